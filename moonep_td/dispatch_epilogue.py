"""``moonep_td.dispatch_epilogue`` -> ``moonep_b200.ops.launch.launch_dispatch_epilogue``: zero fill and duplicate expansion (reference moonep_td/dispatch_epilogue.py:45)."""

from moonep_b200.ops.launch import launch_dispatch_epilogue  # noqa: F401
