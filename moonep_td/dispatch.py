"""``moonep_td.dispatch`` -> ``moonep_b200.ops.launch.launch_dispatch``: row push of the dispatch (reference moonep_td/dispatch.py:126)."""

from moonep_b200.ops.launch import launch_dispatch  # noqa: F401
