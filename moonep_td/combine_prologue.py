"""``moonep_td.combine_prologue`` -> ``moonep_b200.ops.launch.launch_combine_prologue``: duplicate fold (reference moonep_td/combine_prologue.py:45)."""

from moonep_b200.ops.launch import launch_combine_prologue  # noqa: F401
