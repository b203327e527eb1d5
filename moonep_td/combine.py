"""``moonep_td.combine`` -> ``moonep_b200.ops.launch.launch_combine``: per-token gather and K-sum (reference moonep_td/combine.py:77)."""

from moonep_b200.ops.launch import launch_combine  # noqa: F401
