"""``moonep_td.prefetch`` -> ``moonep_b200.ops.launch.launch_prefetch``: expert-weight prefetch (reference moonep_td/prefetch.py:73)."""

from moonep_b200.ops.launch import launch_prefetch  # noqa: F401
