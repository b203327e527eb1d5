"""``moonep_td._dedup_builder`` -> ``moonep_b200.ops.launch.launch_dedup_builder``: duplicate-map rebuild (reference moonep_td/_dedup_builder.py:113)."""

from moonep_b200.ops.launch import launch_dedup_builder  # noqa: F401
