"""``moonep_td.inter_rank_sync`` -> ``moonep_b200.ops.launch.launch_inter_rank_sync``: cross-rank flag round (reference moonep_td/inter_rank_sync.py:8)."""

from moonep_b200.ops.launch import launch_inter_rank_sync  # noqa: F401
