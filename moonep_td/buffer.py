"""``moonep_td.buffer`` -> symmetric-tensor helpers of ``moonep_b200.parallel.symm``."""

from moonep_b200.layout import pad_dim0_for_alignment, pad_to_granularity  # noqa: F401
from moonep_b200.parallel.symm import (  # noqa: F401
    create_full_expert_weight,
    create_nvl_dist_tensor,
    create_nvl_single_owner_tensor,
    nvl_dist_peer_row,
    release_nvl_dist_tensor,
    view_nvl_dist_rows,
)
