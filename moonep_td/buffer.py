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


def ensure_nvshmem_initialized(group=None) -> None:
    """Kept for code written against the reference (moonep_td/buffer.py:40), which initialises NVSHMEM here.  This
    implementation has no such runtime: symmetric memory comes from its own CUDA-VMM allocator, set up when the first
    ``Buffer`` or symmetric tensor of a process group is created.  Only checks that a process group exists."""
    import torch.distributed as dist

    if group is None and not dist.is_initialized():
        raise RuntimeError("initialise torch.distributed (backend 'nccl' on GPUs) before creating symmetric memory")
