"""Symmetric ("NVL distributed") tensors for expert weights and gradient buffers.

``create_nvl_dist_tensor([B, H, Hp], dtype, world)`` returns ``[R*B_pad, H, Hp]``:
chunk r (rows ``[r*B_pad, (r+1)*B_pad)``) is physically on rank r and every rank sees
all chunks in one address range, so plain indexing reaches peer memory over NVLink.
``create_full_expert_weight`` builds the ``[E+B, H, Hp]`` weight layout the Buffer
expects: experts ``[0, E)`` distributed over their owners, slots ``[E, E+B)`` local.

Parity: reference ``moonep_td/buffer.py:62-135`` (``view_nvl_dist_rows``,
``nvl_dist_peer_row``, ``create_nvl_dist_tensor``, ``release_nvl_dist_tensor``,
``create_nvl_single_owner_tensor``).  There a peer's rows must be fetched through
``nvshmem.core.get_peer_tensor``; here they are ordinary rows of the tensor.
"""

from __future__ import annotations

import torch

from ..layout import pad_dim0_for_alignment, pad_to_granularity  # noqa: F401  (re-exported)
from .world import SymmetricTensor, World

_LIVE: dict[int, SymmetricTensor] = {}


def _inner(shape) -> int:
    n = 1
    for d in shape[1:]:
        n *= int(d)
    return n


def create_nvl_dist_tensor(shape, dtype: torch.dtype, world: World, *, pad_dim0: bool = True) -> torch.Tensor:
    """Collective.  ``shape`` is one rank's chunk; returns the ``[R*dim0_padded, ...]`` tensor."""
    shape = [int(s) for s in shape]
    gran = world.granularity()
    dim0 = pad_dim0_for_alignment(shape, dtype, gran) if pad_dim0 else shape[0]
    chunk_numel = dim0 * _inner(shape)
    st = world.alloc_symmetric(chunk_numel, dtype, gran)
    full = st.full.view(world.size * dim0, *shape[1:])
    _LIVE[full.data_ptr()] = st
    return full


def release_nvl_dist_tensor(tensor: torch.Tensor) -> None:
    """Collective on real worlds: free a tensor made by ``create_nvl_dist_tensor``."""
    st = _LIVE.pop(tensor.data_ptr(), None)
    if st is not None:
        st.release()


def view_nvl_dist_rows(full: torch.Tensor, world_size: int, B: int) -> torch.Tensor:
    """View ``[R*B, ...]`` as ``[R, B, ...]``."""
    assert full.shape[0] == world_size * B, f"expected dim0={world_size * B}, got {full.shape[0]}"
    return full.view(world_size, B, *full.shape[1:])


def nvl_dist_peer_row(full: torch.Tensor, row: int, rank: int, world_size: int, B: int) -> torch.Tensor:
    """Rank ``row``'s ``[B, ...]`` slice (peer memory is directly addressable)."""
    del rank
    if full.ndim >= 2 and full.shape[0] == world_size and full.shape[1] == B:
        return full[row]
    return view_nvl_dist_rows(full, world_size, B)[row]


def create_nvl_single_owner_tensor(shape, dtype, owner_rank: int, world: World) -> torch.Tensor:
    """``[E, H, Hp]`` tensor whose storage lives on ``owner_rank`` and is readable by every rank."""
    full = create_nvl_dist_tensor(shape, dtype, world)
    dim0 = full.shape[0] // world.size
    view = full[owner_rank * dim0 : owner_rank * dim0 + int(shape[0])]
    _LIVE[view.data_ptr()] = _LIVE[full.data_ptr()]
    return view


def create_full_expert_weight(E: int, B: int, H: int, Hp: int, world: World, dtype=torch.bfloat16) -> torch.Tensor:
    """Collective.  Weight tensor ``[E+B, H, Hp]``: experts ``[0, E)`` live on their owners
    (rank r holds experts ``[r*E/R, (r+1)*E/R)``), slots ``[E, E+B)`` are local.

    On a multi-process CUDA world the peers' experts and the local slots are mapped back to
    back in one address range (``E/R * H * Hp`` elements must fill whole VMM granules).  On
    emulated and host worlds there is no peer mapping: a plain local tensor is returned and
    the caller fills ``[:E]`` with all experts.
    """
    R = world.size
    assert E % R == 0
    if world.is_cuda and not world.emulated and R > 1:
        from .vmm import VmmAllocator

        full, st = VmmAllocator.get(world).alloc_expert_weight(E // R, B, H, Hp, dtype)
        _LIVE[full.data_ptr()] = st
        return full
    return torch.zeros(E + B, H, Hp, dtype=dtype, device=world.device)
