"""Grouped expert GEMM: ``y[rows of group g] = x[rows of group g] @ w[g].T`` on tcgen05 tensor cores.

``cu_seqlens[g]`` is the inclusive padded end of group ``g`` in the dispatched shard (what
``Buffer.dispatch`` returns); with ``token_padding`` a multiple of 128 every group is a whole number
of 128-row blocks, which is what the kernel tiles over.  Weights are ``[G, N, K]`` (K contiguous).

Modes: ``plain``; ``swiglu`` (``silu(x @ w_gate.T) * (x @ w_up.T)`` in one pass); ``scale``
(``(x @ w.T) * row_scale[:, None]``, the down projection times the gate weight of each row).
On CPU tensors, or when the shapes do not fit the kernel's tiling, a per-group fp32 reference runs.
"""

from __future__ import annotations

import torch

from .. import config
from . import _lib

_MODES = {"plain": 0, "swiglu": 1, "scale": 2}


def grouped_gemm_reference(x, w, cu_seqlens, *, w_up=None, row_scale=None, mode="plain", group_map=None):
    """Per-group fp32 matmul; the oracle of the kernel and the CPU path."""
    _, N, K = w.shape
    G = cu_seqlens.numel()
    out = torch.zeros(x.shape[0], N, dtype=torch.bfloat16, device=x.device)
    ends = cu_seqlens.tolist()
    gmap = list(range(G)) if group_map is None else group_map.tolist()
    start = 0
    for g in range(G):
        end = int(ends[g])
        if end > start:
            xs = x[start:end].float()
            ws = max(0, int(gmap[g]))
            y = xs @ w[ws].float().t()
            if mode == "swiglu":
                y = torch.nn.functional.silu(y) * (xs @ w_up[ws].float().t())
            elif mode == "scale" and row_scale is not None:
                y = y * row_scale[start:end, None]
            out[start:end] = y.to(torch.bfloat16)
        start = max(start, end)
    return out


def kernel_supports(x, w, mode: str) -> bool:
    G, N, K = w.shape
    tile_n = 128 if mode == "swiglu" else 256
    return x.is_cuda and x.dtype == torch.bfloat16 and K % 64 == 0 and N % tile_n == 0 and x.shape[0] >= 128


def grouped_gemm(x, w, cu_seqlens, *, w_up=None, row_scale=None, mode="plain", out=None, status=None, num_sms=0,
                 group_map=None):
    """See module docstring.  ``x``: ``[rows, K]`` bf16, ``w``: ``[G, N, K]`` bf16, returns ``[rows, N]`` bf16.

    Rows beyond ``cu_seqlens[-1]`` are not written.  Group ends must be multiples of 128.  With
    ``group_map`` (int32 ``[G]``) group ``g`` uses ``w[group_map[g]]`` and ``w`` may hold fewer experts
    than there are groups (e.g. only the experts a rank owns or has prefetched).
    """
    assert mode in _MODES
    W, N, K = (int(v) for v in w.shape)
    G = int(cu_seqlens.numel())
    assert x.dim() == 2 and x.shape[1] == K and (group_map is not None or W == G)
    if group_map is not None:
        assert group_map.dtype == torch.int32 and group_map.is_contiguous() and group_map.numel() == G
    if not kernel_supports(x, w, mode):
        if x.is_cuda and torch.cuda.is_available() and not _fallback_allowed():
            raise RuntimeError(
                f"grouped_gemm: shapes rows={x.shape[0]}, K={K}, N={N} do not fit the tcgen05 kernel's tiling "
                "(K % 64, N % 256 or 128 for swiglu, rows >= 128); set MOONEP_GEMM_FALLBACK=1 to use the reference"
            )
        res = grouped_gemm_reference(x, w, cu_seqlens, w_up=w_up, row_scale=row_scale, mode=mode, group_map=group_map)
        if out is not None:
            out.copy_(res)
            return out
        return res
    assert x.is_contiguous() and w.is_contiguous() and w.dtype == torch.bfloat16
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.is_contiguous() and cu_seqlens.is_cuda
    if mode == "swiglu":
        assert w_up is not None and w_up.shape == w.shape and w_up.is_contiguous() and w_up.dtype == torch.bfloat16
    if row_scale is not None:
        assert row_scale.dtype == torch.float32 and row_scale.is_contiguous() and row_scale.numel() >= x.shape[0]
    if out is None:
        out = torch.empty(x.shape[0], N, dtype=torch.bfloat16, device=x.device)
    assert out.is_contiguous() and out.shape == (x.shape[0], N) and out.dtype == torch.bfloat16
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.moonep_grouped_gemm(
            x.data_ptr(), w.data_ptr(), None if w_up is None else w_up.data_ptr(), out.data_ptr(),
            None if row_scale is None else row_scale.data_ptr(), cu_seqlens.data_ptr(), G, int(x.shape[0]), K, N,
            _MODES[mode], None if status is None else status.data_ptr(), config.timeout_ms(), int(num_sms),
            None if group_map is None else group_map.data_ptr(), W, torch.cuda.current_stream().cuda_stream,
        )  # fmt: skip
    _lib.check(rc, "moonep_grouped_gemm")
    return out


def _fallback_allowed() -> bool:
    import os

    return os.environ.get("MOONEP_GEMM_FALLBACK", "0") not in ("0", "", "false", "False")
