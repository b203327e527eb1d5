"""Grouped expert GEMM: ``y[rows of group g] = x[rows of group g] @ w[g].T`` on tcgen05 tensor cores.

``cu_seqlens[g]`` is the inclusive padded end of group ``g`` in the dispatched shard (what
``Buffer.dispatch`` returns); with ``token_padding`` a multiple of 128 every group is a whole number
of 128-row blocks, which is what the kernel tiles over.  Weights are ``[G, N, K]`` (K contiguous).

Modes: ``plain``; ``swiglu`` (``silu(x @ w_gate.T) * (x @ w_up.T)`` in one pass); ``scale``
(``(x @ w.T) * row_scale[:, None]``, the down projection times the gate weight of each row).
On CPU tensors, or when the shapes do not fit the kernel's tiling, a per-group fp32 reference runs.
"""

from __future__ import annotations

import ctypes

import torch

from .. import config
from . import _lib

_MODES = {"plain": 0, "swiglu": 1, "scale": 2}


class GemmHooks(ctypes.Structure):
    """Tile-by-tile hand-off between the communication kernels and the CTA-pair GEMM (``MoonepGemmHooks`` in
    ``csrc/moonep.h``): per-row arrival flags of a dispatch, the dispatch's "tables ready" word, per-slot flags of a
    weight prefetch, and a per-row-block counter of finished output tiles.  Build one with ``Buffer.gemm_hooks``."""

    _fields_ = [
        ("row_flags", ctypes.c_void_p), ("row_bias", ctypes.c_void_p), ("row_epoch", ctypes.c_int),
        ("tables_epoch", ctypes.c_int), ("tables_ready", ctypes.c_void_p), ("tables_bias", ctypes.c_void_p),
        ("slot_flags", ctypes.c_void_p), ("slot_bias", ctypes.c_void_p), ("slot_epoch", ctypes.c_int),
        ("slot_first_group", ctypes.c_int), ("done_counter", ctypes.c_void_p),
    ]  # fmt: skip


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
            ws = int(gmap[g])
            if ws < 0:
                raise IndexError(f"grouped_gemm: group {g} has rows but no weights on this rank (group_map[{g}] = {ws})")
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
                 group_map=None, save_pre=None, pair=None, hooks=None):
    """See module docstring.  ``x``: ``[rows, K]`` bf16, ``w``: ``[G, N, K]`` bf16, returns ``[rows, N]`` bf16.

    Rows beyond ``cu_seqlens[-1]`` are not written.  Group ends must be multiples of 128.  With
    ``group_map`` (int32 ``[G]``) group ``g`` uses ``w[group_map[g]]`` and ``w`` may hold fewer experts
    than there are groups (e.g. only the experts a rank owns or has prefetched).  ``save_pre=(a, u)`` (SwiGLU
    only, two ``[rows, N]`` bf16 tensors) also stores the pre-activations ``x @ w.T`` and ``x @ w_up.T``.
    ``pair`` selects the kernel: True = CTA pairs (``cta_group::2``), False = one CTA per tile, None = ``MOONEP_GEMM_PAIR``.
    ``hooks`` (a ``GemmHooks``, CTA-pair kernel only) lets the kernel run beside the communication kernels: it waits
    per row block / weight slot for their flags and counts finished output tiles per row block.
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
        if save_pre is not None:
            save_pre[0].copy_(grouped_gemm_reference(x, w, cu_seqlens, group_map=group_map))
            save_pre[1].copy_(grouped_gemm_reference(x, w_up, cu_seqlens, group_map=group_map))
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
    if save_pre is not None:
        assert mode == "swiglu", "save_pre goes with mode='swiglu'"
        for t in save_pre:
            assert t.is_contiguous() and t.shape == out.shape and t.dtype == torch.bfloat16 and t.device == out.device
    lib = _lib.load()
    use_pair = config.gemm_on_cta_pairs() if pair is None else pair
    assert hooks is None or use_pair, "hooks need the CTA-pair kernel"
    with torch.cuda.device(x.device):
        args = (
            x.data_ptr(), w.data_ptr(), None if w_up is None else w_up.data_ptr(), out.data_ptr(),
            None if row_scale is None else row_scale.data_ptr(), cu_seqlens.data_ptr(), G, int(x.shape[0]), K, N,
            _MODES[mode], None if status is None else status.data_ptr(), config.timeout_ms(), int(num_sms),
            None if group_map is None else group_map.data_ptr(), W,
            None if save_pre is None else save_pre[0].data_ptr(), None if save_pre is None else save_pre[1].data_ptr(),
        )  # fmt: skip
        st = torch.cuda.current_stream().cuda_stream
        if hooks is not None:
            rc = lib.moonep_grouped_gemm_pair_hooked(*args, ctypes.byref(hooks), st)
        else:
            rc = (lib.moonep_grouped_gemm_pair if use_pair else lib.moonep_grouped_gemm)(*args, st)
    _lib.check(rc, "moonep_grouped_gemm")
    return out


def grouped_gemm_kn_reference(x, ws, cu_seqlens):
    """``y[rows of g] = x[rows of g] @ cat([w[g] for w in ws], dim=0)`` per group in fp32."""
    N = int(ws[0].shape[2])
    out = torch.zeros(x.shape[0], N, dtype=torch.bfloat16, device=x.device)
    start = 0
    for g, end in enumerate(cu_seqlens.tolist()):
        if end > start:
            wcat = torch.cat([w[g].float() for w in ws], dim=0)
            out[start:end] = (x[start:end].float() @ wcat).to(torch.bfloat16)
        start = max(start, int(end))
    return out


def kn_kernel_supports(x, ws) -> bool:
    N = int(ws[0].shape[2])
    return (x.is_cuda and x.dtype == torch.bfloat16 and N % 256 == 0 and all(int(w.shape[1]) % 64 == 0 for w in ws)
            and x.shape[0] >= 128 and len(ws) in (1, 2) and config.gemm_on_cta_pairs())  # fmt: skip


def grouped_gemm_kn(x, ws, cu_seqlens, *, out=None, status=None, num_sms=0):
    """``y[rows of g] = x[rows of g] @ W[g]`` with the weights given as ``[G, K, N]`` (N contiguous): the product an
    activation gradient needs from forward weights stored ``[G, out, in]``, without transposed copies.  ``ws`` is one
    tensor or two that continue the contraction (``x = [a | b]``, ``W = [ws[0]; ws[1]]``).  Runs on the CTA-pair kernel
    (MN-major W tiles); a per-group fp32 reference elsewhere."""
    ws = list(ws)
    G, _, N = (int(v) for v in ws[0].shape)
    Ks = [int(w.shape[1]) for w in ws]
    assert x.dim() == 2 and x.shape[1] == sum(Ks) and cu_seqlens.numel() == G
    assert all(w.shape[0] == G and w.shape[2] == N for w in ws)
    if not kn_kernel_supports(x, ws):
        res = grouped_gemm_kn_reference(x, ws, cu_seqlens)
        if out is not None:
            out.copy_(res)
            return out
        return res
    assert x.is_contiguous() and all(w.is_contiguous() and w.dtype == torch.bfloat16 for w in ws)
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.is_contiguous() and cu_seqlens.is_cuda
    if out is None:
        out = torch.empty(x.shape[0], N, dtype=torch.bfloat16, device=x.device)
    assert out.is_contiguous() and out.shape == (x.shape[0], N) and out.dtype == torch.bfloat16
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.moonep_grouped_gemm_pair_kn(
            x.data_ptr(), ws[0].data_ptr(), Ks[0], ws[1].data_ptr() if len(ws) == 2 else None, Ks[1] if len(ws) == 2 else 0,
            out.data_ptr(), cu_seqlens.data_ptr(), G, int(x.shape[0]), N, G, None if status is None else status.data_ptr(),
            config.timeout_ms(), int(num_sms), torch.cuda.current_stream().cuda_stream,
        )  # fmt: skip
    _lib.check(rc, "moonep_grouped_gemm_pair_kn")
    return out


WGRAD_STORE, WGRAD_ACCUMULATE, WGRAD_STORE_NONEMPTY = 0, 1, 2
WGRAD_MAX_GROUPS = 512  # groups per launch of the weight-gradient kernel (its work list lives in shared memory)


def grouped_wgrad_reference(left, right, cu_seqlens, targets, flags):
    """Per-group matmuls: ``targets[g] (=, +=) left[rows of g].T @ right[rows of g]`` (the oracle and CPU path).
    ``targets[g]`` is an fp32 ``[P, Q]`` tensor or None; ``flags`` as in ``grouped_wgrad``."""
    ends = cu_seqlens.tolist()
    start = 0
    for g, tgt in enumerate(targets):
        end = int(ends[g])
        flag = int(flags[g])
        if tgt is not None:
            if end > start:
                mm = left[start:end].float().t() @ right[start:end].float()
                if flag == WGRAD_ACCUMULATE:
                    tgt.add_(mm)
                else:
                    tgt.copy_(mm)
            elif flag == WGRAD_STORE:
                tgt.zero_()
        start = max(start, end)


def wgrad_kernel_supports(P: int, Q: int, ld: int, device) -> bool:
    return torch.device(device).type == "cuda" and P % 128 == 0 and Q % 256 == 0 and ld % 64 == 0 and ld > 0


def grouped_wgrad(left_t, right_t, cu_seqlens, out_ptrs, flags, *, status=None, num_sms=0):
    """Weight gradients of every group in one launch of the tcgen05 kernel.

    ``left_t``: ``[P, ld]`` bf16 and ``right_t``: ``[Q, ld]`` bf16 are the TRANSPOSED operands (column index =
    row of the dispatched shard), so that the contraction over a group's rows is K-major for both.  For group
    ``g`` with rows ``[cu[g-1], cu[g])`` (multiples of 16): the fp32 ``[P, Q]`` matrix at address ``out_ptrs[g]``
    (int64 device tensor, 0 = skip) is overwritten (``flags[g] == 0``; zeros if the group is empty), added to
    (``1``) or overwritten unless the group is empty (``2``).  ``flags``: int32 device tensor ``[G]``.
    """
    P, ld = (int(v) for v in left_t.shape)
    Q = int(right_t.shape[0])
    G = int(cu_seqlens.numel())
    assert right_t.shape[1] == ld and left_t.dtype == torch.bfloat16 and right_t.dtype == torch.bfloat16
    assert left_t.is_contiguous() and right_t.is_contiguous()
    assert wgrad_kernel_supports(P, Q, ld, left_t.device), f"grouped_wgrad: P={P}, Q={Q}, ld={ld} do not fit the tiling"
    assert G <= WGRAD_MAX_GROUPS, f"grouped_wgrad: at most {WGRAD_MAX_GROUPS} groups per launch"
    assert out_ptrs.dtype == torch.int64 and out_ptrs.numel() == G and out_ptrs.is_cuda and out_ptrs.is_contiguous()
    assert flags.dtype == torch.int32 and flags.numel() == G and flags.is_cuda and flags.is_contiguous()
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.is_contiguous() and cu_seqlens.is_cuda
    lib = _lib.load()
    with torch.cuda.device(left_t.device):
        rc = lib.moonep_grouped_wgrad(
            left_t.data_ptr(), right_t.data_ptr(), ld, P, Q, cu_seqlens.data_ptr(), G, out_ptrs.data_ptr(),
            flags.data_ptr(), ld, None if status is None else status.data_ptr(), config.timeout_ms(), int(num_sms),
            torch.cuda.current_stream().cuda_stream,
        )  # fmt: skip
    _lib.check(rc, "moonep_grouped_wgrad")


def grouped_wgrad_rows(left, right, cu_seqlens, out_ptrs, flags, *, status=None, num_sms=0):
    """``grouped_wgrad`` from the operands as they are: ``left`` ``[rows, P]`` and ``right`` ``[rows, Q]`` bf16 with unit
    column stride (column slices of wider tensors are fine), no transposed copies.  Same targets and flags."""
    rows, P = (int(v) for v in left.shape)
    Q = int(right.shape[1])
    G = int(cu_seqlens.numel())
    assert right.shape[0] == rows and left.dtype == torch.bfloat16 and right.dtype == torch.bfloat16
    assert left.stride(1) == 1 and right.stride(1) == 1 and left.is_cuda
    ldl, ldr = int(left.stride(0)), int(right.stride(0))
    assert P % 128 == 0 and Q % 256 == 0 and ldl % 8 == 0 and ldr % 8 == 0, f"P={P}, Q={Q}, strides {ldl}, {ldr}"
    assert G <= WGRAD_MAX_GROUPS, f"grouped_wgrad_rows: at most {WGRAD_MAX_GROUPS} groups per launch"
    assert left.data_ptr() % 16 == 0 and right.data_ptr() % 16 == 0
    assert out_ptrs.dtype == torch.int64 and out_ptrs.numel() == G and out_ptrs.is_cuda and out_ptrs.is_contiguous()
    assert flags.dtype == torch.int32 and flags.numel() == G and flags.is_cuda and flags.is_contiguous()
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.is_contiguous() and cu_seqlens.is_cuda
    lib = _lib.load()
    with torch.cuda.device(left.device):
        rc = lib.moonep_grouped_wgrad_rows(
            left.data_ptr(), ldl, right.data_ptr(), ldr, rows, P, Q, cu_seqlens.data_ptr(), G, out_ptrs.data_ptr(),
            flags.data_ptr(), None if status is None else status.data_ptr(), config.timeout_ms(), int(num_sms),
            torch.cuda.current_stream().cuda_stream,
        )  # fmt: skip
    _lib.check(rc, "moonep_grouped_wgrad_rows")


def _fallback_allowed() -> bool:
    import os

    return os.environ.get("MOONEP_GEMM_FALLBACK", "0") not in ("0", "", "false", "False")
