"""Dense helpers of the MoE layer's backward pass: batched expert transposes and the SwiGLU backward.

CUDA tensors run the kernels of ``csrc/moe_kernels.cu``; CPU tensors run the same arithmetic in torch.
"""

from __future__ import annotations

import torch

from . import _lib


def transpose_experts(src: torch.Tensor, dst: torch.Tensor, col0: int = 0, active=None) -> torch.Tensor:
    """``dst[n, j, col0 + i] = src[n, i, j]``; ``src`` is ``[n, d0, d1]`` bf16, ``dst`` ``[n, d1, >= col0 + d0]``.
    ``active`` (int32 ``[n]``, optional): matrices whose entry is negative are skipped."""
    n, d0, d1 = (int(v) for v in src.shape)
    assert dst.shape[0] == n and dst.shape[1] == d1 and dst.shape[2] >= col0 + d0 and dst.is_contiguous()
    if active is not None:
        assert active.dtype == torch.int32 and active.numel() == n and active.is_contiguous()
    if not src.is_cuda:
        for i in range(n):
            if active is None or int(active[i]) >= 0:
                dst[i, :, col0 : col0 + d0] = src[i].transpose(0, 1)
        return dst
    assert src.is_contiguous() and src.dtype == torch.bfloat16 and dst.dtype == torch.bfloat16
    with torch.cuda.device(src.device):
        rc = _lib.load().moonep_transpose_experts(
            src.data_ptr(), dst.data_ptr(), n, d0, d1, int(dst.shape[2]), int(dst.shape[1]) * int(dst.shape[2]), int(col0),
            None if active is None else active.data_ptr(), torch.cuda.current_stream().cuda_stream,
        )  # fmt: skip
    _lib.check(rc, "moonep_transpose_experts")
    return dst


def swiglu_bwd(a, u, g, w, total_rows, dadu, hsw, dgate) -> None:
    """See ``csrc/moe_kernels.cu``: fills ``dadu[rows, 2I]``, ``hsw[rows, I]``, ``dgate[rows]`` for rows < total."""
    rows, I = (int(v) for v in a.shape)
    if not a.is_cuda:
        n = int(total_rows[0]) if total_rows is not None else rows
        af, uf, gf = a[:n].float(), u[:n].float(), g[:n].float()
        s = torch.sigmoid(af)
        h = af * s * uf
        dgate[:n] = (gf * h).sum(dim=1)
        dh = gf * w[:n, None]
        dadu[:n, :I] = (dh * uf * s * (1 + af * (1 - s))).to(dadu.dtype)
        dadu[:n, I:] = (dh * af * s).to(dadu.dtype)
        hsw[:n] = (h * w[:n, None]).to(hsw.dtype)
        return
    for t in (a, u, g, dadu, hsw):
        assert t.is_contiguous() and t.dtype == torch.bfloat16
    assert w.dtype == torch.float32 and dgate.dtype == torch.float32 and w.is_contiguous() and dgate.is_contiguous()
    with torch.cuda.device(a.device):
        rc = _lib.load().moonep_swiglu_bwd(
            a.data_ptr(), u.data_ptr(), g.data_ptr(), w.data_ptr(), None if total_rows is None else total_rows.data_ptr(),
            rows, I, dadu.data_ptr(), hsw.data_ptr(), dgate.data_ptr(), torch.cuda.current_stream().cuda_stream,
        )  # fmt: skip
    _lib.check(rc, "moonep_swiglu_bwd")


def sgd_update(w: torch.Tensor, g: torch.Tensor, lr: float) -> None:
    """``w -= lr * g`` for a bf16 weight tensor and its fp32 gradient (same shape, contiguous)."""
    assert w.shape == g.shape
    if not w.is_cuda or w.numel() % 8 != 0:
        w.add_(g, alpha=-lr)
        return
    assert w.is_contiguous() and g.is_contiguous() and w.dtype == torch.bfloat16 and g.dtype == torch.float32
    with torch.cuda.device(w.device):
        rc = _lib.load().moonep_sgd_update(w.data_ptr(), g.data_ptr(), w.numel(), float(lr),
                                           torch.cuda.current_stream().cuda_stream)  # fmt: skip
    _lib.check(rc, "moonep_sgd_update")
