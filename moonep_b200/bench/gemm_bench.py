"""Time the tcgen05 grouped GEMM on MoE-layer shapes and report the fraction of the measured peak.

    python -m moonep_b200.bench.gemm_bench [--rows 32768 --groups 40 --H 7168 --I 2048 --iters 10]

Prints one JSON line per GEMM (SwiGLU gate/up, down projection, weight gradient of the down projection with
and without the operand transposes) with TFLOP/s, the cuBLAS figure from MEASURED_PEAKS.json if present, and a
torch batched-matmul baseline on the same data.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from moonep_b200 import config
from moonep_b200.ops.grouped_gemm import grouped_gemm, grouped_wgrad, grouped_wgrad_rows
from moonep_b200.ops.moe_ops import transpose_experts


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        flush.zero_()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in ev)
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--groups", type=int, default=40)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--I", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--small", action="store_true", help="few hundred MB case for profilers")
    a = ap.parse_args()
    if a.small:
        a.rows, a.groups, a.H, a.I, a.iters = 8192, 8, 2048, 2048, 2
    dev = "cuda"
    peaks = {}
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        peaks = json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("bf16_tflops", 1590.0))
    per = a.rows // a.groups // 128 * 128
    ends = torch.tensor([per * (g + 1) for g in range(a.groups)], dtype=torch.int32, device=dev)
    total = per * a.groups
    x = (torch.randn(total, a.H, device=dev) * 0.5).to(torch.bfloat16)
    wg = (torch.randn(a.groups, a.I, a.H, device=dev) * 0.02).to(torch.bfloat16)
    wu = (torch.randn(a.groups, a.I, a.H, device=dev) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(a.groups, a.H, a.I, device=dev) * 0.02).to(torch.bfloat16)
    scale = torch.rand(total, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    h = torch.empty(total, a.I, dtype=torch.bfloat16, device=dev)
    y = torch.empty(total, a.H, dtype=torch.bfloat16, device=dev)

    t1 = _time(lambda: grouped_gemm(x, wg, ends, w_up=wu, mode="swiglu", out=h, status=status), a.iters, flush)
    t2 = _time(lambda: grouped_gemm(h, wd, ends, row_scale=scale, mode="scale", out=y, status=status), a.iters, flush)
    assert status.tolist()[0] == 0, status.tolist()

    xs = x.view(a.groups, per, a.H)

    def torch_up():
        g = torch.bmm(xs, wg.transpose(1, 2))
        u = torch.bmm(xs, wu.transpose(1, 2))
        return torch.nn.functional.silu(g) * u

    hs = h.view(a.groups, per, a.I)
    t1_ref = _time(torch_up, a.iters, flush)
    t2_ref = _time(lambda: torch.bmm(hs, wd.transpose(1, 2)) * scale.view(a.groups, per, 1), a.iters, flush)
    ref = torch_up().reshape(total, a.I).float()
    err = (h.float() - ref).abs().max().item() / max(1e-6, ref.abs().max().item())
    f1 = 2.0 * total * a.H * a.I * 2
    f2 = 2.0 * total * a.H * a.I
    for name, t, tr, f in (("swiglu_gate_up", t1, t1_ref, f1), ("down_scale", t2, t2_ref, f2)):
        print(json.dumps({
            "gemm": name, "kernel": "cta_pair (cta_group::2)" if config.gemm_on_cta_pairs() else "one CTA per tile",
            "rows": total, "groups": a.groups, "H": a.H, "I": a.I, "ms": round(t, 4),
            "tflops": round(f / t / 1e9, 1), "frac_of_measured_cublas_peak": round(f / t / 1e9 / peak, 3),
            "torch_bmm_plus_elementwise_ms": round(tr, 4), "speedup_vs_torch": round(tr / t, 2),
            "rel_err_vs_torch": round(err, 5), "measured_peak_tflops": peak,
        }))  # fmt: skip

    # weight gradient of the down projection: dW[g] (H x I, fp32) += dy_g^T h_g, contraction over the rows of a group
    if total % 64 == 0 and a.H % 256 == 0 and a.I % 256 == 0:
        dw = torch.zeros(a.groups, a.H, a.I, device=dev)
        ptrs = torch.tensor([dw[g].data_ptr() for g in range(a.groups)], dtype=torch.int64, device=dev)
        flags = torch.ones(a.groups, dtype=torch.int32, device=dev)  # accumulate, as in a training step
        yt = torch.empty(1, a.H, total, dtype=torch.bfloat16, device=dev)
        ht = torch.empty(1, a.I, total, dtype=torch.bfloat16, device=dev)

        def transposes():
            transpose_experts(y.unsqueeze(0), yt)
            transpose_experts(h.unsqueeze(0), ht)

        transposes()
        t3 = _time(lambda: grouped_wgrad(yt[0], ht[0], ends, ptrs, flags, status=status), a.iters, flush)
        t3t = _time(transposes, a.iters, flush)
        t3r = _time(lambda: grouped_wgrad_rows(y, h, ends, ptrs, flags, status=status), a.iters, flush)
        assert status.tolist()[0] == 0, status.tolist()
        ys = y.view(a.groups, per, a.H)
        t3_ref = _time(lambda: dw.add_(torch.bmm(ys.transpose(1, 2), hs)), a.iters, flush)  # bf16 bmm, fp32 add
        dw.zero_()
        flags.zero_()
        grouped_wgrad(yt[0], ht[0], ends, ptrs, flags, status=status)
        ref3 = torch.bmm(ys[:2].transpose(1, 2).float(), hs[:2].float())
        err3 = (dw[:2] - ref3).abs().max().item() / max(1e-6, ref3.abs().max().item())
        print(json.dumps({
            "gemm": "wgrad_down_accumulate", "rows": total, "groups": a.groups, "H": a.H, "I": a.I, "ms": round(t3, 4),
            "tflops": round(f2 / t3 / 1e9, 1), "frac_of_measured_cublas_peak": round(f2 / t3 / 1e9 / peak, 3),
            "operand_transposes_ms": round(t3t, 4), "ms_from_row_major_operands": round(t3r, 4),
            "tflops_from_row_major_operands": round(f2 / t3r / 1e9, 1), "torch_bmm_then_add_ms": round(t3_ref, 4),
            "speedup_vs_torch": round(t3_ref / t3, 2), "speedup_vs_torch_with_transposes": round(t3_ref / (t3 + t3t), 2),
            "rel_err_vs_torch": round(err3, 6), "measured_peak_tflops": peak,
        }))  # fmt: skip


if __name__ == "__main__":
    main()
