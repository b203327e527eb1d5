"""Small, self-terminating workloads for profilers (a few hundred MB to a few GB on the device, inputs larger than
L2, a handful of launches), used as the targets of the ``ncu`` captures summarised under ``profiles/``.

    python -m moonep_b200.bench.profile_case --what roundtrip --ranks 4 --S 2048 --steps 2
    python -m moonep_b200.bench.profile_case --what weights --ranks 2 --steps 2
    python -m moonep_b200.bench.profile_case --what moe --ranks 1 --S 2048 --steps 2

``roundtrip``: R emulated ranks on one GPU run dispatch + combine (emulated ranks launch the dispatch and combine
kernels one role at a time, so every role shows up as a launch of its own; with ``--ranks 1`` set ``MOONEP_PHASED=1``
for the same effect).  ``weights``: ``prefetch_weight`` and ``reduce_grad`` with every slot in use.  ``moe``: forward
and backward of the SwiGLU MoE layer (grouped GEMMs with their hand-off hooks, weight-gradient kernel, SwiGLU
backward).
"""

from __future__ import annotations

import argparse
import dataclasses

import torch

from moonep_b200 import Buffer
from moonep_b200.models.routing import make_routing
from moonep_b200.parallel.world import LocalWorld


def roundtrip(a, lw, R):
    bufs = lw.run(lambda r: Buffer(a.S, a.H, a.K, a.E, R, num_sms=a.num_sms, token_padding=128, world=lw.view(r)))
    inputs = []
    for r in range(R):
        topk, tpe, gates = make_routing("softmax", a.S, a.K, a.E, R, r, seed=2026, device="cuda:0")
        inputs.append((torch.randn(a.S, a.H, device="cuda:0").to(torch.bfloat16), gates, topk, tpe))

    def body(r):
        x, gates, topk, tpe = inputs[r]
        for _ in range(a.steps):
            xn, wn, cu, plan = bufs[r].dispatch(x, gates, topk, tpe, zero_copy=True)
            out, wb, _ = bufs[r].combine(plan, xn, wn, zero_copy=True)
        torch.cuda.synchronize()
        bufs[r].check_status()
        return float((out.float() - a.K * x.float()).abs().max())

    errs = lw.run(body)
    assert max(errs) <= 0.25, errs
    lw.run(lambda r: bufs[r].destroy())
    return errs


def weights(a, lw, R):
    from moonep_b200.parallel.symm import create_full_expert_weight, create_nvl_dist_tensor, view_nvl_dist_rows

    E, H, inter, S, K = a.E, a.H, a.inter, 256, a.K
    epn = E // R
    B = min(epn, a.slots)
    bufs = lw.run(lambda r: Buffer(S, H, K, E, R, num_sms=a.num_sms, token_padding=128, B=B, world=lw.view(r)))
    shapes = ((inter, H), (inter, H), (H, inter))

    def body(r):
        w = lw.view(r)
        dev = "cuda:0"
        topk, tpe, gates = make_routing("softmax", S, K, E, R, r, seed=1, device=dev)
        x = torch.randn(S, H, device=dev).to(torch.bfloat16)
        plan = bufs[r].dispatch(x, gates, topk, tpe)[3]
        etc = torch.full((R, B), -1, dtype=torch.int32)
        for q in range(R):
            etc[q] = torch.arange(B, dtype=torch.int32) + ((q + 1) % R) * epn
        plan = dataclasses.replace(plan, experts_to_copy=etc.to(dev))
        ws = [create_full_expert_weight(E, B, d0, d1, w) for d0, d1 in shapes]
        for t in ws:
            t[:E].normal_(0, 0.02)
        reds = [view_nvl_dist_rows(create_nvl_dist_tensor([B, d0, d1], torch.float32, w, pad_dim0=False), R, B)
                for d0, d1 in shapes]  # fmt: skip
        grads = [torch.zeros(epn, d0, d1, dtype=torch.float32, device=dev) for d0, d1 in shapes]
        for _ in range(a.steps):
            for t in reds:
                t[r].fill_(1.0)
            w.step()
            bufs[r].prefetch_weight(plan, full_gate_weight=ws[0], full_up_weight=ws[1], full_down_weight=ws[2])
            bufs[r].reduce_grad(plan, False, grads[0], grads[1], grads[2], reds[0], reds[1], reds[2], owner_local=True)
        torch.cuda.synchronize()
        bufs[r].check_status()
        return float(grads[0].abs().max())

    out = lw.run(body)
    lw.run(lambda r: bufs[r].destroy())
    return out


def moe(a, lw, R):
    from moonep_b200.models.moe_layer import ExpertParallelMoE

    bufs = lw.run(lambda r: Buffer(a.S, a.H, a.K, a.E, R, num_sms=a.num_sms, token_padding=128, B=min(a.E // R, a.slots),
                                   world=lw.view(r)))  # fmt: skip
    layers = lw.run(lambda r: ExpertParallelMoE(bufs[r], a.inter, init_std=0.02, seed=1))

    def body(r):
        dev = "cuda:0"
        topk, tpe, gates = make_routing("softmax", a.S, a.K, a.E, R, r, seed=3, device=dev)
        x = torch.randn(a.S, a.H, device=dev).to(torch.bfloat16)
        go = (torch.randn(a.S, a.H, device=dev) * 0.1).to(torch.bfloat16)
        for _ in range(a.steps):
            out, saved = layers[r].forward(x, gates, topk, tpe)
            dx, dg = layers[r].backward(saved, go)
            layers[r].sgd_step(1e-5)
            layers[r].zero_grad()
        layers[r].check()
        return bool(torch.isfinite(out.float()).all() and torch.isfinite(dx.float()).all())

    ok = lw.run(body)
    assert all(ok), ok
    lw.run(lambda r: layers[r].destroy())
    lw.run(lambda r: bufs[r].destroy())
    return ok


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="roundtrip", choices=["roundtrip", "weights", "moe"])
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--S", type=int, default=2048)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--E", type=int, default=256)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--slots", type=int, default=4)
    ap.add_argument("--num-sms", type=int, default=32)
    ap.add_argument("--steps", type=int, default=2)
    a = ap.parse_args()
    lw = LocalWorld(a.ranks, "cuda:0")
    res = {"roundtrip": roundtrip, "weights": weights, "moe": moe}[a.what](a, lw, a.ranks)
    print(f"profile_case {a.what} ok", res)


if __name__ == "__main__":
    main()
