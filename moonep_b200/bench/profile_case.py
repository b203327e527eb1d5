"""Small, self-terminating workload for profilers: R emulated ranks on one GPU run a few
dispatch+combine steps (inputs larger than L2, a few hundred MB on the device).

    python -m moonep_b200.bench.profile_case --ranks 4 --S 2048 --steps 2

Used as the target of the ``ncu`` captures summarised under ``profiles/``.
"""

from __future__ import annotations

import argparse

import torch

from moonep_b200 import Buffer
from moonep_b200.models.routing import make_routing
from moonep_b200.parallel.world import LocalWorld


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--S", type=int, default=2048)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--E", type=int, default=256)
    ap.add_argument("--num-sms", type=int, default=32)
    ap.add_argument("--steps", type=int, default=2)
    a = ap.parse_args()
    R = a.ranks
    lw = LocalWorld(R, "cuda:0")
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
    print("profile_case ok", errs)


if __name__ == "__main__":
    main()
