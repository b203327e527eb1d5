"""Planner + dispatch/combine round trip on the host backend with emulated ranks (no GPU):

    python -m moonep_b200.bench.cpu_roundtrip [--ranks 2 --S 512 --H 256 --E 16 --K 4 --steps 3]

Top-k indices are drawn per token without replacement, gates are a softmax over the chosen logits; the expert stage
multiplies every received row by the gate weight that travelled with it, so the result must equal
``sum_k gate[k] * x`` (checked), and the planner outputs are checked against the loop oracle of the package.
Prints one JSON line with the wall time per round trip (all ranks, one thread each).
"""

from __future__ import annotations

import argparse
import json
import time

import numpy as np
import torch

from moonep_b200 import Buffer
from moonep_b200.cpu import planner as P
from moonep_b200.models.routing import make_routing
from moonep_b200.parallel.world import LocalWorld


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--S", type=int, default=512)
    ap.add_argument("--H", type=int, default=256)
    ap.add_argument("--E", type=int, default=16)
    ap.add_argument("--K", type=int, default=4)
    ap.add_argument("--token-padding", type=int, default=128)
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args()
    R, S, H, E, K = a.ranks, a.S, a.H, a.E, a.K
    lw = LocalWorld(R, "cpu")
    bufs = lw.run(lambda r: Buffer(S, H, K, E, R, token_padding=a.token_padding, world=lw.view(r)))
    data = []
    for r in range(R):
        topk, tpe, gates = make_routing("softmax", S, K, E, R, r, seed=2026)
        x = torch.randn(S, H, generator=torch.Generator().manual_seed(r)).to(torch.bfloat16)
        data.append((x, gates, topk, tpe))

    def step(r):
        x, gates, topk, tpe = data[r]
        x_nvs, w_nvs, cu, plan = bufs[r].dispatch(x, gates, topk, tpe, zero_copy=True)
        x_nvs.copy_((x_nvs.float() * w_nvs[:, None]).to(torch.bfloat16))
        out, gates_back, _ = bufs[r].combine(plan, x_nvs, w_nvs, zero_copy=True)
        return out, gates_back, cu, plan

    res = lw.run(step)  # warm-up and correctness
    tpe_all = np.stack([d[3].numpy() for d in data])
    lay = bufs[0]._require_ctx()
    tabs = P.global_tables(tpe_all, S=S, K=K, B=lay["B"], token_padding=a.token_padding, NvS=lay["NvS"])
    ok = True
    err = 0.0
    for r in range(R):
        out, gates_back, cu, plan = res[r]
        x, gates = data[r][0], data[r][1]
        want = x.float() * gates.sum(dim=1, keepdim=True)
        err = max(err, (out.float() - want).abs().max().item())
        ok = ok and bool(torch.equal(gates_back, gates)) and np.array_equal(cu.numpy(), tabs["cu_seqlens"][r])
        ok = ok and np.array_equal(plan.experts_to_copy.numpy(), tabs["experts_to_copy"])
    ok = ok and err <= 0.05 * max(1.0, float(K))
    t0 = time.perf_counter()
    for _ in range(a.steps):
        lw.run(step)
    dt = (time.perf_counter() - t0) / a.steps
    lw.run(lambda r: bufs[r].destroy())
    print(json.dumps({
        "metric": "cpu_emulated_round_trip_seconds", "value": dt, "unit": "s", "higher_is_better": False, "ranks": R,
        "config": {"S_per_rank": S, "H": H, "E": E, "K": K, "token_padding": a.token_padding, "backend": "host (torch/numpy)"},
        "correct": bool(ok), "max_abs_err_vs_sum_gate_x": err, "steps": a.steps,
    }))  # fmt: skip


if __name__ == "__main__":
    main()
