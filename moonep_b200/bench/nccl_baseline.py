"""Baseline for the dispatch/combine benchmark: the textbook NCCL ``all_to_all_single`` round trip.

Not a product path.  Per step: the (token, destination rank) pairs are deduplicated per rank
(same traffic as the library's per-rank dedup), sorted by destination, the row counts are
exchanged, the rows go out with ``all_to_all_single`` (split sizes need a host sync, as in
common MoE implementations), and come back the same way to be summed per token.  No load
balancing, no expert-major layout, no weights channel: this is the cheapest thing NCCL can
do for the same routing, so it bounds what "just call NCCL" achieves on the box.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def run_nccl_baseline(args, rank: int, n: int) -> dict:
    from ..models.routing import make_routing
    from ..utils.clocks import ClockSampler

    S, H, K, E = args.S, args.H, args.K, args.E
    dev = torch.device("cuda", torch.cuda.current_device())
    epn = E // n
    topk, tpe, gates = make_routing(args.routing, S, K, E, n, rank, seed=2026, device=dev)
    g = torch.Generator().manual_seed(7 + rank)
    x = torch.randn(S, H, generator=g).to(torch.bfloat16).to(dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def dispatch():
        dest = (topk // epn).long()  # [S, K]
        hit = torch.zeros(S, n, dtype=torch.bool, device=dev)
        hit.scatter_(1, dest, True)
        tok, rk = hit.nonzero(as_tuple=True)  # sorted by token, then rank
        order = torch.argsort(rk, stable=True)
        tok, rk = tok[order], rk[order]
        send_counts = torch.bincount(rk, minlength=n)
        recv_counts = torch.empty_like(send_counts)
        if n > 1:
            dist.all_to_all_single(recv_counts, send_counts)
        else:
            recv_counts.copy_(send_counts)
        sc, rc = send_counts.tolist(), recv_counts.tolist()  # host sync
        send = x[tok]
        recv = torch.empty(sum(rc), H, dtype=x.dtype, device=dev)
        if n > 1:
            dist.all_to_all_single(recv, send, rc, sc)
        else:
            recv.copy_(send)
        return recv, tok, sc, rc

    def combine(y, tok, sc, rc):
        back = torch.empty(sum(sc), H, dtype=y.dtype, device=dev)
        if n > 1:
            dist.all_to_all_single(back, y, sc, rc)
        else:
            back.copy_(y)
        out = torch.zeros(S, H, dtype=torch.float32, device=dev)
        out.index_add_(0, tok, back.float())
        return out.to(torch.bfloat16)

    for _ in range(max(args.warmup, 3)):
        recv, tok, sc, rc = dispatch()
        out = combine(recv, tok, sc, rc)
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    if n > 1:
        dist.barrier(device_ids=[dev.index])
    torch.cuda.synchronize()
    with ClockSampler(dev.index) as clocks:
        for i in range(args.steps):
            flush.zero_()
            ev[i][0].record()
            recv, tok, sc, rc = dispatch()
            ev[i][1].record()
            out = combine(recv, tok, sc, rc)
            ev[i][2].record()
        torch.cuda.synchronize()
        if n > 1:
            dist.barrier(device_ids=[dev.index])
    t = [sum(e[a].elapsed_time(e[b]) for e in ev) / args.steps for a, b in ((0, 1), (1, 2), (0, 2))]
    if n > 1:
        tt = torch.tensor(t, dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t = tt.tolist()
    return {
        "metric": "ep_dispatch_combine_tokens_per_s",
        "value": n * S / (t[2] / 1e3),
        "unit": "tokens/s",
        "n_gpus": n,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": t[2],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": {"model": "NCCL all_to_all_single baseline (per-rank dedup, no balancing)", "S_per_rank": S, "H": H,
                   "K": K, "E": E, "parallelism": f"ep{n}", "routing": args.routing},
        "dispatch_us": t[0] * 1e3,
        "combine_us": t[1] * 1e3,
        "rows_sent_per_rank": int(sum(sc)),
        "clocks": clocks.summary(),
        "gpu_launches": 0,
    }  # fmt: skip
