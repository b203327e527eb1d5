"""Synthetic routing: who goes where, for tests and benchmarks.

``make_routing`` returns ``(topk[S,K] int32, tokens_per_expert[E] int32, gates[S,K] fp32)``.

Patterns
--------
balanced        round-robin over ranks and experts, per-rank random permutation
                of the local experts (perfectly even load).
biased          experts drawn without replacement from lognormal(sigma=bias)
                popularities shared by all ranks (seed), draws seeded per rank.
softmax         router logits ~ N(0,1) per (token, expert), top-k experts,
                gates = softmax over the chosen logits (DeepSeek-V3 style bench).
zipf            experts drawn without replacement with probability proportional
                to rank^-alpha over a seeded permutation of the experts.
all_local / all_remote / single_expert / duplicate_topk   corner cases.

Parity: reference ``tests/generate_topk_routing.py:6-40`` (balanced, biased) and
``tests/kernel_test_utils.py:76-107`` (corner-case patterns); ``softmax`` and
``zipf`` are the shapes named by the benchmark configurations.
"""

from __future__ import annotations

import torch


def make_routing(pattern, S, K, E, R, rank, *, bias=1.0, alpha=1.2, seed=42, device="cpu"):
    dev = torch.device(device)
    epn = E // R
    g_shared = torch.Generator(device="cpu").manual_seed(int(seed))
    g_local = torch.Generator(device="cpu").manual_seed(int(seed) * 1009 + int(rank) + 1)
    s = torch.arange(S)[:, None]
    k = torch.arange(K)[None, :]
    gates = None
    if pattern == "balanced":
        perm = torch.randperm(epn, generator=g_local)
        topk = ((s + k) % R) * epn + perm[((s // R) + k) % epn]
    elif pattern == "biased":
        pop = torch.exp(torch.normal(0.0, float(bias), size=(E,), generator=g_shared))
        topk = torch.multinomial(pop[None, :].expand(S, E), K, replacement=K > E, generator=g_local)
    elif pattern == "zipf":
        order = torch.randperm(E, generator=g_shared)
        pop = torch.empty(E)
        pop[order] = torch.arange(1, E + 1, dtype=torch.float32) ** (-float(alpha))
        topk = torch.multinomial(pop[None, :].expand(S, E), K, replacement=K > E, generator=g_local)
    elif pattern == "softmax":
        logits = torch.randn(S, E, generator=g_local)
        top_logits, topk = torch.topk(logits, K, dim=1)
        gates = torch.softmax(top_logits, dim=1)
    elif pattern == "all_local":
        topk = rank * epn + ((s + k) % epn)
    elif pattern == "all_remote":
        topk = ((rank + 1) % R) * epn + ((s + k) % epn)
    elif pattern == "single_expert":
        topk = torch.zeros(S, K, dtype=torch.long)
    elif pattern == "duplicate_topk":
        topk = torch.full((S, K), ((rank + 1) % R) * epn, dtype=torch.long)
    else:
        raise ValueError(f"unknown routing pattern: {pattern}")
    topk = topk.to(torch.int32).contiguous()
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    if gates is None:
        gates = torch.softmax(torch.randn(S, K, generator=g_local), dim=1)
    return topk.to(dev), tpe.to(dev), gates.to(torch.float32).contiguous().to(dev)
