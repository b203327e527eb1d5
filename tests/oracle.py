"""Slow, literal planner used only to cross-check the vectorised host planner on small cases.

Written with plain Python lists and explicit loops so that it shares no code (and no
vectorisation trick) with ``moonep_b200.cpu.planner``.  Semantics: reference
``tests/planning_reference.py:33-329``.
"""

from __future__ import annotations


def first_argmax(v):
    best = 0
    for i in range(1, len(v)):
        if v[i] > v[best]:
            best = i
    return best


def first_argmin(v):
    best = 0
    for i in range(1, len(v)):
        if v[i] < v[best]:
            best = i
    return best


def plan_all_ranks(topk, tpe, *, S, K, R, E, B, P, NvS):
    """topk[r] = flat list of N expert ids, tpe[r][e] counts.  Returns a dict of per-rank results."""
    epn = E // R
    cap = S * K
    count = [sum(tpe[r][e] for r in range(R)) for e in range(E)]
    balance = [sum(count[h * epn : (h + 1) * epn]) - cap for h in range(R)]
    z = [[0] * R for _ in range(R)]
    while True:
        h, u = first_argmax(balance), first_argmin(balance)
        if balance[h] <= 0:
            break
        move = -balance[u]
        z[h][u] = move
        balance[h] -= move
        balance[u] = 0
    alloc = [[0] * R for _ in range(E)]
    for e in range(E):
        alloc[e][e // epn] = count[e]
    for h in range(R):
        rem = count[h * epn : (h + 1) * epn]
        q = list(z[h])
        while True:
            d = first_argmax(q)
            if q[d] <= 0:
                break
            le = first_argmax(rem)
            take = min(rem[le], q[d])
            alloc[h * epn + le][d] += take
            alloc[h * epn + le][h] -= take
            rem[le] -= take
            q[d] -= take
    etc = [[-1] * B for _ in range(R)]
    stats = [[0, 0] for _ in range(R)]
    cu = [[0] * (E + B) for _ in range(R)]
    off = [[0] * E for _ in range(R)]
    zf = [[[0, 0] for _ in range(E + B)] for _ in range(R)]
    for d in range(R):
        remote = [e for e in range(E) if alloc[e][d] > 0 and e // epn != d]
        remote.sort(key=lambda e: (alloc[e][d], e), reverse=True)
        stats[d][0] = len(remote)
        picked = remote[:B]
        for b, e in enumerate(picked):
            etc[d][b] = e
            stats[e // epn][1] += 1
        start = 0
        for g in range(E + B):
            if g < E:
                e = g if g not in picked else -1
            else:
                e = etc[d][g - E]
            cnt = alloc[e][d] if e >= 0 else 0
            padded = -(-cnt // P) * P if cnt > 0 else 0
            if cnt > 0:
                off[d][e] = start
                if padded > cnt:
                    zf[d][g] = [start + cnt, padded - cnt]
            start += padded
            cu[d][g] = start
        assert start <= NvS
    dst = []
    for r in range(R):
        seen = [0] * E
        out = []
        for i, e in enumerate(topk[r]):
            g = sum(tpe[s][e] for s in range(r)) + seen[e]
            seen[e] += 1
            acc = 0
            for d in range(R):
                if g < acc + alloc[e][d]:
                    out.append(d * NvS + off[d][e] + g - acc)
                    break
                acc += alloc[e][d]
            else:
                raise AssertionError("no destination")
        for s in range(S):
            used = set()
            for k in range(K):
                d = out[s * K + k] // NvS
                if d in used:
                    out[s * K + k] = -out[s * K + k] - 1
                used.add(d)
        dst.append(out)
    return {"alloc": alloc, "experts_to_copy": etc, "remote_stats": stats, "cu_seqlens": cu, "zero_fill": zf, "dst": dst}
