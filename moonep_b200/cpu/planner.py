"""Host planner: the load-balancing routing plan computed with numpy.

This is the specification the sm_100a planner kernels are tested against (exact
equality) and the planner of the CPU backend.  Every rank derives the same
global tables from the gathered ``tpe[R, E]`` counts, then places its own
``S*K`` routing entries.

Algorithm (parity: reference ``tests/planning_reference.py:33-329``)

1. ``expert_count[e] = sum_src tpe[src, e]``; ``balance[h] = tokens homed on
   rank h - CAP`` with ``CAP = S*K``.
2. Quotas ``z[h, u]``: repeatedly take the most overloaded home ``h`` (first
   index wins ties) and the emptiest rank ``u``; ``u`` is filled completely:
   ``z[h, u] = -balance[u]`` (assignment), ``balance[h] -= move``,
   ``balance[u] = 0``; stop when no home is overloaded.
3. Distribution: per home ``h``, repeatedly take the largest remaining quota
   ``d`` and the local expert with most remaining tokens, move
   ``min(remaining, quota)`` tokens of that expert from ``alloc[e, h]`` to
   ``alloc[e, d]``.  Within an expert the global token order (source rank major)
   is cut into per-destination segments in ascending destination-rank order.
4. Layout of destination ``d``: its remote experts sorted by ``(count, e)``
   descending; the first ``B`` occupy prefetch groups ``E..E+B-1``, the others
   stay in their own group ``e``.  Each non-empty group is padded to a multiple
   of ``token_padding`` rows.
5. A local entry with expert ``e`` and in-order index ``g`` among all global
   tokens of ``e`` lands on the first ``d`` with ``alloc_cumsum[e, d] > g``.
6. Later entries of one token on the same destination rank are duplicates and
   are encoded as ``-dst-1``.
"""

from __future__ import annotations

import numpy as np


def compute_quotas(group_tokens: np.ndarray, cap: int) -> np.ndarray:
    R = group_tokens.shape[0]
    balance = group_tokens.astype(np.int64) - cap
    z = np.zeros((R, R), dtype=np.int64)
    while True:
        h = int(np.argmax(balance))
        u = int(np.argmin(balance))
        if balance[h] <= 0:
            break
        move = -balance[u]
        z[h, u] = move
        balance[h] -= move
        balance[u] = 0
    return z


def distribute(expert_count: np.ndarray, z: np.ndarray, R: int) -> np.ndarray:
    E = expert_count.shape[0]
    epn = E // R
    alloc = np.zeros((E, R), dtype=np.int64)
    alloc[np.arange(E), np.arange(E) // epn] = expert_count
    for h in range(R):
        remaining = expert_count[h * epn : (h + 1) * epn].astype(np.int64).copy()
        quotas = z[h].copy()
        while True:
            d = int(np.argmax(quotas))
            if quotas[d] <= 0:
                break
            le = int(np.argmax(remaining))
            take = min(int(remaining[le]), int(quotas[d]))
            e = h * epn + le
            alloc[e, d] += take
            alloc[e, h] -= take
            remaining[le] -= take
            quotas[d] -= take
    return alloc


def layout_for_rank(alloc: np.ndarray, d: int, R: int, B: int, P: int):
    """Group layout of destination rank ``d``.

    Returns (experts_to_copy[B], n_remote, cu_seqlens[E+B], expert_off[E], zero_fill[E+B,2]).
    """
    E = alloc.shape[0]
    epn = E // R
    cnt_d = alloc[:, d]
    is_local = (np.arange(E) // epn) == d
    remote = np.nonzero((cnt_d > 0) & ~is_local)[0]
    # (count, e) descending
    order = np.lexsort((-remote, -cnt_d[remote]))
    remote = remote[order]
    picked = remote[:B]
    etc = np.full(B, -1, dtype=np.int64)
    etc[: picked.shape[0]] = picked

    group_expert = np.full(E + B, -1, dtype=np.int64)
    group_expert[:E] = np.arange(E)
    group_expert[picked] = -1
    group_expert[E : E + picked.shape[0]] = picked
    cnt = np.where(group_expert >= 0, cnt_d[np.maximum(group_expert, 0)], 0)
    padded = np.where(cnt > 0, (cnt + P - 1) // P * P, 0)
    cu = np.cumsum(padded)
    start = cu - padded
    expert_off = np.zeros(E, dtype=np.int64)
    live = cnt > 0
    expert_off[group_expert[live]] = start[live]
    zf = np.zeros((E + B, 2), dtype=np.int64)
    has_pad = live & (padded > cnt)
    zf[has_pad, 0] = (start + cnt)[has_pad]
    zf[has_pad, 1] = (padded - cnt)[has_pad]
    return etc, int(remote.shape[0]), cu, expert_off, zf


def global_tables(tpe: np.ndarray, *, S: int, K: int, B: int, token_padding: int, NvS: int) -> dict:
    """Steps 1-4: tables that are identical on every rank."""
    tpe = np.asarray(tpe, dtype=np.int64)
    R, E = tpe.shape
    epn = E // R
    cap = S * K
    tpe_cumsum = np.cumsum(tpe, axis=0)
    expert_count = tpe_cumsum[R - 1]
    group_tokens = expert_count.reshape(R, epn).sum(axis=1)
    z = compute_quotas(group_tokens, cap)
    alloc = distribute(expert_count, z, R)
    if not np.array_equal(alloc.sum(axis=1), expert_count):
        raise AssertionError("planner: per-expert token conservation failed")
    if (alloc.sum(axis=0) > cap).any():
        raise AssertionError("planner: rank capacity exceeded")

    experts_to_copy = np.full((R, B), -1, dtype=np.int64)
    remote_stats = np.zeros((R, 2), dtype=np.int64)
    cu_seqlens = np.zeros((R, E + B), dtype=np.int64)
    expert_off = np.zeros((R, E), dtype=np.int64)
    zero_fill = np.zeros((R, E + B, 2), dtype=np.int64)
    for d in range(R):
        etc, n_remote, cu, eoff, zf = layout_for_rank(alloc, d, R, B, token_padding)
        experts_to_copy[d] = etc
        remote_stats[d, 0] = n_remote
        for e in etc[etc >= 0]:
            remote_stats[e // epn, 1] += 1
        cu_seqlens[d], expert_off[d], zero_fill[d] = cu, eoff, zf
        if E + B > 0 and cu.max(initial=0) > NvS:
            raise AssertionError("planner: padded layout exceeds NvS")
    return {
        "tpe_cumsum": tpe_cumsum,
        "z": z,
        "alloc": alloc,
        "alloc_cumsum": np.cumsum(alloc, axis=1),
        "experts_to_copy": experts_to_copy,
        "remote_stats": remote_stats,
        "cu_seqlens": cu_seqlens,
        "expert_off": expert_off,
        "zero_fill": zero_fill,
    }


def in_order_rank(keys: np.ndarray) -> np.ndarray:
    """rank[i] = number of j < i with keys[j] == keys[i]."""
    n = keys.shape[0]
    if n == 0:
        return np.zeros(0, dtype=np.int64)
    perm = np.argsort(keys, kind="stable")
    sk = keys[perm]
    new_seg = np.ones(n, dtype=bool)
    new_seg[1:] = sk[1:] != sk[:-1]
    seg_start = np.maximum.accumulate(np.where(new_seg, np.arange(n), 0))
    out = np.empty(n, dtype=np.int64)
    out[perm] = np.arange(n) - seg_start
    return out


def local_destinations(topk_flat: np.ndarray, rank: int, tables: dict, NvS: int) -> np.ndarray:
    """Step 5: canonical (non-negative) dst of every local entry."""
    e = np.asarray(topk_flat, dtype=np.int64)
    tpe_cumsum = tables["tpe_cumsum"]
    alloc_cumsum = tables["alloc_cumsum"]
    R = alloc_cumsum.shape[1]
    prev = tpe_cumsum[rank - 1][e] if rank > 0 else 0
    g = prev + in_order_rank(e)
    ac = alloc_cumsum[e]  # [N, R]
    dest = (ac <= g[:, None]).sum(axis=1)
    if (dest >= R).any():
        raise AssertionError("planner: no destination rank found")
    prev_alloc = np.where(dest > 0, ac[np.arange(e.shape[0]), np.maximum(dest - 1, 0)], 0)
    return dest * NvS + tables["expert_off"][dest, e] + (g - prev_alloc)


def mark_duplicates(dst_pos: np.ndarray, S: int, K: int, NvS: int) -> np.ndarray:
    """Step 6: keep the first entry per (token, destination rank), encode the others."""
    d = dst_pos.reshape(S, K)
    dest = d // NvS
    same = dest[:, :, None] == dest[:, None, :]  # [S, k, k']
    earlier = np.tril(np.ones((K, K), dtype=bool), k=-1)  # k' < k
    is_dup = (same & earlier[None]).any(axis=2)
    return np.where(is_dup, -d - 1, d).reshape(-1)


LINK_PRIMARY = 1 << 30
LINK_HAS_NEXT = 1 << 29
LINK_ORD_SHIFT = 24  # bits 24..28 of a primary's word: its position among the primaries of its token


def link_words(dst_pos: np.ndarray, S: int, K: int, NvS: int) -> np.ndarray:
    """Per local entry, the word its source pushes beside src_info: primary bit, the position of a primary
    among the primaries of its token (ascending k), and the row of the next entry (higher k) of the same
    token on the same destination rank."""
    d = dst_pos.reshape(S, K)
    dest = d // NvS
    loff = d - dest * NvS
    same = dest[:, :, None] == dest[:, None, :]  # [S, k, k']
    earlier = np.tril(np.ones((K, K), dtype=bool), k=-1)
    later = np.triu(np.ones((K, K), dtype=bool), k=1)
    is_dup = (same & earlier[None]).any(axis=2)
    cand = same & later[None]
    has_next = cand.any(axis=2)
    nxt_k = cand.argmax(axis=2)  # first later k' on the same destination
    nxt = np.take_along_axis(loff, nxt_k, axis=1)
    ord_ = np.cumsum(~is_dup, axis=1) - 1  # primaries before k, for primaries
    words = np.where(is_dup, 0, LINK_PRIMARY | (ord_ << LINK_ORD_SHIFT)) | np.where(has_next, LINK_HAS_NEXT | nxt, 0)
    return words.reshape(-1)


def build_dedup(src_info: np.ndarray, *, S: int, K: int, NvS: int):
    """Destination side: duplicate groups from the src_info of the landed rows.

    Rows of one (source rank, token) form a group; the row with the smallest k
    is the primary, the others are listed in ascending k.
    """
    src_info = np.asarray(src_info, dtype=np.int64)
    loff = np.nonzero(src_info >= 0)[0]
    info = src_info[loff]
    src_rank = info // NvS
    slot = info - src_rank * NvS
    token = slot // K
    kidx = slot - token * K
    key = src_rank * S + token
    order = np.lexsort((kidx, key))
    key, loff = key[order], loff[order]
    n = key.shape[0]
    dup_groups = np.zeros((NvS, 3), dtype=np.int64)
    dup_loffs = np.zeros(NvS, dtype=np.int64)
    dup_counts = np.zeros(2, dtype=np.int64)
    if n == 0:
        return dup_groups, dup_loffs, dup_counts
    first = np.ones(n, dtype=bool)
    first[1:] = key[1:] != key[:-1]
    starts = np.nonzero(first)[0]
    sizes = np.diff(np.append(starts, n))
    multi = sizes > 1
    g_starts, g_sizes = starts[multi], sizes[multi]
    n_groups = g_starts.shape[0]
    dup_n = g_sizes - 1
    dup_start = np.cumsum(dup_n) - dup_n
    dup_groups[:n_groups, 0] = loff[g_starts]
    dup_groups[:n_groups, 1] = dup_start
    dup_groups[:n_groups, 2] = dup_n
    is_dup_row = ~first
    total = int(is_dup_row.sum())
    dup_loffs[:total] = loff[is_dup_row]
    dup_counts[0], dup_counts[1] = n_groups, total
    return dup_groups, dup_loffs, dup_counts
