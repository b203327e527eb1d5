"""Shared test machinery: cases, emulated worlds, scenario runners and checkers.

A scenario runs on a ``LocalWorld`` (R emulated ranks, one thread each) on either
``cpu`` or ``cuda``.  The CPU backend is checked against analytic properties and an
independent loop oracle; the CUDA kernels are checked against the CPU backend.

Test strategy parity: reference ``tests/kernel_test_utils.py:18-139`` (case
descriptor, routing patterns, all-rank agreement) and ``tests/test_dispatch.py:137-250``
(traceable payloads).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from moonep_b200 import Buffer
from moonep_b200.cpu import planner as P
from moonep_b200.models.routing import make_routing
from moonep_b200.parallel.world import LocalWorld


@dataclass(frozen=True)
class Case:
    name: str
    S: int
    K: int
    epn: int
    H: int
    num_sms: int = 4
    B: int | None = None
    token_padding: int = 128
    routing: str = "balanced"
    bias: float = 0.0
    seed: int = 42
    min_R: int = 1
    max_R: int | None = None

    def E(self, R):
        return R * self.epn

    def supports(self, R):
        if R < self.min_R or (self.max_R is not None and R > self.max_R):
            return False
        if self.routing in ("balanced", "biased", "zipf", "softmax") and self.K > self.E(R):
            return False
        return True


def routing_for(case: Case, R: int, rank: int, device="cpu"):
    pattern = case.routing
    return make_routing(pattern, case.S, case.K, case.E(R), R, rank, bias=case.bias or 1.0, seed=case.seed, device=device)


def make_buffers(case: Case, lw: LocalWorld):
    R = lw.size
    return lw.run(
        lambda r: Buffer(case.S, case.H, case.K, case.E(R), R, num_sms=case.num_sms, token_padding=case.token_padding,
                         B=case.B, world=lw.view(r))
    )  # fmt: skip


def destroy_buffers(lw: LocalWorld, bufs):
    lw.run(lambda r: bufs[r].destroy())


def traceable_hidden(S, H, rank, device):
    """Rows that identify (rank, token) with bf16-exact values, the rest pseudo-random small integers."""
    x = torch.zeros(S, H, dtype=torch.float32)
    tok = torch.arange(S)
    x[:, 0] = rank + 1
    if H > 1:
        x[:, 1] = tok % 128
    if H > 2:
        x[:, 2] = tok // 128
    if H > 3:
        g = torch.Generator().manual_seed(1234 + rank)
        x[:, 3:] = torch.randint(-8, 9, (S, H - 3), generator=g).float()
    return x.to(torch.bfloat16).to(device)


def traceable_weights(S, K, rank, device):
    return (rank * S * K + torch.arange(S * K, dtype=torch.float32)).view(S, K).contiguous().to(device)


def host_plan_all(case: Case, R: int, topks, tpes, lay):
    """Host planner results for every rank (numpy) from all ranks' routing."""
    tpe = np.stack([t.cpu().numpy() for t in tpes]).astype(np.int64)
    tabs = P.global_tables(tpe, S=case.S, K=case.K, B=lay["B"], token_padding=case.token_padding, NvS=lay["NvS"])
    dst_pos, dst = [], []
    for r in range(R):
        dp = P.local_destinations(topks[r].cpu().numpy().reshape(-1), r, tabs, lay["NvS"])
        dst_pos.append(dp)
        dst.append(P.mark_duplicates(dp, case.S, case.K, lay["NvS"]))
    return tabs, dst_pos, dst


def expected_src_info(R, NvS, dst_pos):
    """src_info of every destination rank from all ranks' canonical dst."""
    out = np.full((R, NvS), -1, dtype=np.int64)
    for r in range(R):
        dest = dst_pos[r] // NvS
        loff = dst_pos[r] - dest * NvS
        out[dest, loff] = r * NvS + np.arange(dst_pos[r].shape[0])
    return out


def dedup_group_map(dup_groups, dup_loffs, dup_counts, NvS):
    """{primary: sorted duplicate rows} plus structural errors; order of groups is free."""
    groups = np.asarray(dup_groups).reshape(-1, 3)
    loffs = np.asarray(dup_loffs).reshape(-1)
    ng, nd = int(dup_counts[0]), int(dup_counts[1])
    errors, mapping, seen = [], {}, []
    if not (0 <= ng <= NvS and 0 <= nd <= NvS):
        return {}, [f"counts out of range: {ng}, {nd}"]
    for g in range(ng):
        primary, ds, dn = (int(v) for v in groups[g])
        if not (0 <= primary < NvS) or dn <= 0 or ds < 0 or ds + dn > nd:
            errors.append(f"group {g} invalid: {(primary, ds, dn)}")
            continue
        dups = [int(v) for v in loffs[ds : ds + dn]]
        if primary in mapping:
            errors.append(f"primary {primary} listed twice")
        if primary in dups:
            errors.append(f"group {g} lists its own primary")
        mapping[primary] = tuple(sorted(dups))
        seen.extend(dups)
    if len(seen) != len(set(seen)):
        errors.append("a duplicate row appears twice")
    if len(seen) != nd:
        errors.append(f"duplicate count mismatch: header {nd}, used {len(seen)}")
    if set(seen) & set(mapping):
        errors.append("a row is both primary and duplicate")
    return mapping, errors


def bf16_ulp(x: torch.Tensor) -> torch.Tensor:
    ax = x.abs().float().clamp(min=2.0**-126)
    return torch.pow(2.0, torch.floor(torch.log2(ax)) - 7)


def assert_within_ulp(actual, expected, max_ulps=1, atol=0.0, what=""):
    diff = (actual.float() - expected.float()).abs()
    tol = torch.maximum(bf16_ulp(expected) * (max_ulps + 0.5), torch.full_like(diff, atol))
    bad = diff > tol
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} elements differ, max err {float(diff.max())}"


def round_trip_rank(buf, case: Case, R: int, r: int, step, *, zero_copy=False, expert_scale=None, with_weights=True,
                    poison=True, async_finish=False):  # fmt: skip
    """One rank's part of: fresh dispatch -> per-row expert function -> combine.  ``step()`` is a host
    rendezvous of all ranks (thread barrier or dist.barrier)."""
    ctx = buf._require_ctx()
    dev = ctx["device"]
    E = case.E(R)
    topk, tpe, _ = routing_for(case, R, r, device=dev)
    x = traceable_hidden(case.S, case.H, r, dev)
    w = traceable_weights(case.S, case.K, r, dev) if with_weights else None
    if poison:
        ctx["hidden_buf_local"].fill_(7.0)
        ctx["weights_buf_local"].fill_(0x55555555)
        if dev.type == "cuda":
            torch.cuda.synchronize()
        step()
    res = buf.dispatch(x, w, topk, tpe, async_finish=async_finish, zero_copy=zero_copy)
    if async_finish:
        res[-1].synchronize() if dev.type == "cpu" else torch.cuda.current_stream().wait_event(res[-1])
    xn, wn, cu, plan = res[:4]
    rec = {
        "topk": topk.cpu(), "tpe": tpe.cpu(), "x": x.cpu(), "w": None if w is None else w.cpu(),
        "hidden_nvsh": xn.detach().cpu().clone(), "weights_nvs": None if wn is None else wn.detach().cpu().clone(),
        "cu_seqlens": cu.cpu(), "dst": plan.dst.cpu(), "experts_to_copy": plan.experts_to_copy.cpu(),
        "zero_fill": plan.zero_fill_ranges.cpu(), "remote_stats": plan.remote_stats.cpu(),
        "dup_groups": plan.dup_groups.cpu(), "dup_loffs": plan.dup_loffs.cpu(), "dup_counts": plan.dup_counts.cpu(),
        "src_info": ctx["meta_buf"][r * ctx["meta_chunk_padded"] + ctx["SRC_INFO_OFF"]:][: ctx["NvS"]].cpu().clone(),
        "link": ctx["meta_buf"][r * ctx["meta_chunk_padded"] + ctx["LINK_OFF"]:][: ctx["NvS"]].cpu().clone(),
        "layout": {k: v for k, v in ctx.items() if isinstance(v, int)},
    }  # fmt: skip
    # expert stage: y = scale(row) * x, applied row-wise on the received rows
    if expert_scale is not None:
        scale = expert_scale(rec, r, E).to(dev)
        y = (xn.float() * scale[:, None]).to(torch.bfloat16)
        if zero_copy:
            xn.copy_(y)
            y = xn
    else:
        y = xn
    out, wb, ev = buf.combine(plan, y, wn, async_finish=async_finish, zero_copy=zero_copy)
    if async_finish and dev.type == "cuda":
        torch.cuda.current_stream().wait_event(ev)
    rec["out"] = out.cpu()
    rec["weights_back"] = None if wb is None else wb.cpu()
    if dev.type == "cuda":
        torch.cuda.synchronize()
        buf.check_status()
    return rec


def run_round_trip(case: Case, R: int, device: str, **kw):
    """``round_trip_rank`` on a LocalWorld; returns the per-rank records."""
    lw = LocalWorld(R, device)
    bufs = make_buffers(case, lw)
    try:
        return lw.run(lambda r: round_trip_rank(bufs[r], case, R, r, lw.view(r).step, **kw))
    finally:
        destroy_buffers(lw, bufs)


def check_dispatch_records(case: Case, R: int, recs):
    """Planner outputs, landed rows/weights, zero fill and dedup map against the host planner."""
    lay = recs[0]["layout"]
    NvS, S, K, H = lay["NvS"], case.S, case.K, case.H
    tabs, dst_pos, dst = host_plan_all(case, R, [r["topk"] for r in recs], [r["tpe"] for r in recs], lay)
    src_info = expected_src_info(R, NvS, dst_pos)
    link = np.zeros((R, NvS), dtype=np.int64)
    for r in range(R):
        link[dst_pos[r] // NvS, dst_pos[r] % NvS] = P.link_words(dst_pos[r], S, K, NvS)
    for r, rec in enumerate(recs):
        occ = src_info[r] >= 0
        assert np.array_equal(rec["link"].numpy()[occ], link[r][occ]), f"rank {r}: link words differ"
        assert np.array_equal(rec["dst"].numpy(), dst[r]), f"rank {r}: dst differs from the host planner"
        assert np.array_equal(rec["cu_seqlens"].numpy(), tabs["cu_seqlens"][r]), f"rank {r}: cu_seqlens"
        assert np.array_equal(rec["experts_to_copy"].numpy(), tabs["experts_to_copy"]), f"rank {r}: experts_to_copy"
        assert np.array_equal(rec["zero_fill"].numpy(), tabs["zero_fill"][r]), f"rank {r}: zero_fill_ranges"
        assert np.array_equal(rec["remote_stats"].numpy(), tabs["remote_stats"][r]), f"rank {r}: remote_stats"
        assert np.array_equal(rec["src_info"].numpy(), src_info[r]), f"rank {r}: src_info"
        # every landed row carries the source token; every slot its weight
        occupied = np.nonzero(src_info[r] >= 0)[0]
        info = src_info[r][occupied]
        src = info // NvS
        slot = info - src * NvS
        token = slot // K
        got = rec["hidden_nvsh"][occupied].float()
        want = torch.stack([recs[s]["x"][t] for s, t in zip(src.tolist(), token.tolist())]).float() if len(occupied) else got
        assert torch.equal(got, want), f"rank {r}: landed rows differ"
        if rec["weights_nvs"] is not None:
            gotw = rec["weights_nvs"][occupied]
            wantw = torch.tensor([float(recs[s]["w"].view(-1)[i]) for s, i in zip(src.tolist(), slot.tolist())])
            assert torch.equal(gotw, wantw), f"rank {r}: landed weights differ"
        # pad rows are zero
        for start, n in tabs["zero_fill"][r][tabs["zero_fill"][r][:, 1] > 0].tolist():
            assert not bool(rec["hidden_nvsh"][start : start + n].float().abs().max() > 0), f"rank {r}: pad rows not zero"
            if rec["weights_nvs"] is not None:
                assert not bool(rec["weights_nvs"][start : start + n].abs().max() > 0), f"rank {r}: pad weights not zero"
        # dedup map as a set of groups
        want_g, want_l, want_c = P.build_dedup(src_info[r], S=S, K=K, NvS=NvS)
        m_got, e_got = dedup_group_map(rec["dup_groups"].numpy(), rec["dup_loffs"].numpy(), rec["dup_counts"].numpy(), NvS)
        m_want, e_want = dedup_group_map(want_g, want_l, want_c, NvS)
        assert not e_got and not e_want, f"rank {r}: dedup structure errors {e_got[:3]} {e_want[:3]}"
        assert np.array_equal(rec["dup_counts"].numpy(), want_c), f"rank {r}: dup_counts"
        assert m_got == m_want, f"rank {r}: dedup groups differ"
    return tabs, dst_pos, dst, src_info


def expected_combine(case: Case, R: int, recs, dst_pos, scale_rows=None):
    """out[token] with the library's two roundings: duplicates folded to bf16, then the K-sum to bf16.

    ``scale_rows[d][loff]`` is the factor the test's expert stage applied to received row ``loff`` of rank ``d``.
    """
    NvS, S, K = recs[0]["layout"]["NvS"], case.S, case.K
    outs = []
    for r in range(R):
        x = recs[r]["x"].float()
        H = x.shape[1]
        dest = torch.from_numpy(dst_pos[r] // NvS).view(S, K)
        loff = torch.from_numpy(dst_pos[r] % NvS).view(S, K)
        contrib = x[:, None, :].expand(S, K, H).clone()
        if scale_rows is not None:
            sc = torch.stack([scale_rows[d][l] for d, l in zip(dest.view(-1).tolist(), loff.view(-1).tolist())]).view(S, K)
            contrib = (contrib * sc[:, :, None]).to(torch.bfloat16).float()
        total = torch.zeros(S, H)
        for k in range(K):  # primaries in ascending k
            primary = ~(dest[:, :k] == dest[:, k : k + 1]).any(1)
            part = torch.zeros(S, H)
            for k2 in range(k, K):  # the primary, then its duplicates in ascending k
                part += contrib[:, k2] * (dest[:, k2] == dest[:, k])[:, None]
            total += part.to(torch.bfloat16).float() * primary[:, None]
        outs.append(total.to(torch.bfloat16))
    return outs
