"""CPU backend: every Buffer operation in plain torch/numpy on host memory.

It serves three purposes: the oracle of the CUDA kernels' tests, an emulated
multi-rank test bed that needs no GPU (``LocalWorld`` threads or gloo processes
sharing a ``/dev/shm`` mapping), and the timed CPU baseline.

The phase structure is the same as on the GPU: a phase only touches peers'
memory in ways that are safe once every rank has finished the previous phase;
``world.step()`` separates phases.

Parity (semantics): reference ``moonep_td/dispatch.py:42-117`` (row/weight push,
zero fill), ``dispatch_epilogue.py:21-40`` (duplicate expansion),
``combine_prologue.py:19-40`` (duplicate fp32 sum, bf16 rounding in place),
``combine.py:22-68`` (K-sum of primary rows, weight gather),
``prefetch.py:22-64``, ``grad_reduce.py:70-178``.
"""

from __future__ import annotations

import numpy as np
import torch

from . import planner as P


def _np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def _dup_pairs(plan):
    """(groups[ng,3], group index, position in group, duplicate row) of every duplicate row."""
    ng = int(plan.dup_counts[0])
    if ng <= 0:
        return None
    g = plan.dup_groups[:ng].to(torch.int64)
    n = g[:, 2]
    total = int(n.sum())
    seg = torch.repeat_interleave(torch.arange(ng), n)
    pos = torch.arange(total) - torch.repeat_interleave(torch.cumsum(n, 0) - n, n)
    dl = plan.dup_loffs.to(torch.int64)[g[seg, 1] + pos]
    return g, seg, pos, dl


class CpuBackend:
    name = "cpu"

    def __init__(self, ctx: dict, world):
        self.ctx = ctx
        self.world = world

    # -- views ---------------------------------------------------------------
    def _meta(self, r: int, off: int, n: int) -> torch.Tensor:
        ms = self.ctx["meta_chunk_padded"]
        return self.ctx["meta_buf"][r * ms + off : r * ms + off + n]

    def _rows(self, r: int) -> torch.Tensor:
        nvsp = self.ctx["NvS_padded"]
        return self.ctx["hidden_buf"][r * nvsp : r * nvsp + self.ctx["NvS"]]

    def destroy(self):
        pass

    # -- synchronisation -------------------------------------------------------
    def barrier(self):
        self.world.step()

    def signal(self, family: int):
        # On the host a signal followed by the matching wait is one barrier.
        self.world.step()

    def check_status(self):
        pass

    def shard_quiesced(self) -> bool:
        return False

    def stats(self) -> dict:
        return {"backend": "cpu"}

    def global_alloc(self) -> torch.Tensor:
        """``[R, E]`` int64 on the host: rows of expert e the last planning placed on rank d."""
        c = self.ctx
        return c["alloc"].cpu().to(torch.int64).view(c["R"], c["E"])

    # -- planning ------------------------------------------------------------
    def plan_publish(self, tokens_per_expert: torch.Tensor, topk_flat=None):
        c = self.ctx
        rank, R, E = c["rank"], c["R"], c["E"]
        self._meta(rank, c["SRC_INFO_OFF"], c["NvS"]).fill_(-1)
        if tokens_per_expert.dim() == 1:
            row = tokens_per_expert.reshape(-1)[:E].to(torch.int32)
            for d in range(R):
                self._meta(d, c["TPE_OFF"] + rank * E, E).copy_(row)
        self.world.step()

    def plan_compute(self, topk_flat, tokens_per_expert, cu_seqlens, plan):
        c = self.ctx
        rank, R, E, S, K, NvS = c["rank"], c["R"], c["E"], c["S"], c["K"], c["NvS"]
        if tokens_per_expert.dim() == 2:
            tpe = _np(tokens_per_expert)
        else:
            tpe = _np(self._meta(rank, c["TPE_OFF"], R * E)).reshape(R, E)
        tabs = P.global_tables(tpe, S=S, K=K, B=c["B"], token_padding=c["token_padding"], NvS=NvS)
        dst_pos = P.local_destinations(_np(topk_flat).reshape(-1), rank, tabs, NvS)
        dst = P.mark_duplicates(dst_pos, S, K, NvS)

        def put(t, a):
            t.copy_(torch.from_numpy(np.ascontiguousarray(a)).to(torch.int32).reshape(t.shape))

        put(plan.dst, dst)
        put(cu_seqlens, tabs["cu_seqlens"][rank])
        put(plan.experts_to_copy, tabs["experts_to_copy"])
        put(plan.remote_stats, tabs["remote_stats"][rank])
        put(plan.zero_fill_ranges, tabs["zero_fill"][rank])
        c["alloc"].copy_(torch.from_numpy(tabs["alloc"].T.copy()).to(torch.int32).reshape(-1))

        dest = dst_pos // NvS
        loff = dst_pos - dest * NvS
        src_val = torch.from_numpy(rank * NvS + np.arange(S * K)).to(torch.int32)
        link = torch.from_numpy(P.link_words(dst_pos, S, K, NvS)).to(torch.int32)
        loff_t = torch.from_numpy(loff)
        dest_t = torch.from_numpy(dest)
        for d in range(R):
            m = dest_t == d
            if bool(m.any()):
                self._meta(d, c["SRC_INFO_OFF"], NvS)[loff_t[m]] = src_val[m]
                self._meta(d, c["LINK_OFF"], NvS)[loff_t[m]] = link[m]
        self.world.step()

    def build_dedup(self, plan):
        c = self.ctx
        src_info = _np(self._meta(c["rank"], c["SRC_INFO_OFF"], c["NvS"]))
        g, l, n = P.build_dedup(src_info, S=c["S"], K=c["K"], NvS=c["NvS"])
        plan.dup_groups.copy_(torch.from_numpy(g).to(torch.int32))
        plan.dup_loffs.copy_(torch.from_numpy(l).to(torch.int32))
        plan.dup_counts.copy_(torch.from_numpy(n).to(torch.int32))
        if plan.src_info is not None:
            plan.src_info.copy_(self._meta(c["rank"], c["SRC_INFO_OFF"], c["NvS"]))
        if plan.link is not None:
            link = self._meta(c["rank"], c["LINK_OFF"], c["NvS"])
            plan.link.copy_(torch.where(plan.src_info >= 0, link, torch.zeros_like(link)) if plan.src_info is not None else link)

    # -- dispatch --------------------------------------------------------------
    def dispatch_send(self, hidden_sh, route_weights_sk, plan, build_dedup_map, wait=None):
        c = self.ctx
        rank, R, K, NvS = c["rank"], c["R"], c["K"], c["NvS"]
        dst = plan.dst.to(torch.int64)
        raw = torch.where(dst < 0, -dst - 1, dst)
        dest = raw // NvS
        loff = raw - dest * NvS
        token = torch.arange(dst.numel()) // K
        primary = dst >= 0
        wflat = route_weights_sk.reshape(-1) if route_weights_sk is not None else None
        for d in range(R):
            m = primary & (dest == d)
            if bool(m.any()):
                self._rows(d)[loff[m]] = hidden_sh[token[m]]
            if wflat is not None:
                m = dest == d
                if bool(m.any()):
                    self._meta(d, c["WEIGHTS_OFF"], NvS).view(torch.float32)[loff[m]] = wflat[m]
        zf = plan.zero_fill_ranges
        rows = self._rows(rank)
        wloc = self._meta(rank, c["WEIGHTS_OFF"], NvS)
        for start, n in zf[zf[:, 1] > 0].tolist():
            rows[start : start + n].zero_()
            if wflat is not None:
                wloc[start : start + n].zero_()
        if build_dedup_map:
            self.build_dedup(plan)
        self.world.step()

    def dispatch_expand(self, plan, out_hidden, out_weights, zero_copy):
        c = self.ctx
        rows = self._rows(c["rank"])
        pairs = _dup_pairs(plan)
        if pairs is not None:
            g, seg, _pos, dl = pairs
            rows[dl] = rows[g[seg, 0]]
        if not zero_copy:
            out_hidden.copy_(rows)
            if out_weights is not None:
                out_weights.copy_(self._meta(c["rank"], c["WEIGHTS_OFF"], c["NvS"]).view(torch.float32))

    # -- combine ---------------------------------------------------------------
    def combine_prologue(self, plan, hidden_nvsh, route_weights_nvs, zero_copy, wait=None):
        c = self.ctx
        rows = self._rows(c["rank"])
        if not zero_copy:
            if hidden_nvsh is not None:
                rows.copy_(hidden_nvsh)
            if route_weights_nvs is not None:
                self._meta(c["rank"], c["WEIGHTS_OFF"], c["NvS"]).copy_(route_weights_nvs.view(torch.int32))
        pairs = _dup_pairs(plan)
        if pairs is not None:
            g, seg, pos, dl = pairs
            acc = rows[g[:, 0]].float()
            for i in range(int(g[:, 2].max())):  # primary first, then duplicates in stored order, fp32
                m = pos == i
                acc.index_add_(0, seg[m], rows[dl[m]].float())
            rows[g[:, 0]] = acc.to(torch.bfloat16)
        self.world.step()

    def combine_pull(self, plan_dst, out_hidden, out_weights_sk):
        c = self.ctx
        R, S, K, NvS, H = c["R"], c["S"], c["K"], c["NvS"], c["H"]
        dst = plan_dst.to(torch.int64)
        raw = torch.where(dst < 0, -dst - 1, dst)
        dest = raw // NvS
        loff = raw - dest * NvS
        primary = (dst >= 0).view(S, K)
        gathered = torch.zeros(S * K, H, dtype=torch.float32)
        wflat = out_weights_sk.view(-1) if out_weights_sk is not None else None
        for d in range(R):
            m = (dest == d) & primary.view(-1)
            if bool(m.any()):
                gathered[m] = self._rows(d)[loff[m]].float()
            if wflat is not None:
                m = dest == d
                if bool(m.any()):
                    wflat[m] = self._meta(d, c["WEIGHTS_OFF"], NvS).view(torch.float32)[loff[m]]
        acc = torch.zeros(S, H, dtype=torch.float32)
        g3 = gathered.view(S, K, H)
        for k in range(K):  # ascending k, fp32
            acc += g3[:, k]
        out_hidden.copy_(acc.to(torch.bfloat16))

    # -- expert weights ----------------------------------------------------------
    def prefetch(self, weights, experts_to_copy):
        E, rank = self.ctx["E"], self.ctx["rank"]
        mine = experts_to_copy[rank].tolist()
        for w in weights:
            for b, e in enumerate(mine):
                if e >= 0:
                    w[E + b].copy_(w[e])

    def prefetch_launch(self, remote_experts, prefetch_buffers, experts_row):
        for src, dst in zip(remote_experts, prefetch_buffers):
            for b, e in enumerate(experts_row.tolist()):
                if e >= 0:
                    dst[b].copy_(src[e])

    def reduce_grad(self, experts_to_copy, grads, reduce_buffers, local=False):
        c = self.ctx
        E, R, rank = c["E"], c["R"], c["rank"]
        epn = E // R
        off = rank * epn if local else 0
        etc = experts_to_copy.tolist()
        Bn = experts_to_copy.shape[1]
        self.world.step()
        for grad, red in zip(grads, reduce_buffers):
            for src in range(R):
                for b in range(Bn):
                    e = etc[src][b]
                    if e >= 0 and rank * epn <= e < (rank + 1) * epn:
                        grad[e - off] += red[src, b]
        self.world.step()
        for red in reduce_buffers:
            for b in range(Bn):
                if etc[rank][b] >= 0:
                    red[rank, b].zero_()
