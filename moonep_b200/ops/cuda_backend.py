"""CUDA backend: launches the sm_100a kernels of ``libmoonep_b200.so`` for one Buffer.

Every method enqueues kernels on the current CUDA stream and returns; nothing
here synchronises with the host.  Cross-rank ordering is carried by epoch flags
in the meta chunks: ``self.epoch[family]`` counts the signals of a family, and
since all ranks issue the same sequence of operations the counters agree
without communication.  ``world.step()`` is a no-op for real multi-GPU worlds
and a thread barrier for in-process emulation (it keeps the emulated ranks'
launches in phase order on their shared stream).

Parity: plays the role of the reference's ``launch_*`` functions
(``moonep_td/dispatch.py:126``, ``combine.py:77``, ``prefetch.py:73``,
``grad_reduce.py:183``, ``_planning_gpu.py:523``).
"""

from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import config
from ..constants import (
    PLAN_BLOCK,
    FLAG_COMB,
    FLAG_GRAD_DONE,
    FLAG_GRAD_READY,
    FLAG_PLAN,
    FLAG_PREFETCH,
    FLAG_READY,
    FLAG_SENT,
    FLAG_TPE,
    NUM_FLAG_FAMILIES,
    STATUS_BAD_INDEX,
    STATUS_TIMEOUT,
)
from ..errors import MoonEPIndexError, MoonEPTimeoutError
from . import _lib

_PATHS = {"ldst": 0, "bulk": 1, "async": 2}
_KERNEL_NAMES = {
    1: "signal", 2: "plan_publish", 3: "plan_tables", 4: "plan_tokens", 5: "dispatch_send", 6: "dispatch_expand",
    7: "combine_prologue", 8: "combine_pull", 9: "prefetch", 10: "grad_accum", 11: "grad_clear", 12: "wait",
    13: "grouped_gemm", 14: "grouped_wgrad", 15: "grouped_gemm_pair", 16: "combine_push", 17: "combine_sum",
}  # fmt: skip
_PHASE_NAMES = ("tables", "tokens", "send", "zero_fill", "wait_plan", "build_expand", "wait_sent", "fold", "push", "sum")
ROLE_TABLES, ROLE_TOKENS, ROLE_SEND, ROLE_EXPAND = 1, 2, 4, 8
ROLE_PUBLISH = 32  # modifier: the launch begins with the exchange that plan_publish does as a kernel of its own
ROLE_LOCAL_ROWS = 16  # modifier: EXPAND writes the rows of this rank's own tokens from the input, SEND skips them
ROLE_PUSH, ROLE_SUM, ROLE_FOLD = 1, 2, 4
ROLE_LOCAL_HOME = 8  # modifier: rows of this rank's own tokens go from FOLD straight into the local staging chunk
_FAMILY_NAMES = {0: "READY", 1: "TPE", 2: "PLAN", 3: "SENT", 4: "COMB", 5: "GRAD_READY", 6: "GRAD_DONE", 7: "PREFETCH"}
_BIAS_OFF, _CTR_TABLES_READY = 32, 18  # words of the counters block (csrc/moonep.h)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class CudaBackend:
    name = "cuda"

    def __init__(self, ctx: dict, world):
        self.ctx = ctx
        self.world = world
        self.lib = _lib.load()
        dev = ctx["device"]
        c = ctx
        R, E, S, K, B = c["R"], c["E"], c["S"], c["K"], c["B"]
        self.epoch = [0] * NUM_FLAG_FAMILIES
        self.bias = [0] * NUM_FLAG_FAMILIES  # host mirror of the device-side epoch bias (in stream order)
        self._capture = None
        self.path = _PATHS[config.copy_path()]
        # with a single rank the send is a local copy, which all warps of a CTA share on the register path
        self.send_path = _PATHS[config.copy_path("send")] if R > 1 else _PATHS["ldst"]
        self.pull_path = _PATHS[config.copy_path("pull")]
        self.grad_path = _PATHS[config.copy_path("grad")]
        # the cp.async ring wins over NVLink (668 against 629 GB/s); on local memory the register kernel is faster
        self.prefetch_path = _PATHS[config.copy_path("prefetch")] if (R > 1 or config.copy_path_is_set("prefetch")) \
            else _PATHS["ldst"]
        self._profile = None
        self._nvtx = config.nvtx()
        self._quiesced = False  # every peer is known to be past its last pull from this rank's shard

        def i32(n):
            return torch.zeros(max(int(n), 1), dtype=torch.int32, device=dev)

        self.status = i32(8)
        self.counters = i32(64)
        self.alloc_cum = i32(E * R)
        self.expert_off = i32(R * E)
        self.tpe_prev = i32(E)
        self.tables = i32(self.lib.moonep_planner_table_words(R, E, B))
        self.stats_buf = torch.zeros(32, dtype=torch.int64, device=dev)
        tokens_per_block = max(1, PLAN_BLOCK // K)
        self.block_hist = i32(-(-S // tokens_per_block) * E)
        sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
        self.sm_count = sm_count
        # the planner's alloc[d*E+e]; only current when its tables did not fit shared memory (use global_alloc())
        c["alloc"] = self.tables[2 * E : 2 * E + R * E]
        # Emulated ranks share one GPU and one stream: a kernel of one rank must never wait for a kernel of another
        # rank that is launched later, so they run the dispatch and combine kernels one role per phase.
        self.phased = (bool(getattr(world, "emulated", False)) and world.size > 1) or config.force_phased()
        self.combine_mode = config.combine_mode()
        self.n_expand = 0  # CTAs of the dispatch kernel's destination-side role; 0 = every SM the senders leave free

        hid_base = c["hidden_buf"].data_ptr()
        meta_base = c["meta_buf"].data_ptr()
        hp = (ctypes.c_ulonglong * R)(*[hid_base + r * c["NvS_padded"] * c["H"] * 2 for r in range(R)])
        mp = (ctypes.c_ulonglong * R)(*[meta_base + r * c["meta_chunk_padded"] * 4 for r in range(R)])
        sp, flag_off, w_off = None, 0, 0
        if c.get("stage_buf") is not None:
            stage_base = c["stage_buf"].data_ptr()
            sp = (ctypes.c_ulonglong * R)(*[stage_base + r * c["stage_chunk_bytes"] for r in range(R)])
            flag_off, w_off = c["stage_flag_off"], c["stage_w_off"]
        params = [
            c["rank"], R, E, S, K, c["H"], B, c["N"], c["NvS"], c["epn"], c["token_padding"], c["num_sms"],
            c["NvS_padded"], c["meta_chunk_padded"], c["WEIGHTS_OFF"], c["TPE_OFF"], c["PLAN_OFF"], c["SRC_INFO_OFF"],
            c["SYNC_OFF"], c["R32"], c["LINK_OFF"], config.local_sms(sm_count), c["ROWFLAG_OFF"], c["Kp"],
            config.timeout_ms(), flag_off, w_off,
            self.status.data_ptr(), self.counters.data_ptr(), self.alloc_cum.data_ptr(), self.expert_off.data_ptr(),
            self.tpe_prev.data_ptr(), self.tables.data_ptr(), self.stats_buf.data_ptr(), self.block_hist.data_ptr(),
        ]  # fmt: skip
        arr = (ctypes.c_longlong * len(params))(*params)
        with torch.cuda.device(dev):
            self.handle = self.lib.moonep_ctx_create(arr, len(params), hp, mp, sp)
        if not self.handle:
            raise _lib.NativeError("moonep_ctx_create failed: " + self.lib.moonep_last_error().decode())

    # -- housekeeping ------------------------------------------------------------------
    def destroy(self):
        if self.handle:
            self.lib.moonep_ctx_destroy(self.handle)
            self.handle = None

    def set_pdl(self, on: bool):
        _lib.check(self.lib.moonep_ctx_set_pdl(self.handle, int(bool(on))), "set_pdl")

    def set_timeout_ms(self, ms: int):
        _lib.check(self.lib.moonep_ctx_set_timeout_ms(self.handle, int(ms)), "set_timeout_ms")

    def check_status(self):
        st = self.status.cpu().tolist()
        if st[0] == 0:
            return
        self.status.zero_()
        kern = _KERNEL_NAMES.get(st[1], str(st[1]))
        if st[0] == STATUS_TIMEOUT:
            raise MoonEPTimeoutError(
                f"rank {self.ctx['rank']}: kernel {kern} gave up waiting for flag "
                f"{_FAMILY_NAMES.get(st[2], st[2])} of rank {st[3]} (expected epoch {st[4]}, saw {st[5]})",
                kernel=kern, family=st[2], peer=st[3], expected=st[4], seen=st[5],
            )  # fmt: skip
        if st[0] == STATUS_BAD_INDEX:
            raise MoonEPIndexError(
                f"rank {self.ctx['rank']}: kernel {kern} met an out-of-range index (kind {st[2]}, value {st[3]}, "
                f"limit {st[4]}, at {st[5]})"
            )
        raise RuntimeError(f"unknown device status {st}")

    def stats(self) -> dict:
        out = {"backend": "cuda", "epochs": list(self.epoch), "status": self.status.cpu().tolist(),
               "native_launches_in_process": int(self.lib.moonep_launch_count()),
               "send_path": "bulk" if self.send_path else "ldst", "pull_path": "bulk" if self.pull_path else "ldst"}  # fmt: skip
        st = self.stats_buf.cpu().tolist()
        out["flag_wait_max_us"] = {_FAMILY_NAMES[f]: st[f] / 1e3 for f in _FAMILY_NAMES if st[8 + f]}
        out["flag_waits_that_spun"] = {_FAMILY_NAMES[f]: st[8 + f] for f in _FAMILY_NAMES if st[8 + f]}
        # longest duration of each phase of the dispatch / combine kernels over their CTAs since reset_wait_stats()
        out["kernel_phase_max_us"] = {name: st[16 + i] / 1e3 for i, name in enumerate(_PHASE_NAMES) if st[16 + i]}
        if self._profile:
            out["phase_times_us"] = self.phase_times()
        return out

    def global_alloc(self) -> torch.Tensor:
        """``[R, E]`` int64 on the host: rows of expert e the last planning placed on rank d.  Derived from the
        planner's inclusive prefix over destination ranks, the form it keeps in global memory (synchronises)."""
        c = self.ctx
        cum = self.alloc_cum.cpu().to(torch.int64).view(c["E"], c["R"])
        alloc = cum.clone()
        alloc[:, 1:] -= cum[:, :-1]
        return alloc.t().contiguous()

    def reset_wait_stats(self):
        self.stats_buf.zero_()

    def _next(self, family: int) -> int:
        """Advance the family's epoch; return it as a launch argument (relative to the device-side bias)."""
        self.epoch[family] += 1
        return self.epoch[family] - self.bias[family]

    def _cur(self, family: int) -> int:
        """The family's current epoch as a launch argument."""
        return self.epoch[family] - self.bias[family]

    # -- CUDA graph support ------------------------------------------------------------------
    # Kernels add a per-family bias kept in device memory to their epoch arguments.  While a graph is
    # captured the host bias is set to the current epochs, so the captured arguments are small numbers
    # relative to the capture point; the graph's last node advances the device bias by the epochs one
    # replay consumes.  Before a replay the device bias is set to the epochs reached so far (one tiny
    # launch, skipped when replays follow each other), so graph replays and ordinary calls can be mixed.
    def _bias_launch(self, values, mode):
        arr = (ctypes.c_int * NUM_FLAG_FAMILIES)(*[int(v) for v in values])
        with torch.cuda.device(self.ctx["device"]):
            _lib.check(self.lib.moonep_epoch_bias(self.handle, arr, int(mode), _stream()), "moonep_epoch_bias")

    def capture_begin(self):
        assert self._capture is None, "a capture of this Buffer is already in progress"
        assert self._profile is None, "stop profiling before capturing a graph"
        assert self.world.size == 1 or not getattr(self.world, "emulated", False), (
            "graph capture needs one process per rank (emulated ranks share a stream and cannot capture)"
        )
        self._capture = {"epoch": list(self.epoch), "bias": list(self.bias), "quiesced": self._quiesced}
        self.bias = list(self.epoch)
        self._quiesced = False  # a replay may follow anything: keep the barrier that protects the shard

    def capture_end(self):
        """Call inside the capture, after the captured work: adds the bias advance as the last graph node and
        rolls the host state back (nothing ran).  Returns what ``replay_done`` needs."""
        st = self._capture
        delta = [e - e0 for e, e0 in zip(self.epoch, st["epoch"])]
        self._bias_launch(delta, 1)
        end = {"delta": delta, "quiesced": self._quiesced}
        self.epoch, self.bias, self._quiesced = st["epoch"], st["bias"], st["quiesced"]
        self._capture = None
        return end

    def capture_abort(self):
        st = self._capture
        if st is not None:
            self.epoch, self.bias, self._quiesced = st["epoch"], st["bias"], st["quiesced"]
            self._capture = None

    def replay_prepare(self):
        if self.bias != self.epoch:
            self._bias_launch(self.epoch, 0)
            self.bias = list(self.epoch)

    def replay_done(self, end):
        for f, d in enumerate(end["delta"]):
            self.epoch[f] += d
            self.bias[f] += d
        self._quiesced = end["quiesced"]

    def _call(self, name, *args, tag=None):
        with torch.cuda.device(self.ctx["device"]):
            if self._nvtx:
                torch.cuda.nvtx.range_push(tag or name)
                try:
                    _lib.check(getattr(self.lib, name)(self.handle, *args), name)
                finally:
                    torch.cuda.nvtx.range_pop()
                return
            if self._profile is None:
                _lib.check(getattr(self.lib, name)(self.handle, *args), name)
                return
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _lib.check(getattr(self.lib, name)(self.handle, *args), name)
            e1.record()
            self._profile.append((tag or name.replace("moonep_", ""), e0, e1))

    def profile(self, on: bool = True):
        """Start (or stop) timing every native call with CUDA events; read with ``phase_times()``."""
        self._profile = [] if on else None

    def phase_times(self) -> dict:
        """Mean device time in microseconds per kind of native call since ``profile(True)``; synchronises."""
        if not self._profile:
            return {}
        torch.cuda.synchronize(self.ctx["device"])
        acc: dict[str, list[float]] = {}
        for name, e0, e1 in self._profile:
            acc.setdefault(name, []).append(e0.elapsed_time(e1) * 1e3)
        self._profile = []
        return {k: sum(v) / len(v) for k, v in acc.items()}

    # -- flags ---------------------------------------------------------------------------
    def signal(self, family: int):
        self._call("moonep_signal_wait", family, self._next(family), -1, 0, _stream())
        self.world.step()

    def wait(self, family: int):
        self._call("moonep_signal_wait", -1, 0, family, self._cur(family), _stream())

    def barrier(self):
        self.signal(FLAG_READY)
        self.wait(FLAG_READY)

    # -- planning ------------------------------------------------------------------------
    def plan_publish(self, tpe: torch.Tensor, topk_flat: torch.Tensor):
        self._topk = topk_flat
        is2d = int(tpe.dim() == 2)
        self._call("moonep_plan_publish", _ptr(self._topk), _ptr(tpe), is2d, self._next(FLAG_TPE), _stream())
        self.world.step()

    def plan_compute(self, topk_flat, tpe, cu_seqlens, plan):
        if not config.planner_on_gpu():
            return self._plan_compute_host(topk_flat, tpe, cu_seqlens, plan)
        tpe2d = _ptr(tpe) if tpe.dim() == 2 else None
        self._call(
            "moonep_plan_compute", _ptr(topk_flat), tpe2d, _ptr(plan.dst), _ptr(cu_seqlens),
            _ptr(plan.experts_to_copy), _ptr(plan.zero_fill_ranges), _ptr(plan.remote_stats), _ptr(plan.dup_counts),
            self._cur(FLAG_TPE), self._next(FLAG_PLAN), _stream(),
        )  # fmt: skip
        self.world.step()

    def _plan_compute_host(self, topk_flat, tpe, cu_seqlens, plan):
        """MOONEP_PLANNER=cpu: the host planner on device data (synchronises; for debugging)."""
        from ..cpu import planner as P

        c = self.ctx
        rank, R, E, S, K, NvS, ms = c["rank"], c["R"], c["E"], c["S"], c["K"], c["NvS"], c["meta_chunk_padded"]
        self.wait(FLAG_TPE)
        meta = c["meta_buf"]
        if tpe.dim() == 2:
            tpe_np = tpe.cpu().numpy()
        else:
            tpe_np = meta[rank * ms + c["TPE_OFF"] : rank * ms + c["TPE_OFF"] + R * E].cpu().numpy().reshape(R, E)
        tabs = P.global_tables(tpe_np, S=S, K=K, B=c["B"], token_padding=c["token_padding"], NvS=NvS)
        dst_pos = P.local_destinations(topk_flat.cpu().numpy().reshape(-1), rank, tabs, NvS)
        dst = P.mark_duplicates(dst_pos, S, K, NvS)
        dev = c["device"]

        def put(t, a):
            t.copy_(torch.from_numpy(np.ascontiguousarray(a)).to(torch.int32).reshape(t.shape).to(dev))

        put(plan.dst, dst)
        put(cu_seqlens, tabs["cu_seqlens"][rank])
        put(plan.experts_to_copy, tabs["experts_to_copy"])
        put(plan.remote_stats, tabs["remote_stats"][rank])
        put(plan.zero_fill_ranges, tabs["zero_fill"][rank])
        plan.dup_counts.zero_()
        dest = dst_pos // NvS
        loff = dst_pos - dest * NvS
        idx = torch.from_numpy(dest * ms + c["SRC_INFO_OFF"] + loff).to(dev)
        meta[idx] = torch.from_numpy(rank * NvS + np.arange(S * K)).to(torch.int32).to(dev)
        idx = torch.from_numpy(dest * ms + c["LINK_OFF"] + loff).to(dev)
        meta[idx] = torch.from_numpy(P.link_words(dst_pos, S, K, NvS)).to(torch.int32).to(dev)
        self._call("moonep_signal_wait", FLAG_PLAN, self._next(FLAG_PLAN), -1, 0, _stream())
        self.world.step()

    # -- dispatch ------------------------------------------------------------------------
    def _dispatch_launch(self, roles, fresh, plan, *, topk=None, tpe=None, cu_seqlens=None, hidden=None, weights=None,
                         with_weights=False, wait_family=-1, wait_epoch=0, epoch_sent=0, n_send=0, build_only=False,
                         tag=None):  # fmt: skip
        """One launch of the dispatch kernel with the given roles (``csrc/dispatch.cu``)."""
        tpe2d = _ptr(tpe) if (tpe is not None and tpe.dim() == 2) else None
        tpe_row = _ptr(tpe) if (tpe is not None and tpe.dim() == 1 and (roles & ROLE_PUBLISH)) else None
        self._call(
            "moonep_dispatch", int(roles), int(bool(fresh)), _ptr(topk), tpe2d, _ptr(plan.dst), _ptr(cu_seqlens),
            _ptr(plan.experts_to_copy), _ptr(plan.zero_fill_ranges), _ptr(plan.remote_stats), _ptr(hidden),
            _ptr(weights), int(bool(with_weights)), _ptr(plan.dup_groups), _ptr(plan.dup_loffs), _ptr(plan.dup_counts),
            _ptr(plan.src_info), _ptr(plan.link), int(wait_family), int(wait_epoch), self._cur(FLAG_TPE),
            self._cur(FLAG_PLAN), int(epoch_sent), self.send_path, int(n_send), int(self.n_expand), int(bool(build_only)),
            tpe_row, _stream(),
            tag=tag,
        )  # fmt: skip

    def dispatch_all(self, hidden_sh, route_weights_sk, plan, planning_args, inter_rank_sync):
        """The whole dispatch.  Fresh plan: ``plan_publish`` plus one fused launch (planner tables, token planning, row
        push, and on the destination side zero fill, duplicate map and duplicate expansion as rows arrive).  Replayed
        plan: an optional READY round plus one launch (push and expansion).  Emulated ranks run one role per phase."""
        with_w = route_weights_sk is not None
        self._sent_weights = with_w
        lr = ROLE_LOCAL_ROWS if config.local_rows_by_expand() else 0
        if planning_args is not None:
            topk_flat, tpe, cu_seqlens = planning_args
            on_dev = config.planner_on_gpu()
            # one launch for everything when nothing forces separate phases: the exchange of plan_publish becomes the
            # first step of the dispatch kernel
            fuse_publish = on_dev and not self.phased and config.fuse_plan_publish()
            if fuse_publish:
                self._topk = topk_flat
                self._next(FLAG_TPE)
            else:
                self.plan_publish(tpe, topk_flat)
            if not on_dev:
                self._plan_compute_host(topk_flat, tpe, cu_seqlens, plan)
                wf, we = FLAG_PLAN, self._cur(FLAG_PLAN)
            else:
                self._next(FLAG_PLAN)
                wf, we = -1, 0
            sent = self._next(FLAG_SENT)
            kw = dict(topk=topk_flat, tpe=tpe, cu_seqlens=cu_seqlens, hidden=hidden_sh, weights=route_weights_sk,
                      with_weights=with_w, wait_family=wf, wait_epoch=we, epoch_sent=sent)  # fmt: skip
            plan_roles = (ROLE_TABLES | ROLE_TOKENS) if on_dev else 0
            if not self.phased:
                self._dispatch_launch(plan_roles | ROLE_SEND | ROLE_EXPAND | lr | (ROLE_PUBLISH if fuse_publish else 0), True,
                                      plan, tag="dispatch_fused", **kw)
            else:
                if config.force_phased() and plan_roles:  # per-role timing: planner and send as separate launches
                    self._dispatch_launch(plan_roles, True, plan, tag="dispatch_plan", **kw)
                    self._dispatch_launch(ROLE_SEND | lr, True, plan, tag="dispatch_send", **kw)
                else:
                    self._dispatch_launch(plan_roles | ROLE_SEND | lr, True, plan, tag="dispatch_plan_send", **kw)
                self.world.step()
                self._dispatch_launch(ROLE_EXPAND | lr, True, plan, tag="dispatch_expand", **kw)
            self._quiesced = True
        else:
            wf, we = -1, 0
            if inter_rank_sync:
                self.signal(FLAG_READY)
                wf, we = FLAG_READY, self._cur(FLAG_READY)
                self._quiesced = True
            sent = self._next(FLAG_SENT)
            kw = dict(hidden=hidden_sh, weights=route_weights_sk, with_weights=with_w, wait_family=wf, wait_epoch=we,
                      epoch_sent=sent)  # fmt: skip
            if not self.phased:
                self._dispatch_launch(ROLE_SEND | ROLE_EXPAND | lr, False, plan, tag="dispatch_replay", **kw)
            else:
                self._dispatch_launch(ROLE_SEND | lr, False, plan, tag="dispatch_send", **kw)
                self.world.step()
                self._dispatch_launch(ROLE_EXPAND | lr, False, plan, tag="dispatch_expand", **kw)
        self.world.step()

    def copy_out(self, out_hidden, out_weights):
        out_hidden.copy_(self.ctx["hidden_buf_local"])
        if out_weights is not None:
            out_weights.copy_(self.ctx["weights_buf_local"].view(torch.float32))

    # launch-level stages (``ops/launch.py``)
    def dispatch_send(self, hidden_sh, route_weights_sk, plan, build_dedup_map, wait=None):
        wf = -1 if wait is None else int(wait)
        we = 0 if wait is None else self._cur(wf)
        self._dispatch_launch(ROLE_SEND, bool(build_dedup_map), plan, hidden=hidden_sh, weights=route_weights_sk,
                              with_weights=route_weights_sk is not None, wait_family=wf, wait_epoch=we,
                              epoch_sent=self._next(FLAG_SENT), tag="dispatch_send")  # fmt: skip
        if wait is not None:
            self._quiesced = True
        self._sent_weights = route_weights_sk is not None
        self.world.step()
        if build_dedup_map:
            self.build_dedup(plan)

    def build_dedup(self, plan):
        """Rebuild the plan's duplicate map (and its copies of src_info and link words) from what the last planning
        published into this rank's meta chunk."""
        self.wait(FLAG_PLAN)
        plan.dup_counts.zero_()
        self._dispatch_launch(ROLE_EXPAND, True, plan, wait_family=FLAG_PLAN, wait_epoch=self._cur(FLAG_PLAN),
                              epoch_sent=self._cur(FLAG_SENT), build_only=True, tag="dedup_builder")  # fmt: skip

    def dispatch_expand(self, plan, out_hidden, out_weights, zero_copy):
        self._dispatch_launch(ROLE_EXPAND, False, plan, with_weights=getattr(self, "_sent_weights", False),
                              epoch_sent=self._cur(FLAG_SENT), tag="dispatch_expand")  # fmt: skip
        if not zero_copy:
            self.copy_out(out_hidden, out_weights)

    # -- combine -------------------------------------------------------------------------
    def can_push(self, plan) -> bool:
        return (self.combine_mode == "push" and (self.ctx.get("stage_buf") is not None or self.ctx["R"] == 1)
                and plan.src_info is not None and plan.link is not None)  # fmt: skip

    def combine_all(self, plan, hidden_nvsh, route_weights_nvs, out_hidden, out_weights_sk, inter_rank_sync,
                    zero_copy, ready=None, ready_expect=0):  # fmt: skip
        """The whole combine.  Push path (default): the expert side folds duplicates while it pushes each token's row
        to the token's home rank, which sums rows as they land; one launch, no copy of the caller's rows into the
        shard.  Pull path (``MOONEP_COMBINE=pull`` or a plan without src_info/link): fold pass, then pull."""
        wf, we = -1, 0
        # A round of READY flags keeps a rank from overwriting staging rows (or shard rows) a peer still reads from
        # the previous combine; a dispatch that waited for all peers since then already gives that guarantee.
        if inter_rank_sync and not self._quiesced:
            self.signal(FLAG_READY)
            wf, we = FLAG_READY, self._cur(FLAG_READY)
        if not self.can_push(plan):
            self.combine_prologue(plan, hidden_nvsh, route_weights_nvs, zero_copy, wait=None if wf < 0 else wf)
            self.combine_pull(plan.dst, out_hidden, out_weights_sk)
            return
        self._quiesced = False
        comb = self._next(FLAG_COMB)
        lh = ROLE_LOCAL_HOME if config.local_home_by_fold() else 0
        fold_buf, fold_flag = self._fold_scratch()
        args = (_ptr(plan.src_info), _ptr(plan.link), _ptr(plan.dst), _ptr(hidden_nvsh), _ptr(route_weights_nvs),
                _ptr(out_hidden), _ptr(out_weights_sk), wf, we, comb, _ptr(ready), int(ready_expect),
                _ptr(plan.dup_groups), _ptr(plan.dup_loffs), _ptr(plan.dup_counts), _ptr(fold_buf), _ptr(fold_flag),
                int(fold_flag.numel()), 0, 0, _stream())  # fmt: skip
        if self.ctx["R"] == 1:  # nothing to stage: the fold role writes the results itself
            self._call("moonep_combine_push", ROLE_FOLD, *args, tag="combine_fold")
        elif not self.phased:
            self._call("moonep_combine_push", ROLE_FOLD | ROLE_PUSH | ROLE_SUM | lh, *args, tag="combine_fused")
        else:
            self._call("moonep_combine_push", ROLE_FOLD | lh, *args, tag="combine_fold")
            self._call("moonep_combine_push", ROLE_PUSH | lh, *args, tag="combine_push")
            self.world.step()
            self._call("moonep_combine_push", ROLE_SUM | lh, *args, tag="combine_sum")
        self.world.step()

    def _fold_scratch(self):
        """Local scratch of the push combine: one folded row and one flag per duplicate group (a group has at least two
        rows of the shard, so there are at most NvS/2 of them).  A single rank folds straight into the output."""
        if getattr(self, "_fold", None) is None:
            c = self.ctx
            rows = 1 if c["R"] == 1 else c["NvS"] // 2 + 1
            dev = c["device"]
            self._fold = (torch.empty(rows, c["H"], dtype=torch.bfloat16, device=dev),
                          torch.zeros(c["NvS"] // 2 + 1, dtype=torch.int32, device=dev))  # fmt: skip
        return self._fold

    def combine_prologue(self, plan, hidden_nvsh, route_weights_nvs, zero_copy, wait=None):
        wf = -1 if wait is None else int(wait)
        if not zero_copy:
            if wait is not None:
                self.wait(wf)  # peers must be done reading the shard before it is overwritten
                wf = -1
            self.ctx["hidden_buf_local"].copy_(hidden_nvsh)
            if route_weights_nvs is not None:
                self.ctx["weights_buf_local"].copy_(route_weights_nvs.view(torch.int32))
        we = 0 if wf < 0 else self._cur(wf)
        self._call(
            "moonep_combine_prologue", _ptr(plan.dup_groups), _ptr(plan.dup_loffs), _ptr(plan.dup_counts),
            None, None, wf, we, self._next(FLAG_COMB), _stream(),
        )  # fmt: skip
        self.world.step()

    def shard_quiesced(self) -> bool:
        return self._quiesced

    def combine_pull(self, plan_dst, out_hidden, out_weights_sk):
        self._quiesced = False
        self._call(
            "moonep_combine_pull", _ptr(plan_dst), _ptr(out_hidden), _ptr(out_weights_sk), self._cur(FLAG_COMB),
            self.pull_path, _stream(),
        )  # fmt: skip

    # -- expert weights --------------------------------------------------------------------
    def prefetch(self, weights, experts_to_copy):
        c = self.ctx
        E, B = c["E"], c["B"]
        ws = [w for w in weights if w is not None]
        if B == 0 or not ws or experts_to_copy.numel() == 0:
            return
        per = int(ws[0].shape[1]) * int(ws[0].shape[2])
        for w in ws:
            assert w.dtype == torch.bfloat16 and w.is_contiguous(), "weights must be contiguous bf16"
            assert w.ndim == 3 and w.shape[0] == E + B, f"weight shape {tuple(w.shape)}: dim 0 must be E+B={E + B}"
            assert int(w.shape[1]) * int(w.shape[2]) == per, "gate, up and down must have equally sized experts"
            assert w.shape[1] % 128 == 0 and w.shape[2] % 128 == 0, f"H and H' must be multiples of 128, got {tuple(w.shape[1:])}"
        assert experts_to_copy.dtype == torch.int32 and experts_to_copy.is_contiguous()
        row = experts_to_copy[c["rank"]]
        self.prefetch_launch([w[:E] for w in ws], [w[E:] for w in ws], row)

    def prefetch_launch(self, remote_experts, prefetch_buffers, experts_row):
        """Launch-level form: ``remote_experts[i]`` is ``[E', H, Hp]``, ``prefetch_buffers[i]`` ``[B', H, Hp]``."""
        n = len(remote_experts)
        nexp, H, Hp = (int(v) for v in remote_experts[0].shape)
        nslots = int(prefetch_buffers[0].shape[0])
        if nslots == 0 or experts_row.numel() == 0:
            return
        for s, d in zip(remote_experts, prefetch_buffers):
            assert s.dtype == torch.bfloat16 and s.is_contiguous() and d.dtype == torch.bfloat16 and d.is_contiguous()
            assert s.shape[0] == nexp and d.shape[0] == nslots and s.shape[1:] == d.shape[1:]
            assert int(s.shape[1]) * int(s.shape[2]) == H * Hp, "all tensors must have equally sized experts"
        assert experts_row.dtype == torch.int32 and experts_row.is_contiguous() and experts_row.numel() == nslots
        assert H % 128 == 0 and Hp % 128 == 0, f"H and H' must be multiples of 128, got ({H}, {Hp})"
        src = (ctypes.c_void_p * n)(*[t.data_ptr() for t in remote_experts])
        dst = (ctypes.c_void_p * n)(*[t.data_ptr() for t in prefetch_buffers])
        flags = done = None
        epoch = 0
        if nslots == self.ctx["B"]:  # the Buffer's own prefetch slots: per-slot flags for a GEMM that runs beside the copy
            flags, done = self._slot_scratch()
            epoch = self._next(FLAG_PREFETCH)
        self._call("moonep_prefetch", src, dst, n, _ptr(experts_row), H * Hp, nslots, nexp, self.prefetch_path, _ptr(flags),
                   _ptr(done), epoch, _stream())  # fmt: skip

    def gemm_hooks(self, *, rows=False, tables=False, slots=False, done_counter=None):
        """``GemmHooks`` for a grouped GEMM on this Buffer's shard, each part optional: ``rows`` waits per 128-row block
        for the row flags of the latest dispatch; ``tables`` delays reading ``cu_seqlens`` until that dispatch's planner
        tables are out; ``slots`` waits per prefetch slot for the latest ``prefetch_weight``; ``done_counter`` (int32
        ``[ceil(NvS / 128)]``, zero-initialised once) is bumped 4 x column tiles times per row block and call."""
        from .grouped_gemm import GemmHooks

        c, h = self.ctx, GemmHooks()
        ctr = self.counters.data_ptr()
        if rows:
            h.row_flags = c["meta_buf"].data_ptr() + 4 * (c["rank"] * c["meta_chunk_padded"] + c["ROWFLAG_OFF"])
            h.row_bias = ctr + 4 * (_BIAS_OFF + FLAG_SENT)
            h.row_epoch = self._cur(FLAG_SENT)
        if tables:
            h.tables_ready = ctr + 4 * _CTR_TABLES_READY
            h.tables_bias = ctr + 4 * (_BIAS_OFF + FLAG_PLAN)
            h.tables_epoch = self._cur(FLAG_PLAN)
        if slots and c["B"] > 0:
            h.slot_flags = self._slot_scratch()[0].data_ptr()
            h.slot_bias = ctr + 4 * (_BIAS_OFF + FLAG_PREFETCH)
            h.slot_epoch = self._cur(FLAG_PREFETCH)
            h.slot_first_group = c["E"]
        if done_counter is not None:
            assert done_counter.dtype == torch.int32 and done_counter.numel() >= -(-c["NvS"] // 128)
            h.done_counter = done_counter.data_ptr()
        return h

    def _slot_scratch(self):
        if getattr(self, "_slots", None) is None:
            dev, B = self.ctx["device"], max(1, self.ctx["B"])
            self._slots = (torch.zeros(B, dtype=torch.int32, device=dev), torch.zeros(B, dtype=torch.int32, device=dev))
        return self._slots

    def reduce_grad(self, experts_to_copy, grads, reduce_buffers, local=False):
        """``local=True``: ``grads[i]`` holds only this rank's experts, ``[E/R, H, H']``."""
        c = self.ctx
        R, E = c["R"], c["E"]
        n_grad_experts = c["epn"] if local else E
        if experts_to_copy.numel() == 0 or any(r.numel() == 0 for r in reduce_buffers):
            return
        Bc = int(experts_to_copy.shape[1])
        H, Hp = int(grads[0].shape[1]), int(grads[0].shape[2])
        assert experts_to_copy.dtype == torch.int32 and experts_to_copy.is_contiguous()
        assert tuple(experts_to_copy.shape) == (R, Bc)
        for g, r in zip(grads, reduce_buffers):
            assert g.dtype == torch.float32 and g.is_contiguous() and g.ndim == 3
            assert r.dtype == torch.float32 and r.is_contiguous() and r.ndim == 4
            assert g.shape[0] == n_grad_experts and tuple(r.shape[:2]) == (R, Bc) and g.shape[1:] == r.shape[2:]
            assert int(g.shape[1]) * int(g.shape[2]) == H * Hp, "all tensors must have equally sized experts"
            assert g.shape[1] % 128 == 0 and g.shape[2] % 128 == 0, f"H and H' must be multiples of 128, got {tuple(g.shape[1:])}"
        n = len(grads)
        # the kernel indexes gradients by global expert id but only touches this rank's experts, so an
        # owner-local tensor is passed with its base moved back by the experts of the lower ranks
        shift = c["rank"] * c["epn"] * H * Hp * 4 if local else 0
        ga = (ctypes.c_void_p * n)(*[g.data_ptr() - shift for g in grads])
        ra = (ctypes.c_void_p * n)(*[r.data_ptr() for r in reduce_buffers])
        self.signal(FLAG_GRAD_READY)
        ready, done = self._cur(FLAG_GRAD_READY), self._next(FLAG_GRAD_DONE)
        self._call("moonep_grad_reduce", ga, ra, n, _ptr(experts_to_copy), Bc, H * Hp, ready, done, 1, self.grad_path,
                   _stream(), tag="grad_accum")  # fmt: skip
        self.world.step()
        self._call("moonep_grad_reduce", ga, ra, n, _ptr(experts_to_copy), Bc, H * Hp, ready, done, 2, self.path,
                   _stream(), tag="grad_clear")  # fmt: skip
