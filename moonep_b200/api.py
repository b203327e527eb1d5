"""Public API: ``Buffer`` — load-balanced, dropless expert-parallel communication.

Typical training step::

    buf = Buffer(S=4096, H=7168, K=8, E=256, num_ep_ranks=8, num_sms=32, token_padding=128)
    x_nvs, w_nvs, cu_seqlens, plan = buf.dispatch(x, gates, topk, tokens_per_expert)
    buf.prefetch_weight(plan, full_gate_weight=wg, full_up_weight=wu, full_down_weight=wd)
    y_nvs = experts(x_nvs, cu_seqlens, ...)            # grouped GEMMs over [E+B] groups
    y, gates_back, _ = buf.combine(plan, y_nvs, w_nvs)
    # backward: dispatch(grad_y, plan=plan) -> expert backward -> combine -> reduce_grad

Parity: reference ``moonep_td/api.py:187-498`` (constructor signature, return
tuples, ``async_finish`` events, ``zero_copy`` aliasing rules, ``destroy``).
Differences by design: a fresh dispatch needs no separate inter-rank barrier
(the planner's first exchange doubles as one) and no host synchronisation happens
inside any operation.
"""

from __future__ import annotations

import logging
import warnings

import torch

from . import config
from .constants import FLAG_PLAN, FLAG_READY
from .layout import check_encoding_bounds, compute_layout
from .parallel.world import World, make_world
from .plan import MoonEPCommPlan, allocate_planning_outputs, check_plan_for_ctx, check_planning_outputs

logger = logging.getLogger(__name__)


def _create_context(S, H, K, E, num_ep_ranks, num_sms=None, token_padding=128, B=None, group=None, world=None) -> dict:
    """Allocate the symmetric buffers and local scratch of one Buffer."""
    w: World = make_world(num_ep_ranks, group=group, world=world)
    ctx = compute_layout(S, H, K, E, w.size, B=B, num_sms=num_sms, token_padding=token_padding, gran_bytes=w.granularity())
    check_encoding_bounds(ctx)
    R, rank, dev = w.size, w.rank, w.device
    ctx.update({"rank": rank, "group": group, "world": w, "device": dev})

    hid = w.alloc_symmetric(ctx["NvS_padded"] * H, torch.bfloat16, ctx["gran_bytes"])
    meta = w.alloc_symmetric(ctx["meta_chunk_padded"], torch.int32, ctx["gran_bytes"])
    ctx["_symm"] = [hid, meta]
    hidden_buf = hid.full.view(R * ctx["NvS_padded"], H)
    meta_buf = meta.full
    nvsp, ms = ctx["NvS_padded"], ctx["meta_chunk_padded"]
    # Fresh or recycled memory: clear this rank's shards so pad rows, weights
    # and flags start from zero.
    hidden_buf[rank * nvsp : (rank + 1) * nvsp].zero_()
    meta_buf[rank * ms : (rank + 1) * ms].zero_()
    ctx["hidden_buf"] = hidden_buf
    ctx["meta_buf"] = meta_buf
    ctx["hidden_buf_local"] = hidden_buf[rank * nvsp : rank * nvsp + ctx["NvS"]]
    ctx["weights_buf_local"] = meta_buf[rank * ms + ctx["WEIGHTS_OFF"] : rank * ms + ctx["WEIGHTS_OFF"] + ctx["NvS"]]

    # planner result kept for Buffer.stats: rows of expert e placed on rank d (the CUDA backend keeps its own tables)
    ctx["alloc"] = torch.empty(max(E * R, 1), dtype=torch.int32, device=dev)

    ctx["stage_buf"] = None
    if w.is_cuda and config.combine_mode() == "push" and R > 1:
        # Staging memory of the push combine: per token up to min(K, R) rows (one per destination rank), their arrival
        # flags and the K gate weights on their way home.
        from .ops import _lib

        import ctypes

        fo, wo = ctypes.c_longlong(0), ctypes.c_longlong(0)
        nbytes = int(_lib.load().moonep_stage_layout(S, K, H, ctx["Kp"], ctypes.byref(fo), ctypes.byref(wo)))
        gran = ctx["gran_bytes"]
        nbytes = (nbytes + gran - 1) // gran * gran
        stage = w.alloc_symmetric(nbytes, torch.uint8, gran)
        ctx["_symm"].append(stage)
        stage.full[rank * nbytes : (rank + 1) * nbytes].zero_()
        ctx["stage_buf"] = stage.full
        ctx["stage_chunk_bytes"], ctx["stage_flag_off"], ctx["stage_w_off"] = nbytes, int(fo.value), int(wo.value)

    if w.is_cuda:
        from .ops.cuda_backend import CudaBackend

        ctx["_backend"] = CudaBackend(ctx, w)
    else:
        from .cpu.backend import CpuBackend

        ctx["_backend"] = CpuBackend(ctx, w)
    if w.is_cuda:
        torch.cuda.synchronize(dev)
    w.host_barrier()
    return ctx


class Buffer:
    """Communication buffer of one EP rank (see module docstring)."""

    def __init__(
        self,
        S: int,
        H: int,
        K: int,
        E: int,
        num_ep_ranks: int,
        num_sms: int | None = None,
        token_padding: int = 128,
        B: int | None = None,
        group=None,
        comm_stream_priority: int = -1,
        enable_pdl: bool = True,
        explicitly_destroy: bool = False,
        *,
        world: World | None = None,
    ):
        self.explicitly_destroy = explicitly_destroy
        self.comm_stream_priority = comm_stream_priority
        self.enable_pdl = enable_pdl
        self._comm_stream = None
        self._destroyed = False
        self._ctx = _create_context(
            S, H, K, E, num_ep_ranks, num_sms=num_sms, token_padding=token_padding, B=B, group=group, world=world
        )
        w = self._ctx["world"]
        if w.is_cuda:
            max_sms = torch.cuda.get_device_properties(w.device).multi_processor_count
            # enable_pdl: the dispatch and combine kernels are launched with programmatic dependent launch, so their
            # set-up overlaps the tail of the kernel before them (the reference accepts the flag and drops it)
            self._ctx["_backend"].set_pdl(bool(enable_pdl) and config.pdl_allowed())
            self._ctx["num_sms_dedup"] = config.num_sms_dedup(max_sms)  # CTAs of the destination-side dedup/expand role
            self._ctx["_backend"].n_expand = self._ctx["num_sms_dedup"] if config.num_sms_dedup_is_set() else 0
            assert 1 <= self._ctx["num_sms"] <= max_sms, f"num_sms must be in [1, {max_sms}]"
        self._comm_stream = w.comm_stream(comm_stream_priority)

    # -- lifetime ----------------------------------------------------------------
    @property
    def destroyed(self) -> bool:
        return self._destroyed

    def _require_ctx(self) -> dict:
        assert not self._destroyed, "Buffer has been destroyed"
        return self._ctx

    def destroy(self, _collective: bool = True) -> None:
        """Collective: wait for outstanding work on every rank, then free the symmetric memory."""
        if self._destroyed:
            return
        ctx = self._ctx
        self._destroyed = True
        if ctx is None:
            return
        w = ctx["world"]
        if w.is_cuda:
            if self._comm_stream is not None:
                self._comm_stream.synchronize()
            torch.cuda.synchronize(w.device)
            try:  # a failure nobody asked about must not disappear with the Buffer
                ctx["_backend"].check_status()
            except Exception as exc:  # noqa: BLE001 - destroy() still has to free the memory on every rank
                warnings.warn(f"Buffer destroyed with an unreported device-side failure: {exc}", RuntimeWarning)
        if _collective:
            w.host_barrier()
        ctx["_backend"].destroy()
        for key in ("hidden_buf", "meta_buf", "hidden_buf_local", "weights_buf_local", "stage_buf"):
            ctx.pop(key, None)
        for st in ctx.pop("_symm", []):
            w.free_symmetric(st)
        ctx.clear()
        self._ctx = None
        self._comm_stream = None

    def __del__(self):
        if getattr(self, "_destroyed", True):
            return
        if getattr(self, "explicitly_destroy", False):
            warnings.warn("Buffer was not destroyed explicitly.", ResourceWarning)
            return
        try:
            # emulated ranks are threads of this process: the garbage collector runs on one of them and a thread
            # barrier would wait for the others forever (e.g. after a failed test), so only local cleanup here
            w = (self._ctx or {}).get("world")
            self.destroy(_collective=not getattr(w, "emulated", False))
        except Exception as exc:  # noqa: BLE001 - never raise from a destructor
            warnings.warn(f"Buffer destructor failed: {exc!r}", ResourceWarning)

    def check_status(self) -> None:
        """Raise ``MoonEPTimeoutError`` / ``MoonEPIndexError`` if a kernel of an earlier operation gave up a wait or met
        an index out of range (reads a few words from the device: synchronises).  Kernels never trap or hang: after a
        failure they record it and every later kernel of this Buffer returns at once, so **the results of all
        operations since the last successful ``check_status()`` are undefined until it passes**.  Call it where a host
        synchronisation is acceptable anyway (after the optimiser step, when a loss is read, before a checkpoint)."""
        self._require_ctx()["_backend"].check_status()

    def synchronize(self) -> None:
        """Wait for every operation of this Buffer (both streams) and raise if one of them failed on the device."""
        ctx = self._require_ctx()
        if ctx["world"].is_cuda:
            if self._comm_stream is not None:
                self._comm_stream.synchronize()
            torch.cuda.synchronize(ctx["device"])
        self.check_status()

    def stats(self, plan: MoonEPCommPlan | None = None) -> dict:
        """Runtime figures.  With ``plan``: rows this rank sends (primary entries), how many of them leave
        the rank, duplicate entries saved by per-rank dedup, rows and duplicate groups received, remote experts
        hosted here and ranks copying this rank's experts (``remote_stats``), and the load balance of the most recent
        fresh dispatch (rows per rank, max/mean with and without the planner's re-homing).  Reads the plan (synchronises).
        Always: the backend's counters (flag epochs, status block, per-call device times when profiling)."""
        ctx = self._require_ctx()
        out = dict(ctx["_backend"].stats())
        if plan is not None:
            dst = plan.dst.cpu().to(torch.int64)
            raw = torch.where(dst < 0, -dst - 1, dst)
            dest = raw // plan.NvS
            primary = dst >= 0
            rs = plan.remote_stats.cpu().tolist()
            dc = plan.dup_counts.cpu().tolist()
            out.update({
                "entries": int(dst.numel()),
                "rows_sent": int(primary.sum()),
                "rows_sent_remote": int((primary & (dest != ctx["rank"])).sum()),
                "entries_deduplicated": int((~primary).sum()),
                "dup_groups_received": int(dc[0]),
                "dup_rows_received": int(dc[1]),
                "remote_experts_hosted": int(rs[0]),
                "ranks_copying_my_experts": int(rs[1]),
                "bytes_sent_remote": int((primary & (dest != ctx["rank"])).sum()) * ctx["H"] * 2,
            })  # fmt: skip
            # load balance of the most recent fresh dispatch, from the planner's global allocation table
            R, E, epn = ctx["R"], ctx["E"], ctx["epn"]
            alloc = ctx["_backend"].global_alloc()  # [R, E]: rows of expert e placed on rank d
            per_rank = alloc.sum(dim=1)
            per_home = alloc.sum(dim=0).view(R, epn).sum(dim=1)  # rows each rank would get without re-homing
            if int(per_rank.sum()) > 0:
                mean = float(per_rank.sum()) / R
                out.update({
                    "rows_per_rank": per_rank.tolist(),
                    "imbalance": float(per_rank.max()) / mean,
                    "imbalance_without_balancing": float(per_home.max()) / mean,
                    "rows_rehomed": int((per_home - per_rank).clamp(min=0).sum()),
                })  # fmt: skip
        return out

    def gemm_hooks(self, **kw):
        """Hand-off hooks for ``ops.grouped_gemm.grouped_gemm(..., hooks=...)`` on this Buffer's shard (CUDA only; see
        ``CudaBackend.gemm_hooks``).  Returns None on the host backend."""
        be = self._require_ctx()["_backend"]
        return be.gemm_hooks(**kw) if hasattr(be, "gemm_hooks") else None

    # -- CUDA graphs ---------------------------------------------------------------
    def capture(self, fn, *, warmup: int = 1, check_every: int = 0):
        """Capture ``fn()`` — any sequence of this Buffer's operations on fixed tensors, plus whatever
        else is capturable — into a CUDA graph and return a ``CapturedStep``; ``step.replay()`` then
        runs the whole sequence with one launch.  Collective: every rank captures the same sequence and
        replays it the same number of times.  ``fn`` runs ``warmup`` times for real before the capture
        (lazy initialisation, allocator warm-up); its return value of the captured run is ``step.outputs``
        (tensors that every replay overwrites).  Ordinary calls and replays can be mixed, in stream order: wait for an
        ``async_finish`` operation of this Buffer before replaying.  A replay does not look at the device-side status
        block (that would synchronise); pass ``check_every=N`` to synchronise and raise on a failure every N replays, or
        call ``Buffer.synchronize()`` yourself.
        No counterpart in the reference, whose barriers are host-driven."""
        ctx = self._require_ctx()
        if not ctx["world"].is_cuda:
            return _EagerStep(fn)  # host backend: same interface, every replay simply runs ``fn``
        return CapturedStep(self, fn, warmup, check_every)

    # -- stream helpers ------------------------------------------------------------
    def _on_comm_stream(self, tensors, fn):
        """Run ``fn`` on the communication stream after the current stream's work; return its event."""
        comm = self._comm_stream
        if comm is None:  # CPU backend: nothing is asynchronous
            fn()
            return _DoneEvent()
        for t in tensors:
            if t is not None:
                t.record_stream(comm)
        comm.wait_event(torch.cuda.current_stream().record_event())
        with torch.cuda.stream(comm):
            fn()
            return comm.record_event()

    # -- dispatch ---------------------------------------------------------------------
    def _run_dispatch(self, ctx, hidden_sh, route_weights_sk, planning_args, plan, hidden_nvsh, route_weights_nvs,
                      *, inter_rank_sync, zero_copy):  # fmt: skip
        be = ctx["_backend"]
        if hasattr(be, "dispatch_all"):  # CUDA: fused launches (one role per phase for emulated ranks)
            be.dispatch_all(hidden_sh, route_weights_sk, plan, planning_args, inter_rank_sync)
            if not zero_copy:
                be.copy_out(hidden_nvsh, route_weights_nvs)
            return
        wait = None
        if planning_args is not None:
            topk_flat, tpe, cu_seqlens = planning_args
            be.plan_publish(tpe, topk_flat)
            be.plan_compute(topk_flat, tpe, cu_seqlens, plan)
            wait = FLAG_PLAN
        elif inter_rank_sync:
            be.signal(FLAG_READY)
            wait = FLAG_READY
        be.dispatch_send(hidden_sh, route_weights_sk, plan, planning_args is not None, wait=wait)
        be.dispatch_expand(plan, hidden_nvsh, route_weights_nvs, zero_copy)

    def dispatch(
        self,
        hidden_sh,
        route_weights_sk=None,
        topk_experts_sk=None,
        tokens_per_expert=None,
        plan=None,
        async_finish=False,
        *,
        inter_rank_sync=True,
        zero_copy=False,
    ):
        """Send every token to the ranks that will run its experts.

        Returns ``(hidden_nvsh[NvS,H], route_weights_nvs[NvS] | None, cu_seqlens[E+B] | None, plan)``
        plus a completion event if ``async_finish``.  With ``plan`` given, the
        routing of that plan is replayed (no planning, ``cu_seqlens`` is None).
        """
        ctx = self._require_ctx()
        S, H, K, NvS = ctx["S"], ctx["H"], ctx["K"], ctx["NvS"]
        dev = ctx["device"]
        assert hidden_sh.dtype == torch.bfloat16 and hidden_sh.is_contiguous(), "hidden_sh must be contiguous bf16"
        assert tuple(hidden_sh.shape) == (S, H), "hidden_sh shape mismatch"
        if route_weights_sk is not None:
            assert route_weights_sk.dtype == torch.float32 and route_weights_sk.is_contiguous(), (
                "route_weights_sk must be contiguous fp32"
            )
            assert tuple(route_weights_sk.shape) == (S, K), "route_weights_sk shape mismatch"
        if plan is None:
            assert topk_experts_sk is not None and tokens_per_expert is not None, (
                "a fresh dispatch needs topk_experts_sk and tokens_per_expert"
            )
            assert topk_experts_sk.numel() == S * K, "topk_experts_sk shape mismatch"
            topk_flat = topk_experts_sk.reshape(-1).to(torch.int32).contiguous()
            tpe = tokens_per_expert.to(torch.int32).contiguous()
            assert tpe.numel() in (ctx["E"], ctx["R"] * ctx["E"]), "tokens_per_expert must be [E] or [R, E]"
            plan, cu_seqlens = allocate_planning_outputs(ctx)
            check_planning_outputs(ctx, cu_seqlens, plan)
            planning_args = (topk_flat, tpe, cu_seqlens)
        else:
            check_plan_for_ctx(ctx, plan, dev)
            cu_seqlens, planning_args = None, None
        if zero_copy:
            hidden_nvsh = ctx["hidden_buf_local"]
            route_weights_nvs = ctx["weights_buf_local"].view(torch.float32) if route_weights_sk is not None else None
        else:
            hidden_nvsh = torch.empty(NvS, H, dtype=torch.bfloat16, device=dev)
            route_weights_nvs = (
                torch.empty(NvS, dtype=torch.float32, device=dev) if route_weights_sk is not None else None
            )

        def run():
            self._run_dispatch(
                ctx, hidden_sh, route_weights_sk, planning_args, plan, hidden_nvsh, route_weights_nvs,
                inter_rank_sync=inter_rank_sync, zero_copy=zero_copy,
            )  # fmt: skip

        if not async_finish:
            run()
            return hidden_nvsh, route_weights_nvs, cu_seqlens, plan
        tensors = [hidden_sh, route_weights_sk, hidden_nvsh, route_weights_nvs, *plan.tensors()]
        if planning_args is not None:
            tensors.extend(planning_args)
        done = self._on_comm_stream(tensors, run)
        return hidden_nvsh, route_weights_nvs, cu_seqlens, plan, done

    # -- expert weights ---------------------------------------------------------------
    def prefetch_weight(
        self, plan=None, async_finish=False, *, full_gate_weight=None, full_up_weight=None, full_down_weight=None
    ):
        """Copy the remote experts this rank was assigned into its slots ``[E, E+B)`` of each weight."""
        ctx = self._require_ctx()
        assert isinstance(plan, MoonEPCommPlan), "prefetch_weight: plan is required"
        weights = (full_gate_weight, full_up_weight, full_down_weight)
        assert all(w is not None for w in weights), "prefetch_weight needs gate, up and down weights"

        def run():
            ctx["_backend"].prefetch(weights, plan.experts_to_copy)

        if not async_finish:
            run()
            return None
        return self._on_comm_stream((plan.experts_to_copy, *weights), run)

    # -- combine ------------------------------------------------------------------------
    def _run_combine(self, ctx, hidden_sh, plan, hidden_nvsh, route_weights_nvs, route_weights_sk,
                     *, inter_rank_sync, zero_copy, ready=None):  # fmt: skip
        be = ctx["_backend"]
        if hasattr(be, "combine_all"):
            rdy, expect = ready if ready is not None else (None, 0)
            be.combine_all(plan, hidden_nvsh, route_weights_nvs, hidden_sh, route_weights_sk, inter_rank_sync, zero_copy,
                           ready=rdy, ready_expect=expect)  # fmt: skip
            return
        wait = None
        # The barrier protects the shard from being rewritten while a peer still pulls from it.  A
        # dispatch that waited for all peers since the last pull already gives that guarantee.
        if inter_rank_sync and not be.shard_quiesced():
            be.signal(FLAG_READY)
            wait = FLAG_READY
        be.combine_prologue(plan, hidden_nvsh, route_weights_nvs, zero_copy, wait=wait)
        be.combine_pull(plan.dst, hidden_sh, route_weights_sk)

    def combine(
        self,
        plan=None,
        hidden_nvsh=None,
        route_weights_nvs=None,
        async_finish=False,
        inter_rank_sync=True,
        *,
        zero_copy=False,
        ready=None,
    ):
        """Bring expert outputs home: ``out[token] = bf16(sum_k row(token, k))`` (unweighted).

        Returns ``(hidden_sh[S,H], route_weights_sk[S,K] | None, event | None)``.  ``ready=(counter, value)`` (CUDA,
        push path): ``counter[b]`` reaches ``value`` when the producer of ``hidden_nvsh`` (a grouped GEMM with a
        ``done_counter`` hook) has finished the 128-row block ``b``; rows are then taken block by block instead of
        after the whole producer.
        """
        ctx = self._require_ctx()
        S, H, K, NvS = ctx["S"], ctx["H"], ctx["K"], ctx["NvS"]
        assert isinstance(plan, MoonEPCommPlan), "Buffer.combine: plan is required"
        check_plan_for_ctx(ctx, plan, ctx["device"])
        assert hidden_nvsh is not None, "Buffer.combine: hidden_nvsh is required"
        assert hidden_nvsh.dtype == torch.bfloat16 and hidden_nvsh.is_contiguous()
        assert tuple(hidden_nvsh.shape) == (NvS, H), "hidden_nvsh shape mismatch"
        if route_weights_nvs is not None:
            assert route_weights_nvs.dtype == torch.float32 and route_weights_nvs.is_contiguous()
            assert tuple(route_weights_nvs.shape) == (NvS,), "route_weights_nvs shape mismatch"
        if zero_copy:
            assert hidden_nvsh.data_ptr() == ctx["hidden_buf_local"].data_ptr(), (
                "combine(zero_copy=True): hidden_nvsh must alias the shard view returned by dispatch(zero_copy=True)"
            )
            if route_weights_nvs is not None:
                assert route_weights_nvs.data_ptr() == ctx["weights_buf_local"].data_ptr(), (
                    "combine(zero_copy=True): route_weights_nvs must alias the weights view "
                    "returned by dispatch(zero_copy=True)"
                )
        dev = hidden_nvsh.device
        hidden_sh = torch.empty(S, H, dtype=torch.bfloat16, device=dev)
        route_weights_sk = torch.empty(S, K, dtype=torch.float32, device=dev) if route_weights_nvs is not None else None

        def run():
            self._run_combine(
                ctx, hidden_sh, plan, hidden_nvsh, route_weights_nvs, route_weights_sk,
                inter_rank_sync=inter_rank_sync, zero_copy=zero_copy, ready=ready,
            )  # fmt: skip

        if not async_finish:
            run()
            return hidden_sh, route_weights_sk, None
        done = self._on_comm_stream((hidden_sh, *plan.tensors(), hidden_nvsh, route_weights_nvs, route_weights_sk), run)
        return hidden_sh, route_weights_sk, done

    # -- gradients ----------------------------------------------------------------------
    def reduce_grad(
        self,
        plan=None,
        async_finish=False,
        full_gate_grad=None,
        full_up_grad=None,
        full_down_grad=None,
        gate_reduce_buffer=None,
        up_reduce_buffer=None,
        down_reduce_buffer=None,
        *,
        owner_local=False,
    ):
        """Add the gradients of prefetched expert copies back into their owners' gradients.

        ``full_*_grad`` are ``[>=E, H, H']`` fp32 indexed by global expert id (only this rank's experts
        are touched).  With ``owner_local=True`` they are ``[E/R, H, H']`` and hold this rank's experts
        only, which saves the memory of the other ranks' rows.  A weight whose gradient and reduce buffer are both
        ``None`` is left out (every rank must leave out the same ones), so that the weights can be reduced one by one
        as their gradients become ready.
        """
        ctx = self._require_ctx()
        assert isinstance(plan, MoonEPCommPlan), "reduce_grad: plan is required"
        pairs = [(g, b) for g, b in ((full_gate_grad, gate_reduce_buffer), (full_up_grad, up_reduce_buffer),
                                     (full_down_grad, down_reduce_buffer)) if g is not None or b is not None]  # fmt: skip
        assert pairs and all(g is not None and b is not None for g, b in pairs), \
            "reduce_grad needs a gradient together with its reduce buffer, for at least one weight"
        grads, bufs = [g for g, _ in pairs], [b for _, b in pairs]

        def run():
            E = ctx["E"]
            gs = list(grads) if owner_local else [g[:E] for g in grads]
            ctx["_backend"].reduce_grad(plan.experts_to_copy, gs, list(bufs), local=owner_local)

        if not async_finish:
            run()
            return None
        return self._on_comm_stream((plan.experts_to_copy, *grads, *bufs), run)


class CapturedStep:
    """A CUDA graph of Buffer operations (see ``Buffer.capture``)."""

    def __init__(self, buffer: Buffer, fn, warmup: int = 1, check_every: int = 0):
        self._buffer = buffer
        self.check_every = int(check_every)  # every so many replays, synchronise and raise on a device-side failure
        be = buffer._require_ctx()["_backend"]
        for _ in range(max(0, warmup)):
            fn()
        torch.cuda.synchronize(be.ctx["device"])
        buffer.check_status()
        self.graph = torch.cuda.CUDAGraph()
        be.capture_begin()
        try:
            with torch.cuda.graph(self.graph):
                self.outputs = fn()
                self._end = be.capture_end()
        except BaseException:
            be.capture_abort()
            raise
        self.replays = 0

    def replay(self):
        """Enqueue one run of the captured sequence on the current stream; returns ``outputs``."""
        be = self._buffer._require_ctx()["_backend"]
        be.replay_prepare()
        self.graph.replay()
        be.replay_done(self._end)
        self.replays += 1
        if self.check_every > 0 and self.replays % self.check_every == 0:
            self._buffer.synchronize()
        return self.outputs


class _EagerStep:
    """``CapturedStep`` interface on the CPU backend, where there is nothing to capture."""

    def __init__(self, fn):
        self._fn = fn
        self.outputs = None
        self.replays = 0

    def replay(self):
        self.outputs = self._fn()
        self.replays += 1
        return self.outputs


class _DoneEvent:
    """Stand-in for a CUDA event on the CPU backend."""

    def synchronize(self):
        pass

    def wait(self, stream=None):
        pass

    def query(self):
        return True
