"""Expert-parallel SwiGLU MoE layer built on ``Buffer`` and the grouped GEMM.

Forward (per rank)::

    x_nvs, w_nvs, cu, plan = buffer.dispatch(x, gates, topk, tokens_per_expert, zero_copy=True)
    buffer.prefetch_weight(plan, gate/up/down)            # hot remote experts -> local slots [E, E+B)
    h     = grouped_gemm(x_nvs, W_gate, cu, w_up=W_up, mode="swiglu")     # [NvS, I]
    y_nvs = grouped_gemm(h, W_down, cu, row_scale=w_nvs, mode="scale")    # gate weight in the epilogue
    out, _, _ = buffer.combine(plan, y_nvs, zero_copy=True)               # sum over the K experts

Backward replays the plan: ``dispatch(grad_out, plan=plan)`` brings the output gradient to the expert
rows, the expert backward runs per group, ``combine`` returns the input gradient together with the
gate gradients (through the weights channel), and ``reduce_grad`` adds the gradients of prefetched
expert copies to their owners.

Weight layout: ``W_gate, W_up: [E+B, I, H]``, ``W_down: [E+B, H, I]`` (output features x input
features, input contiguous); group ``g < E`` is expert ``g``, group ``E+b`` is the expert copied into
prefetch slot ``b``.  On multi-GPU worlds ``[:E]`` is peer mapped (``create_full_expert_weight``), so a
remote expert that did not get a prefetch slot is read in place over NVLink.

Usage pattern of the reference's Buffer API: reference ``README.md:46-48`` and ``tests/test_e2e.py:201-431``.
Every GEMM of the layer is a tcgen05 kernel of this package: forward and activation gradients on CTA pairs
(``grouped_gemm``, ``grouped_gemm_kn``), weight gradients on ``grouped_wgrad_rows``; the backward takes the weights
and activations as they are stored (MN-major tiles), the forward keeps both SwiGLU pre-activations for it.
Per-group torch matmuls remain for CPU tensors and for shapes outside the kernels' tiling.
"""

from __future__ import annotations

import torch

from .. import config
from ..api import Buffer
from ..ops.grouped_gemm import (
    kernel_supports,
    WGRAD_ACCUMULATE,
    WGRAD_STORE,
    WGRAD_STORE_NONEMPTY,
    grouped_gemm,
    grouped_gemm_kn,
    grouped_wgrad,
    kn_kernel_supports,
    WGRAD_MAX_GROUPS,
    grouped_wgrad_rows,
    wgrad_kernel_supports,
)
from ..ops.moe_ops import sgd_update, swiglu_bwd, transpose_experts
from ..parallel.symm import create_full_expert_weight, create_nvl_dist_tensor, view_nvl_dist_rows


class ExpertParallelMoE:
    def __init__(self, buffer: Buffer, inter: int, *, init_std: float = 0.02, seed: int = 0, backward_buffer: bool = True):
        """``backward_buffer`` (CUDA): a second ``Buffer`` of the same shape carries the backward pass, so the rows the
        forward dispatch delivered stay in the first one until the weight gradients need them and nothing is copied
        (about one more shard plus staging per rank).  Without it the forward keeps a copy of the dispatched rows."""
        ctx = buffer._require_ctx()
        self.buffer = buffer
        self.world = ctx["world"]
        # the copy-free path: push combine reads the expert output where it is, the backward has its own Buffer
        self.fast = bool(ctx["world"].is_cuda and ctx["_backend"].combine_mode == "push")
        self.bwd_buffer = None
        if self.fast and backward_buffer:
            self.bwd_buffer = Buffer(ctx["S"], ctx["H"], ctx["K"], ctx["E"], ctx["R"], num_sms=ctx["num_sms"],
                                     token_padding=ctx["token_padding"], B=ctx["B"], world=ctx["world"])  # fmt: skip
        self._y = None      # expert output rows [NvS, H]
        self._done = None   # per 128-row block: output tiles the down projection has finished
        self._down_calls = 0
        self.E, self.B, self.R, self.H, self.K, self.S = ctx["E"], ctx["B"], ctx["R"], ctx["H"], ctx["K"], ctx["S"]
        self.I = int(inter)
        self.rank, self.epn = ctx["rank"], ctx["epn"]
        E, B, H, I, w = self.E, self.B, self.H, self.I, self.world
        self.w_gate = create_full_expert_weight(E, B, I, H, w)
        self.w_up = create_full_expert_weight(E, B, I, H, w)
        self.w_down = create_full_expert_weight(E, B, H, I, w)
        self.mapped = w.is_cuda and not w.emulated and w.size > 1
        self.matmul_dtype = torch.bfloat16 if w.is_cuda else torch.float32
        gm = torch.full((E + B,), -1, dtype=torch.int32)
        gm[self.rank * self.epn : (self.rank + 1) * self.epn] = torch.arange(self.epn, dtype=torch.int32)
        gm[E:] = self.epn + torch.arange(B, dtype=torch.int32)
        self.group_map = gm.to(ctx["device"])  # group -> index among (own experts, prefetch slots)
        dev = ctx["device"]
        for t, (wt, shape) in enumerate(((self.w_gate, (I, H)), (self.w_up, (I, H)), (self.w_down, (H, I)))):
            for e in range(E):
                if self.mapped and e // self.epn != self.rank:
                    continue  # a peer's expert: its owner initialises it
                g = torch.Generator().manual_seed(seed * 1_000_003 + t * 10_007 + e)
                wt[e].copy_((torch.randn(*shape, generator=g) * init_std).to(torch.bfloat16).to(dev))
        # fp32 gradients of the experts this rank owns; gradients of prefetched copies are written into the
        # reduce buffers and added to their owners' gradients by reduce_grad
        n_g = self.epn
        self.g_gate = torch.zeros(n_g, I, H, dtype=torch.float32, device=dev)
        self.g_up = torch.zeros(n_g, I, H, dtype=torch.float32, device=dev)
        self.g_down = torch.zeros(n_g, H, I, dtype=torch.float32, device=dev)
        self._fresh = True
        self._red_full = [create_nvl_dist_tensor([B, d0, d1], torch.float32, w, pad_dim0=False)
                          for d0, d1 in ((I, H), (I, H), (H, I))]  # fmt: skip
        self.red = [view_nvl_dist_rows(t, self.R, B) for t in self._red_full]
        # Worlds without peer mapping (host backend, emulated ranks) keep a private copy of every expert per rank.
        # Changes of the owned experts (optimizer step, checkpoint load) are published to the other ranks' copies
        # through a symmetric staging tensor, which plays the part the peer mapping plays on real GPUs.
        self._pub = None
        if not self.mapped and self.R > 1:
            self._pub = [w.alloc_symmetric(self.epn * d0 * d1, torch.bfloat16, w.granularity())
                         for d0, d1 in ((I, H), (I, H), (H, I))]  # fmt: skip
        # per group: where its weight gradient goes (0 = nowhere: a remote expert without a prefetch slot) and how
        own0 = self.rank * self.epn
        self._wgrad_ptrs, fresh, later = [], [], []
        for t, gt in enumerate((self.g_gate, self.g_up, self.g_down)):
            ptrs = [0] * (E + B)
            for le in range(self.epn):
                ptrs[own0 + le] = gt[le].data_ptr()
            for b in range(B):
                ptrs[E + b] = self.red[t][self.rank, b].data_ptr()
            self._wgrad_ptrs.append(torch.tensor(ptrs, dtype=torch.int64).to(dev))
        for g in range(E + B):
            fresh.append(WGRAD_STORE if g < E else WGRAD_STORE_NONEMPTY)
            later.append(WGRAD_ACCUMULATE if g < E else WGRAD_STORE_NONEMPTY)
        self._wgrad_flags = {True: torch.tensor(fresh, dtype=torch.int32).to(dev),
                             False: torch.tensor(later, dtype=torch.int32).to(dev)}  # fmt: skip
        w.host_barrier()

    def destroy(self):
        """Collective: free the backward Buffer (the forward Buffer belongs to the caller)."""
        if self.bwd_buffer is not None:
            self.bwd_buffer.destroy()
            self.bwd_buffer = None

    # -- forward -------------------------------------------------------------------------------
    def _forward_fast(self, x, gates, topk, tokens_per_expert, save_for_backward):
        """CUDA: dispatch -> prefetch (on the communication stream, beside the GEMMs) -> SwiGLU GEMM -> down projection
        into a separate tensor -> push combine that reads it in place.  The GEMMs take their hand-off from the
        communication kernels tile by tile: row flags of the dispatch, per-slot flags of the prefetch (so only the
        groups that use a prefetched expert wait for it), and a per-row-block counter of finished output tiles that the
        combine's push role consumes.  Nothing is copied and nothing synchronises with the host."""
        buf = self.buffer
        x_nvs, w_nvs, cu, plan = buf.dispatch(x, gates, topk, tokens_per_expert, zero_copy=True)
        fetched = buf.prefetch_weight(plan, async_finish=True, full_gate_weight=self.w_gate,
                                      full_up_weight=self.w_up, full_down_weight=self.w_down)  # fmt: skip
        rows, dev = int(x_nvs.shape[0]), x_nvs.device
        if self._y is None:
            self._y = torch.empty(rows, self.H, dtype=torch.bfloat16, device=dev)
            self._done = torch.zeros(-(-rows // 128), dtype=torch.int32, device=dev)
        status = buf._require_ctx()["_backend"].status
        a = u = None
        if save_for_backward:
            a = torch.empty(rows, self.I, dtype=torch.bfloat16, device=dev)
            u = torch.empty_like(a)
        # the hand-off hooks need the CTA-pair kernel's tiling; other shapes run after the prefetch, in stream order
        hooked = rows >= 128 and self.H % 256 == 0 and self.I % 128 == 0
        if not hooked:
            torch.cuda.current_stream().wait_event(fetched)
        h = grouped_gemm(x_nvs, self.w_gate, cu, w_up=self.w_up, mode="swiglu", status=status,
                         save_pre=None if a is None else (a, u),
                         hooks=buf.gemm_hooks(rows=True, slots=True) if hooked else None)  # fmt: skip
        ready = None
        if hooked:
            self._down_calls += 1
            ready = (self._done, self._down_calls * 4 * (self.H // 256))
        grouped_gemm(h, self.w_down, cu, row_scale=w_nvs, mode="scale", out=self._y, status=status,
                     hooks=buf.gemm_hooks(slots=True, done_counter=self._done) if hooked else None)  # fmt: skip
        out, _, _ = buf.combine(plan, self._y, None, ready=ready)
        if hooked:
            torch.cuda.current_stream().wait_event(fetched)  # later users of the weight slots come after the copy
        if not save_for_backward:
            return out, None
        return out, {"plan": plan, "cu": cu, "x_nvs": x_nvs, "w_nvs": w_nvs, "h": h, "a": a, "u": u}

    def forward(self, x, gates, topk, tokens_per_expert, save_for_backward: bool = True):
        """Returns ``(out[S, H], saved)``.  ``save_for_backward=False`` (inference): nothing is kept, the expert
        GEMMs read the dispatched rows in place, ``saved`` is None."""
        buf = self.buffer
        if self.fast and (self.bwd_buffer is not None or not save_for_backward) and config.gemm_on_cta_pairs():
            return self._forward_fast(x, gates, topk, tokens_per_expert, save_for_backward)
        x_nvs, w_nvs, cu, plan = buf.dispatch(x, gates, topk, tokens_per_expert, zero_copy=True)
        # the weight copies run on the communication stream while this stream saves the dispatched rows
        fetched = buf.prefetch_weight(plan, async_finish=True, full_gate_weight=self.w_gate,
                                      full_up_weight=self.w_up, full_down_weight=self.w_down)  # fmt: skip
        x_saved = x_nvs.clone() if save_for_backward else x_nvs  # training: the shard is reused for the expert output
        if hasattr(fetched, "wait") and x_nvs.is_cuda:
            torch.cuda.current_stream().wait_event(fetched)
        if not save_for_backward:
            h = grouped_gemm(x_nvs, self.w_gate, cu, w_up=self.w_up, mode="swiglu")
            grouped_gemm(h, self.w_down, cu, row_scale=w_nvs, mode="scale", out=x_nvs)
            out, _, _ = buf.combine(plan, x_nvs, None, zero_copy=True)
            return out, None
        # the pre-activations are kept for the backward pass (two bf16 [NvS, I] tensors instead of two more GEMMs)
        a = torch.empty(x_saved.shape[0], self.I, dtype=torch.bfloat16, device=x_saved.device)
        u = torch.empty_like(a)
        h = grouped_gemm(x_saved, self.w_gate, cu, w_up=self.w_up, mode="swiglu", save_pre=(a, u))
        grouped_gemm(h, self.w_down, cu, row_scale=w_nvs, mode="scale", out=x_nvs)
        out, _, _ = buf.combine(plan, x_nvs, None, zero_copy=True)
        saved = {"plan": plan, "cu": cu, "x_nvs": x_saved, "w_nvs": w_nvs.clone(), "h": h, "a": a, "u": u}
        return out, saved

    # -- backward ------------------------------------------------------------------------------
    def _local_transposed(self, weights, plan):
        """K-major copies of the experts this rank owns and of its prefetch slots for the activation-gradient
        GEMMs: ``[epn+B, d1, sum(d0)]`` with the transposes of ``weights`` side by side along the last axis.
        Slots that hold no expert in this step (``experts_to_copy[rank, b] < 0``) are skipped on the device."""
        E, epn, own0, B = self.E, self.epn, self.rank * self.epn, self.B
        d1 = int(weights[0].shape[2])
        width = sum(int(w.shape[1]) for w in weights)
        out = torch.empty(epn + B, d1, width, dtype=weights[0].dtype, device=weights[0].device)
        col = 0
        for w in weights:
            transpose_experts(w[own0 : own0 + epn], out[:epn], col)
            if B:
                transpose_experts(w[E:], out[epn:], col, active=plan.experts_to_copy[self.rank])
            col += int(w.shape[1])
        return out

    def _grad_target(self, t, g):
        """Where the weight gradient of group ``g`` of tensor ``t`` goes: this rank's gradient for an owned
        expert, the reduce-buffer slot that travels to the owner for a prefetched copy."""
        epn, own0 = self.epn, self.rank * self.epn
        if g >= self.E:
            return self.red[t][self.rank, g - self.E], True
        if own0 <= g < own0 + epn:
            return (self.g_gate, self.g_up, self.g_down)[t][g - own0], False
        raise NotImplementedError(
            "a remote expert without a prefetch slot received tokens (more remote experts than B); "
            "its weight gradient has no way home — raise B"
        )

    def backward(self, saved, grad_out):
        """Returns ``(grad_x[S,H], grad_gates[S,K])`` and accumulates the weight gradients.

        The plan is replayed to bring ``grad_out`` to the expert rows.  Activation gradients multiply by the
        forward weights exactly as they are stored; weight gradients contract over the rows of a group and go
        straight into the gradient of an owned expert or into the reduce-buffer slot of a prefetched copy.  The
        pre-activations come from the forward pass.  On the kernel paths nothing synchronises with the host.
        """
        I = self.I
        # the backward Buffer (when there is one) receives the output gradient, so the forward Buffer still holds x
        buf = self.bwd_buffer if (self.bwd_buffer is not None and saved["x_nvs"].data_ptr() ==
                                  self.buffer._require_ctx()["hidden_buf_local"].data_ptr()) else self.buffer
        ctx = buf._require_ctx()
        plan, cu, x_nvs, w_nvs = saved["plan"], saved["cu"], saved["x_nvs"], saved["w_nvs"]
        dy_nvs, _, _, _ = buf.dispatch(grad_out.contiguous(), None, plan=plan, zero_copy=True)
        rows, dev = int(x_nvs.shape[0]), x_nvs.device
        g = self._times_weights(dy_nvs, [self.w_down], cu, plan)  # dL/dh before the gate weight: dy @ W_down
        dadu = torch.empty(rows, 2 * I, dtype=torch.bfloat16, device=dev)
        hsw = torch.empty(rows, I, dtype=torch.bfloat16, device=dev)
        dgate_nvs = ctx["weights_buf_local"].view(torch.float32)  # gate gradients ride the weights channel home
        swiglu_bwd(saved["a"], saved["u"], g, w_nvs, cu[-1:], dadu, hsw, dgate_nvs)
        del g
        # With MOONEP_BWD_OVERLAP=1, weight by weight: as soon as the gradients of one weight exist, its reduce_grad starts
        # on the communication stream and runs beside the GEMMs that follow, which leave the communication kernels their
        # SMs.  Otherwise one reduce_grad for all three weights follows the combine.
        reduced, grads = [], (self.g_gate, self.g_up, self.g_down)

        def reduce_one(i):
            sel = [None] * 6
            sel[i], sel[3 + i] = grads[i], self.red[i]
            reduced.append(self.buffer.reduce_grad(plan, True, *sel, owner_local=True))

        overlap = config.backward_overlap() and x_nvs.is_cuda
        sms = 0
        if overlap:
            total = torch.cuda.get_device_properties(dev).multi_processor_count
            sms = max(2, (total - int(self.buffer._require_ctx()["num_sms"])) // 2 * 2)
        if not self._weight_grads_on_kernel(x_nvs, dy_nvs, dadu, hsw, cu, after=reduce_one if overlap else None, num_sms=sms):
            self._weight_grads_per_group(x_nvs, dy_nvs, dadu, hsw, cu)
        self._times_weights(dadu, [self.w_gate, self.w_up], cu, plan, out=dy_nvs,
                            num_sms=sms if reduced else 0)  # dx rows = da Wg + du Wu
        dx, dgates, _ = buf.combine(plan, dy_nvs, dgate_nvs, zero_copy=True)
        if reduced:
            for ev in reduced:  # the gradients are complete, and the reduce slots cleared, for whatever comes next
                torch.cuda.current_stream().wait_event(ev)
        else:
            self.buffer.reduce_grad(plan, False, *grads, self.red[0], self.red[1], self.red[2], owner_local=True)
        return dx, dgates

    def _times_weights(self, x, ws, cu, plan, out=None, num_sms=0):
        """``x[rows of g] @ cat(ws, dim=1)[g]`` per group: what an activation gradient needs from forward weights
        stored ``[E+B, out, in]`` (which is ``[G, K, N]`` for this product).  The CTA-pair kernel stages them as
        MN-major tiles; elsewhere K-major copies of the local experts feed the ordinary grouped GEMM."""
        if kn_kernel_supports(x, ws):
            return grouped_gemm_kn(x, ws, cu, out=out, num_sms=num_sms)
        return grouped_gemm(x, self._local_transposed(ws, plan), cu, group_map=self.group_map, out=out,
                            status=self.buffer._require_ctx()["_backend"].status if x.is_cuda else None)

    def _weight_grads_on_kernel(self, x_nvs, dy_nvs, dadu, hsw, cu, after=None, num_sms=0) -> bool:
        """All weight gradients with three launches of the grouped tcgen05 kernel (no host synchronisation); every
        group's result goes straight to the owner's gradient or to the reduce-buffer slot of a prefetched copy.
        Returns False (nothing done) when the shapes do not fit the kernel.  ``after(i)`` is called once the
        gradients of weight ``i`` (0 gate, 1 up, 2 down) are enqueued; launches after the first such call use
        ``num_sms`` SMs."""
        I, H = self.I, self.H
        rows = int(x_nvs.shape[0]) // 64 * 64
        dev = x_nvs.device
        ok = (
            config.wgrad_on_kernel() and x_nvs.is_cuda and rows >= 64 and self.E + self.B <= WGRAD_MAX_GROUPS
            and self.buffer._require_ctx()["token_padding"] % 16 == 0
            and wgrad_kernel_supports(I, H, rows, dev) and wgrad_kernel_supports(H, I, rows, dev)
        )  # fmt: skip
        if not ok:
            return False
        flags = self._wgrad_flags[bool(self._fresh)]
        status = self.buffer._require_ctx()["_backend"].status
        ptrs = self._wgrad_ptrs
        done = after if after is not None else (lambda i: None)
        later = num_sms if after is not None else 0
        if config.wgrad_layout() == "rows":  # the kernel stages MN-major tiles: the activations as they are
            grouped_wgrad_rows(dy_nvs, hsw, cu, ptrs[2], flags, status=status)  # dW_down = dy^T (h * gate weight)
            done(2)
            grouped_wgrad_rows(dadu[:, :I], x_nvs, cu, ptrs[0], flags, status=status, num_sms=later)  # dW_gate = da^T x
            done(0)
            grouped_wgrad_rows(dadu[:, I:], x_nvs, cu, ptrs[1], flags, status=status, num_sms=later)  # dW_up   = du^T x
            done(1)
        else:  # K-major tiles from transposed copies

            def transposed(t):
                out = torch.empty(1, int(t.shape[1]), rows, dtype=torch.bfloat16, device=dev)
                return transpose_experts(t[:rows].unsqueeze(0), out)[0]

            xt, dadut, dyt, hswt = transposed(x_nvs), transposed(dadu), transposed(dy_nvs), transposed(hsw)
            grouped_wgrad(dyt, hswt, cu, ptrs[2], flags, status=status)
            done(2)
            grouped_wgrad(dadut[:I], xt, cu, ptrs[0], flags, status=status, num_sms=later)
            done(0)
            grouped_wgrad(dadut[I:], xt, cu, ptrs[1], flags, status=status, num_sms=later)
            done(1)
        self._fresh = False
        return True

    def _weight_grads_per_group(self, x_nvs, dy_nvs, dadu, hsw, cu):
        """Per-group matmuls (the CPU path, and shapes outside the kernel's tiling); reads ``cu`` on the host."""
        E, B, epn, I, md = self.E, self.B, self.epn, self.I, self.matmul_dtype
        start = 0
        visited = set()
        for grp, end in enumerate(int(v) for v in cu.tolist()):
            if end > start:
                sl = slice(start, end)
                xs, dys = x_nvs[sl].to(md), dy_nvs[sl].to(md)
                parts = (dadu[sl, :I].to(md).t() @ xs, dadu[sl, I:].to(md).t() @ xs, dys.t() @ hsw[sl].to(md))
                for t, val in enumerate(parts):
                    tgt, is_slot = self._grad_target(t, grp)
                    if is_slot or self._fresh:
                        tgt.copy_(val)
                    else:
                        tgt.add_(val)
                if grp < E:
                    visited.add(grp - self.rank * epn)
            start = max(start, end)
        assert grp == E + B - 1
        if self._fresh:  # zero_grad() only set a flag: clear the owned experts that got no rows
            for le in range(epn):
                if le not in visited:
                    for gt in (self.g_gate, self.g_up, self.g_down):
                        gt[le].zero_()
            self._fresh = False

    def check(self):
        """Synchronise and raise if a kernel of the layer's Buffers failed on the device since the last check (nothing in
        forward/backward looks at the status block, because that would synchronise with the host).  Call it once per
        step where the loop synchronises anyway, e.g. when it reads the loss."""
        self.buffer.synchronize()
        if self.bwd_buffer is not None:
            self.bwd_buffer.synchronize()

    def zero_grad(self):
        """Lazy: the next backward overwrites (instead of adding to) the gradients of the experts it visits
        and clears the others."""
        self._fresh = True

    def owner_grads(self):
        """fp32 gradients of the experts this rank owns: three tensors ``[E/R, ...]``."""
        return self.g_gate, self.g_up, self.g_down

    def sgd_step(self, lr: float):
        """Plain SGD on the owned experts (enough for a benchmark step)."""
        s = slice(self.rank * self.epn, (self.rank + 1) * self.epn)
        for w, g in ((self.w_gate, self.g_gate), (self.w_up, self.g_up), (self.w_down, self.g_down)):
            sgd_update(w[s], g, lr)
        self.publish_owned()

    def publish_owned(self):
        """Collective on worlds without peer mapping: make every rank's copy of ``w[:E]`` current after the owned
        experts changed.  On peer-mapped worlds (real GPUs) and single-rank worlds there is nothing to do."""
        if self._pub is None:
            return
        E, epn = self.E, self.epn
        own = slice(self.rank * epn, (self.rank + 1) * epn)
        weights = (self.w_gate, self.w_up, self.w_down)
        for wt, st in zip(weights, self._pub):
            st.full.view(self.R, epn, *wt.shape[1:])[self.rank].copy_(wt[own])
        self.world.host_barrier()
        for wt, st in zip(weights, self._pub):
            wt[:E].copy_(st.full.view(E, *wt.shape[1:]))
        self.world.host_barrier()


    # -- owned experts: views, checkpoints --------------------------------------------------------
    def owner_weights(self):
        """bf16 views of the experts this rank owns: three tensors ``[E/R, ...]`` inside the symmetric weights."""
        s = slice(self.rank * self.epn, (self.rank + 1) * self.epn)
        return self.w_gate[s], self.w_up[s], self.w_down[s]

    def state_dict(self) -> dict:
        """This rank's shard of the layer: the experts it owns (host copies), keyed so that a checkpoint written by
        one expert-parallel layout can be checked against another.  Every rank saves its own shard."""
        g, u, d = (t.detach().to("cpu", copy=True) for t in self.owner_weights())
        return {"format": "moonep_b200.expert_shard.v1", "rank": self.rank, "ranks": self.R, "experts": self.E,
                "first_expert": self.rank * self.epn, "hidden": self.H, "inter": self.I,
                "w_gate": g, "w_up": u, "w_down": d}  # fmt: skip

    def load_state_dict(self, state: dict) -> None:
        """Collective: every rank loads the shard it owns; peers see the new weights after the closing barrier
        (their prefetch slots are refilled by the next ``prefetch_weight``)."""
        assert state.get("format") == "moonep_b200.expert_shard.v1", "not an expert shard of this package"
        for key, mine in (("first_expert", self.rank * self.epn), ("experts", self.E), ("hidden", self.H), ("inter", self.I)):
            assert int(state[key]) == int(mine), f"checkpoint {key}={state[key]} does not match this layer ({mine})"
        for dst, key in zip(self.owner_weights(), ("w_gate", "w_up", "w_down")):
            src = state[key]
            assert tuple(src.shape) == tuple(dst.shape) and src.dtype == dst.dtype, f"{key}: shape or dtype mismatch"
            dst.copy_(src.to(dst.device))
        if self.w_gate.is_cuda:
            torch.cuda.synchronize(self.w_gate.device)
        self.world.host_barrier()
        self.publish_owned()


def dense_reference(x, gates, topk, w_gate, w_up, w_down):
    """fp32 reference of the layer on one rank's tokens: sum_k gate * FFN_{topk}(x)."""
    S, K = topk.shape
    out = torch.zeros(S, x.shape[1], dtype=torch.float32)
    for k in range(K):
        e = topk[:, k].long()
        a = torch.einsum("sh,sih->si", x, w_gate[e])
        u = torch.einsum("sh,sih->si", x, w_up[e])
        hs = torch.nn.functional.silu(a) * u
        out = out + gates[:, k, None] * torch.einsum("si,shi->sh", hs, w_down[e])
    return out
