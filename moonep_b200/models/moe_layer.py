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
The backward GEMMs run as per-group torch matmuls in this version.
"""

from __future__ import annotations

import torch

from ..api import Buffer
from ..ops.grouped_gemm import grouped_gemm
from ..parallel.symm import create_full_expert_weight, create_nvl_dist_tensor, view_nvl_dist_rows


class ExpertParallelMoE:
    def __init__(self, buffer: Buffer, inter: int, *, init_std: float = 0.02, seed: int = 0):
        ctx = buffer._require_ctx()
        self.buffer = buffer
        self.world = ctx["world"]
        self.E, self.B, self.R, self.H, self.K, self.S = ctx["E"], ctx["B"], ctx["R"], ctx["H"], ctx["K"], ctx["S"]
        self.I = int(inter)
        self.rank, self.epn = ctx["rank"], ctx["epn"]
        E, B, H, I, w = self.E, self.B, self.H, self.I, self.world
        self.w_gate = create_full_expert_weight(E, B, I, H, w)
        self.w_up = create_full_expert_weight(E, B, I, H, w)
        self.w_down = create_full_expert_weight(E, B, H, I, w)
        self.mapped = w.is_cuda and not w.emulated and w.size > 1
        self.matmul_dtype = torch.bfloat16 if w.is_cuda else torch.float32
        dev = ctx["device"]
        for t, (wt, shape) in enumerate(((self.w_gate, (I, H)), (self.w_up, (I, H)), (self.w_down, (H, I)))):
            for e in range(E):
                if self.mapped and e // self.epn != self.rank:
                    continue  # a peer's expert: its owner initialises it
                g = torch.Generator().manual_seed(seed * 1_000_003 + t * 10_007 + e)
                wt[e].copy_((torch.randn(*shape, generator=g) * init_std).to(torch.bfloat16).to(dev))
        # fp32 gradients of the groups this rank computes: its own experts [0, epn), then the B prefetch slots
        n_g = self.epn + B
        self.g_gate = torch.zeros(n_g, I, H, dtype=torch.float32, device=dev)
        self.g_up = torch.zeros(n_g, I, H, dtype=torch.float32, device=dev)
        self.g_down = torch.zeros(n_g, H, I, dtype=torch.float32, device=dev)
        self._red_full = [create_nvl_dist_tensor([B, d0, d1], torch.float32, w, pad_dim0=False)
                          for d0, d1 in ((I, H), (I, H), (H, I))]  # fmt: skip
        self.red = [view_nvl_dist_rows(t, self.R, B) for t in self._red_full]
        w.host_barrier()

    # -- forward -------------------------------------------------------------------------------
    def forward(self, x, gates, topk, tokens_per_expert):
        buf = self.buffer
        x_nvs, w_nvs, cu, plan = buf.dispatch(x, gates, topk, tokens_per_expert, zero_copy=True)
        buf.prefetch_weight(plan, full_gate_weight=self.w_gate, full_up_weight=self.w_up, full_down_weight=self.w_down)
        x_saved = x_nvs.clone()  # the shard is reused for the expert output
        h = grouped_gemm(x_saved, self.w_gate, cu, w_up=self.w_up, mode="swiglu")
        grouped_gemm(h, self.w_down, cu, row_scale=w_nvs, mode="scale", out=x_nvs)
        out, _, _ = buf.combine(plan, x_nvs, None, zero_copy=True)
        saved = {"plan": plan, "cu": cu, "x_nvs": x_saved, "w_nvs": w_nvs.clone(), "h": h}
        return out, saved

    # -- backward ------------------------------------------------------------------------------
    def backward(self, saved, grad_out):
        """Returns ``(grad_x[S,H], grad_gates[S,K])`` and accumulates the weight gradients."""
        buf, E, B = self.buffer, self.E, self.B
        plan, cu, x_nvs, w_nvs, h = saved["plan"], saved["cu"], saved["x_nvs"], saved["w_nvs"], saved["h"]
        dy_nvs, _, _, _ = buf.dispatch(grad_out.contiguous(), None, plan=plan, zero_copy=True)
        dx_nvs = dy_nvs  # rewritten in place, group by group
        dgate_nvs = torch.zeros_like(w_nvs)
        ends = cu.tolist()
        start = 0
        own0 = self.rank * self.epn
        for g in range(E + B):
            end = int(ends[g])
            if end > start:
                if g >= E:
                    gi = self.epn + (g - E)
                elif own0 <= g < own0 + self.epn:
                    gi = g - own0
                else:
                    raise NotImplementedError(
                        "a remote expert without a prefetch slot received tokens (more remote experts than B); "
                        "its weight gradient has no way home — raise B"
                    )
                md = self.matmul_dtype  # bf16 tensor-core matmuls on CUDA, fp32 on the host

                def mm(p, q):
                    return (p.to(md) @ q.to(md)).float()

                xs, dy = x_nvs[start:end], dy_nvs[start:end].float()
                wg, wu, wd = self.w_gate[g], self.w_up[g], self.w_down[g]
                a, u = mm(xs, wg.t()), mm(xs, wu.t())
                hs = torch.nn.functional.silu(a) * u
                y = mm(hs, wd.t())
                wr = w_nvs[start:end, None]
                dgate_nvs[start:end] = (dy * y).sum(dim=1)
                dys = dy * wr
                self.g_down[gi] += mm(dys.t(), hs)
                dh = mm(dys, wd)
                sig = torch.sigmoid(a)
                da = dh * u * (sig * (1 + a * (1 - sig)))
                du = dh * (a * sig)
                self.g_gate[gi] += mm(da.t(), xs)
                self.g_up[gi] += mm(du.t(), xs)
                dx_nvs[start:end] = (mm(da, wg) + mm(du, wu)).to(torch.bfloat16)
            start = max(start, end)
        dx, dgates, _ = buf.combine(plan, dx_nvs, dgate_nvs, zero_copy=False)
        # gradients of prefetched copies go home
        epn = self.epn
        for red, g in zip(self.red, (self.g_gate, self.g_up, self.g_down)):
            red[self.rank].copy_(g[epn:])
            g[epn:].zero_()
        buf.reduce_grad(plan, False, self.g_gate[:epn], self.g_up[:epn], self.g_down[:epn], self.red[0], self.red[1],
                        self.red[2], owner_local=True)  # fmt: skip
        return dx, dgates

    def zero_grad(self):
        for g in (self.g_gate, self.g_up, self.g_down):
            g.zero_()

    def owner_grads(self):
        """fp32 gradients of the experts this rank owns: three tensors ``[E/R, ...]``."""
        return self.g_gate[: self.epn], self.g_up[: self.epn], self.g_down[: self.epn]

    def sgd_step(self, lr: float):
        """Plain SGD on the owned experts (enough for a benchmark step)."""
        s = slice(self.rank * self.epn, (self.rank + 1) * self.epn)
        for w, g in ((self.w_gate, self.g_gate), (self.w_up, self.g_up), (self.w_down, self.g_down)):
            w[s].add_((-lr * g[: self.epn]).to(torch.bfloat16))


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
