"""A complete MoE block for training scripts: top-k router + expert-parallel SwiGLU experts, with autograd.

    block = MoEBlock(buffer, inter=2048, seed=0)
    y = block(x)                       # x: [S, H] bf16 tokens of this rank
    loss(y).backward()                 # input and router gradients through autograd, expert gradients in the layer
    block.experts.sgd_step(lr); block.experts.zero_grad()

``MoEFunction`` ties ``ExpertParallelMoE.forward/backward`` into autograd: the backward pass replays the plan
(``dispatch(grad, plan=plan)``), runs the expert backward, brings the input and gate gradients home with
``combine`` and calls ``reduce_grad``.  The experts' weights live in symmetric memory and their fp32 gradients in
the layer (``experts.owner_grads()``), not in autograd: they are updated with ``experts.sgd_step`` or by any
optimizer the caller writes over ``owner_grads()``.

The reference stops at the communication API; its README shows this call sequence for a training step
(reference ``README.md:46-48``).  With in-process emulated ranks on a GPU (``LocalWorld``) use the layer's explicit
``forward``/``backward`` instead: autograd runs all CUDA backward passes on one engine thread, which cannot
interleave the ranks' collective phases.
"""

from __future__ import annotations

import torch
from torch import nn

from ..api import Buffer
from .moe_layer import ExpertParallelMoE


class MoEFunction(torch.autograd.Function):
    """``out = MoEFunction.apply(x, gates, topk, tokens_per_expert, layer)``; differentiable in ``x`` and ``gates``."""

    @staticmethod
    def forward(ctx, x, gates, topk, tokens_per_expert, layer: ExpertParallelMoE):
        out, saved = layer.forward(x.detach().contiguous(), gates.detach().contiguous(), topk, tokens_per_expert)
        ctx.layer, ctx.saved = layer, saved
        return out

    @staticmethod
    def backward(ctx, grad_out):
        dx, dgates = ctx.layer.backward(ctx.saved, grad_out.contiguous().to(torch.bfloat16))
        ctx.saved = None
        return dx, dgates, None, None, None


class TopKRouter(nn.Module):
    """Softmax router: ``gates`` are the top-k probabilities renormalised to sum to one (fp32), ``topk`` the expert
    ids (int32), ``tokens_per_expert`` this rank's count per expert (int32, what the planner exchanges)."""

    def __init__(self, hidden: int, num_experts: int, k: int, *, init_std: float = 0.02, seed: int = 0, device=None):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        w = torch.randn(num_experts, hidden, generator=g) * init_std
        self.weight = nn.Parameter(w.to(device) if device is not None else w)
        self.k, self.num_experts = k, num_experts

    def forward(self, x):
        logits = x.float() @ self.weight.t()
        probs = torch.softmax(logits, dim=-1)
        top_p, top_i = torch.topk(probs, self.k, dim=-1)
        gates = top_p / top_p.sum(dim=-1, keepdim=True)
        topk = top_i.to(torch.int32)
        tpe = torch.bincount(top_i.reshape(-1), minlength=self.num_experts).to(torch.int32)
        return gates.contiguous(), topk.contiguous(), tpe


class MoEBlock(nn.Module):
    """Router + expert-parallel experts of one rank (collective: every rank of the Buffer's world calls it)."""

    def __init__(self, buffer: Buffer, inter: int, *, init_std: float = 0.02, seed: int = 0):
        super().__init__()
        ctx = buffer._require_ctx()
        self.experts = ExpertParallelMoE(buffer, inter, init_std=init_std, seed=seed)
        self.router = TopKRouter(ctx["H"], ctx["E"], ctx["K"], init_std=init_std, seed=seed + 17, device=ctx["device"])

    def forward(self, x):
        gates, topk, tpe = self.router(x)
        return MoEFunction.apply(x, gates, topk, tpe, self.experts)

    def destroy(self):
        """Collective: free what the expert layer allocated beyond the caller's Buffer."""
        self.experts.destroy()
