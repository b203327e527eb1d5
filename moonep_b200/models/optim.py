"""Optimizers for the experts a rank owns.

The experts' bf16 weights live in symmetric memory (peers prefetch them), their fp32 gradients in the layer
(``ExpertParallelMoE.owner_grads()``, completed by ``reduce_grad``).  ``ExpertAdamW`` keeps fp32 master weights and
moments for the owned experts only, so optimizer state is sharded exactly like the experts, and writes the rounded
bf16 result back into the symmetric weights.  ``ExpertParallelMoE.sgd_step`` is the fused plain-SGD alternative.
The reference has no optimizer (it stops at the communication API).
"""

from __future__ import annotations

import torch

from .moe_layer import ExpertParallelMoE


class ExpertAdamW:
    def __init__(self, layer: ExpertParallelMoE, lr: float = 1e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.0):  # fmt: skip
        self.layer, self.lr, self.betas, self.eps, self.weight_decay = layer, lr, betas, eps, weight_decay
        self.master = [w.detach().float().clone() for w in layer.owner_weights()]
        self.exp_avg = [torch.zeros_like(p) for p in self.master]
        self.exp_avg_sq = [torch.zeros_like(p) for p in self.master]
        self.steps = 0

    @torch.no_grad()
    def step(self) -> None:
        """Collective on worlds without peer mapping (the new weights are published to the other ranks' copies)."""
        self.steps += 1
        b1, b2 = self.betas
        c1, c2 = 1.0 - b1**self.steps, 1.0 - b2**self.steps
        for p, g, m, v, w in zip(self.master, self.layer.owner_grads(), self.exp_avg, self.exp_avg_sq,
                                 self.layer.owner_weights()):  # fmt: skip
            if self.weight_decay:
                p.mul_(1.0 - self.lr * self.weight_decay)
            m.mul_(b1).add_(g, alpha=1.0 - b1)
            v.mul_(b2).addcmul_(g, g, value=1.0 - b2)
            p.addcdiv_(m, (v / c2).sqrt_().add_(self.eps), value=-self.lr / c1)
            w.copy_(p)
        self.layer.publish_owned()

    def zero_grad(self) -> None:
        self.layer.zero_grad()

    def state_dict(self) -> dict:
        cpu = lambda ts: [t.to("cpu", copy=True) for t in ts]  # noqa: E731
        return {"steps": self.steps, "master": cpu(self.master), "exp_avg": cpu(self.exp_avg), "exp_avg_sq": cpu(self.exp_avg_sq)}

    def load_state_dict(self, state: dict) -> None:
        self.steps = int(state["steps"])
        for name in ("master", "exp_avg", "exp_avg_sq"):
            for dst, src in zip(getattr(self, name), state[name]):
                dst.copy_(src.to(dst.device))
