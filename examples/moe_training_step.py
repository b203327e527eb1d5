"""A few training steps of one expert-parallel SwiGLU MoE layer, one process per rank.

    # CPU (gloo, host backend), two ranks:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29700 \
        examples/moe_training_step.py --backend gloo --S 64 --H 128 --I 128 --experts-per-rank 2 --K 2 --steps 2
    # GPUs (NCCL bootstrap, sm_100a kernels), eight ranks:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29700 \
        examples/moe_training_step.py --backend nccl

Every step: route the rank's tokens (softmax top-K over random logits), run the layer forward
(dispatch -> prefetch_weight -> grouped GEMMs -> combine), take a squared-error loss against a random target,
run the layer backward (plan replay, expert backward, combine, reduce_grad) and apply SGD to the owned experts.
The step's plan statistics show what load balancing and per-rank deduplication did.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moonep_b200 import Buffer  # noqa: E402
from moonep_b200.models.moe_layer import ExpertParallelMoE  # noqa: E402
from moonep_b200.models.routing import make_routing  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="nccl", choices=["nccl", "gloo"])
    ap.add_argument("--S", type=int, default=4096, help="tokens per rank")
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--I", type=int, default=2048, help="expert intermediate size")
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--experts-per-rank", type=int, default=32)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--lr", type=float, default=1e-4)
    a = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if a.backend == "nccl":
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    R = dist.get_world_size()
    E = R * a.experts_per_rank

    buf = Buffer(a.S, a.H, a.K, E, R, num_sms=32 if dev.type == "cuda" else None, token_padding=128,
                 B=min(a.experts_per_rank, 32))  # fmt: skip
    layer = ExpertParallelMoE(buf, a.I, init_std=0.02, seed=0)
    gen = torch.Generator().manual_seed(1234 + rank)
    target = (torch.randn(a.S, a.H, generator=gen) * 0.1).to(dev)

    for step in range(a.steps):
        x = (torch.randn(a.S, a.H, generator=gen) * 0.5).to(torch.bfloat16).to(dev)
        topk, tpe, gates = make_routing("softmax", a.S, a.K, E, R, rank, seed=step, device=dev)
        out, saved = layer.forward(x, gates, topk, tpe)
        diff = out.float() - target
        loss = (diff * diff).mean()
        grad_out = (2.0 / diff.numel() * diff).to(torch.bfloat16)
        dx, dgates = layer.backward(saved, grad_out)
        layer.sgd_step(a.lr)
        layer.zero_grad()
        layer.check()  # the loss is read below anyway: raise here if a kernel gave up a wait or met a bad index
        loss_all = loss.detach().clone()
        dist.all_reduce(loss_all)
        st = buf.stats(saved["plan"])
        if rank == 0:
            print(f"step {step}: mean loss {loss_all.item() / R:.5f} | rank 0 sent {st['rows_sent']} rows "
                  f"({st['rows_sent_remote']} over the network, {st['entries_deduplicated']} entries saved by dedup), "
                  f"hosts {st['remote_experts_hosted']} remote experts, |dx| {dx.float().abs().mean().item():.3e}",
                  flush=True)  # fmt: skip
    dist.barrier()
    layer.destroy()
    buf.destroy()
    dist.destroy_process_group()
    if rank == 0:
        print("done")


if __name__ == "__main__":
    main()
