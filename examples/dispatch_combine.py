"""Dispatch -> (identity expert scaled by the gate weight) -> combine, one process per rank.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29701 \
        examples/dispatch_combine.py --backend gloo --S 128 --H 64 --K 4 --experts-per-rank 4
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29701 \
        examples/dispatch_combine.py --backend nccl --graph

Shows the zero-copy contract (dispatch returns views of the rank's shard; the expert stage writes its result into
the same rows; combine is given the same views), the weights channel (gate weights travel with the rows and come
back bit-exact), plan reuse (the second dispatch replays the saved plan) and, with ``--graph`` on GPUs, a CUDA graph
of the whole round trip.  ``combine`` returns the unweighted sum over a token's K rows, so an expert stage that
multiplies every row by its gate weight yields ``sum_k gate[k] * x``.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moonep_b200 import Buffer  # noqa: E402
from moonep_b200.models.routing import make_routing  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="nccl", choices=["nccl", "gloo"])
    ap.add_argument("--S", type=int, default=4096)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--experts-per-rank", type=int, default=32)
    ap.add_argument("--graph", action="store_true", help="replay the round trip as a CUDA graph (GPUs only)")
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
    buf = Buffer(a.S, a.H, a.K, E, R, num_sms=32 if dev.type == "cuda" else None, token_padding=128)
    topk, tpe, gates = make_routing("softmax", a.S, a.K, E, R, rank, seed=3, device=dev)
    x = torch.randn(a.S, a.H, generator=torch.Generator().manual_seed(rank)).to(torch.bfloat16).to(dev)

    def round_trip(plan=None):
        if plan is None:
            x_nvs, w_nvs, cu_seqlens, plan = buf.dispatch(x, gates, topk, tpe, zero_copy=True)
        else:  # replay: no planning, cu_seqlens is None
            x_nvs, w_nvs, _, plan = buf.dispatch(x, gates, plan=plan, zero_copy=True)
        x_nvs.copy_((x_nvs.float() * w_nvs[:, None]).to(torch.bfloat16))  # the "expert": scale each row by its gate weight
        out, gates_back, _ = buf.combine(plan, x_nvs, w_nvs, zero_copy=True)
        return out, gates_back, plan

    out, gates_back, plan = round_trip()
    saved = plan.clone()
    out2, _, _ = round_trip(saved)
    want = (x.float() * gates.sum(dim=1, keepdim=True)).to(torch.bfloat16)
    err = (out.float() - want.float()).abs().max().item()
    same = bool(torch.equal(out, out2)) and bool(torch.equal(gates_back, gates))
    if a.graph and dev.type == "cuda":
        step = buf.capture(lambda: round_trip()[0])
        x.copy_(-x)
        out3 = step.replay()
        torch.cuda.synchronize()
        buf.check_status()
        same = same and bool(torch.equal(out3, (-out.float()).to(torch.bfloat16)))
    ok = torch.tensor([1.0 if (same and err < 0.1) else 0.0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"max |out - sum_k gate*x| = {err:.4f}; plan replay and gate weights bit-exact: {same}; all ranks ok: {bool(ok.item())}")
    buf.destroy()
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
