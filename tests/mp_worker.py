"""Multi-process worker: one EP rank per process over torch.distributed.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node R --master-addr 127.0.0.1 \
        --master-port P tests/mp_worker.py --backend gloo|nccl

gloo: CPU backend with /dev/shm symmetric memory.  nccl: the sm_100a kernels on real
peer-mapped (CUDA VMM) memory, one GPU per rank.  Every rank gathers all ranks' records and
runs the same checks, so a failure shows on all ranks (parity: reference
tests/kernel_test_utils.py:116-139).  Prints ``WORKER OK`` per rank on success.
"""

from __future__ import annotations

import argparse
import dataclasses
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moonep_b200 import Buffer  # noqa: E402
from moonep_b200.parallel.symm import (  # noqa: E402
    create_full_expert_weight,
    create_nvl_dist_tensor,
    release_nvl_dist_tensor,
    view_nvl_dist_rows,
)
from tests.cases import ROUNDTRIP_CASES  # noqa: E402
from tests.harness import (  # noqa: E402
    Case,
    assert_within_ulp,
    check_dispatch_records,
    expected_combine,
    round_trip_rank,
    routing_for,
    traceable_hidden,
    traceable_weights,
)


def gather(obj, R):
    out = [None] * R
    dist.all_gather_object(out, obj)
    return out


def barrier(dev):
    if dev.type == "cuda":
        torch.cuda.synchronize()
        dist.barrier(device_ids=[dev.index])
    else:
        dist.barrier()


def make_buffer(case: Case, R):
    return Buffer(case.S, case.H, case.K, case.E(R), R, num_sms=case.num_sms, token_padding=case.token_padding, B=case.B)


def scenario_round_trips(rank, R, dev, ulps):
    for case in ROUNDTRIP_CASES:
        if not case.supports(R):
            continue
        buf = make_buffer(case, R)
        for it, kw in enumerate(({}, {"zero_copy": True}, {"async_finish": True})):
            rec = round_trip_rank(buf, case, R, rank, lambda: barrier(dev), **kw)
            recs = gather(rec, R)
            tabs, dst_pos, dst, src_info = check_dispatch_records(case, R, recs)
            want = expected_combine(case, R, recs, dst_pos)
            assert_within_ulp(recs[rank]["out"], want[rank], max_ulps=ulps, what=f"{case.name} it{it} rank {rank}")
            assert torch.equal(recs[rank]["weights_back"], recs[rank]["w"]), f"{case.name}: weights round trip"
        buf.destroy()
        if rank == 0:
            print(f"  round trips ok: {case.name}", flush=True)


def scenario_plan_reuse(rank, R, dev):
    """Hidden-only re-dispatch with a saved plan: same rows, weights and dedup fields untouched."""
    case = ROUNDTRIP_CASES[1]
    buf = make_buffer(case, R)
    ctx = buf._require_ctx()
    topk, tpe, _ = routing_for(case, R, rank, device=dev)
    x = traceable_hidden(case.S, case.H, rank, dev)
    w = traceable_weights(case.S, case.K, rank, dev)
    xn, wn, cu, plan = buf.dispatch(x, w, topk, tpe)
    snap = plan.clone()
    x2 = (x.float() * 2).to(torch.bfloat16)
    barrier(dev)
    wbuf_before = ctx["weights_buf_local"].clone()
    xn2, wn2, cu2, plan2 = buf.dispatch(x2, None, plan=snap)
    barrier(dev)
    assert wn2 is None and cu2 is None and plan2 is snap
    assert torch.equal(ctx["weights_buf_local"], wbuf_before), "hidden-only dispatch touched the weights buffer"
    for f in ("dup_groups", "dup_loffs", "dup_counts", "dst"):
        assert torch.equal(getattr(snap, f), getattr(plan, f)), f"replay changed plan.{f}"
    occupied = (ctx["meta_buf"][rank * ctx["meta_chunk_padded"] + ctx["SRC_INFO_OFF"]:][: ctx["NvS"]] >= 0).cpu()
    assert torch.equal((xn.float() * 2).to(torch.bfloat16).cpu()[occupied], xn2.cpu()[occupied]), "replayed rows differ"
    # combine without weights, twice in a row on one plan
    o1, w1, _ = buf.combine(snap, xn2, None)
    o2, w2, _ = buf.combine(snap, xn2, None, inter_rank_sync=True)
    barrier(dev)
    assert w1 is None and w2 is None and torch.equal(o1, o2)
    if dev.type == "cuda":
        buf.check_status()
    buf.destroy()
    if rank == 0:
        print("  plan reuse ok", flush=True)


def scenario_weights(rank, R, dev):
    """prefetch_weight and reduce_grad on symmetric tensors with a synthetic experts_to_copy table."""
    epn, B, H, Hp = 8, 4, 256, 512
    E = R * epn
    case = Case("w", S=32, K=2, epn=epn, H=64, num_sms=6, B=B, token_padding=8, routing="biased", bias=1.0)
    buf = make_buffer(case, R)
    world = buf._require_ctx()["world"]
    topk, tpe, gates = routing_for(case, R, rank, device=dev)
    x = traceable_hidden(case.S, case.H, rank, dev)
    _, _, _, plan = buf.dispatch(x, gates, topk, tpe)
    g = torch.Generator().manual_seed(99)
    etc = torch.full((R, B), -1, dtype=torch.int32)
    for src in range(R):
        for b in range(B):
            if R > 1 and torch.rand(1, generator=g).item() < 0.8:
                e = int(torch.randint(0, E, (1,), generator=g))
                if e // epn == src:
                    e = (e + epn) % E
                etc[src, b] = e
    plan = dataclasses.replace(plan, experts_to_copy=etc.to(dev))

    def expert_value(t, e):
        return torch.full((H, Hp), float(t * 100 + e), dtype=torch.bfloat16)

    fulls = []
    for t in range(3):
        full = create_full_expert_weight(E, B, H, Hp, world)
        mapped = world.is_cuda and R > 1
        for e in range(E):
            if not mapped or e // epn == rank:
                full[e].copy_(expert_value(t, e))
        full[E:].fill_(-123.0)
        fulls.append(full)
    barrier(dev)
    ev = buf.prefetch_weight(plan, async_finish=True, full_gate_weight=fulls[0], full_up_weight=fulls[1],
                             full_down_weight=fulls[2])  # fmt: skip
    ev.synchronize()
    barrier(dev)
    for t, full in enumerate(fulls):
        for b in range(B):
            e = int(etc[rank, b])
            want = expert_value(t, e) if e >= 0 else torch.full((H, Hp), -123.0, dtype=torch.bfloat16)
            assert torch.equal(full[E + b].cpu(), want), f"prefetch tensor {t} slot {b} (expert {e}) wrong"
        if mapped:
            assert torch.equal(full[E - 1].cpu(), expert_value(t, E - 1)), "peer-mapped expert not visible"

    def slot_data(t, src, b):
        gg = torch.Generator().manual_seed(1000 * t + src * B + b)
        return torch.randn(H, Hp, generator=gg)

    def grad0(t, e):
        gg = torch.Generator().manual_seed(50000 + 1000 * t + e)
        return torch.randn(H, Hp, generator=gg)

    grads, reds, red_fulls = [], [], []
    for t in range(3):
        gfull = torch.stack([grad0(t, e) for e in range(E)] + [torch.zeros(H, Hp)] * B).to(dev)
        rf = create_nvl_dist_tensor([B, H, Hp], torch.float32, world)
        red = view_nvl_dist_rows(rf, R, B)
        for b in range(B):
            red[rank, b].copy_(slot_data(t, rank, b))
        grads.append(gfull)
        reds.append(red)
        red_fulls.append(rf)
    barrier(dev)
    buf.reduce_grad(plan, False, grads[0], grads[1], grads[2], reds[0], reds[1], reds[2])
    barrier(dev)
    for t in range(3):
        for e in range(E):
            want = grad0(t, e)
            if e // epn == rank:  # owner: local value, then slots in ascending (src, b)
                for src in range(R):
                    for b in range(B):
                        if int(etc[src, b]) == e:
                            want = want + slot_data(t, src, b)
            assert torch.equal(grads[t][e].cpu(), want), f"reduce_grad tensor {t} expert {e} not bitwise equal"
        for b in range(B):
            got = reds[t][rank, b].cpu()
            if int(etc[rank, b]) >= 0:
                assert not bool(got.abs().max() > 0), "consumed slot was not cleared"
            else:
                assert torch.equal(got, slot_data(t, rank, b)), "unused slot was modified"
    if dev.type == "cuda":
        torch.cuda.synchronize()
        buf.check_status()
    barrier(dev)
    for rf in red_fulls:
        release_nvl_dist_tensor(rf)
    for full in fulls:
        release_nvl_dist_tensor(full)
    buf.destroy()
    if rank == 0:
        print("  prefetch + reduce_grad ok", flush=True)


def scenario_moe_layer(rank, R, dev):
    """SwiGLU MoE layer forward/backward on real peer-mapped weights against a dense fp32 reference."""
    from moonep_b200.models.moe_layer import ExpertParallelMoE, dense_reference
    from moonep_b200.models.routing import make_routing

    S, H, I, K, epn, B = 96, 256, 256, 2, 16, 8
    E = R * epn
    buf = Buffer(S, H, K, E, R, num_sms=8, token_padding=128, B=B)
    layer = ExpertParallelMoE(buf, I, init_std=0.05, seed=3)
    data = []
    for r in range(R):
        topk, tpe, gates = make_routing("biased", S, K, E, R, r, bias=2.0, seed=11)
        g = torch.Generator().manual_seed(100 + r)
        x = (torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16)
        go = (torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16)
        data.append((x, gates, topk, tpe, go))
    x, gates, topk, tpe, go = (t.to(dev) for t in data[rank])
    for it in range(2):  # second pass: same inputs, gradients were zeroed, weights unchanged
        out, saved = layer.forward(x, gates, topk, tpe)
        dx, dgates = layer.backward(saved, go)
        barrier(dev)
        if dev.type == "cuda":
            buf.check_status()
        grads = [g.cpu().clone() for g in layer.owner_grads()]
        layer.zero_grad()
        barrier(dev)
    mine = (out.cpu(), dx.cpu(), dgates.cpu(), grads)
    # every rank holds (or maps) all experts: take the full weights for the reference
    wg = layer.w_gate[:E].float().cpu().requires_grad_(True)
    wu = layer.w_up[:E].float().cpu().requires_grad_(True)
    wd = layer.w_down[:E].float().cpu().requires_grad_(True)
    if dev.type == "cpu":  # host worlds have no peer mapping: every rank initialised all experts itself
        pass
    ref = None
    for r in range(R):
        xr = data[r][0].float().requires_grad_(True)
        gr = data[r][1].clone().requires_grad_(True)
        o = dense_reference(xr, gr, data[r][2], wg, wu, wd)
        o.backward(data[r][4].float())
        if r == rank:
            ref = (o.detach(), xr.grad, gr.grad)

    def close(a, b, what, tol=4e-2):
        err = (a.float() - b.float()).abs().max().item()
        scale = max(1e-3, b.float().abs().max().item())
        assert err <= tol * scale, f"moe layer rank {rank} {what}: max abs err {err} vs scale {scale}"

    close(mine[0], ref[0], "output")
    close(mine[1], ref[1], "grad_x")
    close(mine[2], ref[2], "grad_gates")
    sl = slice(rank * epn, (rank + 1) * epn)
    close(mine[3][0], wg.grad[sl], "grad W_gate")
    close(mine[3][1], wu.grad[sl], "grad W_up")
    close(mine[3][2], wd.grad[sl], "grad W_down")
    barrier(dev)
    layer.destroy()
    buf.destroy()
    if rank == 0:
        print("  moe layer ok", flush=True)


def scenario_graph(rank, R, dev):
    """A captured dispatch -> combine step replayed by every rank, mixed with ordinary calls."""
    if dev.type != "cuda":
        return
    case = ROUNDTRIP_CASES[1]
    buf = make_buffer(case, R)
    topk, tpe, gates = routing_for(case, R, rank, device=dev)
    x = torch.randn(case.S, case.H, device=dev).to(torch.bfloat16)

    def step():
        xn, wn, _, plan = buf.dispatch(x, gates, topk, tpe, zero_copy=True)
        return buf.combine(plan, xn, wn, zero_copy=True)[:2]

    def done(res):
        torch.cuda.synchronize()
        buf.check_status()
        return [t.clone() for t in res]

    graph_step = buf.capture(step)
    for i in range(3):
        x.copy_(torch.randn(case.S, case.H, device=dev).to(torch.bfloat16))
        want = done(step())  # an ordinary call between replays; same kernels, same summation order
        got = done(graph_step.replay())
        assert torch.equal(got[0], want[0]), f"replay {i}: output differs from the ordinary call"
        assert torch.equal(got[1], gates), f"replay {i}: weights round trip differs"
    a = done(graph_step.replay())
    b = done(graph_step.replay())  # replays back to back: no bias update in between
    assert torch.equal(a[0], b[0]) and torch.equal(a[0], want[0])
    assert_within_ulp(a[0], (x.float() * case.K).to(torch.bfloat16), max_ulps=2, what="graph replay vs K*x")
    barrier(dev)
    buf.destroy()
    if rank == 0:
        print("  graph capture ok", flush=True)


def scenario_moe_block(rank, R, dev):
    """Router + experts with autograd, one process per rank (host backend): output and router gradient against a
    dense model that holds all experts."""
    if dev.type != "cpu":
        return
    from moonep_b200.models.moe_block import MoEBlock
    from moonep_b200.models.moe_layer import dense_reference

    S, H, I, K, epn = 64, 128, 128, 2, 2
    E = R * epn
    buf = Buffer(S, H, K, E, R, token_padding=16, B=2)
    block = MoEBlock(buf, I, init_std=0.05, seed=21)
    g = torch.Generator().manual_seed(300 + rank)
    x = (torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16).requires_grad_(True)
    go = (torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16)
    out = block(x)
    out.backward(go)
    barrier(dev)
    ex = block.experts
    wr = block.router.weight.detach().float().clone().requires_grad_(True)
    xr = x.detach().float().requires_grad_(True)
    probs = torch.softmax(xr @ wr.t(), dim=-1)
    top_p, top_i = torch.topk(probs, K, dim=-1)
    ref = dense_reference(xr, top_p / top_p.sum(dim=-1, keepdim=True), top_i, ex.w_gate[:E].float(), ex.w_up[:E].float(),
                          ex.w_down[:E].float())  # fmt: skip
    ref.backward(go.float())
    for got, want, what in ((out.detach(), ref.detach(), "output"), (x.grad, xr.grad, "input gradient"),
                            (block.router.weight.grad, wr.grad, "router gradient")):  # fmt: skip
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 6e-2 * max(1e-3, want.abs().max().item()), f"moe block rank {rank}: {what} err {err}"
    barrier(dev)
    block.destroy()
    buf.destroy()
    if rank == 0:
        print("  moe block ok", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="gloo", choices=["gloo", "nccl"])
    ap.add_argument("--scenarios", default="round_trips,plan_reuse,weights,moe_layer,graph,moe_block")
    args = ap.parse_args()
    rank = int(os.environ["RANK"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    if args.backend == "nccl":
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    R = dist.get_world_size()
    ulps = 0 if dev.type == "cpu" else 1
    todo = args.scenarios.split(",")
    if "round_trips" in todo:
        scenario_round_trips(rank, R, dev, ulps)
    if "plan_reuse" in todo:
        scenario_plan_reuse(rank, R, dev)
    if "weights" in todo:
        scenario_weights(rank, R, dev)
    if "moe_layer" in todo:
        scenario_moe_layer(rank, R, dev)
    if "graph" in todo:
        scenario_graph(rank, R, dev)
    if "moe_block" in todo:
        scenario_moe_block(rank, R, dev)
    barrier(dev)
    print(f"WORKER OK rank {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
