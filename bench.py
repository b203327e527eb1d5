"""Headline benchmark: expert-parallel dispatch + combine round trip.

Config (DeepSeek-V3 shaped EP): S=4096 tokens per rank, H=7168 bf16, K=8, E=256 experts,
router logits ~ N(0,1) with softmax top-8 gates, num_sms=32, token_padding=128,
identity expert, synthetic data, weak scaling (S per rank fixed).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

Rank 0 prints one JSON line.  ``value`` is aggregate tokens per second through one
fresh-plan dispatch plus one combine (device-timed with CUDA events, max over ranks, L2
flushed between timed steps).  ``e2e`` is the same step through the public API including
the per-step host-to-device copy of the inputs from pinned memory and the device-to-host
read of a checksum of the result.  ``--impl reference`` runs the reference package from
``baseline/_ref`` if its runtime (triton_dist + nvshmem4py) can be imported.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl"])
    p.add_argument("--S", type=int, default=4096)
    p.add_argument("--H", type=int, default=7168)
    p.add_argument("--K", type=int, default=8)
    p.add_argument("--E", type=int, default=256)
    p.add_argument("--num-sms", type=int, default=32)
    p.add_argument("--token-padding", type=int, default=128)
    p.add_argument("--routing", default="softmax")
    p.add_argument("--staged", action="store_true", help="use the copying (non zero-copy) API paths")
    p.add_argument("--profile-phases", action="store_true", help="(kept for old command lines: phases_us is always reported)")
    p.add_argument("--graph", action="store_true", help="also time the step as one CUDA graph replay (Buffer.capture)")
    p.add_argument("--config", default="headline", choices=["headline", "skew", "sweep", "moe_step", "weights", "p2p_peak"],
                   help="headline: S=4096,H=7168,K=8,E=256 softmax routing; skew: S=8192,H=4096,E=64,K=6 Zipf(1.2); "
                        "sweep: S in {128..16384} with uniform routing, ours and NCCL; moe_step: SwiGLU MoE layer "
                        "forward+backward+SGD with intermediate size --inter; weights: worst-case prefetch_weight and "
                        "reduce_grad traffic (every slot in use); p2p_peak: peer-copy bandwidth of the copy engines and "
                        "of SM-driven bulk-copy rings (2 or more GPUs)")  # fmt: skip
    p.add_argument("--inter", type=int, default=2048)
    return p.parse_args()


HOST_AFFINITY: dict = {}


def init_dist(n):
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    # host threads and the pinned staging buffers of the end-to-end loop stay on the GPU's CPU socket
    from moonep_b200.utils.affinity import bind_to_gpu_socket

    global HOST_AFFINITY
    HOST_AFFINITY = bind_to_gpu_socket(local)
    if n > 1:
        import torch.distributed as dist

        assert world == n, f"--gpus {n} but WORLD_SIZE={world}; launch with torch.distributed.run"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, local, world


def max_over_ranks(x: float, n: int) -> float:
    if n == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync(n):
    torch.cuda.synchronize()
    if n > 1:
        import torch.distributed as dist

        dist.barrier(device_ids=[torch.cuda.current_device()])
        torch.cuda.synchronize()


def reference_arm(args):
    out = {"impl": "reference"}
    first = os.environ.get("RANK", "0") == "0"  # under torch.distributed.run every rank gets here: one line in all
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    try:
        import moonep_td  # noqa: F401
    except Exception as exc:  # noqa: BLE001
        out["unavailable"] = f"reference package not installed under baseline/_ref: {exc!r}"
        if first:
            print(json.dumps(out))
        return
    try:
        import nvshmem.core  # noqa: F401
        import triton_dist  # noqa: F401
    except Exception as exc:  # noqa: BLE001
        out["unavailable"] = (
            "reference needs triton_dist (Triton-distributed) and nvshmem4py, neither is in this image "
            f"and there is no network: {exc!r}"
        )
        if first:
            print(json.dumps(out))
        return
    # Both runtimes import: run the reference's own Buffer on the same config.
    from moonep_td import Buffer as RefBuffer

    rank, local, world = init_dist(args.gpus)
    res = run_steps(args, RefBuffer, rank, world, reference=True)
    if rank == 0:
        res["impl"] = "reference"
        print(json.dumps(res))


def run_steps(args, BufferCls, rank, n, reference=False):
    from moonep_b200.models.routing import make_routing
    from moonep_b200.utils.clocks import ClockSampler

    S, H, K, E = args.S, args.H, args.K, args.E
    dev = torch.device("cuda", torch.cuda.current_device())
    buf = BufferCls(S, H, K, E, n, num_sms=args.num_sms, token_padding=args.token_padding)
    zero_copy = not args.staged
    topk_h, tpe_h, gates_h = make_routing(args.routing, S, K, E, n, rank, seed=2026)
    g = torch.Generator().manual_seed(7 + rank)
    x_h = torch.randn(S, H, generator=g).to(torch.bfloat16)
    pinned = [t.pin_memory() for t in (x_h, gates_h, topk_h, tpe_h)]
    x, gates, topk, tpe = (t.to(dev) for t in pinned)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > 126 MB L2

    def step(x, gates, topk, tpe):
        xn, wn, cu, plan = buf.dispatch(x, gates, topk, tpe, zero_copy=zero_copy)
        out, wb, _ = buf.combine(plan, xn, wn, zero_copy=zero_copy)
        return out, wb, plan

    lib = None
    if not reference:
        from moonep_b200.ops import _lib

        lib = _lib.load()

    for _ in range(max(args.warmup, 3)):
        out, wb, plan = step(x, gates, topk, tpe)
    torch.cuda.synchronize()
    if hasattr(buf, "check_status"):
        buf.check_status()
    # Correctness: with an identity expert the result is known exactly.  The rows of a token that land on one rank are
    # added in fp32 and rounded to bf16 (m * x for m entries on that rank), the per-rank results are added in fp32 in
    # ascending k of their first entry and rounded to bf16.  The check allows one bf16 ulp around that value.
    NvS_ = plan.NvS
    d = plan.dst.view(S, K).to(torch.int64)
    dest = torch.where(d < 0, -d - 1, d) // NvS_
    xf = x.float()
    acc = torch.zeros_like(xf)
    for k in range(K):
        m_k = (dest == dest[:, k : k + 1]).sum(dim=1).float()  # entries of the token on the rank of entry k
        part = (xf * m_k[:, None]).to(torch.bfloat16).float()
        acc += part * (d[:, k] >= 0).float()[:, None]
    want = acc.to(torch.bfloat16).float()
    ulp = torch.pow(2.0, torch.floor(torch.log2(want.abs().clamp(min=2.0**-126))) - 7)
    err_ulp = ((out.float() - want).abs() / ulp).max().item()
    err = (out.float() - K * xf).abs().max().item()
    ok = err_ulp <= 1.0 and torch.equal(wb, gates)
    del xf, acc, want, ulp

    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    with ClockSampler(torch.cuda.current_device(), period_ms=1) as clocks:
        # starting the sampler takes tens of milliseconds in which the GPU idles and drops its clocks: two more untimed
        # steps bring it back before the timed region opens
        for _ in range(2):
            step(x, gates, topk, tpe)
        barrier_sync(n)
        clocks.reset()
        launches0 = lib.moonep_launch_count() if lib else 0
        for i in range(args.steps):
            flush.zero_()
            ev[i][0].record()
            xn, wn, cu, plan = buf.dispatch(x, gates, topk, tpe, zero_copy=zero_copy)
            ev[i][1].record()
            out, wb, _ = buf.combine(plan, xn, wn, zero_copy=zero_copy)
            ev[i][2].record()
        barrier_sync(n)
    launches = (lib.moonep_launch_count() - launches0) if lib else 0
    raw_steps = [e[0].elapsed_time(e[2]) for e in ev]
    per_step = sorted(raw_steps)
    t_disp = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps
    t_comb = sum(e[1].elapsed_time(e[2]) for e in ev) / args.steps
    t_step = sum(per_step) / args.steps
    t_disp, t_comb, t_step = (max_over_ranks(t, n) for t in (t_disp, t_comb, t_step))
    step_stats = {"min": max_over_ranks(per_step[0], n), "median": max_over_ranks(per_step[len(per_step) // 2], n),
                  "max": max_over_ranks(per_step[-1], n), "slowest_step_on_rank0": raw_steps.index(per_step[-1])}  # fmt: skip

    # per-kernel device times, so that the record names the limiting kernel
    phases = None
    if not reference:
        be = buf._require_ctx()["_backend"]
        be.profile(True)
        be.reset_wait_stats()
        for _ in range(10):
            flush.zero_()
            step(x, gates, topk, tpe)
        phases = {k: round(max_over_ranks(v, n), 1) for k, v in sorted(be.phase_times().items())}
        be.profile(False)
        # inside the fused kernels: longest duration of each role's phases over the CTAs (device clock)
        inner = be.stats().get("kernel_phase_max_us", {})
        phases["inside_kernels_max_us"] = {k: round(max_over_ranks(v, n), 1) for k, v in sorted(inner.items())}

    # the same step as one CUDA graph replay (one launch from the host per step)
    graph_ms = None
    if args.graph and not reference:
        cap = buf.capture(lambda: step(x, gates, topk, tpe)[0])
        for _ in range(3):
            cap.replay()
        gev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        barrier_sync(n)
        for a_, b_ in gev:
            flush.zero_()
            a_.record()
            cap.replay()
            b_.record()
        barrier_sync(n)
        graph_ms = max_over_ranks(sum(a_.elapsed_time(b_) for a_, b_ in gev) / args.steps, n)
        buf.check_status()

    # end to end: every step copies its inputs from pinned host memory and sends a checksum of its
    # result back to the host.  The copy of step i+1 runs on a second stream while step i computes
    # (two input buffer sets), as a training or serving loop would do it.
    K_e2e = args.steps
    cs_h = torch.empty(K_e2e + 2, dtype=torch.float32).pin_memory()
    sets = [[torch.empty_like(t, device=dev) for t in pinned] for _ in range(2)]
    copy_stream = torch.cuda.Stream()
    main = torch.cuda.current_stream()
    ready = [torch.cuda.Event() for _ in range(2)]
    free = [torch.cuda.Event() for _ in range(2)]

    def issue_h2d(i):
        k = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(free[k])
            for d, h in zip(sets[k], pinned):
                d.copy_(h, non_blocking=True)
            ready[k].record(copy_stream)

    def e2e_loop(steps, base):
        for k in range(2):
            free[k].record(main)
        issue_h2d(0)
        for i in range(steps):
            if i + 1 < steps:
                issue_h2d(i + 1)
            flush.zero_()
            main.wait_event(ready[i % 2])
            out, wb, plan = step(*sets[i % 2])
            free[i % 2].record(main)
            cs_h[base + i : base + i + 1].copy_(out.sum(dtype=torch.float32).reshape(1), non_blocking=True)

    e2e_loop(2, K_e2e)  # warm-up
    barrier_sync(n)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    e2e_loop(K_e2e, 0)
    t1.record()
    barrier_sync(n)
    t_e2e = max_over_ranks(t0.elapsed_time(t1) / K_e2e, n)
    assert bool(torch.isfinite(cs_h[:K_e2e]).all()), "end-to-end checksums are not finite"
    h2d = sum(t.numel() * t.element_size() for t in pinned)

    # bytes that cross to other ranks (primary rows only) for the bandwidth figures
    dst = plan.dst
    NvS = plan.NvS
    dest = torch.where(dst < 0, -dst - 1, dst) // NvS
    remote_rows = int(((dst >= 0) & (dest != rank)).sum().item())
    total_rows = int((dst >= 0).sum().item())
    row_bytes = H * 2
    if hasattr(buf, "check_status"):
        buf.check_status()
    buf.destroy()
    res = {
        "metric": "ep_dispatch_combine_tokens_per_s",
        "value": n * S / (t_step / 1e3),
        "unit": "tokens/s",
        "n_gpus": n,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": t_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic (N(0,1) activations, N(0,1) router logits, softmax top-k gates, identity expert)",
        "config": {
            "model": "DeepSeek-V3-shaped EP dispatch+combine",
            "S_per_rank": S, "H": H, "K": K, "E": E, "global_batch": n * S, "seq_len": S,
            "parallelism": f"ep{n}", "num_sms": args.num_sms, "token_padding": args.token_padding,
            "routing": args.routing, "zero_copy": zero_copy, "l2": "flushed between timed steps (256 MB write)",
        },
        "dispatch_us": t_disp * 1e3,
        "combine_us": t_comb * 1e3,
        "rows_sent_per_rank": total_rows,
        "remote_rows_per_rank": remote_rows,
        "dispatch_nvlink_GBps_per_rank": remote_rows * row_bytes / (t_disp / 1e3) / 1e9,
        "combine_nvlink_GBps_per_rank": remote_rows * row_bytes / (t_comb / 1e3) / 1e9,
        "dispatch_payload_GBps_per_rank": total_rows * row_bytes / (t_disp / 1e3) / 1e9,
        "combine_payload_GBps_per_rank": total_rows * row_bytes / (t_comb / 1e3) / 1e9,
        "correct": bool(ok),
        "max_abs_err": err,
        "max_err_bf16_ulp_vs_two_rounding_model": err_ulp,
        "ms_per_step_stats": step_stats,
        "clocks": clocks.summary(),
        "e2e": {
            "value": n * S / (t_e2e / 1e3), "unit": "tokens/s", "ms_per_step": t_e2e,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
        },
        "gpu_launches": int(launches),
        "host_cpu_affinity": HOST_AFFINITY,
    }  # fmt: skip
    if phases is not None:
        res["phases_us"] = phases
    if graph_ms is not None:
        res["graph_replay_ms_per_step"] = graph_ms
    return res


def run_moe_step(args, rank, n):
    """SwiGLU MoE layer training step: dispatch -> prefetch -> grouped GEMMs -> combine, backward with the
    plan replayed, reduce_grad, SGD on the owned experts.  Device-timed, max over ranks."""
    from moonep_b200 import Buffer, config
    from moonep_b200.models.moe_layer import ExpertParallelMoE
    from moonep_b200.models.routing import make_routing
    from moonep_b200.utils.clocks import ClockSampler

    S, H, K, E, inter = args.S, args.H, args.K, args.E, args.inter
    dev = torch.device("cuda", torch.cuda.current_device())
    slots = min(E // n, 32)  # prefetch slots per rank; bounds weights + gradients + reduce buffers to ~25 GB
    buf = Buffer(S, H, K, E, n, num_sms=args.num_sms, token_padding=128, B=slots)
    layer = ExpertParallelMoE(buf, inter, init_std=0.02, seed=1)
    topk, tpe, gates = make_routing(args.routing, S, K, E, n, rank, seed=2026, device=dev)
    g = torch.Generator().manual_seed(7 + rank)
    x = torch.randn(S, H, generator=g).to(torch.bfloat16).to(dev)
    go = (torch.randn(S, H, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    last = {}

    def step():
        out, saved = layer.forward(x, gates, topk, tpe)
        mid.record()
        dx, dg = layer.backward(saved, go)
        last.update(dx=dx, dgates=dg)
        layer.sgd_step(1e-5)
        layer.zero_grad()
        return out

    mid = torch.cuda.Event(enable_timing=True)
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    buf.check_status()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier_sync(n)
    with ClockSampler(torch.cuda.current_device()) as clocks:
        for i in range(args.steps):
            flush.zero_()
            ev[i][0].record()
            mid = ev[i][1]
            out = step()
            ev[i][2].record()
        barrier_sync(n)
    t_f = max_over_ranks(sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps, n)
    t_all = max_over_ranks(sum(e[0].elapsed_time(e[2]) for e in ev) / args.steps, n)
    buf.check_status()
    # every rank's outputs, input gradients, gate gradients and owned weight gradients must be finite
    finite = all(bool(torch.isfinite(t.float()).all()) for t in (out, last["dx"], last["dgates"], *layer.owner_grads()))
    finite = max_over_ranks(0.0 if finite else 1.0, n) == 0.0
    layer.destroy()
    buf.destroy()
    flops_fwd = 2.0 * S * K * H * inter * 3  # per rank, real rows
    return {
        "metric": "moe_layer_train_tokens_per_s", "value": n * S / (t_all / 1e3), "unit": "tokens/s", "n_gpus": n,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": t_all, "forward_ms": t_f,
        "backward_ms": t_all - t_f, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic, random-init weights ~N(0,0.02)",
        "config": {"model": "SwiGLU MoE layer (dispatch->prefetch->grouped GEMM->combine, backward with reduce_grad)",
                   "S_per_rank": S, "H": H, "K": K, "E": E, "inter": inter, "parallelism": f"ep{n}",
                   "routing": args.routing, "prefetch_slots": slots,
                   "backward_gemms": "activation and weight gradients: tcgen05 grouped GEMMs" if config.wgrad_on_kernel()
                   else "activation grads: tcgen05 grouped GEMM; weight grads: torch matmul per group (bf16)"},
        "forward_tflops_per_gpu": flops_fwd / (t_f / 1e3) / 1e12, "finite": finite,
        "clocks": clocks.summary(),
    }  # fmt: skip


def run_weights(args, rank, n):
    """Worst-case expert-weight traffic: every rank prefetches B experts of the next rank (gate, up, down) and
    every owner reduces B fp32 gradient slots per tensor from the previous rank.  Device-timed, max over ranks."""
    import dataclasses

    from moonep_b200 import Buffer
    from moonep_b200.models.routing import make_routing
    from moonep_b200.parallel.symm import create_full_expert_weight, create_nvl_dist_tensor, view_nvl_dist_rows

    E, H, inter, S, K = args.E, args.H, args.inter, 512, args.K
    epn = E // n
    B = min(epn, 32)
    dev = torch.device("cuda", torch.cuda.current_device())
    buf = Buffer(S, H, K, E, n, num_sms=args.num_sms, token_padding=128, B=B)
    world = buf._require_ctx()["world"]
    topk, tpe, gates = make_routing("softmax", S, K, E, n, rank, seed=1, device=dev)
    x = torch.randn(S, H, device=dev).to(torch.bfloat16)
    plan = buf.dispatch(x, gates, topk, tpe)[3]
    etc = torch.full((n, B), -1, dtype=torch.int32)
    for r in range(n):
        src = (r + 1) % n
        etc[r] = torch.arange(B, dtype=torch.int32) + src * epn
    plan = dataclasses.replace(plan, experts_to_copy=etc.to(dev))
    shapes = ((inter, H), (inter, H), (H, inter))
    ws = [create_full_expert_weight(E, B, d0, d1, world) for d0, d1 in shapes]
    mapped = n > 1
    for w in ws:
        (w[rank * epn : (rank + 1) * epn] if mapped else w[:E]).normal_(0, 0.02)
    reds = [view_nvl_dist_rows(create_nvl_dist_tensor([B, d0, d1], torch.float32, world, pad_dim0=False), n, B)
            for d0, d1 in shapes]  # fmt: skip
    grads = [torch.zeros(epn, d0, d1, dtype=torch.float32, device=dev) for d0, d1 in shapes]
    for r_ in reds:
        r_[rank].fill_(1.0)
    barrier_sync(n)

    def timed(fn):
        for _ in range(3):
            fn()
        barrier_sync(n)
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a_, b_ in ev:
            a_.record()
            fn()
            b_.record()
        barrier_sync(n)
        return max_over_ranks(sum(a_.elapsed_time(b_) for a_, b_ in ev) / args.steps, n)

    t_pf = timed(lambda: buf.prefetch_weight(plan, full_gate_weight=ws[0], full_up_weight=ws[1], full_down_weight=ws[2]))

    def reduce_once():
        for r_ in reds:
            r_[rank].fill_(1.0)  # slots are cleared by every reduce; refill outside the kernel under test
        buf.reduce_grad(plan, False, grads[0], grads[1], grads[2], reds[0], reds[1], reds[2], owner_local=True)

    def fill_only():
        for r_ in reds:
            r_[rank].fill_(1.0)

    t_red = timed(reduce_once) - timed(fill_only)
    buf.check_status()
    pf_bytes = 3 * B * H * inter * 2
    red_bytes = 3 * B * H * inter * 4
    return {
        "metric": "expert_weight_traffic", "n_gpus": n, "B": B, "H": H, "inter": inter,
        "prefetch_ms": t_pf, "prefetch_GB": pf_bytes / 1e9, "prefetch_GBps_per_rank": pf_bytes / (t_pf / 1e3) / 1e9,
        "reduce_grad_ms": t_red, "reduce_grad_GB": red_bytes / 1e9,
        "reduce_grad_pull_GBps_per_rank": red_bytes / (t_red / 1e3) / 1e9,
        "note": "remote pulls over NVLink when n_gpus > 1, local HBM copies when n_gpus == 1; reduce_grad time "
                "includes the accumulate kernel, the flag round and clearing the consumed slots",
    }  # fmt: skip


def run_p2p_peak(args, rank, n):
    """Measured peer-copy bandwidth: every rank copies 1 GiB into the next rank's symmetric chunk with a plain device
    copy (cudaMemcpyAsync through torch), all ranks at once, device-timed, max over ranks.  The denominator of the NVLink
    roofline fractions this repository quotes."""
    from moonep_b200.parallel.world import DistWorld

    assert n > 1, "p2p_peak needs at least two GPUs"
    w = DistWorld()
    nbytes = 1 << 30
    st = w.alloc_symmetric(nbytes, torch.uint8, w.granularity())
    src = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    peer = (rank + 1) % n
    dst = st.full[peer * nbytes : (peer + 1) * nbytes]
    for _ in range(3):
        dst.copy_(src)
    barrier_sync(n)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a_, b_ in ev:
        a_.record()
        dst.copy_(src)
        b_.record()
    barrier_sync(n)
    t = max_over_ranks(min(a_.elapsed_time(b_) for a_, b_ in ev), n)
    t_mean = max_over_ranks(sum(a_.elapsed_time(b_) for a_, b_ in ev) / args.steps, n)
    barrier_sync(n)
    # The same transfer driven by SMs: CTAs stream the buffer through a shared-memory ring of bulk copies, as the
    # dispatch send role does, without routing, flags or weights (csrc/p2p_bench.cu).  The ceiling of the send and
    # push roles, for num_sms CTAs and for all SMs.
    from moonep_b200.ops import _lib

    lib = _lib.load()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    sm_rates = {}
    stream = torch.cuda.current_stream().cuda_stream
    # the last 1 MiB of the peer's chunk receives the helper warps' flag-like stores
    flag_words = dst[nbytes - (1 << 20):].view(torch.int32)
    copy_bytes = nbytes - (1 << 20)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for grid, fence_warps in ((args.num_sms, 0), (2 * args.num_sms, 0), (sms, 0), (args.num_sms, 4)):
        def once():
            rc = lib.moonep_peer_store_bench(dst.data_ptr(), src.data_ptr(), copy_bytes, 14336, grid, err.data_ptr(), 5000,
                                             fence_warps, flag_words.data_ptr() if fence_warps else None, stream)
            assert rc == 0, lib.moonep_last_error().decode()
        for _ in range(3):
            once()
        barrier_sync(n)
        ev2 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a_, b_ in ev2:
            a_.record()
            once()
            b_.record()
        barrier_sync(n)
        t_sm = max_over_ranks(min(a_.elapsed_time(b_) for a_, b_ in ev2), n)
        key = f"{grid}_ctas" + (f"_with_{fence_warps}_fencing_warps" if fence_warps else "")
        sm_rates[key] = copy_bytes / (t_sm / 1e3) / 1e9
    assert int(err.item()) == 0, "the measurement kernel gave up a wait"
    barrier_sync(n)
    w.free_symmetric(st)
    return {"metric": "peer_copy_GBps_per_direction", "n_gpus": n, "bytes": nbytes, "best_ms": t, "mean_ms": t_mean,
            "value": nbytes / (t / 1e3) / 1e9, "mean_GBps": nbytes / (t_mean / 1e3) / 1e9,
            "sm_bulk_store_GBps": sm_rates,
            "note": "every rank writes 1 GiB into the next rank's memory at the same time: device copy engine (value), "
                    "and SM-driven cp.async.bulk rings of 14 KB pieces with the given number of CTAs, once with four more "
                    "warps per CTA that issue system-scope fences and 4-byte peer stores all the while"}  # fmt: skip


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    rank, local, world = init_dist(args.gpus)
    if args.config == "p2p_peak":
        res = run_p2p_peak(args, rank, args.gpus)
        if rank == 0:
            print(json.dumps(res))
        import torch.distributed as dist

        dist.destroy_process_group()
        return
    if args.config == "skew":
        args.S, args.H, args.E, args.K, args.routing = 8192, 4096, 64, 6, "zipf"
    if args.config in ("moe_step", "weights"):
        res = run_moe_step(args, rank, args.gpus) if args.config == "moe_step" else run_weights(args, rank, args.gpus)
        if rank == 0:
            res["impl"] = "ours"
            print(json.dumps(res))
        if args.gpus > 1:
            import torch.distributed as dist

            dist.destroy_process_group()
        return
    if args.config == "sweep":
        from moonep_b200 import Buffer
        from moonep_b200.bench.nccl_baseline import run_nccl_baseline

        for S in (128, 512, 2048, 8192, 16384):
            args.S = S
            args.routing = "softmax"
            ours = run_steps(args, Buffer, rank, args.gpus)
            base = run_nccl_baseline(args, rank, args.gpus)
            if rank == 0:
                print(json.dumps({"S": S, "n_gpus": args.gpus, "ours_dispatch_us": ours["dispatch_us"],
                                  "ours_combine_us": ours["combine_us"], "nccl_dispatch_us": base["dispatch_us"],
                                  "nccl_combine_us": base["combine_us"],
                                  "speedup_round_trip": base["ms_per_step"] / ours["ms_per_step"]}))  # fmt: skip
        if args.gpus > 1:
            import torch.distributed as dist

            dist.destroy_process_group()
        return
    if args.impl == "nccl":
        from moonep_b200.bench.nccl_baseline import run_nccl_baseline

        res = run_nccl_baseline(args, rank, args.gpus)
    else:
        from moonep_b200 import Buffer

        res = run_steps(args, Buffer, rank, args.gpus)
    if rank == 0:
        res["impl"] = args.impl
        print(json.dumps(res))
    if args.gpus > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    t0 = time.time()
    main()
