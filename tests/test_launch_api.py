"""Stage-by-stage ``launch_*`` functions give the same result as ``Buffer.dispatch`` / ``Buffer.combine``;
the ``moonep_td`` import name resolves to this package."""

import pytest
import torch

from moonep_b200.models.routing import make_routing
from moonep_b200.ops import launch as L
from moonep_b200.parallel.world import LocalWorld

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def test_reference_import_name():
    import moonep_td
    from moonep_td.buffer import create_nvl_dist_tensor, pad_dim0_for_alignment  # noqa: F401
    from moonep_td.planning import MoonEPCommPlan, allocate_planning_outputs, launch_planning  # noqa: F401

    from moonep_td._dedup_builder import launch_dedup_builder  # noqa: F401
    from moonep_td.buffer import ensure_nvshmem_initialized  # noqa: F401
    from moonep_td.combine import launch_combine
    from moonep_td.combine_prologue import launch_combine_prologue  # noqa: F401
    from moonep_td.dispatch import launch_dispatch
    from moonep_td.dispatch_epilogue import launch_dispatch_epilogue  # noqa: F401
    from moonep_td.grad_reduce import launch_grad_reduce  # noqa: F401
    from moonep_td.inter_rank_sync import launch_inter_rank_sync  # noqa: F401
    from moonep_td.prefetch import launch_prefetch  # noqa: F401

    import moonep_b200

    assert launch_dispatch is L.launch_dispatch and launch_combine is L.launch_combine
    assert moonep_td.Buffer is moonep_b200.Buffer and moonep_td.MoonEPCommPlan is moonep_b200.MoonEPCommPlan
    assert pad_dim0_for_alignment([3, 48], torch.bfloat16) * 96 % 128 == 0


@pytest.mark.parametrize("device", DEVICES)
def test_launch_functions_match_buffer_methods(device):
    from moonep_td import Buffer

    R, S, H, K, epn, B = 2, 40, 64, 4, 4, 2
    E = R * epn
    lw = LocalWorld(R, device)
    bufs = lw.run(lambda r: Buffer(S, H, K, E, R, num_sms=4, token_padding=16, B=B, world=lw.view(r)))

    def body(r):
        buf = bufs[r]
        ctx = buf._require_ctx()
        topk, tpe, gates = make_routing("biased", S, K, E, R, r, bias=1.5, seed=3, device=device)
        x = torch.randn(S, H, device=device).to(torch.bfloat16)
        xn, wn, cu, plan = buf.dispatch(x, gates, topk, tpe)
        out, wb, _ = buf.combine(plan, xn, wn)
        # the same through the launch-level functions
        plan2, cu2 = L.allocate_planning_outputs(ctx)
        L.launch_inter_rank_sync(ctx)
        L.launch_planning(ctx, topk.reshape(-1), tpe, cu2, plan2)
        L.launch_dispatch(ctx, x, gates, plan2, build_dedup_map=True)
        L.launch_dispatch_epilogue(ctx, plan2)
        xn2 = ctx["hidden_buf_local"].clone()
        wn2 = ctx["weights_buf_local"].view(torch.float32).clone()
        L.launch_combine_prologue(ctx, plan2)
        out2 = torch.empty(S, H, dtype=torch.bfloat16, device=device)
        wb2 = torch.empty(S, K, dtype=torch.float32, device=device)
        L.launch_cross_rank_barrier(ctx)
        L.launch_combine(ctx, out2, plan2.dst, wb2)
        L.launch_cross_rank_barrier(ctx)
        if device == "cuda":
            torch.cuda.synchronize()
            buf.check_status()
        occ = ctx["meta_buf"][r * ctx["meta_chunk_padded"] + ctx["SRC_INFO_OFF"]:][: ctx["NvS"]] >= 0
        return (torch.equal(plan.dst, plan2.dst), torch.equal(cu, cu2), torch.equal(xn[occ], xn2[occ]),
                torch.equal(wn[occ], wn2[occ]), torch.equal(out, out2), torch.equal(wb, wb2))  # fmt: skip

    for r, flags in enumerate(lw.run(body)):
        assert all(flags), f"rank {r}: dst/cu/rows/weights/out/weights_back equal? {flags}"
    lw.run(lambda r: bufs[r].destroy())


@pytest.mark.parametrize("device", DEVICES)
def test_launch_functions_reject_bad_inputs(device):
    """Wrong dtypes and shapes are refused before anything is launched, and the message names the argument (parity:
    reference tests/test_dispatch.py:436-490 and tests/test_combine.py:332-355)."""
    from moonep_td import Buffer

    S, H, K, E = 8, 64, 2, 4
    lw = LocalWorld(1, device)
    buf = Buffer(S, H, K, E, 1, num_sms=2, token_padding=16, B=1, world=lw.view(0))
    ctx = buf._require_ctx()
    topk, tpe, gates = make_routing("balanced", S, K, E, 1, 0, device=device)
    x = torch.randn(S, H, device=device).to(torch.bfloat16)
    plan, cu = L.allocate_planning_outputs(ctx)
    L.launch_planning(ctx, topk.reshape(-1).contiguous(), tpe, cu, plan)

    with pytest.raises(AssertionError, match="hidden_sh"):
        L.launch_dispatch(ctx, x.float(), gates, plan, build_dedup_map=True)
    with pytest.raises(AssertionError, match="hidden_sh"):
        L.launch_dispatch(ctx, x[: S // 2].contiguous(), gates, plan, build_dedup_map=True)
    with pytest.raises(AssertionError, match="route_weights_sk"):
        L.launch_dispatch(ctx, x, gates.double(), plan, build_dedup_map=True)
    with pytest.raises(AssertionError, match="route_weights_sk"):
        L.launch_dispatch(ctx, x, gates[:, : K - 1].contiguous(), plan, build_dedup_map=True)
    bad = plan.clone()
    object.__setattr__(bad, "dst", plan.dst.long())
    with pytest.raises(AssertionError, match="dst"):
        L.launch_dispatch(ctx, x, gates, bad, build_dedup_map=True)
    bad = plan.clone()
    object.__setattr__(bad, "dup_loffs", plan.dup_loffs.flatten()[:-1].contiguous())
    with pytest.raises(AssertionError, match="dup_loffs"):
        L.launch_dispatch_epilogue(ctx, bad)
    out = torch.empty(S, H, dtype=torch.bfloat16, device=device)
    with pytest.raises(AssertionError, match="output_sk"):
        L.launch_combine(ctx, out, plan.dst, output_sk=torch.empty(S, K, dtype=torch.bfloat16, device=device))
    with pytest.raises(AssertionError, match="output_sh"):
        L.launch_combine(ctx, out.float(), plan.dst)
    # nothing above consumed the plan: the regular sequence still runs
    L.launch_dispatch(ctx, x, gates, plan, build_dedup_map=True)
    L.launch_dispatch_epilogue(ctx, plan)
    if device == "cuda":
        torch.cuda.synchronize()
        buf.check_status()
    buf.destroy()
