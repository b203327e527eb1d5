"""Dispatch -> expert -> combine on emulated worlds: CPU backend (always) and the sm_100a
kernels on one GPU with R emulated ranks (marked gpu).

Checks (parity: reference tests/test_dispatch.py:200-342, tests/test_combine.py:201-257):
planner outputs equal the host planner; every (source, token, k) row and weight landed where
dst says; pad rows are zero after the shard was poisoned; the dedup map equals the oracle's as
a set of groups; combine returns the K-sum with the library's two roundings; gate weights come
back bit-exact.
"""

import pytest
import torch

from tests.cases import PLANNING_CASES, ROUNDTRIP_CASES
from tests.harness import assert_within_ulp, check_dispatch_records, expected_combine, run_round_trip

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def _check(case, R, device, **kw):
    recs = run_round_trip(case, R, device, **kw)
    tabs, dst_pos, dst, src_info = check_dispatch_records(case, R, recs)
    return recs, tabs, dst_pos


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("R", [1, 2, 4])
@pytest.mark.parametrize("case", ROUNDTRIP_CASES, ids=lambda c: c.name)
def test_identity_round_trip(case, R, device):
    if not case.supports(R):
        pytest.skip("world size not supported by this case")
    recs, tabs, dst_pos = _check(case, R, device)
    want = expected_combine(case, R, recs, dst_pos)
    for r in range(R):
        assert_within_ulp(recs[r]["out"], want[r], max_ulps=0 if device == "cpu" else 1, what=f"rank {r} combine")
        assert torch.equal(recs[r]["weights_back"], recs[r]["w"]), f"rank {r}: weights did not round-trip"


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("R", [2, 4])
@pytest.mark.parametrize("case", ROUNDTRIP_CASES[:4] + ROUNDTRIP_CASES[7:8], ids=lambda c: c.name)
def test_zero_copy_scaled_expert_round_trip(case, R, device):
    """Expert stage multiplies every received row by (row index % 5 + 1); zero-copy buffers."""
    if not case.supports(R):
        pytest.skip("world size not supported by this case")

    def scale(rec, r, E):
        n = rec["hidden_nvsh"].shape[0]
        return (torch.arange(n) % 5 + 1).float()

    recs, tabs, dst_pos = _check(case, R, device, zero_copy=True, expert_scale=scale)
    NvS = recs[0]["layout"]["NvS"]
    scale_rows = [(torch.arange(NvS) % 5 + 1).float() for _ in range(R)]
    want = expected_combine(case, R, recs, dst_pos, scale_rows)
    for r in range(R):
        assert_within_ulp(recs[r]["out"], want[r], max_ulps=0 if device == "cpu" else 1, what=f"rank {r} combine")
        assert torch.equal(recs[r]["weights_back"], recs[r]["w"])


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("R", [1, 2, 4])
@pytest.mark.parametrize("case", PLANNING_CASES, ids=lambda c: c.name)
def test_planning_cases_through_dispatch(case, R, device):
    """The planner matrix, checked through a full dispatch (plan equality + landed rows)."""
    if not case.supports(R):
        pytest.skip("world size not supported by this case")
    if device == "cpu" and case.S * case.K * R > 20000:
        pytest.skip("slow on the CPU backend")
    _check(case, R, device)


@pytest.mark.parametrize("device", DEVICES)
def test_async_finish_matches_sync(device):
    case = ROUNDTRIP_CASES[1]
    a = run_round_trip(case, 2, device, async_finish=False)
    b = run_round_trip(case, 2, device, async_finish=True)
    for r in range(2):
        assert torch.equal(a[r]["out"], b[r]["out"])
        assert torch.equal(a[r]["dst"], b[r]["dst"])
        assert torch.equal(a[r]["weights_back"], b[r]["weights_back"])


@pytest.mark.parametrize("device", DEVICES)
def test_hidden_only_dispatch_without_weights(device):
    case = ROUNDTRIP_CASES[0]
    recs = run_round_trip(case, 2, device, with_weights=False)
    check_dispatch_records(case, 2, recs)
    for r in range(2):
        assert recs[r]["weights_nvs"] is None and recs[r]["weights_back"] is None


@pytest.mark.gpu
@pytest.mark.parametrize("paths", [{"MOONEP_SEND_PATH": "ldst", "MOONEP_PULL_PATH": "bulk"},
                                   {"MOONEP_COPY_PATH": "bulk", "MOONEP_PULL_PATH": "bulk", "MOONEP_GRAD_PATH": "bulk"},
                                   {"MOONEP_COPY_PATH": "ldst"}], ids=["send_ldst_pull_bulk", "all_bulk", "all_ldst"])  # fmt: skip
@pytest.mark.parametrize("case", ROUNDTRIP_CASES[:3] + ROUNDTRIP_CASES[7:10], ids=lambda c: c.name)
def test_round_trip_on_the_alternative_copy_paths(case, paths, monkeypatch):
    """Every kernel keeps a bulk-copy (TMA) and a register implementation; the non-default ones stay correct."""
    for k, v in paths.items():
        monkeypatch.setenv(k, v)
    R = 4 if case.supports(4) else 2
    recs, tabs, dst_pos = _check(case, R, "cuda")
    want = expected_combine(case, R, recs, dst_pos)
    for r in range(R):
        assert_within_ulp(recs[r]["out"], want[r], max_ulps=1, what=f"rank {r} combine")
        assert torch.equal(recs[r]["weights_back"], recs[r]["w"]), f"rank {r}: weights did not round-trip"


@pytest.mark.gpu
@pytest.mark.parametrize("local_rows", ["0", "1"], ids=["send_all", "local_rows"])
@pytest.mark.parametrize("expand", ["bulk", "ldst"])
@pytest.mark.parametrize("R", [1, 2, 4])
@pytest.mark.parametrize("case", ROUNDTRIP_CASES[:4] + ROUNDTRIP_CASES[7:10], ids=lambda c: c.name)
def test_round_trip_with_local_rows_written_by_either_role(case, R, expand, local_rows, monkeypatch):
    """The rows of a rank's own tokens come from the destination-side role (straight from the input, primary row and
    duplicates from one read; ``MOONEP_LOCAL_ROWS=1``) or from the send role like every other row (``0``); both on
    the bulk-copy and the register variant of the expansion, with one rank (every row is local) and several.  On the
    way back the same rows reach the local staging chunk through the fold role (``MOONEP_LOCAL_HOME=1``) or the push
    role."""
    if not case.supports(R):
        pytest.skip("case needs another rank count")
    monkeypatch.setenv("MOONEP_LOCAL_ROWS", local_rows)
    monkeypatch.setenv("MOONEP_LOCAL_HOME", local_rows)  # the same choice on the way back: fold role or push role
    monkeypatch.setenv("MOONEP_EXPAND_PATH", expand)
    recs, tabs, dst_pos = _check(case, R, "cuda")
    want = expected_combine(case, R, recs, dst_pos)
    for r in range(R):
        assert_within_ulp(recs[r]["out"], want[r], max_ulps=1, what=f"rank {r} combine")
        assert torch.equal(recs[r]["weights_back"], recs[r]["w"]), f"rank {r}: weights did not round-trip"


@pytest.mark.gpu
def test_large_stride_dispatch_and_identity_combine():
    """S=8192, K=16, H=7168 on two emulated ranks: every rank's shard is 1.9 GB, so element offsets inside the mapped
    range pass 2**31 and byte offsets inside one shard pass 2**30 by far (parity: reference tests/test_dispatch.py:124-134
    spot check and tests/test_combine.py:321-329 large identity combine).  Plan against the host planner, landed rows
    spot-checked through src_info, weights bit-exact, combine = K * x within the two bf16 roundings."""
    import numpy as np

    from moonep_b200 import Buffer
    from moonep_b200.cpu import planner as P
    from moonep_b200.models.routing import make_routing
    from moonep_b200.parallel.world import LocalWorld

    R, S, K, H, epn = 2, 8192, 16, 7168, 8
    E = R * epn
    lw = LocalWorld(R, "cuda")
    bufs = lw.run(lambda r: Buffer(S, H, K, E, R, num_sms=32, token_padding=128, B=2, world=lw.view(r)))
    routes = [make_routing("biased", S, K, E, R, r, bias=1.0, seed=77, device="cuda") for r in range(R)]
    xs = [(torch.randn(S, H, generator=torch.Generator().manual_seed(5 + r)) * 0.5).to(torch.bfloat16).cuda() for r in range(R)]

    def body(r):
        topk, tpe, gates = routes[r]
        xn, wn, cu, plan = bufs[r].dispatch(xs[r], gates, topk, tpe, zero_copy=True)
        torch.cuda.synchronize()
        lw.view(r).step()
        ctx = bufs[r]._require_ctx()
        src_info = plan.src_info.cpu().numpy().astype(np.int64)
        occupied = np.nonzero(src_info >= 0)[0]
        pick = occupied[np.random.default_rng(r).choice(len(occupied), 256, replace=False)]
        pick = np.concatenate([pick, occupied[-8:]])  # the highest rows of the shard too
        rows = xn[torch.from_numpy(pick).cuda()].cpu()
        wts = wn[torch.from_numpy(pick).cuda()].cpu()
        out, wb, _ = bufs[r].combine(plan, xn, wn, zero_copy=True)
        torch.cuda.synchronize()
        bufs[r].check_status()
        return {"dst": plan.dst.cpu().numpy(), "cu": cu.cpu().numpy(), "pick": pick, "info": src_info[pick], "rows": rows,
                "wts": wts, "out_err": float((out.float() - K * xs[r].float()).abs().max()), "wb_ok": torch.equal(wb, gates),
                "NvS": ctx["NvS"], "B": ctx["B"]}  # fmt: skip

    recs = lw.run(body)
    NvS = recs[0]["NvS"]
    tpe = np.stack([routes[r][1].cpu().numpy() for r in range(R)]).astype(np.int64)
    tabs = P.global_tables(tpe, S=S, K=K, B=recs[0]["B"], token_padding=128, NvS=NvS)
    for r in range(R):
        dst_pos = P.local_destinations(routes[r][0].cpu().numpy().reshape(-1), r, tabs, NvS)
        assert np.array_equal(recs[r]["dst"], P.mark_duplicates(dst_pos, S, K, NvS)), f"rank {r}: dst"
        assert np.array_equal(recs[r]["cu"], tabs["cu_seqlens"][r]), f"rank {r}: cu_seqlens"
        info = recs[r]["info"]
        src, slot = info // NvS, info % NvS
        for i in range(len(info)):
            s, t, k = int(src[i]), int(slot[i]) // K, int(slot[i]) % K
            assert torch.equal(recs[r]["rows"][i], xs[s][t].cpu()), f"rank {r}: row {recs[r]['pick'][i]} is not token {t} of rank {s}"
            assert float(recs[r]["wts"][i]) == float(routes[s][2][t, k]), f"rank {r}: weight of row {recs[r]['pick'][i]}"
        assert recs[r]["wb_ok"], f"rank {r}: gate weights did not come back bit-exact"
        assert recs[r]["out_err"] <= 0.25, f"rank {r}: combine error {recs[r]['out_err']}"
    lw.run(lambda r: bufs[r].destroy())
