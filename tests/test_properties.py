"""Property-based round trips on the host backend: for arbitrary small shapes, routings and paddings the planner
keeps every rank within S*K rows, every (source, token, k) entry lands exactly where ``dst`` says, the dedup map
matches the oracle, and combine returns the K-sum with the library's two roundings (parity: the reference's
structural invariants, tests/kernel_test_utils.py:292-364, here over generated cases instead of a fixed list)."""

import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import HealthCheck, given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from tests.harness import Case, assert_within_ulp, check_dispatch_records, expected_combine, run_round_trip  # noqa: E402


@st.composite
def cases(draw):
    R = draw(st.integers(1, 4))
    epn = draw(st.integers(1, 4))
    routing = draw(st.sampled_from(["balanced", "biased", "zipf", "softmax", "single_expert", "duplicate_topk", "all_remote"]))
    kmax = 6 if routing in ("single_expert", "duplicate_topk") else min(6, R * epn)
    K = draw(st.integers(1, kmax))
    case = Case(
        name="generated", S=draw(st.integers(1, 24)), K=K, epn=epn, H=draw(st.sampled_from([8, 20, 32])),
        num_sms=draw(st.integers(1, 4)), B=draw(st.integers(0, epn)), token_padding=draw(st.sampled_from([1, 4, 8, 16])),
        routing=routing, bias=draw(st.sampled_from([0.5, 1.5, 3.0])), seed=draw(st.integers(0, 10_000)),
        min_R=2 if routing in ("duplicate_topk", "all_remote") else 1,
    )  # fmt: skip
    return case, R


@settings(max_examples=30, deadline=None, suppress_health_check=[HealthCheck.too_slow, HealthCheck.data_too_large])
@given(cases())
def test_generated_round_trips_hold_the_invariants(case_and_R):
    case, R = case_and_R
    if not case.supports(R):
        return
    recs = run_round_trip(case, R, "cpu")
    tabs, dst_pos, dst, src_info = check_dispatch_records(case, R, recs)  # landing rows, weights, dedup map, zero fill
    rows_per_rank = tabs["alloc"].sum(axis=0)
    assert (rows_per_rank <= case.S * case.K).all(), "a rank receives more than S*K rows"
    assert int(rows_per_rank.sum()) == R * case.S * case.K
    want = expected_combine(case, R, recs, dst_pos)
    for r in range(R):
        assert_within_ulp(recs[r]["out"], want[r], max_ulps=0, what=f"rank {r} combine")
        assert torch.equal(recs[r]["weights_back"], recs[r]["w"]), f"rank {r}: weights did not round-trip"
