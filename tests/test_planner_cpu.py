"""Host planner against the literal loop oracle and structural invariants (no GPU)."""

import numpy as np
import pytest

from moonep_b200.cpu import planner as P
from moonep_b200.layout import compute_layout
from tests import oracle
from tests.cases import PLANNING_CASES
from tests.harness import routing_for


@pytest.mark.parametrize("R", [1, 2, 4])
@pytest.mark.parametrize("case", PLANNING_CASES, ids=lambda c: c.name)
def test_host_planner_matches_loop_oracle(case, R):
    if not case.supports(R):
        pytest.skip("world size not supported by this case")
    if case.S * case.K * R > 5000:
        pytest.skip("too large for the loop oracle")
    E = case.E(R)
    lay = compute_layout(case.S, case.H, case.K, E, R, B=case.B, token_padding=case.token_padding)
    routes = [routing_for(case, R, r) for r in range(R)]
    topk = [t[0].reshape(-1).tolist() for t in routes]
    tpe = [t[1].tolist() for t in routes]
    ref = oracle.plan_all_ranks(topk, tpe, S=case.S, K=case.K, R=R, E=E, B=lay["B"], P=case.token_padding, NvS=lay["NvS"])
    tabs = P.global_tables(np.array(tpe), S=case.S, K=case.K, B=lay["B"], token_padding=case.token_padding, NvS=lay["NvS"])
    assert np.array_equal(tabs["alloc"], np.array(ref["alloc"]))
    assert np.array_equal(tabs["experts_to_copy"], np.array(ref["experts_to_copy"]).reshape(R, lay["B"]))
    assert np.array_equal(tabs["remote_stats"], np.array(ref["remote_stats"]))
    assert np.array_equal(tabs["cu_seqlens"], np.array(ref["cu_seqlens"]))
    assert np.array_equal(tabs["zero_fill"], np.array(ref["zero_fill"]))
    for r in range(R):
        dp = P.local_destinations(np.array(topk[r]), r, tabs, lay["NvS"])
        dst = P.mark_duplicates(dp, case.S, case.K, lay["NvS"])
        assert np.array_equal(dst, np.array(ref["dst"][r]))


@pytest.mark.parametrize("R", [2, 8])
@pytest.mark.parametrize("case", PLANNING_CASES, ids=lambda c: c.name)
def test_host_planner_invariants(case, R):
    if not case.supports(R):
        pytest.skip("world size not supported by this case")
    E = case.E(R)
    lay = compute_layout(case.S, case.H, case.K, E, R, B=case.B, token_padding=case.token_padding)
    NvS, Pad = lay["NvS"], case.token_padding
    routes = [routing_for(case, R, r) for r in range(R)]
    tpe = np.stack([t[1].numpy() for t in routes])
    tabs = P.global_tables(tpe, S=case.S, K=case.K, B=lay["B"], token_padding=Pad, NvS=NvS)
    assert (tabs["alloc"].sum(axis=0) <= case.S * case.K).all(), "a rank receives more than S*K rows"
    assert np.array_equal(tabs["alloc"].sum(axis=1), tpe.sum(axis=0))
    seg = np.diff(np.concatenate([np.zeros((R, 1), dtype=np.int64), tabs["cu_seqlens"]], axis=1), axis=1)
    assert (seg >= 0).all() and (seg % Pad == 0).all() and (tabs["cu_seqlens"][:, -1] <= NvS).all()
    etc = tabs["experts_to_copy"]
    assert ((etc == -1) | ((etc >= 0) & (etc < E))).all()
    landed = [set() for _ in range(R)]
    for r in range(R):
        dp = P.local_destinations(routes[r][0].numpy().reshape(-1), r, tabs, NvS)
        dest, loff = dp // NvS, dp % NvS
        assert ((dest >= 0) & (dest < R)).all()
        for d, l in zip(dest.tolist(), loff.tolist()):
            assert l not in landed[d], "two entries share a destination row"
            landed[d].add(l)
    for d in range(R):
        assert len(landed[d]) == int(tabs["alloc"][:, d].sum())
