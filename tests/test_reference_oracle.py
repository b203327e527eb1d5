"""Cross-check of the host planner against the reference implementation's own planning oracle, when a copy of the
reference is available (``MOONEP_REFERENCE_DIR``, default: a directory ``reference`` beside this repository); skipped
otherwise.

The reference's ``tests/planning_reference.launch_planning_torch_reference(ctx, topk, tokens_per_expert)`` accepts a
2-D tokens-per-expert table, in which case it needs no process group (with ``materialize_dedup=False`` for more than
one rank, because its duplicate marking gathers ``dst`` over the group).  It returns
``(dst, cu_seqlens, experts_to_copy, remote_stats, zero_fill_ranges, dedup_plan)`` for one rank.
"""

import importlib.util
import os
import sys

import numpy as np
import pytest
import torch

from moonep_b200.cpu import planner as P
from moonep_b200.layout import compute_layout
from moonep_b200.models.routing import make_routing
from tests.cases import PLANNING_CASES

_BESIDE = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
REF_DIR = os.environ.get("MOONEP_REFERENCE_DIR", _BESIDE)
REF_FILE = os.path.join(REF_DIR, "tests", "planning_reference.py")
_ref = None


def _reference():
    global _ref
    if _ref is None:
        if not os.path.isfile(REF_FILE):
            pytest.skip(f"no copy of the reference at {REF_DIR}")
        spec = importlib.util.spec_from_file_location("_moonep_reference_planning", REF_FILE)
        mod = importlib.util.module_from_spec(spec)
        try:
            spec.loader.exec_module(mod)
        except Exception as exc:  # noqa: BLE001 - its imports may need packages this machine lacks
            pytest.skip(f"the reference's planner cannot be imported here: {exc!r}")
        _ref = mod
    return _ref


SMALL = [c for c in PLANNING_CASES if c.S * c.K <= 2048][:12]


@pytest.mark.parametrize("R", [1, 2, 4, 8])
@pytest.mark.parametrize("case", SMALL, ids=lambda c: c.name)
def test_host_planner_equals_the_reference_oracle(case, R):
    if not case.supports(R) or case.E(R) > 512:
        pytest.skip("not a case for this world size (or too slow in the reference's Python loops)")
    fn = _reference().launch_planning_torch_reference
    E, S, K, pad = case.E(R), case.S, case.K, case.token_padding
    lay = compute_layout(S, case.H, K, E, R, B=case.B, token_padding=pad)
    NvS = lay["NvS"]
    routes = [make_routing(case.routing, S, K, E, R, r, bias=case.bias or 1.0, seed=case.seed) for r in range(R)]
    tpe = torch.stack([routes[r][1] for r in range(R)]).to(torch.int32)
    tabs = P.global_tables(tpe.numpy().astype(np.int64), S=S, K=K, B=lay["B"], token_padding=pad, NvS=NvS)
    for r in range(R):
        ctx = dict(lay)
        ctx["rank"] = r
        topk = routes[r][0].to(torch.int32)
        ref = fn(ctx, topk, tpe, materialize_dedup=(R == 1))
        dst_pos = P.local_destinations(topk.numpy().reshape(-1), r, tabs, NvS)
        dst = P.mark_duplicates(dst_pos, S, K, NvS) if R == 1 else dst_pos
        assert np.array_equal(dst, ref[0].numpy()), f"rank {r}: dst differs from the reference oracle"
        assert np.array_equal(tabs["cu_seqlens"][r], ref[1].numpy()), f"rank {r}: cu_seqlens"
        assert np.array_equal(tabs["experts_to_copy"], ref[2].numpy()), f"rank {r}: experts_to_copy"
        assert np.array_equal(tabs["remote_stats"][r], ref[3].numpy()), f"rank {r}: remote_stats"
        assert np.array_equal(tabs["zero_fill"][r], ref[4].numpy()), f"rank {r}: zero_fill_ranges"
        if R == 1:  # the reference's duplicate map (deterministic order) against ours, as sets of groups
            src_info = np.full(NvS, -1, dtype=np.int64)
            src_info[dst_pos % NvS] = r * NvS + np.arange(S * K)
            g, l, n = P.build_dedup(src_info, S=S, K=K, NvS=NvS)
            rd = ref[5]
            assert np.array_equal(n, rd.dup_counts.numpy())
            ours = {int(a): tuple(sorted(l[b : b + c].tolist())) for a, b, c in g[: n[0]]}
            theirs = {int(a): tuple(sorted(rd.dup_loffs[b : b + c].tolist())) for a, b, c in rd.dup_groups[: n[0]].tolist()}
            assert ours == theirs
