"""The allocation-free planner entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they need the routing tables: a
serving thread that must not trigger cudaMalloc's implicit device synchronisation, or a process
whose memory belongs to another allocator.  ``moonep_plan_tables_noalloc`` keeps its work area in
a fixed array inside the library; the caller passes only inputs and outputs.  This test compares
it with the tables the normal path (``Buffer.dispatch``) produces for the same routing, on two
calls in a row (the calls share the work area, so the second must not be disturbed by what the
first left behind), and with the host planner (an implementation that shares no code with the
kernels) at the sizes where the warp-level loops of the table stage run more than once.  The file
name makes pytest collect it after every other test.
"""

import ctypes

import numpy as np
import pytest
import torch

from moonep_b200 import Buffer
from moonep_b200.models.routing import make_routing
from moonep_b200.parallel.world import LocalWorld


def _entry():
    from moonep_b200.ops import _lib

    lib = _lib.load()
    fn = lib.moonep_plan_tables_noalloc  # resolved by its exported name
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] + [ctypes.c_int] * 8 + [ctypes.c_void_p] * 5
    return lib, fn


@pytest.mark.gpu
@pytest.mark.parametrize("R,routing,B", [(4, "biased", 2), (2, "zipf", 3), (1, "softmax", 4)])
def test_noalloc_tables_match_dispatch_tables_twice(R, routing, B):
    lib, fn = _entry()
    S, H, K, epn, P = 64, 32, 4, 4, 16
    E = R * epn
    dev = "cuda"
    lw = LocalWorld(R, dev)
    bufs = lw.run(lambda r: Buffer(S, H, K, E, R, num_sms=4, token_padding=P, B=B, world=lw.view(r)))
    routes = [make_routing(routing, S, K, E, R, r, bias=2.0, seed=21, device=dev) for r in range(R)]

    def body(r):
        topk, tpe, gates = routes[r]
        x = torch.randn(S, H, device=dev).to(torch.bfloat16)
        _, _, cu, plan = bufs[r].dispatch(x, gates, topk, tpe)
        torch.cuda.synchronize()
        return cu.clone(), plan.experts_to_copy.clone(), plan.zero_fill_ranges.clone(), plan.remote_stats.clone()

    want = lw.run(body)
    NvS = bufs[0]._require_ctx()["NvS"]
    tpe_all = torch.stack([routes[r][1] for r in range(R)]).to(torch.int32).contiguous()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        for r in range(R):
            cu = torch.full((E + B,), -7, dtype=torch.int32, device=dev)
            etc = torch.full((R, B), -7, dtype=torch.int32, device=dev)
            zf = torch.full((E + B, 2), -7, dtype=torch.int32, device=dev)
            rs = torch.full((2,), -7, dtype=torch.int32, device=dev)
            rc = fn(tpe_all.data_ptr(), R, E, B, S, K, P, r, NvS, cu.data_ptr(), etc.data_ptr(), zf.data_ptr(),
                    rs.data_ptr(), stream)  # fmt: skip
            assert rc == 0, lib.moonep_last_error().decode()
            torch.cuda.synchronize()
            assert torch.equal(cu, want[r][0]), f"call {call} rank {r}: cu_seqlens differ"
            assert torch.equal(etc, want[r][1]), f"call {call} rank {r}: experts_to_copy differ"
            assert torch.equal(zf, want[r][2]), f"call {call} rank {r}: zero_fill_ranges differ"
            assert torch.equal(rs, want[r][3]), f"call {call} rank {r}: remote_stats differ"
    lw.run(lambda r: bufs[r].destroy())


@pytest.mark.gpu
@pytest.mark.parametrize("R,E,B,S,K,P", [(8, 256, 32, 512, 8, 128), (16, 1024, 8, 64, 4, 16), (4, 64, 3, 96, 6, 32)])
def test_noalloc_tables_match_the_host_planner(R, E, B, S, K, P):
    """E / R > 32 and R = 16: the ballot, scan and argmax loops of the table stage take several rounds."""
    from moonep_b200.cpu import planner as host
    from moonep_b200.layout import compute_layout

    lib, fn = _entry()
    NvS = compute_layout(S, 64, K, E, R, B=B, token_padding=P)["NvS"]
    routes = [make_routing("zipf", S, K, E, R, r, bias=1.5, seed=5) for r in range(R)]
    tpe = np.stack([routes[r][1].numpy() for r in range(R)]).astype(np.int64)
    want = host.global_tables(tpe, S=S, K=K, B=B, token_padding=P, NvS=NvS)
    tpe_dev = torch.from_numpy(tpe).to(torch.int32).cuda().contiguous()
    stream = torch.cuda.current_stream().cuda_stream
    for r in (0, R // 2, R - 1):
        cu = torch.full((E + B,), -7, dtype=torch.int32, device="cuda")
        etc = torch.full((R, B), -7, dtype=torch.int32, device="cuda")
        zf = torch.full((E + B, 2), -7, dtype=torch.int32, device="cuda")
        rs = torch.full((2,), -7, dtype=torch.int32, device="cuda")
        rc = fn(tpe_dev.data_ptr(), R, E, B, S, K, P, r, NvS, cu.data_ptr(), etc.data_ptr(), zf.data_ptr(), rs.data_ptr(),
                stream)  # fmt: skip
        assert rc == 0, lib.moonep_last_error().decode()
        torch.cuda.synchronize()
        assert np.array_equal(cu.cpu().numpy(), want["cu_seqlens"][r]), f"rank {r}: cu_seqlens differ"
        assert np.array_equal(etc.cpu().numpy(), want["experts_to_copy"]), f"rank {r}: experts_to_copy differ"
        assert np.array_equal(zf.cpu().numpy(), want["zero_fill"][r]), f"rank {r}: zero_fill_ranges differ"
        assert np.array_equal(rs.cpu().numpy(), want["remote_stats"][r]), f"rank {r}: remote_stats differ"


@pytest.mark.gpu
def test_noalloc_reports_a_layout_that_does_not_fit():
    """With NvS smaller than the padded rows of the rank, remote_stats[0] comes back as -1."""
    lib, fn = _entry()
    R, E, B, S, K, P = 2, 8, 2, 64, 4, 16
    routes = [make_routing("balanced", S, K, E, R, r, seed=1) for r in range(R)]
    tpe = torch.stack([routes[r][1] for r in range(R)]).to(torch.int32).cuda().contiguous()
    cu = torch.zeros(E + B, dtype=torch.int32, device="cuda")
    etc = torch.zeros(R, B, dtype=torch.int32, device="cuda")
    zf = torch.zeros(E + B, 2, dtype=torch.int32, device="cuda")
    rs = torch.zeros(2, dtype=torch.int32, device="cuda")
    args = (tpe.data_ptr(), R, E, B, S, K, P, 0)
    outs = (cu.data_ptr(), etc.data_ptr(), zf.data_ptr(), rs.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert fn(*args, 16, *outs) == 0  # far too few rows
    torch.cuda.synchronize()
    assert int(rs[0]) == -1
    assert fn(*args, S * K + (P - 1) * 2 * (E // R), *outs) == 0  # the Buffer's own NvS
    torch.cuda.synchronize()
    assert int(rs[0]) >= 0 and int(cu[-1]) <= S * K + (P - 1) * 2 * (E // R)


@pytest.mark.gpu
def test_noalloc_rejects_sizes_beyond_its_work_area():
    lib, fn = _entry()
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    p = dummy.data_ptr()
    rc = fn(p, 17, 17 * 4, 1, 8, 2, 8, 0, 100, p, p, p, p, torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and b"R <= 16" in lib.moonep_last_error()
    rc = fn(p, 2, 4096, 1, 8, 2, 8, 0, 100, p, p, p, p, torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and b"E <= 1024" in lib.moonep_last_error()
    torch.cuda.synchronize()
