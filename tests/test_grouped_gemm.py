"""tcgen05 grouped GEMM against a per-group fp32 torch reference."""

import pytest
import torch

from moonep_b200.ops.grouped_gemm import grouped_gemm, grouped_gemm_reference


def grouped_gemm_reference_fp32(x, w, cu):
    """``x[rows of g] @ w[g].T`` in fp32 without the final rounding to bf16."""
    out = torch.zeros(x.shape[0], w.shape[1], dtype=torch.float32, device=x.device)
    start = 0
    for g, end in enumerate(cu.tolist()):
        if end > start:
            out[start:end] = x[start:end].float() @ w[g].float().t()
        start = max(start, end)
    return out


def _case(G, rows_per_group, K, N, seed=0, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    ends, total = [], 0
    for r in rows_per_group:
        total += r
        ends.append(total)
    rows_cap = total + 256
    x = (torch.randn(rows_cap, K, generator=g) * 0.5).to(torch.bfloat16).to(device)
    w = (torch.randn(G, N, K, generator=g) * 0.05).to(torch.bfloat16).to(device)
    w2 = (torch.randn(G, N, K, generator=g) * 0.05).to(torch.bfloat16).to(device)
    cu = torch.tensor(ends, dtype=torch.int32, device=device)
    scale = torch.rand(rows_cap, generator=g).to(device)
    return x, w, w2, cu, scale, total


def _group_of_rows(cu, total):
    """Group index of every row below ``total`` (ends are cumulative)."""
    ends = cu.to(torch.int64)
    return torch.searchsorted(ends, torch.arange(total, device=cu.device), right=True)


def _abs_dot(x, w, cu, total):
    """``sum_k |x[r, k]| * |w[g(r), n, k]|``: the scale of the rounding error of one output element."""
    out = torch.zeros(total, w.shape[1], dtype=torch.float32, device=x.device)
    start = 0
    for g, end in enumerate(cu.tolist()):
        if end > start:
            out[start:end] = x[start:end].float().abs() @ w[g].float().abs().t()
        start = max(start, end)
    return out


# A bf16 result is within one rounding (2^-9 relative) of the exact value plus the error of the fp32 accumulation,
# which over K / 16 tensor-core steps stays below (K / 16) * 2^-23 of the sum of absolute products: 1.6e-5 at K = 2048.
BF16_REL = 2.0**-8
ACC_REL = 5e-5


def _assert_elementwise(got, want, scale, what):
    """|got - want| <= 2^-8 |want| + ACC_REL * scale, element by element; a lost 64-wide K block is far outside."""
    bound = BF16_REL * want.abs() + ACC_REL * scale + 1e-30
    excess = ((got - want).abs() / bound).max().item()
    assert excess <= 1.0, f"{what}: an element is {excess:.2f} times its error bound away from the fp32 reference"


def test_elementwise_bound_catches_a_dropped_k_block():
    x, w, w2, cu, scale, total = _case(2, [128, 128], 256, 128, device="cpu")
    want = torch.cat([x[:128].float() @ w[0].float().t(), x[128:256].float() @ w[1].float().t()])
    ad = _abs_dot(x, w, cu, total)
    _assert_elementwise(want.to(torch.bfloat16).float(), want, ad, "exact")
    xd = x.clone()
    xd[:, 64:128] = 0  # the second K block never reaches the accumulator
    bad = torch.cat([xd[:128].float() @ w[0].float().t(), xd[128:256].float() @ w[1].float().t()])
    with pytest.raises(AssertionError):
        _assert_elementwise(bad.to(torch.bfloat16).float(), want, ad, "dropped block")


def test_reference_on_cpu_matches_dense():
    x, w, w2, cu, scale, total = _case(3, [128, 0, 256], 64, 256, device="cpu")
    y = grouped_gemm(x, w, cu)
    assert torch.allclose(y[:128].float(), (x[:128].float() @ w[0].float().t()), atol=2e-2, rtol=2e-2)
    assert torch.allclose(y[128:384].float(), (x[128:384].float() @ w[2].float().t()), atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("pair", [False, True], ids=["cta", "cta_pair"])
@pytest.mark.parametrize("mode", ["plain", "swiglu", "scale"])
@pytest.mark.parametrize(
    "G,rows,K,N",
    [
        (1, [128], 64, 256),
        (2, [128, 256], 256, 512),
        (5, [256, 0, 128, 384, 0], 512, 256),
        (8, [1024, 128, 0, 640, 256, 128, 0, 512], 1024, 768),
        (36, [128 * ((i * 7) % 5) for i in range(36)], 2048, 512),
    ],
)
def test_grouped_gemm_matches_fp32_reference(mode, G, rows, K, N, pair):
    x, w, w2, cu, scale, total = _case(G, rows, K, N)
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    kw = {"w_up": w2} if mode == "swiglu" else ({"row_scale": scale} if mode == "scale" else {})
    kw["pair"] = pair
    y = grouped_gemm(x, w, cu, mode=mode, status=status, **kw)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, f"kernel reported status {status.tolist()}"
    kw.pop("pair")
    ref = grouped_gemm_reference(x, w, cu, mode=mode, **kw)
    kw["pair"] = pair
    # the oracle in fp32 before its final rounding, and the error scale of every element
    got = y[:total].float()
    ad = _abs_dot(x, w, cu, total)
    acc = grouped_gemm_reference_fp32(x, w, cu)[:total]
    if mode == "plain":
        want, scale_el = acc, ad
    elif mode == "scale":
        want, scale_el = acc * scale[:total, None], ad * scale[:total, None].abs()
    else:
        up = grouped_gemm_reference_fp32(x, w2, cu)[:total]
        sig = torch.sigmoid(acc)
        want = acc * sig * up
        # d silu / d a is bounded by 1.1; the fast exponential adds a few 2^-22 relative
        scale_el = 1.1 * ad * up.abs() + _abs_dot(x, w2, cu, total) * (acc * sig).abs() + 0.05 * want.abs()
    _assert_elementwise(got, want, scale_el, mode)
    assert (got - ref[:total].float()).abs().max().item() <= 2.0**-7 * max(1e-3, want.abs().max().item())
    # twice in a row on the same buffers (TMEM and barriers are re-initialised per launch)
    y2 = grouped_gemm(x, w, cu, mode=mode, status=status, **kw)
    torch.cuda.synchronize()
    assert torch.equal(y[:total], y2[:total])
    if mode == "swiglu":  # the same pass can keep both pre-activations
        pre = (torch.zeros_like(y), torch.zeros_like(y))
        y3 = grouped_gemm(x, w, cu, mode=mode, status=status, save_pre=pre, **kw)
        torch.cuda.synchronize()
        assert torch.equal(y3[:total], y[:total])
        for got_pre, wt in zip(pre, (w, w2)):
            want_pre = grouped_gemm_reference_fp32(x, wt, cu)[:total]
            _assert_elementwise(got_pre[:total].float(), want_pre, _abs_dot(x, wt, cu, total), "pre-activation")


def _wgrad_case(rows, P, Q, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    ends, total = [], 0
    for r in rows:
        total += r
        ends.append(total)
    cap = (total + 64 + 63) // 64 * 64
    left = (torch.randn(cap, P, generator=g) * 0.5).to(torch.bfloat16).to(device)
    right = (torch.randn(cap, Q, generator=g) * 0.5).to(torch.bfloat16).to(device)
    cu = torch.tensor(ends, dtype=torch.int32, device=device)
    return left, right, cu, cap


def test_wgrad_reference_semantics_on_cpu():
    from moonep_b200.ops.grouped_gemm import grouped_wgrad_reference

    left, right, cu, cap = _wgrad_case([32, 0, 16, 0], 8, 4)
    tg = [torch.full((8, 4), 7.0) for _ in range(4)]
    tg[2] = None
    grouped_wgrad_reference(left, right, cu, tg, [1, 0, 0, 2])
    assert torch.allclose(tg[0], 7.0 + left[:32].float().t() @ right[:32].float())
    assert not bool(tg[1].abs().max() > 0), "an empty group with the store flag is zeroed"
    assert bool((tg[3] == 7.0).all()), "an empty group with the keep flag is left alone"


@pytest.mark.gpu
@pytest.mark.parametrize("layout", ["transposed", "rows"])
@pytest.mark.parametrize(
    "rows,P,Q",
    [
        ([128], 128, 256),
        ([64, 0, 192, 16, 80], 256, 256),
        ([256, 128, 0, 0, 1024, 48, 128, 0], 128, 512),
        ([128 * ((i * 5) % 4) for i in range(20)], 384, 768),
    ],
)
def test_grouped_wgrad_matches_fp32_reference(rows, P, Q, layout):
    from moonep_b200.ops.grouped_gemm import grouped_wgrad, grouped_wgrad_reference, grouped_wgrad_rows
    from moonep_b200.ops.moe_ops import transpose_experts

    G = len(rows)
    left, right, cu, cap = _wgrad_case(rows, P, Q, seed=len(rows), device="cuda")
    if layout == "transposed":
        lt = transpose_experts(left.unsqueeze(0), torch.empty(1, P, cap, dtype=torch.bfloat16, device="cuda"))[0]
        rt = transpose_experts(right.unsqueeze(0), torch.empty(1, Q, cap, dtype=torch.bfloat16, device="cuda"))[0]

        def run(ptrs_t, flags_t):
            grouped_wgrad(lt, rt, cu, ptrs_t, flags_t, status=status)
    else:  # the operands as they are, the left one as a column slice of a wider tensor
        wide = torch.cat([torch.full_like(left, 3.0), left], dim=1)
        left_view = wide[:, P:]

        def run(ptrs_t, flags_t):
            grouped_wgrad_rows(left_view, right, cu, ptrs_t, flags_t, status=status)
    flag_list = [(0, 1, 2)[g % 3] for g in range(G)]
    skipped = G - 1 if rows[-1] == 0 else None  # a group without a target is allowed when it has no rows
    init = torch.randn(G, P, Q, device="cuda")
    out = init.clone()
    ptrs = [out[g].data_ptr() for g in range(G)]
    if skipped is not None:
        ptrs[skipped] = 0
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    flags = torch.tensor(flag_list, dtype=torch.int32, device="cuda")
    run(torch.tensor(ptrs, dtype=torch.int64, device="cuda"), flags)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, f"kernel reported status {status.tolist()}"
    want = init.clone().cpu()
    targets = [None if g == skipped else want[g] for g in range(G)]
    grouped_wgrad_reference(left.cpu(), right.cpu(), cu.cpu(), targets, flag_list)
    # fp32 results: the accumulation error only, scaled by the sum of absolute products of each element
    ad = torch.zeros(G, P, Q)
    start = 0
    for g, end in enumerate(cu.tolist()):
        if end > start:
            ad[g] = left[start:end].float().abs().cpu().t() @ right[start:end].float().abs().cpu()
        start = max(start, end)
    bound = ACC_REL * ad + 2.0**-22 * want.abs() + 1e-30
    excess = ((out.cpu() - want).abs() / bound).max().item()
    assert excess <= 1.0, f"an element is {excess:.2f} times its error bound away from the fp32 reference"
    # again on the same buffers: accumulating groups add a second time, the others give the same result
    run(torch.tensor(ptrs, dtype=torch.int64, device="cuda"), flags)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    grouped_wgrad_reference(left.cpu(), right.cpu(), cu.cpu(), targets, flag_list)
    excess = ((out.cpu() - want).abs() / (2 * bound)).max().item()
    assert excess <= 1.0, f"second launch: an element is {excess:.2f} times its error bound away"


def test_kn_reference_on_cpu():
    from moonep_b200.ops.grouped_gemm import grouped_gemm_kn

    g = torch.Generator().manual_seed(1)
    x = torch.randn(48, 24, generator=g).to(torch.bfloat16)
    w0 = torch.randn(2, 16, 8, generator=g).to(torch.bfloat16)
    w1 = torch.randn(2, 8, 8, generator=g).to(torch.bfloat16)
    cu = torch.tensor([16, 48], dtype=torch.int32)
    y = grouped_gemm_kn(x, [w0, w1], cu)
    want = x[16:48].float() @ torch.cat([w0[1], w1[1]]).float()
    assert torch.allclose(y[16:48].float(), want, atol=0.1, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize(
    "rows,Ks,N",
    [
        ([128], [64], 256),
        ([256, 0, 128], [128, 64], 256),
        ([384, 128, 0, 640], [512], 512),
        ([128 * ((i * 3) % 4) for i in range(12)], [256, 256], 768),
    ],
)
def test_grouped_gemm_kn_matches_fp32_reference(rows, Ks, N):
    """Weights given as [G, K, N] (the activation-gradient product), staged as MN-major tiles by the CTA-pair kernel."""
    from moonep_b200.ops.grouped_gemm import grouped_gemm_kn, grouped_gemm_kn_reference

    g = torch.Generator().manual_seed(len(rows))
    G, total = len(rows), sum(rows)
    cu = torch.tensor([sum(rows[: i + 1]) for i in range(G)], dtype=torch.int32, device="cuda")
    x = (torch.randn(total + 256, sum(Ks), generator=g) * 0.5).to(torch.bfloat16).cuda()
    ws = [(torch.randn(G, k, N, generator=g) * 0.05).to(torch.bfloat16).cuda() for k in Ks]
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    y = grouped_gemm_kn(x, ws, cu, status=status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, f"kernel reported status {status.tolist()}"
    wcat = torch.cat(ws, dim=1).transpose(1, 2).contiguous()  # [G, N, K]
    want = grouped_gemm_reference_fp32(x, wcat, cu)[:total]
    _assert_elementwise(y[:total].float(), want, _abs_dot(x, wcat, cu, total), "kn")
    ref = grouped_gemm_kn_reference(x, ws, cu)[:total].float()
    assert (y[:total].float() - ref).abs().max().item() <= 2.0**-7 * max(1e-3, want.abs().max().item())


@pytest.mark.parametrize("seed", range(6))
def test_pair_tile_schedule_covers_every_block_once(seed):
    """The CTA-pair kernel's tile walk (compiled host-side from the same code): over all pairs, every 128-row
    block of every group appears exactly once per column tile, in its own group, and a pair never straddles groups."""
    import ctypes

    import numpy as np

    from moonep_b200.ops import _lib

    lib = _lib.load()
    rng = np.random.default_rng(seed)
    G = int(rng.integers(1, 40))
    blocks = rng.integers(0, 6, size=G) * (rng.random(G) < 0.7)
    ends = np.cumsum(blocks * 128).astype(np.int32)
    rows_cap = int(ends[-1]) + 256 if seed % 2 else max(128, int(ends[-1]) - 128)  # also a capacity that cuts the tail
    n_tiles, npairs = int(rng.integers(1, 5)), int(rng.integers(1, 9))
    seen = {}
    for pair in range(npairs):
        out = np.zeros(4 * 4096, dtype=np.int32)
        n = lib.moonep_pair_schedule(ends.ctypes.data_as(ctypes.c_void_p), G, rows_cap, n_tiles, pair, npairs,
                                     out.ctypes.data_as(ctypes.c_void_p), 4096)  # fmt: skip
        assert 0 <= n <= 4096
        for g, r0, r1, nb in out[: 4 * n].reshape(n, 4):
            start = min(int(ends[g - 1]), rows_cap) if g > 0 else 0
            end = min(int(ends[g]), rows_cap)
            for r in (r0, r1):
                if r >= 0:
                    assert start <= r and r + 128 <= end, f"block at row {r} is not inside group {g}"
                    assert (int(r), int(nb)) not in seen, "a block was scheduled twice"
                    seen[(int(r), int(nb))] = g
            assert r0 >= 0 and (r1 == -1 or r1 == r0 + 128)
    want = set()
    for g in range(G):
        start = min(int(ends[g - 1]), rows_cap) if g > 0 else 0
        end = min(int(ends[g]), rows_cap)
        for r in range(start, end - 127, 128):
            for nb in range(n_tiles):
                want.add((r, nb))
    assert set(seen) == want
