"""tcgen05 grouped GEMM against a per-group fp32 torch reference."""

import pytest
import torch

from moonep_b200.ops.grouped_gemm import grouped_gemm, grouped_gemm_reference


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


def test_reference_on_cpu_matches_dense():
    x, w, w2, cu, scale, total = _case(3, [128, 0, 256], 64, 256, device="cpu")
    y = grouped_gemm(x, w, cu)
    assert torch.allclose(y[:128].float(), (x[:128].float() @ w[0].float().t()), atol=2e-2, rtol=2e-2)
    assert torch.allclose(y[128:384].float(), (x[128:384].float() @ w[2].float().t()), atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
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
def test_grouped_gemm_matches_fp32_reference(mode, G, rows, K, N):
    x, w, w2, cu, scale, total = _case(G, rows, K, N)
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    kw = {"w_up": w2} if mode == "swiglu" else ({"row_scale": scale} if mode == "scale" else {})
    y = grouped_gemm(x, w, cu, mode=mode, status=status, **kw)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, f"kernel reported status {status.tolist()}"
    ref = grouped_gemm_reference(x, w, cu, mode=mode, **kw)
    got, want = y[:total].float(), ref[:total].float()
    err = (got - want).abs().max().item()
    tol = 2e-2 * max(1.0, want.abs().max().item())
    assert err <= tol, f"max abs err {err} > {tol}"
    # twice in a row on the same buffers (TMEM and barriers are re-initialised per launch)
    y2 = grouped_gemm(x, w, cu, mode=mode, status=status, **kw)
    torch.cuda.synchronize()
    assert torch.equal(y[:total], y2[:total])
