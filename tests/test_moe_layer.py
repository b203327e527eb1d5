"""Expert-parallel SwiGLU MoE layer (dispatch -> prefetch -> grouped GEMM -> combine, and its backward
with reduce_grad) against a dense fp32 autograd reference, on emulated worlds."""

import pytest
import torch

from moonep_b200 import Buffer
from moonep_b200.models.moe_layer import ExpertParallelMoE, dense_reference
from moonep_b200.models.routing import make_routing
from moonep_b200.parallel.world import LocalWorld

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("R,routing", [(1, "softmax"), (2, "biased"), (4, "zipf")])
def test_moe_layer_forward_backward_matches_dense_reference(device, R, routing):
    _layer_against_dense(device, R, routing)


@pytest.mark.gpu
@pytest.mark.parametrize("R,routing", [(2, "biased"), (4, "zipf")])
def test_moe_layer_backward_with_reduce_grad_beside_the_gemms(R, routing, monkeypatch):
    """``MOONEP_BWD_OVERLAP=1``: each weight's gradients are reduced on the communication stream as soon as they
    exist, one ``reduce_grad`` per weight, while the remaining GEMMs run on fewer SMs; same results."""
    monkeypatch.setenv("MOONEP_BWD_OVERLAP", "1")
    _layer_against_dense("cuda", R, routing)


def _layer_against_dense(device, R, routing):
    S, H, I, K, epn, Bslots = 96, 256, 256, 2, 2, 1
    E = R * epn
    lw = LocalWorld(R, device)
    bufs = lw.run(lambda r: Buffer(S, H, K, E, R, num_sms=8, token_padding=128, B=Bslots, world=lw.view(r)))
    layers = lw.run(lambda r: ExpertParallelMoE(bufs[r], I, init_std=0.05, seed=3))
    data = []
    for r in range(R):
        topk, tpe, gates = make_routing(routing, S, K, E, R, r, bias=2.0, seed=11)
        g = torch.Generator().manual_seed(100 + r)
        x = (torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16)
        go = (torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16)
        data.append((x, gates, topk, tpe, go))

    def body(r):
        x, gates, topk, tpe, go = (t.to(device) for t in data[r])
        out, saved = layers[r].forward(x, gates, topk, tpe)
        dx, dgates = layers[r].backward(saved, go)
        if device == "cuda":
            torch.cuda.synchronize()
            bufs[r].check_status()
        return out.cpu(), dx.cpu(), dgates.cpu(), [g.cpu().clone() for g in layers[r].owner_grads()]

    res = lw.run(body)
    # dense reference with autograd, all ranks' tokens
    wg = layers[0].w_gate[:E].float().cpu().requires_grad_(True)
    wu = layers[0].w_up[:E].float().cpu().requires_grad_(True)
    wd = layers[0].w_down[:E].float().cpu().requires_grad_(True)
    refs = []
    for r in range(R):
        x, gates, topk, tpe, go = data[r]
        xr = x.float().requires_grad_(True)
        gr = gates.clone().requires_grad_(True)
        out = dense_reference(xr, gr, topk, wg, wu, wd)
        out.backward(go.float())
        refs.append((out.detach(), xr.grad, gr.grad))

    def close(a, b, what, tol=4e-2):
        err = (a.float() - b.float()).abs().max().item()
        scale = max(1e-3, b.float().abs().max().item())
        assert err <= tol * scale, f"{what}: max abs err {err} vs scale {scale}"

    for r in range(R):
        close(res[r][0], refs[r][0], f"rank {r} output")
        close(res[r][1], refs[r][1], f"rank {r} grad_x")
        close(res[r][2], refs[r][2], f"rank {r} grad_gates")
        s = slice(r * epn, (r + 1) * epn)
        close(res[r][3][0], wg.grad[s], f"rank {r} grad W_gate")
        close(res[r][3][1], wu.grad[s], f"rank {r} grad W_up")
        close(res[r][3][2], wd.grad[s], f"rank {r} grad W_down")
    lw.run(lambda r: layers[r].destroy())
    lw.run(lambda r: bufs[r].destroy())


@pytest.mark.parametrize("device", DEVICES)
def test_moe_helper_ops_match_torch(device):
    """Batched expert transpose, SwiGLU backward and the SGD update against plain torch."""
    from moonep_b200.ops.moe_ops import sgd_update, swiglu_bwd, transpose_experts

    g = torch.Generator().manual_seed(5)
    src = torch.randn(3, 128, 192, generator=g).to(torch.bfloat16).to(device)
    dst = torch.zeros(3, 192, 128 + 64, dtype=torch.bfloat16, device=device)
    transpose_experts(src, dst, 64)
    assert torch.equal(dst[:, :, 64:].cpu(), src.transpose(1, 2).cpu()) and not bool(dst[:, :, :64].abs().max() > 0)

    dst2 = torch.full((3, 192, 128), 7.0, dtype=torch.bfloat16, device=device)
    transpose_experts(src, dst2, 0, active=torch.tensor([4, -1, 0], dtype=torch.int32, device=device))
    assert torch.equal(dst2[0].cpu(), src[0].t().cpu()) and torch.equal(dst2[2].cpu(), src[2].t().cpu())
    assert bool((dst2[1] == 7.0).all()), "a skipped matrix was written"

    rows, I, n = 70, 256, 50
    a, u, gg = (torch.randn(rows, I, generator=g).to(torch.bfloat16).to(device) for _ in range(3))
    w = torch.rand(rows, generator=g).to(device)
    dadu = torch.zeros(rows, 2 * I, dtype=torch.bfloat16, device=device)
    hsw = torch.zeros(rows, I, dtype=torch.bfloat16, device=device)
    dgate = torch.zeros(rows, device=device)
    swiglu_bwd(a, u, gg, w, torch.tensor([n], dtype=torch.int32, device=device), dadu, hsw, dgate)
    af, uf, gf, wf = a.float().cpu(), u.float().cpu(), gg.float().cpu(), w.cpu()
    s = torch.sigmoid(af)
    h = af * s * uf
    dh = gf * wf[:, None]
    assert torch.allclose(dgate.cpu()[:n], (gf * h).sum(1)[:n], rtol=2e-3, atol=2e-2)
    assert torch.allclose(dadu.float().cpu()[:n, :I], (dh * uf * s * (1 + af * (1 - s)))[:n], rtol=2e-2, atol=2e-2)
    assert torch.allclose(dadu.float().cpu()[:n, I:], (dh * af * s)[:n], rtol=2e-2, atol=2e-2)
    assert torch.allclose(hsw.float().cpu()[:n], (h * wf[:, None])[:n], rtol=2e-2, atol=2e-2)
    assert not bool(dadu[n:].abs().max() > 0), "rows beyond the total were written"

    wt = torch.randn(4, 128, 64, generator=g).to(torch.bfloat16).to(device)
    gr = torch.randn(4, 128, 64, generator=g).to(device)
    want = (wt.float() - 0.5 * gr).to(torch.bfloat16)
    sgd_update(wt, gr, 0.5)
    assert torch.allclose(wt.float().cpu(), want.float().cpu(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("device", ["cpu"])
def test_moe_block_autograd_matches_dense_reference(device):
    """Router + experts through autograd on one rank: output, input gradient and router gradient against a dense
    fp32 model with the same weights (emulated multi-rank worlds use the layer's explicit backward, see moe_block.py)."""
    from moonep_b200.models.moe_block import MoEBlock

    S, H, I, K, E = 96, 256, 256, 2, 4
    buf = Buffer(S, H, K, E, 1, num_sms=8, token_padding=128, B=1)
    block = MoEBlock(buf, I, init_std=0.05, seed=5)
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16).to(device).requires_grad_(True)
    go = (torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16).to(device)
    out = block(x)
    out.backward(go)
    if device == "cuda":
        torch.cuda.synchronize()
        buf.check_status()
    # dense reference with the same router and expert weights
    wr = block.router.weight.detach().float().cpu().requires_grad_(True)
    ex = block.experts
    wg, wu, wd = (w[:E].float().cpu() for w in (ex.w_gate, ex.w_up, ex.w_down))
    xr = x.detach().float().cpu().requires_grad_(True)
    probs = torch.softmax(xr @ wr.t(), dim=-1)
    top_p, top_i = torch.topk(probs, K, dim=-1)
    gates = top_p / top_p.sum(dim=-1, keepdim=True)
    ref = dense_reference(xr, gates, top_i, wg, wu, wd)
    ref.backward(go.float().cpu())

    def close(a, b, what, tol=4e-2):
        err = (a.float().cpu() - b.float()).abs().max().item()
        scale = max(1e-3, b.float().abs().max().item())
        assert err <= tol * scale, f"{what}: max abs err {err} vs scale {scale}"

    close(out.detach(), ref.detach(), "output")
    close(block.router.weight.grad, wr.grad, "router gradient", tol=6e-2)
    # the input gradient has two parts: through the experts (from the layer) and through the router (from autograd)
    close(x.grad, xr.grad, "input gradient", tol=6e-2)
    block.destroy()
    buf.destroy()


@pytest.mark.parametrize("device", ["cpu"])
def test_expert_shards_save_and_load(device, tmp_path):
    """Every rank checkpoints the experts it owns; a fresh layer that loads the shards computes the same output."""
    R, S, H, I, K, epn = 2, 32, 128, 128, 2, 2
    E = R * epn
    lw = LocalWorld(R, device)
    bufs = lw.run(lambda r: Buffer(S, H, K, E, R, token_padding=16, B=1, world=lw.view(r)))
    layers = lw.run(lambda r: ExpertParallelMoE(bufs[r], I, init_std=0.05, seed=3))
    others = lw.run(lambda r: ExpertParallelMoE(bufs[r], I, init_std=0.05, seed=99))  # different weights

    def body(r):
        path = tmp_path / f"shard{r}.pt"
        torch.save(layers[r].state_dict(), path)
        others[r].load_state_dict(torch.load(path))
        topk, tpe, gates = make_routing("biased", S, K, E, R, r, bias=1.0, seed=4)
        x = (torch.randn(S, H, generator=torch.Generator().manual_seed(r)) * 0.5).to(torch.bfloat16)
        a, _ = layers[r].forward(x, gates, topk, tpe)
        b, _ = others[r].forward(x, gates, topk, tpe)
        return torch.equal(a, b)

    assert all(lw.run(body))
    with pytest.raises(AssertionError):
        bad = layers[0].state_dict()
        bad["first_expert"] = 1
        layers[0].load_state_dict(bad)
    lw.run(lambda r: layers[r].destroy())
    lw.run(lambda r: others[r].destroy())
    lw.run(lambda r: bufs[r].destroy())


@pytest.mark.parametrize("device", ["cpu"])
def test_owned_expert_updates_reach_the_other_ranks_copies(device):
    """Without peer mapping every rank keeps a copy of all experts: an optimizer step on the owners must show up in
    every copy (what the peer mapping gives for free on real GPUs), so that later prefetches read current weights."""
    R, S, H, I, K, epn = 2, 32, 128, 128, 2, 2
    E = R * epn
    lw = LocalWorld(R, device)
    bufs = lw.run(lambda r: Buffer(S, H, K, E, R, token_padding=16, B=1, world=lw.view(r)))
    layers = lw.run(lambda r: ExpertParallelMoE(bufs[r], I, init_std=0.05, seed=3))

    def body(r):
        topk, tpe, gates = make_routing("biased", S, K, E, R, r, bias=1.0, seed=4)
        g = torch.Generator().manual_seed(r)
        x = (torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16)
        go = (torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16)
        before = layers[r].w_gate[:E].clone()
        out, saved = layers[r].forward(x, gates, topk, tpe)
        layers[r].backward(saved, go)
        layers[r].sgd_step(0.5)
        return before, layers[r].w_gate[:E].clone(), layers[r].w_down[:E].clone()

    res = lw.run(body)
    assert torch.equal(res[0][1], res[1][1]) and torch.equal(res[0][2], res[1][2]), "the ranks' copies diverged"
    assert not torch.equal(res[0][0], res[0][1]), "the step changed nothing"
    lw.run(lambda r: layers[r].destroy())
    lw.run(lambda r: bufs[r].destroy())


def test_expert_adamw_matches_torch_adamw():
    """fp32 master weights and moments for the owned experts; the same numbers as torch.optim.AdamW on fp32 copies."""
    from moonep_b200.models.optim import ExpertAdamW

    S, H, I, K, E = 32, 128, 128, 2, 2
    buf = Buffer(S, H, K, E, 1, token_padding=16, B=1)
    layer = ExpertParallelMoE(buf, I, init_std=0.05, seed=3)
    opt = ExpertAdamW(layer, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref_params = [torch.nn.Parameter(w.float().clone()) for w in layer.owner_weights()]
    ref = torch.optim.AdamW(ref_params, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    g = torch.Generator().manual_seed(0)
    for _ in range(3):
        for p, gr in zip(ref_params, layer.owner_grads()):
            gr.copy_(torch.randn(gr.shape, generator=g) * 0.1)
            p.grad = gr.clone()
        opt.step()
        ref.step()
    for p, m, w in zip(ref_params, opt.master, layer.owner_weights()):
        assert torch.allclose(m, p.detach(), rtol=1e-5, atol=1e-6)
        assert torch.equal(w, m.to(torch.bfloat16)), "the symmetric bf16 weights are the rounded master weights"
    state = opt.state_dict()
    opt2 = ExpertAdamW(layer)
    opt2.load_state_dict(state)
    assert opt2.steps == 3 and torch.equal(opt2.exp_avg[0], opt.exp_avg[0])
    layer.destroy()
    buf.destroy()


@pytest.mark.parametrize("device", ["cpu"])
@pytest.mark.parametrize("R", [1, 2])
def test_inference_forward_equals_training_forward(device, R):
    """``save_for_backward=False`` keeps nothing and reads the dispatched rows in place; same output."""
    S, H, I, K, epn = 48, 128, 128, 2, 2
    E = R * epn
    lw = LocalWorld(R, device)
    bufs = lw.run(lambda r: Buffer(S, H, K, E, R, token_padding=16, B=1, world=lw.view(r)))
    layers = lw.run(lambda r: ExpertParallelMoE(bufs[r], I, init_std=0.05, seed=3))

    def body(r):
        topk, tpe, gates = make_routing("biased", S, K, E, R, r, bias=1.5, seed=4, device=device)
        x = (torch.randn(S, H, generator=torch.Generator().manual_seed(r)) * 0.5).to(torch.bfloat16).to(device)
        a, saved = layers[r].forward(x, gates, topk, tpe)
        b, none = layers[r].forward(x, gates, topk, tpe, save_for_backward=False)
        return saved is not None and none is None and torch.equal(a, b)

    assert all(lw.run(body))
    lw.run(lambda r: layers[r].destroy())
    lw.run(lambda r: bufs[r].destroy())
