"""CUDA-graph capture of Buffer operations: one captured dispatch -> combine step is replayed with
changing inputs, mixed with ordinary calls, and must keep the flag epochs of all kernels in step."""

import pytest
import torch

from moonep_b200 import Buffer
from moonep_b200.models.routing import make_routing

pytestmark = pytest.mark.gpu


def _expected(x, K):
    return (x.float() * K).to(torch.bfloat16)


@pytest.mark.parametrize("fuse_publish", ["0", "1"], ids=["publish_kernel", "publish_fused"])
def test_captured_round_trip_replays_and_mixes_with_eager_calls(fuse_publish, monkeypatch):
    # with MOONEP_FUSE_PUBLISH=1 the tokens-per-expert exchange is the first step of the dispatch kernel
    monkeypatch.setenv("MOONEP_FUSE_PUBLISH", fuse_publish)
    S, H, K, E = 256, 512, 4, 8
    buf = Buffer(S, H, K, E, 1, num_sms=8, token_padding=16, explicitly_destroy=True)
    be = buf._require_ctx()["_backend"]
    be.set_timeout_ms(2000)
    topk, tpe, gates = make_routing("biased", S, K, E, 1, 0, bias=1.5, seed=3, device="cuda")
    x = torch.randn(S, H, device="cuda").to(torch.bfloat16)

    def step():
        xn, wn, cu, plan = buf.dispatch(x, gates, topk, tpe, zero_copy=True)
        out, wb, _ = buf.combine(plan, xn, wn, zero_copy=True)
        return out, wb, cu

    graph_step = buf.capture(step)
    epochs_before = list(be.epoch)
    for i in range(3):
        x.copy_(torch.randn(S, H, device="cuda").to(torch.bfloat16))
        out, wb, cu = graph_step.replay()
        torch.cuda.synchronize()
        buf.check_status()
        assert torch.equal(out, _expected(x, K)), f"replay {i}"
        assert torch.equal(wb, gates)
        assert int(cu[-1]) >= S * K
    per_replay = [b - a for a, b in zip(epochs_before, be.epoch)]
    assert all(d % 3 == 0 for d in per_replay) and sum(per_replay) > 0
    # an ordinary call between replays: its kernels must see the epochs the replays left behind
    x2 = torch.randn(S, H, device="cuda").to(torch.bfloat16)
    xn, wn, cu2, plan = buf.dispatch(x2, gates, topk, tpe)
    out2, wb2, _ = buf.combine(plan, xn, wn)
    torch.cuda.synchronize()
    buf.check_status()
    assert torch.equal(out2, _expected(x2, K)) and torch.equal(wb2, gates)
    # and a replay after the ordinary call (needs the bias to be set again)
    x.copy_(x2)
    out, wb, _ = graph_step.replay()
    out_b, _, _ = graph_step.replay()
    torch.cuda.synchronize()
    buf.check_status()
    assert torch.equal(out, _expected(x2, K)) and out_b.data_ptr() == out.data_ptr()
    assert graph_step.replays == 5
    st = buf.stats()
    assert "flag_wait_max_us" in st and "flag_waits_that_spun" in st
    buf.destroy()


def test_captured_plan_replay_and_async_operations():
    """A captured step that re-dispatches with a saved plan on the communication stream."""
    S, H, K, E = 128, 256, 2, 4
    buf = Buffer(S, H, K, E, 1, num_sms=4, token_padding=8, explicitly_destroy=True)
    buf._require_ctx()["_backend"].set_timeout_ms(2000)
    topk, tpe, gates = make_routing("balanced", S, K, E, 1, 0, device="cuda")
    x = torch.randn(S, H, device="cuda").to(torch.bfloat16)
    _, _, _, plan = buf.dispatch(x, gates, topk, tpe)
    saved = plan.clone()

    def step():
        xn, wn, cu, _, ev = buf.dispatch(x, plan=saved, async_finish=True)
        ev.wait()
        out, _, ev2 = buf.combine(saved, xn, None, async_finish=True)
        ev2.wait()
        return out

    graph_step = buf.capture(step)
    for _ in range(2):
        x.copy_(torch.randn(S, H, device="cuda").to(torch.bfloat16))
        out = graph_step.replay()
        torch.cuda.synchronize()
        buf.check_status()
        assert torch.equal(out, _expected(x, K))
    buf.destroy()
