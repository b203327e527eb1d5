"""prefetch_weight, reduce_grad, plan replay and failure reporting on emulated worlds
(CPU backend always; the sm_100a kernels with R emulated ranks on one GPU when marked gpu).

Parity: reference tests/test_prefetch.py:45-156 (holes, duplicates, empty plan, sentinel slots),
tests/test_grad_reduce.py:232-350 (bitwise order, fan-in, empty plan, repeated launch) and
tests/test_dispatch.py:345-411 (hidden-only dispatch with a saved plan).
"""

import dataclasses

import pytest
import torch

from moonep_b200 import Buffer
from moonep_b200.models.routing import make_routing
from moonep_b200.parallel.world import LocalWorld

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def _world(R, device, S=32, H=64, K=2, epn=4, B=3, num_sms=5):
    lw = LocalWorld(R, device)
    bufs = lw.run(lambda r: Buffer(S, H, K, R * epn, R, num_sms=num_sms, token_padding=8, B=B, world=lw.view(r)))
    return lw, bufs


def _plans(lw, bufs, R, S, H, K, E, device):
    def body(r):
        topk, tpe, gates = make_routing("biased", S, K, E, R, r, bias=1.5, seed=5, device=device)
        x = torch.randn(S, H, device=device).to(torch.bfloat16)
        return bufs[r].dispatch(x, gates, topk, tpe)[3]

    return lw.run(body)


TABLES = {
    "holes_and_duplicates": lambda R, B, E, epn: [[(-1 if b == 1 else ((r + 1) % R) * epn) for b in range(B)] for r in range(R)],
    "empty": lambda R, B, E, epn: [[-1] * B for _ in range(R)],
    "fan_in": lambda R, B, E, epn: [[(0 if r != 0 else epn) for _ in range(B)] for r in range(R)],
    # one rank only sends (to the last rank's experts), the others only receive or idle
    "send_only_rank0": lambda R, B, E, epn: [[(E - 1 - b % epn if r == 0 else -1) for b in range(B)] for r in range(R)],
    # a rank's slot may hold one of its own experts, and the same expert twice
    "self_send": lambda R, B, E, epn: [[r * epn + (b // 2) % epn for b in range(B)] for r in range(R)],
    "random": None,
    "random_seed2": None,
    "random_seed3": None,
}
_SEEDS = {"random": 17, "random_seed2": 202, "random_seed3": 3003}


def _table(name, R, B, E, epn):
    if TABLES[name] is not None:
        return torch.tensor(TABLES[name](R, B, E, epn), dtype=torch.int32)
    g = torch.Generator().manual_seed(_SEEDS[name])
    t = torch.randint(-1, E, (R, B), generator=g).to(torch.int32)
    return t


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize(
    "Hw,Hp,epn,B,num_sms",
    [(128, 128, 1, 1, 1), (256, 128, 2, 2, 7), (128, 384, 3, 4, 2), (384, 256, 2, 1, 64)],
    ids=["one_tile_epn1_one_sm", "tall", "wide_more_slots", "more_sms_than_pieces"],
)
def test_prefetch_and_reduce_grad_shapes(device, Hw, Hp, epn, B, num_sms):
    """Expert shapes, slot counts and SM budgets around the kernels' piece sizes (parity: reference
    tests/test_prefetch.py:45-156 single tile / rectangular / more SMs than tiles, tests/test_grad_reduce.py epn=1)."""
    _prefetch_and_reduce_grad(device, "random_seed2", 2, Hw=Hw, Hp=Hp, epn=epn, B=B, num_sms=num_sms)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("table", list(TABLES))
@pytest.mark.parametrize("R", [2, 4])
def test_prefetch_and_reduce_grad(device, table, R):
    _prefetch_and_reduce_grad(device, table, R)


@pytest.mark.gpu
@pytest.mark.parametrize("table", ["fan_in", "random"])
@pytest.mark.parametrize("path", ["bulk", "ldst"])
def test_reduce_grad_on_every_copy_path(table, path, monkeypatch):
    """The TMA-ring (``MOONEP_GRAD_PATH=bulk``) and register (``ldst``) variants of the gradient accumulation keep the
    bitwise order of the additions; the prefetch runs on its register kernel (``ldst``) and its cp.async ring."""
    monkeypatch.setenv("MOONEP_GRAD_PATH", path)
    monkeypatch.setenv("MOONEP_PREFETCH_PATH", "ldst" if path == "ldst" else "async")
    _prefetch_and_reduce_grad("cuda", table, 4)


@pytest.mark.gpu
@pytest.mark.parametrize("path", ["async", "ldst"])
@pytest.mark.parametrize("stages", ["2", "4", "6"])
def test_prefetch_paths_on_odd_sizes(path, stages, monkeypatch):
    """Experts that are a few 2 KB stages long (fewer than the ring is deep, with one SM) and many slots per expert,
    on the register kernel and on cp.async rings of several depths."""
    monkeypatch.setenv("MOONEP_PREFETCH_PATH", path)
    monkeypatch.setenv("MOONEP_RING_STAGES", stages)
    _prefetch_and_reduce_grad("cuda", "fan_in", 4, Hw=384, Hp=128, epn=2, B=4, num_sms=3)
    _prefetch_and_reduce_grad("cuda", "random_seed2", 2, Hw=128, Hp=128, epn=1, B=1, num_sms=1)
    # 36 slots hold the same expert
    _prefetch_and_reduce_grad("cuda", "fan_in", 4, Hw=128, Hp=128, epn=2, B=12, num_sms=2)


@pytest.mark.parametrize("device", DEVICES)
def test_reduce_grad_one_weight_at_a_time(device):
    """A weight whose gradient and reduce buffer are both None is left out; three calls with one weight each
    (the first two asynchronous, on the communication stream) give what one call with all three gives."""
    _prefetch_and_reduce_grad(device, "random", 2, one_by_one=True)


def _prefetch_and_reduce_grad(device, table, R, Hw=128, Hp=256, epn=4, B=3, num_sms=5, one_by_one=False):
    S, H, K = 32, 64, 2
    E = R * epn
    lw, bufs = _world(R, device, S, H, K, epn, B, num_sms=num_sms)
    plans = _plans(lw, bufs, R, S, H, K, E, device)
    etc = _table(table, R, B, E, epn)

    def expert(t, e):
        return torch.full((Hw, Hp), float(10 * t + e % 7), dtype=torch.bfloat16)

    def slot(t, src, b):
        return torch.randn(Hw, Hp, generator=torch.Generator().manual_seed(1000 * t + src * B + b))

    def grad0(t, e):
        return torch.randn(Hw, Hp, generator=torch.Generator().manual_seed(77000 + 100 * t + e))

    shared_red = [torch.zeros(R, B, Hw, Hp, dtype=torch.float32, device=device) for _ in range(3)]

    def body(r):
        plan = dataclasses.replace(plans[r], experts_to_copy=etc.to(device))
        fulls = []
        for t in range(3):
            full = torch.stack([expert(t, e) for e in range(E)] + [torch.full((Hw, Hp), -123.0, dtype=torch.bfloat16)] * B)
            fulls.append(full.to(device).contiguous())
        bufs[r].prefetch_weight(plan, full_gate_weight=fulls[0], full_up_weight=fulls[1], full_down_weight=fulls[2])
        grads = [torch.stack([grad0(t, e) for e in range(E)] + [torch.zeros(Hw, Hp)] * B).to(device) for t in range(3)]
        for t in range(3):
            for b in range(B):
                shared_red[t][r, b].copy_(slot(t, r, b))
        if device == "cuda":
            torch.cuda.synchronize()
        lw.view(r).step()
        for _rep in range(2):  # the second call finds the consumed slots cleared and must add zeros
            if one_by_one:
                for t in (2, 0, 1):
                    sel = [None] * 6
                    sel[t], sel[3 + t] = grads[t], shared_red[t]
                    ev = bufs[r].reduce_grad(plan, t != 1, *sel)
                    if ev is not None:
                        ev.wait()
                continue
            bufs[r].reduce_grad(plan, False, grads[0], grads[1], grads[2], shared_red[0], shared_red[1], shared_red[2])
        if device == "cuda":
            torch.cuda.synchronize()
            bufs[r].check_status()
        lw.view(r).step()
        return [f.cpu() for f in fulls], [g.cpu() for g in grads]

    res = lw.run(body)
    for r in range(R):
        fulls, grads = res[r]
        for t in range(3):
            for b in range(B):
                e = int(etc[r, b])
                want = expert(t, e) if e >= 0 else torch.full((Hw, Hp), -123.0, dtype=torch.bfloat16)
                assert torch.equal(fulls[t][E + b], want), f"rank {r} tensor {t} slot {b}"
            for e in range(E):
                want = grad0(t, e)
                if e // epn == r:
                    for src in range(R):
                        for b in range(B):
                            if int(etc[src, b]) == e:
                                want = want + slot(t, src, b)
                assert torch.equal(grads[t][e], want), f"rank {r} tensor {t} expert {e}: reduce_grad not bitwise equal"
    for t in range(3):
        red = shared_red[t].cpu()
        for r in range(R):
            for b in range(B):
                if int(etc[r, b]) >= 0:
                    assert not bool(red[r, b].abs().max() > 0), "consumed slot not cleared"
                else:
                    assert torch.equal(red[r, b], slot(t, r, b)), "unused slot modified"
    lw.run(lambda r: bufs[r].destroy())


@pytest.mark.parametrize("device", DEVICES)
def test_saved_plan_replay_leaves_weights_and_dedup_untouched(device):
    R, S, H, K, epn, B = 2, 48, 32, 4, 2, 1
    E = R * epn
    lw, bufs = _world(R, device, S, H, K, epn, B)

    def body(r):
        buf = bufs[r]
        ctx = buf._require_ctx()
        topk, tpe, gates = make_routing("biased", S, K, E, R, r, bias=2.0, seed=9, device=device)
        x = torch.randn(S, H, device=device).to(torch.bfloat16)
        xn, wn, cu, plan = buf.dispatch(x, gates, topk, tpe)
        snap = plan.clone()
        wbuf = ctx["weights_buf_local"].clone()
        x2 = (x.float() * 3).to(torch.bfloat16)
        xn2, wn2, cu2, plan2 = buf.dispatch(x2, None, plan=snap)
        assert wn2 is None and cu2 is None and plan2 is snap
        occ = ctx["meta_buf"][r * ctx["meta_chunk_padded"] + ctx["SRC_INFO_OFF"]:][: ctx["NvS"]] >= 0
        ok_rows = torch.equal((xn.float() * 3).to(torch.bfloat16)[occ], xn2[occ])
        ok_w = torch.equal(ctx["weights_buf_local"], wbuf)
        ok_plan = all(torch.equal(getattr(plan, f), getattr(snap, f)) for f in ("dst", "dup_groups", "dup_loffs", "dup_counts"))
        o1, _, _ = buf.combine(snap, xn2, None)
        o2, _, _ = buf.combine(snap, xn2, None, inter_rank_sync=True)
        if device == "cuda":
            torch.cuda.synchronize()
            buf.check_status()
        return ok_rows, ok_w, ok_plan, torch.equal(o1, o2)

    for r, flags in enumerate(lw.run(body)):
        assert all(flags), f"rank {r}: rows/weights/plan/combine checks {flags}"
    lw.run(lambda r: bufs[r].destroy())


@pytest.mark.parametrize("device", DEVICES)
def test_api_rejects_bad_arguments(device):
    lw, bufs = _world(1, device, S=8, H=16, K=2, epn=4, B=1)
    buf = bufs[0]
    topk, tpe, gates = make_routing("balanced", 8, 2, 4, 1, 0, device=device)
    x = torch.randn(8, 16, device=device).to(torch.bfloat16)
    with pytest.raises(AssertionError):
        buf.dispatch(x.float(), gates, topk, tpe)
    with pytest.raises(AssertionError):
        buf.dispatch(x[:, :8], gates, topk, tpe)
    with pytest.raises(AssertionError):
        buf.dispatch(x, gates[:, :1].contiguous(), topk, tpe)
    with pytest.raises(AssertionError):
        buf.dispatch(x)  # neither routing nor plan
    xn, wn, cu, plan = buf.dispatch(x, gates, topk, tpe)
    with pytest.raises(AssertionError):
        buf.combine(None, xn, wn)
    with pytest.raises(AssertionError):
        buf.combine(plan, xn[:-1], wn)
    with pytest.raises(AssertionError):
        buf.combine(plan, xn, wn, zero_copy=True)  # not the shard view
    with pytest.raises(TypeError):
        buf.combine(plan, xn, wn, hidden_sh=x)
    buf.destroy()
    assert buf.destroyed
    with pytest.raises(AssertionError):
        buf.dispatch(x, gates, topk, tpe)


@pytest.mark.gpu
def test_wait_that_nothing_satisfies_reports_timeout_and_buffer_recovers():
    """A flag that no rank sets: the wait gives up after its budget, the kernel returns, the host
    reads the status; after check_status() the same Buffer works again."""
    from moonep_b200.constants import FLAG_GRAD_DONE
    from moonep_b200.errors import MoonEPTimeoutError

    lw, bufs = _world(1, "cuda", S=16, H=32, K=2, epn=4, B=1)
    buf = bufs[0]
    be = buf._require_ctx()["_backend"]
    be.set_timeout_ms(200)
    be.epoch[FLAG_GRAD_DONE] += 1  # an epoch nobody will ever signal
    be.wait(FLAG_GRAD_DONE)
    torch.cuda.synchronize()
    with pytest.raises(MoonEPTimeoutError) as ei:
        buf.check_status()
    assert ei.value.kernel == "wait" and ei.value.peer == 0
    be.epoch[FLAG_GRAD_DONE] -= 1
    topk, tpe, gates = make_routing("balanced", 16, 2, 4, 1, 0, device="cuda")
    x = torch.randn(16, 32, device="cuda").to(torch.bfloat16)
    xn, wn, cu, plan = buf.dispatch(x, gates, topk, tpe)
    out, wb, _ = buf.combine(plan, xn, wn)
    torch.cuda.synchronize()
    buf.check_status()
    assert torch.equal(wb, gates)
    buf.destroy()


@pytest.mark.gpu
def test_prefetch_and_reduce_grad_with_offsets_beyond_2_31():
    """Experts of 7168 x 3072 elements: byte and element offsets cross 2**31 (parity: reference
    tests/test_prefetch.py:112-124 and tests/test_grad_reduce.py large-offset case)."""
    R, S, H, K, epn, B = 2, 16, 32, 2, 52, 52
    E, Hw, Hp = R * epn, 7168, 3072
    per = Hw * Hp
    lw, bufs = _world(R, "cuda", S, H, K, epn, B, num_sms=32)
    plans = _plans(lw, bufs, R, S, H, K, E, "cuda")
    etc = torch.full((R, B), -1, dtype=torch.int32)
    etc[0, 51] = 103  # expert 103 of rank 1: source offset 103 * per * 2 bytes = 4.5 GB
    etc[1, 50] = 3
    # one shared pool of experts (emulated ranks see all of it) and per-rank slots
    experts = torch.empty(E, Hw, Hp, dtype=torch.bfloat16, device="cuda")
    experts[103].copy_(torch.arange(per, device="cuda").remainder(251).to(torch.bfloat16).view(Hw, Hp))
    experts[3].fill_(3.0)
    red = torch.zeros(R, B, Hw, Hp, dtype=torch.float32, device="cuda")  # slot (1, 50) starts at element 2.2e9
    red[0, 51].fill_(0.5)
    red[1, 50].copy_(torch.arange(per, device="cuda").remainder(127).float().view(Hw, Hp))

    def body(r):
        plan = dataclasses.replace(plans[r], experts_to_copy=etc.cuda())
        slots = torch.full((B, Hw, Hp), -123.0, dtype=torch.bfloat16, device="cuda")
        be = bufs[r]._require_ctx()["_backend"]
        be.prefetch_launch([experts], [slots], etc[r].cuda().contiguous())
        grad = torch.ones(epn, Hw, Hp, dtype=torch.float32, device="cuda")
        lw.view(r).step()
        be.reduce_grad(plan.experts_to_copy, [grad], [red], local=True)
        torch.cuda.synchronize()
        bufs[r].check_status()
        lw.view(r).step()
        if r == 0:
            ok_pf = torch.equal(slots[51], experts[103]) and bool((slots[50] == -123.0).all())
            want = torch.ones(Hw, Hp, device="cuda") + torch.arange(per, device="cuda").remainder(127).float().view(Hw, Hp)
            ok_gr = torch.equal(grad[3], want) and bool((grad[4] == 1).all())
        else:
            ok_pf = torch.equal(slots[50], experts[3]) and bool((slots[51] == -123.0).all())
            ok_gr = torch.equal(grad[103 - epn], torch.full((Hw, Hp), 1.5, device="cuda")) and bool((grad[0] == 1).all())
        return ok_pf, ok_gr

    for r, (ok_pf, ok_gr) in enumerate(lw.run(body)):
        assert ok_pf, f"rank {r}: prefetch with large offsets wrong"
        assert ok_gr, f"rank {r}: reduce_grad with large offsets wrong"
    assert not bool(red[0, 51].abs().max() > 0) and not bool(red[1, 50].abs().max() > 0), "consumed slots not cleared"
    lw.run(lambda r: bufs[r].destroy())


@pytest.mark.parametrize("device", DEVICES)
def test_stats_report_rows_and_dedup(device):
    R, S, H, K, epn, B = 2, 32, 32, 4, 2, 1
    lw, bufs = _world(R, device, S, H, K, epn, B)
    plans = _plans(lw, bufs, R, S, H, K, R * epn, device)

    def body(r):
        return bufs[r].stats(plans[r])

    st = lw.run(body)
    for r in range(R):
        assert st[r]["entries"] == S * K and st[r]["rows_sent"] + st[r]["entries_deduplicated"] == S * K
        assert st[r]["rows_sent_remote"] <= st[r]["rows_sent"] and st[r]["bytes_sent_remote"] == st[r]["rows_sent_remote"] * H * 2
    assert sum(s["entries_deduplicated"] for s in st) == sum(s["dup_rows_received"] for s in st)
    # load balance: all ranks see the same global table; no rank gets more than S*K rows; re-homing never hurts
    assert st[0]["rows_per_rank"] == st[1]["rows_per_rank"] and sum(st[0]["rows_per_rank"]) == R * S * K
    assert max(st[0]["rows_per_rank"]) <= S * K
    assert 1.0 <= st[0]["imbalance"] <= st[0]["imbalance_without_balancing"] + 1e-9
    lw.run(lambda r: bufs[r].destroy())


def test_reduce_grad_needs_a_gradient_with_its_buffer():
    """Leaving a weight out means leaving out both its gradient and its reduce buffer; leaving out all is an error."""
    lw, bufs = _world(1, "cpu", S=8, H=16, K=2, epn=4, B=1)
    buf = bufs[0]
    topk, tpe, gates = make_routing("balanced", 8, 2, 4, 1, 0)
    x = torch.randn(8, 16).to(torch.bfloat16)
    plan = buf.dispatch(x, gates, topk, tpe)[3]
    g = torch.zeros(4, 128, 128)
    red = torch.zeros(1, 1, 128, 128)
    with pytest.raises(AssertionError, match="reduce buffer"):
        buf.reduce_grad(plan, False, g, None, None, None, None, None)  # a gradient without its buffer
    with pytest.raises(AssertionError, match="at least one"):
        buf.reduce_grad(plan, False)
    buf.reduce_grad(plan, False, None, None, g, None, None, red)  # the down projection alone
    buf.destroy()
