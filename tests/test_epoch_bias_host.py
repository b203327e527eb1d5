"""Host-side bookkeeping of the epoch bias that makes Buffer operations capturable in CUDA graphs: launch
arguments are relative to the bias, a capture rolls the host state back, replays advance it, and the device bias
is only rewritten when ordinary calls happened in between.  Runs without a GPU (the bias launch is stubbed)."""

from moonep_b200.constants import FLAG_READY, FLAG_SENT, NUM_FLAG_FAMILIES
from moonep_b200.ops.cuda_backend import CudaBackend


class _World:
    size = 1
    emulated = True


def _backend(epochs):
    be = CudaBackend.__new__(CudaBackend)
    be.epoch = list(epochs)
    be.bias = [0] * NUM_FLAG_FAMILIES
    be._capture = None
    be._profile = None
    be._quiesced = True
    be.world = _World()
    be.bias_launches = []
    be._bias_launch = lambda values, mode: be.bias_launches.append((list(values), mode))
    return be


def test_capture_rolls_back_and_replays_advance():
    start = [5, 3, 3, 7, 7, 0, 0, 0]
    be = _backend(start)
    be.capture_begin()
    assert be._quiesced is False, "a captured sequence must not rely on the state before the capture"
    args = (be._next(FLAG_SENT), be._cur(FLAG_SENT), be._next(FLAG_READY), be._next(FLAG_SENT))
    assert args == (1, 1, 1, 2), "captured arguments are relative to the capture point"
    be._quiesced = True
    end = be.capture_end()
    assert be.bias_launches[-1] == ([1, 0, 0, 2, 0, 0, 0, 0], 1), "the graph ends by advancing the device bias"
    assert be.epoch == start and be.bias == [0] * NUM_FLAG_FAMILIES and be._quiesced is True, "nothing ran: state is back"

    be.replay_prepare()
    assert be.bias_launches[-1] == (start, 0), "before the first replay the device bias is set to the epochs reached"
    be.replay_done(end)
    assert be.epoch == [6, 3, 3, 9, 7, 0, 0, 0] and be.bias == be.epoch and be._quiesced is True
    n = len(be.bias_launches)
    be.replay_prepare()
    assert len(be.bias_launches) == n, "replays back to back need no bias launch"
    be.replay_done(end)
    assert be.epoch[FLAG_SENT] == 11

    # an ordinary call after replays: absolute epoch 12, passed relative to the bias the device holds (11)
    assert be._next(FLAG_SENT) == 1 and be.epoch[FLAG_SENT] == 12 and be._cur(FLAG_SENT) == 1
    be.replay_prepare()
    assert be.bias_launches[-1][1] == 0 and be.bias_launches[-1][0][FLAG_SENT] == 12, "the bias follows ordinary calls"


def test_capture_abort_restores_the_state():
    be = _backend([2] * NUM_FLAG_FAMILIES)
    be.capture_begin()
    be._next(FLAG_READY)
    be.capture_abort()
    assert be.epoch == [2] * NUM_FLAG_FAMILIES and be.bias == [0] * NUM_FLAG_FAMILIES and be._capture is None
    be.capture_begin()  # a new capture can start
    be.capture_abort()


def test_capture_on_the_cpu_backend_runs_eagerly():
    import torch

    from moonep_b200 import Buffer
    from moonep_b200.models.routing import make_routing

    S, H, K, E = 16, 32, 2, 4
    buf = Buffer(S, H, K, E, 1, token_padding=8)
    topk, tpe, gates = make_routing("balanced", S, K, E, 1, 0)
    x = torch.randn(S, H).to(torch.bfloat16)

    def step():
        xn, wn, _, plan = buf.dispatch(x, gates, topk, tpe)
        return buf.combine(plan, xn, wn)[0]

    st = buf.capture(step)
    for _ in range(2):
        x.copy_(torch.randn(S, H).to(torch.bfloat16))
        assert torch.equal(st.replay(), (x.float() * K).to(torch.bfloat16))
    assert st.replays == 2
    buf.destroy()
