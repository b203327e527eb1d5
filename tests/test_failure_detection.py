"""Failure detection without faulting anything: a rank that leaves between steps is noticed by its
peers on the host (the next rendezvous fails within the process-group timeout) instead of hanging."""

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import datetime, os, sys, torch, torch.distributed as dist
sys.path.insert(0, {root!r})
from moonep_b200 import Buffer
from moonep_b200.models.routing import make_routing
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8))
rank, R = dist.get_rank(), dist.get_world_size()
S, H, K, E = 16, 32, 2, 4
buf = Buffer(S, H, K, E, R, token_padding=8, explicitly_destroy=True)
topk, tpe, gates = make_routing("balanced", S, K, E, R, rank)
x = torch.randn(S, H).to(torch.bfloat16)
xn, wn, cu, plan = buf.dispatch(x, gates, topk, tpe)
out, wb, _ = buf.combine(plan, xn, wn)
assert torch.equal(wb, gates)
print("STEP1 OK", rank, flush=True)
if rank == 1:
    os._exit(0)  # leaves between two steps, nothing of its own in flight
try:
    buf.dispatch(x, gates, topk, tpe)
    print("UNEXPECTED: second step completed", flush=True)
    os._exit(3)
except Exception as exc:
    print("PEER LOSS DETECTED:", type(exc).__name__, flush=True)
    os._exit(0)
"""


def test_rank_leaving_between_steps_is_detected_on_the_host(tmp_path):
    script = tmp_path / "leave.py"
    script.write_text(WORKER.format(root=ROOT))
    import socket

    with socket.socket() as sk:  # a fixed port can still be in TIME_WAIT from the previous run
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", str(port), str(script)],
        capture_output=True, text=True, timeout=180, env=env, cwd=ROOT,
    )  # fmt: skip
    assert out.stdout.count("STEP1 OK") == 2, out.stdout + out.stderr[-2000:]
    assert "PEER LOSS DETECTED" in out.stdout, out.stdout + out.stderr[-2000:]
    assert "UNEXPECTED" not in out.stdout
