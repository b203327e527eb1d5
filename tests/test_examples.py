"""The example programs run as documented (two gloo ranks on the host backend)."""

import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(script, *args):
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "examples", script), "--backend", "gloo", *args]  # fmt: skip
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT, env=dict(os.environ, MASTER_ADDR="127.0.0.1"))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    return out.stdout


def test_dispatch_combine_example():
    out = _torchrun("dispatch_combine.py", "--S", "128", "--H", "64", "--K", "4", "--experts-per-rank", "4")
    assert "all ranks ok: True" in out


@pytest.mark.parametrize("steps", [2])
def test_moe_training_step_example(steps):
    out = _torchrun("moe_training_step.py", "--S", "64", "--H", "128", "--I", "128", "--experts-per-rank", "2", "--K", "2",
                    "--steps", str(steps))  # fmt: skip
    assert out.count("mean loss") == steps and "done" in out
