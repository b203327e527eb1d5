"""One process per rank over torch.distributed: gloo + /dev/shm on CPU, NCCL + CUDA VMM on GPUs."""

import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    import socket

    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _run_worker(nproc, backend, port, timeout, extra_env=None, scenarios=None):
    port = _free_port()  # a fixed port can still be in TIME_WAIT from the previous run
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MOONEP_TIMEOUT_MS=os.environ.get("MOONEP_TIMEOUT_MS", "5000"))
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mp_worker.py"), "--backend", backend]  # fmt: skip
    if scenarios:
        cmd += ["--scenarios", scenarios]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert out.returncode == 0, f"worker failed:\n{out.stdout[-4000:]}\n{out.stderr[-6000:]}"
    assert out.stdout.count("WORKER OK") == nproc, out.stdout[-4000:]


def test_cpu_backend_two_gloo_processes():
    _run_worker(2, "gloo", 29621, 600)


def test_cpu_backend_four_gloo_processes():
    """Four ranks: every rank has three peers, experts_to_copy rows differ per rank, a token's entries spread over up
    to four destinations."""
    _run_worker(4, "gloo", 29622, 900, scenarios="round_trips,plan_reuse,weights")


@pytest.mark.gpu
def test_cuda_backend_nccl_processes():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    # up to four ranks (MOONEP_TEST_MP_RANKS changes the bound), one per GPU present
    want = int(os.environ.get("MOONEP_TEST_MP_RANKS", "4"))
    # NVLS off: a rank that dies while its memory is bound to an in-switch reduction object can fault its peers
    _run_worker(max(2, min(n, want)), "nccl", 29631, 900, {"NCCL_NVLS_ENABLE": "0"})
