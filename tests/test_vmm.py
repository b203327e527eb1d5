"""CUDA-VMM allocator pieces on one GPU: create, export, import, map twice, wrap as a tensor."""

import ctypes
import os

import pytest
import torch


@pytest.mark.gpu
def test_vmm_export_import_alias_on_one_gpu():
    from moonep_b200.ops import _lib
    from moonep_b200.parallel.vmm import tensor_from_ptr

    lib = _lib.load()
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    gran = ctypes.c_ulonglong(0)
    _lib.check(lib.moonep_vmm_granularity(0, ctypes.byref(gran)), "granularity")
    g = int(gran.value)
    assert g >= 4096 and g % 4096 == 0
    handle, fd = ctypes.c_ulonglong(0), ctypes.c_int(-1)
    _lib.check(lib.moonep_vmm_create(0, g, ctypes.byref(handle), ctypes.byref(fd)), "create")
    h2 = ctypes.c_ulonglong(0)
    _lib.check(lib.moonep_vmm_import(fd.value, ctypes.byref(h2)), "import")
    os.close(fd.value)
    va = ctypes.c_ulonglong(0)
    _lib.check(lib.moonep_vmm_reserve(2 * g, g, ctypes.byref(va)), "reserve")
    _lib.check(lib.moonep_vmm_map(va.value, g, handle.value, 0), "map 0")
    _lib.check(lib.moonep_vmm_map(va.value + g, g, h2.value, 0), "map 1")
    n = 2 * g // 4
    t = tensor_from_ptr(va.value, n, torch.int32, torch.device("cuda", 0))
    assert t.data_ptr() == va.value and t.numel() == n
    t[: n // 2] = torch.arange(n // 2, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    # the second half maps the same physical memory through the imported handle
    assert torch.equal(t[n // 2 :].cpu(), torch.arange(n // 2, dtype=torch.int32))
    bf = tensor_from_ptr(va.value, 2 * g // 2, torch.bfloat16, torch.device("cuda", 0))
    assert bf.dtype == torch.bfloat16 and bf.data_ptr() == va.value
    del t, bf
    torch.cuda.synchronize()
    _lib.check(lib.moonep_vmm_unmap(va.value, g), "unmap 0")
    _lib.check(lib.moonep_vmm_unmap(va.value + g, g), "unmap 1")
    _lib.check(lib.moonep_vmm_release(handle.value), "release 0")
    _lib.check(lib.moonep_vmm_release(h2.value), "release 1")
    _lib.check(lib.moonep_vmm_free_va(va.value, 2 * g), "free va")


def test_fd_exchange_over_unix_sockets_gloo(tmp_path):
    """The descriptor exchange used by the allocator, with ordinary files and two gloo ranks."""
    import subprocess
    import sys

    script = tmp_path / "fdx.py"
    script.write_text(
        "import os, sys, torch.distributed as dist\n"
        f"sys.path.insert(0, {os.path.dirname(os.path.dirname(os.path.abspath(__file__)))!r})\n"
        "from moonep_b200.parallel.vmm import exchange_fds\n"
        "dist.init_process_group('gloo')\n"
        "r, n = dist.get_rank(), dist.get_world_size()\n"
        "fd = os.memfd_create(f'rank{r}')\n"
        "os.write(fd, f'hello from {r}'.encode())\n"
        "fds = exchange_fds(None, r, n, fd)\n"
        "for p in range(n):\n"  # pread: the received descriptors share one file offset with every other rank's copy
        "    assert os.pread(fds[p], 64, 0) == f'hello from {p}'.encode(), (r, p)\n"
        "dist.barrier()\n"
        "print('ok', r)\n"
    )
    import socket

    with socket.socket() as sk:  # a fixed port can still be in TIME_WAIT from the previous run
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
         "--master-port", str(port), str(script)],
        capture_output=True, text=True, timeout=120, env=env,
    )  # fmt: skip
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.count("ok") == 3
