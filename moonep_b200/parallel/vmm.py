"""CUDA-VMM symmetric allocator: one physical chunk per rank, all chunks in one address range.

``alloc(chunk_numel, dtype)``: every rank creates an exportable allocation of
``chunk_bytes`` (a multiple of the VMM granularity), the POSIX file descriptors
are exchanged over Unix-domain sockets (``SCM_RIGHTS``), and each rank maps the
R allocations back to back into a reserved range, so chunk r starts
``r * chunk_bytes`` after the base on every rank.  The range is wrapped into a
torch tensor through ``__cuda_array_interface__`` (no copy, no ownership).

Parity: replaces the reference's NVSHMEM heap (``moonep_td/buffer.py:86-109``:
``nvshmem_create_tensor`` / ``nvshmem_free_tensor_sync``), which allocates all R
chunks on every PE; here each rank pays for its own chunk only.
"""

from __future__ import annotations

import ctypes
import os
import socket
import uuid

import torch
import torch.distributed as dist

from ..ops import _lib
from .world import SymmetricTensor

_TYPESTR = {1: "|u1", 2: "<i2", 4: "<i4", 8: "<i8"}
_VIEW_AS = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}


class _RawCudaArray:
    """Minimal ``__cuda_array_interface__`` carrier for a device address."""

    def __init__(self, ptr: int, numel: int, itemsize: int):
        self.__cuda_array_interface__ = {
            "shape": (numel,),
            "typestr": _TYPESTR[itemsize],
            "data": (ptr, False),
            "version": 3,
            "strides": None,
        }


def tensor_from_ptr(ptr: int, numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    itemsize = torch.empty(0, dtype=dtype).element_size()
    raw = torch.as_tensor(_RawCudaArray(ptr, numel, itemsize), device=device)
    assert raw.data_ptr() == ptr, "torch copied the buffer instead of aliasing it"
    return raw.view(dtype)


def exchange_fds(group, rank: int, size: int, fd: int) -> list[int]:
    """All-to-all exchange of one file descriptor per rank; returns fds indexed by owner rank."""
    name = f"\0moonep_b200-{os.getpid()}-{uuid.uuid4().hex}"  # abstract socket, no file to clean up
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(name)
    srv.listen(size + 8)
    names = [None] * size
    dist.all_gather_object(names, name, group=group)
    out = [-1] * size
    out[rank] = fd
    conns = []
    for peer in range(size):
        if peer == rank:
            continue
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        s.connect(names[peer])
        socket.send_fds(s, [rank.to_bytes(4, "little")], [fd])
        conns.append(s)
    for _ in range(size - 1):
        c, _addr = srv.accept()
        msg, fds, _flags, _a = socket.recv_fds(c, 4, 1)
        out[int.from_bytes(msg, "little")] = fds[0]
        c.close()
    dist.barrier(group=group)
    for s in conns:
        s.close()
    srv.close()
    return out


class VmmAllocator:
    _instances: dict = {}

    @classmethod
    def get(cls, world) -> "VmmAllocator":
        key = (id(world.group), world.device.index)
        inst = cls._instances.get(key)
        if inst is None:
            inst = cls._instances[key] = cls(world)
        return inst

    def __init__(self, world):
        self.world = world
        self.lib = _lib.load()
        self.dev_index = world.device.index
        g = ctypes.c_ulonglong(0)
        with torch.cuda.device(world.device):
            torch.cuda.current_stream().synchronize()  # make sure the primary context exists
            _lib.check(self.lib.moonep_vmm_granularity(self.dev_index, ctypes.byref(g)), "moonep_vmm_granularity")
        self.granularity = int(g.value)

    def alloc(self, chunk_numel: int, dtype: torch.dtype, tail_numel: int = 0) -> SymmetricTensor:
        """Map all ranks' chunks back to back, optionally followed by ``tail_numel`` rank-private elements."""
        w, lib = self.world, self.lib
        R, rank = w.size, w.rank
        itemsize = torch.empty(0, dtype=dtype).element_size()
        chunk_bytes = chunk_numel * itemsize
        assert chunk_bytes % self.granularity == 0, (
            f"chunk of {chunk_bytes} bytes is not a multiple of the VMM granularity {self.granularity}"
        )
        with torch.cuda.device(w.device):
            handle, fd = ctypes.c_ulonglong(0), ctypes.c_int(-1)
            _lib.check(lib.moonep_vmm_create(self.dev_index, chunk_bytes, ctypes.byref(handle), ctypes.byref(fd)),
                       "moonep_vmm_create")  # fmt: skip
            fds = exchange_fds(w.group, rank, R, fd.value)
            tail_bytes = -(-tail_numel * itemsize // self.granularity) * self.granularity
            va = ctypes.c_ulonglong(0)
            _lib.check(lib.moonep_vmm_reserve(R * chunk_bytes + tail_bytes, self.granularity, ctypes.byref(va)),
                       "moonep_vmm_reserve")  # fmt: skip
            handles = []
            for r in range(R):
                if r == rank:
                    hr = handle.value
                else:
                    h2 = ctypes.c_ulonglong(0)
                    _lib.check(lib.moonep_vmm_import(fds[r], ctypes.byref(h2)), "moonep_vmm_import")
                    hr = h2.value
                _lib.check(lib.moonep_vmm_map(va.value + r * chunk_bytes, chunk_bytes, hr, self.dev_index), "moonep_vmm_map")
                handles.append(hr)
            for f in fds:
                if f >= 0:
                    os.close(f)
            tail_handle = None
            if tail_bytes:
                th, tfd = ctypes.c_ulonglong(0), ctypes.c_int(-1)
                _lib.check(lib.moonep_vmm_create(self.dev_index, tail_bytes, ctypes.byref(th), ctypes.byref(tfd)),
                           "moonep_vmm_create(tail)")  # fmt: skip
                os.close(tfd.value)
                _lib.check(lib.moonep_vmm_map(va.value + R * chunk_bytes, tail_bytes, th.value, self.dev_index),
                           "moonep_vmm_map(tail)")  # fmt: skip
                tail_handle = th.value
        full = tensor_from_ptr(va.value, R * chunk_numel + tail_numel, dtype, w.device)
        base, total = va.value, R * chunk_bytes + tail_bytes

        def release():
            torch.cuda.synchronize(w.device)
            for r in range(R):
                lib.moonep_vmm_unmap(base + r * chunk_bytes, chunk_bytes)
                lib.moonep_vmm_release(handles[r])
            if tail_handle is not None:
                lib.moonep_vmm_unmap(base + R * chunk_bytes, tail_bytes)
                lib.moonep_vmm_release(tail_handle)
            lib.moonep_vmm_free_va(base, total)

        full[rank * chunk_numel : (rank + 1) * chunk_numel].zero_()
        if tail_numel:
            full[R * chunk_numel :].zero_()
        torch.cuda.synchronize(w.device)
        dist.barrier(group=w.group, device_ids=[self.dev_index])
        return SymmetricTensor(full, chunk_numel, on_release=release)

    def alloc_expert_weight(self, epn: int, B: int, H: int, Hp: int, dtype: torch.dtype):
        """``[R*epn + B, H, Hp]``: every owner's experts mapped in rank order, then B local slots."""
        per = H * Hp
        itemsize = torch.empty(0, dtype=dtype).element_size()
        assert (epn * per * itemsize) % self.granularity == 0, (
            f"experts per rank * H * H' * {itemsize} bytes must be a multiple of the VMM granularity "
            f"({self.granularity}); got {epn}*{H}*{Hp}"
        )
        st = self.alloc(epn * per, dtype, tail_numel=B * per)
        full = st.full.view(self.world.size * epn + B, H, Hp)
        return full, st
