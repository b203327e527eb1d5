"""Communication worlds: who the EP ranks are and how the host meets them.

A ``World`` gives a ``Buffer`` three things: its rank and size, symmetric
memory (one chunk per rank, all chunks in one address range), and ``step()``,
the host-side rendezvous between two phases of a collective operation.

``DistWorld``   one process per rank over ``torch.distributed``.
                CUDA: chunks are CUDA-VMM allocations mapped into every
                process; ordering between phases is done by epoch flags inside
                the kernels, so ``step()`` does nothing.
                CPU (gloo): chunks live in one ``/dev/shm`` file mapped by all
                processes; ``step()`` is ``dist.barrier``.
``LocalWorld``  R emulated ranks inside one process, each driven by its own
                Python thread (``LocalWorld.run``).  All chunks live in one
                ordinary tensor on one device; ``step()`` is a thread barrier,
                so phase p of every rank is issued before phase p+1 of any.  On
                CUDA all ranks share one stream, hence a kernel never waits for
                a kernel that has not been launched before it.

The reference has only the first kind (NVSHMEM heap, ``moonep_td/buffer.py:40-60``).
"""

from __future__ import annotations

import os
import threading
import uuid

import torch
import torch.distributed as dist


class World:
    rank: int
    size: int
    device: torch.device
    emulated = False

    @property
    def is_cuda(self) -> bool:
        return self.device.type == "cuda"

    def step(self) -> None:
        """Host rendezvous of all ranks between two phases."""

    def host_barrier(self) -> None:
        """Unconditional host barrier (creation / destruction)."""

    def alloc_symmetric(self, chunk_numel: int, dtype: torch.dtype, gran_bytes: int) -> "SymmetricTensor":
        raise NotImplementedError

    def free_symmetric(self, st: "SymmetricTensor") -> None:
        st.release()

    def granularity(self) -> int:
        return 128

    def comm_stream(self, priority: int):
        if not self.is_cuda:
            return None
        return torch.cuda.Stream(device=self.device, priority=priority)


class SymmetricTensor:
    """``full`` is a 1-D tensor over all R chunks; chunk r = full[r*chunk_numel:(r+1)*chunk_numel]."""

    def __init__(self, full: torch.Tensor, chunk_numel: int, owner=None, on_release=None):
        self.full = full
        self.chunk_numel = chunk_numel
        self._owner = owner
        self._on_release = on_release
        self.released = False

    def release(self) -> None:
        if self.released:
            return
        self.released = True
        self.full = None
        if self._on_release is not None:
            self._on_release()
        self._owner = None


# ----------------------------------------------------------------------------
# In-process emulation
# ----------------------------------------------------------------------------


class LocalWorld:
    """R emulated ranks in one process; ``view(r)`` is rank r's ``World``."""

    def __init__(self, size: int, device="cpu"):
        self.size = int(size)
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self._barrier = threading.Barrier(self.size)
        self._lock = threading.Lock()
        self._allocs: dict[int, SymmetricTensor] = {}
        self._alloc_seq = [0] * self.size
        self._comm_stream = None
        self._views = [_LocalRank(self, r) for r in range(self.size)]

    def view(self, rank: int) -> "World":
        return self._views[rank]

    def run(self, fn, *, timeout: float | None = 600.0):
        """Call ``fn(rank)`` on one thread per rank and return the list of results."""
        results = [None] * self.size
        errors = [None] * self.size

        def body(r):
            try:
                if self.device.type == "cuda":
                    torch.cuda.set_device(self.device)
                results[r] = fn(r)
            except BaseException as exc:  # noqa: BLE001 - re-raised on the caller's thread
                errors[r] = exc
                self._barrier.abort()

        if self.size == 1:
            body(0)
        else:
            threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(self.size)]
            for t in threads:
                t.start()
            for t in threads:
                t.join(timeout)
        self._barrier.reset()
        real = [e for e in errors if e is not None and not isinstance(e, threading.BrokenBarrierError)]
        if real:
            raise real[0]
        broken = [e for e in errors if e is not None]
        if broken:
            raise broken[0]
        return results

    def _step(self):
        if self.size > 1:
            self._barrier.wait()

    def _alloc(self, rank, chunk_numel, dtype, gran_bytes):
        with self._lock:
            seq = self._alloc_seq[rank]
            self._alloc_seq[rank] += 1
            st = self._allocs.get(seq)
            if st is None:
                full = torch.zeros(self.size * chunk_numel, dtype=dtype, device=self.device)
                st = SymmetricTensor(full, chunk_numel)
                st._users = 0
                self._allocs[seq] = st
            assert st.chunk_numel == chunk_numel and st.full.dtype == dtype, "ranks disagree on a symmetric allocation"
            st._users += 1
            if st._users == self.size:
                del self._allocs[seq]
        return SymmetricTensor(st.full, chunk_numel)

    def _get_comm_stream(self, priority):
        if self.device.type != "cuda":
            return None
        with self._lock:
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=self.device, priority=priority)
        return self._comm_stream


class _LocalRank(World):
    emulated = True

    def __init__(self, parent: LocalWorld, rank: int):
        self.parent = parent
        self.rank = rank
        self.size = parent.size
        self.device = parent.device

    def step(self):
        self.parent._step()

    def host_barrier(self):
        self.parent._step()

    def alloc_symmetric(self, chunk_numel, dtype, gran_bytes):
        return self.parent._alloc(self.rank, chunk_numel, dtype, gran_bytes)

    def comm_stream(self, priority):
        # One stream for all emulated ranks keeps their phases in issue order.
        return self.parent._get_comm_stream(priority)


# ----------------------------------------------------------------------------
# torch.distributed
# ----------------------------------------------------------------------------


class DistWorld(World):
    """One process per rank.  ``device`` decides between the CUDA and the CPU backend."""

    def __init__(self, group=None, device=None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialized before a Buffer is created")
        self.group = group
        self.rank = dist.get_rank(group=group)
        self.size = dist.get_world_size(group=group)
        if device is None:
            backend = dist.get_backend(group)
            use_cuda = torch.cuda.is_available() and "nccl" in str(backend)
            device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self._vmm = None

    def step(self):
        if not self.is_cuda:
            dist.barrier(group=self.group)

    def host_barrier(self):
        if self.is_cuda:
            dist.barrier(group=self.group, device_ids=[self.device.index])
        else:
            dist.barrier(group=self.group)

    def granularity(self) -> int:
        if self.is_cuda and self.size > 1:
            from .vmm import VmmAllocator

            return VmmAllocator.get(self).granularity
        return 128

    def alloc_symmetric(self, chunk_numel, dtype, gran_bytes):
        if self.is_cuda:
            if self.size == 1:
                full = torch.zeros(chunk_numel, dtype=dtype, device=self.device)
                return SymmetricTensor(full, chunk_numel)
            from .vmm import VmmAllocator

            return VmmAllocator.get(self).alloc(chunk_numel, dtype)
        return _alloc_shm(self, chunk_numel, dtype)


def _alloc_shm(world: DistWorld, chunk_numel: int, dtype: torch.dtype) -> SymmetricTensor:
    """CPU symmetric memory: one /dev/shm file mapped by every process of the group."""
    nbytes = world.size * chunk_numel * torch.empty(0, dtype=dtype).element_size()
    name = [None]
    if world.rank == 0:
        name[0] = f"/dev/shm/moonep_b200_{os.getpid()}_{uuid.uuid4().hex}"
        with open(name[0], "wb") as f:
            f.truncate(max(nbytes, 1))
    dist.broadcast_object_list(name, src=dist.get_global_rank(world.group, 0) if world.group else 0, group=world.group)
    raw = torch.from_file(name[0], shared=True, size=max(nbytes, 1), dtype=torch.uint8)
    dist.barrier(group=world.group)
    if world.rank == 0:
        os.unlink(name[0])  # the mappings keep the memory alive
    full = raw[:nbytes].view(dtype)
    return SymmetricTensor(full, chunk_numel, owner=raw)


def make_world(num_ep_ranks: int, group=None, world: World | None = None) -> World:
    if world is not None:
        assert world.size == num_ep_ranks, f"world has {world.size} ranks, Buffer asked for {num_ep_ranks}"
        return world
    if not dist.is_initialized():
        if num_ep_ranks == 1:
            dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
            return LocalWorld(1, dev).view(0)
        raise RuntimeError(
            "torch.distributed must be initialized before a multi-rank Buffer is created "
            "(or pass world=LocalWorld(R, device).view(rank) for in-process emulation)"
        )
    w = DistWorld(group=group)
    assert w.size == num_ep_ranks, f"process group has {w.size} ranks, Buffer asked for {num_ep_ranks}"
    return w
