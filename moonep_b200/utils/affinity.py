"""Keep a rank's host threads (and therefore its pinned staging buffers, which are placed on the node of the thread
that first touches them) on the CPU socket its GPU hangs off.  With eight ranks per host the host-to-device copies of
the ranks whose process runs on the far socket otherwise cross the socket interconnect.

Only the calling process is affected (``os.sched_setaffinity``); nothing of the GPU or the host is reconfigured.
``MOONEP_NO_AFFINITY=1`` disables it.  NVML is only read (``nvmlDeviceGetCpuAffinity``).
"""

from __future__ import annotations

import os

from .clocks import _physical_index


def gpu_cpu_set(index: int) -> set[int] | None:
    """CPUs NVML reports as local to GPU ``index`` (a CUDA device index of this process), or None if unknown."""
    try:
        import pynvml

        pynvml.nvmlInit()
        try:
            handle = pynvml.nvmlDeviceGetHandleByIndex(_physical_index(index))
            ncpu = os.cpu_count() or 1
            words = pynvml.nvmlDeviceGetCpuAffinity(handle, (ncpu + 63) // 64)
        finally:
            pynvml.nvmlShutdown()
    except Exception:  # noqa: BLE001 - no NVML, no permission, no such device: leave the affinity alone
        return None
    cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
    return cpus or None


def bind_to_gpu_socket(index: int, min_cpus: int = 2) -> dict:
    """Restrict this process to the CPUs local to GPU ``index`` that it is allowed to use anyway.  Returns what was
    done: ``{"applied": bool, "cpus": number of CPUs now allowed, "reason": why not}``."""
    if os.environ.get("MOONEP_NO_AFFINITY", "0") not in ("0", "", "false", "False"):
        return {"applied": False, "reason": "disabled by MOONEP_NO_AFFINITY"}
    if not hasattr(os, "sched_setaffinity"):
        return {"applied": False, "reason": "no sched_setaffinity on this platform"}
    local = gpu_cpu_set(index)
    if not local:
        return {"applied": False, "reason": "NVML reports no CPU affinity for the GPU"}
    allowed = os.sched_getaffinity(0)
    target = allowed & local
    if len(target) < min_cpus:
        return {"applied": False, "reason": f"only {len(target)} of the GPU's CPUs are available to this process"}
    if target == allowed:
        return {"applied": False, "cpus": len(allowed), "reason": "already on the GPU's socket"}
    try:
        os.sched_setaffinity(0, target)
    except OSError as exc:
        return {"applied": False, "reason": f"sched_setaffinity failed: {exc}"}
    return {"applied": True, "cpus": len(target)}
