"""Build and load the native library ``libmoonep_b200.so`` (ctypes).

The library is compiled in-tree with nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and linked against the static
CUDA runtime, so it also loads on a machine without a GPU driver (where only
the build and the CPU backend are used).  ``load()`` rebuilds when the hash of
the sources differs from the one stored beside the binary.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent.parent
CSRC = _PKG / "csrc"
LIBDIR = _PKG / "lib"
LIBPATH = LIBDIR / "libmoonep_b200.so"
_HASHFILE = LIBDIR / "libmoonep_b200.hash"

NVCC_FLAGS = [
    "-shared",
    "-Xcompiler",
    "-fPIC",
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "--threads",
    "0",
]

_lock = threading.Lock()
_lib = None


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _source_hash() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def nvcc_path() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc")
    if cand:
        return cand
    p = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
    return str(p) if p.exists() else None


def is_stale() -> bool:
    if not LIBPATH.exists() or not _HASHFILE.exists():
        return True
    return _HASHFILE.read_text().strip() != _source_hash()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu file of the package into one shared object."""
    with _lock:
        if not force and not is_stale():
            return LIBPATH
        nvcc = nvcc_path()
        if nvcc is None:
            raise RuntimeError("nvcc not found; cannot build libmoonep_b200.so")
        LIBDIR.mkdir(exist_ok=True)
        tmp = LIBDIR / f"libmoonep_b200.{os.getpid()}.tmp.so"
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-o", str(tmp), *[str(s) for s in sources()]]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp, LIBPATH)
        _HASHFILE.write_text(_source_hash() + "\n")
        if verbose:
            print(proc.stderr)
        return LIBPATH


_vp, _i, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_ull = ctypes.c_ulonglong

_SIGNATURES = {
    "moonep_version": (_i, []),
    "moonep_last_error": (ctypes.c_char_p, []),
    "moonep_sizeof_devctx": (_i, []),
    "moonep_launch_count": (_ll, []),
    "moonep_planner_table_words": (_ll, [_i, _i, _i]),
    "moonep_ctx_create": (_vp, [ctypes.POINTER(_ll), _i, ctypes.POINTER(_ull), ctypes.POINTER(_ull), ctypes.POINTER(_ull)]),
    "moonep_ctx_destroy": (None, [_vp]),
    "moonep_ctx_set_timeout_ms": (_i, [_vp, _ll]),
    "moonep_ctx_set_pdl": (_i, [_vp, _i]),
    "moonep_signal_wait": (_i, [_vp, _i, _i, _i, _i, _vp]),
    "moonep_epoch_bias": (_i, [_vp, _vp, _i, _vp]),
    "moonep_plan_publish": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "moonep_plan_compute": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "moonep_dispatch": (_i, [_vp, _i, _i] + [_vp] * 9 + [_i] + [_vp] * 5 + [_i] * 9 + [_vp, _vp]),
    "moonep_peer_store_bench": (_i, [_vp, _vp, _ll, _i, _i, _vp, _ll, _i, _vp, _vp]),
    "moonep_stage_layout": (_ll, [_i, _i, _i, _i, ctypes.POINTER(_ll), ctypes.POINTER(_ll)]),
    "moonep_combine_push": (_i, [_vp, _i] + [_vp] * 7 + [_i, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "moonep_combine_prologue": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "moonep_combine_pull": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "moonep_prefetch": (_i, [_vp, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i, _vp, _ll, _i, _i, _i, _vp, _vp, _i, _vp]),
    "moonep_grad_reduce": (_i, [_vp, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i, _vp, _i, _ll, _i, _i, _i, _i, _vp]),
    "moonep_grouped_gemm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _ll, _i, _vp, _i, _vp, _vp, _vp]),
    "moonep_grouped_gemm_pair": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _ll, _i, _vp, _i, _vp, _vp, _vp]),
    "moonep_grouped_gemm_pair_hooked": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _ll, _i, _vp, _i, _vp, _vp, _vp, _vp]),
    "moonep_grouped_gemm_pair_kn": (_i, [_vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _ll, _i, _vp]),
    "moonep_pair_schedule": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _i]),
    "moonep_grouped_wgrad": (_i, [_vp, _vp, _ll, _i, _i, _vp, _i, _vp, _vp, _i, _vp, _ll, _i, _vp]),
    "moonep_grouped_wgrad_rows": (_i, [_vp, _ll, _vp, _ll, _i, _i, _i, _vp, _i, _vp, _vp, _vp, _ll, _i, _vp]),
    "moonep_transpose_experts": (_i, [_vp, _vp, _i, _i, _i, _ll, _ll, _i, _vp, _vp]),
    "moonep_sgd_update": (_i, [_vp, _vp, _ll, ctypes.c_float, _vp]),
    "moonep_swiglu_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp]),
    "moonep_vmm_granularity": (_i, [_i, ctypes.POINTER(_ull)]),
    "moonep_vmm_create": (_i, [_i, _ull, ctypes.POINTER(_ull), ctypes.POINTER(_i)]),
    "moonep_vmm_import": (_i, [_i, ctypes.POINTER(_ull)]),
    "moonep_vmm_reserve": (_i, [_ull, _ull, ctypes.POINTER(_ull)]),
    "moonep_vmm_map": (_i, [_ull, _ull, _ull, _i]),
    "moonep_vmm_unmap": (_i, [_ull, _ull]),
    "moonep_vmm_release": (_i, [_ull]),
    "moonep_vmm_free_va": (_i, [_ull, _ull]),
}


def load():
    """Return the loaded library, building it first if needed."""
    global _lib
    if _lib is not None:
        return _lib
    if is_stale():
        build()
    with _lock:
        if _lib is None:
            lib = ctypes.CDLL(str(LIBPATH))
            for name, (res, args) in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


class NativeError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().moonep_last_error().decode(errors="replace")
        raise NativeError(f"{what} failed (code {rc}): {msg}")
