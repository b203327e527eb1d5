"""Environment toggles.

MOONEP_PLANNER        ``gpu`` (default) or ``cpu``: run the planner kernels or the host planner.
MOONEP_TIMEOUT_MS     budget of every device-side wait (default 10000).
MOONEP_COPY_PATH      ``bulk`` (default: TMA bulk copies through shared memory) or ``ldst``
                      (plain 16-byte loads/stores) for dispatch/combine/prefetch;
                      ``MOONEP_SEND_PATH`` / ``MOONEP_PULL_PATH`` / ``MOONEP_GRAD_PATH`` / ``MOONEP_PREFETCH_PATH`` set one
                      kernel only; the prefetch defaults to ``async`` (cp.async rings in shared memory; ``ldst`` for
                      register copies) whatever ``MOONEP_COPY_PATH`` says.
MOONEP_RING_STAGES    2..6 (default 4): 2 KB stages per warp of the prefetch kernel's cp.async ring (read by the native
                      library).
MOONEP_FUSE_PUBLISH   ``1``: ``plan_publish`` runs as the first step of the dispatch kernel, so a fresh dispatch is one launch
                      (default 0: measured the same as the separate kernel).
MOONEP_LOCAL_ROWS     ``0``: the send role of dispatch also writes the rows that stay on the rank (default: the
                      destination-side role writes them from the input).
MOONEP_LOCAL_HOME     ``0``: the push role of combine also moves the rows whose token lives on the rank (default: the fold
                      role puts them into the local staging chunk).
MOONEP_SUM_SLOTS      ``2``: a warp of combine's sum role holds two tokens and sums the one that completes first (read by
                      the native library; default 1: measured equal or slower on 2 GPUs, not measured on more).
MOONEP_BWD_OVERLAP    ``1``: the MoE layer reduces each weight's gradients beside the remaining backward GEMMs (default 0).
MOONEP_EXPAND_PATH    ``bulk`` (default) or ``ldst``: how the destination side of dispatch copies duplicate rows and clears
                      pad rows (read by the native library).
MOONEP_COMBINE        ``push`` (default: the expert side folds duplicates and pushes rows to the tokens' home ranks,
                      which sum them as they arrive) or ``pull`` (fold pass, then the home ranks pull).
MOONEP_PHASED         ``1``: launch the dispatch and combine kernels one role at a time even on real multi-GPU worlds
                      (what emulated ranks always do); for per-role timing and debugging.
MOONEP_PDL            ``0`` turns programmatic dependent launch off even for Buffers created with ``enable_pdl=True``.
MOONEP_LOCAL_SMS      CTAs of the kernels that only touch local memory (default: all SMs); ``num_sms`` of
                      the Buffer bounds the kernels that move data between ranks.
MOONEP_NUM_SMS_DEDUP  CTAs of the dispatch kernel's destination-side role (zero fill, dedup builder, duplicate
                      expansion); validated, 1..SM count; default: every SM the senders leave free.
MOONEP_NVTX           ``1`` wraps every native call in an NVTX range.
MOONEP_GEMM_PAIR      ``1`` (default): grouped GEMMs on CTA pairs (tcgen05 cta_group::2); ``0``: one CTA per tile.
MOONEP_WGRAD          ``kernel`` (default) or ``torch``: weight gradients of the MoE layer.
MOONEP_WGRAD_LAYOUT   ``rows`` (default: activations as stored, MN-major tiles) or ``transposed``.

Parity: reference ``moonep_td/_pipeline.py:1-14``, ``moonep_td/api.py:40-47``,
``moonep_td/_planning_gpu.py:14-16`` (``MOONEP_TD_PLANNING_TRITON`` is accepted as an alias).
"""

from __future__ import annotations

import os

from .constants import DEFAULT_TIMEOUT_MS

_FALSE = ("0", "false", "False", "")


def planner_on_gpu() -> bool:
    raw = os.environ.get("MOONEP_PLANNER")
    if raw is not None:
        return raw.lower() != "cpu"
    return os.environ.get("MOONEP_TD_PLANNING_TRITON", "1") not in _FALSE


def timeout_ms() -> int:
    return max(1, int(os.environ.get("MOONEP_TIMEOUT_MS", DEFAULT_TIMEOUT_MS)))


def copy_path(which: str = "") -> str:
    """Copy path of the send (``which="send"``), pull (``"pull"``), gradient accumulation (``"grad"``) or prefetch
    (``"prefetch"``) kernel.

    ``MOONEP_SEND_PATH`` / ``MOONEP_PULL_PATH`` / ``MOONEP_GRAD_PATH`` / ``MOONEP_PREFETCH_PATH`` override
    ``MOONEP_COPY_PATH`` for one kernel.
    """
    raw = os.environ.get(f"MOONEP_{which.upper()}_PATH") if which else None
    if not raw:
        # measured on 8 B200: bulk stores win for the send, register loads for the pull
        # (bulk loads from peer memory measured below LSU loads, bulk stores to peer memory above LSU stores)
        if which == "prefetch":
            raw = "async"  # measured 668 GB/s against 629 GB/s of the register kernel on 2 B200
        else:
            raw = os.environ.get("MOONEP_COPY_PATH", "ldst" if which in ("pull", "grad") else "bulk")
    raw = raw.lower()
    # "async": 16-byte cp.async copies into per-warp shared-memory rings (prefetch only)
    allowed = ("bulk", "ldst", "async") if which == "prefetch" else ("bulk", "ldst")
    if raw not in allowed:
        raise ValueError(f"copy path must be one of {allowed}, got {raw!r}")
    return raw


def copy_path_is_set(which: str) -> bool:
    """True when the environment names the copy path of this kernel explicitly."""
    return bool(os.environ.get(f"MOONEP_{which.upper()}_PATH"))


def local_sms(sm_count: int) -> int:
    """CTAs for kernels that only touch local memory (planner, dedup expansion, duplicate folding)."""
    raw = os.environ.get("MOONEP_LOCAL_SMS")
    if raw is None or raw == "":
        return sm_count
    return max(1, min(int(raw), sm_count))


def pdl_allowed() -> bool:
    return os.environ.get("MOONEP_PDL", "1") not in _FALSE


def force_phased() -> bool:
    return os.environ.get("MOONEP_PHASED", "0") not in _FALSE


def combine_mode() -> str:
    """``push`` or ``pull`` (see the module docstring)."""
    v = os.environ.get("MOONEP_COMBINE", "push").lower()
    if v not in ("push", "pull"):
        raise ValueError(f"MOONEP_COMBINE must be 'push' or 'pull', got {v!r}")
    return v


def wgrad_on_kernel() -> bool:
    """MOONEP_WGRAD=torch: the MoE layer computes weight gradients with per-group torch matmuls instead of the
    grouped tcgen05 kernel (for comparisons)."""
    return os.environ.get("MOONEP_WGRAD", "kernel").lower() != "torch"


def fuse_plan_publish() -> bool:
    """MOONEP_FUSE_PUBLISH=1: a fresh dispatch is one launch; the tokens-per-expert exchange (``plan_publish``) runs as
    the first step of the dispatch kernel.  Default 0: with programmatic dependent launch the separate kernel already
    overlaps the dispatch kernel's set-up, and the fused form measured the same (0.310 against 0.304 ms per round trip
    on 1 GPU, 0.411 against 0.415 ms on 2)."""
    return os.environ.get("MOONEP_FUSE_PUBLISH", "0") not in _FALSE


def local_rows_by_expand() -> bool:
    """The rows of a rank's own tokens are written by the destination-side role of the dispatch kernel straight from
    the input (primary row and duplicates from one read) instead of by the CTAs that drive NVLink.
    MOONEP_LOCAL_ROWS=0: the send role writes them like every other row."""
    return os.environ.get("MOONEP_LOCAL_ROWS", "1") not in _FALSE


def local_home_by_fold() -> bool:
    """Push combine: the rows of a rank's own tokens skip the CTAs that drive NVLink; the fold role writes them
    (folded, or as they are) straight into the rank's own staging chunk.  MOONEP_LOCAL_HOME=0: they go through the
    push role like every other row."""
    return os.environ.get("MOONEP_LOCAL_HOME", "1") not in _FALSE


def backward_overlap() -> bool:
    """MOONEP_BWD_OVERLAP=1: the MoE layer's backward starts ``reduce_grad`` of each weight on the communication stream
    as soon as that weight's gradients exist, beside the remaining GEMMs (which then leave ``num_sms`` SMs to it).
    Default 0: one ``reduce_grad`` for all three weights after the backward's combine (with balanced routing few
    prefetch slots are in use and the smaller GEMM grid costs more than the overlap returns)."""
    return os.environ.get("MOONEP_BWD_OVERLAP", "0") not in _FALSE


def gemm_on_cta_pairs() -> bool:
    """The grouped GEMM runs on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles; measured 9-10 % faster);
    MOONEP_GEMM_PAIR=0 selects the kernel with one CTA per 128 x 256 tile."""
    return os.environ.get("MOONEP_GEMM_PAIR", "1") not in _FALSE


def wgrad_layout() -> str:
    """MOONEP_WGRAD_LAYOUT: ``rows`` (default) feeds the weight-gradient kernel the activations as they are
    (MN-major tiles), ``transposed`` makes K-major copies first."""
    v = os.environ.get("MOONEP_WGRAD_LAYOUT", "rows").lower()
    assert v in ("rows", "transposed"), f"MOONEP_WGRAD_LAYOUT={v!r}: expected rows or transposed"
    return v


def nvtx() -> bool:
    """MOONEP_NVTX=1: wrap every native call in an NVTX range named after the kernel."""
    return os.environ.get("MOONEP_NVTX", "0") not in _FALSE


def num_sms_dedup_is_set() -> bool:
    return bool(os.environ.get("MOONEP_NUM_SMS_DEDUP"))


def num_sms_dedup(max_sms: int) -> int:
    raw = os.environ.get("MOONEP_NUM_SMS_DEDUP")
    if raw is None or raw == "":
        return max_sms
    value = int(raw)
    if not (1 <= value <= max_sms):
        raise ValueError(f"MOONEP_NUM_SMS_DEDUP must be in [1, {max_sms}], got {value}")
    return value
