"""Constants shared by the Python layer and the CUDA sources.

The numeric values that describe packed encodings and the meta-chunk layout
must agree with ``csrc/moonep.h``; ``tests/test_layout.py`` checks them against
the values the compiled library reports.

Parity: reference ``moonep_td/constants.py:1-9`` (bit widths, barrier slots,
planner block size).
"""

from __future__ import annotations

# Packed int32 encodings used by the destination-side dedup builder:
#   primary_packed = (kidx << NVS_BITS) | loff
RANK_BITS = 7
KIDX_BITS = 7
NVS_BITS = 32 - 1 - KIDX_BITS
NVS_MASK = (1 << NVS_BITS) - 1
MAX_TOPK = 32
MAX_RANKS = 1 << RANK_BITS

# Three legacy barrier words are kept in every meta chunk for layout parity.
BARRIER_SLOTS = 3

# Planner token phase: routing entries are processed in blocks of at most this
# many (token, k) entries; blocks are aligned to whole tokens.
BLOCK_SIZE_P2 = 2048

# Planner kernels work on blocks of whole tokens with at most this many routing entries.
PLAN_BLOCK = 512

# Vestigial tags of the reference's grid barrier; the flag protocol here uses
# monotonically increasing epochs instead.
GRID_SYNC_TAG = 0x80000000
WARP_SYNC_TAG = 0x80000000
DEDUP_BUILDER_WARPS = 4

# Cross-rank flag families (one int32 flag per source rank and family, placed
# after the logical end of each meta chunk).  A signal stores the family's
# current epoch into the receiver's flag; a wait spins until flag >= epoch.
FLAG_READY = 0  # peer finished every earlier use of the symmetric buffers
FLAG_TPE = 1  # peer pushed its tokens-per-expert row
FLAG_PLAN = 2  # peer pushed the src_info of every row it will send here
FLAG_SENT = 3  # peer pushed all hidden rows / route weights
FLAG_COMB = 4  # peer's shard is final and may be pulled by combine
FLAG_GRAD_READY = 5  # peer's reduce buffers are final
FLAG_GRAD_DONE = 6  # peer finished pulling gradient slots
FLAG_PREFETCH = 7  # no cross-rank flag: epoch of the prefetch_weight calls (their per-slot flags are local)
NUM_FLAG_FAMILIES = 8

# Status codes written by kernels into the host-visible status block.
STATUS_OK = 0
STATUS_TIMEOUT = 1
STATUS_BAD_INDEX = 2

# Default budget of a device-side wait, in milliseconds.
DEFAULT_TIMEOUT_MS = 10_000
