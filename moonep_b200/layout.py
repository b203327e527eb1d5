"""Sizes and offsets of the two symmetric buffers of a ``Buffer``.

Every rank owns one chunk of each buffer; chunk ``r`` of the *hidden* buffer is
``[NvS_padded, H]`` bf16 and chunk ``r`` of the *meta* buffer is
``meta_chunk_padded`` int32 words laid out as::

    WEIGHTS_OFF   [NvS]      fp32 gate weight of every received row
    TPE_OFF       [R*E]      tokens-per-expert row of every source rank
    PLAN_OFF      [...]      planner broadcast area (global tables)
    TOPK0_OFF     [N4]       scratch
    ORDER_OFF     [N4]       scratch
    ORDER0_OFF    [N4]       scratch
    BARRIER_OFF   [3]        legacy barrier words
    SRC_INFO_OFF  [NvS]      src_rank*NvS + slot of the row that lands here, or -1
    SYNC_OFF      [F*R32]    epoch flags, one per (family, source rank)
    LINK_OFF      [NvS]      per landed row: primary bit, position among the token's primaries, and the next
                             row of the same (source, token)
    ROWFLAG_OFF   [NvS]      per row: epoch of the dispatch that last put data into it (rows are flagged one by
                             one as they land, so consumers need not wait for the whole all-to-all)

All chunks of a buffer are mapped back to back in one virtual address range, so
chunk ``r`` starts ``r * chunk_bytes`` after the base on every rank.  The chunk
size is rounded up to ``gran_bytes``: 128 B for host/emulated memory, the CUDA
VMM allocation granularity (2 MiB) for real peer-mapped memory.

Parity: reference ``moonep_td/api.py:50-149`` (``_create_context``) and
``moonep_td/buffer.py:22-37`` (padding helpers).  Offsets up to ``SRC_INFO_OFF``
are the reference's; ``SYNC_OFF``, ``LINK_OFF`` and ``ROWFLAG_OFF`` are additions placed past the reference's logical end.
"""

from __future__ import annotations

from .constants import BARRIER_SLOTS, BLOCK_SIZE_P2, KIDX_BITS, MAX_RANKS, MAX_TOPK, NUM_FLAG_FAMILIES, NVS_BITS

_ELEM_SIZE = {"bfloat16": 2, "float16": 2, "float32": 4, "int32": 4, "int64": 8, "uint8": 1, "int16": 2}


def align_up(x: int, alignment: int) -> int:
    return ((x + alignment - 1) // alignment) * alignment


def elem_size(dtype) -> int:
    name = str(dtype).replace("torch.", "")
    return _ELEM_SIZE[name]


def pad_to_granularity(nbytes: int, gran_bytes: int = 128) -> int:
    return align_up(nbytes, gran_bytes)


def pad_dim0_for_alignment(chunk_shape, dtype, gran_bytes: int = 128) -> int:
    """Smallest dim0 >= chunk_shape[0] whose chunk size is a multiple of gran_bytes."""
    inner = elem_size(dtype)
    for d in chunk_shape[1:]:
        inner *= int(d)
    dim0 = align_up(int(chunk_shape[0]) * inner, gran_bytes) // inner
    while (dim0 * inner) % gran_bytes:
        dim0 += 1
    return dim0


def planner_block_entries(K: int) -> int:
    """Routing entries per planner block: whole tokens, at most BLOCK_SIZE_P2 entries."""
    return max(1, BLOCK_SIZE_P2 // K) * K


def compute_layout(S, H, K, E, R, *, B=None, num_sms=None, token_padding=128, gran_bytes=128) -> dict:
    """Return the integer part of a Buffer context (no tensors)."""
    S, H, K, E, R = int(S), int(H), int(K), int(E), int(R)
    assert R >= 1 and E % R == 0, f"E={E} must be a multiple of num_ep_ranks={R}"
    assert S >= 1 and K >= 1 and H >= 1 and token_padding >= 1
    epn = E // R
    if B is None:
        B = epn
    if num_sms is None:
        num_sms = 32
    N = S * K
    NvS_capacity = N
    token_padding_extra = (token_padding - 1) * 2 * epn
    NvS = NvS_capacity + token_padding_extra
    num_vblocks = (N + BLOCK_SIZE_P2 - 1) // BLOCK_SIZE_P2
    NvS_padded = pad_dim0_for_alignment([NvS, H], "bfloat16", gran_bytes)

    WEIGHTS_OFF = 0
    TPE_OFF = align_up(NvS, 4)
    PLAN_OFF = align_up(TPE_OFF + R * E, 4)
    broadcast_elems = 3 * E * R
    planning_out_elems = broadcast_elems + R * (E + B) + 2 * R * (E + B) + B * R + 2 * R
    N4 = align_up(N, 4)
    TOPK0_OFF = align_up(PLAN_OFF + planning_out_elems, 4)
    ORDER_OFF = TOPK0_OFF + N4
    ORDER0_OFF = ORDER_OFF + N4
    BARRIER_OFF = ORDER0_OFF + N4
    SRC_INFO_OFF = BARRIER_OFF + BARRIER_SLOTS
    R32 = align_up(R, 32)
    SYNC_OFF = align_up(SRC_INFO_OFF + NvS, 32)
    LINK_OFF = SYNC_OFF + NUM_FLAG_FAMILIES * R32
    ROWFLAG_OFF = align_up(LINK_OFF + NvS, 32)  # 16-byte aligned: consumers read four flags per load
    meta_chunk_logical = ROWFLAG_OFF + NvS
    meta_chunk_padded = align_up(meta_chunk_logical * 4, gran_bytes) // 4

    return {
        "R": R,
        "E": E,
        "S": S,
        "K": K,
        "H": H,
        "B": int(B),
        "N": N,
        "epn": epn,
        "NvS": NvS,
        "NvS_capacity": NvS_capacity,
        "NvS_padded": NvS_padded,
        "num_sms": int(num_sms),
        "num_sms_dedup": int(num_sms),
        "token_padding": int(token_padding),
        "token_padding_extra": token_padding_extra,
        "num_vblocks": num_vblocks,
        "gran_bytes": int(gran_bytes),
        "meta_chunk_padded": meta_chunk_padded,
        "WEIGHTS_OFF": WEIGHTS_OFF,
        "TPE_OFF": TPE_OFF,
        "PLAN_OFF": PLAN_OFF,
        "TOPK0_OFF": TOPK0_OFF,
        "ORDER_OFF": ORDER_OFF,
        "ORDER0_OFF": ORDER0_OFF,
        "BARRIER_OFF": BARRIER_OFF,
        "SRC_INFO_OFF": SRC_INFO_OFF,
        "SYNC_OFF": SYNC_OFF,
        "LINK_OFF": LINK_OFF,
        "ROWFLAG_OFF": ROWFLAG_OFF,
        "Kp": min(K, R),
        "R32": R32,
    }


def check_encoding_bounds(lay: dict) -> None:
    """Limits of the packed int32 encodings (dst, src_info, primary_packed)."""
    R, S, K, NvS = lay["R"], lay["S"], lay["K"], lay["NvS"]
    assert S * K <= NvS
    assert R * NvS <= 2**31 - 1, "R*NvS must fit in int32"
    assert R <= MAX_RANKS, f"at most {MAX_RANKS} ranks"
    assert K <= (1 << KIDX_BITS) - 1 and K <= MAX_TOPK, f"K must be <= {MAX_TOPK}"
    assert NvS <= (1 << NVS_BITS) - 1, "NvS must fit in 24 bits"
