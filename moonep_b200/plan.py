"""``MoonEPCommPlan``: everything a rank needs to replay one routing decision.

A plan is produced by a fresh ``Buffer.dispatch`` and is consumed by
``combine``, ``prefetch_weight``, ``reduce_grad`` and by a later hidden-only
``dispatch(plan=...)`` (the backward re-dispatch).

Fields
------
dst[N]                  destination of local entry ``token*K + k``:
                        ``dest_rank*NvS + loff`` for the first entry of a token
                        on that rank (*primary*, its row crosses the link) and
                        ``-(dest_rank*NvS + loff) - 1`` for later entries on
                        the same rank (expanded on the destination).
experts_to_copy[R, B]   global table: remote experts rank ``d`` hosts in its
                        prefetch slots ``[E, E+B)``; ``-1`` = empty slot.
zero_fill_ranges[E+B,2] ``(first pad row, number of pad rows)`` per group.
remote_stats[2]         ``(#remote experts received here, #ranks copying my experts)``.
dup_groups[NvS,3]       destination side: ``(primary loff, dup_start, dup_n)``.
dup_loffs[NvS]          duplicate row offsets, indexed by ``dup_start``.
dup_counts[2]           ``(#groups, #duplicate rows)``.
src_info[NvS]           (optional) destination side: ``src_rank*NvS + token*K + k`` of the entry that landed in
                        each row, ``-1`` for unused rows.
link[NvS]               (optional) destination side: the link word of each row (primary bit, position among the
                        token's primaries, next row of the same token).  With ``src_info`` it lets ``combine``
                        push rows to the tokens' home ranks; plans without them are combined by pulling.

Parity: reference ``moonep_td/planning.py:12-115``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .layout import check_encoding_bounds


@dataclass(frozen=True, slots=True)
class MoonEPCommPlan:
    dst: torch.Tensor
    experts_to_copy: torch.Tensor
    zero_fill_ranges: torch.Tensor
    remote_stats: torch.Tensor
    N: int
    R: int
    E: int
    B: int
    NvS: int
    K: int
    dup_groups: torch.Tensor
    dup_loffs: torch.Tensor
    dup_counts: torch.Tensor
    src_info: torch.Tensor | None = None
    link: torch.Tensor | None = None

    def __post_init__(self) -> None:
        N, R, E, B, NvS = int(self.N), int(self.R), int(self.E), int(self.B), int(self.NvS)
        assert self.dst.dtype == torch.int32 and self.dst.is_contiguous(), "dst must be contiguous int32"
        assert self.dst.numel() == N, "dst must hold one entry per (token, k)"
        for name, shape in (
            ("experts_to_copy", (R, B)),
            ("zero_fill_ranges", (E + B, 2)),
            ("remote_stats", (2,)),
            ("dup_groups", (NvS, 3)),
            ("dup_loffs", (NvS,)),
            ("dup_counts", (2,)),
        ):
            got = tuple(getattr(self, name).shape)
            assert got == shape, f"{name} has shape {got}, expected {shape}"
        for name in ("src_info", "link"):
            t = getattr(self, name)
            assert t is None or tuple(t.shape) == (NvS,), f"{name} must have shape ({NvS},)"

    def tensors(self):
        """The tensors a stream must keep alive while it uses this plan."""
        base = (
            self.dst,
            self.experts_to_copy,
            self.zero_fill_ranges,
            self.remote_stats,
            self.dup_groups,
            self.dup_loffs,
            self.dup_counts,
        )
        return base + tuple(t for t in (self.src_info, self.link) if t is not None)

    def clone(self) -> "MoonEPCommPlan":
        """Deep copy, e.g. to keep a plan for the backward pass."""
        return type(self)(
            dst=self.dst.clone(),
            experts_to_copy=self.experts_to_copy.clone(),
            zero_fill_ranges=self.zero_fill_ranges.clone(),
            remote_stats=self.remote_stats.clone(),
            dup_groups=self.dup_groups.clone(),
            dup_loffs=self.dup_loffs.clone(),
            dup_counts=self.dup_counts.clone(),
            src_info=None if self.src_info is None else self.src_info.clone(),
            link=None if self.link is None else self.link.clone(),
            N=self.N,
            R=self.R,
            E=self.E,
            B=self.B,
            NvS=self.NvS,
            K=self.K,
        )


def _round4(n: int) -> int:
    return (n + 3) & ~3


def _i32(n: int, dev) -> torch.Tensor:
    # Over-allocated to a multiple of four words so kernels may use 16-byte accesses.
    return torch.empty(_round4(n), dtype=torch.int32, device=dev)[:n]


def allocate_planning_outputs(ctx: dict) -> tuple[MoonEPCommPlan, torch.Tensor]:
    """Allocate an empty plan and the ``cu_seqlens[E+B]`` tensor for ``ctx``."""
    E, B, N, NvS, R, K = ctx["E"], ctx["B"], ctx["N"], ctx["NvS"], ctx["R"], ctx["K"]
    dev = ctx["meta_buf"].device
    plan = MoonEPCommPlan(
        dst=_i32(N, dev),
        experts_to_copy=_i32(R * B, dev).view(R, B),
        zero_fill_ranges=_i32((E + B) * 2, dev).view(E + B, 2),
        remote_stats=_i32(2, dev),
        dup_groups=_i32(NvS * 3, dev).view(NvS, 3),
        dup_loffs=_i32(NvS, dev),
        dup_counts=_i32(2, dev),
        src_info=_i32(NvS, dev),
        link=_i32(NvS, dev),
        N=N,
        R=R,
        E=E,
        B=B,
        NvS=NvS,
        K=K,
    )
    return plan, _i32(E + B, dev)


def check_planning_outputs(ctx: dict, cu_seqlens: torch.Tensor, plan: MoonEPCommPlan) -> None:
    E, B = ctx["E"], ctx["B"]
    assert plan.N == ctx["N"] and plan.R == ctx["R"] and plan.E == E and plan.B == B
    assert plan.NvS == ctx["NvS"] and plan.K == ctx["K"]
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.is_contiguous()
    assert tuple(cu_seqlens.shape) == (E + B,)
    check_encoding_bounds(ctx)


def check_plan_for_ctx(ctx: dict, plan: MoonEPCommPlan, device) -> None:
    """Shape/dtype/device checks before a plan is handed to a kernel; the message names the field that is wrong
    (parity: the assertions of reference moonep_td/dispatch.py:126-160 and moonep_td/dispatch_epilogue.py:45-60)."""
    assert isinstance(plan, MoonEPCommPlan), "plan must be a MoonEPCommPlan"
    assert plan.N == ctx["N"] and plan.R == ctx["R"] and plan.K == ctx["K"] and plan.NvS == ctx["NvS"]
    assert plan.E == ctx["E"] and plan.B == ctx["B"]
    E, B, N, NvS, R = ctx["E"], ctx["B"], ctx["N"], ctx["NvS"], ctx["R"]
    shapes = {
        "dst": (N,), "experts_to_copy": (R, B), "zero_fill_ranges": (E + B, 2), "remote_stats": (2,),
        "dup_groups": (NvS, 3), "dup_loffs": (NvS,), "dup_counts": (2,), "src_info": (NvS,), "link": (NvS,),
    }  # fmt: skip
    for name, shape in shapes.items():
        t = getattr(plan, name)
        if t is None:  # the two optional trailing fields
            continue
        assert t.dtype == torch.int32 and t.is_contiguous(), f"plan.{name} must be contiguous int32"
        assert tuple(t.shape) == shape, f"plan.{name} must have shape {shape}, got {tuple(t.shape)}"
        assert t.device == torch.device(device), f"plan.{name} is on the wrong device"
