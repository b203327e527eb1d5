"""Launch-level API: the ``launch_*`` functions that take a Buffer context dict.

They exist for users (and tests) that drive single stages instead of ``Buffer.dispatch`` /
``Buffer.combine``.  ``ctx = buffer._require_ctx()``.  Each function is collective across the
ranks of the Buffer's world and enqueues on the current stream (CUDA) or runs at once (CPU).

Parity: reference ``launch_planning`` (``moonep_td/planning.py:164``), ``launch_dispatch``
(``dispatch.py:126``), ``launch_dispatch_epilogue`` (``dispatch_epilogue.py:45``),
``launch_combine_prologue`` (``combine_prologue.py:45``), ``launch_combine`` (``combine.py:77``),
``launch_prefetch`` (``prefetch.py:73``), ``launch_grad_reduce`` (``grad_reduce.py:183``),
``launch_dedup_builder`` (``_dedup_builder.py:113``), ``launch_inter_rank_sync``
(``inter_rank_sync.py:1-9``), ``launch_cross_rank_barrier`` (``_common.py:75``).
"""

from __future__ import annotations

import torch

from ..constants import FLAG_PLAN, FLAG_READY, FLAG_SENT
from ..plan import MoonEPCommPlan, allocate_planning_outputs, check_plan_for_ctx, check_planning_outputs

__all__ = [
    "allocate_planning_outputs",
    "launch_planning",
    "launch_dispatch",
    "launch_dispatch_epilogue",
    "launch_dedup_builder",
    "launch_combine_prologue",
    "launch_combine",
    "launch_prefetch",
    "launch_grad_reduce",
    "launch_inter_rank_sync",
    "launch_cross_rank_barrier",
]


def _be(ctx):
    return ctx["_backend"]


def launch_cross_rank_barrier(ctx: dict) -> None:
    """All ranks' earlier work on the symmetric buffers is complete and visible when this returns (in stream order)."""
    _be(ctx).barrier()


launch_inter_rank_sync = launch_cross_rank_barrier


def launch_planning(ctx, topk_experts_flat, tokens_per_expert, cu_seqlens, plan: MoonEPCommPlan) -> None:
    """Fill ``plan`` (dst, experts_to_copy, zero_fill_ranges, remote_stats) and ``cu_seqlens``; publish
    src_info and link words to the destination ranks.  Ends with a wait for every rank's planner."""
    check_planning_outputs(ctx, cu_seqlens, plan)
    be = _be(ctx)
    topk = topk_experts_flat.reshape(-1).to(torch.int32).contiguous()
    tpe = tokens_per_expert.to(torch.int32).contiguous()
    be.plan_publish(tpe, topk)
    be.plan_compute(topk, tpe, cu_seqlens, plan)
    if ctx["world"].is_cuda:
        be.wait(FLAG_PLAN)
    ctx["_standalone_plan"] = True


def launch_dispatch(ctx, hidden_sh, route_weights_sk, plan, *, build_dedup_map=False, pdl_trigger=False) -> None:
    """Push rows and weights (and build the dedup map when asked); all rows have landed when this returns."""
    del pdl_trigger
    S, H, K = ctx["S"], ctx["H"], ctx["K"]
    assert hidden_sh.dtype == torch.bfloat16 and hidden_sh.is_contiguous(), "hidden_sh must be contiguous bf16"
    assert tuple(hidden_sh.shape) == (S, H), "hidden_sh shape mismatch"
    if route_weights_sk is not None:
        assert route_weights_sk.dtype == torch.float32 and route_weights_sk.is_contiguous(), \
            "route_weights_sk must be contiguous fp32"
        assert tuple(route_weights_sk.shape) == (S, K), "route_weights_sk shape mismatch"
    check_plan_for_ctx(ctx, plan, hidden_sh.device)
    be = _be(ctx)
    fresh = bool(ctx.pop("_standalone_plan", False))
    if not fresh:
        be.signal(FLAG_READY)
    be.dispatch_send(hidden_sh, route_weights_sk, plan, build_dedup_map, wait=FLAG_PLAN if fresh else FLAG_READY)
    if ctx["world"].is_cuda:
        be.wait(FLAG_SENT)


def launch_dedup_builder(ctx, plan) -> None:
    """Rebuild ``dup_groups / dup_loffs / dup_counts`` of ``plan`` (and its copies of src_info and the link words)
    from what the last planning published into this rank's meta chunk."""
    _be(ctx).build_dedup(plan)


def launch_dispatch_epilogue(ctx, plan, *, pdl_launch=False) -> None:
    """Zero the pad rows and copy every primary row to its duplicates inside the local shard."""
    del pdl_launch
    check_plan_for_ctx(ctx, plan, plan.dst.device)
    _be(ctx).dispatch_expand(plan, None, None, True)


def launch_combine_prologue(ctx, plan, *, pdl_trigger=False) -> None:
    """Fold duplicate rows into their primaries (fp32 sum, bf16 in place) in the local shard."""
    del pdl_trigger
    _be(ctx).combine_prologue(plan, None, None, True, wait=None)


def launch_combine(ctx, output_sh, dst, output_sk=None, *, pdl_launch=False) -> None:
    """Pull the primary rows of every token and sum them into ``output_sh``; gather weights into ``output_sk``."""
    del pdl_launch
    assert output_sh.dtype == torch.bfloat16 and output_sh.is_contiguous(), "output_sh must be contiguous bf16"
    assert dst.dtype == torch.int32 and dst.is_contiguous(), "dst must be contiguous int32"
    if output_sk is not None:
        assert output_sk.dtype == torch.float32 and output_sk.is_contiguous(), "output_sk must be contiguous fp32"
        assert tuple(output_sk.shape) == (ctx["S"], ctx["K"]), "output_sk shape mismatch"
    _be(ctx).combine_pull(dst, output_sh, output_sk)


def launch_prefetch(ctx, remote_expert, prefetch_buffers, experts_to_copy_row) -> None:
    """Copy ``remote_expert[experts_to_copy_row[b]]`` into ``prefetch_buffers[b]`` for every ``b`` with a valid id."""
    if prefetch_buffers.numel() == 0 or experts_to_copy_row.numel() == 0:
        return
    _be(ctx).prefetch_launch([remote_expert], [prefetch_buffers], experts_to_copy_row)


def launch_grad_reduce(ctx, remote_expert_grads, remote_reduce_buffers, experts_to_copy) -> None:
    """``grad[e] += sum of reduce slots holding e`` on the owner (ascending slot order), then clear own slots."""
    if remote_reduce_buffers.numel() == 0 or experts_to_copy.numel() == 0:
        return
    _be(ctx).reduce_grad(experts_to_copy, [remote_expert_grads], [remote_reduce_buffers])
