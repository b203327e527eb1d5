"""Drop-in import name for code written against MoonEP-Triton-Distributed.

``from moonep_td import Buffer, MoonEPCommPlan`` resolves to the sm_100a implementation in
``moonep_b200``.  The helper modules keep their names: ``moonep_td.buffer`` (symmetric tensors and
padding helpers), ``moonep_td.planning`` (plan dataclass, ``allocate_planning_outputs``,
``launch_planning``), ``moonep_td.api``, and one module per launch-level function (``moonep_td.dispatch``,
``dispatch_epilogue``, ``combine``, ``combine_prologue``, ``prefetch``, ``grad_reduce``, ``inter_rank_sync``,
``_dedup_builder``).  The launch-level functions take the same arguments as there, except that the ones which the
reference gives a bare tensor list also take the context.
"""

from moonep_b200 import Buffer, MoonEPCommPlan

__all__ = ["Buffer", "MoonEPCommPlan"]
