"""``moonep_td.planning`` -> plan dataclass and planner launch of ``moonep_b200``."""

from moonep_b200.ops.launch import launch_planning  # noqa: F401
from moonep_b200.plan import MoonEPCommPlan, allocate_planning_outputs  # noqa: F401
