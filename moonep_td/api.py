"""``moonep_td.api`` -> ``moonep_b200.api``."""

from moonep_b200.api import Buffer, _create_context  # noqa: F401
from moonep_b200.plan import MoonEPCommPlan  # noqa: F401
