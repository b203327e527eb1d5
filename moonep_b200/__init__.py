"""moonep_b200: load-balanced expert-parallel MoE communication for NVIDIA B200 (sm_100a).

Public surface (parity: reference ``moonep_td/__init__.py:1-7``)::

    from moonep_b200 import Buffer, MoonEPCommPlan
"""

from .api import Buffer, CapturedStep
from .plan import MoonEPCommPlan

__all__ = ["Buffer", "CapturedStep", "MoonEPCommPlan"]
__version__ = "0.1.0"
