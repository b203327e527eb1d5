"""``moonep_td.constants`` -> ``moonep_b200.constants``."""

from moonep_b200.constants import *  # noqa: F401,F403
