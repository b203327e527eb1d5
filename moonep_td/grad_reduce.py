"""``moonep_td.grad_reduce`` -> ``moonep_b200.ops.launch.launch_grad_reduce``: gradient reduction to the owners (reference moonep_td/grad_reduce.py:183)."""

from moonep_b200.ops.launch import launch_grad_reduce  # noqa: F401
