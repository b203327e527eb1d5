"""Models built on the Buffer API: the expert-parallel SwiGLU MoE layer, a router + experts block with autograd,
and routing generators for tests and benchmarks."""
