"""B200-native W4G128 / W4A8 matmul path behind mollm's accelerator-backend boundary.

  csrc/      hand-written sm_100a kernels and the extern "C" layer (libb200w4.so)
  capi.py    ctypes binding of that C ABI (tests, bench)
  synth.py   seeded synthetic weights / activations of the benchmark shapes
  shard.py   tensor-parallel (row) and expert-parallel sharding of weights across ranks
  expert_parallel.py  routed MoE over ranks: local expert outputs, all-reduce, ordered combine
  decoder.py a Qwen3-shaped dense decoder driven through the C ABI (benchmark configuration 3)
  package.py reader for the reference's .mollm packages (dense Qwen3, W4G128 weights)
  build.py   in-tree nvcc build

The directory name carries a hyphen, so load it with importlib (see __graft_entry__.py)
under the module name `palm_infra_b200`.
"""
from . import capi, decoder, expert_parallel, package, shard, synth  # noqa: F401
from .build import build as build_library  # noqa: F401
