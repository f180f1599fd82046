"""iris_testing_b200 -- Blackwell-native (sm_100a) expert-parallel MoE library.

Layout: ``ops`` (router, plan, dispatch, shuffle, expert GEMM, combine), ``parallel``
(symmetric heap, gloo backend, NCCL baseline), ``models`` (``MoELayer``), ``utils``
(generators, packing front-end, buffer sets, comparisons), ``csrc`` (CUDA sources).
"""
__version__ = "0.1.0"

from .config import PRESETS, MoEConfig, preset  # noqa: F401
