"""Ops of the expert-parallel pipeline.  CUDA tensors run the hand-written sm_100a
kernels; CPU tensors run the PyTorch restatements in :mod:`.cpu_ref`."""
from . import cpu_ref
from ._common import check_default_status, default_status
from .activation import silu_gate
from .combine import padded_return, weighted_gather
from .dispatch import AllToAllOp, custom_a2a, zero_padding
from .expert import Expert, expert, grouped_gemm, to_kmajor
from .plan import Plan, make_plan, pack_rows
from .router import router_topk
from .shuffle import TokenShuffle, shuffle, unshuffle
