"""SiLU gate ``silu(gate) * up`` as a stand-alone op (the fused path does this
inside the first GEMM's epilogue).  No counterpart in the reference."""
from __future__ import annotations

import ctypes as C

import torch

from . import cpu_ref
from ._common import contiguous_bf16, declare, ptr, require, stream_ptr, use_native


def silu_gate(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    require(gate.shape == up.shape, "gate and up must have the same shape")
    if not use_native(gate):
        return cpu_ref.silu_gate_ref(gate, up).to(gate.dtype)
    gate, up = contiguous_bf16(gate, "gate"), contiguous_bf16(up, "up")
    require(gate.numel() % 2 == 0, "element count must be even")
    fn = declare("b200_silu_gate", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p])
    out = torch.empty_like(gate)
    rc = fn(ptr(gate), ptr(up), ptr(out), gate.numel(), stream_ptr(gate))
    if rc != 0:
        raise RuntimeError(f"silu_gate launch failed ({rc})")
    return out
