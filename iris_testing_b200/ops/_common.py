"""Helpers shared by the op wrappers: stream handles, pointer casts, dispatch rule."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as nv


def use_native(t: torch.Tensor) -> bool:
    """CUDA tensors always take the native kernels (a missing library raises);
    CPU tensors take the PyTorch restatement."""
    return t.is_cuda


def stream_ptr(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def ptr(t) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def contiguous_bf16(t: torch.Tensor, name: str) -> torch.Tensor:
    require(t.dtype == torch.bfloat16, f"{name} must be bfloat16 on the CUDA path (got {t.dtype})")
    return t if t.is_contiguous() else t.contiguous()


_declared = set()


def declare(name: str, argtypes, restype=C.c_int):
    if name not in _declared:
        nv.declare(name, argtypes, restype)
        _declared.add(name)
    return getattr(nv.lib(), name)
