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


_DEFAULT_STATUS = {}


def default_status(device) -> torch.Tensor:
    """The device's default status word (int32 [4], zero = ok): where a kernel launched
    without a caller-owned status tensor records timeouts, overflows and bad indices, so that
    such a report is never dropped.  Read it with :func:`check_default_status`."""
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _DEFAULT_STATUS.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _DEFAULT_STATUS[idx] = t
    return t


def check_default_status(device=None, reset: bool = True) -> None:
    """Raise if a kernel that was launched without a caller-owned status tensor has reported
    an error on ``device`` (default: the current device).  Synchronises."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    st = default_status(device).tolist()
    if st[0] != 0:
        if reset:
            default_status(device).zero_()
        extra = f" (rows needed: {st[1]})" if st[0] == 10 and st[1] > 0 else ""
        raise nv.NativeError(f"device status {st[0]}: {nv.status_message(st[0])}{extra}")
