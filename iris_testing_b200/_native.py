"""ctypes binding of ``libb200moe.so`` (the hand-written sm_100a kernels).

The library is built in-tree by :mod:`iris_testing_b200.csrc.build`.  Loading is
lazy: importing the package on a machine without a GPU (or without nvcc) works,
and the CPU reference paths never touch this module.  On a machine *with* a GPU
a missing or unloadable library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Optional

MAX_WORLD = 8
MAX_GROUPS = 128
MAX_EXPERTS = 128

EPI_STORE = 0
EPI_SILU_GATE = 1
EPI_COMBINE = 2
EPI_ROUTER = 3

ST_OVERFLOW = 10      # status code: routed rows exceed a buffer's capacity

STATUS_NAMES = {
    0: "ok",
    1: "timeout: TMA data never arrived in shared memory",
    2: "timeout: MMA never released a shared-memory stage",
    3: "timeout: accumulator never completed",
    4: "timeout: epilogue never released an accumulator",
    5: "timeout: a peer's routing counts never arrived",
    6: "timeout: a dispatched token tile never arrived",
    7: "timeout: combine rows never arrived",
    8: "timeout: a peer never reached the barrier",
    9: "timeout: a peer never finished the previous iteration",
    10: "overflow: routed rows exceed the receive capacity",
    11: "bad index: a computed row/peer index was out of bounds",
    12: "timeout: in-flight async work did not retire at teardown",
}


class NativeError(RuntimeError):
    """Raised when a kernel launch fails or a kernel reports a non-zero status."""


class DispatchArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int),
        ("rank", C.c_int),
        ("e_local", C.c_int),
        ("topk", C.c_int),
        ("num_tokens", C.c_int),
        ("x", C.c_void_p),
        ("send_order", C.c_void_p),
        ("topk_weight", C.c_void_p),
        ("counts_all", C.c_void_p),
        ("counts_flag", C.c_void_p),
        ("epoch", C.c_uint32),
        ("cap_rows", C.c_int),
        ("cap_mtiles", C.c_int),
        ("drop_signal", C.c_int),
        ("peer_recv", C.c_ulonglong * MAX_WORLD),
        ("peer_meta", C.c_ulonglong * MAX_WORLD),
        ("peer_ready", C.c_ulonglong * MAX_WORLD),
        ("group_rows_out", C.c_void_p),
        ("iter_ptr", C.c_void_p),
        ("stride_counts", C.c_ulonglong),
        ("stride_flag", C.c_ulonglong),
        ("stride_recv", C.c_ulonglong),
        ("stride_meta", C.c_ulonglong),
        ("stride_ready", C.c_ulonglong),
        ("trace", C.c_void_p),
        ("trace_tiles", C.c_int),
    ]


class CombineArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int),
        ("row_meta", C.c_void_p),
        ("out_row_stride", C.c_longlong),
        ("max_slots", C.c_int),
        ("peer_out", C.c_ulonglong * MAX_WORLD),
        ("peer_arrived", C.c_ulonglong * MAX_WORLD),
        ("iter_ptr", C.c_void_p),
        ("stride_meta", C.c_ulonglong),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("num_groups", C.c_int),
        ("N", C.c_int),
        ("K", C.c_int),
        ("n_out", C.c_int),
        ("group_m", C.c_int),
        ("group_rows", C.c_void_p),
        ("out", C.c_void_p),
        ("ldo", C.c_longlong),
        ("status", C.c_void_p),
        ("wait_budget_ns", C.c_ulonglong),
        ("single_group_rows", C.c_int),
        ("mma_n", C.c_int),
        ("cta_pair", C.c_int),
        ("a_base", C.c_void_p),
        ("a_rows", C.c_longlong),
        ("l2_hints", C.c_int),
        ("tma_store", C.c_int),
        ("wide_tiles", C.c_int),
        ("dbg", C.c_void_p),
    ]


class RouterArgs(C.Structure):
    _fields_ = [
        ("num_experts", C.c_int),
        ("topk", C.c_int),
        ("renorm", C.c_int),
        ("bias", C.c_void_p),
        ("topk_idx", C.c_void_p),
        ("topk_w", C.c_void_p),
    ]


_LIB: Optional[C.CDLL] = None


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "libb200moe.so"


def available() -> bool:
    """True when the native library has been built (it may still need a GPU to run)."""
    return lib_path().exists()


def _declare(lib: C.CDLL) -> None:
    vp, i32, i64, u64 = C.c_void_p, C.c_int, C.c_longlong, C.c_ulonglong
    sigs = {
        "b200_grouped_gemm": ([vp, i64, vp, i32, i32, C.POINTER(GemmArgs), C.POINTER(DispatchArgs),
                               C.POINTER(CombineArgs), C.POINTER(RouterArgs), i32, vp], i32),
        "b200_gemm_smem_bytes": ([], i32),
    }
    for name, (argtypes, restype) in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype


def declare(name: str, argtypes, restype=C.c_int) -> None:
    """Declare the signature of one more exported symbol (used by op modules)."""
    fn = getattr(lib(), name)
    fn.argtypes = argtypes
    fn.restype = restype


def lib() -> C.CDLL:
    """Load (building first if stale and nvcc is present) and return the library."""
    global _LIB
    if _LIB is None:
        path = lib_path()
        try:
            from .csrc.build import build, is_current
            if not is_current():
                build()
        except Exception as exc:  # no nvcc: fall back to a prebuilt library if there is one
            if not path.exists():
                raise NativeError(f"native library missing and cannot be built: {exc}") from exc
        _LIB = C.CDLL(str(path))
        _declare(_LIB)
    return _LIB


def check(code: int, what: str) -> None:
    if code != 0:
        raise NativeError(f"{what} failed with code {code}"
                          + (" (cudaError)" if code > 0 else " (argument/descriptor error)"))


def status_message(code: int) -> str:
    return STATUS_NAMES.get(int(code), f"unknown status {code}")
