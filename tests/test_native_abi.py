"""The ctypes mirrors of the native argument blocks must match the C structs byte for byte.
Loading the library needs no GPU, so this runs everywhere the library has been built."""
import ctypes as C

import pytest


def _lib():
    from iris_testing_b200 import _native
    try:
        return _native.lib()
    except Exception as exc:        # no nvcc and no prebuilt library on this machine
        pytest.skip(f"native library unavailable: {exc}")


def test_argument_block_sizes_match():
    from iris_testing_b200 import _native as nv
    from iris_testing_b200.models.moe_layer import RetireArgs
    from iris_testing_b200.ops.plan import PlanPushArgs
    lib = _lib()
    sizes = (C.c_int * 4)()
    lib.b200_abi_sizes_gemm(sizes)
    assert list(sizes) == [C.sizeof(nv.GemmArgs), C.sizeof(nv.DispatchArgs), C.sizeof(nv.CombineArgs),
                           C.sizeof(nv.RouterArgs)]
    lib.b200_abi_size_retire_args.restype = C.c_int
    lib.b200_abi_size_plan_push_args.restype = C.c_int
    assert lib.b200_abi_size_retire_args() == C.sizeof(RetireArgs)
    assert lib.b200_abi_size_plan_push_args() == C.sizeof(PlanPushArgs)
    from iris_testing_b200.parallel.padded_a2a import _CapacityArgs
    lib.b200_abi_size_capacity_args.restype = C.c_int
    assert lib.b200_abi_size_capacity_args() == C.sizeof(_CapacityArgs)


def test_limits_agree():
    from iris_testing_b200 import _native as nv
    lib = _lib()
    lib.b200_gemm_smem_bytes.restype = C.c_int
    assert 0 < lib.b200_gemm_smem_bytes() <= 232448
    lib.b200_plan_noalloc_max.restype = C.c_int
    assert lib.b200_plan_noalloc_max() == 1 << 20
    assert nv.MAX_WORLD == 8 and nv.MAX_EXPERTS == 128 and nv.MAX_GROUPS == 128
