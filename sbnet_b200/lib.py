"""ctypes binding of ``libsbnet_b200.so`` (the C ABI declared in ``include/sbnet_b200.h``).

There is no fallback: if the library has not been built, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# SBNET_B200_LIB selects another build of the same library (e.g. an instrumented one)
LIB_PATH = os.environ.get("SBNET_B200_LIB") or os.path.join(PKG, "libsbnet_b200.so")

SBNET_F32, SBNET_F16, SBNET_BF16 = 0, 1, 2
SBNET_SCRATCH_CLEAN = 1
SBNET_COUNT_POLL = 2
SBNET_MASK_STABLE = 4
SBNET_COUNT_YIELD = 8
SBNET_COUNT_NOWAIT = 16
SBNET_COUNT_PENDING = -(2 ** 31)
SBNET_REDUCE_MASK_SCRATCH_INTS = 4

_i, _f, _p, _sz = C.c_int, C.c_float, C.c_void_p, C.c_size_t
_GEOM = [_i] * 6
_TENSOR = [_p, _i, _i, _i, _i, _i, _p]  # x, dtype, N, H, W, C, y

# name -> (restype, argtypes); one entry per declaration in include/sbnet_b200.h
SIGNATURES = {
    "sbnet_version": (_i, []),
    "sbnet_last_error": (C.c_char_p, []),
    "sbnet_reduce_mask": (_i, [_p, _i, _i, _i, _f, _i] + _GEOM + [_i, _i, _p, _p, _p, _i, _p]),
    "sbnet_sparse_gather": (_i, _TENSOR + _GEOM + [_i, _p, _i, _p]),
    "sbnet_sparse_gather_dyn": (_i, _TENSOR + _GEOM + [_i, _p, _p, _i, _p]),
    "sbnet_sparse_scatter": (_i, _TENSOR + _GEOM + [_i, _p, _i, _i, _i, _p]),
    "sbnet_sparse_scatter_dyn": (_i, _TENSOR + _GEOM + [_i, _p, _p, _i, _i, _i, _p]),
    "sbnet_copy_tensor": (_i, [_p, _p, _sz, _p]),
    "sbnet_cuda_timer_start": (_i, [C.POINTER(C.c_int64)]),
    "sbnet_cuda_timer_end": (_i, [C.c_int64, C.POINTER(_f)]),
    "sbnet_wait_timeouts": (_i, [C.POINTER(C.c_uint)]),
    "sbnet_set_option": (_i, [C.c_char_p, _i]),
    "sbnet_get_option": (_i, [C.c_char_p, C.POINTER(_i)]),
    "sbnet_reduce_mask_static": (_i, [_p, _i, _i, _i, _f, _i] + _GEOM + [_i, _i, _p, _p, _p, _p]),
}

_lib = None


class SbnetError(RuntimeError):
    """A CUDA runtime error reported by the library (positive status)."""


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m sbnet_b200.build` "
                "(needs nvcc; there is no CPU or PyTorch fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int) -> None:
    """0 -> ok; negative -> ValueError (the reference raises InvalidArgument); positive -> CUDA error."""
    if status == 0:
        return
    msg = load().sbnet_last_error().decode("utf-8", "replace")
    if status < 0:
        raise ValueError(msg)
    raise SbnetError(msg)


def set_option(name: str, value: int) -> None:
    """Sets one of the library's process-wide switches (``sbnet_set_option``)."""
    check(load().sbnet_set_option(name.encode(), int(value)))


def get_option(name: str) -> int:
    out = _i(0)
    check(load().sbnet_get_option(name.encode(), C.byref(out)))
    return out.value


def wait_timeouts() -> int:
    """Bounded device-side waits that gave up since the library was loaded (0 in a healthy process)."""
    out = C.c_uint(0)
    check(load().sbnet_wait_timeouts(C.byref(out)))
    return out.value
