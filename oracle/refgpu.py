"""ctypes front end for the reference's own CUDA kernels recompiled for sm_100a.  TEST / BENCHMARK
INFRASTRUCTURE ONLY (never imported by the product package).

``oracle/_ref/libsbnet_refgpu.so`` is built by ``make -C oracle refgpu`` from
``oracle/ref_gpu_harness.cu`` plus the reference's kernel headers included in place
(``sbnet_ops/sparse_blocks.cu.h``, ``sbnet_ops/reduce_mask.cu.h``, ``sbnet_ops/zero_block_counters.cu.h``).
The functions mirror the op-level interface on torch CUDA tensors (fp32 only, as in the reference) and
launch on torch's current stream.  ``available()`` is False where neither the reference tree nor a
prebuilt library exists.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(_HERE, "_ref", "libsbnet_refgpu.so")

_i, _f, _p = C.c_int, C.c_float, C.c_void_p
_GEOM = [_i] * 6
_SIGS = {
    "refgpu_sparse_gather": (_i, [_p, _i, _i, _i, _i, _p] + _GEOM + [_i, _p, _i, _p]),
    "refgpu_sparse_scatter": (_i, [_p, _i, _i, _i, _i, _p] + _GEOM + [_i, _p, _i, _i, _i, _p]),
    "refgpu_reduce_mask": (_i, [_p, _i, _i, _i, _f, _i] + _GEOM + [_i, _i, _p, _p, _p]),
}
_lib = None


def build() -> None:
    """``make -C oracle refgpu`` (a no-op with a message when the reference tree is absent)."""
    from . import oracle
    oracle.make(["refgpu"])


def available() -> bool:
    return os.path.exists(LIB)


def _load():
    global _lib
    if _lib is None:
        lib = C.CDLL(LIB)
        for name, (res, args) in _SIGS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class Unsupported(Exception):
    """The shape is one this harness does not cover (status -2)."""


def _check(status: int, what: str) -> None:
    if status == -2:
        raise Unsupported(what)
    if status != 0:
        raise RuntimeError(f"{what}: CUDA error {status}")


def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _f32(t, name):
    import torch
    if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
        raise ValueError(f"{name}: contiguous fp32 CUDA tensor expected")
    return C.c_void_p(t.data_ptr())


def sparse_gather(x, num_active: int, idx, bsize, bstride, boffset, transpose: bool, out):
    N, H, W, Cc = x.shape
    _check(_load().refgpu_sparse_gather(_f32(x, "x"), N, H, W, Cc, _f32(out, "out"), boffset[0], boffset[1],
                                        bsize[0], bsize[1], bstride[0], bstride[1], int(num_active),
                                        C.c_void_p(idx.data_ptr()), int(transpose), _stream()),
           "refgpu_sparse_gather")
    return out


def sparse_scatter_var(stack, num_active: int, idx, ybase, bsize, bstride, boffset, add: bool,
                       atomic: bool = False, transpose: bool = False):
    N, H, W, Cc = ybase.shape
    _check(_load().refgpu_sparse_scatter(_f32(stack, "stack"), N, H, W, Cc, _f32(ybase, "ybase"), boffset[0],
                                         boffset[1], bsize[0], bsize[1], bstride[0], bstride[1],
                                         int(num_active), C.c_void_p(idx.data_ptr()), int(add),
                                         int(transpose), int(atomic), _stream()),
           "refgpu_sparse_scatter")
    return ybase


def reduce_mask_launch(mask, bcount, bsize, bstride, boffset, tol: float, avgpool: bool, idx, count_dev):
    """Asynchronous: ``idx`` (int16 ``[N*bCntH*bCntW, 3]``) and ``count_dev`` (int32 ``[1]``) are CUDA
    tensors the kernels fill; the raw count (no empty-mask rule) is in ``count_dev`` afterwards."""
    N, H, W = mask.shape[0], mask.shape[1], mask.shape[2]
    _check(_load().refgpu_reduce_mask(_f32(mask, "mask"), N, H, W, float(tol), int(avgpool), boffset[0],
                                      boffset[1], bsize[0], bsize[1], bstride[0], bstride[1], bcount[0],
                                      bcount[1], C.c_void_p(idx.data_ptr()), C.c_void_p(count_dev.data_ptr()),
                                      _stream()),
           "refgpu_reduce_mask")
