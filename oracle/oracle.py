"""ctypes front end for the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Two libraries export the same ``oracle_*`` table:

* ``port`` -- ``oracle/libsbnet_oracle.so``, built from ``oracle/sbnet_oracle.c`` (the C restatement
  kept in this repository);
* ``ref``  -- ``oracle/_ref/libsbnet_ref.so``, the reference's own CPU functors
  (``sbnet_ops/reduce_mask.cc:46-98``, ``sbnet_ops/sparse_gather.cc:61-142``) compiled unchanged by
  ``oracle/Makefile``.

The functions below mirror the reference's op-level interface (``REGISTER_OP`` blocks in
``sbnet_ops/reduce_mask.cc:100-110`` and ``sbnet_ops/sparse_gather.cc:48-57,242-268``) on numpy
arrays: geometry arrives as length-2 ``[H, W]`` sequences, ``bin_counts`` is a length-1 int32 array,
``active_block_indices`` is ``[N*bCntH*bCntW, 3]`` int16.  Only tests, the smoke check and the
benchmark's CPU legs may import this module; the product never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_LIB = os.path.join(_HERE, "libsbnet_oracle.so")
REF_LIB = os.path.join(_HERE, "_ref", "libsbnet_ref.so")

_i, _f, _p = C.c_int, C.c_float, C.c_void_p
_GEOM = [_i] * 6
_SIGS = {
    "oracle_set_threads": (None, [_i]),
    "oracle_max_threads": (_i, []),
    "oracle_reduce_mask": (None, [_p, _i, _i, _i, _f] + _GEOM + [_i, _i, _p, _p, _i]),
    "oracle_reduce_mask_op": (None, [_p, _i, _i, _i, _f] + _GEOM + [_i, _i, _p, _p, _i]),
    "oracle_sparse_gather_f32": (None, [_p, _i, _i, _i, _i, _p] + _GEOM + [_i, _p, _i]),
    "oracle_sparse_gather_f16": (None, [_p, _i, _i, _i, _i, _p] + _GEOM + [_i, _p, _i]),
    "oracle_sparse_scatter_f32": (None, [_p, _i, _i, _i, _i, _p] + _GEOM + [_i, _p, _i, _i, _i]),
    "oracle_sparse_scatter_f16": (None, [_p, _i, _i, _i, _i, _p] + _GEOM + [_i, _p, _i, _i, _i]),
    "oracle_sparse_gather_bf16": (None, [_p, _i, _i, _i, _i, _p] + _GEOM + [_i, _p, _i]),
    "oracle_sparse_scatter_bf16": (None, [_p, _i, _i, _i, _i, _p] + _GEOM + [_i, _p, _i, _i, _i]),
    "oracle_copy_tensor": (None, [_p, _p, C.c_size_t]),
}


def reference_ops_dir():
    """``sbnet_tensorflow/sbnet_ops`` of the reference tree, or None: ``$SBNET_REFERENCE`` names the
    tree's root, else a directory called ``reference`` beside this repository is tried."""
    root = os.environ.get("SBNET_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    ops = os.path.join(root, "sbnet_tensorflow", "sbnet_ops")
    return ops if os.path.isfile(os.path.join(ops, "sparse_gather.cc")) else None


def make(targets) -> None:
    ops = reference_ops_dir()
    subprocess.run(["make", "-s", "-C", _HERE] + list(targets) + ([f"REF={ops}"] if ops else []), check=True)


def build(ref: bool = True) -> None:
    """Compile the checkers (``make -C oracle``).  Building the checker is not using it."""
    make(["port"] + (["ref"] if ref else []))


class OracleLib:
    """One loaded checker library (``kind`` is ``"port"`` or ``"ref"``)."""

    def __init__(self, kind: str = "port"):
        path = {"port": PORT_LIB, "ref": REF_LIB}[kind]
        if not os.path.exists(path):
            if kind == "port":
                build(ref=False)
            else:
                raise FileNotFoundError(path)
        self.kind = kind
        self.lib = C.CDLL(path)
        for name, (res, args) in _SIGS.items():
            fn = getattr(self.lib, name)
            fn.restype, fn.argtypes = res, args

    # ---- helpers -------------------------------------------------------------------------------
    @staticmethod
    def _ptr(a: np.ndarray):
        return a.ctypes.data_as(C.c_void_p)

    @staticmethod
    def _pair(v, name):
        v = np.asarray(v)
        if v.ndim != 1 or v.shape[0] != 2:  # reduce_mask.cc:132-138, sparse_gather.cc:170-175
            raise ValueError(f"{name} should be one-dimensional with shape[0] == 2")
        return int(v[0]), int(v[1])

    def set_threads(self, n: int) -> None:
        self.lib.oracle_set_threads(int(n))

    def max_threads(self) -> int:
        return int(self.lib.oracle_max_threads())

    # ---- ops -----------------------------------------------------------------------------------
    def reduce_mask(self, mask, dynamic_bcount, dynamic_bsize, dynamic_bstride, dynamic_boffset,
                    tol, avgpool=False, op_fixup=True):
        """``ReduceMask``: returns ``(active_block_indices [N*bCntH*bCntW,3] int16, bin_counts [1] int32)``.
        Rows past ``bin_counts[0]`` are zero here (the reference leaves them undefined)."""
        mask = np.ascontiguousarray(mask, dtype=np.float32)
        N, H, W = mask.shape[0], mask.shape[1], mask.shape[2]
        bch, bcw = self._pair(dynamic_bcount, "dynamic_bcount")
        bsh, bsw = self._pair(dynamic_bsize, "dynamic_bsize")
        bth, btw = self._pair(dynamic_bstride, "dynamic_bstride")
        boh, bow = self._pair(dynamic_boffset, "dynamic_boffset")
        idx = np.zeros((max(N * bch * bcw, 1), 3), dtype=np.int16)
        cnt = np.zeros(1, dtype=np.int32)
        fn = self.lib.oracle_reduce_mask_op if op_fixup else self.lib.oracle_reduce_mask
        fn(self._ptr(mask), N, H, W, float(tol), boh, bow, bsh, bsw, bth, btw, bch, bcw,
           self._ptr(idx), self._ptr(cnt), int(bool(avgpool)))
        return idx[: N * bch * bcw], cnt

    def _fns(self, dtype):
        if dtype == np.float32:
            return self.lib.oracle_sparse_gather_f32, self.lib.oracle_sparse_scatter_f32
        if dtype == np.float16:
            return self.lib.oracle_sparse_gather_f16, self.lib.oracle_sparse_scatter_f16
        if np.dtype(dtype).name == "bfloat16":   # ml_dtypes.bfloat16 (numpy itself has no bfloat16)
            return self.lib.oracle_sparse_gather_bf16, self.lib.oracle_sparse_scatter_bf16
        raise TypeError(f"unsupported dtype {dtype}")

    def sparse_gather(self, x, bin_counts, active_block_indices, dynamic_bsize, dynamic_bstride,
                      dynamic_boffset, transpose=False):
        """``SparseGather``: ``[nB,bSzH,bSzW,C]`` or, transposed, ``[nB,C,bSzH,bSzW]``."""
        x = np.ascontiguousarray(x)
        if x.ndim != 4:  # sparse_gather.cc:164
            raise ValueError("x must be rank 4")
        N, H, W, Cc = x.shape
        bsh, bsw = self._pair(dynamic_bsize, "dynamic_bsize")
        bth, btw = self._pair(dynamic_bstride, "dynamic_bstride")
        boh, bow = self._pair(dynamic_boffset, "dynamic_boffset")
        nb = int(np.asarray(bin_counts).reshape(-1)[0])
        idx = np.ascontiguousarray(active_block_indices, dtype=np.int16)
        shape = (nb, Cc, bsh, bsw) if transpose else (nb, bsh, bsw, Cc)
        y = np.empty(shape, dtype=x.dtype)
        gather, _ = self._fns(x.dtype)
        gather(self._ptr(x), N, H, W, Cc, self._ptr(y), boh, bow, bsh, bsw, bth, btw, nb,
               self._ptr(idx), int(bool(transpose)))
        return y

    def sparse_scatter_var(self, x, bin_counts, active_block_indices, ybase, dynamic_bsize,
                           dynamic_bstride, dynamic_boffset, add, atomic=False, transpose=False):
        """``SparseScatterVar``: scatters into ``ybase`` in place and returns it."""
        if ybase.ndim != 4:  # sparse_gather.cc:327
            raise ValueError("ybase must be rank 4")
        if not ybase.flags["C_CONTIGUOUS"]:
            raise ValueError("ybase must be contiguous")
        N, H, W, Cc = ybase.shape
        bsh, bsw = self._pair(dynamic_bsize, "dynamic_bsize")
        bth, btw = self._pair(dynamic_bstride, "dynamic_bstride")
        boh, bow = self._pair(dynamic_boffset, "dynamic_boffset")
        if add and not atomic and not (bth >= bsh and btw >= bsw):  # sparse_gather.cc:322-326
            raise ValueError("Only non-overlapping blocks are supported with add=True, atomic=False")
        x = np.ascontiguousarray(x, dtype=ybase.dtype)
        nb = int(np.asarray(bin_counts).reshape(-1)[0])
        idx = np.ascontiguousarray(active_block_indices, dtype=np.int16)
        _, scatter = self._fns(ybase.dtype)
        scatter(self._ptr(x), N, H, W, Cc, self._ptr(ybase), boh, bow, bsh, bsw, bth, btw, nb,
                self._ptr(idx), int(bool(add)), int(bool(transpose)), int(bool(atomic)))
        return ybase

    def sparse_scatter(self, x, bin_counts, active_block_indices, ybase, dynamic_bsize,
                       dynamic_bstride, dynamic_boffset, add, atomic=False, transpose=False):
        """``SparseScatter``: copy of ``ybase`` (sparse_gather.cc:338-347) with the blocks applied."""
        ybase = np.ascontiguousarray(ybase)
        y = np.empty_like(ybase)
        self.lib.oracle_copy_tensor(self._ptr(y), self._ptr(ybase), ybase.nbytes)
        return self.sparse_scatter_var(x, bin_counts, active_block_indices, y, dynamic_bsize,
                                       dynamic_bstride, dynamic_boffset, add, atomic, transpose)


_CACHE: dict = {}


def get(kind: str = "port") -> OracleLib:
    if kind not in _CACHE:
        _CACHE[kind] = OracleLib(kind)
    return _CACHE[kind]


def have_ref() -> bool:
    return os.path.exists(REF_LIB)


def sort_blocks(indices: np.ndarray, count: int, bcount):
    """Order in which the reference's own test compares GPU results with CPU results
    (``sbnet_ops/tests/test_sparse_blocks.py:310-314``): ascending key n*BCH*BCW + h*BCW + w."""
    idx = np.asarray(indices[:count]).astype(np.int64)
    key = idx[:, 0] * int(bcount[0]) * int(bcount[1]) + idx[:, 1] * int(bcount[1]) + idx[:, 2]
    return np.argsort(key, kind="stable")
