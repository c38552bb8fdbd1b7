"""Runs one reference-style case (mask -> reduce_mask -> gather -> scatter) through any
implementation of the four ops and normalises the result for comparison.

``ops`` is an object with the reference op names (``reduce_mask``, ``sparse_gather``,
``sparse_scatter``, ``sparse_scatter_var``) working on numpy arrays: the CPU checker
(``oracle.oracle.OracleLib``) or the numpy adapter over the CUDA library.  Block order is
normalised the way the reference's own test does it
(``sbnet_ops/tests/test_sparse_blocks.py:310-317``): sort by n*BCH*BCW + h*BCW + w and permute the
gathered stack accordingly.
"""
from __future__ import annotations

import hashlib

import numpy as np

from ref_cases import RefCase, make_inputs


def sort_order(indices, count, bcount):
    idx = np.asarray(indices[:count]).astype(np.int64)
    key = idx[:, 0] * bcount[0] * bcount[1] + idx[:, 1] * bcount[1] + idx[:, 2]
    return np.argsort(key, kind="stable")


def run_case(ops, case: RefCase, transpose: bool, inputs=None):
    mask, x, tol, bcount = inputs if inputs is not None else make_inputs(case)
    idx, cnt = ops.reduce_mask(mask, list(bcount), list(case.RS), list(case.UV), list(case.BOFFS),
                               tol=tol, avgpool=case.avgpool)
    count = int(cnt[0])
    stack = ops.sparse_gather(x, cnt, idx, list(case.RS), list(case.UV), list(case.BOFFS),
                              transpose=transpose)
    base = (x * 0.0 + 10.0).astype(np.float32)
    scatter = ops.sparse_scatter_var if case.test_var else ops.sparse_scatter
    y = scatter(stack, cnt, idx, base, list(case.RS), list(case.UV), list(case.BOFFS),
                add=case.do_add, atomic=case.use_atomics, transpose=transpose)
    order = sort_order(idx, count, bcount)
    return dict(count=count, indices=np.asarray(idx[:count])[order].copy(),
                stack=np.asarray(stack)[order].copy(), y=np.asarray(y).copy())


def digest(a: np.ndarray) -> str:
    a = np.ascontiguousarray(a)
    return hashlib.sha256(a.tobytes()).hexdigest()[:32]
