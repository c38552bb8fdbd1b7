"""Exact (fp64) evaluation of an accumulating scatter, and the bars an add in ANY order must meet.
TEST INFRASTRUCTURE ONLY (numpy): imported by tests and the smoke check, never by the product.

An accumulating scatter over overlapping blocks (``sbnet_ops/sparse_gather.cc:105-130`` with
``add=True``) adds up to ``k`` block values onto each destination element, in an order that the
GPU's reductions -- and the reference's own OpenMP loop -- leave to the schedule.  Two orders differ
in their roundings and in nothing else, and that is checked here instead of being assumed:

* ``exact`` = base + sum of the addends, in fp64 (exact for a handful of fp32 / fp16 terms up to one
  fp64 rounding);
* ``M`` = |base| + sum of |addends| bounds every partial sum of every order, so a result of ``k``
  rounded additions lies within ``k * eps * M`` of ``exact`` (eps = half an ulp of the element type).
  Both the CUDA result and the CPU checker's must lie inside that bound: then the summation order is
  the only thing that separates them;
* where nothing cancels (``|exact| >= sum|addends| / cover``) the difference is also a small RELATIVE
  error of the result: 1e-6 for fp32 (at most four addends, cover four: 16 * 2^-24 < 1e-6, so this
  follows from the bound above).  For 16-bit types 1e-3 is two roundings of the result, which one
  addend meets and two or more addends in different orders cannot, whatever computes them
  (``tests/test_exact_sum_cpu.py`` shows the CPU checker missing it against itself); there the
  k-roundings bound is the bar.
"""
from __future__ import annotations

import numpy as np

EPS = {"float32": 2.0 ** -24, "float16": 2.0 ** -11, "bfloat16": 2.0 ** -8}
RELATIVE_BAR = {"float32": 1e-6, "float16": 1e-3, "bfloat16": 2.0 ** -7}
# red.global.add.f32 flushes subnormal results; fp16 / bf16 reductions are .noftz
FLUSH = {"float32": 2.0 ** -126, "float16": 0.0, "bfloat16": 0.0}


def exact_add(stack, count, indices, base, bsize, bstride, boffset, transpose=False):
    """fp64 sum of ``base`` and every in-range element of the first ``count`` blocks of ``stack``.
    Returns ``(exact, M, k)``: the sum, the sum of magnitudes (both ``[N,H,W,C]`` fp64) and the number
    of addends per pixel (``[N,H,W]`` int32)."""
    N, H, W, C = base.shape
    exact = base.astype(np.float64)
    mag = np.abs(exact)
    k = np.zeros((N, H, W), dtype=np.int32)
    R, S = int(bsize[0]), int(bsize[1])
    for b in range(int(count)):
        n, bh, bw = (int(v) for v in indices[b])
        h0, w0 = int(boffset[0]) + bh * int(bstride[0]), int(boffset[1]) + bw * int(bstride[1])
        ha, hb = max(h0, 0), min(h0 + R, H)
        wa, wb = max(w0, 0), min(w0 + S, W)
        if ha >= hb or wa >= wb:
            continue
        blk = stack[b]
        blk = (blk[:, ha - h0:hb - h0, wa - w0:wb - w0].transpose(1, 2, 0) if transpose
               else blk[ha - h0:hb - h0, wa - w0:wb - w0, :]).astype(np.float64)
        exact[n, ha:hb, wa:wb, :] += blk
        mag[n, ha:hb, wa:wb, :] += np.abs(blk)
        k[n, ha:hb, wa:wb] += 1
    return exact, mag, k


def check_add(result, exact, mag, k, base, cover, what=""):
    """Asserts the two bars of the module docstring on one result array.  Returns the largest
    error in units of the k-roundings bound and the largest relative error on the no-cancellation set."""
    name = np.dtype(result.dtype).name
    eps, bar, flush = EPS[name], RELATIVE_BAR[name], FLUSH[name]
    r = result.astype(np.float64)
    kk = k[..., None].astype(np.float64)
    err = np.abs(r - exact)
    bound = 1.01 * kk * eps * mag + kk * flush
    untouched = (k == 0)
    assert np.array_equal(result[untouched], base[untouched]), f"{what}: elements no block covers were changed"
    worst = float(np.max(np.where(kk > 0, err / np.maximum(bound, 1e-300), 0.0), initial=0.0))
    assert worst <= 1.0, f"{what}: a sum is {worst:.3f}x outside the bound of k rounded additions"
    addends = mag - np.abs(base.astype(np.float64))
    steady = (np.abs(exact) >= addends / max(cover, 1)) & (kk > 0) & (np.abs(exact) > 1e-30)
    if name != "float32":
        steady &= (kk <= 1)          # 16-bit types: see the module docstring
    elif cover > 4:
        # more than four addends per element (the benchmark geometry has at most four): the worst case
        # of k-1 misrounded partial sums grows as (cover-1)*(2*cover+1); same margin as at cover = 4
        bar *= (cover - 1) * (2 * cover + 1) / 27.0
    rel = float(np.max(np.where(steady, err / np.maximum(np.abs(exact), 1e-300), 0.0), initial=0.0))
    assert rel <= bar, f"{what}: relative error {rel:.3e} above {bar:g} where nothing cancels"
    return worst, rel
