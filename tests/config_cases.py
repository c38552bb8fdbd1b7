"""Benchmark-configuration shaped cases at sizes the CPU checker finishes in well under a second.

Same generators, geometries, dtypes and flag combinations as the full-size configurations
(sbnet_b200/configs.py), smaller tensors.  ``run(ops, name)`` pushes one case through any
implementation of the reference op interface (numpy in, numpy out) and returns the arrays to compare
plus their digests.  Arrays listed in ``tol`` come from atomic adds over overlapping halos, whose
floating-point add order is schedule dependent: they are held to the fp64 exact-sum bars
(``tests/atomic_check.py``) from the inputs returned under ``atomic``; every other array must match
bit for bit.
"""
from __future__ import annotations

import numpy as np

from sbnet_b200 import configs as cfg
import pipeline


def _sorted_stack(stack, idx, cnt, bcount):
    order = pipeline.sort_order(idx, int(cnt[0]), bcount)
    return np.asarray(stack)[order]


def _c1(ops):
    c = cfg.config1(0)
    g, go = c["geom"], c["geom_out"]
    idx, cnt = ops.reduce_mask(c["mask"], *g.as_lists(), tol=c["tol"], avgpool=c["avgpool"])
    out = {}
    order = pipeline.sort_order(idx, int(cnt[0]), g.bcount)
    out["indices"] = np.asarray(idx[: int(cnt[0])])[order]
    for t in (False, True):
        st = ops.sparse_gather(c["x"], cnt, idx, g.bsize, g.bstride, g.boffset, transpose=t)
        out[f"stack_t{int(t)}"] = np.asarray(st)[order]
        # stand-in for a 3x3 VALID conv on the 10x10 windows: their 8x8 interior
        inner = st[:, :, 1:9, 1:9] if t else st[:, 1:9, 1:9, :]
        y = ops.sparse_scatter(np.ascontiguousarray(inner), cnt, idx, np.zeros_like(c["x"]),
                               go.bsize, go.bstride, go.boffset, add=False, transpose=t)
        out[f"y_t{int(t)}"] = y
    return out, ()


def _c2(ops):
    mask = cfg.rect_union_mask(2, 160, 176, seed=3, n_rects=10)
    g = cfg.halo_geom(160, 176)
    out = {}
    for name, avg, tol in (("avg", True, 0.1), ("max", False, 0.5)):
        idx, cnt = ops.reduce_mask(mask, *g.as_lists(), tol=tol, avgpool=avg)
        order = pipeline.sort_order(idx, int(cnt[0]), g.bcount)
        out[f"indices_{name}"] = np.asarray(idx[: int(cnt[0])])[order]
    return out, ()


def _c3(ops, dtype, density):
    N, H, W, C = 2, 64, 64, 32
    x = cfg.normal((N, H, W, C), 11, dtype)
    g = cfg.halo_geom(H, W)
    idx, cnt = cfg.random_block_list(N, g.bcount, density, seed=5)
    out = {}
    for t in (False, True):
        st = ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=t)
        out[f"stack_t{int(t)}"] = st
    return out, ()


def _c4a(ops, density):
    N, H, W, C = 2, 64, 64, 16
    g = cfg.halo_geom(H, W)
    idx, cnt = cfg.random_block_list(N, g.bcount, density, seed=6)
    nb = int(cnt[0])
    stack = cfg.normal((nb, 18, 18, C), 12)
    base = cfg.normal((N, H, W, C), 13)
    y = ops.sparse_scatter(stack, cnt, idx, base, g.bsize, g.bstride, g.boffset, add=True,
                           atomic=True, transpose=False)
    yv = base.copy()
    yv = ops.sparse_scatter_var(stack, cnt, idx, yv, g.bsize, g.bstride, g.boffset, add=True,
                                atomic=True, transpose=False)
    # the inputs of the accumulation, for the exact-sum check of the order-dependent arrays
    return dict(y=y, y_var=yv), ("y", "y_var"), dict(stack=stack, count=cnt, indices=idx, base=base, geom=g)


def _c4b(ops, density):
    N, H, W, C = 2, 64, 64, 16
    g = cfg.inner_geom(H, W)
    idx, cnt = cfg.random_block_list(N, g.bcount, density, seed=7)
    nb = int(cnt[0])
    stack = cfg.normal((nb, C, 16, 16), 14, np.float16)
    base = cfg.normal((N, H, W, C), 15, np.float16)
    y = ops.sparse_scatter(stack, cnt, idx, base, g.bsize, g.bstride, g.boffset, add=False,
                           transpose=True)
    return dict(y=y), ()


def _c5(ops):
    N, H, W, C = 2, 64, 48, 32
    x = cfg.normal((N, H, W, C), 21, np.float16)
    mask = cfg.rect_union_mask(N, H, W, seed=22, occupancy=0.3, side=(4, 16))
    g, go = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    idx, cnt = ops.reduce_mask(mask, *g.as_lists(), tol=0.5, avgpool=False)
    order = pipeline.sort_order(idx, int(cnt[0]), g.bcount)
    st = ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=True)
    q = np.ascontiguousarray(st[:, :, 1:17, 1:17])  # stand-in for the bottleneck convs
    y = ops.sparse_scatter_var(q, cnt, idx, x.copy(), go.bsize, go.bstride, go.boffset, add=True,
                               transpose=True)
    return dict(indices=np.asarray(idx[: int(cnt[0])])[order], stack=np.asarray(st)[order], y=y), ()


_CASES = {
    "c1": _c1,
    "c2_small": _c2,
    "c3_f32_d20": lambda ops: _c3(ops, np.float32, 0.2),
    "c3_f32_d50": lambda ops: _c3(ops, np.float32, 0.5),
    "c3_f16_d20": lambda ops: _c3(ops, np.float16, 0.2),
    "c3_f16_d50": lambda ops: _c3(ops, np.float16, 0.5),
    "c4a_d20": lambda ops: _c4a(ops, 0.2),
    "c4a_d50": lambda ops: _c4a(ops, 0.5),
    "c4b_d20": lambda ops: _c4b(ops, 0.2),
    "c4b_d50": lambda ops: _c4b(ops, 0.5),
    "c5_small": _c5,
}
NAMES = list(_CASES)


def run(ops, name):
    res = _CASES[name](ops)
    arrays, tol = res[0], res[1]
    return dict(arrays=arrays, tol=tuple(tol), atomic=res[2] if len(res) > 2 else None,
                digests={k: pipeline.digest(v) for k, v in arrays.items()})
