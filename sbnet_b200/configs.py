"""Seeded synthetic workloads for the block ops (numpy only; no device code here).

The reference ships no data: its own benchmark draws a synthetic top-left-square mask
(``benchmark/sparse_conv_perf.py:47-63``) and its op test draws ``randn`` masks
(``sbnet_ops/tests/test_sparse_blocks.py:124-134``).  The generators below produce the shapes, block
geometries and value distributions of the benchmark configurations (LiDAR bird's-eye-view style
rectangle-union masks, uniformly random active-block lists, N(0,1) activations) from a seed, so the
CPU checker and the CUDA library always see identical inputs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence, Tuple

import numpy as np


@dataclass(frozen=True)
class BlockGeom:
    """Block geometry in the order the ops take it: every field is ``(H, W)``."""

    bsize: Tuple[int, int]
    bstride: Tuple[int, int]
    boffset: Tuple[int, int]
    bcount: Tuple[int, int]

    def as_lists(self):
        return list(self.bcount), list(self.bsize), list(self.bstride), list(self.boffset)


def calc_block_count_1d(size: int, bstride: int, boffset: int) -> int:
    """Blocks needed so the last block still owns at least one in-range pixel
    (``sbnet_ops/tests/test_sparse_blocks.py:100-111``)."""
    return 1 + (size - boffset - 1) // bstride


def geom_for(H: int, W: int, bsize: Sequence[int], bstride: Sequence[int],
             boffset: Sequence[int]) -> BlockGeom:
    return BlockGeom(tuple(bsize), tuple(bstride), tuple(boffset),
                     (calc_block_count_1d(H, bstride[0], boffset[0]),
                      calc_block_count_1d(W, bstride[1], boffset[1])))


# Geometry of the large configurations: 18x18 windows on a 16-pixel pitch with a one-pixel halo.
def halo_geom(H: int, W: int) -> BlockGeom:
    assert H % 16 == 0 and W % 16 == 0
    return BlockGeom((18, 18), (16, 16), (-1, -1), (H // 16, W // 16))


def inner_geom(H: int, W: int) -> BlockGeom:
    """Geometry of the block stack after a 3x3 VALID conv on 18x18 windows: 16x16, no halo."""
    assert H % 16 == 0 and W % 16 == 0
    return BlockGeom((16, 16), (16, 16), (0, 0), (H // 16, W // 16))


def cell_mask(N: int, H: int, W: int, cell: int, p: float, seed: int) -> np.ndarray:
    """Bernoulli(p) on a ``cell x cell`` pixel grid, nearest-upsampled to ``[N,H,W,1]`` fp32."""
    rng = np.random.default_rng(seed)
    grid = (rng.random((N, H // cell, W // cell)) < p).astype(np.float32)
    return np.repeat(np.repeat(grid, cell, axis=1), cell, axis=2)[..., None].copy()


def rect_union_mask(N: int, H: int, W: int, seed: int, n_rects: int | None = 96,
                    occupancy: float | None = None, side=(8, 64)) -> np.ndarray:
    """``[N,H,W,1]`` fp32 mask: per image (seed + n) a union of axis-aligned rectangles with sides
    uniform in ``side`` placed fully inside the image.  Either a fixed number of rectangles, or --
    when ``occupancy`` is given -- rectangles are added until that fraction of pixels is set."""
    out = np.zeros((N, H, W, 1), dtype=np.float32)
    for n in range(N):
        rng = np.random.default_rng(seed + n)
        img = out[n, :, :, 0]
        k = 0
        while True:
            if occupancy is None:
                if k >= n_rects:
                    break
            elif img.mean() >= occupancy:
                break
            hh = int(rng.integers(side[0], min(side[1], H) + 1))
            ww = int(rng.integers(side[0], min(side[1], W) + 1))
            h0 = int(rng.integers(0, H - hh + 1))
            w0 = int(rng.integers(0, W - ww + 1))
            img[h0:h0 + hh, w0:w0 + ww] = 1.0
            k += 1
    return out


def random_block_list(N: int, bcount: Sequence[int], density: float, seed: int):
    """Each of the ``N*bCntH*bCntW`` candidate blocks is kept with probability ``density``; the kept
    blocks are listed in random order (reduce_mask's compaction order is arbitrary too).
    Returns ``(active_block_indices [N*bCntH*bCntW,3] int16, bin_counts [1] int32)``."""
    rng = np.random.default_rng(seed)
    total = N * bcount[0] * bcount[1]
    keep = np.flatnonzero(rng.random(total) < density)
    if keep.size == 0:
        keep = np.array([0])
    keep = rng.permutation(keep)
    idx = np.zeros((total, 3), dtype=np.int16)
    n, rem = np.divmod(keep, bcount[0] * bcount[1])
    bh, bw = np.divmod(rem, bcount[1])
    idx[: keep.size] = np.stack([n, bh, bw], axis=1)
    return idx, np.array([keep.size], dtype=np.int32)


def normal(shape, seed: int, dtype=np.float32) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal(shape, dtype=np.float32).astype(dtype)


def union_pixels(idx: np.ndarray, count: int, geom: BlockGeom, N: int, H: int, W: int) -> int:
    """Number of distinct in-range pixels covered by the listed blocks (the ``U`` of the
    algorithmic-byte formulas)."""
    cover = np.zeros((N, H, W), dtype=bool)
    for n, bh, bw in np.asarray(idx[:count]).astype(np.int64):
        h0 = geom.boffset[0] + bh * geom.bstride[0]
        w0 = geom.boffset[1] + bw * geom.bstride[1]
        cover[n, max(h0, 0):max(min(h0 + geom.bsize[0], H), 0),
              max(w0, 0):max(min(w0 + geom.bsize[1], W), 0)] = True
    return int(cover.sum())


def algorithmic_bytes(op: str, *, nB: int, geom: BlockGeom, C: int, itemsize: int, U: int,
                      N: int = 0, H: int = 0, W: int = 0, count: int = 0) -> int:
    """Minimum DRAM traffic of one call (the numerator of every roofline figure).

    reduce_mask: mask read once + 6 B per emitted index + the 4-byte count.
    gather: every distinct in-range source pixel read once, every stack element written once.
    scatter overwrite: stack read once, every distinct destination pixel written once.
    scatter add / atomic: stack read once, destination read and written.
    scatter_copy: the non-Var op's extra full copy of the base tensor."""
    blk = nB * geom.bsize[0] * geom.bsize[1] * C * itemsize
    if op == "reduce_mask":
        return N * H * W * 4 + 6 * count + 4
    if op == "gather":
        return U * C * itemsize + blk + 6 * nB
    if op == "scatter":
        return blk + U * C * itemsize + 6 * nB
    if op == "scatter_add":
        return blk + 2 * U * C * itemsize + 6 * nB
    if op == "scatter_copy":
        return 2 * N * H * W * C * itemsize
    raise ValueError(op)


# ---- the named configurations -------------------------------------------------------------------

def config1(seed: int = 0):
    """CPU-plumbing case: x fp32 [2,64,64,32], 8x8-cell Bernoulli(0.15) mask, 10x10 windows on an
    8-pixel pitch with a one-pixel halo; scatter geometry is the 8x8 interior."""
    x = normal((2, 64, 64, 32), seed)
    mask = cell_mask(2, 64, 64, 8, 0.15, seed + 1)
    g_in = BlockGeom((10, 10), (8, 8), (-1, -1), (8, 8))
    g_out = BlockGeom((8, 8), (8, 8), (0, 0), (8, 8))
    return dict(x=x, mask=mask, geom=g_in, geom_out=g_out, tol=0.5, avgpool=False)


def config2(seed: int = 0, N: int = 8, H: int = 800, W: int = 704):
    """reduce_mask at bird's-eye-view scale: 96 rectangles per image."""
    mask = rect_union_mask(N, H, W, seed, n_rects=96)
    return dict(mask=mask, geom=halo_geom(H, W), runs=[dict(avgpool=True, tol=0.1),
                                                       dict(avgpool=False, tol=0.5)])
