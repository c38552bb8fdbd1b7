"""Seeded random geometries through all ops on the GPU against the CPU checker (through the C ABI).

Each case draws image size, channel count, block size / stride / offset (overlaps, gaps, blocks
hanging over every border), dtype, layout and a block list from a seed, then checks reduce_mask
(both pooling modes), gather (bit-exact), overwrite scatter of gathered values (bit-exact), atomic
add (tolerance per addend) and, where blocks are disjoint, non-atomic add (bit-exact)."""
import numpy as np
import pytest

from sbnet_b200 import configs as cfg
from atomic_check import check_atomic_add

pytestmark = pytest.mark.gpu

CHANNELS = [1, 2, 3, 4, 5, 8, 12, 16, 20, 32, 33, 48, 64, 96, 128, 130]


def _draw(seed):
    rng = np.random.default_rng(1000 + seed)
    N = int(rng.integers(1, 4))
    H, W = int(rng.integers(1, 40)), int(rng.integers(1, 40))
    C = int(rng.choice(CHANNELS))
    bsize = (int(rng.integers(1, min(H, 20) + 1)), int(rng.integers(1, min(W, 20) + 1)))
    bstride = (int(rng.integers(1, bsize[0] + 3)), int(rng.integers(1, bsize[1] + 3)))
    boffset = (int(rng.integers(-bsize[0] + 1, 1)), int(rng.integers(-bsize[1] + 1, 1)))
    dtype = np.float16 if rng.random() < 0.5 else np.float32
    return N, H, W, C, bsize, bstride, boffset, dtype, rng


@pytest.mark.parametrize("seed", range(120))
def test_random_geometry(cuda_ops, oracle_port, seed):
    N, H, W, C, bsize, bstride, boffset, dtype, rng = _draw(seed)
    g = cfg.geom_for(H, W, bsize, bstride, boffset)
    # reduce_mask on a real-valued mask, both modes
    mask = rng.standard_normal((N, H, W, 1)).astype(np.float32)
    for avg, tol in ((False, 0.8), (True, 0.05)):
        gi, gc = cuda_ops.reduce_mask(mask, *g.as_lists(), tol=tol, avgpool=avg)
        oi, oc = oracle_port.reduce_mask(mask, *g.as_lists(), tol=tol, avgpool=avg)
        n = int(oc[0])
        assert int(gc[0]) == n
        assert sorted(map(tuple, gi[:n].tolist())) == sorted(map(tuple, oi[:n].tolist()))
    idx, cnt = cfg.random_block_list(N, g.bcount, 0.6, seed=seed)
    nb = int(cnt[0])
    x = cfg.normal((N, H, W, C), seed, dtype)
    base = cfg.normal((N, H, W, C), seed + 1, dtype)
    disjoint = bstride[0] >= bsize[0] and bstride[1] >= bsize[1]
    cover = -(-bsize[0] // bstride[0]) * -(-bsize[1] // bstride[1])
    for transpose in (False, True):
        exp = oracle_port.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=transpose)
        got = cuda_ops.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=transpose)
        np.testing.assert_array_equal(got, exp)
        e = oracle_port.sparse_scatter(exp, cnt, idx, base, bsize, bstride, boffset, add=False, transpose=transpose)
        o = cuda_ops.sparse_scatter(exp, cnt, idx, base, bsize, bstride, boffset, add=False, transpose=transpose)
        np.testing.assert_array_equal(o, e)
        shape = (nb, C, *bsize) if transpose else (nb, *bsize, C)
        stack = cfg.normal(shape, seed + 2, dtype)
        e = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                           atomic=True, transpose=transpose)
        o = cuda_ops.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                        atomic=True, transpose=transpose)
        check_atomic_add({"cuda": o, "cpu checker": e}, stack, cnt, idx, base, bsize, bstride, boffset, transpose)
        if disjoint:
            e = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                               transpose=transpose)
            o = cuda_ops.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                            transpose=transpose)
            np.testing.assert_array_equal(o, e)


def _draw_tile(seed):
    """Shapes the tile CTAs of the transposed layout take: pixels of a multiple of 16 bytes, blocks
    from one pixel to beyond one tile (pixel chunks), a forced number of blocks per tile."""
    rng = np.random.default_rng(5000 + seed)
    N = int(rng.integers(1, 3))
    H, W = int(rng.integers(8, 90)), int(rng.integers(8, 90))
    kind = int(rng.integers(0, 3))            # 0 fp32, 1 fp16, 2 bfloat16
    C = int(rng.choice([4, 8, 12, 32, 36, 64]) if kind == 0 else rng.choice([8, 16, 24, 64, 72, 128, 200]))
    lo, hi = [(1, 13), (12, 19), (20, 40)][int(rng.integers(0, 3))]   # several per tile / one tile / pixel chunks
    H, W = max(H, lo), max(W, lo)
    bsize = (int(rng.integers(lo, min(H, hi) + 1)), int(rng.integers(lo, min(W, hi) + 1)))
    bstride = (int(rng.integers(max(1, bsize[0] - 2), bsize[0] + 3)), int(rng.integers(max(1, bsize[1] - 2), bsize[1] + 3)))
    boffset = (int(rng.integers(-bsize[0] + 1, 1)), int(rng.integers(-bsize[1] + 1, 1)))
    pack = str(rng.choice([1, 2, 5, 1000]))
    return N, H, W, C, bsize, bstride, boffset, kind, pack


@pytest.mark.parametrize("seed", range(60))
def test_random_tile_shapes(cuda_ops, oracle_port, seed):
    N, H, W, C, bsize, bstride, boffset, kind, pack = _draw_tile(seed)
    if kind == 2:
        ml_dtypes = pytest.importorskip("ml_dtypes")
        dtype, rtol1 = ml_dtypes.bfloat16, 2.0 ** -7
    else:
        dtype, rtol1 = (np.float32, 1e-6) if kind == 0 else (np.float16, 1e-3)
    bits = np.uint32 if kind == 0 else np.uint16
    g = cfg.geom_for(H, W, bsize, bstride, boffset)
    idx, cnt = cfg.random_block_list(N, g.bcount, 0.7, seed=seed)
    nb = int(cnt[0])
    x = cfg.normal((N, H, W, C), seed, dtype)
    base = cfg.normal((N, H, W, C), seed + 1, dtype)
    stack = cfg.normal((nb, C, *bsize), seed + 2, dtype)
    disjoint = bstride[0] >= bsize[0] and bstride[1] >= bsize[1]
    cover = -(-bsize[0] // bstride[0]) * -(-bsize[1] // bstride[1])
    from conftest import library_options
    with library_options(tile_blocks=int(pack), planes=3 if seed % 2 else 0):   # odd seeds: tile CTAs whatever the launch size
        exp = oracle_port.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=True)
        got = cuda_ops.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=True)
        np.testing.assert_array_equal(got.view(bits), exp.view(bits))
        e = oracle_port.sparse_scatter_var(exp, cnt, idx, base.copy(), bsize, bstride, boffset, add=False, transpose=True)
        o = cuda_ops.sparse_scatter_var(exp, cnt, idx, base.copy(), bsize, bstride, boffset, add=False, transpose=True)
        np.testing.assert_array_equal(o.view(bits), e.view(bits))
        if disjoint:
            e = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                               transpose=True)
            o = cuda_ops.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                            transpose=True)
            np.testing.assert_array_equal(o.view(bits), e.view(bits))
        e = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True, atomic=True,
                                           transpose=True)
        o = cuda_ops.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True, atomic=True,
                                        transpose=True)
        check_atomic_add({"cuda": o, "cpu checker": e}, stack, cnt, idx, base, bsize, bstride, boffset, True)
