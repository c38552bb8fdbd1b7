"""bfloat16 through the C ABI (SBNET_BF16, an extension like fp16: the reference registers float only)
against the CPU checker instantiated for bfloat16.  Gather and overwrite move bit patterns; add and
atomic add accumulate in bfloat16 with one round-to-nearest-even per add (``red.add.noftz.bf16x2``),
which is what the checker's ``y += v`` does, so non-overlapping adds are bit-exact."""
import numpy as np
import pytest

from sbnet_b200 import configs as cfg

pytestmark = pytest.mark.gpu
ml_dtypes = pytest.importorskip("ml_dtypes")
BF16 = ml_dtypes.bfloat16

# (N, H, W, C, bsize, bstride, boffset)
SHAPES = [
    (2, 64, 48, 64, (18, 18), (16, 16), (-1, -1)),     # tile CTAs, rows of 162 words
    (2, 64, 48, 256, (16, 16), (16, 16), (0, 0)),      # tile CTAs, rows of 128 words
    (1, 50, 45, 40, (6, 5), (4, 3), (-2, -3)),         # partial channel chunk, overlapping
    (1, 50, 50, 64, (5, 5), (5, 5), (0, 0)),           # odd pixel count: rows of an odd number of halves
    (1, 100, 90, 64, (34, 34), (32, 32), (-1, -1)),    # pixel chunks
    (2, 23, 31, 7, (5, 4), (3, 4), (-2, -1)),          # 14-byte pixels: general kernels, 2-byte vectors
    (2, 23, 31, 6, (5, 4), (5, 4), (0, 0)),            # 12-byte pixels: 4-byte vectors
    (1, 30, 30, 12, (8, 8), (8, 8), (0, 0)),           # 24-byte pixels: 8-byte vectors
]


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


@pytest.mark.parametrize("transpose", [False, True], ids=["rows", "planes"])
@pytest.mark.parametrize("shape", SHAPES, ids=[f"C{s[3]}_b{s[4][0]}x{s[4][1]}" for s in SHAPES])
def test_bf16_gather_and_scatter(cuda_ops, oracle_port, shape, transpose):
    N, H, W, C, bsize, bstride, boffset = shape
    g = cfg.geom_for(H, W, bsize, bstride, boffset)
    idx, cnt = cfg.random_block_list(N, g.bcount, 0.6, seed=C + bsize[0])
    nb = int(cnt[0])
    x = cfg.normal((N, H, W, C), 3, BF16)
    exp = oracle_port.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=transpose)
    got = cuda_ops.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=transpose)
    np.testing.assert_array_equal(_bits(got), _bits(exp))

    shp = (nb, C, *bsize) if transpose else (nb, *bsize, C)
    stack = cfg.normal(shp, 4, BF16)
    base = cfg.normal((N, H, W, C), 5, BF16)
    disjoint = bstride[0] >= bsize[0] and bstride[1] >= bsize[1]
    src = stack if disjoint else exp   # overlapping overwrite: every copy of a pixel must agree
    e = oracle_port.sparse_scatter_var(src, cnt, idx, base.copy(), bsize, bstride, boffset, add=False,
                                       transpose=transpose)
    o = cuda_ops.sparse_scatter_var(src, cnt, idx, base.copy(), bsize, bstride, boffset, add=False,
                                    transpose=transpose)
    np.testing.assert_array_equal(_bits(o), _bits(e))
    if disjoint:
        e = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                           transpose=transpose)
        o = cuda_ops.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                        transpose=transpose)
        np.testing.assert_array_equal(_bits(o), _bits(e))
    e = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True, atomic=True,
                                       transpose=transpose)
    o = cuda_ops.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True, atomic=True,
                                    transpose=transpose)
    # bfloat16 keeps 8 significant bits: one add rounds by at most 2^-8 of the partial sum; both results
    # within k such roundings of the fp64 sum
    from atomic_check import check_atomic_add
    check_atomic_add({"cuda": o, "cpu checker": e}, stack, cnt, idx, base, bsize, bstride, boffset, transpose)


def test_bf16_subnormal_addends_are_not_flushed(cuda_ops, oracle_port):
    """Accumulation must keep subnormal bfloat16 values (``noftz``), as the CPU does."""
    N, H, W, C = 1, 16, 16, 64
    bsize = bstride = (8, 8)
    g = cfg.geom_for(H, W, bsize, bstride, (0, 0))
    idx, cnt = cfg.random_block_list(N, g.bcount, 1.0, seed=0)
    nb = int(cnt[0])
    rng = np.random.default_rng(0)
    tiny = (rng.integers(1, 0x7F, size=(nb, 8, 8, C)).astype(np.uint16)).view(BF16)   # subnormal patterns
    base = (rng.integers(0, 0x7F, size=(N, H, W, C)).astype(np.uint16)).view(BF16)
    for transpose in (False, True):
        stack = np.ascontiguousarray(tiny.transpose(0, 3, 1, 2)) if transpose else tiny
        e = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, (0, 0), add=True,
                                           transpose=transpose)
        o = cuda_ops.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, (0, 0), add=True,
                                        transpose=transpose)
        np.testing.assert_array_equal(_bits(o), _bits(e))
        assert (_bits(e) != _bits(base)).any()
