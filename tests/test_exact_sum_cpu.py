"""The fp64 exact-sum checker on the CPU checker itself: an accumulating scatter over overlapping
blocks evaluated in two block orders differs only by roundings (both inside the k-roundings bound),
fp32 keeps 1e-6 relative where nothing cancels, and fp16 with several addends does NOT keep 1e-3 --
which is why the GPU tests hold 16-bit sums to the k-roundings bound instead."""
import numpy as np
import pytest

from oracle import exact
from sbnet_b200 import configs as cfg


def _two_orders(oracle_port, dtype, seed):
    N, H, W, C = 2, 64, 48, 16
    g = cfg.geom_for(H, W, (18, 18), (16, 16), (-1, -1))      # halos shared by up to four blocks
    idx, cnt = cfg.random_block_list(N, g.bcount, 0.8, seed=seed)
    nb = int(cnt[0])
    stack = cfg.normal((nb, 18, 18, C), seed + 1, dtype)
    base = cfg.normal((N, H, W, C), seed + 2, dtype)
    oracle_port.set_threads(1)      # a fixed block order per call
    fwd = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), g.bsize, g.bstride, g.boffset, add=True,
                                         atomic=True)
    rev_idx = np.ascontiguousarray(idx[:nb][::-1])
    rev = oracle_port.sparse_scatter_var(np.ascontiguousarray(stack[::-1]), cnt, rev_idx, base.copy(), g.bsize,
                                         g.bstride, g.boffset, add=True, atomic=True)
    oracle_port.set_threads(oracle_port.max_threads())
    ex, mag, k = exact.exact_add(stack, nb, idx, base, g.bsize, g.bstride, g.boffset)
    return fwd, rev, ex, mag, k, base


@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["f32", "f16"])
def test_block_order_changes_roundings_only(oracle_port, dtype):
    fwd, rev, ex, mag, k, base = _two_orders(oracle_port, dtype, 3)
    assert int(k.max()) == 4
    assert not np.array_equal(fwd, rev)                        # the order does show
    for name, res in (("forward", fwd), ("reversed", rev)):
        worst, rel = exact.check_add(res, ex, mag, k, base, cover=4, what=name)
        assert 0.3 < worst <= 1.0                              # the bound is tight, not loose


def test_half_precision_cannot_hold_1e_3_over_several_addends(oracle_port):
    fwd, rev, ex, mag, k, base = _two_orders(oracle_port, np.float16, 4)
    steady = (np.abs(ex) >= (mag - np.abs(base.astype(np.float64))) / 4) & (k[..., None] >= 2)
    rel = np.abs(fwd.astype(np.float64) - rev.astype(np.float64)) / np.maximum(np.abs(ex), 1e-300)
    assert float(rel[steady].max()) > 1e-3                    # the CPU checker against itself
    single = (np.abs(ex) >= (mag - np.abs(base.astype(np.float64))) / 4) & (k[..., None] == 1)
    assert float(rel[single].max()) == 0.0                    # one addend: no order to differ in


def test_checker_flags_a_wrong_sum(oracle_port):
    fwd, rev, ex, mag, k, base = _two_orders(oracle_port, np.float32, 5)
    bad = fwd.copy()
    n, h, w = np.argwhere(k == 4)[0]
    bad[n, h, w, 0] += np.float32(1e-3)
    with pytest.raises(AssertionError, match="outside the bound"):
        exact.check_add(bad, ex, mag, k, base, cover=4)
    bad = fwd.copy()
    n, h, w = np.argwhere(k == 0)[0]
    bad[n, h, w, 0] += np.float32(1.0)
    with pytest.raises(AssertionError, match="no block covers"):
        exact.check_add(bad, ex, mag, k, base, cover=4)
