"""CPU checks of the benchmark's own bookkeeping: block counts, covered pixels and algorithmic bytes
must agree with the CPU checker and with hand-computed figures."""
import importlib.util
import os

import numpy as np

from sbnet_b200 import configs as cfg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_union_stats_and_per_image_counts_match_the_checker(oracle_port):
    bench = _bench()
    N, H, W = 3, 64, 48
    mask = cfg.rect_union_mask(N, H, W, seed=5, occupancy=0.2, side=(4, 12))
    g_in, g_out = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    nB, U_in, U_out, idx = bench.union_stats(mask, g_in, g_out, N, H, W)
    oi, oc = oracle_port.reduce_mask(mask, *g_in.as_lists(), tol=0.5)
    assert nB == int(oc[0])
    assert sorted(map(tuple, idx.tolist())) == sorted(map(tuple, oi[:nB].tolist()))
    assert U_out == nB * 256                       # disjoint 16x16 interiors, all inside the image
    assert U_in == cfg.union_pixels(oi, nB, g_in, N, H, W) <= nB * 324
    per = bench.per_image_blocks(mask, g_in, N, H, W)
    assert per.tolist() == [int((oi[:nB, 0] == n).sum()) for n in range(N)]


def test_algorithmic_bytes_of_the_benchmark_shapes():
    g, gi = cfg.halo_geom(512, 512), cfg.inner_geom(512, 512)
    # one interior 18x18x128 fp32 block: 165,888 B each way
    assert cfg.algorithmic_bytes("gather", nB=1, geom=g, C=128, itemsize=4, U=324) == 2 * 165888 + 6
    assert cfg.algorithmic_bytes("scatter_add", nB=1, geom=g, C=64, itemsize=4, U=324) == 3 * 82944 + 6
    assert cfg.algorithmic_bytes("scatter", nB=1, geom=gi, C=64, itemsize=2, U=256) == 2 * 32768 + 6
    assert cfg.algorithmic_bytes("scatter_add", nB=1, geom=gi, C=256, itemsize=2, U=256) == 393216 + 6
    assert cfg.algorithmic_bytes("reduce_mask", nB=0, geom=g, C=1, itemsize=4, U=0, N=8, H=800, W=704, count=0) == 18022400 + 4
    assert cfg.algorithmic_bytes("scatter_copy", nB=0, geom=g, C=64, itemsize=4, U=0, N=8, H=512, W=512) == 2 * 536870912


def test_random_block_list_is_seeded_and_unique():
    g = cfg.halo_geom(512, 512)
    a, ca = cfg.random_block_list(8, g.bcount, 0.2, seed=11)
    b, cb = cfg.random_block_list(8, g.bcount, 0.2, seed=11)
    assert np.array_equal(a, b) and ca[0] == cb[0]
    n = int(ca[0])
    assert len({tuple(r) for r in a[:n].tolist()}) == n
    assert abs(n / (8 * 32 * 32) - 0.2) < 0.02


def test_rect_union_mask_hits_its_occupancy():
    m = cfg.rect_union_mask(2, 400, 352, seed=7, occupancy=0.10)
    occ = m.reshape(2, -1).mean(axis=1)
    assert (occ >= 0.10).all() and (occ < 0.13).all()
    assert set(np.unique(m)) == {0.0, 1.0}
