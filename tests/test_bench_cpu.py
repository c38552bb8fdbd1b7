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


def test_roofline_traffic_comes_from_the_committed_profiles():
    """`roofline.traffic` = DRAM bytes per block read from the committed profiler summary of the
    dominant kernel x the blocks of the launch; the summary must hold the three figures, and they
    must stay close to the algorithmic bytes of the same launch (no wasted re-reads)."""
    import re
    bench = _bench()
    for op, key in (("gather", "gather"), ("scatter", "scatter_add")):
        per_block, name = bench.traffic_per_block(op)
        text = open(os.path.join(ROOT, "profiles", name)).read()
        assert per_block is not None and name in bench.TRAFFIC_PROFILES.values()
        blocks = int(re.search(r"blocks in this launch\s+(\d+)", text).group(1))
        read = float(re.search(r"DRAM read\s+([0-9.]+) Mbyte", text).group(1)) * 1e6
        write = float(re.search(r"DRAM write\s+([0-9.]+) Mbyte", text).group(1)) * 1e6
        assert abs(per_block * blocks - (read + write)) < 1.0
        alg = int(re.search(r"algorithmic bytes (\d+)", text).group(1))
        assert 0.7 < per_block * blocks / alg < 1.15, (op, per_block * blocks, alg)


def test_default_scaling_is_the_configured_split():
    """With N GPUs the benchmark shards ONE batch of 32 (the configured multi-GPU case)."""
    import subprocess
    import sys
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True, text=True).stdout
    assert "--scaling" in out
    bench = _bench()
    import argparse
    src = open(os.path.join(ROOT, "bench.py")).read()
    assert 'choices=["weak", "strong"], default="strong"' in src
    from sbnet_b200.dist import shard_bounds
    assert [shard_bounds(32, w, 0)[1] for w in (1, 2, 4, 8)] == [32, 16, 8, 4]
    del bench, argparse


def test_top_left_mask_and_tables_follow_the_reference_harness():
    """The synthetic mask of the dense-vs-sparse benchmark (``benchmark/sparse_conv_perf.py:47-63``: a
    top-left rectangle with edge ratio sqrt(1 - sparsity), edges rounded up) and its tables
    (``benchmark/benchmark_configs.py:23-44``, ``benchmark/benchmark_topleft.py:45-53``)."""
    import bench_topleft as tl
    m = tl.top_left_mask(1, 400, 700, 0.9)
    assert m.shape == (1, 400, 700, 1) and m.dtype == np.float32
    h, w = int(np.ceil(np.sqrt(0.1) * 400)), int(np.ceil(np.sqrt(0.1) * 700))
    assert m[0, :h, :w, 0].all() and m.sum() == h * w and (h, w) == (127, 222)
    assert abs(float(m.mean()) - 0.1) < 0.002
    assert tl.INPUT_SIZES["resnet-50"][0] == [400, 700, 256, 64] and tl.INPUT_SIZES["resnet-v2"][3] == [50, 88, 384, 96]
    assert tl.SPARSITIES[0] == 0.6 and tl.SPARSITIES[-1] == 0.99 and len(tl.SPARSITIES) == 9
    assert [list(r)[0] for r in tl.BLOCK_SIZES] == [11, 7, 5, 5] and [list(r)[-1] for r in tl.BLOCK_SIZES] == [31, 23, 19, 19]
    assert (tl.BATCH, tl.TOL, tl.AVGPOOL, tl.N_REPEAT, tl.N_WARMUP, tl.N_RUN) == (1, 0.05, True, 5, 3, 3)
