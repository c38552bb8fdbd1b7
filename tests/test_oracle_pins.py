"""Pins the CPU checker before anything is compared against it.

1. Known answers held by the reference's own tests (read from their source):
   * empty mask -> bin_counts == 1 and first index (0,0,0)
     (sbnet_ops/tests/test_sparse_blocks.py:303-306, rule in sbnet_ops/reduce_mask.cc:203-220);
   * the hand-written 5x5 expected output of reduce_mask -> gather -> 3x3 ones conv -> scatter_var
     (benchmark/sparse_conv_tests.py:437-460);
   * the hand-drawn 5x5 / 8x8 masks of benchmark/reduce_mask_tests.py:49-82, whose expected index
     sets the reference derives from max-pool + where (benchmark/sparse_conv_lib.py:279-318),
     restated here in numpy.
2. Golden vectors generated from the reference's CPU functors compiled unchanged
   (tests/golden/make_golden.py) -- checked against the C restatement.
3. When the compiled reference library is present, restatement == reference bit for bit, live.
"""
import json
import os

import numpy as np
import pytest

import config_cases
import pipeline
import ref_cases

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

MASK_5x5 = np.array([[[0, 0, 0, 0, 0],
                      [0, 0, 1, 0, 0],
                      [1, 0, 0, 0, 0],
                      [0, 0, 0, 0, 0],
                      [0, 0, 0, 0, 0]]], dtype=np.float32)
YEXP_5x5 = np.array([[0, 6, 6, 6, 0],
                     [6, 9, 9, 9, 0],
                     [6, 9, 9, 9, 0],
                     [6, 9, 0, 0, 0],
                     [0, 0, 0, 0, 0]], dtype=np.float32)
MASK_8x8 = np.zeros((1, 8, 8), dtype=np.float32)
MASK_8x8[0, 0:5, 5:8] = 1
MASK_8x8[0, 2, 0] = 1


def test_empty_mask_reports_one_block(oracle_port):
    idx, cnt = oracle_port.reduce_mask(np.zeros((1, 2, 2, 1), np.float32), [2, 2], [1, 1], [1, 1],
                                       [0, 0], tol=1e32)
    assert cnt.tolist() == [1] and idx[0].tolist() == [0, 0, 0]
    idx, cnt = oracle_port.reduce_mask(np.zeros((1, 2, 2, 1), np.float32), [2, 2], [1, 1], [1, 1],
                                       [0, 0], tol=1e32, op_fixup=False)
    assert cnt.tolist() == [0]


def test_sparse_conv_same_known_answer(oracle_port):
    # calc_block_params([1,5,5,1], bsize 3x3, ksize 3x3, stride 1, SAME):
    # bstride 1, boffset (-1,-1), bcount (5,5), bsize_out (1,1)   (sparse_conv_lib.py:343-397)
    o = oracle_port
    idx, cnt = o.reduce_mask(MASK_5x5[..., None], [5, 5], [3, 3], [1, 1], [-1, -1], tol=0.0)
    x = np.ones((1, 5, 5, 1), np.float32)
    for transpose in (False, True):
        p = o.sparse_gather(x, cnt, idx, [3, 3], [1, 1], [-1, -1], transpose=transpose)
        q = p.reshape(p.shape[0], -1).sum(1).reshape(-1, 1, 1, 1)  # 3x3 ones kernel, VALID
        y = o.sparse_scatter_var(q, cnt, idx, x.copy(), [1, 1], [1, 1], [0, 0], add=False,
                                 transpose=transpose)
        exp = np.where(YEXP_5x5 == 0, 1.0, YEXP_5x5).astype(np.float32)
        np.testing.assert_array_equal(y[0, :, :, 0], exp)


def _maxpool_where(mask, bsize, bstride, boffset, bcount, tol):
    """numpy restatement of convert_mask_to_indices: pad, max-pool, where(> tol)."""
    out = set()
    N, H, W = mask.shape
    for n in range(N):
        for bh in range(bcount[0]):
            for bw in range(bcount[1]):
                h0, w0 = boffset[0] + bh * bstride[0], boffset[1] + bw * bstride[1]
                win = mask[n, max(h0, 0):max(min(h0 + bsize[0], H), 0),
                           max(w0, 0):max(min(w0 + bsize[1], W), 0)]
                if win.size and win.max() > tol:
                    out.add((n, bh, bw))
    return out


@pytest.mark.parametrize("mask,bsize,bstride,boffset,bcount", [
    (MASK_5x5, (3, 3), (1, 1), (-1, -1), (5, 5)),       # reduce_mask_tests.py:49-63 (SAME)
    (MASK_8x8, (5, 5), (4, 4), (0, 0), (2, 2)),         # reduce_mask_tests.py:65-82 (VALID, k=2)
])
def test_reduce_mask_hand_drawn_masks(oracle_port, mask, bsize, bstride, boffset, bcount):
    idx, cnt = oracle_port.reduce_mask(mask[..., None], bcount, bsize, bstride, boffset, tol=0.0)
    got = {tuple(r) for r in idx[: int(cnt[0])].tolist()}
    assert got == _maxpool_where(mask, bsize, bstride, boffset, bcount, 0.0)


def test_gather_matches_numpy_slicing(oracle_port):
    # sparse_gather_tests.py:81-122 compares with tf.gather_nd on x = arange; numpy slicing here.
    x = np.arange(1 * 8 * 8 * 3, dtype=np.float32).reshape(1, 8, 8, 3)
    idx, cnt = oracle_port.reduce_mask(MASK_8x8[..., None], [2, 2], [5, 5], [4, 4], [0, 0], tol=0.0)
    st = oracle_port.sparse_gather(x, cnt, idx, [5, 5], [4, 4], [0, 0])
    for k in range(int(cnt[0])):
        n, bh, bw = idx[k]
        exp = np.zeros((5, 5, 3), np.float32)
        sl = x[n, bh * 4:bh * 4 + 5, bw * 4:bw * 4 + 5]
        exp[: sl.shape[0], : sl.shape[1]] = sl
        np.testing.assert_array_equal(st[k], exp)
    stt = oracle_port.sparse_gather(x, cnt, idx, [5, 5], [4, 4], [0, 0], transpose=True)
    np.testing.assert_array_equal(stt, st.transpose(0, 3, 1, 2))


def test_scatter_overlap_rule(oracle_port):
    x = np.zeros((1, 2, 2, 1), np.float32)
    with pytest.raises(ValueError):
        oracle_port.sparse_scatter_var(x, [1], np.zeros((1, 3), np.int16), np.zeros((1, 4, 4, 1), np.float32),
                                       [2, 2], [1, 1], [0, 0], add=True, atomic=False)


def _golden(name):
    path = os.path.join(GOLDEN, name)
    if not os.path.exists(path):
        pytest.skip(f"{name} not generated")
    with open(path) as f:
        return json.load(f)


SMALL = [c for c in ref_cases.CASES if not c.big]


@pytest.mark.parametrize("case", SMALL, ids=[c.name for c in SMALL])
def test_port_matches_reference_golden(oracle_port, case):
    gold = _golden("ref_cases.json")[case.name]
    inputs = ref_cases.make_inputs(case)
    for transpose in (False, True):
        r = pipeline.run_case(oracle_port, case, transpose, inputs)
        g = gold["T" if transpose else "N"]
        assert r["count"] == g["count"]
        if g["indices"] is not None:
            assert r["indices"].tolist() == g["indices"]
        assert pipeline.digest(r["indices"]) == g["indices_sha"]
        assert pipeline.digest(r["stack"]) == g["stack_sha"]
        assert pipeline.digest(r["y"]) == g["y_sha"]
        if case.sparsity == 100:  # test_sparse_blocks.py:303-306
            assert r["count"] == 1 and r["indices"][0].tolist() == [0, 0, 0]


@pytest.mark.parametrize("name", config_cases.NAMES)
def test_port_matches_reference_golden_configs(oracle_port, name):
    gold = _golden("config_cases.json")[name]
    assert config_cases.run(oracle_port, name)["digests"] == gold


LIVE = [c for c in SMALL if not c.name.startswith("perm_")] + \
       [c for c in SMALL if c.name.startswith("perm_")][::7]


@pytest.mark.parametrize("case", LIVE, ids=[c.name for c in LIVE])
def test_port_matches_compiled_reference_live(oracle_port, oracle_ref, case):
    oracle_ref.set_threads(1)
    inputs = ref_cases.make_inputs(case)
    for transpose in (False, True):
        a = pipeline.run_case(oracle_port, case, transpose, inputs)
        b = pipeline.run_case(oracle_ref, case, transpose, inputs)
        assert a["count"] == b["count"]
        for k in ("indices", "stack", "y"):
            np.testing.assert_array_equal(a[k], b[k])


def test_threaded_port_is_deterministic_where_disjoint(oracle_port):
    name = "c4b_d50"
    oracle_port.set_threads(1)
    a = config_cases.run(oracle_port, name)["digests"]
    oracle_port.set_threads(4)
    try:
        b = config_cases.run(oracle_port, name)["digests"]
    finally:
        oracle_port.set_threads(1)
    assert a == b


def test_reference_cuda_kernel_library_exports_its_entry_points():
    """The second checker (the reference's CUDA kernels for sm_100a) loads without a GPU and exports
    the three launchers; no launch is made here."""
    from oracle import refgpu
    if not refgpu.available():
        try:
            refgpu.build()
        except Exception:
            pass
    if not refgpu.available():
        pytest.skip("reference CUDA kernels not built (no reference tree and no prebuilt library)")
    lib = refgpu._load()
    for name in ("refgpu_sparse_gather", "refgpu_sparse_scatter", "refgpu_reduce_mask"):
        assert getattr(lib, name) is not None


def test_bf16_restatement_matches_compiled_reference(oracle_port, oracle_ref):
    """bfloat16 instantiations of both checkers agree bit for bit, and one add equals a float
    addition rounded to nearest even (checked against torch's CPU bfloat16 add)."""
    ml_dtypes = pytest.importorskip("ml_dtypes")
    import torch
    from sbnet_b200 import configs as cfg
    bf = ml_dtypes.bfloat16
    oracle_ref.set_threads(1)
    N, H, W, C = 2, 40, 40, 24
    g = cfg.geom_for(H, W, (6, 6), (4, 4), (-1, -1))
    idx, cnt = cfg.random_block_list(N, g.bcount, 0.6, seed=1)
    x = cfg.normal((N, H, W, C), 1, bf)
    for tr in (False, True):
        a = oracle_port.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=tr)
        b = oracle_ref.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=tr)
        np.testing.assert_array_equal(a.view(np.uint16), b.view(np.uint16))
        stack, base = cfg.normal(a.shape, 2, bf), cfg.normal((N, H, W, C), 3, bf)
        ya = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), g.bsize, g.bstride, g.boffset,
                                            add=True, atomic=True, transpose=tr)
        yb = oracle_ref.sparse_scatter_var(stack, cnt, idx, base.copy(), g.bsize, g.bstride, g.boffset,
                                           add=True, atomic=True, transpose=tr)
        np.testing.assert_array_equal(ya.view(np.uint16), yb.view(np.uint16))
    a = cfg.normal((50000,), 5, bf)
    b = (cfg.normal((50000,), 6, np.float32) * 1e-2).astype(bf)
    ta = torch.from_numpy(a.view(np.int16)).view(torch.bfloat16)
    tb = torch.from_numpy(b.view(np.int16)).view(torch.bfloat16)
    y = oracle_port.sparse_scatter_var(b.reshape(1, 1, 1, -1), np.array([1], np.int32), np.zeros((1, 3), np.int16),
                                       a.reshape(1, 1, 1, -1).copy(), (1, 1), (1, 1), (0, 0), add=True)
    np.testing.assert_array_equal(y.view(np.int16).reshape(-1), (ta + tb).view(torch.int16).numpy())
