"""reduce_mask corner cases on the GPU against the CPU checker (through the C ABI)."""
import numpy as np
import pytest

from sbnet_b200 import configs as cfg

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["tile", "tile_many_ctas", "tile_few_ctas", "tile_no_pdl", "tile_two_resident", "band", "per_block"])
def rm_kernel(request):
    """Every case runs through each reduce_mask kernel: the TMA-fed tile kernel (default column
    tiling, the narrowest and the widest tiles, without programmatic serialization, and with a cap on
    the CTAs resident per SM), the
    register-fed band kernel, and the one-thread-per-block kernel."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from conftest import library_options
    opts = {"tile": {}, "tile_many_ctas": {"rm_ctas_per_sm": 10000}, "tile_few_ctas": {"rm_ctas_per_sm": 1},
            "tile_no_pdl": {"pdl": 0}, "tile_two_resident": {"rm_resident": 2}, "band": {"rm_kernel": 1}, "per_block": {"rm_kernel": 2}}[request.param]
    with library_options(**{"rm_kernel": 0, "rm_ctas_per_sm": 8, "pdl": 1, "rm_resident": 0, **opts}):
        yield request.param


def _sets_equal(cuda_ops, oracle_port, mask, g, tol, avg):
    gi, gc = cuda_ops.reduce_mask(mask, *g.as_lists(), tol=tol, avgpool=avg)
    oi, oc = oracle_port.reduce_mask(mask, *g.as_lists(), tol=tol, avgpool=avg)
    assert int(gc[0]) == int(oc[0])
    n = int(oc[0])
    got = sorted(map(tuple, gi[:n].tolist()))
    assert got == sorted(map(tuple, oi[:n].tolist()))
    return n


@pytest.mark.parametrize("seed", range(6))
def test_average_threshold_on_a_block_value(cuda_ops, oracle_port, seed):
    """Real-valued masks with the threshold set EXACTLY to one block's average as the reference
    computes it (row-major fp32 sum / area): the verdict of that block depends on the last bit of
    the sum, so the GPU must reproduce the reference's summation order there."""
    rng = np.random.default_rng(seed)
    N, H, W = 2, 96, 80 + 4 * (seed % 2) + (seed % 3)       # W not always a multiple of 4
    mask = rng.standard_normal((N, H, W, 1)).astype(np.float32)
    g = cfg.geom_for(H, W, (18, 18), (16, 16), (-1, -1))
    for _ in range(8):
        n, bh, bw = rng.integers(0, N), rng.integers(0, g.bcount[0]), rng.integers(0, g.bcount[1])
        h0, w0 = -1 + 16 * bh, -1 + 16 * bw
        s = np.float32(0)
        for hh in range(max(h0, 0), min(h0 + 18, H)):
            for ww in range(max(w0, 0), min(w0 + 18, W)):
                s = np.float32(s + mask[n, hh, ww, 0])
        tol = float(np.float32(s / np.float32(324)))
        _sets_equal(cuda_ops, oracle_port, mask, g, tol, True)
        _sets_equal(cuda_ops, oracle_port, mask, g, float(np.nextafter(np.float32(tol), np.float32(-1e9))), True)


def test_zero_threshold_on_binary_mask(cuda_ops, oracle_port):
    mask = cfg.rect_union_mask(2, 160, 176, seed=1, n_rects=6)
    g = cfg.halo_geom(160, 176)
    for avg in (True, False):
        n = _sets_equal(cuda_ops, oracle_port, mask, g, 0.0, avg)
        assert 0 < n < 2 * 10 * 11


def test_negative_threshold_activates_out_of_range_blocks(cuda_ops, oracle_port):
    # block rows/cols entirely outside the image: avg of nothing is 0 > tol when tol < 0
    mask = np.zeros((1, 8, 8, 1), np.float32)
    g = cfg.BlockGeom((2, 2), (4, 4), (-6, -6), (5, 5))
    for avg in (True, False):
        _sets_equal(cuda_ops, oracle_port, mask, g, -0.5, avg)


def test_nan_and_inf_pixels(cuda_ops, oracle_port):
    rng = np.random.default_rng(0)
    mask = rng.standard_normal((1, 64, 64, 1)).astype(np.float32)
    mask[0, 5, 5, 0] = np.nan
    mask[0, 40, 40, 0] = np.inf
    mask[0, 41, 41, 0] = -np.inf
    mask[0, 20, 50, 0] = np.inf
    g = cfg.halo_geom(64, 64)
    for avg in (True, False):
        _sets_equal(cuda_ops, oracle_port, mask, g, 0.1, avg)


def test_scratch_is_reusable_across_calls_and_empty_results(cuda_ops, oracle_port):
    g = cfg.halo_geom(64, 64)
    full = np.ones((3, 64, 64, 1), np.float32)
    empty = np.zeros((3, 64, 64, 1), np.float32)
    for mask in (full, empty, full, empty, empty, full):
        for avg in (False, True):
            gi, gc = cuda_ops.reduce_mask(mask, *g.as_lists(), tol=0.5, avgpool=avg)
            oi, oc = oracle_port.reduce_mask(mask, *g.as_lists(), tol=0.5, avgpool=avg)
            assert int(gc[0]) == int(oc[0])
            if mask is empty:
                assert int(gc[0]) == 1 and gi[0].tolist() == [0, 0, 0]


def test_many_narrow_blocks_span_several_tiles(cuda_ops, oracle_port):
    rng = np.random.default_rng(3)
    mask = (rng.random((1, 6, 9000, 1)) < 0.02).astype(np.float32)
    g = cfg.geom_for(6, 9000, (3, 3), (2, 1), (-1, -1))        # 9001 block columns, stride 1
    _sets_equal(cuda_ops, oracle_port, mask, g, 0.5, False)
    _sets_equal(cuda_ops, oracle_port, mask, g, 0.2, True)


def test_window_wider_than_the_staging_area_uses_the_fallback(cuda_ops, oracle_port):
    rng = np.random.default_rng(4)
    mask = rng.standard_normal((1, 5, 12000, 1)).astype(np.float32)
    g = cfg.geom_for(5, 12000, (2, 5000), (2, 3000), (0, -10))
    _sets_equal(cuda_ops, oracle_port, mask, g, 3.5, False)
    _sets_equal(cuda_ops, oracle_port, mask, g, 0.001, True)


def test_full_size_bev_mask_matches(cuda_ops, oracle_port):
    c2 = cfg.config2(0)
    for run in c2["runs"]:
        _sets_equal(cuda_ops, oracle_port, c2["mask"], c2["geom"], run["tol"], run["avgpool"])


def test_misaligned_scratch_is_rejected(cuda_ops):
    import torch
    from sbnet_b200 import lib
    m = torch.zeros((1, 8, 8, 1), device="cuda")
    idx = torch.zeros((16, 3), dtype=torch.int16, device="cuda")
    scratch = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = lib.load().sbnet_reduce_mask(m.data_ptr(), 1, 8, 8, 0.5, 0, 0, 0, 2, 2, 2, 2, 4, 4, idx.data_ptr(),
                                      scratch.data_ptr() + 4, None, 0, None)
    assert rc == -1


def test_pageable_count_host(cuda_ops):
    """count_host in ordinary (unpinned) memory takes the copy path."""
    import ctypes as C
    import torch
    from sbnet_b200 import lib
    m = torch.ones((2, 16, 16, 1), device="cuda")
    idx = torch.zeros((2 * 4 * 4, 3), dtype=torch.int16, device="cuda")
    scratch = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = C.c_int32(-7)
    rc = lib.load().sbnet_reduce_mask(m.data_ptr(), 2, 16, 16, 0.5, 0, 0, 0, 4, 4, 4, 4, 4, 4, idx.data_ptr(),
                                      scratch.data_ptr(), C.addressof(out), 0,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and out.value == 32
    assert scratch.cpu().tolist() == [32, 0, 0, 0]


def test_two_thousand_calls_on_self_resetting_scratch(cuda_ops):
    """A scratch slot is zero-filled once and then only reset by the kernel itself.  Alternate masks
    of different counts for many calls: through the op wrappers (polled and device-side counts, each
    call on a fresh slot of a slab) and through the raw entry point on ONE slot for every call."""
    import ctypes as C
    import torch
    from sbnet_b200 import lib, ops
    g = cfg.halo_geom(160, 176)
    masks_h = [cfg.rect_union_mask(2, 160, 176, seed=s, n_rects=k) for s, k in ((1, 3), (2, 12), (3, 0), (4, 30))]
    masks = [torch.from_numpy(m).cuda() for m in masks_h]
    expect = []
    for m in masks:
        idx, cnt = ops.reduce_mask(m, *g.as_lists(), tol=0.5)
        expect.append(int(cnt[0]))
    assert expect[2] == 1 and len(set(expect)) == 4
    for i in range(2000):
        k = (i * 7 + i // 3) % 4
        if i % 5 == 0:
            idx, cnt_dev = ops.reduce_mask_async(masks[k], *g.as_lists(), tol=0.5)
            got = int(cnt_dev.cpu()[0])
        else:
            idx, cnt = ops.reduce_mask(masks[k], *g.as_lists(), tol=0.5)
            got = int(cnt[0])
        assert got == expect[k], (i, k, got, expect[k])
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    slab = ops._scratch[(masks[0].device.index, stream)][0].cpu().view(-1, 4)
    assert int(slab[:, 2:].abs().sum()) == 0          # every cursor word was left at zero
    # the raw entry point, one caller-owned slot reused by every call
    scratch = torch.zeros(4, dtype=torch.int32, device="cuda")
    idx = torch.zeros((2 * g.bcount[0] * g.bcount[1], 3), dtype=torch.int16, device="cuda")
    out = C.c_int32(0)
    for i in range(600):
        k = (i * 5 + i // 7) % 4
        rc = lib.load().sbnet_reduce_mask(masks[k].data_ptr(), 2, 160, 176, 0.5, 0, g.boffset[0], g.boffset[1],
                                          g.bsize[0], g.bsize[1], g.bstride[0], g.bstride[1], g.bcount[0],
                                          g.bcount[1], idx.data_ptr(), scratch.data_ptr(), C.addressof(out),
                                          lib.SBNET_SCRATCH_CLEAN | (lib.SBNET_MASK_STABLE if i % 2 else 0), stream)
        assert rc == 0 and out.value == expect[k], (i, k, rc, out.value)
    assert scratch.cpu().tolist() == [expect[k], 0, 0, 0]


def test_results_of_several_calls_may_be_outstanding(cuda_ops):
    """Every asynchronous call owns its count word: two results in flight on one stream do not alias,
    and a synchronous call in between does not disturb them."""
    import torch
    from sbnet_b200 import ops
    g = cfg.halo_geom(160, 176)
    a = torch.from_numpy(cfg.rect_union_mask(2, 160, 176, seed=5, n_rects=5)).cuda()
    b = torch.from_numpy(cfg.rect_union_mask(2, 160, 176, seed=6, n_rects=25)).cuda()
    na = int(ops.reduce_mask(a, *g.as_lists(), tol=0.5)[1][0])
    nb = int(ops.reduce_mask(b, *g.as_lists(), tol=0.5)[1][0])
    assert na != nb
    ia, ca = ops.reduce_mask_async(a, *g.as_lists(), tol=0.5)
    ib, cb = ops.reduce_mask_async(b, *g.as_lists(), tol=0.5, mask_stable=True)
    _, cs = ops.reduce_mask(a, *g.as_lists(), tol=0.5)
    x = torch.randn((2, 160, 176, 16), device="cuda")
    max_blocks = ia.shape[0]
    ya = ops.sparse_gather_dyn(x, ca, max_blocks, ia, g.bsize, g.bstride, g.boffset)
    yb = ops.sparse_gather_dyn(x, cb, max_blocks, ib, g.bsize, g.bstride, g.boffset)
    torch.cuda.synchronize()
    assert int(ca[0]) == na and int(cb[0]) == nb and int(cs[0]) == na
    assert torch.equal(ya[:na], ops.sparse_gather(x, [na], ia, g.bsize, g.bstride, g.boffset))
    assert torch.equal(yb[:nb], ops.sparse_gather(x, [nb], ib, g.bsize, g.bstride, g.boffset))


def test_two_streams_with_their_own_scratch_do_not_interfere(cuda_ops):
    import torch
    from sbnet_b200 import ops
    g = cfg.halo_geom(160, 176)
    a = torch.from_numpy(cfg.rect_union_mask(2, 160, 176, seed=5, n_rects=5)).cuda()
    b = torch.from_numpy(cfg.rect_union_mask(2, 160, 176, seed=6, n_rects=25)).cuda()
    na = int(ops.reduce_mask(a, *g.as_lists(), tol=0.5)[1][0])
    nb = int(ops.reduce_mask(b, *g.as_lists(), tol=0.5)[1][0])
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for i in range(200):
        with torch.cuda.stream(s1):
            outs.append((ops.reduce_mask_async(a, *g.as_lists(), tol=0.5)[1], na))
        with torch.cuda.stream(s2):
            outs.append((ops.reduce_mask_async(b, *g.as_lists(), tol=0.5)[1], nb))
    torch.cuda.synchronize()
    assert all(int(c[0]) == n for c, n in outs)


def test_count_without_waiting(cuda_ops):
    """SBNET_COUNT_NOWAIT: the call returns after the launch, the pinned word reads SBNET_COUNT_PENDING until
    the kernel stores the count; several calls may be in flight; pageable memory is refused."""
    import ctypes as C
    import torch
    from sbnet_b200 import lib, ops
    g = cfg.halo_geom(160, 176)
    masks = [torch.from_numpy(cfg.rect_union_mask(2, 160, 176, seed=s, n_rects=k)).cuda() for s, k in ((1, 4), (2, 0), (3, 19))]
    expect = [int(ops.reduce_mask(m, *g.as_lists(), tol=0.5)[1][0]) for m in masks]
    call = ops.bind_reduce_mask(masks[0], *g.as_lists(), tol=0.5, wait=False)
    for _ in range(50):
        out = [call(m) for m in masks]                    # three launches in flight, nothing waited for
        got = [ops.wait_count(cnt) for _, cnt, _ in out]
        assert got == expect
        assert all(ops.count_ready(cnt) for _, cnt, _ in out)
    torch.cuda.synchronize()
    assert [int(c[0]) for _, _, c in out] == expect       # the device-side counts agree
    idx = torch.zeros((2 * g.bcount[0] * g.bcount[1], 3), dtype=torch.int16, device="cuda")
    scratch = torch.zeros(4, dtype=torch.int32, device="cuda")
    pageable = C.c_int32(5)
    rc = lib.load().sbnet_reduce_mask(masks[0].data_ptr(), 2, 160, 176, 0.5, 0, g.boffset[0], g.boffset[1], g.bsize[0],
                                      g.bsize[1], g.bstride[0], g.bstride[1], g.bcount[0], g.bcount[1], idx.data_ptr(),
                                      scratch.data_ptr(), C.addressof(pageable), lib.SBNET_COUNT_NOWAIT, None)
    assert rc == -1 and "pinned" in lib.load().sbnet_last_error().decode() and pageable.value == 5
