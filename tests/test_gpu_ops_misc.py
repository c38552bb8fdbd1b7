"""Gather / scatter mode matrix, vector-width fallbacks, device-count variants, copy and timers on
the GPU against the CPU checker (through the C ABI)."""
import numpy as np
import pytest

from sbnet_b200 import configs as cfg

pytestmark = pytest.mark.gpu


from atomic_check import check_atomic_add


# channel counts chosen to hit every vector width: C*sizeof(T) in {2,4,6,8,12,14,16,30,48,...}
@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("C", [1, 2, 3, 4, 6, 7, 8, 15, 24, 40])
@pytest.mark.parametrize("transpose", [False, "rows_vectors", True, "elementwise", "raw_rows_narrow"],
                         ids=["rows", "rows_vector_kernel", "planes", "planes_elementwise", "planes_raw_rows_narrow"])
def test_mode_matrix(cuda_ops, oracle_port, dtype, C, transpose):
    """``rows`` / ``planes``: pixels that are not 8- / 16-byte multiples run the raw-row kernel of the general
    path; ``rows_vector_kernel`` and ``planes_elementwise`` send the same calls through the kernels it replaced,
    ``planes_raw_rows_narrow`` through the raw-row kernel with element-wide stack accesses."""
    from conftest import library_options
    with library_options(planes={"rows_vectors": 4, "elementwise": 4, "raw_rows_narrow": 6}.get(transpose, 0)):
        _mode_matrix(cuda_ops, oracle_port, dtype, C, transpose not in (False, "rows_vectors"))


def _mode_matrix(cuda_ops, oracle_port, dtype, C, transpose):
    N, H, W = 2, 23, 31
    bsize, bstride, boffset = (5, 4), (3, 4), (-2, -1)      # rows overlap, columns touch
    g = cfg.geom_for(H, W, bsize, bstride, boffset)
    idx, cnt = cfg.random_block_list(N, g.bcount, 0.7, seed=C)
    nb = int(cnt[0])
    x = cfg.normal((N, H, W, C), 1, dtype)
    exp = oracle_port.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=transpose)
    got = cuda_ops.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=transpose)
    np.testing.assert_array_equal(got, exp)

    shape = (nb, C, *bsize) if transpose else (nb, *bsize, C)
    stack = cfg.normal(shape, 2, dtype)
    base = cfg.normal((N, H, W, C), 3, dtype)
    # atomic add over overlapping rows
    e = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                       atomic=True, transpose=transpose)
    o = cuda_ops.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                    atomic=True, transpose=transpose)
    check_atomic_add({"cuda": o, "cpu checker": e}, stack, cnt, idx, base, bsize, bstride, boffset, transpose)
    # overwrite with equal values on shared pixels (a gathered stack)
    e = oracle_port.sparse_scatter(exp, cnt, idx, base, bsize, bstride, boffset, add=False, transpose=transpose)
    o = cuda_ops.sparse_scatter(exp, cnt, idx, base, bsize, bstride, boffset, add=False, transpose=transpose)
    np.testing.assert_array_equal(o, e)
    # disjoint geometry: overwrite and non-atomic add are bit-exact
    g2 = cfg.geom_for(H, W, bsize, (5, 6), (-1, -3))
    idx2, cnt2 = cfg.random_block_list(N, g2.bcount, 0.7, seed=C + 1)
    shape2 = (int(cnt2[0]), C, *bsize) if transpose else (int(cnt2[0]), *bsize, C)
    st2 = cfg.normal(shape2, 4, dtype)
    for add in (False, True):
        e = oracle_port.sparse_scatter_var(st2, cnt2, idx2, base.copy(), bsize, (5, 6), (-1, -3), add=add,
                                           transpose=transpose)
        o = cuda_ops.sparse_scatter_var(st2, cnt2, idx2, base.copy(), bsize, (5, 6), (-1, -3), add=add,
                                        transpose=transpose)
        np.testing.assert_array_equal(o, e)


def test_add_with_subnormals_is_bit_exact(cuda_ops, oracle_port):
    """Non-atomic add must not flush subnormal inputs or results (fp32 and fp16)."""
    g = cfg.geom_for(8, 8, (4, 4), (4, 4), (0, 0))
    idx, cnt = cfg.random_block_list(1, g.bcount, 1.0, seed=0)
    for dtype, tiny in ((np.float32, 1e-41), (np.float16, 3e-7)):
        for transpose in (False, True):
            C = 64 if dtype == np.float16 else 32
            shape = (4, C, 4, 4) if transpose else (4, 4, 4, C)
            stack = np.full(shape, tiny, dtype)
            base = np.full((1, 8, 8, C), tiny, dtype)
            base[0, ::2] = -base[0, ::2] * 3
            e = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), (4, 4), (4, 4), (0, 0), add=True,
                                               transpose=transpose)
            o = cuda_ops.sparse_scatter_var(stack, cnt, idx, base.copy(), (4, 4), (4, 4), (0, 0), add=True,
                                            transpose=transpose)
            assert (e != 0).any()
            np.testing.assert_array_equal(o.view(np.uint8), e.view(np.uint8))


def test_overlapping_add_without_atomics_is_rejected(cuda_ops):
    x = np.zeros((1, 2, 2, 1), np.float32)
    with pytest.raises(ValueError, match="non-overlapping"):
        cuda_ops.sparse_scatter_var(x, [1], np.zeros((1, 3), np.int16), np.zeros((1, 4, 4, 1), np.float32),
                                    [2, 2], [1, 1], [0, 0], add=True, atomic=False)
    with pytest.raises(ValueError, match="non-overlapping"):
        cuda_ops.sparse_scatter(x, [1], np.zeros((1, 3), np.int16), np.zeros((1, 4, 4, 1), np.float32),
                                [2, 2], [1, 1], [0, 0], add=True, atomic=False)


def test_outputs_are_not_written_past_their_end(cuda_ops, oracle_port):
    """Guard bands: the stack and the image live in the middle of larger allocations."""
    import torch
    from sbnet_b200 import ops
    N, H, W, C = 1, 40, 40, 32
    g = cfg.halo_geom(32, 32)
    g = cfg.geom_for(H, W, (18, 18), (16, 16), (-1, -1))
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, 1.0, seed=0)
    nb = int(cnt_h[0])
    dev = "cuda"
    x = torch.randn((N, H, W, C), device=dev)
    idx = torch.from_numpy(idx_h).to(dev)
    cnt = torch.from_numpy(cnt_h)
    pad = 4096
    for tr in (False, True):
        n_out = nb * 18 * 18 * C
        big = torch.full((n_out + 2 * pad,), 7.0, device=dev)
        out = big[pad:pad + n_out].view((nb, C, 18, 18) if tr else (nb, 18, 18, C))
        ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=tr, out=out)
        assert bool((big[:pad] == 7.0).all()) and bool((big[pad + n_out:] == 7.0).all())
        bigy = torch.full((N * H * W * C + 2 * pad,), 7.0, device=dev)
        y = bigy[pad:pad + N * H * W * C].view(N, H, W, C)
        ops.sparse_scatter_var(out, cnt, idx, y, g.bsize, g.bstride, g.boffset, add=False, transpose=tr)
        assert bool((bigy[:pad] == 7.0).all()) and bool((bigy[pad + N * H * W * C:] == 7.0).all())
        np.testing.assert_array_equal(y.cpu().numpy(), x.cpu().numpy())   # full coverage: y == x


def test_device_count_pipeline_matches_host_count_pipeline(cuda_ops, oracle_port):
    import torch
    from sbnet_b200 import ops
    c = cfg.config1(0)
    g, go = c["geom"], c["geom_out"]
    dev = "cuda"
    x = torch.from_numpy(c["x"]).to(dev)
    mask = torch.from_numpy(c["mask"]).to(dev)
    idx, cnt = ops.reduce_mask(mask, *g.as_lists(), tol=0.5)
    nb = int(cnt[0])
    max_blocks = idx.shape[0]
    for tr in (False, True):
        ref = ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=tr)
        idx2, cnt_dev = ops.reduce_mask_async(mask, *g.as_lists(), tol=0.5)
        out = torch.full((max_blocks, 32, 10, 10) if tr else (max_blocks, 10, 10, 32), -3.0, device=dev)
        ops.sparse_gather_dyn(x, cnt_dev, max_blocks, idx2, g.bsize, g.bstride, g.boffset, transpose=tr, out=out)
        torch.cuda.synchronize()
        assert int(cnt_dev[0]) == nb
        # same blocks (order may differ between the two reduce_mask calls)
        key = lambda i: (i[:, 0].long() * 64 + i[:, 1].long() * 8 + i[:, 2].long()).argsort()  # noqa: E731
        assert torch.equal(out[:nb][key(idx2[:nb])], ref[key(idx[:nb])])
        assert bool((out[nb:] == -3.0).all())
        inner = (out[:, :, 1:9, 1:9] if tr else out[:, 1:9, 1:9, :]).contiguous()
        y1 = ops.sparse_scatter_var_dyn(inner, cnt_dev, max_blocks, idx2, torch.zeros_like(x), go.bsize,
                                        go.bstride, go.boffset, add=True, transpose=tr)
        y2 = ops.sparse_scatter_var(inner[:nb].contiguous(), cnt, idx2, torch.zeros_like(x), go.bsize,
                                    go.bstride, go.boffset, add=True, transpose=tr)
        assert torch.equal(y1, y2)


@pytest.mark.parametrize("nbytes,off", [(1, 0), (15, 0), (16, 0), (4097, 0), (1 << 20, 0), (1000, 1), (5000, 8)])
def test_copy_tensor(cuda_ops, nbytes, off):
    import torch
    from sbnet_b200 import lib
    src = torch.randint(0, 255, (nbytes + 64,), dtype=torch.uint8, device="cuda")
    dst = torch.zeros(nbytes + 64, dtype=torch.uint8, device="cuda")
    lib.check(lib.load().sbnet_copy_tensor(dst.data_ptr() + off, src.data_ptr() + off, nbytes,
                                           torch.cuda.current_stream().cuda_stream))
    assert torch.equal(dst[off:off + nbytes], src[off:off + nbytes])
    assert int(dst[off + nbytes:].sum()) == 0 and int(dst[:off].sum()) == 0


def test_cuda_timers(cuda_ops):
    import torch
    from sbnet_b200 import ops
    h = ops.cuda_timer_start()
    a = torch.randn(1 << 22, device="cuda")
    (a * 2).sum().item()
    ms = ops.cuda_timer_end(h)
    assert 0.0 < ms < 5000.0


def test_device_count_pipeline_replays_from_a_cuda_graph(cuda_ops, oracle_port):
    """mask -> gather -> scatter captured once, replayed on two different masks written into the same
    buffers: the block count never visits the host, so the graph adapts to each mask by itself."""
    import torch
    from sbnet_b200 import ops
    dev = "cuda"
    N, H, W, C = 2, 64, 48, 64
    g, go = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    max_blocks = N * g.bcount[0] * g.bcount[1]
    x_h = cfg.normal((N, H, W, C), 1, np.float16)
    masks = [cfg.rect_union_mask(N, H, W, seed=s, occupancy=occ, side=(4, 12)) for s, occ in ((1, 0.1), (2, 0.35))]
    mask = torch.from_numpy(masks[0]).to(dev)
    x = torch.from_numpy(x_h).to(dev)
    y = torch.zeros_like(x)
    stack = torch.zeros((max_blocks, C, 18, 18), dtype=torch.float16, device=dev)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())

    def enqueue():
        idx, cnt_dev = ops.reduce_mask_async(mask, *g.as_lists(), tol=0.5)
        ops.sparse_gather_dyn(x, cnt_dev, max_blocks, idx, g.bsize, g.bstride, g.boffset, transpose=True, out=stack)
        inner = stack[:, :, 1:17, 1:17].contiguous()
        ops.sparse_scatter_var_dyn(inner, cnt_dev, max_blocks, idx, y, go.bsize, go.bstride, go.boffset, add=True,
                                   transpose=True)
        return idx, cnt_dev

    with torch.cuda.stream(side):
        enqueue()                                   # warm-up: scratch allocation, lazy loading
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        idx, cnt_dev = enqueue()
    counts = []
    for m_h in masks:
        mask.copy_(torch.from_numpy(m_h))
        y.zero_()
        graph.replay()
        torch.cuda.synchronize()
        oi, oc = oracle_port.reduce_mask(m_h, *g.as_lists(), tol=0.5)
        n = int(oc[0])
        counts.append(n)
        assert int(cnt_dev[0]) == n
        got_idx = idx[:n].cpu().numpy()
        assert sorted(map(tuple, got_idx.tolist())) == sorted(map(tuple, oi[:n].tolist()))
        # reference result: gather interiors of the active blocks added onto zeros == x on those pixels
        st = oracle_port.sparse_gather(x_h, oc, oi, g.bsize, g.bstride, g.boffset, transpose=True)
        exp = oracle_port.sparse_scatter_var(np.ascontiguousarray(st[:, :, 1:17, 1:17]), oc, oi, np.zeros_like(x_h),
                                             go.bsize, go.bstride, go.boffset, add=True, transpose=True)
        np.testing.assert_array_equal(y.cpu().numpy(), exp)
    assert counts[0] != counts[1]


def test_bound_calls_match_the_ordinary_wrappers(cuda_ops):
    """bind_reduce_mask / bind_sparse_gather / bind_sparse_scatter_var (arguments validated once) give the
    results of the per-call wrappers, also on a stream passed by handle, and still reject what changes
    shape under them."""
    import torch
    from sbnet_b200 import ops
    dev = "cuda"
    N, H, W, C = 2, 64, 48, 64
    g, gi = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    masks = [torch.from_numpy(cfg.rect_union_mask(N, H, W, seed=s, occupancy=0.3, side=(4, 16))).to(dev) for s in (1, 2)]
    x = torch.randn((N, H, W, C), device=dev).half()
    cap = N * g.bcount[0] * g.bcount[1]
    stack = torch.empty((cap, C, 18, 18), dtype=torch.float16, device=dev)
    q = (torch.randn((cap, C, 16, 16), device=dev) * 0.1).half()
    side = torch.cuda.Stream()
    for stream in (None, side.cuda_stream):
        rm = ops.bind_reduce_mask(masks[0], *g.as_lists(), tol=0.5, mask_stable=True, stream=stream)
        ga = ops.bind_sparse_gather(x, stack, g.bsize, g.bstride, g.boffset, transpose=True, stream=stream)
        y = x.clone()
        sc = ops.bind_sparse_scatter_var(q, y, gi.bsize, gi.bstride, gi.boffset, add=True, transpose=True, stream=stream)
        torch.cuda.synchronize()
        ref = x.clone()
        for m in masks:
            idx, cnt, cnt_dev = rm(m)
            ridx, rcnt = ops.reduce_mask(m, *g.as_lists(), tol=0.5)
            n = int(cnt[0])
            assert n == int(rcnt[0])
            ga(cnt, idx)
            sc(cnt, idx)
            torch.cuda.synchronize()
            assert int(cnt_dev[0]) == n
            assert sorted(map(tuple, idx[:n].tolist())) == sorted(map(tuple, ridx[:n].tolist()))
            assert torch.equal(stack[:n], ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=True))
            # the same stack rows onto the same block list through the ordinary wrapper
            ops.sparse_scatter_var(q[:n].contiguous(), cnt, idx, ref, gi.bsize, gi.bstride, gi.boffset, add=True,
                                   transpose=True)
        torch.cuda.synchronize()
        assert torch.equal(y, ref)
    # an index list of the caller's: written in place, same list as a fresh one
    mine = torch.full((cap, 3), -7, dtype=torch.int16, device=dev)
    idx2, cnt2, _ = rm(masks[1], None, mine)
    torch.cuda.synchronize()
    assert idx2 is mine and int(cnt2[0]) == n
    assert sorted(map(tuple, mine[:n].tolist())) == sorted(map(tuple, idx[:n].tolist()))
    assert bool((mine[n:] == -7).all())
    with pytest.raises(ValueError):
        rm(masks[1], None, mine[:-1])
    with pytest.raises(ValueError):
        rm(masks[1], None, mine.to(torch.int32))
    with pytest.raises(ValueError):
        rm(masks[0][:1])
    with pytest.raises(ValueError):
        ga([cap + 1], idx)
    with pytest.raises(ValueError):
        sc([1], idx.to(torch.int32))
