"""The benchmark configurations at their FULL sizes on the GPU against the CPU checker, whole launches,
through the C ABI -- with the assertions of the reference's own integration test
(``sbnet_ops/tests/test_sparse_blocks.py:296-342``: equal counts, equal sorted indices, gathered blocks
bit-equal, transposed == transpose of untransposed, scattered outputs bit-equal):

* sparse_gather on x [8,512,512,128], fp16 and fp32, both layouts, 5 / 20 / 50 % of the blocks;
* sparse_scatter_var transposed overwrite of fp16 [nB,64,16,16] stacks onto [8,512,512,64];
* sparse_scatter / sparse_scatter_var fp32 atomic add over overlapping 18x18 halos onto [8,512,512,64]
  (order dependent: both results inside the fp64 exact-sum bars, image by image);
* the sparse bottleneck's block ops on x fp16 [32,400,352,256] at 10 % and 30 % mask occupancy:
  reduce_mask, transposed gather with its halo rows, non-atomic transposed add;
* pixels that are not 16-byte multiples ([8,512,512,33] fp32, [8,512,512,100] fp16): gather, overwrite,
  read-add-write, atomic add.

Size-independent properties of the same launches (layout identities, round trips, exact coverage
counts from atomic adds of ones) ride along.  Tensors of a gigabyte and more are compared on the
device (the checker's result is uploaded) so the host holds one copy at a time.
"""
import numpy as np
import pytest
import torch

from atomic_check import check_atomic_add
from sbnet_b200 import configs as cfg

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _coverage(idx_h, nb, g, N, H, W):
    cov = np.zeros((N, H, W), dtype=np.int32)
    for n, bh, bw in np.asarray(idx_h[:nb]).astype(np.int64):
        h0, w0 = g.boffset[0] + bh * g.bstride[0], g.boffset[1] + bw * g.bstride[1]
        cov[n, max(h0, 0):min(h0 + g.bsize[0], H), max(w0, 0):min(w0 + g.bsize[1], W)] += 1
    return cov


def _same_bits(dev_tensor, host_array):
    """Bit-equality of a device tensor with a numpy array, compared on the device."""
    exp = torch.from_numpy(host_array).to(dev_tensor.device)
    return exp.shape == dev_tensor.shape and torch.equal(dev_tensor.view(torch.int16 if exp.element_size() == 2 else torch.int32),
                                                         exp.view(torch.int16 if exp.element_size() == 2 else torch.int32))


def _border_blocks_present(idx_h, nb, bcount):
    """The list holds blocks on all four image borders and in at least one corner."""
    bh, bw = idx_h[:nb, 1], idx_h[:nb, 2]
    edges = [(bh == 0).any(), (bh == bcount[0] - 1).any(), (bw == 0).any(), (bw == bcount[1] - 1).any()]
    corner = (((bh == 0) | (bh == bcount[0] - 1)) & ((bw == 0) | (bw == bcount[1] - 1))).any()
    return all(edges) and bool(corner)


@pytest.mark.parametrize("dtype", [np.float16, np.float32], ids=["f16", "f32"])
def test_config3_gather_whole_launches_against_cpu(cuda_ops, oracle_port, dtype):
    from sbnet_b200 import ops
    N, H, W, C = 8, 512, 512, 128
    g, gi = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    xd = torch.randn((N, H, W, C), device=DEV, generator=torch.Generator(DEV).manual_seed(3)).to(
        torch.float16 if dtype == np.float16 else torch.float32)
    xh = xd.cpu().numpy()
    oracle_port.set_threads(oracle_port.max_threads())
    for dens in (0.05, 0.20, 0.50):
        idx_h, cnt_h = cfg.random_block_list(N, g.bcount, dens, seed=int(dens * 100))
        nb = int(cnt_h[0])
        assert _border_blocks_present(idx_h, nb, g.bcount)
        idx, cnt = torch.from_numpy(idx_h).to(DEV), torch.from_numpy(cnt_h)
        rows = ops.sparse_gather(xd, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=False)
        planes = ops.sparse_gather(xd, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=True)
        exp = oracle_port.sparse_gather(xh, cnt_h, idx_h, g.bsize, g.bstride, g.boffset, transpose=False)
        assert _same_bits(rows, exp), f"rows layout differs from the CPU checker at {dens}"
        del exp
        exp_t = oracle_port.sparse_gather(xh, cnt_h, idx_h, g.bsize, g.bstride, g.boffset, transpose=True)
        assert _same_bits(planes, exp_t), f"planes layout differs from the CPU checker at {dens}"
        del exp_t
        assert torch.equal(planes, rows.permute(0, 3, 1, 2))          # test_sparse_blocks.py:341-342
        if dens == 0.50:
            # round trip: the 16x16 interiors written back onto zeros reproduce x on covered pixels
            inner = rows[:, 1:17, 1:17, :].contiguous()
            y = ops.sparse_scatter_var(inner, cnt, idx, torch.zeros_like(xd), gi.bsize, gi.bstride, gi.boffset, add=False)
            cov = torch.from_numpy(_coverage(idx_h, nb, gi, N, H, W) > 0).to(DEV)
            assert torch.equal(y[cov], xd[cov]) and float(y[~cov].abs().max()) == 0.0
            inner_t = planes[:, :, 1:17, 1:17].contiguous()
            y2 = ops.sparse_scatter_var(inner_t, cnt, idx, torch.zeros_like(xd), gi.bsize, gi.bstride, gi.boffset,
                                        add=False, transpose=True)
            assert torch.equal(y2, y)
            del y, y2, inner, inner_t
        del rows, planes


def test_config4b_transposed_overwrite_whole_launches_against_cpu(cuda_ops, oracle_port):
    from sbnet_b200 import ops
    N, H, W, C = 8, 512, 512, 64
    gi = cfg.inner_geom(H, W)
    base_h = cfg.normal((N, H, W, C), 4, np.float16)
    base_d = torch.from_numpy(base_h).to(DEV)
    oracle_port.set_threads(oracle_port.max_threads())
    for dens in (0.05, 0.20, 0.50):
        idx_h, cnt_h = cfg.random_block_list(N, gi.bcount, dens, seed=int(dens * 100) + 1)
        nb = int(cnt_h[0])
        assert _border_blocks_present(idx_h, nb, gi.bcount)
        stack_h = cfg.normal((nb, C, 16, 16), 5, np.float16)
        idx, cnt = torch.from_numpy(idx_h).to(DEV), torch.from_numpy(cnt_h)
        stack_d = torch.from_numpy(stack_h).to(DEV)
        y_var = ops.sparse_scatter_var(stack_d, cnt, idx, base_d.clone(), gi.bsize, gi.bstride, gi.boffset, add=False,
                                       transpose=True)
        y = ops.sparse_scatter(stack_d, cnt, idx, base_d, gi.bsize, gi.bstride, gi.boffset, add=False, transpose=True)
        exp = oracle_port.sparse_scatter_var(stack_h, cnt_h, idx_h, base_h.copy(), gi.bsize, gi.bstride, gi.boffset,
                                             add=False, transpose=True)
        assert _same_bits(y_var, exp) and _same_bits(y, exp), f"overwrite differs from the CPU checker at {dens}"
        assert _same_bits(base_d, base_h)                               # the non-Var op left its base alone


@pytest.mark.parametrize("dens", [0.05, 0.20, 0.50])
def test_config4a_atomic_add_whole_launches_within_exact_sum_bars(cuda_ops, oracle_port, dens):
    from sbnet_b200 import ops
    N, H, W, C = 8, 512, 512, 64
    g = cfg.halo_geom(H, W)
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, dens, seed=int(dens * 100) + 1)
    nb = int(cnt_h[0])
    assert _border_blocks_present(idx_h, nb, g.bcount)
    stack_h = cfg.normal((nb, 18, 18, C), 6, np.float32)
    base_h = cfg.normal((N, H, W, C), 7, np.float32)
    idx, cnt = torch.from_numpy(idx_h).to(DEV), torch.from_numpy(cnt_h)
    stack_d, base_d = torch.from_numpy(stack_h).to(DEV), torch.from_numpy(base_h).to(DEV)
    y_var = ops.sparse_scatter_var(stack_d, cnt, idx, base_d.clone(), g.bsize, g.bstride, g.boffset, add=True,
                                   atomic=True).cpu().numpy()
    y = ops.sparse_scatter(stack_d, cnt, idx, base_d, g.bsize, g.bstride, g.boffset, add=True, atomic=True).cpu().numpy()
    exp = oracle_port.sparse_scatter_var(stack_h, cnt_h, idx_h, base_h.copy(), g.bsize, g.bstride, g.boffset,
                                         add=True, atomic=True)         # one thread, list order
    worst = 0.0
    for n in range(N):          # image by image: the fp64 work arrays stay small
        sel = np.flatnonzero(idx_h[:nb, 0] == n)
        sub_idx = idx_h[sel].copy()
        sub_idx[:, 0] = 0
        out = check_atomic_add({"scatter_var": y_var[n:n + 1], "scatter": y[n:n + 1], "cpu checker": exp[n:n + 1]},
                               stack_h[sel], [len(sel)], sub_idx, base_h[n:n + 1], g.bsize, g.bstride, g.boffset)
        worst = max(worst, max(v[1] for v in out.values()))
    assert worst <= 1e-6          # the relative bar where nothing cancels, over the whole tensor
    if dens == 0.50:
        # ones scattered with atomic adds give the exact number of covering blocks (small integers)
        ones = torch.ones((nb, 18, 18, C), device=DEV)
        cov = torch.from_numpy(_coverage(idx_h, nb, g, N, H, W)).to(DEV).to(torch.float32)
        yy = ops.sparse_scatter_var(ones, cnt, idx, torch.zeros((N, H, W, C), device=DEV), g.bsize, g.bstride,
                                    g.boffset, add=True, atomic=True)
        assert torch.equal(yy, cov[..., None].expand(-1, -1, -1, C)) and int(cov.max()) == 4


@pytest.mark.parametrize("occupancy", [0.10, 0.30], ids=["occ10", "occ30"])
def test_config5_pipeline_whole_launches_against_cpu(cuda_ops, oracle_port, occupancy):
    from sbnet_b200 import ops
    import pipeline
    N, H, W, C = 32, 400, 352, 256
    g, gi = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    mask_h = cfg.rect_union_mask(N, H, W, seed=7, occupancy=occupancy)
    mask = torch.from_numpy(mask_h).to(DEV)
    x = torch.empty((N, H, W, C), dtype=torch.float16, device=DEV)
    gen = torch.Generator(DEV).manual_seed(11)
    for n in range(N):
        x[n] = torch.randn((H, W, C), device=DEV, generator=gen).half()
    xh = x.cpu().numpy()
    oracle_port.set_threads(oracle_port.max_threads())

    # reduce_mask: count and sorted index list
    idx, cnt = ops.reduce_mask(mask, *g.as_lists(), tol=0.5)
    oi, oc = oracle_port.reduce_mask(mask_h, *g.as_lists(), tol=0.5, avgpool=False)
    nb = int(cnt[0])
    assert nb == int(oc[0])
    idx_h = idx.cpu().numpy()
    order = pipeline.sort_order(idx_h, nb, g.bcount)
    np.testing.assert_array_equal(idx_h[:nb][order], oi[:nb])       # the checker lists blocks in key order
    assert _border_blocks_present(idx_h, nb, g.bcount)

    # gather (transposed, halo rows and columns included), in the GPU's own block order
    p = ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=True)
    exp = oracle_port.sparse_gather(xh, cnt.numpy(), idx_h, g.bsize, g.bstride, g.boffset, transpose=True)
    assert _same_bits(p, exp), "gather differs from the CPU checker"
    # halo rows of a border block are the zero padding, those of interior blocks are image rows
    top = int(np.flatnonzero(idx_h[:nb, 1] == 0)[0])
    assert float(p[top, :, 0, :].abs().max()) == 0.0
    inner_blk = int(np.flatnonzero((idx_h[:nb, 1] > 0) & (idx_h[:nb, 2] > 0) & (idx_h[:nb, 2] < g.bcount[1] - 1))[0])
    n0, bh, bw = (int(v) for v in idx_h[inner_blk])
    assert torch.equal(p[inner_blk, :, 0, :], x[n0, 16 * bh - 1, 16 * bw - 1:16 * bw + 17, :].t())
    del exp

    # conv-output-shaped stack, non-atomic transposed add onto x (disjoint 16x16 interiors)
    q = (torch.randn((nb, C, 16, 16), device=DEV, generator=gen) * 0.5).half()
    qh = q.cpu().numpy()
    ops.sparse_scatter_var(q, cnt, idx, x, gi.bsize, gi.bstride, gi.boffset, add=True, transpose=True)
    exp = oracle_port.sparse_scatter_var(qh, cnt.numpy(), idx_h, xh, gi.bsize, gi.bstride, gi.boffset, add=True,
                                         transpose=True)
    assert _same_bits(x, exp), "scatter-add differs from the CPU checker"
    del exp, xh

    if occupancy == 0.10:
        # x + gathered interiors == 2x on active interiors (doubling is exact in fp16), x elsewhere
        x0 = x.clone()
        p = ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=True)
        ops.sparse_scatter_var(p[:, :, 1:17, 1:17].contiguous(), cnt, idx, x, gi.bsize, gi.bstride, gi.boffset, add=True,
                               transpose=True)
        cov = torch.from_numpy(_coverage(idx_h, nb, gi, N, H, W) > 0).to(DEV)
        assert torch.equal(x[cov], x0[cov] * 2) and torch.equal(x[~cov], x0[~cov])


@pytest.mark.parametrize("dtype,C", [(np.float32, 33), (np.float16, 100)], ids=["f32_C33", "f16_C100"])
def test_pixels_that_are_not_16_byte_multiples_whole_launches_against_cpu(cuda_ops, oracle_port, dtype, C):
    """[8,512,512,C] with C = 33 (fp32) and C = 100 (fp16) at 20 % of the blocks -- the shapes of the benchmark
    table's odd-channel rows, which run the raw-row kernel in the plane layout and the narrow-vector kernel in the
    row layout: gather in both layouts, overwrite and read-add-write of the 16x16 interiors (disjoint blocks), all
    bit-equal to the CPU checker; atomic add of the 18x18 halos inside the exact-sum bars."""
    from sbnet_b200 import ops
    N, H, W = 8, 512, 512
    g, gi = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    xh = cfg.normal((N, H, W, C), 51, dtype)
    xd = torch.from_numpy(xh).to(DEV)
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, 0.20, seed=52)
    nb = int(cnt_h[0])
    assert _border_blocks_present(idx_h, nb, g.bcount)
    idx, cnt = torch.from_numpy(idx_h).to(DEV), torch.from_numpy(cnt_h)
    oracle_port.set_threads(oracle_port.max_threads())
    rows = ops.sparse_gather(xd, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=False)
    planes = ops.sparse_gather(xd, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=True)
    exp = oracle_port.sparse_gather(xh, cnt_h, idx_h, g.bsize, g.bstride, g.boffset, transpose=True)
    assert _same_bits(planes, exp)
    del exp
    assert torch.equal(planes, rows.permute(0, 3, 1, 2))
    del rows, planes
    for tr in (False, True):
        sshape = (nb, C, 16, 16) if tr else (nb, 16, 16, C)
        stack_h = cfg.normal(sshape, 53, dtype)
        stack_d = torch.from_numpy(stack_h).to(DEV)
        for add in (False, True):
            y = ops.sparse_scatter_var(stack_d, cnt, idx, xd.clone(), gi.bsize, gi.bstride, gi.boffset, add=add, transpose=tr)
            exp = oracle_port.sparse_scatter_var(stack_h, cnt_h, idx_h, xh.copy(), gi.bsize, gi.bstride, gi.boffset,
                                                 add=add, transpose=tr)
            assert _same_bits(y, exp), (tr, add)
            del y, exp
    # overlapping halos, one image's blocks at a time (fp64 work arrays stay small)
    halo_h = cfg.normal((nb, C, 18, 18), 54, dtype)
    y = ops.sparse_scatter_var(torch.from_numpy(halo_h).to(DEV), cnt, idx, xd.clone(), g.bsize, g.bstride, g.boffset,
                               add=True, atomic=True, transpose=True).cpu().numpy()
    for n in (0, N - 1):
        sel = np.flatnonzero(idx_h[:nb, 0] == n)
        sub_idx = idx_h[sel].copy()
        sub_idx[:, 0] = 0
        check_atomic_add({"cuda": y[n:n + 1]}, halo_h[sel], [len(sel)], sub_idx, xh[n:n + 1], g.bsize, g.bstride,
                         g.boffset, True)
