"""Full benchmark sizes on the GPU, checked through size-independent properties (the CPU checker
would take minutes here): layout identities, gather -> scatter round trips, exact coverage counts
from atomic adds of ones, and x + x == 2x for the add pipeline.  Everything goes through the C ABI."""
import numpy as np
import pytest
import torch

from sbnet_b200 import configs as cfg

pytestmark = pytest.mark.gpu


def _coverage(idx_h, nb, g, N, H, W, dev):
    cov = np.zeros((N, H, W), dtype=np.int32)
    for n, bh, bw in np.asarray(idx_h[:nb]).astype(np.int64):
        h0, w0 = g.boffset[0] + bh * g.bstride[0], g.boffset[1] + bw * g.bstride[1]
        cov[n, max(h0, 0):min(h0 + g.bsize[0], H), max(w0, 0):min(w0 + g.bsize[1], W)] += 1
    return torch.from_numpy(cov).to(dev)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32], ids=["f16", "f32"])
def test_gather_layouts_and_round_trip_at_config3_size(cuda_ops, dtype):
    from sbnet_b200 import ops
    dev = "cuda"
    N, H, W, C = 8, 512, 512, 128
    g, gi = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, 0.5, seed=3)
    nb = int(cnt_h[0])
    idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
    x = torch.randn((N, H, W, C), device=dev, dtype=torch.float32).to(dtype)
    rows = ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=False)
    planes = ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=True)
    assert torch.equal(planes, rows.permute(0, 3, 1, 2))          # test_sparse_blocks.py:341-342
    # border handling: a block at the image corner has zero first row / column
    first = int(np.flatnonzero((idx_h[:nb, 1] == 0) & (idx_h[:nb, 2] == 0))[0])
    assert float(rows[first, 0].abs().max()) == 0.0 and float(rows[first, :, 0].abs().max()) == 0.0
    n0 = int(idx_h[first, 0])
    assert torch.equal(rows[first, 1:, 1:], x[n0, :17, :17])
    # round trip: the 16x16 interiors written back onto zeros reproduce x on covered pixels
    inner = rows[:, 1:17, 1:17, :].contiguous()
    y = ops.sparse_scatter_var(inner, cnt, idx, torch.zeros_like(x), gi.bsize, gi.bstride, gi.boffset, add=False)
    cov = _coverage(idx_h, nb, gi, N, H, W, dev) > 0
    assert torch.equal(y[cov], x[cov]) and float(y[~cov].abs().max()) == 0.0
    inner_t = planes[:, :, 1:17, 1:17].contiguous()
    y2 = ops.sparse_scatter_var(inner_t, cnt, idx, torch.zeros_like(x), gi.bsize, gi.bstride, gi.boffset,
                                add=False, transpose=True)
    assert torch.equal(y2, y)


def test_atomic_scatter_counts_coverage_exactly_at_config4_size(cuda_ops):
    """Ones scattered with atomic adds over overlapping 18x18 halos give the exact number of blocks
    covering each pixel (small integers are exact in fp32 whatever the order)."""
    from sbnet_b200 import ops
    dev = "cuda"
    N, H, W, C = 8, 512, 512, 64
    g = cfg.halo_geom(H, W)
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, 0.5, seed=4)
    nb = int(cnt_h[0])
    idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
    ones = torch.ones((nb, 18, 18, C), device=dev)
    for make in (lambda: ops.sparse_scatter_var(ones, cnt, idx, torch.zeros((N, H, W, C), device=dev), g.bsize,
                                                g.bstride, g.boffset, add=True, atomic=True),
                 lambda: ops.sparse_scatter(ones, cnt, idx, torch.zeros((N, H, W, C), device=dev), g.bsize,
                                            g.bstride, g.boffset, add=True, atomic=True)):
        y = make()
        cov = _coverage(idx_h, nb, g, N, H, W, dev).to(torch.float32)
        assert torch.equal(y, cov[..., None].expand(-1, -1, -1, C))
    assert int(cov.max()) == 4      # halo corners are shared by four blocks


def test_pipeline_adds_x_to_itself_at_config5_size(cuda_ops):
    """mask -> gather(transpose) -> scatter_var(add, transpose) of the gathered interiors onto x gives
    exactly 2x on active interiors (doubling is exact in fp16) and x elsewhere."""
    from sbnet_b200 import ops
    dev = "cuda"
    N, H, W, C = 32, 400, 352, 256
    g, gi = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    mask_h = cfg.rect_union_mask(N, H, W, seed=7, occupancy=0.10)
    mask = torch.from_numpy(mask_h).to(dev)
    x = torch.empty((N, H, W, C), dtype=torch.float16, device=dev)
    for n in range(N):
        x[n] = torch.randn((H, W, C), device=dev).half()
    idx, cnt = ops.reduce_mask(mask, *g.as_lists(), tol=0.5)
    nb = int(cnt[0])
    idx_h = idx.cpu().numpy()
    # every active block contains a set pixel, every inactive one none (max pooling)
    act = np.zeros((N, g.bcount[0], g.bcount[1]), bool)
    act[idx_h[:nb, 0], idx_h[:nb, 1], idx_h[:nb, 2]] = True
    m = mask_h[..., 0] > 0.5
    for n in (0, N - 1):
        for bh in (0, 7, g.bcount[0] - 1):
            for bw in range(g.bcount[1]):
                win = m[n, max(16 * bh - 1, 0):16 * bh + 17, max(16 * bw - 1, 0):16 * bw + 17]
                assert act[n, bh, bw] == bool(win.any())
    p = ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=True)
    q = p[:, :, 1:17, 1:17].contiguous()
    x0 = x.clone()
    ops.sparse_scatter_var(q, cnt, idx, x, gi.bsize, gi.bstride, gi.boffset, add=True, transpose=True)
    cov = _coverage(idx_h, nb, gi, N, H, W, dev) > 0
    assert torch.equal(x[cov], x0[cov] * 2) and torch.equal(x[~cov], x0[~cov])
