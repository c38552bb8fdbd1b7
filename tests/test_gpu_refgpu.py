"""Second parity authority: the reference's OWN CUDA kernels (sbnet_ops/sparse_blocks.cu.h,
sbnet_ops/reduce_mask.cu.h), recompiled for sm_100a by ``make -C oracle refgpu``, run on the same
device and the same inputs as this library's kernels.  fp32 only, as in the reference.

gather and overwrite / non-overlapping add scatter: bit-exact.  Atomic add over overlapping blocks:
1e-6 relative per addend (arrival order differs between any two runs).  reduce_mask: equal as sets
(both compact in arrival order)."""
import numpy as np
import pytest

from sbnet_b200 import configs as cfg

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def refgpu():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import refgpu as r
    if not r.available():
        try:
            r.build()
        except Exception:
            pass
    if not r.available():
        pytest.skip("reference CUDA kernels not built (no reference tree and no prebuilt library)")
    return r


# (N, H, W, C, bsize, bstride, boffset): 16x16 and 18x18 take the reference's compile-time kernels,
# the others its run-time-size kernels
SHAPES = [
    (2, 64, 64, 32, (10, 10), (8, 8), (-1, -1)),
    (2, 96, 80, 64, (18, 18), (16, 16), (-1, -1)),
    (2, 96, 80, 128, (16, 16), (16, 16), (0, 0)),
    (1, 50, 45, 40, (18, 18), (16, 16), (-1, -1)),     # 40 channels: tail channel tile
    (3, 33, 29, 7, (6, 5), (4, 3), (-2, -3)),
    (1, 70, 70, 20, (35, 37), (30, 30), (-3, -4)),     # blocks above 1,024 pixels
]


@pytest.mark.parametrize("shape", SHAPES, ids=[f"C{s[3]}_b{s[4][0]}x{s[4][1]}" for s in SHAPES])
@pytest.mark.parametrize("transpose", [False, True])
def test_gather_scatter_match_reference_kernels(cuda_ops, refgpu, shape, transpose):
    import torch
    from sbnet_b200 import ops
    N, H, W, C, bsize, bstride, boffset = shape
    dev = torch.device("cuda:0")
    g = cfg.geom_for(H, W, bsize, bstride, boffset)
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, 0.6, seed=C)
    nb = int(cnt_h[0])
    idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
    x = torch.from_numpy(cfg.normal((N, H, W, C), 11, np.float32)).to(dev)
    shp = (nb, C, bsize[0], bsize[1]) if transpose else (nb, bsize[0], bsize[1], C)

    ours = ops.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=transpose)
    ref = refgpu.sparse_gather(x, nb, idx, bsize, bstride, boffset, transpose,
                               torch.full(shp, float("nan"), device=dev))
    torch.cuda.synchronize()
    assert torch.equal(ours.view(torch.int32), ref.view(torch.int32))

    stack = torch.from_numpy(cfg.normal(shp, 12, np.float32)).to(dev)
    base = torch.from_numpy(cfg.normal((N, H, W, C), 13, np.float32)).to(dev)
    disjoint = bstride[0] >= bsize[0] and bstride[1] >= bsize[1]
    src = stack if disjoint else ours   # overlapping overwrite: every copy of a pixel must agree
    a = ops.sparse_scatter_var(src, cnt, idx, base.clone(), bsize, bstride, boffset, add=False,
                               transpose=transpose)
    b = refgpu.sparse_scatter_var(src, nb, idx, base.clone(), bsize, bstride, boffset, add=False,
                                  transpose=transpose)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    if disjoint:
        a = ops.sparse_scatter_var(stack, cnt, idx, base.clone(), bsize, bstride, boffset, add=True,
                                   transpose=transpose)
        b = refgpu.sparse_scatter_var(stack, nb, idx, base.clone(), bsize, bstride, boffset, add=True,
                                      transpose=transpose)
        torch.cuda.synchronize()
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    a = ops.sparse_scatter_var(stack, cnt, idx, base.clone(), bsize, bstride, boffset, add=True, atomic=True,
                               transpose=transpose)
    b = refgpu.sparse_scatter_var(stack, nb, idx, base.clone(), bsize, bstride, boffset, add=True,
                                  atomic=True, transpose=transpose)
    torch.cuda.synchronize()
    from atomic_check import check_atomic_add
    check_atomic_add({"this library": a, "reference kernels": b}, stack, [nb], idx, base, bsize, bstride, boffset,
                     transpose)


# avg thresholds sit between attainable block averages: the reference kernel divides with -use_fast_math
@pytest.mark.parametrize("avgpool,tol", [(False, 0.5), (True, 0.105), (True, 0.305)])
def test_reduce_mask_matches_reference_kernel(cuda_ops, refgpu, avgpool, tol):
    import torch
    from sbnet_b200 import ops
    dev = torch.device("cuda:0")
    for (N, H, W, bsize, bstride, boffset, seed) in [
        (2, 64, 64, (10, 10), (8, 8), (-1, -1), 1),
        (3, 200, 176, (18, 18), (16, 16), (-1, -1), 2),
        (1, 90, 110, (35, 37), (30, 30), (-3, -4), 3),   # more pixels than threads in the reference CTA
    ]:
        if avgpool and bsize[0] * bsize[1] > 1024:
            # sbnet_ops/reduce_mask.cu.h:84-113 keeps each lane's running sum across its 1,024-thread
            # passes, so earlier partial sums are counted again: on blocks above 1,024 pixels the
            # reference kernel's average is not the CPU functor's (the authority).  Max is unaffected.
            continue
        g = cfg.geom_for(H, W, bsize, bstride, boffset)
        mask = torch.from_numpy(cfg.rect_union_mask(N, H, W, seed, n_rects=12)).to(dev)
        idx, cnt = ops.reduce_mask(mask, g.bcount, bsize, bstride, boffset, tol=tol, avgpool=avgpool)
        nb = int(cnt[0])
        ridx = torch.zeros((N * g.bcount[0] * g.bcount[1], 3), dtype=torch.int16, device=dev)
        rcnt = torch.zeros(1, dtype=torch.int32, device=dev)
        refgpu.reduce_mask_launch(mask, g.bcount, bsize, bstride, boffset, tol, avgpool, ridx, rcnt)
        torch.cuda.synchronize()
        rn = int(rcnt.item())
        assert rn >= 1, "the case is meant to have active blocks"
        assert nb == rn
        ours = {tuple(r) for r in idx[:nb].cpu().numpy().tolist()}
        ref = {tuple(r) for r in ridx[:rn].cpu().numpy().tolist()}
        assert ours == ref
