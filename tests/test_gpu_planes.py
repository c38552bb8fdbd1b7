"""Plane-layout ([nB,C,R,S]) gather / scatter on the shapes the TMA pipeline takes (C*sizeof(T) a
multiple of 128 bytes, blocks of at most 384 pixels), the wider set the tile CTAs take (partial
channel chunks, blocks of any size cut into pixel chunks) and shapes outside both, against the CPU
checker; the general kernels are run on the same inputs by switching the others off."""

import numpy as np
import pytest

from sbnet_b200 import configs as cfg
from atomic_check import check_atomic_add

pytestmark = pytest.mark.gpu

# (dtype, N, H, W, C, bsize, bstride, boffset)
SHAPES = [
    (np.float16, 2, 64, 48, 64, (18, 18), (16, 16), (-1, -1)),
    (np.float16, 2, 64, 48, 256, (18, 18), (16, 16), (-1, -1)),
    (np.float16, 1, 40, 40, 128, (16, 16), (16, 16), (0, 0)),
    (np.float16, 3, 33, 29, 64, (6, 5), (4, 3), (-2, -3)),      # 30 pixels, all four borders
    (np.float16, 1, 50, 50, 64, (19, 20), (7, 9), (-5, -4)),    # 380 pixels
    (np.float16, 1, 50, 50, 64, (5, 5), (5, 5), (0, 0)),        # odd pixel count: rows of an odd number of halves
    (np.float16, 2, 64, 48, 128, (17, 17), (15, 15), (-1, -1)), # 289 pixels, overlapping
    (np.float16, 1, 60, 60, 40, (19, 19), (19, 19), (-9, -9)),  # 361 pixels, partial channel chunk
    (np.float16, 1, 37, 41, 64, (7, 3), (5, 3), (-3, -1)),      # 21 pixels
    (np.float16, 1, 9, 400, 64, (1, 383), (1, 383), (0, 5)),    # the largest odd block of one tile
    (np.float16, 1, 64, 64, 64, (20, 20), (16, 16), (-2, -2)),  # 400 pixels: two pixel chunks
    (np.float32, 2, 64, 48, 32, (18, 18), (16, 16), (-1, -1)),
    (np.float32, 2, 64, 48, 128, (18, 18), (16, 16), (-1, -1)),
    (np.float32, 1, 37, 41, 64, (7, 3), (5, 3), (-3, -1)),      # 21 pixels (odd is fine for fp32)
    (np.float32, 1, 50, 50, 32, (19, 20), (19, 20), (-9, -9)),
    (np.float32, 1, 20, 20, 32, (1, 1), (1, 1), (0, 0)),
    # plane rows a multiple of 32 words: the swizzled scatter tile
    (np.float32, 2, 40, 56, 64, (16, 16), (16, 16), (0, 0)),
    (np.float32, 1, 30, 30, 32, (8, 8), (5, 6), (-3, -2)),
    (np.float16, 1, 30, 30, 128, (8, 8), (8, 8), (-3, -2)),
    (np.float16, 2, 64, 48, 256, (16, 16), (16, 16), (0, 0)),
    (np.float16, 1, 50, 70, 64, (16, 24), (11, 13), (-7, -9)),   # 384 pixels, overlapping
    # pixels that are not a multiple of 128 bytes: the last channel chunk is partial (tile CTAs only)
    (np.float32, 2, 40, 56, 48, (18, 18), (16, 16), (-1, -1)),
    (np.float32, 1, 30, 30, 12, (8, 8), (8, 8), (0, 0)),
    (np.float16, 1, 30, 30, 24, (6, 6), (5, 5), (-1, -1)),
    (np.float16, 2, 64, 48, 200, (16, 16), (16, 16), (0, 0)),
    (np.float16, 1, 40, 40, 40, (18, 18), (16, 16), (-1, -1)),
    # blocks of more than 384 pixels: pixel chunks in the tile CTAs
    (np.float16, 1, 100, 90, 64, (34, 34), (32, 32), (-1, -1)),   # rows of 578 words: 8-byte copy-in, word stores
    (np.float32, 1, 100, 90, 32, (34, 34), (32, 32), (-1, -1)),   # rows of 1156 words: 16-byte aligned
    (np.float32, 1, 70, 70, 32, (21, 21), (21, 21), (-3, -3)),    # 441 pixels (odd): gather chunks, general scatter
    (np.float32, 2, 80, 70, 48, (27, 22), (20, 17), (-5, -4)),    # 594 pixels, overlapping, partial channel chunk
    (np.float16, 1, 130, 150, 128, (41, 48), (41, 48), (0, 0)),   # 1968 pixels: six chunks of 328
    (np.float16, 2, 140, 130, 40, (64, 64), (61, 59), (-9, -7)),  # 4096 pixels, partial channel chunk
    (np.float16, 1, 170, 170, 64, (81, 81), (81, 81), (-4, -4)),  # 6561 pixels (odd), fp16: gather chunks shift odd rows
    (np.float16, 2, 70, 70, 128, (21, 21), (19, 19), (-1, -1)),   # 441 pixels (odd), overlapping: chunks of 224 + 217
    (np.float16, 1, 80, 70, 40, (25, 19), (25, 19), (-3, -3)),    # 475 pixels (odd), partial channel chunk
    (np.float32, 1, 170, 170, 16, (81, 81), (70, 70), (-4, -4)),  # 6561 pixels (odd), fp32 gather chunks
]


def _ids():
    return [f"{np.dtype(s[0]).name}_C{s[4]}_b{s[5][0]}x{s[5][1]}_s{s[6][0]}x{s[6][1]}" for s in SHAPES]


@pytest.fixture(params=["default", "tma_tile", "tile_ctas", "tma_pipeline", "general", "general_elementwise",
                        "general_raw_rows_narrow"])
def tma_off(request):
    """Selects which plane-layout implementation takes the call: the default dispatch (which sends
    launches as small as these tests' gathers to the TMA pipeline where the shape allows), the tile CTAs
    fed by TMA whatever the launch size, the tile CTAs with plain loads, the persistent TMA pipeline, or the
    general kernels (whole rows as raw bytes; element-wise; raw rows with element-wide stack accesses)."""
    from conftest import library_options
    planes = {"default": 0, "general": 0, "tma_pipeline": 1, "tile_ctas": 2, "tma_tile": 3, "general_elementwise": 4,
              "general_raw_rows_narrow": 6}[request.param]
    with library_options(planes=planes, disable_tma=int(request.param.startswith("general")), tile_blocks=0):
        yield request.param


@pytest.mark.parametrize("shape", SHAPES, ids=_ids())
def test_planes_gather_and_scatter(cuda_ops, oracle_port, tma_off, shape):
    _run_shape(cuda_ops, oracle_port, shape)


def _run_shape(cuda_ops, oracle_port, shape):
    dtype, N, H, W, C, bsize, bstride, boffset = shape
    g = cfg.geom_for(H, W, bsize, bstride, boffset)
    idx, cnt = cfg.random_block_list(N, g.bcount, 0.6, seed=C + bsize[0])
    nb = int(cnt[0])
    x = cfg.normal((N, H, W, C), 3, dtype)
    exp = oracle_port.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=True)
    got = cuda_ops.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=True)
    np.testing.assert_array_equal(got, exp)

    stack = cfg.normal((nb, C, bsize[0], bsize[1]), 4, dtype)
    base = cfg.normal((N, H, W, C), 5, dtype)
    disjoint = bstride[0] >= bsize[0] and bstride[1] >= bsize[1]
    # overwrite: with overlapping blocks the winner is schedule dependent unless the values agree,
    # so overlapping layouts scatter a gathered stack (all copies of a pixel are equal)
    src = stack if disjoint else exp
    e = oracle_port.sparse_scatter_var(src, cnt, idx, base.copy(), bsize, bstride, boffset, add=False,
                                       transpose=True)
    o = cuda_ops.sparse_scatter_var(src, cnt, idx, base.copy(), bsize, bstride, boffset, add=False,
                                    transpose=True)
    np.testing.assert_array_equal(o, e)
    if disjoint:
        e = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset,
                                           add=True, transpose=True)
        o = cuda_ops.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset,
                                        add=True, transpose=True)
        np.testing.assert_array_equal(o, e)
    e = oracle_port.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                       atomic=True, transpose=True)
    o = cuda_ops.sparse_scatter_var(stack, cnt, idx, base.copy(), bsize, bstride, boffset, add=True,
                                    atomic=True, transpose=True)
    # both results within k rounded additions of the fp64 sum; relative bars where nothing cancels
    check_atomic_add({"cuda": o, "cpu checker": e}, stack, cnt, idx, base, bsize, bstride, boffset, True)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_device_count_calls_on_blocks_above_384_pixels(cuda_ops, dtype):
    """The ``*_dyn`` entry points (block count read on the device) against the host-count calls on
    34x34 blocks: the scatter runs the pixel-chunked tile kernel as one resident wave, the gather the
    general kernel."""
    import torch
    from sbnet_b200 import ops
    N, H, W, C = 2, 100, 90, 64
    bsize, bstride, boffset = (34, 34), (32, 32), (-1, -1)
    g = cfg.geom_for(H, W, bsize, bstride, boffset)
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, 0.7, seed=5)
    nb, max_blocks = int(cnt_h[0]), idx_h.shape[0]
    dev = torch.device("cuda:0")
    idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
    cnt_dev = cnt.to(dev)
    x = torch.from_numpy(cfg.normal((N, H, W, C), 21, dtype)).to(dev)
    ref = ops.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=True)
    out = torch.full((max_blocks, C, 34, 34), -3.0, dtype=x.dtype, device=dev)
    ops.sparse_gather_dyn(x, cnt_dev, max_blocks, idx, bsize, bstride, boffset, transpose=True, out=out)
    torch.cuda.synchronize()
    assert torch.equal(out[:nb], ref) and bool((out[nb:] == -3.0).all())
    base = torch.from_numpy(cfg.normal((N, H, W, C), 22, dtype)).to(dev)
    for add, atomic in ((False, False), (True, True)):
        src = ref if not add else torch.from_numpy(cfg.normal(tuple(ref.shape), 23, dtype)).to(dev)
        full = torch.cat([src, torch.full((max_blocks - nb, C, 34, 34), float("nan"), dtype=x.dtype, device=dev)])
        y1 = ops.sparse_scatter_var_dyn(full, cnt_dev, max_blocks, idx, base.clone(), bsize, bstride, boffset,
                                        add=add, atomic=atomic, transpose=True)
        y2 = ops.sparse_scatter_var(src, cnt, idx, base.clone(), bsize, bstride, boffset, add=add, atomic=atomic,
                                    transpose=True)
        torch.cuda.synchronize()
        if add:   # overlapping halos: arrival order differs between the two runs
            check_atomic_add({"device count": y1, "host count": y2}, src, cnt_h, idx_h, base, bsize, bstride, boffset, True)
        else:
            assert torch.equal(y1, y2)


# Small blocks: several whole blocks share one tile of the tile CTAs.
SMALL_BLOCKS = [
    (np.float16, 2, 40, 40, 64, (6, 6), (4, 4), (-1, -1)),      # 36 pixels, overlapping
    (np.float16, 1, 33, 29, 200, (4, 6), (4, 6), (0, 0)),       # 24 pixels, partial last channel chunk
    (np.float32, 2, 40, 40, 32, (5, 5), (3, 3), (-1, -1)),      # 25 pixels: rows of an odd number of words
    (np.float32, 1, 50, 50, 48, (8, 8), (8, 8), (0, 0)),        # 64 pixels, partial last channel chunk
    (np.float16, 1, 50, 50, 128, (10, 10), (8, 8), (-1, -1)),   # rows of 50 words: 8-byte copy-in
    (np.float32, 1, 30, 30, 32, (1, 1), (1, 1), (0, 0)),        # one pixel per block
    (np.float32, 1, 64, 64, 32, (12, 16), (12, 16), (0, 0)),    # 192 pixels: two blocks per tile
    (np.float16, 1, 64, 64, 64, (2, 1), (2, 1), (0, 0)),        # two pixels per block
    # fp16, odd pixel counts: the gather pairs pixels inside each block
    (np.float16, 2, 40, 40, 64, (5, 5), (3, 3), (-1, -1)),
    (np.float16, 1, 33, 29, 200, (3, 3), (3, 3), (0, 0)),
    (np.float16, 1, 30, 30, 64, (1, 1), (1, 1), (0, 0)),
    (np.float16, 1, 64, 64, 32, (13, 13), (11, 11), (-1, -1)),  # 169 pixels: two blocks per tile
]


@pytest.mark.parametrize("gather_loads", ["plain", "tma"])
@pytest.mark.parametrize("blocks_per_tile", ["2", "7", "1000"])
@pytest.mark.parametrize("shape", SMALL_BLOCKS,
                         ids=[f"{np.dtype(s[0]).name}_C{s[4]}_b{s[5][0]}x{s[5][1]}" for s in SMALL_BLOCKS])
def test_several_blocks_per_tile(cuda_ops, oracle_port, shape, blocks_per_tile, gather_loads):
    """``plain``: the plain-load kernels of the tile CTAs; ``tma``: the default dispatch, whose gather
    feeds the shared tile with one TMA load per block where it can."""
    from conftest import library_options
    with library_options(tile_blocks=int(blocks_per_tile), planes=2 if gather_loads == "plain" else 3, disable_tma=0):
        _run_shape(cuda_ops, oracle_port, shape)


def test_several_blocks_per_tile_chosen_by_launch_size(cuda_ops, oracle_port):
    """Enough 8x8 blocks that the dispatcher packs several per tile on its own; also through the
    device-count scatter."""
    import torch
    from sbnet_b200 import ops
    _run_shape(cuda_ops, oracle_port, (np.float16, 2, 256, 256, 64, (8, 8), (6, 6), (-1, -1)))
    N, H, W, C = 2, 256, 256, 64
    bsize, bstride, boffset = (8, 8), (8, 8), (0, 0)
    g = cfg.geom_for(H, W, bsize, bstride, boffset)
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, 0.8, seed=9)
    nb, max_blocks = int(cnt_h[0]), idx_h.shape[0]
    dev = torch.device("cuda:0")
    idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
    stack = torch.from_numpy(cfg.normal((max_blocks, C, 8, 8), 31, np.float32)).to(dev)
    base = torch.from_numpy(cfg.normal((N, H, W, C), 32, np.float32)).to(dev)
    y1 = ops.sparse_scatter_var_dyn(stack, cnt.to(dev), max_blocks, idx, base.clone(), bsize, bstride, boffset,
                                    add=True, transpose=True)
    y2 = ops.sparse_scatter_var(stack[:nb].contiguous(), cnt, idx, base.clone(), bsize, bstride, boffset, add=True,
                                transpose=True)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    exp = oracle_port.sparse_scatter_var(stack[:nb].cpu().numpy(), cnt_h, idx_h, base.cpu().numpy(), bsize, bstride,
                                         boffset, add=True, transpose=True)
    np.testing.assert_array_equal(y2.cpu().numpy(), exp)


@pytest.mark.parametrize("case", [
    (np.float16, 40, (8, 8), (6, 6), (-1, -1)),      # several blocks per tile
    (np.float32, 24, (18, 18), (16, 16), (-1, -1)),  # one block per tile, partial channel chunk
    (np.float16, 72, (17, 17), (15, 15), (-1, -1)),  # odd pixel count
    (np.float32, 32, (40, 30), (40, 30), (0, 0)),    # row chunks
], ids=["shared_tile", "one_block", "odd_pixels", "row_chunks"])
def test_device_count_gather_outside_the_pipeline(cuda_ops, case):
    """Gathers with the block count on the device whose pixels are not 128-byte multiples (or whose
    blocks exceed one tile): the TMA-fed tile kernels run over a grid sized for every candidate block
    and the surplus CTAs leave at once.  Compared with the host-count call; rows past the count stay
    untouched."""
    import torch
    from sbnet_b200 import ops
    from cuda_ops import to_torch
    dtype, C, bsize, bstride, boffset = case
    N, H, W = 2, 128, 120
    g = cfg.geom_for(H, W, bsize, bstride, boffset)
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, 0.4, seed=C)
    nb, max_blocks = int(cnt_h[0]), idx_h.shape[0]
    dev = torch.device("cuda:0")
    idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
    x = to_torch(cfg.normal((N, H, W, C), 41, dtype)).to(dev)
    ref = ops.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=True)
    out = torch.full((max_blocks, C, *bsize), -3.0, dtype=x.dtype, device=dev)
    ops.sparse_gather_dyn(x, cnt.to(dev), max_blocks, idx, bsize, bstride, boffset, transpose=True, out=out)
    torch.cuda.synchronize()
    assert torch.equal(out[:nb], ref)
    assert bool((out[nb:] == -3.0).all())


def test_no_bounded_wait_gave_up(cuda_ops):
    import torch
    from sbnet_b200 import lib
    torch.cuda.synchronize()
    assert lib.wait_timeouts() == 0


def test_shared_memory_limit_is_consistent_across_host_threads(cuda_ops):
    """A kernel's dynamic shared-memory limit belongs to the function, not to the calling thread: a small
    launch of the same kernel from a second host thread (as an autograd engine's backward pass makes)
    must not lower the limit under a later large launch from the first."""
    import threading
    import torch
    from conftest import library_options
    from sbnet_b200 import ops
    dev = "cuda"
    x = torch.randn((2, 64, 64, 32), device=dev)            # fp32, 128-byte pixels: the TMA pipeline's shape
    big = cfg.halo_geom(64, 64)                             # 18x18 blocks: ~205 KB of stages
    small = cfg.geom_for(64, 64, (3, 3), (3, 3), (0, 0))    # 3x3 blocks: a few KB
    lists = {k: cfg.random_block_list(2, g.bcount, 0.6, seed=3) for k, g in (("big", big), ("small", small))}

    def gather(kind):
        g = big if kind == "big" else small
        idx_h, cnt_h = lists[kind]
        out = ops.sparse_gather(x, torch.from_numpy(cnt_h), torch.from_numpy(idx_h).to(dev), g.bsize, g.bstride,
                                g.boffset, transpose=True)
        torch.cuda.synchronize()
        return out

    with library_options(planes=1):                         # the persistent pipeline, whatever the launch size
        ref_big, ref_small = gather("big").clone(), gather("small").clone()
        result = {}
        t = threading.Thread(target=lambda: result.update(small=gather("small")))
        t.start()
        t.join()
        assert torch.equal(result["small"], ref_small)
        assert torch.equal(gather("big"), ref_big)          # failed with "invalid argument" when limits were cached per thread


@pytest.mark.parametrize("transpose", [True, False], ids=["planes", "rows"])
@pytest.mark.parametrize("dtype,C", [(np.float32, 5), (np.float16, 6), (np.float16, 7)])
def test_device_count_calls_on_general_shapes_loop_over_items(cuda_ops, dtype, C, transpose):
    """Pixels that are not a multiple of 16 bytes with the block count on the device: the raw-row kernel runs as
    one resident wave whose CTAs each take several blocks in turn (4,000 blocks on about 1,200 CTAs), reusing
    their row buffers and their barrier.  Every mode must give what the host-count call (one CTA per block) gives."""
    import torch
    from sbnet_b200 import ops
    N, H, W = 4, 256, 256
    bsize, bstride, boffset = (6, 6), (6, 6), (-2, -3)
    g = cfg.geom_for(H, W, bsize, bstride, boffset)
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, 0.6, seed=15)
    nb, max_blocks = int(cnt_h[0]), idx_h.shape[0]
    assert nb > 3000
    dev = torch.device("cuda:0")
    idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
    cnt_dev = cnt.to(dev)
    x = torch.from_numpy(cfg.normal((N, H, W, C), 31, dtype)).to(dev)
    ref = ops.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=transpose)
    out = torch.full((max_blocks, C, 6, 6) if transpose else (max_blocks, 6, 6, C), -3.0, dtype=x.dtype, device=dev)
    ops.sparse_gather_dyn(x, cnt_dev, max_blocks, idx, bsize, bstride, boffset, transpose=transpose, out=out)
    torch.cuda.synchronize()
    assert torch.equal(out[:nb], ref) and bool((out[nb:] == -3.0).all())
    base = torch.from_numpy(cfg.normal((N, H, W, C), 32, dtype)).to(dev)
    src = torch.from_numpy(cfg.normal(tuple(ref.shape), 33, dtype)).to(dev)
    full = torch.cat([src, torch.full((max_blocks - nb,) + tuple(ref.shape[1:]), float("nan"), dtype=x.dtype, device=dev)])
    for add, atomic in ((False, False), (True, False), (True, True)):      # the blocks do not overlap: all bit-exact
        y1 = ops.sparse_scatter_var_dyn(full, cnt_dev, max_blocks, idx, base.clone(), bsize, bstride, boffset,
                                        add=add, atomic=atomic, transpose=transpose)
        y2 = ops.sparse_scatter_var(src, cnt, idx, base.clone(), bsize, bstride, boffset, add=add, atomic=atomic,
                                    transpose=transpose)
        torch.cuda.synchronize()
        assert torch.equal(y1, y2), (add, atomic)
    from sbnet_b200 import lib
    assert lib.wait_timeouts() == 0


def _carve(torch, shape, dtype, dev, lead, fill):
    """A contiguous tensor of ``shape`` that starts ``lead`` elements into a larger buffer (so its address is
    element-aligned only), and the buffer, pre-filled with ``fill`` as a guard band on both sides."""
    n = int(np.prod(shape))
    buf = torch.full((n + lead + 37,), fill, dtype=dtype, device=dev)
    return buf[lead:lead + n].view(*shape), buf


@pytest.mark.parametrize("transpose", [False, True], ids=["rows", "planes"])
@pytest.mark.parametrize("dtype,C,lead_x,lead_s", [(np.float32, 8, 1, 3), (np.float32, 33, 3, 1), (np.float16, 100, 1, 5),
                                                   (np.float16, 64, 7, 2), (np.float16, 9, 3, 3)])
def test_buffers_aligned_to_an_element_only(cuda_ops, dtype, C, lead_x, lead_s, transpose):
    """Image and stack that start at odd element offsets of their allocations (views into larger buffers): same
    results as on aligned copies, and nothing written outside the views (guard bands on both sides)."""
    import torch
    from sbnet_b200 import ops
    dev = torch.device("cuda:0")
    N, H, W = 2, 50, 44
    bsize, bstride, boffset = (10, 12), (10, 12), (-3, -5)      # blocks do not overlap; they hang over every border
    g = cfg.geom_for(H, W, bsize, bstride, boffset)
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, 0.8, seed=3)
    nb = int(cnt_h[0])
    idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
    tdt = torch.float32 if dtype == np.float32 else torch.float16
    x_al = torch.from_numpy(cfg.normal((N, H, W, C), 41, dtype)).to(dev)
    sshape = (nb, C, *bsize) if transpose else (nb, *bsize, C)
    s_al = torch.from_numpy(cfg.normal(sshape, 42, dtype)).to(dev)
    x, xbuf = _carve(torch, (N, H, W, C), tdt, dev, lead_x, 77.0)
    x.copy_(x_al)
    s, sbuf = _carve(torch, sshape, tdt, dev, lead_s, 55.0)
    assert x.data_ptr() % 16 != 0 and s.data_ptr() % 16 != 0

    def guards_intact(buf, lead, n, fill):
        return bool((buf[:lead] == fill).all()) and bool((buf[lead + n:] == fill).all())

    ref = ops.sparse_gather(x_al, cnt, idx, bsize, bstride, boffset, transpose=transpose)
    ops.sparse_gather(x, cnt, idx, bsize, bstride, boffset, transpose=transpose, out=s)
    torch.cuda.synchronize()
    assert torch.equal(s, ref)
    assert guards_intact(sbuf, lead_s, s.numel(), 55.0)
    s.copy_(s_al)
    for add, atomic in ((False, False), (True, False), (True, True)):
        y_ref = ops.sparse_scatter_var(s_al, cnt, idx, x_al.clone(), bsize, bstride, boffset, add=add, atomic=atomic,
                                       transpose=transpose)
        x.copy_(x_al)
        y = ops.sparse_scatter_var(s, cnt, idx, x, bsize, bstride, boffset, add=add, atomic=atomic, transpose=transpose)
        torch.cuda.synchronize()
        assert y.data_ptr() == x.data_ptr()
        assert torch.equal(y, y_ref), (add, atomic)
        assert guards_intact(xbuf, lead_x, x.numel(), 77.0), (add, atomic)
