"""sbnet_reduce_mask_static -- the reduce_mask entry point for callers that cannot allocate device
scratch (plug-ins inside a framework that owns all GPU memory, allocation-free sections, allocator-less
C wrappers) -- against the ordinary entry point, through the C ABI.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test.  Passes alone in a fresh process and after the rest of the suite; the scratch it
uses is shared by every call in the process, so each case makes two calls in a row and the second
must not see anything of the first.
"""
import ctypes as C

import numpy as np
import pytest

from sbnet_b200 import configs as cfg

pytestmark = pytest.mark.gpu


def _run(lib, torch, fn_static, mask_h, g, tol, avg):
    """Returns (sorted index tuples, count) from the ordinary or the static entry point."""
    dev = "cuda"
    mask = torch.from_numpy(mask_h).to(dev)
    N, H, W = mask_h.shape[:3]
    total = N * g.bcount[0] * g.bcount[1]
    idx = torch.full((total, 3), -1, dtype=torch.int16, device=dev)
    host = torch.full((1,), -5, dtype=torch.int32).pin_memory()
    stream = torch.cuda.current_stream().cuda_stream
    geom = (g.boffset[0], g.boffset[1], g.bsize[0], g.bsize[1], g.bstride[0], g.bstride[1], g.bcount[0], g.bcount[1])
    if fn_static:
        count_dev = torch.full((1,), -9, dtype=torch.int32, device=dev)
        lib.check(lib.load().sbnet_reduce_mask_static(mask.data_ptr(), N, H, W, tol, int(avg), *geom,
                                                      idx.data_ptr(), count_dev.data_ptr(), host.data_ptr(), stream))
        torch.cuda.synchronize()
        assert int(count_dev[0]) == int(host[0])
    else:
        scratch = torch.zeros(4, dtype=torch.int32, device=dev)
        lib.check(lib.load().sbnet_reduce_mask(mask.data_ptr(), N, H, W, tol, int(avg), *geom, idx.data_ptr(),
                                               scratch.data_ptr(), host.data_ptr(), 0, stream))
        torch.cuda.synchronize()
    n = int(host[0])
    return sorted(map(tuple, idx[:n].cpu().tolist())), n


def test_static_scratch_matches_ordinary_entry_point_twice_in_a_row(cuda_ops):
    import torch
    from sbnet_b200 import lib
    g = cfg.halo_geom(160, 176)
    dense = cfg.rect_union_mask(3, 160, 176, seed=5, n_rects=14)
    empty = np.zeros_like(dense)
    real = np.random.default_rng(0).standard_normal(dense.shape).astype(np.float32)
    # consecutive calls on the shared scratch: many blocks, then none, then a real-valued mask, ...
    for mask_h, tol, avg in [(dense, 0.5, False), (empty, 0.5, False), (dense, 0.1, True), (real, 0.02, True),
                             (empty, 0.1, True), (real, 1.5, False)]:
        exp, n_exp = _run(lib, torch, False, mask_h, g, tol, avg)
        for _ in range(2):                       # two calls in a row, both must agree exactly
            got, n_got = _run(lib, torch, True, mask_h, g, tol, avg)
            assert n_got == n_exp
            assert got == exp
    # the ordinary entry point still works afterwards
    exp2, n2 = _run(lib, torch, False, dense, g, 0.5, False)
    assert (exp2, n2) == _run(lib, torch, False, dense, g, 0.5, False)


def test_static_scratch_rejects_more_blocks_than_its_limit(cuda_ops):
    from sbnet_b200 import lib
    h = lib.load()
    # 32767 * 32767 * 1 candidate blocks > 2^24; rejected before anything touches the device
    rc = h.sbnet_reduce_mask_static(None, 1, 40000, 40000, 0.5, 0, 0, 0, 1, 1, 1, 1, 32767, 32767, None, None,
                                    None, None)
    assert rc == -1
    msg = h.sbnet_last_error().decode()
    assert "product" in msg and str(1 << 24) in msg
    # factors past the int16 range are refused one by one, before their product is formed
    rc = h.sbnet_reduce_mask_static(None, 2 ** 31 - 1, 8, 8, 0.5, 0, 0, 0, 1, 1, 1, 1, 2 ** 31 - 1, 2 ** 31 - 1,
                                    None, None, None, None)
    assert rc == -1 and "32767" in h.sbnet_last_error().decode()


def test_static_scratch_count_stays_on_the_device_and_feeds_a_gather(cuda_ops):
    """The stream-ordered use: no host count at all (count_host NULL), the count lands in the caller's
    device word and is read there by the device-count gather -- on a stream of the caller's own, twice
    in a row, against the ordinary entry point followed by the host-count gather."""
    import torch
    from sbnet_b200 import lib, ops
    dev = "cuda"
    g = cfg.halo_geom(160, 176)
    N, H, W, Cc = 2, 160, 176, 32
    x = torch.randn((N, H, W, Cc), device=dev)
    geom = (g.boffset[0], g.boffset[1], g.bsize[0], g.bsize[1], g.bstride[0], g.bstride[1], g.bcount[0], g.bcount[1])
    total = N * g.bcount[0] * g.bcount[1]
    side = torch.cuda.Stream()
    for seed, rects in ((11, 9), (12, 0), (13, 21)):
        mask = torch.from_numpy(cfg.rect_union_mask(N, H, W, seed=seed, n_rects=rects)).to(dev)
        idx_ref, cnt_ref = ops.reduce_mask(mask, *g.as_lists(), tol=0.5)
        n = int(cnt_ref[0])
        ref = ops.sparse_gather(x, cnt_ref, idx_ref, g.bsize, g.bstride, g.boffset, transpose=True)
        key = lambda t: (t[:, 0].long() * g.bcount[0] + t[:, 1].long()) * g.bcount[1] + t[:, 2].long()  # noqa: E731
        ref_sorted = ref[torch.argsort(key(idx_ref[:n]))]
        torch.cuda.synchronize()
        for _ in range(2):
            with torch.cuda.stream(side):
                idx = torch.full((total, 3), -1, dtype=torch.int16, device=dev)
                count_dev = torch.full((1,), -9, dtype=torch.int32, device=dev)
                out = torch.full((total, Cc, 18, 18), 7.0, device=dev)
                lib.check(lib.load().sbnet_reduce_mask_static(mask.data_ptr(), N, H, W, 0.5, 0, *geom, idx.data_ptr(),
                                                              count_dev.data_ptr(), None, side.cuda_stream))
                ops.sparse_gather_dyn(x, count_dev, total, idx, g.bsize, g.bstride, g.boffset, transpose=True, out=out)
            side.synchronize()
            assert int(count_dev[0]) == n
            assert torch.equal(out[torch.argsort(key(idx[:n]))], ref_sorted)
            assert bool((out[n:] == 7.0).all())
