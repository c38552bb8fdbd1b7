"""Op-level measurements behind ``bench.py --suite ops``: one JSON line per case.

Cases are the op-level benchmark configurations: reduce_mask on a bird's-eye-view sized mask
([8,800,704], avg and max pooling), sparse_gather on x [8,512,512,128] (fp32 / fp16, both layouts,
5 / 20 / 50 % active blocks) and sparse_scatter[_var] (fp32 atomic add with overlapping halos onto
[8,512,512,64]; fp16 transposed overwrite).  Every launch is timed on its own with CUDA events on the
launching stream after an L2 flush (a 256 MiB fill), so small cases are measured from DRAM; the
median is reported with the algorithmic bytes of the call and the fraction of the HBM peak.
"""
from __future__ import annotations

import json
import statistics

import numpy as np

from . import configs as cfg


def _peak():
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class Timer:
    def __init__(self, torch, dev, steps, warmup):
        self.t, self.dev, self.steps, self.warmup = torch, dev, steps, warmup
        self.flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def run(self, fn, flush=True):
        t = self.t
        for _ in range(self.warmup):
            fn()
        t.cuda.synchronize()
        pairs = []
        for _ in range(self.steps):
            if flush:   # two fills: evicts L2 and keeps the device busy while the host queues the launch
                self.flush_buf.fill_(1)
                self.flush_buf.fill_(2)
            a, b = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            pairs.append((a, b))
        t.cuda.synchronize()
        ms = [a.elapsed_time(b) for a, b in pairs]
        return statistics.median(ms), min(ms)


def emit(name, med_ms, min_ms, nbytes, extra):
    peak, kind = _peak()
    gbs = nbytes / (med_ms * 1e-3) / 1e9
    line = {"case": name, "us": med_ms * 1e3, "us_min": min_ms * 1e3, "algorithmic_bytes": int(nbytes),
            "GB/s": gbs, "frac_of_" + kind: gbs / peak, "peak_GB/s": peak}
    line.update(extra)
    print(json.dumps(line), flush=True)


def one(args):
    """``bench.py --suite one --case NAME [--density D] [--one-channels C] [--one-block SIZE,STRIDE,OFFSET]``: a few launches of ONE op on a mid-sized
    input (larger than L2, well under a GB), for profiler captures.  Prints one JSON line."""
    import torch
    from . import build, ops
    build.build_library()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tm = Timer(torch, dev, max(args.steps, 3), 3)
    name, dens = args.case, args.density
    N, H, W = 8, 512, 512
    if name.startswith("reduce_mask"):
        c2 = cfg.config2(0)
        g = c2["geom"]
        m = torch.from_numpy(c2["mask"]).to(dev)
        avg = name.endswith("avg")
        fn = lambda: ops.reduce_mask_async(m, *g.as_lists(), tol=0.1 if avg else 0.5, avgpool=avg)  # noqa: E731
        nbytes = m.numel() * 4
    else:
        kind, tname, layout = name.split("_")[:3]           # gather_f16_t1, scatter_f32_t0_atomic ...
        mode = name.split("_")[3] if kind == "scatter" else None
        dtype = torch.float16 if tname == "f16" else torch.float32
        tr = layout == "t1"
        C = args.one_channels or (128 if kind == "gather" else 64)
        halo = kind == "gather" or mode == "atomic"
        g = cfg.halo_geom(H, W) if halo else cfg.inner_geom(H, W)
        if getattr(args, "one_block", None):   # --one-block SIZE,STRIDE,OFFSET: square blocks of another geometry
            b, stride, off = (int(v) for v in args.one_block.split(","))
            g = cfg.geom_for(H, W, (b, b), (stride, stride), (off, off))
        idx_h, cnt_h = cfg.random_block_list(N, g.bcount, dens, seed=11)
        nb = int(cnt_h[0])
        U = cfg.union_pixels(idx_h, nb, g, N, H, W)
        idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
        x = torch.randn((N, H, W, C), device=dev).to(dtype)
        shape = (nb, C, *g.bsize) if tr else (nb, *g.bsize, C)
        st = torch.randn(shape, device=dev).to(dtype)
        if kind == "gather":
            fn = lambda: ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=tr, out=st)  # noqa: E731
            nbytes = cfg.algorithmic_bytes("gather", nB=nb, geom=g, C=C, itemsize=x.element_size(), U=U)
        else:
            add, atomic = mode in ("add", "atomic"), mode == "atomic"
            fn = lambda: ops.sparse_scatter_var(st, cnt, idx, x, g.bsize, g.bstride, g.boffset, add=add,  # noqa: E731
                                                atomic=atomic, transpose=tr)
            nbytes = cfg.algorithmic_bytes("scatter_add" if add else "scatter", nB=nb, geom=g, C=C,
                                           itemsize=x.element_size(), U=U)
    med, mn = tm.run(fn, flush=True)
    emit(name, med, mn, nbytes, {"density": dens})


def resblock(args):
    """``bench.py --suite resblock``: the full sparse bottleneck (x fp16 [batch,400,352,256], 1x1 256->64,
    3x3 VALID 64->64, 1x1 64->256 by torch / cuDNN between gather and scatter) with the share of the
    block ops in the block time.  The convolutions are the host framework's, identical whichever op
    library is used; they are reported, not optimised here."""
    import torch
    from . import build, ops
    from .resblock import SparseBottleneck
    build.build_library()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    N, H, W, C = args.batch, args.height, args.width, args.channels
    m = SparseBottleneck(C, C // 4, dtype=torch.float16).eval()
    x = torch.randn((N, H, W, C), device=dev, dtype=torch.float32).half() if N * H * W * C < 2 ** 29 else None
    if x is None:
        x = torch.empty((N, H, W, C), device=dev, dtype=torch.float16)
        for n in range(N):
            x[n] = torch.randn((H, W, C), device=dev).half()
    mask = torch.from_numpy(cfg.rect_union_mask(N, H, W, seed=7, occupancy=args.occupancy)).to(dev)
    bp = m.block_params(x.shape)
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    rows = []
    with torch.no_grad():
        for it in range(args.warmup + args.steps):
            e = [ev() for _ in range(5)]
            e[0].record()
            idx, cnt = ops.reduce_mask(mask, bp.bcount, bp.bsize, bp.bstrides, bp.boffset, tol=0.5)
            e[1].record()
            p = ops.sparse_gather(x, cnt, idx, bp.bsize, bp.bstrides, bp.boffset, transpose=True)
            e[2].record()
            q = m.residual(p).contiguous()
            e[3].record()
            ops.sparse_scatter_var(q, cnt, idx, x, bp.bsize_out, bp.bsize_out, [0, 0], add=True, transpose=True)
            e[4].record()
            torch.cuda.synchronize()
            if it >= args.warmup:
                rows.append([e[i].elapsed_time(e[i + 1]) for i in range(4)])
            del p, q
    med = [statistics.median(r[i] for r in rows) for i in range(4)]
    total = sum(med)
    nb = int(cnt[0])
    print(json.dumps({"case": "sparse_bottleneck_block", "x": [N, H, W, C], "occupancy": args.occupancy,
                      "active_blocks": nb, "ms": {"reduce_mask": med[0], "gather": med[1], "convs_bn_relu": med[2],
                                                  "scatter": med[3], "total": total},
                      "block_ops_share_of_block_time": (med[0] + med[1] + med[3]) / total,
                      "blocks/s": nb / (total * 1e-3)}), flush=True)


def main(args):
    import torch
    from . import build, ops
    if getattr(args, "suite", None) == "one":
        return one(args)
    if getattr(args, "suite", None) == "resblock":
        return resblock(args)
    build.build_library()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tm = Timer(torch, dev, max(args.steps, 5), max(args.warmup, 3))

    # ---- reduce_mask, bird's-eye-view scale ----
    c2 = cfg.config2(0)
    g = c2["geom"]
    masks = [torch.from_numpy(c2["mask"]).to(dev) for _ in range(8)]
    occ = float(c2["mask"].mean())
    for run in c2["runs"]:
        idx, cnt = ops.reduce_mask(masks[0], *g.as_lists(), tol=run["tol"], avgpool=run["avgpool"])
        nb = int(cnt[0])
        nbytes = cfg.algorithmic_bytes("reduce_mask", nB=nb, geom=g, C=1, itemsize=4, U=0, N=8, H=800,
                                       W=704, count=nb)
        tag = "avg" if run["avgpool"] else "max"
        med, mn = tm.run(lambda: ops.reduce_mask_async(masks[0], *g.as_lists(), tol=run["tol"],
                                                       avgpool=run["avgpool"]))
        emit(f"reduce_mask_{tag}_kernel", med, mn, nbytes, {"active": nb, "occupancy": occ})
        med, mn = tm.run(lambda: ops.reduce_mask(masks[0], *g.as_lists(), tol=run["tol"],
                                                 avgpool=run["avgpool"]))
        emit(f"reduce_mask_{tag}_with_count_readback", med, mn, nbytes, {"active": nb})
        # back to back over rotating copies (144 MB of masks > L2), no flush: launch-amortised figure
        k = [0]

        def rot():
            k[0] += 1
            ops.reduce_mask_async(masks[k[0] % 8], *g.as_lists(), tol=run["tol"], avgpool=run["avgpool"])
        for _ in range(8):
            rot()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(64):
            rot()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / 64
        emit(f"reduce_mask_{tag}_back_to_back", ms, ms, nbytes, {"active": nb, "launches": 64})
    # the op as a C caller sees it: one sbnet_reduce_mask call per mask with preallocated buffers and the
    # count polled in pinned memory (host wall clock per call, rotating masks; includes ~2 us of ctypes)
    import ctypes as C
    import time
    from . import lib as _lib
    handle = _lib.load()
    idx_buf = torch.empty((8 * g.bcount[0] * g.bcount[1], 3), dtype=torch.int16, device=dev)
    cnt_pin = torch.empty(1, dtype=torch.int32, pin_memory=True)
    scratch = torch.zeros(_lib.SBNET_REDUCE_MASK_SCRATCH_INTS, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for run in c2["runs"]:
        def call(k):
            _lib.check(handle.sbnet_reduce_mask(
                masks[k % 8].data_ptr(), 8, 800, 704, float(run["tol"]), int(run["avgpool"]), g.boffset[0], g.boffset[1],
                g.bsize[0], g.bsize[1], g.bstride[0], g.bstride[1], g.bcount[0], g.bcount[1], idx_buf.data_ptr(),
                scratch.data_ptr(), cnt_pin.data_ptr(), _lib.SBNET_SCRATCH_CLEAN | _lib.SBNET_COUNT_POLL, stream))
        for k in range(16):
            call(k)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for k in range(200):
            call(k)
        dt = (time.perf_counter() - t0) / 200
        tag = "avg" if run["avgpool"] else "max"
        emit(f"reduce_mask_{tag}_c_abi_call_with_count", dt * 1e3, dt * 1e3, 18022400, {"active": int(cnt_pin[0]), "calls": 200})
    del masks

    # ---- sparse_gather on [8,512,512,128] ----
    N, H, W, C = 8, 512, 512, 128
    g = cfg.halo_geom(H, W)
    for dtype, tname in ((torch.float32, "f32"), (torch.float16, "f16")):
        x = torch.randn((N, H, W, C), device=dev, dtype=torch.float32).to(dtype)
        for dens in (0.05, 0.20, 0.50):
            idx_h, cnt_h = cfg.random_block_list(N, g.bcount, dens, seed=int(dens * 100))
            nb = int(cnt_h[0])
            U = cfg.union_pixels(idx_h, nb, g, N, H, W)
            idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
            nbytes = cfg.algorithmic_bytes("gather", nB=nb, geom=g, C=C, itemsize=x.element_size(), U=U)
            for tr in (False, True):
                shape = (nb, C, 18, 18) if tr else (nb, 18, 18, C)
                out = torch.empty(shape, dtype=dtype, device=dev)
                med, mn = tm.run(lambda: ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset,
                                                           transpose=tr, out=out))
                emit(f"gather_{tname}_t{int(tr)}_d{int(dens*100)}", med, mn, nbytes,
                     {"blocks": nb, "blocks/s": nb / (med * 1e-3)})
                del out
        # the 5 % case again with the launch cost amortised: 8 launches over 8 different block lists and
        # 8 output buffers (together larger than L2) captured in one CUDA graph, time per launch
        lists = [cfg.random_block_list(N, g.bcount, 0.05, seed=100 + k) for k in range(8)]
        for tr in (False, True):
            jobs, total = [], 0
            for idx_h, cnt_h in lists:
                nb = int(cnt_h[0])
                total += cfg.algorithmic_bytes("gather", nB=nb, geom=g, C=C, itemsize=x.element_size(),
                                               U=cfg.union_pixels(idx_h, nb, g, N, H, W))
                jobs.append((torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h),
                             torch.empty((nb, C, 18, 18) if tr else (nb, 18, 18, C), dtype=dtype, device=dev)))

            def launch_all():
                for idx, cnt, out in jobs:
                    ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=tr, out=out)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                launch_all()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                launch_all()
            med, mn = tm.run(graph.replay, flush=True)
            emit(f"gather_{tname}_t{int(tr)}_d5_graph_per_launch", med / 8, mn / 8, total / 8, {"launches_per_replay": 8})
            del jobs, graph
        del x

    # ---- sparse_scatter on [8,512,512,64] ----
    C = 64
    for dens in (0.05, 0.20, 0.50):
        idx_h, cnt_h = cfg.random_block_list(N, g.bcount, dens, seed=int(dens * 100) + 1)
        nb = int(cnt_h[0])
        idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
        # (a) fp32 atomic add with overlapping halos, Var (in place) and non-Var (copy + scatter)
        U = cfg.union_pixels(idx_h, nb, g, N, H, W)
        base = torch.randn((N, H, W, C), device=dev)
        stack = torch.randn((nb, 18, 18, C), device=dev)
        nbytes = cfg.algorithmic_bytes("scatter_add", nB=nb, geom=g, C=C, itemsize=4, U=U)
        med, mn = tm.run(lambda: ops.sparse_scatter_var(stack, cnt, idx, base, g.bsize, g.bstride,
                                                        g.boffset, add=True, atomic=True))
        emit(f"scatter_var_f32_atomic_d{int(dens*100)}", med, mn, nbytes,
             {"blocks": nb, "blocks/s": nb / (med * 1e-3)})
        ybuf = torch.empty_like(base)

        def nonvar():
            ops.copy_tensor(ybuf, base)
            ops.sparse_scatter_var(stack, cnt, idx, ybuf, g.bsize, g.bstride, g.boffset, add=True,
                                   atomic=True)
        med, mn = tm.run(nonvar)
        emit(f"scatter_f32_atomic_d{int(dens*100)}", med, mn,
             nbytes + cfg.algorithmic_bytes("scatter_copy", nB=0, geom=g, C=C, itemsize=4, U=0, N=N, H=H, W=W),
             {"blocks": nb, "blocks/s": nb / (med * 1e-3)})
        del base, stack, ybuf
        # (b) fp16 transposed overwrite, 16x16 disjoint blocks
        gi = cfg.inner_geom(H, W)
        U = cfg.union_pixels(idx_h, nb, gi, N, H, W)
        base = torch.randn((N, H, W, C), device=dev).half()
        stack = torch.randn((nb, C, 16, 16), device=dev).half()
        nbytes = cfg.algorithmic_bytes("scatter", nB=nb, geom=gi, C=C, itemsize=2, U=U)
        med, mn = tm.run(lambda: ops.sparse_scatter_var(stack, cnt, idx, base, gi.bsize, gi.bstride,
                                                        gi.boffset, add=False, transpose=True))
        emit(f"scatter_var_f16_t1_set_d{int(dens*100)}", med, mn, nbytes,
             {"blocks": nb, "blocks/s": nb / (med * 1e-3)})
        del base, stack

    # ---- blocks of more than 384 pixels in the plane layout: 34x34 over stride 32 on [8,512,512,128] ----
    C = 128
    gl = cfg.geom_for(H, W, (34, 34), (32, 32), (-1, -1))
    idx_h, cnt_h = cfg.random_block_list(N, gl.bcount, 0.20, seed=34)
    nb = int(cnt_h[0])
    idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
    U = cfg.union_pixels(idx_h, nb, gl, N, H, W)
    for dtype, tname in ((torch.float32, "f32"), (torch.float16, "f16")):
        x = torch.randn((N, H, W, C), device=dev, dtype=torch.float32).to(dtype)
        out = torch.empty((nb, C, 34, 34), dtype=dtype, device=dev)
        nbytes = cfg.algorithmic_bytes("gather", nB=nb, geom=gl, C=C, itemsize=x.element_size(), U=U)
        med, mn = tm.run(lambda: ops.sparse_gather(x, cnt, idx, gl.bsize, gl.bstride, gl.boffset,
                                                   transpose=True, out=out))
        emit(f"gather_{tname}_t1_b34_d20", med, mn, nbytes, {"blocks": nb, "blocks/s": nb / (med * 1e-3)})
        nbytes = cfg.algorithmic_bytes("scatter_add", nB=nb, geom=gl, C=C, itemsize=x.element_size(), U=U)
        med, mn = tm.run(lambda: ops.sparse_scatter_var(out, cnt, idx, x, gl.bsize, gl.bstride, gl.boffset,
                                                        add=True, atomic=True, transpose=True))
        emit(f"scatter_var_{tname}_t1_atomic_b34_d20", med, mn, nbytes,
             {"blocks": nb, "blocks/s": nb / (med * 1e-3)})
        del x, out

    # ---- plain copy (the non-Var op's base copy), with torch's own copy beside it as a yardstick ----
    a = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    b = torch.empty_like(a)
    med, mn = tm.run(lambda: ops.copy_tensor(b, a))
    emit("copy_tensor_1GiB", med, mn, 2 << 30, {})
    a16, b16 = a.view(torch.bfloat16), b.view(torch.bfloat16)
    med, mn = tm.run(lambda: b16.copy_(a16))
    emit("yardstick_torch_copy_1GiB", med, mn, 2 << 30, {})

    # ---- launch floor: the same reduce_mask entry point on a 32x32 mask ----
    tiny = torch.zeros((1, 32, 32, 1), device=dev)
    med, mn = tm.run(lambda: ops.reduce_mask_async(tiny, [2, 2], [18, 18], [16, 16], [-1, -1], tol=0.5))
    emit("floor_reduce_mask_32x32_event_timed", med, mn, 4096, {})

    # ---- reduce_mask replayed from a CUDA graph: 32 launches over 8 rotating masks, no host in the loop ----
    c2 = cfg.config2(0)
    g = c2["geom"]
    masks = [torch.from_numpy(c2["mask"]).to(dev) for _ in range(8)]
    for run in c2["runs"]:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for m in masks:   # warm-up on the capture stream (also zero-fills that stream's scratch)
                ops.reduce_mask_async(m, *g.as_lists(), tol=run["tol"], avgpool=run["avgpool"])
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        keep = []
        with torch.cuda.graph(graph, stream=side):
            for i in range(32):
                keep.append(ops.reduce_mask_async(masks[i % 8], *g.as_lists(), tol=run["tol"], avgpool=run["avgpool"]))
        med, mn = tm.run(graph.replay, flush=False)
        tag = "avg" if run["avgpool"] else "max"
        emit(f"reduce_mask_{tag}_graph_replay_per_launch", med / 32, mn / 32, 18022400, {"launches_per_replay": 32})

