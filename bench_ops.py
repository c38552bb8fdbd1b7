"""Op-level measurements behind ``bench.py --suite ops`` and the ``suite`` table of the benchmark line.

Benchmark tooling, kept beside ``bench.py`` and outside the library package.  Cases are the op-level
benchmark configurations: reduce_mask on a bird's-eye-view sized mask ([8,800,704], avg and max
pooling) with its yardsticks (an empty launch and a load-only pass over the same mask), sparse_gather
on x [8,512,512,128] (fp32 / fp16, both layouts, 5 / 20 / 50 % active blocks) and sparse_scatter[_var]
(fp32 atomic add with overlapping halos onto [8,512,512,64], Var and non-Var; fp16 transposed
overwrite).  Protocol (the reference's own harness: warm-up, repeats, CUDA-event time,
``benchmark/sparse_conv_perf.py:202-262``): every launch is timed on its own with CUDA events on the
launching stream after an L2 flush (a 256 MiB fill), at least 5 warm-ups and 20 timed launches, median
and minimum reported with the algorithmic bytes of the call and the fraction of the HBM peak.  The small
cases are measured a second time per launch inside a CUDA graph of eight launches over eight different
inputs (together larger than L2), which takes the host's launch cost out.
"""
from __future__ import annotations

import ctypes
import json
import os
import statistics
import subprocess

from sbnet_b200 import configs as cfg

ROOT = os.path.dirname(os.path.abspath(__file__))
YARD_SRC = os.path.join(ROOT, "bench_yardsticks.cu")
YARD_LIB = os.path.join(ROOT, "bench_yardsticks.so")


def _peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def build_yardsticks(force: bool = False) -> str:
    """Compiles ``bench_yardsticks.cu`` for sm_100a next to its source (nvcc cross-compiles without a GPU)."""
    if not force and os.path.exists(YARD_LIB) and os.path.getmtime(YARD_LIB) >= os.path.getmtime(YARD_SRC):
        return YARD_LIB
    from sbnet_b200.build import _nvcc
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--cudart", "static",
           "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared", "-o", YARD_LIB, YARD_SRC]
    if os.path.exists("/usr/bin/g++"):
        cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
    subprocess.run(cmd, check=True)
    return YARD_LIB


_yard = None


def yardsticks():
    global _yard
    if _yard is None:
        lib = ctypes.CDLL(build_yardsticks())
        lib.yard_launch.restype = ctypes.c_int
        lib.yard_launch.argtypes = [ctypes.c_int, ctypes.c_void_p] + [ctypes.c_int] * 7 + [ctypes.c_void_p, ctypes.c_void_p]
        _yard = lib
    return _yard


class Timer:
    def __init__(self, torch, dev, steps, warmup):
        self.t, self.dev, self.steps, self.warmup = torch, dev, max(steps, 20), max(warmup, 5)
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

    def graph_per_launch(self, launch_all, n_launches):
        """``launch_all`` enqueues ``n_launches`` launches; they are captured into one CUDA graph and the
        replay is timed after an L2 flush.  Returns (median, min) per launch."""
        t = self.t
        side = t.cuda.Stream()
        side.wait_stream(t.cuda.current_stream())
        with t.cuda.stream(side):
            launch_all()
        t.cuda.current_stream().wait_stream(side)
        t.cuda.synchronize()
        graph = t.cuda.CUDAGraph()
        with t.cuda.graph(graph, stream=side):
            launch_all()
        med, mn = self.run(graph.replay, flush=True)
        del graph
        return med / n_launches, mn / n_launches


class Table:
    """Collects the rows; prints each as a JSON line unless ``quiet``."""

    def __init__(self, quiet=False):
        self.rows, self.quiet = {}, quiet
        self.peak, self.kind = _peak()

    def emit(self, name, med_ms, min_ms, nbytes, extra=None):
        gbs = nbytes / (med_ms * 1e-3) / 1e9
        row = {"us": round(med_ms * 1e3, 3), "us_min": round(min_ms * 1e3, 3), "algorithmic_bytes": int(nbytes),
               "GB/s": round(gbs, 1), "frac_of_" + self.kind: round(gbs / self.peak, 4)}
        row.update(extra or {})
        self.rows[name] = row
        if not self.quiet:
            print(json.dumps(dict(case=name, **row, **{"peak_GB/s": self.peak})), flush=True)


def _set_one_case(name, dens, channels, block, torch, dev):
    """Inputs and the launch closure of one gather / scatter case (``--suite one``)."""
    from sbnet_b200 import ops
    N, H, W = 8, 512, 512
    kind, tname, layout = name.split("_")[:3]           # gather_f16_t1, scatter_f32_t0_atomic ...
    mode = name.split("_")[3] if kind == "scatter" else None
    dtype = torch.float16 if tname == "f16" else torch.float32
    tr = layout == "t1"
    C = channels or (128 if kind == "gather" else 64)
    halo = kind == "gather" or mode == "atomic"
    g = cfg.halo_geom(H, W) if halo else cfg.inner_geom(H, W)
    if block:   # SIZE,STRIDE,OFFSET: square blocks of another geometry
        b, stride, off = (int(v) for v in block.split(","))
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
    return fn, nbytes, nb


def one(args):
    """``bench.py --suite one --case NAME [--density D] [--one-channels C] [--one-block SIZE,STRIDE,OFFSET]``:
    a few launches of ONE op on a mid-sized input (larger than L2, well under a GB), for profiler
    captures.  NAME is an op case (gather_f16_t1, scatter_f32_t0_atomic, reduce_mask_max, reduce_mask_avg)
    or a yardstick (yard_empty, yard_load, yard_bulk).  Prints one JSON line."""
    import torch
    from sbnet_b200 import build, ops
    build.build_library()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tm = Timer(torch, dev, 0, 0)
    tm.steps, tm.warmup = max(args.steps, 3), 3
    name, dens = args.case, args.density
    extra = {"density": dens}
    if name.startswith("reduce_mask") or name.startswith("yard_"):
        c2 = cfg.config2(0)
        g = c2["geom"]
        m = torch.from_numpy(c2["mask"]).to(dev)
        nbytes = m.numel() * 4
        if name.startswith("yard_"):
            fn = _yard_fn(torch, m, g, {"yard_empty": 0, "yard_load": 1, "yard_bulk": 2}[name])
        else:
            avg = name.endswith("avg")
            fn = lambda: ops.reduce_mask_async(m, *g.as_lists(), tol=0.1 if avg else 0.5, avgpool=avg)  # noqa: E731
    else:
        fn, nbytes, nb = _set_one_case(name, dens, args.one_channels, getattr(args, "one_block", None), torch, dev)
        extra["blocks"] = nb
    med, mn = tm.run(fn, flush=True)
    Table().emit(name, med, mn, nbytes, extra)


def _yard_fn(torch, mask, g, kind):
    lib = yardsticks()
    N, H, W = mask.shape[0], mask.shape[1], mask.shape[2]
    out = torch.zeros(4, dtype=torch.int32, device=mask.device)

    def fn():
        rc = lib.yard_launch(kind, mask.data_ptr(), N, H, W, g.bsize[0], g.bstride[0], g.boffset[0], g.bcount[0],
                             out.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0, rc
    fn.keep = out
    return fn


def resblock(args):
    """``bench.py --suite resblock``: the full sparse bottleneck (x fp16 [batch,400,352,256], 1x1 256->64,
    3x3 VALID 64->64, 1x1 64->256 by torch / cuDNN between gather and scatter) with the share of the
    block ops in the block time.  The convolutions are the host framework's, identical whichever op
    library is used; they are reported, not optimised here."""
    import torch
    from sbnet_b200 import build, ops
    from sbnet_b200.resblock import SparseBottleneck
    build.build_library()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    N, H, W, C = args.batch, args.height, args.width, args.channels
    m = SparseBottleneck(C, C // 4, dtype=torch.float16).eval()
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


# ---- the table ----------------------------------------------------------------------------------

def reduce_mask_rows(tb, tm, torch, dev):
    """Config 2: [8,800,704] mask, avg (tol 0.1) and max (tol 0.5): the kernel alone, the op with the
    count read back to the host, per launch inside a CUDA graph, and the yardsticks."""
    import time
    from sbnet_b200 import lib as _lib, ops
    c2 = cfg.config2(0)
    g = c2["geom"]
    masks = [torch.from_numpy(c2["mask"]).to(dev) for _ in range(8)]   # 144 MB of copies: larger than L2
    occ = float(c2["mask"].mean())
    nbytes_mask = masks[0].numel() * 4
    for run in c2["runs"]:
        tag = "avg" if run["avgpool"] else "max"
        idx, cnt = ops.reduce_mask(masks[0], *g.as_lists(), tol=run["tol"], avgpool=run["avgpool"])
        nb = int(cnt[0])
        nbytes = cfg.algorithmic_bytes("reduce_mask", nB=nb, geom=g, C=1, itemsize=4, U=0, N=8, H=800, W=704, count=nb)
        med, mn = tm.run(lambda: ops.reduce_mask_async(masks[0], *g.as_lists(), tol=run["tol"], avgpool=run["avgpool"]))
        tb.emit(f"c2_reduce_mask_{tag}_kernel", med, mn, nbytes, {"active": nb, "occupancy": round(occ, 4)})
        med, mn = tm.run(lambda: ops.reduce_mask(masks[0], *g.as_lists(), tol=run["tol"], avgpool=run["avgpool"]))
        tb.emit(f"c2_reduce_mask_{tag}_with_count_readback", med, mn, nbytes, {"active": nb})

        def graph_body():
            for i in range(32):
                keep.append(ops.reduce_mask_async(masks[i % 8], *g.as_lists(), tol=run["tol"], avgpool=run["avgpool"]))
        keep = []
        med, mn = tm.graph_per_launch(graph_body, 32)
        tb.emit(f"c2_reduce_mask_{tag}_graph_per_launch", med, mn, nbytes, {"launches_per_replay": 32})
        keep.clear()
    # the op as a C caller sees it: one sbnet_reduce_mask call per mask with preallocated buffers and the
    # count polled in pinned memory (host wall clock per call, rotating masks; includes ~2 us of ctypes)
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
        tb.emit(f"c2_reduce_mask_{tag}_c_abi_call_with_count", dt * 1e3, dt * 1e3, nbytes_mask,
                {"active": int(cnt_pin[0]), "calls": 200, "clock": "host wall clock"})
    # yardsticks on the same mask: an empty launch of 400 CTAs, and the 18 MB loaded once (plain 128-bit
    # loads / bulk copies into shared memory) with nothing else to do
    for name, kind in (("empty_launch", 0), ("load_only", 1), ("bulk_load_only", 2)):
        fns = [_yard_fn(torch, m, g, kind) for m in masks]
        med, mn = tm.run(fns[0])
        tb.emit(f"c2_yardstick_{name}", med, mn, nbytes_mask if kind else 0, {})

        def body():
            for i in range(32):
                fns[i % 8]()
        med, mn = tm.graph_per_launch(body, 32)
        tb.emit(f"c2_yardstick_{name}_graph_per_launch", med, mn, nbytes_mask if kind else 0, {"launches_per_replay": 32})
    # launch floor of the entry point itself: the same call on a 32x32 mask
    tiny = torch.zeros((1, 32, 32, 1), device=dev)
    med, mn = tm.run(lambda: ops.reduce_mask_async(tiny, [2, 2], [18, 18], [16, 16], [-1, -1], tol=0.5))
    tb.emit("floor_reduce_mask_32x32_event_timed", med, mn, 4096, {})


def gather_rows(tb, tm, torch, dev):
    """Config 3: x [8,512,512,128] fp32 and fp16, both layouts, 5 / 20 / 50 %."""
    from sbnet_b200 import ops
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
                out = torch.empty((nb, C, 18, 18) if tr else (nb, 18, 18, C), dtype=dtype, device=dev)
                med, mn = tm.run(lambda: ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=tr, out=out))
                tb.emit(f"c3_gather_{tname}_t{int(tr)}_d{int(dens*100)}", med, mn, nbytes, {"blocks": nb})
                del out
        # the 5 % case with the launch cost amortised: 8 launches over 8 different block lists and 8
        # output buffers (together larger than L2) in one CUDA graph, time per launch
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
            med, mn = tm.graph_per_launch(launch_all, 8)
            tb.emit(f"c3_gather_{tname}_t{int(tr)}_d5_graph_per_launch", med, mn, total / 8, {"launches_per_replay": 8})
            del jobs
        del x


def scatter_rows(tb, tm, torch, dev):
    """Config 4: (a) fp32 atomic add of [nB,18,18,64] stacks with overlapping halos onto [8,512,512,64], Var and
    non-Var; (b) fp16 transposed overwrite of [nB,64,16,16] stacks.  5 / 20 / 50 %."""
    from sbnet_b200 import ops
    N, H, W, C = 8, 512, 512, 64
    g, gi = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    base = torch.randn((N, H, W, C), device=dev)
    ybuf = torch.empty_like(base)
    base16 = torch.randn((N, H, W, C), device=dev).half()
    ybuf16 = torch.empty_like(base16)
    copy_bytes = cfg.algorithmic_bytes("scatter_copy", nB=0, geom=g, C=C, itemsize=4, U=0, N=N, H=H, W=W)
    for dens in (0.05, 0.20, 0.50):
        idx_h, cnt_h = cfg.random_block_list(N, g.bcount, dens, seed=int(dens * 100) + 1)
        nb = int(cnt_h[0])
        idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
        d = int(dens * 100)
        # (a) fp32 atomic add with overlapping halos, Var (in place) and non-Var (copy + scatter)
        U = cfg.union_pixels(idx_h, nb, g, N, H, W)
        stack = torch.randn((nb, 18, 18, C), device=dev)
        nbytes = cfg.algorithmic_bytes("scatter_add", nB=nb, geom=g, C=C, itemsize=4, U=U)
        med, mn = tm.run(lambda: ops.sparse_scatter_var(stack, cnt, idx, base, g.bsize, g.bstride, g.boffset, add=True,
                                                        atomic=True))
        tb.emit(f"c4a_scatter_var_f32_atomic_d{d}", med, mn, nbytes, {"blocks": nb})

        def nonvar():
            ops.copy_tensor(ybuf, base)
            ops.sparse_scatter_var(stack, cnt, idx, ybuf, g.bsize, g.bstride, g.boffset, add=True, atomic=True)
        med, mn = tm.run(nonvar)
        tb.emit(f"c4a_scatter_f32_atomic_d{d}", med, mn, nbytes + copy_bytes, {"blocks": nb})
        del stack
        # (b) fp16 transposed overwrite, 16x16 disjoint blocks, Var and non-Var
        U = cfg.union_pixels(idx_h, nb, gi, N, H, W)
        stack = torch.randn((nb, C, 16, 16), device=dev).half()
        nbytes = cfg.algorithmic_bytes("scatter", nB=nb, geom=gi, C=C, itemsize=2, U=U)
        med, mn = tm.run(lambda: ops.sparse_scatter_var(stack, cnt, idx, base16, gi.bsize, gi.bstride, gi.boffset,
                                                        add=False, transpose=True))
        tb.emit(f"c4b_scatter_var_f16_t1_set_d{d}", med, mn, nbytes, {"blocks": nb})

        def nonvar16():
            ops.copy_tensor(ybuf16, base16)
            ops.sparse_scatter_var(stack, cnt, idx, ybuf16, gi.bsize, gi.bstride, gi.boffset, add=False, transpose=True)
        med, mn = tm.run(nonvar16)
        tb.emit(f"c4b_scatter_f16_t1_set_d{d}", med, mn, nbytes + copy_bytes // 2, {"blocks": nb})
        del stack
    # the small launches per launch inside a CUDA graph: 8 launches over 8 block lists / stacks
    for tag, dens, dtype, shape, geom, kw, op, isz, b in (
            ("c4a_scatter_var_f32_atomic_d5", 0.05, torch.float32, (18, 18, C), g, dict(add=True, atomic=True), "scatter_add", 4, base),
            ("c4b_scatter_var_f16_t1_set_d5", 0.05, torch.float16, (C, 16, 16), gi, dict(add=False, transpose=True), "scatter", 2, base16),
            ("c4b_scatter_var_f16_t1_set_d20", 0.20, torch.float16, (C, 16, 16), gi, dict(add=False, transpose=True), "scatter", 2, base16),
            ("c4b_scatter_var_f16_t1_set_d50", 0.50, torch.float16, (C, 16, 16), gi, dict(add=False, transpose=True), "scatter", 2, base16)):
        jobs, total = [], 0
        for k in range(8):
            idx_h, cnt_h = cfg.random_block_list(N, geom.bcount, dens, seed=200 + k)
            nb = int(cnt_h[0])
            total += cfg.algorithmic_bytes(op, nB=nb, geom=geom, C=C, itemsize=isz, U=cfg.union_pixels(idx_h, nb, geom, N, H, W))
            jobs.append((torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h), torch.randn((nb, *shape), device=dev).to(dtype)))

        def launch_all():
            for idx, cnt, st in jobs:
                ops.sparse_scatter_var(st, cnt, idx, b, geom.bsize, geom.bstride, geom.boffset, **kw)
        med, mn = tm.graph_per_launch(launch_all, 8)
        tb.emit(f"{tag}_graph_per_launch", med, mn, total / 8, {"launches_per_replay": 8})
        del jobs


def large_block_rows(tb, tm, torch, dev):
    """Blocks of more than 384 pixels in the plane layout: 34x34 over stride 32 on [8,512,512,128]; and pixels
    that are not a multiple of 16 bytes (C = 33 fp32, C = 100 fp16), which run the general kernels."""
    from sbnet_b200 import ops
    N, H, W, C = 8, 512, 512, 128
    gl = cfg.geom_for(H, W, (34, 34), (32, 32), (-1, -1))
    idx_h, cnt_h = cfg.random_block_list(N, gl.bcount, 0.20, seed=34)
    nb = int(cnt_h[0])
    idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
    U = cfg.union_pixels(idx_h, nb, gl, N, H, W)
    for dtype, tname in ((torch.float32, "f32"), (torch.float16, "f16")):
        x = torch.randn((N, H, W, C), device=dev, dtype=torch.float32).to(dtype)
        out = torch.empty((nb, C, 34, 34), dtype=dtype, device=dev)
        nbytes = cfg.algorithmic_bytes("gather", nB=nb, geom=gl, C=C, itemsize=x.element_size(), U=U)
        med, mn = tm.run(lambda: ops.sparse_gather(x, cnt, idx, gl.bsize, gl.bstride, gl.boffset, transpose=True, out=out))
        tb.emit(f"gather_{tname}_t1_b34_d20", med, mn, nbytes, {"blocks": nb})
        nbytes = cfg.algorithmic_bytes("scatter_add", nB=nb, geom=gl, C=C, itemsize=x.element_size(), U=U)
        med, mn = tm.run(lambda: ops.sparse_scatter_var(out, cnt, idx, x, gl.bsize, gl.bstride, gl.boffset, add=True,
                                                        atomic=True, transpose=True))
        tb.emit(f"scatter_var_{tname}_t1_atomic_b34_d20", med, mn, nbytes, {"blocks": nb})
        del x, out
    g = cfg.halo_geom(H, W)
    idx_h, cnt_h = cfg.random_block_list(N, g.bcount, 0.20, seed=21)
    nb = int(cnt_h[0])
    idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
    U = cfg.union_pixels(idx_h, nb, g, N, H, W)
    for dtype, tname, Cx in ((torch.float32, "f32", 33), (torch.float16, "f16", 100)):
        x = torch.randn((N, H, W, Cx), device=dev, dtype=torch.float32).to(dtype)
        for tr in (False, True):
            out = torch.empty((nb, Cx, 18, 18) if tr else (nb, 18, 18, Cx), dtype=dtype, device=dev)
            nbytes = cfg.algorithmic_bytes("gather", nB=nb, geom=g, C=Cx, itemsize=x.element_size(), U=U)
            med, mn = tm.run(lambda: ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=tr, out=out))
            tb.emit(f"gather_{tname}_C{Cx}_t{int(tr)}_d20", med, mn, nbytes, {"blocks": nb})
            nbytes = cfg.algorithmic_bytes("scatter_add", nB=nb, geom=g, C=Cx, itemsize=x.element_size(), U=U)
            med, mn = tm.run(lambda: ops.sparse_scatter_var(out, cnt, idx, x, g.bsize, g.bstride, g.boffset, add=True,
                                                            atomic=True, transpose=tr))
            tb.emit(f"scatter_var_{tname}_C{Cx}_t{int(tr)}_atomic_d20", med, mn, nbytes, {"blocks": nb})
            del out
        del x


def copy_rows(tb, tm, torch, dev):
    """Plain copy (the non-Var op's base copy), with torch's own copy beside it as a yardstick."""
    from sbnet_b200 import ops
    a = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    b = torch.empty_like(a)
    med, mn = tm.run(lambda: ops.copy_tensor(b, a))
    tb.emit("copy_tensor_1GiB", med, mn, 2 << 30, {})
    a16, b16 = a.view(torch.bfloat16), b.view(torch.bfloat16)
    med, mn = tm.run(lambda: b16.copy_(a16))
    tb.emit("yardstick_torch_copy_1GiB", med, mn, 2 << 30, {})


def suite_table(torch, dev, steps=20, warmup=5, quiet=True, extended=False, other_shapes=False):
    """All rows of the op-level table as {case: row}.  ``other_shapes`` adds the large-block and odd-channel
    rows (shapes outside the configured cases that run other kernels), ``extended`` those and the copy rows
    (``--suite ops`` prints them all)."""
    from sbnet_b200 import build
    build.build_library()
    tm = Timer(torch, dev, steps, warmup)
    tb = Table(quiet=quiet)
    reduce_mask_rows(tb, tm, torch, dev)
    gather_rows(tb, tm, torch, dev)
    scatter_rows(tb, tm, torch, dev)
    if extended or other_shapes:
        large_block_rows(tb, tm, torch, dev)
    if extended:
        copy_rows(tb, tm, torch, dev)
    del tm
    torch.cuda.empty_cache()
    return tb.rows


def main(args):
    import torch
    if getattr(args, "suite", None) == "one":
        return one(args)
    if getattr(args, "suite", None) == "resblock":
        return resblock(args)
    if getattr(args, "suite", None) == "topleft":
        from bench_topleft import topleft
        return topleft(args)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    suite_table(torch, dev, steps=args.steps if args.steps != 100 else 20, warmup=args.warmup, quiet=False, extended=True)
