#!/usr/bin/env python
"""Benchmark of the block-op hot path: reduce_mask -> sparse_gather -> sparse_scatter_var.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--occupancy 0.1] [--scaling weak|strong] [--suite ops]

Workload (one "step" = one pass of the three ops over one batch): the sparse ResNet-bottleneck
configuration -- x fp16 [32,400,352,256], a rectangle-union mask, 18x18 windows on a 16 pixel pitch
with a one pixel halo: reduce_mask (max, tol 0.5) -> sparse_gather(transpose=True) ->
sparse_scatter_var(add=True, transpose=True, 16x16 interior) of a conv-output-shaped stack back onto
x.  The dense convolutions between gather and scatter belong to the host framework and are not part
of this library, so they are not in the step.  Data is synthetic and seeded (sbnet_b200/configs.py).

One JSON line is printed by rank 0.  `value` is blocks/s over all ranks with inputs resident in HBM;
`e2e` is the same pipeline fed from pinned host buffers with the copies inside the timed region;
`roofline` describes the kernel that takes the largest share of the step; `cpu_baseline` is the
reference's CPU functors timed on this machine's cores on a bounded sample.

`--impl reference` times the reference's own CPU implementation (oracle/_ref when it was compiled
from the reference tree, else the C restatement) on bounded samples of the same workload.
`--suite ops` prints one JSON line per op-level configuration (mask / gather / scatter sizes of the
other benchmark configurations) instead of the pipeline line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from sbnet_b200 import configs as cfg  # noqa: E402

FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 * 1024 * 1024


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi.  The sampler is started
    well before the timed region (nvidia-smi takes a moment to come up); `summary(t0, t1)` keeps the
    samples that arrived inside the wall-clock window of the load."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self, t0, t1):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, r in self.rows:
            if not (t0 <= t <= t1 + 0.06):
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                for nm, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
            except Exception:
                continue
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ---- workload ------------------------------------------------------------------------------------

def make_host_inputs(args, rank, world):
    """Seeded host-side inputs of one rank (numpy).  Weak scaling: every rank owns a full batch of its
    own images; strong scaling: the ranks split ONE batch into contiguous slices."""
    from sbnet_b200.dist import shard_bounds
    H, W, C = args.height, args.width, args.channels
    if args.scaling == "weak":
        first, N = rank * args.batch, args.batch
    else:
        lo, hi = shard_bounds(args.batch, world, rank)
        first, N = lo, max(hi - lo, 1)
    # image n of the global batch always gets seed 7 + n, whichever rank owns it
    mask = cfg.rect_union_mask(N, H, W, seed=7 + first, occupancy=args.occupancy)
    return N, H, W, C, mask


def union_stats(mask, g_in, g_out, N, H, W):
    """Active blocks and distinct covered pixels (for the algorithmic-byte formulas), on the CPU."""
    m = mask[..., 0] > 0.5
    bch, bcw = g_in.bcount
    act = np.zeros((N, bch, bcw), dtype=bool)
    for bh in range(bch):
        h0 = g_in.boffset[0] + bh * g_in.bstride[0]
        rows = m[:, max(h0, 0):min(h0 + g_in.bsize[0], H), :]
        for bw in range(bcw):
            w0 = g_in.boffset[1] + bw * g_in.bstride[1]
            act[:, bh, bw] = rows[:, :, max(w0, 0):min(w0 + g_in.bsize[1], W)].any(axis=(1, 2))
    nB = int(act.sum())
    idx = np.argwhere(act).astype(np.int16)
    U_in = cfg.union_pixels(idx, nB, g_in, N, H, W)
    U_out = cfg.union_pixels(idx, nB, g_out, N, H, W)
    return nB, U_in, U_out, idx


def per_image_blocks(mask, g_in, N, H, W):
    """Active blocks of every image (max pooling, tol 0.5 on a 0/1 mask), on the CPU."""
    m = mask[..., 0] > 0.5
    out = np.zeros(N, dtype=np.int64)
    for bh in range(g_in.bcount[0]):
        h0 = g_in.boffset[0] + bh * g_in.bstride[0]
        rows = m[:, max(h0, 0):min(h0 + g_in.bsize[0], H), :]
        for bw in range(g_in.bcount[1]):
            w0 = g_in.boffset[1] + bw * g_in.bstride[1]
            out += rows[:, :, max(w0, 0):min(w0 + g_in.bsize[1], W)].any(axis=(1, 2))
    return out


# ---- our arm -------------------------------------------------------------------------------------

def run_ours(args):
    import torch
    import torch.distributed as dist
    from sbnet_b200 import build, lib, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in the product)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if rank == 0:
        build.build_library()
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
    lib.load()

    N, H, W, C, mask_h = make_host_inputs(args, rank, world)
    g_in, g_out = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    nB, U_in, U_out, _ = union_stats(mask_h, g_in, g_out, N, H, W)
    sz = 2
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    x = torch.empty((N, H, W, C), dtype=torch.float16, device=dev)
    for n in range(N):  # generated in slices: a one-shot fp32 randn of this size would double the footprint
        x[n] = torch.randn((H, W, C), generator=gen, device=dev, dtype=torch.float32).half()
    # conv-output-shaped stack [nB,C,16,16]; small magnitudes so K accumulations stay far from fp16 max
    q = (torch.randn((nB, C, 16, 16), generator=gen, device=dev, dtype=torch.float32) * 0.01).half()
    stack = torch.empty((nB, C, 18, 18), dtype=torch.float16, device=dev)
    # masks rotate through enough copies to exceed L2 on their own
    n_masks = max(2, int(L2_BYTES // mask_h.nbytes) + 2)
    masks = [torch.from_numpy(mask_h).to(dev) for _ in range(min(n_masks, 8))]
    torch.cuda.synchronize()

    bytes_mask = cfg.algorithmic_bytes("reduce_mask", nB=nB, geom=g_in, C=1, itemsize=4, U=0, N=N,
                                       H=H, W=W, count=nB)
    bytes_gather = cfg.algorithmic_bytes("gather", nB=nB, geom=g_in, C=C, itemsize=sz, U=U_in)
    bytes_scatter = cfg.algorithmic_bytes("scatter_add", nB=nB, geom=g_out, C=C, itemsize=sz, U=U_out)

    from sbnet_b200 import dist as sbdist
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731

    last_counts = [None]
    pending = [None]
    side = torch.cuda.Stream() if world > 1 else None

    def step(i, marks=None, exchange=True):
        m = masks[i % len(masks)]
        if pending[0] is not None:   # the previous step's all-gather has read the device count by now
            pending[0].wait()
            pending[0] = None
        if marks is not None:
            marks[0].record()
        idx, cnt = ops.reduce_mask(m, *g_in.as_lists(), tol=0.5, avgpool=False)
        if marks is not None:
            marks[1].record()
        nb = int(cnt[0])
        assert nb == nB, (nb, nB)
        if marks is not None:
            marks[2].record()
        ops.sparse_gather(x, cnt, idx, g_in.bsize, g_in.bstride, g_in.boffset, transpose=True, out=stack)
        if marks is not None:
            marks[3].record()
        ops.sparse_scatter_var(q, cnt, idx, x, g_out.bsize, g_out.bstride, g_out.boffset, add=True,
                               transpose=True)
        if marks is not None:
            marks[4].record()
        if world > 1 and exchange:
            # The only exchange of the path: every rank's block count, read from device memory.  It is
            # issued after gather and scatter are queued, on a side stream (the count is final: the op
            # interface already synchronised for it), so it overlaps them and nothing waits for it
            # until the next reduce_mask is about to overwrite the count.
            count_dev = ops.scratch_for(dev, torch.cuda.current_stream(dev).cuda_stream)[0][:1]
            with torch.cuda.stream(side):
                counts_all, pending[0] = sbdist.all_gather_counts(count_dev, async_op=True)
            last_counts[0] = counts_all
        return nb

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    clocks = ClockSampler(local).start()
    for i in range(args.warmup):
        step(i)
    fence()
    marks = [[ev() for _ in range(5)] for _ in range(args.steps)]
    t0, t1 = ev(), ev()
    fence()
    wall0 = time.time()
    t0.record()
    blocks = 0
    for i in range(args.steps):
        blocks += step(args.warmup + i, marks[i])
    t1.record()
    if pending[0] is not None:
        pending[0].wait()
        pending[0] = None
    fence()
    ms_total = t0.elapsed_time(t1)
    # a short timed region may fall between two clock samples: keep the same load running (untimed)
    # until at least half a second of it has been sampled
    extra = 0
    while time.time() - wall0 < 0.5:
        step(extra, exchange=False)   # ranks may run different numbers of these: no collective here
        extra += 1
    torch.cuda.synchronize()
    wall1 = time.time()
    if pending[0] is not None:
        pending[0].wait()
        pending[0] = None
    fence()
    clocks.stop()
    op_ms = {"reduce_mask": [], "gather": [], "scatter": []}
    for mk in marks:
        op_ms["reduce_mask"].append(mk[0].elapsed_time(mk[1]))
        op_ms["gather"].append(mk[2].elapsed_time(mk[3]))
        op_ms["scatter"].append(mk[3].elapsed_time(mk[4]))

    # ---- end to end: host buffers in, host result out, copies inside the timed region ----
    # The batch is cut into image groups; three streams (host->device, compute, device->host) are
    # chained with events so that the upload of group g+1, the ops on group g and the download of
    # group g-1 overlap.  PCIe is full duplex, so a step costs about max(upload, download) instead of
    # their sum.  Every byte of mask, x and the conv-output stack goes up and every byte of the
    # updated x comes down inside the timed region, every step.
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(1, min(args.steps, args.e2e_steps))
        G = max(1, min(args.e2e_groups, N))
        bounds = [(N * g) // G for g in range(G + 1)]
        per_image = per_image_blocks(mask_h, g_in, N, H, W)
        qoff = [0]
        for g in range(G):
            qoff.append(qoff[-1] + int(per_image[bounds[g]:bounds[g + 1]].sum()))
        hx = torch.empty((N, H, W, C), dtype=torch.float16, pin_memory=True)
        hx.copy_(x)
        hq = torch.empty(q.shape, dtype=torch.float16, pin_memory=True)
        hq.copy_(q)
        hm = torch.from_numpy(mask_h).pin_memory()
        hy = torch.empty((N, H, W, C), dtype=torch.float16, pin_memory=True)
        dm = masks[0]
        s_in, s_c, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        out_done = [None] * G
        fence()

        def e2e_step():
            in_done = []
            with torch.cuda.stream(s_in):
                for g in range(G):
                    lo, hi = bounds[g], bounds[g + 1]
                    if out_done[g] is not None:      # x[lo:hi] of the previous step must be downloaded first
                        s_in.wait_event(out_done[g])
                    dm[lo:hi].copy_(hm[lo:hi], non_blocking=True)
                    x[lo:hi].copy_(hx[lo:hi], non_blocking=True)
                    q[qoff[g]:qoff[g + 1]].copy_(hq[qoff[g]:qoff[g + 1]], non_blocking=True)
                    e = torch.cuda.Event()
                    e.record(s_in)
                    in_done.append(e)
            total = 0
            for g in range(G):
                lo, hi = bounds[g], bounds[g + 1]
                with torch.cuda.stream(s_c):
                    s_c.wait_event(in_done[g])
                    idx, cnt = ops.reduce_mask(dm[lo:hi], *g_in.as_lists(), tol=0.5, avgpool=False)
                    nb = int(cnt[0])
                    assert nb == qoff[g + 1] - qoff[g] or qoff[g + 1] == qoff[g], (nb, g)
                    if qoff[g + 1] > qoff[g]:
                        ops.sparse_gather(x[lo:hi], cnt, idx, g_in.bsize, g_in.bstride, g_in.boffset,
                                          transpose=True, out=stack[:nb])
                        ops.sparse_scatter_var(q[qoff[g]:qoff[g + 1]], cnt, idx, x[lo:hi], g_out.bsize,
                                               g_out.bstride, g_out.boffset, add=True, transpose=True)
                        total += nb
                    e = torch.cuda.Event()
                    e.record(s_c)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(e)
                    hy[lo:hi].copy_(x[lo:hi], non_blocking=True)
                    d = torch.cuda.Event()
                    d.record(s_out)
                    out_done[g] = d
            return total

        def e2e_fence():
            for st in (s_in, s_c, s_out):
                st.synchronize()
            fence()

        e2e_step()
        e2e_fence()
        a, b = ev(), ev()
        a.record()
        s_in.wait_event(a)
        eb = 0
        for _ in range(e2e_steps):
            eb += e2e_step()
        for st in (s_in, s_c, s_out):
            torch.cuda.current_stream().wait_stream(st)
        b.record()
        e2e_fence()
        e2e_ms = a.elapsed_time(b)
        e2e = dict(ms=e2e_ms, blocks=eb, steps=e2e_steps, groups=G,
                   h2d=hx.numel() * 2 + hq.numel() * 2 + hm.numel() * 4, d2h=hy.numel() * 2)
        del hx, hq, hy

    # ---- the same three ops with the block count kept on the device, replayed from a CUDA graph ----
    # (outside the op interface, which needs bin_counts on the host; offered by the *_dyn entry points)
    sync_free = None
    if world == 1 and not args.no_sync_free:
        max_blocks = N * g_in.bcount[0] * g_in.bcount[1]
        big_stack = torch.empty((max_blocks, C, 18, 18), dtype=torch.float16, device=dev)
        big_q = torch.empty((max_blocks, C, 16, 16), dtype=torch.float16, device=dev)
        big_q[:nB] = q
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())

        def dyn_step(m):
            idx, cnt_dev = ops.reduce_mask_async(m, *g_in.as_lists(), tol=0.5, avgpool=False)
            ops.sparse_gather_dyn(x, cnt_dev, max_blocks, idx, g_in.bsize, g_in.bstride, g_in.boffset,
                                  transpose=True, out=big_stack)
            ops.sparse_scatter_var_dyn(big_q, cnt_dev, max_blocks, idx, x, g_out.bsize, g_out.bstride,
                                       g_out.boffset, add=True, transpose=True)
            return idx

        with torch.cuda.stream(side):
            dyn_step(masks[0])
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph, keep = torch.cuda.CUDAGraph(), []
        with torch.cuda.graph(graph, stream=side):
            for m in masks[:4]:
                keep.append(dyn_step(m))
        for _ in range(2):
            graph.replay()
        fence()
        a, b = ev(), ev()
        reps = max(1, args.steps // 4)
        a.record()
        for _ in range(reps):
            graph.replay()
        b.record()
        fence()
        ms = a.elapsed_time(b) / (reps * 4)
        sync_free = {"value": nB / (ms * 1e-3), "unit": "blocks/s", "ms_per_step": ms,
                     "how": "reduce_mask -> gather_dyn -> scatter_dyn, count read on the device, 4 steps per CUDA graph replay"}
        del big_stack, big_q, graph, keep

    # ---- reduce over ranks: max time, summed blocks ----
    stats = torch.tensor([ms_total, e2e["ms"] if e2e else 0.0], dtype=torch.float64, device=dev)
    sums = torch.tensor([blocks, e2e["blocks"] if e2e else 0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    ms_total, e2e_ms = stats.tolist()
    blocks_all, e2e_blocks_all = sums.tolist()

    global_blocks = None
    if world > 1 and last_counts[0] is not None:
        global_blocks = int(last_counts[0].sum().item())   # from the all-gathered device counts
        assert global_blocks * args.steps == int(blocks_all), (global_blocks, blocks_all)
    if rank == 0:
        peak, peak_kind = measured_peak()
        med = {k: statistics.median(v) for k, v in op_ms.items()}
        alg = {"reduce_mask": bytes_mask, "gather": bytes_gather, "scatter": bytes_scatter}
        gbs = {k: alg[k] / (med[k] * 1e-3) / 1e9 for k in med}
        dom = max(("gather", "scatter"), key=lambda k: med[k])
        kernel_name = {"gather": "planes_gather_tma_tile<__half> (sparse_gather transpose=True)",
                       "scatter": "planes_scatter_simt<atomic,__half,4> (sparse_scatter_var add=True transpose=True)"}[dom]
        # DRAM bytes per active block from one ncu capture of each kernel on a smaller case of the same
        # shape (1,641 blocks; profiles/planes_*_c256_d20.txt), scaled by the blocks of this launch
        # (traffic is proportional to the block count: every block moves the same tile)
        traffic = {"gather": 295860, "scatter": 357910}[dom] * nB
        line = {
            "metric": "sparse block pipeline throughput (reduce_mask -> sparse_gather -> sparse_scatter_var)",
            "value": blocks_all / (ms_total * 1e-3),
            "unit": "blocks/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {
                "workload": "sparse ResNet bottleneck block ops, batch-sharded (BASELINE config 5 without the framework's convs)",
                "x": [N, H, W, C], "per_rank_batch": N, "global_batch": N * world,
                "mask": f"rectangle union, {args.occupancy:.0%} pixel occupancy",
                "bsize": [18, 18], "bstride": [16, 16], "boffset": [-1, -1],
                "active_blocks_per_rank": nB, "candidate_blocks_per_rank": N * g_in.bcount[0] * g_in.bcount[1],
                "l2": "x (2.3 GB per rank) exceeds L2; masks rotate through copies and are evicted by the x traffic between uses",
                "parallelism": f"dp{world}", "global_blocks_per_step": global_blocks if world > 1 else nB,
                "collective": "all-gather of one int32 block count per rank per step (NCCL), off the critical path",
            },
            "ops": {k: {"us": med[k] * 1e3, "algorithmic_bytes": alg[k], "GB/s": gbs[k],
                        "frac_of_" + peak_kind: gbs[k] / peak} for k in med},
            "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": gbs[dom], "peak": peak,
                         "peak_source": peak_kind, "unit": "GB/s", "frac": gbs[dom] / peak,
                         "traffic": traffic, "algorithmic_bytes": alg[dom]},
            "gpu_launches": 3 * args.steps,
            "clocks": clocks.summary(wall0, wall1),
        }
        if sync_free:
            line["sync_free"] = sync_free
        if e2e:
            line["e2e"] = {"value": e2e_blocks_all / (e2e_ms * 1e-3), "unit": "blocks/s",
                           "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                           "steps": e2e["steps"], "ms_per_step": e2e_ms / e2e["steps"],
                           "pipelining": f"{e2e['groups']} image groups on 3 streams (upload / ops / download overlap)"}
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_pipeline(args, mask_h, N, H, W, C, budget_s=args.cpu_budget)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ---- CPU legs ------------------------------------------------------------------------------------

def cpu_pipeline(args, mask_h, N, H, W, C, budget_s=12.0, steps=1):
    """Times the reference CPU functors on a bounded sample: the first image(s) of the batch for
    reduce_mask and the first M active blocks for gather / scatter-add, M grown until one pass takes
    a few seconds.  blocks/s = M / (t_mask * M/nB_image + t_gather + t_scatter)."""
    from oracle import oracle
    kind = "ref" if oracle.have_ref() else "port"
    if kind == "port":
        oracle.build(ref=False)
    o = oracle.get(kind)
    cores = o.max_threads()
    o.set_threads(cores)
    g_in, g_out = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    m1 = np.ascontiguousarray(mask_h[:1])
    t = time.perf_counter()
    idx, cnt = o.reduce_mask(m1, *g_in.as_lists(), tol=0.5, avgpool=False)
    t_mask = time.perf_counter() - t
    nb_img = int(cnt[0])
    x1 = cfg.normal((1, H, W, C), 5, np.float16)
    M, per_block = min(8, nb_img), None
    spent = 0.0
    res = None
    while True:
        c = np.array([M], dtype=np.int32)
        t = time.perf_counter()
        st = o.sparse_gather(x1, c, idx, g_in.bsize, g_in.bstride, g_in.boffset, transpose=True)
        t_g = time.perf_counter() - t
        qh = np.ascontiguousarray(st[:, :, 1:17, 1:17])
        t = time.perf_counter()
        o.sparse_scatter_var(qh, c, idx, x1, g_out.bsize, g_out.bstride, g_out.boffset, add=True,
                             transpose=True)
        t_s = time.perf_counter() - t
        spent += t_g + t_s
        res = (M, t_g, t_s)
        per_block = (t_g + t_s) / M
        nxt = min(nb_img, int(M * 4))
        if nxt == M or spent + per_block * nxt > budget_s:
            break
        M = nxt
    M, t_g, t_s = res
    total = t_mask * (M / max(nb_img, 1)) + t_g + t_s
    return {"value": M / total, "unit": "blocks/s", "cores": cores,
            "kind": "reference" if kind == "ref" else "port",
            "sample": f"image 0 of the batch: reduce_mask on 1 image ({t_mask*1e3:.1f} ms, single thread), "
                      f"gather+scatter-add on its first {M} of {nb_img} active blocks "
                      f"({t_g:.2f} s + {t_s:.2f} s)",
            "us_per_block": {"gather": t_g / M * 1e6, "scatter_add": t_s / M * 1e6}}


def cpu_suite(args):
    """``bench.py --suite cpu``: the reference's CPU functors (compiled from the reference tree when
    available, else the C restatement) on bounded samples of the op-level configurations, all host
    threads.  One JSON line per case; reported beside the GPU numbers, not a target."""
    from oracle import oracle   # the checker, timed here as the CPU baseline (never used by the product)
    kind = "ref" if oracle.have_ref() else "port"
    if kind == "port":
        oracle.build(ref=False)
    o = oracle.get(kind)
    cores = o.max_threads()
    o.set_threads(cores)

    def line(case, seconds, units, unit_name, nbytes, sample):
        print(json.dumps({"case": "cpu_" + case, "kind": "reference" if kind == "ref" else "port", "cores": cores,
                          "seconds": seconds, unit_name + "/s": units / seconds, "GB/s": nbytes / seconds / 1e9,
                          "sample": sample}), flush=True)

    def best(fn, reps=3):
        out = []
        for _ in range(reps):
            t = time.perf_counter()
            fn()
            out.append(time.perf_counter() - t)
        return min(out)

    c2 = cfg.config2(0)
    g = c2["geom"]
    for run in c2["runs"]:
        dt = best(lambda: o.reduce_mask(c2["mask"], *g.as_lists(), tol=run["tol"], avgpool=run["avgpool"]))
        line("reduce_mask_" + ("avg" if run["avgpool"] else "max"), dt, 1, "masks", c2["mask"].nbytes,
             "full [8,800,704] mask, single thread (the functor is not threaded)")
    N, H, W = 8, 512, 512
    g = cfg.halo_geom(H, W)
    idx, cnt = cfg.random_block_list(N, g.bcount, 0.2, seed=20)
    for dtype, tname, C in ((np.float32, "f32", 128), (np.float16, "f16", 128)):
        x = cfg.normal((N, H, W, C), 1, dtype)
        nb = min(int(cnt[0]), 1600)
        m = np.array([nb], np.int32)
        for tr in (False, True):
            dt = best(lambda: o.sparse_gather(x, m, idx, g.bsize, g.bstride, g.boffset, transpose=tr))
            line(f"gather_{tname}_t{int(tr)}", dt, nb, "blocks", 2 * nb * 324 * C * x.itemsize,
                 f"first {nb} blocks of the 20 % list on x [8,512,512,128]")
    C = 64
    base = cfg.normal((N, H, W, C), 2)
    m = np.array([64], np.int32)
    stack = cfg.normal((64, 18, 18, C), 3)
    dt = best(lambda: o.sparse_scatter_var(stack, m, idx, base, g.bsize, g.bstride, g.boffset, add=True, atomic=True), 2)
    line("scatter_f32_add", dt, 64, "blocks", 3 * 64 * 324 * C * 4,
         "first 64 blocks, add=True (one global lock per added element in the reference)")
    gi = cfg.inner_geom(H, W)
    base16 = cfg.normal((N, H, W, C), 4, np.float16)
    nb = min(int(cnt[0]), 1600)
    m = np.array([nb], np.int32)
    stack16 = cfg.normal((nb, C, 16, 16), 5, np.float16)
    dt = best(lambda: o.sparse_scatter_var(stack16, m, idx, base16, gi.bsize, gi.bstride, gi.boffset, add=False,
                                           transpose=True))
    line("scatter_f16_t1_set", dt, nb, "blocks", 2 * nb * 256 * C * 2, f"first {nb} blocks, overwrite, transposed stack")


def refgpu_suite(args):
    """``bench.py --suite refgpu``: the reference's own CUDA kernels recompiled for sm_100a
    (``make -C oracle refgpu``) timed beside this library's kernels on the same device, inputs and
    timing protocol (CUDA events, L2 flushed between launches, median).  fp32, as the reference is
    fp32-only; the last cases add this library's fp16 path on the same shapes.  Informational: the
    parity authority stays the CPU functors."""
    import torch
    from oracle import refgpu   # test / benchmark infrastructure, never used by the product
    from sbnet_b200 import build, ops
    from sbnet_b200.opbench import Timer, _peak
    if not refgpu.available():
        try:
            refgpu.build()
        except Exception:
            pass
    if not refgpu.available():
        print(json.dumps({"suite": "refgpu", "unavailable": "reference CUDA kernels not built (no reference tree, no prebuilt library)"}))
        return
    build.build_library()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tm = Timer(torch, dev, max(args.steps if args.steps != 100 else 20, 5), max(args.warmup, 3))
    peak, kind = _peak()

    def line(case, nbytes, ref_ms, ours_ms, extra=None):
        extra = extra or {}
        rbytes = extra.get("ref_algorithmic_bytes", nbytes)   # differs when this library runs fp16
        d = {"case": case, "algorithmic_bytes": int(nbytes), "ref_us": ref_ms * 1e3, "ours_us": ours_ms * 1e3,
             "speedup": ref_ms / ours_ms, "ref_GB/s": rbytes / ref_ms / 1e6, "ours_GB/s": nbytes / ours_ms / 1e6,
             "ref_frac_of_" + kind: rbytes / ref_ms / 1e6 / peak, "ours_frac_of_" + kind: nbytes / ours_ms / 1e6 / peak}
        d.update(extra)
        print(json.dumps(d), flush=True)

    # ---- reduce_mask at bird's-eye-view scale (two reference launches: zero the counter, reduce) ----
    c2 = cfg.config2(0)
    g = c2["geom"]
    mask = torch.from_numpy(c2["mask"]).to(dev)
    ridx = torch.zeros((8 * g.bcount[0] * g.bcount[1], 3), dtype=torch.int16, device=dev)
    rcnt = torch.zeros(1, dtype=torch.int32, device=dev)
    for run in c2["runs"]:
        idx, cnt = ops.reduce_mask(mask, *g.as_lists(), tol=run["tol"], avgpool=run["avgpool"])
        nb = int(cnt[0])
        nbytes = cfg.algorithmic_bytes("reduce_mask", nB=nb, geom=g, C=1, itemsize=4, U=0, N=8, H=800, W=704, count=nb)
        r, _ = tm.run(lambda: refgpu.reduce_mask_launch(mask, g.bcount, g.bsize, g.bstride, g.boffset, run["tol"],
                                                        run["avgpool"], ridx, rcnt))
        o, _ = tm.run(lambda: ops.reduce_mask_async(mask, *g.as_lists(), tol=run["tol"], avgpool=run["avgpool"]))
        line("reduce_mask_" + ("avg" if run["avgpool"] else "max"), nbytes, r, o, {"active": nb, "ref_active": int(rcnt.item())})
    del mask

    # ---- sparse_gather on [8,512,512,128] fp32 ----
    N, H, W, C = 8, 512, 512, 128
    g = cfg.halo_geom(H, W)
    x = torch.randn((N, H, W, C), device=dev)
    for dens in (0.05, 0.20, 0.50):
        idx_h, cnt_h = cfg.random_block_list(N, g.bcount, dens, seed=int(dens * 100))
        nb = int(cnt_h[0])
        U = cfg.union_pixels(idx_h, nb, g, N, H, W)
        idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
        nbytes = cfg.algorithmic_bytes("gather", nB=nb, geom=g, C=C, itemsize=4, U=U)
        for tr in (False, True):
            out = torch.empty((nb, C, 18, 18) if tr else (nb, 18, 18, C), device=dev)
            r, _ = tm.run(lambda: refgpu.sparse_gather(x, nb, idx, g.bsize, g.bstride, g.boffset, tr, out))
            o, _ = tm.run(lambda: ops.sparse_gather(x, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=tr, out=out))
            line(f"gather_f32_t{int(tr)}_d{int(dens * 100)}", nbytes, r, o, {"blocks": nb})
            del out
    del x

    # ---- sparse_scatter_var on [8,512,512,64] fp32: atomic add with halos; transposed overwrite ----
    C = 64
    gi = cfg.inner_geom(H, W)
    base = torch.randn((N, H, W, C), device=dev)
    for dens in (0.05, 0.20, 0.50):
        idx_h, cnt_h = cfg.random_block_list(N, g.bcount, dens, seed=int(dens * 100) + 1)
        nb = int(cnt_h[0])
        idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
        stack = torch.randn((nb, 18, 18, C), device=dev)
        nbytes = cfg.algorithmic_bytes("scatter_add", nB=nb, geom=g, C=C, itemsize=4,
                                       U=cfg.union_pixels(idx_h, nb, g, N, H, W))
        r, _ = tm.run(lambda: refgpu.sparse_scatter_var(stack, nb, idx, base, g.bsize, g.bstride, g.boffset,
                                                        add=True, atomic=True))
        o, _ = tm.run(lambda: ops.sparse_scatter_var(stack, cnt, idx, base, g.bsize, g.bstride, g.boffset,
                                                     add=True, atomic=True))
        line(f"scatter_var_f32_atomic_d{int(dens * 100)}", nbytes, r, o, {"blocks": nb})
        stack = torch.randn((nb, C, 16, 16), device=dev)
        nbytes = cfg.algorithmic_bytes("scatter", nB=nb, geom=gi, C=C, itemsize=4,
                                       U=cfg.union_pixels(idx_h, nb, gi, N, H, W))
        r, _ = tm.run(lambda: refgpu.sparse_scatter_var(stack, nb, idx, base, gi.bsize, gi.bstride, gi.boffset,
                                                        add=False, transpose=True))
        o, _ = tm.run(lambda: ops.sparse_scatter_var(stack, cnt, idx, base, gi.bsize, gi.bstride, gi.boffset,
                                                     add=False, transpose=True))
        line(f"scatter_var_f32_t1_set_d{int(dens * 100)}", nbytes, r, o, {"blocks": nb})
        del stack
    del base

    # ---- small blocks: 8x8 on a 6-pixel pitch and 10x10 on an 8-pixel pitch over [8,512,512,64], 20 % ----
    x = torch.randn((8, 512, 512, 64), device=dev)
    for b, stride in ((8, 6), (10, 8)):
        gs = cfg.geom_for(512, 512, (b, b), (stride, stride), (-1, -1))
        idx_h, cnt_h = cfg.random_block_list(8, gs.bcount, 0.20, seed=b)
        nb = int(cnt_h[0])
        U = cfg.union_pixels(idx_h, nb, gs, 8, 512, 512)
        idx, cnt = torch.from_numpy(idx_h).to(dev), torch.from_numpy(cnt_h)
        for tr in (False, True):
            out = torch.empty((nb, 64, b, b) if tr else (nb, b, b, 64), device=dev)
            nbytes = cfg.algorithmic_bytes("gather", nB=nb, geom=gs, C=64, itemsize=4, U=U)
            r, _ = tm.run(lambda: refgpu.sparse_gather(x, nb, idx, gs.bsize, gs.bstride, gs.boffset, tr, out))
            o, _ = tm.run(lambda: ops.sparse_gather(x, cnt, idx, gs.bsize, gs.bstride, gs.boffset, transpose=tr, out=out))
            line(f"gather_f32_t{int(tr)}_b{b}_d20", nbytes, r, o, {"blocks": nb})
            nbytes = cfg.algorithmic_bytes("scatter_add", nB=nb, geom=gs, C=64, itemsize=4, U=U)
            r, _ = tm.run(lambda: refgpu.sparse_scatter_var(out, nb, idx, x, gs.bsize, gs.bstride, gs.boffset,
                                                            add=True, atomic=True, transpose=tr))
            o, _ = tm.run(lambda: ops.sparse_scatter_var(out, cnt, idx, x, gs.bsize, gs.bstride, gs.boffset, add=True,
                                                         atomic=True, transpose=tr))
            line(f"scatter_var_f32_t{int(tr)}_atomic_b{b}_d20", nbytes, r, o, {"blocks": nb})
            del out
    del x

    # ---- the sparse bottleneck's block ops, 8 of the 32 images: [8,400,352,256] ----
    # reference fp32 (its only type) against this library's fp32 and fp16 paths on the same block list
    N, H, W, C = 8, 400, 352, 256
    g, gi = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
    mask = torch.from_numpy(cfg.rect_union_mask(N, H, W, 7, n_rects=None, occupancy=0.10)).to(dev)
    idx, cnt = ops.reduce_mask(mask, *g.as_lists(), tol=0.5, avgpool=False)
    nb = int(cnt[0])
    idx_h = idx.cpu().numpy()
    x32 = torch.randn((N, H, W, C), device=dev)
    x16 = x32.half()
    for t, tname, sz in ((x32, "f32", 4), (x16, "f16", 2)):
        out = torch.empty((nb, C, 18, 18), dtype=t.dtype, device=dev)
        nbytes = cfg.algorithmic_bytes("gather", nB=nb, geom=g, C=C, itemsize=sz, U=cfg.union_pixels(idx_h, nb, g, N, H, W))
        if sz == 4:
            r_g, _ = tm.run(lambda: refgpu.sparse_gather(t, nb, idx, g.bsize, g.bstride, g.boffset, True, out))
            nbytes32 = nbytes
        o, _ = tm.run(lambda: ops.sparse_gather(t, cnt, idx, g.bsize, g.bstride, g.boffset, transpose=True, out=out))
        line(f"bottleneck_gather_t1_ours_{tname}_vs_ref_f32", nbytes, r_g, o,
             {"blocks": nb, "ref_algorithmic_bytes": int(nbytes32)})
        stack = torch.randn((nb, C, 16, 16), device=dev).to(t.dtype)
        nbytes = cfg.algorithmic_bytes("scatter_add", nB=nb, geom=gi, C=C, itemsize=sz,
                                       U=cfg.union_pixels(idx_h, nb, gi, N, H, W))
        if sz == 4:
            r_s, _ = tm.run(lambda: refgpu.sparse_scatter_var(stack, nb, idx, t, gi.bsize, gi.bstride, gi.boffset,
                                                              add=True, transpose=True))
            nbytes32s = nbytes
        o, _ = tm.run(lambda: ops.sparse_scatter_var(stack, cnt, idx, t, gi.bsize, gi.bstride, gi.boffset, add=True,
                                                     transpose=True))
        line(f"bottleneck_scatter_add_t1_ours_{tname}_vs_ref_f32", nbytes, r_s, o,
             {"blocks": nb, "ref_algorithmic_bytes": int(nbytes32s)})
        del out, stack


def run_reference(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    N, H, W, C, mask_h = make_host_inputs(args, 0, world)
    vals = []
    base = None
    t_all = time.perf_counter()
    step_ms = []
    for _ in range(args.warmup + args.steps):
        t_step = time.perf_counter()
        base = cpu_pipeline(args, mask_h, N, H, W, C, budget_s=args.cpu_budget / 2)
        step_ms.append((time.perf_counter() - t_step) * 1e3)
        vals.append(base["value"])
        if time.perf_counter() - t_all > 150:
            break
    timed = vals[min(args.warmup, len(vals) - 1):]
    value = statistics.median(timed)
    base["value"] = value
    g_in = cfg.halo_geom(H, W)
    line = {
        "impl": "reference",
        "metric": "sparse block pipeline throughput (reduce_mask -> sparse_gather -> sparse_scatter_var)",
        "value": value, "unit": "blocks/s", "n_gpus": world, "steps": len(timed),
        "warmup": min(args.warmup, len(vals) - 1), "ms_per_step": statistics.median(step_ms),
        "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "sparse ResNet bottleneck block ops (BASELINE config 5 without the framework's convs), CPU functors on a bounded sample",
                   "x": [N, H, W, C], "mask": f"rectangle union, {args.occupancy:.0%} pixel occupancy",
                   "bsize": [18, 18], "bstride": [16, 16], "boffset": [-1, -1],
                   "candidate_blocks_per_rank": N * g_in.bcount[0] * g_in.bcount[1]},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "blocks/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak")
    ap.add_argument("--occupancy", type=float, default=0.10)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--height", type=int, default=400)
    ap.add_argument("--width", type=int, default=352)
    ap.add_argument("--channels", type=int, default=256)
    ap.add_argument("--e2e-steps", type=int, default=4)
    ap.add_argument("--e2e-groups", type=int, default=8)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-sync-free", action="store_true")
    ap.add_argument("--cpu-budget", type=float, default=12.0)
    ap.add_argument("--suite", choices=["ops", "one", "resblock", "cpu", "refgpu"], default=None)
    ap.add_argument("--case", default="gather_f16_t1")
    ap.add_argument("--density", type=float, default=0.2)
    ap.add_argument("--one-channels", type=int, default=None)
    ap.add_argument("--one-block", default=None, help="--suite one: square block SIZE,STRIDE,OFFSET instead of 18,16,-1")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.suite == "refgpu":
        refgpu_suite(args)
    elif args.suite == "cpu":
        cpu_suite(args)
    elif args.suite in ("ops", "one", "resblock"):
        from sbnet_b200 import opbench
        opbench.main(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
