#!/usr/bin/env python
"""Benchmark of the block-op hot path: reduce_mask -> sparse_gather -> sparse_scatter_var.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--occupancy 0.1] [--scaling strong|weak] [--suite ops|one|resblock|topleft|cpu|refgpu]

Workload (one "step" = one pass of the three ops over one batch): the sparse ResNet-bottleneck
configuration -- x fp16 [32,400,352,256], a rectangle-union mask, 18x18 windows on a 16 pixel pitch
with a one pixel halo: reduce_mask (max, tol 0.5) -> sparse_gather(transpose=True) ->
sparse_scatter_var(add=True, transpose=True, 16x16 interior) of a conv-output-shaped stack back onto
x.  The dense convolutions between gather and scatter belong to the host framework and are not part
of this library, so they are not in the step.  Data is synthetic and seeded (sbnet_b200/configs.py).

One JSON line is printed by rank 0.  `value` is blocks/s over all ranks with inputs resident in HBM;
with N GPUs ONE batch of 32 images is sharded 32/N per rank (`"scaling": "strong"`, the configured
split) and the weak-scaling figure -- a full batch per rank -- is reported beside it under `weak`;
`e2e` is the same pipeline fed from pinned host buffers with the copies inside the timed region;
`roofline` describes the kernel that takes the largest share of the step; `suite` (1 GPU) is the
op-level table of the other configurations (reduce_mask at bird's-eye-view scale with its yardsticks,
every gather and scatter cell at 5 / 20 / 50 %, the pipeline at 30 % occupancy); `cpu_baseline` is
the reference's CPU functors timed on this machine's cores on a bounded sample.

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

TRAFFIC_PROFILES = {
    # dominant kernel -> the committed profiler summary its DRAM traffic per block is read from
    "gather": "planes_gather_tma_tile_f16_c256_d20.txt",
    "scatter": "planes_scatter_simt_f16_add_c256_d20.txt",
}


def traffic_per_block(op):
    """DRAM bytes per active block of the dominant kernel, read from the committed summary of one
    profiler capture of that kernel on a smaller case of the same shape (``DRAM read`` + ``DRAM write``
    divided by ``blocks in this launch``).  Every block moves the same tile, so traffic is proportional
    to the block count.  Returns (bytes per block, file name) or (None, file name)."""
    import re
    name = TRAFFIC_PROFILES[op]
    try:
        text = open(os.path.join(ROOT, "profiles", name)).read()
        unit = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
        rd = re.search(r"DRAM read\s+([0-9.]+)\s+(\w+)", text)
        wr = re.search(r"DRAM write\s+([0-9.]+)\s+(\w+)", text)
        nb = re.search(r"blocks in this launch\s+(\d+)", text)
        total = float(rd.group(1)) * unit[rd.group(2)] + float(wr.group(1)) * unit[wr.group(2)]
        return total / int(nb.group(1)), name
    except Exception:
        return None, name


def bind_cores(local, per_node):
    """Gives this rank its own slice of the cores the process may run on, before any pinned buffer is
    allocated (first touch then lands near those cores).  Returns the cores, or None when unsupported."""
    try:
        allowed = sorted(os.sched_getaffinity(0))
        per = len(allowed) // max(per_node, 1)
        if per_node <= 1 or per < 1:
            return allowed
        mine = allowed[local * per:(local + 1) * per]
        os.sched_setaffinity(0, mine)
        return mine
    except Exception:
        return None


class FastEvents:
    """cudaEventRecord / cudaStreamWaitEvent on torch's events and streams through ctypes: torch's own
    methods cost 4-7 us of interpreter time per call, which is a tenth of a rank's step when eight GPUs
    share one batch.  Falls back to the torch methods where the runtime library cannot be opened."""

    def __init__(self, torch):
        import ctypes
        self.rt = None
        for name in ("libcudart.so.12", "libcudart.so"):
            try:
                rt = ctypes.CDLL(name)
                rt.cudaEventRecord.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
                rt.cudaStreamWaitEvent.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint]
                self.rt = rt
                break
            except OSError:
                continue

    def record(self, event, stream):
        if self.rt is None or not event.cuda_event:     # a torch event gets its handle at its first record
            event.record(stream)
        elif self.rt.cudaEventRecord(event.cuda_event, stream.cuda_stream) != 0:
            raise RuntimeError("cudaEventRecord failed")

    def wait(self, stream, event):
        if self.rt is None:
            stream.wait_event(event)
        elif self.rt.cudaStreamWaitEvent(stream.cuda_stream, event.cuda_event, 0) != 0:
            raise RuntimeError("cudaStreamWaitEvent failed")


class Workload:
    """Device-resident inputs of one rank for `n_images` images at one mask occupancy."""

    def __init__(self, torch, dev, args, first_image, n_images, occupancy, x_all, gen):
        H, W, C = args.height, args.width, args.channels
        self.N, self.H, self.W, self.C = n_images, H, W, C
        self.g_in, self.g_out = cfg.halo_geom(H, W), cfg.inner_geom(H, W)
        # image n of the global batch always gets seed 7 + n, whichever rank owns it
        self.mask_h = cfg.rect_union_mask(n_images, H, W, seed=7 + first_image, occupancy=occupancy)
        self.nB, self.U_in, self.U_out, _ = union_stats(self.mask_h, self.g_in, self.g_out, n_images, H, W)
        self.x = x_all[:n_images]
        # conv-output-shaped stack [nB,C,16,16]; small magnitudes so K accumulations stay far from fp16 max
        self.q = (torch.randn((self.nB, C, 16, 16), generator=gen, device=dev, dtype=torch.float32) * 0.01).half()
        self.stack = torch.empty((self.nB, C, 18, 18), dtype=torch.float16, device=dev)
        # masks rotate through enough copies to exceed L2 on their own
        n_masks = max(2, int(L2_BYTES // self.mask_h.nbytes) + 2)
        self.masks = [torch.from_numpy(self.mask_h).to(dev) for _ in range(min(n_masks, 8))]
        sz = 2
        self.bytes = {
            "reduce_mask": cfg.algorithmic_bytes("reduce_mask", nB=self.nB, geom=self.g_in, C=1, itemsize=4, U=0,
                                                 N=n_images, H=H, W=W, count=self.nB),
            "gather": cfg.algorithmic_bytes("gather", nB=self.nB, geom=self.g_in, C=C, itemsize=sz, U=self.U_in),
            "scatter": cfg.algorithmic_bytes("scatter_add", nB=self.nB, geom=self.g_out, C=C, itemsize=sz, U=self.U_out),
        }


def run_pipeline(torch, dist, ops, w, steps, warmup, world, exchange=None, marks=False, common_start=True,
                 prefetch=False, ahead=2):
    """`warmup` untimed and `steps` timed passes of reduce_mask -> gather -> scatter over workload `w`.
    Returns (ms of the timed region on this rank, blocks processed, per-op event times or None, wall-clock
    window).  The timed steps carry no per-op events (they cost host time between the launches); a
    separate call with marks=True takes those."""
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    g_in, g_out = w.g_in, w.g_out
    yield_core = world > 1

    main = torch.cuda.current_stream()
    side = torch.cuda.Stream(priority=-1) if prefetch else None
    # the same buffers and geometry every step: arguments are validated once (ops.bind_*), which takes
    # about 7 us of interpreter time off each call -- it matters when a rank's step is only tens of us.
    # The mask has been resident since start-up and the kernel queued before a reduce_mask never writes
    # it, so its loads may overlap that kernel's tail (mask_stable).
    mask_fn = ops.bind_reduce_mask(w.masks[0], *g_in.as_lists(), tol=0.5, avgpool=False, mask_stable=True,
                                   yield_core=yield_core, stream=side.cuda_stream if side is not None else None,
                                   wait=side is None)
    mask_nowait = ops.bind_reduce_mask(w.masks[0], *g_in.as_lists(), tol=0.5, avgpool=False, mask_stable=True,
                                       wait=False) if marks else None
    gather_fn = ops.bind_sparse_gather(w.x, w.stack, g_in.bsize, g_in.bstride, g_in.boffset, transpose=True)
    scatter_fn = ops.bind_sparse_scatter_var(w.q, w.x, g_out.bsize, g_out.bstride, g_out.boffset, add=True, transpose=True)
    fast = FastEvents(torch)
    RING = 8
    ready_ev = [torch.cuda.Event() for _ in range(RING)]  # index list of step j written (side stream)
    free_ev = [torch.cuda.Event() for _ in range(RING)]   # index list of step j read for the last time (main stream)
    # the index lists rotate through a few buffers allocated once (a fresh tensor per step would send the
    # first pass over a new batch through the caching allocator's slow path every few steps); a buffer is
    # rewritten only after the scatter that read it last, which the side stream waits for
    idx_ring = [torch.empty((w.N * g_in.bcount[0] * g_in.bcount[1], 3), dtype=torch.int16, device=w.x.device)
                for _ in range(RING)] if side is not None else None
    launched = {}   # step -> (idx, count, event): reduce_mask calls issued ahead on the side stream
    AHEAD = ahead   # steps the masks run ahead: the count of step i+1 is on the host before it is needed
    assert 1 <= AHEAD < RING - 1

    def launch_mask(j, ex):
        if j >= RING:
            fast.wait(side, free_ev[j % RING])             # recorded behind the scatter of step j - RING
        idx, cnt, _ = mask_fn(w.masks[j % len(w.masks)], ex.slot(j, side) if ex is not None else None,
                              idx_ring[j % RING])          # returns at once
        ev = ready_ev[j % RING]
        fast.record(ev, side)
        launched[j] = (idx, cnt, ev)

    def step(i, mk=None, ex=None):
        if side is None:
            if mk is not None:
                # instrumented pass: the op's device time is taken between events around a launch that does not
                # wait for the count (launch gap + kernel); the count's way to the host is not part of it
                mk[0].record()
                idx, cnt, _ = mask_nowait(w.masks[i % len(w.masks)], None)
                mk[1].record()
                nb = ops.wait_count(cnt)
            else:
                idx, cnt, _ = mask_fn(w.masks[i % len(w.masks)], ex.slot(i) if ex is not None else None)
                nb = int(cnt[0])
        else:
            # software pipelining over steps: reduce_mask depends on nothing of the steps before it, so
            # the masks of the next steps are issued ahead on a second stream and their counts come back
            # through pinned memory without the host ever waiting inside a call.  Every step issues
            # exactly one reduce_mask, one gather and one scatter (the last steps' reduce_masks serve
            # steps that are never run)
            for j in range(i, i + AHEAD):          # only at the very first step is anything missing here
                if j not in launched:
                    launch_mask(j, ex)
            idx, cnt, ready = launched.pop(i)
            nb = ops.wait_count(cnt)
            fast.wait(main, ready)                 # the gather reads the index list written on the side stream
        assert nb == w.nB, (nb, w.nB)
        if mk is not None:
            mk[2].record()
        gather_fn(cnt, idx)
        if mk is not None:
            mk[3].record()
        if side is not None:
            launch_mask(i + AHEAD, ex)
        scatter_fn(cnt, idx)
        if side is not None:
            fast.record(free_ev[i % RING], main)
        if mk is not None:
            mk[4].record()
        if ex is not None:
            ex.step_done(i, warmup + steps)
        return nb

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(warmup):
        step(i, ex=exchange)
    fence()
    mks = [[ev() for _ in range(5)] for _ in range(steps)] if marks else None
    t0, t1 = ev(), ev()
    if world > 1 and common_start:
        # every rank enters the timed region at the same wall-clock instant (one node, one clock), so
        # the barrier's exit skew is not part of a region that lasts only milliseconds
        go = torch.zeros(1, dtype=torch.float64, device=w.x.device)
        if dist.get_rank() == 0:
            go[0] = time.time() + 0.01
        dist.broadcast(go, 0)
        t_go = float(go.item())
        while time.time() < t_go:
            pass
    wall0 = time.time()
    t0.record()
    blocks = 0
    for i in range(steps):
        blocks += step(warmup + i, mks[i] if marks else None, exchange)
    t1.record()
    run_pipeline.host_issue_s = time.time() - wall0     # how long the host took to queue the timed steps
    torch.cuda.synchronize()
    wall1 = time.time()
    fence()
    ms = t0.elapsed_time(t1)
    op_ms = None
    if marks:
        op_ms = {"reduce_mask": [m[0].elapsed_time(m[1]) for m in mks], "gather": [m[2].elapsed_time(m[3]) for m in mks],
                 "scatter": [m[3].elapsed_time(m[4]) for m in mks]}
    return ms, blocks, op_ms, (wall0, wall1)


def run_ours(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cores = bind_cores(local, int(os.environ.get("LOCAL_WORLD_SIZE", str(world))))
    import torch
    import torch.distributed as dist
    from sbnet_b200 import build, lib, ops
    from sbnet_b200 import dist as sbdist
    from sbnet_b200.dist import shard_bounds

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in the product)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if rank == 0:
        build.build_library()
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # the communicator's banner ("NCCL version ...") goes to the process's stdout, which is to carry the one
        # JSON line and nothing else: file descriptor 1 points at stderr while the communicator comes up
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    lib.load()

    H, W, C = args.height, args.width, args.channels
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    # the configured split: ONE batch of `--batch` images sharded over the ranks (strong scaling); the
    # weak-scaling figure (every rank a full batch of its own) is measured beside it when there are peers
    lo, hi = shard_bounds(args.batch, world, rank)
    n_strong = max(hi - lo, 1)
    n_alloc = args.batch if (world > 1 and not args.no_weak) or args.scaling == "weak" else n_strong
    x_all = torch.empty((n_alloc, H, W, C), dtype=torch.float16, device=dev)
    for n in range(n_alloc):  # generated in slices: a one-shot fp32 randn of this size would double the footprint
        x_all[n] = torch.randn((H, W, C), generator=gen, device=dev, dtype=torch.float32).half()
    if args.scaling == "strong":
        main_w = Workload(torch, dev, args, lo, n_strong, args.occupancy, x_all, gen)
    else:
        main_w = Workload(torch, dev, args, rank * args.batch, args.batch, args.occupancy, x_all, gen)
    torch.cuda.synchronize()

    def exchange():
        # The only exchange of the path: every rank's block count per step, read from device memory.
        return sbdist.CountExchange(dev, depth=32, timeout_s=60.0) if world > 1 else None

    clocks = ClockSampler(local).start()
    # One untimed rehearsal of the pass (same loop, same exchange protocol): the first uses of the streams, events,
    # the collective inside the loop and the allocator's pools happen here.  Without it single ranks were seen to
    # lose several milliseconds once, somewhere in their first pass, which is a third of a 20 ms timed region.
    ex = exchange()
    run_pipeline(torch, dist, ops, main_w, min(args.steps, 50), args.warmup, world, ex, prefetch=not args.in_order)
    if ex is not None:
        ex.finish()
    ex = exchange()
    ms_total, blocks, _, (wall0, _) = run_pipeline(torch, dist, ops, main_w, args.steps, args.warmup, world, ex,
                                                   prefetch=not args.in_order)
    global_counts = ex.finish() if ex is not None else None
    # a short timed region may fall between two clock samples: keep the same load running (untimed)
    # until at least half a second of it has been sampled; the per-op event times come from these passes
    op_ms = {"reduce_mask": [], "gather": [], "scatter": []}
    while True:
        _, _, more, _ = run_pipeline(torch, dist, ops, main_w, min(args.steps, 25), 1, 1, None, marks=True)
        for k in op_ms:
            op_ms[k] += more[k]
        if time.time() - wall0 >= 0.5:
            break
    wall1 = time.time()
    clocks.stop()
    if world > 1:
        dist.barrier()

    # ---- the other scaling mode beside it (per-rank batch fixed / one batch split), N > 1 only ----
    other = None
    if world > 1 and not args.no_weak:
        if args.scaling == "strong":
            ow = Workload(torch, dev, args, rank * args.batch, args.batch, args.occupancy, x_all, gen)
        else:
            ow = Workload(torch, dev, args, lo, n_strong, args.occupancy, x_all, gen)
        oex = exchange()
        oms, oblocks, _, _ = run_pipeline(torch, dist, ops, ow, args.steps, args.warmup, world, oex,
                                          prefetch=not args.in_order)
        oex.finish()
        other = (oms, oblocks, ow.N)
        del ow

    # ---- end to end: host buffers in, host result out, copies inside the timed region ----
    e2e = run_e2e(torch, dist, ops, args, main_w, world) if not args.no_e2e else None
    sync_free = run_sync_free(torch, ops, args, main_w) if world == 1 and not args.no_sync_free else None

    # ---- the configured op-level cells and the 30 % pipeline, single GPU only ----
    suite = None
    if world == 1 and not args.no_suite:
        import bench_ops
        suite = {}
        w30 = Workload(torch, dev, args, 0, main_w.N, 0.30, x_all, gen)
        ms30, b30, op30, _ = run_pipeline(torch, dist, ops, w30, 20, 5, 1, None, marks=True)
        peak, peak_kind = measured_peak()
        for k in ("reduce_mask", "gather", "scatter"):
            med = statistics.median(op30[k])
            gbs = w30.bytes[k] / (med * 1e-3) / 1e9
            suite[f"c5_occ30_{k}"] = {"us": round(med * 1e3, 2), "us_min": round(min(op30[k]) * 1e3, 2),
                                      "algorithmic_bytes": int(w30.bytes[k]), "GB/s": round(gbs, 1),
                                      "frac_of_" + peak_kind: round(gbs / peak, 4), "blocks": w30.nB}
        suite["c5_occ30_step"] = {"us": round(ms30 / 20 * 1e3, 2), "blocks": w30.nB, "blocks/s": round(b30 / (ms30 * 1e-3))}
        del w30
        torch.cuda.empty_cache()
        suite.update(bench_ops.suite_table(torch, dev, steps=20, warmup=5, quiet=True, other_shapes=True))

    # ---- reduce over ranks: max time, summed blocks; per-op medians of the slowest rank ----
    med_local = [statistics.median(op_ms[k]) for k in ("reduce_mask", "gather", "scatter")]
    stats = torch.tensor([ms_total, e2e["ms"] if e2e else 0.0, other[0] if other else 0.0] + med_local,
                         dtype=torch.float64, device=dev)
    sums = torch.tensor([blocks, e2e["blocks"] if e2e else 0, other[1] if other else 0], dtype=torch.float64, device=dev)
    per_rank = None
    if world > 1:
        gathered = [torch.zeros_like(stats) for _ in range(world)]
        dist.all_gather(gathered, stats)
        per_rank = torch.stack(gathered).cpu().tolist()
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    ms_total, e2e_ms, other_ms = stats.tolist()[:3]
    med_slowest = dict(zip(("reduce_mask", "gather", "scatter"), stats.tolist()[3:6]))
    blocks_all, e2e_blocks_all, other_blocks_all = sums.tolist()
    e2e_rates = None
    if e2e and world > 1:
        t = torch.tensor([e2e["h2d"] / (e2e["ms"] / e2e["steps"] * 1e-3) / 1e9, e2e["d2h"] / (e2e["ms"] / e2e["steps"] * 1e-3) / 1e9],
                         dtype=torch.float64, device=dev)
        g = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(g, t)
        e2e_rates = [[round(v, 2) for v in r] for r in torch.stack(g).cpu().tolist()]

    global_blocks = None
    if global_counts:
        # the timed steps only: a partly filled last ring also reports its unused slots
        per_step = [sum(v) for k, v in sorted(global_counts.items()) if args.warmup <= k < args.warmup + args.steps]
        global_blocks = per_step[0]
        assert len(per_step) == args.steps and all(p == global_blocks for p in per_step) \
            and global_blocks * args.steps == int(blocks_all), \
            (per_step[:4], blocks_all)
    if rank == 0:
        peak, peak_kind = measured_peak()
        w = main_w
        med0 = dict(zip(("reduce_mask", "gather", "scatter"), med_local))
        gbs = {k: w.bytes[k] / (med_slowest[k] * 1e-3) / 1e9 for k in med_slowest}
        dom = max(("gather", "scatter"), key=lambda k: med_slowest[k])
        kernel_name = {"gather": "planes_gather_tma_tile<__half> (sparse_gather transpose=True)",
                       "scatter": "planes_scatter_simt<atomic,__half,4> (sparse_scatter_var add=True transpose=True)"}[dom]
        per_block, source = traffic_per_block(dom)
        line = {
            "metric": "sparse block pipeline throughput (reduce_mask -> sparse_gather -> sparse_scatter_var)",
            "value": blocks_all / (ms_total * 1e-3),
            "unit": "blocks/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {
                "workload": "sparse ResNet bottleneck block ops, one batch sharded over the GPUs (BASELINE config 5 without the framework's convs)"
                            if args.scaling == "strong" else
                            "sparse ResNet bottleneck block ops, one full batch per GPU (BASELINE config 5 without the framework's convs)",
                "x": [w.N, H, W, C], "per_rank_batch": w.N,
                "global_batch": args.batch if args.scaling == "strong" else args.batch * world,
                "mask": f"rectangle union, {args.occupancy:.0%} pixel occupancy",
                "bsize": [18, 18], "bstride": [16, 16], "boffset": [-1, -1],
                "active_blocks_per_rank": w.nB, "candidate_blocks_per_rank": w.N * w.g_in.bcount[0] * w.g_in.bcount[1],
                "l2": "x (72 MB per image) exceeds L2 from two images on; masks rotate through copies and are evicted by the x traffic between uses",
                "parallelism": f"dp{world}", "global_blocks_per_step": global_blocks if world > 1 else w.nB,
                "collective": "all-gather of the ranks' int32 block counts, 32 steps per call (NCCL), off the critical path",
                "rehearsal": "one untimed pass of min(steps, 50) steps precedes the warm-up and the timed steps",
            },
            "ops": {k: {"us": med_slowest[k] * 1e3, "us_rank0": med0[k] * 1e3, "algorithmic_bytes": w.bytes[k], "GB/s": gbs[k],
                        "frac_of_" + peak_kind: gbs[k] / peak} for k in med_slowest},
            "ops_note": "median CUDA-event time per op on the slowest rank, from instrumented in-order passes of the same "
                        "steps; reduce_mask: events around a launch that does not wait for the count (launch gap + kernel; "
                        "the suite's c2 rows time the call with its count read-back)",
            "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": gbs[dom], "peak": peak,
                         "peak_source": peak_kind, "unit": "GB/s", "frac": gbs[dom] / peak,
                         "traffic": per_block * w.nB if per_block else None, "traffic_source": "profiles/" + source,
                         "algorithmic_bytes": w.bytes[dom]},
            "gpu_launches": 3 * args.steps,
            "clocks": clocks.summary(wall0, wall1),
            "host_cores_per_rank": len(cores) if cores else None,
        }
        if other:
            mode = "weak" if args.scaling == "strong" else "strong"
            line[mode] = {"value": other_blocks_all / (other_ms * 1e-3), "unit": "blocks/s", "ms_per_step": other_ms / args.steps,
                          "per_rank_batch": other[2],
                          "global_batch": args.batch * world if mode == "weak" else args.batch}
        if per_rank:
            line["per_rank"] = {"ms_per_step": [r[0] / args.steps for r in per_rank],
                                "reduce_mask_us": [r[3] * 1e3 for r in per_rank],
                                "gather_us": [r[4] * 1e3 for r in per_rank], "scatter_us": [r[5] * 1e3 for r in per_rank]}
        if sync_free:
            line["sync_free"] = sync_free
        if e2e:
            line["e2e"] = {"value": e2e_blocks_all / (e2e_ms * 1e-3), "unit": "blocks/s",
                           "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                           "steps": e2e["steps"], "ms_per_step": e2e_ms / e2e["steps"],
                           "pipelining": f"{e2e['groups']} image groups on 3 streams (upload / ops / download overlap)"}
            if e2e_rates:
                line["e2e"]["per_rank_h2d_d2h_GB/s"] = e2e_rates
        if suite:
            line["suite"] = suite
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_pipeline(args, w.mask_h, w.N, H, W, C, budget_s=args.cpu_budget)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_e2e(torch, dist, ops, args, w, world):
    """The same pipeline fed from pinned host buffers.  The batch is cut into image groups; three streams
    (host->device, compute, device->host) are chained with events so that the upload of group g+1, the
    ops on group g and the download of group g-1 overlap.  PCIe is full duplex, so a step costs about
    max(upload, download) instead of their sum.  Every byte of mask, x and the conv-output stack goes up
    and every byte of the updated x comes down inside the timed region, every step."""
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    N, H, W, C = w.N, w.H, w.W, w.C
    g_in, g_out, x, q, stack = w.g_in, w.g_out, w.x, w.q, w.stack
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    G = max(1, min(args.e2e_groups, N))
    bounds = [(N * g) // G for g in range(G + 1)]
    per_image = per_image_blocks(w.mask_h, g_in, N, H, W)
    qoff = [0]
    for g in range(G):
        qoff.append(qoff[-1] + int(per_image[bounds[g]:bounds[g + 1]].sum()))
    hx = torch.empty((N, H, W, C), dtype=torch.float16, pin_memory=True)
    hx.copy_(x)
    hq = torch.empty(q.shape, dtype=torch.float16, pin_memory=True)
    hq.copy_(q)
    hm = torch.from_numpy(w.mask_h).pin_memory()
    hy = torch.empty((N, H, W, C), dtype=torch.float16, pin_memory=True)
    dm = w.masks[0]
    s_in, s_c, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    out_done = [None] * G

    def fence():
        for st in (s_in, s_c, s_out):
            st.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

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
                idx, cnt = ops.reduce_mask(dm[lo:hi], *g_in.as_lists(), tol=0.5, avgpool=False, yield_core=world > 1)
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

    fence()
    e2e_step()
    fence()
    a, b = ev(), ev()
    a.record()
    s_in.wait_event(a)
    eb = 0
    for _ in range(e2e_steps):
        eb += e2e_step()
    for st in (s_in, s_c, s_out):
        torch.cuda.current_stream().wait_stream(st)
    b.record()
    fence()
    res = dict(ms=a.elapsed_time(b), blocks=eb, steps=e2e_steps, groups=G,
               h2d=hx.numel() * 2 + hq.numel() * 2 + hm.numel() * 4, d2h=hy.numel() * 2)
    del hx, hq, hy
    return res


def run_sync_free(torch, ops, args, w):
    """The same three ops with the block count kept on the device, replayed from a CUDA graph (outside
    the op interface, which needs bin_counts on the host; offered by the *_dyn entry points)."""
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    dev = w.x.device
    g_in, g_out, x = w.g_in, w.g_out, w.x
    max_blocks = w.N * g_in.bcount[0] * g_in.bcount[1]
    big_stack = torch.empty((max_blocks, w.C, 18, 18), dtype=torch.float16, device=dev)
    big_q = torch.empty((max_blocks, w.C, 16, 16), dtype=torch.float16, device=dev)
    big_q[:w.nB] = w.q
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())

    def dyn_step(m):
        idx, cnt_dev = ops.reduce_mask_async(m, *g_in.as_lists(), tol=0.5, avgpool=False, mask_stable=True)
        ops.sparse_gather_dyn(x, cnt_dev, max_blocks, idx, g_in.bsize, g_in.bstride, g_in.boffset,
                              transpose=True, out=big_stack)
        ops.sparse_scatter_var_dyn(big_q, cnt_dev, max_blocks, idx, x, g_out.bsize, g_out.bstride,
                                   g_out.boffset, add=True, transpose=True)
        return idx, cnt_dev

    with torch.cuda.stream(side):
        dyn_step(w.masks[0])
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph, keep = torch.cuda.CUDAGraph(), []
    with torch.cuda.graph(graph, stream=side):
        for m in w.masks[:4]:
            keep.append(dyn_step(m))
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    a, b = ev(), ev()
    reps = max(1, args.steps // 4)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / (reps * 4)
    del big_stack, big_q, graph, keep
    return {"value": w.nB / (ms * 1e-3), "unit": "blocks/s", "ms_per_step": ms,
            "how": "reduce_mask -> gather_dyn -> scatter_dyn, count read on the device, 4 steps per CUDA graph replay"}


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
    from bench_ops import Timer, _peak
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
    ap.add_argument("--scaling", choices=["weak", "strong"], default="strong")
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
    ap.add_argument("--in-order", action="store_true",
                    help="issue every step's reduce_mask behind the previous step's scatter on one stream "
                         "(default: two steps ahead on a second stream, counts fetched without blocking)")
    ap.add_argument("--no-suite", action="store_true", help="skip the op-level table of configurations 2-4 and 5 at 30 percent")
    ap.add_argument("--no-weak", action="store_true", help="N > 1: skip the second pass in the other scaling mode")
    ap.add_argument("--cpu-budget", type=float, default=12.0)
    ap.add_argument("--suite", choices=["ops", "one", "resblock", "topleft", "cpu", "refgpu"], default=None)
    ap.add_argument("--arch", choices=["resnet-50", "resnet-v2"], default="resnet-v2", help="--suite topleft: size table")
    ap.add_argument("--topleft-test", choices=["conv", "res"], default="res")
    ap.add_argument("--topleft-dtype", choices=["f16", "f32"], default="f16")
    ap.add_argument("--topleft-eager", action="store_true", help="--suite topleft: time eager launches instead of CUDA graphs")
    ap.add_argument("--topleft-stage", type=int, default=None, help="--suite topleft: one stage (0-3) instead of all")
    ap.add_argument("--topleft-sparsity", type=float, default=None, help="--suite topleft: one sparsity instead of the list")
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
    elif args.suite in ("ops", "one", "resblock", "topleft"):
        import bench_ops
        bench_ops.main(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
