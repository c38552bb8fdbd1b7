"""``bench.py --suite topleft``: dense versus block-sparse evaluation on a synthetic top-left mask.

What the reference's own harness measures (``benchmark/benchmark_topleft.py:45-133``,
``benchmark/sparse_conv_perf.py:47-63,112-262``, tables ``benchmark/benchmark_configs.py:23-44``): for
every feature-map size of a ResNet variant, a dense convolution (or bottleneck residual block) on the
whole tensor against the block-sparse version on a mask whose top-left square holds ``1 - sparsity``
of the pixels, over a sweep of square block sizes; per sparsity the best block size, its block
sparsity, dense time, sparse time and speed-up.  Protocol as there: batch 1, average pooling with
tol 0.05, block indices computed once outside the timed region, five independent input tensors per
run, three warm-up runs, three timed runs, CUDA-event time divided by five.

The convolutions are the host framework's (torch / cuDNN here, TensorFlow in the reference) in both
arms; this library contributes reduce_mask, sparse_gather and sparse_scatter[_var].  Benchmark tooling,
kept beside ``bench.py`` and outside the library package.  One JSON line per (size, sparsity).
"""
from __future__ import annotations

import json
import math

import numpy as np

# [H, W, C, K] per stage: input channels C, bottleneck (or conv output) channels K
INPUT_SIZES = {
    "resnet-50": [[400, 700, 256, 64], [200, 350, 512, 128], [100, 175, 1024, 256], [50, 88, 2048, 512]],
    "resnet-v2": [[400, 700, 96, 24], [200, 350, 192, 48], [100, 175, 256, 64], [50, 88, 384, 96]],
}
SPARSITIES = [0.6, 0.65, 0.7, 0.75, 0.8, 0.85, 0.9, 0.95, 0.99]
BLOCK_SIZES = [range(11, 33, 2), range(7, 25, 2), range(5, 21, 2), range(5, 21, 2)]   # one sweep per stage
BATCH, TOL, AVGPOOL = 1, 0.05, True
N_REPEAT, N_WARMUP, N_RUN = 5, 3, 3


def top_left_mask(N: int, H: int, W: int, sparsity: float) -> np.ndarray:
    """``[N,H,W,1]`` fp32: ones on a top-left rectangle with the image's aspect ratio that holds
    ``1 - sparsity`` of the pixels (edges rounded up), zeros elsewhere."""
    edge = math.sqrt(1.0 - sparsity)
    m = np.zeros((N, H, W, 1), dtype=np.float32)
    m[:, :int(math.ceil(edge * H)), :int(math.ceil(edge * W))] = 1.0
    return m


def _time_runs(torch, fn_of_repeat, graph=True):
    """Three warm-ups, then three runs of five repeats each between CUDA events; mean time of one repeat.
    The five repeats are captured into one CUDA graph and replayed (the reference's harness runs a
    TensorFlow graph, which has no per-op interpreter cost either); ``graph=False`` times eager launches."""
    def run_all():
        for i in range(N_REPEAT):
            fn_of_repeat(i)
    for _ in range(N_WARMUP):
        run_all()
    torch.cuda.synchronize()
    replay = run_all
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            run_all()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            run_all()
        replay = g.replay
        for _ in range(N_WARMUP):
            replay()
        torch.cuda.synchronize()
    times = []
    for _ in range(N_RUN):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) / N_REPEAT)
    return sum(times) / len(times)


def topleft(args):
    import torch
    import torch.nn.functional as F
    from sbnet_b200 import build, geometry, ops
    from sbnet_b200.resblock import SparseBottleneck
    build.build_library()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    res_block = args.topleft_test == "res"
    dtype = torch.float32 if args.topleft_dtype == "f32" else torch.float16
    sizes = INPUT_SIZES[args.arch]
    stages = range(len(sizes)) if args.topleft_stage is None else [args.topleft_stage]
    sparsities = SPARSITIES if args.topleft_sparsity is None else [args.topleft_sparsity]
    for stage in stages:
        H, W, C, K = sizes[stage]
        Cin = C if res_block else K            # the single-convolution test runs K -> K channels
        with torch.no_grad():
            xs = [torch.empty((BATCH, H, W, Cin), device=dev, dtype=dtype).uniform_(-1, 1) for _ in range(N_REPEAT)]
            if res_block:
                net = SparseBottleneck(C, K, dtype=dtype, device=dev).eval()
                xs_nchw = [x.permute(0, 3, 1, 2).contiguous() for x in xs]

                def dense(i):   # the whole tensor, SAME padding on the 3x3
                    x = xs_nchw[i]
                    q = net.conv1(F.relu(net.bn[0](x)))
                    q = F.conv2d(F.relu(net.bn[1](q)), net.conv2.weight, padding=1)
                    return x + net.conv3(F.relu(net.bn[2](q)))
            else:
                w = torch.empty((K, K, 3, 3), device=dev, dtype=dtype).uniform_(-1, 1)
                xs_nchw = [x.permute(0, 3, 1, 2).contiguous() for x in xs]

                def dense(i):
                    return F.conv2d(xs_nchw[i], w, padding=1)
            dense_ms = _time_runs(torch, dense, graph=not args.topleft_eager)
            for sparsity in sparsities:
                mask = torch.from_numpy(top_left_mask(BATCH, H, W, sparsity)).to(dev)
                best = None
                for b in BLOCK_SIZES[stage]:
                    if b > H or b > W:
                        continue
                    ks = [[1, 1, C, K], [3, 3, K, K], [1, 1, K, C]] if res_block else [[3, 3, K, K]]
                    bp = geometry.calc_block_params_res_block([BATCH, H, W, Cin], [1, b, b, 1], ks, [1, 1, 1, 1], "SAME")
                    idx, cnt = ops.reduce_mask(mask, bp.bcount, bp.bsize, bp.bstrides, bp.boffset, tol=TOL, avgpool=AVGPOOL)
                    nb = int(cnt[0])
                    block_sparsity = 1.0 - nb / float(idx.shape[0])

                    if res_block:
                        def sparse(i):
                            p = ops.sparse_gather(xs[i], cnt, idx, bp.bsize, bp.bstrides, bp.boffset, transpose=True)
                            q = net.residual(p).contiguous()
                            return ops.sparse_scatter_var(q, cnt, idx, xs[i], bp.bsize_out, bp.bsize_out, [0, 0],
                                                          add=True, transpose=True)
                    else:
                        def sparse(i):
                            p = ops.sparse_gather(xs[i], cnt, idx, bp.bsize, bp.bstrides, bp.boffset, transpose=True)
                            q = F.conv2d(p, w).contiguous()
                            return ops.sparse_scatter_var(q, cnt, idx, xs[i], bp.bsize_out, bp.bsize_out, [0, 0],
                                                          add=False, transpose=True)
                    ms = _time_runs(torch, sparse, graph=not args.topleft_eager)
                    if best is None or ms < best["sparse_ms"]:
                        best = {"BH": b, "BW": b, "sparse_ms": ms, "block_sparsity": block_sparsity, "active_blocks": nb}
                print(json.dumps({"case": f"topleft_{args.topleft_test}", "arch": args.arch, "dtype": args.topleft_dtype,
                                  "H": H, "W": W, "C": C, "K": K, "sparsity": sparsity,
                                  "block_sparsity": round(best["block_sparsity"], 4), "BH": best["BH"], "BW": best["BW"],
                                  "active_blocks": best["active_blocks"], "dense_ms": round(dense_ms, 4),
                                  "sparse_ms": round(best["sparse_ms"], 4),
                                  "speedup": round(dense_ms / best["sparse_ms"], 3),
                                  "timing": "eager" if args.topleft_eager else "cuda graph of 5 repeats"}), flush=True)
            del xs, xs_nchw
            torch.cuda.empty_cache()
