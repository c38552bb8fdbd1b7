// sparse_gather / sparse_scatter for sm_100a: the row-layout kernels, the general plane-layout
// kernel (any block size, stride, offset, channel count and element type), the flat copy, and the
// dispatch between these and the aligned plane-layout kernels of planes_simt.cu / planes_tma.cu.
//
// Replaces the reference's blockGatherTiled0/1 and blockScatterTiled0/1 families and their launcher
// (sbnet_ops/sparse_blocks.cu.h:68-366, sbnet_ops/sparse_gather.cu:41-266).  Semantics follow the
// reference CPU functors (sbnet_ops/sparse_gather.cc:61-132): the in-range test is per PIXEL, so
// gather zero-fills and scatter drops whatever part of a block hangs over any image border.
//
// Two layouts of the block stack:
//  * [nB, R, S, C] ("rows"): a block row of S pixels is one contiguous run of S*C elements both in
//    the NHWC image and in the stack, so the op is a clipped copy of contiguous runs.  Threads move
//    the widest vector (16/8/4/2 bytes) that divides C*sizeof(T), several per thread in flight, no
//    shared memory.  Where that vector is only 4 or 2 bytes the raw-row kernel below takes the call:
//    bulk copies on the image side, 16-byte vectors aligned to the stack on the stack side.
//  * [nB, C, R, S] ("planes", transpose=true): pixels of a multiple of 16 bytes go to the kernels of
//    planes_simt.cu / planes_tma.cu.  The kernels here take every other shape.  planes_rows_kernel:
//    whole block rows travel between the image and shared memory as raw bytes through the TMA
//    engine (untiled bulk copies, bulk stores / reductions), and warps transpose between those row
//    buffers and the stack.  planes_kernel (block rows too long for the tile; the A/B option): a CTA
//    stages a tile of pixels x channels in shared memory with an odd word pitch and moves both sides
//    element-wise.
// Scatter has three write modes: overwrite, read-add-write (legal only for disjoint blocks) and
// vector reductions (red.global.add .v4.f32 / .v4.f16x2 / .v4.bf16x2 and narrower) for overlapping halos.
//
// With the block count on the host every work item gets its own short CTA (measured faster on B200
// than a resident grid); when the count lives in device memory (written by reduce_mask earlier on
// the same stream) a fixed-size grid strides over the items instead.
#include <stdlib.h>

#include "async_ptx.cuh"
#include "common.cuh"
#include "kernels.h"
#include "options.h"

namespace sbnet {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

__device__ __forceinline__ int active_count(const BlockArgs& a)
{
    if (a.num_active_dev == nullptr)
        return a.numActive;
    const int n = __ldg(a.num_active_dev);
    return n < a.numActive ? n : a.numActive;
}

// ---- [nB,R,S,C] layout ---------------------------------------------------------------------------
// A block is vecsPerBlock = R * vecsPerRow vectors, contiguous in the stack; a work item is a chunk of
// at most kThreads * kUnroll of them.  With the block count known on the host every item gets its own
// small CTA (measured on B200: many short CTAs stream ~12 % faster than a resident grid looping over
// the same chunks); with the count in device memory a resident grid strides over the items instead.
struct RowPlan {
    FastDiv vecsPerRow;      // S * C * sizeof(T) / VB
    FastDiv chunksPerBlock;
    int vecsPerPixel;        // C * sizeof(T) / VB
    int vecsPerBlock;
    int chunkVecs;           // vectors per item (<= kThreads * kUnroll)
};

template <int VB, int MODE, typename T>
__device__ __forceinline__ void rows_item(const BlockArgs& a, const RowPlan& p, uint32_t ib, uint32_t chunk)
{
    typedef typename Vec<VB>::type V;
    const int vBeg = (int)chunk * p.chunkVecs;
    const int vEnd = min(vBeg + p.chunkVecs, p.vecsPerBlock);
    const int n = a.idx[ib * 3 + 0];
    const int h0 = a.bOffsH + a.idx[ib * 3 + 1] * a.bStrH;
    const int w0 = a.bOffsW + a.idx[ib * 3 + 2] * a.bStrW;
    // in-range part of a block row, in vectors from the row's first pixel
    const int qLo = max(0, -w0) * p.vecsPerPixel;
    const int qHi = max(0, min(a.bSzW, a.W - w0)) * p.vecsPerPixel;
    const long long rowPitch = (long long)a.W * p.vecsPerPixel;   // image row, in vectors
    V* img = reinterpret_cast<V*>(a.image) + (((long long)n * a.H + h0) * a.W + w0) * (long long)p.vecsPerPixel;
    V* stk = reinterpret_cast<V*>(a.stack) + (long long)ib * p.vecsPerBlock;

    V val[kUnroll], old[kUnroll];
    long long ioff[kUnroll];
    bool inr[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int v = vBeg + (int)threadIdx.x + u * kThreads;
        uint32_t r, q;
        p.vecsPerRow.divmod((uint32_t)min(v, vEnd - 1), r, q);
        const int h = h0 + (int)r;
        inr[u] = v < vEnd && h >= 0 && h < a.H && (int)q >= qLo && (int)q < qHi;
        ioff[u] = (long long)r * rowPitch + q;
        if constexpr (MODE == kGather) {
            val[u] = inr[u] ? ld_stream(img + ioff[u]) : vzero<VB>();
        } else {
            val[u] = inr[u] ? ld_stream(stk + v) : vzero<VB>();
            if constexpr (MODE == kScatterAdd)
                old[u] = inr[u] ? ld_plain<VB>(img + ioff[u]) : vzero<VB>();
        }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int v = vBeg + (int)threadIdx.x + u * kThreads;
        if constexpr (MODE == kGather) {
            if (v < vEnd)
                stk[v] = val[u];
        } else {
            if (inr[u])
                image_write<VB, MODE, T>(img + ioff[u], val[u], old[u]);
        }
    }
}

template <int VB, int MODE, typename T>
__global__ void __launch_bounds__(kThreads) rows_kernel(const BlockArgs a, const RowPlan p)
{
    pdl_wait();   // nothing is read or written before the kernel queued ahead of this one is done
    uint32_t ib, chunk;
    p.chunksPerBlock.divmod(blockIdx.x, ib, chunk);
    rows_item<VB, MODE, T>(a, p, ib, chunk);
    pdl_launch_dependents();
}

template <int VB, int MODE, typename T>
__global__ void __launch_bounds__(kThreads) rows_kernel_dyn(const BlockArgs a, const RowPlan p)
{
    pdl_wait();   // nothing is read or written before the kernel queued ahead of this one is done
    const long long nItems = (long long)active_count(a) * p.chunksPerBlock.div;
    for (long long item = blockIdx.x; item < nItems; item += gridDim.x) {
        uint32_t ib, chunk;
        p.chunksPerBlock.divmod((uint32_t)item, ib, chunk);
        rows_item<VB, MODE, T>(a, p, ib, chunk);
    }
    pdl_launch_dependents();
}

// ---- [nB,C,R,S] layout ---------------------------------------------------------------------------
constexpr int kTileBytes = 44352;   // 336 pixels x 33 words

struct PlanePlan {
    FastDiv blockW;          // S
    FastDiv cChunks;         // channel chunks per block
    FastDiv pChunks;         // pixel chunks per block
    FastDiv vecsPerPixelFull, vecsPerPixelLast;   // vectors per pixel in a full / the last chunk
    FastDiv pixFull, pixLast;                     // pixels in a full / the last pixel chunk
    int chanPerChunk;        // channels per chunk (128 bytes worth, or all of C)
    int pixPerChunk;
    int pitch;               // shared-memory pitch of one pixel, in elements (odd number of words)
};

template <int VB, typename T> __device__ __forceinline__ void tile_store(T* p, typename Vec<VB>::type v)
{
    if constexpr (VB == 2) {
        *reinterpret_cast<uint16_t*>(p) = v;
    } else {
        uint32_t w[VB / 4];
        memcpy(w, &v, VB);
#pragma unroll
        for (int i = 0; i < VB / 4; ++i)
            reinterpret_cast<uint32_t*>(p)[i] = w[i];
    }
}
template <int VB, typename T> __device__ __forceinline__ typename Vec<VB>::type tile_load(const T* p)
{
    typename Vec<VB>::type v;
    if constexpr (VB == 2) {
        v = *reinterpret_cast<const uint16_t*>(p);
    } else {
        uint32_t w[VB / 4];
#pragma unroll
        for (int i = 0; i < VB / 4; ++i)
            w[i] = reinterpret_cast<const uint32_t*>(p)[i];
        memcpy(&v, w, VB);
    }
    return v;
}

// Narrow vectors need more of them in flight: the general kernel keeps 64 bytes of image loads (and 16
// stack elements) per thread outstanding whatever the vector width.
template <int VB> struct PlaneUnroll { static constexpr int image = VB >= 16 ? 4 : (VB == 8 ? 8 : 16); };
constexpr int kStackUnroll = 16;

template <int VB, int MODE, typename T>
__global__ void __launch_bounds__(kThreads, 4) planes_kernel(const BlockArgs a, const PlanePlan p)
{
    pdl_wait();   // nothing is read or written before the kernel queued ahead of this one is done
    typedef typename Vec<VB>::type V;
    constexpr int EPV = VB / (int)sizeof(T);   // elements per vector
    constexpr int kUI = PlaneUnroll<VB>::image;
    __shared__ __align__(16) unsigned char tileRaw[kTileBytes];
    T* tile = reinterpret_cast<T*>(tileRaw);

    const int nActive = active_count(a);
    const uint32_t itemsPerBlock = p.cChunks.div * p.pChunks.div;
    const long long nItems = (long long)nActive * itemsPerBlock;
    const int RS = a.bSzH * a.bSzW;
    T* image = reinterpret_cast<T*>(a.image);
    T* stack = reinterpret_cast<T*>(a.stack);

    for (long long item = blockIdx.x; item < nItems; item += gridDim.x) {
        uint32_t rest, cc, ib, pc;
        p.cChunks.divmod((uint32_t)item, rest, cc);   // channel chunk varies fastest
        p.pChunks.divmod(rest, ib, pc);
        const bool lastC = cc + 1 == p.cChunks.div, lastP = pc + 1 == p.pChunks.div;
        const int c0 = (int)cc * p.chanPerChunk;
        const int nChan = min(p.chanPerChunk, a.C - c0);
        const int p0 = (int)pc * p.pixPerChunk;
        const int nPix = min(p.pixPerChunk, RS - p0);
        const FastDiv vpp = lastC ? p.vecsPerPixelLast : p.vecsPerPixelFull;
        const FastDiv pixDiv = lastP ? p.pixLast : p.pixFull;
        const int n = a.idx[ib * 3 + 0];
        const int h0 = a.bOffsH + a.idx[ib * 3 + 1] * a.bStrH;
        const int w0 = a.bOffsW + a.idx[ib * 3 + 2] * a.bStrW;
        const T* imgN = image + (long long)n * a.H * a.W * a.C + c0;
        T* planes = stack + ((long long)ib * a.C + c0) * RS + p0;   // [nChan][RS] view, pixel p0
        const int nVec = nPix * (int)vpp.div;
        const int nElem = nPix * nChan;

        if constexpr (MODE == kGather) {
            // image -> tile: one vector of channels per thread-step, kUI loads in flight
            for (int v0 = threadIdx.x; v0 < nVec; v0 += kThreads * kUI) {
                V val[kUI];
#pragma unroll
                for (int u = 0; u < kUI; ++u) {
                    const int v = v0 + u * kThreads;
                    uint32_t px, j, r, s;
                    vpp.divmod((uint32_t)min(v, nVec - 1), px, j);
                    p.blockW.divmod((uint32_t)p0 + px, r, s);
                    const int h = h0 + (int)r, w = w0 + (int)s;
                    const bool inr = v < nVec && h >= 0 && h < a.H && w >= 0 && w < a.W;
                    val[u] = inr ? ld_stream(reinterpret_cast<const V*>(
                                       imgN + ((long long)h * a.W + w) * a.C + j * EPV))
                                 : vzero<VB>();
                }
#pragma unroll
                for (int u = 0; u < kUI; ++u) {
                    const int v = v0 + u * kThreads;
                    if (v < nVec) {
                        uint32_t px, j;
                        vpp.divmod((uint32_t)v, px, j);   // recomputed: cheaper than keeping it across the loads
                        tile_store<VB, T>(tile + px * p.pitch + j * EPV, val[u]);
                    }
                }
            }
            __syncthreads();
            // tile -> stack: consecutive threads write consecutive pixels of one channel plane
            for (int o = threadIdx.x; o < nElem; o += kThreads) {
                uint32_t c, px;
                pixDiv.divmod((uint32_t)o, c, px);
                planes[(long long)c * RS + px] = tile[px * p.pitch + c];
            }
            __syncthreads();
        } else {
            // stack -> tile
            for (int o0 = threadIdx.x; o0 < nElem; o0 += kThreads * kStackUnroll) {
                T val[kStackUnroll];
#pragma unroll
                for (int u = 0; u < kStackUnroll; ++u) {
                    const int o = o0 + u * kThreads;
                    uint32_t c, px;
                    pixDiv.divmod((uint32_t)min(o, nElem - 1), c, px);
                    val[u] = planes[(long long)c * RS + px];
                }
#pragma unroll
                for (int u = 0; u < kStackUnroll; ++u) {
                    const int o = o0 + u * kThreads;
                    if (o < nElem) {
                        uint32_t c, px;
                        pixDiv.divmod((uint32_t)o, c, px);
                        tile[px * p.pitch + c] = val[u];
                    }
                }
            }
            __syncthreads();
            // tile -> image
            for (int v = threadIdx.x; v < nVec; v += kThreads) {
                uint32_t px, j, r, s;
                vpp.divmod((uint32_t)v, px, j);
                p.blockW.divmod((uint32_t)p0 + px, r, s);
                const int h = h0 + (int)r, w = w0 + (int)s;
                if (h >= 0 && h < a.H && w >= 0 && w < a.W) {
                    V* dst = reinterpret_cast<V*>(const_cast<T*>(imgN) +
                                                  ((long long)h * a.W + w) * a.C + j * EPV);
                    const V val = tile_load<VB, T>(tile + px * p.pitch + j * EPV);
                    V old = vzero<VB>();
                    if constexpr (MODE == kScatterAdd)
                        old = *dst;
                    image_write<VB, MODE, T>(dst, val, old);
                }
            }
            __syncthreads();
        }
    }
    pdl_launch_dependents();
}

// ---- [nB,C,R,S] layout, any pixel size: whole image rows staged as raw bytes -----------------------
// The general kernel above spends ~40 integer instructions per element (two divisions and a 64-bit
// address per element in each phase) and is issue-bound on the shapes it exists for (pixels that are
// not a multiple of 16 bytes).  This kernel takes the same shapes whenever a block row's pixels fit
// the tile.  A block row of S pixels x C channels is ONE contiguous run of the image, so whatever
// C*sizeof(T) is, the run moves between the image and a row buffer as raw bytes through the TMA
// engine -- one untiled bulk copy per block row, no thread touches it: the buffer keeps the run's
// misalignment (byte b of the run lands at offset (address & 15) + b), which makes both ends of the
// copy 16-byte aligned.
//   image -> buffer: the 16-byte vectors that hold the run clipped to the image (a vector that holds
//     one byte of the tensor lies in the same page as that byte, so the few bytes read beside the run
//     belong to the same allocation; they are never used).
//   buffer -> image: the whole 16-byte vectors inside the clipped run as one bulk store -- or one
//     bulk reduction (cp.reduce.async.bulk .add), element-wise adds in L2 like red.global.add, for
//     overlapping blocks -- and the run's two ragged ends (< 16 bytes each) element by element, so
//     nothing outside the run is written.  Read-add-write of fp32 (kept apart from the reduction,
//     which flushes subnormals) loads the rows first, adds in shared memory and stores them.
// The transposition happens between the row buffers and the stack: a warp takes 32 consecutive runs
// of Q pixels x a group of channels at a time, one run per lane -- one division and one range test
// per task, then only constant offsets on the shared-memory side and one plane pitch per channel on
// the stack side, where a warp access covers 32 consecutive runs of one plane (Q pixels = 16 bytes
// per lane where the planes are aligned for it, 4 bytes for 16-bit planes on 4-byte boundaries, else
// one element).  16-bit accumulation reduces with packed red.global.add (.v4.f16x2 / .bf16x2) from
// the row buffers instead of the engine's reduction, which adds one 16-bit element at a time.
// A CTA of the raw-row kernel: 128 threads and 24 KB of row buffers, eight per SM.  (256 threads and 44 KB, four per
// SM, measured 3-8 % slower on C = 33 fp32 and C = 100 fp16: a CTA's load and transposition phases do not overlap,
// so more and smaller CTAs interleave them better.)
constexpr int kRawThreads = 128;
constexpr int kRawTileBytes = 24576;
constexpr int kRawMaxRows = 1024;     // block rows per work item (a bound on the loop of the issuing warp)
template <typename T> struct RawChans { static constexpr int n = sizeof(T) == 4 ? 12 : 16; };   // channels per task

__device__ unsigned int g_rows_wait_timeouts = 0;   // bounded waits of planes_rows_kernel that gave up

struct RawPlan {
    FastDiv rChunks;       // row chunks per block
    FastDiv blockW;        // S
    FastDiv chanGroups;    // channel groups per pixel group
    int chansPerGroup;     // channels of one group (the last may hold fewer), <= RawChans<T>::n
    int rowsPerItem;       // block rows per work item
    int rowPitch;          // bytes of one row buffer: S*C*sizeof(T) + its possible misalignment, a multiple of 16
    int rowBytes;          // S*C*sizeof(T)
    FastDiv stackSlots;    // row layout of the stack: 16-byte vectors a row can touch there
};

// Q: consecutive pixels of one channel plane a lane moves at a time on the stack side -- 1 (any shape), 2 (16-bit
// planes on 4-byte boundaries), or the 16 bytes' worth (4 / 8 pixels as ONE 16-byte access) when every plane of an
// item starts on a 16-byte boundary.
template <int MODE, typename T, int Q>
__global__ void __launch_bounds__(kRawThreads, 8) planes_rows_kernel(const BlockArgs a, const RawPlan p)
{
    __shared__ __align__(128) unsigned char tile[kRawTileBytes];
    __shared__ __align__(8) unsigned long long barWord;
    __shared__ int abortFlag;
    constexpr int SZ = (int)sizeof(T);
    constexpr int G = RawChans<T>::n;
    constexpr bool kLoads = MODE == kGather || MODE == kScatterAdd;   // image rows come into the buffers
    typedef typename Vec<SZ>::type E;                 // one element as plain bits
    const uint32_t tileAddr = smem_u32(tile), bar = smem_u32(&barWord);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        abortFlag = 0;
        if constexpr (kLoads) {
            mbar_init(bar, 1);
            mbar_init_fence();
        }
    }
    __syncthreads();
    pdl_wait();   // nothing is read or written before the kernel queued ahead of this one is done
    const int nActive = active_count(a);
    const long long nItems = (long long)nActive * p.rChunks.div;
    const int S = a.bSzW, P = a.bSzH * a.bSzW;
    const int pixBytes = a.C * SZ;
    const long long imgRowBytes = (long long)a.W * pixBytes;
    const int rowMis = (int)(imgRowBytes & 15);       // how the misalignment moves from one image row to the next
    uint32_t parity = 0;

    for (long long item = blockIdx.x; item < nItems; item += gridDim.x) {
        uint32_t ib, rc;
        p.rChunks.divmod((uint32_t)item, ib, rc);
        const int r0 = (int)rc * p.rowsPerItem;
        const int rows = min(p.rowsPerItem, a.bSzH - r0);
        const int n = a.idx[ib * 3 + 0];
        const int h0 = a.bOffsH + a.idx[ib * 3 + 1] * a.bStrH + r0;
        const int w0 = a.bOffsW + a.idx[ib * 3 + 2] * a.bStrW;
        const int sLo = max(0, -w0), sHi = max(sLo, min(S, a.W - w0));   // in-range pixels of every row: [sLo, sHi)
        const int bLo = sLo * pixBytes, bHi = sHi * pixBytes;            // ... as bytes of the row's run
        // address the run of row 0 WOULD start at: its pixel 0 may lie left of, above or below the image; such an
        // address only tells the alignment and is never dereferenced
        const long long g00 = (long long)reinterpret_cast<uintptr_t>(a.image)
            + (((long long)n * a.H + h0) * a.W + w0) * (long long)pixBytes;
        const int ph0 = (int)(g00 & 15);
        T* planes = reinterpret_cast<T*>(a.stack) + (long long)ib * a.C * P + (long long)r0 * S;   // [C][P] view at row r0
        const int nPix = rows * S;
        const int nTasks = Q == 0 ? 0 : ((nPix + 32 * (Q ? Q : 1) - 1) / (32 * (Q ? Q : 1))) * (int)p.chanGroups.div;

        // Row rl of the item: the clipped run [lo, hi) as global addresses and the shared-memory address
        // of the 16-byte vector that holds the run's (unclipped) first byte.
        struct Row {
            long long lo, hi;   // lo >= hi: nothing of the row is inside the image
            long long base;     // global address of that first vector
            uint32_t buf;       // its shared-memory address
        };
        auto row_of = [&](int rl) -> Row {
            Row r;
            const long long g0 = g00 + rl * imgRowBytes;
            r.base = g0 & ~15ll;
            r.buf = tileAddr + (uint32_t)(rl * p.rowPitch);
            r.lo = g0 + bLo, r.hi = g0 + bHi;
            if ((unsigned)(h0 + rl) >= (unsigned)a.H)
                r.hi = r.lo;
            return r;
        };
        // A task of the transposition: 32 consecutive pixels of the item (one per lane) x one channel group.
        struct Task {
            uint32_t at;        // row-buffer address of the lane's pixel, first channel of the group
            E* g;               // the same element in the stack; channel c + 1 lies P elements further
            int nc;             // channels of the group; 0 for a lane beyond the item's last pixel
            bool inr;           // the pixel lies inside the image
        };
        auto task_of = [&](int t) -> Task {
            Task k;
            uint32_t pg, cg, rl, s;
            p.chanGroups.divmod((uint32_t)t, pg, cg);
            const int px = (int)pg * 32 + lane, c0 = (int)cg * p.chansPerGroup;
            k.nc = px < nPix ? min(p.chansPerGroup, a.C - c0) : 0;
            p.blockW.divmod((uint32_t)min(px, nPix - 1), rl, s);
            k.inr = (unsigned)(h0 + (int)rl) < (unsigned)a.H && (unsigned)(w0 + (int)s) < (unsigned)a.W;
            k.at = tileAddr + rl * (uint32_t)p.rowPitch + (uint32_t)((ph0 + (int)rl * rowMis) & 15)
                + (uint32_t)(((int)s * a.C + c0) * SZ);
            k.g = reinterpret_cast<E*>(planes) + (long long)c0 * P + px;
            return k;
        };

        if constexpr (kLoads) {
            // image -> row buffers: warp 0 announces the bytes and issues one bulk copy per row
            if (warp == 0) {
                uint32_t bytes = 0;
                for (int rl = lane; rl < rows; rl += 32) {
                    const Row r = row_of(rl);
                    if (r.lo < r.hi)
                        bytes += (uint32_t)(((r.hi + 15) & ~15ll) - (r.lo & ~15ll));
                }
                bytes = __reduce_add_sync(0xffffffffu, bytes);
                if (lane == 0)
                    mbar_expect_tx(bar, bytes);
                __syncwarp();
                for (int rl = lane; rl < rows; rl += 32) {
                    const Row r = row_of(rl);
                    if (r.lo < r.hi) {
                        const long long src = r.lo & ~15ll;
                        bulk_load_1d(r.buf + (uint32_t)(src - r.base), reinterpret_cast<const void*>(src),
                                     (uint32_t)(((r.hi + 15) & ~15ll) - src), bar);
                    }
                }
            }
            // every warp waits (bounded); one that gives up waits once more, again bounded, so that the copies are
            // not left in flight over shared memory this CTA has given back
            int ok = 1;
            if (lane == 0) {
                ok = mbar_wait_bounded(bar, parity, &abortFlag, &g_rows_wait_timeouts) ? 1 : 0;
                if (!ok) {
                    int again = 0;
                    (void)mbar_wait_bounded(bar, parity, &again, &g_rows_wait_timeouts);
                }
            }
            if (!__shfl_sync(0xffffffffu, ok, 0))
                break;
            parity ^= 1u;
        }

        if constexpr (Q == 0) {
            // ---- [nB,R,S,C] stack: the item's rows are one contiguous run of the stack, each row a copy of its row
            // buffer at another alignment.  A thread takes a 16-byte vector of the STACK (aligned there) and the
            // 4 words -- or, 16-bit elements an odd half away, 8 halves -- of the row buffer that belong to it; the
            // partial vectors at a row's two ends go element by element.
            const long long sItem = (long long)reinterpret_cast<uintptr_t>(a.stack)
                + ((long long)ib * a.bSzH + r0) * (long long)p.rowBytes;
            const int nSlots = rows * (int)p.stackSlots.div;
            struct Slot {
                long long A;          // the vector's address in the stack (16-byte aligned)
                uint32_t src;         // row-buffer address of the vector's first byte that belongs to the row
                int lo, hi;           // [lo, hi): the vector's bytes that belong to the row (empty: lo >= hi)
                int off;              // offset of byte lo inside the row's run
                bool rowIn;           // the row lies inside the image (gather zero-fills otherwise)
            };
            auto slot_of = [&](int k) -> Slot {
                Slot t;
                t.A = 0, t.src = 0, t.lo = t.hi = t.off = 0, t.rowIn = false;
                if (k >= nSlots)
                    return t;
                uint32_t rl, q;
                p.stackSlots.divmod((uint32_t)k, rl, q);
                const long long sRow = sItem + (long long)rl * p.rowBytes;
                const int ph2 = (int)(sRow & 15), b0 = 16 * (int)q;
                t.A = (sRow & ~15ll) + b0;
                t.lo = max(b0, ph2) - b0, t.hi = max(t.lo, min(b0 + 16, ph2 + p.rowBytes) - b0);
                t.off = b0 + t.lo - ph2;
                t.src = tileAddr + rl * (uint32_t)p.rowPitch + (uint32_t)((ph0 + (int)rl * rowMis) & 15) + (uint32_t)t.off;
                t.rowIn = (unsigned)(h0 + (int)rl) < (unsigned)a.H;
                return t;
            };
            auto read16 = [&](uint32_t src) -> uint4 {   // 16 bytes of a row buffer from an element-aligned address
                uint4 v;
                if (SZ == 4 || (src & 3u) == 0) {
                    v.x = lds32(src), v.y = lds32(src + 4), v.z = lds32(src + 8), v.w = lds32(src + 12);
                } else {
                    v.x = lds16(src) | (lds16(src + 2) << 16), v.y = lds16(src + 4) | (lds16(src + 6) << 16);
                    v.z = lds16(src + 8) | (lds16(src + 10) << 16), v.w = lds16(src + 12) | (lds16(src + 14) << 16);
                }
                return v;
            };
            if constexpr (MODE == kGather) {
                for (int k = threadIdx.x; k < nSlots; k += kRawThreads) {
                    const Slot t = slot_of(k);
                    if (t.lo >= t.hi)
                        continue;
                    const bool allIn = t.rowIn && t.off >= bLo && t.off + (t.hi - t.lo) <= bHi;
                    if (t.hi - t.lo == 16 && allIn) {
                        *reinterpret_cast<uint4*>(t.A) = read16(t.src);
                    } else {   // a row's end, or a stretch outside the image (zeros): element by element
                        for (int b = t.lo; b < t.hi; b += SZ) {
                            const int o = t.off + (b - t.lo);
                            E e = 0;
                            if (t.rowIn && o >= bLo && o < bHi)
                                e = SZ == 4 ? (E)lds32(t.src + (uint32_t)(b - t.lo)) : (E)lds16(t.src + (uint32_t)(b - t.lo));
                            *reinterpret_cast<E*>(t.A + b) = e;
                        }
                    }
                }
            } else {
                constexpr int kSU = 4;   // stack vectors in flight per thread
                for (int k0 = threadIdx.x; k0 < nSlots; k0 += kRawThreads * kSU) {
                    Slot t[kSU];
                    uint4 v[kSU];
#pragma unroll
                    for (int u = 0; u < kSU; ++u) {
                        t[u] = slot_of(k0 + u * kRawThreads);
                        if (t[u].hi - t[u].lo == 16)
                            v[u] = ld_stream(reinterpret_cast<const uint4*>(t[u].A));
                    }
#pragma unroll
                    for (int u = 0; u < kSU; ++u) {
                        if (t[u].hi - t[u].lo == 16) {
                            const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
                            if (SZ == 4 || (t[u].src & 3u) == 0) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    uint32_t e = w[j];
                                    if constexpr (MODE == kScatterAdd)   // the buffer holds the image's value
                                        e = vadd<T>(lds32(t[u].src + 4 * j), e);
                                    sts32(t[u].src + 4 * j, e);
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    uint32_t e = (j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xffffu);
                                    if constexpr (MODE == kScatterAdd)
                                        e = vadd<T>((E)lds16(t[u].src + 2 * j), (E)e);
                                    sts16(t[u].src + 2 * j, e);
                                }
                            }
                        } else {
                            for (int b = t[u].lo; b < t[u].hi; b += SZ) {
                                const uint32_t dst = t[u].src + (uint32_t)(b - t[u].lo);
                                E e = ld_stream(reinterpret_cast<const E*>(t[u].A + b));
                                if constexpr (MODE == kScatterAdd)
                                    e = vadd<T>(SZ == 4 ? (E)lds32(dst) : (E)lds16(dst), e);
                                if constexpr (SZ == 4)
                                    sts32(dst, e);
                                else
                                    sts16(dst, e);
                            }
                        }
                    }
                }
            }
        } else if constexpr (Q > 1) {
            // ---- vector stack accesses: a lane owns Q consecutive pixels (NW words), the channels of its group in
            // batches of kB
            constexpr int kB = 4, NW = Q * SZ / 4;
            typedef typename Vec<4 * NW>::type V;
            for (int t = warp; t < nTasks; t += kRawThreads / 32) {
                uint32_t pg, cg, rl, sx;
                p.chanGroups.divmod((uint32_t)t, pg, cg);
                const int px0 = ((int)pg * 32 + lane) * Q, c0 = (int)cg * p.chansPerGroup;
                const int nc = px0 < nPix ? min(p.chansPerGroup, a.C - c0) : 0;   // nPix is a multiple of Q
                p.blockW.divmod((uint32_t)min(px0, nPix - Q), rl, sx);
                uint32_t at[Q], inMask = 0;      // row-buffer address of every pixel (first channel of the group); in the image?
#pragma unroll
                for (int j = 0; j < Q; ++j) {
                    at[j] = tileAddr + rl * (uint32_t)p.rowPitch + (uint32_t)((ph0 + (int)rl * rowMis) & 15)
                        + (uint32_t)(((int)sx * a.C + c0) * SZ);
                    if ((unsigned)(h0 + (int)rl) < (unsigned)a.H && (unsigned)(w0 + (int)sx) < (unsigned)a.W)
                        inMask |= 1u << j;
                    if (++sx == (uint32_t)S)
                        sx = 0, ++rl;
                }
                V* g = reinterpret_cast<V*>(reinterpret_cast<E*>(planes) + (long long)c0 * P + px0);
                const long long planeVecs = (long long)P / Q;     // P is a multiple of Q here
                for (int u0 = 0; u0 < nc; u0 += kB, g += kB * planeVecs) {
                    uint32_t w[kB][NW];
                    if constexpr (MODE == kGather) {
#pragma unroll
                        for (int u = 0; u < kB; ++u) {
                            if (u0 + u < nc) {
#pragma unroll
                                for (int j = 0; j < NW; ++j) {
                                    if constexpr (SZ == 4) {
                                        const uint32_t e = lds32(at[j] + (uint32_t)(u * SZ));
                                        w[u][j] = ((inMask >> j) & 1u) ? e : 0u;
                                    } else {
                                        const uint32_t lo = lds16(at[2 * j] + (uint32_t)(u * SZ));
                                        const uint32_t hi = lds16(at[2 * j + 1] + (uint32_t)(u * SZ));
                                        w[u][j] = (((inMask >> (2 * j)) & 1u) ? lo : 0u)
                                            | ((((inMask >> (2 * j + 1)) & 1u) ? hi : 0u) << 16);
                                    }
                                }
                            }
                        }
#pragma unroll
                        for (int u = 0; u < kB; ++u) {
                            if (u0 + u < nc) {
                                if constexpr (NW == 4)
                                    g[u * planeVecs] = make_uint4(w[u][0], w[u][1], w[u][2], w[u][3]);
                                else if constexpr (NW == 2)
                                    g[u * planeVecs] = make_uint2(w[u][0], w[u][1]);
                                else
                                    g[u * planeVecs] = w[u][0];
                            }
                        }
                    } else {
#pragma unroll
                        for (int u = 0; u < kB; ++u) {
                            if (u0 + u < nc) {
                                const V v = ld_stream(g + u * planeVecs);
                                if constexpr (NW == 4)
                                    w[u][0] = v.x, w[u][1] = v.y, w[u][2] = v.z, w[u][3] = v.w;
                                else if constexpr (NW == 2)
                                    w[u][0] = v.x, w[u][1] = v.y;
                                else
                                    w[u][0] = v;
                            }
                        }
#pragma unroll
                        for (int u = 0; u < kB; ++u) {
                            if (u0 + u < nc) {
#pragma unroll
                                for (int j = 0; j < Q; ++j) {
                                    const uint32_t dst = at[j] + (uint32_t)(u * SZ);
                                    E e = SZ == 4 ? (E)w[u][j] : (E)((j & 1) ? (w[u][j >> 1] >> 16) : (w[u][j >> 1] & 0xffffu));
                                    if constexpr (MODE == kScatterAdd)   // the buffer holds the image's value
                                        e = vadd<T>(SZ == 4 ? (E)lds32(dst) : (E)lds16(dst), e);
                                    if constexpr (SZ == 4)
                                        sts32(dst, e);
                                    else
                                        sts16(dst, e);
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int j = 0; j < Q; ++j)
                        at[j] += kB * SZ;
                }
            }
        } else if constexpr (MODE == kGather) {
            // row buffers -> stack; pixels outside the image are zeros
            for (int t = warp; t < nTasks; t += kRawThreads / 32) {
                const Task k = task_of(t);
                E e[G];
#pragma unroll
                for (int u = 0; u < G; ++u) {
                    e[u] = 0;
                    if (u < k.nc && k.inr)
                        e[u] = SZ == 4 ? (E)lds32(k.at + u * SZ) : (E)lds16(k.at + u * SZ);
                }
#pragma unroll
                for (int u = 0; u < G; ++u)
                    if (u < k.nc)
                        k.g[(long long)u * P] = e[u];
            }
        } else {
            // stack -> row buffers (pixels outside the image too: the stack holds them, the image never gets them)
            for (int t = warp; t < nTasks; t += kRawThreads / 32) {
                const Task k = task_of(t);
                E e[G];
#pragma unroll
                for (int u = 0; u < G; ++u)
                    if (u < k.nc)
                        e[u] = ld_stream(k.g + (long long)u * P);
#pragma unroll
                for (int u = 0; u < G; ++u) {
                    if (u < k.nc) {
                        E v = e[u];
                        if constexpr (MODE == kScatterAdd)   // the buffer holds the image's value
                            v = vadd<T>(SZ == 4 ? (E)lds32(k.at + u * SZ) : (E)lds16(k.at + u * SZ), v);
                        if constexpr (SZ == 4)
                            sts32(k.at + u * SZ, v);
                        else
                            sts16(k.at + u * SZ, v);
                    }
                }
            }
        }
        if constexpr (MODE != kGather) {
            fence_async_smem();   // the bulk copies below read what the threads wrote
            __syncthreads();
            // row buffers -> image: whole vectors inside the clipped run by the TMA engine ...
            constexpr bool kEngine = !(MODE == kScatterAtomic && SZ == 2);
            if constexpr (!kEngine) {
                // ... except 16-bit accumulation: the engine's reduction adds one 16-bit element at a time (measured
                // 2-3 times slower than the packed form), so a warp takes a row and reduces 16 bytes per lane
                // (red.global.add.noftz.v4.f16x2 / .bf16x2)
                for (int rl = warp; rl < rows; rl += kRawThreads / 32) {
                    const Row r = row_of(rl);
                    const long long aLo = (r.lo + 15) & ~15ll, aHi = r.hi & ~15ll;
                    if (r.lo < r.hi)
                        for (long long b = aLo + 16 * lane; b < aHi; b += 16 * 32)
                            Red<T>::add(reinterpret_cast<uint4*>(b), lds128(r.buf + (uint32_t)(b - r.base)));
                }
            } else if (warp == 0) {
                for (int rl = lane; rl < rows; rl += 32) {
                    const Row r = row_of(rl);
                    const long long aLo = (r.lo + 15) & ~15ll, aHi = r.hi & ~15ll;
                    if (r.lo < r.hi && aLo < aHi) {
                        if constexpr (MODE == kScatterAtomic)
                            bulk_reduce_add_1d<T>(reinterpret_cast<void*>(aLo), r.buf + (uint32_t)(aLo - r.base), (uint32_t)(aHi - aLo));
                        else
                            bulk_store_1d_nocommit(reinterpret_cast<void*>(aLo), r.buf + (uint32_t)(aLo - r.base), (uint32_t)(aHi - aLo));
                    }
                }
                bulk_commit();
            }
            // ... and the two ragged ends of every run element by element (side 0: head, side 1: tail)
            for (int t = threadIdx.x; t < 2 * rows; t += kRawThreads) {
                const Row r = row_of(t >> 1);
                if (r.lo >= r.hi)
                    continue;
                const long long aLo = (r.lo + 15) & ~15ll, aHi = r.hi & ~15ll;
                long long b, end;
                if (aLo >= aHi)            // no whole vector inside the run: all of it is the head
                    b = r.lo, end = (t & 1) ? r.lo : r.hi;
                else if (t & 1)
                    b = aHi, end = r.hi;
                else
                    b = r.lo, end = aLo;
                constexpr int kEnd = MODE == kScatterAtomic ? kScatterAtomic : kScatterSet;
                while (b < end) {
                    const uint32_t at = r.buf + (uint32_t)(b - r.base);
                    if (SZ == 2 && (b & 3) == 0 && b + 4 <= end) {
                        // two 16-bit elements as one word (a packed reduction; the one-element form is far slower)
                        const uint32_t e2 = lds32(at);
                        image_write<4, kEnd, T>(reinterpret_cast<uint32_t*>(b), e2, e2);
                        b += 4;
                    } else {
                        const E e = SZ == 4 ? (E)lds32(at) : (E)lds16(at);
                        image_write<SZ, kEnd, T>(reinterpret_cast<E*>(b), e, e);
                        b += SZ;
                    }
                }
            }
            if (kEngine && warp == 0)
                bulk_wait_read<0>();   // the engine has read the buffers
        }
        __syncthreads();   // the row buffers are reused by the next item
    }
    pdl_launch_dependents();
}

// ---- host side -----------------------------------------------------------------------------------
int sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// CTAs of `kernel` that fit one SM at once (a property of the kernel and of sm_100a, the only target);
// persistent grids are sized to exactly one resident wave of the CURRENT device.
template <typename K> static int ctas_per_sm(K kernel, int threads)
{
    int perSm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kernel, threads, 0) != cudaSuccess || perSm < 1) {
        (void)cudaGetLastError();
        perSm = 1;
    }
    return perSm;
}

static int pick_vector_bytes(const BlockArgs& a, int itemsize)
{
    const size_t pixelBytes = (size_t)a.C * itemsize;
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(a.image) | reinterpret_cast<uintptr_t>(a.stack);
    for (int vb = 16; vb > itemsize; vb >>= 1)
        if (pixelBytes % vb == 0 && (ptrs & (vb - 1)) == 0)
            return vb;
    return itemsize;
}

template <int MODE, typename T> static bool launch_planes_rows(const BlockArgs& a, cudaStream_t stream, bool rowsLayout);

template <int VB, int MODE, typename T>
static void launch_rows(const BlockArgs& a, cudaStream_t stream)
{
    // Vectors of 4 or 2 bytes (pixels that are not 8-byte multiples, or buffers aligned no better): the raw-row
    // kernel, which moves 16-byte vectors on both sides whatever the pixel size, where a block row fits its tile.
    // Measured on [8,512,512,C] at 20 %, this kernel -> raw rows: C = 33 fp32 gather 38.9 -> 32.7 us, overwrite
    // 40.9 -> 30.7 us, atomic add 45.1 -> 45.0 us; C = 33 fp16 (2-byte vectors, one-element reductions) atomic add
    // 191 -> 38.9 us, overwrite 37.0 -> 20.4 us.  8-byte vectors stay here (C = 100 fp16: 41.0 vs 42.9 us gather,
    // 57.4 vs 69.7 us atomic add).  Option planes=4 keeps this kernel for every width.
    if (VB <= 4 && options().planes != 4 && launch_planes_rows<MODE, T>(a, stream, true))
        return;
    const int itemsize = (int)sizeof(T);
    RowPlan p;
    p.vecsPerPixel = (int)((size_t)a.C * itemsize / VB);
    const long long vpr = (long long)a.bSzW * p.vecsPerPixel;
    p.vecsPerRow = FastDiv((uint32_t)vpr);
    p.vecsPerBlock = (int)(vpr * a.bSzH);
    // equal chunks of at most kThreads*kUnroll vectors, rounded up to whole warps
    const int maxChunk = kThreads * kUnroll;
    const int nChunks = (p.vecsPerBlock + maxChunk - 1) / maxChunk;
    p.chunkVecs = (((p.vecsPerBlock + nChunks - 1) / nChunks) + 31) & ~31;
    p.chunksPerBlock = FastDiv((uint32_t)nChunks);
    const long long nItems = (long long)a.numActive * nChunks;
    if (a.num_active_dev == nullptr && nItems <= 0x7fffffffll) {
        launch_pdl(rows_kernel<VB, MODE, T>, dim3((unsigned)nItems), dim3(kThreads), 0, stream, a, p);
    } else {
        static const int perSm = ctas_per_sm(rows_kernel_dyn<VB, MODE, T>, kThreads);
        const int wave = perSm * sm_count();
        const int grid = (int)(nItems < wave ? nItems : wave);
        launch_pdl(rows_kernel_dyn<VB, MODE, T>, dim3(grid), dim3(kThreads), 0, stream, a, p);
    }
}

// Whole block rows as raw bytes (planes_rows_kernel) whenever one row's pixels fit the tile.
template <int MODE, typename T> static bool launch_planes_rows(const BlockArgs& a, cudaStream_t stream, bool rowsLayout)
{
    const long long rowBytes = (long long)a.bSzW * a.C * (long long)sizeof(T);
    const long long rowPitch = ((rowBytes + 15 + 15) / 16) * 16;   // the run, its misalignment (< 16), rounded up
    if (rowPitch > kRawTileBytes)
        return false;
    RawPlan p;
    p.rowPitch = (int)rowPitch;
    p.rowBytes = (int)rowBytes;
    p.stackSlots = FastDiv((uint32_t)((rowBytes + 15 + 15) / 16));
    int rows = (int)(kRawTileBytes / rowPitch);
    rows = rows < a.bSzH ? rows : a.bSzH;
    rows = rows < kRawMaxRows ? rows : kRawMaxRows;
    const int nChunks = (a.bSzH + rows - 1) / rows;
    p.rowsPerItem = (a.bSzH + nChunks - 1) / nChunks;               // the fewest, nearly equal chunks of rows
    // ... of a row count that keeps every item's planes on 16-byte boundaries (vector stack accesses), if that fits
    if (nChunks > 1 && !rowsLayout) {
        int m = 1;
        while (((long long)m * a.bSzW * (long long)sizeof(T)) % 16 != 0)
            m *= 2;
        const int rounded = ((p.rowsPerItem + m - 1) / m) * m;
        if (rounded <= rows)
            p.rowsPerItem = rounded;
    }
    p.rChunks = FastDiv((uint32_t)((a.bSzH + p.rowsPerItem - 1) / p.rowsPerItem));
    p.blockW = FastDiv((uint32_t)a.bSzW);
    // vector stack accesses when every plane of every item starts on the vector's boundary and holds whole vectors:
    // 16 bytes, else (16-bit elements) 8 or 4 bytes
    constexpr int kQuad = 16 / (int)sizeof(T);
    const long long planeBytes = (long long)a.bSzH * a.bSzW * (long long)sizeof(T);
    const long long itemBytes = (long long)p.rowsPerItem * a.bSzW * (long long)sizeof(T);
    auto fits = [&](int vb) {
        return (reinterpret_cast<uintptr_t>(a.stack) & (vb - 1)) == 0 && planeBytes % vb == 0
            && (p.rChunks.div == 1 || itemBytes % vb == 0) && options().planes != 6;
    };
    const bool wide = fits(16);
    // (8-byte vectors for the scatter modes only: measured on C = 100 fp16 18x18 blocks against 4-byte vectors, atomic
    // scatter 86 -> 72 us, but gather 49 -> 53 us -- four pixel runs of 200 bytes apart per lane fall on four banks)
    const int q = wide ? kQuad
                       : (sizeof(T) == 2 && MODE != kGather && fits(8) ? 4 : (sizeof(T) == 2 && fits(4) ? 2 : 1));
    // channel groups: a warp task is 32 lanes x q pixels x one group.  Fewest rounds of the CTA's warps first, then
    // the fewest tasks (each pays its address arithmetic once); the narrow path keeps a group in registers.
    const int pixGroups = (p.rowsPerItem * a.bSzW + 32 * q - 1) / (32 * q);
    const int warps = kRawThreads / 32, maxGroup = q > 1 ? a.C : RawChans<T>::n;
    long long bestCost = -1;
    int bestGroups = 1;
    for (int groups = (a.C + maxGroup - 1) / maxGroup; groups <= a.C; ++groups) {
        const int per = (a.C + groups - 1) / groups;
        if ((long long)(groups - 1) * per >= a.C)
            continue;                                                // an empty last group
        const long long rounds = ((long long)pixGroups * groups + warps - 1) / warps;
        const long long cost = rounds * ((long long)per * q * 3 + 60);   // ~3 instructions per element, ~60 per task
        if (bestCost < 0 || cost < bestCost)
            bestCost = cost, bestGroups = groups;
    }
    p.chanGroups = FastDiv((uint32_t)bestGroups);
    p.chansPerGroup = (a.C + bestGroups - 1) / bestGroups;
    const long long nItems = (long long)a.numActive * p.rChunks.div;
    const bool perItem = a.num_active_dev == nullptr && nItems <= 0x7fffffffll;
    auto go = [&](auto kernel) {
        const int wave = ctas_per_sm(kernel, kRawThreads) * sm_count();
        const unsigned grid = (unsigned)(perItem ? nItems : (nItems < wave ? nItems : wave));
        launch_pdl(kernel, dim3(grid), dim3(kRawThreads), 0, stream, a, p);
    };
    if (rowsLayout) {
        go(planes_rows_kernel<MODE, T, 0>);
    } else if (wide) {
        go(planes_rows_kernel<MODE, T, kQuad>);
    } else if (q == 4) {
        if constexpr (sizeof(T) == 2)
            go(planes_rows_kernel<MODE, T, 4>);
    } else if (q == 2) {
        if constexpr (sizeof(T) == 2)
            go(planes_rows_kernel<MODE, T, 2>);
    } else {
        go(planes_rows_kernel<MODE, T, 1>);
    }
    return true;
}

template <int VB, int MODE, typename T>
static void launch_planes(const BlockArgs& a, cudaStream_t stream)
{
    // The raw-row kernel takes every shape whose block row fits its tile: measured on [8,512,512,C] at 20 %
    // against the element-wise kernel below, C = 33 fp32 gather 65 -> 31 us, atomic scatter 70 -> 43 us; C = 100 fp16
    // gather 93 -> 49 us, atomic scatter 117 -> 86 us.  Option planes=4 keeps the element-wise kernel.
    if (options().planes != 4 && launch_planes_rows<MODE, T>(a, stream, false))
        return;
    const int itemsize = (int)sizeof(T);
    PlanePlan p;
    const int RS = a.bSzH * a.bSzW;
    // channel chunks of at most 256 bytes (a pixel of up to 256 bytes is moved whole, so image rows stay
    // contiguous runs), as even as the vector width allows: 100 fp16 channels run as one chunk, 160 as
    // 80 + 80, never as 128 + 32
    const int chunkElems = 256 / itemsize, epv = VB / itemsize;
    const int wantChunks = (a.C + chunkElems - 1) / chunkElems;
    p.chanPerChunk = (((a.C + wantChunks - 1) / wantChunks + epv - 1) / epv) * epv;
    if (p.chanPerChunk > chunkElems)
        p.chanPerChunk = chunkElems;
    // pitch: an odd number of 32-bit words (2-byte elements with a 2-byte vector: any odd count)
    if (itemsize == 4 || VB == 2) {
        p.pitch = p.chanPerChunk | 1;
    } else {
        const int words = (p.chanPerChunk + 1) / 2;
        p.pitch = (words | 1) * 2;
    }
    const int maxPix = kTileBytes / (p.pitch * itemsize);
    p.pixPerChunk = RS < maxPix ? RS : maxPix;
    const int nC = (a.C + p.chanPerChunk - 1) / p.chanPerChunk;
    const int nP = (RS + p.pixPerChunk - 1) / p.pixPerChunk;
    const int lastChan = a.C - (nC - 1) * p.chanPerChunk;
    const int lastPix = RS - (nP - 1) * p.pixPerChunk;
    p.blockW = FastDiv((uint32_t)a.bSzW);
    p.cChunks = FastDiv((uint32_t)nC);
    p.pChunks = FastDiv((uint32_t)nP);
    p.vecsPerPixelFull = FastDiv((uint32_t)(p.chanPerChunk * itemsize / VB));
    p.vecsPerPixelLast = FastDiv((uint32_t)(lastChan * itemsize / VB));
    p.pixFull = FastDiv((uint32_t)p.pixPerChunk);
    p.pixLast = FastDiv((uint32_t)lastPix);
    const long long nItems = (long long)a.numActive * nC * nP;
    // host-side count: one CTA per item (short CTAs stream faster than a resident grid); device-side
    // count: one resident wave striding over the items
    static const int perSm = ctas_per_sm(planes_kernel<VB, MODE, T>, kThreads);
    const int wave = perSm * sm_count();
    const bool perItem = a.num_active_dev == nullptr && nItems <= 0x7fffffffll;
    const unsigned grid = (unsigned)(perItem ? nItems : (nItems < wave ? nItems : wave));
    launch_pdl(planes_kernel<VB, MODE, T>, dim3(grid), dim3(kThreads), 0, stream, a, p);
}

template <int MODE, typename T>
static void dispatch_vb(const BlockArgs& a, bool transpose, int vb, cudaStream_t stream)
{
#define SBNET_GO(VBYTES)                                       \
    do {                                                       \
        if (transpose)                                         \
            launch_planes<VBYTES, MODE, T>(a, stream);         \
        else                                                   \
            launch_rows<VBYTES, MODE, T>(a, stream);           \
    } while (0)
    switch (vb) {
    case 16: SBNET_GO(16); break;
    case 8: SBNET_GO(8); break;
    case 4: SBNET_GO(4); break;
    default:
        if constexpr (sizeof(T) == 2)
            SBNET_GO(2);
        break;
    }
#undef SBNET_GO
}

template <typename T>
static void dispatch_mode(const BlockArgs& a, int mode, bool transpose, int vb, cudaStream_t stream)
{
    switch (mode) {
    case kGather: dispatch_vb<kGather, T>(a, transpose, vb, stream); break;
    case kScatterSet: dispatch_vb<kScatterSet, T>(a, transpose, vb, stream); break;
    case kScatterAdd: dispatch_vb<kScatterAdd, T>(a, transpose, vb, stream); break;
    default: dispatch_vb<kScatterAtomic, T>(a, transpose, vb, stream); break;
    }
}

cudaError_t launch_blocks(const BlockArgs& a, int dtype, int mode, bool transpose,
                          cudaStream_t stream)
{
    if (a.numActive <= 0)
        return cudaSuccess;
    // fp16 read-add-write over disjoint blocks is done with the packed-half reduction instead: every
    // destination element receives exactly one addend, and red.add.noftz.f16x2 rounds to nearest even
    // without flushing subnormals, so the result is bit-identical while the SM never waits on the
    // destination read.  (fp32 keeps the explicit read-add-write: red.add.f32 flushes subnormals.)
    if (mode == kScatterAdd && dtype != 0)
        mode = kScatterAtomic;
    // bf16 (dtype 2): gather and overwrite move bytes, so they run the fp16 instantiations; only
    // accumulation (red.add.noftz.bf16x2, same argument as for fp16) has kernels of its own.
    if (dtype == 2 && (mode == kGather || mode == kScatterSet))
        dtype = 1;
    const int itemsize = dtype == 0 ? 4 : 2;
    if (transpose) {
        // Aligned shapes have two implementations: one short CTA per tile (planes_simt.cu) and the
        // persistent TMA pipeline (planes_tma.cu, the only one that can read the count on the device).
        // Scatter goes to the tile CTAs, whose swizzled tile lets every warp-level store / reduction
        // cover whole 128-byte image lines (about 20 % faster than the pipeline's dense tile); for
        // gather the two are within a few percent (tile CTAs +3 % at the largest sizes), so the
        // pipeline only serves calls whose block count lives on the device.
        // The `planes` option (SBNET_PLANES=tma|tile) forces one of them (A/B measurements).
        bool taken = false;
        const bool tileFirst = options().planes != 1;
        if (tileFirst) {
            if (cudaError_t e = launch_planes_simt(a, dtype, mode, stream, &taken))
                return e;
            if (taken)
                return cudaSuccess;
        }
        if (cudaError_t e = launch_planes_tma(a, dtype, mode, stream, &taken))
            return e;
        if (taken)
            return cudaSuccess;
    }
    const int vb = pick_vector_bytes(a, itemsize);
    note_site(transpose ? "launch of planes_kernel" : "launch of rows_kernel");
    if (dtype == 0)
        dispatch_mode<float>(a, mode, transpose, vb, stream);
    else if (dtype == 2)
        dispatch_vb<kScatterAtomic, __nv_bfloat16>(a, transpose, vb, stream);
    else
        dispatch_mode<__half>(a, mode, transpose, vb, stream);
    return cudaGetLastError();
}

cudaError_t read_rows_wait_timeouts(unsigned int* out)
{
    return cudaMemcpyFromSymbol(out, g_rows_wait_timeouts, sizeof(unsigned int));
}

// ---- flat copy (the non-Var scatter's "y = ybase") -----------------------------------------------
// One short CTA per 8 KB: two 16-byte vectors per thread, both loads issued before the stores.
constexpr int kCopyUnroll = 2;
__global__ void __launch_bounds__(kThreads) copy_kernel(uint4* __restrict__ dst,
                                                        const uint4* __restrict__ src, size_t nVec,
                                                        unsigned char* dstTail,
                                                        const unsigned char* srcTail, int tailBytes)
{
    pdl_wait();   // nothing is read or written before the kernel queued ahead of this one is done
    const size_t base = (size_t)blockIdx.x * (kThreads * kCopyUnroll) + threadIdx.x;
    uint4 v[kCopyUnroll];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u)
        if (base + u * kThreads < nVec)
            v[u] = src[base + u * kThreads];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u)
        if (base + u * kThreads < nVec)
            dst[base + u * kThreads] = v[u];
    if (blockIdx.x == 0 && (int)threadIdx.x < tailBytes)
        dstTail[threadIdx.x] = srcTail[threadIdx.x];
    pdl_launch_dependents();
}

__global__ void copy_bytes_kernel(unsigned char* dst, const unsigned char* src, size_t n)
{
    pdl_wait();   // nothing is read or written before the kernel queued ahead of this one is done
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = src[i];
    pdl_launch_dependents();
}

cudaError_t launch_copy(void* dst, const void* src, size_t bytes, cudaStream_t stream)
{
    if (bytes == 0 || dst == src)
        return cudaSuccess;
    const long long cap = (long long)sm_count() * 8;
    if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0 &&
        bytes / 16 / (kThreads * kCopyUnroll) < 0x7fffffffull) {
        const size_t nVec = bytes / 16;
        const int tail = (int)(bytes - nVec * 16);
        const size_t want = (nVec + kThreads * kCopyUnroll - 1) / (kThreads * kCopyUnroll);
        const unsigned grid = (unsigned)(want < 1 ? 1 : want);
        launch_pdl(copy_kernel, dim3(grid), dim3(kThreads), 0, stream, reinterpret_cast<uint4*>(dst),
                   reinterpret_cast<const uint4*>(src), nVec, reinterpret_cast<unsigned char*>(dst) + nVec * 16,
                   reinterpret_cast<const unsigned char*>(src) + nVec * 16, tail);
    } else {
        long long want = (long long)((bytes + kThreads - 1) / kThreads);
        const int grid = (int)(want < cap ? want : cap);
        launch_pdl(copy_bytes_kernel, dim3(grid), dim3(kThreads), 0, stream, reinterpret_cast<unsigned char*>(dst),
                   reinterpret_cast<const unsigned char*>(src), bytes);
    }
    return cudaGetLastError();
}

} // namespace sbnet
