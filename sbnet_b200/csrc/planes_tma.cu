// Transposed ([nB,C,R,S]) gather and scatter through the TMA unit (sm_100a).
//
// Three things live here, all of them users of tiled TMA loads from the NHWC image (semantics as the
// reference: sbnet_ops/sparse_gather.cc:61-132, transposed branches of
// sbnet_ops/sparse_blocks.cu.h:135-171 and :217-251):
//  * planes_gather_tma_tile / planes_gather_tma_rows (further down): the default gather when the
//    block count is on the host -- one short CTA per tile, the tile filled by TMA;
//  * planes_gather_tma / planes_scatter_tma (next): a persistent pipeline for C*sizeof(T) a multiple
//    of 128 bytes and blocks of at most 384 pixels.  It serves gather calls whose block count lives
//    in device memory (a resident grid does not need the count at launch) and is the A/B partner of
//    the one-CTA-per-tile kernels.
//
// One persistent CTA per SM: a producer warp keeps a ring of shared-memory stages filled through
// the async proxy, eight consumer warps transpose out of them.  A work item is one active block x
// one 128-byte channel chunk, i.e. a tile of P = R*S pixels x 128 bytes.
//
//  gather : the producer issues ONE tiled TMA load per item from the NHWC image, box
//           (128 B of channels, S, R); coordinates may start before 0 or run past the image and the
//           TMA unit zero-fills there, which is exactly the op's padding rule.  The stage uses the
//           128-byte swizzle, so consumers read 16-byte channel groups without bank conflicts,
//           regroup them into words of one channel (1 fp32 pixel or 2 fp16 pixels), and build the
//           tile in [channel][pixel] order in a second stage, which leaves as ONE bulk store: the
//           channel planes of a chunk are contiguous in the stack.
//  scatter: the producer issues ONE 1-D bulk load per item (the chunk's planes are contiguous),
//           consumers regroup words into 16-byte channel groups and write / add / reduce them into
//           the image with a per-pixel in-range test.  For the read-add-write mode every thread
//           first issues all of its destination loads for the tile, so the SM keeps ~50 KB of image
//           reads in flight despite running a single CTA.
//
// Every wait on an mbarrier is bounded (about a second of SM clock); a wait that gives up raises a
// CTA-wide abort flag, counts itself in g_wait_timeouts, and the CTA drains and returns.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <stdlib.h>

#include <algorithm>
#include <mutex>

#include "async_ptx.cuh"
#include "common.cuh"
#include "kernels.h"
#include "options.h"

namespace sbnet {

constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kTmaThreads = kConsumers + 32;
constexpr int kMaxPixels = 384;                     // 48 KB stages

__device__ unsigned int g_wait_timeouts = 0;

struct TmaPlan {
    FastDiv cChunks;      // 128-byte channel chunks per pixel
    FastDiv blockW;       // S
    int pixels;           // P = R*S
    int units;            // 32-bit words per channel plane row: P (fp32) or P/2 (fp16)
    int tileBytes;        // 128 * P
    int inStages, outStages;
    int inStageBytes, outStageBytes;
};

// ---- PTX wrappers (mbarriers, TMA loads: async_ptx.cuh) -------------------------------------------
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abortFlag)
{
    return mbar_wait_bounded(bar, parity, abortFlag, &g_wait_timeouts);
}
// Barrier among the consumer warps only (the producer warp never joins), with an OR vote.
__device__ __forceinline__ bool consumers_any(bool pred)
{
    uint32_t out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(out)
        : "r"((uint32_t)pred), "n"(kConsumers)
        : "memory");
    return out != 0;
}
__device__ __forceinline__ void consumers_sync()
{
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
}

struct Ring {
    uint32_t in0, out0, full0, empty0;   // shared-space addresses
};

// Carves the dynamic shared memory: swizzled input stages need 1024-byte alignment.
__device__ __forceinline__ Ring carve(unsigned char* dyn, const TmaPlan& p)
{
    Ring r;
    r.in0 = (smem_u32(dyn) + 1023u) & ~1023u;
    r.out0 = r.in0 + (uint32_t)p.inStages * p.inStageBytes;
    r.full0 = r.out0 + (uint32_t)p.outStages * p.outStageBytes;
    r.empty0 = r.full0 + 8u * p.inStages;
    return r;
}

__device__ __forceinline__ void ring_init(const Ring& r, const TmaPlan& p, int* abortFlag)
{
    if (threadIdx.x == 0) {
        *abortFlag = 0;
        for (int s = 0; s < p.inStages; ++s) {
            mbar_init(r.full0 + 8u * s, 1);
            mbar_init(r.empty0 + 8u * s, kConsumerWarps);
        }
        mbar_init_fence();
        fence_async_smem();
    }
    __syncthreads();
}

// Producer, after its last issue: waits (bounded, on a flag of its own, so that an abort raised by
// the consumers does not cut it short) until the last loads it issued -- `issued` in total, at most
// one per stage still open -- have landed.  The CTA's shared memory is therefore never given back
// with a copy in flight over it, whether the consumers finished their items or gave up.
__device__ __forceinline__ void drain_loads(const Ring& r, const TmaPlan& p, int issued)
{
    int gaveUp = 0;
    for (int j = max(issued - p.inStages, 0); j < issued; ++j)
        if (!mbar_wait(r.full0 + 8u * (uint32_t)(j % p.inStages), (uint32_t)(j / p.inStages) & 1u, &gaveUp))
            break;
}

__device__ __forceinline__ int device_count(const BlockArgs& a)
{
    if (a.num_active_dev == nullptr)
        return a.numActive;
    const int n = __ldg(a.num_active_dev);
    return n < a.numActive ? n : a.numActive;
}

// ---- gather -------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kTmaThreads, 1)
planes_gather_tma(const __grid_constant__ CUtensorMap imageMap, const BlockArgs a, const TmaPlan p)
{
    extern __shared__ unsigned char dynSmem[];
    __shared__ int abortFlag;
    constexpr int EPW = 4 / (int)sizeof(T);        // pixels per 32-bit word of a channel plane
    constexpr int CPG = 16 / (int)sizeof(T);       // channels per 16-byte group
    const Ring ring = carve(dynSmem, p);
    ring_init(ring, p, &abortFlag);
    pdl_wait();   // nothing global is read or written before the kernel queued ahead of this one is done

    const long long nItems = (long long)device_count(a) * p.cChunks.div;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (warp == kConsumerWarps) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int k = 0;
            for (long long item = blockIdx.x; item < nItems; item += gridDim.x, ++k) {
                const int s = k % p.inStages;
                const uint32_t parity = (uint32_t)(k / p.inStages) & 1u;
                if (!mbar_wait(ring.empty0 + 8u * s, parity ^ 1u, &abortFlag))
                    break;
                uint32_t ib, cc;
                p.cChunks.divmod((uint32_t)item, ib, cc);
                const int n = a.idx[ib * 3 + 0];
                const int h0 = a.bOffsH + a.idx[ib * 3 + 1] * a.bStrH;
                const int w0 = a.bOffsW + a.idx[ib * 3 + 2] * a.bStrW;
                mbar_expect_tx(ring.full0 + 8u * s, (uint32_t)p.tileBytes);
                tma_load_4d(ring.in0 + (uint32_t)s * p.inStageBytes, &imageMap,
                            (int)cc * (128 / (int)sizeof(T)), w0, h0, n, ring.full0 + 8u * s);
            }
            drain_loads(ring, p, k);
        }
        pdl_launch_dependents();
        return;
    }

    // ---------------- consumers ----------------
    T* stack = reinterpret_cast<T*>(a.stack);
    const int U = p.units;
    const int nTasks = ((U + 15) >> 4) * 128;
    int k = 0;
    for (long long item = blockIdx.x; item < nItems; item += gridDim.x, ++k) {
        const int s = k % p.inStages, o = k % p.outStages;
        const uint32_t parity = (uint32_t)(k / p.inStages) & 1u;
        int ok = 1;
        if (lane == 0)
            ok = mbar_wait(ring.full0 + 8u * s, parity, &abortFlag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);   // reconverges the warp before the CTA-level vote
        if (consumers_any(ok == 0))   // also orders: thread 0 has drained the store that used out[o]
            break;
        const uint32_t in = ring.in0 + (uint32_t)s * p.inStageBytes;
        const uint32_t out = ring.out0 + (uint32_t)o * p.outStageBytes;
        for (int t = threadIdx.x; t < nTasks; t += kConsumers) {
            int j, u;
            transpose_task<EPW>(t, j, u);
            if (u >= U)
                continue;
            if constexpr (EPW == 2) {
                const int r0 = 2 * u, r1 = 2 * u + 1;
                const uint4 A = lds128(in + r0 * 128 + ((j ^ (r0 & 7)) << 4));
                const uint4 B = lds128(in + r1 * 128 + ((j ^ (r1 & 7)) << 4));
                const uint32_t base = out + ((uint32_t)(CPG * j) * U + u) * 4u;
                sts32(base + 0u * U * 4u, __byte_perm(A.x, B.x, 0x5410));
                sts32(base + 1u * U * 4u, __byte_perm(A.x, B.x, 0x7632));
                sts32(base + 2u * U * 4u, __byte_perm(A.y, B.y, 0x5410));
                sts32(base + 3u * U * 4u, __byte_perm(A.y, B.y, 0x7632));
                sts32(base + 4u * U * 4u, __byte_perm(A.z, B.z, 0x5410));
                sts32(base + 5u * U * 4u, __byte_perm(A.z, B.z, 0x7632));
                sts32(base + 6u * U * 4u, __byte_perm(A.w, B.w, 0x5410));
                sts32(base + 7u * U * 4u, __byte_perm(A.w, B.w, 0x7632));
            } else {
                const uint4 A = lds128(in + u * 128 + ((j ^ (u & 7)) << 4));
                const uint32_t base = out + ((uint32_t)(CPG * j) * U + u) * 4u;
                sts32(base + 0u * U * 4u, A.x);
                sts32(base + 1u * U * 4u, A.y);
                sts32(base + 2u * U * 4u, A.z);
                sts32(base + 3u * U * 4u, A.w);
            }
        }
        fence_async_smem();     // the bulk store reads what the generic proxy just wrote
        __syncwarp();
        consumers_sync();
        if (lane == 0)
            mbar_arrive(ring.empty0 + 8u * s);
        if (threadIdx.x == 0) {
            uint32_t ib, cc;
            p.cChunks.divmod((uint32_t)item, ib, cc);
            T* dst = stack + ((long long)ib * a.C + (long long)cc * (128 / (int)sizeof(T))) * p.pixels;
            bulk_store_1d(dst, out, (uint32_t)p.tileBytes);
            // the other out stage is written next: its previous store must have finished reading
            bulk_wait_read<1>();
        }
        __syncwarp();
    }
    pdl_launch_dependents();
    if (threadIdx.x == 0)
        bulk_wait_all();
}

// ---- scatter ------------------------------------------------------------------------------------
template <int MODE, typename T>
__global__ void __launch_bounds__(kTmaThreads, 1) planes_scatter_tma(const BlockArgs a, const TmaPlan p)
{
    extern __shared__ unsigned char dynSmem[];
    __shared__ int abortFlag;
    constexpr int EPW = 4 / (int)sizeof(T);
    constexpr int CPG = 16 / (int)sizeof(T);
    // tasks per thread: ceil(units/16) groups of 16 units x 8 channel groups over 256 threads
    constexpr int kMaxTasks = ((kMaxPixels / EPW + 15) / 16 + 1) / 2;
    const Ring ring = carve(dynSmem, p);
    ring_init(ring, p, &abortFlag);
    pdl_wait();   // nothing global is read or written before the kernel queued ahead of this one is done

    const long long nItems = (long long)device_count(a) * p.cChunks.div;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* stack = reinterpret_cast<const T*>(a.stack);

    if (warp == kConsumerWarps) {
        if (lane == 0) {
            int k = 0;
            for (long long item = blockIdx.x; item < nItems; item += gridDim.x, ++k) {
                const int s = k % p.inStages;
                const uint32_t parity = (uint32_t)(k / p.inStages) & 1u;
                if (!mbar_wait(ring.empty0 + 8u * s, parity ^ 1u, &abortFlag))
                    break;
                uint32_t ib, cc;
                p.cChunks.divmod((uint32_t)item, ib, cc);
                const T* src = stack + ((long long)ib * a.C + (long long)cc * (128 / (int)sizeof(T))) * p.pixels;
                mbar_expect_tx(ring.full0 + 8u * s, (uint32_t)p.tileBytes);
                bulk_load_1d(ring.in0 + (uint32_t)s * p.inStageBytes, src, (uint32_t)p.tileBytes,
                             ring.full0 + 8u * s);
            }
            drain_loads(ring, p, k);
        }
        pdl_launch_dependents();
        return;
    }

    T* image = reinterpret_cast<T*>(a.image);
    const int U = p.units;
    const int nTasks = ((U + 15) >> 4) * 128;
    int k = 0;
    for (long long item = blockIdx.x; item < nItems; item += gridDim.x, ++k) {
        const int s = k % p.inStages;
        const uint32_t parity = (uint32_t)(k / p.inStages) & 1u;
        uint32_t ib, cc;
        p.cChunks.divmod((uint32_t)item, ib, cc);
        const int n = a.idx[ib * 3 + 0];
        const int h0 = a.bOffsH + a.idx[ib * 3 + 1] * a.bStrH;
        const int w0 = a.bOffsW + a.idx[ib * 3 + 2] * a.bStrW;
        T* imgN = image + (long long)n * a.H * a.W * a.C + (long long)cc * (128 / (int)sizeof(T));

        // destination vector of (pixel, 16-byte group), or nullptr when the pixel is outside
        auto dest = [&](int pix, int j) -> uint4* {
            uint32_t r, sx;
            p.blockW.divmod((uint32_t)pix, r, sx);
            const int h = h0 + (int)r, w = w0 + (int)sx;
            if (h < 0 || h >= a.H || w < 0 || w >= a.W)
                return nullptr;
            return reinterpret_cast<uint4*>(imgN + ((long long)h * a.W + w) * a.C + j * CPG);
        };

        // read-add-write: all destination loads of this thread's share of the tile go out first
        uint4 old[kMaxTasks][EPW];
        if constexpr (MODE == kScatterAdd) {
#pragma unroll
            for (int q = 0; q < kMaxTasks; ++q) {
                const int t = threadIdx.x + q * kConsumers;
                const int uLocal = t & 15, grp = t >> 4;
                const int j = grp & 7, u = ((grp >> 3) << 4) + uLocal;
#pragma unroll
                for (int e = 0; e < EPW; ++e) {
                    old[q][e] = make_uint4(0, 0, 0, 0);
                    if (t < nTasks && u < U) {
                        const uint4* d = dest(u * EPW + e, j);
                        if (d)
                            old[q][e] = *d;
                    }
                }
            }
        }

        // warps run independently: each polls the stage itself and releases it itself
        int ok = 1;
        if (lane == 0)
            ok = mbar_wait(ring.full0 + 8u * s, parity, &abortFlag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok == 0)
            break;
        const uint32_t in = ring.in0 + (uint32_t)s * p.inStageBytes;
#pragma unroll
        for (int q = 0; q < kMaxTasks; ++q) {
            const int t = threadIdx.x + q * kConsumers;
            const int uLocal = t & 15, grp = t >> 4;
            const int j = grp & 7, u = ((grp >> 3) << 4) + uLocal;
            if (t >= nTasks || u >= U)
                continue;
            const uint32_t base = in + ((uint32_t)(CPG * j) * U + u) * 4u;
            if constexpr (EPW == 2) {
                uint32_t w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    w[i] = lds32(base + (uint32_t)i * U * 4u);
                const uint4 v0 = make_uint4(__byte_perm(w[0], w[1], 0x5410), __byte_perm(w[2], w[3], 0x5410),
                                            __byte_perm(w[4], w[5], 0x5410), __byte_perm(w[6], w[7], 0x5410));
                const uint4 v1 = make_uint4(__byte_perm(w[0], w[1], 0x7632), __byte_perm(w[2], w[3], 0x7632),
                                            __byte_perm(w[4], w[5], 0x7632), __byte_perm(w[6], w[7], 0x7632));
                if (uint4* d = dest(2 * u, j))
                    image_write<16, MODE, T>(d, v0, old[q][0]);
                if (uint4* d = dest(2 * u + 1, j))
                    image_write<16, MODE, T>(d, v1, old[q][EPW - 1]);
            } else {
                const uint4 v = make_uint4(lds32(base), lds32(base + (uint32_t)U * 4u),
                                           lds32(base + 2u * U * 4u), lds32(base + 3u * U * 4u));
                if (uint4* d = dest(u, j))
                    image_write<16, MODE, T>(d, v, old[q][0]);
            }
        }
        __syncwarp();          // this warp is done reading the stage
        if (lane == 0)
            mbar_arrive(ring.empty0 + 8u * s);
    }
    pdl_launch_dependents();
}

// ---- gather, one short CTA per tile, fed by TMA ---------------------------------------------------
// The default gather for blocks of at most 384 pixels when the block count is on the host: the tile
// of planes_simt.cu (one block, or several small blocks sharing the 48 KB), but filled by one tiled
// TMA load per block issued by one thread (zero fill outside the image included) instead of by
// plain loads.  That frees the registers and instructions of the load phase -- the 256 threads only
// transpose -- which is worth about 3 % on one-block tiles (four CTAs per SM for fp32 too) and up
// to 20 % on shared tiles, where plain loads are issue-bound (two divisions and an index lookup per
// 16-byte load).  Block b's box lands at region b of the tile; regions are padded to a multiple of 8
// pixels (1,024 bytes) so that the 128-byte swizzle pattern of every box starts at its own first
// pixel.  Each region is transposed in place and leaves as its own bulk store.
struct TmaTilePlan {
    FastDiv cChunks;    // 128-byte channel chunks per pixel
    FastDiv unitsDiv;   // units
    int pixels;         // P
    int units;          // words per channel plane row: P (fp32) or P/2 (16-bit types, P even)
    int regionPixels;   // P rounded up to a multiple of 8
    int blocksPerItem;
    int groups;         // 16-byte channel groups per pixel; the last chunk may hold fewer than 8
};
constexpr int kTileThreads = 256;
constexpr int kTileBytesMax = 128 * kMaxPixels;

// Whole CTA: waits for the tile's TMA loads.  Every warp's lane 0 waits (bounded); a warp that
// gives up waits once more, again bounded, so that this CTA's copies are not left in flight over
// shared memory it has given back.  false (for every thread) if any warp gave up.
__device__ __forceinline__ bool tile_arrived(uint32_t bar, int* abortFlag)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) {
        ok = mbar_wait(bar, 0, abortFlag) ? 1 : 0;
        if (!ok) {
            int again = 0;
            (void)mbar_wait(bar, 0, &again);
        }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return __syncthreads_or(ok == 0) == 0;
}

// ODD (16-bit blocks of an odd pixel count): plane rows are an odd number of halves, so a channel's
// row starts on a word boundary only for even channels; words of odd channels are written as two
// halves, and p.units counts a row's words rounded up.
template <typename T, bool ODD = false>
__global__ void __launch_bounds__(kTileThreads, 4)
planes_gather_tma_tile(const __grid_constant__ CUtensorMap imageMap, const BlockArgs a, const TmaTilePlan p)
{
    static_assert(!ODD || sizeof(T) == 2, "odd rows of halves: 16-bit types only");
    extern __shared__ unsigned char dynSmem[];
    __shared__ __align__(8) unsigned long long barStorage;
    __shared__ int abortFlag;
    constexpr int EPW = 4 / (int)sizeof(T);
    constexpr int CPG = 16 / (int)sizeof(T);
    constexpr int kMaxTasks = ((kMaxPixels / EPW + 15) / 16 + 1) / 2;
    const uint32_t tile = (smem_u32(dynSmem) + 1023u) & ~1023u;
    const uint32_t bar = smem_u32(&barStorage);

    uint32_t grp, cc;
    p.cChunks.divmod(blockIdx.x, grp, cc);
    const uint32_t ib = grp * (uint32_t)p.blocksPerItem;
    if (threadIdx.x == 0) {
        abortFlag = 0;
        mbar_init(bar, 1);
        mbar_init_fence();
        fence_async_smem();
    }
    __syncthreads();
    pdl_wait();   // nothing global is read or written before the kernel queued ahead of this one is done
    // With the block count on the device the grid covers the largest possible count and the CTAs
    // past the actual one leave at once.
    const int nActive = device_count(a);
    if ((int)ib >= nActive)
        return;
    const int nBlk = min(p.blocksPerItem, nActive - (int)ib);
    const int nG = min(8, p.groups - 8 * (int)cc);
    const uint32_t regionBytes = (uint32_t)p.regionPixels * 128u;
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar, (uint32_t)nBlk * (uint32_t)p.pixels * 128u);
        for (int b = 0; b < nBlk; ++b) {
            const int16_t* ix = a.idx + (size_t)(ib + b) * 3;
            tma_load_4d(tile + (uint32_t)b * regionBytes, &imageMap, (int)cc * (128 / (int)sizeof(T)),
                        a.bOffsW + ix[2] * a.bStrW, a.bOffsH + ix[1] * a.bStrH, ix[0], bar);
        }
    }
    if (!tile_arrived(bar, &abortFlag))
        return;
    pdl_launch_dependents();   // this CTA's loads have landed: the next kernel's CTAs may take the slots that free up

    // ---- tile -> registers (16-byte channel groups), then registers -> tile in [channel][pixel] order
    const int U = nBlk * p.units;
    const int nTasks = ((U + 15) >> 4) * 128;
    uint4 A[kMaxTasks], B[kMaxTasks];
#pragma unroll
    for (int q = 0; q < kMaxTasks; ++q) {
        const int t = threadIdx.x + q * kTileThreads;
        int j, u;
        transpose_task<EPW>(t, j, u);
        if (t < nTasks && u < U && j < nG) {
            uint32_t b, uIn;
            p.unitsDiv.divmod((uint32_t)u, b, uIn);
            const uint32_t region = tile + b * regionBytes;
            const uint32_t r0 = EPW * uIn;   // pixel inside the block: the swizzle restarts with every region
            A[q] = lds128(region + r0 * 128u + ((j ^ (r0 & 7u)) << 4));
            if constexpr (EPW == 2) {
                B[q] = make_uint4(0, 0, 0, 0);
                if (!ODD || (int)r0 + 1 < p.pixels)   // an odd row's last word holds one pixel
                    B[q] = lds128(region + (r0 + 1u) * 128u + ((j ^ ((r0 + 1u) & 7u)) << 4));
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kMaxTasks; ++q) {
        const int t = threadIdx.x + q * kTileThreads;
        int j, u;
        transpose_task<EPW>(t, j, u);
        if (t < nTasks && u < U && j < nG) {
            uint32_t b, uIn;
            p.unitsDiv.divmod((uint32_t)u, b, uIn);
            const uint32_t base = tile + b * regionBytes + ((uint32_t)(CPG * j) * p.units + uIn) * 4u;
            const uint32_t pitch = (uint32_t)p.units * 4u;
            if constexpr (ODD) {
                const uint32_t region = tile + b * regionBytes;
                const bool second = (int)(2u * uIn) + 1 < p.pixels;
                const uint32_t wd[8] = {__byte_perm(A[q].x, B[q].x, 0x5410), __byte_perm(A[q].x, B[q].x, 0x7632),
                                        __byte_perm(A[q].y, B[q].y, 0x5410), __byte_perm(A[q].y, B[q].y, 0x7632),
                                        __byte_perm(A[q].z, B[q].z, 0x5410), __byte_perm(A[q].z, B[q].z, 0x7632),
                                        __byte_perm(A[q].w, B[q].w, 0x5410), __byte_perm(A[q].w, B[q].w, 0x7632)};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    // half index of (channel 8j+i, pixel 2*uIn): even exactly for even channels
                    const uint32_t at = region + ((uint32_t)(CPG * j + i) * (uint32_t)p.pixels + 2u * uIn) * 2u;
                    if ((i & 1) == 0 && second) {
                        sts32(at, wd[i]);
                    } else {
                        sts16(at, wd[i] & 0xffffu);
                        if (second)
                            sts16(at + 2u, wd[i] >> 16);
                    }
                }
            } else if constexpr (EPW == 2) {
                sts32(base + 0u * pitch, __byte_perm(A[q].x, B[q].x, 0x5410));
                sts32(base + 1u * pitch, __byte_perm(A[q].x, B[q].x, 0x7632));
                sts32(base + 2u * pitch, __byte_perm(A[q].y, B[q].y, 0x5410));
                sts32(base + 3u * pitch, __byte_perm(A[q].y, B[q].y, 0x7632));
                sts32(base + 4u * pitch, __byte_perm(A[q].z, B[q].z, 0x5410));
                sts32(base + 5u * pitch, __byte_perm(A[q].z, B[q].z, 0x7632));
                sts32(base + 6u * pitch, __byte_perm(A[q].w, B[q].w, 0x5410));
                sts32(base + 7u * pitch, __byte_perm(A[q].w, B[q].w, 0x7632));
            } else {
                sts32(base + 0u * pitch, A[q].x);
                sts32(base + 1u * pitch, A[q].y);
                sts32(base + 2u * pitch, A[q].z);
                sts32(base + 3u * pitch, A[q].w);
            }
        }
    }
    fence_async_smem();   // the bulk stores read what the generic proxy just wrote
    __syncthreads();
    if ((int)threadIdx.x < nBlk) {   // block b's planes of this chunk: one contiguous run of the stack
        T* dst = reinterpret_cast<T*>(a.stack) +
                 ((long long)(ib + threadIdx.x) * a.C + (long long)cc * (128 / (int)sizeof(T))) * p.pixels;
        bulk_store_1d(dst, tile + threadIdx.x * regionBytes, (uint32_t)(16 * nG * p.pixels));
        bulk_wait_read<0>();
    }
}

// ---- gather of blocks of more than 384 pixels: row chunks fed by TMA -----------------------------
// A work item is (block, chunk of whole block rows, channel chunk): the chunk is a box of the image,
// so one TMA load fills the tile; two tensor maps, one for full chunks and one for the shorter last
// chunk of a block.  After the in-place transposition the tile holds one word-aligned row per channel
// plane, which leaves as a run of the stack's plane row: one bulk store per plane where runs are
// 16-byte multiples, else 8- or 4-byte stores, else (16-bit runs that start on an odd half) the first
// half, words funnel-shifted out of two tile words, and the last half.
struct TmaRowsPlan {
    FastDiv cChunks;     // 128-byte channel chunks per pixel
    FastDiv rChunks;     // row chunks per block
    int groups;          // 16-byte channel groups per pixel
    int pixels;          // P = R*S
    int blockW;          // S
    int blockH;          // R
    int chunkRows;       // block rows per chunk; the last chunk of a block holds blockH - (rChunks-1)*chunkRows
};

template <typename T>
__global__ void __launch_bounds__(kTileThreads, 4)
planes_gather_tma_rows(const __grid_constant__ CUtensorMap mapFull, const __grid_constant__ CUtensorMap mapLast,
                       const BlockArgs a, const TmaRowsPlan p)
{
    extern __shared__ unsigned char dynSmem[];
    __shared__ __align__(8) unsigned long long barStorage;
    __shared__ int abortFlag;
    constexpr int EPW = 4 / (int)sizeof(T);
    constexpr int CPG = 16 / (int)sizeof(T);
    constexpr int kMaxTasks = ((kMaxPixels / EPW + 15) / 16 + 1) / 2;
    const uint32_t tile = (smem_u32(dynSmem) + 1023u) & ~1023u;
    const uint32_t bar = smem_u32(&barStorage);

    uint32_t rest, cc, ib, kc;
    p.cChunks.divmod(blockIdx.x, rest, cc);
    p.rChunks.divmod(rest, ib, kc);
    pdl_wait();   // nothing global is read or written before the kernel queued ahead of this one is done
    if ((int)ib >= device_count(a))   // count on the device: the grid covers the largest possible count
        return;
    const bool last = kc + 1 == p.rChunks.div;
    const int rows = last ? p.blockH - (int)kc * p.chunkRows : p.chunkRows;
    const int P = rows * p.blockW;            // pixels of this chunk
    const int p0 = (int)kc * p.chunkRows * p.blockW;
    const int U = (P + EPW - 1) / EPW;        // words per tile row
    const int nG = min(8, p.groups - 8 * (int)cc);

    if (threadIdx.x == 0) {
        abortFlag = 0;
        mbar_init(bar, 1);
        mbar_init_fence();
        fence_async_smem();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int16_t* ix = a.idx + (size_t)ib * 3;
        mbar_expect_tx(bar, (uint32_t)P * 128u);
        tma_load_4d(tile, last ? &mapLast : &mapFull, (int)cc * (128 / (int)sizeof(T)), a.bOffsW + ix[2] * a.bStrW,
                    a.bOffsH + ix[1] * a.bStrH + (int)kc * p.chunkRows, ix[0], bar);
    }
    if (!tile_arrived(bar, &abortFlag))
        return;
    pdl_launch_dependents();

    // ---- tile -> registers (16-byte channel groups), then registers -> tile in [channel][pixel] order
    const int nTasks = ((U + 15) >> 4) * 128;
    uint4 A[kMaxTasks], B[kMaxTasks];
#pragma unroll
    for (int q = 0; q < kMaxTasks; ++q) {
        const int t = threadIdx.x + q * kTileThreads;
        int j, u;
        transpose_task<EPW>(t, j, u);
        if (t < nTasks && u < U && j < nG) {
            const uint32_t r0 = EPW * u;
            A[q] = lds128(tile + r0 * 128u + ((j ^ (r0 & 7u)) << 4));
            if constexpr (EPW == 2) {
                B[q] = make_uint4(0, 0, 0, 0);
                if ((int)r0 + 1 < P)   // a chunk of an odd pixel count: the last word holds one pixel
                    B[q] = lds128(tile + (r0 + 1u) * 128u + ((j ^ ((r0 + 1u) & 7u)) << 4));
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kMaxTasks; ++q) {
        const int t = threadIdx.x + q * kTileThreads;
        int j, u;
        transpose_task<EPW>(t, j, u);
        if (t < nTasks && u < U && j < nG) {
            const uint32_t base = tile + ((uint32_t)(CPG * j) * U + u) * 4u;
            const uint32_t pitch = (uint32_t)U * 4u;
            if constexpr (EPW == 2) {
                sts32(base + 0u * pitch, __byte_perm(A[q].x, B[q].x, 0x5410));
                sts32(base + 1u * pitch, __byte_perm(A[q].x, B[q].x, 0x7632));
                sts32(base + 2u * pitch, __byte_perm(A[q].y, B[q].y, 0x5410));
                sts32(base + 3u * pitch, __byte_perm(A[q].y, B[q].y, 0x7632));
                sts32(base + 4u * pitch, __byte_perm(A[q].z, B[q].z, 0x5410));
                sts32(base + 5u * pitch, __byte_perm(A[q].z, B[q].z, 0x7632));
                sts32(base + 6u * pitch, __byte_perm(A[q].w, B[q].w, 0x5410));
                sts32(base + 7u * pitch, __byte_perm(A[q].w, B[q].w, 0x7632));
            } else {
                sts32(base + 0u * pitch, A[q].x);
                sts32(base + 1u * pitch, A[q].y);
                sts32(base + 2u * pitch, A[q].z);
                sts32(base + 3u * pitch, A[q].w);
            }
        }
    }
    fence_async_smem();   // bulk stores read what the generic proxy just wrote
    __syncthreads();

    // ---- tile rows -> runs of the stack's plane rows (p.pixels elements apart, starting at pixel p0)
    const int planes = nG * CPG;
    T* dst = reinterpret_cast<T*>(a.stack) + ((long long)ib * a.C + (long long)cc * (128 / (int)sizeof(T))) * p.pixels + p0;
    const int sz = (int)sizeof(T);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // alignment that every run of this chunk shares (the stack base is 16-byte aligned and a block
    // starts on a 16-byte boundary, so only the row pitch, the chunk's first pixel and its length count)
    const int common = (p.pixels * sz) | (p0 * sz) | (P * sz);
    if ((common & 15) == 0) {
        if ((int)threadIdx.x < planes) {
            bulk_store_1d(dst + (long long)threadIdx.x * p.pixels, tile + threadIdx.x * (uint32_t)U * 4u, (uint32_t)(P * sz));
            bulk_wait_read<0>();
        }
    } else if ((common & 7) == 0) {
        const int U2 = U / 2;
        for (int c = warp; c < planes; c += kTileThreads / 32) {
            uint2* row = reinterpret_cast<uint2*>(dst + (long long)c * p.pixels);
            for (int u = lane; u < U2; u += 32) {
                uint2 v;
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(tile + (uint32_t)(c * U2 + u) * 8u));
                row[u] = v;
            }
        }
    } else if ((common & 3) == 0) {
        for (int c = warp; c < planes; c += kTileThreads / 32) {
            uint32_t* row = reinterpret_cast<uint32_t*>(dst + (long long)c * p.pixels);
            for (int u = lane; u < U; u += 32)
                row[u] = lds32(tile + (uint32_t)(c * U + u) * 4u);
        }
    } else if constexpr (EPW == 2) {
        // 16-bit runs of which some start on an odd half (odd row pitch and / or odd first pixel)
        unsigned short* dstH = reinterpret_cast<unsigned short*>(dst);
        for (int c = warp; c < planes; c += kTileThreads / 32) {
            unsigned short* row = dstH + (long long)c * p.pixels;
            const uint32_t trow = tile + (uint32_t)(c * U) * 4u;
            if ((((long long)c * p.pixels + p0) & 1) == 0) {
                uint32_t* rowW = reinterpret_cast<uint32_t*>(row);
                for (int u = lane; u < P / 2; u += 32)
                    rowW[u] = lds32(trow + (uint32_t)u * 4u);
                if ((P & 1) && lane == 0)
                    row[P - 1] = (unsigned short)lds16(trow + (uint32_t)(P - 1) * 2u);
            } else {
                uint32_t* rowW = reinterpret_cast<uint32_t*>(row + 1);
                const int nW = (P - 1) / 2;
                if (lane == 0)
                    row[0] = (unsigned short)lds16(trow);
                for (int k = lane; k < nW; k += 32)
                    rowW[k] = __funnelshift_r(lds32(trow + (uint32_t)k * 4u), lds32(trow + (uint32_t)k * 4u + 4u), 16);
                if (((P - 1) & 1) && lane == 0)
                    row[P - 1] = (unsigned short)lds16(trow + (uint32_t)(P - 1) * 2u);
            }
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled encode_fn()
{
    static PFN_cuTensorMapEncodeTiled fn = nullptr;
    static bool tried = false;
    if (!tried) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(ptr);
        else
            (void)cudaGetLastError();
        tried = true;
    }
    return fn;
}

// Tensor map of the NHWC image for boxes of 128 bytes of channels x boxW x boxH pixels (128-byte
// swizzle, zero fill outside the image).  Encoding costs a couple of microseconds on the host, and
// callers tend to come back with the same buffers, so each thread keeps its last few maps.
// false: no encoder in this driver, or a shape the encoder rejects (the caller falls back).
static bool image_map(const BlockArgs& a, int itemsize, int boxW, int boxH, CUtensorMap* out)
{
    struct Entry {
        const void* base;
        int N, H, W, C, itemsize, boxW, boxH, l2;
        CUtensorMap map;
    };
    constexpr int kEntries = 8;
    thread_local Entry cache[kEntries];
    thread_local int used = 0, next = 0;
    for (int i = 0; i < used; ++i) {
        const Entry& e = cache[i];
        if (e.base == a.image && e.N == a.N && e.H == a.H && e.W == a.W && e.C == a.C && e.itemsize == itemsize &&
            e.boxW == boxW && e.boxH == boxH && e.l2 == options().tmaL2) {
            *out = e.map;
            return true;
        }
    }
    PFN_cuTensorMapEncodeTiled enc = encode_fn();
    if (enc == nullptr)
        return false;
    const cuuint64_t dims[4] = {(cuuint64_t)a.C, (cuuint64_t)a.W, (cuuint64_t)a.H, (cuuint64_t)a.N};
    const cuuint64_t strides[3] = {(cuuint64_t)a.C * itemsize, (cuuint64_t)a.W * a.C * itemsize,
                                   (cuuint64_t)a.H * a.W * a.C * itemsize};
    const cuuint32_t box[4] = {(cuuint32_t)(128 / itemsize), (cuuint32_t)boxW, (cuuint32_t)boxH, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    // how much of a line the L2 fetches from DRAM around every 128-byte piece the box touches
    static const CUtensorMapL2promotion promotion[4] = {CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_64B,
                                                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B};
    if (enc(out, itemsize == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, a.image, dims,
            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promotion[options().tmaL2 & 3],
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    Entry& e = cache[next];
    e.base = a.image, e.N = a.N, e.H = a.H, e.W = a.W, e.C = a.C, e.itemsize = itemsize, e.boxW = boxW, e.boxH = boxH;
    e.l2 = options().tmaL2;
    e.map = *out;
    next = (next + 1) % kEntries;
    if (used < kEntries)
        ++used;
    return true;
}

bool planes_tma_eligible(const BlockArgs& a, int itemsize)
{
    if (options().disableTma)
        return false;
    const long long P = (long long)a.bSzH * a.bSzW;
    const size_t pixelBytes = (size_t)a.C * itemsize;
    if (pixelBytes % 128 != 0 || P > kMaxPixels || (itemsize == 2 && (P & 1)))
        return false;
    if (a.bSzH > 256 || a.bSzW > 256)
        return false;
    if ((reinterpret_cast<uintptr_t>(a.image) | reinterpret_cast<uintptr_t>(a.stack)) & 15)
        return false;
    return true;
}

// Raises a kernel's dynamic shared memory limit.  The limit is a property of the function (of the
// context), shared by every host thread, so what has been set is remembered process-wide -- frameworks
// call from several threads (an autograd engine runs backward passes on its own) -- and it is only ever
// raised: a smaller request after a larger one leaves the larger limit in place.
static cudaError_t set_smem(const void* fn, int bytes)
{
    struct Done {
        const void* fn;
        int device, bytes;
    };
    constexpr int kEntries = 64;
    static Done done[kEntries];
    static int used = 0;
    static std::mutex lock;
    int device = 0;
    note_site("cudaGetDevice (shared-memory limit)");
    if (cudaError_t e = cudaGetDevice(&device))
        return e;
    std::lock_guard<std::mutex> guard(lock);
    int slot = -1;
    for (int i = 0; i < used; ++i)
        if (done[i].fn == fn && done[i].device == device) {
            if (done[i].bytes >= bytes)
                return cudaSuccess;
            slot = i;
            break;
        }
    note_site("cudaFuncSetAttribute (shared-memory limit)");
    if (cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes))
        return e;
    if (slot < 0 && used < kEntries)
        slot = used++;
    if (slot >= 0)   // a full table only costs the repeated runtime call
        done[slot] = Done{fn, device, bytes};
    return cudaSuccess;
}

cudaError_t launch_planes_tma(const BlockArgs& a, int dtype, int mode, cudaStream_t stream, bool* taken)
{
    *taken = false;
    if (dtype == 2)
        return cudaSuccess;   // bf16 accumulation: tile CTAs or the general kernel
    const int itemsize = dtype == 0 ? 4 : 2;
    if (!planes_tma_eligible(a, itemsize))
        return cudaSuccess;

    TmaPlan p;
    const int P = a.bSzH * a.bSzW;
    p.cChunks = FastDiv((uint32_t)((size_t)a.C * itemsize / 128));
    p.blockW = FastDiv((uint32_t)a.bSzW);
    p.pixels = P;
    p.units = itemsize == 4 ? P : P / 2;
    p.tileBytes = 128 * P;
    const long long nItems = (long long)a.numActive * p.cChunks.div;
    const int grid = (int)(nItems < sm_count() ? nItems : sm_count());

    if (mode == kGather) {
        CUtensorMap map;
        if (!image_map(a, itemsize, a.bSzW, a.bSzH, &map))
            return cudaSuccess;   // no encoder, or a shape it rejects: the general kernel takes the call
        note_site("launch of planes_gather_tma");
        p.outStages = 2;
        p.inStageBytes = (p.tileBytes + 1023) & ~1023;
        p.outStageBytes = (p.tileBytes + 127) & ~127;
        p.inStages = 3 * p.inStageBytes + 2 * p.outStageBytes <= 225 * 1024 ? 3 : 2;
        const int smem = 1024 + p.inStages * p.inStageBytes + p.outStages * p.outStageBytes + 16 * p.inStages;
        if (dtype == 0) {
            if (cudaError_t e = set_smem((const void*)planes_gather_tma<float>, smem))
                return e;
            launch_pdl(planes_gather_tma<float>, dim3(grid), dim3(kTmaThreads), smem, stream, map, a, p);
        } else {
            if (cudaError_t e = set_smem((const void*)planes_gather_tma<__half>, smem))
                return e;
            launch_pdl(planes_gather_tma<__half>, dim3(grid), dim3(kTmaThreads), smem, stream, map, a, p);
        }
        *taken = true;
        return cudaGetLastError();
    }

    note_site("launch of planes_scatter_tma");
    p.inStages = 4, p.outStages = 0;
    p.inStageBytes = (p.tileBytes + 127) & ~127;
    p.outStageBytes = 0;
    const int smem = 1024 + p.inStages * p.inStageBytes + 16 * p.inStages;
#define SBNET_SCATTER_TMA(MODE_, T_)                                                              \
    do {                                                                                          \
        if (cudaError_t e = set_smem((const void*)planes_scatter_tma<MODE_, T_>, smem))       \
            return e;                                                                             \
        launch_pdl(planes_scatter_tma<MODE_, T_>, dim3(grid), dim3(kTmaThreads), smem, stream, a, p); \
    } while (0)
    if (dtype == 0) {
        if (mode == kScatterSet)
            SBNET_SCATTER_TMA(kScatterSet, float);
        else if (mode == kScatterAdd)
            SBNET_SCATTER_TMA(kScatterAdd, float);
        else
            SBNET_SCATTER_TMA(kScatterAtomic, float);
    } else {
        if (mode == kScatterSet)
            SBNET_SCATTER_TMA(kScatterSet, __half);
        else if (mode == kScatterAdd)
            SBNET_SCATTER_TMA(kScatterAdd, __half);
        else
            SBNET_SCATTER_TMA(kScatterAtomic, __half);
    }
#undef SBNET_SCATTER_TMA
    *taken = true;
    return cudaGetLastError();
}

// Gather with `blocksPerItem` (>= 1) blocks per tile; not taken (the plain-load kernel of
// planes_simt.cu runs instead) for blocks of more than 384 pixels or when the driver has no
// tensor-map encoder.  With the block count on the device the grid covers every candidate block and
// the surplus CTAs leave at once.
cudaError_t launch_gather_tma_tile(const BlockArgs& a, int dtype, int blocksPerItem, cudaStream_t stream, bool* taken)
{
    *taken = false;
    const int itemsize = dtype == 0 ? 4 : 2;
    const int P = a.bSzH * a.bSzW;
    if (a.bSzH > 256 || a.bSzW > 256 || ((size_t)a.C * itemsize) % 16 != 0)
        return cudaSuccess;
    const bool odd = itemsize == 2 && (P & 1);
    TmaTilePlan p;
    p.pixels = P;
    p.units = itemsize == 4 ? P : (P + 1) / 2;
    p.regionPixels = (P + 7) & ~7;
    // what fits: 384 pixels in padded regions, and 384/EPW words per tile row (odd rows round up)
    p.blocksPerItem = std::min(blocksPerItem, std::min(kMaxPixels / p.regionPixels, (kMaxPixels * itemsize / 4) / p.units));
    if (p.blocksPerItem < 1)
        return cudaSuccess;
    p.groups = (int)((size_t)a.C * itemsize / 16);
    p.cChunks = FastDiv((uint32_t)((p.groups + 7) / 8));
    p.unitsDiv = FastDiv((uint32_t)p.units);
    CUtensorMap map;
    if (!image_map(a, itemsize, a.bSzW, a.bSzH, &map))
        return cudaSuccess;
    const long long nItems = (long long)((a.numActive + p.blocksPerItem - 1) / p.blocksPerItem) * p.cChunks.div;
    if (nItems > 0x7fffffffll)
        return cudaSuccess;
    const int smem = kTileBytesMax + 1024;
    note_site("launch of planes_gather_tma_tile");
    if (dtype == 0) {
        if (cudaError_t e = set_smem((const void*)planes_gather_tma_tile<float>, smem))
            return e;
        launch_pdl(planes_gather_tma_tile<float>, dim3((unsigned)nItems), dim3(kTileThreads), smem, stream, map, a, p);
    } else if (odd) {
        if (cudaError_t e = set_smem((const void*)planes_gather_tma_tile<__half, true>, smem))
            return e;
        launch_pdl(planes_gather_tma_tile<__half, true>, dim3((unsigned)nItems), dim3(kTileThreads), smem, stream, map, a, p);
    } else {
        if (cudaError_t e = set_smem((const void*)planes_gather_tma_tile<__half>, smem))
            return e;
        launch_pdl(planes_gather_tma_tile<__half>, dim3((unsigned)nItems), dim3(kTileThreads), smem, stream, map, a, p);
    }
    *taken = true;
    return cudaGetLastError();
}

// Gather of blocks of more than 384 pixels by row chunks; not taken (the pixel chunks of
// planes_simt.cu run instead) for blocks wider than 256 pixels or when the driver has no tensor-map
// encoder.  With the block count on the device the grid covers every candidate block.
cudaError_t launch_gather_tma_rows(const BlockArgs& a, int dtype, cudaStream_t stream, bool* taken)
{
    *taken = false;
    const int itemsize = dtype == 0 ? 4 : 2;
    if (a.bSzW > 256 || ((size_t)a.C * itemsize) % 16 != 0)
        return cudaSuccess;
    TmaRowsPlan p;
    p.blockW = a.bSzW, p.blockH = a.bSzH, p.pixels = a.bSzH * a.bSzW;
    const int maxRows = std::min(kMaxPixels / a.bSzW, 256);
    if (maxRows < 1)
        return cudaSuccess;
    const int nChunks = (a.bSzH + maxRows - 1) / maxRows;
    p.chunkRows = (a.bSzH + nChunks - 1) / nChunks;                   // the fewest, nearly equal chunks
    p.rChunks = FastDiv((uint32_t)((a.bSzH + p.chunkRows - 1) / p.chunkRows));
    const int lastRows = a.bSzH - ((int)p.rChunks.div - 1) * p.chunkRows;
    p.groups = (int)((size_t)a.C * itemsize / 16);
    p.cChunks = FastDiv((uint32_t)((p.groups + 7) / 8));
    CUtensorMap maps[2];
    if (!image_map(a, itemsize, a.bSzW, p.chunkRows, &maps[0]) || !image_map(a, itemsize, a.bSzW, lastRows, &maps[1]))
        return cudaSuccess;
    const long long nItems = (long long)a.numActive * p.rChunks.div * p.cChunks.div;
    if (nItems > 0x7fffffffll)
        return cudaSuccess;
    const int smem = kTileBytesMax + 1024;
    note_site("launch of planes_gather_tma_rows");
    if (dtype == 0) {
        if (cudaError_t e = set_smem((const void*)planes_gather_tma_rows<float>, smem))
            return e;
        launch_pdl(planes_gather_tma_rows<float>, dim3((unsigned)nItems), dim3(kTileThreads), smem, stream, maps[0], maps[1], a, p);
    } else {
        if (cudaError_t e = set_smem((const void*)planes_gather_tma_rows<__half>, smem))
            return e;
        launch_pdl(planes_gather_tma_rows<__half>, dim3((unsigned)nItems), dim3(kTileThreads), smem, stream, maps[0], maps[1], a, p);
    }
    *taken = true;
    return cudaGetLastError();
}

cudaError_t read_wait_timeouts(unsigned int* out)
{
    return cudaMemcpyFromSymbol(out, g_wait_timeouts, sizeof(unsigned int));
}

} // namespace sbnet
