// reduce_mask for sm_100a: block-local max / average pooling of a dense [N,H,W] fp32 mask,
// thresholding, and compaction of the active (n, bh, bw) triples -- in ONE launch.
//
// Replaces the reference's zeroBlockCounters + reduceMask pair and the host-side empty-mask fix-up
// (sbnet_ops/reduce_mask.cu:69-85, reduce_mask.cu.h:54-157, zero_block_counters.cu.h:26-51,
// reduce_mask.cc:203-220).  Results follow the reference CPU functor (reduce_mask.cc:66-96): same
// set of indices, same count; the order of the list is arrival order, as on the reference GPU path.
//
// Layout of the work: one CTA owns a TILE of the image -- the rows of one block row bh of one image
// n, cut into runs of at most 32 consecutive block columns.  Every mask byte is fetched from DRAM
// once (neighbouring tiles share their halo rows and columns through L2).
//  * reduce_mask_tile (rows of a multiple of four pixels, 16-byte aligned mask, tile fits shared
//    memory -- every benchmark shape): the tile's in-range rows are brought into shared memory by
//    the TMA engine, one untiled bulk copy per row issued by the lanes of one warp onto one
//    mbarrier, so the load phase costs no registers and no load instructions.  Eight lanes then sum
//    (or test) the window of one block straight out of shared memory, combine by shuffles, and the
//    first warp ballots the verdicts, reserves the tile's run of the index list with ONE 64-bit atomic
//    and writes the triples.  Like every kernel of the library it is launched with programmatic stream
//    serialization; when the caller vouches for the mask, not only its prologue but its loads too
//    overlap the tail of the kernel queued before it.
//  * reduce_mask_band (any other shape): threads own image columns (four at a time, one 128-bit load
//    per row) and run down the band's rows keeping all loads of a batch in flight; per-column partial
//    results go to shared memory, then one thread per block combines the columns of its window.
//
// Exactness.  Max pooling is "any pixel > tol", which does not depend on evaluation order.  Average
// pooling compares fl(sum/area) with tol, and the reference sums the window row-major in fp32; the
// column-then-row order used here can differ in the last bits.  Each block therefore also carries
// the sum of magnitudes, which bounds the difference between ANY two summation orders; only when
// the threshold falls inside that bound (practically never for 0/1 masks, rarely for real-valued
// ones) is the block re-evaluated by one thread in the reference's exact order.
#include "async_ptx.cuh"
#include "common.cuh"
#include "kernels.h"
#include "options.h"

namespace sbnet {

__device__ unsigned int g_rm_wait_timeouts = 0;   // bounded waits of reduce_mask_tile that gave up

constexpr int kRmThreads = 192;      // 176 threads cover a 704-pixel row with 128-bit loads; 3 CTAs per SM
                                    // keep the 400 bands of an [8,800,704] mask in a single wave
constexpr int kRmMaxCols = 4096;   // image columns one CTA stages (x2 floats of shared memory)
constexpr int kRowBatch = 18;      // loads kept in flight per thread while running down a band

struct RmArgs {
    const float* mask;
    int16_t* idx;
    int32_t* scratch;      // [0] published count, [2..3] 64-bit cursor|ticket word (16-byte aligned)
    int32_t* host_count;   // optional device-visible address of a pinned host int
    int N, H, W;
    float tol;
    int bOffsH, bOffsW, bSzH, bSzW, bStrH, bStrW, bCntH, bCntW;
    int tileBlocks;        // block columns per CTA
    int earlyLoads;        // tile kernel: the mask may be read before the preceding kernel has finished
    int tileFloats;        // tile kernel: floats of shared memory reserved for the tile itself
    int tileCols;          // tile kernel: columns reserved per partial-result array behind the tile
    float area;            // (float)(bSzH*bSzW)
};

// The reference's evaluation order for one block, used for the rare ambiguous average and by the
// fallback kernel for geometries the band kernel does not take.
template <bool AVG>
__device__ bool block_active_exact(const RmArgs& a, int n, int bh, int bw)
{
    const int h0 = a.bOffsH + bh * a.bStrH, w0 = a.bOffsW + bw * a.bStrW;
    const int hBeg = max(h0, 0), wBeg = max(w0, 0);
    const int hEnd = min(h0 + a.bSzH, a.H), wEnd = min(w0 + a.bSzW, a.W);
    const float* img = a.mask + (size_t)n * a.H * a.W;
    float sum = 0.0f;
    bool any = false;
    for (int hh = hBeg; hh < hEnd; ++hh) {
        const float* row = img + (size_t)hh * a.W;
        // nine loads are issued before the nine dependent adds, so the serial chain waits for memory
        // once per batch instead of once per pixel (the order of the adds is unchanged)
        for (int w0b = wBeg; w0b < wEnd; w0b += 9) {
            float v[9];
#pragma unroll
            for (int k = 0; k < 9; ++k)
                v[k] = (w0b + k < wEnd) ? __ldg(row + w0b + k) : 0.0f;
#pragma unroll
            for (int k = 0; k < 9; ++k) {
                if (w0b + k < wEnd) {
                    if (AVG)
                        sum = __fadd_rn(sum, v[k]);
                    else
                        any |= (v[k] > a.tol);
                }
            }
        }
    }
    return AVG ? (__fdiv_rn(sum, a.area) > a.tol) : any;
}

// scratch words [2..3] form one 64-bit word: low half = append cursor, high half = CTAs finished.
__device__ __forceinline__ unsigned long long* cursor64(const RmArgs& a)
{
    return reinterpret_cast<unsigned long long*>(a.scratch + 2);
}

// The CTA that finishes last publishes the count (an empty result becomes the single block
// (0,0,0), as the reference op does on the host) and leaves the cursor word at zero for the next
// call.  `count` is the final number of appended blocks.
__device__ __forceinline__ void publish(const RmArgs& a, int count)
{
    if (count == 0) {
        a.idx[0] = a.idx[1] = a.idx[2] = 0;
        count = 1;
    }
    a.scratch[0] = count;
    *cursor64(a) = 0ull;
    if (a.host_count) {
        // a host that sees the count may hand scratch[0] (or the indices) to other work at once:
        // everything published so far must be visible system-wide before the host-visible store
        __threadfence_system();
        *reinterpret_cast<volatile int32_t*>(a.host_count) = count;
        __threadfence_system();
    }
}

// Verdict of an average-pooled block from its window sum s and sum of magnitudes m, both taken in
// an arbitrary order over `terms` in-range pixels: decided from the error bound where that is
// conclusive, else re-evaluated in the reference's order.
__device__ __forceinline__ bool avg_verdict(const RmArgs& a, float s, float m, float terms, int n, int bh, int bw)
{
    // |sum in any order - exact sum| <= ~terms * 2^-24 * m; two orders differ by at most twice
    // that.  A factor-two margin on top covers the rounding of m itself.
    const float rel = terms * 5.9604645e-8f;
    const float delta = 4.0f * rel * m;   // exactly 0 for an all-zero window
    const bool yes = __fdiv_rn(s - delta, a.area) > a.tol;
    const bool no = !(__fdiv_rn(s + delta, a.area) > a.tol);
    if (rel < 0.125f && m < 3.0e38f && yes)
        return true;
    if (rel < 0.125f && m < 3.0e38f && no)
        return false;
    return block_active_exact<true>(a, n, bh, bw);
}

// ---- tile kernel ------------------------------------------------------------------------------------
constexpr int kRmLanesPerBlock = 8;     // lanes that share one block's window
constexpr int kRmTileMaxBlocks = 32;    // block columns per tile: one warp ballots and appends them
constexpr int kRmTileMaxThreads = kRmLanesPerBlock * kRmTileMaxBlocks;
constexpr int kRmTileSmemMax = 96 * 1024;

template <bool AVG>
__global__ void __launch_bounds__(kRmTileMaxThreads) reduce_mask_tile(const RmArgs a)
{
    extern __shared__ __align__(128) unsigned char rmSmem[];   // [nRows][pitch] fp32
    __shared__ __align__(8) unsigned long long barStorage;
    __shared__ int abortFlag;
    __shared__ unsigned char verdict[kRmTileMaxBlocks];

    const int n = blockIdx.z, bh = blockIdx.y;
    const int bw0 = blockIdx.x * a.tileBlocks;
    const int nBlk = min(a.tileBlocks, a.bCntW - bw0);
    const int h0 = a.bOffsH + bh * a.bStrH;
    const int hBeg = max(h0, 0), hEnd = min(h0 + a.bSzH, a.H);
    const int nRows = max(hEnd - hBeg, 0);
    // columns this tile touches, widened to whole 16-byte groups (W is a multiple of four)
    const int cBeg = max(a.bOffsW + bw0 * a.bStrW, 0) & ~3;
    const int cEnd = min((min(a.bOffsW + (bw0 + nBlk - 1) * a.bStrW + a.bSzW, a.W) + 3) & ~3, a.W);
    const int nCols = max(cEnd - cBeg, 0);
    const bool haveTile = nRows > 0 && nCols > 0;
    const uint32_t tile = smem_u32(rmSmem);
    const uint32_t bar = smem_u32(&barStorage);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        abortFlag = 0;
        mbar_init(bar, 1);
        mbar_init_fence();
        fence_async_smem();
    }
    __syncthreads();
    if (!a.earlyLoads)
        pdl_wait();   // the mask may be the output of the kernel queued before this one
    if (warp == 0 && haveTile) {
        if (lane == 0)
            mbar_expect_tx(bar, (uint32_t)nRows * (uint32_t)nCols * 4u);
        __syncwarp();
        const float* src = a.mask + ((size_t)n * a.H + hBeg) * a.W + cBeg;
        for (int r = lane; r < nRows; r += 32)
            bulk_load_1d(tile + (uint32_t)(r * nCols) * 4u, src + (size_t)r * a.W, (uint32_t)nCols * 4u, bar);
    }
    if (haveTile) {
        // every warp waits for the tile (bounded); a warp that gives up waits once more, again
        // bounded, so that copies are not left in flight over shared memory the CTA has given back
        int ok = 1;
        if (lane == 0) {
            ok = mbar_wait_bounded(bar, 0, &abortFlag, &g_rm_wait_timeouts) ? 1 : 0;
            if (!ok) {
                int again = 0;
                (void)mbar_wait_bounded(bar, 0, &again, &g_rm_wait_timeouts);
            }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (__syncthreads_or(ok == 0)) {
            // The tile never arrived: the CTA still takes its finish ticket (appending nothing), so the
            // call completes and the wait counter tells the host that the result is incomplete.
            if (threadIdx.x == 0) {
                pdl_wait();
                const unsigned long long old = atomicAdd(cursor64(a), 1ull << 32);
                if ((unsigned)(old >> 32) == gridDim.x * gridDim.y * gridDim.z - 1)
                    publish(a, (int)(unsigned)old);
            }
            return;
        }
    }

    pdl_launch_dependents();   // the tile is here: the next kernel's CTAs may take the slots that free up
    // ---- columns: a thread owns four neighbouring columns and runs down the tile's rows with 128-bit
    // shared-memory loads (a warp reads 512 contiguous bytes per instruction: no bank conflicts), leaving
    // one partial result per column behind the tile
    float* colVal = reinterpret_cast<float*>(rmSmem) + (size_t)a.tileFloats;   // [nCols] sum / any-flag
    float* colMag = colVal + a.tileCols;                                        // [nCols] sum of magnitudes (AVG)
    for (int c4 = threadIdx.x; c4 < (nCols >> 2); c4 += blockDim.x) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, mag[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint32_t at = tile + (uint32_t)c4 * 16u;
#pragma unroll 6
        for (int r = 0; r < nRows; ++r) {
            const uint4 q = lds128(at + (uint32_t)(r * nCols) * 4u);
            const float v[4] = {__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z), __uint_as_float(q.w)};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (AVG) {
                    acc[j] = __fadd_rn(acc[j], v[j]);
                    mag[j] = __fadd_rn(mag[j], fabsf(v[j]));
                } else {
                    acc[j] = (v[j] > a.tol) ? 1.0f : acc[j];
                }
            }
        }
        *reinterpret_cast<float4*>(colVal + 4 * c4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        if (AVG)
            *reinterpret_cast<float4*>(colMag + 4 * c4) = make_float4(mag[0], mag[1], mag[2], mag[3]);
    }
    __syncthreads();

    // ---- window of block b: eight lanes stride over its columns' partial results and combine by shuffles
    // (whole warps take every trip: lanes past the last block hold zeros and shuffle along)
    for (int t0 = warp * 32; t0 < nBlk * kRmLanesPerBlock; t0 += blockDim.x) {
        const int t = t0 + lane;
        const int b = t / kRmLanesPerBlock, g = t % kRmLanesPerBlock;
        const bool mine = b < nBlk;
        const int w0 = a.bOffsW + (bw0 + b) * a.bStrW;
        const int wBeg = max(w0, 0), wEnd = (mine && haveTile) ? min(w0 + a.bSzW, a.W) : 0;
        float s = 0.0f, m = 0.0f;
        for (int c = wBeg + g - cBeg; c < wEnd - cBeg; c += kRmLanesPerBlock) {
            if (AVG) {
                s = __fadd_rn(s, colVal[c]);
                m = __fadd_rn(m, colMag[c]);
            } else {
                s = fmaxf(s, colVal[c]);
            }
        }
#pragma unroll
        for (int d = kRmLanesPerBlock / 2; d > 0; d >>= 1) {   // a block's lanes are neighbours in one warp
            if (AVG) {
                s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, d));
                m = __fadd_rn(m, __shfl_xor_sync(0xffffffffu, m, d));
            } else {
                s = fmaxf(s, __shfl_xor_sync(0xffffffffu, s, d));
            }
        }
        if (g == 0 && mine) {
            bool active;
            if (AVG) {
                const float terms = (float)nRows * (float)max(min(w0 + a.bSzW, a.W) - wBeg, 0);
                active = avg_verdict(a, s, m, terms, n, bh, bw0 + b);
            } else {
                active = s > 0.0f;
            }
            verdict[b] = active ? 1 : 0;
        }
    }
    __syncthreads();

    // ---- first warp: ballot, ONE atomic reserves the tile's run and takes the finish ticket, append
    if (warp == 0) {
        const bool act = lane < nBlk && verdict[lane] != 0;
        const unsigned ballot = __ballot_sync(0xffffffffu, act);
        const unsigned total = __popc(ballot);
        unsigned long long old = 0ull;
        pdl_wait();   // scratch and the index list may still be in use by the kernel queued before this one
        if (lane == 0)
            old = atomicAdd(cursor64(a), (1ull << 32) | total);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (act) {
            int16_t* out = a.idx + (size_t)((unsigned)old + __popc(ballot & ((1u << lane) - 1u))) * 3;
            out[0] = (int16_t)n;
            out[1] = (int16_t)bh;
            out[2] = (int16_t)(bw0 + lane);
        }
        if (lane == 0 && (unsigned)(old >> 32) == gridDim.x * gridDim.y * gridDim.z - 1)
            publish(a, (int)((unsigned)old + total));
    }
}


template <bool AVG, bool VEC4>
__global__ void __launch_bounds__(kRmThreads, 3) reduce_mask_band(const RmArgs a)
{
    // per staged column: sum (or any-flag) and, for AVG, the sum of magnitudes
    __shared__ float colVal[kRmMaxCols];
    __shared__ float colMag[AVG ? kRmMaxCols : 1];
    __shared__ unsigned ballots[kRmMaxCols / 32 + 1];   // verdicts of the tile, 32 blocks per word
    __shared__ unsigned wordBase[kRmMaxCols / 32 + 1];  // exclusive prefix of popc(ballots)
    __shared__ unsigned ctaBase;

    pdl_wait();   // nothing global is read or written before the kernel queued ahead of this one is done
    const int n = blockIdx.z, bh = blockIdx.y;
    const int bw0 = blockIdx.x * a.tileBlocks;
    const int bwEnd = min(bw0 + a.tileBlocks, a.bCntW);
    const int h0 = a.bOffsH + bh * a.bStrH;
    const int hBeg = max(h0, 0), hEnd = min(h0 + a.bSzH, a.H);

    // columns this tile touches, widened to whole 4-column groups when loads are vectorised
    int cBeg = max(a.bOffsW + bw0 * a.bStrW, 0);
    int cEnd = min(a.bOffsW + (bwEnd - 1) * a.bStrW + a.bSzW, a.W);
    if (VEC4) {
        cBeg &= ~3;
        cEnd = min((cEnd + 3) & ~3, a.W);
    }
    const int nCols = max(cEnd - cBeg, 0);
    const float* img = a.mask + (size_t)n * a.H * a.W;

    constexpr int V = VEC4 ? 4 : 1;
    for (int cv = threadIdx.x * V; cv < nCols; cv += kRmThreads * V) {
        float acc[V], mag[V];
#pragma unroll
        for (int j = 0; j < V; ++j)
            acc[j] = 0.0f, mag[j] = 0.0f;
        const float* colp = img + cBeg + cv;
        for (int hb = hBeg; hb < hEnd; hb += kRowBatch) {
            float v[kRowBatch][V];
#pragma unroll
            for (int k = 0; k < kRowBatch; ++k) {   // all loads of the batch are issued before any use
#pragma unroll
                for (int j = 0; j < V; ++j)
                    v[k][j] = 0.0f;
                if (hb + k < hEnd) {
                    if constexpr (VEC4) {
                        const float4 q = __ldg(reinterpret_cast<const float4*>(colp + (size_t)(hb + k) * a.W));
                        v[k][0] = q.x, v[k][1] = q.y, v[k][2] = q.z, v[k][3] = q.w;
                    } else {
                        v[k][0] = __ldg(colp + (size_t)(hb + k) * a.W);
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < kRowBatch; ++k) {
                if (hb + k < hEnd) {
#pragma unroll
                    for (int j = 0; j < V; ++j) {
                        if (AVG) {
                            acc[j] = __fadd_rn(acc[j], v[k][j]);
                            mag[j] = __fadd_rn(mag[j], fabsf(v[k][j]));
                        } else {
                            acc[j] = (v[k][j] > a.tol) ? 1.0f : acc[j];
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
            colVal[cv + j] = acc[j];
            if (AVG)
                colMag[cv + j] = mag[j];
        }
    }
    __syncthreads();

    // verdicts: one thread per block column of the tile, 32 verdicts per ballot word
    const int nBlk = bwEnd - bw0;
    const int nWords = (nBlk + 31) >> 5;
    for (int b = threadIdx.x; b < nWords * 32; b += kRmThreads) {
        bool active = false;
        const int bw = bw0 + b;
        if (b < nBlk && hBeg < hEnd) {
            const int w0 = a.bOffsW + bw * a.bStrW;
            const int wBeg = max(w0, 0), wEnd = min(w0 + a.bSzW, a.W);
            float s = 0.0f, m = 0.0f;
            for (int ww = wBeg; ww < wEnd; ++ww) {
                if (AVG) {
                    s = __fadd_rn(s, colVal[ww - cBeg]);
                    m = __fadd_rn(m, colMag[ww - cBeg]);
                } else {
                    s = fmaxf(s, colVal[ww - cBeg]);
                }
            }
            if (!AVG) {
                active = s > 0.0f;
            } else {
                const float terms = (float)(hEnd - hBeg) * (float)max(wEnd - wBeg, 0);
                active = avg_verdict(a, s, m, terms, n, bh, bw);
            }
        } else if (b < nBlk) {
            // a band with no in-range row: empty window => max: inactive; avg: 0/area > tol
            active = AVG ? (__fdiv_rn(0.0f, a.area) > a.tol) : false;
        }
        const unsigned ballot = __ballot_sync(0xffffffffu, active);
        if ((threadIdx.x & 31) == 0)
            ballots[b >> 5] = ballot;
    }
    __syncthreads();

    // ONE atomic per CTA reserves its run of the index list and takes a finish ticket with it
    if (threadIdx.x == 0) {
        unsigned total = 0;
        for (int w = 0; w < nWords; ++w) {
            wordBase[w] = total;
            total += __popc(ballots[w]);
        }
        const unsigned long long old = atomicAdd(cursor64(a), (1ull << 32) | total);
        ctaBase = (unsigned)old;
        if ((unsigned)(old >> 32) == gridDim.x * gridDim.y * gridDim.z - 1)
            publish(a, (int)((unsigned)old + total));
    }
    __syncthreads();
    for (int b = threadIdx.x; b < nBlk; b += kRmThreads) {
        const unsigned ballot = ballots[b >> 5], bit = 1u << (b & 31);
        if (ballot & bit) {
            int16_t* out = a.idx + (size_t)(ctaBase + wordBase[b >> 5] + __popc(ballot & (bit - 1u))) * 3;
            out[0] = (int16_t)n;
            out[1] = (int16_t)bh;
            out[2] = (int16_t)(bw0 + b);
        }
    }
}

// Fallback for windows wider than a CTA can stage: one thread per block, reference order; one
// reservation per warp (ballot, popc), one finish ticket per CTA.
template <bool AVG>
__global__ void __launch_bounds__(kRmThreads) reduce_mask_naive(const RmArgs a)
{
    pdl_wait();   // nothing global is read or written before the kernel queued ahead of this one is done
    const long long total = (long long)a.N * a.bCntH * a.bCntW;
    const long long stride = (long long)gridDim.x * kRmThreads;
    const long long rounds = (total + stride - 1) / stride;
    const int lane = threadIdx.x & 31;
    for (long long r = 0; r < rounds; ++r) {
        const long long i = r * stride + (long long)blockIdx.x * kRmThreads + threadIdx.x;
        bool active = false;
        int n = 0, bh = 0, bw = 0;
        if (i < total) {
            bw = (int)(i % a.bCntW);
            bh = (int)((i / a.bCntW) % a.bCntH);
            n = (int)(i / ((long long)a.bCntW * a.bCntH));
            active = block_active_exact<AVG>(a, n, bh, bw);
        }
        const unsigned ballot = __ballot_sync(0xffffffffu, active);
        if (ballot == 0)
            continue;
        const int leader = __ffs(ballot) - 1;
        unsigned base = 0;
        if (lane == leader)
            base = (unsigned)atomicAdd(cursor64(a), (unsigned long long)__popc(ballot));
        base = __shfl_sync(0xffffffffu, base, leader);
        if (active) {
            int16_t* out = a.idx + (size_t)(base + __popc(ballot & ((1u << lane) - 1u))) * 3;
            out[0] = (int16_t)n;
            out[1] = (int16_t)bh;
            out[2] = (int16_t)bw;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned long long old = atomicAdd(cursor64(a), 1ull << 32);
        if ((unsigned)(old >> 32) == gridDim.x - 1)
            publish(a, (int)(unsigned)old);
    }
}

// Raises the tile kernel's dynamic shared memory limit once per device.
template <bool AVG> static cudaError_t tile_smem_limit()
{
    static bool done[64] = {false};
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev))
        return e;
    if (dev >= 0 && dev < 64 && done[dev])
        return cudaSuccess;
    if (cudaError_t e = cudaFuncSetAttribute(reduce_mask_tile<AVG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kRmTileSmemMax))
        return e;
    if (dev >= 0 && dev < 64)
        done[dev] = true;
    return cudaSuccess;
}

// Column tiles per block row for the tile kernel: about `kRmCtasPerSm` CTAs per SM in total, at most
// 32 block columns per tile, and a tile that fits shared memory.  0: the shape is not eligible.
static int tile_blocks_for(int N, int H, int W, int bSzH, int bSzW, int bStrW, int bCntH, int bCntW)
{
    const long long rows = bSzH < H ? bSzH : H;
    // widest run of block columns whose pixel span (plus the rounding to 16-byte groups) fits
    const long long maxCols = kRmTileSmemMax / 4 / (rows + 2);
    long long fit = (maxCols - 9 - bSzW) >= 0 ? (maxCols - 9 - bSzW) / bStrW + 1 : 0;
    if (fit > kRmTileMaxBlocks)
        fit = kRmTileMaxBlocks;
    if (fit < 1)
        return 0;
    const long long want = (long long)sm_count() * (options().rmCtasPerSm > 0 ? options().rmCtasPerSm : 8);
    const long long bands = (long long)bCntH * N;
    long long tiles = (want + bands / 2) / bands;       // column tiles per band, rounded to nearest
    if (tiles < 1)
        tiles = 1;
    if (tiles > bCntW)
        tiles = bCntW;
    long long tb = (bCntW + tiles - 1) / tiles;
    if (tb > fit)
        tb = fit;
    tiles = (bCntW + tb - 1) / tb;
    return (int)((bCntW + tiles - 1) / tiles);          // equal tiles
}

cudaError_t launch_reduce_mask(const float* mask, int N, int H, int W, float tol, bool avgpool,
                               int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH, int bStrW,
                               int bCntH, int bCntW, int16_t* idx, int32_t* scratch,
                               int32_t* host_count_dev, bool maskStable, cudaStream_t stream)
{
    RmArgs a;
    a.mask = mask, a.idx = idx, a.scratch = scratch, a.host_count = host_count_dev;
    a.N = N, a.H = H, a.W = W, a.tol = tol;
    a.bOffsH = bOffsH, a.bOffsW = bOffsW, a.bSzH = bSzH, a.bSzW = bSzW;
    a.bStrH = bStrH, a.bStrW = bStrW, a.bCntH = bCntH, a.bCntW = bCntW;
    a.area = (float)(bSzH * bSzW);
    a.earlyLoads = maskStable ? 1 : 0;

    const bool vec4 = (W % 4 == 0) && ((reinterpret_cast<uintptr_t>(mask) & 15) == 0);
    const int tb = vec4 && options().rmKernel == 0
                       ? tile_blocks_for(N, H, W, bSzH, bSzW, bStrW, bCntH, bCntW) : 0;
    if (tb >= 1) {
        a.tileBlocks = tb;
        const int rows = bSzH < H ? bSzH : H;
        long long cols = ((long long)(tb - 1) * bStrW + bSzW + 9) & ~3ll;
        if (cols > W)
            cols = W;
        a.tileFloats = (int)(rows * cols), a.tileCols = (int)cols;
        size_t smem = ((size_t)rows + 2) * (size_t)cols * 4;   // the tile + two rows of per-column partial results
        // fewer, larger shared-memory claims per SM keep that many CTAs from being resident at once: the
        // CTAs of a later wave then load while those of an earlier one reduce
        if (options().rmResident > 0) {
            const size_t want = (size_t)(220 * 1024) / (size_t)options().rmResident - 1024;
            if (want > smem && want <= (size_t)kRmTileSmemMax)
                smem = want;
        }
        const dim3 grid((bCntW + tb - 1) / tb, bCntH, N);
        const dim3 block((unsigned)((tb * kRmLanesPerBlock + 31) & ~31));
        if (avgpool) {
            if (cudaError_t e = tile_smem_limit<true>())
                return e;
            return launch_pdl(reduce_mask_tile<true>, grid, block, smem, stream, a);
        }
        if (cudaError_t e = tile_smem_limit<false>())
            return e;
        return launch_pdl(reduce_mask_tile<false>, grid, block, smem, stream, a);
    }

    // widest run of block columns whose pixel span (plus 4-column rounding) fits the staging area
    const long long spare = (long long)kRmMaxCols - 8 - bSzW;
    if (spare >= 0 && options().rmKernel != 2) {
        long long tb = spare / bStrW + 1;
        a.tileBlocks = (int)(tb < bCntW ? tb : bCntW);
        const dim3 grid((bCntW + a.tileBlocks - 1) / a.tileBlocks, bCntH, N);
        if (avgpool) {
            if (vec4)
                launch_pdl(reduce_mask_band<true, true>, grid, dim3(kRmThreads), 0, stream, a);
            else
                launch_pdl(reduce_mask_band<true, false>, grid, dim3(kRmThreads), 0, stream, a);
        } else {
            if (vec4)
                launch_pdl(reduce_mask_band<false, true>, grid, dim3(kRmThreads), 0, stream, a);
            else
                launch_pdl(reduce_mask_band<false, false>, grid, dim3(kRmThreads), 0, stream, a);
        }
    } else {
        a.tileBlocks = 1;
        const long long total = (long long)N * bCntH * bCntW;
        const int grid = (int)((total + kRmThreads - 1) / kRmThreads < 1184
                                   ? (total + kRmThreads - 1) / kRmThreads
                                   : 1184);
        if (avgpool)
            launch_pdl(reduce_mask_naive<true>, dim3(grid), dim3(kRmThreads), 0, stream, a);
        else
            launch_pdl(reduce_mask_naive<false>, dim3(grid), dim3(kRmThreads), 0, stream, a);
    }
    return cudaGetLastError();
}

cudaError_t read_rm_wait_timeouts(unsigned int* out)
{
    return cudaMemcpyFromSymbol(out, g_rm_wait_timeouts, sizeof(unsigned int));
}

} // namespace sbnet
