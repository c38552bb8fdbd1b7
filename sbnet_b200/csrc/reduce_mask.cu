// reduce_mask for sm_100a: block-local max / average pooling of a dense [N,H,W] fp32 mask,
// thresholding, and compaction of the active (n, bh, bw) triples -- in ONE launch.
//
// Replaces the reference's zeroBlockCounters + reduceMask pair and the host-side empty-mask fix-up
// (sbnet_ops/reduce_mask.cu:69-85, reduce_mask.cu.h:54-157, zero_block_counters.cu.h:26-51,
// reduce_mask.cc:203-220).  Results follow the reference CPU functor (reduce_mask.cc:66-96): same
// set of indices, same count; the order of the list is arrival order, as on the reference GPU path.
//
// Layout of the work: one CTA owns a horizontal BAND of the image -- the rows of one block row bh
// of one image n -- and a tile of consecutive block columns.  Threads own image columns (four at a
// time, one 128-bit load per row) and run down the band's rows keeping all loads of a batch in
// flight; the per-column partial results go to shared memory, then one thread per block combines
// the columns of its window.  Every mask byte is fetched from DRAM once (neighbouring bands share
// their halo rows through L2).
//
// Exactness.  Max pooling is "any pixel > tol", which does not depend on evaluation order.  Average
// pooling compares fl(sum/area) with tol, and the reference sums the window row-major in fp32; the
// column-then-row order used here can differ in the last bits.  Each block therefore also carries
// the sum of magnitudes, which bounds the difference between ANY two summation orders; only when
// the threshold falls inside that bound (practically never for 0/1 masks, rarely for real-valued
// ones) is the block re-evaluated by one thread in the reference's exact order.
#include "common.cuh"
#include "kernels.h"

namespace sbnet {

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
        *reinterpret_cast<volatile int32_t*>(a.host_count) = count;
        __threadfence_system();
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
                // |sum in any order - exact sum| <= ~terms * 2^-24 * m; two orders differ by at
                // most twice that.  A factor-two margin on top covers the rounding of m itself.
                const float terms = (float)(hEnd - hBeg) * (float)max(wEnd - wBeg, 0);
                const float rel = terms * 5.9604645e-8f;
                const float delta = 4.0f * rel * m;   // exactly 0 for an all-zero window
                const bool yes = __fdiv_rn(s - delta, a.area) > a.tol;
                const bool no = !(__fdiv_rn(s + delta, a.area) > a.tol);
                if (rel < 0.125f && m < 3.0e38f && yes)
                    active = true;
                else if (rel < 0.125f && m < 3.0e38f && no)
                    active = false;
                else
                    active = block_active_exact<true>(a, n, bh, bw);
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

cudaError_t launch_reduce_mask(const float* mask, int N, int H, int W, float tol, bool avgpool,
                               int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH, int bStrW,
                               int bCntH, int bCntW, int16_t* idx, int32_t* scratch,
                               int32_t* host_count_dev, cudaStream_t stream)
{
    RmArgs a;
    a.mask = mask, a.idx = idx, a.scratch = scratch, a.host_count = host_count_dev;
    a.N = N, a.H = H, a.W = W, a.tol = tol;
    a.bOffsH = bOffsH, a.bOffsW = bOffsW, a.bSzH = bSzH, a.bSzW = bSzW;
    a.bStrH = bStrH, a.bStrW = bStrW, a.bCntH = bCntH, a.bCntW = bCntW;
    a.area = (float)(bSzH * bSzW);

    // widest run of block columns whose pixel span (plus 4-column rounding) fits the staging area
    const long long spare = (long long)kRmMaxCols - 8 - bSzW;
    if (spare >= 0) {
        long long tb = spare / bStrW + 1;
        a.tileBlocks = (int)(tb < bCntW ? tb : bCntW);
        const dim3 grid((bCntW + a.tileBlocks - 1) / a.tileBlocks, bCntH, N);
        const bool vec4 = (W % 4 == 0) && ((reinterpret_cast<uintptr_t>(mask) & 15) == 0);
        if (avgpool) {
            if (vec4)
                reduce_mask_band<true, true><<<grid, kRmThreads, 0, stream>>>(a);
            else
                reduce_mask_band<true, false><<<grid, kRmThreads, 0, stream>>>(a);
        } else {
            if (vec4)
                reduce_mask_band<false, true><<<grid, kRmThreads, 0, stream>>>(a);
            else
                reduce_mask_band<false, false><<<grid, kRmThreads, 0, stream>>>(a);
        }
    } else {
        a.tileBlocks = 1;
        const long long total = (long long)N * bCntH * bCntW;
        const int grid = (int)((total + kRmThreads - 1) / kRmThreads < 1184
                                   ? (total + kRmThreads - 1) / kRmThreads
                                   : 1184);
        if (avgpool)
            reduce_mask_naive<true><<<grid, kRmThreads, 0, stream>>>(a);
        else
            reduce_mask_naive<false><<<grid, kRmThreads, 0, stream>>>(a);
    }
    return cudaGetLastError();
}

} // namespace sbnet
