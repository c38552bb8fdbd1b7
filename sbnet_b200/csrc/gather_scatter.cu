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
//    shared memory.
//  * [nB, C, R, S] ("planes", transpose=true): pixels of a multiple of 16 bytes go to the kernels of
//    planes_simt.cu / planes_tma.cu.  The kernel here takes every other shape: a CTA stages a tile
//    of pixels x channels (128 bytes of channels per pixel) in shared memory with an odd word pitch,
//    so that the image side moves channel runs and the stack side moves runs of consecutive pixels
//    of one channel plane, both conflict-free.
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
// the tile: a block row of S pixels x C channels is ONE contiguous run of the image, so it is moved as
// raw bytes with aligned 16-byte accesses -- whatever C*sizeof(T) is -- into a row buffer that keeps the
// run's misalignment (the copy "shifts" nothing: byte b of the run lands at offset (address & 15) + b),
// ragged ends element by element, so nothing outside the clipped run is ever touched.  The transposition
// then happens between the row buffers and the stack: a warp owns a channel plane at a time and its
// lanes walk the pixels with running (row, column) counters -- no divisions -- so stack accesses are
// consecutive elements of one plane.
constexpr int kRawMaxRows = 256;      // block rows per work item (their phases are kept in shared memory)
constexpr int kRawUnroll = 4;         // 16-byte slots (image side) / elements (stack side) in flight per thread

struct RawPlan {
    FastDiv rChunks;       // row chunks per block
    FastDiv slotsPerRow;   // 16-byte slots a row buffer holds
    int rowsPerItem;       // block rows per work item
    int rowBytes;          // S * C * sizeof(T)
    int rowPitch;          // bytes of one row buffer: rowBytes + its possible misalignment, a multiple of 16
    int stepS, stepR;      // 32 % S, 32 / S: how (row, column) advance when a lane moves on by 32 pixels
};

template <int MODE, typename T>
__global__ void __launch_bounds__(kThreads, 4) planes_rows_kernel(const BlockArgs a, const RawPlan p)
{
    pdl_wait();   // nothing is read or written before the kernel queued ahead of this one is done
    __shared__ __align__(16) unsigned char tile[kTileBytes];
    __shared__ unsigned char rowPhase[kRawMaxRows];   // (address of the row's first byte) & 15
    constexpr int SZ = (int)sizeof(T);
    typedef typename Vec<SZ>::type E;                 // one element as plain bits
    const int nActive = active_count(a);
    const long long nItems = (long long)nActive * p.rChunks.div;
    const int S = a.bSzW, P = a.bSzH * a.bSzW;
    const long long pixBytes = (long long)a.C * SZ;
    const uintptr_t imgBase = reinterpret_cast<uintptr_t>(a.image);
    const uint32_t tileAddr = smem_u32(tile);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    for (long long item = blockIdx.x; item < nItems; item += gridDim.x) {
        uint32_t ib, rc;
        p.rChunks.divmod((uint32_t)item, ib, rc);
        const int r0 = (int)rc * p.rowsPerItem;
        const int rows = min(p.rowsPerItem, a.bSzH - r0);
        const int n = a.idx[ib * 3 + 0];
        const int h0 = a.bOffsH + a.idx[ib * 3 + 1] * a.bStrH + r0;
        const int w0 = a.bOffsW + a.idx[ib * 3 + 2] * a.bStrW;
        const int sLo = max(0, -w0), sHi = max(sLo, min(S, a.W - w0));   // in-range pixels of every row: [sLo, sHi)
        const long long bLo = sLo * pixBytes, bHi = sHi * pixBytes;      // ... as bytes of the row's run
        // address the run of row rl WOULD start at (its pixel 0 may lie left of the image: never dereferenced there)
        auto row_start = [&](int rl) -> long long {
            return (long long)imgBase + (((long long)n * a.H + (h0 + rl)) * a.W + w0) * pixBytes;
        };
        if ((int)threadIdx.x < rows)
            rowPhase[threadIdx.x] = (unsigned char)(row_start((int)threadIdx.x) & 15);
        T* planes = reinterpret_cast<T*>(a.stack) + (long long)ib * a.C * P + (long long)r0 * S;   // [C][P] view at row r0
        const int nPix = rows * S;

        // One 16-byte slot of a row buffer and the piece of the row's clipped run it holds.
        struct Slot {
            long long lo, hi;   // global byte range [lo, hi) of the slot that belongs to the run (empty: lo >= hi)
            long long A;        // the slot's global address (16-byte aligned)
            uint32_t at;        // the slot's shared-memory address
        };
        const int nSlots = rows * (int)p.slotsPerRow.div;
        auto slot_of = [&](int k) -> Slot {
            Slot t;
            t.lo = 0, t.hi = 0, t.A = 0, t.at = 0;
            if (k >= nSlots)
                return t;
            uint32_t rl, q;
            p.slotsPerRow.divmod((uint32_t)k, rl, q);
            const int h = h0 + (int)rl;
            if (h < 0 || h >= a.H)
                return t;
            const long long g0 = row_start((int)rl);
            t.A = (g0 & ~15ll) + 16ll * q;
            t.lo = max(t.A, g0 + bLo), t.hi = min(t.A + 16, g0 + bHi);
            t.at = tileAddr + rl * (uint32_t)p.rowPitch + 16u * q;
            return t;
        };
        // Lane's pixel px of the item -> (its row buffer address for channel c, in range?); (rl, s) are the
        // pixel's row and column inside the item and advance by 32 pixels per step without a division.
        auto advance = [&](int& rl, int& s) {
            s += p.stepS, rl += p.stepR;
            if (s >= S)
                s -= S, ++rl;
        };
        auto pixel_at = [&](int rl, int s, int c, bool& inr) -> uint32_t {
            const int h = h0 + rl, w = w0 + s;
            inr = h >= 0 && h < a.H && w >= 0 && w < a.W;
            return tileAddr + (uint32_t)(rl * p.rowPitch) + rowPhase[min(rl, kRawMaxRows - 1)] + (uint32_t)((s * a.C + c) * SZ);
        };
        __syncthreads();   // rowPhase is set (and the previous item's buffers are no longer read)

        if constexpr (MODE == kGather) {
            // image -> row buffers: all loads of a batch are issued before its stores
            for (int k0 = threadIdx.x; k0 < nSlots; k0 += kThreads * kRawUnroll) {
                Slot t[kRawUnroll];
                uint4 v[kRawUnroll];
#pragma unroll
                for (int u = 0; u < kRawUnroll; ++u) {
                    t[u] = slot_of(k0 + u * kThreads);
                    if (t[u].hi - t[u].lo == 16)
                        v[u] = ld_stream(reinterpret_cast<const uint4*>(t[u].A));
                }
#pragma unroll
                for (int u = 0; u < kRawUnroll; ++u) {
                    if (t[u].hi - t[u].lo == 16) {
                        sts128(t[u].at, v[u]);
                    } else {   // a ragged end of the run (or nothing): element by element
                        uint32_t at = t[u].at + (uint32_t)(t[u].lo - t[u].A);
                        for (long long b = t[u].lo; b < t[u].hi; b += SZ, at += SZ) {
                            const E e = ld_stream(reinterpret_cast<const E*>(b));
                            if constexpr (SZ == 4)
                                sts32(at, e);
                            else
                                sts16(at, e);
                        }
                    }
                }
            }
            __syncthreads();
            // row buffers -> stack: a warp writes consecutive pixels of one channel plane
            for (int c = warp; c < a.C; c += kThreads / 32) {
                int rl = lane / S, s = lane - rl * S;     // one division per plane, none per element
                E* plane = reinterpret_cast<E*>(planes) + (long long)c * P;
                for (int px = lane; px < nPix; px += 32) {
                    bool inr;
                    const uint32_t at = pixel_at(rl, s, c, inr);
                    E e = 0;
                    if (inr)
                        e = SZ == 4 ? (E)lds32(at) : (E)lds16(at);
                    plane[px] = e;
                    advance(rl, s);
                }
            }
        } else {
            // stack -> row buffers: a warp reads consecutive pixels of one channel plane, a batch of loads at a time
            for (int c = warp; c < a.C; c += kThreads / 32) {
                int rl = lane / S, s = lane - rl * S;
                const E* plane = reinterpret_cast<const E*>(planes) + (long long)c * P;
                for (int px0 = lane; px0 < nPix; px0 += 32 * kRawUnroll) {
                    E e[kRawUnroll];
                    uint32_t at[kRawUnroll];
                    bool inr[kRawUnroll];
#pragma unroll
                    for (int u = 0; u < kRawUnroll; ++u) {
                        const int px = px0 + 32 * u;
                        inr[u] = false, at[u] = 0, e[u] = 0;
                        if (px < nPix) {
                            at[u] = pixel_at(rl, s, c, inr[u]);
                            if (inr[u])
                                e[u] = ld_stream(plane + px);
                            advance(rl, s);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kRawUnroll; ++u) {
                        if (inr[u]) {
                            if constexpr (SZ == 4)
                                sts32(at[u], e[u]);
                            else
                                sts16(at[u], e[u]);
                        }
                    }
                }
            }
            __syncthreads();
            // row buffers -> image: whole slots as 16-byte stores / adds / reductions, ragged ends by element
            for (int k0 = threadIdx.x; k0 < nSlots; k0 += kThreads * kRawUnroll) {
                Slot t[kRawUnroll];
                uint4 old[kRawUnroll];
#pragma unroll
                for (int u = 0; u < kRawUnroll; ++u) {
                    t[u] = slot_of(k0 + u * kThreads);
                    old[u] = make_uint4(0, 0, 0, 0);
                    if constexpr (MODE == kScatterAdd)
                        if (t[u].hi - t[u].lo == 16)
                            old[u] = *reinterpret_cast<const uint4*>(t[u].A);
                }
#pragma unroll
                for (int u = 0; u < kRawUnroll; ++u) {
                    if (t[u].hi - t[u].lo == 16) {
                        image_write<16, MODE, T>(reinterpret_cast<uint4*>(t[u].A), lds128(t[u].at), old[u]);
                    } else {
                        uint32_t at = t[u].at + (uint32_t)(t[u].lo - t[u].A);
                        for (long long b = t[u].lo; b < t[u].hi; b += SZ, at += SZ) {
                            E* g = reinterpret_cast<E*>(b);
                            const E e = SZ == 4 ? (E)lds32(at) : (E)lds16(at);
                            E prev = 0;
                            if constexpr (MODE == kScatterAdd)
                                prev = *g;
                            image_write<SZ, MODE, T>(g, e, prev);
                        }
                    }
                }
            }
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

template <int VB, int MODE, typename T>
static void launch_rows(const BlockArgs& a, cudaStream_t stream)
{
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
template <int MODE, typename T> static bool launch_planes_rows(const BlockArgs& a, cudaStream_t stream)
{
    const long long rowBytes = (long long)a.bSzW * a.C * (long long)sizeof(T);
    const long long rowPitch = ((rowBytes + 15 + 15) / 16) * 16;   // the run, its misalignment (< 16), rounded up
    if (rowPitch > kTileBytes)
        return false;
    RawPlan p;
    p.rowBytes = (int)rowBytes, p.rowPitch = (int)rowPitch;
    int rows = (int)(kTileBytes / rowPitch);
    rows = rows < a.bSzH ? rows : a.bSzH;
    rows = rows < kRawMaxRows ? rows : kRawMaxRows;
    const int nChunks = (a.bSzH + rows - 1) / rows;
    p.rowsPerItem = (a.bSzH + nChunks - 1) / nChunks;               // the fewest, nearly equal chunks of rows
    p.rChunks = FastDiv((uint32_t)((a.bSzH + p.rowsPerItem - 1) / p.rowsPerItem));
    p.slotsPerRow = FastDiv((uint32_t)(rowPitch / 16));
    p.stepS = 32 % a.bSzW, p.stepR = 32 / a.bSzW;
    const long long nItems = (long long)a.numActive * p.rChunks.div;
    static const int perSm = ctas_per_sm(planes_rows_kernel<MODE, T>, kThreads);
    const int wave = perSm * sm_count();
    const bool perItem = a.num_active_dev == nullptr && nItems <= 0x7fffffffll;
    const unsigned grid = (unsigned)(perItem ? nItems : (nItems < wave ? nItems : wave));
    launch_pdl(planes_rows_kernel<MODE, T>, dim3(grid), dim3(kThreads), 0, stream, a, p);
    return true;
}

template <int VB, int MODE, typename T>
static void launch_planes(const BlockArgs& a, cudaStream_t stream)
{
    // 32-bit elements only: measured on [8,512,512,C] at 20 %, C = 33 fp32 gains (gather 61 -> 53 us, atomic
    // scatter 66 -> 64 us) while C = 100 fp16 loses (92 -> 117 us, 115 -> 164 us: 2-byte accesses on both sides of
    // the transposition).  Option planes=4 keeps the element-wise kernel for every shape.
    if constexpr (sizeof(T) == 4)
        if (options().planes != 4 && launch_planes_rows<MODE, T>(a, stream))
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
