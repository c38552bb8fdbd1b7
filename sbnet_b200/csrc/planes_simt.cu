// Transposed ([nB,C,R,S]) gather and scatter, one short CTA per tile (sm_100a).
//
// Default implementation of the plane-layout ops for pixels of a multiple of 16 bytes; other shapes
// run the general kernel of gather_scatter.cu.  Semantics follow the reference CPU functors
// (sbnet_ops/sparse_gather.cc:61-132, transposed branches).  On B200 a grid of many short CTAs
// streams measurably faster than a resident grid looping over the same tiles, so with a host-side
// block count every work item gets its own CTA.  A work item is one active block x one 128-byte
// channel chunk (the last chunk of a pixel may be narrower): a tile of P = R*S pixels x up to 128
// bytes, staged ONCE in shared memory (48 KB = 384 pixels).  Blocks of more than 384 pixels are cut
// into pixel chunks; blocks of at most 192 pixels share a tile with their neighbours in the list.
//
//  gather : every thread issues all of its 16-byte image loads (out-of-image pixels become zeros),
//           stores them to the tile in [pixel][128 B] order with the 16-byte groups XOR-swizzled by
//           the pixel index; each thread then reads its share back as 16-byte channel groups, the
//           CTA synchronises, and the same threads write words of one channel (1 fp32 pixel / 2
//           16-bit pixels, regrouped with prmt) in [channel][pixel] order into the same buffer
//           (in-place transpose through registers).  The tile leaves as ONE bulk store (TMA engine):
//           a chunk's channel planes are contiguous in the stack.
//  scatter: the tile (contiguous in the stack) is copied in, swizzled so that eight neighbouring
//           lanes can own the eight 16-byte groups of one pixel; words are regrouped into 16-byte
//           channel groups and written / added / reduced into the image, whole 128-byte lines per
//           warp instruction, with a per-pixel in-range test.  With a device-side block count the
//           same kernel runs as one resident wave striding over the items.
//
// Element types: float, __half and (accumulating scatter only) __nv_bfloat16; 16-bit gathers and
// overwrites of any type run the __half instantiations, which only move bits.
#include <stdlib.h>

#include <algorithm>

#include "async_ptx.cuh"
#include "common.cuh"
#include "kernels.h"
#include "options.h"

namespace sbnet {

constexpr int kPsThreads = 256;
constexpr int kPsMaxPixels = 384;
constexpr int kPsTileBytes = 128 * kPsMaxPixels;          // 48 KB
constexpr int kPsMaxVecs = (8 * kPsMaxPixels) / kPsThreads;   // 16-byte vectors per thread

struct SimtPlan {
    FastDiv cChunks;   // 128-byte channel chunks per pixel
    FastDiv pChunks;   // pixel chunks per block (1 unless the block has more than 384 pixels)
    FastDiv unitsPerRowLast; // unitsPerRow of a block's last (shorter) pixel chunk
    int chunkPixels;   // pixels per pixel chunk (a multiple of 8); the last chunk of a block may hold fewer
    int rowsAligned;   // every plane row of every pixel chunk starts and ends on a 16-byte boundary
    FastDiv blockW;    // S
    FastDiv unitsPerRow; // copy-in units (GW words each) per channel plane (swizzled scatter only)
    int pitchWords;    // tile row pitch of the swizzled scatter: the tile's words per row rounded up to 32
    int groups;        // 16-byte channel groups per pixel (C*sizeof(T)/16); the last chunk may hold fewer than 8
    int pixels;        // P
    int units;         // words per channel plane: P (fp32) or P/2 rounded up (16-bit types)
    // several small blocks per work item (kTileMulti)
    int blocksPerItem; // blocks sharing one tile
    FastDiv pixelsDiv; // P
    FastDiv unitsDiv;  // units
    FastDiv runVecs, runVecsLast; // 16-byte vectors of one block's chunk (full / last channel chunk)
};

// How a work item maps onto the 384-pixel tile.
constexpr int kTileSingle = 0;   // one block (at most 384 pixels) x one channel chunk
constexpr int kTileChunked = 1;  // blocks of more than 384 pixels, cut into pixel chunks
constexpr int kTileMulti = 2;    // blocks of at most 192 pixels: as many whole blocks as fit share the tile

// kTileChunked: a work item is (block, pixel chunk, channel chunk) and its transposed tile leaves as
// one run per channel plane.
// kTileMulti: the tile holds the pixels of several consecutive blocks of the list back to back; each
// block's region is transposed in place on its own and leaves as its own bulk store.
// ODD (16-bit blocks of an odd pixel count, whole blocks): plane rows are an odd number of halves,
// so a channel's row starts on a word boundary only for even channels; words of odd channels are
// written as two halves, and p.units counts a row's words rounded up.  (Pixel chunks of such
// blocks keep word-aligned tile rows and shift the rows of odd channels on their way out.)
template <typename T, int SHAPE, bool ODD = false>
__global__ void __launch_bounds__(kPsThreads, sizeof(T) == 2 ? 4 : 3) planes_gather_simt(const BlockArgs a, const SimtPlan p)
{
    pdl_wait();   // nothing global is read or written before the kernel queued ahead of this one is done
    constexpr bool PCH = SHAPE == kTileChunked, MB = SHAPE == kTileMulti;
    static_assert(!ODD || (sizeof(T) == 2 && !PCH), "odd rows: fp16, whole blocks only");
    __shared__ __align__(1024) unsigned char tileRaw[kPsTileBytes];
    constexpr int EPW = 4 / (int)sizeof(T);
    constexpr int CPG = 16 / (int)sizeof(T);
    constexpr int kMaxTasks = ((kPsMaxPixels / EPW + 15) / 16 + 1) / 2;
    const uint32_t tile = smem_u32(tileRaw);

    uint32_t ib, cc;                          // (first) block of the item, channel chunk
    int p0 = 0, P = p.pixels, U = p.units;   // first pixel, pixels and words per plane row of this item
    int nBlk = 1;                            // blocks sharing the tile
    if constexpr (PCH) {
        uint32_t rest, pc;
        p.cChunks.divmod(blockIdx.x, rest, cc);
        p.pChunks.divmod(rest, ib, pc);
        p0 = (int)pc * p.chunkPixels;
        P = min(p.chunkPixels, p.pixels - p0);
        U = (P + EPW - 1) / EPW;   // a 16-bit block of an odd pixel count ends in a chunk of an odd count
    } else if constexpr (MB) {
        uint32_t grp;
        p.cChunks.divmod(blockIdx.x, grp, cc);
        ib = grp * (uint32_t)p.blocksPerItem;
        nBlk = min(p.blocksPerItem, a.numActive - (int)ib);
        P = nBlk * p.pixels;   // the tile's pixel slots: block b owns slots [b*pixels, (b+1)*pixels)
        U = nBlk * p.units;
    } else {
        p.cChunks.divmod(blockIdx.x, ib, cc);
    }
    // image plane of a block's batch index, at this item's channel chunk, and the block's window origin
    auto locate = [&](uint32_t blk, int& h0, int& w0) -> const T* {
        const int n = a.idx[blk * 3 + 0];
        h0 = a.bOffsH + a.idx[blk * 3 + 1] * a.bStrH;
        w0 = a.bOffsW + a.idx[blk * 3 + 2] * a.bStrW;
        return reinterpret_cast<const T*>(a.image) + (long long)n * a.H * a.W * a.C + (long long)cc * (128 / (int)sizeof(T));
    };
    int h0 = 0, w0 = 0;
    const T* imgN = nullptr;
    if constexpr (!MB)
        imgN = locate(ib, h0, w0);
    const int nG = min(8, p.groups - 8 * (int)cc);   // 16-byte groups in this chunk

    // ---- image -> tile: thread owns 16-byte group j of pixels px0, px0+32, ...
    {
        const int j = threadIdx.x & 7, px0 = threadIdx.x >> 3;
        uint4 v[kPsMaxVecs];
#pragma unroll
        for (int k = 0; k < kPsMaxVecs; ++k) {
            const int px = px0 + 32 * k;
            v[k] = make_uint4(0, 0, 0, 0);
            if (px < P && j < nG) {
                uint32_t r, s, inBlock = (uint32_t)(px + p0);
                if constexpr (MB) {
                    uint32_t b;
                    p.pixelsDiv.divmod((uint32_t)px, b, inBlock);
                    imgN = locate(ib + b, h0, w0);
                }
                p.blockW.divmod(inBlock, r, s);
                const int h = h0 + (int)r, w = w0 + (int)s;
                if (h >= 0 && h < a.H && w >= 0 && w < a.W)
                    v[k] = ld_stream(reinterpret_cast<const uint4*>(imgN + ((long long)h * a.W + w) * a.C + j * CPG));
            }
        }
        const uint32_t dst = tile + ((uint32_t)(j ^ (px0 & 7)) << 4);   // (px & 7) == (px0 & 7)
#pragma unroll
        for (int k = 0; k < kPsMaxVecs; ++k)
            if (px0 + 32 * k < P)
                sts128(dst + (uint32_t)(px0 + 32 * k) * 128u, v[k]);
    }
    __syncthreads();
    pdl_launch_dependents();   // this CTA's loads have landed: the next kernel's CTAs may take the slots that free up

    // ---- tile -> registers (16-byte channel groups), then registers -> tile in [channel][pixel] order
    const int nTasks = ((U + 15) >> 4) * 128;
    uint4 A[kMaxTasks], B[kMaxTasks];
#pragma unroll
    for (int q = 0; q < kMaxTasks; ++q) {
        const int t = threadIdx.x + q * kPsThreads;
        int j, u;
        transpose_task<EPW>(t, j, u);
        if (t < nTasks && u < U && j < nG) {
            if constexpr (ODD) {   // word u = word uIn of block b: pixels 2*uIn and (if it exists) 2*uIn+1
                uint32_t b = 0, uIn = (uint32_t)u;
                if constexpr (MB)
                    p.unitsDiv.divmod((uint32_t)u, b, uIn);
                const int r0 = (int)(b * (uint32_t)p.pixels + 2u * uIn), r1 = r0 + 1;
                A[q] = lds128(tile + r0 * 128 + ((j ^ (r0 & 7)) << 4));
                B[q] = make_uint4(0, 0, 0, 0);
                if ((int)(2u * uIn) + 1 < p.pixels)
                    B[q] = lds128(tile + r1 * 128 + ((j ^ (r1 & 7)) << 4));
            } else if constexpr (EPW == 2) {
                const int r0 = 2 * u, r1 = 2 * u + 1;
                A[q] = lds128(tile + r0 * 128 + ((j ^ (r0 & 7)) << 4));
                B[q] = lds128(tile + r1 * 128 + ((j ^ (r1 & 7)) << 4));
            } else {
                A[q] = lds128(tile + u * 128 + ((j ^ (u & 7)) << 4));
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kMaxTasks; ++q) {
        const int t = threadIdx.x + q * kPsThreads;
        int j, u;
        transpose_task<EPW>(t, j, u);
        if (t < nTasks && u < U && j < nG) {
            uint32_t base = tile + ((uint32_t)(CPG * j) * U + u) * 4u;
            uint32_t pitch = (uint32_t)U * 4u;
            if constexpr (MB) {   // word u of the tile = word uIn of block b's region
                uint32_t b, uIn;
                p.unitsDiv.divmod((uint32_t)u, b, uIn);
                base = tile + b * (uint32_t)p.pixels * 128u + ((uint32_t)(CPG * j) * p.units + uIn) * 4u;
                pitch = (uint32_t)p.units * 4u;
            }
            if constexpr (ODD) {
                uint32_t b = 0, uIn = (uint32_t)u;
                if constexpr (MB)
                    p.unitsDiv.divmod((uint32_t)u, b, uIn);
                const uint32_t region = tile + b * (uint32_t)p.pixels * 128u;
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
    fence_async_smem();   // the bulk store reads what the generic proxy just wrote
    __syncthreads();
    T* dst = reinterpret_cast<T*>(a.stack) +
             ((long long)ib * a.C + (long long)cc * (128 / (int)sizeof(T))) * p.pixels + p0;
    if constexpr (PCH) {
        // one run of U words per channel plane, p.pixels elements apart
        const int rows = nG * CPG;
        if (EPW == 2 && (p.pixels & 1)) {
            // 16-bit rows of an odd length: the rows of odd channels start on an odd half.  Tile rows
            // are word aligned, so such a row leaves as its first half, then words made of the high
            // half of one tile word and the low half of the next, then (even chunk) its last half.
            unsigned short* dstH = reinterpret_cast<unsigned short*>(dst);
            const int lane = threadIdx.x & 31;
            for (int c = threadIdx.x >> 5; c < rows; c += kPsThreads / 32) {
                unsigned short* row = dstH + (long long)c * p.pixels;
                const uint32_t trow = tile + (uint32_t)(c * U) * 4u;
                if ((c & 1) == 0) {
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
        } else if (p.rowsAligned) {
            if ((int)threadIdx.x < rows) {
                bulk_store_1d(dst + (long long)threadIdx.x * p.pixels, tile + threadIdx.x * (uint32_t)U * 4u, (uint32_t)U * 4u);
                bulk_wait_read<0>();
            }
        } else if ((p.pixels / EPW) % 2 == 0) {   // rows of an even number of words: 8-byte stores
            uint2* dst2 = reinterpret_cast<uint2*>(dst);
            const long long row2 = p.pixels / EPW / 2;
            const int U2 = U / 2;
            for (int c = threadIdx.x >> 5; c < rows; c += kPsThreads / 32)
                for (int u = threadIdx.x & 31; u < U2; u += 32) {
                    uint2 v;
                    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(tile + (uint32_t)(c * U2 + u) * 8u));
                    dst2[c * row2 + u] = v;
                }
        } else {
            uint32_t* dstW = reinterpret_cast<uint32_t*>(dst);   // rows start on word boundaries (fp16: P even)
            const long long rowW = p.pixels / EPW;
            for (int c = threadIdx.x >> 5; c < rows; c += kPsThreads / 32)
                for (int u = threadIdx.x & 31; u < U; u += 32)
                    dstW[c * rowW + u] = lds32(tile + (uint32_t)(c * U + u) * 4u);
        }
    } else if constexpr (MB) {
        if ((int)threadIdx.x < nBlk) {   // block b's planes of this chunk: one contiguous run of the stack
            bulk_store_1d(dst + (long long)threadIdx.x * a.C * p.pixels, tile + threadIdx.x * (uint32_t)p.pixels * 128u,
                          (uint32_t)(16 * nG * p.pixels));
            bulk_wait_read<0>();
        }
    } else if (threadIdx.x == 0) {
        bulk_store_1d(dst, tile, (uint32_t)(16 * nG * P));
        bulk_wait_read<0>();   // shared memory must outlive the engine's read of it
    }
}

// GW >= 1 (plane rows of a multiple of GW = 1, 2 or 4 words): the tile is stored with a row pitch rounded
// up to 32 words and its 16-byte column groups XOR-ed by the channel-group index, which lets eight
// neighbouring lanes own the eight 16-byte groups of ONE pixel without bank conflicts -- every
// warp-level store / reduction then covers whole 128-byte lines of the image (four pixels) instead
// of sixteen scattered sectors (measured: 5.3 -> 6.4 TB/s on the fp16 add scatter).  GW is the
// copy-in unit in words (a unit must not straddle plane rows; with one block per item the chunk is
// one contiguous run, read with 16-byte loads and split into GW-word pieces when it is stored, so
// rows of an odd number of words, GW == 1, get the same tile).  GW == 0 (fp16 blocks of an odd
// pixel count): dense copy of the chunk, rows of an odd number of halves; words of odd channels are
// read as two halves.  That layout needs no swizzle: channel groups are 4*P words apart, and with
// P odd the eight groups land on eight different bank quads.
// kTileChunked (GW >= 2 only) / kTileMulti: as in the gather.  kTileMulti keeps block b's words in
// columns [b*units, (b+1)*units) of every tile row (GW == 0: the blocks' dense copies back to back).
template <int MODE, typename T, int GW, int SHAPE>
__global__ void __launch_bounds__(kPsThreads, MODE == kScatterAdd ? 2 : 3)
planes_scatter_simt(const BlockArgs a, const SimtPlan p)
{
    pdl_wait();   // nothing global is read or written before the kernel queued ahead of this one is done
    constexpr bool PCH = SHAPE == kTileChunked, MB = SHAPE == kTileMulti;
    static_assert(!PCH || GW > 1, "pixel chunks copy in whole 8- or 16-byte units");
    static_assert(GW != 0 || sizeof(T) == 2, "odd rows of halves: fp16 only");
    constexpr bool ODD = GW == 0;
    __shared__ __align__(128) unsigned char tileRaw[kPsTileBytes];
    constexpr int EPW = 4 / (int)sizeof(T);
    constexpr int CPG = 16 / (int)sizeof(T);
    constexpr bool SWZ = GW > 0;
    constexpr int kMaxTasks = (8 * (kPsMaxPixels / EPW)) / kPsThreads;
    const uint32_t tile = smem_u32(tileRaw);

    // One item per CTA when the grid was sized from a host-side count; with a device-side count the
    // grid is one resident wave and every CTA strides over the items.
    int nActive = a.numActive;
    if (a.num_active_dev != nullptr)
        nActive = min(__ldg(a.num_active_dev), a.numActive);
    long long nItems = (long long)nActive * p.cChunks.div * (PCH ? p.pChunks.div : 1u);
    if constexpr (MB)
        nItems = (long long)((nActive + p.blocksPerItem - 1) / p.blocksPerItem) * p.cChunks.div;
    for (long long item = blockIdx.x; item < nItems; item += gridDim.x) {
    uint32_t ib, cc;                          // (first) block of the item, channel chunk
    int p0 = 0, P = p.pixels, U = p.units;   // first pixel, pixels and words per plane row of this item
    int nBlk = 1;                            // blocks sharing the tile
    FastDiv unitsPerRow = p.unitsPerRow;
    if constexpr (PCH) {
        uint32_t rest, pc;
        p.cChunks.divmod((uint32_t)item, rest, cc);
        p.pChunks.divmod(rest, ib, pc);
        p0 = (int)pc * p.chunkPixels;
        P = min(p.chunkPixels, p.pixels - p0);
        U = P / EPW;
        if (pc + 1 == p.pChunks.div)
            unitsPerRow = p.unitsPerRowLast;
    } else if constexpr (MB) {
        uint32_t grp;
        p.cChunks.divmod((uint32_t)item, grp, cc);
        ib = grp * (uint32_t)p.blocksPerItem;
        nBlk = min(p.blocksPerItem, nActive - (int)ib);
        P = nBlk * p.pixels;   // the tile's pixel slots: block b owns slots [b*pixels, (b+1)*pixels)
        U = nBlk * p.units;
    } else {
        p.cChunks.divmod((uint32_t)item, ib, cc);
    }
    const int nG = min(8, p.groups - 8 * (int)cc);   // 16-byte groups in this chunk
    const int nTasks = 8 * U;
    const uint32_t pitchW = SWZ ? (uint32_t)p.pitchWords : (uint32_t)U;   // tile row pitch in words

    // A block's window: image plane of its batch index at this item's channel chunk + window origin.
    struct Window {
        T* img;
        int h0, w0;
    };
    auto window = [&](uint32_t blk) -> Window {
        Window wn;
        const int n = a.idx[blk * 3 + 0];
        wn.h0 = a.bOffsH + a.idx[blk * 3 + 1] * a.bStrH;
        wn.w0 = a.bOffsW + a.idx[blk * 3 + 2] * a.bStrW;
        wn.img = reinterpret_cast<T*>(a.image) + (long long)n * a.H * a.W * a.C + (long long)cc * (128 / (int)sizeof(T));
        return wn;
    };
    Window own = {nullptr, 0, 0};
    if constexpr (!MB)
        own = window(ib);
    // tile pixel slot -> its block's window and the pixel index inside that block
    auto locate = [&](int slot, int& pix) -> Window {
        if constexpr (MB && ODD) {   // blocks of an odd pixel count: a block's words do not tile its slots
            uint32_t b, uIn;
            p.unitsDiv.divmod((uint32_t)slot >> 1, b, uIn);
            pix = (int)(2u * uIn);
            return window(ib + b);
        } else if constexpr (MB) {
            uint32_t b, q;
            p.pixelsDiv.divmod((uint32_t)slot, b, q);
            pix = (int)q;
            return window(ib + b);
        } else {
            pix = slot + p0;
            return own;
        }
    };
    auto dest = [&](const Window& wn, int pix, int j) -> uint4* {
        uint32_t r, sx;
        p.blockW.divmod((uint32_t)pix, r, sx);
        const int h = wn.h0 + (int)r, w = wn.w0 + (int)sx;
        if (h < 0 || h >= a.H || w < 0 || w >= a.W)
            return nullptr;
        return reinterpret_cast<uint4*>(wn.img + ((long long)h * a.W + w) * a.C + j * CPG);
    };
    // task t of this thread -> (16-byte channel group j, word column u): eight neighbouring lanes
    // own the 128 bytes of one pixel (pair)
    auto task = [&](int t, int& j, int& u) {
        j = t & 7;
        u = t >> 3;
    };

    // ---- stack -> tile: the chunk's planes are one contiguous run of 32*P words (pixel chunks: one
    // run of U words per plane, p.pixels elements apart; shared tile: one run per block)
    {
        const T* srcT = reinterpret_cast<const T*>(a.stack) +
                        ((long long)ib * a.C + (long long)cc * (128 / (int)sizeof(T))) * p.pixels + p0;
        constexpr uint32_t G = GW > 0 ? GW : 1;
        const uint32_t rowUnits = (uint32_t)(p.pixels / EPW) / G;               // one whole plane row
        const FastDiv runDiv = (int)cc + 1 == (int)p.cChunks.div ? p.runVecsLast : p.runVecs;
        // copy-in unit vi -> its offset from srcT (in units) and its word in the tile (one block per item)
        auto place = [&](uint32_t vi, uint32_t& srcUnit, uint32_t& tileW) {
            uint32_t c, col;
            unitsPerRow.divmod(vi, c, col);
            srcUnit = PCH ? c * rowUnits + col : vi;
            tileW = c * pitchW + ((col * G) ^ (4u * ((c / CPG) & 7u)));
        };
        if constexpr ((GW >= 1 && MB) || ((GW == 2 || GW == 1) && SHAPE == kTileSingle)) {
            // A block's chunk is one contiguous 16-byte aligned run: 16-byte loads even where plane
            // rows are only 8- or 4-byte multiples; a vector is stored as 4/GW pieces of GW words,
            // each placed in its own row and column.
            const uint4* src = reinterpret_cast<const uint4*>(srcT);
            const int nVec = nG * P;
            const uint32_t blockVecs = (uint32_t)((long long)a.C * p.pixels * (int)sizeof(T) / 16);
            uint4 v[kPsMaxVecs];
#pragma unroll
            for (int k = 0; k < kPsMaxVecs; ++k) {
                const int vi = (int)threadIdx.x + k * kPsThreads;
                if (vi < nVec) {
                    uint32_t at = (uint32_t)vi;
                    if constexpr (MB) {   // vector rest of block b's run
                        uint32_t b, rest;
                        runDiv.divmod((uint32_t)vi, b, rest);
                        at = b * blockVecs + rest;
                    }
                    v[k] = ld_stream(src + at);
                }
            }
#pragma unroll
            for (int k = 0; k < kPsMaxVecs; ++k) {
                const int vi = (int)threadIdx.x + k * kPsThreads;
                if (vi < nVec) {
                    uint32_t b = 0, rest = (uint32_t)vi;
                    if constexpr (MB)
                        runDiv.divmod((uint32_t)vi, b, rest);
                    uint32_t c, col;   // row and column (in GW-word units) of the vector's first piece
                    p.unitsPerRow.divmod((uint32_t)(4 / GW) * rest, c, col);
                    const uint32_t colBase = b * (uint32_t)p.units;
                    const uint32_t piece[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
                    for (int h = 0; h < 4 / GW; ++h) {
                        const uint32_t w = c * pitchW + ((colBase + col * GW) ^ (4u * ((c / CPG) & 7u)));
                        if constexpr (GW == 4)
                            sts128(tile + w * 4u, v[k]);
                        else if constexpr (GW == 2)
                            asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(tile + w * 4u), "r"(piece[2 * h]),
                                         "r"(piece[2 * h + 1])
                                         : "memory");
                        else
                            sts32(tile + w * 4u, piece[h]);
                        if (++col == p.unitsPerRow.div) {
                            col = 0;
                            ++c;
                        }
                    }
                }
            }
        } else if constexpr (GW == 2) {
            const uint2* src = reinterpret_cast<const uint2*>(srcT);
            const int nUnit = 2 * nG * P;
#pragma unroll
            for (int half = 0; half < 2; ++half) {   // two batches keep the register count under the launch bound
                uint2 v[kPsMaxVecs];
#pragma unroll
                for (int k = 0; k < kPsMaxVecs; ++k) {
                    const int vi = (int)threadIdx.x + (half * kPsMaxVecs + k) * kPsThreads;
                    if (vi < nUnit) {
                        uint32_t srcUnit, w;
                        place((uint32_t)vi, srcUnit, w);
                        v[k] = ld_stream(src + srcUnit);
                    }
                }
#pragma unroll
                for (int k = 0; k < kPsMaxVecs; ++k) {
                    const int vi = (int)threadIdx.x + (half * kPsMaxVecs + k) * kPsThreads;
                    if (vi < nUnit) {
                        uint32_t srcUnit, w;
                        place((uint32_t)vi, srcUnit, w);
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(tile + w * 4u), "r"(v[k].x), "r"(v[k].y)
                                     : "memory");
                    }
                }
            }
        } else {
            const uint4* src = reinterpret_cast<const uint4*>(srcT);
            const int nVec = nG * P;
            // pixel chunks / shared tiles: the per-unit arithmetic costs registers, so two batches as above
            constexpr int kBatches = SHAPE == kTileSingle ? 1 : 2, kPer = kPsMaxVecs / kBatches;
#pragma unroll
            for (int b = 0; b < kBatches; ++b) {
                uint4 v[kPer];
#pragma unroll
                for (int k = 0; k < kPer; ++k) {
                    const int vi = (int)threadIdx.x + (b * kPer + k) * kPsThreads;
                    if (vi < nVec) {
                        uint32_t srcUnit = (uint32_t)vi, w;
                        if constexpr (ODD && MB) {   // dense regions packed back to back: only the source needs the block
                            uint32_t blk, rest;
                            runDiv.divmod((uint32_t)vi, blk, rest);
                            srcUnit = blk * (uint32_t)((long long)a.C * p.pixels * (int)sizeof(T) / 16) + rest;
                        } else if constexpr (SHAPE != kTileSingle) {
                            place((uint32_t)vi, srcUnit, w);
                        }
                        v[k] = ld_stream(src + srcUnit);
                    }
                }
#pragma unroll
                for (int k = 0; k < kPer; ++k) {
                    const int vi = (int)threadIdx.x + (b * kPer + k) * kPsThreads;
                    if (vi < nVec) {
                        uint32_t srcUnit, w = (uint32_t)vi * 4u;
                        if constexpr (GW == 4)   // row = channel; XOR the 16-byte column group with the channel group
                            place((uint32_t)vi, srcUnit, w);
                        sts128(tile + w * 4u, v[k]);
                    }
                }
            }
        }
    }
    // read-add-write: the destination loads go out while the tile settles
    uint4 old[kMaxTasks][EPW];
    if constexpr (MODE == kScatterAdd) {
#pragma unroll
        for (int q = 0; q < kMaxTasks; ++q) {
            const int t = threadIdx.x + q * kPsThreads;
            int j, u;
            task(t, j, u);
#pragma unroll
            for (int e = 0; e < EPW; ++e)
                old[q][e] = make_uint4(0, 0, 0, 0);
            if (t < nTasks && u < U && j < nG) {
                int pix;
                const Window wn = locate(u * EPW, pix);
#pragma unroll
                for (int e = 0; e < EPW; ++e)
                    if (!ODD || pix + e < p.pixels)
                        if (const uint4* d = dest(wn, pix + e, j))
                            old[q][e] = *d;
            }
        }
    }
    __syncthreads();

    // ---- tile -> image
#pragma unroll
    for (int q = 0; q < kMaxTasks; ++q) {
        const int t = threadIdx.x + q * kPsThreads;
        int j, u;
        task(t, j, u);
        if (t >= nTasks || u >= U || j >= nG)
            continue;
        const uint32_t col = SWZ ? ((uint32_t)u ^ (4u * ((uint32_t)j & 7u))) : (uint32_t)u;
        const uint32_t base = tile + ((uint32_t)(CPG * j) * pitchW + col) * 4u;
        const uint32_t pitch = pitchW * 4u;
        int pix;
        const Window wn = locate(u * EPW, pix);   // fp16: both pixels of a word lie in one block (P is even)
        if constexpr (EPW == 2) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if constexpr (ODD) {   // half index of (channel 8j+i, pixel 2u): even exactly for even channels
                    uint32_t region = tile, uIn = (uint32_t)u;
                    if constexpr (MB) {   // block b's dense copy starts b runs into the tile
                        uint32_t b;
                        p.unitsDiv.divmod((uint32_t)u, b, uIn);
                        region = tile + b * (uint32_t)(16 * nG * p.pixels);
                    }
                    const uint32_t at = region + ((uint32_t)(CPG * j + i) * (uint32_t)p.pixels + 2u * uIn) * 2u;
                    w[i] = (i & 1) == 0 ? lds32(at) : (lds16(at) | (lds16(at + 2u) << 16));
                } else {
                    w[i] = lds32(base + (uint32_t)i * pitch);
                }
            }
            const uint4 v0 = make_uint4(__byte_perm(w[0], w[1], 0x5410), __byte_perm(w[2], w[3], 0x5410),
                                        __byte_perm(w[4], w[5], 0x5410), __byte_perm(w[6], w[7], 0x5410));
            const uint4 v1 = make_uint4(__byte_perm(w[0], w[1], 0x7632), __byte_perm(w[2], w[3], 0x7632),
                                        __byte_perm(w[4], w[5], 0x7632), __byte_perm(w[6], w[7], 0x7632));
            if (uint4* d = dest(wn, pix, j))
                image_write<16, MODE, T>(d, v0, old[q][0]);
            if (!ODD || pix + 1 < p.pixels)   // an odd row's last word holds one pixel
                if (uint4* d = dest(wn, pix + 1, j))
                    image_write<16, MODE, T>(d, v1, old[q][EPW - 1]);
        } else {
            const uint4 v = make_uint4(lds32(base), lds32(base + pitch), lds32(base + 2u * pitch),
                                       lds32(base + 3u * pitch));
            if (uint4* d = dest(wn, pix, j))
                image_write<16, MODE, T>(d, v, old[q][0]);
        }
    }
    __syncthreads();   // the tile is reused by the next item
    }
    pdl_launch_dependents();
}

// Pixels of a multiple of 16 bytes (the last 128-byte chunk may be partial), 16-byte aligned buffers.
// Blocks of more than 384 pixels run as pixel chunks (the scatter then needs plane rows of an even
// number of words).
static bool planes_simt_eligible(const BlockArgs& a, int itemsize)
{
    if (options().disableTma)
        return false;
    const long long P = (long long)a.bSzH * a.bSzW;
    if (((size_t)a.C * itemsize) % 16 != 0 || P > (1 << 24))
        return false;
    return ((reinterpret_cast<uintptr_t>(a.image) | reinterpret_cast<uintptr_t>(a.stack)) & 15) == 0;
}

cudaError_t launch_planes_simt(const BlockArgs& a, int dtype, int mode, cudaStream_t stream, bool* taken)
{
    *taken = false;
    const int itemsize = dtype == 0 ? 4 : 2;
    if (!planes_simt_eligible(a, itemsize))
        return cudaSuccess;
    // Gather with the block count on the device: shapes the persistent TMA pipeline takes go there (a
    // resident grid does not need the count at launch: 449 vs 460 us per step of the sync-free
    // pipeline benchmark); the others run the TMA-fed tile kernels over a grid sized for the largest
    // possible count, whose surplus CTAs leave at once.
    const bool dynGather = a.num_active_dev != nullptr && mode == kGather;
    if (dynGather && planes_tma_eligible(a, itemsize))
        return cudaSuccess;
    // Small gathers go to the pipeline as well: under about three resident waves of tile CTAs (4 per SM) the
    // rounds of load -> transpose -> store CTAs do not overlap and the last, partly filled round costs as
    // much as a full one, whereas the pipeline's CTAs keep loads running ahead of their transposition
    // (per launch inside a CUDA graph, [8,512,512,128] at 5 %: fp32 28.2 -> 25.7 us, fp16 15.4 -> 14.9 us;
    // at 20 % the tile CTAs are ahead again, 45.1 vs 47.0 us).
    if (mode == kGather && options().planes == 0 && planes_tma_eligible(a, itemsize) &&
        (long long)a.numActive * (((long long)a.C * itemsize + 127) / 128) <= 12ll * sm_count())
        return cudaSuccess;
    SimtPlan p;
    const int P = a.bSzH * a.bSzW;
    p.groups = (int)((size_t)a.C * itemsize / 16);
    p.cChunks = FastDiv((uint32_t)((p.groups + 7) / 8));
    p.blockW = FastDiv((uint32_t)a.bSzW);
    p.pixels = P;
    const bool odd = itemsize == 2 && (P & 1);   // fp16 rows of an odd number of halves
    p.units = itemsize == 4 ? P : (P + 1) / 2;
    const int gw = odd ? 0 : (p.units % 4 == 0 ? 4 : (p.units % 2 == 0 ? 2 : 1));   // words per copy-in unit
    // Blocks of more than 384 pixels: the fewest equal pixel chunks, each a multiple of 8 pixels.
    const int nPc = (P + kPsMaxPixels - 1) / kPsMaxPixels;
    const bool pch = nPc > 1;
    if (pch && mode != kGather && gw < 2)
        return cudaSuccess;
    const int epw = 4 / itemsize;
    p.chunkPixels = pch ? (((P + nPc - 1) / nPc + 7) & ~7) : P;
    p.pChunks = FastDiv((uint32_t)((P + p.chunkPixels - 1) / p.chunkPixels));
    const int chunkUnits = p.chunkPixels / epw;
    const int lastUnits = (P - ((int)p.pChunks.div - 1) * p.chunkPixels) / epw;
    p.rowsAligned = ((size_t)P * itemsize) % 16 == 0;
    p.unitsPerRow = FastDiv((uint32_t)(gw >= 1 ? (pch ? chunkUnits : p.units) / gw : 1));
    p.unitsPerRowLast = FastDiv((uint32_t)(gw >= 1 ? (pch ? lastUnits : p.units) / gw : 1));
    p.pitchWords = ((pch ? chunkUnits : p.units) + 31) & ~31;
    // Blocks of at most 192 pixels: pack as many whole blocks into the tile as fit, but never so many
    // that fewer than four items per SM remain (small launches keep one block per item).
    // The gather gains at every size (more bytes in flight per SM); the scatter up to about 100
    // pixels (measured, of copy bandwidth: 5x5 fp32 0.27 -> 0.80, 8x8 0.62 -> 0.80, 10x10 0.76 -> 0.80,
    // but 12x12 0.88 -> 0.75), so larger blocks keep one block per scatter item.
    p.blocksPerItem = 1;
    if (!pch && (mode == kGather || P <= 100)) {
        long long perSm = (long long)a.numActive * p.cChunks.div / ((long long)sm_count() * 4);
        if (options().tileBlocks > 0)   // tests: pack up to this many blocks regardless of the launch size
            perSm = options().tileBlocks;
        // what fits: 384 pixels, and (rows rounded up to words) 384/EPW words per tile row
        const long long fit = std::min<long long>(kPsMaxPixels / P, (kPsMaxPixels / epw) / p.units);
        const long long k = std::min<long long>(std::min<long long>(fit, kPsThreads), perSm);
        if (k >= 2)
            p.blocksPerItem = (int)k;
    }
    const bool multi = p.blocksPerItem > 1;
    // Gathers of at most 384 pixels per block are fed by TMA where possible (planes_tma.cu: same tile,
    // one TMA load per block instead of plain loads; measured +3 % on one-block tiles, up to +20 % on
    // shared tiles).  The `planes` option set to 2 (SBNET_PLANES=tile) keeps the plain-load kernel (A/B measurements, tests).
    if (mode == kGather) {
        if (options().planes != 2) {
            if (cudaError_t e = pch ? launch_gather_tma_rows(a, dtype, stream, taken)
                                    : launch_gather_tma_tile(a, dtype, p.blocksPerItem, stream, taken))
                return e;
            if (*taken)
                return cudaSuccess;
        }
    }
    if (dynGather)
        return cudaSuccess;   // the plain-load gather needs the count at launch
    p.pixelsDiv = FastDiv((uint32_t)P);
    p.unitsDiv = FastDiv((uint32_t)std::max(p.units, 1));
    const int lastGroups = p.groups - 8 * ((int)p.cChunks.div - 1);
    p.runVecs = FastDiv((uint32_t)(8 * P));
    p.runVecsLast = FastDiv((uint32_t)(lastGroups * P));
    if (multi)
        p.pitchWords = (p.blocksPerItem * p.units + 31) & ~31;
    const long long nItems = multi ? (long long)((a.numActive + p.blocksPerItem - 1) / p.blocksPerItem) * p.cChunks.div
                                   : (long long)a.numActive * p.cChunks.div * p.pChunks.div;
    if (nItems > 0x7fffffffll)
        return cudaSuccess;
    note_site("launch of a planes_simt kernel");
    unsigned grid = (unsigned)nItems;
    if (a.num_active_dev != nullptr) {   // count on the device: one resident wave strides over the items
        const long long wave = (long long)sm_count() * 3;
        grid = (unsigned)(nItems < wave ? nItems : wave);
    }
#define SBNET_PS(KERNEL) launch_pdl(KERNEL, dim3(grid), dim3(kPsThreads), 0, stream, a, p)
    const int shape = pch ? kTileChunked : (multi ? kTileMulti : kTileSingle);
#define SBNET_PS_G(T_)                                                \
    do {                                                              \
        if (shape == kTileChunked)                                    \
            SBNET_PS((planes_gather_simt<T_, kTileChunked>));         \
        else if (shape == kTileMulti)                                 \
            SBNET_PS((planes_gather_simt<T_, kTileMulti>));           \
        else                                                          \
            SBNET_PS((planes_gather_simt<T_, kTileSingle>));          \
    } while (0)
#define SBNET_PS_SG(M, T_, GW_)                                       \
    do {                                                              \
        if (shape == kTileChunked)                                    \
            SBNET_PS((planes_scatter_simt<M, T_, GW_, kTileChunked>)); \
        else if (shape == kTileMulti)                                 \
            SBNET_PS((planes_scatter_simt<M, T_, GW_, kTileMulti>));  \
        else                                                          \
            SBNET_PS((planes_scatter_simt<M, T_, GW_, kTileSingle>)); \
    } while (0)
#define SBNET_PS_SC(M, T_)                                            \
    do {                                                              \
        if (gw == 4)                                                  \
            SBNET_PS_SG(M, T_, 4);                                    \
        else if (gw == 2)                                             \
            SBNET_PS_SG(M, T_, 2);                                    \
        else if (shape == kTileMulti)                                 \
            SBNET_PS((planes_scatter_simt<M, T_, 1, kTileMulti>));    \
        else                                                          \
            SBNET_PS((planes_scatter_simt<M, T_, 1, kTileSingle>));   \
    } while (0)
    if (mode == kGather) {
        if (dtype == 0)
            SBNET_PS_G(float);
        else if (odd && multi)
            SBNET_PS((planes_gather_simt<__half, kTileMulti, true>));
        else if (odd && !pch)
            SBNET_PS((planes_gather_simt<__half, kTileSingle, true>));
        else
            SBNET_PS_G(__half);
    } else if (odd) {
#define SBNET_PS_ODD(M, T_)                                           \
    do {                                                              \
        if (multi)                                                    \
            SBNET_PS((planes_scatter_simt<M, T_, 0, kTileMulti>));    \
        else                                                          \
            SBNET_PS((planes_scatter_simt<M, T_, 0, kTileSingle>));   \
    } while (0)
        if (mode == kScatterSet)
            SBNET_PS_ODD(kScatterSet, __half);
        else if (dtype == 2)
            SBNET_PS_ODD(kScatterAtomic, __nv_bfloat16);
        else
            SBNET_PS_ODD(kScatterAtomic, __half);
#undef SBNET_PS_ODD
    } else if (dtype == 2) {
        SBNET_PS_SC(kScatterAtomic, __nv_bfloat16);   // gather / overwrite arrive as fp16
    } else if (dtype == 0) {
        if (mode == kScatterSet)
            SBNET_PS_SC(kScatterSet, float);
        else if (mode == kScatterAdd)
            SBNET_PS_SC(kScatterAdd, float);
        else
            SBNET_PS_SC(kScatterAtomic, float);
    } else {
        if (mode == kScatterSet)
            SBNET_PS_SC(kScatterSet, __half);
        else
            SBNET_PS_SC(kScatterAtomic, __half);   // fp16 add arrives as a reduction
    }
#undef SBNET_PS_SC
#undef SBNET_PS_SG
#undef SBNET_PS_G
#undef SBNET_PS
    *taken = true;
    return cudaGetLastError();
}

} // namespace sbnet
