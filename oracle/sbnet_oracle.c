/*
 * CPU oracle for the SBNet block ops.  TEST INFRASTRUCTURE ONLY: this file is the checker the
 * parity tests, the smoke test and the benchmark's CPU-baseline leg compare the CUDA library
 * against.  Nothing in the product library links, loads or calls it.
 *
 * It restates, in plain C, the arithmetic of the reference's CPU functors
 * (sbnet_tensorflow/sbnet_ops):
 *   oracle_reduce_mask      <- ReduceMaskFunctor<CPUDevice,T>      reduce_mask.cc:46-98
 *   oracle_reduce_mask_op   <- + ReduceMaskOp::Compute fix-up      reduce_mask.cc:203-220
 *   oracle_sparse_gather_*  <- SparseGatherFunctor<CPUDevice,T>    sparse_gather.cc:61-90
 *   oracle_sparse_scatter_* <- SparseScatterFunctor<CPUDevice,T>   sparse_gather.cc:94-132
 *   oracle_copy_tensor      <- CopyTensorFunctor<CPUDevice,T>      sparse_gather.cc:135-142
 *
 * Parity pin: tests/test_oracle_pins.py checks this file against (a) the known answers the
 * reference's own tests hold (empty mask => one block (0,0,0); the hand-written 5x5 expected output
 * of reduce_mask -> gather -> 3x3 ones conv -> scatter), (b) the reference's CPU functors compiled
 * unchanged from the reference tree (oracle/Makefile target `ref`) when that build is present, and
 * (c) committed golden vectors generated from that compiled reference (tests/golden/).
 *
 * Everything is sequential by default: the scatter-add order is then the block-list order, which
 * makes overlapping-halo sums reproducible.  oracle_set_threads(n) spreads blocks over n OpenMP
 * threads for gather and for scatter with disjoint blocks (stride >= size); overlapping scatter
 * always stays on one thread.  (The reference instead threads over blocks and takes one global lock
 * per added element, sparse_gather.cc:100-125; results are the same up to fp add order.)
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

static int g_threads = 1;

ORACLE_API void oracle_set_threads(int n) { g_threads = n < 1 ? 1 : n; }

ORACLE_API int oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* reduce_mask.cc:66-96.  Blocks are visited in (n, bh, bw) lexicographic order; the window is
 * clipped to the image; max mode is "any pixel strictly above the threshold"; average mode sums the
 * in-range pixels in row-major order in fp32 and divides by the FULL block area. */
ORACLE_API void oracle_reduce_mask(const float* mask, int N, int H, int W, float threshold,
                                   int bOffsH0, int bOffsW0, int bSzH, int bSzW, int bStrH,
                                   int bStrW, int bCntH, int bCntW, int16_t* activeBlockIndices,
                                   int32_t* binCounts, int avgPool)
{
    int count = 0;
    for (int n = 0; n < N; ++n)
        for (int bh = 0; bh < bCntH; ++bh)
            for (int bw = 0; bw < bCntW; ++bw) {
                const int h0 = bOffsH0 + bh * bStrH;
                const int w0 = bOffsW0 + bw * bStrW;
                const int hBeg = h0 > 0 ? h0 : 0, wBeg = w0 > 0 ? w0 : 0;
                int active = 0;
                float sum = 0.0f;
                for (int hh = hBeg; hh < h0 + bSzH && hh < H; ++hh)
                    for (int ww = wBeg; ww < w0 + bSzW && ww < W; ++ww) {
                        const float val = mask[((size_t)n * H + hh) * W + ww];
                        if (avgPool)
                            sum += val;
                        else
                            active |= (val > threshold);
                    }
                if (avgPool)
                    active = (sum / (bSzH * bSzW)) > threshold;
                if (active) {
                    activeBlockIndices[count * 3 + 0] = (int16_t)n;
                    activeBlockIndices[count * 3 + 1] = (int16_t)bh;
                    activeBlockIndices[count * 3 + 2] = (int16_t)bw;
                    count++;
                }
            }
    binCounts[0] = count;
}

/* reduce_mask.cc:203-220: an empty result is reported as ONE block with index (0,0,0). */
ORACLE_API void oracle_reduce_mask_op(const float* mask, int N, int H, int W, float threshold,
                                      int bOffsH0, int bOffsW0, int bSzH, int bSzW, int bStrH,
                                      int bStrW, int bCntH, int bCntW, int16_t* activeBlockIndices,
                                      int32_t* binCounts, int avgPool)
{
    oracle_reduce_mask(mask, N, H, W, threshold, bOffsH0, bOffsW0, bSzH, bSzW, bStrH, bStrW, bCntH,
                       bCntW, activeBlockIndices, binCounts, avgPool);
    if (binCounts[0] == 0) {
        activeBlockIndices[0] = activeBlockIndices[1] = activeBlockIndices[2] = 0;
        binCounts[0] = 1;
    }
}

/* sparse_gather.cc:66-89 (gather) and :102-129 (scatter), generated per element type. */
#define DEFINE_GATHER_SCATTER(SUFFIX, T)                                                           \
    ORACLE_API void oracle_sparse_gather_##SUFFIX(                                                 \
        const T* x, int N, int H, int W, int C, T* y, int bOffsH0, int bOffsW0, int bSzH,          \
        int bSzW, int bStrH, int bStrW, int numActive, const int16_t* idx, int transpose)          \
    {                                                                                              \
        (void)N;                                                                                   \
        const size_t R = (size_t)bSzH, S = (size_t)bSzW, CC = (size_t)C;                           \
        _Pragma("omp parallel for num_threads(g_threads) schedule(static)")                        \
        for (int ib = 0; ib < numActive; ib++) {                                                   \
            const int biN = idx[ib * 3 + 0];                                                       \
            const int h0 = bOffsH0 + idx[ib * 3 + 1] * bStrH;                                      \
            const int w0 = bOffsW0 + idx[ib * 3 + 2] * bStrW;                                      \
            T* yb = y + (size_t)ib * R * S * CC;                                                   \
            for (size_t r = 0; r < R; ++r)                                                         \
                for (size_t s = 0; s < S; ++s) {                                                   \
                    const int hh = h0 + (int)r, ww = w0 + (int)s;                                  \
                    const int inside = hh >= 0 && ww >= 0 && hh < H && ww < W;                     \
                    const T* px = inside ? x + (((size_t)biN * H + hh) * W + ww) * CC : NULL;      \
                    for (size_t c = 0; c < CC; ++c) {                                              \
                        const T v = inside ? px[c] : (T)0.0f;                                      \
                        if (transpose)                                                             \
                            yb[c * R * S + r * S + s] = v;                                         \
                        else                                                                       \
                            yb[(r * S + s) * CC + c] = v;                                          \
                    }                                                                              \
                }                                                                                  \
        }                                                                                          \
    }                                                                                              \
    static void scatter_block_##SUFFIX(const T* xb, int H, int W, size_t CC, T* y, int biN,        \
                                       int h0, int w0, size_t R, size_t S, int add, int transpose) \
    {                                                                                              \
        for (size_t r = 0; r < R; ++r)                                                             \
            for (size_t s = 0; s < S; ++s) {                                                       \
                const int hh = h0 + (int)r, ww = w0 + (int)s;                                      \
                if (!(hh >= 0 && ww >= 0 && hh < H && ww < W))                                     \
                    continue;                                                                      \
                T* py = y + (((size_t)biN * H + hh) * W + ww) * CC;                                \
                for (size_t c = 0; c < CC; ++c) {                                                  \
                    const T v = transpose ? xb[c * R * S + r * S + s] : xb[(r * S + s) * CC + c];  \
                    if (add)                                                                       \
                        py[c] += v;                                                                \
                    else                                                                           \
                        py[c] = v;                                                                 \
                }                                                                                  \
            }                                                                                      \
    }                                                                                              \
    ORACLE_API void oracle_sparse_scatter_##SUFFIX(                                                \
        const T* x, int N, int H, int W, int C, T* y, int bOffsH0, int bOffsW0, int bSzH,          \
        int bSzW, int bStrH, int bStrW, int numActive, const int16_t* idx, int add, int transpose, \
        int atomic)                                                                                \
    {                                                                                              \
        (void)N;                                                                                   \
        (void)atomic; /* ignored on the CPU, sparse_gather.cc:98 */                                \
        const size_t R = (size_t)bSzH, S = (size_t)bSzW, CC = (size_t)C;                           \
        /* Blocks may overlap when stride < size; adding (or overwriting with different values) */ \
        /* must then follow one fixed order, so only provably disjoint layouts run threaded. */    \
        const int disjoint = bStrH >= bSzH && bStrW >= bSzW;                                       \
        const int nthr = disjoint ? g_threads : 1;                                                 \
        _Pragma("omp parallel for num_threads(nthr) schedule(static)")                             \
        for (int ib = 0; ib < numActive; ib++) {                                                   \
            const int h0 = bOffsH0 + idx[ib * 3 + 1] * bStrH;                                      \
            const int w0 = bOffsW0 + idx[ib * 3 + 2] * bStrW;                                      \
            scatter_block_##SUFFIX(x + (size_t)ib * R * S * CC, H, W, CC, y, idx[ib * 3 + 0], h0,  \
                                   w0, R, S, add, transpose);                                      \
        }                                                                                          \
    }

DEFINE_GATHER_SCATTER(f32, float)
DEFINE_GATHER_SCATTER(f16, _Float16)
/* bfloat16: gcc evaluates `py[c] += v` as a float addition converted back with round-to-nearest-even */
DEFINE_GATHER_SCATTER(bf16, __bf16)

/* sparse_gather.cc:135-142 */
ORACLE_API void oracle_copy_tensor(void* dst, const void* src, size_t bytes)
{
    memcpy(dst, src, bytes);
}
