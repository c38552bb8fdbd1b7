/*
 * A plain C99 consumer of the C ABI: no Python, no C++, no framework -- device memory from the CUDA runtime,
 * the library through its header, the result checked against the CPU checker (oracle/sbnet_oracle.c, linked in
 * by the test that builds this file).  It is what a host in any language with a C FFI does: the mask -> gather ->
 * per-block work -> scatter sequence of one sparse layer, in both stack layouts, with the host-count and the
 * device-count entry points.  Prints "PASS" and returns 0, or says what differed.
 */
#include <cuda_runtime_api.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "sbnet_b200.h"

void oracle_reduce_mask_op(const float* mask, int N, int H, int W, float threshold, int bOffsH0, int bOffsW0, int bSzH,
                           int bSzW, int bStrH, int bStrW, int bCntH, int bCntW, int16_t* activeBlockIndices,
                           int32_t* binCounts, int avgPool);
void oracle_sparse_gather_f32(const float* x, int N, int H, int W, int C, float* y, int bOffsH0, int bOffsW0, int bSzH,
                              int bSzW, int bStrH, int bStrW, int numActive, const int16_t* idx, int transpose);
void oracle_sparse_scatter_f32(const float* x, int N, int H, int W, int C, float* y, int bOffsH0, int bOffsW0, int bSzH,
                               int bSzW, int bStrH, int bStrW, int numActive, const int16_t* idx, int add, int transpose,
                               int atomic);

#define CUDA_OK(call)                                                                         \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess) {                                                              \
            fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_));                       \
            return 2;                                                                         \
        }                                                                                     \
    } while (0)
#define SBNET_OK_(call)                                                                       \
    do {                                                                                      \
        int rc_ = (call);                                                                     \
        if (rc_ != SBNET_OK) {                                                                \
            fprintf(stderr, "%s -> %d: %s\n", #call, rc_, sbnet_last_error());                \
            return 3;                                                                         \
        }                                                                                     \
    } while (0)

static uint32_t g_seed = 12345u;
static float rnd(void)   /* uniform in [-1, 1), the same sequence on every run */
{
    g_seed = g_seed * 1664525u + 1013904223u;
    return (float)(g_seed >> 8) / 8388608.0f - 1.0f;
}

static int cmp_triples(const void* a, const void* b)
{
    return memcmp(a, b, 3 * sizeof(int16_t));
}

int main(void)
{
    enum { N = 2, H = 40, W = 36, C = 12, BS = 10, STR = 8, OFF = -1, BCH = 5, BCW = 5, MAXB = N * BCH * BCW };
    const size_t nImg = (size_t)N * H * W * C, nBlk = (size_t)BS * BS * C;
    float* mask = (float*)calloc((size_t)N * H * W, sizeof(float));
    float* x = (float*)malloc(nImg * sizeof(float));
    float* stack = (float*)malloc(MAXB * nBlk * sizeof(float));
    float* expect = (float*)malloc(MAXB * nBlk * sizeof(float));
    float* y = (float*)malloc(nImg * sizeof(float));
    float* yExpect = (float*)malloc(nImg * sizeof(float));
    int16_t idx[MAXB * 3], idxExpect[MAXB * 3];
    int32_t count = -1, countExpect = -1;
    for (size_t i = 0; i < nImg; ++i)
        x[i] = rnd();
    for (int n = 0; n < N; ++n)   /* two rectangles per image, one touching a corner */
        for (int h = 0; h < H; ++h)
            for (int w = 0; w < W; ++w)
                mask[((size_t)n * H + h) * W + w] = ((h < 9 && w < 7 + 5 * n) || (h > 20 + n && h < 31 && w > 17 && w < 30)) ? 1.0f : 0.0f;

    float *dMask, *dX, *dStack, *dY;
    int16_t* dIdx;
    int32_t* dScratch;
    CUDA_OK(cudaMalloc((void**)&dMask, (size_t)N * H * W * sizeof(float)));
    CUDA_OK(cudaMalloc((void**)&dX, nImg * sizeof(float)));
    CUDA_OK(cudaMalloc((void**)&dY, nImg * sizeof(float)));
    CUDA_OK(cudaMalloc((void**)&dStack, MAXB * nBlk * sizeof(float)));
    CUDA_OK(cudaMalloc((void**)&dIdx, sizeof(idx)));
    CUDA_OK(cudaMalloc((void**)&dScratch, 4 * sizeof(int32_t)));
    CUDA_OK(cudaMemcpy(dMask, mask, (size_t)N * H * W * sizeof(float), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dX, x, nImg * sizeof(float), cudaMemcpyHostToDevice));
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));

    /* reduce_mask: the count comes back in host memory, the index list stays on the device */
    SBNET_OK_(sbnet_reduce_mask(dMask, N, H, W, 0.5f, 0, OFF, OFF, BS, BS, STR, STR, BCH, BCW, dIdx, dScratch, &count, 0, stream));
    CUDA_OK(cudaMemcpy(idx, dIdx, sizeof(idx), cudaMemcpyDeviceToHost));
    oracle_reduce_mask_op(mask, N, H, W, 0.5f, OFF, OFF, BS, BS, STR, STR, BCH, BCW, idxExpect, &countExpect, 0);
    if (count != countExpect || count < 4) {
        fprintf(stderr, "count %d, expected %d\n", count, countExpect);
        return 1;
    }
    qsort(idx, (size_t)count, 3 * sizeof(int16_t), cmp_triples);
    qsort(idxExpect, (size_t)count, 3 * sizeof(int16_t), cmp_triples);
    if (memcmp(idx, idxExpect, (size_t)count * 3 * sizeof(int16_t)) != 0) {
        fprintf(stderr, "index lists differ\n");
        return 1;
    }
    CUDA_OK(cudaMemcpy(idx, dIdx, sizeof(idx), cudaMemcpyDeviceToHost));   /* the device's own order from here on */

    for (int transpose = 0; transpose < 2; ++transpose) {
        for (int dyn = 0; dyn < 2; ++dyn) {
            /* gather; the device-count variant reads the count reduce_mask left in scratch word 0 */
            CUDA_OK(cudaMemsetAsync(dStack, 0xff, MAXB * nBlk * sizeof(float), stream));
            if (dyn)
                SBNET_OK_(sbnet_sparse_gather_dyn(dX, SBNET_F32, N, H, W, C, dStack, OFF, OFF, BS, BS, STR, STR, MAXB,
                                                  dScratch, dIdx, transpose, stream));
            else
                SBNET_OK_(sbnet_sparse_gather(dX, SBNET_F32, N, H, W, C, dStack, OFF, OFF, BS, BS, STR, STR, count, dIdx,
                                              transpose, stream));
            CUDA_OK(cudaMemcpyAsync(stack, dStack, (size_t)count * nBlk * sizeof(float), cudaMemcpyDeviceToHost, stream));
            CUDA_OK(cudaStreamSynchronize(stream));
            oracle_sparse_gather_f32(x, N, H, W, C, expect, OFF, OFF, BS, BS, STR, STR, count, idx, transpose);
            if (memcmp(stack, expect, (size_t)count * nBlk * sizeof(float)) != 0) {
                fprintf(stderr, "gather differs (transpose %d, device count %d)\n", transpose, dyn);
                return 1;
            }
            /* the layer's own work on the stack (here: halve it), then accumulate it back over the halos */
            for (size_t i = 0; i < (size_t)count * nBlk; ++i)
                stack[i] *= 0.5f;
            CUDA_OK(cudaMemcpyAsync(dStack, stack, (size_t)count * nBlk * sizeof(float), cudaMemcpyHostToDevice, stream));
            SBNET_OK_(sbnet_copy_tensor(dY, dX, nImg * sizeof(float), stream));
            if (dyn)
                SBNET_OK_(sbnet_sparse_scatter_dyn(dStack, SBNET_F32, N, H, W, C, dY, OFF, OFF, BS, BS, STR, STR, MAXB,
                                                   dScratch, dIdx, 1, transpose, 1, stream));
            else
                SBNET_OK_(sbnet_sparse_scatter(dStack, SBNET_F32, N, H, W, C, dY, OFF, OFF, BS, BS, STR, STR, count, dIdx, 1,
                                               transpose, 1, stream));
            CUDA_OK(cudaMemcpyAsync(y, dY, nImg * sizeof(float), cudaMemcpyDeviceToHost, stream));
            CUDA_OK(cudaStreamSynchronize(stream));
            memcpy(yExpect, x, nImg * sizeof(float));
            oracle_sparse_scatter_f32(stack, N, H, W, C, yExpect, OFF, OFF, BS, BS, STR, STR, count, idx, 1, transpose, 1);
            /* overlapping halos: up to four addends per element in an order the schedule picks */
            for (size_t i = 0; i < nImg; ++i) {
                const float d = y[i] - yExpect[i], tol = 4.0f * 1.2e-7f * 4.0f;   /* 4 additions of values below 4 */
                if (d > tol || d < -tol) {
                    fprintf(stderr, "scatter differs at %zu: %g vs %g (transpose %d, device count %d)\n", i, y[i],
                            yExpect[i], transpose, dyn);
                    return 1;
                }
            }
        }
    }
    unsigned int timeouts = 1;
    SBNET_OK_(sbnet_wait_timeouts(&timeouts));
    if (timeouts != 0) {
        fprintf(stderr, "%u bounded waits gave up\n", timeouts);
        return 1;
    }
    /* an argument the reference rejects as InvalidArgument comes back as a negative status, not as a crash */
    if (sbnet_sparse_scatter(dStack, SBNET_F32, N, H, W, C, dY, OFF, OFF, BS, BS, STR, STR, count, dIdx, 1, 0, 0, stream) >= 0) {
        fprintf(stderr, "overlapping add without atomics was accepted\n");
        return 1;
    }
    printf("PASS %d blocks, library version %d\n", count, sbnet_version());
    return 0;
}
