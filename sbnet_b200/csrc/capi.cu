// The C ABI (include/sbnet_b200.h): argument checks the reference performs in its OpKernels
// (sbnet_ops/reduce_mask.cc:132-138, sbnet_ops/sparse_gather.cc:164,173,322-327), then the launch.
#include <limits.h>
#include <stdarg.h>
#include <stdio.h>
#include <sched.h>
#include <time.h>

#include "../../include/sbnet_b200.h"
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "options.h"

#define SBNET_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

thread_local char g_err[320] = "";
thread_local const char* g_site = "";
constexpr int32_t kCountSentinel = SBNET_COUNT_PENDING;

int reject(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

inline int cuda_status(cudaError_t e)
{
    if (e != cudaSuccess)
        snprintf(g_err, sizeof(g_err), "CUDA error %d: %s%s%s", (int)e, cudaGetErrorString(e), g_site[0] ? " at " : "",
                 g_site);
    return (int)e;
}

// Geometry limits shared by all ops: positive sizes/strides and every pixel coordinate inside 31 bits.
int check_geometry(const char* op, int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH, int bStrW,
                   long long maxBlockH, long long maxBlockW)
{
    if (bSzH < 1 || bSzW < 1)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: block size must be positive, got [%d, %d]", op,
                      bSzH, bSzW);
    if (bStrH < 1 || bStrW < 1)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: block stride must be positive, got [%d, %d]",
                      op, bStrH, bStrW);
    const long long lim = 1ll << 30;
    const long long absH = bOffsH < 0 ? -(long long)bOffsH : bOffsH;
    const long long absW = bOffsW < 0 ? -(long long)bOffsW : bOffsW;
    if (absH + maxBlockH * bStrH + bSzH >= lim || absW + maxBlockW * bStrW + bSzW >= lim ||
        (long long)bSzH * bSzW >= lim)
        return reject(SBNET_ERR_UNSUPPORTED, "%s: block geometry exceeds 2^30 pixels", op);
    return SBNET_OK;
}

int blocks_call(const char* op, int mode, int dtype, int N, int H, int W, int C,
                void* image, void* stack, int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH,
                int bStrW, int numActive, const int32_t* numActiveDev, const int16_t* idx,
                int transpose, void* stream)
{
    g_site = "";
    if (dtype != SBNET_F32 && dtype != SBNET_F16 && dtype != SBNET_BF16)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: unknown dtype %d", op, dtype);
    if (N < 1 || H < 1 || W < 1 || C < 1)
        return reject(SBNET_ERR_INVALID_ARGUMENT,
                      "%s: tensor must be rank 4 with positive dimensions, got [%d, %d, %d, %d]", op,
                      N, H, W, C);
    if (numActive < 0)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: negative block count %d", op, numActive);
    if (int rc = check_geometry(op, bOffsH, bOffsW, bSzH, bSzW, bStrH, bStrW, 32767, 32767))
        return rc;
    if (numActive == 0)
        return SBNET_OK;
    if (image == nullptr || stack == nullptr || idx == nullptr)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: null tensor pointer", op);
    // a pointer off its element's boundary would be a misaligned access on the device, not an error code
    const uintptr_t elem = dtype == SBNET_F32 ? 4 : 2;
    if (((reinterpret_cast<uintptr_t>(image) | reinterpret_cast<uintptr_t>(stack)) & (elem - 1)) != 0 ||
        (reinterpret_cast<uintptr_t>(idx) & 1) != 0 || (reinterpret_cast<uintptr_t>(numActiveDev) & 3) != 0)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: tensor pointer not aligned to its element size", op);
    const long long lim = 1ll << 31;
    const long long blockElems = (long long)bSzH * bSzW * C;
    const long long chunks = ((long long)C * 4 + 127) / 128;
    if (blockElems >= lim || (long long)numActive * bSzH >= lim ||
        (long long)numActive * chunks * ((long long)bSzH * bSzW / 128 + 1) >= lim)
        return reject(SBNET_ERR_UNSUPPORTED, "%s: more than 2^31 work items", op);

    sbnet::BlockArgs a;
    a.image = image, a.stack = stack, a.idx = idx, a.num_active_dev = numActiveDev;
    a.numActive = numActive, a.N = N, a.H = H, a.W = W, a.C = C;
    a.bOffsH = bOffsH, a.bOffsW = bOffsW, a.bSzH = bSzH, a.bSzW = bSzW, a.bStrH = bStrH,
    a.bStrW = bStrW;
    return cuda_status(sbnet::launch_blocks(a, dtype, mode, transpose != 0, (cudaStream_t)stream));
}

int scatter_mode(const char* op, int add, int atomic, int bSzH, int bSzW, int bStrH, int bStrW,
                 int* mode)
{
    if (add && !atomic && !(bStrH >= bSzH && bStrW >= bSzW))
        return reject(SBNET_ERR_INVALID_ARGUMENT,
                      "%s: Only non-overlapping blocks are supported with add=True, atomic=False", op);
    *mode = !add ? sbnet::kScatterSet : (atomic ? sbnet::kScatterAtomic : sbnet::kScatterAdd);
    return SBNET_OK;
}

} // namespace

namespace sbnet {
// Lets other translation units of the library report through sbnet_last_error().
void set_last_error(const char* text) { snprintf(g_err, sizeof(g_err), "%s", text); }
void note_site(const char* site) { g_site = site; }

static int env_number(const char* name, int dflt)
{
    const char* v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

Options& options()
{
    static Options opt;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* planes = getenv("SBNET_PLANES");
        opt.planes = (planes && planes[0] == 't') ? (planes[1] == 'i' ? 2 : 1) : env_number("SBNET_PLANES", 0);   // tma | tile | 0..5
        opt.disableTma = env_number("SBNET_DISABLE_TMA", 0) == 1;
        opt.tileBlocks = env_number("SBNET_TILE_BLOCKS", 0);
        opt.rmKernel = env_number("SBNET_RM_KERNEL", 0);
        opt.rmCtasPerSm = env_number("SBNET_RM_CTAS_PER_SM", 8);
        opt.rmResident = env_number("SBNET_RM_RESIDENT", 0);
        opt.pdl = env_number("SBNET_PDL", 1);
        opt.tmaL2 = env_number("SBNET_TMA_L2", 3);
    });
    return opt;
}
} // namespace sbnet

namespace {
struct OptionName {
    const char* name;
    int sbnet::Options::*field;
};
const OptionName kOptionNames[] = {
    {"planes", &sbnet::Options::planes},          {"disable_tma", &sbnet::Options::disableTma},
    {"tile_blocks", &sbnet::Options::tileBlocks}, {"rm_kernel", &sbnet::Options::rmKernel},
    {"rm_ctas_per_sm", &sbnet::Options::rmCtasPerSm}, {"pdl", &sbnet::Options::pdl},
    {"rm_resident", &sbnet::Options::rmResident},
    {"tma_l2", &sbnet::Options::tmaL2},
};
} // namespace

SBNET_EXPORT int sbnet_set_option(const char* name, int value)
{
    for (const OptionName& o : kOptionNames)
        if (name != nullptr && strcmp(name, o.name) == 0) {
            sbnet::options().*(o.field) = value;
            return SBNET_OK;
        }
    return reject(SBNET_ERR_INVALID_ARGUMENT, "sbnet_set_option: unknown option '%s'", name ? name : "(null)");
}

SBNET_EXPORT int sbnet_get_option(const char* name, int* value)
{
    for (const OptionName& o : kOptionNames)
        if (name != nullptr && value != nullptr && strcmp(name, o.name) == 0) {
            *value = sbnet::options().*(o.field);
            return SBNET_OK;
        }
    return reject(SBNET_ERR_INVALID_ARGUMENT, "sbnet_get_option: unknown option '%s'", name ? name : "(null)");
}

SBNET_EXPORT int sbnet_version(void) { return 100; }

SBNET_EXPORT const char* sbnet_last_error(void) { return g_err; }

SBNET_EXPORT int sbnet_reduce_mask(const float* mask, int N, int H, int W, float tol, int avgpool,
                                   int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH, int bStrW,
                                   int bCntH, int bCntW, int16_t* active_block_indices,
                                   int32_t* scratch_dev, int32_t* count_host, int flags,
                                   void* stream)
{
    const char* op = "ReduceMask";
    if (N < 1 || H < 1 || W < 1)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: mask must be [N,H,W,1] with positive dimensions, "
                      "got [%d, %d, %d]", op, N, H, W);
    if (bCntH < 1 || bCntW < 1)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: block counts must be positive, got [%d, %d]", op,
                      bCntH, bCntW);
    if (N > 32767 || bCntH > 32767 || bCntW > 32767)
        return reject(SBNET_ERR_INVALID_ARGUMENT,
                      "%s: N, bCntH and bCntW must fit the int16 index triples (<= 32767), got %d, %d, %d",
                      op, N, bCntH, bCntW);
    if ((long long)N * bCntH * bCntW >= (1ll << 31))
        return reject(SBNET_ERR_UNSUPPORTED, "%s: N*bCntH*bCntW = %lld candidate blocks do not fit the int32 count",
                      op, (long long)N * bCntH * bCntW);
    if (int rc = check_geometry(op, bOffsH, bOffsW, bSzH, bSzW, bStrH, bStrW, bCntH, bCntW))
        return rc;
    if (mask == nullptr || active_block_indices == nullptr || scratch_dev == nullptr)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: null tensor pointer", op);
    if (reinterpret_cast<uintptr_t>(scratch_dev) & 15)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: scratch_dev must be 16-byte aligned", op);
    if ((reinterpret_cast<uintptr_t>(mask) & 3) != 0 || (reinterpret_cast<uintptr_t>(active_block_indices) & 1) != 0)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: tensor pointer not aligned to its element size", op);

    cudaStream_t s = (cudaStream_t)stream;
    int32_t* hostDev = nullptr;   // device-visible alias of count_host when it is pinned
    if (count_host != nullptr) {
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, count_host) == cudaSuccess &&
            attr.type == cudaMemoryTypeHost && attr.devicePointer != nullptr)
            hostDev = static_cast<int32_t*>(attr.devicePointer);
        else
            (void)cudaGetLastError();
    }
    if ((flags & SBNET_COUNT_NOWAIT) && hostDev == nullptr)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "%s: SBNET_COUNT_NOWAIT needs count_host in pinned host memory", op);
    if (hostDev != nullptr && (flags & (SBNET_COUNT_POLL | SBNET_COUNT_NOWAIT)))
        *count_host = kCountSentinel;
    if (!(flags & SBNET_SCRATCH_CLEAN))
        if (cudaError_t e = cudaMemsetAsync(scratch_dev, 0, sizeof(int32_t) * SBNET_REDUCE_MASK_SCRATCH_INTS, s))
            return cuda_status(e);
    if (cudaError_t e = sbnet::launch_reduce_mask(mask, N, H, W, tol, avgpool != 0, bOffsH, bOffsW, bSzH,
                                                  bSzW, bStrH, bStrW, bCntH, bCntW,
                                                  active_block_indices, scratch_dev, hostDev,
                                                  (flags & SBNET_MASK_STABLE) != 0, s))
        return cuda_status(e);
    if (count_host != nullptr && !(flags & SBNET_COUNT_NOWAIT)) {
        if (hostDev != nullptr && (flags & SBNET_COUNT_POLL)) {
            // The kernel stores the count straight into pinned memory: watching that word is several
            // times quicker than putting the thread to sleep in a stream synchronisation.  A count is
            // never negative, so the sentinel written before the launch cannot be mistaken for one.
            volatile int32_t* word = count_host;
            timespec t0;
            clock_gettime(CLOCK_MONOTONIC, &t0);
            const bool yield = (flags & SBNET_COUNT_YIELD) != 0;
            for (unsigned spins = 0; *word == kCountSentinel; ++spins) {
                if (yield)
                    sched_yield();   // several such threads (one per GPU) may share this core
                if (yield || (spins & 1023u) == 1023u) {
                    timespec t1;
                    clock_gettime(CLOCK_MONOTONIC, &t1);
                    if ((t1.tv_sec - t0.tv_sec) * 1000000000ll + (t1.tv_nsec - t0.tv_nsec) > 200000000ll)
                        break;   // 0.2 s: let the runtime wait (and report a failed launch, if any)
                }
            }
            if (*word != kCountSentinel)
                return SBNET_OK;
        }
        if (hostDev == nullptr)
            if (cudaError_t e = cudaMemcpyAsync(count_host, scratch_dev, sizeof(int32_t),
                                                cudaMemcpyDeviceToHost, s))
                return cuda_status(e);
        if (cudaError_t e = cudaStreamSynchronize(s))
            return cuda_status(e);
    }
    return SBNET_OK;
}

SBNET_EXPORT int sbnet_sparse_gather(const void* x, int dtype, int N, int H, int W, int C, void* y,
                                     int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH,
                                     int bStrW, int numActive, const int16_t* active_block_indices,
                                     int transpose, void* stream)
{
    return blocks_call("SparseGather", sbnet::kGather, dtype, N, H, W, C, const_cast<void*>(x), y,
                       bOffsH, bOffsW, bSzH, bSzW, bStrH, bStrW, numActive, nullptr,
                       active_block_indices, transpose, stream);
}

SBNET_EXPORT int sbnet_sparse_gather_dyn(const void* x, int dtype, int N, int H, int W, int C,
                                         void* y, int bOffsH, int bOffsW, int bSzH, int bSzW,
                                         int bStrH, int bStrW, int maxActive,
                                         const int32_t* num_active_dev,
                                         const int16_t* active_block_indices, int transpose,
                                         void* stream)
{
    if (num_active_dev == nullptr)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "SparseGather: num_active_dev is null");
    return blocks_call("SparseGather", sbnet::kGather, dtype, N, H, W, C, const_cast<void*>(x), y,
                       bOffsH, bOffsW, bSzH, bSzW, bStrH, bStrW, maxActive, num_active_dev,
                       active_block_indices, transpose, stream);
}

SBNET_EXPORT int sbnet_sparse_scatter(const void* x, int dtype, int N, int H, int W, int C, void* y,
                                      int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH,
                                      int bStrW, int numActive, const int16_t* active_block_indices,
                                      int add, int transpose, int atomic, void* stream)
{
    int mode = 0;
    if (int rc = scatter_mode("SparseScatter", add, atomic, bSzH, bSzW, bStrH, bStrW, &mode))
        return rc;
    return blocks_call("SparseScatter", mode, dtype, N, H, W, C, y, const_cast<void*>(x), bOffsH,
                       bOffsW, bSzH, bSzW, bStrH, bStrW, numActive, nullptr, active_block_indices,
                       transpose, stream);
}

SBNET_EXPORT int sbnet_sparse_scatter_dyn(const void* x, int dtype, int N, int H, int W, int C,
                                          void* y, int bOffsH, int bOffsW, int bSzH, int bSzW,
                                          int bStrH, int bStrW, int maxActive,
                                          const int32_t* num_active_dev,
                                          const int16_t* active_block_indices, int add,
                                          int transpose, int atomic, void* stream)
{
    int mode = 0;
    if (num_active_dev == nullptr)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "SparseScatter: num_active_dev is null");
    if (int rc = scatter_mode("SparseScatter", add, atomic, bSzH, bSzW, bStrH, bStrW, &mode))
        return rc;
    return blocks_call("SparseScatter", mode, dtype, N, H, W, C, y, const_cast<void*>(x), bOffsH,
                       bOffsW, bSzH, bSzW, bStrH, bStrW, maxActive, num_active_dev,
                       active_block_indices, transpose, stream);
}

SBNET_EXPORT int sbnet_copy_tensor(void* dst, const void* src, size_t bytes, void* stream)
{
    if (bytes != 0 && (dst == nullptr || src == nullptr))
        return reject(SBNET_ERR_INVALID_ARGUMENT, "CopyTensor: null pointer");
    return cuda_status(sbnet::launch_copy(dst, src, bytes, (cudaStream_t)stream));
}

SBNET_EXPORT int sbnet_cuda_timer_start(int64_t* handle)
{
    if (handle == nullptr)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "CudaTimerStart: null handle");
    cudaEvent_t ev;
    if (cudaError_t e = cudaEventCreate(&ev))
        return cuda_status(e);
    if (cudaError_t e = cudaEventRecord(ev, 0)) {
        cudaEventDestroy(ev);
        return cuda_status(e);
    }
    *handle = (int64_t)reinterpret_cast<intptr_t>(ev);
    return SBNET_OK;
}

SBNET_EXPORT int sbnet_cuda_timer_end(int64_t handle, float* elapsed_ms)
{
    if (handle == 0 || elapsed_ms == nullptr)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "CudaTimerEnd: null handle or output");
    cudaEvent_t start = reinterpret_cast<cudaEvent_t>((intptr_t)handle), stop;
    if (cudaError_t e = cudaEventCreate(&stop))
        return cuda_status(e);
    cudaError_t e = cudaEventRecord(stop, 0);
    if (e == cudaSuccess)
        e = cudaEventSynchronize(stop);
    if (e == cudaSuccess)
        e = cudaEventElapsedTime(elapsed_ms, start, stop);
    cudaEventDestroy(stop);
    cudaEventDestroy(start);
    return cuda_status(e);
}

SBNET_EXPORT int sbnet_wait_timeouts(unsigned int* count)
{
    if (count == nullptr)
        return reject(SBNET_ERR_INVALID_ARGUMENT, "sbnet_wait_timeouts: null output");
    unsigned int planes = 0, mask = 0, rows = 0;
    if (cudaError_t e = sbnet::read_wait_timeouts(&planes))
        return cuda_status(e);
    if (cudaError_t e = sbnet::read_rm_wait_timeouts(&mask))
        return cuda_status(e);
    if (cudaError_t e = sbnet::read_rows_wait_timeouts(&rows))
        return cuda_status(e);
    *count = planes + mask + rows;
    return SBNET_OK;
}
