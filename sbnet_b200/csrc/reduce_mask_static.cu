// sbnet_reduce_mask_static: reduce_mask for callers that cannot hand the library any device scratch.
//
// The ordinary entry point, sbnet_reduce_mask, needs a few words of device memory for its append
// cursor and finish ticket, and the caller has to allocate them.  Some hosts cannot: a plug-in that
// runs inside a framework which has already claimed the whole GPU for its own memory pool (a raw
// cudaMalloc there fails, and the plug-in is not handed the framework's allocator), code that runs in
// a section where the driver's allocation calls are forbidden (e.g. a latency-critical loop that
// pins down all memory at start-up), or a thin C wrapper with no allocator of its own.  For them the
// scratch lives in a fixed array inside this library's device image.
//
// Consequences a caller must know:
//  * The array exists once per GPU that loads this library and stays until the process exits.
//  * ALL calls on one GPU share it.  Two calls whose kernels overlap in time (different streams,
//    different host threads) race on it and corrupt each other's counts; order them on one stream or
//    with events.  The array keeps whatever the last call left there, so the words that must start
//    at zero are cleared on the caller's stream at the start of every call.
//  * The first call on each GPU looks up the array's device address (a host-side symbol is only a
//    stand-in; the kernel is given the address the runtime reports).  That look-up is not a stream
//    operation: make the first call on a device before any stream capture begins.
//  * Nothing is allocated here or in anything this function calls: no cudaMalloc / cudaFree, no
//    library routine that allocates.
#include <mutex>
#include <stdio.h>

#include "../../include/sbnet_b200.h"
#include "kernels.h"

#define SBNET_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kMaxDevices = 64;

// One 256-byte line; the kernel uses the first SBNET_REDUCE_MASK_SCRATCH_INTS words
// ([0] published count, [2..3] the 64-bit cursor|ticket word).
static __device__ __align__(256) int32_t g_static_scratch[SBNET_STATIC_SCRATCH_BYTES / sizeof(int32_t)];

static int32_t* g_scratch_addr[kMaxDevices] = {nullptr};
static std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device, resolved once per device.
cudaError_t scratch_for_current_device(int32_t** out)
{
    int dev = -1;
    if (cudaError_t e = cudaGetDevice(&dev))
        return e;
    if (dev < 0 || dev >= kMaxDevices)
        return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        int32_t* ptr = nullptr;
        if (cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch))
            return e;
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return cudaSuccess;
}

} // namespace

SBNET_EXPORT int sbnet_reduce_mask_static(const float* mask, int N, int H, int W, float tol, int avgpool,
                                          int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH,
                                          int bStrW, int bCntH, int bCntW,
                                          int16_t* active_block_indices, int32_t* count_dev,
                                          int32_t* count_host, void* stream)
{
    char msg[256];
    // The 32-bit cursor kept in the fixed scratch counts candidate blocks; this variant states its
    // limit instead of inheriting the int16 bound of the index triples.
    // each factor is bounded first (the int16 index triples allow no more), so the product cannot overflow
    const bool factorsOk = N >= 1 && bCntH >= 1 && bCntW >= 1 && N <= 32767 && bCntH <= 32767 && bCntW <= 32767;
    const long long candidates = factorsOk ? (long long)N * bCntH * bCntW : -1;
    if (!factorsOk || candidates > (long long)SBNET_STATIC_MAX_BLOCKS) {
        snprintf(msg, sizeof(msg),
                 "ReduceMask (static scratch): N, bCntH, bCntW = %d, %d, %d must each lie in 1..32767 and their "
                 "product must not exceed %d, the most this entry point's fixed scratch is specified for",
                 N, bCntH, bCntW, SBNET_STATIC_MAX_BLOCKS);
        sbnet::set_last_error(msg);
        return SBNET_ERR_INVALID_ARGUMENT;
    }
    if (static_cast<size_t>(SBNET_REDUCE_MASK_SCRATCH_INTS) * sizeof(int32_t) > SBNET_STATIC_SCRATCH_BYTES) {
        sbnet::set_last_error("ReduceMask (static scratch): scratch array too small");
        return SBNET_ERR_UNSUPPORTED;
    }
    int32_t* scratch = nullptr;
    if (cudaError_t e = scratch_for_current_device(&scratch)) {
        snprintf(msg, sizeof(msg), "CUDA error %d resolving the scratch array: %s", (int)e,
                 cudaGetErrorString(e));
        sbnet::set_last_error(msg);
        return (int)e;
    }
    // flags = 0: the ordinary entry point clears the scratch words on `stream` (cudaMemsetAsync) before
    // its kernel, which is exactly the "start from zero" this shared array needs on every call.
    const int rc = sbnet_reduce_mask(mask, N, H, W, tol, avgpool, bOffsH, bOffsW, bSzH, bSzW, bStrH, bStrW,
                                     bCntH, bCntW, active_block_indices, scratch, count_host, 0, stream);
    if (rc != SBNET_OK)
        return rc;   // sbnet_last_error() already describes it
    if (count_dev != nullptr) {   // hand the published count to the caller's own device word
        if (cudaError_t e = cudaMemcpyAsync(count_dev, scratch, sizeof(int32_t), cudaMemcpyDeviceToDevice,
                                            (cudaStream_t)stream)) {
            snprintf(msg, sizeof(msg), "CUDA error %d copying the count: %s", (int)e, cudaGetErrorString(e));
            sbnet::set_last_error(msg);
            return (int)e;
        }
    }
    return SBNET_OK;
}
