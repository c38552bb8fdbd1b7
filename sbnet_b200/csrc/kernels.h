// Launchers behind the C ABI (internal; the public surface is include/sbnet_b200.h).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sbnet {

struct BlockArgs;

// scratch: 4 x int32 on the device; [2] and [3] must be zero on entry and are zero again on exit.
// maskStable: the mask is not written by the operation queued just before this call on `stream`.
cudaError_t launch_reduce_mask(const float* mask, int N, int H, int W, float tol, bool avgpool,
                               int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH, int bStrW,
                               int bCntH, int bCntW, int16_t* idx, int32_t* scratch,
                               int32_t* host_count_dev, bool maskStable, cudaStream_t stream);
cudaError_t read_rm_wait_timeouts(unsigned int* out);

// mode: 0 gather, 1 scatter overwrite, 2 scatter add (disjoint blocks), 3 scatter atomic add
cudaError_t launch_blocks(const BlockArgs& a, int dtype, int mode, bool transpose,
                          cudaStream_t stream);
cudaError_t read_rows_wait_timeouts(unsigned int* out);   // bounded waits of the raw-row plane kernel that gave up

// Plane-layout fast path (TMA pipeline); *taken tells whether it accepted the call.
cudaError_t launch_planes_tma(const BlockArgs& a, int dtype, int mode, cudaStream_t stream, bool* taken);

// Same shapes as launch_planes_tma, one short CTA per tile; host-side block count only.
cudaError_t launch_planes_simt(const BlockArgs& a, int dtype, int mode, cudaStream_t stream, bool* taken);
cudaError_t launch_gather_tma_rows(const BlockArgs& a, int dtype, cudaStream_t stream, bool* taken);
cudaError_t launch_gather_tma_tile(const BlockArgs& a, int dtype, int blocksPerItem, cudaStream_t stream, bool* taken);
bool planes_tma_eligible(const BlockArgs& a, int itemsize);

// Bounded device-side waits that gave up since the library was loaded (0 in a healthy process).
cudaError_t read_wait_timeouts(unsigned int* out);

cudaError_t launch_copy(void* dst, const void* src, size_t bytes, cudaStream_t stream);

int sm_count();

// Sets the calling thread's sbnet_last_error() text.
void set_last_error(const char* text);

// Names the runtime call a launcher is about to make; a CUDA error reported by the C ABI carries the
// last name noted on the calling thread.
void note_site(const char* site);

} // namespace sbnet
