/*
 * sbnet_b200 -- C ABI of the B200 (sm_100a) implementation of SBNet's block ops.
 *
 * Every entry point replaces one seam of the reference library (paths below are relative to
 * sbnet_tensorflow/sbnet_ops/ of uber-research/sbnet).  A TensorFlow OpKernel (or any other host)
 * calls these with raw device pointers exactly where the reference's Compute() methods call their
 * functors (the repository's integration notes show the binding).
 *
 * Conventions
 *  - All tensor pointers are DEVICE pointers unless a parameter says "host".  The caller owns every
 *    buffer; the library allocates nothing.  A tensor pointer must be a multiple of its element size
 *    (rejected otherwise); beyond that any alignment is served, wider alignment by faster kernels.
 *  - Geometry is passed as in the reference functors: offsets may be negative, strides may be
 *    smaller (overlap) or larger (gaps) than sizes, blocks may hang over any image border.
 *  - `stream` is a cudaStream_t passed as void*.  Work is enqueued on it; only sbnet_reduce_mask with
 *    a non-NULL count_host waits for it.
 *  - Return value: 0 = success; negative = SBNET_ERR_* (the argument was rejected, nothing was
 *    launched; sbnet_last_error() has the text); positive = a cudaError_t from the CUDA runtime.
 *    The library never terminates the process (the reference calls exit(), op_utils.h:27-37).
 *  - Threads and streams: calls may be made from several host threads and on several streams at once
 *    as long as they do not share scratch or output buffers.  State the library keeps: per-thread
 *    caches (the last error text, the last few TMA tensor maps -- keyed by base address, shape and
 *    element size, so a buffer freed and re-allocated at the same address with the same shape reuses
 *    a still-valid map -- and which kernels already had their shared-memory limit raised); per-device
 *    caches (SM count, resolved address of the static scratch); three device-side counters of bounded
 *    waits that gave up (sbnet_wait_timeouts); the process-wide option table (sbnet_set_option), which
 *    is initialised from the environment once, at first use; and the fixed scratch array of
 *    sbnet_reduce_mask_static, which all calls of that one entry point on a GPU share.
 *  - A call that returns 0 has enqueued its work.  The TMA-fed kernels bound their waits on
 *    shared-memory barriers; should one ever give up, the kernel returns early, the output is
 *    incomplete and sbnet_wait_timeouts() reports it -- success of the launch does not imply that.
 */
#ifndef SBNET_B200_H
#define SBNET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SBNET_OK 0
#define SBNET_ERR_INVALID_ARGUMENT (-1) /* maps to tensorflow::errors::InvalidArgument */
#define SBNET_ERR_UNSUPPORTED (-2)      /* valid but outside what the kernels index (>= 2^31 items) */

/* element types of x / y / block stacks */
#define SBNET_F32 0
#define SBNET_F16 1 /* extension: the reference registers T = float only (sparse_gather.cc:49) */
#define SBNET_BF16 2 /* extension: bfloat16; accumulation rounds to nearest even once per add, no flush */

/* sbnet_reduce_mask flags */
#define SBNET_SCRATCH_CLEAN 1 /* scratch[2..3] are already zero (see below): skip the memset */
#define SBNET_COUNT_POLL 2    /* pinned count_host: return as soon as the count has arrived (see below) */
#define SBNET_MASK_STABLE 4   /* the mask is not written by the operation queued just before this call on
                                 `stream`: its loads may overlap the tail of that operation (see below) */
#define SBNET_COUNT_YIELD 8   /* with SBNET_COUNT_POLL: give the core away between looks at the count */
#define SBNET_COUNT_NOWAIT 16 /* pinned count_host: return right after the launch; the word reads
                                 SBNET_COUNT_PENDING until the kernel has stored the count (see below) */
#define SBNET_COUNT_PENDING INT32_MIN

/* int32 words of device scratch sbnet_reduce_mask needs */
#define SBNET_REDUCE_MASK_SCRATCH_INTS 4

int sbnet_version(void);

/* Text of the last SBNET_ERR_* returned on the calling thread ("" if none). */
const char* sbnet_last_error(void);

/*
 * ReduceMask -- replaces ReduceMaskFunctor<GPUDevice,T>::operator() (reduce_mask.h:23-44, launcher
 * reduce_mask.cu:39-88, kernels reduce_mask.cu.h:54-188 and zero_block_counters.cu.h:26-51) plus the
 * count read-back and empty-mask rule of ReduceMaskOp::Compute (reduce_mask.cc:198-220).
 *
 *   mask                  [N,H,W] (or [N,H,W,1]) fp32
 *   tol, avgpool          op attrs: a block is active if any pixel > tol (max) or
 *                         sum(in-range pixels)/(bSzH*bSzW) > tol (avg)
 *   active_block_indices  [N*bCntH*bCntW, 3] int16 (n, bh, bw); the first count rows are written,
 *                         in arbitrary order
 *   scratch_dev           SBNET_REDUCE_MASK_SCRATCH_INTS int32, 16-byte aligned.  On return (stream
 *                         order) scratch_dev[0] holds the published count, which device-side
 *                         consumers (the *_dyn entry points) may read without a host round trip;
 *                         scratch_dev[2..3] are internal and are left at zero.  Pass
 *                         SBNET_SCRATCH_CLEAN in `flags` when the buffer was zero-filled once and has
 *                         since only been used by stream-ordered calls of this function; otherwise
 *                         the library clears it with a cudaMemsetAsync first.
 *   count_host            host int32 (the op's bin_counts output, reduce_mask.cc:198-220) or NULL.
 *                         When given, the call synchronises `stream` and stores the count.  Pinned
 *                         host memory is written directly by the kernel; pageable memory costs an
 *                         extra copy.  With SBNET_COUNT_POLL (pinned memory only) the call watches that
 *                         word instead of synchronising the stream and returns as soon as the count is
 *                         there: the kernel's last index writes may still be in flight, but they are
 *                         ordered before anything enqueued on `stream` afterwards (use an event or a
 *                         stream synchronisation before reading the indices from another stream).
 *                         The poll spins on one core for at most 0.2 s; SBNET_COUNT_YIELD makes it call
 *                         sched_yield() between looks (for hosts that run one such thread per GPU on
 *                         shared cores).  An empty result is reported as ONE block with index (0,0,0),
 *                         as the reference does.
 *   SBNET_COUNT_NOWAIT    (pinned memory only; other memory is rejected) the call stores SBNET_COUNT_PENDING
 *                         in *count_host, enqueues the kernel and returns; the kernel stores the count
 *                         (never negative) there when it is done, and the host looks when it needs it --
 *                         a loop that issues the next masks ahead never blocks on a count.
 *   SBNET_MASK_STABLE     every kernel of the library is launched with programmatic stream serialization:
 *                         its CTAs may become resident while the kernel queued before it on `stream`
 *                         drains, and touch global memory only once that kernel has completed.  With this
 *                         flag reduce_mask reads the MASK before that point as well (scratch_dev and
 *                         active_block_indices still wait), which is only correct when the mask is not
 *                         produced by that preceding kernel (e.g. the previous layer's scatter precedes,
 *                         and the mask has been resident for longer).
 *   Limits                N, bCntH, bCntW <= 32767 (int16 triples); N*bCntH*bCntW < 2^31 (int32 count),
 *                         larger products are rejected with SBNET_ERR_UNSUPPORTED.
 */
int sbnet_reduce_mask(const float* mask, int N, int H, int W, float tol, int avgpool,
                      int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH, int bStrW,
                      int bCntH, int bCntW, int16_t* active_block_indices, int32_t* scratch_dev,
                      int32_t* count_host, int flags, void* stream);

/*
 * SparseGather -- replaces SparseGatherFunctor<GPUDevice,T>::operator() (sparse_gather.h:23-41,
 * launcher sparse_gather.cu:62-154, kernels sparse_blocks.cu.h:68-172,292-347).
 *
 *   x  [N,H,W,C] NHWC;  y  [numActive,bSzH,bSzW,C], or [numActive,C,bSzH,bSzW] when transpose != 0.
 *   Pixels outside the image read as zero.  numActive == 0 is a successful no-op.
 *   dtype (here and below): SBNET_F32, SBNET_F16 or SBNET_BF16, the element type of x and y.
 */
int sbnet_sparse_gather(const void* x, int dtype, int N, int H, int W, int C, void* y,
                        int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH, int bStrW,
                        int numActive, const int16_t* active_block_indices, int transpose,
                        void* stream);

/*
 * SparseScatter / SparseScatterVar -- replaces SparseScatterFunctor<GPUDevice,T>::operator()
 * (sparse_gather.h:43-65, launcher sparse_gather.cu:158-266, kernels sparse_blocks.cu.h:174-289,
 * 309-366) and the argument rule of SparseScatterOp::Compute (sparse_gather.cc:322-326).
 *
 *   x  block stack ([numActive,bSzH,bSzW,C] or transposed [numActive,C,bSzH,bSzW]);
 *   y  [N,H,W,C], updated in place: y = x (add == 0), y += x (add != 0).  Pixels outside the image
 *   are dropped.  add != 0 with atomic == 0 requires disjoint blocks (bStr >= bSz in both
 *   dimensions) and is rejected with SBNET_ERR_INVALID_ARGUMENT otherwise; atomic != 0 uses vector
 *   reductions and accepts any overlap.  With add == 0 and overlapping blocks the surviving value
 *   of a shared pixel is whichever block wrote last (as in the reference).
 *   The non-Var op is sbnet_copy_tensor(y, ybase) followed by this call on the same stream.
 */
int sbnet_sparse_scatter(const void* x, int dtype, int N, int H, int W, int C, void* y,
                         int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH, int bStrW,
                         int numActive, const int16_t* active_block_indices, int add,
                         int transpose, int atomic, void* stream);

/*
 * Device-count variants (no counterpart in the reference, whose op interface forces a host read of
 * bin_counts between reduce_mask and gather, reduce_mask.cc:204 / sparse_gather.cc:190-192):
 * the number of blocks is read on the device from *num_active_dev (e.g. scratch_dev of
 * sbnet_reduce_mask) and clamped to maxActive, so mask -> gather -> scatter can be enqueued without
 * a host synchronisation.  Buffers must be sized for maxActive blocks.
 */
int sbnet_sparse_gather_dyn(const void* x, int dtype, int N, int H, int W, int C, void* y,
                            int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH, int bStrW,
                            int maxActive, const int32_t* num_active_dev,
                            const int16_t* active_block_indices, int transpose, void* stream);
int sbnet_sparse_scatter_dyn(const void* x, int dtype, int N, int H, int W, int C, void* y,
                             int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH, int bStrW,
                             int maxActive, const int32_t* num_active_dev,
                             const int16_t* active_block_indices, int add, int transpose,
                             int atomic, void* stream);

/*
 * CopyTensor -- replaces CopyTensorFunctor<GPUDevice,T>::operator() (sparse_gather.h:68-76,
 * sparse_gather.cu:268-276): dst[0..bytes) = src[0..bytes), stream ordered, WITHOUT the
 * reference's cudaStreamSynchronize.  The size is in bytes (the reference's int element count
 * overflows past 2^31 elements).
 */
int sbnet_copy_tensor(void* dst, const void* src, size_t bytes, void* stream);

/*
 * CudaTimerStart / CudaTimerEnd -- replace the two timing ops (sparse_gather.cc:390-466): start
 * records an event on the legacy default stream and returns its handle; end records a second
 * event, waits for it, returns the elapsed milliseconds and destroys both events.
 */
int sbnet_cuda_timer_start(int64_t* handle);
int sbnet_cuda_timer_end(int64_t handle, float* elapsed_ms);

/*
 * Diagnostic with no counterpart in the reference: the TMA-pipelined kernels bound every wait on a
 * shared-memory barrier (about a second); a wait that gives up makes its thread block drain and
 * return, and is counted here.  *count stays 0 in a healthy process; a non-zero value means some
 * output was left incomplete.  Synchronises the device.
 */
int sbnet_wait_timeouts(unsigned int* count);

/*
 * Process-wide switches (no counterpart in the reference), for A/B measurements and for tests that
 * push one input through every kernel family.  Initialised once from the environment variables in
 * brackets; afterwards only these calls change them.  Not synchronised with launches in flight on other
 * threads.  Unknown names are rejected with SBNET_ERR_INVALID_ARGUMENT.
 *   "planes"          0 default dispatch, 1 persistent TMA pipeline, 2 tile CTAs with plain loads [SBNET_PLANES=tma|tile],
 *                     3 tile CTAs fed by TMA whatever the launch size, 4 general shapes on the element-wise / narrow-vector
 *                     kernels instead of the raw-row kernel,
 *                     6 general shapes on the raw-row kernel with element-wide accesses on the stack side
 *   "disable_tma"     1: plane layouts run the general kernel only                               [SBNET_DISABLE_TMA]
 *   "tile_blocks"     > 0: small blocks sharing one tile, whatever the launch size               [SBNET_TILE_BLOCKS]
 *   "rm_kernel"       reduce_mask: 0 default, 1 register-fed band kernel, 2 one thread per block  [SBNET_RM_KERNEL]
 *   "rm_ctas_per_sm"  reduce_mask: CTAs per SM the column tiling aims at (default 8)             [SBNET_RM_CTAS_PER_SM]
 *   "rm_resident"     reduce_mask: at most this many CTAs resident per SM, 0 = no cap            [SBNET_RM_RESIDENT]
 *   "pdl"             0: launch kernels without programmatic stream serialization (default 1)    [SBNET_PDL]
 *   "tma_l2"          L2 promotion of image tensor maps: 0 none, 1 64 B, 2 128 B, 3 256 B (default) [SBNET_TMA_L2]
 */
int sbnet_set_option(const char* name, int value);
int sbnet_get_option(const char* name, int* value);

/*
 * ReduceMask without caller-provided scratch.  No counterpart in the reference.
 *
 * For hosts that cannot give the library device memory of their own: a plug-in inside a framework
 * that has already reserved the whole GPU for its memory pool (a plain cudaMalloc fails there), code
 * in a section where allocation calls are not allowed, or a thin C wrapper with no allocator.  Same
 * result as sbnet_reduce_mask; the cursor / ticket words live in a fixed SBNET_STATIC_SCRATCH_BYTES
 * array inside the library's device image (one per GPU that loads the library, held until exit).
 *
 *   count_dev   optional DEVICE int32 that receives the published count in stream order (what
 *               scratch_dev[0] is for sbnet_reduce_mask); count_host as in sbnet_reduce_mask.
 *
 * Limits and rules: N*bCntH*bCntW must not exceed SBNET_STATIC_MAX_BLOCKS (rejected with
 * SBNET_ERR_INVALID_ARGUMENT otherwise).  All calls on one GPU share the array: calls whose kernels
 * can overlap (different streams or threads without ordering) race; the words that must start at zero
 * are cleared on `stream` at the start of every call, so a previous call's leftovers never leak.
 * The first call on each GPU resolves the array's device address (not a stream operation): make it
 * before any stream capture.  The function and everything it calls allocate nothing.
 */
#define SBNET_STATIC_SCRATCH_BYTES 256
#define SBNET_STATIC_MAX_BLOCKS (1 << 24)
int sbnet_reduce_mask_static(const float* mask, int N, int H, int W, float tol, int avgpool,
                             int bOffsH, int bOffsW, int bSzH, int bSzW, int bStrH, int bStrW,
                             int bCntH, int bCntW, int16_t* active_block_indices, int32_t* count_dev,
                             int32_t* count_host, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SBNET_B200_H */
