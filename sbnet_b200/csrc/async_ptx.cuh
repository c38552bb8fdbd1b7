// Thin wrappers over the PTX used by the TMA-fed kernels: shared-memory accesses by 32-bit
// shared-space address, bulk (TMA engine) copies in both directions, mbarriers with bounded waits,
// and the programmatic-dependent-launch controls.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace sbnet {

constexpr long long kWaitCycles = 1ll << 31;        // bound of every mbarrier wait: ~1.1 s at 1.9 GHz

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void bulk_store_1d(void* dst, uint32_t src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// The same copy without closing the group: several copies, then one bulk_commit().
__device__ __forceinline__ void bulk_store_1d_nocommit(void* dst, uint32_t src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes)
                 : "memory");
}
// dst[i] += src[i] for every element of the run, each an addition performed in L2 (round to nearest even,
// 16-bit types without flushing subnormals), like red.global.add.  Both addresses 16-byte aligned, size a
// multiple of 16 bytes.  T: float, __half or __nv_bfloat16.
template <typename T> __device__ __forceinline__ void bulk_reduce_add_1d(void* dst, uint32_t src, uint32_t bytes);
template <> __device__ __forceinline__ void bulk_reduce_add_1d<float>(void* dst, uint32_t src, uint32_t bytes)
{
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst), "r"(src),
                 "r"(bytes)
                 : "memory");
}
template <> __device__ __forceinline__ void bulk_reduce_add_1d<__half>(void* dst, uint32_t src, uint32_t bytes)
{
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.f16 [%0], [%1], %2;" ::"l"(dst),
                 "r"(src), "r"(bytes)
                 : "memory");
}
template <> __device__ __forceinline__ void bulk_reduce_add_1d<__nv_bfloat16>(void* dst, uint32_t src, uint32_t bytes)
{
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.bf16 [%0], [%1], %2;" ::"l"(dst),
                 "r"(src), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int N> __device__ __forceinline__ void bulk_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void bulk_wait_all()
{
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

__device__ __forceinline__ void fence_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v)
{
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// 16-bit accesses (plane rows of an odd number of halves start on odd half boundaries)
__device__ __forceinline__ uint32_t lds16(uint32_t addr)
{
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ void sts16(uint32_t addr, uint32_t v)
{
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v) : "memory");
}

__device__ __forceinline__ void sts128(uint32_t addr, uint4 v)
{
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// ---- mbarriers ----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  false: gave up (or another role of this CTA did): the CTA-wide abort flag is then
// set and the wait has counted itself in *timeouts (a __device__ counter of the calling file).
static __device__ __noinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abortFlag,
                                               unsigned int* timeouts)
{
    const long long t0 = clock64();
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((i & 31u) == 31u) {
            if (*abortFlag)
                return false;
            if (clock64() - t0 > kWaitCycles)
                break;
        }
    }
    atomicAdd(timeouts, 1u);
    *abortFlag = 1;
    return false;
}

// ---- loads through the TMA engine (this GPU's memory only; never multicast) -----------------------
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            int c3, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
        : "memory");
}
// Untiled bulk copy: both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// ---- in-place transposition of a swizzled tile -----------------------------------------------------
// Task t of a tile's transposition -> (16-byte channel group j, word column u); 128 tasks cover 16
// word columns x 8 groups.  A quarter warp's eight 16-byte reads of the [pixel][128 B] tile (groups
// XOR-swizzled by pixel & 7) are conflict-free when they hit eight different groups.  32-bit elements:
// word column u is pixel u, so eight neighbouring columns of one group do.  16-bit elements: word
// column u is the pixel pair (2u, 2u+1), whose swizzle phases are all even (or all odd) -- four
// values only -- so every eight lanes pair two channel groups with four columns instead.
template <int EPW> __device__ __forceinline__ void transpose_task(int t, int& j, int& u)
{
    if constexpr (EPW == 2) {
        j = (t & 1) | (((t >> 5) & 3) << 1);
        u = ((t >> 7) << 4) + ((t >> 1) & 15);
    } else {
        j = (t >> 4) & 7;
        u = ((t >> 7) << 4) + (t & 15);
    }
}

// ---- programmatic dependent launch ----------------------------------------------------------------
// wait: blocks until the kernel this one was launched behind (with the programmatic-serialization
// attribute) has completed and its writes are visible; a no-op for an ordinary launch.
__device__ __forceinline__ void pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// launch_dependents: lets a kernel queued behind this one with that attribute start its prologue
// once every CTA of this grid has passed this point; a no-op when nothing of the kind is queued.
__device__ __forceinline__ void pdl_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

} // namespace sbnet
