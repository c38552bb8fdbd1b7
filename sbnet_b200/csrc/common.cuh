// Shared device/host helpers for the block-op kernels (sm_100a only).
#pragma once
#include <type_traits>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "options.h"

namespace sbnet {

// Every kernel of the library is launched with programmatic stream serialization: its CTAs may become
// resident while the kernel queued before it on the stream drains, and they start their first global
// memory access only behind griddepcontrol.wait (pdl_wait(), async_ptx.cuh), i.e. once that kernel has
// completed and its writes are visible -- stream order as seen through memory is unchanged, the launch
// latency and the prologue are hidden.  The `pdl` option set to 0 launches the ordinary way.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = options().pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// ---- exact unsigned division by a runtime constant ----------------------------------------------
// q = n / d for 0 <= n < 2^31, 1 <= d < 2^31, with one mul.hi, one add and one shift.
// (Round-up multiplier: m = floor(2^32 * (2^s - d) / d) + 1 with s = ceil(log2 d); then
//  q = (mulhi(n, m) + n) >> s.  n < 2^31 keeps the sum inside 32 bits.)
struct FastDiv {
    uint32_t mul, shr, div;
    __host__ FastDiv() : mul(0), shr(0), div(1) {}
    __host__ explicit FastDiv(uint32_t d) : div(d)
    {
        uint32_t s = 0;
        while ((1ull << s) < d)
            ++s;
        shr = s;
        mul = (uint32_t)((((1ull << s) - d) << 32) / d + 1);
    }
    __host__ __device__ __forceinline__ uint32_t quot(uint32_t n) const
    {
#ifdef __CUDA_ARCH__
        return (__umulhi(n, mul) + n) >> shr;
#else
        return (uint32_t)((((uint64_t)n * mul) >> 32) + n) >> shr;
#endif
    }
    __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const
    {
        q = quot(n);
        r = n - q * div;
    }
};

// ---- plain-old-data vectors of 2..16 bytes ------------------------------------------------------
template <int BYTES> struct Vec;
template <> struct Vec<16> { typedef uint4 type; };
template <> struct Vec<8> { typedef uint2 type; };
template <> struct Vec<4> { typedef uint32_t type; };
template <> struct Vec<2> { typedef uint16_t type; };

template <int BYTES> __device__ __forceinline__ typename Vec<BYTES>::type vzero();
template <> __device__ __forceinline__ uint4 vzero<16>() { return make_uint4(0, 0, 0, 0); }
template <> __device__ __forceinline__ uint2 vzero<8>() { return make_uint2(0, 0); }
template <> __device__ __forceinline__ uint32_t vzero<4>() { return 0u; }
template <> __device__ __forceinline__ uint16_t vzero<2>() { return (uint16_t)0; }

// Streaming loads: every byte of the image and of the block stack is touched once per call, so
// neither side is worth keeping in L1.
__device__ __forceinline__ uint4 ld_stream(const uint4* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream(const uint2* p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint16_t ld_stream(const uint16_t* p)
{
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// ---- element-wise add on packed words -----------------------------------------------------------
template <typename T> __device__ __forceinline__ uint32_t add_word(uint32_t a, uint32_t b);
template <> __device__ __forceinline__ uint32_t add_word<float>(uint32_t a, uint32_t b)
{
    return __float_as_uint(__fadd_rn(__uint_as_float(a), __uint_as_float(b)));
}
template <> __device__ __forceinline__ uint32_t add_word<__half>(uint32_t a, uint32_t b)
{
    __half2 r = __hadd2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

template <> __device__ __forceinline__ uint32_t add_word<__nv_bfloat16>(uint32_t a, uint32_t b)
{
    __nv_bfloat162 r = __hadd2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

template <typename T> __device__ __forceinline__ uint4 vadd(uint4 a, uint4 b)
{
    return make_uint4(add_word<T>(a.x, b.x), add_word<T>(a.y, b.y), add_word<T>(a.z, b.z),
                      add_word<T>(a.w, b.w));
}
template <typename T> __device__ __forceinline__ uint2 vadd(uint2 a, uint2 b)
{
    return make_uint2(add_word<T>(a.x, b.x), add_word<T>(a.y, b.y));
}
template <typename T> __device__ __forceinline__ uint32_t vadd(uint32_t a, uint32_t b)
{
    return add_word<T>(a, b);
}
template <typename T> __device__ __forceinline__ uint16_t vadd(uint16_t a, uint16_t b)
{
    // only reachable for 2-byte element types (a 2-byte vector cannot hold a float)
    if constexpr (sizeof(T) == 2 && !std::is_same<T, __half>::value) {
        __nv_bfloat16 r = __hadd(__ushort_as_bfloat16(a), __ushort_as_bfloat16(b));
        return __bfloat16_as_ushort(r);
    } else {
        __half r = __hadd(__ushort_as_half(a), __ushort_as_half(b));
        return __half_as_ushort(r);
    }
}

// ---- vector reductions into global memory (no return value, resolved in L2) ----------------------
template <typename T> struct Red;
template <> struct Red<float> {
    static __device__ __forceinline__ void add(uint4* p, uint4 v)
    {
        asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(__uint_as_float(v.x)),
                     "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                     : "memory");
    }
    static __device__ __forceinline__ void add(uint2* p, uint2 v)
    {
        asm volatile("red.global.add.v2.f32 [%0], {%1,%2};" ::"l"(p), "f"(__uint_as_float(v.x)),
                     "f"(__uint_as_float(v.y))
                     : "memory");
    }
    static __device__ __forceinline__ void add(uint32_t* p, uint32_t v)
    {
        asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(__uint_as_float(v)) : "memory");
    }
    static __device__ __forceinline__ void add(uint16_t*, uint16_t) {}
};
template <> struct Red<__half> {
    static __device__ __forceinline__ void add(uint4* p, uint4 v)
    {
        asm volatile("red.global.add.noftz.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
                     "r"(v.z), "r"(v.w)
                     : "memory");
    }
    static __device__ __forceinline__ void add(uint2* p, uint2 v)
    {
        asm volatile("red.global.add.noftz.v2.f16x2 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y)
                     : "memory");
    }
    static __device__ __forceinline__ void add(uint32_t* p, uint32_t v)
    {
        asm volatile("red.global.add.noftz.f16x2 [%0], %1;" ::"l"(p), "r"(v) : "memory");
    }
    static __device__ __forceinline__ void add(uint16_t* p, uint16_t v)
    {
        asm volatile("red.global.add.noftz.f16 [%0], %1;" ::"l"(p), "h"(v) : "memory");
    }
};

template <> struct Red<__nv_bfloat16> {
    static __device__ __forceinline__ void add(uint4* p, uint4 v)
    {
        asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
                     "r"(v.z), "r"(v.w)
                     : "memory");
    }
    static __device__ __forceinline__ void add(uint2* p, uint2 v)
    {
        asm volatile("red.global.add.noftz.v2.bf16x2 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y)
                     : "memory");
    }
    static __device__ __forceinline__ void add(uint32_t* p, uint32_t v)
    {
        asm volatile("red.global.add.noftz.bf16x2 [%0], %1;" ::"l"(p), "r"(v) : "memory");
    }
    static __device__ __forceinline__ void add(uint16_t* p, uint16_t v)
    {
        asm volatile("red.global.add.noftz.bf16 [%0], %1;" ::"l"(p), "h"(v) : "memory");
    }
};

enum Mode : int { kGather = 0, kScatterSet = 1, kScatterAdd = 2, kScatterAtomic = 3 };

template <int VB> __device__ __forceinline__ typename Vec<VB>::type ld_plain(const typename Vec<VB>::type* p)
{
    return *p;
}

// Applies one vector to the image in the given scatter mode.
template <int VB, int MODE, typename T>
__device__ __forceinline__ void image_write(typename Vec<VB>::type* dst, typename Vec<VB>::type v,
                                            typename Vec<VB>::type old)
{
    if constexpr (MODE == kScatterSet)
        *dst = v;
    else if constexpr (MODE == kScatterAdd)
        *dst = vadd<T>(old, v);
    else
        Red<T>::add(dst, v);
}

// Geometry + buffers shared by the gather and scatter launches.  `image` is the NHWC tensor,
// `stack` the block stack ([nB,R,S,C], or [nB,C,R,S] when transposed).
struct BlockArgs {
    void* image;
    void* stack;
    const int16_t* idx;           // [numActive,3] (n, bh, bw)
    const int32_t* num_active_dev; // optional device-side count (nullptr: use numActive)
    int numActive;                // block count, or its upper bound when num_active_dev is set
    int N, H, W, C;
    int bOffsH, bOffsW, bSzH, bSzW, bStrH, bStrW;
};

} // namespace sbnet
