// Device helpers shared by the kernels: streaming 128-bit loads, warp reductions.
#ifndef BPL_CSRC_COMMON_CUH_
#define BPL_CSRC_COMMON_CUH_

#include <cstdint>
#include <cuda_runtime.h>

namespace bpl {

constexpr unsigned FULL_MASK = 0xffffffffu;

// 128-bit read-only load that bypasses L1 allocation: matrix entries are touched once per call.
__device__ __forceinline__ uint4 ldg_stream_u4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ldg_stream_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ uint2 ldg_stream_u2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

template<typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL_MASK, v, o);
    return v;
}

// Sum inside aligned groups of `width` lanes (width a power of two <= 32, uniform in the warp).
template<typename T>
__device__ __forceinline__ T group_sum(T v, int width) {
    for (int o = width >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(FULL_MASK, v, o);
    return v;
}

// Truthiness of one event element, as `if (x[i])` in the reference kernels
// (lib/gpu_event_csr_matvec.cu:65,88): bool as is, floating point != 0 (NaN is truthy).
__device__ __forceinline__ bool is_event(bool e) { return e; }
__device__ __forceinline__ bool is_event(uint8_t e) { return e != 0; }
__device__ __forceinline__ bool is_event(float e) { return e != 0.0f; }
__device__ __forceinline__ bool is_event(double e) { return e != 0.0; }

}  // namespace bpl

#endif  // BPL_CSRC_COMMON_CUH_
