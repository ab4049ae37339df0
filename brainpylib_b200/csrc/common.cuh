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

// Programmatic dependent launch (scan -> scatter pairs): the scan lets its dependents start as soon as it runs, the
// scatter does everything that needs no input from the scan (clearing its shared memory) and then waits here until
// the scan has completed and its writes are visible.  In a kernel that was launched the ordinary way the wait returns
// at once.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch of a kernel that may start before the kernel in front of it on the stream has finished (it must call
// pdl_wait() before it touches anything that kernel writes).
template<typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Reduction without a return value (one L2 operation, nothing travels back), spelled out so that no
// call site can turn into the value-returning form.
__device__ __forceinline__ void red_add(float *p, float v) {
    asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" :: "l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void red_add(double *p, double v) {
    asm volatile("red.relaxed.gpu.global.add.f64 [%0], %1;" :: "l"(p), "d"(v) : "memory");
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

// Packs the truthiness of n events into a bitmask (bit i of word i / 32 = event i) held in shared
// memory, cooperatively by the whole block.  Where the event array is 16-byte aligned each lane reads
// 16 bytes at a time (16 bools, 4 floats or 2 doubles), so a block needs one or two rounds of loads
// even for a million events; the unaligned case and the ragged end use one ballot per 32 events.
template<typename E>
__device__ __forceinline__ void pack_event_mask(const E *__restrict__ x, const uint32_t n, uint32_t *mask) {
    constexpr uint32_t PER_LANE = 16 / sizeof(E);          // events per 128-bit load
    constexpr uint32_t SPAN = 32 * PER_LANE;               // events per warp-wide load
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    const uint32_t n_vec = vec_ok ? (n / SPAN) * SPAN : 0u;
    for (uint32_t base = warp * SPAN; base < n_vec; base += n_warps * SPAN) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(x + base + lane * PER_LANE);
        const E *e = reinterpret_cast<const E *>(&raw);
        uint32_t bits = 0;
#pragma unroll
        for (uint32_t k = 0; k < PER_LANE; ++k) bits |= (is_event(e[k]) ? 1u : 0u) << k;
        // PER_LANE bits per lane -> 32 / PER_LANE lanes make one word
        constexpr uint32_t LANES_PER_WORD = 32 / PER_LANE;
        uint32_t word = bits << (PER_LANE * (lane % LANES_PER_WORD));
#pragma unroll
        for (uint32_t o = 1; o < LANES_PER_WORD; o <<= 1) word |= __shfl_xor_sync(FULL_MASK, word, o);
        if (lane % LANES_PER_WORD == 0) mask[base / 32 + lane / LANES_PER_WORD] = word;
    }
    const uint32_t n_words = (n + 31u) >> 5;
    for (uint32_t w = n_vec / 32 + warp; w < n_words; w += n_warps) {
        const uint32_t i = w * 32u + lane;
        const uint32_t bits = __ballot_sync(FULL_MASK, (i < n) && is_event(x[i]));
        if (lane == 0) mask[w] = bits;
    }
}

}  // namespace bpl

#endif  // BPL_CSRC_COMMON_CUH_
