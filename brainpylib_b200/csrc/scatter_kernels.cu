// Legacy scatter operators of the `compat` API for sm_100a:
//   gpu_csr_event_sum_*   replaces lib/gpu_event_sum.cu:30-117   (one THREAD per row there)
//   gpu_coo_event_sum_*   replaces lib/gpu_event_sum.cu:122-206
//   gpu_coo_atomic_sum_*  replaces lib/gpu_atomic_sum.cu:27-97
//   gpu_coo_atomic_prod_* replaces lib/gpu_atomic_prod.cu:27-97  (the reference adds onto a
//                         byte-pattern memset; here the product is formed, starting from 1,
//                         as the reference's CPU kernel does, lib/cpu_atomic_prod.cc:6-43)
// Index type I is uint32 (`_i32`) or uint64 (`_i64`), as in the reference's instantiations.
#include "abi.h"
#include "common.cuh"

namespace bpl {
namespace {

constexpr int THREADS = 256;

template<typename T>
__global__ void fill_kernel(T *__restrict__ y, const uint32_t n, const T value) {
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<uint64_t>(gridDim.x) * blockDim.x)
        y[i] = value;
}

// one warp per pre-synaptic row; silent rows cost one byte load
template<typename T, typename I, bool HOMO>
__global__ void __launch_bounds__(THREADS)
csr_event_sum_kernel(const uint32_t pre_size, const bool *__restrict__ events, const I *__restrict__ indices,
                     const I *__restrict__ indptr, const T *__restrict__ values, T *__restrict__ y) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t n_warps = static_cast<uint64_t>(gridDim.x) * (THREADS / 32);
    const T w0 = values[0];
    for (uint64_t row = static_cast<uint64_t>(blockIdx.x) * (THREADS / 32) + (threadIdx.x >> 5); row < pre_size;
         row += n_warps) {
        if (!events[row]) continue;
        const I start = indptr[row], end = indptr[row + 1];
        for (I j = start + lane; j < end; j += 32) atomicAdd(y + indices[j], HOMO ? w0 : values[j]);
    }
}

template<typename T, typename I, bool HOMO>
__global__ void __launch_bounds__(THREADS)
coo_event_sum_kernel(const uint32_t size, const bool *__restrict__ events, const I *__restrict__ pre_ids,
                     const I *__restrict__ post_ids, const T *__restrict__ values, T *__restrict__ y) {
    const T w0 = values[0];
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * THREADS + threadIdx.x; i < size;
         i += static_cast<uint64_t>(gridDim.x) * THREADS)
        if (events[pre_ids[i]]) atomicAdd(y + post_ids[i], HOMO ? w0 : values[i]);
}

__device__ __forceinline__ void atomic_mul(float *addr, float v) {
    unsigned int *a = reinterpret_cast<unsigned int *>(addr);
    unsigned int old = *a, assumed;
    do {
        assumed = old;
        old = atomicCAS(a, assumed, __float_as_uint(__uint_as_float(assumed) * v));
    } while (assumed != old);   // integer comparison: terminates for NaN as well
}
__device__ __forceinline__ void atomic_mul(double *addr, double v) {
    unsigned long long *a = reinterpret_cast<unsigned long long *>(addr);
    unsigned long long old = *a, assumed;
    do {
        assumed = old;
        old = atomicCAS(a, assumed, __double_as_longlong(__longlong_as_double(assumed) * v));
    } while (assumed != old);
}

// y[post[i]] (+|*)= HOMO ? values[0] : values[pre[i]]
template<typename T, typename I, bool HOMO, bool PROD>
__global__ void __launch_bounds__(THREADS)
coo_atomic_kernel(const uint32_t size, const T *__restrict__ values, const I *__restrict__ pre_ids,
                  const I *__restrict__ post_ids, T *__restrict__ y) {
    const T w0 = values[0];
    // a block takes 4 * THREADS consecutive entries, four per thread: the id loads, then the gathers of `values`, then
    // the reductions, so that four dependent chains (id -> value -> reduction) are in flight instead of one.  One
    // block per tile, not a persistent grid: with many more blocks than the SMs hold the L2 reductions spread better
    // (a persistent grid of 8 blocks per SM measured 73-75 us for 1e7 entries, this form the reduction floor).
    const uint64_t i0 = static_cast<uint64_t>(blockIdx.x) * (4 * THREADS) + threadIdx.x;
    I pre[4], post[4];
    T v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const uint64_t i = i0 + u * THREADS;
        if (i < size) {
            post[u] = post_ids[i];
            if (!HOMO) pre[u] = pre_ids[i];
        }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
        if (i0 + u * THREADS < size) v[u] = HOMO ? w0 : values[pre[u]];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        if (i0 + u * THREADS < size) {
            if (PROD) atomic_mul(y + post[u], v[u]);
            else red_add(y + post[u], v[u]);
        }
    }
}

inline int grid_for(uint64_t n_threads) {
    const uint64_t cap = static_cast<uint64_t>(sm_count()) * 8;
    const uint64_t need = (n_threads + THREADS - 1) / THREADS;
    return static_cast<int>(need < 1 ? 1 : (need < cap ? need : cap));
}

template<typename T>
bool fill(cudaStream_t stream, T *y, uint32_t n, T value) {
    if (n == 0) return true;
    if (value == T(0)) {
        if (cudaMemsetAsync(y, 0, sizeof(T) * static_cast<size_t>(n), stream) != cudaSuccess) return launch_ok();
        return true;
    }
    fill_kernel<T><<<grid_for(n), THREADS, 0, stream>>>(y, n, value);
    return launch_ok();
}

template<typename T, typename I, bool HOMO>
void csr_event_sum_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    const DoubleSizeDescriptor *d = unpack<DoubleSizeDescriptor>(opaque, opaque_len);
    if (!d) return;
    const uint32_t pre_size = d->size_x, post_size = d->size_y;
    T *y = static_cast<T *>(buffers[4]);
    if (!fill<T>(stream, y, post_size, T(0)) || pre_size == 0) return;
    csr_event_sum_kernel<T, I, HOMO><<<grid_for(static_cast<uint64_t>(pre_size) * 32), THREADS, 0, stream>>>(
        pre_size, static_cast<const bool *>(buffers[0]), static_cast<const I *>(buffers[1]),
        static_cast<const I *>(buffers[2]), static_cast<const T *>(buffers[3]), y);
    launch_ok();
}

template<typename T, typename I, bool HOMO>
void coo_event_sum_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    const DoubleSizeDescriptor *d = unpack<DoubleSizeDescriptor>(opaque, opaque_len);
    if (!d) return;
    const uint32_t conn_size = d->size_x, post_size = d->size_y;
    T *y = static_cast<T *>(buffers[4]);
    if (!fill<T>(stream, y, post_size, T(0)) || conn_size == 0) return;
    coo_event_sum_kernel<T, I, HOMO><<<grid_for(conn_size), THREADS, 0, stream>>>(
        conn_size, static_cast<const bool *>(buffers[0]), static_cast<const I *>(buffers[1]),
        static_cast<const I *>(buffers[2]), static_cast<const T *>(buffers[3]), y);
    launch_ok();
}

template<typename T, typename I, bool HOMO, bool PROD>
void coo_atomic_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    const DoubleSizeDescriptor *d = unpack<DoubleSizeDescriptor>(opaque, opaque_len);
    if (!d) return;
    const uint32_t conn_size = d->size_x, post_size = d->size_y;
    const T *values = static_cast<const T *>(buffers[0]);
    const I *pre_ids = HOMO ? nullptr : static_cast<const I *>(buffers[1]);
    const I *post_ids = static_cast<const I *>(buffers[HOMO ? 1 : 2]);
    T *y = static_cast<T *>(buffers[HOMO ? 2 : 3]);
    if (!fill<T>(stream, y, post_size, PROD ? T(1) : T(0)) || conn_size == 0) return;
    const uint64_t tiles = (static_cast<uint64_t>(conn_size) + 4 * THREADS - 1) / (4 * THREADS);
    if (tiles > 0x7fffffffull) {
        set_status(BPL_ERR_ARGUMENT, "coo_atomic: too many entries for one launch");
        return;
    }
    coo_atomic_kernel<T, I, HOMO, PROD><<<static_cast<unsigned int>(tiles), THREADS, 0, stream>>>(
        conn_size, values, pre_ids, post_ids, y);
    launch_ok();
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {

#define FI_VARIANTS(M, stem, ...)                                   \
    M(stem##_f32_i32, float, uint32_t, __VA_ARGS__)                 \
    M(stem##_f32_i64, float, uint64_t, __VA_ARGS__)                 \
    M(stem##_f64_i32, double, uint32_t, __VA_ARGS__)                \
    M(stem##_f64_i64, double, uint64_t, __VA_ARGS__)

#define CSR_EVENT_SUM(name, T, I, HOMO) \
    void name(bpl_stream_t s, void **b, const char *o, size_t n) { csr_event_sum_impl<T, I, HOMO>(s, b, o, n); }
FI_VARIANTS(CSR_EVENT_SUM, gpu_csr_event_sum_homo, true)
FI_VARIANTS(CSR_EVENT_SUM, gpu_csr_event_sum_heter, false)

#define COO_EVENT_SUM(name, T, I, HOMO) \
    void name(bpl_stream_t s, void **b, const char *o, size_t n) { coo_event_sum_impl<T, I, HOMO>(s, b, o, n); }
FI_VARIANTS(COO_EVENT_SUM, gpu_coo_event_sum_homo, true)
FI_VARIANTS(COO_EVENT_SUM, gpu_coo_event_sum_heter, false)

#define COO_ATOMIC(name, T, I, HOMO, PROD) \
    void name(bpl_stream_t s, void **b, const char *o, size_t n) { coo_atomic_impl<T, I, HOMO, PROD>(s, b, o, n); }
FI_VARIANTS(COO_ATOMIC, gpu_coo_atomic_sum_homo, true, false)
FI_VARIANTS(COO_ATOMIC, gpu_coo_atomic_sum_heter, false, false)
FI_VARIANTS(COO_ATOMIC, gpu_coo_atomic_prod_homo, true, true)
FI_VARIANTS(COO_ATOMIC, gpu_coo_atomic_prod_heter, false, true)

}  // extern "C"
