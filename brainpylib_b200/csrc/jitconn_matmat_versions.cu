// Versions 'v2' and 'v3' of Y = X @ M with a just-in-time matrix M (normal weights only), registered by the
// reference as gpu_matmat_prob_prob_normal_{float,double}_{v2,v3} (lib/gpu_ops.cc:166-169) and selected by
// `version=` in brainpylib/_src/jitconn_ops/matmat.py:443-452.  They generate DIFFERENT matrices from 'v1'
// (other `curand_init` arguments), so each has to reproduce its own reference kernel:
//
//   v2  lib/gpu_jitconn_matmat.cu:138-231.  Column n of M is cut into 32 ranges of ceil(k / 32) rows; lane t of a
//       warp owns range t with the stream curand_init(seed + n, t * ceil(k / 32), 0): first gap from the start of
//       the range, then weight, gap, weight, ... while inside the range (and inside k).  A lane accumulates
//       X[r][pos] * w for its rows in its own register; the 32 partial sums of a row are added with the shuffle
//       tree (offsets 16, 8, 4, 2, 1) and lane 0 writes Y[r][n].
//   v3  lib/gpu_jitconn_matmat.cu:19-135.  One block per (column n, group of B rows), B = m rounded up to a
//       multiple of 32, at most 512.  Thread r has the stream curand_init(seed + n, row(r) * n_columns, 0).  In
//       rounds, every thread draws ONE (gap, weight) pair into shared memory and then every row walks the B pairs
//       in thread order: pos += gap_i, Y += X[row][pos] * w_i while pos < k.  All rows of a block therefore see the
//       same connectivity, built from B interleaved streams.
//
// Differences from the reference, none visible where the reference works: loads of X are guarded (the reference
// reads beyond X for rows >= m); v3 has the barrier the reference omits between a round's reads and the next
// round's writes, and its threads for rows >= m leave the loop with the others (in the reference they never see
// the position advance and spin for ever, so it only terminates when m is a multiple of its block size).
#include <curand_kernel.h>

#include "abi.h"
#include "common.cuh"

namespace bpl {
namespace {

template<typename T, int SIZE>
__global__ void __launch_bounds__(512)
jit_matmat_v2_kernel(const T *__restrict__ X, const unsigned int seed, const double log_prob, const double w_mu,
                     const double w_sigma, const unsigned int m, const unsigned int k, const unsigned int n,
                     const unsigned int k_per_lane, const unsigned long long n_warps, T *__restrict__ Y) {
    const unsigned long long warp_id = static_cast<unsigned long long>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    if (warp_id >= n_warps) return;            // whole warps only: the shuffles below need all 32 lanes
    const unsigned int m_i = static_cast<unsigned int>(warp_id / n) * SIZE;
    const unsigned int n_i = static_cast<unsigned int>(warp_id % n);
    const unsigned int lane = threadIdx.x % 32;
    unsigned int pos = k_per_lane * lane;
    const unsigned int k_max = min(pos + k_per_lane, k);

    curandState state;
    curand_init(seed + n_i, k_per_lane * lane, 0, &state);
    pos += (unsigned int) ceil(log(curand_uniform(&state)) / log_prob);
    T sum[SIZE];
#pragma unroll
    for (int i = 0; i < SIZE; ++i) sum[i] = 0;
    while (pos < k_max) {
        const T rand = (T) (curand_normal(&state) * w_sigma + w_mu);
#pragma unroll
        for (int i = 0; i < SIZE; ++i) {
            const T x = (m_i + i < m) ? X[static_cast<size_t>(m_i + i) * k + pos] : T(0);
            sum[i] += (x * rand);
        }
        pos += (unsigned int) ceil(log(curand_uniform(&state)) / log_prob);
    }
#pragma unroll
    for (int i = 0; i < SIZE; ++i) {
        T v = sum[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(FULL_MASK, v, o);
        if (m_i + i < m && lane == 0) Y[static_cast<size_t>(m_i + i) * n + n_i] = v;
    }
}

template<typename T>
__global__ void __launch_bounds__(512)
jit_matmat_v3_kernel(const T *__restrict__ X, const unsigned int seed, const double log_prob, const double w_mu,
                     const double w_sigma, const unsigned int m, const unsigned int k, const unsigned int n,
                     T *__restrict__ Y) {
    __shared__ T pair_w[512];
    __shared__ int pair_gap[512];
    const unsigned int t = threadIdx.x, B = blockDim.x;
    const unsigned int m_i = blockIdx.y * B + t;
    int pos = 0;
    T sum = 0;
    curandState state;
    curand_init(seed + blockIdx.x, static_cast<unsigned long long>(m_i * n), 0, &state);   // 32-bit product, as there
    while (pos < static_cast<int>(k)) {        // `pos` advances identically in every thread of the block
        pair_gap[t] = (int) ceil(log(curand_uniform(&state)) / log_prob);
        pair_w[t] = (T) (curand_normal(&state) * w_sigma + w_mu);
        __syncthreads();
        for (unsigned int i = 0; i < B; ++i) {
            pos += pair_gap[i];
            if (pos >= static_cast<int>(k)) break;
            if (m_i < m) sum += (X[static_cast<size_t>(m_i) * k + pos] * pair_w[i]);
        }
        __syncthreads();
    }
    if (m_i < m) Y[static_cast<size_t>(m_i) * n + blockIdx.x] = sum;
}

template<typename T, int VERSION>
void jit_matmat_version_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    const MatMatJITProbDescriptor1 *d = unpack<MatMatJITProbDescriptor1>(opaque, opaque_len);
    if (!d) return;
    const T *X = static_cast<const T *>(buffers[0]);
    T *Y = static_cast<T *>(buffers[1]);
    const unsigned int m = d->m, k = d->k, n = d->n;
    if (m == 0 || n == 0) return;
    if (VERSION == 2) {
        const unsigned int k_per_lane = (k + 31) / 32;
        const unsigned int size = m <= 8 ? 8 : (m <= 16 ? 16 : (m <= 24 ? 24 : 32));
        const unsigned long long n_warps = static_cast<unsigned long long>((m + size - 1) / size) * n;
        const unsigned long long blocks = (n_warps * 32 + 511) / 512;
        if (blocks > 0x7fffffffull) {
            set_status(BPL_ERR_ARGUMENT, "matmat v2: too many (row group, column) pairs for one launch");
            return;
        }
        const unsigned int grid = static_cast<unsigned int>(blocks);
#define BPL_V2(SIZE) jit_matmat_v2_kernel<T, SIZE><<<grid, 512, 0, stream>>>(X, d->seed, d->log_p, d->w1, d->w2, m, k, n, \
                                                                                k_per_lane, n_warps, Y)
        if (size == 8) BPL_V2(8); else if (size == 16) BPL_V2(16); else if (size == 24) BPL_V2(24); else BPL_V2(32);
#undef BPL_V2
    } else {
        const unsigned int B = m >= 481 ? 512u : ((m + 31u) / 32u) * 32u;     // the reference's ladder of block sizes
        const unsigned int gy = (m + B - 1) / B;
        if (gy > 65535u) {
            set_status(BPL_ERR_ARGUMENT, "matmat v3: more than 65535 * 512 rows in the dense operand");
            return;
        }
        jit_matmat_v3_kernel<T><<<dim3(n, gy), B, 0, stream>>>(X, d->seed, d->log_p, d->w1, d->w2, m, k, n, Y);
    }
    launch_ok();
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {
void gpu_matmat_prob_prob_normal_float_v2(bpl_stream_t s, void **b, const char *o, size_t n) { jit_matmat_version_impl<float, 2>(s, b, o, n); }
void gpu_matmat_prob_prob_normal_double_v2(bpl_stream_t s, void **b, const char *o, size_t n) { jit_matmat_version_impl<double, 2>(s, b, o, n); }
void gpu_matmat_prob_prob_normal_float_v3(bpl_stream_t s, void **b, const char *o, size_t n) { jit_matmat_version_impl<float, 3>(s, b, o, n); }
void gpu_matmat_prob_prob_normal_double_v3(bpl_stream_t s, void **b, const char *o, size_t n) { jit_matmat_version_impl<double, 3>(s, b, o, n); }
}  // extern "C"
