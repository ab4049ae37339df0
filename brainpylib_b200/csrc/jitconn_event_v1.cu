// The counter-based ("v1") just-in-time-connectivity event product: the connection between output row r and
// input column c is decided by a stateless generator seeded with `seed + n_col * r + c` (32-bit wrap-around), so
// only the columns that fired are visited and any (r, c) can be evaluated on its own.
//
//   gpu_event_matvec_prob_{homo,uniform,normal}_{float,double}
//   replaces lib/gpu_jitconn_event_matvec.cu:10-51, 138-183, 281-331 with the generators of
//   lib/kernel_helpers_random.cuh:12-71 (registered lib/gpu_ops.cc:107-112).
//   opaque  JITConnProb{Homo,Uniform,Normal}Descriptor; `prob` holds the RAW connection probability
//   buffers [event_ids i32(>= event_num), event_num i32(1), y T(n_row)]   (what event_info returns, then the output)
//
//   y[r] = sum over the listed events c of  [lfsr113(seed + n_col * r + c) < prob] * w(seed + n_col * r + c)
//   w = 1 | taus88 * w_range + w_min | w_mu + sqrt(-2 log u) cos(2 pi v) * w_sigma with (u, v) two taus88 steps
//
// The reference's wrappers read `event_num[0]` on the HOST from the device buffer (lib/gpu_jitconn_event_matvec.cu:67,75
// and the uniform / normal twins) and hand the kernel a reference to it, so they cannot have run as shipped and no
// Python code of the reference builds these target names; the kernel text, however, defines the function above, and
// that is what is computed here, with the count read on the device.  The two generators are L'Ecuyer's combined
// Tausworthe generators taus88 and lfsr113, one step from the states (s+1, s+7, s+15[, s+127]).
#include "abi.h"
#include "common.cuh"

namespace bpl {
namespace {

enum { V1_HOMO = 0, V1_UNIFORM = 1, V1_NORMAL = 2 };
constexpr int V1_THREADS = 256;

struct Taus88 {
    unsigned int s1, s2, s3;
    __device__ __forceinline__ explicit Taus88(unsigned int seed) : s1(seed + 1u), s2(seed + 7u), s3(seed + 15u) {}
    __device__ __forceinline__ double next() {
        unsigned int b;
        b = (((s1 << 13) ^ s1) >> 19);
        s1 = (((s1 & 4294967294u) << 12) ^ b);
        b = (((s2 << 2) ^ s2) >> 25);
        s2 = (((s2 & 4294967288u) << 4) ^ b);
        b = (((s3 << 3) ^ s3) >> 11);
        s3 = (((s3 & 4294967280u) << 17) ^ b);
        return ((s1 ^ s2 ^ s3) * 2.3283064365386963e-10);
    }
};

__device__ __forceinline__ double lfsr113_first(unsigned int seed) {
    unsigned int z1 = seed + 1u, z2 = seed + 7u, z3 = seed + 15u, z4 = seed + 127u, b;
    b = ((z1 << 6) ^ z1) >> 13;
    z1 = ((z1 & 4294967294u) << 18) ^ b;
    b = ((z2 << 2) ^ z2) >> 27;
    z2 = ((z2 & 4294967288u) << 2) ^ b;
    b = ((z3 << 13) ^ z3) >> 21;
    z3 = ((z3 & 4294967280u) << 7) ^ b;
    b = ((z4 << 3) ^ z4) >> 12;
    z4 = ((z4 & 4294967168u) << 13) ^ b;
    return (z1 ^ z2 ^ z3 ^ z4) * 2.3283064365386963e-10;
}

template<typename T, int KIND>
__global__ void __launch_bounds__(V1_THREADS)
jit_event_v1_kernel(const int *__restrict__ event_ids, const int *__restrict__ event_num, const unsigned int conn_seed,
                    const double conn_prob, const double w1, const double w2, const unsigned int num_row,
                    const unsigned int num_col, T *__restrict__ out) {
    __shared__ int tile[V1_THREADS];
    const unsigned int idx = threadIdx.x;
    const unsigned int row_i = blockIdx.x * blockDim.x + idx;
    const int n_ev = max(*event_num, 0);
    const unsigned int seed_base = conn_seed + num_col * row_i;
    T sum = 0;
    for (int e0 = 0; e0 < n_ev; e0 += V1_THREADS) {
        const int n_tile = min(V1_THREADS, n_ev - e0);
        if (static_cast<int>(idx) < n_tile) tile[idx] = event_ids[e0 + idx];
        __syncthreads();
        for (int i = 0; i < n_tile; ++i) {
            const unsigned int seed = seed_base + tile[i];
            if (lfsr113_first(seed) < conn_prob) {
                if (KIND == V1_HOMO) {
                    sum += 1;
                } else if (KIND == V1_UNIFORM) {
                    Taus88 g(seed);
                    sum += (g.next() * w2 + w1);
                } else {
                    Taus88 g(seed);
                    const double u = g.next(), v = g.next();
                    sum += (w1 + sqrt(-2 * log(u)) * cos(2 * 3.14159265358979323846 * v) * w2);
                }
            }
        }
        __syncthreads();
    }
    if (row_i < num_row) out[row_i] = sum;
}

template<typename T, int KIND>
void jit_event_v1_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    unsigned int n_row, n_col, seed;
    double prob, w1 = 0.0, w2 = 0.0;
    if (KIND == V1_HOMO) {
        const JITConnProbHomoDescriptor *d = unpack<JITConnProbHomoDescriptor>(opaque, opaque_len);
        if (!d) return;
        n_row = d->n_row; n_col = d->n_col; seed = d->seed; prob = d->prob;
    } else {
        const JITConnProbWeightedDescriptor *d = unpack<JITConnProbWeightedDescriptor>(opaque, opaque_len);
        if (!d) return;
        n_row = d->n_row; n_col = d->n_col; seed = d->seed; prob = d->prob; w1 = d->w1; w2 = d->w2;
    }
    if (n_row == 0) return;
    if (buffers[0] == nullptr || buffers[1] == nullptr || buffers[2] == nullptr) {
        set_status(BPL_ERR_ARGUMENT, "counter-based event product: null event list, count or output");
        return;
    }
    const unsigned int grid = (n_row + V1_THREADS - 1) / V1_THREADS;
    jit_event_v1_kernel<T, KIND><<<grid, V1_THREADS, 0, stream>>>(
        static_cast<const int *>(buffers[0]), static_cast<const int *>(buffers[1]), seed, prob, w1, w2, n_row, n_col,
        static_cast<T *>(buffers[2]));
    launch_ok();
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {
#define JIT_EVENT_V1(name, T, KIND) \
    void name(bpl_stream_t s, void **b, const char *o, size_t n) { jit_event_v1_impl<T, KIND>(s, b, o, n); }
JIT_EVENT_V1(gpu_event_matvec_prob_homo_float, float, V1_HOMO)
JIT_EVENT_V1(gpu_event_matvec_prob_homo_double, double, V1_HOMO)
JIT_EVENT_V1(gpu_event_matvec_prob_uniform_float, float, V1_UNIFORM)
JIT_EVENT_V1(gpu_event_matvec_prob_uniform_double, double, V1_UNIFORM)
JIT_EVENT_V1(gpu_event_matvec_prob_normal_float, float, V1_NORMAL)
JIT_EVENT_V1(gpu_event_matvec_prob_normal_double, double, V1_NORMAL)
}  // extern "C"
