// Just-in-time connectivity products for sm_100a: the matrix is never stored, every row
// (or column) regenerates its synapses from the stream `seed + index`.
//   gpu_matvec{,_atomic}_prob_*_v2        replaces lib/gpu_jitconn_matvec{,_atomic}.cu
//   gpu_event_matvec{,_atomic}_prob_*_v2  replaces lib/gpu_jitconn_event_matvec{,_atomic}.cu
//   gpu_matmat_prob_prob_*_v1             replaces lib/gpu_jitconn_matmat.cu
//
// Generator scheme (must stay bit-identical to the reference, whose sampled connectivity is
// the contract): cuRAND XORWOW, `curand_init(seed + i, 0, 0)`; position of the next synapse
//     pos += (int) ceil( log(curand_uniform(&st)) / log_p )
// with a float `log`, a float/double division carried out in double, `ceil`, and a
// conversion to int (lib/gpu_jitconn_matvec.cu:99-106).  The weight of a synapse is drawn
// after its position and before the next gap: uniform `(T)(u * w_range + w_min)`,
// normal `(T)(n * w_sigma + w_mu)`, both evaluated in double (lib/gpu_jitconn_matvec.cu:243,386).
// The same cuRAND device functions and the same expressions are used here, compiled
// without fast-math, so the bits agree.
#include <curand_kernel.h>

#include "abi.h"
#include "common.cuh"

namespace bpl {
namespace {

enum { W_HOMO = 0, W_UNIFORM = 1, W_NORMAL = 2 };

struct Stream {
    curandState st;
    double log_p;
    float inv_log_p;   // float(1 / log_p)
    float tol_k;       // |inv_log_p| * 2^-20; negative when the shortcuts are switched off

    __device__ __forceinline__ Stream(unsigned int stream_seed, double lp) : log_p(lp) {
        curand_init(stream_seed, 0, 0, &st);
        inv_log_p = (float) (1.0 / lp);
        // log(u) lies in [-22.9, 0]; the shortcuts need 0 <= q = log(u) / log_p < 2^20
        const bool ok = inv_log_p < 0.0f && inv_log_p > -45000.0f;
        tol_k = ok ? -inv_log_p * 9.5367432e-7f : -1.0f;
    }

    // The reference's gap is (int) ceil(log(u) / log_p): float log, double division, ceil.
    // It is reproduced exactly in up to three stages, each falling through to the next when it
    // cannot prove the result:
    //  (1) q = __logf(u) * float(1 / log_p).  __logf is within 2^-21.41 (absolute, u in [0.5, 2])
    //      or 3 ulp of the true logarithm and logf within 1 ulp; with the float rounding of the
    //      product (2^-23 q) q is within |1 / log_p| * max(2^-21.19 + 2^-23 |log u|, 1.25 * 2^-21 |log u|)
    //      of the reference's quotient.  The test distance |1 / log_p| * 2^-20 * (1 + 1.5 |log u|) is
    //      more than 2.2x that bound everywhere, so when q is farther than it from the nearest
    //      integer the reference's quotient lies strictly between the same two integers: same ceil.
    //  (2) the same test with the accurate logf (the value the reference uses): error < 2^-22.9 q,
    //      margin 2^-21 q.
    //  (3) the reference's own expression.
    // rint(q) and its integer value come from adding 1.5 * 2^23, exact for 0 <= q < 2^22.
    // At a mean gap of 1000 about 1 draw in 200 leaves stage 1 and 1 in 1000 stage 2.
    __device__ __forceinline__ int gap() {
        const float u = curand_uniform(&st);
        if (tol_k > 0.0f) {
            const float a = __logf(u);
            const float q = a * inv_log_p;
            const float t = q + 12582912.0f;
            const float frac = q - (t - 12582912.0f);
            if (fabsf(frac) > fmaf(fabsf(a), 1.5f * tol_k, tol_k))
                return (__float_as_int(t) - 0x4B400000) + (frac > 0.0f ? 1 : 0);
            const float lg = log(u);
            const float q2 = lg * inv_log_p;
            const float t2 = q2 + 12582912.0f;
            const float frac2 = q2 - (t2 - 12582912.0f);
            if (fabsf(frac2) > q2 * 4.8e-7f)
                return (__float_as_int(t2) - 0x4B400000) + (frac2 > 0.0f ? 1 : 0);
            return (int) ceil(lg / log_p);
        }
        return (int) ceil(log(u) / log_p);
    }
    // the matmat kernels of the reference hold positions as `unsigned int` (lib/gpu_jitconn_matmat.cu:252);
    // the shortcuts only return non-negative values, for which both conversions agree
    __device__ __forceinline__ unsigned int ugap() {
        const float u = curand_uniform(&st);
        if (tol_k > 0.0f) {
            const float a = __logf(u);
            const float q = a * inv_log_p;
            const float t = q + 12582912.0f;
            const float frac = q - (t - 12582912.0f);
            if (fabsf(frac) > fmaf(fabsf(a), 1.5f * tol_k, tol_k))
                return (unsigned int) ((__float_as_int(t) - 0x4B400000) + (frac > 0.0f ? 1 : 0));
            const float lg = log(u);
            const float q2 = lg * inv_log_p;
            const float t2 = q2 + 12582912.0f;
            const float frac2 = q2 - (t2 - 12582912.0f);
            if (fabsf(frac2) > q2 * 4.8e-7f)
                return (unsigned int) ((__float_as_int(t2) - 0x4B400000) + (frac2 > 0.0f ? 1 : 0));
            return (unsigned int) ceil(lg / log_p);
        }
        return (unsigned int) ceil(log(u) / log_p);
    }
    template<typename T, int KIND>
    __device__ __forceinline__ T weight(double w1, double w2) {
        if (KIND == W_UNIFORM) return (T) (curand_uniform(&st) * w2 + w1);
        if (KIND == W_NORMAL) return (T) (curand_normal(&st) * w2 + w1);
        return T(1);
    }
};

// A synapse weight whose raw draws are taken immediately (the stream must advance exactly as in
// the reference) but whose value is only computed when asked for.  Event products ask for it on
// a hit only, which skips the conversions, the double multiply-add and (normal) the Box-Muller
// transform for every silent input.  The value is produced by cuRAND's own conversion functions
// on the same raw draws, in the same pairing as curand_normal (two draws on odd calls, the
// second half of the pair on even calls), so it is bit-identical.
template<typename T, int KIND>
struct LazyWeight {
    unsigned int x, y;
    int second;   // normal: 1 when the current value is the second half of the pair
    int have;     // normal: 1 when an unused second half is pending

    __device__ __forceinline__ LazyWeight() : x(0), y(0), second(0), have(0) {}
    __device__ __forceinline__ void draw(curandState *st) {
        if (KIND == W_UNIFORM) {
            x = curand(st);
        } else if (KIND == W_NORMAL) {
            if (!have) { x = curand(st); y = curand(st); have = 1; second = 0; }
            else { have = 0; second = 1; }
        }
    }
    __device__ __forceinline__ T value(double w1, double w2) const {
        if (KIND == W_UNIFORM) return (T) (_curand_uniform(x) * w2 + w1);
        if (KIND == W_NORMAL) {
            const float2 v = _curand_box_muller(x, y);
            return (T) ((second ? v.y : v.x) * w2 + w1);
        }
        return T(1);
    }
};

constexpr int JIT_THREADS = 256;

// ------------------------------------------------------------------------------------------
// Row-parallel (outdim_parallel = True): one thread owns one output row.
// ------------------------------------------------------------------------------------------
// Dense input: lib/gpu_jitconn_matvec.cu:84-112, :220-251, :363-394.
template<typename T, int KIND>
__global__ void __launch_bounds__(JIT_THREADS)
jit_rows_dense_kernel(const T *__restrict__ vector, const unsigned int seed, const double log_p,
                      const double w1, const double w2, const unsigned int num_row,
                      const unsigned int num_col, T *__restrict__ out) {
    const unsigned int row_i = blockIdx.x * blockDim.x + threadIdx.x;
    if (row_i >= num_row) return;
    Stream s(seed + row_i, log_p);
    T sum = 0;
    int pos = s.gap();
    while (pos < num_col) {
        if (KIND == W_HOMO) {
            sum += vector[pos];
        } else {
            const T rand = s.template weight<T, KIND>(w1, w2);
            sum += (vector[pos] * rand);
        }
        pos += s.gap();
    }
    out[row_i] = sum;
}

// Version 'v1' of the dense-vector product: a Bernoulli test per (row, column) instead of the
// geometric skip, `conn_prob` being the raw probability (lib/gpu_jitconn_matvec.cu:10-54, :141-187,
// :284-331).  One `curand_uniform` per column, the weight drawn only on a connection; a different
// random matrix from 'v2'.  The input vector is staged through shared memory tile by tile as in the
// reference (plus the barrier the reference omits before a tile is overwritten).
template<typename T, int KIND>
__global__ void __launch_bounds__(JIT_THREADS)
jit_rows_dense_v1_kernel(const T *__restrict__ vector, const unsigned int seed, const double conn_prob,
                         const double w1, const double w2, const unsigned int num_row,
                         const unsigned int num_col, T *__restrict__ out) {
    __shared__ T tile[JIT_THREADS];
    const unsigned int idx = threadIdx.x;
    const unsigned int row_i = blockIdx.x * blockDim.x + idx;
    curandState state;
    curand_init(seed + row_i, 0, 0, &state);
    T sum = 0;
    for (unsigned int c0 = 0; c0 < num_col; c0 += JIT_THREADS) {
        const unsigned int n_tile = min(static_cast<unsigned int>(JIT_THREADS), num_col - c0);
        if (idx < n_tile) tile[idx] = vector[c0 + idx];
        __syncthreads();
        for (unsigned int sh_i = 0; sh_i < n_tile; ++sh_i) {
            if (curand_uniform(&state) < conn_prob) {
                if (KIND == W_HOMO) sum += tile[sh_i];
                else if (KIND == W_UNIFORM) sum += tile[sh_i] * (curand_uniform(&state) * w2 + w1);
                else sum += tile[sh_i] * (curand_normal(&state) * w2 + w1);
            }
        }
        __syncthreads();
    }
    if (row_i < num_row) out[row_i] = sum;
}

// Event input read straight from global memory: lib/gpu_jitconn_event_matvec.cu:81-108
// (homogeneous: adds the event VALUE), :217-248, :365-396 (weight drawn for every synapse,
// added when the event is truthy).
template<typename T, typename E, int KIND>
__global__ void __launch_bounds__(JIT_THREADS)
jit_rows_event_kernel(const E *__restrict__ events, const unsigned int seed, const double log_p,
                      const double w1, const double w2, const unsigned int num_row,
                      const unsigned int num_col, T *__restrict__ out) {
    const unsigned int row_i = blockIdx.x * blockDim.x + threadIdx.x;
    if (row_i >= num_row) return;
    Stream s(seed + row_i, log_p);
    LazyWeight<T, KIND> lw;
    T sum = 0;
    int pos = s.gap();
    while (pos < num_col) {
        if (KIND == W_HOMO) {
            sum += events[pos];
        } else {
            lw.draw(&s.st);
            if (events[pos]) sum += lw.value(w1, w2);
        }
        pos += s.gap();
    }
    out[row_i] = sum;
}

// Event input held as a bitmask in shared memory (one bit per input neuron).  Used when only
// the truthiness of an event matters (bool events, or weighted variants) and the mask fits:
// 1e6 inputs = 125 KB.  One persistent block per SM packs the events once and then walks rows
// `block + k * grid`; a random 1-byte gather from L2 per synapse becomes a shared-memory read.
constexpr int MASK_THREADS = 1024;
constexpr unsigned int MASK_MAX_BITS = 200u * 1024u * 8u;   // 200 KB of shared memory

template<typename T, typename E, int KIND>
__global__ void __launch_bounds__(MASK_THREADS, 1)
jit_rows_event_mask_kernel(const E *__restrict__ events, const unsigned int seed, const double log_p,
                           const double w1, const double w2, const unsigned int num_row,
                           const unsigned int num_col, T *__restrict__ out) {
    extern __shared__ uint32_t mask[];
    pack_event_mask(events, num_col, mask);
    __syncthreads();

    for (unsigned int row_i = blockIdx.x * MASK_THREADS + threadIdx.x; row_i < num_row;
         row_i += gridDim.x * MASK_THREADS) {
        Stream s(seed + row_i, log_p);
        LazyWeight<T, KIND> lw;
        T sum = 0;
        unsigned int hits = 0;   // homogeneous: events are 0 or 1, their float sum is the exact count (< 2^24)
        int pos = s.gap();
        while (pos < num_col) {
            const unsigned int hit = (mask[pos >> 5] >> (pos & 31)) & 1u;
            if (KIND == W_HOMO) {
                hits += hit;
            } else {
                lw.draw(&s.st);
                if (hit) sum += lw.value(w1, w2);
            }
            pos += s.gap();
        }
        if (KIND == W_HOMO) sum = (T) hits;
        out[row_i] = sum;
    }
}

// ------------------------------------------------------------------------------------------
// Column-parallel (outdim_parallel = False): one thread owns one input column and scatters.
// ------------------------------------------------------------------------------------------
// Dense input: lib/gpu_jitconn_matvec_atomic.cu:27-52, :82-110, :143-171.
template<typename T, int KIND>
__global__ void __launch_bounds__(JIT_THREADS)
jit_cols_dense_kernel(const T *__restrict__ vector, const unsigned int seed, const double log_p,
                      const double w1, const double w2, const unsigned int num_row,
                      const unsigned int num_col, T *__restrict__ out) {
    const unsigned int col_i = blockIdx.x * blockDim.x + threadIdx.x;
    if (col_i >= num_col) return;
    Stream s(seed + col_i, log_p);
    const T v = vector[col_i];
    int row_i = s.gap();
    while (row_i < num_row) {
        if (KIND == W_HOMO) {
            atomicAdd(&out[row_i], v);
        } else {
            const T rand = s.template weight<T, KIND>(w1, w2);
            atomicAdd(&out[row_i], v * rand);
        }
        row_i += s.gap();
    }
}

// Event input: lib/gpu_jitconn_event_matvec_atomic.cu:30-58, :88-117, :150-178.  There every
// column walks its stream and only the atomicAdd is conditional; a silent column therefore
// contributes nothing and its stream is private, so it is skipped here.  Each block compacts
// the firing columns of its chunk into shared memory and gives one thread to each of them.
constexpr int COL_CHUNK = JIT_THREADS * 8;

template<typename T, typename E, int KIND>
__global__ void __launch_bounds__(JIT_THREADS)
jit_cols_event_kernel(const E *__restrict__ events, const unsigned int seed, const double log_p,
                      const double w1, const double w2, const unsigned int num_row,
                      const unsigned int num_col, T *__restrict__ out) {
    __shared__ unsigned int active[COL_CHUNK];
    __shared__ unsigned int n_active;
    if (threadIdx.x == 0) n_active = 0;
    __syncthreads();
    const unsigned long long base = static_cast<unsigned long long>(blockIdx.x) * COL_CHUNK;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const unsigned long long c = base + k * JIT_THREADS + threadIdx.x;
        if (c < num_col && is_event(events[c])) active[atomicAdd(&n_active, 1u)] = static_cast<unsigned int>(c);
    }
    __syncthreads();
    const unsigned int n = n_active;
    for (unsigned int i = threadIdx.x; i < n; i += JIT_THREADS) {
        const unsigned int col_i = active[i];
        Stream s(seed + col_i, log_p);
        int row_i = s.gap();
        while (row_i < num_row) {
            if (KIND == W_HOMO) {
                atomicAdd(&out[row_i], T(1));
            } else {
                const T weight = s.template weight<T, KIND>(w1, w2);
                atomicAdd(&out[row_i], weight);
            }
            row_i += s.gap();
        }
    }
}

// ------------------------------------------------------------------------------------------
// Y = X @ M, M just-in-time with one stream per output column
// (lib/gpu_jitconn_matmat.cu:236-276 normal, :321-361 uniform).
// ------------------------------------------------------------------------------------------
// A thread owns one output column and 32 rows of X, as in the reference, and accumulates
// `sum += X[row][pos] * w` in synapse order (same bits).  What changes is where X comes from: the
// reference reads X[(m_i + i) * k + pos] from global memory, one 32-byte sector per float; here a
// K-tile of the 32 rows is staged TRANSPOSED in shared memory ([k][row]), so a synapse reads 32
// consecutive floats with 128-bit shared loads.  The lanes of a warp read different tile rows
// (their synapses sit at unrelated positions), which would put them on the same banks; instead
// lane l reads the 16-byte chunks of its row in the rotated order (c + l) mod CHUNKS, so the
// eight lanes served together always touch eight different chunks.  The accumulator register
// (c, i) of lane l therefore belongs to row ((c + l) mod CHUNKS) * PER_CHUNK + i; the rotation is
// undone when Y is written.
constexpr int MM_THREADS = 512;
constexpr int MM_ROWS = 32;

template<typename T> struct MMTile;
template<> struct MMTile<float> { static constexpr int KT = 512; static constexpr int CHUNKS = 8; };    // 64 KB
template<> struct MMTile<double> { static constexpr int KT = 256; static constexpr int CHUNKS = 16; };  // 64 KB

// Stages X[m_i .. m_i+31][k0 .. k0+KT) transposed into `tile` ([KT][MM_ROWS]): lane = row of X, so the 32 stores of
// a warp go to 32 consecutive words (no bank conflict); each lane reads VEC consecutive k from its own row (the
// other half of a touched sector is picked up from L1 by the next iteration).  Rows and columns past the matrix read
// as zero.
template<typename T, int KT>
__device__ __forceinline__ void mm_stage_tile(T *tile, const T *__restrict__ X, const unsigned int m_i,
                                              const unsigned int m, const unsigned int k, const unsigned int k0,
                                              const bool vec_ok, const unsigned int lane, const unsigned int warp) {
    constexpr int VEC = 16 / sizeof(T);
    const unsigned int r = lane;
    const bool row_ok = m_i + r < m;
    const T *src = X + static_cast<size_t>(m_i + r) * k + k0;
    for (unsigned int kk = warp * VEC; kk < KT; kk += (MM_THREADS / 32) * VEC) {
        T v[VEC];
        if (vec_ok && row_ok && k0 + kk + VEC <= k) {
            const uint4 u = *reinterpret_cast<const uint4 *>(src + kk);
            *reinterpret_cast<uint4 *>(v) = u;
        } else {
#pragma unroll
            for (int q = 0; q < VEC; ++q) v[q] = (row_ok && k0 + kk + q < k) ? src[kk + q] : T(0);
        }
#pragma unroll
        for (int q = 0; q < VEC; ++q) tile[(kk + q) * MM_ROWS + r] = v[q];
    }
}

template<typename T, int KIND>
__global__ void __launch_bounds__(MM_THREADS, (sizeof(T) == 8 ? 1 : 2))     // 32 double sums: more than 64 registers
jit_matmat_kernel(const T *__restrict__ X, const unsigned int seed, const double log_p, const double w1,
                  const double w2, const unsigned int m, const unsigned int k, const unsigned int n,
                  T *__restrict__ Y, const unsigned int col0 = 0, const unsigned int *__restrict__ cnt = nullptr,
                  const unsigned int cap = 0, const unsigned int *__restrict__ n_over = nullptr) {
    constexpr int KT = MMTile<T>::KT, CHUNKS = MMTile<T>::CHUNKS, PER_CHUNK = 16 / sizeof(T);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T *tile = reinterpret_cast<T *>(smem_raw);   // [KT][MM_ROWS]

    // columns col0 + blockIdx.x * MM_THREADS + threadIdx.x, below n.  With `cnt`: only the columns whose connection
    // list did not fit its `cap` slots (the list-driven kernel leaves those to this one); normally there are none
    // and every block returns at once.
    const unsigned long long n_i64 = col0 + static_cast<unsigned long long>(blockIdx.x) * MM_THREADS + threadIdx.x;
    bool live = n_i64 < n;
    const unsigned int n_i = static_cast<unsigned int>(n_i64);
    if (cnt != nullptr) {
        if (*n_over == 0u) return;
        live = live && cnt[n_i - col0] > cap;
        if (!__syncthreads_or(live)) return;
    }
    const unsigned int m_i = blockIdx.y * MM_ROWS;
    const unsigned int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool vec_ok = (k % (16 / sizeof(T)) == 0) && ((reinterpret_cast<uintptr_t>(X) & 15u) == 0);

    Stream s(seed + n_i, log_p);
    curandState &st = s.st;
    unsigned int pos = live ? s.ugap() : 0xffffffffu;
    T sum[MM_ROWS];
#pragma unroll
    for (int i = 0; i < MM_ROWS; ++i) sum[i] = 0;

    for (unsigned int k0 = 0; k0 < k; k0 += KT) {
        mm_stage_tile<T, KT>(tile, X, m_i, m, k, k0, vec_ok, lane, warp);
        __syncthreads();
        const unsigned int k_end = min(k0 + KT, k);
        while (pos < k_end) {
            T rand;
            if (KIND == W_NORMAL) rand = (T) (curand_normal(&st) * w2 + w1);
            else rand = (T) (curand_uniform(&st) * w2 + w1);
            const unsigned int kk = pos - k0;
            const T *row = tile + kk * MM_ROWS;
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                const unsigned int chunk = (c + lane) & (CHUNKS - 1);
                if (sizeof(T) == 4) {
                    const float4 x = *reinterpret_cast<const float4 *>(row + chunk * PER_CHUNK);
                    sum[c * 4 + 0] += (x.x * rand);
                    sum[c * 4 + 1] += (x.y * rand);
                    sum[c * 4 + 2] += (x.z * rand);
                    sum[c * 4 + 3] += (x.w * rand);
                } else {
                    const double2 x = *reinterpret_cast<const double2 *>(row + chunk * PER_CHUNK);
                    sum[c * 2 + 0] += (x.x * rand);
                    sum[c * 2 + 1] += (x.y * rand);
                }
            }
            pos += s.ugap();
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const unsigned int chunk = (c + lane) & (CHUNKS - 1);
#pragma unroll
            for (int i = 0; i < PER_CHUNK; ++i) {
                const unsigned int row = m_i + chunk * PER_CHUNK + i;
                if (row < m) Y[static_cast<size_t>(row) * n + n_i] = sum[c * PER_CHUNK + i];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Y = X @ M with every column's stream generated ONCE (targets *_v1_ws: one more buffer, a workspace)
// ------------------------------------------------------------------------------------------
// jit_matmat_kernel regenerates the stream of a column for every group of 32 rows of X (8 times for 256 rows), as
// the reference does, and that generator work is most of its time.  Here one pass walks every column's stream once
// and writes its connections, position and weight (the same draws, the same conversions), into a workspace; a second
// pass is the multiply alone: the same thread = (column, 32 rows) mapping, the same transposed K-tiles of X in shared
// memory, the same order of additions (same bits), with (position, weight) read from the list.
//
// Workspace of one chunk of C columns (C a multiple of MM_THREADS; the host walks the columns chunk by chunk):
//   n_over u32 (+ padding to 256 B) | cnt u32[C] | Xt T[k * m_pad] (X transposed, see below) | entries MMEntry<T>[C * stride]
// Entry j of column c sits at c * stride + j (stride = cap + 1 rounded up to even), position and weight side by side (8 bytes for float, 16 for double),
// and a column's list ends with an entry whose position is 0xffffffff: a
// thread walks its own column's entries front to back at its own pace, so what matters is that consecutive
// entries of ONE column share 32-byte sectors (the first touch of a sector fetches the next entries too); an
// interleaved-by-warp layout was measured first and cost a sector per entry (7.1 ms instead of the inline 6.1).
// cap = expected connections per column + 10 standard deviations + 16.  A column with more (never seen; the bound
// is not a proof) is counted in n_over and recomputed whole by jit_matmat_kernel in its overflow-only mode, so the
// result is exact whatever the draws.
template<typename T> struct MMEntry;
template<> struct __align__(8) MMEntry<float> { unsigned int pos; float w; };
template<> struct __align__(16) MMEntry<double> { unsigned int pos, pad; double w; };
template<typename T> struct __align__(16) MMEntryPair { MMEntry<T> a, b; };
// slots per column: the entries, the terminating entry, rounded up to whole pairs
__host__ __device__ inline unsigned int mm_list_stride(unsigned int cap) { return (cap + 2u) & ~1u; }

template<typename T, int KIND>
__global__ void __launch_bounds__(256)
jit_matmat_fill_kernel(const unsigned int seed, const double log_p, const double w1, const double w2,
                       const unsigned int k, const unsigned int n, const unsigned int col0, const unsigned int cap,
                       unsigned int *__restrict__ cnt, MMEntry<T> *__restrict__ entries,
                       unsigned int *__restrict__ n_over) {
    const unsigned int c = blockIdx.x * 256u + threadIdx.x;     // column within the chunk
    const unsigned long long n_i64 = static_cast<unsigned long long>(col0) + c;
    if (n_i64 >= n) return;
    Stream s(seed + static_cast<unsigned int>(n_i64), log_p);
    curandState &st = s.st;
    MMEntry<T> *mine = entries + static_cast<size_t>(c) * mm_list_stride(cap);
    unsigned int count = 0;
    unsigned int pos = s.ugap();
    // The stream is a chain (state -> draw -> logarithm -> position -> loop test) and a column is one thread, so the
    // walk is bound by latency, not by issue slots.  The draws of the next FOUR connections (weight, gap, weight, gap,
    // ... in the stream's order) are therefore taken ahead of the loop test: only the cheap state update chains them,
    // their logarithms and normal transforms overlap.  Draws behind the last connection of the column are thrown away;
    // nobody else reads this column's stream.
    while (pos < k) {
        T w4[4];
        unsigned int g4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (KIND == W_NORMAL) w4[u] = (T) (curand_normal(&st) * w2 + w1);
            else w4[u] = (T) (curand_uniform(&st) * w2 + w1);
            g4[u] = s.ugap();
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (pos < k) {
                if (count < cap) {
                    MMEntry<T> e;
                    e.pos = pos;
                    e.w = w4[u];
                    mine[count] = e;
                }
                ++count;
                pos += g4[u];
            }
        }
    }
    cnt[c] = count;
    // the list ends with a position no tile contains; a list that overflowed reads as empty
    MMEntry<T> last;
    last.pos = 0xffffffffu;
    last.w = T(0);
    mine[count <= cap ? count : 0u] = last;
    if (count > cap) atomicAdd(n_over, 1u);
}

// ---- the multiply ----
// X is first transposed into the workspace (Xt[k][m_pad]): the values of a group of rows at position pos are then
// contiguous, and a K-tile of a row group is copied into shared memory as is, by 16-byte asynchronous copies, while
// the previous tile is being multiplied (two buffers).
//
// Mapping: a thread owns one column and 32 rows of X, as in the inline kernel, and walks its own list; the block is
// one per SM with up to 1024 threads and two tiles of 768 positions (96 KB each).  What bounds it is the spread of
// the number of connections per thread and tile (Poisson, mean 7.7 at C5): every tile ends at a block-wide barrier,
// so the slowest thread sets its length, and shared memory caps the tile.  Measured alternatives, same workload
// (inline kernel, generator included: 6.1 ms):
//   * row-major X staged through registers, 512 threads, tiles of 768, two blocks per SM          6.2 ms
//   * Xt tiles copied asynchronously, 512 threads, two tiles of 384, two blocks per SM            4.4 ms
//   * lanes as rows (a warp owns 8-16 columns x 128 rows, every lane works on every connection, no spread at all):
//     10 ms with a column's entry loaded when the column is visited, 7.7 ms with the next entry of every column kept
//     in registers — a block then covers only 192 columns, so a staged tile is used by too few connections and the
//     copies of Xt (22 GB instead of 4 GB) bound it.
// Each (row, column) sum receives its products in stream order: same bits as the inline kernel.
template<typename T> struct MMApply;
template<> struct MMApply<float> { static constexpr int MAX_THREADS = 896; };      // up to 72 registers per thread
template<> struct MMApply<double> { static constexpr int MAX_THREADS = 512; };     // 32 double sums: up to 128
constexpr int MMA_TILE_BYTES = 96 * 1024;      // per buffer, two buffers, one block per SM

__device__ __forceinline__ void mm_cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 :: "r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(__cvta_generic_to_global(src))
                 : "memory");
}

// 32 x 32 tiles through shared memory; grid = (ceil(k / 32), m_pad / 32), block = (32, 8)
template<typename T>
__global__ void __launch_bounds__(256)
jit_matmat_transpose_kernel(const T *__restrict__ X, const unsigned int m, const unsigned int k,
                            const unsigned int m_pad, T *__restrict__ Xt) {
    __shared__ T t[32][33];
    const unsigned int k0 = blockIdx.x * 32u, m0 = blockIdx.y * 32u;
    for (unsigned int i = threadIdx.y; i < 32u; i += 8u) {
        const unsigned int r = m0 + i, c = k0 + threadIdx.x;
        t[i][threadIdx.x] = (r < m && c < k) ? X[static_cast<size_t>(r) * k + c] : T(0);
    }
    __syncthreads();
    for (unsigned int i = threadIdx.y; i < 32u; i += 8u) {
        const unsigned int c = k0 + i;
        if (c < k) Xt[static_cast<size_t>(c) * m_pad + m0 + threadIdx.x] = t[threadIdx.x][i];
    }
}

// grid = (row groups of 32, column blocks of blockDim.x columns): the blocks that walk the same columns' lists are
// launched side by side, so the lists come from DRAM once and from L2 for the other row groups.
template<typename T>
__global__ void __launch_bounds__(MMApply<T>::MAX_THREADS, 1)
jit_matmat_apply_kernel(const T *__restrict__ Xt, const unsigned int m, const unsigned int m_pad, const unsigned int k,
                        const unsigned int n, const unsigned int col0, const unsigned int cols,
                        const unsigned int cap, const unsigned int *__restrict__ cnt,
                        const MMEntry<T> *__restrict__ entries, T *__restrict__ Y) {
    constexpr int CHUNKS = MMTile<T>::CHUNKS, PER_CHUNK = 16 / sizeof(T);
    constexpr int KT = MMA_TILE_BYTES / (MM_ROWS * static_cast<int>(sizeof(T)));   // positions per tile
    constexpr int ROW_PIECES = MM_ROWS * sizeof(T) / 16;                           // 16-byte pieces per position
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T *tiles = reinterpret_cast<T *>(smem_raw);   // [2][KT][MM_ROWS]

    const unsigned int c = blockIdx.y * blockDim.x + threadIdx.x;       // column within the chunk
    const bool live = c < cols;
    const unsigned int n_i = col0 + c;
    const unsigned int m_i = blockIdx.x * MM_ROWS;
    const unsigned int lane = threadIdx.x & 31;

    const bool fits = live && cnt[c] <= cap;                           // else: the overflow pass writes this column
    // The list is read two entries at a time (one 16-byte load per lane every other connection: every lane reads its
    // own list, so a warp's load touches 32 different lines and costs the load/store pipe as much as all shared loads
    // of a connection together).  `cur` holds the pair being consumed, `nxt` the pair after it, requested when `cur`
    // is entered; `j` counts consumed entries.
    const MMEntryPair<T> *pairs =
        reinterpret_cast<const MMEntryPair<T> *>(entries + static_cast<size_t>(c) * mm_list_stride(cap));
    MMEntryPair<T> cur, nxt;
    cur.a.pos = cur.b.pos = nxt.a.pos = nxt.b.pos = 0xffffffffu;
    cur.a.w = cur.b.w = nxt.a.w = nxt.b.w = T(0);
    unsigned int j = 0;
    if (live) {                                                         // an overflowed list reads as empty
        cur = pairs[0];
        if (cur.a.pos != 0xffffffffu && cur.b.pos != 0xffffffffu) nxt = pairs[1];
    }
    unsigned int pos = cur.a.pos;
    T rand = cur.a.w;
    T sum[MM_ROWS];
#pragma unroll
    for (int i = 0; i < MM_ROWS; ++i) sum[i] = 0;

    // tile t = positions [t * KT, min((t + 1) * KT, k)) of the row group, into buffer t & 1
    auto issue = [&](unsigned int t) {
        const unsigned int k0 = t * KT;
        const unsigned int rows = min(static_cast<unsigned int>(KT), k - k0);
        T *dst = tiles + static_cast<size_t>(t & 1u) * KT * MM_ROWS;
        const T *src = Xt + static_cast<size_t>(k0) * m_pad + m_i;
        for (unsigned int q = threadIdx.x; q < rows * ROW_PIECES; q += blockDim.x) {
            const unsigned int kk = q / ROW_PIECES, piece = q % ROW_PIECES;
            mm_cp_async16(dst + kk * MM_ROWS + piece * PER_CHUNK, src + static_cast<size_t>(kk) * m_pad + piece * PER_CHUNK);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const unsigned int n_tiles = (k + KT - 1) / KT;
    issue(0);
    for (unsigned int t = 0; t < n_tiles; ++t) {
        if (t + 1 < n_tiles) {
            issue(t + 1);                                            // its buffer was last read in iteration t - 1
            asm volatile("cp.async.wait_group 1;" ::: "memory");    // this thread's copies of tile t have landed
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                                             // everyone's have
        const unsigned int k0 = t * KT;
        const unsigned int k_end = min(k0 + KT, k);
        const T *tile = tiles + static_cast<size_t>(t & 1u) * KT * MM_ROWS;
        while (pos < k_end) {
            const T *row = tile + (pos - k0) * MM_ROWS;
            const T w = rand;
            ++j;
            if (j & 1u) {                                            // second entry of the pair
                pos = cur.b.pos;
                rand = cur.b.w;
            } else {                                                 // next pair; request the one after it unless the
                cur = nxt;                                           // list ends inside (position 0xffffffff ends it)
                pos = cur.a.pos;
                rand = cur.a.w;
                if (cur.a.pos != 0xffffffffu && cur.b.pos != 0xffffffffu) nxt = pairs[(j >> 1) + 1];
            }
#pragma unroll
            for (int cc = 0; cc < CHUNKS; ++cc) {
                const unsigned int chunk = (cc + lane) & (CHUNKS - 1);
                if (sizeof(T) == 4) {
                    const float4 x = *reinterpret_cast<const float4 *>(row + chunk * PER_CHUNK);
                    sum[cc * 4 + 0] += (x.x * w);
                    sum[cc * 4 + 1] += (x.y * w);
                    sum[cc * 4 + 2] += (x.z * w);
                    sum[cc * 4 + 3] += (x.w * w);
                } else {
                    const double2 x = *reinterpret_cast<const double2 *>(row + chunk * PER_CHUNK);
                    sum[cc * 2 + 0] += (x.x * w);
                    sum[cc * 2 + 1] += (x.y * w);
                }
            }
        }
        __syncthreads();                                             // tile t is free for the copies of tile t + 2
    }
    if (fits && static_cast<unsigned long long>(col0) + c < n) {
#pragma unroll
        for (int cc = 0; cc < CHUNKS; ++cc) {
            const unsigned int chunk = (cc + lane) & (CHUNKS - 1);
#pragma unroll
            for (int i = 0; i < PER_CHUNK; ++i) {
                const unsigned int row = m_i + chunk * PER_CHUNK + i;
                if (row < m) Y[static_cast<size_t>(row) * n + n_i] = sum[cc * PER_CHUNK + i];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
struct JitArgs {
    unsigned int n_row, n_col, seed;
    double log_p, w1, w2;
};

template<int KIND>
inline bool unpack_jit(const char *opaque, size_t opaque_len, JitArgs &a) {
    if (KIND == W_HOMO) {
        const JITConnProbHomoDescriptor *d = unpack<JITConnProbHomoDescriptor>(opaque, opaque_len);
        if (!d) return false;
        a = JitArgs{d->n_row, d->n_col, d->seed, d->prob, 0.0, 0.0};
    } else {
        const JITConnProbWeightedDescriptor *d = unpack<JITConnProbWeightedDescriptor>(opaque, opaque_len);
        if (!d) return false;
        a = JitArgs{d->n_row, d->n_col, d->seed, d->prob, d->w1, d->w2};
    }
    return true;
}

inline unsigned int blocks_for(unsigned int n, unsigned int per_block) {
    return static_cast<unsigned int>((static_cast<unsigned long long>(n) + per_block - 1) / per_block);
}

template<typename T, int KIND, bool ROWS>
void jit_matvec_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    JitArgs a;
    if (!unpack_jit<KIND>(opaque, opaque_len, a)) return;
    const T *vector = static_cast<const T *>(buffers[0]);
    T *y = static_cast<T *>(buffers[1]);
    if (a.n_row == 0) return;
    if (ROWS) {
        jit_rows_dense_kernel<T, KIND><<<blocks_for(a.n_row, JIT_THREADS), JIT_THREADS, 0, stream>>>(
            vector, a.seed, a.log_p, a.w1, a.w2, a.n_row, a.n_col, y);
    } else {
        if (cudaMemsetAsync(y, 0, sizeof(T) * static_cast<size_t>(a.n_row), stream) != cudaSuccess) {
            launch_ok();
            return;
        }
        if (a.n_col == 0) return;
        jit_cols_dense_kernel<T, KIND><<<blocks_for(a.n_col, JIT_THREADS), JIT_THREADS, 0, stream>>>(
            vector, a.seed, a.log_p, a.w1, a.w2, a.n_row, a.n_col, y);
    }
    launch_ok();
}

template<typename T, int KIND>
void jit_matvec_v1_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    JitArgs a;
    if (!unpack_jit<KIND>(opaque, opaque_len, a)) return;   // a.log_p holds the raw probability here
    if (a.n_row == 0) return;
    jit_rows_dense_v1_kernel<T, KIND><<<blocks_for(a.n_row, JIT_THREADS), JIT_THREADS, 0, stream>>>(
        static_cast<const T *>(buffers[0]), a.seed, a.log_p, a.w1, a.w2, a.n_row, a.n_col,
        static_cast<T *>(buffers[1]));
    launch_ok();
}

template<typename T, typename E, int KIND>
bool enable_mask_kernel(size_t bytes) {
    static thread_local int configured_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_device != dev) {
        if (cudaFuncSetAttribute(jit_rows_event_mask_kernel<T, E, KIND>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(MASK_MAX_BITS / 8)) != cudaSuccess) {
            launch_ok();
            return false;
        }
        configured_device = dev;
    }
    (void) bytes;
    return true;
}

template<typename T, typename E, int KIND, bool ROWS>
void jit_event_matvec_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    JitArgs a;
    if (!unpack_jit<KIND>(opaque, opaque_len, a)) return;
    const E *events = static_cast<const E *>(buffers[0]);
    T *y = static_cast<T *>(buffers[1]);
    if (a.n_row == 0) return;
    if (ROWS) {
        // the bitmask holds truthiness only: enough unless a homogeneous product must add float event values
        const bool truth_only = (KIND != W_HOMO) || (sizeof(E) == 1);
        const bool big_enough = static_cast<unsigned long long>(a.n_row) >= 4ull * MASK_THREADS;
        if (truth_only && big_enough && a.n_col <= MASK_MAX_BITS) {
            const size_t bytes = static_cast<size_t>((a.n_col + 31u) >> 5) * 4;
            if (!enable_mask_kernel<T, E, KIND>(bytes)) return;
            const unsigned int grid = min(static_cast<unsigned int>(sm_count()), blocks_for(a.n_row, MASK_THREADS));
            jit_rows_event_mask_kernel<T, E, KIND><<<grid, MASK_THREADS, bytes, stream>>>(
                events, a.seed, a.log_p, a.w1, a.w2, a.n_row, a.n_col, y);
        } else {
            jit_rows_event_kernel<T, E, KIND><<<blocks_for(a.n_row, JIT_THREADS), JIT_THREADS, 0, stream>>>(
                events, a.seed, a.log_p, a.w1, a.w2, a.n_row, a.n_col, y);
        }
    } else {
        if (cudaMemsetAsync(y, 0, sizeof(T) * static_cast<size_t>(a.n_row), stream) != cudaSuccess) {
            launch_ok();
            return;
        }
        if (a.n_col == 0) return;
        jit_cols_event_kernel<T, E, KIND><<<blocks_for(a.n_col, COL_CHUNK), JIT_THREADS, 0, stream>>>(
            events, a.seed, a.log_p, a.w1, a.w2, a.n_row, a.n_col, y);
    }
    launch_ok();
}

template<typename T, int KIND>
void jit_matmat_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    const MatMatJITProbDescriptor1 *d = unpack<MatMatJITProbDescriptor1>(opaque, opaque_len);
    if (!d) return;
    const T *X = static_cast<const T *>(buffers[0]);
    T *Y = static_cast<T *>(buffers[1]);
    if (d->m == 0 || d->n == 0) return;
    const unsigned int gy = blocks_for(d->m, MM_ROWS);
    if (gy > 65535u) {
        set_status(BPL_ERR_ARGUMENT, "matmat: more than 65535 * 32 rows in the dense operand");
        return;
    }
    constexpr size_t smem = static_cast<size_t>(MMTile<T>::KT) * MM_ROWS * sizeof(T);
    static thread_local int configured_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_device != dev) {
        if (cudaFuncSetAttribute(jit_matmat_kernel<T, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem)) != cudaSuccess) {
            launch_ok();
            return;
        }
        configured_device = dev;
    }
    const dim3 grid(blocks_for(d->n, MM_THREADS), gy);
    jit_matmat_kernel<T, KIND><<<grid, MM_THREADS, smem, stream>>>(
        X, d->seed, d->log_p, d->w1, d->w2, d->m, d->k, d->n, Y);
    launch_ok();
}

// ---- list-driven matmat: capacity, chunking, workspace ----
constexpr size_t MM_LIST_BUDGET = 768ull << 20;     // bytes of lists one chunk of columns may take
// tests: force a small capacity (the overflow pass runs) or a small budget (several chunks of columns)
unsigned int g_mm_list_cap_override = 0;
size_t g_mm_list_budget_override = 0;

struct MMListPlan {
    unsigned int cap;        // list slots per column
    unsigned int chunk;      // columns per chunk (multiple of MM_THREADS)
    unsigned int m_pad;      // rows of X rounded up to MM_ROWS
    size_t cnt_off, xt_off, entries_off, bytes;
};

inline MMListPlan mm_list_plan(unsigned int m, unsigned int k, unsigned int n, double log_p, size_t elem) {
    MMListPlan p;
    const double prob = -expm1(log_p);                        // log_p = log(1 - conn_prob)
    const double mean = static_cast<double>(k) * prob;
    const double cap_d = ceil(mean + 10.0 * sqrt(mean * (1.0 - prob) + 1.0)) + 16.0;
    p.cap = static_cast<unsigned int>(cap_d < static_cast<double>(k) + 16.0 ? cap_d : static_cast<double>(k) + 16.0);
    if (g_mm_list_cap_override != 0) p.cap = g_mm_list_cap_override;
    const size_t entry = elem == 8 ? 16 : 8;        // sizeof(MMEntry<T>)
    const size_t per_col = static_cast<size_t>(mm_list_stride(p.cap)) * entry + 4;
    const size_t n_round = (static_cast<size_t>(n) + MM_THREADS - 1) / MM_THREADS * MM_THREADS;
    const size_t budget = g_mm_list_budget_override != 0 ? g_mm_list_budget_override : MM_LIST_BUDGET;
    size_t chunk = budget / per_col / MM_THREADS * MM_THREADS;
    if (chunk < static_cast<size_t>(MM_THREADS)) chunk = MM_THREADS;
    if (chunk > n_round) chunk = n_round;
    p.chunk = static_cast<unsigned int>(chunk);
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    p.cnt_off = 256;
    p.m_pad = (m + MM_ROWS - 1) / MM_ROWS * MM_ROWS;
    p.xt_off = up(p.cnt_off + 4 * chunk);
    p.entries_off = up(p.xt_off + elem * static_cast<size_t>(k) * p.m_pad);
    p.bytes = up(p.entries_off + entry * chunk * static_cast<size_t>(mm_list_stride(p.cap)));
    return p;
}

template<typename T, int KIND>
void jit_matmat_list_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    const MatMatJITProbDescriptor1 *d = unpack<MatMatJITProbDescriptor1>(opaque, opaque_len);
    if (!d) return;
    const T *X = static_cast<const T *>(buffers[0]);
    T *Y = static_cast<T *>(buffers[1]);
    unsigned char *ws = static_cast<unsigned char *>(buffers[2]);
    if (d->m == 0 || d->n == 0) return;
    const unsigned int gy = blocks_for(d->m, MM_ROWS);
    if (gy > 65535u) {
        set_status(BPL_ERR_ARGUMENT, "matmat: more than 65535 * 32 rows in the dense operand");
        return;
    }
    if (ws == nullptr || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) {
        set_status(BPL_ERR_ARGUMENT, "matmat: the workspace is missing or not aligned to 256 bytes");
        return;
    }
    if (d->k == 0) {
        if (cudaMemsetAsync(Y, 0, sizeof(T) * static_cast<size_t>(d->m) * d->n, stream) != cudaSuccess) launch_ok();
        return;
    }
    const MMListPlan p = mm_list_plan(d->m, d->k, d->n, d->log_p, sizeof(T));
    constexpr size_t smem_apply = 2 * static_cast<size_t>(MMA_TILE_BYTES);
    constexpr size_t smem_inline = static_cast<size_t>(MMTile<T>::KT) * MM_ROWS * sizeof(T);
    static thread_local int configured_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_device != dev) {
        if (cudaFuncSetAttribute(jit_matmat_apply_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem_apply)) != cudaSuccess ||
            cudaFuncSetAttribute(jit_matmat_kernel<T, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem_inline)) != cudaSuccess) {
            launch_ok();
            return;
        }
        configured_device = dev;
    }
    unsigned int *n_over = reinterpret_cast<unsigned int *>(ws);
    unsigned int *cnt = reinterpret_cast<unsigned int *>(ws + p.cnt_off);
    MMEntry<T> *entries = reinterpret_cast<MMEntry<T> *>(ws + p.entries_off);
    T *Xt = reinterpret_cast<T *>(ws + p.xt_off);
    const unsigned int sms = static_cast<unsigned int>(sm_count());
    jit_matmat_transpose_kernel<T><<<dim3(blocks_for(d->k, 32), p.m_pad / 32), dim3(32, 8), 0, stream>>>(
        X, d->m, d->k, p.m_pad, Xt);
    for (unsigned long long col0 = 0; col0 < d->n; col0 += p.chunk) {
        const unsigned int cols = static_cast<unsigned int>(
            d->n - col0 < p.chunk ? d->n - col0 : static_cast<unsigned long long>(p.chunk));
        const unsigned int c0 = static_cast<unsigned int>(col0);
        if (cudaMemsetAsync(n_over, 0, sizeof(unsigned int), stream) != cudaSuccess) {
            launch_ok();
            return;
        }
        jit_matmat_fill_kernel<T, KIND><<<blocks_for(cols, 256), 256, 0, stream>>>(
            d->seed, d->log_p, d->w1, d->w2, d->k, d->n, c0, p.cap, cnt, entries, n_over);
        const dim3 grid(blocks_for(cols, MM_THREADS), gy);
        // threads per block (= columns per block): the size whose last wave of blocks, one per SM, wastes least
        unsigned int threads = 128, best_cost = 0xffffffffu;
        for (unsigned int th = 256; th <= static_cast<unsigned int>(MMApply<T>::MAX_THREADS); th += 128) {
            const unsigned long long blocks = static_cast<unsigned long long>(blocks_for(cols, th)) * gy;
            const unsigned long long waves = (blocks + sms - 1) / sms;
            const unsigned long long cost = waves * th;
            if (cost <= best_cost) {
                best_cost = static_cast<unsigned int>(cost < 0xffffffffull ? cost : 0xfffffffeull);
                threads = th;
            }
        }
        const dim3 grid_apply(gy, blocks_for(cols, threads));
        jit_matmat_apply_kernel<T><<<grid_apply, threads, smem_apply, stream>>>(Xt, d->m, p.m_pad, d->k, d->n, c0, cols,
                                                                               p.cap, cnt, entries, Y);
        jit_matmat_kernel<T, KIND><<<grid, MM_THREADS, smem_inline, stream>>>(
            X, d->seed, d->log_p, d->w1, d->w2, d->m, d->k, d->n, Y, c0, cnt, p.cap, n_over);
    }
    launch_ok();
}

}  // namespace

size_t matmat_list_workspace_bytes(const char *opaque, size_t opaque_len, size_t elem) {
    if (opaque == nullptr || opaque_len != sizeof(MatMatJITProbDescriptor1)) return 0;
    const MatMatJITProbDescriptor1 *d = reinterpret_cast<const MatMatJITProbDescriptor1 *>(opaque);
    if (d->n == 0) return 256;
    return mm_list_plan(d->m, d->k, d->n, d->log_p, elem).bytes;
}

}  // namespace bpl

using namespace bpl;

extern "C" {

#define JIT_MATVEC(name, T, KIND, ROWS) \
    void name(bpl_stream_t s, void **b, const char *o, size_t n) { jit_matvec_impl<T, KIND, ROWS>(s, b, o, n); }
#define JIT_MATVEC_ALL(kind, KIND)                                           \
    JIT_MATVEC(gpu_matvec_prob_##kind##_v2_float, float, KIND, true)          \
    JIT_MATVEC(gpu_matvec_prob_##kind##_v2_double, double, KIND, true)        \
    JIT_MATVEC(gpu_matvec_atomic_prob_##kind##_v2_float, float, KIND, false)  \
    JIT_MATVEC(gpu_matvec_atomic_prob_##kind##_v2_double, double, KIND, false)
JIT_MATVEC_ALL(homo, W_HOMO)
JIT_MATVEC_ALL(uniform, W_UNIFORM)
JIT_MATVEC_ALL(normal, W_NORMAL)

#define JIT_MATVEC_V1(name, T, KIND) \
    void name(bpl_stream_t s, void **b, const char *o, size_t n) { jit_matvec_v1_impl<T, KIND>(s, b, o, n); }
JIT_MATVEC_V1(gpu_matvec_prob_homo_v1_float, float, W_HOMO)
JIT_MATVEC_V1(gpu_matvec_prob_homo_v1_double, double, W_HOMO)
JIT_MATVEC_V1(gpu_matvec_prob_uniform_v1_float, float, W_UNIFORM)
JIT_MATVEC_V1(gpu_matvec_prob_uniform_v1_double, double, W_UNIFORM)
JIT_MATVEC_V1(gpu_matvec_prob_normal_v1_float, float, W_NORMAL)
JIT_MATVEC_V1(gpu_matvec_prob_normal_v1_double, double, W_NORMAL)

#define JIT_EVENT(name, T, E, KIND, ROWS) \
    void name(bpl_stream_t s, void **b, const char *o, size_t n) { jit_event_matvec_impl<T, E, KIND, ROWS>(s, b, o, n); }
#define JIT_EVENT_ALL(kind, KIND)                                                               \
    JIT_EVENT(gpu_event_matvec_prob_##kind##_v2_float_bool, float, bool, KIND, true)             \
    JIT_EVENT(gpu_event_matvec_prob_##kind##_v2_float_float, float, float, KIND, true)           \
    JIT_EVENT(gpu_event_matvec_prob_##kind##_v2_double_bool, double, bool, KIND, true)           \
    JIT_EVENT(gpu_event_matvec_prob_##kind##_v2_double_double, double, double, KIND, true)       \
    JIT_EVENT(gpu_event_matvec_atomic_prob_##kind##_v2_float_bool, float, bool, KIND, false)     \
    JIT_EVENT(gpu_event_matvec_atomic_prob_##kind##_v2_float_float, float, float, KIND, false)   \
    JIT_EVENT(gpu_event_matvec_atomic_prob_##kind##_v2_double_bool, double, bool, KIND, false)   \
    JIT_EVENT(gpu_event_matvec_atomic_prob_##kind##_v2_double_double, double, double, KIND, false)
JIT_EVENT_ALL(homo, W_HOMO)
JIT_EVENT_ALL(uniform, W_UNIFORM)
JIT_EVENT_ALL(normal, W_NORMAL)

#define JIT_MATMAT(name, T, KIND) \
    void name(bpl_stream_t s, void **b, const char *o, size_t n) { jit_matmat_impl<T, KIND>(s, b, o, n); }
JIT_MATMAT(gpu_matmat_prob_prob_normal_float_v1, float, W_NORMAL)
JIT_MATMAT(gpu_matmat_prob_prob_normal_double_v1, double, W_NORMAL)
JIT_MATMAT(gpu_matmat_prob_prob_uniform_float_v1, float, W_UNIFORM)
JIT_MATMAT(gpu_matmat_prob_prob_uniform_double_v1, double, W_UNIFORM)
#define JIT_MATMAT_LIST(name, T, KIND) \
    void name(bpl_stream_t s, void **b, const char *o, size_t n) { jit_matmat_list_impl<T, KIND>(s, b, o, n); }
JIT_MATMAT_LIST(gpu_matmat_prob_prob_normal_float_v1_ws, float, W_NORMAL)
JIT_MATMAT_LIST(gpu_matmat_prob_prob_normal_double_v1_ws, double, W_NORMAL)
JIT_MATMAT_LIST(gpu_matmat_prob_prob_uniform_float_v1_ws, float, W_UNIFORM)
JIT_MATMAT_LIST(gpu_matmat_prob_prob_uniform_double_v1_ws, double, W_UNIFORM)

// Tests only: non-zero values replace the computed list capacity per column and the byte budget of one chunk of
// columns (0 restores them), so that a small matrix overflows its lists (the recomputation pass runs) or is walked
// in several chunks.
void bpl_matmat_list_limits_for_tests(uint32_t cap, size_t budget_bytes) {
    g_mm_list_cap_override = cap;
    g_mm_list_budget_override = budget_bytes;
}

}  // extern "C"
