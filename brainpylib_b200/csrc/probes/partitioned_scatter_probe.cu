// Probe: can the transposed event product on a PLAIN CSR matrix get past the L2 reduction rate by
// partitioning the active synapses by column range first?
//
// The scatter of one step (about 1e7 synapses of 1e4 active rows into 1e6 outputs) costs one L2
// reduction per synapse, 155 G/s on a B200 = 64 us, while the rows themselves stream in 11 us.  Here the
// step is done in two passes without any per-synapse global reduction:
//
//   pass 1  (partition)   A CTA takes batches of 2..16 active rows, loads them with 128-bit loads, bins the
//                         entries by column bucket (4096 columns per bucket) in shared memory - integer
//                         shared-memory atomics hand out the positions - reserves room in each bucket's
//                         global array with one global atomic per (batch, bucket) and copies each bin out
//                         as one contiguous run of {local column, weight} pairs.
//   pass 2  (accumulate)  One CTA per bucket streams its array (coalesced, mostly from L2), accumulates
//                         into 4096 floats of shared memory and adds the slice to y with plain stores.
//
// Entries that do not fit a bucket's array (capacity 2.3x the mean here) fall back to a global reduction in
// pass 1, so the result is always complete.  The probe builds a pool of rows, runs K steps with different
// active rows (the matrix data of a step is cold in DRAM/L2), checks both passes against the plain
// reduction kernel and prints the times.
//
// Measured on one B200 (SM clock 1965 MHz): reduction kernel about 66 us per step; partition 55 us
// (1024 threads x 16 rows) to 87 us (256 threads x 2 rows) + accumulate 30.7 us, i.e. 0.77x at best: the
// phases of pass 1 run one after the other between block-wide barriers, and pass 2 manages about 1.1
// shared-memory float atomics per clock per SM on its 4096 hot addresses.  Results equal the reduction
// kernel's exactly (the weights are multiples of 2^-20, so every order of additions gives the same float).
//
// Build and run:
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o partitioned_scatter_probe partitioned_scatter_probe.cu
//   ./partitioned_scatter_probe
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_runtime.h>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
    std::printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); std::exit(1); } } while (0)

constexpr uint32_t N_COL = 1000000;        // outputs
constexpr uint32_t DEGREE = 1000;          // entries per row (a multiple of 4: rows start 16-byte aligned)
constexpr uint32_t POOL_ROWS = 100000;     // rows held in memory (800 MB); a step activates 1e4 of them
constexpr uint32_t N_ACT = 10000;
constexpr int STEPS = 8;

constexpr uint32_t BUCKET_SHIFT = 12;                      // 4096 columns per bucket
constexpr uint32_t BUCKET_COLS = 1u << BUCKET_SHIFT;
constexpr uint32_t N_BUCKETS = (N_COL + BUCKET_COLS - 1) / BUCKET_COLS;   // 245
constexpr uint32_t BUCKET_CAP = 96 * 1024;                 // entries per bucket array (mean 40.8 K per step)

static_assert(DEGREE % 4 == 0, "rows must start on 16-byte boundaries in this probe");

__device__ __forceinline__ uint4 ldg_stream_u4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// ---------------------------------------------------------------------------------------------------------
// reference: one warp per active row, one global reduction per synapse (what the library does today)
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
red_scatter_kernel(const uint32_t *__restrict__ cols, const float *__restrict__ w,
                   const uint32_t *__restrict__ act, const uint32_t n_act, float *__restrict__ y) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, n_warps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t i = warp; i < n_act; i += n_warps) {
        const size_t base = static_cast<size_t>(act[i]) * DEGREE;
        for (uint32_t g = lane; g < DEGREE / 4; g += 32) {
            const uint4 c = ldg_stream_u4(cols + base + 4 * g);
            const uint4 v = ldg_stream_u4(w + base + 4 * g);
            atomicAdd(y + c.x, __uint_as_float(v.x));
            atomicAdd(y + c.y, __uint_as_float(v.y));
            atomicAdd(y + c.z, __uint_as_float(v.z));
            atomicAdd(y + c.w, __uint_as_float(v.w));
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// pass 1: partition the active synapses into per-bucket arrays
// ---------------------------------------------------------------------------------------------------------
// shared memory: stage[BATCH_ENTRIES] uint2 {local column, weight bits}; count[N_BUCKETS], start[N_BUCKETS + 1],
// gbase[N_BUCKETS].  P1_THREADS x BATCH_ROWS is swept by main(): bigger batches give longer contiguous runs per
// bucket, smaller ones let several CTAs share an SM and overlap their load, bin and copy phases.
template<int P1_THREADS, uint32_t BATCH_ROWS>
constexpr size_t p1_smem() { return static_cast<size_t>(BATCH_ROWS) * DEGREE * 8 + (3 * N_BUCKETS + 1) * 4 + 64; }

template<int P1_THREADS, uint32_t BATCH_ROWS>
__global__ void __launch_bounds__(P1_THREADS)
partition_kernel(const uint32_t *__restrict__ cols, const float *__restrict__ w, const uint32_t *__restrict__ act,
                 const uint32_t n_act, uint2 *__restrict__ buckets, uint32_t *__restrict__ cursor,
                 float *__restrict__ y, uint32_t *__restrict__ overflowed) {
    constexpr uint32_t BATCH_ENTRIES = BATCH_ROWS * DEGREE;
    constexpr int PER_THREAD = 4 * static_cast<int>((BATCH_ENTRIES / 4 + P1_THREADS - 1) / P1_THREADS);
    extern __shared__ __align__(16) unsigned char smem[];
    uint2 *stage = reinterpret_cast<uint2 *>(smem);
    uint32_t *count = reinterpret_cast<uint32_t *>(smem + static_cast<size_t>(BATCH_ENTRIES) * 8);
    uint32_t *start = count + N_BUCKETS;            // N_BUCKETS + 1
    uint32_t *gbase = start + N_BUCKETS + 1;        // N_BUCKETS
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // this CTA's contiguous share of the active rows, in batches of BATCH_ROWS
    const uint32_t per_cta = (n_act + gridDim.x - 1) / gridDim.x;
    const uint32_t row_begin = min(n_act, blockIdx.x * per_cta), row_end = min(n_act, row_begin + per_cta);

    for (uint32_t r0 = row_begin; r0 < row_end; r0 += BATCH_ROWS) {
        const uint32_t rows_here = min(BATCH_ROWS, row_end - r0);
        const uint32_t groups_here = rows_here * (DEGREE / 4);        // 128-bit groups of the batch
        for (uint32_t b = tid; b < N_BUCKETS; b += P1_THREADS) count[b] = 0;
        __syncthreads();

        // (a) load: thread t takes the 128-bit groups t, t + P1_THREADS, ... of the batch
        uint4 c[PER_THREAD / 4], v[PER_THREAD / 4];
        uint32_t pos[PER_THREAD];
#pragma unroll
        for (int k = 0; k < PER_THREAD / 4; ++k) {
            const uint32_t g = tid + k * P1_THREADS;
            if (g < groups_here) {
                const uint32_t r = g / (DEGREE / 4), in_row = g % (DEGREE / 4);
                const size_t at = static_cast<size_t>(act[r0 + r]) * DEGREE + 4 * in_row;
                c[k] = ldg_stream_u4(cols + at);
                v[k] = ldg_stream_u4(w + at);
            }
        }
        // (b) position of every entry inside its bucket's bin of this batch (integer shared-memory atomics)
#pragma unroll
        for (int k = 0; k < PER_THREAD / 4; ++k) {
            const uint32_t g = tid + k * P1_THREADS;
            if (g < groups_here) {
                pos[4 * k + 0] = atomicAdd(count + (c[k].x >> BUCKET_SHIFT), 1u);
                pos[4 * k + 1] = atomicAdd(count + (c[k].y >> BUCKET_SHIFT), 1u);
                pos[4 * k + 2] = atomicAdd(count + (c[k].z >> BUCKET_SHIFT), 1u);
                pos[4 * k + 3] = atomicAdd(count + (c[k].w >> BUCKET_SHIFT), 1u);
            }
        }
        __syncthreads();
        // (c) bin starts in the staging array (exclusive prefix over the counts, one warp) and room in the
        //     global arrays (one global atomic per bucket and batch)
        if (warp == 0) {
            uint32_t running = 0;
            for (uint32_t b0 = 0; b0 < N_BUCKETS; b0 += 32) {
                const uint32_t b = b0 + lane;
                const uint32_t n = b < N_BUCKETS ? count[b] : 0u;
                uint32_t incl = n;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= static_cast<uint32_t>(o)) incl += t;
                }
                if (b < N_BUCKETS) start[b] = running + incl - n;
                running += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) start[N_BUCKETS] = running;
        }
        for (uint32_t b = tid; b < N_BUCKETS; b += P1_THREADS) {
            const uint32_t n = count[b];
            gbase[b] = n ? atomicAdd(cursor + b, n) : 0u;
        }
        __syncthreads();
        // (d) place the entries into their bins
#pragma unroll
        for (int k = 0; k < PER_THREAD / 4; ++k) {
            const uint32_t g = tid + k * P1_THREADS;
            if (g < groups_here) {
                const uint32_t cc[4] = {c[k].x, c[k].y, c[k].z, c[k].w};
                const uint32_t vv[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t b = cc[e] >> BUCKET_SHIFT;
                    stage[start[b] + pos[4 * k + e]] = make_uint2(cc[e] & (BUCKET_COLS - 1), vv[e]);
                }
            }
        }
        __syncthreads();
        // (e) copy every bin out as one contiguous run; entries beyond a bucket's capacity are reduced into y
        //     directly (correct, slow, and counted)
        for (uint32_t b = warp; b < N_BUCKETS; b += P1_THREADS / 32) {
            const uint32_t s = start[b], n = start[b + 1] - s, g0 = gbase[b];
            for (uint32_t i = lane; i < n; i += 32) {
                const uint2 ent = stage[s + i];
                const uint32_t at = g0 + i;
                if (at < BUCKET_CAP) {
                    buckets[static_cast<size_t>(b) * BUCKET_CAP + at] = ent;
                } else {
                    atomicAdd(y + (b << BUCKET_SHIFT) + ent.x, __uint_as_float(ent.y));
                    atomicAdd(overflowed, 1u);
                }
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------------------
// pass 2: one CTA per bucket accumulates its array in shared memory and adds the slice to y
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024, 1)
accumulate_kernel(const uint2 *__restrict__ buckets, uint32_t *__restrict__ cursor, float *__restrict__ y) {
    __shared__ float acc[BUCKET_COLS];
    const uint32_t b = blockIdx.x;
    for (uint32_t j = threadIdx.x; j < BUCKET_COLS; j += blockDim.x) acc[j] = 0.0f;
    __syncthreads();
    const uint32_t n = min(cursor[b], BUCKET_CAP);
    const uint4 *src = reinterpret_cast<const uint4 *>(buckets + static_cast<size_t>(b) * BUCKET_CAP);   // 2 entries
    for (uint32_t i = threadIdx.x; i < n / 2; i += blockDim.x) {
        const uint4 two = src[i];
        atomicAdd(acc + two.x, __uint_as_float(two.y));
        atomicAdd(acc + two.z, __uint_as_float(two.w));
    }
    if ((n & 1u) && threadIdx.x == 0) {
        const uint2 last = buckets[static_cast<size_t>(b) * BUCKET_CAP + n - 1];
        atomicAdd(acc + last.x, __uint_as_float(last.y));
    }
    __syncthreads();
    const uint32_t col0 = b << BUCKET_SHIFT;
    for (uint32_t j = threadIdx.x; j < BUCKET_COLS; j += blockDim.x)
        if (col0 + j < N_COL) y[col0 + j] += acc[j];      // only this CTA touches these outputs in this pass
    __syncthreads();
    if (threadIdx.x == 0) cursor[b] = 0;                  // ready for the next step
}

struct Buffers {
    const uint32_t *cols; const float *w; const uint32_t *act; uint2 *buckets; uint32_t *cursor; float *y;
    uint32_t *over; cudaEvent_t e0, e1, e2; int sms; float red_ms; const std::vector<float> *yref;
};

// One configuration of the partition kernel: check step 0 against the reduction kernel, then time all steps
// (every step uses different rows, so its matrix data is cold) for a few grid sizes.
template<int P1_THREADS, uint32_t BATCH_ROWS>
void sweep(const Buffers &b) {
    static_assert(N_BUCKETS <= 1024, "bucket tables are sized for at most 1024 buckets");
    constexpr size_t smem = p1_smem<P1_THREADS, BATCH_ROWS>();
    auto kernel = partition_kernel<P1_THREADS, BATCH_ROWS>;
    CK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    int per_sm = 0;
    CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, P1_THREADS, smem));
    if (per_sm < 1) { std::printf("%d threads x %u rows: does not fit an SM\n", P1_THREADS, BATCH_ROWS); return; }

    CK(cudaMemset(b.y, 0, N_COL * 4));
    CK(cudaMemset(b.over, 0, 4));
    kernel<<<b.sms * per_sm, P1_THREADS, smem>>>(b.cols, b.w, b.act, N_ACT, b.buckets, b.cursor, b.y, b.over);
    accumulate_kernel<<<N_BUCKETS, 1024>>>(b.buckets, b.cursor, b.y);
    CK(cudaDeviceSynchronize());
    std::vector<float> y(N_COL);
    uint32_t over = 0;
    CK(cudaMemcpy(y.data(), b.y, N_COL * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(&over, b.over, 4, cudaMemcpyDeviceToHost));
    double worst = 0;
    for (uint32_t j = 0; j < N_COL; ++j) worst = std::max(worst, static_cast<double>(std::fabs(y[j] - (*b.yref)[j])));
    std::printf("%4d threads x %2u rows per batch, %zu KB shared, %d CTAs per SM: max |y - y_ref| = %.3g, overflowed %u -> %s\n",
                P1_THREADS, BATCH_ROWS, smem / 1024, per_sm, worst, over, worst < 1e-3 ? "OK" : "MISMATCH");

    for (int grid : {b.sms * per_sm, b.sms * per_sm * 2}) {
        float best_p1 = 1e9f, best_p2 = 1e9f;
        for (int rep = 0; rep < 3; ++rep)
            for (int k = 0; k < STEPS; ++k) {
                const uint32_t *act = b.act + static_cast<size_t>(k) * N_ACT;
                CK(cudaMemsetAsync(b.y, 0, N_COL * 4));
                CK(cudaEventRecord(b.e0));
                kernel<<<grid, P1_THREADS, smem>>>(b.cols, b.w, act, N_ACT, b.buckets, b.cursor, b.y, b.over);
                CK(cudaEventRecord(b.e1));
                accumulate_kernel<<<N_BUCKETS, 1024>>>(b.buckets, b.cursor, b.y);
                CK(cudaEventRecord(b.e2));
                CK(cudaEventSynchronize(b.e2));
                float p1, p2;
                CK(cudaEventElapsedTime(&p1, b.e0, b.e1));
                CK(cudaEventElapsedTime(&p2, b.e1, b.e2));
                if (p1 + p2 < best_p1 + best_p2) { best_p1 = p1; best_p2 = p2; }
            }
        std::printf("     grid %4d: partition %.1f us + accumulate %.1f us = %.1f us  (%.2fx the reduction kernel)\n", grid,
                    best_p1 * 1e3, best_p2 * 1e3, (best_p1 + best_p2) * 1e3, b.red_ms / (best_p1 + best_p2));
    }
}

int main() {
    int sms = 0;
    CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
    const size_t nse = static_cast<size_t>(POOL_ROWS) * DEGREE;
    std::printf("pool %u rows x %u = %.1f MB per array; %u active rows per step; %u buckets of %u columns, "
                "capacity %u entries each (%.0f MB of bucket arrays); %d SMs\n",
                POOL_ROWS, DEGREE, nse * 4e-6, N_ACT, N_BUCKETS, BUCKET_COLS, BUCKET_CAP,
                static_cast<double>(N_BUCKETS) * BUCKET_CAP * 8e-6, sms);

    // matrix pool: random columns, weights U(0,1), generated on the host with a fixed LCG
    std::vector<uint32_t> h_cols(nse);
    std::vector<float> h_w(nse);
    uint64_t s = 0x9E3779B97F4A7C15ull;
    for (size_t i = 0; i < nse; ++i) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        h_cols[i] = static_cast<uint32_t>((s >> 33) % N_COL);
        h_w[i] = static_cast<float>((s >> 11) & 0xFFFFF) / 1048576.0f;
    }
    std::vector<uint32_t> h_act(static_cast<size_t>(STEPS) * N_ACT);
    for (int k = 0; k < STEPS; ++k)                       // disjoint, ascending active rows per step
        for (uint32_t i = 0; i < N_ACT; ++i) h_act[static_cast<size_t>(k) * N_ACT + i] = (i * STEPS + k) % POOL_ROWS;

    uint32_t *d_cols, *d_act, *d_cursor, *d_over;
    float *d_w, *d_y, *d_yref;
    uint2 *d_buckets;
    CK(cudaMalloc(&d_cols, nse * 4));
    CK(cudaMalloc(&d_w, nse * 4));
    CK(cudaMalloc(&d_act, h_act.size() * 4));
    CK(cudaMalloc(&d_y, N_COL * 4));
    CK(cudaMalloc(&d_yref, N_COL * 4));
    CK(cudaMalloc(&d_buckets, static_cast<size_t>(N_BUCKETS) * BUCKET_CAP * 8));
    CK(cudaMalloc(&d_cursor, N_BUCKETS * 4));
    CK(cudaMalloc(&d_over, 4));
    CK(cudaMemcpy(d_cols, h_cols.data(), nse * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_w, h_w.data(), nse * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_act, h_act.data(), h_act.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemset(d_cursor, 0, N_BUCKETS * 4));
    CK(cudaMemset(d_over, 0, 4));

    cudaEvent_t e0, e1, e2;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1)); CK(cudaEventCreate(&e2));

    // ---- the reduction kernel: reference result of step 0 and its time over all steps ----
    std::vector<float> yref(N_COL);
    CK(cudaMemset(d_yref, 0, N_COL * 4));
    red_scatter_kernel<<<sms * 4, 256>>>(d_cols, d_w, d_act, N_ACT, d_yref);
    CK(cudaMemcpy(yref.data(), d_yref, N_COL * 4, cudaMemcpyDeviceToHost));
    float best_red = 1e9f;
    for (int rep = 0; rep < 3; ++rep)
        for (int k = 0; k < STEPS; ++k) {
            const uint32_t *act = d_act + static_cast<size_t>(k) * N_ACT;
            CK(cudaMemsetAsync(d_yref, 0, N_COL * 4));
            CK(cudaEventRecord(e0));
            red_scatter_kernel<<<sms * 4, 256>>>(d_cols, d_w, act, N_ACT, d_yref);
            CK(cudaEventRecord(e1));
            CK(cudaEventSynchronize(e1));
            float ms;
            CK(cudaEventElapsedTime(&ms, e0, e1));
            best_red = std::min(best_red, ms);
        }
    std::printf("reductions: %.1f us per step\n", best_red * 1e3);

    Buffers buf{d_cols, d_w, d_act, d_buckets, d_cursor, d_y, d_over, e0, e1, e2, sms, best_red, &yref};
    sweep<1024, 16>(buf);
    sweep<512, 8>(buf);
    sweep<256, 4>(buf);
    sweep<256, 2>(buf);
    CK(cudaDeviceSynchronize());
    std::printf("%s\n", cudaGetErrorString(cudaGetLastError()));
    return 0;
}
