// Scatter direction of the CSR products (y += A^T x over a list of rows): one warp per piece of a
// row, 128-bit streaming loads, one `red.global.add` per synapse.  Shared by the stand-alone
// operators and by the sharded step kernel that fuses the spike exchange with the scatter.
#ifndef BPL_CSRC_ROW_SCATTER_CUH_
#define BPL_CSRC_ROW_SCATTER_CUH_

#include "abi.h"
#include "common.cuh"
#include "spike_scan.cuh"

namespace bpl {
namespace {

// ------------------------------------------------------------------------------------------
// Row streaming helpers: 4 consecutive matrix entries at a 16-byte aligned position
// ------------------------------------------------------------------------------------------
template<typename T>
struct Quad { T v[4]; };

__device__ __forceinline__ void load_quad(const float *p, Quad<float> &q) {
    const uint4 u = ldg_stream_u4(p);
    q.v[0] = __uint_as_float(u.x); q.v[1] = __uint_as_float(u.y);
    q.v[2] = __uint_as_float(u.z); q.v[3] = __uint_as_float(u.w);
}
__device__ __forceinline__ void load_quad(const double *p, Quad<double> &q) {
    const uint4 a = ldg_stream_u4(p), b = ldg_stream_u4(p + 2);
    q.v[0] = __hiloint2double(a.y, a.x); q.v[1] = __hiloint2double(a.w, a.z);
    q.v[2] = __hiloint2double(b.y, b.x); q.v[3] = __hiloint2double(b.w, b.z);
}

constexpr int ROW_THREADS = 256;
constexpr int ROW_WARPS = ROW_THREADS / 32;

// How many pieces a row is cut into so that work items stay near 256 entries: keeps the
// last wave of a persistent grid short.  Uniform over the grid (a function of the mean row length).
__device__ __forceinline__ uint32_t pieces_per_row(uint32_t nse, uint32_t n_row) {
    const uint32_t mean = n_row ? nse / n_row : 0;
    const uint32_t s = mean / 320u;
    return s < 1u ? 1u : (s > 16u ? 16u : s);
}

// Boundary h (0..S) of row [start, end) cut into S pieces; interior cuts fall on multiples of 4
// entries so that every piece starts on a 16-byte boundary of the index and weight arrays.
__device__ __forceinline__ uint32_t piece_cut(uint32_t start, uint32_t end, uint32_t h, uint32_t S) {
    if (h == 0) return start;
    if (h >= S) return end;
    const uint64_t c = start + static_cast<uint64_t>(end - start) * h / S;
    const uint64_t r = (c + 3u) & ~static_cast<uint64_t>(3u);
    return static_cast<uint32_t>(r < end ? r : end);
}

// One reduction into y.  ASM_RED = false: `atomicAdd` with the result unused, which the stand-alone kernels
// compile to a reduction (measured at the L2 reduction rate).  ASM_RED = true: the reduction spelled out;
// inside the sharded step kernel the `atomicAdd` form ran at half that rate.
template<bool ASM_RED, typename T>
__device__ __forceinline__ void reduce_into(T *p, T v) {
    if (ASM_RED) red_add(p, v); else atomicAdd(p, v);
}

// One warp scatters entries [a, b) of the matrix: y[indices[e]] += weight(e) * scale.
template<typename T, bool HOMO, bool SCALED, bool VEC, bool ASM_RED>
__device__ __forceinline__ void scatter_span(const uint32_t *__restrict__ indices, const T *__restrict__ data,
                                             const T homo_w, const T scale, const uint32_t a, const uint32_t b,
                                             const uint32_t nse, T *__restrict__ y, const uint32_t lane) {
    if (VEC) {
        const uint32_t g_begin = a >> 2, g_end = (b + 3u) >> 2;   // 4-entry groups touched
        const uint32_t g_full = nse >> 2;                         // groups lying wholly inside the arrays
        for (uint32_t g0 = g_begin; g0 < g_end; g0 += 128u) {
            uint4 ix[4];
            Quad<T> wq[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t g = g0 + lane + 32u * u;
                if (g < g_end && g < g_full) {
                    ix[u] = ldg_stream_u4(indices + 4ull * g);
                    if (!HOMO) load_quad(data + 4ull * g, wq[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t g = g0 + lane + 32u * u;
                if (g >= g_end) continue;
                if (g < g_full) {
                    const uint32_t c[4] = {ix[u].x, ix[u].y, ix[u].z, ix[u].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t pos = 4u * g + e;
                        if (pos >= a && pos < b) {
                            T w = HOMO ? homo_w : wq[u].v[e];
                            if (SCALED) w = w * scale;
                            reduce_into<ASM_RED>(y + c[e], w);
                        }
                    }
                } else {  // ragged tail of the arrays: element-wise
                    for (uint32_t pos = max(4u * g, a); pos < b; ++pos) {
                        T w = HOMO ? homo_w : data[pos];
                        if (SCALED) w = w * scale;
                        reduce_into<ASM_RED>(y + indices[pos], w);
                    }
                }
            }
        }
    } else {
        for (uint32_t pos = a + lane; pos < b; pos += 32u) {
            T w = HOMO ? homo_w : data[pos];
            if (SCALED) w = w * scale;
            reduce_into<ASM_RED>(y + indices[pos], w);
        }
    }
}

// Scatter product over a list of rows.
//   LIST = true : rows come from the compacted spike list (event-driven, scale = 1).
//   LIST = false: every row, scaled by x[row]  (y = A^T x for a dense x).
template<typename T, bool HOMO, bool LIST, bool VEC, bool ASM_RED = false, bool LANE_PARALLEL = false>
__device__ __forceinline__ void
row_scatter_body(const uint32_t *__restrict__ indices, const uint32_t *__restrict__ indptr,
                 const T *__restrict__ data, const T *__restrict__ x, const uint32_t n_row,
                 const uint32_t chunk, const uint32_t n_chunks, const uint32_t *__restrict__ counts,
                 const uint32_t *__restrict__ ids, T *__restrict__ y,
                 uint32_t *prefix /* shared, MAX_CHUNKS + 1 */, uint32_t *warp_total /* shared, ROW_WARPS */,
                 const uint32_t block_index, const uint32_t block_count /* the blocks that share the work */) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t n_list = n_row;
    if (LIST) {
        pdl_wait();                                    // the spike list (and the zeroed y) are ready
        n_list = chunk_prefix(counts, n_chunks, prefix, warp_total);
    }
    if (n_list == 0) return;

    const uint32_t nse = indptr[n_row];
    const uint32_t S = pieces_per_row(nse, n_row);
    const T homo_w = HOMO ? data[0] : T(0);
    const uint64_t n_items = static_cast<uint64_t>(n_list) * S;
    const uint64_t n_warps = static_cast<uint64_t>(block_count) * ROW_WARPS;

    // A warp owns the items first, first + n_warps, ...
    const uint64_t first = static_cast<uint64_t>(block_index) * ROW_WARPS + warp;
    if (!LANE_PARALLEL) {
        // One item at a time: resolve it (list entry -> row -> row pointers -> piece bounds), stream it.  With
        // many long pieces per warp the other warps hide the resolution latency, and this form measured 4 %
        // faster on a million-row matrix (66.2 against 69.2 us per launch on one GPU, same run).
        for (uint64_t item = first; item < n_items; item += n_warps) {
            const uint32_t li = static_cast<uint32_t>(item / S), h = static_cast<uint32_t>(item % S);
            const uint32_t row = LIST ? list_row(prefix, n_chunks, chunk, ids, li) : li;
            const T scale = LIST ? T(1) : x[row];
            const uint32_t start = indptr[row], end = indptr[row + 1];
            const uint32_t a = piece_cut(start, end, h, S), b = piece_cut(start, end, h + 1, S);
            if (a < b) scatter_span<T, HOMO, !LIST, VEC, ASM_RED>(indices, data, homo_w, scale, a, b, nse, y, lane);
        }
        return;
    }
    // LANE_PARALLEL (column shards: a few short pieces per warp, nothing to hide latency behind): the warp
    // resolves up to 32 of its items at once, one per lane, so the dependent loads of all its rows overlap,
    // and then streams the pieces one after the other with all lanes.
    for (uint64_t base = first; base < n_items; base += n_warps * 32u) {
        const uint64_t item = base + static_cast<uint64_t>(lane) * n_warps;
        uint32_t a = 0, b = 0;
        T scale = T(1);
        if (item < n_items) {
            const uint32_t li = static_cast<uint32_t>(item / S), h = static_cast<uint32_t>(item % S);
            const uint32_t row = LIST ? list_row(prefix, n_chunks, chunk, ids, li) : li;
            if (!LIST) scale = x[row];
            const uint32_t start = indptr[row], end = indptr[row + 1];
            a = piece_cut(start, end, h, S);
            b = piece_cut(start, end, h + 1, S);
        }
        const uint64_t left = (n_items - base + n_warps - 1) / n_warps;
        const uint32_t count = left < 32u ? static_cast<uint32_t>(left) : 32u;
        for (uint32_t t = 0; t < count; ++t) {
            const uint32_t ta = __shfl_sync(FULL_MASK, a, t), tb = __shfl_sync(FULL_MASK, b, t);
            const T ts = __shfl_sync(FULL_MASK, scale, t);
            if (ta < tb) scatter_span<T, HOMO, !LIST, VEC, ASM_RED>(indices, data, homo_w, ts, ta, tb, nse, y, lane);
        }
    }
}

template<typename T, bool HOMO, bool LIST, bool VEC, bool LANE_PARALLEL = false>
__global__ void __launch_bounds__(ROW_THREADS)
row_scatter_kernel(const uint32_t *__restrict__ indices, const uint32_t *__restrict__ indptr,
                   const T *__restrict__ data, const T *__restrict__ x, const uint32_t n_row,
                   const uint32_t chunk, const uint32_t n_chunks, const uint32_t *__restrict__ counts,
                   const uint32_t *__restrict__ ids, T *__restrict__ y) {
    __shared__ uint32_t prefix[MAX_CHUNKS + 1];
    __shared__ uint32_t warp_total[ROW_WARPS];
    row_scatter_body<T, HOMO, LIST, VEC, false, LANE_PARALLEL>(indices, indptr, data, x, n_row, chunk, n_chunks, counts,
                                                               ids, y, prefix, warp_total, blockIdx.x, gridDim.x);
}

}  // namespace
}  // namespace bpl

#endif  // BPL_CSRC_ROW_SCATTER_CUH_
