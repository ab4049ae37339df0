// Builder of the column-blocked matrix format (cb_scatter.cuh) from a CSR matrix, on the GPU.
//
// Takes the place of the host-side layout step of the reference (brainpylib/_src/sparse_ops/utils.py:21-51
// builds CSR from COO with host array code) for the one layout this library adds.  A column range
// [col_lo, col_hi) can be given: synapses outside it are dropped and columns are re-based to col_lo,
// which yields one rank's shard of a matrix that is partitioned by post-synaptic neuron.
//
// Two calls, because the size of the result is only known after the first:
//   bpl_cbcsr_plan   counts, per row and column block, the groups of 8 synapses (one warp per row, a
//                    histogram in shared memory), writes them as row-relative offsets, and prefix-sums the
//                    row totals; the total number of groups lands in the first 8 bytes of the workspace.
//   bpl_cbcsr_fill   re-bases the offsets and places every synapse: the order inside a (row, block)
//                    segment is the CSR order (ranks from __match_any_sync, no atomics), so the layout is a
//                    fixed function of the input.  Padding synapses are zero (the array is cleared first).
#include "abi.h"
#include "common.cuh"
#include "cb_scatter.cuh"

namespace bpl {
namespace {

constexpr int BUILD_THREADS = 256;
constexpr int BUILD_WARPS = BUILD_THREADS / 32;
constexpr uint32_t SCAN_ROWS = 4096;   // rows per block of the row-total prefix sum (1024 threads x 4)

// workspace: [0] u64 total groups, [1 .. 1 + n_scan_blocks] u64 block bases, then u32 row totals / row starts
inline uint32_t scan_blocks(uint32_t n_row) { return (n_row + SCAN_ROWS - 1) / SCAN_ROWS; }
inline size_t build_workspace_bytes(uint32_t n_row) {
    return (2 + static_cast<size_t>(scan_blocks(n_row))) * 8 + static_cast<size_t>(n_row) * 4 + 16;
}
inline uint64_t *ws_block_base(void *ws) { return static_cast<uint64_t *>(ws) + 1; }
inline uint32_t *ws_row_start(void *ws, uint32_t n_row) {
    return reinterpret_cast<uint32_t *>(static_cast<uint64_t *>(ws) + 2 + scan_blocks(n_row));
}

// One warp per row: groups per block, row-relative exclusive offsets, row total.
__global__ void __launch_bounds__(BUILD_THREADS)
cb_count_kernel(const uint32_t *__restrict__ indices, const uint32_t *__restrict__ indptr, const uint32_t n_row,
                const uint32_t col_lo, const uint32_t col_hi, const uint32_t width, const uint32_t n_blocks,
                uint32_t *__restrict__ offsets, uint32_t *__restrict__ row_total) {
    extern __shared__ uint32_t hist_all[];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t *hist = hist_all + warp * n_blocks;
    const uint64_t stride = static_cast<uint64_t>(n_blocks) + 1;
    for (uint64_t row = static_cast<uint64_t>(blockIdx.x) * BUILD_WARPS + warp; row < n_row;
         row += static_cast<uint64_t>(gridDim.x) * BUILD_WARPS) {
        for (uint32_t b = lane; b < n_blocks; b += 32) hist[b] = 0;
        __syncwarp();
        const uint32_t start = indptr[row], end = indptr[row + 1];
        for (uint32_t e = start + lane; e < end; e += 32) {
            const uint32_t c = ldg_stream_u32(indices + e);
            if (c >= col_lo && c < col_hi) atomicAdd(hist + (c - col_lo) / width, 1u);
        }
        __syncwarp();
        uint32_t run = 0;
        for (uint32_t b0 = 0; b0 < n_blocks; b0 += 32) {
            const uint32_t b = b0 + lane;
            const uint32_t g = b < n_blocks ? (hist[b] + 7u) >> 3 : 0u;
            uint32_t incl = g;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(FULL_MASK, incl, o);
                if (lane >= static_cast<uint32_t>(o)) incl += t;
            }
            if (b < n_blocks) offsets[row * stride + b] = run + incl - g;
            run += __shfl_sync(FULL_MASK, incl, 31);
        }
        if (lane == 0) {
            offsets[row * stride + n_blocks] = run;
            row_total[row] = run;
        }
        __syncwarp();
    }
}

// Block-wide inclusive scan of one value per thread (1024 threads); returns the inclusive value, total in *total.
__device__ __forceinline__ uint64_t block_scan_1024(uint64_t v, uint64_t *warp_sums, uint64_t *total) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint64_t incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint64_t t = __shfl_up_sync(FULL_MASK, incl, o);
        if (lane >= static_cast<uint32_t>(o)) incl += t;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    uint64_t base = 0, all = 0;
    for (uint32_t w = 0; w < 32; ++w) {
        const uint64_t t = warp_sums[w];
        if (w < warp) base += t;
        all += t;
    }
    __syncthreads();
    *total = all;
    return base + incl;
}

__global__ void __launch_bounds__(1024)
cb_block_sum_kernel(const uint32_t *__restrict__ row_total, const uint32_t n_row, uint64_t *__restrict__ block_sum) {
    __shared__ uint64_t warp_sums[32];
    const uint64_t first = static_cast<uint64_t>(blockIdx.x) * SCAN_ROWS + threadIdx.x * 4ull;
    uint64_t s = 0;
    for (int k = 0; k < 4; ++k)
        if (first + k < n_row) s += row_total[first + k];
    uint64_t total;
    block_scan_1024(s, warp_sums, &total);
    if (threadIdx.x == 0) block_sum[blockIdx.x] = total;
}

// One CTA turns the block sums into exclusive bases (in place) and writes the grand total.
__global__ void __launch_bounds__(1024)
cb_scan_blocks_kernel(uint64_t *__restrict__ block_sum, const uint32_t n_blocks_scan, uint64_t *__restrict__ grand_total) {
    __shared__ uint64_t warp_sums[32];
    uint64_t run = 0;
    for (uint32_t b0 = 0; b0 < n_blocks_scan; b0 += 1024) {
        const uint32_t b = b0 + threadIdx.x;
        const uint64_t v = b < n_blocks_scan ? block_sum[b] : 0ull;
        uint64_t total;
        const uint64_t incl = block_scan_1024(v, warp_sums, &total);
        if (b < n_blocks_scan) block_sum[b] = run + incl - v;
        run += total;
    }
    if (threadIdx.x == 0) *grand_total = run;
}

// Row totals -> exclusive row starts (in place).
__global__ void __launch_bounds__(1024)
cb_scan_rows_kernel(uint32_t *__restrict__ row_total, const uint32_t n_row, const uint64_t *__restrict__ block_base) {
    __shared__ uint64_t warp_sums[32];
    const uint64_t first = static_cast<uint64_t>(blockIdx.x) * SCAN_ROWS + threadIdx.x * 4ull;
    uint32_t v[4];
    uint64_t s = 0;
    for (int k = 0; k < 4; ++k) {
        v[k] = first + k < n_row ? row_total[first + k] : 0u;
        s += v[k];
    }
    uint64_t total;
    const uint64_t incl = block_scan_1024(s, warp_sums, &total);
    uint64_t run = block_base[blockIdx.x] + incl - s;
    for (int k = 0; k < 4; ++k) {
        if (first + k < n_row) row_total[first + k] = static_cast<uint32_t>(run);
        run += v[k];
    }
}

// One warp per row: re-base the row's offsets, then place its synapses.
template<bool HOMO, bool FIXED>
__global__ void __launch_bounds__(BUILD_THREADS)
cb_fill_kernel(const float *__restrict__ data, const uint32_t *__restrict__ indices, const uint32_t *__restrict__ indptr,
               const uint32_t n_row, const uint32_t col_lo, const uint32_t col_hi, const uint32_t width,
               const uint32_t n_blocks, uint32_t *__restrict__ offsets, const uint32_t *__restrict__ row_start,
               unsigned char *__restrict__ groups, const float scale /* FIXED: units per 1.0 */) {
    extern __shared__ uint32_t cursor_all[];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t *cursor = cursor_all + warp * n_blocks;   // next free synapse slot of each segment, relative to the row
    const uint64_t stride = static_cast<uint64_t>(n_blocks) + 1;
    const float homo_w = HOMO ? data[0] : 0.0f;
    for (uint64_t row = static_cast<uint64_t>(blockIdx.x) * BUILD_WARPS + warp; row < n_row;
         row += static_cast<uint64_t>(gridDim.x) * BUILD_WARPS) {
        const uint32_t base = row_start[row];
        for (uint32_t b = lane; b <= n_blocks; b += 32) {
            const uint32_t rel = offsets[row * stride + b];
            offsets[row * stride + b] = rel + base;
            if (b < n_blocks) cursor[b] = rel * 8u;
        }
        __syncwarp();
        const uint32_t start = indptr[row], end = indptr[row + 1];
        for (uint32_t e0 = start; e0 < end; e0 += 32) {
            const uint32_t e = e0 + lane;
            const bool valid = e < end;
            const uint32_t c = valid ? ldg_stream_u32(indices + e) : 0u;
            const bool in = valid && c >= col_lo && c < col_hi;
            const uint32_t b = in ? (c - col_lo) / width : 0u;
            const uint32_t members = __ballot_sync(FULL_MASK, in);
            uint32_t pos = 0, peers = 0;
            if (in) {
                peers = __match_any_sync(members, b);
                pos = cursor[b] + __popc(peers & ((1u << lane) - 1u));
            }
            __syncwarp();
            if (in && (peers >> lane) == 1u) cursor[b] += __popc(peers);   // the highest lane of each set updates
            __syncwarp();
            if (in) {
                const uint64_t slot = static_cast<uint64_t>(base) * 8u + pos;
                unsigned char *g = groups + (slot >> 3) * CB_GROUP_BYTES;
                const uint32_t k = static_cast<uint32_t>(slot & 7u);
                const float w = HOMO ? homo_w : data[e];
                if (FIXED) reinterpret_cast<int *>(g)[k] = __float2int_rn(w * scale);
                else reinterpret_cast<float *>(g)[k] = w;
                reinterpret_cast<uint16_t *>(g + 32)[k] = static_cast<uint16_t>(c - col_lo - b * width);
            }
        }
        __syncwarp();
    }
}

// Sum of |w| per kept column (float reductions), then the largest of them as float bits (non-negative floats
// order like their bit patterns): what bounds any column's accumulator when every row spikes.
template<bool HOMO>
__global__ void __launch_bounds__(256)
cb_column_abs_sum_kernel(const float *__restrict__ data, const uint32_t *__restrict__ indices, const uint64_t nse,
                         const uint32_t col_lo, const uint32_t col_hi, float *__restrict__ colsum) {
    const float homo_w = HOMO ? fabsf(data[0]) : 0.0f;
    for (uint64_t e = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; e < nse;
         e += static_cast<uint64_t>(gridDim.x) * 256) {
        const uint32_t c = ldg_stream_u32(indices + e);
        if (c >= col_lo && c < col_hi) red_add(colsum + (c - col_lo), HOMO ? homo_w : fabsf(data[e]));
    }
}
__global__ void __launch_bounds__(256)
cb_max_kernel(const float *__restrict__ colsum, const uint32_t n, uint32_t *__restrict__ max_bits) {
    uint32_t m = 0;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; i < n; i += static_cast<uint64_t>(gridDim.x) * 256) {
        const float v = colsum[i];
        const uint32_t bits = (v == v) ? __float_as_uint(v) : 0x7f800000u;   // NaN counts as infinity
        m = max(m, bits);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(FULL_MASK, m, o));
    if ((threadIdx.x & 31) == 0 && m != 0) atomicMax(max_bits, m);
}

bool build_arguments_ok(uint32_t col_lo, uint32_t col_hi, uint32_t width, uint32_t *n_blocks) {
    if (col_hi < col_lo || width == 0 || width > CB_MAX_WIDTH || (width & 31u) != 0) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked build: block_width must be a multiple of 32 in 32..32256 "
                                     "and col_lo <= col_hi");
        return false;
    }
    const uint64_t nb = (static_cast<uint64_t>(col_hi - col_lo) + width - 1) / width;
    if (nb > CB_MAX_BLOCKS) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked build: more than 1024 column blocks; use a wider block");
        return false;
    }
    *n_blocks = nb < 1 ? 1u : static_cast<uint32_t>(nb);
    return true;
}

inline int build_grid(uint32_t n_row) {
    const uint64_t need = (static_cast<uint64_t>(n_row) + BUILD_WARPS - 1) / BUILD_WARPS;
    const uint64_t cap = static_cast<uint64_t>(sm_count()) * 8;
    return static_cast<int>(need < 1 ? 1 : (need < cap ? need : cap));
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {

size_t bpl_cbcsr_build_workspace_bytes(uint32_t n_row) { return build_workspace_bytes(n_row); }

uint32_t bpl_cbcsr_n_blocks(uint32_t n_col, uint32_t block_width) {
    if (block_width == 0) return 0;
    const uint64_t nb = (static_cast<uint64_t>(n_col) + block_width - 1) / block_width;
    return nb < 1 ? 1u : static_cast<uint32_t>(nb);
}

void bpl_cbcsr_plan(bpl_stream_t stream, const void *indices, const void *indptr, uint32_t n_row, uint32_t col_lo,
                    uint32_t col_hi, uint32_t block_width, void *offsets, void *workspace) {
    uint32_t n_blocks = 0;
    if (!build_arguments_ok(col_lo, col_hi, block_width, &n_blocks)) return;
    // `indices` may be null: a matrix without entries has none
    if (workspace == nullptr || (n_row != 0 && (indptr == nullptr || offsets == nullptr))) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked build: null row pointers, offsets or workspace");
        return;
    }
    uint64_t *total = static_cast<uint64_t *>(workspace);
    if (n_row == 0) {
        cudaMemsetAsync(total, 0, 8, stream);
        launch_ok();
        return;
    }
    uint32_t *row_total = ws_row_start(workspace, n_row);
    const size_t smem = static_cast<size_t>(BUILD_WARPS) * n_blocks * 4;
    cb_count_kernel<<<build_grid(n_row), BUILD_THREADS, smem, stream>>>(
        static_cast<const uint32_t *>(indices), static_cast<const uint32_t *>(indptr), n_row, col_lo, col_hi,
        block_width, n_blocks, static_cast<uint32_t *>(offsets), row_total);
    if (!launch_ok()) return;
    const uint32_t nsb = scan_blocks(n_row);
    cb_block_sum_kernel<<<nsb, 1024, 0, stream>>>(row_total, n_row, ws_block_base(workspace));
    cb_scan_blocks_kernel<<<1, 1024, 0, stream>>>(ws_block_base(workspace), nsb, total);
    cb_scan_rows_kernel<<<nsb, 1024, 0, stream>>>(row_total, n_row, ws_block_base(workspace));
    launch_ok();
}

// Largest column sum of |w| over the kept columns -> max_out[0] (float32).  colsum: scratch, col_hi - col_lo floats.
void bpl_cbcsr_max_column_abs_sum(bpl_stream_t stream, const void *data, int homogeneous, const void *indices,
                                  uint64_t nse, uint32_t col_lo, uint32_t col_hi, void *colsum, void *max_out) {
    if (col_hi < col_lo || max_out == nullptr || (col_hi > col_lo && colsum == nullptr) ||
        (nse != 0 && (data == nullptr || indices == nullptr))) {
        set_status(BPL_ERR_ARGUMENT, "column sums: null operand or col_lo > col_hi");
        return;
    }
    const uint32_t n = col_hi - col_lo;
    cudaMemsetAsync(max_out, 0, 4, stream);
    if (n == 0 || nse == 0) { launch_ok(); return; }
    cudaMemsetAsync(colsum, 0, static_cast<size_t>(n) * 4, stream);
    const uint64_t need = (nse + 255) / 256;
    const uint64_t cap = static_cast<uint64_t>(sm_count()) * 16;
    const int grid = static_cast<int>(need < cap ? need : cap);
    if (homogeneous)
        cb_column_abs_sum_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const float *>(data),
            static_cast<const uint32_t *>(indices), nse, col_lo, col_hi, static_cast<float *>(colsum));
    else
        cb_column_abs_sum_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const float *>(data),
            static_cast<const uint32_t *>(indices), nse, col_lo, col_hi, static_cast<float *>(colsum));
    const uint64_t need2 = (static_cast<uint64_t>(n) + 255) / 256;
    cb_max_kernel<<<static_cast<int>(need2 < cap ? need2 : cap), 256, 0, stream>>>(
        static_cast<const float *>(colsum), n, static_cast<uint32_t *>(max_out));
    launch_ok();
}

void bpl_cbcsr_fill(bpl_stream_t stream, const void *data, int homogeneous, const void *indices, const void *indptr,
                    uint32_t n_row, uint32_t col_lo, uint32_t col_hi, uint32_t block_width, void *offsets,
                    const void *workspace, void *groups, uint64_t n_groups, int fixed_point, int scale_log2) {
    uint32_t n_blocks = 0;
    if (!build_arguments_ok(col_lo, col_hi, block_width, &n_blocks)) return;
    if (n_groups >= (1ull << 32)) {
        set_status(BPL_ERR_TOO_LARGE, "column-blocked build: 2^32 or more groups of 8 synapses");
        return;
    }
    if (n_row == 0 || n_groups == 0) return;
    if (data == nullptr || indices == nullptr || indptr == nullptr || offsets == nullptr || workspace == nullptr ||
        groups == nullptr || !aligned16(groups)) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked build: null operand, or a group array that is not 16-byte aligned");
        return;
    }
    if (cudaMemsetAsync(groups, 0, n_groups * CB_GROUP_BYTES, stream) != cudaSuccess) {
        launch_ok();
        return;
    }
    const uint32_t *row_start = ws_row_start(const_cast<void *>(workspace), n_row);
    const size_t smem = static_cast<size_t>(BUILD_WARPS) * n_blocks * 4;
    if (fixed_point && (scale_log2 < -100 || scale_log2 > 100)) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked build: scale_log2 must be in -100..100");
        return;
    }
    const float scale = fixed_point ? ldexpf(1.0f, scale_log2) : 1.0f;
#define BPL_FILL(HOMO, FIXED)                                                                                    \
    cb_fill_kernel<HOMO, FIXED><<<build_grid(n_row), BUILD_THREADS, smem, stream>>>(                             \
        static_cast<const float *>(data), static_cast<const uint32_t *>(indices),                                \
        static_cast<const uint32_t *>(indptr), n_row, col_lo, col_hi, block_width, n_blocks,                     \
        static_cast<uint32_t *>(offsets), row_start, static_cast<unsigned char *>(groups), scale)
    if (homogeneous) { if (fixed_point) BPL_FILL(true, true); else BPL_FILL(true, false); }
    else             { if (fixed_point) BPL_FILL(false, true); else BPL_FILL(false, false); }
#undef BPL_FILL
    launch_ok();
}

}  // extern "C"
