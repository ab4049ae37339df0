// Stored-matrix (CSR) synaptic propagation for sm_100a:
//   event_csr_matvec  (replaces lib/gpu_event_csr_matvec.cu of the reference)
//   csr_matvec        (replaces lib/gpu_csr_matvec.cu) and its transposed form
//   gpu_csr_event_sum (replaces the CSR half of lib/gpu_event_sum.cu)
//
// Scatter direction (y = A^T x, "transpose"): the spike vector is first compacted into a
// list of active rows (scan_events_kernel, which also zero-fills y), then only those rows
// are streamed with 128-bit loads and scattered with one `red.global.add` per synapse
// (row_scatter_kernel).  Homogeneous weights use the same float reductions: k additions
// of one value give the same float in any order, so the result equals the reference's
// sequential sum bit for bit.
//
// Gather direction (y = A x): a sub-warp per row streams the whole matrix with 128-bit
// loads and reduces with shuffles (row_gather_kernel).
#include "abi.h"
#include "common.cuh"
#include "spike_scan.cuh"
#include "row_scatter.cuh"

namespace bpl {
namespace {

// ------------------------------------------------------------------------------------------
// Gather direction: y[r] = sum_j w_j * f(x[col_j]) with a group of `lpr` lanes per row
// ------------------------------------------------------------------------------------------
// EVENT = true : f = truthiness of the event; homogeneous weights count hits and scale once
//                (equal to the reference CPU kernel's float64 accumulation,
//                brainpylib/_src/event_ops/event_csr_matvec.py:334-357).
// EVENT = false: f = x, products accumulated with fused multiply-adds as the reference
//                `sum += data[e] * x[col]` compiles to (lib/gpu_csr_matvec.cu:163).
//
// MASK = true (events only): the block first packs the event vector into a bitmask in shared memory
// (one ballot per 32 events) and tests bits instead of gathering event bytes through L1/L2; the
// whole-matrix stream then runs at HBM speed.  Blocks of 1024 threads, mask of n_col / 8 bytes.
constexpr int GATHER_MASK_THREADS = 1024;
constexpr uint32_t GATHER_MASK_MAX_BITS = 200u * 1024u * 8u;

template<typename T, typename X, bool HOMO, bool EVENT, bool VEC, bool MASK = false>
__global__ void __launch_bounds__(MASK ? GATHER_MASK_THREADS : ROW_THREADS)
row_gather_kernel(const uint32_t *__restrict__ indices, const uint32_t *__restrict__ indptr,
                  const T *__restrict__ data, const X *__restrict__ x, const uint32_t n_row,
                  T *__restrict__ y, const uint32_t n_col = 0) {
    extern __shared__ uint32_t event_mask[];
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warps_per_block = blockDim.x >> 5;
    if (MASK) {
        pack_event_mask(x, n_col, event_mask);
        __syncthreads();
    }
    auto hit = [&](uint32_t col) -> bool {
        if (MASK) return (event_mask[col >> 5] >> (col & 31u)) & 1u;
        return is_event(x[col]);
    };
    const uint32_t nse = indptr[n_row];
    const uint32_t mean = n_row ? nse / n_row : 0;
    // Lanes per row: a lane takes 4 consecutive entries per 128-bit load and up to GATHER_UNROLL such
    // loads per step, so mean / 16 lanes cover an average row in one step.  Few lanes per row means
    // several rows per warp in flight, which is what hides the pointer -> entries -> gather latency
    // chain when rows are short.
    const uint32_t want = (mean + 15u) / 16u;
    const uint32_t lpr = want <= 4u ? 4u : (want <= 8u ? 8u : (want <= 16u ? 16u : 32u));
    const uint32_t rows_per_warp = 32u / lpr;
    const uint32_t sub = lane / lpr, sl = lane % lpr;
    const T homo_w = HOMO ? data[0] : T(0);
    const uint64_t n_warps = static_cast<uint64_t>(gridDim.x) * warps_per_block;
    const uint64_t n_groups = (static_cast<uint64_t>(n_row) + rows_per_warp - 1) / rows_per_warp;
    const uint32_t g_full = nse >> 2;
    constexpr int GATHER_UNROLL = 4;

    for (uint64_t wg = static_cast<uint64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); wg < n_groups;
         wg += n_warps) {
        const uint64_t row64 = wg * rows_per_warp + sub;
        const bool live = row64 < n_row;
        const uint32_t row = live ? static_cast<uint32_t>(row64) : 0u;
        const uint32_t start = live ? indptr[row] : 0u, end = live ? indptr[row + 1] : 0u;
        T acc = T(0);
        uint32_t hits = 0;
        if (VEC) {
            const uint32_t g_begin = start >> 2, g_end = (end + 3u) >> 2;
            for (uint32_t g0 = g_begin + sl; g0 < g_end; g0 += lpr * GATHER_UNROLL) {
                uint4 ix[GATHER_UNROLL];
                Quad<T> wq[GATHER_UNROLL];
#pragma unroll
                for (int u = 0; u < GATHER_UNROLL; ++u) {
                    const uint32_t g = g0 + u * lpr;
                    if (g < g_end && g < g_full) {
                        ix[u] = ldg_stream_u4(indices + 4ull * g);
                        if (!HOMO) load_quad(data + 4ull * g, wq[u]);
                    }
                }
#pragma unroll
                for (int u = 0; u < GATHER_UNROLL; ++u) {
                    const uint32_t g = g0 + u * lpr;
                    if (g >= g_end) continue;
                    if (g < g_full) {
                        const uint32_t c[4] = {ix[u].x, ix[u].y, ix[u].z, ix[u].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t pos = 4u * g + e;
                            if (pos >= start && pos < end) {
                                if (EVENT) {
                                    if (hit(c[e])) { if (HOMO) ++hits; else acc += wq[u].v[e]; }
                                } else {
                                    acc += (HOMO ? homo_w : wq[u].v[e]) * static_cast<T>(x[c[e]]);
                                }
                            }
                        }
                    } else {   // ragged tail of the arrays: element-wise
                        for (uint32_t pos = max(4u * g, start); pos < end; ++pos) {
                            const uint32_t col = indices[pos];
                            if (EVENT) {
                                if (hit(col)) { if (HOMO) ++hits; else acc += data[pos]; }
                            } else {
                                acc += (HOMO ? homo_w : data[pos]) * static_cast<T>(x[col]);
                            }
                        }
                    }
                }
            }
        } else {
            for (uint32_t pos = start + sl; pos < end; pos += lpr) {
                const uint32_t col = indices[pos];
                if (EVENT) {
                    if (hit(col)) { if (HOMO) ++hits; else acc += data[pos]; }
                } else {
                    acc += (HOMO ? homo_w : data[pos]) * static_cast<T>(x[col]);
                }
            }
        }
        if (EVENT && HOMO) {
            hits = group_sum(hits, static_cast<int>(lpr));
            // no hit leaves +0 like an empty sum (the product with a negative weight would give -0)
            acc = hits ? static_cast<T>(static_cast<double>(hits) * static_cast<double>(homo_w)) : T(0);
        } else {
            acc = group_sum(acc, static_cast<int>(lpr));
        }
        if (live && sl == 0) y[row] = acc;
    }
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
inline int persistent_blocks(int blocks_per_sm, uint64_t work_warps) {
    const uint64_t cap = static_cast<uint64_t>(sm_count()) * blocks_per_sm;
    const uint64_t need = (work_warps + ROW_WARPS - 1) / ROW_WARPS;
    return static_cast<int>(need < 1 ? 1 : (need < cap ? need : cap));
}

template<typename T, typename E, bool HOMO>
void event_csr_matvec_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    const TwoUintOneBoolDescriptor *d = unpack<TwoUintOneBoolDescriptor>(opaque, opaque_len);
    if (!d) return;
    const uint32_t n_row = d->uint_x, n_col = d->uint_y;
    const T *data = static_cast<const T *>(buffers[0]);
    const uint32_t *indices = static_cast<const uint32_t *>(buffers[1]);
    const uint32_t *indptr = static_cast<const uint32_t *>(buffers[2]);
    const E *events = static_cast<const E *>(buffers[3]);
    T *y = static_cast<T *>(buffers[4]);
    const bool vec = aligned16(indices) && (HOMO || aligned16(data));

    if (d->bool_x) {
        if (n_col == 0) return;
        uint32_t *ws = static_cast<uint32_t *>(buffers[5]);
        if (ws == nullptr) {
            set_status(BPL_ERR_ARGUMENT, "event_csr_matvec(transpose=True) needs a workspace buffer");
            return;
        }
        uint32_t *counts = ws, *ids = ws + MAX_CHUNKS;
        const ScanPlan p = plan_scan(n_row);
        const uint64_t zero_blocks = (static_cast<uint64_t>(n_col) + SCAN_TILE - 1) / SCAN_TILE;
        const uint64_t zero_cap = static_cast<uint64_t>(sm_count()) * 8;
        const uint32_t scan_grid = static_cast<uint32_t>(
            max(static_cast<uint64_t>(p.n_chunks), min(zero_blocks, zero_cap)));
        scan_events_kernel<T, E><<<scan_grid, SCAN_THREADS, 0, stream>>>(
            events, n_row, p.chunk, p.n_chunks, y, n_col, counts, ids);
        if (!launch_ok()) return;
        if (n_row == 0) return;
        // one warp per work item; the grid is sized for the worst case (every row active) but capped
        // four blocks per SM are resident; for large matrices four times as many are launched: with more blocks than
        // the SMs hold the L2 reductions spread better (1e7 synapses per call: 70.3 us with 4 per SM, 64.3 with 16,
        // 66.8 with 32).  Small matrices keep one wave: every block prefix-sums the chunk counts first, which a
        // launch-bound call (4000 rows: 6.6 us) would pay several times over (9.1 us).
        const int grid = persistent_blocks(n_row >= 262144u ? 16 : 4, static_cast<uint64_t>(n_row) * 16);
        if (profile_before()) cudaEventRecord(profile_before(), stream);
        // a dependent launch behind the scan: the blocks are resident and wait only where they first read the list
        const cudaError_t e =
            vec ? launch_dependent(row_scatter_kernel<T, HOMO, true, true>, dim3(grid), dim3(ROW_THREADS), 0, stream, indices,
                                   indptr, data, static_cast<const T *>(nullptr), n_row, p.chunk, p.n_chunks, counts, ids, y)
                : launch_dependent(row_scatter_kernel<T, HOMO, true, false>, dim3(grid), dim3(ROW_THREADS), 0, stream,
                                   indices, indptr, data, static_cast<const T *>(nullptr), n_row, p.chunk, p.n_chunks, counts,
                                   ids, y);
        if (e != cudaSuccess) set_status(BPL_ERR_CUDA, cudaGetErrorString(e));
        if (profile_after()) cudaEventRecord(profile_after(), stream);
        launch_ok();
    } else {
        if (n_row == 0) return;
        if (vec && n_col >= 8192u && n_col <= GATHER_MASK_MAX_BITS && n_row >= 4096u) {
            const size_t smem = static_cast<size_t>((n_col + 31u) >> 5) * 4;
            static thread_local int configured_device = -1;
            int dev = 0;
            cudaGetDevice(&dev);
            if (configured_device != dev) {
                if (cudaFuncSetAttribute(row_gather_kernel<T, E, HOMO, true, true, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(GATHER_MASK_MAX_BITS / 8)) != cudaSuccess) {
                    launch_ok();
                    return;
                }
                configured_device = dev;
            }
            const int per_sm = smem <= 100u * 1024u ? 2 : 1;
            const uint64_t need = (static_cast<uint64_t>(n_row) + GATHER_MASK_THREADS / 32 - 1) / (GATHER_MASK_THREADS / 32);
            const uint64_t cap = static_cast<uint64_t>(sm_count()) * per_sm;
            const int grid = static_cast<int>(need < cap ? need : cap);
            row_gather_kernel<T, E, HOMO, true, true, true><<<grid, GATHER_MASK_THREADS, smem, stream>>>(
                indices, indptr, data, events, n_row, y, n_col);
            launch_ok();
            return;
        }
        const int grid = persistent_blocks(8, n_row);
        if (vec)
            row_gather_kernel<T, E, HOMO, true, true><<<grid, ROW_THREADS, 0, stream>>>(
                indices, indptr, data, events, n_row, y);
        else
            row_gather_kernel<T, E, HOMO, true, false><<<grid, ROW_THREADS, 0, stream>>>(
                indices, indptr, data, events, n_row, y);
        launch_ok();
    }
}

template<typename T, bool HOMO>
void csr_matvec_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len,
                     bool transpose, int vector_slot) {
    const DoubleSizeDescriptor *d = unpack<DoubleSizeDescriptor>(opaque, opaque_len);
    if (!d) return;
    const uint32_t n_row = d->size_x, n_col = d->size_y;
    const T *data = static_cast<const T *>(buffers[0]);
    const uint32_t *indices = static_cast<const uint32_t *>(buffers[1]);
    const uint32_t *indptr = static_cast<const uint32_t *>(buffers[2]);
    const T *x = static_cast<const T *>(buffers[vector_slot]);
    T *y = static_cast<T *>(buffers[vector_slot + 1]);
    const bool vec = aligned16(indices) && (HOMO || aligned16(data));

    if (transpose) {
        if (n_col == 0) return;
        if (cudaMemsetAsync(y, 0, sizeof(T) * static_cast<size_t>(n_col), stream) != cudaSuccess) {
            launch_ok();
            return;
        }
        if (n_row == 0) return;
        // more blocks than the SMs hold: the L2 reductions spread better (1e7 entries: 74.9 us with 4 blocks per SM,
        // 66.5 with 16, 64.9 with 32: the reduction floor)
        const int grid = persistent_blocks(32, static_cast<uint64_t>(n_row) * 16);
        if (vec)
            row_scatter_kernel<T, HOMO, false, true><<<grid, ROW_THREADS, 0, stream>>>(
                indices, indptr, data, x, n_row, 0, 0, nullptr, nullptr, y);
        else
            row_scatter_kernel<T, HOMO, false, false><<<grid, ROW_THREADS, 0, stream>>>(
                indices, indptr, data, x, n_row, 0, 0, nullptr, nullptr, y);
    } else {
        if (n_row == 0) return;
        const int grid = persistent_blocks(8, n_row);
        if (vec)
            row_gather_kernel<T, T, HOMO, false, true><<<grid, ROW_THREADS, 0, stream>>>(
                indices, indptr, data, x, n_row, y);
        else
            row_gather_kernel<T, T, HOMO, false, false><<<grid, ROW_THREADS, 0, stream>>>(
                indices, indptr, data, x, n_row, y);
    }
    launch_ok();
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {

size_t bpl_event_csr_workspace_bytes(uint32_t n_row, int transpose) {
    return transpose ? scatter_workspace_bytes(n_row) : 0;
}

#define EVENT_CSR_TARGET(name, T, E, HOMO) \
    void name(bpl_stream_t s, void **b, const char *o, size_t n) { event_csr_matvec_impl<T, E, HOMO>(s, b, o, n); }

EVENT_CSR_TARGET(event_csr_matvec_homo_float_bool, float, uint8_t, true)
EVENT_CSR_TARGET(event_csr_matvec_homo_float_float, float, float, true)
EVENT_CSR_TARGET(event_csr_matvec_homo_double_bool, double, uint8_t, true)
EVENT_CSR_TARGET(event_csr_matvec_homo_double_double, double, double, true)
EVENT_CSR_TARGET(event_csr_matvec_heter_float_bool, float, uint8_t, false)
EVENT_CSR_TARGET(event_csr_matvec_heter_float_float, float, float, false)
EVENT_CSR_TARGET(event_csr_matvec_heter_double_bool, double, uint8_t, false)
EVENT_CSR_TARGET(event_csr_matvec_heter_double_double, double, double, false)

// The reference's scalar / vector / adaptive methods (lib/gpu_csr_matvec.cu) differ only in
// how rows are mapped to threads; here all three names run the same kernel.  'adaptive'
// carries its row_blocks operand at slot 3, which is ignored.
#define CSR_TARGET(name, T, HOMO, TRANSPOSE, SLOT) \
    void name(bpl_stream_t s, void **b, const char *o, size_t n) { csr_matvec_impl<T, HOMO>(s, b, o, n, TRANSPOSE, SLOT); }

CSR_TARGET(csr_matvec_homo_scalar_float, float, true, false, 3)
CSR_TARGET(csr_matvec_homo_scalar_double, double, true, false, 3)
CSR_TARGET(csr_matvec_homo_vector_float, float, true, false, 3)
CSR_TARGET(csr_matvec_homo_vector_double, double, true, false, 3)
CSR_TARGET(csr_matvec_homo_adaptive_float, float, true, false, 4)
CSR_TARGET(csr_matvec_homo_adaptive_double, double, true, false, 4)
CSR_TARGET(csr_matvec_heter_scalar_float, float, false, false, 3)
CSR_TARGET(csr_matvec_heter_scalar_double, double, false, false, 3)
CSR_TARGET(csr_matvec_heter_vector_float, float, false, false, 3)
CSR_TARGET(csr_matvec_heter_vector_double, double, false, false, 3)
CSR_TARGET(csr_matvec_heter_adaptive_float, float, false, false, 4)
CSR_TARGET(csr_matvec_heter_adaptive_double, double, false, false, 4)
CSR_TARGET(csr_matvec_transpose_homo_float, float, true, true, 3)
CSR_TARGET(csr_matvec_transpose_homo_double, double, true, true, 3)
CSR_TARGET(csr_matvec_transpose_heter_float, float, false, true, 3)
CSR_TARGET(csr_matvec_transpose_heter_double, double, false, true, 3)

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Transposed event product that allocates nothing and takes no workspace buffer
// ------------------------------------------------------------------------------------------
// Who needs it: a caller that runs as an XLA custom call (or inside any framework's stream
// capture) receives exactly the buffers the framework planned for it and must not call
// cudaMalloc itself: allocation is illegal while a stream is being captured, synchronises
// the device, and takes memory behind the back of the framework's own allocator.  The
// regular targets solve this by asking for one extra workspace buffer; a caller that cannot
// even declare that extra buffer (it must keep the reference's exact five-buffer list) can
// use this entry point instead.  Its scratch (the compacted spike list) lives in a
// file-scope device array of fixed size, so the number of matrix rows is limited.
//
// Cost and rules of the fixed array:
//  * every GPU that loads this library holds BPL_NOALLOC_MAX_ROWS * 4 + 4096 bytes (about
//    8.4 MB) from the first use of the library on that GPU until the process exits;
//  * all calls on one GPU share it.  Nothing in it has to start at zero (every word that is
//    read was written earlier in the same call), so stale contents of an earlier call are
//    harmless, but two calls that overlap on the GPU (different streams, no ordering between
//    them) race on it and give wrong results: keep such calls on one stream or order them;
//  * the first call on a device looks the array's device address up (cudaGetSymbolAddress,
//    with that device current).  That one call should be made before any stream capture
//    begins; later calls only launch kernels.
constexpr uint32_t NOALLOC_MAX_ROWS = 1u << 21;   // 2,097,152 rows
static __device__ __align__(256) uint32_t g_noalloc_scratch[MAX_CHUNKS + NOALLOC_MAX_ROWS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
uint32_t *g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the current device.  In host code the array's name
// is only a handle for the runtime, not a pointer a kernel could use.
uint32_t *noalloc_scratch_address() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
        set_status(BPL_ERR_CUDA, "no-allocation entry point: cannot identify the current device");
        return nullptr;
    }
    uint32_t *p = __atomic_load_n(&g_noalloc_ptr[dev], __ATOMIC_ACQUIRE);
    if (p != nullptr) return p;
    void *addr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&addr, g_noalloc_scratch);
    if (e != cudaSuccess || addr == nullptr) {
        set_status(BPL_ERR_CUDA, e != cudaSuccess ? cudaGetErrorString(e) : "cudaGetSymbolAddress returned null");
        return nullptr;
    }
    // a racing first call on another host thread stores the same address
    __atomic_store_n(&g_noalloc_ptr[dev], static_cast<uint32_t *>(addr), __ATOMIC_RELEASE);
    return static_cast<uint32_t *>(addr);
}
}  // namespace

extern "C" {

uint32_t bpl_noalloc_max_rows(void) { return NOALLOC_MAX_ROWS; }

// y = A^T events for heterogeneous float32 weights and float32 events, transpose only.
// buffers: [data f32(nse), indices u32(nse), indptr u32(n_row+1), events f32(n_row), y f32(n_col)]
// opaque : TwoUintOneBoolDescriptor{n_row, n_col, transpose = true}
void event_csr_matvec_heter_float_float_noalloc(bpl_stream_t stream, void **buffers, const char *opaque,
                                                size_t opaque_len) {
    const TwoUintOneBoolDescriptor *d = unpack<TwoUintOneBoolDescriptor>(opaque, opaque_len);
    if (!d) return;
    if (!d->bool_x) {
        set_status(BPL_ERR_ARGUMENT, "the no-allocation entry point computes transpose=True only");
        return;
    }
    const uint32_t n_row = d->uint_x, n_col = d->uint_y;
    if (n_row > NOALLOC_MAX_ROWS) {
        set_status(BPL_ERR_TOO_LARGE,
                   "event_csr_matvec_heter_float_float_noalloc: more than 2097152 matrix rows; "
                   "use event_csr_matvec_heter_float_float with a workspace buffer");
        return;
    }
    if (n_col == 0) return;
    uint32_t *scratch = noalloc_scratch_address();
    if (scratch == nullptr) return;
    const float *data = static_cast<const float *>(buffers[0]);
    const uint32_t *indices = static_cast<const uint32_t *>(buffers[1]);
    const uint32_t *indptr = static_cast<const uint32_t *>(buffers[2]);
    const float *events = static_cast<const float *>(buffers[3]);
    float *y = static_cast<float *>(buffers[4]);
    uint32_t *counts = scratch, *ids = scratch + MAX_CHUNKS;

    const ScanPlan p = plan_scan(n_row);
    const uint64_t zero_blocks = (static_cast<uint64_t>(n_col) + SCAN_TILE - 1) / SCAN_TILE;
    const uint64_t zero_cap = static_cast<uint64_t>(sm_count()) * 8;
    const uint32_t scan_grid = static_cast<uint32_t>(
        max(static_cast<uint64_t>(p.n_chunks), min(zero_blocks, zero_cap)));
    scan_events_kernel<float, float><<<scan_grid, SCAN_THREADS, 0, stream>>>(
        events, n_row, p.chunk, p.n_chunks, y, n_col, counts, ids);
    if (!launch_ok() || n_row == 0) return;
    const int grid = persistent_blocks(4, static_cast<uint64_t>(n_row) * 16);
    if (aligned16(indices) && aligned16(data))
        row_scatter_kernel<float, false, true, true><<<grid, ROW_THREADS, 0, stream>>>(
            indices, indptr, data, nullptr, n_row, p.chunk, p.n_chunks, counts, ids, y);
    else
        row_scatter_kernel<float, false, true, false><<<grid, ROW_THREADS, 0, stream>>>(
            indices, indptr, data, nullptr, n_row, p.chunk, p.n_chunks, counts, ids, y);
    launch_ok();
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Transposed event product driven by a ready-made spike list (no counterpart in the reference)
// ------------------------------------------------------------------------------------------
// The scatter half of event_csr_matvec_heter_float_* on its own, for callers that already hold the
// compacted spike list in the layout of the workspace (counts[1024], then row ids in 4096-entry chunk
// segments): the multi-GPU exchange assembles exactly that on every rank.  y must be zero-filled by
// the caller (the exchange's wait does it).
//   buffers [data f32(nse), indices u32(nse), indptr u32(n_row + 1), list u32, y f32(n_col)]
//   opaque  TripleSizeDescriptor{n_row, n_col, n_chunks}
extern "C" void event_csr_matvec_list_heter_float(bpl_stream_t stream, void **buffers, const char *opaque,
                                                  size_t opaque_len) {
    struct Triple { unsigned int n_row, n_col, n_chunks; };
    const Triple *d = unpack<Triple>(opaque, opaque_len);
    if (!d) return;
    if (d->n_chunks > static_cast<unsigned int>(MAX_CHUNKS)) {
        set_status(BPL_ERR_ARGUMENT, "spike list: more than 1024 chunks");
        return;
    }
    if (d->n_row == 0 || d->n_col == 0 || d->n_chunks == 0) return;
    const float *data = static_cast<const float *>(buffers[0]);
    const uint32_t *indices = static_cast<const uint32_t *>(buffers[1]);
    const uint32_t *indptr = static_cast<const uint32_t *>(buffers[2]);
    const uint32_t *list = static_cast<const uint32_t *>(buffers[3]);
    float *y = static_cast<float *>(buffers[4]);
    const int grid = persistent_blocks(4, static_cast<uint64_t>(d->n_row) * 16);
    if (profile_before()) cudaEventRecord(profile_before(), stream);
    if (aligned16(indices) && aligned16(data))
        row_scatter_kernel<float, false, true, true, true><<<grid, ROW_THREADS, 0, stream>>>(
            indices, indptr, data, nullptr, d->n_row, SCAN_TILE, d->n_chunks, list, list + MAX_CHUNKS, y);
    else
        row_scatter_kernel<float, false, true, false, true><<<grid, ROW_THREADS, 0, stream>>>(
            indices, indptr, data, nullptr, d->n_row, SCAN_TILE, d->n_chunks, list, list + MAX_CHUNKS, y);
    if (profile_after()) cudaEventRecord(profile_after(), stream);
    launch_ok();
}
