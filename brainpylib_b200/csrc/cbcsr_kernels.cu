// Transposed event product on a column-blocked CSR matrix (no counterpart in the reference).
//
// Why a second format: on a plain CSR matrix every active synapse costs one scattered
// `red.global.add` = one 32-byte L2 sector operation, and the L2 of a B200 retires about 155 G of
// them per second - 64 us for the 1e7 synapses of a 1 %-firing step of a 1e6 x 1000 network, while
// the same 80 MB stream from HBM in 11 us.  Here the post-synaptic neurons are cut into blocks of
// at most 45056 columns.  The matrix stays row-major (a CSR row keeps its place), but inside a row
// the synapses are grouped by block, with 16-bit local column ids, and a per-row table
// offsets[row][0..n_blocks] says where each block's group starts.  A CTA owns one block's slice of
// y in shared memory, walks the active rows, reads only its block's group of each row, accumulates
// with shared-memory atomics (which do not touch L2) and flushes the slice once with coalesced
// reductions.  The groups of one row lie side by side and are read by the CTAs of the different
// blocks within microseconds of each other, so HBM delivers each row once and L2 hands the pieces
// out.  `P` CTAs share a block, each taking every P-th active row, so that all SMs work; the flush
// then costs P * n_col / 8 sector operations instead of one per synapse.
//
//   event_cbcsr_matvec_heter_float_{bool,float}
//   opaque  {u32 n_row, u32 n_col, u32 block_width}
//   buffers [data f32(nse), cols u16(nse), offsets u32(n_row, n_blocks + 1), events E(n_row), y f32(n_col), workspace]
//   workspace: as for event_csr_matvec with transpose (4 KB + 4 B per row): the compacted spike list
#include "abi.h"
#include "common.cuh"
#include "spike_scan.cuh"

namespace bpl {
namespace {

constexpr int CB_THREADS = 1024;
constexpr int CB_WARPS = CB_THREADS / 32;
constexpr int CB_ROW_CACHE = 4096;      // active rows per pass whose pointer pairs are held in shared memory
constexpr int CB_UNROLL = 8;            // rows in flight per warp
constexpr uint32_t CB_MAX_WIDTH = 45056;

struct TripleSizeDescriptor {   // same layout as the reference's (lib/kernel_helper_descriptor.cuh:125-129)
    unsigned int size_x, size_y, size_z;
};

__global__ void __launch_bounds__(CB_THREADS, 1)
event_cb_scatter_kernel(const float *__restrict__ data, const uint16_t *__restrict__ cols,
                        const uint32_t *__restrict__ offsets, const uint32_t n_row, const uint32_t n_col,
                        const uint32_t width, const uint32_t P, const uint32_t chunk, const uint32_t n_chunks,
                        const uint32_t *__restrict__ counts, const uint32_t *__restrict__ ids, float *__restrict__ y) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *acc = reinterpret_cast<float *>(smem_raw);                           // [width]
    uint2 *seg = reinterpret_cast<uint2 *>(smem_raw + static_cast<size_t>(width) * 4);   // [CB_ROW_CACHE]
    __shared__ uint32_t prefix[MAX_CHUNKS + 1];
    __shared__ uint32_t warp_total[CB_WARPS];

    const uint32_t b = blockIdx.x / P, p = blockIdx.x % P;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t col0 = b * width;
    const uint32_t my_width = min(width, n_col - col0);
    for (uint32_t j = threadIdx.x; j < my_width; j += CB_THREADS) acc[j] = 0.0f;

    const uint32_t n_act = chunk_prefix(counts, n_chunks, prefix, warp_total);   // ends with a barrier
    const uint32_t mine = n_act > p ? (n_act - p + P - 1) / P : 0;               // rows p, p + P, ...
    const uint32_t n_blocks = (n_col + width - 1) / width;
    const uint64_t stride = static_cast<uint64_t>(n_blocks) + 1;

    for (uint32_t base = 0; base < mine; base += CB_ROW_CACHE) {
        const uint32_t n_here = min(static_cast<uint32_t>(CB_ROW_CACHE), mine - base);
        // phase 1: every thread resolves a few of this pass's rows (list entry -> row -> pointer pair);
        // the dependent loads of all rows of the pass are in flight together
        for (uint32_t j = threadIdx.x; j < n_here; j += CB_THREADS) {
            const uint32_t row = list_row(prefix, n_chunks, chunk, ids, p + (base + j) * P);
            const uint32_t *o = offsets + row * stride + b;
            seg[j] = make_uint2(o[0], o[1]);
        }
        __syncthreads();
        // phase 2: a warp takes CB_UNROLL rows at a time, one lane per synapse of a segment: all loads of the
        // batch are issued, then the shared-memory atomics.  (Issuing the next batch's loads before the
        // atomics, more rows per batch, or fewer and fatter warps all measured slower: the accumulation is
        // bound by shared-memory float atomics, ~3.4 per clock per SM, and overlaps best across many warps.)
        for (uint32_t j0 = warp * CB_UNROLL; j0 < n_here; j0 += CB_WARPS * CB_UNROLL) {
            uint32_t c[CB_UNROLL];
            float w[CB_UNROLL];
            uint32_t live = 0u;   // bit u: this lane holds a synapse of row u; bit 16 + u: row u is longer than a warp
#pragma unroll
            for (int u = 0; u < CB_UNROLL; ++u) {
                if (j0 + u < n_here) {
                    const uint2 sg = seg[j0 + u];
                    const uint32_t e = sg.x + lane;
                    if (e < sg.y) {
                        c[u] = cols[e];
                        w[u] = __uint_as_float(ldg_stream_u32(data + e));
                        live |= 1u << u;
                    }
                    if (sg.y - sg.x > 32u) live |= 0x10000u << u;
                }
            }
#pragma unroll
            for (int u = 0; u < CB_UNROLL; ++u)
                if (live & (1u << u)) atomicAdd(acc + c[u], w[u]);
            if (live >> 16) {   // segments longer than a warp (uniform across the warp)
#pragma unroll
                for (int u = 0; u < CB_UNROLL; ++u)
                    if (live & (0x10000u << u)) {
                        const uint2 sg = seg[j0 + u];
                        for (uint32_t e = sg.x + 32u + lane; e < sg.y; e += 32u) atomicAdd(acc + cols[e], data[e]);
                    }
            }
        }
        __syncthreads();
    }
    // flush the slice: coalesced reductions, P CTAs add into the same zero-filled y
    if (mine > 0)
        for (uint32_t j = threadIdx.x; j < my_width; j += CB_THREADS) {
            const float v = acc[j];
            if (v != 0.0f) atomicAdd(y + col0 + j, v);
        }
}

template<typename E>
void event_cbcsr_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    const TripleSizeDescriptor *d = unpack<TripleSizeDescriptor>(opaque, opaque_len);
    if (!d) return;
    const uint32_t n_row = d->size_x, n_col = d->size_y, width = d->size_z;
    if (width == 0 || width > CB_MAX_WIDTH) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked CSR: block_width must be in 1..45056");
        return;
    }
    if (n_col == 0) return;
    const float *data = static_cast<const float *>(buffers[0]);
    const uint16_t *cols = static_cast<const uint16_t *>(buffers[1]);
    const uint32_t *offsets = static_cast<const uint32_t *>(buffers[2]);
    const E *events = static_cast<const E *>(buffers[3]);
    float *y = static_cast<float *>(buffers[4]);
    uint32_t *ws = static_cast<uint32_t *>(buffers[5]);
    if (ws == nullptr) {
        set_status(BPL_ERR_ARGUMENT, "event_cbcsr_matvec needs a workspace buffer");
        return;
    }
    uint32_t *counts = ws, *ids = ws + MAX_CHUNKS;
    const ScanPlan p = plan_scan(n_row);
    const uint64_t zero_blocks = (static_cast<uint64_t>(n_col) + SCAN_TILE - 1) / SCAN_TILE;
    const uint64_t zero_cap = static_cast<uint64_t>(sm_count()) * 8;
    const uint32_t scan_grid = static_cast<uint32_t>(max(static_cast<uint64_t>(p.n_chunks), min(zero_blocks, zero_cap)));
    scan_events_kernel<float, E><<<scan_grid, SCAN_THREADS, 0, stream>>>(events, n_row, p.chunk, p.n_chunks, y, n_col,
                                                                         counts, ids);
    if (!launch_ok() || n_row == 0) return;

    const uint32_t n_blocks = (n_col + width - 1) / width;
    uint32_t P = static_cast<uint32_t>(sm_count()) / n_blocks;
    P = P < 1 ? 1 : (P > 8 ? 8 : P);
    const size_t smem = static_cast<size_t>(width) * 4 + static_cast<size_t>(CB_ROW_CACHE) * sizeof(uint2);
    static thread_local int configured_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_device != dev) {
        if (cudaFuncSetAttribute(event_cb_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(CB_MAX_WIDTH * 4 + CB_ROW_CACHE * sizeof(uint2))) != cudaSuccess) {
            launch_ok();
            return;
        }
        configured_device = dev;
    }
    event_cb_scatter_kernel<<<n_blocks * P, CB_THREADS, smem, stream>>>(
        data, cols, offsets, n_row, n_col, width, P, p.chunk, p.n_chunks, counts, ids, y);
    launch_ok();
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {

void event_cbcsr_matvec_heter_float_bool(bpl_stream_t s, void **b, const char *o, size_t n) {
    event_cbcsr_impl<uint8_t>(s, b, o, n);
}
void event_cbcsr_matvec_heter_float_float(bpl_stream_t s, void **b, const char *o, size_t n) {
    event_cbcsr_impl<float>(s, b, o, n);
}

size_t bpl_build_triple_size_descriptor(uint32_t size_x, uint32_t size_y, uint32_t size_z, void *out, size_t cap) {
    if (out == nullptr || cap < sizeof(TripleSizeDescriptor)) return 0;
    const TripleSizeDescriptor d{size_x, size_y, size_z};
    __builtin_memcpy(out, &d, sizeof(d));
    return sizeof(d);
}

}  // extern "C"
