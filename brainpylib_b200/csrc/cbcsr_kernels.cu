// Transposed event product on a column-blocked matrix (no counterpart in the reference).
//
// Why a second format: on a plain CSR matrix every active synapse costs one scattered
// `red.global.add` = one 32-byte L2 sector operation, and the L2 of a B200 retires about 155 G of
// them per second - 64 us for the 1e7 synapses of a 1 %-firing step of a 1e6 x 1000 network, while
// the same bytes stream from HBM in 11 us.  Here a CTA keeps one block of y in shared memory and
// accumulates there; see cb_scatter.cuh for the format and the kernel, cbcsr_build.cu for the
// builder.
//
//   event_cbcsr_matvec_heter_float_{bool,float}
//   opaque  {u32 n_row, u32 n_col, u32 block_width, i32 fixed_point, i32 scale_log2, u32 team_lanes_log2}
//           (bpl_build_cbcsr_descriptor).  fixed_point = 0: float accumulators; 1: 32-bit fixed point with
//           2^scale_log2 units per 1.0.  team_lanes_log2 = 2..5: a (row, block) segment is copied by 4, 8, 16 or 32
//           lanes, up to that many groups per round; pick the smallest that covers most segments.
//   buffers [groups u8(48 * n_groups), offsets u32(n_row, n_blocks + 1), events E(n_row), y f32(n_col), workspace]
//   workspace: as for event_csr_matvec with transpose (4 KB + 4 B per row): the compacted spike list
#include <type_traits>

#include "abi.h"
#include "common.cuh"
#include "spike_scan.cuh"
#include "cb_scatter.cuh"

namespace bpl {
namespace {

struct TripleSizeDescriptor {   // same layout as the reference's (lib/kernel_helper_descriptor.cuh:125-129)
    unsigned int size_x, size_y, size_z;
};
struct CbDescriptor {
    unsigned int n_row, n_col, block_width;
    int fixed_point, scale_log2;
    unsigned int team_lanes_log2;   // 2..5: lanes (and groups per round) a segment gets; 0 = 2
};
static_assert(sizeof(CbDescriptor) == 24, "layout");

// Optional phase stamps of the next launches made by this host thread (see cb_stamp): 8 words per CTA.
thread_local unsigned long long *g_cb_trace = nullptr;

template<int NBUF, bool FIXED, int LOG_L>
__global__ void __launch_bounds__(CB_THREADS, 1)
event_cb_scatter_kernel(const unsigned char *__restrict__ groups, const uint32_t *__restrict__ offsets,
                        const uint32_t n_col, const uint32_t width, const uint32_t n_blocks, const uint32_t P,
                        const uint32_t chunk, const uint32_t n_chunks, const uint32_t *__restrict__ counts,
                        const uint32_t *__restrict__ ids, float *__restrict__ y, const uint32_t acc_bytes,
                        const float inv_scale, unsigned long long *__restrict__ trace) {
    extern __shared__ __align__(128) unsigned char cb_smem[];
    __shared__ uint32_t prefix[MAX_CHUNKS + 1];
    __shared__ uint32_t warp_total[CB_WARPS];
    cb_scatter_body<NBUF, FIXED, LOG_L>(groups, offsets, n_col, width, n_blocks, blockIdx.x / P, blockIdx.x % P, P, chunk,
                                        n_chunks, counts, ids, y, acc_bytes, cb_smem, prefix, warp_total, inv_scale, trace,
                                        blockIdx.x);
}

// y = A^T x for a dense float vector x on the same storage: every row with x[row] != 0 is walked, weights scaled by x[row].
// GATHER: y = A x instead: the block's slice of x sits in shared memory, a team sums a row's segment against it.
template<int NBUF, int LOG_L, bool GATHER>
__global__ void __launch_bounds__(CB_THREADS, 1)
dense_cb_scatter_kernel(const unsigned char *__restrict__ groups, const uint32_t *__restrict__ offsets,
                        const uint32_t n_row, const uint32_t n_col, const uint32_t width, const uint32_t n_blocks,
                        const uint32_t P, const float *__restrict__ x, float *__restrict__ y, const uint32_t acc_bytes) {
    extern __shared__ __align__(128) unsigned char cb_smem[];
    __shared__ uint32_t prefix[2];            // unused by the dense walk
    __shared__ uint32_t warp_total[CB_WARPS];
    cb_scatter_body<NBUF, false, LOG_L, true, GATHER>(groups, offsets, n_col, width, n_blocks, blockIdx.x / P,
                                                      blockIdx.x % P, P, 0, n_row, nullptr, nullptr, y, acc_bytes, cb_smem,
                                                      prefix, warp_total, 1.0f, nullptr, 0, x);
}

using CbDenseKernel = void (*)(const unsigned char *, const uint32_t *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
                               const float *, float *, uint32_t);
template<int NBUF, bool GATHER>
CbDenseKernel cb_dense_kernel_for_lanes(uint32_t log_l) {
    switch (log_l) {
        case 3: return dense_cb_scatter_kernel<NBUF, 3, GATHER>;
        case 4: return dense_cb_scatter_kernel<NBUF, 4, GATHER>;
        case 5: return dense_cb_scatter_kernel<NBUF, 5, GATHER>;
        default: return dense_cb_scatter_kernel<NBUF, 2, GATHER>;
    }
}
CbDenseKernel cb_dense_kernel(uint32_t n_buf, uint32_t log_l, bool gather) {
    if (gather) return n_buf == 3 ? cb_dense_kernel_for_lanes<3, true>(log_l) : cb_dense_kernel_for_lanes<2, true>(log_l);
    return n_buf == 3 ? cb_dense_kernel_for_lanes<3, false>(log_l) : cb_dense_kernel_for_lanes<2, false>(log_l);
}

using CbKernel = void (*)(const unsigned char *, const uint32_t *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
                          const uint32_t *, const uint32_t *, float *, uint32_t, float, unsigned long long *);

template<int NBUF, bool FIXED>
CbKernel cb_kernel_for_lanes(uint32_t log_l) {
    switch (log_l) {
        case 3: return event_cb_scatter_kernel<NBUF, FIXED, 3>;
        case 4: return event_cb_scatter_kernel<NBUF, FIXED, 4>;
        case 5: return event_cb_scatter_kernel<NBUF, FIXED, 5>;
        default: return event_cb_scatter_kernel<NBUF, FIXED, 2>;
    }
}
CbKernel cb_kernel(uint32_t n_buf, bool fixed, uint32_t log_l) {
    if (n_buf == 3) return fixed ? cb_kernel_for_lanes<3, true>(log_l) : cb_kernel_for_lanes<3, false>(log_l);
    return fixed ? cb_kernel_for_lanes<2, true>(log_l) : cb_kernel_for_lanes<2, false>(log_l);
}

bool cb_kernel_configured() {
    static thread_local int configured_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_device != dev) {
        for (uint32_t n_buf = 2; n_buf <= 3; ++n_buf)
            for (int fixed = 0; fixed < 2; ++fixed)
                for (uint32_t log_l = 2; log_l <= 5; ++log_l)
                    if (cudaFuncSetAttribute(cb_kernel(n_buf, fixed != 0, log_l), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(CB_SMEM_LIMIT)) != cudaSuccess) {
                        launch_ok();
                        return false;
                    }
        configured_device = dev;
    }
    return true;
}

// CTAs that share one column block (each takes every P-th active row), so that all SMs work.
inline uint32_t cb_shares(uint32_t n_blocks) {
    const uint32_t P = static_cast<uint32_t>(sm_count()) / (n_blocks ? n_blocks : 1u);
    return P < 1 ? 1u : (P > 32 ? 32u : P);
}

// E = void: the spike list is an operand (buffers [groups, offsets, list, y]; y must already be zero) instead of
// being compacted from an event vector here.
template<typename E>
void event_cbcsr_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    constexpr bool FROM_LIST = std::is_void<E>::value;
    const CbDescriptor *d = unpack<CbDescriptor>(opaque, opaque_len);
    if (!d) return;
    const uint32_t n_row = d->n_row, n_col = d->n_col, width = d->block_width;
    if (d->fixed_point != 0 && (d->scale_log2 < -100 || d->scale_log2 > 100)) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: scale_log2 must be in -100..100");
        return;
    }
    const float inv_scale = d->fixed_point ? ldexpf(1.0f, -d->scale_log2) : 1.0f;
    if (width == 0 || width > CB_MAX_WIDTH || (width & 31u) != 0) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: block_width must be a multiple of 32 in 32..32256");
        return;
    }
    if (d->team_lanes_log2 != 0 && (d->team_lanes_log2 < 2 || d->team_lanes_log2 > 5)) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: team_lanes_log2 must be 2..5");
        return;
    }
    if (n_col == 0) return;
    const uint32_t n_blocks = (n_col + width - 1) / width;
    if (n_blocks > CB_MAX_BLOCKS) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: more than 1024 column blocks");
        return;
    }
    const unsigned char *groups = static_cast<const unsigned char *>(buffers[0]);
    const uint32_t *offsets = static_cast<const uint32_t *>(buffers[1]);
    float *y = static_cast<float *>(buffers[3]);
    uint32_t *ws = static_cast<uint32_t *>(FROM_LIST ? buffers[2] : buffers[4]);
    if (ws == nullptr) {
        set_status(BPL_ERR_ARGUMENT, FROM_LIST ? "event_cbcsr_matvec_list needs a spike list"
                                               : "event_cbcsr_matvec needs a workspace buffer");
        return;
    }
    if (!aligned16(groups)) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: the group array must be 16-byte aligned");
        return;
    }
    uint32_t *counts = ws, *ids = ws + MAX_CHUNKS;
    const ScanPlan p = plan_scan(n_row);
    const uint64_t zero_blocks = (static_cast<uint64_t>(n_col) + SCAN_TILE - 1) / SCAN_TILE;
    const uint64_t zero_cap = static_cast<uint64_t>(sm_count()) * 8;
    const uint32_t scan_grid = static_cast<uint32_t>(max(static_cast<uint64_t>(p.n_chunks), min(zero_blocks, zero_cap)));
    if constexpr (!FROM_LIST) {
        scan_events_kernel<float, E><<<scan_grid, SCAN_THREADS, 0, stream>>>(static_cast<const E *>(buffers[2]), n_row,
                                                                             p.chunk, p.n_chunks, y, n_col, counts, ids);
        if (!launch_ok()) return;
    }
    (void) scan_grid;
    if (n_row == 0) return;
    const uint32_t P = cb_shares(n_blocks);
    if (!cb_kernel_configured()) return;
    const CbPlan plan = cb_plan(width);
    if (!plan.ok) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: block_width leaves no shared memory for the copy buffers");
        return;
    }
    const uint32_t log_l = d->team_lanes_log2 == 0 ? 2u : d->team_lanes_log2;
    if (profile_before()) cudaEventRecord(profile_before(), stream);
    // behind the scan of this call the scatter is a dependent launch: it clears its slice while the scan still runs
    const cudaError_t e = launch_dependent(cb_kernel(plan.n_buf, d->fixed_point != 0, log_l), dim3(n_blocks * P),
                                           dim3(CB_THREADS), plan.smem_bytes, stream, groups, offsets, n_col, width,
                                           n_blocks, P, p.chunk, p.n_chunks, counts, ids, y, plan.acc_bytes, inv_scale,
                                           g_cb_trace);
    if (e != cudaSuccess) set_status(BPL_ERR_CUDA, cudaGetErrorString(e));
    if (profile_after()) cudaEventRecord(profile_after(), stream);
    launch_ok();
}

// gather = false: y(n_col) = A^T x(n_row); gather = true: y(n_row) = A x(n_col)
void cbcsr_matvec_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len, const bool gather) {
    const CbDescriptor *d = unpack<CbDescriptor>(opaque, opaque_len);
    if (!d) return;
    const uint32_t n_row = d->n_row, n_col = d->n_col, width = d->block_width;
    if (d->fixed_point != 0) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: the dense-vector product needs float weights (not fixed point)");
        return;
    }
    if (width == 0 || width > CB_MAX_WIDTH || (width & 31u) != 0) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: block_width must be a multiple of 32 in 32..32256");
        return;
    }
    if (d->team_lanes_log2 != 0 && (d->team_lanes_log2 < 2 || d->team_lanes_log2 > 5)) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: team_lanes_log2 must be 2..5");
        return;
    }
    if (n_col == 0) {
        if (gather && n_row != 0 && cudaMemsetAsync(buffers[3], 0, sizeof(float) * static_cast<size_t>(n_row), stream) != cudaSuccess)
            launch_ok();
        return;
    }
    const uint32_t n_blocks = (n_col + width - 1) / width;
    if (n_blocks > CB_MAX_BLOCKS) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: more than 1024 column blocks");
        return;
    }
    const unsigned char *groups = static_cast<const unsigned char *>(buffers[0]);
    const uint32_t *offsets = static_cast<const uint32_t *>(buffers[1]);
    const float *x = static_cast<const float *>(buffers[2]);
    float *y = static_cast<float *>(buffers[3]);
    if (!aligned16(groups)) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: the group array must be 16-byte aligned");
        return;
    }
    const size_t n_out = gather ? n_row : n_col;
    if (n_out != 0 && cudaMemsetAsync(y, 0, sizeof(float) * n_out, stream) != cudaSuccess) {
        launch_ok();
        return;
    }
    if (n_row == 0) return;
    const CbPlan plan = cb_plan(width);
    if (!plan.ok) {
        set_status(BPL_ERR_ARGUMENT, "column-blocked matrix: block_width leaves no shared memory for the copy buffers");
        return;
    }
    static thread_local int configured_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_device != dev) {
        for (uint32_t n_buf = 2; n_buf <= 3; ++n_buf)
            for (uint32_t log_l = 2; log_l <= 5; ++log_l)
                for (int g = 0; g < 2; ++g)
                    if (cudaFuncSetAttribute(cb_dense_kernel(n_buf, log_l, g != 0),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(CB_SMEM_LIMIT)) != cudaSuccess) {
                        launch_ok();
                        return;
                    }
        configured_device = dev;
    }
    const uint32_t P = cb_shares(n_blocks);
    const uint32_t log_l = d->team_lanes_log2 == 0 ? 2u : d->team_lanes_log2;
    if (profile_before()) cudaEventRecord(profile_before(), stream);
    cb_dense_kernel(plan.n_buf, log_l, gather)<<<n_blocks * P, CB_THREADS, plan.smem_bytes, stream>>>(
        groups, offsets, n_row, n_col, width, n_blocks, P, x, y, plan.acc_bytes);
    if (profile_after()) cudaEventRecord(profile_after(), stream);
    launch_ok();
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {

// y = A^T x for a dense float32 vector x on the column-blocked storage (no counterpart in the reference, which takes
// this product from cuSPARSE): buffers [groups, offsets, x f32(n_row), y f32(n_col)]; opaque as event_cbcsr_matvec_*
// with fixed_point = 0.
void cbcsr_matvec_transpose_heter_float(bpl_stream_t s, void **b, const char *o, size_t n) {
    cbcsr_matvec_impl(s, b, o, n, false);
}
// y = A x on the same storage: buffers [groups, offsets, x f32(n_col), y f32(n_row)].  The block's slice of x is staged
// in shared memory, so the gathers of x never leave the SM.
void cbcsr_matvec_heter_float(bpl_stream_t s, void **b, const char *o, size_t n) {
    cbcsr_matvec_impl(s, b, o, n, true);
}

void event_cbcsr_matvec_heter_float_bool(bpl_stream_t s, void **b, const char *o, size_t n) {
    event_cbcsr_impl<uint8_t>(s, b, o, n);
}
void event_cbcsr_matvec_heter_float_float(bpl_stream_t s, void **b, const char *o, size_t n) {
    event_cbcsr_impl<float>(s, b, o, n);
}
// The scatter alone, from a ready-made spike list (the layout of the workspace: counts[1024], then row ids in chunk
// segments of bpl-defined size for n_row rows), e.g. the one lif_exp_step_float writes.  y must already be zero.
//   buffers [groups, offsets, list u32, y f32(n_col)]; opaque as above
void event_cbcsr_matvec_list_heter_float(bpl_stream_t s, void **b, const char *o, size_t n) {
    event_cbcsr_impl<void>(s, b, o, n);
}

// Debugging aid: while `buffer` (device memory, 64 bytes per CTA of the launch) is not null, every
// event_cbcsr_matvec_* launch of this host thread stamps its phases into it with the global nanosecond timer.
void bpl_cbcsr_trace(void *buffer) { g_cb_trace = static_cast<unsigned long long *>(buffer); }

size_t bpl_build_cbcsr_descriptor(uint32_t n_row, uint32_t n_col, uint32_t block_width, int fixed_point,
                                  int scale_log2, uint32_t team_lanes_log2, void *out, size_t cap) {
    if (out == nullptr || cap < sizeof(CbDescriptor)) return 0;
    const CbDescriptor d{n_row, n_col, block_width, fixed_point, scale_log2, team_lanes_log2};
    __builtin_memcpy(out, &d, sizeof(d));
    return sizeof(d);
}

size_t bpl_build_triple_size_descriptor(uint32_t size_x, uint32_t size_y, uint32_t size_z, void *out, size_t cap) {
    if (out == nullptr || cap < sizeof(TripleSizeDescriptor)) return 0;
    const TripleSizeDescriptor d{size_x, size_y, size_z};
    __builtin_memcpy(out, &d, sizeof(d));
    return sizeof(d);
}

}  // extern "C"
