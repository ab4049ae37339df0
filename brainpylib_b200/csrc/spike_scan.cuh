// Spike compaction shared by the transposed event products: the event vector becomes a list of
// active rows (ascending, deterministic, no atomics) plus per-chunk counts, and the output vector
// is zero-filled in the same launch.
#ifndef BPL_CSRC_SPIKE_SCAN_CUH_
#define BPL_CSRC_SPIKE_SCAN_CUH_

#include "abi.h"
#include "common.cuh"

namespace bpl {
namespace {

// ------------------------------------------------------------------------------------------
// Spike compaction
// ------------------------------------------------------------------------------------------
constexpr int SCAN_THREADS = 256;
constexpr int SCAN_WARP_SPAN = 512;                                   // events per warp per tile
constexpr int SCAN_TILE = (SCAN_THREADS / 32) * SCAN_WARP_SPAN;       // 4096 events per block per tile
constexpr int MAX_CHUNKS = 1024;                                      // chunk = what one block compacts

struct ScanPlan {
    uint32_t chunk;     // events per chunk, a multiple of SCAN_TILE
    uint32_t n_chunks;  // <= MAX_CHUNKS
};

inline ScanPlan plan_scan(uint32_t n_row) {
    const uint64_t tiles = (static_cast<uint64_t>(n_row) + SCAN_TILE - 1) / SCAN_TILE;
    const uint64_t tiles_per_chunk = tiles == 0 ? 1 : (tiles + MAX_CHUNKS - 1) / MAX_CHUNKS;
    ScanPlan p;
    p.chunk = static_cast<uint32_t>(tiles_per_chunk * SCAN_TILE);
    p.n_chunks = static_cast<uint32_t>((static_cast<uint64_t>(n_row) + p.chunk - 1) / p.chunk);
    return p;
}

// Workspace of the transposed event product: counts[MAX_CHUNKS] then ids[n_row] (uint32).
// Chunk c owns ids[c * chunk, (c + 1) * chunk): its active rows, ascending, counts[c] of them.
// Nothing in it needs initialising and no atomics are used, so the list is a fixed function
// of the events (ascending row order).
inline size_t scatter_workspace_bytes(uint32_t n_row) {
    return (static_cast<size_t>(MAX_CHUNKS) + n_row) * sizeof(uint32_t);
}

template<typename T, typename E>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_events_kernel(const E *__restrict__ events, const uint32_t n_row, const uint32_t chunk,
                   const uint32_t n_chunks, T *__restrict__ y, const uint32_t n_out,
                   uint32_t *__restrict__ counts, uint32_t *__restrict__ ids) {
    pdl_launch_dependents();   // the scatter behind this kernel may set itself up now; it waits before reading the list
    // (1) zero-fill the output (the reference does it with a cudaMemset on the wrong stream,
    //     lib/gpu_event_csr_matvec.cu:170).
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * SCAN_THREADS + threadIdx.x; i < n_out;
         i += static_cast<uint64_t>(gridDim.x) * SCAN_THREADS)
        y[i] = T(0);

    if (blockIdx.x >= n_chunks) return;

    // (2) compact this block's chunk.  A warp reads 512 consecutive events as 16 coalesced
    //     loads; each ballot is one word of the natural-order bitmap.
    __shared__ uint32_t warp_total[SCAN_THREADS / 32];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t chunk_begin = static_cast<uint64_t>(blockIdx.x) * chunk;
    const uint64_t chunk_end = min(chunk_begin + chunk, static_cast<uint64_t>(n_row));
    uint32_t *out = ids + chunk_begin;
    uint32_t running = 0;

    for (uint64_t tile = chunk_begin; tile < chunk_end; tile += SCAN_TILE) {
        const uint64_t base = tile + static_cast<uint64_t>(warp) * SCAN_WARP_SPAN;
        bool act[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const uint64_t i = base + k * 32 + lane;
            act[k] = (i < chunk_end) && is_event(events[i]);
        }
        uint32_t bits[16];
        uint32_t total = 0;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            bits[k] = __ballot_sync(FULL_MASK, act[k]);
            total += __popc(bits[k]);
        }
        if (lane == 0) warp_total[warp] = total;
        __syncthreads();
        uint32_t offset = running, tile_total = 0;
#pragma unroll
        for (int w = 0; w < SCAN_THREADS / 32; ++w) {
            const uint32_t t = warp_total[w];
            if (w < static_cast<int>(warp)) offset += t;
            tile_total += t;
        }
        __syncthreads();
        const uint32_t below = (1u << lane) - 1u;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            if (act[k]) out[offset + __popc(bits[k] & below)] = static_cast<uint32_t>(base + k * 32 + lane);
            offset += __popc(bits[k]);
        }
        running += tile_total;
    }
    if (threadIdx.x == 0) counts[blockIdx.x] = running;
}


// Exclusive prefix over the chunk counts into shared memory (prefix[k] for k < n_chunks; entries
// beyond hold the total), for a block of at least 256 threads; returns the total (all threads).
// `warp_total` must have room for blockDim.x / 32 values.
__device__ __forceinline__ uint32_t chunk_prefix(const uint32_t *__restrict__ counts, const uint32_t n_chunks,
                                                 uint32_t *prefix, uint32_t *warp_total) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const uint32_t per = (MAX_CHUNKS + blockDim.x - 1) / blockDim.x;   // counts per thread
    uint32_t c[4];
    uint32_t s = 0;
    for (uint32_t j = 0; j < per; ++j) {
        const uint32_t k = threadIdx.x * per + j;
        c[j] = k < n_chunks ? counts[k] : 0u;
        s += c[j];
    }
    uint32_t incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(FULL_MASK, incl, o);
        if (lane >= static_cast<uint32_t>(o)) incl += t;
    }
    if (lane == 31) warp_total[warp] = incl;
    __syncthreads();
    uint32_t base = 0, total = 0;
    for (uint32_t w = 0; w < n_warps; ++w) {
        const uint32_t t = warp_total[w];
        if (w < warp) base += t;
        total += t;
    }
    uint32_t run = base + incl - s;
    for (uint32_t j = 0; j < per; ++j) {
        const uint32_t k = threadIdx.x * per + j;
        if (k < MAX_CHUNKS) prefix[k] = run;
        run += c[j];
    }
    if (threadIdx.x == 0) prefix[MAX_CHUNKS] = total;
    __syncthreads();
    return total;
}

// Row id of entry `li` of the compacted list (li < total).
__device__ __forceinline__ uint32_t list_row(const uint32_t *prefix, const uint32_t n_chunks, const uint32_t chunk,
                                             const uint32_t *__restrict__ ids, const uint32_t li) {
    uint32_t lo = 0, hi = n_chunks;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (prefix[mid] <= li) lo = mid; else hi = mid;
    }
    return ids[static_cast<uint64_t>(lo) * chunk + (li - prefix[lo])];
}

}  // namespace
}  // namespace bpl

#endif  // BPL_CSRC_SPIKE_SCAN_CUH_
