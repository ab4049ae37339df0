// Spike compaction as an operator: nonzero_{bool,int,long,float,double}
// (replaces lib/gpu_event_info.cu:11-67, registered lib/gpu_ops.cc:72-76).
//
// For every row of a (batch, size) array: the indices of its non-zero entries in ASCENDING order,
// padded with -1, and their count.  The reference appends with shared and global atomics and
// returns the indices in an arbitrary order that changes from run to run
// (lib/gpu_event_info.cu:28-43); here the order is fixed, which costs a second read of the events:
// pass 1 counts per chunk, pass 2 turns the counts into offsets and writes.
//   buffers [events T(batch, size), event_ids i32(batch, size), event_num i32(batch), workspace u32(batch * 1024)]
//   opaque  NonZeroDescriptor{event_size, batch_size}
#include "abi.h"
#include "common.cuh"

namespace bpl {
namespace {

constexpr int THREADS = 256;
constexpr int WARP_SPAN = 512;
constexpr int TILE = (THREADS / 32) * WARP_SPAN;   // 4096 events per block per tile
constexpr int MAX_CHUNKS = 1024;

struct Plan {
    uint32_t chunk, n_chunks;
};
inline Plan plan(uint32_t size) {
    const uint64_t tiles = (static_cast<uint64_t>(size) + TILE - 1) / TILE;
    const uint64_t per = tiles == 0 ? 1 : (tiles + MAX_CHUNKS - 1) / MAX_CHUNKS;
    Plan p;
    p.chunk = static_cast<uint32_t>(per * TILE);
    p.n_chunks = static_cast<uint32_t>((static_cast<uint64_t>(size) + p.chunk - 1) / p.chunk);
    return p;
}

template<typename E>
__device__ __forceinline__ bool nonzero(E e) { return e != E(0); }

// Shared by both passes: visits the chunk tile by tile; `emit(position, rank_in_chunk)` is called
// for every non-zero entry.  Returns the chunk's count (same value in every thread).
template<typename E, typename F>
__device__ __forceinline__ uint32_t walk_chunk(const E *__restrict__ events, uint64_t begin, uint64_t end, F emit) {
    __shared__ uint32_t warp_total[THREADS / 32];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t running = 0;
    for (uint64_t tile = begin; tile < end; tile += TILE) {
        const uint64_t base = tile + static_cast<uint64_t>(warp) * WARP_SPAN;
        bool act[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const uint64_t i = base + k * 32 + lane;
            act[k] = (i < end) && nonzero(events[i]);
        }
        uint32_t bits[16], total = 0;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            bits[k] = __ballot_sync(FULL_MASK, act[k]);
            total += __popc(bits[k]);
        }
        if (lane == 0) warp_total[warp] = total;
        __syncthreads();
        uint32_t offset = running, tile_total = 0;
#pragma unroll
        for (int w = 0; w < THREADS / 32; ++w) {
            const uint32_t t = warp_total[w];
            if (w < static_cast<int>(warp)) offset += t;
            tile_total += t;
        }
        __syncthreads();
        const uint32_t below = (1u << lane) - 1u;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            if (act[k]) emit(base + k * 32 + lane, offset + __popc(bits[k] & below));
            offset += __popc(bits[k]);
        }
        running += tile_total;
    }
    return running;
}

template<typename E>
__global__ void __launch_bounds__(THREADS)
count_kernel(const E *__restrict__ events, const uint32_t size, const uint32_t chunk, uint32_t *__restrict__ counts) {
    const uint64_t row = blockIdx.y;
    const uint64_t begin = static_cast<uint64_t>(blockIdx.x) * chunk;
    const uint64_t end = min(begin + chunk, static_cast<uint64_t>(size));
    const uint32_t n = walk_chunk(events + row * size, begin, end, [](uint64_t, uint32_t) {});
    if (threadIdx.x == 0) counts[row * MAX_CHUNKS + blockIdx.x] = n;
}

template<typename E>
__global__ void __launch_bounds__(THREADS)
write_kernel(const E *__restrict__ events, const uint32_t size, const uint32_t chunk, const uint32_t n_chunks,
             const uint32_t *__restrict__ counts, int *__restrict__ event_ids, int *__restrict__ event_num) {
    __shared__ uint32_t part[2][THREADS / 32];
    const uint64_t row = blockIdx.y;
    const uint32_t *c = counts + row * MAX_CHUNKS;
    // offset of this chunk = counts before it; total = all counts (<= 1024 values, 4 per thread)
    uint32_t before = 0, total = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t k = threadIdx.x * 4 + j;
        const uint32_t v = k < n_chunks ? c[k] : 0u;
        total += v;
        if (k < blockIdx.x) before += v;
    }
    before = warp_sum(before);
    total = warp_sum(total);
    if ((threadIdx.x & 31) == 0) { part[0][threadIdx.x >> 5] = before; part[1][threadIdx.x >> 5] = total; }
    __syncthreads();
    before = 0; total = 0;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) { before += part[0][w]; total += part[1][w]; }
    __syncthreads();

    int *ids = event_ids + row * size;
    const uint64_t begin = static_cast<uint64_t>(blockIdx.x) * chunk;
    const uint64_t end = min(begin + chunk, static_cast<uint64_t>(size));
    walk_chunk(events + row * size, begin, end,
               [=](uint64_t pos, uint32_t rank) { ids[before + rank] = static_cast<int>(pos); });
    // padding: this block owns the output positions of its own chunk range
    for (uint64_t p = max(begin, static_cast<uint64_t>(total)) + threadIdx.x; p < end; p += THREADS) ids[p] = -1;
    if (blockIdx.x == 0 && threadIdx.x == 0) event_num[row] = static_cast<int>(total);
}

template<typename E>
void nonzero_impl(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    const DoubleSizeDescriptor *d = unpack<DoubleSizeDescriptor>(opaque, opaque_len);
    if (!d) return;
    const uint32_t size = d->size_x, batch = d->size_y;
    if (batch == 0) return;
    if (batch > 65535u) {
        set_status(BPL_ERR_ARGUMENT, "nonzero: more than 65535 batch rows");
        return;
    }
    const E *events = static_cast<const E *>(buffers[0]);
    int *event_ids = static_cast<int *>(buffers[1]);
    int *event_num = static_cast<int *>(buffers[2]);
    uint32_t *counts = static_cast<uint32_t *>(buffers[3]);
    if (size == 0) {
        cudaMemsetAsync(event_num, 0, sizeof(int) * batch, stream);
        launch_ok();
        return;
    }
    if (counts == nullptr) {
        set_status(BPL_ERR_ARGUMENT, "nonzero needs a workspace buffer");
        return;
    }
    const Plan p = plan(size);
    const dim3 grid(p.n_chunks, batch);
    count_kernel<E><<<grid, THREADS, 0, stream>>>(events, size, p.chunk, counts);
    if (!launch_ok()) return;
    write_kernel<E><<<grid, THREADS, 0, stream>>>(events, size, p.chunk, p.n_chunks, counts, event_ids, event_num);
    launch_ok();
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {

size_t bpl_nonzero_workspace_bytes(uint32_t batch_size) { return static_cast<size_t>(batch_size) * MAX_CHUNKS * 4; }

void nonzero_bool(bpl_stream_t s, void **b, const char *o, size_t n) { nonzero_impl<uint8_t>(s, b, o, n); }
void nonzero_int(bpl_stream_t s, void **b, const char *o, size_t n) { nonzero_impl<int>(s, b, o, n); }
void nonzero_long(bpl_stream_t s, void **b, const char *o, size_t n) { nonzero_impl<long long>(s, b, o, n); }
void nonzero_float(bpl_stream_t s, void **b, const char *o, size_t n) { nonzero_impl<float>(s, b, o, n); }
void nonzero_double(bpl_stream_t s, void **b, const char *o, size_t n) { nonzero_impl<double>(s, b, o, n); }

}  // extern "C"
