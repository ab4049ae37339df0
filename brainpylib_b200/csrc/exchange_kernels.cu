// Spike exchange between the GPUs of one node without a collective (no counterpart in the
// reference, which has no multi-device code).
//
// Every rank owns 1/world of the spike sources.  Per step it PUSHES its slice of the event vector
// straight into a slot of every peer's buffer with plain peer stores over NVLink and then bumps a
// per-(slot, source) arrival counter on that peer (system-scope atomic after a system fence).  A
// consumer waits until all `world` counters of the slot have reached the value it expects, with a
// BOUNDED number of polls: if they have not, it records a timeout in a status word and returns, so a
// missing or late peer can never hang the GPU.  The operators that follow on the same stream then
// read the assembled event vector from local memory; no load ever goes to a peer.
//
// Buffers (the caller allocates them so that every rank can address every peer's copy, e.g. with
// torch's symmetric memory; with world = 1 ordinary device memory will do):
//   data  [slots][world * slice_bytes]   assembled event vectors
//   flags [slots][world] u32             arrival counters, zero-initialised once
//   state [slots + 1 + 32] u32           local: arrivals already consumed per slot, the status word, then the
//                                        counters of the push and step kernels (all zero at start)
// Slot reuse: with `slots` >= 4 a producer that runs at most one step ahead of its own consumer
// cannot overwrite a slot a peer is still reading (see sharded.py).
#include "abi.h"
#include "common.cuh"
#include "spike_scan.cuh"
#include "row_scatter.cuh"
#include "cb_scatter.cuh"

namespace bpl {
namespace {

constexpr int MAX_WORLD = 16;
constexpr int PUSH_THREADS = 1024;

struct PeerTable {
    unsigned char *data[MAX_WORLD];   // peer p's data buffer
    uint32_t *flags[MAX_WORLD];       // peer p's flag array
};

// grid = (ctas_per_dst, world): the CTAs of column `dst` copy the slice to peer `dst` together; the one that
// finishes last (local counter) publishes the arrival on the peer.
__global__ void __launch_bounds__(PUSH_THREADS)
spike_push_kernel(const unsigned char *__restrict__ local, const size_t slice_bytes, const PeerTable peers,
                  const int world, const int rank, const int slot, uint32_t *__restrict__ cta_counter) {
    const int dst = blockIdx.y;
    const uint32_t part = blockIdx.x, parts = gridDim.x;
    unsigned char *out = peers.data[dst] + (static_cast<size_t>(slot) * world + rank) * slice_bytes;
    const bool vec = ((reinterpret_cast<uintptr_t>(local) | reinterpret_cast<uintptr_t>(out) | slice_bytes) & 15u) == 0;
    if (vec) {
        const uint4 *src4 = reinterpret_cast<const uint4 *>(local);
        uint4 *dst4 = reinterpret_cast<uint4 *>(out);
        const size_t n4 = slice_bytes / 16;
        for (size_t i = static_cast<size_t>(part) * PUSH_THREADS + threadIdx.x; i < n4;
             i += static_cast<size_t>(parts) * PUSH_THREADS)
            dst4[i] = src4[i];
    } else {
        for (size_t i = static_cast<size_t>(part) * PUSH_THREADS + threadIdx.x; i < slice_bytes;
             i += static_cast<size_t>(parts) * PUSH_THREADS)
            out[i] = local[i];
    }
    __threadfence_system();   // this CTA's stores are visible system-wide before it reports in
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t done = atomicAdd(cta_counter + dst, 1u);
        if (done == parts - 1) {               // every CTA of this destination has fenced and reported
            cta_counter[dst] = 0u;             // ready for the next push (pushes of one rank are stream-ordered)
            __threadfence_system();
            atomicAdd_system(peers.flags[dst] + slot * world + rank, 1u);
        }
    }
}

// Compaction fused with the exchange: block j compacts chunk j (<= 4096 events) of this rank's own
// spike sources and writes the ascending list of GLOBAL row ids, and its length, straight into the
// spike list of EVERY rank (peer stores), at chunk index rank * chunks_per_rank + j.  The assembled
// list has exactly the layout the scatter kernel consumes (counts[1024] then ids in 4096-entry chunk
// segments), so a consumer needs no scan of its own.  The block that finishes last publishes the
// arrival on every peer.
struct ListTable {
    uint32_t *list[MAX_WORLD];    // peer p's list buffer for this slot: counts[MAX_CHUNKS] then ids
    uint32_t *flags[MAX_WORLD];
};

// Block-wide: compacts chunk `chunk_in_rank` (<= 4096 events) of this rank's events and stores the ids and
// the count into every peer's list (`lists[p] + list_offset`) at chunk index `chunk_index`.  Ends with the
// block's stores issued but not fenced.  `warp_total`: shared, SCAN_THREADS / 32 words.  `stage`: shared, 16-byte
// aligned, SCAN_TILE words: the ids are compacted there first and leave as 16-byte stores, a few per peer
// instead of one 4-byte peer store per spike (an SM keeps only so many peer stores in flight).
// `tid`: index of the thread in its team of 256 (the whole block for 256-thread blocks); `bar`: 0 = the block
// barrier, else the id of a named barrier that the 256 threads of the team share (1024-thread blocks run four teams).
__device__ __forceinline__ void team_sync(const int bar) {
    if (bar == 0) __syncthreads();
    else asm volatile("bar.sync %0, 256;" :: "r"(bar) : "memory");
}

template<typename E>
__device__ __forceinline__ void compact_and_push_chunk(const E *__restrict__ events, const uint32_t n_local,
                                                       const uint32_t row_offset, uint32_t *const *lists,
                                                       const size_t list_offset, const int world,
                                                       const uint32_t chunk_in_rank, const uint32_t chunk_index,
                                                       uint32_t *warp_total, uint32_t *stage,
                                                       const uint32_t tid = threadIdx.x, const int bar = 0) {
    const uint32_t lane = tid & 31, warp = tid >> 5;
    const uint32_t begin = chunk_in_rank * SCAN_TILE;
    const uint32_t end = min(begin + static_cast<uint32_t>(SCAN_TILE), n_local);
    const uint32_t base = begin + warp * SCAN_WARP_SPAN;
    bool act[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const uint32_t i = base + k * 32 + lane;
        act[k] = (i < end) && is_event(events[i]);
    }
    uint32_t bits[16], total = 0;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        bits[k] = __ballot_sync(FULL_MASK, act[k]);
        total += __popc(bits[k]);
    }
    team_sync(bar);                // warp_total may still be read from an earlier use
    if (lane == 0) warp_total[warp] = total;
    team_sync(bar);
    uint32_t offset = 0, chunk_total = 0;
#pragma unroll
    for (int w = 0; w < SCAN_THREADS / 32; ++w) {
        const uint32_t t = warp_total[w];
        if (w < static_cast<int>(warp)) offset += t;
        chunk_total += t;
    }
    const uint32_t below = (1u << lane) - 1u;
    const size_t seg = list_offset + static_cast<size_t>(MAX_CHUNKS) + static_cast<size_t>(chunk_index) * SCAN_TILE;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        if (act[k]) stage[offset + __popc(bits[k] & below)] = row_offset + base + k * 32 + lane;
        offset += __popc(bits[k]);
    }
    team_sync(bar);
    // whole 16-byte words: up to three entries behind the count are written too (they stay inside the chunk's
    // segment and nobody reads behind the count)
    const uint32_t n4 = (chunk_total + 3u) >> 2;
    const uint4 *src = reinterpret_cast<const uint4 *>(stage);
    for (int p = 0; p < world; ++p) {
        uint4 *dst = reinterpret_cast<uint4 *>(lists[p] + seg);
        for (uint32_t i = tid; i < n4; i += SCAN_THREADS) dst[i] = src[i];
    }
    if (tid < static_cast<uint32_t>(world)) lists[tid][list_offset + chunk_index] = chunk_total;
}

// Block-wide, after the block's peer stores: the block reports in on `counter`; the last of `n_blocks`
// reporting blocks resets the counter and bumps this rank's arrival counter of `slot` on every peer.
// One system-scope fence per block: the barrier orders the block's peer stores before it and the fence is
// cumulative over them, so they are visible to every GPU before the counter moves.
__device__ __forceinline__ void publish_arrival(uint32_t *counter, const uint32_t n_blocks, uint32_t *const *flags,
                                                const int world, const int rank, const int slot) {
    __shared__ bool last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t done = atomicAdd(counter, 1u);
        last = (done == n_blocks - 1);
        if (last) *counter = 0u;
    }
    __syncthreads();
    if (last && threadIdx.x < static_cast<uint32_t>(world)) {
        __threadfence_system();
        atomicAdd_system(flags[threadIdx.x] + slot * world + rank, 1u);
    }
}

// Bounded wait of one warp (lanes < world poll one source each) for generation `expected` of `slot`.
// Acquire loads at system scope: what a producer wrote before bumping its counter is visible to this
// thread, and through a barrier or a kernel boundary to whoever runs after it.
__device__ __forceinline__ bool poll_arrivals(const uint32_t *flags, const int world, const int slot,
                                              const uint32_t expected, const uint32_t max_polls) {
    bool ok = true;
    if (static_cast<int>(threadIdx.x & 31) < world) {
        const uint32_t *f = flags + slot * world + (threadIdx.x & 31);
        uint32_t polls = 0;
        for (;;) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
            if (seen >= expected) break;
            if (++polls > max_polls) { ok = false; break; }
            __nanosleep(100);
        }
    }
    return __all_sync(FULL_MASK, ok);
}

template<typename E>
__global__ void __launch_bounds__(SCAN_THREADS)
spike_scan_push_kernel(const E *__restrict__ events, const uint32_t n_local, const uint32_t row_offset,
                       const ListTable peers, const int world, const int rank, const int slot,
                       const uint32_t chunks_per_rank, uint32_t *__restrict__ cta_counter) {
    __shared__ uint32_t warp_total[SCAN_THREADS / 32];
    __shared__ __align__(16) uint32_t stage[SCAN_TILE];
    compact_and_push_chunk(events, n_local, row_offset, peers.list, 0, world, blockIdx.x,
                           rank * chunks_per_rank + blockIdx.x, warp_total, stage);
    publish_arrival(cta_counter + MAX_WORLD, gridDim.x, peers.flags, world, rank, slot);   // counter 16
}

// ------------------------------------------------------------------------------------------
// One launch per simulation step on a sharded matrix: exchange of the NEXT step's spikes fused with
// the scatter of THIS step's.
// ------------------------------------------------------------------------------------------
// The first `pushers` blocks (at most one per chunk of the rank's own events and 1/16 of the grid) only exchange:
//   they compact the rank's spikes of step t + 1 and store the list into slot (t + 1) % slots of every
//   peer (plain peer stores), fence, and publish the arrival on every peer.
// The other blocks only compute: they wait, bounded, until the lists of step t have arrived from every
//   rank (pushed by the peers' previous launch, so normally the first poll succeeds) and scatter step t
//   from the assembled list in local memory into `y_cur` (row_scatter_body).
// All blocks zero-fill a share of `y_next` (the output buffer of step t + 1; outputs are double-buffered)
// and take an exit ticket; the last one out advances the step counter t kept in `state`.
// Nothing here waits on a kernel that has not been launched yet: the lists of step t come from each
// peer's PREVIOUS launch (or its prime call), which waits only on launches before this one.
// ctr = state + slots + 1: ctr[17] push counter, ctr[18] exit tickets, ctr[19] step counter t.
constexpr int CTR_STEP_PUSH = 17, CTR_STEP_EXIT = 18, CTR_STEP_T = 19;

// The exchange half of the step kernel, kept out of line (and everything it needs re-derived from the
// kernel parameters after it) so that it takes no registers from the scatter loop, which wants all 64 a
// thread can have at four blocks per SM for its loads in flight.  Returns through `arrived` (shared)
// whether this block should scatter (false for pushing blocks and after a timeout, which is recorded).
template<typename E>
__device__ __noinline__ void step_exchange(float *__restrict__ y_next, const uint32_t n_out,
                                           const E *__restrict__ next_events, const uint32_t n_local,
                                           const uint32_t row_offset, const uint32_t chunks_per_rank,
                                           const ListTable &peers, const size_t slot_words, uint32_t *state,
                                           const int world, const int rank, const int slots,
                                           const uint32_t max_polls, const uint32_t pushers, bool *arrived,
                                           uint32_t *warp_total, uint32_t *stage) {
    uint32_t *ctr = state + slots + 1;
    const uint32_t t = ctr[CTR_STEP_T];
    const int slot = static_cast<int>(t % slots), next_slot = static_cast<int>((t + 1u) % slots);
    const uint32_t expected = t / slots + 1u;
    if (y_next != nullptr)
        for (uint32_t i = blockIdx.x * ROW_THREADS + threadIdx.x; i < n_out; i += gridDim.x * ROW_THREADS)
            y_next[i] = 0.0f;
    if (blockIdx.x < pushers) {
        for (uint32_t c = blockIdx.x; c < chunks_per_rank; c += pushers)
            compact_and_push_chunk(next_events, n_local, row_offset, peers.list,
                                   static_cast<size_t>(next_slot) * slot_words, world, c,
                                   rank * chunks_per_rank + c, warp_total, stage);
        publish_arrival(ctr + CTR_STEP_PUSH, pushers, peers.flags, world, rank, next_slot);
        if (threadIdx.x == 0) *arrived = false;
    } else if (threadIdx.x < 32) {
        const bool ok = poll_arrivals(peers.flags[rank], world, slot, expected, max_polls);
        if (threadIdx.x == 0) {
            *arrived = ok;
            if (!ok) state[slots] = 1u;        // timed out: the output of this step must not be trusted
        }
    }
    __syncthreads();
}

template<typename E, bool VEC>
__global__ void __launch_bounds__(ROW_THREADS, 4)
sharded_step_kernel(const uint32_t *__restrict__ indices, const uint32_t *__restrict__ indptr,
                    const float *__restrict__ data, const uint32_t n_row, float *__restrict__ y_cur,
                    float *__restrict__ y_next, const uint32_t n_out, const E *__restrict__ next_events,
                    const uint32_t n_local, const uint32_t row_offset, const uint32_t chunks_per_rank,
                    const __grid_constant__ ListTable peers, const size_t slot_words, uint32_t *state,
                    const int world, const int rank, const int slots, const uint32_t max_polls) {
    __shared__ uint32_t prefix[MAX_CHUNKS + 1];
    __shared__ uint32_t warp_total[ROW_WARPS];
    __shared__ __align__(16) uint32_t stage[SCAN_TILE];
    __shared__ bool arrived;
    // few enough pushing blocks that the scatter keeps (nearly) the whole grid, each taking several chunks in
    // turn: their work is short next to the scatter and off its critical path
    const uint32_t pushers = next_events == nullptr ? 0u : min(chunks_per_rank, max(gridDim.x / 16u, 1u));
    step_exchange(y_next, n_out, next_events, n_local, row_offset, chunks_per_rank, peers, slot_words, state, world,
                  rank, slots, max_polls, pushers, &arrived, warp_total, stage);
    if (arrived) {
        const uint32_t slot = state[slots + 1 + CTR_STEP_T] % slots;
        const uint32_t *list = peers.list[rank] + static_cast<size_t>(slot) * slot_words;
        row_scatter_body<float, false, true, VEC, true, true>(indices, indptr, data, nullptr, n_row, SCAN_TILE,
                                                  chunks_per_rank * world, list, list + MAX_CHUNKS, y_cur, prefix,
                                                  warp_total, blockIdx.x - pushers, gridDim.x - pushers);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t *ctr = state + slots + 1;
        const uint32_t done = atomicAdd(ctr + CTR_STEP_EXIT, 1u);
        if (done == gridDim.x - 1) {           // every block has read t and finished
            const uint32_t t = ctr[CTR_STEP_T];
            ctr[CTR_STEP_EXIT] = 0u;
            state[t % slots] = t / slots + 1u;
            ctr[CTR_STEP_T] = t + 1u;
        }
    }
}

// The same step on a shard stored in the column-blocked layout (cb_scatter.cuh): blocks [0, n_scatter) are the
// (column block, row share) CTAs of the scatter, with the block's slice of the output in shared memory; the blocks
// behind them exchange, four 256-thread teams per block, each compacting and pushing one chunk at a time.
template<int NBUF, bool FIXED, int LOG_L>
__global__ void __launch_bounds__(CB_THREADS, 1)
sharded_cb_step_kernel(const unsigned char *__restrict__ groups, const uint32_t *__restrict__ offsets, const uint32_t n_out,
                       const uint32_t width, const uint32_t n_blocks, const uint32_t P, float *__restrict__ y_cur,
                       float *__restrict__ y_next, const void *__restrict__ next_events, const int ev_is_float,
                       const uint32_t n_local, const uint32_t row_offset, const uint32_t chunks_per_rank,
                       const __grid_constant__ ListTable peers, const size_t slot_words, uint32_t *state, const int world,
                       const int rank, const int slots, const uint32_t max_polls, const uint32_t acc_bytes,
                       const float inv_scale) {
    extern __shared__ __align__(128) unsigned char cb_smem[];
    __shared__ uint32_t prefix[MAX_CHUNKS + 1];
    __shared__ uint32_t warp_total[CB_WARPS];
    __shared__ bool arrived;
    uint32_t *ctr = state + slots + 1;
    const uint32_t n_scatter = n_blocks * P;
    const uint32_t t = ctr[CTR_STEP_T];
    const int slot = static_cast<int>(t % slots), next_slot = static_cast<int>((t + 1u) % slots);
    if (y_next != nullptr)
        for (uint32_t i = blockIdx.x * CB_THREADS + threadIdx.x; i < n_out; i += gridDim.x * CB_THREADS) y_next[i] = 0.0f;
    if (blockIdx.x >= n_scatter) {
        // ---- exchange: the rank's spikes of step t + 1 go to slot (t + 1) % slots of every peer ----
        const uint32_t team = threadIdx.x >> 8, tid = threadIdx.x & 255u;
        const uint32_t n_teams = (gridDim.x - n_scatter) * 4u;
        for (uint32_t c = (blockIdx.x - n_scatter) * 4u + team; c < chunks_per_rank; c += n_teams) {
            if (ev_is_float)
                compact_and_push_chunk(static_cast<const float *>(next_events), n_local, row_offset, peers.list,
                                       static_cast<size_t>(next_slot) * slot_words, world, c, rank * chunks_per_rank + c,
                                       warp_total + team * 8u, reinterpret_cast<uint32_t *>(cb_smem) + team * SCAN_TILE,
                                       tid, 1 + static_cast<int>(team));
            else
                compact_and_push_chunk(static_cast<const uint8_t *>(next_events), n_local, row_offset, peers.list,
                                       static_cast<size_t>(next_slot) * slot_words, world, c, rank * chunks_per_rank + c,
                                       warp_total + team * 8u, reinterpret_cast<uint32_t *>(cb_smem) + team * SCAN_TILE,
                                       tid, 1 + static_cast<int>(team));
        }
        publish_arrival(ctr + CTR_STEP_PUSH, gridDim.x - n_scatter, peers.flags, world, rank, next_slot);
    } else {
        // ---- scatter of step t from the lists every rank pushed during its previous launch ----
        if (threadIdx.x < 32) {
            const bool ok = poll_arrivals(peers.flags[rank], world, slot, t / slots + 1u, max_polls);
            if (threadIdx.x == 0) {
                arrived = ok;
                if (!ok) state[slots] = 1u;    // timed out: the output of this step must not be trusted
            }
        }
        __syncthreads();
        if (arrived) {
            const uint32_t *list = peers.list[rank] + static_cast<size_t>(slot) * slot_words;
            cb_scatter_body<NBUF, FIXED, LOG_L>(groups, offsets, n_out, width, n_blocks, blockIdx.x / P, blockIdx.x % P, P,
                                                SCAN_TILE, chunks_per_rank * world, list, list + MAX_CHUNKS, y_cur,
                                                acc_bytes, cb_smem, prefix, warp_total, inv_scale);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t done = atomicAdd(ctr + CTR_STEP_EXIT, 1u);
        if (done == gridDim.x - 1) {           // every block has read t and finished
            ctr[CTR_STEP_EXIT] = 0u;
            state[t % slots] = t / slots + 1u;
            ctr[CTR_STEP_T] = t + 1u;
        }
    }
}

using CbStepKernel = void (*)(const unsigned char *, const uint32_t *, uint32_t, uint32_t, uint32_t, uint32_t, float *, float *,
                              const void *, int, uint32_t, uint32_t, uint32_t, const ListTable, size_t, uint32_t *, int, int,
                              int, uint32_t, uint32_t, float);
template<int NBUF, bool FIXED>
CbStepKernel cb_step_for_lanes(uint32_t log_l) {
    switch (log_l) {
        case 3: return sharded_cb_step_kernel<NBUF, FIXED, 3>;
        case 4: return sharded_cb_step_kernel<NBUF, FIXED, 4>;
        case 5: return sharded_cb_step_kernel<NBUF, FIXED, 5>;
        default: return sharded_cb_step_kernel<NBUF, FIXED, 2>;
    }
}
CbStepKernel cb_step_kernel(uint32_t n_buf, bool fixed, uint32_t log_l) {
    if (n_buf == 3) return fixed ? cb_step_for_lanes<3, true>(log_l) : cb_step_for_lanes<3, false>(log_l);
    return fixed ? cb_step_for_lanes<2, true>(log_l) : cb_step_for_lanes<2, false>(log_l);
}

// Pushes the spikes of the step the counter points at (the first step of a run) and zero-fills its output.
template<typename E>
__global__ void __launch_bounds__(SCAN_THREADS)
sharded_prime_kernel(const E *__restrict__ events, const uint32_t n_local, const uint32_t row_offset,
                     const uint32_t chunks_per_rank, const ListTable peers, const size_t slot_words,
                     uint32_t *state, const int world, const int rank, const int slots,
                     float *__restrict__ y_first, const uint32_t n_out) {
    __shared__ uint32_t warp_total[SCAN_THREADS / 32];
    __shared__ __align__(16) uint32_t stage[SCAN_TILE];
    uint32_t *ctr = state + slots + 1;
    const int slot = static_cast<int>(ctr[CTR_STEP_T] % slots);
    for (uint32_t i = blockIdx.x * SCAN_THREADS + threadIdx.x; i < n_out; i += gridDim.x * SCAN_THREADS)
        y_first[i] = 0.0f;
    compact_and_push_chunk(events, n_local, row_offset, peers.list, static_cast<size_t>(slot) * slot_words, world,
                           blockIdx.x, rank * chunks_per_rank + blockIdx.x, warp_total, stage);
    publish_arrival(ctr + CTR_STEP_PUSH, gridDim.x, peers.flags, world, rank, slot);
}

// grid > 1: the extra blocks only zero-fill `zero` (the consumer's output vector) while block 0 polls.
__global__ void spike_wait_kernel(uint32_t *__restrict__ flags, uint32_t *__restrict__ state, const int world,
                                  const int slot, const int slots, const uint32_t max_polls,
                                  float *__restrict__ zero, const uint32_t n_zero) {
    if (gridDim.x > 1) {
        if (blockIdx.x != 0) {      // blocks 1.. zero-fill; block 0 only polls, with no stores of its own in flight
            for (uint32_t i = (blockIdx.x - 1) * blockDim.x + threadIdx.x; i < n_zero; i += (gridDim.x - 1) * blockDim.x)
                zero[i] = 0.0f;
            return;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < n_zero; i += blockDim.x) zero[i] = 0.0f;
    }
    if (threadIdx.x >= 32) return;
    const uint32_t expected = state[slot] + 1u;
    const bool all_ok = poll_arrivals(flags, world, slot, expected, max_polls);
    if (threadIdx.x == 0) {
        if (all_ok) state[slot] = expected;
        else state[slots] = 1u;   // timed out: the data of this slot must not be trusted
    }
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {

// Enqueue the push of `slice_bytes` bytes at `local` into slot `slot` of every peer.
// peer_data / peer_flags: host arrays of `world` device pointers (entry `rank` is this rank's own).
void bpl_spike_exchange_push(bpl_stream_t stream, const void *local, size_t slice_bytes, void *const *peer_data,
                             void *const *peer_flags, void *state, int world, int rank, int slot, int slots) {
    if (world < 1 || world > MAX_WORLD || rank < 0 || rank >= world || slot < 0 || slot >= slots || state == nullptr) {
        set_status(BPL_ERR_ARGUMENT, "spike exchange: world must be 1..16, rank and slot in range");
        return;
    }
    PeerTable t;
    for (int p = 0; p < MAX_WORLD; ++p) {
        t.data[p] = p < world ? static_cast<unsigned char *>(peer_data[p]) : nullptr;
        t.flags[p] = p < world ? static_cast<uint32_t *>(peer_flags[p]) : nullptr;
    }
    // enough CTAs per destination to fill the NVLink pipe (16 KB per CTA pass), at most 16
    size_t parts = (slice_bytes + 65535) / 65536;
    parts = parts < 1 ? 1 : (parts > 16 ? 16 : parts);
    const dim3 grid(static_cast<unsigned int>(parts), static_cast<unsigned int>(world));
    spike_push_kernel<<<grid, PUSH_THREADS, 0, stream>>>(static_cast<const unsigned char *>(local), slice_bytes, t,
                                                        world, rank, slot,
                                                        static_cast<uint32_t *>(state) + slots + 1);
    launch_ok();
}

// Enqueue the bounded wait for all `world` arrivals in slot `slot`.  `max_polls` polls of ~0.2 us each per
// source; on timeout state[slots] becomes 1 and the kernel returns.
void bpl_spike_exchange_wait(bpl_stream_t stream, void *flags, void *state, int world, int slot, int slots,
                             uint32_t max_polls) {
    if (world < 1 || world > MAX_WORLD || slot < 0 || slot >= slots) {
        set_status(BPL_ERR_ARGUMENT, "spike exchange: world must be 1..16 and slot < slots");
        return;
    }
    spike_wait_kernel<<<1, 32, 0, stream>>>(static_cast<uint32_t *>(flags), static_cast<uint32_t *>(state), world,
                                            slot, slots, max_polls, nullptr, 0u);
    launch_ok();
}

// As bpl_spike_exchange_wait, and the same launch zero-fills `zero[0 .. n_zero)` (float32): the output vector
// the list-driven scatter will accumulate into.
void bpl_spike_exchange_wait_zero(bpl_stream_t stream, void *flags, void *state, int world, int slot, int slots,
                                  uint32_t max_polls, void *zero, uint32_t n_zero) {
    if (world < 1 || world > MAX_WORLD || slot < 0 || slot >= slots) {
        set_status(BPL_ERR_ARGUMENT, "spike exchange: world must be 1..16 and slot < slots");
        return;
    }
    const unsigned int blocks = n_zero == 0 ? 1u : min(64u, (n_zero + 4095u) / 4096u + 1u);
    spike_wait_kernel<<<blocks, 256, 0, stream>>>(static_cast<uint32_t *>(flags), static_cast<uint32_t *>(state),
                                                  world, slot, slots, max_polls, static_cast<float *>(zero), n_zero);
    launch_ok();
}

// Number of 4096-event chunks one rank contributes, and the size in bytes of one slot of the spike-list buffer.
uint32_t bpl_spike_list_chunks_per_rank(uint32_t n_local) { return (n_local + SCAN_TILE - 1) / SCAN_TILE; }
size_t bpl_spike_list_slot_bytes(uint32_t n_local, int world) {
    return (static_cast<size_t>(MAX_CHUNKS) +
            static_cast<size_t>(bpl_spike_list_chunks_per_rank(n_local)) * world * SCAN_TILE) * sizeof(uint32_t);
}

// Enqueue compaction + push of this rank's `n_local` events (bool when ev_is_float == 0, else float32);
// global row id of local event i is row_offset + i.  peer_lists[p]: peer p's list buffer OF THIS SLOT.
void bpl_spike_exchange_push_compacted(bpl_stream_t stream, const void *local_events, int ev_is_float,
                                       uint32_t n_local, uint32_t row_offset, void *const *peer_lists,
                                       void *const *peer_flags, void *state, int world, int rank, int slot,
                                       int slots) {
    const uint32_t cpr = bpl_spike_list_chunks_per_rank(n_local);
    if (world < 1 || world > MAX_WORLD || rank < 0 || rank >= world || slot < 0 || slot >= slots ||
        state == nullptr || n_local == 0 || static_cast<uint64_t>(cpr) * world > MAX_CHUNKS) {
        set_status(BPL_ERR_ARGUMENT, "spike exchange: bad rank/slot, or more than 1024 chunks of 4096 events in total");
        return;
    }
    ListTable t;
    for (int p = 0; p < MAX_WORLD; ++p) {
        t.list[p] = p < world ? static_cast<uint32_t *>(peer_lists[p]) : nullptr;
        t.flags[p] = p < world ? static_cast<uint32_t *>(peer_flags[p]) : nullptr;
    }
    uint32_t *counters = static_cast<uint32_t *>(state) + slots + 1;
    if (ev_is_float)
        spike_scan_push_kernel<float><<<cpr, SCAN_THREADS, 0, stream>>>(
            static_cast<const float *>(local_events), n_local, row_offset, t, world, rank, slot, cpr, counters);
    else
        spike_scan_push_kernel<uint8_t><<<cpr, SCAN_THREADS, 0, stream>>>(
            static_cast<const uint8_t *>(local_events), n_local, row_offset, t, world, rank, slot, cpr, counters);
    launch_ok();
}

// ---- one launch per step on a sharded matrix (sharded_step_kernel) ----
// peer_lists[p] / peer_flags[p]: peer p's list buffer (slot 0; slots are slot_bytes apart) and flag array.
// The step counter lives in `state`, so the same call sequence can be captured in a CUDA graph and replayed.

static bool step_arguments_ok(uint32_t n_local, int world, int rank, int slots, const void *state) {
    const uint32_t cpr = bpl_spike_list_chunks_per_rank(n_local);
    if (world < 1 || world > MAX_WORLD || rank < 0 || rank >= world || slots < 4 || state == nullptr ||
        n_local == 0 || static_cast<uint64_t>(cpr) * world > MAX_CHUNKS) {
        set_status(BPL_ERR_ARGUMENT,
                   "sharded step: world 1..16, rank < world, slots >= 4, at most 1024 chunks of 4096 events in total");
        return false;
    }
    return true;
}

static ListTable list_table(void *const *peer_lists, void *const *peer_flags, int world) {
    ListTable t;
    for (int p = 0; p < MAX_WORLD; ++p) {
        t.list[p] = p < world ? static_cast<uint32_t *>(peer_lists[p]) : nullptr;
        t.flags[p] = p < world ? static_cast<uint32_t *>(peer_flags[p]) : nullptr;
    }
    return t;
}

// Before the first step of a run: push the spikes of that step and zero-fill its output vector.
void bpl_sharded_prime(bpl_stream_t stream, const void *events, int ev_is_float, uint32_t n_local,
                       uint32_t row_offset, void *const *peer_lists, size_t slot_bytes, void *const *peer_flags,
                       void *state, int world, int rank, int slots, void *y_first, uint32_t n_out) {
    if (!step_arguments_ok(n_local, world, rank, slots, state)) return;
    if (events == nullptr || peer_lists == nullptr || peer_flags == nullptr || (y_first == nullptr && n_out != 0)) {
        set_status(BPL_ERR_ARGUMENT, "sharded prime: null events, output or peer table");
        return;
    }
    const uint32_t cpr = bpl_spike_list_chunks_per_rank(n_local);
    const ListTable t = list_table(peer_lists, peer_flags, world);
    if (ev_is_float)
        sharded_prime_kernel<float><<<cpr, SCAN_THREADS, 0, stream>>>(
            static_cast<const float *>(events), n_local, row_offset, cpr, t, slot_bytes / 4,
            static_cast<uint32_t *>(state), world, rank, slots, static_cast<float *>(y_first), n_out);
    else
        sharded_prime_kernel<uint8_t><<<cpr, SCAN_THREADS, 0, stream>>>(
            static_cast<const uint8_t *>(events), n_local, row_offset, cpr, t, slot_bytes / 4,
            static_cast<uint32_t *>(state), world, rank, slots, static_cast<float *>(y_first), n_out);
    launch_ok();
}

// One step: y_cur (already zero) += A_shard^T spikes(t) from the assembled list; pushes `next_events`
// (this rank's spikes of step t + 1; may be null at the end of a run) and zero-fills `y_next` (may be null).
void bpl_sharded_step(bpl_stream_t stream, const void *data, const void *indices, const void *indptr,
                      uint32_t n_row, uint32_t n_out, void *y_cur, void *y_next, const void *next_events,
                      int ev_is_float, uint32_t n_local, uint32_t row_offset, void *const *peer_lists,
                      size_t slot_bytes, void *const *peer_flags, void *state, int world, int rank, int slots,
                      uint32_t max_polls) {
    if (!step_arguments_ok(n_local, world, rank, slots, state)) return;
    if (data == nullptr || indices == nullptr || indptr == nullptr || y_cur == nullptr || peer_lists == nullptr ||
        peer_flags == nullptr || slot_bytes % 16 != 0) {
        set_status(BPL_ERR_ARGUMENT, "sharded step: null matrix, output or peer table, or a slot size that is not a "
                                     "multiple of 16 bytes");
        return;
    }
    const uint32_t cpr = bpl_spike_list_chunks_per_rank(n_local);
    const ListTable t = list_table(peer_lists, peer_flags, world);
    const int grid = sm_count() * 4;
    const bool vec = aligned16(indices) && aligned16(data);
#define BPL_STEP_LAUNCH(E, VEC)                                                                                  \
    sharded_step_kernel<E, VEC><<<grid, ROW_THREADS, 0, stream>>>(                                               \
        static_cast<const uint32_t *>(indices), static_cast<const uint32_t *>(indptr),                           \
        static_cast<const float *>(data), n_row, static_cast<float *>(y_cur), static_cast<float *>(y_next),      \
        n_out, static_cast<const E *>(next_events), n_local, row_offset, cpr, t, slot_bytes / 4,                 \
        static_cast<uint32_t *>(state), world, rank, slots, max_polls)
    if (ev_is_float) { if (vec) BPL_STEP_LAUNCH(float, true); else BPL_STEP_LAUNCH(float, false); }
    else             { if (vec) BPL_STEP_LAUNCH(uint8_t, true); else BPL_STEP_LAUNCH(uint8_t, false); }
#undef BPL_STEP_LAUNCH
    launch_ok();
}

// The same step on a shard prepared into the column-blocked layout (bpl_cbcsr_plan / bpl_cbcsr_fill with the rank's
// column range): groups / offsets / block_width / fixed_point / scale_log2 / team_lanes_log2 as for
// event_cbcsr_matvec_*; n_out = columns of the shard.  y_cur must already be zero.
void bpl_sharded_cb_step(bpl_stream_t stream, const void *groups, const void *offsets, uint32_t n_out, uint32_t block_width,
                         int fixed_point, int scale_log2, uint32_t team_lanes_log2, void *y_cur, void *y_next,
                         const void *next_events, int ev_is_float, uint32_t n_local, uint32_t row_offset,
                         void *const *peer_lists, size_t slot_bytes, void *const *peer_flags, void *state, int world,
                         int rank, int slots, uint32_t max_polls) {
    if (!step_arguments_ok(n_local, world, rank, slots, state)) return;
    if (groups == nullptr || offsets == nullptr || y_cur == nullptr || peer_lists == nullptr || peer_flags == nullptr ||
        slot_bytes % 16 != 0 || !aligned16(groups) || n_out == 0) {
        set_status(BPL_ERR_ARGUMENT, "sharded step: null or misaligned matrix, output or peer table, or a slot size that is "
                                     "not a multiple of 16 bytes");
        return;
    }
    if (block_width == 0 || block_width > CB_MAX_WIDTH || (block_width & 31u) != 0 ||
        (team_lanes_log2 != 0 && (team_lanes_log2 < 2 || team_lanes_log2 > 5)) ||
        (fixed_point && (scale_log2 < -100 || scale_log2 > 100))) {
        set_status(BPL_ERR_ARGUMENT, "sharded step: bad block_width, team_lanes_log2 or scale_log2");
        return;
    }
    const uint32_t n_blocks = (n_out + block_width - 1) / block_width;
    const CbPlan plan = cb_plan(block_width);
    if (n_blocks > CB_MAX_BLOCKS || !plan.ok) {
        set_status(BPL_ERR_ARGUMENT, "sharded step: too many column blocks, or no shared memory left for the copy buffers");
        return;
    }
    const uint32_t cpr = bpl_spike_list_chunks_per_rank(n_local);
    const uint32_t sms = static_cast<uint32_t>(sm_count());
    // exchange blocks: four chunks at a time each, at most four blocks; the rest of the SMs scatter
    uint32_t pushers = next_events == nullptr ? 0u : (cpr + 3u) / 4u;
    pushers = pushers > 4u ? 4u : pushers;
    uint32_t P = (sms > pushers ? sms - pushers : 1u) / n_blocks;
    P = P < 1 ? 1u : (P > 32 ? 32u : P);
    const uint32_t log_l = team_lanes_log2 == 0 ? 2u : team_lanes_log2;
    const CbStepKernel kernel = cb_step_kernel(plan.n_buf, fixed_point != 0, log_l);
    static thread_local int configured_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_device != dev) {
        for (uint32_t nb = 2; nb <= 3; ++nb)
            for (int fx = 0; fx < 2; ++fx)
                for (uint32_t ll = 2; ll <= 5; ++ll)
                    if (cudaFuncSetAttribute(cb_step_kernel(nb, fx != 0, ll), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(CB_SMEM_LIMIT)) != cudaSuccess) {
                        launch_ok();
                        return;
                    }
        configured_device = dev;
    }
    const ListTable t = list_table(peer_lists, peer_flags, world);
    const float inv_scale = fixed_point ? ldexpf(1.0f, -scale_log2) : 1.0f;
    kernel<<<n_blocks * P + pushers, CB_THREADS, plan.smem_bytes, stream>>>(
        static_cast<const unsigned char *>(groups), static_cast<const uint32_t *>(offsets), n_out, block_width, n_blocks, P,
        static_cast<float *>(y_cur), static_cast<float *>(y_next), next_events, ev_is_float, n_local, row_offset, cpr, t,
        slot_bytes / 4, static_cast<uint32_t *>(state), world, rank, slots, max_polls, plan.acc_bytes, inv_scale);
    launch_ok();
}

}  // extern "C"
