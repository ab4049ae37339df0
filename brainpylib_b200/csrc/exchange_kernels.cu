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
//   state [slots + 1 + 17] u32           local: arrivals already consumed per slot, the status word, then the
//                                        CTA counters of the push kernels (all zero at start)
// Slot reuse: with `slots` >= 4 a producer that runs at most one step ahead of its own consumer
// cannot overwrite a slot a peer is still reading (see sharded.py).
#include "abi.h"
#include "common.cuh"
#include "spike_scan.cuh"

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

template<typename E>
__global__ void __launch_bounds__(SCAN_THREADS)
spike_scan_push_kernel(const E *__restrict__ events, const uint32_t n_local, const uint32_t row_offset,
                       const ListTable peers, const int world, const int rank, const int slot,
                       const uint32_t chunks_per_rank, uint32_t *__restrict__ cta_counter) {
    __shared__ uint32_t warp_total[SCAN_THREADS / 32];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t chunk_index = rank * chunks_per_rank + blockIdx.x;
    const uint32_t begin = blockIdx.x * SCAN_TILE;
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
    if (lane == 0) warp_total[warp] = total;
    __syncthreads();
    uint32_t offset = 0, chunk_total = 0;
#pragma unroll
    for (int w = 0; w < SCAN_THREADS / 32; ++w) {
        const uint32_t t = warp_total[w];
        if (w < static_cast<int>(warp)) offset += t;
        chunk_total += t;
    }
    const uint32_t below = (1u << lane) - 1u;
    const size_t seg = static_cast<size_t>(MAX_CHUNKS) + static_cast<size_t>(chunk_index) * SCAN_TILE;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        if (act[k]) {
            const uint32_t at = offset + __popc(bits[k] & below);
            const uint32_t row = row_offset + base + k * 32 + lane;
            for (int p = 0; p < world; ++p) peers.list[p][seg + at] = row;
        }
        offset += __popc(bits[k]);
    }
    if (threadIdx.x < static_cast<uint32_t>(world)) peers.list[threadIdx.x][chunk_index] = chunk_total;
    __threadfence_system();
    __syncthreads();
    __shared__ bool last;
    if (threadIdx.x == 0) {
        const uint32_t done = atomicAdd(cta_counter + MAX_WORLD, 1u);   // counter 16: this kernel's own
        last = (done == gridDim.x - 1);
        if (last) cta_counter[MAX_WORLD] = 0u;
    }
    __syncthreads();
    if (last && threadIdx.x < static_cast<uint32_t>(world)) {
        __threadfence_system();
        atomicAdd_system(peers.flags[threadIdx.x] + slot * world + rank, 1u);
    }
}

// grid > 1: the extra blocks only zero-fill `zero` (the consumer's output vector) while block 0 polls.
__global__ void spike_wait_kernel(uint32_t *__restrict__ flags, uint32_t *__restrict__ state, const int world,
                                  const int slot, const int slots, const uint32_t max_polls,
                                  float *__restrict__ zero, const uint32_t n_zero) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_zero; i += gridDim.x * blockDim.x) zero[i] = 0.0f;
    if (blockIdx.x != 0 || threadIdx.x >= 32) return;
    const int src = threadIdx.x;
    const uint32_t expected = state[slot] + 1u;
    bool ok = true;
    if (src < world) {
        const volatile uint32_t *f = flags + slot * world + src;
        uint32_t polls = 0;
        while (*f < expected) {
            if (++polls > max_polls) { ok = false; break; }
            __nanosleep(200);
        }
    }
    __threadfence_system();   // acquire: what the producers wrote before bumping is visible from here on
    const bool all_ok = __all_sync(FULL_MASK, ok);
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

}  // extern "C"
