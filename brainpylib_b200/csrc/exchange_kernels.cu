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
//   state [slots + 1 + 16] u32           local: arrivals already consumed per slot, the status word, then one
//                                        CTA counter per destination used by the push kernel (all zero at start)
// Slot reuse: with `slots` >= 4 a producer that runs at most one step ahead of its own consumer
// cannot overwrite a slot a peer is still reading (see sharded.py).
#include "abi.h"
#include "common.cuh"

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

__global__ void spike_wait_kernel(uint32_t *__restrict__ flags, uint32_t *__restrict__ state, const int world,
                                  const int slot, const int slots, const uint32_t max_polls) {
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
                                            slot, slots, max_polls);
    launch_ok();
}

}  // extern "C"
