// Runs of many steps on HOST-resident spike trains (no counterpart in the reference, whose callers feed one
// device array per call from Python): every step's spikes come from pinned host memory and every step's result
// goes back to pinned host memory, with the copy in, the compute launch and the copy out of neighbouring steps
// overlapped on three streams over rings of three device buffers.  The whole run is enqueued by native code in
// one call, so the dozen runtime calls a step needs cost microseconds, not an interpreter's dispatch each.
//
// Ordering inside a run.  Steps are handled in groups of `group` consecutive steps and the rings hold 3 * group
// buffers; b = (step / group) % 3 is the group's place in the ring:
//   copy-in stream : [wait until the launches that last read the group's input buffers are done]
//                    H2D spikes(step) -> in_ring[b * group + step % group] for every step of the group, back to back
//   compute stream : wait for those copies [and for the copy-outs that last read the group's output buffers];
//                    one launch per step
//   copy-out stream: wait for the launches; D2H of every step's result -> host result slot step % out_slots
// Cross-stream waits sit only between groups: with one per step (group = 1) the copy engines idled ~20 us per
// step between copies on a link that moves 4 MB in 77 us.
// At entry the two copy streams wait for what is already enqueued on the compute stream, at exit the compute
// stream waits for the last copy in either direction: an event recorded on the compute stream before / after
// the call brackets the whole run.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#include "abi.h"

namespace bpl {
namespace {

constexpr int RING = 3;

struct Events {
    cudaEvent_t done_in[RING], read_in[RING], done_c[RING], done_out[RING], edge;
    bool ok = false;
    Events() {
        cudaEvent_t *all[] = {done_in, read_in, done_c, done_out};
        ok = true;
        for (auto *group : all)
            for (int i = 0; i < RING; ++i)
                if (cudaEventCreateWithFlags(&group[i], cudaEventDisableTiming) != cudaSuccess) ok = false;
        if (cudaEventCreateWithFlags(&edge, cudaEventDisableTiming) != cudaSuccess) ok = false;
    }
    ~Events() {
        cudaEvent_t *all[] = {done_in, read_in, done_c, done_out};
        for (auto *group : all)
            for (int i = 0; i < RING; ++i) cudaEventDestroy(group[i]);
        cudaEventDestroy(edge);
    }
};

struct Runtime {
    bool failed = false;
    void operator()(cudaError_t e) {
        if (e != cudaSuccess && !failed) {
            failed = true;
            set_status(BPL_ERR_CUDA, cudaGetErrorString(e));
        }
    }
};

constexpr uint32_t MAX_GROUP = 16;

bool rings_ok(void *const *ring, uint32_t group = 1) {
    if (ring == nullptr) return false;
    for (uint32_t i = 0; i < RING * group; ++i)
        if (ring[i] == nullptr) return false;
    return true;
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {

// One registered target called n_steps times.  buffers[in_index] / buffers[out_index] / buffers[ws_index] are
// replaced per step by a buffer of in_ring / out_ring / ws_ring (3 * group buffers each; ws_index < 0: the target
// needs no workspace, or all steps may share the one in `buffers`: the launches are ordered on one stream).
void bpl_run_host_steps(const char *target_name, const char *opaque, size_t opaque_len, void *const *buffers,
                        int n_buffers, int in_index, int out_index, int ws_index, void *const *in_ring,
                        void *const *out_ring, void *const *ws_ring, uint32_t group, const void *host_in,
                        size_t in_bytes, void *host_out, size_t out_bytes, uint32_t out_slots, uint32_t n_steps,
                        bpl_stream_t s_in, bpl_stream_t s_compute, bpl_stream_t s_out) {
    const bpl_custom_call_t target = target_name == nullptr ? nullptr : bpl_find_target(target_name);
    if (target == nullptr) {
        set_status(BPL_ERR_ARGUMENT, "host steps: unknown target");
        return;
    }
    if (group == 0 || group > MAX_GROUP) {
        set_status(BPL_ERR_ARGUMENT, "host steps: group must be 1..16");
        return;
    }
    if (buffers == nullptr || n_buffers <= 0 || n_buffers > 16 || in_index < 0 || in_index >= n_buffers || out_index < 0 ||
        out_index >= n_buffers || in_index == out_index || ws_index >= n_buffers || !rings_ok(in_ring, group) ||
        !rings_ok(out_ring, group) || (ws_index >= 0 && !rings_ok(ws_ring, group)) || host_in == nullptr ||
        host_out == nullptr || out_slots == 0 || s_in == s_compute || s_out == s_compute || s_in == s_out) {
        set_status(BPL_ERR_ARGUMENT, "host steps: null buffer, index out of range, or streams that are not distinct");
        return;
    }
    if (n_steps == 0) return;
    Events ev;
    if (!ev.ok) {
        set_status(BPL_ERR_CUDA, "host steps: could not create the events");
        return;
    }
    Runtime rt;
    rt(cudaEventRecord(ev.edge, s_compute));
    rt(cudaStreamWaitEvent(s_in, ev.edge, 0));
    rt(cudaStreamWaitEvent(s_out, ev.edge, 0));
    void *args[16];
    std::memcpy(args, buffers, sizeof(void *) * n_buffers);
    const unsigned char *in = static_cast<const unsigned char *>(host_in);
    unsigned char *out = static_cast<unsigned char *>(host_out);
    const uint32_t n_groups = (n_steps + group - 1) / group;
    for (uint32_t g = 0; g < n_groups && !rt.failed; ++g) {
        const int b = static_cast<int>(g % RING);
        const uint32_t first = g * group, last = first + group < n_steps ? first + group : n_steps;
        if (g >= RING) {
            rt(cudaStreamWaitEvent(s_in, ev.done_c[b], 0));        // the launches that read these input buffers are done
            rt(cudaStreamWaitEvent(s_compute, ev.done_out[b], 0)); // the copy-outs that read these output buffers are done
        }
        for (uint32_t i = first; i < last; ++i)
            rt(cudaMemcpyAsync(in_ring[b * group + (i - first)], in + static_cast<size_t>(i) * in_bytes, in_bytes,
                               cudaMemcpyHostToDevice, s_in));
        rt(cudaEventRecord(ev.done_in[b], s_in));
        rt(cudaStreamWaitEvent(s_compute, ev.done_in[b], 0));
        for (uint32_t i = first; i < last; ++i) {
            const uint32_t slot = b * group + (i - first);
            args[in_index] = in_ring[slot];
            args[out_index] = out_ring[slot];
            if (ws_index >= 0) args[ws_index] = ws_ring[slot];
            target(s_compute, args, opaque, opaque_len);
        }
        rt(cudaEventRecord(ev.done_c[b], s_compute));
        rt(cudaStreamWaitEvent(s_out, ev.done_c[b], 0));
        for (uint32_t i = first; i < last; ++i)
            rt(cudaMemcpyAsync(out + static_cast<size_t>(i % out_slots) * out_bytes, out_ring[b * group + (i - first)],
                               out_bytes, cudaMemcpyDeviceToHost, s_out));
        rt(cudaEventRecord(ev.done_out[b], s_out));
    }
    rt(cudaEventRecord(ev.edge, s_in));
    rt(cudaStreamWaitEvent(s_compute, ev.edge, 0));
    rt(cudaStreamWaitEvent(s_compute, ev.done_out[(n_groups - 1) % RING], 0));
}

}  // extern "C"

namespace bpl {
namespace {

// The one-launch sharded step (bpl_sharded_prime, then one step launch per step) on host-resident spike trains:
// host_events holds n_steps slices of this rank's own n_local spike sources, host_out takes this rank's n_out outputs
// per step (slot step % out_slots).  Step i scatters the spikes of step i and pushes those of step i + 1, so the
// spikes of steps g * group + 1 .. (g + 1) * group are the inputs of the group of steps g * group .. (g + 1) * group - 1.
// ev_ring: 3 * group + 1 buffers of n_local events (the last one takes the spikes of step 0, which the prime call
// pushes; the spikes of step j >= 1 go to buffer (j - 1) % (3 * group)); y_ring: 3 * group buffers of n_out floats
// (step i scatters into buffer i % (3 * group) and zero-fills the next one).
// `step(stream, y_cur, y_next, next_events)` enqueues the launch of one step on the rank's shard.
template<typename Step>
void sharded_run_host_steps_impl(Step step, uint32_t n_out, int ev_is_float, uint32_t n_local, uint32_t row_offset,
                                 void *const *peer_lists, size_t slot_bytes, void *const *peer_flags, void *state,
                                 int world, int rank, int slots, void *const *ev_ring, void *const *y_ring,
                                 uint32_t group, const void *host_events, void *host_out, uint32_t out_slots,
                                 uint32_t n_steps, bpl_stream_t s_in, bpl_stream_t s_compute, bpl_stream_t s_out) {
    if (group == 0 || group > MAX_GROUP) {
        set_status(BPL_ERR_ARGUMENT, "sharded host steps: group must be 1..16");
        return;
    }
    if (!rings_ok(ev_ring, group) || ev_ring[RING * group] == nullptr || !rings_ok(y_ring, group) ||
        host_events == nullptr || host_out == nullptr || out_slots == 0 || s_in == s_compute || s_out == s_compute ||
        s_in == s_out) {
        set_status(BPL_ERR_ARGUMENT, "sharded host steps: null buffer or streams that are not distinct");
        return;
    }
    if (n_steps == 0) return;
    Events ev;
    if (!ev.ok) {
        set_status(BPL_ERR_CUDA, "sharded host steps: could not create the events");
        return;
    }
    Runtime rt;
    const uint32_t ring = RING * group;
    const size_t in_bytes = static_cast<size_t>(n_local) * (ev_is_float ? 4 : 1);
    const size_t out_bytes = static_cast<size_t>(n_out) * 4;
    const unsigned char *in = static_cast<const unsigned char *>(host_events);
    unsigned char *out = static_cast<unsigned char *>(host_out);
    rt(cudaEventRecord(ev.edge, s_compute));
    rt(cudaStreamWaitEvent(s_in, ev.edge, 0));
    rt(cudaStreamWaitEvent(s_out, ev.edge, 0));
    // the spikes of step 0, pushed by the prime call, which also zero-fills the first output buffer
    rt(cudaMemcpyAsync(ev_ring[ring], in, in_bytes, cudaMemcpyHostToDevice, s_in));
    rt(cudaEventRecord(ev.read_in[0], s_in));
    rt(cudaStreamWaitEvent(s_compute, ev.read_in[0], 0));
    bpl_sharded_prime(s_compute, ev_ring[ring], ev_is_float, n_local, row_offset, peer_lists, slot_bytes, peer_flags, state,
                      world, rank, slots, y_ring[0], n_out);
    const uint32_t n_groups = (n_steps + group - 1) / group;
    for (uint32_t g = 0; g < n_groups && !rt.failed; ++g) {
        const int b = static_cast<int>(g % RING);
        const uint32_t first = g * group, last = first + group < n_steps ? first + group : n_steps;   // steps [first, last)
        // inputs of the group: the spikes of steps first + 1 .. last (those of step n_steps do not exist)
        if (g >= RING) rt(cudaStreamWaitEvent(s_in, ev.done_c[b], 0));   // the launches that pushed these buffers are done
        for (uint32_t j = first + 1; j <= last && j < n_steps; ++j)
            rt(cudaMemcpyAsync(ev_ring[(j - 1) % ring], in + static_cast<size_t>(j) * in_bytes, in_bytes,
                               cudaMemcpyHostToDevice, s_in));
        rt(cudaEventRecord(ev.done_in[b], s_in));
        rt(cudaStreamWaitEvent(s_compute, ev.done_in[b], 0));
        // the group scatters into its own output buffers and zero-fills the first one of the next group: the copy-outs
        // of the group two back (and, the stream being ordered, of every earlier one) must be done
        if (g >= 2) rt(cudaStreamWaitEvent(s_compute, ev.done_out[(g - 2) % RING], 0));
        for (uint32_t i = first; i < last; ++i) {
            const bool final_step = i + 1 == n_steps;
            step(s_compute, y_ring[i % ring], final_step ? nullptr : y_ring[(i + 1) % ring],
                 final_step ? nullptr : ev_ring[i % ring]);
        }
        rt(cudaEventRecord(ev.done_c[b], s_compute));
        rt(cudaStreamWaitEvent(s_out, ev.done_c[b], 0));
        for (uint32_t i = first; i < last; ++i)
            rt(cudaMemcpyAsync(out + static_cast<size_t>(i % out_slots) * out_bytes, y_ring[i % ring], out_bytes,
                               cudaMemcpyDeviceToHost, s_out));
        rt(cudaEventRecord(ev.done_out[b], s_out));
    }
    rt(cudaEventRecord(ev.edge, s_in));
    rt(cudaStreamWaitEvent(s_compute, ev.edge, 0));
    rt(cudaStreamWaitEvent(s_compute, ev.done_out[(n_groups - 1) % RING], 0));
}

}  // namespace
}  // namespace bpl

extern "C" {

// The shard in the column-blocked layout (bpl_sharded_cb_step per step).
void bpl_sharded_run_host_steps(const void *groups, const void *offsets, uint32_t n_out, uint32_t block_width,
                                int fixed_point, int scale_log2, uint32_t team_lanes_log2, int ev_is_float,
                                uint32_t n_local, uint32_t row_offset, void *const *peer_lists, size_t slot_bytes,
                                void *const *peer_flags, void *state, int world, int rank, int slots, uint32_t max_polls,
                                void *const *ev_ring, void *const *y_ring, uint32_t group, const void *host_events,
                                void *host_out, uint32_t out_slots, uint32_t n_steps, bpl_stream_t s_in,
                                bpl_stream_t s_compute, bpl_stream_t s_out) {
    sharded_run_host_steps_impl(
        [&](bpl_stream_t s, void *y_cur, void *y_next, const void *next_events) {
            bpl_sharded_cb_step(s, groups, offsets, n_out, block_width, fixed_point, scale_log2, team_lanes_log2, y_cur,
                                y_next, next_events, ev_is_float, n_local, row_offset, peer_lists, slot_bytes, peer_flags,
                                state, world, rank, slots, max_polls);
        },
        n_out, ev_is_float, n_local, row_offset, peer_lists, slot_bytes, peer_flags, state, world, rank, slots, ev_ring,
        y_ring, group, host_events, host_out, out_slots, n_steps, s_in, s_compute, s_out);
}

// The shard as plain CSR arrays (bpl_sharded_step per step).
void bpl_sharded_run_host_steps_csr(const void *data, const void *indices, const void *indptr, uint32_t n_row,
                                    uint32_t n_out, int ev_is_float, uint32_t n_local, uint32_t row_offset,
                                    void *const *peer_lists, size_t slot_bytes, void *const *peer_flags, void *state,
                                    int world, int rank, int slots, uint32_t max_polls, void *const *ev_ring,
                                    void *const *y_ring, uint32_t group, const void *host_events, void *host_out,
                                    uint32_t out_slots, uint32_t n_steps, bpl_stream_t s_in, bpl_stream_t s_compute,
                                    bpl_stream_t s_out) {
    sharded_run_host_steps_impl(
        [&](bpl_stream_t s, void *y_cur, void *y_next, const void *next_events) {
            bpl_sharded_step(s, data, indices, indptr, n_row, n_out, y_cur, y_next, next_events, ev_is_float, n_local,
                             row_offset, peer_lists, slot_bytes, peer_flags, state, world, rank, slots, max_polls);
        },
        n_out, ev_is_float, n_local, row_offset, peer_lists, slot_bytes, peer_flags, state, world, rank, slots, ev_ring,
        y_ring, group, host_events, host_out, out_slots, n_steps, s_in, s_compute, s_out);
}

}  // extern "C"
