// Runs of many steps on HOST-resident spike trains (no counterpart in the reference, whose callers feed one
// device array per call from Python): every step's spikes come from pinned host memory and every step's result
// goes back to pinned host memory, with the copy in, the compute launch and the copy out of neighbouring steps
// overlapped on three streams over rings of three device buffers.  The whole run is enqueued by native code in
// one call, so the dozen runtime calls a step needs cost microseconds, not an interpreter's dispatch each.
//
// Ordering inside a run (b = step % 3):
//   copy-in stream : [wait until the launch that last read in_ring[b] is done] H2D spikes(step) -> in_ring[b]
//   compute stream : wait for that copy [and for the copy-out that last read out_ring[b]]; launch
//   copy-out stream: wait for the launch; D2H out_ring[b] -> host result slot step % out_slots
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

bool rings_ok(void *const *ring) {
    if (ring == nullptr) return false;
    for (int i = 0; i < RING; ++i)
        if (ring[i] == nullptr) return false;
    return true;
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {

// One registered target called n_steps times.  buffers[in_index] / buffers[out_index] / buffers[ws_index] are
// replaced per step by in_ring / out_ring / ws_ring[step % 3] (ws_index < 0: the target needs no workspace, or all
// steps may share the one in `buffers`: the launches are ordered on one stream).
void bpl_run_host_steps(const char *target_name, const char *opaque, size_t opaque_len, void *const *buffers,
                        int n_buffers, int in_index, int out_index, int ws_index, void *const *in_ring,
                        void *const *out_ring, void *const *ws_ring, const void *host_in, size_t in_bytes,
                        void *host_out, size_t out_bytes, uint32_t out_slots, uint32_t n_steps, bpl_stream_t s_in,
                        bpl_stream_t s_compute, bpl_stream_t s_out) {
    const bpl_custom_call_t target = target_name == nullptr ? nullptr : bpl_find_target(target_name);
    if (target == nullptr) {
        set_status(BPL_ERR_ARGUMENT, "host steps: unknown target");
        return;
    }
    if (buffers == nullptr || n_buffers <= 0 || n_buffers > 16 || in_index < 0 || in_index >= n_buffers || out_index < 0 ||
        out_index >= n_buffers || in_index == out_index || ws_index >= n_buffers || !rings_ok(in_ring) ||
        !rings_ok(out_ring) || (ws_index >= 0 && !rings_ok(ws_ring)) || host_in == nullptr || host_out == nullptr ||
        out_slots == 0 || s_in == s_compute || s_out == s_compute || s_in == s_out) {
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
    void *args[RING][16];
    for (int b = 0; b < RING; ++b) {
        std::memcpy(args[b], buffers, sizeof(void *) * n_buffers);
        args[b][in_index] = in_ring[b];
        args[b][out_index] = out_ring[b];
        if (ws_index >= 0) args[b][ws_index] = ws_ring[b];
    }
    const unsigned char *in = static_cast<const unsigned char *>(host_in);
    unsigned char *out = static_cast<unsigned char *>(host_out);
    for (uint32_t i = 0; i < n_steps && !rt.failed; ++i) {
        const int b = static_cast<int>(i % RING);
        if (i >= RING) {
            rt(cudaStreamWaitEvent(s_in, ev.done_c[b], 0));        // the launch that read in_ring[b] has finished
            rt(cudaStreamWaitEvent(s_compute, ev.done_out[b], 0)); // the copy-out that read out_ring[b] has finished
        }
        rt(cudaMemcpyAsync(in_ring[b], in + static_cast<size_t>(i) * in_bytes, in_bytes, cudaMemcpyHostToDevice, s_in));
        rt(cudaEventRecord(ev.done_in[b], s_in));
        rt(cudaStreamWaitEvent(s_compute, ev.done_in[b], 0));
        target(s_compute, args[b], opaque, opaque_len);
        rt(cudaEventRecord(ev.done_c[b], s_compute));
        rt(cudaStreamWaitEvent(s_out, ev.done_c[b], 0));
        rt(cudaMemcpyAsync(out + static_cast<size_t>(i % out_slots) * out_bytes, out_ring[b], out_bytes,
                           cudaMemcpyDeviceToHost, s_out));
        rt(cudaEventRecord(ev.done_out[b], s_out));
    }
    rt(cudaEventRecord(ev.edge, s_in));
    rt(cudaStreamWaitEvent(s_compute, ev.edge, 0));
    rt(cudaStreamWaitEvent(s_compute, ev.done_out[(n_steps - 1) % RING], 0));
}

// The one-launch sharded step (bpl_sharded_prime, then bpl_sharded_cb_step per step) on host-resident spike trains:
// host_events holds n_steps slices of this rank's own n_local spike sources, host_out takes this rank's n_out outputs
// per step (slot step % out_slots).  ev_ring[3]: n_local events each; y_ring[3]: n_out floats each.
void bpl_sharded_run_host_steps(const void *groups, const void *offsets, uint32_t n_out, uint32_t block_width,
                                int fixed_point, int scale_log2, uint32_t team_lanes_log2, int ev_is_float,
                                uint32_t n_local, uint32_t row_offset, void *const *peer_lists, size_t slot_bytes,
                                void *const *peer_flags, void *state, int world, int rank, int slots, uint32_t max_polls,
                                void *const *ev_ring, void *const *y_ring, const void *host_events, void *host_out,
                                uint32_t out_slots, uint32_t n_steps, bpl_stream_t s_in, bpl_stream_t s_compute,
                                bpl_stream_t s_out) {
    if (!rings_ok(ev_ring) || !rings_ok(y_ring) || host_events == nullptr || host_out == nullptr || out_slots == 0 ||
        s_in == s_compute || s_out == s_compute || s_in == s_out) {
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
    const size_t in_bytes = static_cast<size_t>(n_local) * (ev_is_float ? 4 : 1);
    const size_t out_bytes = static_cast<size_t>(n_out) * 4;
    const unsigned char *in = static_cast<const unsigned char *>(host_events);
    unsigned char *out = static_cast<unsigned char *>(host_out);
    rt(cudaEventRecord(ev.edge, s_compute));
    rt(cudaStreamWaitEvent(s_in, ev.edge, 0));
    rt(cudaStreamWaitEvent(s_out, ev.edge, 0));
    // read_in[b]: the launch that compacted and pushed ev_ring[b] has finished
    auto copy_in = [&](uint32_t j) {
        const int b = static_cast<int>(j % RING);
        if (j >= RING) rt(cudaStreamWaitEvent(s_in, ev.read_in[b], 0));
        rt(cudaMemcpyAsync(ev_ring[b], in + static_cast<size_t>(j) * in_bytes, in_bytes, cudaMemcpyHostToDevice, s_in));
        rt(cudaEventRecord(ev.done_in[b], s_in));
    };
    copy_in(0);
    rt(cudaStreamWaitEvent(s_compute, ev.done_in[0], 0));
    bpl_sharded_prime(s_compute, ev_ring[0], ev_is_float, n_local, row_offset, peer_lists, slot_bytes, peer_flags, state,
                      world, rank, slots, y_ring[0], n_out);
    rt(cudaEventRecord(ev.read_in[0], s_compute));
    for (uint32_t i = 0; i < n_steps && !rt.failed; ++i) {
        const bool last = i + 1 == n_steps;
        const int b = static_cast<int>(i % RING), nb = static_cast<int>((i + 1) % RING);
        if (!last) {
            copy_in(i + 1);
            rt(cudaStreamWaitEvent(s_compute, ev.done_in[nb], 0));
            if (i + 1 >= RING) rt(cudaStreamWaitEvent(s_compute, ev.done_out[nb], 0));   // this launch zero-fills y_ring[nb]
        }
        bpl_sharded_cb_step(s_compute, groups, offsets, n_out, block_width, fixed_point, scale_log2, team_lanes_log2,
                            y_ring[b], last ? nullptr : y_ring[nb], last ? nullptr : ev_ring[nb], ev_is_float, n_local,
                            row_offset, peer_lists, slot_bytes, peer_flags, state, world, rank, slots, max_polls);
        if (!last) rt(cudaEventRecord(ev.read_in[nb], s_compute));
        rt(cudaEventRecord(ev.done_c[b], s_compute));
        rt(cudaStreamWaitEvent(s_out, ev.done_c[b], 0));
        rt(cudaMemcpyAsync(out + static_cast<size_t>(i % out_slots) * out_bytes, y_ring[b], out_bytes,
                           cudaMemcpyDeviceToHost, s_out));
        rt(cudaEventRecord(ev.done_out[b], s_out));
    }
    rt(cudaEventRecord(ev.edge, s_in));
    rt(cudaStreamWaitEvent(s_compute, ev.edge, 0));
    rt(cudaStreamWaitEvent(s_compute, ev.done_out[(n_steps - 1) % RING], 0));
}

}  // extern "C"
