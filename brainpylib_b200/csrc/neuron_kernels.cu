// The caller's side of synaptic propagation in one kernel (no counterpart in brainpylib, whose operators stop at
// the product): conductance decay, summation of the propagated input, leaky integrate-and-fire update with
// refractory period, threshold and reset, AND the compaction of the new spikes into the spike list that the
// list-driven transposed event products consume.  It is the step pattern of the reference's own network example,
// brainpylib/_src/op_register/tests/ei_net.py:47-72:
//
//     g = g * exp(-dt / tau_syn);  g += event_sum(pre.spike, ...);  post.input += g * (E - post.V)      (:47-54)
//     LIF neurons with exponential-Euler integration, refractory period, threshold, reset               (:57-63)
//
// The neuron and synapse models themselves live in BrainPy (`bp.neurons.LIF`, `bp.odeint(..., method='exp_auto')`),
// a dependency that is not part of the reference tree; their published update rule is restated here:
//     refractory = (t - t_last) <= tau_ref
//     V_inf = V_rest + R * I;   V' = V_inf + (V - V_inf) * exp(-dt / tau);   V' = refractory ? V : V'
//     spike = V' >= V_th;   t_last = spike ? t : t_last;   V = spike ? V_reset : V'
// Every product and sum is rounded on its own (no fused multiply-add), in the order written, so that a float32
// array implementation of the same formulas gives the same bits (the spikes feed back, so a last-bit difference
// would grow into different spike trains).
//
//   lif_exp_step_float
//   opaque  LifExpDescriptor (below)
//   buffers [y f32(K, n)   propagated input per synaptic channel; READ, THEN ZERO-FILLED for the next step
//            g f32(K, n)   conductances, updated in place
//            V f32(n), t_last f32(n)   membrane potential and last spike time, updated in place
//            spikes f32(n) out: 1.0 where the neuron fired, else 0.0
//            list u32      out: counts[1024] then row ids in chunk segments, the layout of the workspace of
//                          event_csr_matvec (bpl_workspace_bytes of that target for n rows)]
// What it saves per step against separate operators: the event-vector round trip (the scatter reads the list, not
// the 4 B per neuron vector), the spike-scan launch, the zero-fill of y, and the elementwise launches of the update.
#include "abi.h"
#include "common.cuh"
#include "spike_scan.cuh"

namespace bpl {
namespace {

constexpr int LIF_MAX_CHANNELS = 4;

struct LifExpDescriptor {
    unsigned int n;             // neurons
    unsigned int n_channels;    // synaptic channels K (1..4), e.g. excitatory and inhibitory
    float t, dt_unused;         // time of this step (for the refractory test); second field reserved
    float syn_decay[LIF_MAX_CHANNELS];   // exp(-dt / tau_syn) per channel
    float E_rev[LIF_MAX_CHANNELS];       // reversal potential per channel
    float ext_input;            // constant external input added to every neuron
    float V_rest, V_th, V_reset, R, lif_decay /* exp(-dt / tau) */, tau_ref;
};
static_assert(sizeof(LifExpDescriptor) == 76, "layout");

// 1024 threads per 4096-neuron tile (4 neurons per thread, a warp covers 128 consecutive neurons): the kernel is a
// stream of ~50 bytes per neuron and needs many loads in flight; with the spike scan's 256 threads per tile (16
// neurons per thread) a million neurons kept only 13 warps per SM busy and ran at 2.5x its memory time.
constexpr int LIF_THREADS = 1024;
constexpr int LIF_PER_THREAD = SCAN_TILE / LIF_THREADS;          // 4
constexpr int LIF_WARP_SPAN = 32 * LIF_PER_THREAD;               // 128

__global__ void __launch_bounds__(LIF_THREADS)
lif_exp_step_kernel(float *__restrict__ y, float *__restrict__ g, float *__restrict__ V, float *__restrict__ t_last,
                    float *__restrict__ spikes, const LifExpDescriptor d, const uint32_t chunk, const uint32_t n_chunks,
                    uint32_t *__restrict__ counts, uint32_t *__restrict__ ids) {
    if (blockIdx.x >= n_chunks) return;
    __shared__ uint32_t warp_total[LIF_THREADS / 32];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t n = d.n;
    const uint64_t chunk_begin = static_cast<uint64_t>(blockIdx.x) * chunk;
    const uint64_t chunk_end = min(chunk_begin + chunk, static_cast<uint64_t>(n));
    uint32_t *out = ids + chunk_begin;
    uint32_t running = 0;
    for (uint64_t tile = chunk_begin; tile < chunk_end; tile += SCAN_TILE) {
        const uint64_t base = tile + static_cast<uint64_t>(warp) * LIF_WARP_SPAN;
        bool act[LIF_PER_THREAD];
#pragma unroll
        for (int k = 0; k < LIF_PER_THREAD; ++k) {
            const uint64_t i = base + k * 32 + lane;
            act[k] = false;
            if (i < chunk_end) {
                const float v = V[i];
                float input = d.ext_input;
                for (uint32_t c = 0; c < d.n_channels; ++c) {
                    const uint64_t at = static_cast<uint64_t>(c) * n + i;
                    const float gc = __fadd_rn(__fmul_rn(g[at], d.syn_decay[c]), y[at]);
                    g[at] = gc;
                    y[at] = 0.0f;
                    input = __fadd_rn(input, __fmul_rn(gc, __fsub_rn(d.E_rev[c], v)));
                }
                const float tl = t_last[i];
                const bool refractory = __fsub_rn(d.t, tl) <= d.tau_ref;
                const float v_inf = __fadd_rn(d.V_rest, __fmul_rn(d.R, input));
                float v_new = __fadd_rn(v_inf, __fmul_rn(__fsub_rn(v, v_inf), d.lif_decay));
                if (refractory) v_new = v;
                const bool spike = v_new >= d.V_th;
                act[k] = spike;
                V[i] = spike ? d.V_reset : v_new;
                if (spike) t_last[i] = d.t;
                spikes[i] = spike ? 1.0f : 0.0f;
            }
        }
        uint32_t bits[LIF_PER_THREAD];
        uint32_t total = 0;
#pragma unroll
        for (int k = 0; k < LIF_PER_THREAD; ++k) {
            bits[k] = __ballot_sync(FULL_MASK, act[k]);
            total += __popc(bits[k]);
        }
        if (lane == 0) warp_total[warp] = total;
        __syncthreads();
        uint32_t offset = running, tile_total = 0;
#pragma unroll
        for (int w = 0; w < LIF_THREADS / 32; ++w) {
            const uint32_t t = warp_total[w];
            if (w < static_cast<int>(warp)) offset += t;
            tile_total += t;
        }
        __syncthreads();
        const uint32_t below = (1u << lane) - 1u;
#pragma unroll
        for (int k = 0; k < LIF_PER_THREAD; ++k) {
            if (act[k]) out[offset + __popc(bits[k] & below)] = static_cast<uint32_t>(base + k * 32 + lane);
            offset += __popc(bits[k]);
        }
        running += tile_total;
    }
    if (threadIdx.x == 0) counts[blockIdx.x] = running;
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {

size_t bpl_build_lif_exp_descriptor(uint32_t n, uint32_t n_channels, float t, const float *syn_decay, const float *E_rev,
                                    float ext_input, float V_rest, float V_th, float V_reset, float R, float lif_decay,
                                    float tau_ref, void *out, size_t cap) {
    if (out == nullptr || cap < sizeof(LifExpDescriptor) || n_channels < 1 || n_channels > LIF_MAX_CHANNELS ||
        syn_decay == nullptr || E_rev == nullptr)
        return 0;
    LifExpDescriptor d;
    __builtin_memset(&d, 0, sizeof(d));
    d.n = n; d.n_channels = n_channels; d.t = t;
    for (uint32_t c = 0; c < n_channels; ++c) { d.syn_decay[c] = syn_decay[c]; d.E_rev[c] = E_rev[c]; }
    d.ext_input = ext_input; d.V_rest = V_rest; d.V_th = V_th; d.V_reset = V_reset; d.R = R; d.lif_decay = lif_decay;
    d.tau_ref = tau_ref;
    __builtin_memcpy(out, &d, sizeof(d));
    return sizeof(d);
}

void lif_exp_step_float(bpl_stream_t stream, void **buffers, const char *opaque, size_t opaque_len) {
    const LifExpDescriptor *d = unpack<LifExpDescriptor>(opaque, opaque_len);
    if (!d) return;
    if (d->n_channels < 1 || d->n_channels > LIF_MAX_CHANNELS) {
        set_status(BPL_ERR_ARGUMENT, "lif_exp_step: 1..4 synaptic channels");
        return;
    }
    for (int b = 0; b < 6; ++b)
        if (buffers[b] == nullptr) {
            set_status(BPL_ERR_ARGUMENT, "lif_exp_step: null buffer");
            return;
        }
    uint32_t *list = static_cast<uint32_t *>(buffers[5]);
    const ScanPlan p = plan_scan(d->n);
    if (d->n == 0) return;
    lif_exp_step_kernel<<<p.n_chunks, LIF_THREADS, 0, stream>>>(
        static_cast<float *>(buffers[0]), static_cast<float *>(buffers[1]), static_cast<float *>(buffers[2]),
        static_cast<float *>(buffers[3]), static_cast<float *>(buffers[4]), *d, p.chunk, p.n_chunks, list,
        list + MAX_CHUNKS);
    launch_ok();
}

}  // extern "C"
