// Transposed event product on a column-blocked matrix: the device code shared by the stand-alone
// operator (cbcsr_kernels.cu) and by the sharded step kernel (exchange_kernels.cu).
//
// Format (built once per matrix by cbcsr_build.cu).  The post-synaptic neurons are cut into blocks
// of `width` columns.  The matrix stays row-major: the synapses of row r lie together, grouped by
// the block of their target, and every (row, block) segment is stored as whole GROUPS of 8
// synapses, 48 bytes each:
//
//     float | int32  w[8]   weights; fixed-point matrices hold round(w * 2^k) as int32   (bytes  0..31)
//     uint16_t       c[8]   column - block * width                                        (bytes 32..47)
//
// A segment whose length is not a multiple of 8 ends in padding synapses (w = 0, c = 0), which
// add nothing.  offsets[r][b] (uint32, in groups, row stride n_blocks + 1) is where row r's segment
// for block b starts, offsets[r][b + 1] where it ends; offsets[r][n_blocks] == offsets[r + 1][0].
//
// Kernel.  A CTA owns one block's slice of y in shared memory and one of P interleaved shares of the
// active rows; its 32 warps split those rows and run independently of one another (no barrier in the
// main loop, no wait on another warp).  A warp resolves 32 of its rows at a time, one per lane (spike
// list -> row -> segment of this block), with the next 32 already in flight, and then streams the
// segments through a private ring of small shared-memory buffers.  A buffer has 32 slots of one group;
// a team of L lanes (L = 4, 8, 16 or 32, chosen from the mean segment length when the matrix is
// prepared) owns L consecutive slots and copies up to L groups of ONE segment into them with 16-byte
// `cp.async`, so a round moves 32 / L segments and needs no packing: where a piece lands is fixed.  The
// round is committed as one group, and while it is in flight the warp adds the oldest buffer into the
// slice: lane l takes slot l (if its team filled it), one shared-memory atomic per synapse.  A segment
// longer than L groups simply stays at the head of the queue for another round.  At the end the P
// slices of a block are added into the zero-filled y with 16-byte vector reductions.
//
// Measured alternatives that lost (1e6 x 1e6, 1000 synapses per row, 1 % of the rows active, 37 blocks):
// one producer warp feeding the others with one `cp.async.bulk` per segment: 4x slower (a segment is
// ~190 bytes and the copy engine has a per-copy cost); one lane per segment with plain 16-byte loads
// into registers: 2x slower (every lane of a load instruction touches a different sector); a ticketed
// combine of the P slices through a scratch area instead of the reductions: 5 us slower; a deeper or
// shallower ring: no change, the loop is bound by the instructions it issues per round, not by memory
// latency; pieces packed back to back (a prefix sum over the teams per round) instead of fixed slots:
// about twice the instructions per row.
//
// FIXED = false: float accumulators.  A float add on shared memory is a compare-and-swap loop on this
// hardware (about 3.4 per clock per SM at random addresses, each a chain of dependent instructions).
// FIXED = true: 32-bit fixed-point accumulators; an integer add on shared memory is one fire-and-forget
// instruction (about 11 per clock per SM).  The weights were rounded to multiples of 2^-k when the
// matrix was prepared, k chosen so that no column can overflow even if every row spikes; the result
// is exact but for that rounding, and does not depend on the order of the additions.
#ifndef BPL_CSRC_CB_SCATTER_CUH_
#define BPL_CSRC_CB_SCATTER_CUH_

#include "abi.h"
#include "common.cuh"
#include "spike_scan.cuh"

namespace bpl {
namespace {

constexpr int CB_THREADS = 1024;
constexpr int CB_WARPS = CB_THREADS / 32;
constexpr uint32_t CB_GROUP_BYTES = 48;
constexpr uint32_t CB_MAX_WIDTH = 32256;           // 126 KB of shared memory for the slice, the rest for two ring buffers per warp
constexpr uint32_t CB_MAX_BLOCKS = 1024;
// static shared memory of a kernel that calls cb_scatter_body (prefix, warp totals), rounded up
constexpr uint32_t CB_STATIC_SMEM = 4608;
constexpr uint32_t CB_SMEM_LIMIT = 232448 - CB_STATIC_SMEM;           // 227 KB per CTA on sm_100

constexpr uint32_t CB_BUF_GROUPS = 32;             // slots per ring buffer: one per lane
constexpr uint32_t CB_BUF_BYTES = CB_BUF_GROUPS * CB_GROUP_BYTES;   // 1536

// ---- shared-memory layout, computed on the host and passed to the kernel ----
//   acc [acc_bytes]   then per warp a ring of n_buf buffers of 32 groups
struct CbPlan {
    uint32_t n_buf;        // ring buffers per warp (2; the kernels also exist for 3)
    uint32_t acc_bytes;    // slice of y, rounded up to 16 bytes
    uint32_t smem_bytes;   // dynamic shared memory of the launch
    bool ok;
};

inline CbPlan cb_plan(uint32_t width, uint32_t extra_bytes = 0) {
    CbPlan p{};
    p.acc_bytes = (width * 4u + 15u) & ~15u;
    const uint32_t limit = CB_SMEM_LIMIT - extra_bytes;
    p.ok = false;
    if (p.acc_bytes + CB_WARPS * 2u * CB_BUF_BYTES > limit) return p;
    // Two buffers per warp even where three would fit: a third adds nothing to the stream (measured with 2, 3 and 4),
    // and the 48 KB it takes from the L1 cache slows the list and offset loads, which go through L1 (shards of 1/2 and
    // 1/4 of the benchmark matrix: 31.8 -> 28.2 us and 22.7 -> 20.1 us per launch).
    p.n_buf = 2u;
    p.smem_bytes = p.acc_bytes + CB_WARPS * p.n_buf * CB_BUF_BYTES;
    p.ok = true;
    return p;
}

// ---- asynchronous 16-byte copies global -> shared ----
__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 :: "r"(smem_addr(dst)), "l"(__cvta_generic_to_global(src)) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template<int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

__device__ __forceinline__ void red_add_v4(float *p, float a, float b, float c, float d) {
    asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

struct CbGroup { uint4 wa, wb, cc; };

template<bool FIXED>
__device__ __forceinline__ void cb_add(float *acc, const uint32_t c, const uint32_t w_bits) {
    if (FIXED) {
        if (w_bits != 0u) atomicAdd(reinterpret_cast<int *>(acc) + c, static_cast<int>(w_bits));
    } else {
        const float w = __uint_as_float(w_bits);
        if (w != 0.0f) atomicAdd(acc + c, w);   // padding synapses and zero weights add nothing
    }
}

// float accumulation of a group whose weights are scaled by the row's factor (dense vector product)
__device__ __forceinline__ void cb_add_scaled(float *acc, const uint32_t c, const uint32_t w_bits, const float scale) {
    const float w = __uint_as_float(w_bits);
    if (w != 0.0f) atomicAdd(acc + c, w * scale);
}
__device__ __forceinline__ void cb_add_group_scaled(float *acc, const CbGroup &g, const float s) {
    cb_add_scaled(acc, g.cc.x & 0xffffu, g.wa.x, s);
    cb_add_scaled(acc, g.cc.x >> 16, g.wa.y, s);
    cb_add_scaled(acc, g.cc.y & 0xffffu, g.wa.z, s);
    cb_add_scaled(acc, g.cc.y >> 16, g.wa.w, s);
    cb_add_scaled(acc, g.cc.z & 0xffffu, g.wb.x, s);
    cb_add_scaled(acc, g.cc.z >> 16, g.wb.y, s);
    cb_add_scaled(acc, g.cc.w & 0xffffu, g.wb.z, s);
    cb_add_scaled(acc, g.cc.w >> 16, g.wb.w, s);
}

// gather direction: sum of weight * xs[column] over a group (xs: the block's slice of the vector in shared memory;
// padding synapses have weight 0 and column 0)
__device__ __forceinline__ float cb_dot_group(const float *xs, const CbGroup &g) {
    float s = __uint_as_float(g.wa.x) * xs[g.cc.x & 0xffffu];
    s = fmaf(__uint_as_float(g.wa.y), xs[g.cc.x >> 16], s);
    s = fmaf(__uint_as_float(g.wa.z), xs[g.cc.y & 0xffffu], s);
    s = fmaf(__uint_as_float(g.wa.w), xs[g.cc.y >> 16], s);
    s = fmaf(__uint_as_float(g.wb.x), xs[g.cc.z & 0xffffu], s);
    s = fmaf(__uint_as_float(g.wb.y), xs[g.cc.z >> 16], s);
    s = fmaf(__uint_as_float(g.wb.z), xs[g.cc.w & 0xffffu], s);
    s = fmaf(__uint_as_float(g.wb.w), xs[g.cc.w >> 16], s);
    return s;
}

template<bool FIXED>
__device__ __forceinline__ void cb_add_group(float *acc, const CbGroup &g) {
    cb_add<FIXED>(acc, g.cc.x & 0xffffu, g.wa.x);
    cb_add<FIXED>(acc, g.cc.x >> 16, g.wa.y);
    cb_add<FIXED>(acc, g.cc.y & 0xffffu, g.wa.z);
    cb_add<FIXED>(acc, g.cc.y >> 16, g.wa.w);
    cb_add<FIXED>(acc, g.cc.z & 0xffffu, g.wb.x);
    cb_add<FIXED>(acc, g.cc.z >> 16, g.wb.y);
    cb_add<FIXED>(acc, g.cc.w & 0xffffu, g.wb.z);
    cb_add<FIXED>(acc, g.cc.w >> 16, g.wb.w);
}

// Lane `lane` adds the group in its slot of a ring buffer into the slice (when its team filled that slot).
// DENSE: the weights are multiplied by `scale`, the vector entry of the row the group belongs to.
template<bool FIXED, bool DENSE = false>
__device__ __forceinline__ void cb_accumulate(float *acc, const unsigned char *buf, const bool filled, const uint32_t lane,
                                              const float scale = 1.0f) {
    if (filled) {
        CbGroup grp;
        grp.wa = *reinterpret_cast<const uint4 *>(buf + lane * CB_GROUP_BYTES);
        grp.wb = *reinterpret_cast<const uint4 *>(buf + lane * CB_GROUP_BYTES + 16);
        grp.cc = *reinterpret_cast<const uint4 *>(buf + lane * CB_GROUP_BYTES + 32);
        if (DENSE) cb_add_group_scaled(acc, grp, scale);
        else cb_add_group<FIXED>(acc, grp);
    }
}

// Exclusive prefix over the chunk counts for a block of 1024 threads (one count per thread): prefix[k] for k < 1024,
// prefix[1024] = total; returns the total.  `warp_total`: shared, 32 words.
__device__ __forceinline__ uint32_t cb_chunk_prefix(const uint32_t *__restrict__ counts, const uint32_t n_chunks,
                                                    uint32_t *prefix, uint32_t *warp_total) {
    const uint32_t t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const uint32_t c = t < n_chunks ? counts[t] : 0u;
    uint32_t incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(FULL_MASK, incl, o);
        if (lane >= static_cast<uint32_t>(o)) incl += v;
    }
    if (lane == 31) warp_total[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const uint32_t w = warp_total[lane];
        uint32_t wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(FULL_MASK, wi, o);
            if (lane >= static_cast<uint32_t>(o)) wi += v;
        }
        warp_total[lane] = wi - w;
        if (lane == 31) prefix[MAX_CHUNKS] = wi;
    }
    __syncthreads();
    prefix[t] = warp_total[warp] + incl - c;
    __syncthreads();
    return prefix[MAX_CHUNKS];
}

// Optional phase stamps (nanoseconds of %globaltimer), 8 words per CTA, written when `trace` is not null:
//   0 entry   1 spike list prefix-summed   2 first rows of warp 0 resolved   3 earliest / 4 latest end of a
//   warp's streaming loop   5 all warps done   6 slice flushed
__device__ __forceinline__ unsigned long long cb_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void cb_stamp(unsigned long long *trace, const uint32_t cta, const int slot) {
    if (trace != nullptr) trace[static_cast<uint64_t>(cta) * 8u + slot] = cb_now();
}

// One CTA's work: block `b` of the columns, share `p` of `P` of the listed rows.
//   counts / ids: the spike list (chunk_prefix / list_row layout); y: this matrix's output, already zero.
//   smem: dynamic shared memory laid out by cb_plan; prefix / warp_total: static shared memory.
//   inv_scale: FIXED only, 2^-k.
//   DENSE (with x): y = A^T x for a dense vector x instead of a spike list: every row whose x is not zero is walked and
//   its weights are multiplied by x[row] (float accumulation only); counts / ids are not read, n_chunks = n_row.
//   GATHER (with DENSE): y = A x instead.  The shared-memory slice holds x[block] (not sums), every row is walked, a
//   lane forms the dot product of its group with the slice, the team's lanes add up and one of them adds the sum to
//   y[row] in global memory (y already zero; a row receives one addition per block and copy round).
template<int NBUF, bool FIXED, int LOG_L, bool DENSE = false, bool GATHER = false>
__device__ __forceinline__ void
cb_scatter_body(const unsigned char *__restrict__ groups, const uint32_t *__restrict__ offsets, const uint32_t n_col,
                const uint32_t width, const uint32_t n_blocks, const uint32_t b, const uint32_t p, const uint32_t P,
                const uint32_t chunk, const uint32_t n_chunks, const uint32_t *__restrict__ counts,
                const uint32_t *__restrict__ ids, float *__restrict__ y, const uint32_t acc_bytes,
                unsigned char *smem, uint32_t *prefix, uint32_t *warp_total, const float inv_scale,
                unsigned long long *trace = nullptr, const uint32_t trace_cta = 0, const float *__restrict__ x = nullptr) {
    static_assert(!(DENSE && FIXED), "the dense product accumulates in float");
    static_assert(DENSE || !GATHER, "the gather direction is a dense-vector product");
    static_assert(NBUF <= 3, "the per-round scale registers cover three rounds in flight");
    constexpr uint32_t L = 1u << LOG_L, TEAMS = 32u / L;          // lanes (= slots) per team, teams per warp
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t team = lane >> LOG_L, sub = lane & (L - 1u);
    float *acc = reinterpret_cast<float *>(smem);
    unsigned char *ring = smem + acc_bytes + warp * (NBUF * CB_BUF_BYTES);
    const uint32_t col0 = b * width;
    const uint32_t my_width = min(width, n_col - col0);
    if (threadIdx.x == 0) {
        cb_stamp(trace, trace_cta, 0);
        if (trace != nullptr) {
            trace[static_cast<uint64_t>(trace_cta) * 8u + 3] = ~0ull;
            trace[static_cast<uint64_t>(trace_cta) * 8u + 4] = 0ull;
        }
    }
    if (GATHER) {
        for (uint32_t j = threadIdx.x; j < my_width; j += CB_THREADS) acc[j] = x[col0 + j];
    } else {
        for (uint32_t j = threadIdx.x; j < my_width; j += CB_THREADS) acc[j] = 0.0f;
    }

    uint32_t n_act;
    if (DENSE) {
        n_act = n_chunks;
        __syncthreads();                                                             // the slice is zero
    } else {
        pdl_wait();                                                                  // the spike list (and the zeroed y) are ready
        n_act = cb_chunk_prefix(counts, n_chunks, prefix, warp_total);               // ends with a barrier
    }
    if (threadIdx.x == 0) cb_stamp(trace, trace_cta, 1);
    const uint32_t mine = n_act > p ? (n_act - p + P - 1) / P : 0;               // the CTA's rows: p, p + P, ...
    const uint32_t K = mine > warp ? (mine - warp + 31u) / 32u : 0u;             // this warp's: warp, warp + 32, ... of those
    const uint64_t stride = static_cast<uint64_t>(n_blocks) + 1;

    // lane `l` resolves the warp's row k: where its segment for block b starts and how many groups it has
    auto resolve = [&](const uint32_t k, uint32_t &src, uint32_t &rem, float &xs) {
        src = 0;
        rem = 0;
        xs = 0.0f;
        if (k < K) {
            const uint32_t at = p + (warp + 32u * k) * P;
            const uint32_t row = DENSE ? at : list_row(prefix, n_chunks, chunk, ids, at);
            if (GATHER) xs = __uint_as_float(row);               // the row rides in the scale registers
            else if (DENSE) xs = x[row];
            if (!DENSE || GATHER || xs != 0.0f) {                // a row whose vector entry is zero adds nothing
                const uint32_t *o = offsets + row * stride + b;
                src = o[0];
                rem = o[1] - src;
            }
        }
    };

    // one round's buffer: scatter adds the lane's group into the slice; gather forms its dot product with the slice,
    // sums over the team (whose slots hold consecutive groups of ONE row's segment) and adds to y[row]
    auto consume = [&](const unsigned char *buf, const bool filled, const float tag) {
        if (GATHER) {
            float part = 0.0f;
            if (filled) {
                CbGroup grp;
                grp.wa = *reinterpret_cast<const uint4 *>(buf + lane * CB_GROUP_BYTES);
                grp.wb = *reinterpret_cast<const uint4 *>(buf + lane * CB_GROUP_BYTES + 16);
                grp.cc = *reinterpret_cast<const uint4 *>(buf + lane * CB_GROUP_BYTES + 32);
                part = cb_dot_group(acc, grp);
            }
#pragma unroll
            for (uint32_t o = L >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(FULL_MASK, part, o);
            if (sub == 0 && filled) atomicAdd(y + __float_as_uint(tag), part);
        } else {
            cb_accumulate<FIXED, DENSE>(acc, buf, filled, lane, tag);
        }
    };

    uint32_t next_src, next_rem;
    float next_xs;
    resolve(lane, next_src, next_rem, next_xs);
    if (trace != nullptr && threadIdx.x == 0 && next_rem != 0xffffffffu) cb_stamp(trace, trace_cta, 2);
    uint32_t issued = 0, consumed = 0;     // rounds committed / accumulated; buffer of round r is r % NBUF
    uint32_t pieces = 0;                   // groups this lane's team copied in the rounds in flight, 8 bits each, oldest lowest
    float sc0 = 1.0f, sc1 = 1.0f, sc2 = 1.0f;   // DENSE: the vector entries of the rows of those rounds, oldest first

    for (uint32_t k0 = 0; k0 < K; k0 += 32u) {
        uint32_t src = next_src, rem = next_rem;
        const float xs = next_xs;
        resolve(k0 + 32u + lane, next_src, next_rem, next_xs);      // in flight while this batch streams
        uint32_t mask = __ballot_sync(FULL_MASK, rem > 0);
        while (mask) {
            // one round: team t copies up to L groups of the segment held by lane first + t into its own slots
            const uint32_t first = __ffs(mask) - 1u;
            const uint32_t owner = first + team;
            const uint32_t o_src = __shfl_sync(FULL_MASK, src, owner & 31u);
            uint32_t o_rem = __shfl_sync(FULL_MASK, rem, owner & 31u);
            if (owner > 31u) o_rem = 0;
            const uint32_t piece = min(o_rem, L);
            unsigned char *dst = ring + (issued % NBUF) * CB_BUF_BYTES + team * (L * CB_GROUP_BYTES);
            const unsigned char *from = groups + static_cast<uint64_t>(o_src) * CB_GROUP_BYTES;
#pragma unroll
            for (uint32_t it = 0; it < 3u; ++it) {         // a group is three 16-byte chunks: 3 * piece <= 3 L chunks
                const uint32_t c = sub + it * L;
                if (c < 3u * piece) cp_async16(dst + c * 16u, from + c * 16u);
            }
            cp_async_commit();
            // the lanes that hold the segments just copied move on
            const uint32_t my_rank = lane - first;
            const uint32_t taken = __shfl_sync(FULL_MASK, piece, (my_rank & (TEAMS - 1u)) << LOG_L);
            if (lane >= first && my_rank < TEAMS) {
                src += taken;
                rem -= taken;
            }
            pieces |= piece << (8u * (issued - consumed));
            if (DENSE) {
                const float o_xs = __shfl_sync(FULL_MASK, xs, owner & 31u);
                const uint32_t d = issued - consumed;
                if (d == 0u) sc0 = o_xs; else if (d == 1u) sc1 = o_xs; else sc2 = o_xs;
            }
            ++issued;
            if (issued - consumed == NBUF) {                // ring full: accumulate the oldest round
                cp_async_wait<NBUF - 1>();
                __syncwarp();
                consume(ring + (consumed % NBUF) * CB_BUF_BYTES, sub < (pieces & 0xffu), sc0);
                __syncwarp();
                pieces >>= 8;
                sc0 = sc1;
                sc1 = sc2;
                ++consumed;
            }
            mask = __ballot_sync(FULL_MASK, rem > 0);
        }
    }
    cp_async_wait<0>();
    __syncwarp();
    while (consumed < issued) {
        consume(ring + (consumed % NBUF) * CB_BUF_BYTES, sub < (pieces & 0xffu), sc0);
        pieces >>= 8;
        sc0 = sc1;
        sc1 = sc2;
        ++consumed;
    }
    if (trace != nullptr && lane == 0) {
        const unsigned long long t = cb_now();
        atomicMin(trace + static_cast<uint64_t>(trace_cta) * 8u + 3, t);
        atomicMax(trace + static_cast<uint64_t>(trace_cta) * 8u + 4, t);
    }
    __syncthreads();
    if (threadIdx.x == 0) cb_stamp(trace, trace_cta, 5);
    // flush the slice: coalesced vector reductions, P CTAs add into the same zero-filled y
    if (mine > 0 && !GATHER) {
        float *out = y + col0;
        auto value = [&](const uint32_t j) -> float {
            return FIXED ? static_cast<float>(reinterpret_cast<const int *>(acc)[j]) * inv_scale : acc[j];
        };
        if ((reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
            const uint32_t n4 = my_width >> 2;
            for (uint32_t j = threadIdx.x; j < n4; j += CB_THREADS) {
                const float a0 = value(4u * j), a1 = value(4u * j + 1u), a2 = value(4u * j + 2u), a3 = value(4u * j + 3u);
                if (a0 != 0.0f || a1 != 0.0f || a2 != 0.0f || a3 != 0.0f) red_add_v4(out + 4u * j, a0, a1, a2, a3);
            }
            for (uint32_t j = 4u * n4 + threadIdx.x; j < my_width; j += CB_THREADS)
                if (value(j) != 0.0f) red_add(out + j, value(j));
        } else {
            for (uint32_t j = threadIdx.x; j < my_width; j += CB_THREADS)
                if (value(j) != 0.0f) red_add(out + j, value(j));
        }
    }
    if (threadIdx.x == 0) cb_stamp(trace, trace_cta, 6);
}

}  // namespace
}  // namespace bpl

#endif  // BPL_CSRC_CB_SCATTER_CUH_
