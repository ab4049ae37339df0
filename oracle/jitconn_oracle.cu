/*
 * CPU restatement of the reference's just-in-time-connectivity algorithms
 * (the live "v2" geometric-skip scheme).  TEST INFRASTRUCTURE ONLY: this file
 * is a checker, nothing that ships may call it.
 *
 * The generator itself lives in a third-party dependency of the reference:
 * cuRAND's device API (`curandState` = XORWOW, `curand_init`, `curand_uniform`,
 * `curand_normal`, header curand_kernel.h of the CUDA toolkit; the reference
 * pins no version, this build uses CUDA 12.9 / cuRAND 10.3.10).  It is CALLED
 * here, not restated: the header is compiled for the host by overriding its
 * QUALIFIERS macro, so the XORWOW bit stream is the toolkit's own.
 *
 * What differs between host and device and therefore limits this oracle:
 *   - `logf`: glibc on the host, CUDA libdevice on the GPU (<= 1 ulp apart).  A
 *     gap `ceil(logf(u) / log_p)` can differ by one when the quotient lies
 *     within an ulp of an integer.  Such draws are counted as "fragile" so a
 *     test can tell a real mismatch from this rounding effect.
 *   - `curand_normal`: the device path uses the fast `__sincosf`, the host path
 *     `sinf`/`cosf`; normal weights agree to about 1e-6, not bitwise.
 * The reference's own tests pin no absolute value of this path (they are
 * relational only).  This oracle is pinned instead against outputs of the
 * reference's own CUDA kernels: tests/golden/jitconn_reference_gpu.npz holds 93
 * of them (event / dense / matmat, homo / uniform / normal, both parallel modes),
 * produced on a B200 by tests/golden/make_golden_jitconn.py, and
 * tests/test_jitconn_golden.py requires this file to reproduce every one (no
 * output outside the tolerance over 1.1e6 sampled connections).  The bitwise
 * check of the CUDA kernels is made on the GPU against the same kernels compiled
 * into oracle/_ref/ and against the same golden file.
 *
 * Citations are paths inside the brainpylib source tree.
 */
#define QUALIFIERS static inline __host__ __device__
#include <curand_kernel.h>
#include <cmath>
#include <cstdint>
#include <cstring>

namespace {

enum { W_HOMO = 0, W_UNIFORM = 1, W_NORMAL = 2 };

/* One gap of the geometric skip: lib/gpu_jitconn_matvec.cu:103,106 —
 * `(int) ceil(log(curand_uniform(&state)) / conn_prob)`: float log, float/double
 * division in double, ceil, conversion to int. */
struct GapSource {
    curandState st;
    double log_p;
    uint64_t fragile;

    GapSource(uint32_t stream_seed, double lp) : log_p(lp), fragile(0) {
        curand_init((unsigned long long) stream_seed, 0, 0, &st);   /* :99 */
    }

    int next_gap() {
        const float u = curand_uniform(&st);
        const float lg = logf(u);
        const double q = (double) lg / log_p;
        const double c = ceil(q);
        /* would one ulp of logf move the quotient across an integer? */
        const double q_lo = (double) nextafterf(lg, -INFINITY) / log_p;
        const double q_hi = (double) nextafterf(lg, INFINITY) / log_p;
        if (ceil(q_lo) != c || ceil(q_hi) != c) ++fragile;
        /* cvt.rzi.s32.f64 saturates on the device; mirror that for huge gaps */
        if (c >= 2147483647.0) return 2147483647;
        return (int) c;
    }

    /* weight of one synapse, drawn after its position and before the next gap
     * (lib/gpu_jitconn_matvec.cu:243 uniform, :386 normal).  The device
     * contracts `a * b + c` in double into one fused multiply-add. */
    template<typename T>
    T next_weight(int kind, double w1, double w2) {
        if (kind == W_UNIFORM) return (T) fma((double) curand_uniform(&st), w2, w1);   /* u * w_range + w_min */
        if (kind == W_NORMAL) return (T) fma((double) curand_normal(&st), w2, w1);     /* n * w_sigma + w_mu */
        return (T) 1;
    }
};

template<typename T>
inline T mul_add(T a, T b, T c);
template<> inline float mul_add<float>(float a, float b, float c) { return fmaf(a, b, c); }
template<> inline double mul_add<double>(double a, double b, double c) { return fma(a, b, c); }

inline bool truthy(const void *ev, int ev_kind, uint32_t i) {
    if (ev_kind == 0) return ((const uint8_t *) ev)[i] != 0;
    if (ev_kind == 1) return ((const float *) ev)[i] != 0.0f;
    return ((const double *) ev)[i] != 0.0;
}

template<typename T>
inline T event_value(const void *ev, int ev_kind, uint32_t i) {
    if (ev_kind == 0) return (T) (((const uint8_t *) ev)[i] != 0);
    if (ev_kind == 1) return (T) ((const float *) ev)[i];
    return (T) ((const double *) ev)[i];
}

/* `while (syn_arrival_id < num_col)` compares an int with an unsigned int:
 * the int is converted to unsigned (lib/gpu_jitconn_matvec.cu:104). */
inline bool in_range(int pos, uint32_t extent) { return (uint32_t) pos < extent; }

/* `syn_arrival_id += gap` on the device wraps in 32 bits; avoid host UB. */
inline int advance(int pos, int gap) { return (int) ((uint32_t) pos + (uint32_t) gap); }

/* Row-parallel product  y[row] = sum_pos v[pos] * w  (outdim_parallel=True):
 * lib/gpu_jitconn_matvec.cu:84-112 (homo), :220-251 (uniform), :363-394 (normal). */
template<typename T>
uint64_t matvec_rows(const T *v, uint32_t seed, double log_p, double w1, double w2,
                     uint32_t n_row, uint32_t n_col, int kind, T *y, uint64_t *n_conn) {
    uint64_t fragile = 0, conn = 0;
    for (uint32_t row = 0; row < n_row; ++row) {
        GapSource g(seed + row, log_p);
        T sum = 0;
        int pos = g.next_gap();
        while (in_range(pos, n_col)) {
            if (kind == W_HOMO) sum += v[pos];
            else sum = mul_add<T>(v[pos], g.next_weight<T>(kind, w1, w2), sum);
            ++conn;
            pos = advance(pos, g.next_gap());
        }
        y[row] = sum;
        fragile += g.fragile;
    }
    if (n_conn) *n_conn = conn;
    return fragile;
}

/* Column-parallel product with scatter (outdim_parallel=False):
 * lib/gpu_jitconn_matvec_atomic.cu:27-52, :82-110, :143-171.  The device adds
 * with atomics in arbitrary order; here columns ascend. */
template<typename T>
uint64_t matvec_cols(const T *v, uint32_t seed, double log_p, double w1, double w2,
                     uint32_t n_row, uint32_t n_col, int kind, T *y, uint64_t *n_conn) {
    uint64_t fragile = 0, conn = 0;
    memset(y, 0, sizeof(T) * (size_t) n_row);
    for (uint32_t col = 0; col < n_col; ++col) {
        GapSource g(seed + col, log_p);
        const T x = v[col];
        int pos = g.next_gap();
        while (in_range(pos, n_row)) {
            if (kind == W_HOMO) y[pos] += x;
            else { volatile T p = g.next_weight<T>(kind, w1, w2) * x; y[pos] += p; }
            ++conn;
            pos = advance(pos, g.next_gap());
        }
        fragile += g.fragile;
    }
    if (n_conn) *n_conn = conn;
    return fragile;
}

/* Row-parallel event product: lib/gpu_jitconn_event_matvec.cu:81-108 (homo adds
 * the event VALUE), :217-248 / :365-396 (weight drawn for every synapse, added
 * only when the event is truthy). */
template<typename T>
uint64_t event_rows(const void *ev, int ev_kind, uint32_t seed, double log_p, double w1, double w2,
                    uint32_t n_row, uint32_t n_col, int kind, T *y, uint64_t *n_conn) {
    uint64_t fragile = 0, conn = 0;
    for (uint32_t row = 0; row < n_row; ++row) {
        GapSource g(seed + row, log_p);
        T sum = 0;
        int pos = g.next_gap();
        while (in_range(pos, n_col)) {
            if (kind == W_HOMO) {
                sum += event_value<T>(ev, ev_kind, (uint32_t) pos);
            } else {
                const T w = g.next_weight<T>(kind, w1, w2);
                if (truthy(ev, ev_kind, (uint32_t) pos)) sum += w;
            }
            ++conn;
            pos = advance(pos, g.next_gap());
        }
        y[row] = sum;
        fragile += g.fragile;
    }
    if (n_conn) *n_conn = conn;
    return fragile;
}

/* Column-parallel event product: lib/gpu_jitconn_event_matvec_atomic.cu:30-58
 * (homo adds 1 when the column's event is truthy), :88-117, :150-178.  A silent
 * column changes nothing, so it is skipped; its stream is private to it. */
template<typename T>
uint64_t event_cols(const void *ev, int ev_kind, uint32_t seed, double log_p, double w1, double w2,
                    uint32_t n_row, uint32_t n_col, int kind, T *y, uint64_t *n_conn) {
    uint64_t fragile = 0, conn = 0;
    memset(y, 0, sizeof(T) * (size_t) n_row);
    for (uint32_t col = 0; col < n_col; ++col) {
        if (!truthy(ev, ev_kind, col)) continue;
        GapSource g(seed + col, log_p);
        int pos = g.next_gap();
        while (in_range(pos, n_row)) {
            y[pos] += g.next_weight<T>(kind, w1, w2);
            ++conn;
            pos = advance(pos, g.next_gap());
        }
        fragile += g.fragile;
    }
    if (n_conn) *n_conn = conn;
    return fragile;
}

/* Y = X @ M with M's column n drawn from stream seed + n:
 * lib/gpu_jitconn_matmat.cu:236-276 (normal), :321-361 (uniform).  Positions are
 * `unsigned int` there.  Per output element the products are accumulated in
 * synapse order with a fused multiply-add (`sum[i] += X[...] * rand`). */
template<typename T>
uint64_t matmat_cols(const T *X, uint32_t m, uint32_t k, uint32_t n, uint32_t seed, double log_p,
                     double w1, double w2, int kind, T *Y, uint64_t *n_conn) {
    uint64_t fragile = 0, conn = 0;
    for (uint32_t col = 0; col < n; ++col) {
        GapSource g(seed + col, log_p);
        for (uint32_t r = 0; r < m; ++r) Y[(size_t) r * n + col] = 0;
        uint32_t pos = (uint32_t) g.next_gap();
        while (pos < k) {
            const T w = g.next_weight<T>(kind, w1, w2);
            for (uint32_t r = 0; r < m; ++r)
                Y[(size_t) r * n + col] = mul_add<T>(X[(size_t) r * k + pos], w, Y[(size_t) r * n + col]);
            ++conn;
            pos += (uint32_t) g.next_gap();
        }
        fragile += g.fragile;
    }
    if (n_conn) *n_conn = conn;
    return fragile;
}

}  // namespace

extern "C" {

#define EXPORT_JITCONN(SUF, T)                                                                             \
uint64_t oracle_jitconn_matvec_##SUF(const T *v, uint32_t seed, double log_p, double w1, double w2,        \
                                     uint32_t n_row, uint32_t n_col, int kind, int outdim_parallel,        \
                                     T *y, uint64_t *n_conn) {                                             \
    return outdim_parallel ? matvec_rows<T>(v, seed, log_p, w1, w2, n_row, n_col, kind, y, n_conn)         \
                           : matvec_cols<T>(v, seed, log_p, w1, w2, n_row, n_col, kind, y, n_conn);        \
}                                                                                                          \
uint64_t oracle_jitconn_event_matvec_##SUF(const void *ev, int ev_kind, uint32_t seed, double log_p,       \
                                           double w1, double w2, uint32_t n_row, uint32_t n_col,           \
                                           int kind, int outdim_parallel, T *y, uint64_t *n_conn) {        \
    return outdim_parallel                                                                                 \
        ? event_rows<T>(ev, ev_kind, seed, log_p, w1, w2, n_row, n_col, kind, y, n_conn)                   \
        : event_cols<T>(ev, ev_kind, seed, log_p, w1, w2, n_row, n_col, kind, y, n_conn);                  \
}                                                                                                          \
uint64_t oracle_jitconn_matmat_##SUF(const T *X, uint32_t m, uint32_t k, uint32_t n, uint32_t seed,        \
                                     double log_p, double w1, double w2, int kind, T *Y,                   \
                                     uint64_t *n_conn) {                                                   \
    return matmat_cols<T>(X, m, k, n, seed, log_p, w1, w2, kind, Y, n_conn);                               \
}

EXPORT_JITCONN(f32, float)
EXPORT_JITCONN(f64, double)

/* The sampled positions (and weights) of ONE stream `stream_seed` = seed + row
 * (or + column) over `extent` positions.  Returns the number of connections;
 * at most `cap` are written.  `*n_fragile` receives the number of gaps whose
 * value depends on the last bit of logf. */
uint64_t oracle_jitconn_stream(uint32_t stream_seed, double log_p, double w1, double w2,
                               uint32_t extent, int kind, int32_t *pos_out, float *w_out,
                               uint64_t cap, uint64_t *n_fragile) {
    GapSource g(stream_seed, log_p);
    uint64_t count = 0;
    int pos = g.next_gap();
    while (in_range(pos, extent)) {
        const float w = g.next_weight<float>(kind, w1, w2);
        if (count < cap) {
            if (pos_out) pos_out[count] = pos;
            if (w_out) w_out[count] = w;
        }
        ++count;
        pos = advance(pos, g.next_gap());
    }
    if (n_fragile) *n_fragile = g.fragile;
    return count;
}

}  // extern "C"
