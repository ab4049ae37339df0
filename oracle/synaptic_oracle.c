/*
 * CPU restatement of the reference's synaptic-propagation algorithms
 * (stored-matrix ops).  TEST INFRASTRUCTURE ONLY: this file is the checker
 * that the CUDA kernels are compared against.  Nothing that ships may call it.
 *
 * Every function is a serial loop in the reference's own summation order, so
 * that a result computed here equals the reference CPU result bit for bit.
 * Pinned against the reference's own compiled CPU code (lib/cpu_*.cc built
 * into oracle/_ref/) and its numba kernels by tests/test_oracle_pin.py and by
 * the fixtures in tests/golden/.
 *
 * Citations are paths inside the brainpylib source tree.
 */
#include <stdint.h>
#include <string.h>

/* Event truthiness: the reference only ever tests `if (events[i])`
 * (lib/gpu_event_csr_matvec.cu:65,88; brainpylib/_src/event_ops/event_csr_matvec.py:320).
 * ev_kind: 0 = bool (1 byte), 1 = float32, 2 = float64. */
static inline int event_is_set(const void *events, int ev_kind, uint32_t i) {
    switch (ev_kind) {
        case 0: return ((const uint8_t *) events)[i] != 0;
        case 1: return ((const float *) events)[i] != 0.0f;   /* NaN != 0 is true, as in C truthiness */
        default: return ((const double *) events)[i] != 0.0;
    }
}

#define DEFINE_STORED_MATRIX_OPS(SUF, T)                                                          \
/* event-driven CSR product.                                                                      \
 * transpose=1 follows lib/cpu_event_sum.cc:6-24 (homo), :49-67 (heter) and                       \
 *   brainpylib/_src/event_ops/event_csr_matvec.py:313-331: y[col[j]] += w_j over active rows,    \
 *   rows ascending, j ascending, accumulation in T.                                              \
 * transpose=0 follows event_csr_matvec.py:334-357: per row a float64 accumulator                 \
 *   (`r = 0.` is a Python float) that is narrowed to T on store. */                              \
void oracle_event_csr_matvec_##SUF(const T *data, int homo, const uint32_t *indices,              \
                                   const uint32_t *indptr, const void *events, int ev_kind,       \
                                   uint32_t n_row, uint32_t n_col, int transpose, T *y) {         \
    if (transpose) {                                                                              \
        memset(y, 0, sizeof(T) * (size_t) n_col);                                                 \
        for (uint32_t r = 0; r < n_row; ++r) {                                                    \
            if (!event_is_set(events, ev_kind, r)) continue;                                      \
            for (uint32_t j = indptr[r]; j < indptr[r + 1]; ++j)                                  \
                y[indices[j]] += homo ? data[0] : data[j];                                        \
        }                                                                                         \
    } else {                                                                                      \
        for (uint32_t r = 0; r < n_row; ++r) {                                                    \
            double acc = 0.0;                                                                     \
            for (uint32_t j = indptr[r]; j < indptr[r + 1]; ++j)                                  \
                if (event_is_set(events, ev_kind, indices[j]))                                    \
                    acc += (double) (homo ? data[0] : data[j]);                                   \
            y[r] = (T) acc;                                                                       \
        }                                                                                         \
    }                                                                                             \
}                                                                                                 \
                                                                                                  \
/* CSR matrix times dense vector.                                                                 \
 * transpose=0 follows brainpylib/_src/sparse_ops/sparse_csr_matvec.py:108-126 (product in T,     \
 *   float64 row accumulator).                                                                    \
 * transpose=1 follows brainpylib/_src/sparse_ops/cusparse_matvec.py:195-212 (serial scatter,     \
 *   product and accumulation in T). */                                                           \
void oracle_csr_matvec_##SUF(const T *data, int homo, const uint32_t *indices,                    \
                             const uint32_t *indptr, const T *x,                                  \
                             uint32_t n_row, uint32_t n_col, int transpose, T *y) {               \
    if (transpose) {                                                                              \
        memset(y, 0, sizeof(T) * (size_t) n_col);                                                 \
        for (uint32_t r = 0; r < n_row; ++r) {                                                    \
            const T v = x[r];                                                                     \
            for (uint32_t j = indptr[r]; j < indptr[r + 1]; ++j) {                                \
                volatile T prod = homo ? data[0] * v : v * data[j];                               \
                y[indices[j]] += prod;                                                            \
            }                                                                                     \
        }                                                                                         \
    } else {                                                                                      \
        for (uint32_t r = 0; r < n_row; ++r) {                                                    \
            double acc = 0.0;                                                                     \
            for (uint32_t j = indptr[r]; j < indptr[r + 1]; ++j) {                                \
                volatile T prod = x[indices[j]] * (homo ? data[0] : data[j]);                     \
                acc += (double) prod;                                                             \
            }                                                                                     \
            y[r] = (T) acc;                                                                       \
        }                                                                                         \
    }                                                                                             \
}                                                                                                 \
                                                                                                  \
/* COO scatter-add: lib/cpu_atomic_sum.cc:6-41.  homo: y[post[i]] += value;                       \
 * heter: y[post[i]] += values[pre[i]]. */                                                        \
void oracle_coo_atomic_sum_##SUF(const T *values, int homo, const uint32_t *pre_ids,              \
                                 const uint32_t *post_ids, uint32_t conn_size,                    \
                                 uint32_t out_size, T *y) {                                       \
    memset(y, 0, sizeof(T) * (size_t) out_size);                                                  \
    for (uint32_t i = 0; i < conn_size; ++i)                                                      \
        y[post_ids[i]] += homo ? values[0] : values[pre_ids[i]];                                  \
}                                                                                                 \
                                                                                                  \
/* COO scatter-multiply from 1.0: lib/cpu_atomic_prod.cc:6-43 (the CPU semantics;                 \
 * the reference GPU kernel adds instead of multiplying and is not followed). */                  \
void oracle_coo_atomic_prod_##SUF(const T *values, int homo, const uint32_t *pre_ids,             \
                                  const uint32_t *post_ids, uint32_t conn_size,                   \
                                  uint32_t out_size, T *y) {                                      \
    for (uint32_t i = 0; i < out_size; ++i) y[i] = (T) 1;                                         \
    for (uint32_t i = 0; i < conn_size; ++i)                                                      \
        y[post_ids[i]] *= homo ? values[0] : values[pre_ids[i]];                                  \
}                                                                                                 \
                                                                                                  \
/* COO event scatter: lib/gpu_event_sum.cu:122-137 (homo), :165-180 (heter):                      \
 * if events[pre[i]]: y[post[i]] += value (homo) or values[i] (heter). */                         \
void oracle_coo_event_sum_##SUF(const uint8_t *events, const uint32_t *pre_ids,                   \
                                const uint32_t *post_ids, const T *values, int homo,              \
                                uint32_t conn_size, uint32_t out_size, T *y) {                    \
    memset(y, 0, sizeof(T) * (size_t) out_size);                                                  \
    for (uint32_t i = 0; i < conn_size; ++i)                                                      \
        if (events[pre_ids[i]]) y[post_ids[i]] += homo ? values[0] : values[i];                   \
}

DEFINE_STORED_MATRIX_OPS(f32, float)
DEFINE_STORED_MATRIX_OPS(f64, double)

/* Sum of the rows' lengths over active rows: the number of synaptic operations
 * one transposed event-CSR call performs (used to report throughput). */
uint64_t oracle_count_active_synapses(const uint32_t *indptr, const void *events, int ev_kind,
                                      uint32_t n_row) {
    uint64_t s = 0;
    for (uint32_t r = 0; r < n_row; ++r)
        if (event_is_set(events, ev_kind, r)) s += indptr[r + 1] - indptr[r];
    return s;
}

/* ------------------------------------------------------------------------------------------
 * Counter-based ("v1") just-in-time-connectivity event product, restated from the kernel text
 * lib/gpu_jitconn_event_matvec.cu:10-51 (homo), :138-183 (uniform), :281-331 (normal) with the
 * generators of lib/kernel_helpers_random.cuh:12-71 (one step of L'Ecuyer's lfsr113 / taus88 from
 * the states seed + 1, + 7, + 15 [, + 127]):
 *   y[r] = sum over listed events c of [lfsr113(seed + n_col * r + c) < prob] * w
 * The reference's wrappers cannot run (they dereference the device count on the host), so this
 * restatement of the kernel arithmetic is the only pin these targets have.  The products that the
 * device compiler fuses are written as fma() here.
 * ------------------------------------------------------------------------------------------ */
#include <math.h>

static double v1_lfsr113(uint32_t seed) {
    uint32_t z1 = seed + 1u, z2 = seed + 7u, z3 = seed + 15u, z4 = seed + 127u, b;
    b = ((z1 << 6) ^ z1) >> 13;   z1 = ((z1 & 4294967294u) << 18) ^ b;
    b = ((z2 << 2) ^ z2) >> 27;   z2 = ((z2 & 4294967288u) << 2) ^ b;
    b = ((z3 << 13) ^ z3) >> 21;  z3 = ((z3 & 4294967280u) << 7) ^ b;
    b = ((z4 << 3) ^ z4) >> 12;   z4 = ((z4 & 4294967168u) << 13) ^ b;
    return (z1 ^ z2 ^ z3 ^ z4) * 2.3283064365386963e-10;
}

static double v1_taus88_step(uint32_t *s1, uint32_t *s2, uint32_t *s3) {
    uint32_t b;
    b = (((*s1 << 13) ^ *s1) >> 19);  *s1 = (((*s1 & 4294967294u) << 12) ^ b);
    b = (((*s2 << 2) ^ *s2) >> 25);   *s2 = (((*s2 & 4294967288u) << 4) ^ b);
    b = (((*s3 << 3) ^ *s3) >> 11);   *s3 = (((*s3 & 4294967280u) << 17) ^ b);
    return ((*s1 ^ *s2 ^ *s3) * 2.3283064365386963e-10);
}

/* kind: 0 homo, 1 uniform (w1 = w_min, w2 = w_range), 2 normal (w1 = mu, w2 = sigma); out_f64: 0 float, 1 double */
void oracle_jitconn_event_v1(const int32_t *event_ids, int32_t event_num, uint32_t conn_seed, double prob,
                             int kind, double w1, double w2, uint32_t n_row, uint32_t n_col, int out_f64,
                             void *out) {
    for (uint32_t r = 0; r < n_row; ++r) {
        const uint32_t seed_base = conn_seed + n_col * r;
        float sum_f = 0.0f;
        double sum_d = 0.0;
        for (int32_t i = 0; i < event_num; ++i) {
            const uint32_t seed = seed_base + (uint32_t) event_ids[i];
            if (!(v1_lfsr113(seed) < prob)) continue;
            double w = 1.0;
            if (kind != 0) {
                uint32_t s1 = seed + 1u, s2 = seed + 7u, s3 = seed + 15u;
                const double u = v1_taus88_step(&s1, &s2, &s3);
                if (kind == 1) {
                    w = fma(u, w2, w1);
                } else {
                    const double v = v1_taus88_step(&s1, &s2, &s3);
                    w = fma(sqrt(-2 * log(u)) * cos(2 * 3.14159265358979323846 * v), w2, w1);
                }
            }
            if (out_f64) sum_d += w; else sum_f = (float) ((double) sum_f + w);
        }
        if (out_f64) ((double *) out)[r] = sum_d; else ((float *) out)[r] = sum_f;
    }
}
