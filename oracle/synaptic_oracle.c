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
