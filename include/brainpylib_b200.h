/*
 * brainpylib_b200 — C ABI of the B200 synaptic-propagation library.
 *
 * Every operator is an XLA GPU custom-call target with the legacy (API version 0)
 * signature the reference library uses (lib/gpu_event_csr_matvec.cuh:14-15):
 *
 *     void target(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len);
 *
 * `buffers` holds device pointers: the operands in call order, then the outputs,
 * then (only where stated) ONE trailing workspace buffer that the caller owns.
 * `opaque` is a packed descriptor, byte-identical to the reference's
 * (lib/kernel_helper_descriptor.cuh:49-144).  A target only enqueues work on
 * `stream`; it never synchronises, allocates, frees or keeps a pointer.  Outputs
 * may arrive uninitialised.  Errors never cross the boundary as C++ exceptions
 * (the reference throws, lib/kernel_helpers.h:36-38): they are recorded per
 * host thread and read with bpl_last_status().
 *
 * The C symbol of a target is the registration name the reference uses in
 * lib/gpu_ops.cc:28-174, so a registry built from bpl_registration_*() is a
 * drop-in for `gpu_ops.registrations()`.
 */
#ifndef BRAINPYLIB_B200_H_
#define BRAINPYLIB_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st *bpl_stream_t; /* == cudaStream_t */
typedef void (*bpl_custom_call_t)(bpl_stream_t stream, void **buffers, const char *opaque, size_t opaque_len);

/* ---- status (replaces the reference's C++ exceptions: lib/kernel_helpers.h:34-40,
 *      lib/kernel_helpers_gpu.cuh:15-19) ------------------------------------------------- */
enum {
    BPL_OK = 0,
    BPL_ERR_OPAQUE_SIZE = 1,  /* "Invalid opaque object size" */
    BPL_ERR_CUDA = 2,         /* launch / runtime error, message = cudaGetErrorString */
    BPL_ERR_ARGUMENT = 3,     /* a size the kernels cannot take */
    BPL_ERR_TOO_LARGE = 4     /* beyond the fixed capacity of a no-allocation entry point */
};
/* Status of the last target called on THIS host thread; copies the message (may be NULL). */
int bpl_last_status(char *message, size_t capacity);
void bpl_clear_status(void);

/* ---- registry (replaces Registrations() of lib/gpu_ops.cc:24-177) ------------------------- */
int bpl_registration_count(void);
const char *bpl_registration_name(int i);
bpl_custom_call_t bpl_registration_target(int i);
bpl_custom_call_t bpl_find_target(const char *name); /* NULL when unknown */

/* ---- descriptor builders (replace build_*_descriptor of lib/kernel_helper_descriptor.cu:13-102,
 *      lib/gpu_event_sum.cu, lib/gpu_atomic_sum.cu, lib/gpu_atomic_prod.cu).  Each writes the packed
 *      struct to `out` (capacity `cap` bytes) and returns its size, or 0 when `cap` is too small.
 *      As in the reference, real-valued fields arrive as `float` and are stored as `double`. ---- */
size_t bpl_build_twouint_onebool_descriptor(uint32_t uint_x, uint32_t uint_y, int bool_x, void *out, size_t cap);
size_t bpl_build_double_size_descriptor(uint32_t size_x, uint32_t size_y, void *out, size_t cap);
size_t bpl_build_triple_size_descriptor(uint32_t size_x, uint32_t size_y, uint32_t size_z, void *out, size_t cap);
size_t bpl_build_jitconn_prob_homo_descriptor(uint32_t n_row, uint32_t n_col, uint32_t seed, float prob,
                                              void *out, size_t cap);
size_t bpl_build_jitconn_prob_uniform_descriptor(uint32_t n_row, uint32_t n_col, uint32_t seed, float prob,
                                                 float w_min, float w_range, void *out, size_t cap);
size_t bpl_build_jitconn_prob_normal_descriptor(uint32_t n_row, uint32_t n_col, uint32_t seed, float prob,
                                                float w_mu, float w_sigma, void *out, size_t cap);
size_t bpl_build_matmat_jit_prob_descriptor1(uint32_t m, uint32_t k, uint32_t n, uint32_t seed, float log_p,
                                             float w1, float w2, void *out, size_t cap);
size_t bpl_build_csr_event_sum_descriptor(uint32_t pre_size, uint32_t post_size, void *out, size_t cap);
size_t bpl_build_coo_event_sum_descriptor(uint32_t conn_size, uint32_t post_size, void *out, size_t cap);
size_t bpl_build_coo_atomic_sum_descriptor(uint32_t conn_size, uint32_t post_size, void *out, size_t cap);
size_t bpl_build_coo_atomic_prod_descriptor(uint32_t conn_size, uint32_t post_size, void *out, size_t cap);
size_t bpl_build_nonzero_descriptor(uint32_t event_size, uint32_t batch_size, void *out, size_t cap);
size_t bpl_build_lif_exp_descriptor(uint32_t n, uint32_t n_channels, float t, const float *syn_decay, const float *E_rev,
                                    float ext_input, float V_rest, float V_th, float V_reset, float R, float lif_decay,
                                    float tau_ref, void *out, size_t cap);
size_t bpl_build_cbcsr_descriptor(uint32_t n_row, uint32_t n_col, uint32_t block_width, int fixed_point,
                                  int scale_log2, uint32_t team_lanes_log2, void *out, size_t cap);

/* ---- workspace -------------------------------------------------------------------------
 * Bytes of the trailing workspace buffer a target needs for the given opaque descriptor
 * (0 = the target takes no workspace buffer).  The workspace is scratch: its contents
 * need not be initialised and are undefined afterwards.  Under XLA it is declared as one
 * more (discarded) uint8 output, the way the reference's `event_info` returns a second
 * array (brainpylib/_src/event_ops/event_info_collection.py:115-122). */
size_t bpl_workspace_bytes(const char *target_name, const char *opaque, size_t opaque_len);
/* Tests only: non-zero values replace the per-column list capacity and the byte budget of one chunk of columns of
 * the *_v1_ws matmat targets (0 restores the computed ones), so that a small matrix overflows its lists (the
 * recomputation pass runs) or is walked in several chunks. */
void bpl_matmat_list_limits_for_tests(uint32_t cap, size_t budget_bytes);

/* ---- profiling hook (no counterpart in the reference) -------------------------------------
 * When both are non-NULL cudaEvent_t handles, every later event_csr_matvec_* call with
 * transpose=true and every event_cbcsr_matvec_* call made by THIS host thread records `before` /
 * `after` on its stream directly around its scatter kernel, so that kernel can be timed on its
 * own.  NULL switches it off. */
void bpl_profile_scatter_events(void *before, void *after);

/* ---- targets ----------------------------------------------------------------------------
 * E = events element: bool (1 byte) or the float type of the op; T = float | double.
 *
 * event_csr_matvec_{homo,heter}_{float_bool,float_float,double_bool,double_double}
 *   replaces lib/gpu_event_csr_matvec.cu:148-217 (registered lib/gpu_ops.cc:95-104)
 *   opaque  TwoUintOneBoolDescriptor{n_row, n_col, transpose}
 *   buffers [data T(1|nse), indices u32(nse), indptr u32(n_row+1), events E, y T, workspace]
 *   workspace: bpl_workspace_bytes() bytes when transpose, none otherwise (slot ignored).
 *
 * event_cbcsr_matvec_heter_float_{bool,float}   (no counterpart in the reference)
 *   y = A^T events on a COLUMN-BLOCKED matrix built once by bpl_cbcsr_plan / bpl_cbcsr_fill (below): the
 *   post-synaptic neurons are cut into blocks of `block_width` columns (a multiple of 32, <= 32256); the
 *   matrix stays row-major, the synapses of a row are grouped by block and stored in records of 8
 *   (8 x float32 weight - or int32 round(w * 2^k) for fixed-point matrices - then 8 x uint16 column offset
 *   into the block; a segment is padded with zero-weight synapses to whole records); offsets[row][b] ..
 *   offsets[row][b + 1] are the records of row's segment for block b.  One block's slice of y is accumulated
 *   in shared memory, which lifts the scattered-reduction limit of the plain CSR scatter.
 *   opaque  {u32 n_row, u32 n_col, u32 block_width, i32 fixed_point, i32 scale_log2, u32 team_lanes_log2}
 *           (bpl_build_cbcsr_descriptor; team_lanes_log2 2..5: lanes and groups per round a segment gets)
 *   buffers [groups u8(48 * n_groups), offsets u32(n_row, n_blocks + 1), events E(n_row), y f32(n_col), workspace]
 *   workspace: bpl_workspace_bytes() (as for event_csr_matvec with transpose)
 *
 * cbcsr_matvec_transpose_heter_float   (no counterpart in the reference, which takes this product from cuSPARSE)
 *   y = A^T x for a dense float32 vector x on the same storage: every row with x[row] != 0 is walked and its weights
 *   are multiplied by x[row]; float accumulation (fixed_point must be 0).
 *   buffers [groups, offsets, x f32(n_row), y f32(n_col)]; opaque as above
 * cbcsr_matvec_heter_float             (no counterpart in the reference)
 *   y = A x on the same storage: a block's slice of x is staged in shared memory and a row's segment is summed against
 *   it, so the gathers of x never leave the SM; a row receives one global addition per column block and copy round.
 *   buffers [groups, offsets, x f32(n_col), y f32(n_row)]; opaque as above
 *
 * event_cbcsr_matvec_list_heter_float / event_csr_matvec_list_heter_float   (no counterpart in the reference)
 *   the scatter half alone, driven by a ready-made spike list (counts[1024], then row ids in chunk segments: the
 *   layout of the event_csr_matvec workspace, written e.g. by lif_exp_step_float); y must already be zero.
 *   buffers [groups, offsets, list u32, y f32(n_col)] (opaque as event_cbcsr_matvec) resp.
 *           [data f32, indices u32, indptr u32(n_row + 1), list u32, y f32(n_col)] (opaque {n_row, n_col, n_chunks})
 *
 * lif_exp_step_float   (no counterpart in the reference: the caller's side of the step, fused)
 *   The step pattern of the reference's network example (brainpylib/_src/op_register/tests/ei_net.py:47-72) in one
 *   launch: per synaptic channel g = g * decay + y (y is then zero-filled for the next step), input += g * (E - V);
 *   leaky integrate-and-fire update with refractory period, threshold and reset; and the new spikes are compacted
 *   into the spike list the *_list_* products read, so no event vector has to be scanned and y needs no zero-fill.
 *   Products and sums are rounded one by one (no fused multiply-add) so that a float32 array implementation agrees
 *   bit for bit.
 *   opaque  bpl_build_lif_exp_descriptor()
 *   buffers [y f32(K, n) in/zeroed, g f32(K, n) in/out, V f32(n) in/out, t_last f32(n) in/out, spikes f32(n) out,
 *            list u32 out (bpl_workspace_bytes of event_csr_matvec_* with transpose for n rows)]
 *
 * csr_matvec_{homo,heter}_{scalar,vector,adaptive}_{float,double}
 *   replaces lib/gpu_csr_matvec.cu:84-141,195-246,505-560 (lib/gpu_ops.cc:79-92); the three
 *   method names run the same kernel; 'adaptive' ignores its extra row_blocks operand.
 *   opaque  DoubleSizeDescriptor{n_row, n_col}
 *   buffers [data, indices, indptr, vector T(n_col), y T(n_row)]   (adaptive: row_blocks at 3)
 * csr_matvec_transpose_{homo,heter}_{float,double}
 *   y = A^T x; replaces the jaxlib cuSPARSE lowering the reference's AD rules call
 *   (brainpylib/_src/sparse_ops/cusparse_matvec.py:266-278; math :195-212).
 *   opaque  DoubleSizeDescriptor{n_row, n_col}; buffers [data, indices, indptr, vector T(n_row), y T(n_col)]
 *
 * gpu_matvec_prob_{homo,uniform,normal}_v1_{float,double}
 *   replaces lib/gpu_jitconn_matvec.cu:57-81,190-217,334-360 (lib/gpu_ops.cc:143-148): Bernoulli test per
 *   (row, column); the descriptor's `prob` field holds the raw connection probability, not its log.
 *   opaque and buffers as for v2.
 * gpu_matvec{,_atomic}_prob_{homo,uniform,normal}_v2_{float,double}
 *   replaces lib/gpu_jitconn_matvec.cu:115-139,254-281,397-424 and
 *   lib/gpu_jitconn_matvec_atomic.cu:55-78,113-139,174-200 (lib/gpu_ops.cc:151-164)
 *   opaque  JITConnProb{Homo,Uniform,Normal}Descriptor; buffers [vector T(n_col), y T(n_row)]
 * gpu_event_matvec{,_atomic}_prob_{homo,uniform,normal}_v2_{float_bool,float_float,double_bool,double_double}
 *   replaces lib/gpu_jitconn_event_matvec.cu:111-135,251-278,399-426 and
 *   lib/gpu_jitconn_event_matvec_atomic.cu:61-85,120-147,181-208 (lib/gpu_ops.cc:115-140)
 *   opaque  as above; buffers [events E(n_col), y T(n_row)]
 * gpu_event_matvec_prob_{homo,uniform,normal}_{float,double}      (the counter-based "v1" scheme)
 *   replaces lib/gpu_jitconn_event_matvec.cu:10-51,138-183,281-331 + lib/kernel_helpers_random.cuh:12-71
 *   (lib/gpu_ops.cc:107-112).  Connection (row r, column c) exists iff lfsr113(seed + n_col * r + c) < prob (RAW
 *   probability in the descriptor); its weight comes from taus88 on the same seed.  Only listed events are visited.
 *   opaque  JITConnProb{Homo,Uniform,Normal}Descriptor; buffers [event_ids i32, event_num i32(1), y T(n_row)].
 *   The count is read on the device (the reference's wrapper dereferences the device pointer on the host).
 * gpu_matmat_prob_prob_{normal,uniform}_{float,double}_v1
 *   replaces lib/gpu_jitconn_matmat.cu:279-317,364-402 (lib/gpu_ops.cc:171-174)
 *   opaque  MatMatJITProbDescriptor1{m,k,n,seed,log_p,w1,w2}; buffers [X T(m,k), Y T(m,n)] row-major
 * gpu_matmat_prob_prob_{normal,uniform}_{float,double}_v1_ws      (no counterpart in the reference)
 *   The same product, bit for bit, with every column's stream generated once instead of once per 32 rows of X:
 *   one pass writes the connections (position, weight) of a chunk of columns into the workspace, a second multiplies
 *   from the lists.  buffers [X T(m,k), Y T(m,n), workspace (bpl_workspace_bytes(), 256-byte aligned)]; same opaque.
 * gpu_matmat_prob_prob_normal_{float,double}_{v2,v3}
 *   replace lib/gpu_jitconn_matmat.cu:138-231 (v2: 32 streams per column, one per range of ceil(k / 32) rows) and
 *   :19-135 (v3: one stream per row of X, pairs shared by a block of rows); registered lib/gpu_ops.cc:166-169.
 *   Each generates its own matrix, different from v1's.  Same opaque and buffers.
 *
 * nonzero_{bool,int,long,float,double}   replaces lib/gpu_event_info.cu:48-118 (lib/gpu_ops.cc:72-76)
 *   opaque NonZeroDescriptor{event_size, batch_size}
 *   buffers [events E(batch, size), event_ids i32(batch, size), event_num i32(batch), workspace]
 *   event_ids: ascending indices of the non-zero entries of each row, padded with -1 (the reference
 *   returns them in an arbitrary, run-dependent order); workspace: bpl_workspace_bytes() = 4096 B per row.
 *
 * gpu_csr_event_sum_{homo,heter}_{f32,f64}_{i32,i64}   replaces lib/gpu_event_sum.cu:50-117
 *   opaque {pre_size, post_size}; buffers [events bool, indices I, indptr I, values T, y T]
 * gpu_coo_event_sum_{homo,heter}_{f32,f64}_{i32,i64}   replaces lib/gpu_event_sum.cu:140-206
 *   opaque {conn_size, post_size}; buffers [events bool, pre_ids I, post_ids I, values T, y T]
 * gpu_coo_atomic_sum_{homo,heter}_{f32,f64}_{i32,i64}  replaces lib/gpu_atomic_sum.cu:39-97
 * gpu_coo_atomic_prod_{homo,heter}_{f32,f64}_{i32,i64} replaces lib/gpu_atomic_prod.cu:39-97
 *   opaque {conn_size, post_size}; buffers homo [values T(1), post_ids I, y T]
 *                                          heter [values T, pre_ids I, post_ids I, y T]
 *   y[post[i]] op= values[pre[i]].  The heter operand order is the one the reference's Python
 *   side passes (brainpylib/_src/compat/atomic_sum.py:128-131) and its CPU kernel reads
 *   (lib/cpu_atomic_sum.cc:8-10); the reference's CUDA wrapper reads the two id arrays the other
 *   way round (lib/gpu_atomic_sum.cu:86-87), which is not followed.  "prod" multiplies from 1.0
 *   as lib/cpu_atomic_prod.cc:6-43 does (the reference's CUDA "prod" adds).
 */
#define BPL_DECLARE_TARGET(name) \
    void name(bpl_stream_t stream, void **buffers, const char *opaque, size_t opaque_len)

#define BPL_FOR_EACH_TE(X, stem) X(stem##_float_bool) X(stem##_float_float) X(stem##_double_bool) X(stem##_double_double)
#define BPL_FOR_EACH_T(X, stem) X(stem##_float) X(stem##_double)
#define BPL_FOR_EACH_FI(X, stem) X(stem##_f32_i32) X(stem##_f32_i64) X(stem##_f64_i32) X(stem##_f64_i64)

#define BPL_FOR_EACH_TARGET(X)                                      \
    BPL_FOR_EACH_TE(X, event_csr_matvec_homo)                       \
    BPL_FOR_EACH_TE(X, event_csr_matvec_heter)                      \
    X(event_csr_matvec_heter_float_float_noalloc)                   \
    X(event_cbcsr_matvec_heter_float_bool) X(event_cbcsr_matvec_heter_float_float) \
    X(event_cbcsr_matvec_list_heter_float) X(event_csr_matvec_list_heter_float) X(lif_exp_step_float) \
    BPL_FOR_EACH_T(X, csr_matvec_homo_scalar)                       \
    BPL_FOR_EACH_T(X, csr_matvec_homo_vector)                       \
    BPL_FOR_EACH_T(X, csr_matvec_homo_adaptive)                     \
    BPL_FOR_EACH_T(X, csr_matvec_heter_scalar)                      \
    BPL_FOR_EACH_T(X, csr_matvec_heter_vector)                      \
    BPL_FOR_EACH_T(X, csr_matvec_heter_adaptive)                    \
    BPL_FOR_EACH_T(X, csr_matvec_transpose_homo)                    \
    BPL_FOR_EACH_T(X, csr_matvec_transpose_heter)                   \
    BPL_FOR_EACH_T(X, gpu_matvec_prob_homo_v1)                      \
    BPL_FOR_EACH_T(X, gpu_matvec_prob_uniform_v1)                   \
    BPL_FOR_EACH_T(X, gpu_matvec_prob_normal_v1)                    \
    BPL_FOR_EACH_T(X, gpu_matvec_prob_homo_v2)                      \
    BPL_FOR_EACH_T(X, gpu_matvec_prob_uniform_v2)                   \
    BPL_FOR_EACH_T(X, gpu_matvec_prob_normal_v2)                    \
    BPL_FOR_EACH_T(X, gpu_matvec_atomic_prob_homo_v2)               \
    BPL_FOR_EACH_T(X, gpu_matvec_atomic_prob_uniform_v2)            \
    BPL_FOR_EACH_T(X, gpu_matvec_atomic_prob_normal_v2)             \
    BPL_FOR_EACH_T(X, gpu_event_matvec_prob_homo)                   \
    BPL_FOR_EACH_T(X, gpu_event_matvec_prob_uniform)                \
    BPL_FOR_EACH_T(X, gpu_event_matvec_prob_normal)                 \
    BPL_FOR_EACH_TE(X, gpu_event_matvec_prob_homo_v2)               \
    BPL_FOR_EACH_TE(X, gpu_event_matvec_prob_uniform_v2)            \
    BPL_FOR_EACH_TE(X, gpu_event_matvec_prob_normal_v2)             \
    BPL_FOR_EACH_TE(X, gpu_event_matvec_atomic_prob_homo_v2)        \
    BPL_FOR_EACH_TE(X, gpu_event_matvec_atomic_prob_uniform_v2)     \
    BPL_FOR_EACH_TE(X, gpu_event_matvec_atomic_prob_normal_v2)      \
    X(gpu_matmat_prob_prob_normal_float_v1)                         \
    X(gpu_matmat_prob_prob_normal_double_v1)                        \
    X(gpu_matmat_prob_prob_normal_float_v2)                         \
    X(gpu_matmat_prob_prob_normal_double_v2)                        \
    X(gpu_matmat_prob_prob_normal_float_v3)                         \
    X(gpu_matmat_prob_prob_normal_double_v3)                        \
    X(gpu_matmat_prob_prob_uniform_float_v1)                        \
    X(gpu_matmat_prob_prob_uniform_double_v1)                       \
    X(cbcsr_matvec_transpose_heter_float) X(cbcsr_matvec_heter_float) \
    X(gpu_matmat_prob_prob_normal_float_v1_ws)                      \
    X(gpu_matmat_prob_prob_normal_double_v1_ws)                     \
    X(gpu_matmat_prob_prob_uniform_float_v1_ws)                     \
    X(gpu_matmat_prob_prob_uniform_double_v1_ws)                    \
    X(nonzero_bool) X(nonzero_int) X(nonzero_long) X(nonzero_float) X(nonzero_double) \
    BPL_FOR_EACH_FI(X, gpu_csr_event_sum_homo)                      \
    BPL_FOR_EACH_FI(X, gpu_csr_event_sum_heter)                     \
    BPL_FOR_EACH_FI(X, gpu_coo_event_sum_homo)                      \
    BPL_FOR_EACH_FI(X, gpu_coo_event_sum_heter)                     \
    BPL_FOR_EACH_FI(X, gpu_coo_atomic_sum_homo)                     \
    BPL_FOR_EACH_FI(X, gpu_coo_atomic_sum_heter)                    \
    BPL_FOR_EACH_FI(X, gpu_coo_atomic_prod_homo)                    \
    BPL_FOR_EACH_FI(X, gpu_coo_atomic_prod_heter)

#define BPL_DECLARE_ONE(name) BPL_DECLARE_TARGET(name);
BPL_FOR_EACH_TARGET(BPL_DECLARE_ONE)
#undef BPL_DECLARE_ONE

/* ---- builder of the column-blocked format (takes the place of the host-side layout code of
 *      brainpylib/_src/sparse_ops/utils.py:21-51 for the one layout this library adds) ---------
 * From a CSR matrix (float32 weights, one shared weight when `homogeneous`; uint32 ids) on the device.
 * [col_lo, col_hi): the columns kept, re-based to col_lo (one rank's shard of a matrix partitioned by
 * post-synaptic neuron; 0 .. n_col keeps everything).  Calls, all enqueued on `stream`:
 *   bpl_cbcsr_plan   fills offsets (n_row x (n_blocks + 1) uint32, row-relative for now) and prefix-sums the
 *                    row totals; afterwards the first 8 bytes of `workspace`
 *                    (bpl_cbcsr_build_workspace_bytes(n_row) bytes) hold the number of 48-byte records.
 *   bpl_cbcsr_max_column_abs_sum   (fixed point only) max_out[0] = largest sum of |w| over a kept column;
 *                    colsum: scratch of col_hi - col_lo floats.  scale_log2 = floor(log2(2^30 / that)).
 *   bpl_cbcsr_fill   after the caller has read the record count and provided `groups` (48 * n_groups bytes,
 *                    16-byte aligned): makes the offsets absolute and writes the records; the order inside a
 *                    segment is the CSR order, so the result is a fixed function of the input. */
size_t bpl_cbcsr_build_workspace_bytes(uint32_t n_row);
uint32_t bpl_cbcsr_n_blocks(uint32_t n_col, uint32_t block_width);
void bpl_cbcsr_plan(bpl_stream_t stream, const void *indices, const void *indptr, uint32_t n_row, uint32_t col_lo,
                    uint32_t col_hi, uint32_t block_width, void *offsets, void *workspace);
void bpl_cbcsr_max_column_abs_sum(bpl_stream_t stream, const void *data, int homogeneous, const void *indices,
                                  uint64_t nse, uint32_t col_lo, uint32_t col_hi, void *colsum, void *max_out);
void bpl_cbcsr_fill(bpl_stream_t stream, const void *data, int homogeneous, const void *indices, const void *indptr,
                    uint32_t n_row, uint32_t col_lo, uint32_t col_hi, uint32_t block_width, void *offsets,
                    const void *workspace, void *groups, uint64_t n_groups, int fixed_point, int scale_log2);
/* Debugging aid: while `buffer` (device memory, 64 bytes per CTA of the launch) is not NULL, every
 * event_cbcsr_matvec_* launch of this host thread stamps its phases into it with the global nanosecond timer. */
void bpl_cbcsr_trace(void *buffer);

/* ---- spike exchange between the GPUs of one node (no counterpart in the reference) -----------
 * push: copies `slice_bytes` bytes at `local` into slot `slot` of every peer's data buffer (at offset
 *       (slot * world + rank) * slice_bytes) with peer stores, then bumps the peer's arrival counter
 *       flags[slot * world + rank].  peer_data / peer_flags: HOST arrays of `world` device pointers.
 * wait: polls this rank's own counters of `slot` until all `world` have passed state[slot]; at most
 *       `max_polls` polls (~0.2 us each) per source, then state[slots] = 1 (timeout) and it returns:
 *       the wait is bounded by construction.  state: slots + 1 + 17 u32 of this rank's own memory,
 *       zero-initialised by the caller (consumed counts, status word, CTA counters of the push).
 * world <= 16.  Both only enqueue on `stream`. */
void bpl_spike_exchange_push(bpl_stream_t stream, const void *local, size_t slice_bytes, void *const *peer_data,
                             void *const *peer_flags, void *state, int world, int rank, int slot, int slots);
void bpl_spike_exchange_wait(bpl_stream_t stream, void *flags, void *state, int world, int slot, int slots,
                             uint32_t max_polls);
/* Fused form: compaction of this rank's own events pushed straight into every rank's spike LIST (the layout the
 * scatter consumes: counts[1024], then row ids in 4096-entry chunk segments; rank r owns chunk indices
 * r * chunks_per_rank ...), so that consumers need no scan: wait_zero (bounded wait + zero-fill of the output
 * in one launch), then event_csr_matvec_list_heter_float.  peer_lists[p] = peer p's list buffer of this slot
 * (bpl_spike_list_slot_bytes bytes each); ev_is_float: 0 = bool events, 1 = float32. */
uint32_t bpl_spike_list_chunks_per_rank(uint32_t n_local);
size_t bpl_spike_list_slot_bytes(uint32_t n_local, int world);
void bpl_spike_exchange_push_compacted(bpl_stream_t stream, const void *local_events, int ev_is_float,
                                       uint32_t n_local, uint32_t row_offset, void *const *peer_lists,
                                       void *const *peer_flags, void *state, int world, int rank, int slot,
                                       int slots);
void bpl_spike_exchange_wait_zero(bpl_stream_t stream, void *flags, void *state, int world, int slot, int slots,
                                  uint32_t max_polls, void *zero, uint32_t n_zero);

/* One launch per simulation step on a column-sharded matrix (no reference counterpart): the kernel pushes
 * this rank's spikes of step t + 1 as a compacted list into every peer (peer stores), zero-fills y_next,
 * waits (bounded by max_polls) for the lists of step t from every rank, and scatters step t into y_cur,
 * which must already be zero (bpl_sharded_prime zero-fills the first one).  The step counter t lives in
 * `state` (slots + 1 + 32 zero-initialised uint32), so a captured sequence of steps can be replayed.
 * peer_lists[p] / peer_flags[p]: peer p's list buffer (slots x slot_bytes, see bpl_spike_list_slot_bytes)
 * and arrival counters (slots x world uint32, zero-initialised).  slots >= 4.  A timeout sets the status
 * word state[slots] to 1 and skips the scatter.  An exchange object is driven either by these two calls or
 * by the push / wait calls above, not by both. */
void bpl_sharded_prime(bpl_stream_t stream, const void *events, int ev_is_float, uint32_t n_local,
                       uint32_t row_offset, void *const *peer_lists, size_t slot_bytes, void *const *peer_flags,
                       void *state, int world, int rank, int slots, void *y_first, uint32_t n_out);
void bpl_sharded_step(bpl_stream_t stream, const void *data, const void *indices, const void *indptr,
                      uint32_t n_row, uint32_t n_out, void *y_cur, void *y_next, const void *next_events,
                      int ev_is_float, uint32_t n_local, uint32_t row_offset, void *const *peer_lists,
                      size_t slot_bytes, void *const *peer_flags, void *state, int world, int rank, int slots,
                      uint32_t max_polls);
/* The same step on a shard prepared into the column-blocked layout (bpl_cbcsr_plan / bpl_cbcsr_fill with the rank's
 * column range; arguments as in the opaque of event_cbcsr_matvec_*): the scatter accumulates in shared memory. */
void bpl_sharded_cb_step(bpl_stream_t stream, const void *groups, const void *offsets, uint32_t n_out,
                         uint32_t block_width, int fixed_point, int scale_log2, uint32_t team_lanes_log2, void *y_cur,
                         void *y_next, const void *next_events, int ev_is_float, uint32_t n_local, uint32_t row_offset,
                         void *const *peer_lists, size_t slot_bytes, void *const *peer_flags, void *state, int world,
                         int rank, int slots, uint32_t max_polls);

/* ---- runs of many steps on host-resident spike trains (no counterpart in the reference) ----
 * Every step's spikes come from pinned host memory and every step's result goes back to pinned host memory; copy
 * in, launch and copy out of neighbouring steps overlap on the three (distinct) streams over rings of three
 * device buffers, and the whole run is enqueued by this one call.  An event recorded on s_compute before / after
 * the call brackets the run.  host_in: n_steps x in_bytes; host_out: out_slots x out_bytes (step i lands in slot
 * i % out_slots).
 * bpl_run_host_steps: target_name (any registered target) is called once per step with buffers[in_index],
 * buffers[out_index] and, if ws_index >= 0, buffers[ws_index] replaced by a buffer of in_ring / out_ring / ws_ring,
 * which hold 3 * group buffers each; cross-stream waits sit between groups of `group` (1..16) consecutive steps, the
 * copies of a group run back to back. */
void bpl_run_host_steps(const char *target_name, const char *opaque, size_t opaque_len, void *const *buffers,
                        int n_buffers, int in_index, int out_index, int ws_index, void *const *in_ring,
                        void *const *out_ring, void *const *ws_ring, uint32_t group, const void *host_in,
                        size_t in_bytes, void *host_out, size_t out_bytes, uint32_t out_slots, uint32_t n_steps,
                        bpl_stream_t s_in, bpl_stream_t s_compute, bpl_stream_t s_out);
/* bpl_sharded_prime, then bpl_sharded_cb_step per step: host_events holds n_steps slices of this rank's own n_local
 * spike sources (float32 if ev_is_float, else one byte each), host_out takes this rank's n_out float32 outputs per
 * step; ev_ring: 3 * group + 1 buffers of n_local events, y_ring: 3 * group buffers of n_out floats (device). */
void bpl_sharded_run_host_steps(const void *groups, const void *offsets, uint32_t n_out, uint32_t block_width,
                                int fixed_point, int scale_log2, uint32_t team_lanes_log2, int ev_is_float,
                                uint32_t n_local, uint32_t row_offset, void *const *peer_lists, size_t slot_bytes,
                                void *const *peer_flags, void *state, int world, int rank, int slots,
                                uint32_t max_polls, void *const *ev_ring, void *const *y_ring, uint32_t group,
                                const void *host_events, void *host_out, uint32_t out_slots, uint32_t n_steps,
                                bpl_stream_t s_in, bpl_stream_t s_compute, bpl_stream_t s_out);
/* The same run on a shard kept as plain CSR arrays (bpl_sharded_step per step). */
void bpl_sharded_run_host_steps_csr(const void *data, const void *indices, const void *indptr, uint32_t n_row,
                                    uint32_t n_out, int ev_is_float, uint32_t n_local, uint32_t row_offset,
                                    void *const *peer_lists, size_t slot_bytes, void *const *peer_flags, void *state,
                                    int world, int rank, int slots, uint32_t max_polls, void *const *ev_ring,
                                    void *const *y_ring, uint32_t group, const void *host_events, void *host_out,
                                    uint32_t out_slots, uint32_t n_steps, bpl_stream_t s_in, bpl_stream_t s_compute,
                                    bpl_stream_t s_out);

/* ---- transposed event product without workspace and without allocation ------------------
 * No counterpart in the reference.  Same computation as event_csr_matvec_heter_float_float
 * with transpose=true, for callers that may neither allocate device memory nor pass the extra
 * workspace buffer (an XLA custom call that must keep the reference's exact buffer list, code
 * running under stream capture): the scratch is a fixed device array inside the library.
 *   buffers [data f32(nse), indices u32(nse), indptr u32(n_row+1), events f32(n_row), y f32(n_col)]
 *   opaque  TwoUintOneBoolDescriptor{n_row, n_col, transpose=true}
 * Limits: n_row <= bpl_noalloc_max_rows() (2,097,152), else status BPL_ERR_TOO_LARGE and nothing
 * runs; about 8.4 MB of device memory per GPU for the life of the process; calls that overlap on
 * one GPU race on the shared scratch (serialise them); the first call on a device resolves the
 * scratch address and should precede any stream capture. */
uint32_t bpl_noalloc_max_rows(void);
BPL_DECLARE_TARGET(event_csr_matvec_heter_float_float_noalloc);

#ifdef __cplusplus
}
#endif
#endif /* BRAINPYLIB_B200_H_ */
