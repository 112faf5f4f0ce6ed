/* gatzk_b200.h — C ABI of libgatzk_b200.so, the B200 (sm_100a) compute backend for
 * the data-parallel core of the GAT-ZKML prover.
 *
 * Conventions
 *  - every function returns 0 on success and a non-zero GZK_E_* code otherwise;
 *    gzk_last_error() gives the message of the last failure on the context.  No
 *    exception crosses this boundary.
 *  - Fr values cross the boundary as 32-byte little-endian canonical integers, the
 *    format of FieldElement::write_little_endian / from_little_endian_mod
 *    (include/gatzk/algebra/field.hpp:79-84, 193-201).
 *  - G1 points cross the boundary affine, x || y, 2 x 48 bytes little-endian
 *    canonical; 96 zero bytes are the point at infinity.
 *  - `gzk_buf` handles name device-resident arrays.  A buffer has a kind: FR
 *    (canonical 32-byte elements, the upload format), FR_MONT (Montgomery form,
 *    what kernels of this library produce), I64 / U32 (small-integer columns that
 *    are widened to Fr inside the kernels, as FieldElement::from_signed does,
 *    field.hpp:71-76).
 *  - one context per GPU and per host thread that issues work; calls on one
 *    context are ordered on the context's CUDA stream.
 *  - there is no CPU fallback: every entry point fails with GZK_E_CUDA when no
 *    sm_100 device is usable.
 */
#ifndef GATZK_B200_H
#define GATZK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GZK_OK 0
#define GZK_E_INVALID 1   /* bad argument: the reference would have thrown std::runtime_error */
#define GZK_E_CUDA 2      /* CUDA runtime failure or no usable device */
#define GZK_E_DOMAIN 3    /* evaluation point lies on the domain / zero denominator in a batch inversion */
#define GZK_E_TIMEOUT 4   /* a bounded device-side wait gave up */

#define GZK_KIND_FR 0
#define GZK_KIND_FR_MONT 1
#define GZK_KIND_I64 2
#define GZK_KIND_U32 3
#define GZK_KIND_F64 4   /* IEEE doubles: the fp64 forward pass and the input of gzk_quantize */
#define GZK_KIND_G1 5    /* affine G1 points, 96 bytes; wire format on upload/download, Montgomery on the device */

typedef struct gzk_ctx gzk_ctx;
typedef struct gzk_buf gzk_buf;

/* ---- context ------------------------------------------------------------------
 * Replaces the runtime probe `cuda_backend_runtime_available()`
 * (src/algebra/cuda_backend.cu:10-14, used by src/main.cpp:134-142) and owns what
 * the reference keeps in process-wide caches: domain tables
 * (RootOfUnityDomain::create, src/algebra/polynomial.cpp:37-91). */
int gzk_ctx_create(int device, gzk_ctx** out);
void gzk_ctx_destroy(gzk_ctx* ctx);
const char* gzk_last_error(const gzk_ctx* ctx);
int gzk_ctx_synchronize(gzk_ctx* ctx);
/* Deferred mode: calls whose results stay on the device (the column builders, row folds,
 * gathers, histograms ...) return as soon as their kernels are queued, so the host runs
 * ahead of the GPU as a chain of kernels; an error raised on the device (zero denominator,
 * index out of range) is then reported by the next gzk_ctx_synchronize instead of by the
 * call itself.  Calls that return values to the host always synchronise.  Off by default
 * (every call reports its own errors, like the reference's exceptions). */
int gzk_ctx_set_deferred(gzk_ctx* ctx, int on);
/* the CUDA stream (cudaStream_t) all work of this context is issued on */
void* gzk_ctx_stream(gzk_ctx* ctx);
/* Orders two contexts of one GPU on the device: what is queued on `ctx` after this call runs after what
 * was queued on `other` before it.  Nothing waits on the host.  For a host thread that deals independent
 * chains of short calls over several contexts (each context is one stream) and joins them again; the
 * reference runs such chains as concurrent std::async tasks (src/protocol/trace.cpp:2737-2772). */
int gzk_ctx_wait_for(gzk_ctx* ctx, gzk_ctx* other);

/* ---- measurement ---------------------------------------------------------------
 * Per kernel family: number of launches since the last reset and, while timing is
 * enabled, the summed CUDA-event duration on the context stream.  Replaces the
 * steady_clock stage metrics of RunMetrics (include/gatzk/protocol/proof.hpp:119-272)
 * for device work. */
int gzk_timing_enable(gzk_ctx* ctx, int on);
int gzk_timing_reset(gzk_ctx* ctx);
int gzk_timing_family_count(gzk_ctx* ctx);
int gzk_timing_get(gzk_ctx* ctx, int index, const char** name, uint64_t* launches, double* total_ms);
/* Work of the packed-evaluation launches since the last gzk_timing_reset, for rooflines: out[0]
 * algorithmic bytes (every column element once per launch at its stored width of 4 / 8 / 32 bytes,
 * the weight vector once per rotation), out[1] 32x32-bit limb products of the inner loops (64 per
 * term for field-element columns, 16 for I64, 8 for U32), out[2] (row, column, rotation) terms. */
int gzk_eval_work_counters(gzk_ctx* ctx, uint64_t out[3]);

/* Test facility for the device-side failure handling.  The packed-evaluation kernel waits
 * for its bulk copies with a bounded number of polls; when a wait runs out the kernel raises
 * GZK_E_TIMEOUT in the status word and returns.  While this switch is on (process-wide),
 * every launch of that kernel arms its chunk barriers but issues no copy and polls only a
 * few hundred times, so the waits do run out - with nothing in flight and no fault - and the
 * error path can be exercised: gzk_eval_batch returns GZK_E_TIMEOUT, gzk_eval_batch_static
 * poisons its outputs.  No reference counterpart (the reference has no device-side waits). */
int gzk_debug_inject_eval_stall(int on);

/* ---- device buffers -----------------------------------------------------------
 * Replace the host std::vector<FieldElement> column storage of
 * Polynomial::from_evaluations (src/algebra/polynomial.cpp:364-379) and the
 * interleaved copy of the PackedEvaluationBackend constructor
 * (src/algebra/eval_backend.cpp:61-87): columns stay column-major in HBM. */
int gzk_buf_alloc(gzk_ctx* ctx, int kind, size_t count, gzk_buf** out);
int gzk_buf_free(gzk_ctx* ctx, gzk_buf* buf);
/* A buffer over device memory the caller owns (its own pool, a tensor of its framework, a
 * communication buffer): nothing is allocated or copied, gzk_buf_free releases only the
 * handle.  The pointer must be 32-byte aligned memory of the context's GPU and stay valid
 * while the handle is in use. */
int gzk_buf_wrap(gzk_ctx* ctx, int kind, size_t count, void* device_ptr, gzk_buf** out);
/* Declares which of the two 32-byte forms (GZK_KIND_FR canonical, GZK_KIND_FR_MONT) the
 * buffer holds from now on, for work areas that are refilled by copies (gzk_transpose,
 * gzk_swap_outer, an exchange between GPUs); nothing is converted. */
int gzk_buf_retag(gzk_buf* buf, int kind);
/* Copies `count` elements from host memory (canonical form; an FR_MONT or G1 buffer converts on the
 * device).  The host memory may be reused as soon as the call returns.  The call waits for the copy,
 * except in deferred mode for uploads of at most 256 KiB, which are staged and ordered on the
 * context's stream like a kernel (another context sees them after gzk_ctx_synchronize). */
int gzk_buf_upload(gzk_ctx* ctx, gzk_buf* buf, size_t offset, const void* host, size_t count);
/* gzk_buf_upload_async queues the copy on a second stream so that it overlaps with kernels
 * in flight (host memory should be pinned and must stay valid); gzk_copy_fence makes all
 * work issued afterwards wait for the uploads queued so far. */
int gzk_buf_upload_async(gzk_ctx* ctx, gzk_buf* buf, size_t offset, const void* host, size_t count);
int gzk_copy_fence(gzk_ctx* ctx);
/* Page-locks / releases a range of the caller's host memory (the reference keeps its inputs in
 * ordinary std::vector storage): uploads from a registered range are direct DMA transfers. */
int gzk_host_register(void* host, size_t bytes);
int gzk_host_unregister(void* host);
/* downloads always deliver the wire format: FR_MONT buffers are converted to
 * canonical on the device first */
int gzk_buf_download(gzk_ctx* ctx, const gzk_buf* buf, size_t offset, void* host, size_t count);
size_t gzk_buf_count(const gzk_buf* buf);
int gzk_buf_kind(const gzk_buf* buf);
void* gzk_buf_device_ptr(gzk_buf* buf);

/* ---- a1: field helpers ---------------------------------------------------------
 * omega_n = 5^((r-1)/n): FieldElement::root_of_unity (field.hpp:87-101). */
int gzk_root_of_unity(gzk_ctx* ctx, uint64_t size, uint8_t out[32]);
/* FieldElement +, -, *, inv on the host (field.hpp:112-179) for the caller's scalar
 * glue: op 0 add, 1 sub, 2 mul, 3 inverse of a (GZK_E_DOMAIN for zero). */
int gzk_fr_op(int op, const uint8_t a[32], const uint8_t b[32], uint8_t out[32]);

/* ---- a2: barycentric weights ----------------------------------------------------
 * w_i(x) = (x^n - 1) * omega^i / n / (x - omega^i), i < n = 2^log2n.
 * Replaces RootOfUnityDomain::barycentric_weights_native
 * (src/algebra/polynomial.cpp:131-316) and cached_barycentric_weights_native
 * (src/protocol/trace.cpp:181-201).  `out` must be FR_MONT with count >= n.
 * GZK_E_DOMAIN when x is a domain point (the reference then takes the
 * direct-index branch of build_domain_evaluation_weights,
 * include/gatzk/algebra/domain_evaluation.hpp:40-71, which the caller handles). */
int gzk_bary_weights(gzk_ctx* ctx, unsigned log2n, const uint8_t x[32], gzk_buf* out);
/* The same vector when only w[0 .. keep), w[n-2] and w[n-1] will be read (every column of the domain is stored
 * as a prefix of at most `keep` rows; the last two are what rows 0 and 1 meet at rotations 1 and 2): the other
 * entries of `out` are not written, which saves their share of the arithmetic. */
int gzk_bary_weights_prefix(gzk_ctx* ctx, unsigned log2n, const uint8_t x[32], uint64_t keep, gzk_buf* out);
/* Weight vectors of one domain at `count` points (points: count x 32 bytes) into outs[0 .. count): for a domain of at
 * most 2^18 points and up to four points one launch (the binding points a head draws at the same transcript stage,
 * src/protocol/trace.cpp:2461-2530, are independent dependent-chains); otherwise one gzk_bary_weights per point. */
int gzk_bary_weights_multi(gzk_ctx* ctx, unsigned log2n, const uint8_t* points, size_t count, gzk_buf* const* outs);

/* ---- a3 / a4: packed evaluation and commit inner products ------------------------
 * out[p][k] = sum_{c < len} col_k[c] * w[(c - rot_p) mod n]
 *           = sum_c w[c] * col_k[(c + rot_p) mod n]   (columns are zero beyond len).
 * Replaces PackedEvaluationBackend::evaluate_with_native_weights and
 * ::evaluate_with_native_weight_rotations (src/algebra/eval_backend.cpp:191-292,
 * 309-444), evaluate_polynomials_with_shared_domain_weights
 * (src/crypto/kzg.cpp:161-282; valid prefix = len, one rotation 0) and
 * dot_product_native_weights (src/algebra/vector_ops.cpp:168-219).
 * cols: K buffers of kind FR / FR_MONT / I64 / U32 with count >= len;
 * weights: FR_MONT with count >= n; out_host: P*K*32 bytes, [p][k].
 * The sums are exact integers reduced once: field-element columns form them from byte products on the tensor
 * cores, small-integer columns on the integer pipe or, at two points, in groups of four on the tensor cores; a call
 * launches one kernel per kind of column present.  The results do not depend on which kernel took a column. */
int gzk_eval_batch(gzk_ctx* ctx, gzk_buf* const* cols, size_t k_count, size_t len, unsigned log2n,
                   const gzk_buf* weights, const uint64_t* rotations, size_t p_count, uint8_t* out_host);

/* The same sums left on the device, for consumers that are themselves on the device (the
 * same-base G1 multiplication of a commit barrier, an exchange of partial sums between GPUs):
 * out[out_offset + p*k_count + k], canonical for an FR buffer, Montgomery for an FR_MONT one.
 * Nothing is read back, so in deferred mode these calls only queue kernels.  Together with
 * gzk_matrix_horner_device and gzk_g1_fixed_base_mul they form KZG::commit_batch
 * (src/crypto/kzg.cpp:458-542) with ONE read-back per batch of columns. */
int gzk_eval_batch_device(gzk_ctx* ctx, gzk_buf* const* cols, size_t k_count, size_t len, unsigned log2n,
                          const gzk_buf* weights, const uint64_t* rotations, size_t p_count, gzk_buf* out, size_t out_offset);

/* The edge side of a route whose query of edge e is the table row of the node the edge points at
 * (query columns = node columns gathered by `index`, as build_route_trace's callers construct them,
 * src/protocol/trace.cpp:1776-1794, 2737-2772): 1/(query_e + beta) = 1/(table_{index[e]} + beta), so the
 * node_count table inverses are computed once and the running sum fetches them.  Same output as
 * gzk_route_edge_accumulator on the gathered query column; an index outside the table raises
 * GZK_E_INVALID. */
int gzk_route_edge_accumulator_indexed(gzk_ctx* ctx, const gzk_buf* table, size_t node_count, const gzk_buf* index, size_t valid_length,
                                       size_t domain_size, const uint8_t beta[32], gzk_buf* out);
/* The same accumulator for a lookup into a banded static table, computed without one inversion per
 * row.  Every query (x[i], y[i]) equals some table row - the lookup argument proves exactly that, and
 * gzk_banded_lookup_multiplicity has located the row already - so 1/(query_i + beta) is one of the
 * table_size values 1/(table_t + beta).  Those are inverted once (pass 0), and the accumulator's
 * term of row i becomes  [i < table_size] multiplicity[i] / (table_i + beta)  -  1/(table_{hit(i)} + beta),
 * a 32-byte fetch per row.  The selectors are taken to be the prefix indicators the reference builds
 * (table rows first, queries on rows < active_count; src/protocol/prover.cpp:460-535), x_min / band /
 * table_y describe the table as in gzk_banded_lookup_multiplicity.  Same output as
 * gzk_logup_accumulator on the packed columns (src/protocol/lookup.cpp:100-157); a query outside
 * the table raises GZK_E_INVALID. */
int gzk_logup_accumulator_indexed(gzk_ctx* ctx, const gzk_buf* table, const gzk_buf* multiplicity, const gzk_buf* x, const gzk_buf* y,
                                  size_t active_count, int64_t x_min, size_t band, const gzk_buf* table_y, size_t table_size, size_t n,
                                  const uint8_t beta[32], gzk_buf* out);
/* ---- a7: LogUp and route running sums ----------------------------------------------
 * Input columns may be of any kind; `out` is FR_MONT with count >= n.  One batch
 * inversion per call; GZK_E_DOMAIN ("batch_invert encountered zero") when a
 * denominator is zero, as the reference throws.
 * gzk_logup_accumulator: R_0 = 0, R_{i+1} = R_i + q_table_i*m_i/(T_i+beta) - q_query_i/(Q_i+beta)
 * for i < active_count (clamped to n-1), tail filled with the last value.  Replaces
 * build_logup_accumulator_with_active_count (src/protocol/lookup.cpp:100-157).
 * gzk_route_node_accumulator / gzk_route_edge_accumulator: running sums of
 * m_i/(T_i+beta) resp. 1/(Q_i+beta) over the first valid_length rows (must be <
 * domain_size).  Replace build_route_node_accumulator / build_route_edge_accumulator
 * (src/protocol/trace.cpp:298-361). */
int gzk_logup_accumulator(gzk_ctx* ctx, const gzk_buf* table, const gzk_buf* query, const gzk_buf* multiplicity,
                          const gzk_buf* q_table, const gzk_buf* q_query, size_t n, const uint8_t beta[32],
                          size_t active_count, gzk_buf* out);
int gzk_route_node_accumulator(gzk_ctx* ctx, const gzk_buf* table, const gzk_buf* multiplicity, size_t valid_length,
                               size_t domain_size, const uint8_t beta[32], gzk_buf* out);
int gzk_route_edge_accumulator(gzk_ctx* ctx, const gzk_buf* query, size_t valid_length, size_t domain_size,
                               const uint8_t beta[32], gzk_buf* out);

/* Several independent running sums in ONE pair of launches.  The accumulators that sit between two
 * Fiat-Shamir points of one attention head (the lookup sums, the node and edge sums of a routing
 * argument, the segmented states, the small inner-product accumulators: src/protocol/trace.cpp:2565-2772)
 * do not depend on one another; alone each is a short latency chain on a fraction of the GPU, queued
 * together they fill it.  A job is one call of the single-column functions, with the same meaning of
 * its fields and the same errors:
 *   GZK_SCAN_LOGUP        c0..c4 = table, query, multiplicity, q_table, q_query; count = active_count
 *   GZK_SCAN_ROUTE_NODE   c0, c1 = table, multiplicity; count = valid_length
 *   GZK_SCAN_ROUTE_EDGE   c0 = query; count = valid_length
 *   GZK_SCAN_ZKMAP        c0, c1 = a, b; count = number of products (the total is out[count])
 *   GZK_SCAN_GROUP_PREFIX c0, c1 = values, q_new; count ignored (the whole domain)
 * beta: 32 bytes for the first three operations, NULL otherwise.  At most 2^20 rows per job. */
#define GZK_SCAN_LOGUP 0
#define GZK_SCAN_ROUTE_NODE 1
#define GZK_SCAN_ROUTE_EDGE 2
#define GZK_SCAN_ZKMAP 3
#define GZK_SCAN_GROUP_PREFIX 4
typedef struct gzk_scan_job
{
    int op;
    const gzk_buf* c0;
    const gzk_buf* c1;
    const gzk_buf* c2;
    const gzk_buf* c3;
    const gzk_buf* c4;
    size_t count;
    size_t domain_size;
    const uint8_t* beta;
    gzk_buf* out;
} gzk_scan_job;
int gzk_running_sums_batch(gzk_ctx* ctx, const gzk_scan_job* jobs, size_t job_count);

/* ---- a8: segmented prefix states over the dst-sorted edge list ------------------------
 * out[0] = v[0]; out[i] = q_new[i] ? v[i] : out[i-1] + v[i].  q_new must hold only
 * 0 and 1 (the reference's selector; other values give GZK_E_INVALID).  Replaces
 * build_group_prefix_state and build_max_counter_state (src/protocol/psq.cpp:7-39). */
int gzk_group_prefix_state(gzk_ctx* ctx, const gzk_buf* values, const gzk_buf* q_new, size_t n, gzk_buf* out);

/* ---- a9: inner-product accumulator ------------------------------------------------------
 * acc[0] = 0, acc[i+1] = acc[i] + a[i]*b[i] for i < count, tail filled with the
 * total, which is also returned in mu_out.  Replaces build_zkmap_trace
 * (src/protocol/zkmap.cpp:7-32) and the accumulator of build_binding_trace
 * (src/protocol/trace.cpp:1595-1621). */
int gzk_zkmap_accumulator(gzk_ctx* ctx, const gzk_buf* a, const gzk_buf* b, size_t count, size_t domain_size,
                          gzk_buf* out_acc, uint8_t mu_out[32]);

/* ---- a6 / a9 / a12: matrices and coefficient polynomials ----------------------------------
 * gzk_matrix_horner: the rows x cols row-major matrix read as one coefficient
 * polynomial sum_{i,j} M[i][j] x^(i*cols+j).  Replaces matrix_row_major_evaluation /
 * row_polynomial_at_point (src/protocol/trace.cpp:508-573, twin at
 * src/protocol/prover.cpp:414-440) and, with rows = 1, horner / the coefficient
 * branch of Polynomial::evaluate (src/algebra/polynomial.cpp:415-421, 499-508).
 * gzk_fold_rows: out[c] = sum_{row < row_count} w[row] * M[row][c]; `out` is an FR
 * buffer (canonical).  Replaces weighted_column_sum_native (trace.cpp:203-271).
 * gzk_linear_form_rows: out[row] = sum_c M[row][c] * powers[c]; out FR_MONT.  Replaces
 * linear_form_by_powers / compress_rows_with_challenge (trace.cpp:273-296, 1358-1364).
 * gzk_powers: 1, c, c^2, ... (the `powers` helper those callers use). */
int gzk_matrix_horner(gzk_ctx* ctx, const gzk_buf* matrix, size_t rows, size_t cols, const uint8_t x[32], uint8_t out[32]);
int gzk_fold_rows(gzk_ctx* ctx, const gzk_buf* matrix, size_t rows, size_t cols, const gzk_buf* row_weights, size_t row_count,
                  gzk_buf* out);
int gzk_linear_form_rows(gzk_ctx* ctx, const gzk_buf* matrix, size_t rows, size_t cols, const gzk_buf* column_powers, gzk_buf* out);
int gzk_powers(gzk_ctx* ctx, const uint8_t challenge[32], size_t count, gzk_buf* out);
/* gzk_matrix_horner with the value left in out[out_offset] on the device (FR: canonical, FR_MONT:
 * Montgomery form). */
int gzk_matrix_horner_device(gzk_ctx* ctx, const gzk_buf* matrix, size_t rows, size_t cols, const uint8_t x[32], gzk_buf* out,
                             size_t out_offset);

/* ---- a10: witness-column leaves ---------------------------------------------------------------
 * gzk_weighted_sum: out[i] = left[i] + lambda*right[i], i < count, zero tail
 *   (build_weighted_sum and the query pack of build_pair_lookup_artifacts,
 *   src/protocol/trace.cpp:2073, 2098-2108).
 * gzk_feature_lookup_rows: out[row*width+c] = row_id[row] + eta_i*feature_index[c]
 *   + eta_v*features[row*width+c] (fill_feature_lookup_rows, trace.cpp:579-607).
 * gzk_broadcast_node_values: out[e] = node_values[index[e]], e < edge_count, zero tail;
 *   index is a U32 or I64 buffer, out has the kind of node_values
 *   (broadcast_node_values and the gathers of quantize_*_witness_cpu,
 *   trace.cpp:1366-1381, 1143-1279).
 * gzk_histogram: out[b] = #{i : indices[i] = b}, out is a U32 column
 *   (multiplicity_from_indices, trace.cpp:1916-1933, and lookup_histogram_indices_cuda,
 *   src/algebra/cuda_backend.cu:21-102).
 * gzk_quantize: F64 -> I64, round half away from zero at scale 16 (quantize_float,
 *   trace.cpp:973-976).
 * gzk_first_zero_marker: out[k] = 1 for the first row k of every [begin,end) group
 *   with delta[k] = 0, else 0; out is a U32 column (s_max, trace.cpp:2610-2618). */
int gzk_weighted_sum(gzk_ctx* ctx, const gzk_buf* left, const uint8_t lambda[32], const gzk_buf* right, size_t count,
                     size_t domain_size, gzk_buf* out);
int gzk_feature_lookup_rows(gzk_ctx* ctx, const gzk_buf* row_ids, const gzk_buf* feature_indices, const gzk_buf* features,
                            size_t rows, size_t width, const uint8_t eta_index[32], const uint8_t eta_value[32], gzk_buf* out);
int gzk_broadcast_node_values(gzk_ctx* ctx, const gzk_buf* node_values, size_t node_count, const gzk_buf* index, size_t edge_count,
                              size_t domain_size, gzk_buf* out);
int gzk_histogram(gzk_ctx* ctx, const gzk_buf* indices, size_t count, size_t domain_size, gzk_buf* out);
int gzk_quantize(gzk_ctx* ctx, const gzk_buf* values, size_t count, gzk_buf* out);
/* gzk_quantize that also counts, into flagged[0] (a U32 buffer; added to, not cleared), the values
 * whose 16*|v| lies within `guard` of a rounding boundary k + 1/2.  The forward pass on the GPU is
 * bit-identical to the host's up to exp / expm1, whose last bit may differ between the CUDA and the
 * host math library; a quantised value can then differ from the reference's only if 16*v is that
 * close to a boundary.  A caller that needs the byte-identical witness re-computes on the host,
 * with the reference's own loop (src/model/gat.cpp:474-615), whenever the count is not zero. */
int gzk_quantize_guarded(gzk_ctx* ctx, const gzk_buf* values, size_t count, double guard, gzk_buf* out, gzk_buf* flagged);
int gzk_first_zero_marker(gzk_ctx* ctx, const gzk_buf* delta, const gzk_buf* group_begin, const gzk_buf* group_end, size_t groups,
                          size_t domain_size, gzk_buf* out);

/* ---- a10: column packs and lookup multiplicities ---------------------------------------------------
 * gzk_linear_combination: out[i] = sum_j coefficients[j] * cols[j][i] for i < count, zero tail;
 *   1 to 8 terms, coefficients = terms x 32 bytes.  The routing-table packs with up to six
 *   challenge powers (src/protocol/trace.cpp:2978-3006), table packs T_x + eta*T_y
 *   (cached_pair_lookup_table, trace.cpp:1958-1988) and the average of the output heads
 *   (average_field_matrices, trace.cpp:994-1018) are of this shape.
 * gzk_mul_columns: out[i] = left[i] * right[i] for i < count, zero tail (the products
 *   alpha * H_star_edge of trace.cpp:2716-2719).
 * gzk_banded_lookup_multiplicity: multiplicity column of a lookup into one of the static
 *   tables.  The reference finds the table row of every query in a hash map and counts the hits
 *   (build_single_lookup_artifacts / build_pair_lookup_artifacts + multiplicity_from_indices,
 *   trace.cpp:1916-1933, 2011-2096).  Its tables (make_range_table, make_lrelu_table,
 *   make_elu_table, make_exp_table, src/protocol/prover.cpp:460-535) are all "banded": row
 *   band*(x - x_min) + j holds the j-th candidate second component for first component x, so the
 *   row is arithmetic on x plus a scan of `band` candidates table_y[...] (first match wins, as the
 *   hash map keeps the first of equal pairs).  x / y: I64 or U32 query columns (y and table_y NULL
 *   for the single-column range table, band 1); out: U32 column of domain_size.  A query that is
 *   not in the table gives GZK_E_INVALID "lookup query escaped static table", as the reference throws.
 * gzk_buf_zero: clears a buffer (the zero tails of padded columns).
 * gzk_copy_block: dst[dst_offset + r*dst_stride + c] = src[src_offset + r*src_stride + c] for
 *   r < rows, c < width: concatenation of per-head matrices (model::forward_note_style,
 *   src/model/gat.cpp:1155-1194) and flattening / padding of matrices into columns; src_stride 0
 *   repeats one source row (the quantised output bias under every row, trace.cpp:1257-1268). */
int gzk_linear_combination(gzk_ctx* ctx, const gzk_buf* const* cols, const uint8_t* coefficients, size_t terms, size_t count,
                           size_t domain_size, gzk_buf* out);
int gzk_mul_columns(gzk_ctx* ctx, const gzk_buf* left, const gzk_buf* right, size_t count, size_t domain_size, gzk_buf* out);
int gzk_banded_lookup_multiplicity(gzk_ctx* ctx, const gzk_buf* x, const gzk_buf* y, size_t count, int64_t x_min, size_t band,
                                   const gzk_buf* table_y, size_t table_size, size_t domain_size, gzk_buf* out);
int gzk_buf_zero(gzk_ctx* ctx, gzk_buf* buf);
int gzk_copy_block(gzk_ctx* ctx, const gzk_buf* src, size_t src_offset, size_t src_stride, gzk_buf* dst, size_t dst_offset,
                   size_t dst_stride, size_t rows, size_t width);

/* ---- a11: public feature-domain columns that are never materialised ---------------------------
 * out[0..4] = sum_{i < rows*feature_count} w[i] * {1, i / fc, i % fc, abs_ids[i / fc],
 * features[i]} (32 bytes each; abs_ids / features may be NULL, their slot is then
 * zero).  Replaces evaluate_truncated_domain_polynomial and
 * evaluate_lazy_large_fh_public_group(_points) (src/protocol/prover.cpp:224-276,
 * 1205-1675), which stream the same generated columns on the CPU for n_FH >= 2^24.
 * Weights at the wanted point come from gzk_bary_weights. */
int gzk_fh_public_eval(gzk_ctx* ctx, const gzk_buf* features, size_t rows, size_t feature_count, const gzk_buf* abs_ids,
                       const gzk_buf* weights, uint8_t out[5 * 32]);
/* The same five sums at the rotated point omega^rotation * z, from the weights at z of the whole
 * 2^log2n domain: entry i then meets weights[(i - rotation) mod n], as the rotated evaluations of
 * evaluate_with_native_weight_rotations do (src/algebra/eval_backend.cpp:309-444). */
int gzk_fh_public_eval_rotated(gzk_ctx* ctx, const gzk_buf* features, size_t rows, size_t feature_count, const gzk_buf* abs_ids,
                               const gzk_buf* weights, unsigned log2n, uint64_t rotation, uint8_t out[5 * 32]);

/* ---- a5: G1 -----------------------------------------------------------------------------------
 * gzk_g1_mul_same_base: points[k] = [scalars[k]] base for K host scalars (32-byte
 * canonical) -> K affine points (96 bytes each).  Replaces g1_mul_same_base_batch /
 * mcl::G1::mulEach (src/crypto/curve.cpp:138-238) and batch_quotient_commitments
 * (src/protocol/prover.cpp:2220-2247).  A window table of the base is built on first
 * use and stays resident on the context.  The base is an argument because the
 * reference derives its generator with mcl's hashAndMapToG1 (src/crypto/kzg.cpp:383).
 * gzk_g1_fixed_base_mul: same for a device scalar buffer (FR or FR_MONT) into a G1 buffer.
 * gzk_commit_batch: tau-evaluations (gzk_eval_batch, rotation 0, valid prefix len) followed
 * by the same-base multiplication: KZG::commit_batch (src/crypto/kzg.cpp:458-542);
 * returns both the scalars p_k(tau) (Commitment::tau_evaluation) and the points. */
int gzk_g1_mul_same_base(gzk_ctx* ctx, const uint8_t base[96], const uint8_t* scalars_host, size_t count, uint8_t* points_out_host);
int gzk_g1_fixed_base_mul(gzk_ctx* ctx, const uint8_t base[96], const gzk_buf* scalars, size_t count, gzk_buf* out);
int gzk_commit_batch(gzk_ctx* ctx, gzk_buf* const* cols, size_t k_count, size_t len, unsigned log2n, const gzk_buf* weights_tau,
                     const uint8_t base[96], uint8_t* tau_evals_out, uint8_t* points_out);

/* ---- fp64 forward pass of one attention head -----------------------------------------------------
 * Replaces attention_head_forward_impl (src/model/gat.cpp:474-615, with matmul / matvec /
 * leaky_relu / elu of :354-401): H' = X W, the two score vectors, per destination node the
 * softmax statistics M / Sum / inv and the alpha-weighted aggregation over its incoming
 * edges, the per-edge columns S, Z, Delta, U, alpha, and H_agg = ELU(H_agg_pre + bias).
 * Every sum runs serially in index order with separate multiply and add, as on the host,
 * so H', E_src, E_dst, S, Z, M, Delta are bit-identical to the reference; U, Sum, inv, alpha
 * and H_agg inherit the last-place behaviour of the CUDA exp / expm1.
 * The incoming list (incoming_ptr[node_count+1], incoming_src[incoming_count]) holds, per
 * destination node, its sources in edge order followed by the node itself when the edges
 * carry no self loop - the `incoming_sources` the reference builds on the host
 * (gat.cpp:521-538); edge_src / edge_dst are the edges in their original order.
 * All matrices are row-major F64 buffers; index lists are U32 buffers.  Outputs marked
 * optional may be NULL.  Errors: GZK_E_INVALID for an endpoint out of range (the
 * reference throws "edge out of bounds while running attention head forward"). */
typedef struct gzk_gat_head
{
    const gzk_buf* features;         /* node_count x input_width */
    uint32_t input_width;
    uint32_t output_width;
    const gzk_buf* seq_kernel;       /* input_width x output_width */
    const gzk_buf* attn_src_kernel;  /* output_width */
    const gzk_buf* attn_dst_kernel;  /* output_width */
    double attn_src_bias;
    double attn_dst_bias;
    const gzk_buf* output_bias;      /* output_bias_count entries, or NULL (apply_output_bias = false) */
    size_t output_bias_count;
    int apply_activation;            /* ELU on the output when non-zero */
} gzk_gat_head;
typedef struct gzk_gat_graph
{
    size_t node_count;
    size_t edge_count;
    const gzk_buf* edge_src;         /* edge_count */
    const gzk_buf* edge_dst;         /* edge_count */
    size_t incoming_count;
    const gzk_buf* incoming_ptr;     /* node_count + 1 */
    const gzk_buf* incoming_src;     /* incoming_count */
} gzk_gat_graph;
typedef struct gzk_gat_trace
{
    gzk_buf* H_prime;                /* node_count x output_width */
    gzk_buf* E_src;                  /* node_count */
    gzk_buf* E_dst;                  /* node_count */
    gzk_buf* M;                      /* node_count */
    gzk_buf* Sum;                    /* node_count */
    gzk_buf* inv;                    /* node_count */
    gzk_buf* S;                      /* edge_count, optional */
    gzk_buf* Z;                      /* edge_count, optional */
    gzk_buf* Delta;                  /* edge_count, optional */
    gzk_buf* U;                      /* edge_count, optional */
    gzk_buf* alpha;                  /* edge_count, optional */
    gzk_buf* H_agg_pre_bias;         /* node_count x output_width, optional */
    gzk_buf* H_agg;                  /* node_count x output_width, optional */
} gzk_gat_trace;
int gzk_gat_head_forward(gzk_ctx* ctx, const gzk_gat_head* head, const gzk_gat_graph* graph, const gzk_gat_trace* out);

/* ---- MSM (kernel sweep; honest-prover commitment) ----------------------------------------------
 * gzk_msm: out = sum_i [scalars[i]] points[i]; scalars FR or FR_MONT, points a G1
 * buffer.  Pippenger with signed-digit windows and XYZZ buckets.  No reference caller:
 * the reference commits with the trapdoor (src/crypto/kzg.cpp:402-419); against the
 * Lagrange SRS of gzk_srs_lagrange the MSM of a column equals that commitment.
 * gzk_srs_lagrange: out_points[i] = [L_i(tau)] base over the 2^log2n domain. */
int gzk_msm(gzk_ctx* ctx, const gzk_buf* scalars, const gzk_buf* points, size_t n, uint8_t out[96]);
int gzk_srs_lagrange(gzk_ctx* ctx, unsigned log2n, const uint8_t base[96], const uint8_t tau[32], gzk_buf* out_points);
/* MSM against a FIXED point set that stays resident (an SRS): gzk_msm_precompute fills `table`
 * (a G1 buffer of gzk_msm_table_points(n, window_bits) points) with 2^(window_bits*w) P_i for
 * every window w of the signed-digit decomposition; gzk_msm_precomputed then adds the digits
 * of all windows into one set of 2^(window_bits-1) buckets - same result as gzk_msm, without
 * the per-window reductions and the chain of ~254 doublings at the end.
 * gzk_msm_window_bits(n) is the recommended window for n points.  The table costs
 * ceil(255/window_bits) times the memory of the points and one pass of doublings to build. */
unsigned gzk_msm_window_bits(size_t n);
size_t gzk_msm_table_points(size_t n, unsigned window_bits);
int gzk_msm_precompute(gzk_ctx* ctx, const gzk_buf* points, size_t n, unsigned window_bits, gzk_buf* table);
int gzk_msm_precomputed(gzk_ctx* ctx, const gzk_buf* scalars, const gzk_buf* table, size_t n, unsigned window_bits, uint8_t out[96]);

/* ---- NTT / coset LDE / multilinear fold (kernel sweep) -------------------------------------------
 * No reference caller: the reference evaluates by barycentric weights and never
 * builds quotient polynomials (src/algebra/polynomial.cpp:131-316, 415-508).  The
 * domain is the reference's: omega_n = 5^((r-1)/n) (field.hpp:87-101).
 * gzk_ntt: out[b][j] = sum_i in[b][i] * (shift*omega^j)^i (forward) or its inverse;
 * natural order in and out, `batch` vectors stored back to back; coset_shift may
 * be NULL (shift 1).  `out` is FR_MONT and must differ from `in`.
 * gzk_coset_lde: evaluations on the 2^log2n domain -> evaluations on shift * the
 * 2^(log2n+log2_blowup) domain.
 * gzk_fold: out[i] = t[2i] + r*(t[2i+1] - t[2i]), i < n/2 (one sumcheck round); out is an FR or
 *   FR_MONT buffer - a table kept in one form (canonical in and out, or Montgomery in and out) costs
 *   one multiplication per output, a change of form one more. */
int gzk_ntt(gzk_ctx* ctx, const gzk_buf* in, gzk_buf* out, unsigned log2n, size_t batch, int inverse, const uint8_t* coset_shift);
int gzk_coset_lde(gzk_ctx* ctx, const gzk_buf* in, unsigned log2n, unsigned log2_blowup, const uint8_t shift[32], gzk_buf* out);
int gzk_fold(gzk_ctx* ctx, const gzk_buf* table, size_t n, const uint8_t challenge[32], gzk_buf* out);

/* ---- row-sharded transform (kernel sweep at 2^24 and above, several GPUs) -----------------------
 * No reference caller.  n = n1*n2, element i = i1*n2 + i2, each GPU owns a block of rows i1.
 * Forward: pack (gzk_swap_outer) -> all-to-all -> gzk_transpose -> gzk_ntt of length n1 on
 * every row -> gzk_ntt_twiddle -> pack -> all-to-all -> gzk_transpose -> gzk_ntt of length
 * n2; the GPU that owns k1 in its block ends with X[k1 + n1*k2] stored as [k1][k2].  The
 * inverse runs the same steps backwards.  The all-to-all is the caller's (NCCL): data
 * lands in the receiver's own memory before any kernel reads it.
 * gzk_swap_outer: out[b][a][c] = in[a][b][c] for a < d0, b < d1, c < d2.
 * gzk_transpose: out[c][r] = in[r][c].  Both move FR / FR_MONT elements unchanged.
 * gzk_ntt_twiddle: buf[r][c] *= omega_n^((row_first + r) * c) (inverse: the inverse power). */
int gzk_swap_outer(gzk_ctx* ctx, const gzk_buf* in, size_t d0, size_t d1, size_t d2, gzk_buf* out);
int gzk_transpose(gzk_ctx* ctx, const gzk_buf* in, size_t rows, size_t cols, gzk_buf* out);
int gzk_ntt_twiddle(gzk_ctx* ctx, gzk_buf* buf, unsigned log2n, uint64_t row_first, size_t rows, size_t cols, int inverse);
/* the three values (at 0, 1, 2) of the round polynomial of the same table: what a rank
 * contributes to the per-round 3-element all-gather before the Fiat-Shamir squeeze */
int gzk_sumcheck_round_sums(gzk_ctx* ctx, const gzk_buf* table, size_t n, uint8_t out[3 * 32]);

/* ---- sharding across GPUs (one context per GPU, one process per GPU) ---------------------------
 * The reference is a single process; these entry points let the rows of a domain be
 * split over GPUs with only tiny exchanges, which the host performs (NCCL / MPI
 * all-gather of the partial results below):
 * gzk_bary_weights_range: the slice w[first .. first+count) (indices modulo n) of the
 *   barycentric weight vector; no exchange needed, the batch inversion is per slice.
 * gzk_eval_batch_range: partial sums of gzk_eval_batch over the local rows
 *   [row_offset, row_offset+len) given a weight slice starting at weights_first that
 *   covers row_offset-rot .. row_offset+len-1-rot for every rotation.
 * gzk_eval_batch_range_device: the same partial sums left in a device buffer (see
 *   gzk_eval_batch_device), ready for an all-gather between GPUs.
 * gzk_fr_sum: out[i] = sum_g values[g][i] over `groups` GPUs (host arithmetic).
 * gzk_g1_sum: sum of `count` affine points (host arithmetic): the per-GPU results of an
 *   MSM whose point range was split over the GPUs. */
int gzk_bary_weights_range(gzk_ctx* ctx, unsigned log2n, const uint8_t x[32], uint64_t first, uint64_t count, gzk_buf* out);
int gzk_eval_batch_range(gzk_ctx* ctx, gzk_buf* const* cols, size_t k_count, size_t len, uint64_t row_offset, unsigned log2n,
                         const gzk_buf* weights, uint64_t weights_first, const uint64_t* rotations, size_t p_count,
                         uint8_t* out_host);
int gzk_eval_batch_range_device(gzk_ctx* ctx, gzk_buf* const* cols, size_t k_count, size_t len, uint64_t row_offset, unsigned log2n,
                                const gzk_buf* weights, uint64_t weights_first, const uint64_t* rotations, size_t p_count,
                                gzk_buf* out, size_t out_offset);
int gzk_fr_sum(const uint8_t* values, size_t groups, size_t count, uint8_t* out);
int gzk_g1_sum(const uint8_t* points, size_t count, uint8_t out[96]);

/* ---- exchange between GPUs (one process and one context per GPU) -----------------------------------
 * The reference is a single process; this is what `--gpus N` of a multi-GPU host needs beside the
 * range entry points above.  A communicator wraps NCCL (bound at run time: libnccl.so.2) and issues
 * its collectives on the context's stream, so they are ordered with the kernels around them; data
 * always lands in the receiving GPU's own memory before a kernel of this library reads it.
 * gzk_comm_unique_id: rank 0 makes the 128-byte id and hands it to the other ranks by any host
 *   channel; gzk_comm_create: collective over all ranks.
 * gzk_comm_allgather: out[g*count .. ) = rank g's in[0 .. count) (any buffer kind; raw elements).
 * gzk_comm_allgather_fr_sum: out[i] = sum over all ranks of their in[i] mod r - the partial sums of
 *   gzk_eval_batch_range_device, combined on the device (replaces the host's gzk_fr_sum).
 * gzk_comm_alltoall: chunk g of `in` goes to rank g, chunk h of `out` comes from rank h.
 * gzk_ntt_sharded: the row-sharded forward transform of 2^log2n elements as one call (see the
 *   row-sharded transform above): `rows` = this rank's rows, result X[k1 + n1*k2] for k1 in this
 *   rank's block in `out` (Montgomery form); `work` = a second buffer of the local size.
 * gzk_comm_wait: host-side wait for everything queued on the context's stream, bounded by the
 *   communicator's time limit (gzk_comm_set_timeout, default 30 s).  When the limit runs out - a
 *   peer never joined a collective - the communicator is aborted (ncclCommAbort), the call returns
 *   GZK_E_TIMEOUT and every later exchange on this communicator fails at once; the context itself
 *   stays usable. */
typedef struct gzk_comm gzk_comm;
int gzk_comm_unique_id(uint8_t out[128]);
int gzk_comm_create(gzk_ctx* ctx, int nranks, int rank, const uint8_t unique_id[128], gzk_comm** out);
void gzk_comm_destroy(gzk_comm* comm);
int gzk_comm_set_timeout(gzk_comm* comm, double seconds);
int gzk_comm_rank(const gzk_comm* comm);
int gzk_comm_size(const gzk_comm* comm);
int gzk_comm_wait(gzk_comm* comm);
int gzk_comm_allgather(gzk_comm* comm, const gzk_buf* in, size_t count, gzk_buf* out);
int gzk_comm_allgather_fr_sum(gzk_comm* comm, const gzk_buf* in, size_t count, gzk_buf* out);
int gzk_comm_alltoall(gzk_comm* comm, const gzk_buf* in, size_t count_per_rank, gzk_buf* out);
int gzk_ntt_sharded(gzk_comm* comm, const gzk_buf* rows, unsigned log2n, gzk_buf* work, gzk_buf* out);

/* ---- generated public columns; carry of a sharded running sum ---------------------------------
 * gzk_generated_column: columns the reference materialises on the host although they are
 * pure functions of the row index: what = 0 selector (1 for i < valid, build_selector,
 * src/protocol/lookup.cpp:75-81), 1 index i, 2 i / width, 3 i % width (the row-id /
 * column-id columns of the feature domain, src/protocol/prover.cpp:2794-2867); zero
 * beyond `valid`; out is a U32 or I64 column.
 * gzk_fr_add_scalar: buf[offset .. offset+count) += scalar: applies the carry (sum of the
 * totals of the lower ranks) to a running-sum column whose rows are split over GPUs. */
int gzk_generated_column(gzk_ctx* ctx, int what, size_t valid, size_t width, size_t domain_size, gzk_buf* out);
int gzk_fr_add_scalar(gzk_ctx* ctx, gzk_buf* buf, size_t offset, size_t count, const uint8_t scalar[32]);

/* ---- packed evaluation without any allocation ------------------------------------
 * No counterpart in the reference.  Same result as gzk_eval_batch, for callers that
 * cannot call cudaMalloc while they run: a prover host that has already given all
 * HBM to its own column pool (an allocation would fail), or one that cannot accept
 * the device-wide synchronisation an allocation implies in the middle of a proof.
 * Nothing is allocated or freed here, by CUDA or by any library: the work area is a
 * fixed ~2.1 MiB array inside the library image, resident on every GPU that loads
 * the library until the process exits.
 *  - limits: k_count <= 256 columns and p_count <= 2 rotations per call; larger
 *    requests are rejected with GZK_E_INVALID and a message in `err`.
 *  - col_ptrs / col_kinds: HOST arrays of k_count DEVICE pointers and their
 *    GZK_KIND_*; weights_mont: device pointer to n Montgomery-form weights (what
 *    gzk_bary_weights writes); out_device: device pointer to p_count*k_count*32
 *    bytes, receives canonical Fr values [p][k].  Work is queued on `stream`
 *    (a cudaStream_t; NULL = default stream) on `device`, which is made current;
 *    the results are complete once the caller has synchronised that stream.
 *  - the first call on each device also looks up the device address of the array
 *    and the SM count; make that first call before starting any stream capture.
 *  - all calls on a device share the one array, which keeps whatever the previous
 *    call left in it.  The call clears the one word that must start at zero (its
 *    status word) on `stream` before the kernels; every other slot a call reads it
 *    has written itself first.  Two calls that overlap on the GPU (different streams,
 *    or different host threads) race on the array: serialise them.
 *  - pointers are checked before anything is launched: field-element columns, the
 *    weights and out_device must be 32-byte aligned, I64 columns 8-byte, U32 columns
 *    4-byte aligned, and all must be device memory of `device`; otherwise
 *    GZK_E_INVALID and nothing runs.
 *  - device-side failure: if a bounded wait inside the kernel gives up (GZK_E_TIMEOUT
 *    in gzk_eval_batch), this entry point has no host-side result to put a code in -
 *    it returns when the work is queued - so every one of the call's outputs is set
 *    to 32 bytes of 0xFF, which is not a canonical field element.  A caller that
 *    reads 0xFF..FF from out_device must treat the whole call as failed.
 *  - err / err_cap: optional buffer for a failure message. */
int gzk_eval_batch_static(int device, void* stream, const void* const* col_ptrs, const int* col_kinds, size_t k_count,
                          size_t len, unsigned log2n, const void* weights_mont, const uint64_t* rotations,
                          size_t p_count, void* out_device, char* err, size_t err_cap);

#ifdef __cplusplus
}
#endif
#endif
