/* gatzk_b200_flow.h — C entry points of libgatzk_b200_flow.so: the commit + prove flow of the
 * multi-head GAT prover (project_b200/host/prover_flow.hpp) driven over libgatzk_b200.so.
 *
 * The flow is the host orchestration of one proof: forward pass and quantised witness of every
 * attention head, the column builders, the commit barriers chained by the Fiat-Shamir
 * transcript, and the evaluations of the prove phase.  It mirrors build_multihead_trace
 * (src/protocol/trace.cpp:2110-4270) and the multi-head branch of prove
 * (src/protocol/prover.cpp:3050-3398) on a model, graph and feature matrix handed over as
 * plain arrays; benchmarks and parity tests call it through these functions.
 *
 * All functions return 0 on success; gzk_flow_error() gives the message of the last failure
 * on the calling thread. */
#ifndef GATZK_B200_FLOW_H
#define GATZK_B200_FLOW_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gzk_flow gzk_flow;

typedef struct gzk_flow_config
{
    uint64_t node_count, feature_count, class_count, edge_count;
    uint64_t hidden_layer_count;
    const uint64_t* hidden_heads;     /* heads per hidden layer */
    const uint64_t* hidden_head_dim;  /* output width of a head, per hidden layer */
    uint64_t output_heads;
    uint32_t range_bits;              /* size of the range table: 2^range_bits (config key range_bits) */
    uint64_t seed;                    /* KZG::setup: tau = seed + 17 (src/crypto/kzg.cpp:378) */
    const double* features;           /* node_count x feature_count, row-major */
    const uint32_t* edge_src;         /* edge_count endpoints, edges sorted by destination, one self loop per node */
    const uint32_t* edge_dst;
    /* model parameters, one block per head, hidden heads in layer order then output heads:
     * seq_kernel (input_dim x width, row-major), attn_src (width), attn_dst (width),
     * attn_src_bias, attn_dst_bias, output_bias (width; used by output heads only) */
    const double* params;
    uint64_t param_count;
    const uint8_t* generator;         /* affine G1 generator, 96 bytes (x || y, little-endian) */
    /* not zero: edge-domain columns are stored as prefixes (the rows that carry data; a running sum up to
     * its final value, which the remaining rows repeat) instead of whole-domain vectors.  The committed
     * polynomials and the proof are the same; memory drops from (columns x domain size) to
     * (columns x edge count), which is what lets the 169k-node configuration (edge domain 2^26, about
     * 300 opened edge columns) run on one device.  The reference stores whole-domain vectors
     * (0.3-0.65 TB of host memory at that size).  Not combinable with gzk_flow_set_msm_commit. */
    uint32_t compact_columns;
} gzk_flow_config;

const char* gzk_flow_error(void);
/* Prepares everything that depends only on the key, the graph, the tables and the model
 * parameters (domains, weights at tau, public and static commitments): the reference's
 * build_context (src/protocol/prover.cpp:2579-3030). */
int gzk_flow_create(int device, const gzk_flow_config* config, gzk_flow** out);
void gzk_flow_destroy(gzk_flow* flow);
/* One commit + prove pass from the host inputs; everything witness-dependent is recomputed.
 * gzk_flow_prove_resident does the same with the feature matrix already on the device (uploaded
 * when the flow was created) instead of uploading it again. */
int gzk_flow_prove(gzk_flow* flow);
int gzk_flow_prove_resident(gzk_flow* flow);
/* Honest-prover commitments.  The reference commits with the trapdoor: [p(tau)] G from the scalar
 * p(tau) (src/crypto/kzg.cpp:402-419).  With the switch on, every later proof run ALSO commits each
 * column as a multi-scalar multiplication against a resident structured reference string (the
 * Lagrange basis [L_i(tau)] G of its domain; the monomial basis [tau^i] G for the matrices, which are
 * coefficient polynomials) and compares the point with the trapdoor one.  counts (optional) receives
 * the number of commitments checked so far and the number of mismatches. */
int gzk_flow_set_msm_commit(gzk_flow* flow, int on, uint64_t counts[2]);
/* Text listing of the last proof run, one value per line (challenges, tau-evaluations,
 * commitments, quotient scalars, opened values, witnesses, external evaluations, witness
 * scalars): returns the length; copies at most cap bytes. */
size_t gzk_flow_dump(gzk_flow* flow, char* out, size_t cap);
/* The proof as bytes in the layout proof_size_bytes counts (src/protocol/prover.cpp:3831-3905). */
size_t gzk_flow_proof_bytes(gzk_flow* flow, uint8_t* out, size_t cap);
/* counters of the last run: commit barriers, challenges, dynamic commitments, opened columns,
 * the seven domain sizes FH, edge, in, d, cat, C, N, the bytes uploaded to and downloaded from the
 * backend during the run, and the number of forward-pass values found within the guard band of a
 * rounding boundary (when not zero the forward pass was repeated on the host, see
 * gzk_quantize_guarded) */
int gzk_flow_stats(gzk_flow* flow, uint64_t out[14]);
/* A committed column of the last run by label: its buffer kind (GZK_KIND_*), stored length and,
 * when out is not NULL, its first min(length, cap_elements) elements in the wire format of
 * gzk_buf_download. */
int gzk_flow_column(gzk_flow* flow, const char* label, int* kind, uint64_t* length, void* out, size_t cap_elements);
/* Row check of the quotient numerators of the last proof run (src/protocol/quotients.cpp:311-1303 as restated
 * in the flow): a constraint must vanish on every row of its domain when it reads the committed columns
 * themselves (rows i and i+1; L_0 and L_{n-1} become the indicators of the first and the last row).  Checked are
 * the constraints that the witness of the reference's own builders satisfies (not those that tie quantised values
 * to exact arithmetic, the LogUp steps of accumulators the builders cut short, the source route; a running sum's
 * step is not checked across the wrap-around).  out[d] = rows of domain d (FH, edge, in, d, cat, C, N) on which a
 * checked constraint does not vanish; failures (optional) receives up to cap
 * triples (domain index, index of the constraint in the order the reference adds them, rows it failed on), count
 * their number.  Reads every column back: a diagnostic for small models. */
int gzk_flow_constraint_violations(gzk_flow* flow, uint64_t out[7], uint64_t* failures, size_t cap, size_t* count);
/* Honest quotient of one domain of the last proof run (a diagnostic: the reference commits t_D = N(tau)/Z(tau) by
 * the trapdoor and never divides a polynomial, src/protocol/prover.cpp:3076-3160).  Every column the domain's
 * numerator reads is interpolated (gzk_ntt, inverse) and evaluated on the domain of n << log2_blowup points
 * (gzk_ntt, forward); the numerator of the constraint classes in `classes` (bit 0: constraints that vanish on every
 * row, bit 1: those that vanish except across the wrap-around, bit 2: those the reference's own witness does not
 * satisfy) is formed pointwise, transformed to coefficients and divided by X^n - 1: N = t (X^n - 1) + R.
 * out: n, points, degree of N, rows on which R does not vanish, 1 when t(x)(x^n - 1) + R(x) equals the numerator
 * formed directly at a point x outside the domains (0: the blow-up is too small for the degree), degree of t.
 * log2_blowup 1..4, at most 2^22 points; the pointwise part runs on the host: for small models. */
int gzk_flow_honest_quotient(gzk_flow* flow, const char* domain, unsigned log2_blowup, unsigned classes, uint64_t out[6]);
/* newline-separated labels of the opened columns of a domain ("FH", "edge", "in", "d", "cat", "C", "N") */
size_t gzk_flow_domain_labels(gzk_flow* flow, const char* domain, char* out, size_t cap);
/* the gzk_ctx the flow issues its work on (for gzk_timing_* and stream queries) */
void* gzk_flow_context(gzk_flow* flow);
/* The further contexts of the same GPU the flow deals independent chains of short calls over (the
 * indexed accumulators of one commit barrier): index 0, 1, ...; NULL past the last one.  Their kernel
 * families and launch counts are kept per context like those of the main one. */
void* gzk_flow_side_context(gzk_flow* flow, size_t index);
/* Test hook (no counterpart in the reference): while on, every device buffer the flow allocates is
 * filled with a byte pattern first, so a builder that reads a row nobody wrote gives a wrong proof
 * deterministically instead of depending on what the memory held before. */
void gzk_flow_debug_poison_allocations(int on);

#ifdef __cplusplus
}
#endif
#endif
