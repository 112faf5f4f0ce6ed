// Commit + prove flow of the multi-head GAT prover over an abstract compute backend.
//
// This is the host orchestration that sits ABOVE the hot path: which data-parallel leaf runs
// when, on which columns, and how the Fiat-Shamir transcript chains the commit barriers.  It
// follows the reference's build_multihead_trace (src/protocol/trace.cpp:2110-4270) and the
// multi-head branch of prove (src/protocol/prover.cpp:3050-3398): one transcript for the whole
// proof, heads in transcript order, per hidden head the barrier groups of trace.cpp:2392-2414
// (16 columns), :2454-2459 (H_star), :2774-2823 (43 columns), :3023-3046 (17) and :3047-3058 (5),
// the layer concatenation of :3076-3133, the output heads of :3185-3650 and the final challenges
// of :4241-4257; then the quotient scalars from the evaluations at {tau, omega*tau}
// (src/protocol/quotients.cpp:311-1303) and, after the quotient commitments, the evaluation of every
// opened column at {z, omega*z} per domain with the quotients' own values there.  Labels and challenge names are those of
// src/protocol/challenges.cpp:138-309, 396-507 and src/protocol/schema.cpp.
//
// All O(domain) work goes through `Backend`; this file only does O(#columns) scalar glue.  The
// same flow runs over the GPU backend (libgatzk_b200.so) and, in tests and in the CPU baseline,
// over a CPU backend, so that the two can be compared value by value.
//
// Deliberate differences from the reference, all in host glue outside the hot path:
//  - the G1 generator is an input and points are serialised by a local 48-byte encoding (the
//    reference takes both from the mcl library: src/crypto/kzg.cpp:383, src/crypto/curve.cpp:63-73);
//  - a quotient numerator reads only the running columns at a rotated point, so only those are
//    evaluated at omega*tau and at omega^2*z (prover_flow_quotients.hpp); the reference evaluates every
//    dependency label at every point, which changes no value of the proof;
//  - public and static columns are limited to those the transcript absorbs and the builders read
//    (ids, endpoints, selectors, tables, model parameters).
#pragma once

#include <algorithm>
#include <array>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <set>
#include <stdexcept>
#include <string>
#include <thread>
#include <utility>
#include <vector>

#include "host_forward.hpp"
#include "proof_codec.hpp"

namespace gatzk_flow
{
    using Fe = std::array<std::uint8_t, 32>;   // canonical little-endian Fr
    using G1 = std::array<std::uint8_t, 96>;   // affine x || y, little-endian; all zero = infinity

    // buffer kinds, numbered as in the C ABI
    enum Kind : int { kFr = 0, kFrMont = 1, kI64 = 2, kU32 = 3, kF64 = 4, kG1 = 5 };

    struct Col
    {
        virtual ~Col() = default;
        std::size_t count = 0;
        int kind = kFr;
    };
    using ColP = std::shared_ptr<Col>;

    struct HeadDesc
    {
        ColP features;  // node_count x input_width, F64
        std::size_t input_width = 0, output_width = 0;
        ColP seq_kernel, attn_src, attn_dst, output_bias;  // F64; output_bias may be null
        double attn_src_bias = 0.0, attn_dst_bias = 0.0;
        bool apply_activation = false;
    };
    struct GraphCols
    {
        std::size_t node_count = 0, edge_count = 0, incoming_count = 0;
        ColP edge_src, edge_dst, incoming_ptr, incoming_src;  // U32
    };
    struct HeadTraceCols
    {
        ColP H_prime, E_src, E_dst, M, Sum, inv, S, Z, Delta, U, alpha, H_agg_pre_bias, H_agg;  // F64
    };

    // One running-sum column to build: the arguments of Backend::logup / route_node / route_edge /
    // zkmap / group_prefix_state, so that independent ones can be handed over together.
    struct ScanJob
    {
        enum Op : int { kLogup = 0, kRouteNode = 1, kRouteEdge = 2, kZkmap = 3, kGroupPrefix = 4 };
        int op = kLogup;
        ColP c0, c1, c2, c3, c4;
        std::size_t count = 0, domain_size = 0;
        Fe beta{};
        ColP out;
        // kLogup of a lookup into a banded static table: the integer keys of the queries and the shape of the
        // table, for backends that fetch the inverses from the table instead of inverting every row
        ColP key_x, key_y, table_y;
        std::int64_t x_min = 0;
        std::size_t band = 0, table_size = 0;
    };

    // The compute backend: every call is one data-parallel leaf of the hot path.
    class Backend
    {
    public:
        virtual ~Backend() = default;
        // host scalar arithmetic: 0 add, 1 sub, 2 mul, 3 inverse of a
        virtual Fe fr_op(int op, const Fe& a, const Fe& b) = 0;
        virtual Fe root_of_unity(std::uint64_t size) = 0;
        // buffers
        virtual ColP alloc(int kind, std::size_t count) = 0;
        virtual void upload(const ColP& col, const void* host, std::size_t count) = 0;
        virtual void download(const ColP& col, std::size_t offset, std::size_t count, void* host) = 0;
        virtual void zero(const ColP& col) = 0;
        virtual void copy_block(const ColP& src, std::size_t src_offset, std::size_t src_stride, const ColP& dst, std::size_t dst_offset,
                                std::size_t dst_stride, std::size_t rows, std::size_t width) = 0;
        // a10: forward pass and witness leaves
        virtual void head_forward(const HeadDesc& head, const GraphCols& graph, const HeadTraceCols& out) = 0;
        virtual void quantize(const ColP& values, std::size_t count, const ColP& out) = 0;
        // quantize + count (added to flagged[0], a U32 buffer) of the values within `guard` of a rounding
        // boundary; a backend whose forward pass IS the reference's host loop has nothing to flag
        virtual void quantize_guarded(const ColP& values, std::size_t count, double guard, const ColP& out, const ColP& flagged)
        {
            (void)guard;
            (void)flagged;
            quantize(values, count, out);
        }
        virtual void gather(const ColP& node_values, std::size_t node_count, const ColP& index, std::size_t edge_count, std::size_t domain_size,
                            const ColP& out) = 0;
        virtual void linear_combination(const std::vector<ColP>& cols, const std::vector<Fe>& coefficients, std::size_t count,
                                        std::size_t domain_size, const ColP& out) = 0;
        virtual void mul_columns(const ColP& left, const ColP& right, std::size_t count, std::size_t domain_size, const ColP& out) = 0;
        virtual void linear_form_rows(const ColP& matrix, std::size_t rows, std::size_t cols, const ColP& powers, const ColP& out) = 0;
        virtual void powers(const Fe& challenge, std::size_t count, const ColP& out) = 0;
        virtual void lookup_multiplicity(const ColP& x, const ColP& y, std::size_t count, std::int64_t x_min, std::size_t band, const ColP& table_y,
                                         std::size_t table_size, std::size_t domain_size, const ColP& out) = 0;
        virtual void first_zero_marker(const ColP& delta, const ColP& group_begin, const ColP& group_end, std::size_t groups, std::size_t domain_size,
                                       const ColP& out) = 0;
        // a7 / a8 / a9: running sums
        virtual void logup(const ColP& table, const ColP& query, const ColP& multiplicity, const ColP& q_table, const ColP& q_query, std::size_t n,
                           const Fe& beta, std::size_t active_count, const ColP& out) = 0;
        virtual void route_node(const ColP& table, const ColP& multiplicity, std::size_t valid, std::size_t domain_size, const Fe& beta,
                                const ColP& out) = 0;
        virtual void route_edge(const ColP& query, std::size_t valid, std::size_t domain_size, const Fe& beta, const ColP& out) = 0;
        virtual void group_prefix_state(const ColP& values, const ColP& q_new, std::size_t n, const ColP& out) = 0;
        virtual void zkmap(const ColP& a, const ColP& b, std::size_t count, std::size_t domain_size, const ColP& out) = 0;
        // independent running sums of one phase; a backend may run them in one launch
        virtual void running_sums_batch(const std::vector<ScanJob>& jobs)
        {
            for (const auto& j : jobs)
            {
                switch (j.op)
                {
                case ScanJob::kLogup: logup(j.c0, j.c1, j.c2, j.c3, j.c4, j.domain_size, j.beta, j.count, j.out); break;
                case ScanJob::kRouteNode: route_node(j.c0, j.c1, j.count, j.domain_size, j.beta, j.out); break;
                case ScanJob::kRouteEdge: route_edge(j.c0, j.count, j.domain_size, j.beta, j.out); break;
                case ScanJob::kZkmap: zkmap(j.c0, j.c1, j.count, j.domain_size, j.out); break;
                default: group_prefix_state(j.c0, j.c1, j.domain_size, j.out); break;
                }
            }
        }
        // a2 / a9: weights and row folds
        virtual void bary_weights(unsigned log2n, const Fe& x, const ColP& out) = 0;
        // weights of one domain at several points; a backend may compute them side by side
        virtual void bary_weights_multi(unsigned log2n, const std::vector<Fe>& xs, const std::vector<ColP>& outs)
        {
            for (std::size_t i = 0; i < xs.size(); ++i) bary_weights(log2n, xs[i], outs[i]);
        }
        // the same when only the first `keep` weights and the last two will be read (every column of the domain is a
        // prefix of at most `keep` rows); a backend may leave the other entries unwritten
        virtual void bary_weights_prefix(unsigned log2n, const Fe& x, std::size_t keep, const ColP& out)
        {
            (void)keep;
            bary_weights(log2n, x, out);
        }
        virtual void fold_rows(const ColP& matrix, std::size_t rows, std::size_t cols, const ColP& weights, std::size_t row_count, const ColP& out) = 0;
        // a3 / a4 / a5 / a6 / a11: evaluation and commitment; results stay in backend buffers
        virtual void eval_device(const std::vector<ColP>& cols, std::size_t len, unsigned log2n, const ColP& weights,
                                 const std::vector<std::uint64_t>& rotations, const ColP& out, std::size_t out_offset) = 0;
        virtual void horner_device(const ColP& matrix, std::size_t rows, std::size_t cols, const Fe& x, const ColP& out, std::size_t out_offset) = 0;
        virtual void g1_fixed_base(const G1& base, const ColP& scalars, std::size_t count, const ColP& out_points) = 0;
        // weights: those of the whole 2^log2n domain at a point z; rotation r gives the sums at omega^r * z
        virtual void fh_public_eval(const ColP& features, std::size_t rows, std::size_t feature_count, const ColP& abs_ids, const ColP& weights,
                                    unsigned log2n, std::uint64_t rotation, Fe out[5]) = 0;
        virtual void synchronize() = 0;
        // Number-theoretic transform of a host vector in place (length a power of two; natural order; forward:
        // out[j] = sum_i in[i] omega^(ij) with omega = root_of_unity(length); inverse undoes it).  Only the
        // honest-quotient diagnostic calls it.
        virtual void transform(std::vector<Fe>& data, bool inverse) = 0;
        virtual void transform_many(std::vector<std::vector<Fe>>& vectors, bool inverse)
        {
            for (auto& v : vectors) transform(v, inverse);
        }
        // Honest-prover commitment by multi-scalar multiplication (optional): structured reference strings
        // [L_i(tau)] G of a domain / [tau^i] G, the resident table of shifted bases of such a point set,
        // and sum_i scalars[i] * P_i against it.  `scalars` is a field-element column (kFr / kFrMont).
        virtual bool supports_msm() const { return false; }
        // the backend's running_sums_batch takes kLogup jobs without a packed query column (c1 null) when the
        // job carries the integer keys and the shape of the banded table
        virtual bool supports_indexed_logup() const { return false; }
        virtual ColP srs_lagrange(unsigned, const G1&, const Fe&) { throw std::runtime_error("this backend has no MSM commitment path"); }
        virtual ColP msm_table(const ColP&, std::size_t, unsigned*) { throw std::runtime_error("this backend has no MSM commitment path"); }
        virtual G1 msm(const ColP&, const ColP&, std::size_t, unsigned) { throw std::runtime_error("this backend has no MSM commitment path"); }
        // bytes moved between host and backend since the last reset (end-to-end accounting)
        std::uint64_t uploaded_bytes = 0, downloaded_bytes = 0;
    };

    // ---- host scalars -------------------------------------------------------------------------
    inline Fe fe_u64(std::uint64_t v)
    {
        Fe out{};
        std::memcpy(out.data(), &v, 8);
        return out;
    }
    inline bool fe_is_zero(const Fe& a) { return std::all_of(a.begin(), a.end(), [](std::uint8_t b) { return b == 0; }); }

    // decimal string of a canonical value (what FieldElement::to_string gives, include/gatzk/algebra/field.hpp:182-185)
    inline std::string fe_to_decimal(const Fe& a)
    {
        std::uint32_t limbs[8];
        std::memcpy(limbs, a.data(), 32);
        std::string digits;
        bool any = true;
        while (any)
        {
            std::uint64_t rem = 0;
            any = false;
            for (int i = 7; i >= 0; --i)
            {
                const std::uint64_t cur = (rem << 32) | limbs[i];
                limbs[i] = static_cast<std::uint32_t>(cur / 1000000000ULL);
                rem = cur % 1000000000ULL;
                if (limbs[i] != 0) any = true;
            }
            std::string chunk = std::to_string(rem);
            if (any) chunk = std::string(9 - chunk.size(), '0') + chunk;
            digits = chunk + digits;
        }
        return digits;
    }

    // Local 48-byte encoding of a G1 point for the transcript and the proof stream: x little-endian,
    // bit 7 of the last byte = lowest bit of y, bit 6 alone = infinity.  (The reference uses the mcl
    // library's own serialisation, which is not available here.)
    inline gatzk_b200::protocol::PointBytes point_bytes(const G1& p)
    {
        gatzk_b200::protocol::PointBytes out{};
        if (std::all_of(p.begin(), p.end(), [](std::uint8_t b) { return b == 0; }))
        {
            out[47] = 0x40;
            return out;
        }
        std::memcpy(out.data(), p.data(), 48);
        if (p[48] & 1U) out[47] |= 0x80;
        return out;
    }

    // src/crypto/transcript.cpp:10-55
    class Transcript
    {
    public:
        explicit Transcript(const std::string& label) { append(label); }
        void absorb_scalar(const std::string& label, const Fe& value)
        {
            append("|");
            append(label);
            append("=");
            append(fe_to_decimal(value));
        }
        void absorb_commitment(const std::string& label, const G1& point)
        {
            append("|");
            append(label);
            append("=");
            static const char kHex[] = "0123456789abcdef";
            char hex[2 * sizeof(G1)];
            std::size_t n = 0;
            for (const auto byte : point_bytes(point))
            {
                hex[n++] = kHex[(byte >> 4U) & 0x0FU];
                hex[n++] = kHex[byte & 0x0FU];
            }
            append(std::string(hex, n));
        }
        // FNV-1a of everything absorbed so far followed by "|label|count".  The hash is a byte-serial
        // recurrence, so the digest of the absorbed text is carried along instead of the text: a
        // challenge costs its own few bytes, not a pass over the whole history.
        Fe challenge(const std::string& label)
        {
            const auto hash = fnv1a("|" + label + "|" + std::to_string(issued_), digest_);
            ++issued_;
            const Fe value = fe_u64(hash);
            absorb_scalar(label, value);
            return value;
        }
        static constexpr std::uint64_t kFnvOffset = 1469598103934665603ULL;
        static std::uint64_t fnv1a(const std::string& data, std::uint64_t hash = kFnvOffset)
        {
            for (const unsigned char ch : data)
            {
                hash ^= ch;
                hash *= 1099511628211ULL;
            }
            return hash;
        }

    private:
        void append(const std::string& text) { digest_ = fnv1a(text, digest_); }
        std::uint64_t digest_ = kFnvOffset;
        std::size_t issued_ = 0;
    };

    // ---- model, graph and configuration ---------------------------------------------------------
    struct HeadParams
    {
        std::vector<double> seq_kernel;  // input_dim x output_dim, row-major
        std::vector<double> attn_src, attn_dst, output_bias;
        double attn_src_bias = 0.0, attn_dst_bias = 0.0;
    };
    struct LayerParams
    {
        std::size_t input_dim = 0, head_dim = 0;
        std::vector<HeadParams> heads;
    };
    struct FlowInputs
    {
        std::size_t node_count = 0, feature_count = 0, class_count = 0;
        std::vector<double> features;                 // node_count x feature_count
        std::vector<std::uint32_t> edge_src, edge_dst;  // sorted by destination, one self loop per node
        std::vector<LayerParams> hidden_layers;
        LayerParams output_layer;                     // head_dim = class_count
        unsigned range_bits = 12;
        std::uint64_t seed = 11;
        G1 generator{};
        std::string dataset_name = "synthetic";
        // Store the edge-domain columns as prefixes: the rows that carry data, plus for a running sum the
        // constant it stays at afterwards (see ProverFlow::ColumnEntry).  Same polynomials, same proof;
        // the only way the 169k-node configuration (edge domain 2^26, about 300 opened edge columns)
        // fits the memory of one device.
        bool compact_columns = false;
    };

    struct Commitment
    {
        G1 point{};
        Fe tau_evaluation{};
    };

    struct FlowStats
    {
        std::size_t commit_barriers = 0, challenges = 0, dynamic_commitments = 0, opened_columns = 0;
        std::size_t guard_flags = 0;  // forward-pass values within the guard band of a rounding boundary (host re-check ran when > 0)
    };

    // Guard band of the quantisation, in units of 16*v: the forward pass on the GPU equals the host's bit
    // for bit up to exp / expm1 (relative difference <= 2^-51 per call); sums of at most 2^20 such terms,
    // values below 2^9 and two layers of amplification by at most 2^10 each keep |16 v_gpu - 16 v_host|
    // far below 2^-30, so a value outside the band rounds the same way on both sides.
    constexpr double kQuantizeGuard = 1.0 / 1073741824.0;

    inline std::size_t next_power_of_two(std::size_t v)
    {
        std::size_t p = 1;
        while (p < v) p <<= 1;
        return p;
    }
    inline unsigned log2_of(std::size_t pow2)
    {
        unsigned l = 0;
        while ((static_cast<std::size_t>(1) << l) < pow2) ++l;
        return l;
    }
    // trace.cpp:973-976 / prover.cpp:468-475
    inline std::int64_t quantize_value(double value) { return static_cast<std::int64_t>(value >= 0.0 ? value * 16.0 + 0.5 : value * 16.0 - 0.5); }

    struct Domain
    {
        std::string name;
        std::size_t size = 0;
        unsigned log2n = 0;
        Fe omega{};
        ColP w_tau;  // barycentric weights at tau, resident (the reference caches them per key: kzg.cpp:118-146)
    };

    // ---- the flow ----------------------------------------------------------------------------------
    class ProverFlow
    {
    public:
        ProverFlow(Backend& backend, FlowInputs inputs) : be_(backend), in_(std::move(inputs)) { setup(); }

        // One commit + prove pass from the host inputs (features, parameters, graph).  Nothing that
        // depends on the witness is reused between calls.  inputs_resident: the fp64 feature matrix is
        // taken from the copy uploaded at set-up instead of being uploaded again.
        void prove(bool inputs_resident = false);

        const gatzk_b200::protocol::Proof& proof() const { return proof_; }
        const std::vector<std::pair<std::string, Fe>>& challenges() const { return challenge_log_; }
        const std::vector<std::pair<std::string, Fe>>& tau_evaluations() const { return tau_eval_log_; }
        const std::vector<std::pair<std::string, Fe>>& quotient_scalars() const { return quotient_log_; }
        const FlowStats& stats() const { return stats_; }
        const FlowInputs& inputs() const { return in_; }
        // Commit every column ALSO as an MSM against the resident SRS (Lagrange basis of its domain, monomial
        // basis for the matrices) and compare the point with the trapdoor commitment [p(tau)] G: the honest
        // prover's commitment path.  The SRS tables are built on first use and stay resident.
        void set_msm_commit(bool on) { msm_commit_ = on; }
        std::size_t msm_commitments() const { return msm_checked_; }
        std::size_t msm_mismatches() const { return msm_mismatches_; }
        std::size_t domain_size(const std::string& name) const { return dom_.at(name).size; }
        // a column of the last proof by label (tests compare a few against the CPU restatement)
        std::vector<std::uint64_t> constraint_violations(std::vector<std::array<std::uint64_t, 3>>* first_failures = nullptr);
        std::array<std::uint64_t, 6> honest_quotient(const std::string& domain, unsigned log2_blowup, unsigned classes);
        ColP column(const std::string& label, std::size_t* length = nullptr) const
        {
            const auto it = columns_.find(label);
            if (it == columns_.end()) return nullptr;
            if (length != nullptr) *length = it->second.length;
            return it->second.col;
        }
        std::vector<std::string> domain_labels(const std::string& domain) const
        {
            const auto it = opened_.find(domain);
            return it == opened_.end() ? std::vector<std::string>{} : it->second;
        }

    private:
        struct ColumnEntry
        {
            ColP col;
            std::string domain;
            std::size_t length = 0;  // stored prefix; beyond it the column is zero, or `tail` when const_tail
            bool const_tail = false;
            Fe tail{};               // the column's value on rows length .. domain size - 1 (its last stored element)
            // a column that is a fixed linear combination of other opened columns of its domain (the packed
            // table / query columns of a lookup): its value at any point is that combination of theirs
            std::vector<std::pair<std::string, Fe>> derived_from;
        };
        struct CommitItem
        {
            std::string label;
            bool matrix = false;
            ColP col;
            std::string domain;       // columns
            std::size_t length = 0;   // columns: valid prefix; matrices: rows * cols
            std::size_t rows = 0, cols = 0;
            bool opened = true;       // matrices are commitment-only
            bool const_tail = false;  // rows beyond `length` repeat the last stored element (a running sum after its last term)
            std::vector<std::pair<std::string, Fe>> derived_from;  // see ColumnEntry
        };

        // scalar helpers
        Fe add(const Fe& a, const Fe& b) { return be_.fr_op(0, a, b); }
        Fe sub(const Fe& a, const Fe& b) { return be_.fr_op(1, a, b); }
        Fe mul(const Fe& a, const Fe& b) { return be_.fr_op(2, a, b); }
        Fe inv(const Fe& a) { return be_.fr_op(3, a, a); }
        Fe pow(Fe base, std::uint64_t e)
        {
            Fe out = fe_u64(1);
            while (e != 0)
            {
                if (e & 1U) out = mul(out, base);
                base = mul(base, base);
                e >>= 1U;
            }
            return out;
        }
        Fe from_signed(std::int64_t v) { return v >= 0 ? fe_u64(static_cast<std::uint64_t>(v)) : sub(fe_u64(0), fe_u64(~static_cast<std::uint64_t>(v) + 1)); }

        ColP upload_i64(const std::vector<std::int64_t>& v, std::size_t count = 0)
        {
            ColP c = be_.alloc(kI64, std::max<std::size_t>(count, v.size()));
            if (count > v.size()) be_.zero(c);
            if (!v.empty()) be_.upload(c, v.data(), v.size());
            return c;
        }
        ColP upload_u32(const std::vector<std::uint32_t>& v, std::size_t count = 0)
        {
            ColP c = be_.alloc(kU32, std::max<std::size_t>(count, v.size()));
            if (count > v.size()) be_.zero(c);
            if (!v.empty()) be_.upload(c, v.data(), v.size());
            return c;
        }
        ColP upload_f64(const std::vector<double>& v)
        {
            ColP c = be_.alloc(kF64, std::max<std::size_t>(1, v.size()));
            if (!v.empty()) be_.upload(c, v.data(), v.size());
            return c;
        }
        ColP upload_fe(const std::vector<Fe>& v, std::size_t count)
        {
            ColP c = be_.alloc(kFr, std::max<std::size_t>(count, std::max<std::size_t>(1, v.size())));
            be_.zero(c);
            if (!v.empty()) be_.upload(c, v.data(), v.size());
            return c;
        }
        std::vector<Fe> powers_host(const Fe& base, std::size_t count)
        {
            std::vector<Fe> out(count);
            Fe cur = fe_u64(1);
            for (std::size_t i = 0; i < count; ++i)
            {
                out[i] = cur;
                cur = mul(cur, base);
            }
            return out;
        }

        void setup();
        void add_domain(const std::string& name, std::size_t size);
        Commitment commit_static(const std::string& label, const ColP& col, const std::string& domain, std::size_t length);
        Commitment commit_static_matrix(const std::string& label, const ColP& matrix, std::size_t rows, std::size_t cols);

        // a commit barrier: tau-evaluation of every item, same-base multiplication, ONE read-back
        void commit_batch(const std::vector<CommitItem>& items);
        CommitItem column_item(const std::string& label, const ColP& col, const std::string& domain, std::size_t length)
        {
            CommitItem it;
            it.label = label;
            it.col = col;
            it.domain = domain;
            it.length = length;
            return it;
        }
        // a running sum stored up to (and including) its final value
        CommitItem tail_item(const std::string& label, const ColP& col, const std::string& domain, std::size_t length)
        {
            CommitItem it = column_item(label, col, domain, length);
            it.const_tail = compact_ && length < dom_.at(domain).size;
            return it;
        }
        CommitItem matrix_item(const std::string& label, const ColP& matrix, std::size_t rows, std::size_t cols)
        {
            CommitItem it;
            it.label = label;
            it.matrix = true;
            it.col = matrix;
            it.rows = rows;
            it.cols = cols;
            it.opened = false;
            return it;
        }
        Fe challenge(Transcript& t, const std::string& name)
        {
            const Fe c = t.challenge(name);
            challenges_[name] = c;
            challenge_log_.push_back({name, c});
            ++stats_.challenges;
            return c;
        }
        void absorb_dyn(Transcript& t, const std::string& label) { t.absorb_commitment(label, commitments_.at(label).point); }
        void absorb_static(Transcript& t, const std::string& label) { t.absorb_commitment(label, static_commitments_.at(label).point); }

        // running sums are queued and handed to the backend together at the next commit barrier
        std::vector<ScanJob> scan_queue_;
        void queue_scan(int op, const ColP& c0, const ColP& c1, const ColP& c2, const ColP& c3, const ColP& c4, std::size_t count,
                        std::size_t domain_size, const Fe& beta, const ColP& out)
        {
            ScanJob j;
            j.op = op;
            j.c0 = c0;
            j.c1 = c1;
            j.c2 = c2;
            j.c3 = c3;
            j.c4 = c4;
            j.count = count;
            j.domain_size = domain_size;
            j.beta = beta;
            j.out = out;
            scan_queue_.push_back(j);
        }
        void flush_scans()
        {
            if (scan_queue_.empty()) return;
            be_.running_sums_batch(scan_queue_);
            scan_queue_.clear();
        }
        struct PendingTotal
        {
            std::string name;
            ColP column;
            std::size_t index;
        };
        std::vector<PendingTotal> pending_totals_;
        void resolve_totals()
        {
            flush_scans();
            for (const auto& p : pending_totals_)
            {
                Fe v{};
                be_.download(p.column, p.index, 1, v.data());
                witness_scalars_.push_back({p.name, v});
            }
            pending_totals_.clear();
        }

        struct Binding
        {
            ColP a, b, acc;
        };
        Binding build_binding(const ColP& matrix, std::size_t rows, std::size_t cols, const Fe& point, const ColP& parameter_values,
                              const std::string& dim_domain, ColP* weights_out = nullptr, const ColP& ready_weights = nullptr);
        // node-domain weights at the binding points drawn at one transcript stage, side by side
        std::vector<ColP> node_weights_at(const std::vector<Fe>& points)
        {
            const Domain& n = dom_.at("N");
            std::vector<ColP> outs;
            for (std::size_t i = 0; i < points.size(); ++i) outs.push_back(be_.alloc(kFrMont, n.size));
            be_.bary_weights_multi(n.log2n, points, outs);
            return outs;
        }
        struct Lookup
        {
            ColP table, query, multiplicity, acc;
            std::size_t store = 0;        // stored rows of the accumulator (and of the other columns unless table_store says otherwise)
            std::size_t table_store = 0;  // stored rows of table and multiplicity
            Fe eta{};
            bool pair = false;
        };
        Lookup build_pair_lookup(const ColP& table_x, const ColP& table_y, std::size_t table_size, std::int64_t x_min, std::size_t band,
                                 const ColP& left, const ColP& right, std::size_t valid, const Fe& eta, const Fe& beta, const ColP& q_table,
                                 const ColP& q_query);
        // The packed columns of a lookup as commit items.  Prefix-stored runs do not evaluate them: table =
        // table_x + eta * table_y and query = left + eta * right are combinations of columns that are opened
        // anyway (x_label / y_label), so their value at any point follows from those.
        CommitItem packed_item(const std::string& label, const ColP& col, std::size_t length, const Lookup& lookup, const std::string& x_label,
                               const std::string& y_label)
        {
            CommitItem it = column_item(label, col, "edge", length);
            if (compact_)
            {
                it.derived_from.push_back({x_label, fe_u64(1)});
                if (lookup.pair) it.derived_from.push_back({y_label, lookup.eta});
            }
            return it;
        }
        struct Route
        {
            ColP table, query, node_acc, edge_acc;  // the routed total is node_acc[node_count]
        };
        Route build_route(const std::vector<ColP>& node_cols, const std::vector<ColP>& edge_cols, const Fe& eta, const ColP& multiplicity,
                          const Fe& beta);
        struct HeadWitness
        {
            ColP h_prime, h_agg_pre, h_agg;                       // I64 matrices node_count x width
            ColP e_src, e_dst, m, sum, inv;                        // I64, node_count
            ColP s, z, delta, u, alpha;                            // I64, edge domain (zero tail)
            ColP e_src_edge, e_dst_edge, m_edge, sum_edge, inv_edge;
            ColP h_agg_f64;                                        // the head's fp64 output (next layer's input)
        };
        // host_input: when set, the forward pass of the head runs on the host (host_head_forward) on this
        // row-major input instead of on the backend; host_output receives the head's fp64 output
        HeadWitness run_head(const ColP& layer_input_f64, std::size_t input_dim, std::size_t width, const HeadParams& p, bool output_head,
                             const std::vector<double>* host_input = nullptr, std::vector<double>* host_output = nullptr);
        void forward_all(bool inputs_resident, bool on_host, std::vector<std::vector<HeadWitness>>& hidden_witness, std::vector<ColP>& concat_q,
                         std::vector<HeadWitness>& output_witness, std::size_t& final_width);
        ColP guard_counter_;
        void commit_hidden_head(Transcript& t, std::size_t head_index, std::size_t layer_index, std::size_t local_head, const HeadWitness& w);
        void commit_hidden_concat(Transcript& t, std::size_t layer_index, const ColP& concat_q, std::size_t width);
        void commit_output_head(Transcript& t, std::size_t head_index, const HeadWitness& w, const ColP& h_cat_q, std::size_t cat_width,
                                std::vector<ColP>* y_lin_all, std::vector<ColP>* y_all);
        void prove_openings(Transcript& t);
        Fe eval_column_at(const ColP& col, std::size_t length, const std::string& domain, const ColP& weights);

        struct SrsTable
        {
            ColP table;
            unsigned window_bits = 0;
        };
        const SrsTable& srs_for(bool monomial, const std::string& domain, std::size_t n);
        G1 msm_commit(const CommitItem& item);
        bool msm_commit_ = false;
        std::size_t msm_checked_ = 0, msm_mismatches_ = 0;
        std::map<std::pair<int, std::size_t>, SrsTable> srs_tables_;  // (0 = Lagrange of a domain size / 1 = monomial, point count)

        Backend& be_;
        FlowInputs in_;
        std::map<std::string, Domain> dom_;
        Fe tau_{};
        std::size_t n_nodes_ = 0, n_edges_ = 0;
        bool compact_ = false;
        std::size_t es_ = 0;      // stored rows of an edge-domain column: the domain size, or (compact) the data rows + 1
        ColP ones_;               // a column of ones (compact): weight of a prefix = its evaluation
        std::size_t ones_len_ = 0;
        static std::size_t round64(std::size_t v) { return (v + 63) / 64 * 64; }
        // stored rows of the columns of a lookup with `active` data rows
        std::size_t lookup_store(std::size_t active) const
        {
            return compact_ ? std::min(dom_.at("edge").size, std::max(es_, round64(active + 1))) : dom_.at("edge").size;
        }
        ColP ones_col(std::size_t length)
        {
            if (ones_len_ < length)
            {
                const std::vector<std::uint32_t> host(length, 1u);
                ones_ = upload_u32(host);
                ones_len_ = length;
            }
            return ones_;
        }
        GraphCols graph_;
        // public / static columns
        ColP ids_i64_, src_i64_, dst_i64_, src_u32_, dst_u32_, q_new_, q_edge_valid_, group_begin_, group_end_, features_q_;
        ColP src_multiplicity_, dst_multiplicity_, features_f64_;
        ColP t_range_, t_l_x_, t_l_y_, t_exp_x_, t_exp_y_, t_elu_x_, t_elu_y_;
        ColP q_tbl_l_, q_qry_l_, q_tbl_r_, q_qry_r_, q_tbl_exp_, q_qry_exp_, q_tbl_elu_, q_qry_elu_;
        std::size_t range_size_ = 0, lrelu_bound_ = 0, groups_ = 0;
        std::map<std::string, std::vector<Fe>> param_vectors_;  // quantised attn_src / attn_dst per head label
        std::map<std::string, ColP> param_matrices_;            // quantised seq_kernel per head label (I64)
        std::map<std::string, Commitment> static_commitments_;
        std::map<std::string, ColumnEntry> static_columns_;
        std::map<std::string, Fe> static_omega_tau_;  // value of a key-dependent column at omega * tau (filled by the first proof)
        Fe fh_public_tau_[5], fh_public_omega_tau_[5];
        // per-proof state
        std::map<std::string, Commitment> commitments_;
        std::vector<std::string> commitment_order_;
        std::map<std::string, ColumnEntry> columns_;
        std::map<std::string, std::vector<std::string>> opened_;  // domain -> labels in commitment order
        std::map<std::string, Fe> challenges_;
        std::vector<std::pair<std::string, Fe>> challenge_log_, tau_eval_log_, quotient_log_;
        std::vector<std::pair<std::string, Fe>> external_evaluations_, witness_scalars_;
        std::vector<std::pair<std::string, Fe>> external_sources_;  // per external evaluation: committed label, evaluation point
        std::map<std::size_t, ColP> layer_inputs_q_;                 // quantised input matrix of hidden layer i >= 1
        // constraint numerators of the quotients (prover_flow_quotients.hpp)
        using PointValues = std::function<Fe(const std::string&, int)>;
        std::vector<std::string> rotated_labels(const std::string& domain) const;
        Fe quotient_numerator(const std::string& domain, const PointValues& at, const Fe& first, const Fe& last);
        std::map<std::string, std::vector<Fe>> domain_cells(const std::string& domain);
        static std::string numerator_column(const std::string& label);
        unsigned term_classes_ = 7u;  // classes of constraints that enter the numerator (bit c = class c); all, except inside the honest-quotient diagnostic
        std::map<std::string, Fe> quotient_scalars_, quotient_externals_;  // witness scalars and external evaluations by name
        std::vector<std::size_t>* nonzero_terms_ = nullptr;                // row check: indices of the constraints that did not vanish
        // L_0(x) and L_{n-1}(x) of a domain (RootOfUnityDomain::lagrange_basis_eval, src/algebra/polynomial.cpp:122-127)
        std::array<Fe, 2> boundary_basis(const Domain& d, const Fe& x)
        {
            const Fe zero_eval = sub(pow(x, d.size), fe_u64(1)), scale = mul(zero_eval, inv(fe_u64(d.size)));
            const Fe last_point = inv(d.omega);
            return {mul(scale, inv(sub(x, fe_u64(1)))), mul(mul(scale, last_point), inv(sub(x, last_point)))};
        }
        void add_external(const std::string& name, const Fe& value, const std::string& label, const Fe& point)
        {
            external_evaluations_.push_back({name, value});
            external_sources_.push_back({label, point});
        }
        gatzk_b200::protocol::Proof proof_;
        FlowStats stats_;
    };

    // =================================================================================================
    inline void ProverFlow::add_domain(const std::string& name, std::size_t size)
    {
        Domain d;
        d.name = name;
        d.size = size;
        d.log2n = log2_of(size);
        d.omega = be_.root_of_unity(size);
        d.w_tau = be_.alloc(kFrMont, size);
        be_.bary_weights(d.log2n, tau_, d.w_tau);
        dom_[name] = d;
    }

    inline Fe ProverFlow::eval_column_at(const ColP& col, std::size_t length, const std::string& domain, const ColP& weights)
    {
        const ColP out = be_.alloc(kFr, 1);
        be_.eval_device({col}, length, dom_.at(domain).log2n, weights, {0}, out, 0);
        Fe v{};
        be_.download(out, 0, 1, v.data());
        return v;
    }

    inline Commitment ProverFlow::commit_static(const std::string& label, const ColP& col, const std::string& domain, std::size_t length)
    {
        Commitment c;
        c.tau_evaluation = eval_column_at(col, length, domain, dom_.at(domain).w_tau);
        const ColP scalar = upload_fe({c.tau_evaluation}, 1);
        const ColP point = be_.alloc(kG1, 1);
        be_.g1_fixed_base(in_.generator, scalar, 1, point);
        be_.download(point, 0, 1, c.point.data());
        static_commitments_[label] = c;
        static_columns_[label] = ColumnEntry{col, domain, length, false, Fe{}, {}};
        return c;
    }

    inline Commitment ProverFlow::commit_static_matrix(const std::string& label, const ColP& matrix, std::size_t rows, std::size_t cols)
    {
        Commitment c;
        const ColP scalar = be_.alloc(kFr, 1);
        be_.horner_device(matrix, rows, cols, tau_, scalar, 0);
        be_.download(scalar, 0, 1, c.tau_evaluation.data());
        const ColP point = be_.alloc(kG1, 1);
        be_.g1_fixed_base(in_.generator, scalar, 1, point);
        be_.download(point, 0, 1, c.point.data());
        static_commitments_[label] = c;
        return c;
    }

    // Everything that depends only on the key, the graph, the tables and the model parameters: what
    // the reference's build_context prepares and caches (src/protocol/prover.cpp:2579-3030).
    inline void ProverFlow::setup()
    {
        n_nodes_ = in_.node_count;
        n_edges_ = in_.edge_src.size();
        if (in_.edge_dst.size() != n_edges_ || in_.features.size() != n_nodes_ * in_.feature_count)
            throw std::runtime_error("flow: input size mismatch");
        tau_ = fe_u64(in_.seed + 17);  // KZG::setup, src/crypto/kzg.cpp:378

        // domain sizes: prover.cpp:2682-2727
        std::size_t d_h = 0, d_cat = 0, max_in = in_.feature_count;
        for (const auto& layer : in_.hidden_layers)
        {
            d_h = std::max(d_h, layer.head_dim);
            d_cat = std::max(d_cat, layer.head_dim * layer.heads.size());
            max_in = std::max(max_in, layer.input_dim);
        }
        range_size_ = static_cast<std::size_t>(1) << in_.range_bits;
        lrelu_bound_ = std::max<std::size_t>(4096, range_size_);
        const std::size_t lrelu_table_size = lrelu_bound_ * 2 + 1;
        const std::size_t elu_table_size = lrelu_table_size * 3;
        const std::size_t exp_table_size = range_size_ * 5;
        const std::size_t fh_size = next_power_of_two(n_nodes_ * in_.feature_count + 2);
        const std::size_t edge_size =
            next_power_of_two(std::max({n_nodes_, n_edges_, n_nodes_ * d_h, lrelu_table_size, elu_table_size, exp_table_size, range_size_}) + 2);
        add_domain("FH", fh_size);
        add_domain("edge", edge_size);
        compact_ = in_.compact_columns;
        es_ = compact_ ? std::min(edge_size, round64(std::max({n_nodes_, n_edges_, lrelu_table_size, elu_table_size, exp_table_size, range_size_}) + 1)) : edge_size;
        add_domain("in", next_power_of_two(max_in + 2));
        add_domain("d", next_power_of_two(d_h + 2));
        add_domain("cat", next_power_of_two(d_cat + 2));
        add_domain("C", next_power_of_two(in_.class_count + 2));
        add_domain("N", next_power_of_two(n_nodes_ + 2));
        const std::size_t n_size = dom_.at("N").size;

        // graph: endpoints, incoming lists (src/model/gat.cpp:521-538), destination groups (trace.cpp:1407-1422)
        std::vector<std::vector<std::uint32_t>> incoming(n_nodes_);
        for (std::size_t e = 0; e < n_edges_; ++e)
        {
            if (in_.edge_src[e] >= n_nodes_ || in_.edge_dst[e] >= n_nodes_) throw std::runtime_error("edge out of bounds while running attention head forward");
            incoming[in_.edge_dst[e]].push_back(in_.edge_src[e]);
        }
        std::vector<std::uint32_t> in_ptr(n_nodes_ + 1, 0), in_src;
        for (std::size_t d = 0; d < n_nodes_; ++d)
        {
            if (std::find(incoming[d].begin(), incoming[d].end(), static_cast<std::uint32_t>(d)) == incoming[d].end())
                incoming[d].push_back(static_cast<std::uint32_t>(d));
            in_src.insert(in_src.end(), incoming[d].begin(), incoming[d].end());
            in_ptr[d + 1] = static_cast<std::uint32_t>(in_src.size());
        }
        graph_.node_count = n_nodes_;
        graph_.edge_count = n_edges_;
        graph_.incoming_count = in_src.size();
        graph_.edge_src = upload_u32(in_.edge_src);
        graph_.edge_dst = upload_u32(in_.edge_dst);
        graph_.incoming_ptr = upload_u32(in_ptr);
        graph_.incoming_src = upload_u32(in_src);
        src_u32_ = graph_.edge_src;
        dst_u32_ = graph_.edge_dst;
        std::vector<std::int64_t> ids(n_nodes_), src64(n_edges_), dst64(n_edges_);
        std::vector<std::uint32_t> q_new(edge_size, 0), q_end(edge_size, 0), q_valid(edge_size, 0), gb, ge, src_mult(n_size, 0), dst_mult(n_size, 0);
        for (std::size_t i = 0; i < n_nodes_; ++i) ids[i] = static_cast<std::int64_t>(i);
        for (std::size_t e = 0; e < n_edges_; ++e)
        {
            src64[e] = in_.edge_src[e];
            dst64[e] = in_.edge_dst[e];
            q_valid[e] = 1;
            const bool starts = e == 0 || in_.edge_dst[e] != in_.edge_dst[e - 1];
            const bool ends = e + 1 == n_edges_ || in_.edge_dst[e + 1] != in_.edge_dst[e];
            if (starts)
            {
                q_new[e] = 1;
                gb.push_back(static_cast<std::uint32_t>(e));
            }
            if (ends)
            {
                q_end[e] = 1;
                ge.push_back(static_cast<std::uint32_t>(e + 1));
            }
            src_mult[in_.edge_src[e]] += 1;   // count_by_src / count_by_dst, trace.cpp:1383-1405
            dst_mult[in_.edge_dst[e]] += 1;
        }
        groups_ = gb.size();
        ids_i64_ = upload_i64(ids, n_size);
        src_i64_ = upload_i64(src64, edge_size);
        dst_i64_ = upload_i64(dst64, edge_size);
        q_new_ = upload_u32(q_new);
        q_edge_valid_ = upload_u32(q_valid);
        group_begin_ = upload_u32(gb);
        group_end_ = upload_u32(ge);
        src_multiplicity_ = upload_u32(src_mult);
        dst_multiplicity_ = upload_u32(dst_mult);

        // static tables: prover.cpp:460-535
        // A selector is zero beyond its last 1, so only that prefix has to be evaluated (prefix-stored runs; the
        // whole-domain run keeps the reference's full-length evaluation).
        auto sel_len = [&](std::size_t valid) { return compact_ ? std::min(edge_size, valid) : edge_size; };
        auto selector = [&](std::size_t valid) {
            std::vector<std::uint32_t> s(edge_size, 0);
            for (std::size_t i = 0; i < valid && i < edge_size; ++i) s[i] = 1;
            return upload_u32(s);
        };
        {
            std::vector<std::int64_t> range(range_size_), lx, ly, ex, ey, ux, uy;
            for (std::size_t i = 0; i < range_size_; ++i) range[i] = static_cast<std::int64_t>(i);
            for (std::int64_t raw = -static_cast<std::int64_t>(lrelu_bound_); raw <= static_cast<std::int64_t>(lrelu_bound_); ++raw)
            {
                const double input = static_cast<double>(raw) / 16.0;
                lx.push_back(raw);
                ly.push_back(quantize_value(input >= 0.0 ? input : 0.2 * input));
                const std::int64_t central = quantize_value(input >= 0.0 ? input : std::exp(input) - 1.0);
                for (std::int64_t offset = -1; offset <= 1; ++offset)
                {
                    ux.push_back(raw);
                    uy.push_back(central + offset);
                }
            }
            for (std::size_t i = 0; i < range_size_; ++i)
            {
                const std::int64_t central = quantize_value(std::exp(-static_cast<double>(i) / 16.0));
                for (std::int64_t offset = -2; offset <= 2; ++offset)
                {
                    ex.push_back(static_cast<std::int64_t>(i));
                    ey.push_back(std::max<std::int64_t>(0, central + offset));
                }
            }
            t_range_ = upload_i64(range, edge_size);
            t_l_x_ = upload_i64(lx, edge_size);
            t_l_y_ = upload_i64(ly, edge_size);
            t_exp_x_ = upload_i64(ex, edge_size);
            t_exp_y_ = upload_i64(ey, edge_size);
            t_elu_x_ = upload_i64(ux, edge_size);
            t_elu_y_ = upload_i64(uy, edge_size);
        }
        q_tbl_l_ = selector(lrelu_table_size);
        q_qry_l_ = selector(n_edges_);
        q_tbl_r_ = selector(range_size_);
        q_qry_r_ = selector(n_edges_);
        q_tbl_exp_ = selector(exp_table_size);
        q_qry_exp_ = selector(n_edges_);
        q_tbl_elu_ = selector(elu_table_size);
        q_qry_elu_ = selector(n_nodes_ * d_h);

        // public commitments the transcript absorbs (prover.cpp:2750-2977)
        commit_static("P_I", ids_i64_, "N", n_nodes_);
        commit_static("P_src", src_i64_, "edge", n_edges_);
        commit_static("P_dst", dst_i64_, "edge", n_edges_);
        commit_static("P_Q_new_edge", q_new_, "edge", sel_len(n_edges_));
        commit_static("P_Q_end_edge", upload_u32(q_end), "edge", sel_len(n_edges_));
        commit_static("P_Q_edge_valid", q_edge_valid_, "edge", sel_len(n_edges_));
        {
            auto valid_selector = [&](const std::string& domain, std::size_t valid) {
                std::vector<std::uint32_t> s(dom_.at(domain).size, 0);
                for (std::size_t i = 0; i < valid; ++i) s[i] = 1;
                return upload_u32(s);
            };
            commit_static("P_Q_N", valid_selector("N", n_nodes_), "N", n_size);
            commit_static("P_Q_proj_valid", valid_selector("in", max_in), "in", dom_.at("in").size);
            commit_static("P_Q_d_valid", valid_selector("d", d_h), "d", dom_.at("d").size);
            commit_static("P_Q_cat_valid", valid_selector("cat", d_cat), "cat", dom_.at("cat").size);
            commit_static("P_Q_C_valid", valid_selector("C", in_.class_count), "C", dom_.at("C").size);
        }
        commit_static("V_T_range", t_range_, "edge", range_size_);
        commit_static("V_T_L_x", t_l_x_, "edge", lrelu_table_size);
        commit_static("V_T_L_y", t_l_y_, "edge", lrelu_table_size);
        commit_static("V_T_exp_x", t_exp_x_, "edge", exp_table_size);
        commit_static("V_T_exp_y", t_exp_y_, "edge", exp_table_size);
        commit_static("V_T_ELU_x", t_elu_x_, "edge", elu_table_size);
        commit_static("V_T_ELU_y", t_elu_y_, "edge", elu_table_size);
        commit_static("P_Q_tbl_L", q_tbl_l_, "edge", sel_len(lrelu_table_size));
        commit_static("P_Q_qry_L", q_qry_l_, "edge", sel_len(n_edges_));
        commit_static("P_Q_tbl_R", q_tbl_r_, "edge", sel_len(range_size_));
        commit_static("P_Q_qry_R", q_qry_r_, "edge", sel_len(n_edges_));
        commit_static("P_Q_tbl_exp", q_tbl_exp_, "edge", sel_len(exp_table_size));
        commit_static("P_Q_qry_exp", q_qry_exp_, "edge", sel_len(n_edges_));
        commit_static("P_Q_tbl_ELU", q_tbl_elu_, "edge", sel_len(elu_table_size));
        commit_static("P_Q_qry_ELU", q_qry_elu_, "edge", sel_len(n_nodes_ * d_h));

        // model parameters, quantised as cached_quantized_*_head_parameters do (trace.cpp:1027-1139)
        auto quantise_vector = [&](const std::vector<double>& v) {
            std::vector<std::int64_t> q(v.size());
            for (std::size_t i = 0; i < v.size(); ++i) q[i] = quantize_value(v[i]);
            return q;
        };
        auto register_head = [&](const std::string& w_label, const std::string& src_label, const std::string& dst_label, const HeadParams& p,
                                 std::size_t input_dim, std::size_t width) {
            if (p.seq_kernel.size() != input_dim * width || p.attn_src.size() != width || p.attn_dst.size() != width)
                throw std::runtime_error("flow: head parameter size mismatch");
            const ColP w = upload_i64(quantise_vector(p.seq_kernel));
            param_matrices_[w_label] = w;
            commit_static_matrix(w_label, w, input_dim, width);
            for (const auto& item : {std::make_pair(src_label, &p.attn_src), std::make_pair(dst_label, &p.attn_dst)})
            {
                std::vector<Fe> values;
                for (const auto q : quantise_vector(*item.second)) values.push_back(from_signed(q));
                param_vectors_[item.first] = values;
                commit_static_matrix(item.first, upload_i64(quantise_vector(*item.second)), 1, width);
            }
        };
        std::size_t global_head = 0;
        for (const auto& layer : in_.hidden_layers)
            for (const auto& head : layer.heads)
            {
                const auto h = std::to_string(global_head++);
                register_head("V_h" + h + "_W", "V_h" + h + "_a_src", "V_h" + h + "_a_dst", head, layer.input_dim, layer.head_dim);
            }
        const bool legacy = in_.output_layer.heads.size() == 1;
        for (std::size_t k = 0; k < in_.output_layer.heads.size(); ++k)
        {
            const std::string base = legacy ? "V_out" : "V_out" + std::to_string(k);
            register_head(base + "_W", base + "_a_src", base + "_a_dst", in_.output_layer.heads[k], in_.output_layer.input_dim, in_.class_count);
        }

        // feature domain: quantised features (loader.cpp:62-64 quantises at the same scale), the table
        // commitment V_T_H and the generated public columns at tau and omega*tau (prover.cpp:1205-1675)
        {
            std::vector<std::int64_t> fq(in_.features.size());
            for (std::size_t i = 0; i < fq.size(); ++i) fq[i] = quantize_value(in_.features[i]);
            features_q_ = upload_i64(fq);
            features_f64_ = upload_f64(in_.features);
            commit_static_matrix("V_T_H", features_q_, n_nodes_, in_.feature_count);
            const Domain& fh = dom_.at("FH");
            be_.fh_public_eval(features_q_, n_nodes_, in_.feature_count, ids_i64_, fh.w_tau, fh.log2n, 0, fh_public_tau_);
            be_.fh_public_eval(features_q_, n_nodes_, in_.feature_count, ids_i64_, fh.w_tau, fh.log2n, 1, fh_public_omega_tau_);
        }
        be_.synchronize();
    }

    // KZG::commit_batch (src/crypto/kzg.cpp:458-542) as add_dynamic_commitment_batch calls it
    // (src/protocol/trace.cpp:762-902): tau-evaluations grouped by (domain, stored length), matrices by
    // Horner, all scalars multiplied onto the generator in one same-base batch, one read-back.
    inline void ProverFlow::commit_batch(const std::vector<CommitItem>& items)
    {
        if (items.empty()) return;
        flush_scans();
        // Scalars are laid out group by group (matrices first, then the columns of each (domain, stored
        // length) group), so that a group is ONE evaluation call; `slot` maps an item to its place and
        // the results are put back into label order on the host after the single read-back.
        ColP scalars = be_.alloc(kFr, items.size());
        std::map<std::pair<std::string, std::size_t>, std::vector<std::size_t>> groups;
        std::vector<std::size_t> slot(items.size());
        std::size_t next = 0;
        for (std::size_t i = 0; i < items.size(); ++i)
        {
            if (items[i].matrix)
            {
                slot[i] = next;
                be_.horner_device(items[i].col, items[i].rows, items[i].cols, tau_, scalars, next++);
            }
            else if (items[i].derived_from.empty())
            {
                groups[{items[i].domain, items[i].length}].push_back(i);
            }
        }
        // prefix-stored running sums: the rows beyond the prefix hold the column's last stored value, so
        // p(tau) = (sum over the prefix) + tail * (weight of the remaining rows), and that weight is
        // 1 - (evaluation of a column of ones over the prefix) because the weights of a domain sum to 1
        std::vector<std::size_t> tail_items;
        std::map<std::pair<std::string, std::size_t>, std::size_t> ones_slot;
        for (const auto& group : groups)
            for (const auto i : group.second)
                if (items[i].const_tail)
                {
                    tail_items.push_back(i);
                    ones_slot.emplace(group.first, ones_slot.size());
                }
        const ColP ones_out = tail_items.empty() ? nullptr : be_.alloc(kFr, ones_slot.size());
        for (const auto& group : groups)
        {
            const Domain& d = dom_.at(group.first.first);
            std::vector<ColP> cols;
            for (const auto i : group.second)
            {
                cols.push_back(items[i].col);
                slot[i] = next + cols.size() - 1;
            }
            be_.eval_device(cols, group.first.second, d.log2n, d.w_tau, {0}, scalars, next);
            next += cols.size();
            const auto ones = ones_slot.find(group.first);
            if (ones != ones_slot.end()) be_.eval_device({ones_col(group.first.second)}, group.first.second, d.log2n, d.w_tau, {0}, ones_out, ones->second);
        }
        std::vector<Fe> evals(items.size()), evals_by_slot(items.size());
        std::vector<Fe> tails(items.size());
        std::vector<std::size_t> derived_items;
        for (std::size_t i = 0; i < items.size(); ++i)
            if (!items[i].matrix && !items[i].derived_from.empty())
            {
                slot[i] = next++;
                derived_items.push_back(i);
            }
        const bool host_fix = !tail_items.empty() || !derived_items.empty();
        if (host_fix)
        {
            std::vector<Fe> ones_host(ones_slot.size());
            be_.download(scalars, 0, items.size(), evals_by_slot.data());
            if (!tail_items.empty()) be_.download(ones_out, 0, ones_host.size(), ones_host.data());
            for (const auto i : tail_items)
            {
                be_.download(items[i].col, items[i].length - 1, 1, &tails[i]);
                const Fe rest = sub(fe_u64(1), ones_host[ones_slot.at({items[i].domain, items[i].length})]);
                evals_by_slot[slot[i]] = add(evals_by_slot[slot[i]], mul(tails[i], rest));
            }
            // combinations of columns that are evaluated in this barrier, were committed earlier, or are static
            std::map<std::string, std::size_t> here;
            for (std::size_t i = 0; i < items.size(); ++i) here[items[i].label] = i;
            for (const auto i : derived_items)
            {
                Fe value = fe_u64(0);
                for (const auto& term : items[i].derived_from)
                {
                    Fe source;
                    const auto in_batch = here.find(term.first);
                    const auto earlier = commitments_.find(term.first);
                    if (in_batch != here.end())
                        source = evals_by_slot[slot[in_batch->second]];
                    else if (earlier != commitments_.end())
                        source = earlier->second.tau_evaluation;
                    else
                        source = static_commitments_.at(term.first).tau_evaluation;
                    value = add(value, mul(term.second, source));
                }
                evals_by_slot[slot[i]] = value;
            }
            scalars = upload_fe(evals_by_slot, items.size());
        }
        const ColP points = be_.alloc(kG1, items.size());
        be_.g1_fixed_base(in_.generator, scalars, items.size(), points);
        std::vector<G1> pts(items.size()), pts_by_slot(items.size());
        if (!host_fix) be_.download(scalars, 0, items.size(), evals_by_slot.data());
        be_.download(points, 0, items.size(), pts_by_slot.data());
        for (std::size_t i = 0; i < items.size(); ++i)
        {
            evals[i] = evals_by_slot[slot[i]];
            pts[i] = pts_by_slot[slot[i]];
        }
        if (msm_commit_)
        {
            if (compact_) throw std::runtime_error("flow: the MSM commitment check needs whole-domain columns (compact_columns off)");
            for (std::size_t i = 0; i < items.size(); ++i)
            {
                ++msm_checked_;
                if (msm_commit(items[i]) != pts[i]) ++msm_mismatches_;
            }
        }
        for (std::size_t i = 0; i < items.size(); ++i)
        {
            commitments_[items[i].label] = Commitment{pts[i], evals[i]};
            commitment_order_.push_back(items[i].label);
            tau_eval_log_.push_back({items[i].label, evals[i]});
            if (!items[i].matrix)
            {
                columns_[items[i].label] = ColumnEntry{items[i].col, items[i].domain, items[i].length, items[i].const_tail, tails[i], items[i].derived_from};
                opened_[items[i].domain].push_back(items[i].label);
            }
        }
        ++stats_.commit_barriers;
        stats_.dynamic_commitments += items.size();
    }

    // SRS of `n` points with its table of shifted bases: the Lagrange basis [L_i(tau)] G of a domain (n = the
    // domain size) or the monomial basis [tau^i] G, i < n (for the matrices, which are committed as
    // coefficient polynomials).  What an honest KZG setup would hand the prover instead of tau.
    inline const ProverFlow::SrsTable& ProverFlow::srs_for(bool monomial, const std::string& domain, std::size_t n)
    {
        const auto key = std::make_pair(monomial ? 1 : 0, n);
        const auto it = srs_tables_.find(key);
        if (it != srs_tables_.end()) return it->second;
        ColP points;
        if (monomial)
        {
            const ColP powers = be_.alloc(kFrMont, n);
            be_.powers(tau_, n, powers);
            points = be_.alloc(kG1, n);
            be_.g1_fixed_base(in_.generator, powers, n, points);
        }
        else
        {
            points = be_.srs_lagrange(dom_.at(domain).log2n, in_.generator, tau_);
        }
        SrsTable t;
        t.table = be_.msm_table(points, n, &t.window_bits);
        return srs_tables_.emplace(key, t).first->second;
    }

    inline G1 ProverFlow::msm_commit(const CommitItem& item)
    {
        const std::size_t count = item.matrix ? item.rows * item.cols : item.length;
        if (count == 0) return G1{};
        const std::size_t n = item.matrix ? count : dom_.at(item.domain).size;
        const SrsTable& srs = srs_for(item.matrix, item.domain, n);
        // the MSM reads field elements: small-integer columns are widened first (padded with zeros up to n)
        ColP scalars = item.col;
        if ((item.col->kind != kFr && item.col->kind != kFrMont) || item.col->count < n)
        {
            scalars = be_.alloc(kFrMont, n);
            be_.linear_combination({item.col}, {fe_u64(1)}, count, n, scalars);
        }
        return be_.msm(scalars, srs.table, n, srs.window_bits);
    }

    // build_binding_trace, src/protocol/trace.cpp:1595-1621
    inline ProverFlow::Binding ProverFlow::build_binding(const ColP& matrix, std::size_t rows, std::size_t cols, const Fe& point,
                                                         const ColP& parameter_values, const std::string& dim_domain, ColP* weights_out,
                                                         const ColP& ready_weights)
    {
        const Domain& n = dom_.at("N");
        const Domain& dd = dom_.at(dim_domain);
        ColP weights = ready_weights;
        if (weights == nullptr)
        {
            weights = be_.alloc(kFrMont, n.size);
            be_.bary_weights(n.log2n, point, weights);
        }
        Binding out;
        out.a = be_.alloc(kFr, dd.size);
        be_.zero(out.a);
        be_.fold_rows(matrix, rows, cols, weights, rows, out.a);
        out.b = parameter_values;
        out.acc = be_.alloc(kFrMont, dd.size);
        queue_scan(ScanJob::kZkmap, out.a, out.b, nullptr, nullptr, nullptr, cols, dd.size, Fe{}, out.acc);
        if (weights_out != nullptr) *weights_out = weights;
        return out;
    }

    // cached_pair_lookup_table + build_pair_lookup_artifacts / build_single_lookup_artifacts +
    // build_logup_accumulator_with_active_count (trace.cpp:1935-2096, src/protocol/lookup.cpp:100-157)
    inline ProverFlow::Lookup ProverFlow::build_pair_lookup(const ColP& table_x, const ColP& table_y, std::size_t table_size, std::int64_t x_min,
                                                            std::size_t band, const ColP& left, const ColP& right, std::size_t valid, const Fe& eta,
                                                            const Fe& beta, const ColP& q_table, const ColP& q_query)
    {
        const Domain& e = dom_.at("edge");
        Lookup out;
        const std::size_t store = lookup_store(std::max(table_size, valid));
        out.store = store;
        out.eta = eta;
        out.pair = table_y != nullptr;
        // A long lookup on a backend that fetches the inverses from the inverted table needs neither the packed
        // query column nor table rows beyond the table: nothing reads them (their evaluations are derived).
        const bool keys_only = compact_ && be_.supports_indexed_logup() && valid > (static_cast<std::size_t>(1) << 20) && table_size <= valid;
        const std::size_t table_store = keys_only ? std::min(store, round64(table_size + 1)) : store;
        out.table_store = table_store;
        if (table_y != nullptr)
        {
            out.table = be_.alloc(kFrMont, table_store);
            be_.linear_combination({table_x, table_y}, {fe_u64(1), eta}, table_size, table_store, out.table);
            if (!keys_only)
            {
                out.query = be_.alloc(kFrMont, store);
                be_.linear_combination({left, right}, {fe_u64(1), eta}, valid, store, out.query);
            }
        }
        else
        {
            out.table = table_x;  // cached_single_lookup_table: the padded table itself
            out.query = left;     // build_single_lookup_artifacts copies the query values
        }
        out.multiplicity = be_.alloc(kU32, table_store);
        be_.lookup_multiplicity(left, table_y != nullptr ? right : nullptr, valid, x_min, band, table_y, table_size, table_store, out.multiplicity);
        out.acc = be_.alloc(kFrMont, store);
        queue_scan(ScanJob::kLogup, out.table, keys_only ? nullptr : out.query, out.multiplicity, q_table, q_query, std::min(valid, e.size - 1), store, beta,
                   out.acc);
        ScanJob& job = scan_queue_.back();
        job.key_x = left;
        job.key_y = table_y != nullptr ? right : nullptr;
        job.table_y = table_y;
        job.x_min = x_min;
        job.band = band;
        job.table_size = table_size;
        return out;
    }

    // route packs + build_route_trace (trace.cpp:1776-1794): table = sum_j eta^j node_cols[j],
    // query = sum_j eta^j edge_cols[j]
    inline ProverFlow::Route ProverFlow::build_route(const std::vector<ColP>& node_cols, const std::vector<ColP>& edge_cols, const Fe& eta,
                                                     const ColP& multiplicity, const Fe& beta)
    {
        const Domain& n = dom_.at("N");
        const auto eta_powers = powers_host(eta, node_cols.size());
        Route out;
        out.table = be_.alloc(kFrMont, n.size);
        be_.linear_combination(node_cols, eta_powers, n_nodes_, n.size, out.table);
        out.query = be_.alloc(kFrMont, es_);
        be_.linear_combination(edge_cols, eta_powers, n_edges_, es_, out.query);
        out.node_acc = be_.alloc(kFrMont, n.size);
        queue_scan(ScanJob::kRouteNode, out.table, multiplicity, nullptr, nullptr, nullptr, n_nodes_, n.size, beta, out.node_acc);
        out.edge_acc = be_.alloc(kFrMont, es_);
        queue_scan(ScanJob::kRouteEdge, out.query, nullptr, nullptr, nullptr, nullptr, n_edges_, es_, beta, out.edge_acc);
        {
            // the edge columns are the node columns gathered by the first edge column (the endpoint ids), so a
            // backend may fetch 1/(query + beta) from the inverted node table instead of inverting per edge
            ScanJob& job = scan_queue_.back();
            job.key_x = edge_cols.front();
            job.table_y = out.table;
            job.table_size = n_nodes_;
        }
        return out;
    }

    // attention_head_forward_impl + quantize_hidden_witness_cpu / quantize_output_witness_cpu
    // (src/model/gat.cpp:474-615; trace.cpp:1143-1279)
    inline ProverFlow::HeadWitness ProverFlow::run_head(const ColP& layer_input, std::size_t input_dim, std::size_t width, const HeadParams& p,
                                                        bool output_head, const std::vector<double>* host_input, std::vector<double>* host_output)
    {
        const std::size_t edge_size = es_;
        HeadTraceCols tr;
        auto f64 = [&](std::size_t n) { return be_.alloc(kF64, std::max<std::size_t>(1, n)); };
        tr.H_prime = f64(n_nodes_ * width);
        tr.H_agg_pre_bias = f64(n_nodes_ * width);
        tr.H_agg = f64(n_nodes_ * width);
        tr.E_src = f64(n_nodes_);
        tr.E_dst = f64(n_nodes_);
        tr.M = f64(n_nodes_);
        tr.Sum = f64(n_nodes_);
        tr.inv = f64(n_nodes_);
        tr.S = f64(n_edges_);
        tr.Z = f64(n_edges_);
        tr.Delta = f64(n_edges_);
        tr.U = f64(n_edges_);
        tr.alpha = f64(n_edges_);
        if (host_input == nullptr)
        {
            HeadDesc head;
            head.features = layer_input;
            head.input_width = input_dim;
            head.output_width = width;
            head.seq_kernel = upload_f64(p.seq_kernel);
            head.attn_src = upload_f64(p.attn_src);
            head.attn_dst = upload_f64(p.attn_dst);
            head.attn_src_bias = p.attn_src_bias;
            head.attn_dst_bias = p.attn_dst_bias;
            head.output_bias = output_head && !p.output_bias.empty() ? upload_f64(p.output_bias) : nullptr;
            head.apply_activation = !output_head;
            be_.head_forward(head, graph_, tr);
        }
        else
        {
            const HostHeadTrace h = host_head_forward(*host_input, n_nodes_, input_dim, p.seq_kernel, width, p.attn_src, p.attn_src_bias, p.attn_dst,
                                                      p.attn_dst_bias, p.output_bias, output_head && !p.output_bias.empty(), !output_head, in_.edge_src,
                                                      in_.edge_dst);
            auto put = [&](const ColP& col, const std::vector<double>& v) {
                if (!v.empty()) be_.upload(col, v.data(), v.size());
            };
            put(tr.H_prime, h.H_prime);
            put(tr.H_agg_pre_bias, h.H_agg_pre_bias);
            put(tr.H_agg, h.H_agg);
            put(tr.E_src, h.E_src);
            put(tr.E_dst, h.E_dst);
            put(tr.M, h.M);
            put(tr.Sum, h.Sum);
            put(tr.inv, h.inv);
            put(tr.S, h.S);
            put(tr.Z, h.Z);
            put(tr.Delta, h.Delta);
            put(tr.U, h.U);
            put(tr.alpha, h.alpha);
            if (host_output != nullptr) *host_output = h.H_agg;
        }

        HeadWitness w;
        auto q_nodes = [&](const ColP& v, std::size_t n) {
            const ColP out = be_.alloc(kI64, std::max<std::size_t>(1, n));
            if (host_input == nullptr)
                be_.quantize_guarded(v, n, kQuantizeGuard, out, guard_counter_);
            else
                be_.quantize(v, n, out);
            return out;
        };
        auto q_edges = [&](const ColP& v) {
            const ColP out = be_.alloc(kI64, edge_size);
            be_.zero(out);
            if (host_input == nullptr)
                be_.quantize_guarded(v, n_edges_, kQuantizeGuard, out, guard_counter_);
            else
                be_.quantize(v, n_edges_, out);
            return out;
        };
        w.h_prime = q_nodes(tr.H_prime, n_nodes_ * width);
        w.h_agg_pre = q_nodes(tr.H_agg_pre_bias, n_nodes_ * width);
        w.h_agg = q_nodes(tr.H_agg, n_nodes_ * width);
        w.e_src = q_nodes(tr.E_src, n_nodes_);
        w.e_dst = q_nodes(tr.E_dst, n_nodes_);
        w.m = q_nodes(tr.M, n_nodes_);
        w.sum = q_nodes(tr.Sum, n_nodes_);
        w.inv = q_nodes(tr.inv, n_nodes_);
        w.s = q_edges(tr.S);
        w.z = q_edges(tr.Z);
        w.delta = q_edges(tr.Delta);
        w.u = q_edges(tr.U);
        w.alpha = q_edges(tr.alpha);
        auto to_edges = [&](const ColP& node_values, const ColP& index) {
            const ColP out = be_.alloc(kI64, edge_size);
            be_.gather(node_values, n_nodes_, index, n_edges_, edge_size, out);
            return out;
        };
        w.e_src_edge = to_edges(w.e_src, src_u32_);
        w.e_dst_edge = to_edges(w.e_dst, dst_u32_);
        w.m_edge = to_edges(w.m, dst_u32_);
        w.sum_edge = to_edges(w.sum, dst_u32_);
        w.inv_edge = to_edges(w.inv, dst_u32_);
        w.h_agg_f64 = tr.H_agg;
        return w;
    }

    // commit_hidden_head, trace.cpp:2348-3074
    inline void ProverFlow::commit_hidden_head(Transcript& t, std::size_t head_index, std::size_t layer_index, std::size_t local_head,
                                               const HeadWitness& w)
    {
        (void)local_head;
        const auto& layer = in_.hidden_layers[layer_index];
        const std::size_t d = layer.head_dim;
        const Domain& n = dom_.at("N");
        const std::string h = std::to_string(head_index);
        const std::string prefix = "P_h" + h + "_";
        const std::string input_label = layer_index == 0 ? "P_H" : "P_H_cat_l" + std::to_string(layer_index - 1);

        commit_batch({matrix_item(prefix + "H_prime", w.h_prime, n_nodes_, d), column_item(prefix + "E_src", w.e_src, "N", n_nodes_),
                      column_item(prefix + "E_dst", w.e_dst, "N", n_nodes_), column_item(prefix + "S", w.s, "edge", n_edges_),
                      column_item(prefix + "Z", w.z, "edge", n_edges_), column_item(prefix + "M", w.m, "N", n_nodes_),
                      column_item(prefix + "M_edge", w.m_edge, "edge", es_), column_item(prefix + "Delta", w.delta, "edge", n_edges_),
                      column_item(prefix + "U", w.u, "edge", n_edges_), column_item(prefix + "Sum", w.sum, "N", n_nodes_),
                      column_item(prefix + "Sum_edge", w.sum_edge, "edge", es_), column_item(prefix + "inv", w.inv, "N", n_nodes_),
                      column_item(prefix + "inv_edge", w.inv_edge, "edge", es_), column_item(prefix + "alpha", w.alpha, "edge", n_edges_),
                      matrix_item(prefix + "H_agg_pre", w.h_agg_pre, n_nodes_, d), matrix_item(prefix + "H_agg", w.h_agg, n_nodes_, d)});

        absorb_dyn(t, input_label);
        absorb_dyn(t, prefix + "H_prime");
        absorb_static(t, "V_h" + h + "_W");
        const Fe y_proj = challenge(t, "y_proj_h" + h);
        const Fe xi = challenge(t, "xi_h" + h);
        absorb_dyn(t, prefix + "H_prime");
        absorb_dyn(t, prefix + "E_src");
        absorb_static(t, "V_h" + h + "_a_src");
        const Fe y_src = challenge(t, "y_src_h" + h);
        absorb_dyn(t, prefix + "H_prime");
        absorb_dyn(t, prefix + "E_dst");
        absorb_static(t, "V_h" + h + "_a_dst");
        const Fe y_dst = challenge(t, "y_dst_h" + h);

        // cached_hidden_compressed_trace, trace.cpp:1654-1685
        const ColP xi_powers = be_.alloc(kFrMont, std::max<std::size_t>(1, d));
        be_.powers(xi, d, xi_powers);
        auto compress = [&](const ColP& matrix) {
            const ColP out = be_.alloc(kFrMont, n_nodes_);
            be_.linear_form_rows(matrix, n_nodes_, d, xi_powers, out);
            return out;
        };
        auto to_edges = [&](const ColP& node_values, const ColP& index) {
            const ColP out = be_.alloc(kFrMont, es_);
            be_.gather(node_values, n_nodes_, index, n_edges_, es_, out);
            return out;
        };
        const ColP h_star = compress(w.h_prime), h_agg_pre_star = compress(w.h_agg_pre), h_agg_star = compress(w.h_agg);
        const ColP h_star_edge = to_edges(h_star, src_u32_);
        const ColP h_agg_pre_star_edge = to_edges(h_agg_pre_star, dst_u32_);
        const ColP h_agg_star_edge = to_edges(h_agg_star, dst_u32_);

        commit_batch({column_item(prefix + "H_star", h_star, "N", n_nodes_)});

        // bindings, trace.cpp:2461-2530
        const std::string w_label = "V_h" + h + "_W";
        const ColP y_proj_powers = be_.alloc(kFrMont, std::max<std::size_t>(1, d));
        be_.powers(y_proj, d, y_proj_powers);
        const ColP proj_b_mont = be_.alloc(kFrMont, dom_.at("in").size);
        be_.zero(proj_b_mont);
        be_.linear_form_rows(param_matrices_.at(w_label), layer.input_dim, d, y_proj_powers, proj_b_mont);
        const ColP input_q = layer_index == 0 ? features_q_ : layer_inputs_q_.at(layer_index);
        ColP w_src, w_dst, w_star;
        const std::vector<ColP> stage_weights = node_weights_at({y_proj, y_src, y_dst});
        const Binding proj = build_binding(input_q, n_nodes_, layer.input_dim, y_proj, proj_b_mont, "in", nullptr, stage_weights[0]);
        const ColP a_src_col = upload_fe(param_vectors_.at("V_h" + h + "_a_src"), dom_.at("d").size);
        const ColP a_dst_col = upload_fe(param_vectors_.at("V_h" + h + "_a_dst"), dom_.at("d").size);
        const Binding src_b = build_binding(w.h_prime, n_nodes_, d, y_src, a_src_col, "d", &w_src, stage_weights[1]);
        const Binding dst_b = build_binding(w.h_prime, n_nodes_, d, y_dst, a_dst_col, "d", &w_dst, stage_weights[2]);
        absorb_dyn(t, prefix + "H_star");
        const Fe y_star = challenge(t, "y_star_h" + h);
        const ColP xi_powers_padded = be_.alloc(kFrMont, dom_.at("d").size);
        be_.zero(xi_powers_padded);
        be_.powers(xi, d, xi_powers_padded);
        const Binding star_b = build_binding(w.h_prime, n_nodes_, d, y_star, xi_powers_padded, "d", &w_star);

        absorb_dyn(t, prefix + "E_src");
        absorb_dyn(t, prefix + "H_star");
        const Fe eta_src = challenge(t, "eta_src_h" + h);
        const Fe beta_src = challenge(t, "beta_src_h" + h);
        absorb_dyn(t, prefix + "S");
        absorb_dyn(t, prefix + "Z");
        absorb_static(t, "V_T_L_x");
        absorb_static(t, "V_T_L_y");
        const Fe eta_l = challenge(t, "eta_L_h" + h);
        const Fe beta_l = challenge(t, "beta_L_h" + h);
        absorb_dyn(t, prefix + "M");
        absorb_dyn(t, prefix + "M_edge");
        absorb_dyn(t, prefix + "Delta");
        absorb_static(t, "V_T_range");
        const Fe beta_r = challenge(t, "beta_R_h" + h);
        absorb_dyn(t, prefix + "Delta");
        absorb_dyn(t, prefix + "U");
        absorb_static(t, "V_T_exp_x");
        absorb_static(t, "V_T_exp_y");
        const Fe eta_exp = challenge(t, "eta_exp_h" + h);
        const Fe beta_exp = challenge(t, "beta_exp_h" + h);

        // lookups, s_max / C_max, trace.cpp:2565-2711
        const std::size_t lrelu_size = lrelu_bound_ * 2 + 1;
        const Lookup lrelu = build_pair_lookup(t_l_x_, t_l_y_, lrelu_size, -static_cast<std::int64_t>(lrelu_bound_), 1, w.s, w.z, n_edges_, eta_l,
                                               beta_l, q_tbl_l_, q_qry_l_);
        const ColP s_max = be_.alloc(kU32, es_);
        be_.first_zero_marker(w.delta, group_begin_, group_end_, groups_, es_, s_max);
        const ColP c_max = be_.alloc(kFrMont, es_);
        queue_scan(ScanJob::kGroupPrefix, s_max, q_new_, nullptr, nullptr, nullptr, es_, es_, Fe{}, c_max);
        const Lookup range = build_pair_lookup(t_range_, nullptr, range_size_, 0, 1, w.delta, nullptr, n_edges_, fe_u64(0), beta_r, q_tbl_r_, q_qry_r_);
        const Lookup exp_l = build_pair_lookup(t_exp_x_, t_exp_y_, range_size_ * 5, 0, 5, w.delta, w.u, n_edges_, eta_exp, beta_exp, q_tbl_exp_, q_qry_exp_);

        const Fe lambda_psq = challenge(t, "lambda_psq_h" + h);
        const ColP widehat = be_.alloc(kFrMont, es_);
        be_.mul_columns(w.alpha, h_star_edge, n_edges_, es_, widehat);
        const ColP w_psq = be_.alloc(kFrMont, es_);
        be_.linear_combination({w.u, widehat}, {fe_u64(1), lambda_psq}, es_, es_, w_psq);  // build_weighted_sum runs over the whole column
        const ColP t_psq = be_.alloc(kFrMont, n_nodes_);
        be_.linear_combination({w.sum, h_agg_pre_star}, {fe_u64(1), lambda_psq}, n_nodes_, n_nodes_, t_psq);
        const ColP t_psq_edge = to_edges(t_psq, dst_u32_);
        const ColP psq = be_.alloc(kFrMont, es_);
        queue_scan(ScanJob::kGroupPrefix, w_psq, q_new_, nullptr, nullptr, nullptr, es_, es_, Fe{}, psq);
        // the source route packs ids + eta * value with powers(eta, 2) = {1, eta} (trace.cpp:2737-2772)
        const Route src_route = build_route({ids_i64_, w.e_src}, {src_i64_, h_star_edge}, eta_src, src_multiplicity_, beta_src);

        const std::size_t dd = dom_.at("d").size, di = dom_.at("in").size;
        commit_batch({column_item(prefix + "a_proj", proj.a, "in", di), column_item(prefix + "b_proj", proj.b, "in", di),
                      column_item(prefix + "Acc_proj", proj.acc, "in", di), column_item(prefix + "a_src", src_b.a, "d", dd),
                      column_item(prefix + "b_src", src_b.b, "d", dd), column_item(prefix + "Acc_src", src_b.acc, "d", dd),
                      column_item(prefix + "a_dst", dst_b.a, "d", dd), column_item(prefix + "b_dst", dst_b.b, "d", dd),
                      column_item(prefix + "Acc_dst", dst_b.acc, "d", dd), column_item(prefix + "a_star", star_b.a, "d", dd),
                      column_item(prefix + "b_star", star_b.b, "d", dd), column_item(prefix + "Acc_star", star_b.acc, "d", dd),
                      column_item(prefix + "E_src_edge", w.e_src_edge, "edge", es_), column_item(prefix + "E_dst_edge", w.e_dst_edge, "edge", es_),
                      column_item(prefix + "H_src_star_edge", h_star_edge, "edge", es_), column_item(prefix + "Table_src", src_route.table, "N", n.size),
                      column_item(prefix + "Query_src", src_route.query, "edge", es_), column_item(prefix + "m_src", src_multiplicity_, "N", n.size),
                      column_item(prefix + "R_src_node", src_route.node_acc, "N", n.size), tail_item(prefix + "R_src", src_route.edge_acc, "edge", es_),
                      packed_item(prefix + "Table_L", lrelu.table, lrelu.table_store, lrelu, "V_T_L_x", "V_T_L_y"), packed_item(prefix + "Query_L", lrelu.query, lrelu.store, lrelu, prefix + "S", prefix + "Z"),
                      column_item(prefix + "m_L", lrelu.multiplicity, "edge", lrelu.table_store), tail_item(prefix + "R_L", lrelu.acc, "edge", lrelu.store),
                      column_item(prefix + "s_max", s_max, "edge", es_), tail_item(prefix + "C_max", c_max, "edge", es_),
                      packed_item(prefix + "Table_R", range.table, range.table_store, range, "V_T_range", ""), packed_item(prefix + "Query_R", range.query, range.store, range, prefix + "Delta", ""),
                      column_item(prefix + "m_R", range.multiplicity, "edge", range.table_store), tail_item(prefix + "R_R", range.acc, "edge", range.store),
                      packed_item(prefix + "Table_exp", exp_l.table, exp_l.table_store, exp_l, "V_T_exp_x", "V_T_exp_y"), packed_item(prefix + "Query_exp", exp_l.query, exp_l.store, exp_l, prefix + "Delta", prefix + "U"),
                      column_item(prefix + "m_exp", exp_l.multiplicity, "edge", exp_l.table_store), tail_item(prefix + "R_exp", exp_l.acc, "edge", exp_l.store),
                      column_item(prefix + "H_agg_pre_star", h_agg_pre_star, "N", n_nodes_),
                      column_item(prefix + "H_agg_pre_star_edge", h_agg_pre_star_edge, "edge", es_),
                      column_item(prefix + "widehat_v_pre_star", widehat, "edge", es_), column_item(prefix + "w_psq", w_psq, "edge", es_),
                      column_item(prefix + "T_psq", t_psq, "N", n_nodes_), column_item(prefix + "T_psq_edge", t_psq_edge, "edge", es_),
                      tail_item(prefix + "PSQ", psq, "edge", es_), column_item(prefix + "H_agg_star", h_agg_star, "N", n_nodes_),
                      column_item(prefix + "H_agg_star_edge", h_agg_star_edge, "edge", es_)});

        absorb_dyn(t, prefix + "T_psq");
        absorb_dyn(t, prefix + "T_psq_edge");
        const Fe eta_t = challenge(t, "eta_t_h" + h);
        const Fe beta_t = challenge(t, "beta_t_h" + h);
        const Route t_route = build_route({ids_i64_, t_psq}, {dst_i64_, t_psq_edge}, eta_t, dst_multiplicity_, beta_t);
        absorb_dyn(t, prefix + "H_agg_pre");
        absorb_dyn(t, prefix + "H_agg_pre_star");
        const Fe y_agg_pre = challenge(t, "y_agg_pre_h" + h);
        absorb_dyn(t, prefix + "H_agg_pre");
        absorb_dyn(t, prefix + "H_agg");
        absorb_static(t, "V_T_ELU_x");
        absorb_static(t, "V_T_ELU_y");
        const Fe eta_elu = challenge(t, "eta_ELU_h" + h);
        const Fe beta_elu = challenge(t, "beta_ELU_h" + h);
        absorb_dyn(t, prefix + "H_agg");
        absorb_dyn(t, prefix + "H_agg_star");
        const Fe y_agg = challenge(t, "y_agg_h" + h);
        const Fe eta_dst = challenge(t, "eta_dst_h" + h);
        const Fe beta_dst = challenge(t, "beta_dst_h" + h);

        ColP w_agg_pre, w_agg;
        const std::vector<ColP> agg_weights = node_weights_at({y_agg_pre, y_agg});
        const Binding agg_pre_b = build_binding(w.h_agg_pre, n_nodes_, d, y_agg_pre, xi_powers_padded, "d", &w_agg_pre, agg_weights[0]);
        const Binding agg_b = build_binding(w.h_agg, n_nodes_, d, y_agg, xi_powers_padded, "d", &w_agg, agg_weights[1]);
        // ELU lookup over the flattened node_count x d matrices (trace.cpp:2920-2971): the row-major
        // matrix buffers ARE the flat columns
        const std::size_t flat = n_nodes_ * d;
        const Lookup elu = build_pair_lookup(t_elu_x_, t_elu_y_, lrelu_size * 3, -static_cast<std::int64_t>(lrelu_bound_), 3, w.h_agg_pre, w.h_agg, flat,
                                             eta_elu, beta_elu, q_tbl_elu_, q_qry_elu_);
        const Route dst_route = build_route({ids_i64_, w.e_dst, w.m, w.sum, w.inv, h_agg_star},
                                            {dst_i64_, w.e_dst_edge, w.m_edge, w.sum_edge, w.inv_edge, h_agg_star_edge}, eta_dst, dst_multiplicity_,
                                            beta_dst);

        commit_batch({column_item(prefix + "a_agg_pre", agg_pre_b.a, "d", dd), column_item(prefix + "b_agg_pre", agg_pre_b.b, "d", dd),
                      column_item(prefix + "Acc_agg_pre", agg_pre_b.acc, "d", dd), column_item(prefix + "a_agg", agg_b.a, "d", dd),
                      column_item(prefix + "b_agg", agg_b.b, "d", dd), column_item(prefix + "Acc_agg", agg_b.acc, "d", dd),
                      column_item(prefix + "H_agg_pre_flat", w.h_agg_pre, "edge", flat), column_item(prefix + "H_agg_flat", w.h_agg, "edge", flat),
                      packed_item(prefix + "Table_ELU", elu.table, elu.table_store, elu, "V_T_ELU_x", "V_T_ELU_y"), packed_item(prefix + "Query_ELU", elu.query, elu.store, elu, prefix + "H_agg_pre_flat", prefix + "H_agg_flat"),
                      column_item(prefix + "m_ELU", elu.multiplicity, "edge", elu.table_store), tail_item(prefix + "R_ELU", elu.acc, "edge", elu.store),
                      column_item(prefix + "Table_t", t_route.table, "N", n.size), column_item(prefix + "Query_t", t_route.query, "edge", es_),
                      column_item(prefix + "m_t", dst_multiplicity_, "N", n.size), column_item(prefix + "R_t_node", t_route.node_acc, "N", n.size),
                      tail_item(prefix + "R_t", t_route.edge_acc, "edge", es_)});
        commit_batch({column_item(prefix + "Table_dst", dst_route.table, "N", n.size), column_item(prefix + "Query_dst", dst_route.query, "edge", es_),
                      column_item(prefix + "m_dst", dst_multiplicity_, "N", n.size), column_item(prefix + "R_dst_node", dst_route.node_acc, "N", n.size),
                      tail_item(prefix + "R_dst", dst_route.edge_acc, "edge", es_)});

        // route.total = node_acc[real_node_count] (build_route_trace, trace.cpp:1792)
        pending_totals_.push_back({"S_src_h" + h, src_route.node_acc, n_nodes_});
        pending_totals_.push_back({"S_dst_h" + h, dst_route.node_acc, n_nodes_});
        pending_totals_.push_back({"S_t_h" + h, t_route.node_acc, n_nodes_});
        resolve_totals();
        // external evaluations, trace.cpp:3062-3073: Horner of the matrix, barycentric evaluation of the
        // columns at the binding points (the weights at those points exist already)
        {
            const ColP out = be_.alloc(kFr, 6);
            be_.horner_device(w.h_prime, n_nodes_, d, y_proj, out, 0);
            be_.eval_device({w.e_src}, n_nodes_, n.log2n, w_src, {0}, out, 1);
            be_.eval_device({w.e_dst}, n_nodes_, n.log2n, w_dst, {0}, out, 2);
            be_.eval_device({h_star}, n_nodes_, n.log2n, w_star, {0}, out, 3);
            be_.eval_device({h_agg_pre_star}, n_nodes_, n.log2n, w_agg_pre, {0}, out, 4);
            be_.eval_device({h_agg_star}, n_nodes_, n.log2n, w_agg, {0}, out, 5);
            Fe mu[6];
            be_.download(out, 0, 6, mu);
            const char* names[6] = {"_proj", "_src", "_dst", "_star", "_agg_pre", "_agg"};
            const std::string labels[6] = {prefix + "H_prime", prefix + "E_src", prefix + "E_dst", prefix + "H_star", prefix + "H_agg_pre_star", prefix + "H_agg_star"};
            const Fe points[6] = {y_proj, y_src, y_dst, y_star, y_agg_pre, y_agg};
            for (int i = 0; i < 6; ++i) add_external("mu_h" + h + names[i], mu[i], labels[i], points[i]);
        }
    }
}  // namespace gatzk_flow

#include "prover_flow_tail.hpp"
#include "prover_flow_quotients.hpp"
