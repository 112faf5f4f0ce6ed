// Host-side C++ mirror of the reference prover's operator interface for the hot
// path, implemented on top of the C ABI of libgatzk_b200.so.  Names, argument
// meaning and error behaviour (std::runtime_error) follow the reference:
//   gatzk::algebra::FieldElement           include/gatzk/algebra/field.hpp:28-205
//   gatzk::algebra::RootOfUnityDomain      include/gatzk/algebra/polynomial.hpp, src/algebra/polynomial.cpp:37-351
//   gatzk::algebra::Polynomial             src/algebra/polynomial.cpp:353-508
//   gatzk::algebra::PackedEvaluationBackend src/algebra/eval_backend.cpp:61-444
//   gatzk::crypto::KZG::commit_batch        src/crypto/kzg.cpp:458-542
//   gatzk::protocol::build_*                src/protocol/lookup.cpp, psq.cpp, zkmap.cpp, trace.cpp:203-361
// Columns live on the GPU; only scalars, commitments and opened values come back.
#pragma once

#include <algorithm>
#include <array>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/gatzk_b200.h"

namespace gatzk_b200
{
    // One GPU context shared by the objects below (one per host thread that issues work).
    class Context
    {
    public:
        explicit Context(int device = 0)
        {
            if (gzk_ctx_create(device, &ctx_) != GZK_OK) throw std::runtime_error("b200 backend: no usable sm_100 GPU");
        }
        ~Context() { gzk_ctx_destroy(ctx_); }
        Context(const Context&) = delete;
        Context& operator=(const Context&) = delete;
        gzk_ctx* raw() const { return ctx_; }
        // Waits for the queued work; throws what a deferred call raised on the device.
        void synchronize() const { check(gzk_ctx_synchronize(ctx_)); }
        // Builder calls return once queued (errors surface at synchronize()).
        void set_deferred(bool on) const { check(gzk_ctx_set_deferred(ctx_, on ? 1 : 0)); }
        void check(int rc) const
        {
            if (rc != GZK_OK) throw std::runtime_error(gzk_last_error(ctx_));
        }

    private:
        gzk_ctx* ctx_ = nullptr;
    };

    // Owning handle of a device buffer.
    class DeviceBuffer
    {
    public:
        DeviceBuffer(const Context& ctx, int kind, std::size_t count) : ctx_(&ctx)
        {
            ctx.check(gzk_buf_alloc(ctx.raw(), kind, count, &buf_));
        }
        ~DeviceBuffer()
        {
            if (buf_ != nullptr) gzk_buf_free(ctx_->raw(), buf_);
        }
        DeviceBuffer(const DeviceBuffer&) = delete;
        DeviceBuffer& operator=(const DeviceBuffer&) = delete;
        gzk_buf* raw() const { return buf_; }
        std::size_t count() const { return gzk_buf_count(buf_); }
        void upload(const void* host, std::size_t count, std::size_t offset = 0) { ctx_->check(gzk_buf_upload(ctx_->raw(), buf_, offset, host, count)); }
        void download(void* host, std::size_t count, std::size_t offset = 0) const { ctx_->check(gzk_buf_download(ctx_->raw(), buf_, offset, host, count)); }

    private:
        const Context* ctx_;
        gzk_buf* buf_ = nullptr;
    };

    namespace algebra
    {
        // 32-byte little-endian canonical Fr value (the wire format of the C ABI).
        class FieldElement
        {
        public:
            FieldElement() { bytes_.fill(0); }
            explicit FieldElement(std::uint64_t raw)
            {
                bytes_.fill(0);
                std::memcpy(bytes_.data(), &raw, 8);
            }
            static FieldElement zero() { return FieldElement(0); }
            static FieldElement one() { return FieldElement(1); }
            static FieldElement from_signed(std::int64_t value)
            {
                if (value >= 0) return FieldElement(static_cast<std::uint64_t>(value));
                return zero() - FieldElement(~static_cast<std::uint64_t>(value) + 1);
            }
            static FieldElement from_bytes(const std::uint8_t* bytes)
            {
                FieldElement out;
                std::memcpy(out.bytes_.data(), bytes, 32);
                return out;
            }
            const std::uint8_t* bytes() const { return bytes_.data(); }
            std::uint64_t value() const
            {
                std::uint64_t v;
                std::memcpy(&v, bytes_.data(), 8);
                return v;
            }
            bool is_zero() const
            {
                for (auto b : bytes_)
                    if (b != 0) return false;
                return true;
            }
            bool operator==(const FieldElement& o) const { return bytes_ == o.bytes_; }
            FieldElement operator+(const FieldElement& o) const { return op(0, o); }
            FieldElement operator-(const FieldElement& o) const { return op(1, o); }
            FieldElement operator*(const FieldElement& o) const { return op(2, o); }
            FieldElement inv() const
            {
                if (is_zero()) throw std::runtime_error("attempted to invert zero in FieldElement");
                return op(3, *this);
            }
            FieldElement pow(std::uint64_t exponent) const
            {
                FieldElement out = one(), base = *this;
                while (exponent != 0)
                {
                    if (exponent & 1U) out = out * base;
                    base = base * base;
                    exponent >>= 1U;
                }
                return out;
            }

        private:
            FieldElement op(int code, const FieldElement& o) const
            {
                FieldElement out;
                if (gzk_fr_op(code, bytes_.data(), o.bytes_.data(), out.bytes_.data()) != GZK_OK)
                    throw std::runtime_error("FieldElement: non-canonical operand");
                return out;
            }
            std::array<std::uint8_t, 32> bytes_;
        };

        // Device-resident barycentric weight vector (what the reference keeps as std::vector<mcl::Fr>).
        struct NativeWeights
        {
            std::shared_ptr<DeviceBuffer> buffer;
        };

        struct RootOfUnityDomain
        {
            std::string name;
            std::size_t size = 0;
            unsigned log2_size = 0;
            FieldElement omega;
            FieldElement inv_size;
            const Context* context = nullptr;

            static std::shared_ptr<RootOfUnityDomain> create(const Context& ctx, const std::string& name, std::size_t size)
            {
                if (size == 0 || (size & (size - 1U)) != 0U) throw std::runtime_error("domain size must be a non-zero power of two");
                auto d = std::make_shared<RootOfUnityDomain>();
                d->name = name;
                d->size = size;
                while ((static_cast<std::size_t>(1) << d->log2_size) < size) ++d->log2_size;
                std::uint8_t w[32];
                ctx.check(gzk_root_of_unity(ctx.raw(), size, w));
                d->omega = FieldElement::from_bytes(w);
                d->inv_size = FieldElement(static_cast<std::uint64_t>(size)).inv();
                d->context = &ctx;
                return d;
            }
            FieldElement zero_polynomial_eval(const FieldElement& x) const { return x.pow(size) - FieldElement::one(); }
            // polynomial.cpp:131-316; throws when x is a point of the domain (the caller then takes the
            // direct-index branch, as build_domain_evaluation_weights does)
            NativeWeights barycentric_weights_native(const FieldElement& x) const
            {
                NativeWeights w;
                w.buffer = std::make_shared<DeviceBuffer>(*context, GZK_KIND_FR_MONT, size);
                context->check(gzk_bary_weights(context->raw(), log2_size, x.bytes(), w.buffer->raw()));
                return w;
            }
            // polynomial.cpp:330-351 without the O(n) search: x = omega^shift iff x^n = 1; the shift is
            // then recovered bit by bit (the group has order 2^k).
            bool rotation_shift(const FieldElement& to, std::size_t* shift) const
            {
                if (!(to.pow(size) == FieldElement::one())) return false;
                std::size_t s = 0;
                FieldElement rest = to;  // invariant: rest = to * omega^-s
                const FieldElement omega_inv = omega.inv();
                for (unsigned bit = 0; bit < log2_size; ++bit)
                {
                    // rest^(n / 2^(bit+1)) is +1 or -1; -1 means bit `bit` of the shift is set
                    if (!(rest.pow(size >> (bit + 1)) == FieldElement::one()))
                    {
                        s |= static_cast<std::size_t>(1) << bit;
                        rest = rest * omega_inv.pow(static_cast<std::uint64_t>(1) << bit);
                    }
                }
                *shift = s;
                return true;
            }
        };

        enum class PolynomialBasis { Coefficient, Evaluation };

        struct Polynomial
        {
            std::string name;
            PolynomialBasis basis = PolynomialBasis::Coefficient;
            std::shared_ptr<DeviceBuffer> data;  // column or coefficient vector on the device
            std::size_t length = 0;               // number of stored values (valid prefix)
            std::shared_ptr<RootOfUnityDomain> domain;

            static Polynomial from_evaluations(const Context& ctx, const std::string& name, const std::vector<FieldElement>& evaluations,
                                               const std::shared_ptr<RootOfUnityDomain>& domain)
            {
                if (domain == nullptr || evaluations.size() > domain->size) throw std::runtime_error("evaluation polynomial requires a compatible domain");
                Polynomial p = upload(ctx, name, evaluations);
                p.basis = PolynomialBasis::Evaluation;
                p.domain = domain;
                return p;
            }
            static Polynomial from_coefficients(const Context& ctx, const std::string& name, const std::vector<FieldElement>& coefficients)
            {
                return upload(ctx, name, coefficients);
            }
            std::size_t size() const { return length; }

            // polynomial.cpp:415-496: Horner for coefficients; for evaluations the direct value when x is a
            // domain point, otherwise weights + inner product (same field value as the reference's
            // per-element-inversion loop).
            FieldElement evaluate(const Context& ctx, const FieldElement& x) const
            {
                std::uint8_t out[32];
                if (basis == PolynomialBasis::Coefficient)
                {
                    ctx.check(gzk_matrix_horner(ctx.raw(), data ? data->raw() : nullptr, length == 0 ? 0 : 1, length, x.bytes(), out));
                    return FieldElement::from_bytes(out);
                }
                if (domain == nullptr) throw std::runtime_error("evaluation polynomial is missing its domain");
                std::size_t shift = 0;
                if (domain->rotation_shift(x, &shift))
                {
                    if (shift >= length) return FieldElement::zero();
                    data->download(out, 1, shift);
                    return FieldElement::from_bytes(out);
                }
                const auto weights = domain->barycentric_weights_native(x);
                gzk_buf* col = data->raw();
                const std::uint64_t rotation = 0;
                ctx.check(gzk_eval_batch(ctx.raw(), &col, 1, length, domain->log2_size, weights.buffer->raw(), &rotation, 1, out));
                return FieldElement::from_bytes(out);
            }

        private:
            static Polynomial upload(const Context& ctx, const std::string& name, const std::vector<FieldElement>& values)
            {
                Polynomial p;
                p.name = name;
                p.length = values.size();
                p.data = std::make_shared<DeviceBuffer>(ctx, GZK_KIND_FR, values.empty() ? 1 : values.size());
                if (!values.empty())
                {
                    std::vector<std::uint8_t> raw(values.size() * 32);
                    for (std::size_t i = 0; i < values.size(); ++i) std::memcpy(&raw[32 * i], values[i].bytes(), 32);
                    p.data->upload(raw.data(), values.size());
                }
                return p;
            }
        };

        // eval_backend.cpp:61-444.  No interleaved copy is made: the columns stay where they are.
        class PackedEvaluationBackend
        {
        public:
            PackedEvaluationBackend(const Context& ctx, std::shared_ptr<RootOfUnityDomain> domain,
                                    std::vector<std::pair<std::string, const Polynomial*>> polynomials)
                : ctx_(&ctx), domain_(std::move(domain)), polynomials_(std::move(polynomials))
            {
                if (domain_ == nullptr) throw std::runtime_error("domain evaluation backend requires a domain");
                for (std::size_t row = 0; row < polynomials_.size(); ++row)
                {
                    const auto* polynomial = polynomials_[row].second;
                    if (polynomial == nullptr || polynomial->basis != PolynomialBasis::Evaluation || polynomial->domain != domain_)
                        throw std::runtime_error("domain evaluation backend requires same-domain evaluation polynomials");
                    label_to_index_.emplace(polynomials_[row].first, row);
                }
            }
            std::vector<FieldElement> evaluate_with_native_weights(const std::vector<std::string>& labels, const NativeWeights& weights) const
            {
                return evaluate_with_native_weight_rotations(labels, weights, {0}).front();
            }
            std::vector<std::vector<FieldElement>> evaluate_with_native_weight_rotations(const std::vector<std::string>& labels,
                                                                                         const NativeWeights& representative_weights,
                                                                                         const std::vector<std::size_t>& rotations) const
            {
                if (representative_weights.buffer == nullptr || representative_weights.buffer->count() != domain_->size)
                    throw std::runtime_error("domain evaluation backend rotation weight size mismatch");
                if (rotations.empty()) return {};
                // columns of one call must share a stored length; group the labels by length
                std::vector<std::vector<FieldElement>> out(rotations.size(), std::vector<FieldElement>(labels.size()));
                std::map<std::size_t, std::vector<std::size_t>> by_length;
                for (std::size_t i = 0; i < labels.size(); ++i)
                {
                    const auto it = label_to_index_.find(labels[i]);
                    if (it == label_to_index_.end()) throw std::runtime_error("domain evaluation backend is missing label: " + labels[i]);
                    by_length[polynomials_[it->second].second->length].push_back(i);
                }
                std::vector<std::uint64_t> rot(rotations.begin(), rotations.end());
                for (const auto& group : by_length)
                {
                    std::vector<gzk_buf*> cols;
                    for (const auto i : group.second) cols.push_back(polynomials_[label_to_index_.at(labels[i])].second->data->raw());
                    std::vector<std::uint8_t> raw(rot.size() * cols.size() * 32);
                    ctx_->check(gzk_eval_batch(ctx_->raw(), cols.data(), cols.size(), group.first, domain_->log2_size,
                                               representative_weights.buffer->raw(), rot.data(), rot.size(), raw.data()));
                    for (std::size_t p = 0; p < rot.size(); ++p)
                        for (std::size_t k = 0; k < cols.size(); ++k)
                            out[p][group.second[k]] = FieldElement::from_bytes(&raw[(p * cols.size() + k) * 32]);
                }
                return out;
            }

            // eval_backend.cpp:142-189: the values of the named columns at one row (the point is omega^index)
            std::vector<FieldElement> values_at_direct_index(const std::vector<std::string>& labels, std::size_t index) const
            {
                std::vector<FieldElement> out(labels.size());
                for (std::size_t i = 0; i < labels.size(); ++i)
                {
                    const auto it = label_to_index_.find(labels[i]);
                    if (it == label_to_index_.end()) throw std::runtime_error("domain evaluation backend is missing label: " + labels[i]);
                    const auto* polynomial = polynomials_[it->second].second;
                    if (index < polynomial->length)
                    {
                        std::uint8_t raw[32];
                        polynomial->data->download(raw, 1, index);
                        out[i] = FieldElement::from_bytes(raw);
                    }
                }
                return out;
            }
            const std::shared_ptr<RootOfUnityDomain>& domain() const { return domain_; }

        private:
            const Context* ctx_;
            std::shared_ptr<RootOfUnityDomain> domain_;
            std::vector<std::pair<std::string, const Polynomial*>> polynomials_;
            std::map<std::string, std::size_t> label_to_index_;
        };
    }

    namespace protocol
    {
        // The verifier evaluates the PUBLIC columns itself, with the same packed backend the prover uses
        // (PublicEvaluationBackendRegistry + the precompute of VerifierEvaluationCache,
        // src/protocol/verifier.cpp:218-262, 540-565): all public columns of a domain are grouped in one
        // backend, and the first request at a point evaluates the whole group - by direct row access when
        // the point is a domain point (include/gatzk/algebra/domain_evaluation.hpp:40-71), by barycentric
        // weights otherwise.  On the reference's large runs this is most of verify_time (176 s of the
        // 169k-node run); here it is one weights call and one packed evaluation per (domain, point).
        class PublicEvaluationBackendRegistry
        {
        public:
            PublicEvaluationBackendRegistry(const Context& ctx, const std::map<std::string, algebra::Polynomial>& public_polynomials) : ctx_(&ctx)
            {
                std::map<std::string, std::vector<std::pair<std::string, const algebra::Polynomial*>>> groups;
                std::map<std::string, std::shared_ptr<algebra::RootOfUnityDomain>> domains;
                for (const auto& item : public_polynomials)
                {
                    const auto& polynomial = item.second;
                    if (polynomial.basis != algebra::PolynomialBasis::Evaluation || polynomial.domain == nullptr) continue;
                    const auto key = polynomial.domain->name + ":" + std::to_string(polynomial.domain->size);
                    groups[key].push_back({item.first, &polynomial});
                    domains[key] = polynomial.domain;
                    label_domain_[item.first] = key;
                }
                for (auto& group : groups)
                {
                    std::vector<std::string> labels;
                    for (const auto& p : group.second) labels.push_back(p.first);
                    labels_.emplace(group.first, std::move(labels));
                    backends_.emplace(group.first, algebra::PackedEvaluationBackend(ctx, domains.at(group.first), std::move(group.second)));
                }
            }
            // value of one public column at a point; the whole domain group is evaluated on the first request
            // at that point and cached, as the reference's verifier does
            algebra::FieldElement eval(const std::string& label, const algebra::FieldElement& point)
            {
                const auto dom = label_domain_.find(label);
                if (dom == label_domain_.end()) throw std::runtime_error("unsupported verifier public polynomial label: " + label);
                const std::string point_key(reinterpret_cast<const char*>(point.bytes()), 32);
                const auto cache_key = dom->second + "@" + point_key;
                auto hit = cache_.find(cache_key);
                if (hit == cache_.end())
                {
                    const auto& backend = backends_.at(dom->second);
                    const auto& labels = labels_.at(dom->second);
                    std::vector<algebra::FieldElement> values;
                    std::size_t shift = 0;
                    if (backend.domain()->rotation_shift(point, &shift))
                        values = backend.values_at_direct_index(labels, shift);
                    else
                        values = backend.evaluate_with_native_weights(labels, backend.domain()->barycentric_weights_native(point));
                    std::map<std::string, algebra::FieldElement> by_label;
                    for (std::size_t i = 0; i < labels.size(); ++i) by_label.emplace(labels[i], values[i]);
                    hit = cache_.emplace(cache_key, std::move(by_label)).first;
                    ++group_evaluations_;
                }
                return hit->second.at(label);
            }
            std::size_t group_evaluations() const { return group_evaluations_; }

        private:
            const Context* ctx_;
            std::map<std::string, algebra::PackedEvaluationBackend> backends_;
            std::map<std::string, std::vector<std::string>> labels_;
            std::map<std::string, std::string> label_domain_;
            std::map<std::string, std::map<std::string, algebra::FieldElement>> cache_;
            std::size_t group_evaluations_ = 0;
        };
    }

    namespace crypto
    {
        struct G1Point
        {
            std::array<std::uint8_t, 96> affine{};  // x || y little-endian; all zero = infinity
        };
        struct KZGKeyPair
        {
            algebra::FieldElement tau;
            G1Point g1_generator;  // supplied by the host (the reference derives it with mcl's hashAndMapToG1)
        };
        struct Commitment
        {
            std::string name;
            G1Point point;
            algebra::FieldElement tau_evaluation;
        };

        struct KZG
        {
            // kzg.cpp:366-399 without the mcl-specific generator derivation
            static KZGKeyPair setup(std::uint64_t seed, const G1Point& generator)
            {
                return KZGKeyPair{algebra::FieldElement(seed + 17), generator};
            }
            // kzg.cpp:458-542: coefficient polynomials by Horner, evaluation polynomials grouped by
            // (domain, stored length) against the shared weights at tau, then K same-base multiplications.
            static std::vector<Commitment> commit_batch(const Context& ctx,
                                                        const std::vector<std::pair<std::string, const algebra::Polynomial*>>& named_polynomials,
                                                        const KZGKeyPair& key)
            {
                std::vector<Commitment> out(named_polynomials.size());
                if (named_polynomials.empty()) return out;
                std::vector<algebra::FieldElement> tau_evaluations(named_polynomials.size());
                std::map<std::pair<const algebra::RootOfUnityDomain*, std::size_t>, std::vector<std::size_t>> groups;
                for (std::size_t i = 0; i < named_polynomials.size(); ++i)
                {
                    const auto* polynomial = named_polynomials[i].second;
                    if (polynomial->basis == algebra::PolynomialBasis::Coefficient)
                    {
                        tau_evaluations[i] = polynomial->evaluate(ctx, key.tau);
                        continue;
                    }
                    if (polynomial->domain == nullptr) throw std::runtime_error("evaluation polynomial is missing its domain");
                    groups[{polynomial->domain.get(), polynomial->length}].push_back(i);
                }
                std::map<const algebra::RootOfUnityDomain*, algebra::NativeWeights> weight_cache;
                for (const auto& group : groups)
                {
                    const auto* domain = group.first.first;
                    auto it = weight_cache.find(domain);
                    if (it == weight_cache.end()) it = weight_cache.emplace(domain, domain->barycentric_weights_native(key.tau)).first;
                    std::vector<gzk_buf*> cols;
                    for (const auto i : group.second) cols.push_back(named_polynomials[i].second->data->raw());
                    std::vector<std::uint8_t> raw(cols.size() * 32);
                    const std::uint64_t rotation = 0;
                    ctx.check(gzk_eval_batch(ctx.raw(), cols.data(), cols.size(), group.first.second, domain->log2_size, it->second.buffer->raw(),
                                             &rotation, 1, raw.data()));
                    for (std::size_t k = 0; k < cols.size(); ++k) tau_evaluations[group.second[k]] = algebra::FieldElement::from_bytes(&raw[32 * k]);
                }
                std::vector<std::uint8_t> scalars(named_polynomials.size() * 32), points(named_polynomials.size() * 96);
                for (std::size_t i = 0; i < named_polynomials.size(); ++i) std::memcpy(&scalars[32 * i], tau_evaluations[i].bytes(), 32);
                ctx.check(gzk_g1_mul_same_base(ctx.raw(), key.g1_generator.affine.data(), scalars.data(), named_polynomials.size(), points.data()));
                for (std::size_t i = 0; i < named_polynomials.size(); ++i)
                {
                    out[i].name = named_polynomials[i].first;
                    std::memcpy(out[i].point.affine.data(), &points[96 * i], 96);
                    out[i].tau_evaluation = tau_evaluations[i];
                }
                return out;
            }
        };
    }

    namespace protocol
    {
        // lookup.cpp:100-157
        inline std::shared_ptr<DeviceBuffer> build_logup_accumulator_with_active_count(
            const Context& ctx, const DeviceBuffer& table, const DeviceBuffer& query, const DeviceBuffer& multiplicity, const DeviceBuffer& q_table,
            const DeviceBuffer& q_query, std::size_t n, const algebra::FieldElement& beta, std::size_t active_count)
        {
            auto out = std::make_shared<DeviceBuffer>(ctx, GZK_KIND_FR_MONT, n == 0 ? 1 : n);
            ctx.check(gzk_logup_accumulator(ctx.raw(), table.raw(), query.raw(), multiplicity.raw(), q_table.raw(), q_query.raw(), n, beta.bytes(),
                                            active_count, out->raw()));
            return out;
        }
        // trace.cpp:298-361
        inline std::shared_ptr<DeviceBuffer> build_route_node_accumulator(const Context& ctx, const DeviceBuffer& table, const DeviceBuffer& multiplicity,
                                                                          std::size_t valid_length, std::size_t domain_size, const algebra::FieldElement& beta)
        {
            auto out = std::make_shared<DeviceBuffer>(ctx, GZK_KIND_FR_MONT, domain_size == 0 ? 1 : domain_size);
            ctx.check(gzk_route_node_accumulator(ctx.raw(), table.raw(), multiplicity.raw(), valid_length, domain_size, beta.bytes(), out->raw()));
            return out;
        }
        inline std::shared_ptr<DeviceBuffer> build_route_edge_accumulator(const Context& ctx, const DeviceBuffer& query, std::size_t valid_length,
                                                                          std::size_t domain_size, const algebra::FieldElement& beta)
        {
            auto out = std::make_shared<DeviceBuffer>(ctx, GZK_KIND_FR_MONT, domain_size == 0 ? 1 : domain_size);
            ctx.check(gzk_route_edge_accumulator(ctx.raw(), query.raw(), valid_length, domain_size, beta.bytes(), out->raw()));
            return out;
        }
        // psq.cpp:7-39 (build_group_prefix_state and build_max_counter_state share the recurrence)
        inline std::shared_ptr<DeviceBuffer> build_group_prefix_state(const Context& ctx, const DeviceBuffer& values, const DeviceBuffer& q_new, std::size_t n)
        {
            auto out = std::make_shared<DeviceBuffer>(ctx, GZK_KIND_FR_MONT, n == 0 ? 1 : n);
            ctx.check(gzk_group_prefix_state(ctx.raw(), values.raw(), q_new.raw(), n, out->raw()));
            return out;
        }
        // zkmap.cpp:7-32
        struct ZkMapAccumulatorTrace
        {
            std::shared_ptr<DeviceBuffer> accumulator;
            algebra::FieldElement mu;
        };
        inline ZkMapAccumulatorTrace build_zkmap_trace(const Context& ctx, const DeviceBuffer& a_values, const DeviceBuffer& b_values, std::size_t count,
                                                       std::size_t domain_size)
        {
            ZkMapAccumulatorTrace trace;
            trace.accumulator = std::make_shared<DeviceBuffer>(ctx, GZK_KIND_FR_MONT, domain_size == 0 ? 1 : domain_size);
            std::uint8_t mu[32];
            ctx.check(gzk_zkmap_accumulator(ctx.raw(), a_values.raw(), b_values.raw(), count, domain_size, trace.accumulator->raw(), mu));
            trace.mu = algebra::FieldElement::from_bytes(mu);
            return trace;
        }
    }

    // Mirror of the reference's fp64 forward of one attention head (include/gatzk/model/gat.hpp:21-46,
    // src/model/gat.cpp:474-615): same parameter and trace types, same call shape; the loops run on the GPU.
    namespace model
    {
        using FloatMatrix = std::vector<std::vector<double>>;
        struct Edge
        {
            std::size_t src = 0;
            std::size_t dst = 0;
        };
        struct AttentionHeadParameters
        {
            FloatMatrix seq_kernel_fp;
            std::vector<double> attn_dst_kernel_fp;
            double attn_dst_bias_fp = 0.0;
            std::vector<double> attn_src_kernel_fp;
            double attn_src_bias_fp = 0.0;
            std::vector<double> output_bias_fp;
        };
        struct HeadForwardTrace
        {
            FloatMatrix H_prime;
            std::vector<double> E_src, E_dst, S, Z, M, Delta, U, Sum, inv, alpha;
            FloatMatrix H_agg_pre_bias, H_agg;
        };

        inline HeadForwardTrace attention_head_forward(const Context& ctx, const FloatMatrix& features, const std::vector<Edge>& edges,
                                                       const AttentionHeadParameters& parameters, bool apply_output_bias, bool apply_activation)
        {
            HeadForwardTrace trace;
            if (features.empty()) return trace;
            const std::size_t nodes = features.size(), inner = features.front().size();
            const std::size_t width = parameters.seq_kernel_fp.empty() ? 0 : parameters.seq_kernel_fp.front().size();
            if (parameters.seq_kernel_fp.size() != inner) throw std::runtime_error("float matrix multiply dimension mismatch");
            for (const auto& edge : edges)
                if (edge.src >= nodes || edge.dst >= nodes) throw std::runtime_error("edge out of bounds while running attention head forward");
            auto upload_f64 = [&](const std::vector<double>& v) {
                auto b = std::make_shared<DeviceBuffer>(ctx, GZK_KIND_F64, v.empty() ? 1 : v.size());
                if (!v.empty()) b->upload(v.data(), v.size());
                return b;
            };
            auto upload_u32 = [&](const std::vector<std::uint32_t>& v) {
                auto b = std::make_shared<DeviceBuffer>(ctx, GZK_KIND_U32, v.empty() ? 1 : v.size());
                if (!v.empty()) b->upload(v.data(), v.size());
                return b;
            };
            auto flatten = [](const FloatMatrix& m) {
                std::vector<double> out;
                for (const auto& row : m) out.insert(out.end(), row.begin(), row.end());
                return out;
            };
            // incoming sources per destination in edge order, the node itself appended when it has no self loop
            std::vector<std::vector<std::uint32_t>> incoming(nodes);
            std::vector<std::uint32_t> edge_src(edges.size()), edge_dst(edges.size());
            for (std::size_t e = 0; e < edges.size(); ++e)
            {
                edge_src[e] = static_cast<std::uint32_t>(edges[e].src);
                edge_dst[e] = static_cast<std::uint32_t>(edges[e].dst);
                incoming[edges[e].dst].push_back(edge_src[e]);
            }
            std::vector<std::uint32_t> in_ptr(nodes + 1, 0), in_src;
            for (std::size_t d = 0; d < nodes; ++d)
            {
                if (std::find(incoming[d].begin(), incoming[d].end(), static_cast<std::uint32_t>(d)) == incoming[d].end())
                    incoming[d].push_back(static_cast<std::uint32_t>(d));
                in_src.insert(in_src.end(), incoming[d].begin(), incoming[d].end());
                in_ptr[d + 1] = static_cast<std::uint32_t>(in_src.size());
            }
            const auto d_features = upload_f64(flatten(features)), d_w = upload_f64(flatten(parameters.seq_kernel_fp));
            const auto d_asrc = upload_f64(parameters.attn_src_kernel_fp), d_adst = upload_f64(parameters.attn_dst_kernel_fp);
            const auto d_bias = upload_f64(parameters.output_bias_fp);
            const auto d_es = upload_u32(edge_src), d_ed = upload_u32(edge_dst), d_ptr = upload_u32(in_ptr), d_in = upload_u32(in_src);
            gzk_gat_head head{};
            head.features = d_features->raw();
            head.input_width = static_cast<std::uint32_t>(inner);
            head.output_width = static_cast<std::uint32_t>(width);
            head.seq_kernel = d_w->raw();
            head.attn_src_kernel = d_asrc->raw();
            head.attn_dst_kernel = d_adst->raw();
            head.attn_src_bias = parameters.attn_src_bias_fp;
            head.attn_dst_bias = parameters.attn_dst_bias_fp;
            head.output_bias = apply_output_bias ? d_bias->raw() : nullptr;
            head.output_bias_count = apply_output_bias ? parameters.output_bias_fp.size() : 0;
            head.apply_activation = apply_activation ? 1 : 0;
            gzk_gat_graph graph{};
            graph.node_count = nodes;
            graph.edge_count = edges.size();
            graph.edge_src = d_es->raw();
            graph.edge_dst = d_ed->raw();
            graph.incoming_count = in_src.size();
            graph.incoming_ptr = d_ptr->raw();
            graph.incoming_src = d_in->raw();
            const std::size_t e_count = edges.empty() ? 1 : edges.size();
            DeviceBuffer h(ctx, GZK_KIND_F64, nodes * width), pre(ctx, GZK_KIND_F64, nodes * width), agg(ctx, GZK_KIND_F64, nodes * width);
            DeviceBuffer es(ctx, GZK_KIND_F64, nodes), ed(ctx, GZK_KIND_F64, nodes), m(ctx, GZK_KIND_F64, nodes), sum(ctx, GZK_KIND_F64, nodes),
                inv(ctx, GZK_KIND_F64, nodes);
            DeviceBuffer s(ctx, GZK_KIND_F64, e_count), z(ctx, GZK_KIND_F64, e_count), delta(ctx, GZK_KIND_F64, e_count), u(ctx, GZK_KIND_F64, e_count),
                alpha(ctx, GZK_KIND_F64, e_count);
            gzk_gat_trace out{h.raw(), es.raw(), ed.raw(), m.raw(), sum.raw(), inv.raw(), s.raw(), z.raw(), delta.raw(), u.raw(), alpha.raw(), pre.raw(), agg.raw()};
            ctx.check(gzk_gat_head_forward(ctx.raw(), &head, &graph, &out));
            auto vec = [](const DeviceBuffer& b, std::size_t count) {
                std::vector<double> v(count);
                if (count != 0) b.download(v.data(), count);
                return v;
            };
            auto mat = [&](const DeviceBuffer& b) {
                const auto v = vec(b, nodes * width);
                FloatMatrix out_m(nodes, std::vector<double>(width));
                for (std::size_t i = 0; i < nodes; ++i) std::copy(v.begin() + i * width, v.begin() + (i + 1) * width, out_m[i].begin());
                return out_m;
            };
            trace.H_prime = mat(h);
            trace.E_src = vec(es, nodes);
            trace.E_dst = vec(ed, nodes);
            trace.S = vec(s, edges.size());
            trace.Z = vec(z, edges.size());
            trace.M = vec(m, nodes);
            trace.Delta = vec(delta, edges.size());
            trace.U = vec(u, edges.size());
            trace.Sum = vec(sum, nodes);
            trace.inv = vec(inv, nodes);
            trace.alpha = vec(alpha, edges.size());
            trace.H_agg_pre_bias = mat(pre);
            trace.H_agg = mat(agg);
            return trace;
        }
    }
}
