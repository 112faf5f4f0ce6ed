// Byte codec of the proof object: the reference only COUNTS the bytes of a proof
// (proof_size_bytes, src/protocol/prover.cpp:3831-3905: length-prefixed metadata strings and
// block labels, 48-byte commitments, per domain bundle its opened values and witness, the
// external evaluations, the witness scalars and the external witness); this header writes
// and reads exactly those bytes, so that two backends' proofs can be compared as files.
// serialize_proof(p).size() == proof_size_bytes(p) by construction.
//
// Layout (all integers little-endian u64, field elements 32-byte little-endian canonical,
// points 48 bytes as produced by the caller's point serialiser):
//   u64 24, then 24 x (u64 length, bytes)                 public metadata, field order of PublicMetadata
//   u64 #blocks, then (u64 length, bytes) each            block_order
//   u64 #dynamic, then 48 bytes each                      dynamic commitments (names follow the fixed label order)
//   u64 #quotient, then 48 bytes each                     quotient commitments
//   u64 #bundles, per bundle: u64 #rows, per row (u64 #values, 32 bytes each), then 48 bytes witness
//   u64 #external, 32 bytes each;  u64 #scalars, 32 bytes each;  48 bytes external witness
// Names of commitments, rows, evaluations and scalars are not part of the stream (the
// reference does not count them: they are fixed by the protocol's label order); the reader
// takes them from a ProofSchema.  Pure host code, no GPU.
#pragma once

#include <array>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace gatzk_b200
{
    namespace protocol
    {
        using FieldBytes = std::array<std::uint8_t, 32>;
        using PointBytes = std::array<std::uint8_t, 48>;

        // include/gatzk/protocol/proof.hpp:42-67
        struct PublicMetadata
        {
            std::string protocol_id, dataset_name, task_type, report_unit, graph_count, L, hidden_profile, d_in_profile, K_out, C, batching_rule,
                subgraph_rule, self_loop_rule, edge_sort_rule, chunking_rule, model_arch_id, model_param_id, static_table_id, quant_cfg_id, domain_cfg,
                dim_cfg, encoding_id, padding_rule_id, degree_bound_id;
            std::array<const std::string*, 24> fields() const
            {
                return {&protocol_id,    &dataset_name,  &task_type,      &report_unit,   &graph_count,   &L,
                        &hidden_profile, &d_in_profile,  &K_out,          &C,             &batching_rule, &subgraph_rule,
                        &self_loop_rule, &edge_sort_rule, &chunking_rule, &model_arch_id, &model_param_id, &static_table_id,
                        &quant_cfg_id,   &domain_cfg,    &dim_cfg,        &encoding_id,   &padding_rule_id, &degree_bound_id};
            }
            std::array<std::string*, 24> fields()
            {
                return {&protocol_id,    &dataset_name,  &task_type,      &report_unit,   &graph_count,   &L,
                        &hidden_profile, &d_in_profile,  &K_out,          &C,             &batching_rule, &subgraph_rule,
                        &self_loop_rule, &edge_sort_rule, &chunking_rule, &model_arch_id, &model_param_id, &static_table_id,
                        &quant_cfg_id,   &domain_cfg,    &dim_cfg,        &encoding_id,   &padding_rule_id, &degree_bound_id};
            }
        };
        // proof.hpp:95-99 (the opening points are derived from the challenges and are not counted)
        struct DomainOpeningBundle
        {
            std::vector<std::pair<std::string, std::vector<FieldBytes>>> values;
            PointBytes witness{};
        };
        // proof.hpp:101-111
        struct Proof
        {
            PublicMetadata public_metadata;
            std::vector<std::string> block_order;
            std::vector<std::pair<std::string, PointBytes>> dynamic_commitments;
            std::vector<std::pair<std::string, PointBytes>> quotient_commitments;
            std::vector<std::pair<std::string, DomainOpeningBundle>> domain_openings;
            std::vector<std::pair<std::string, FieldBytes>> external_evaluations;
            std::vector<std::pair<std::string, FieldBytes>> witness_scalars;
            PointBytes external_witness{};
        };
        // the names the stream leaves out, in protocol order
        struct ProofSchema
        {
            std::vector<std::string> dynamic_commitments, quotient_commitments, external_evaluations, witness_scalars;
            std::vector<std::pair<std::string, std::vector<std::string>>> domain_openings;  // bundle name, row names
        };

        // prover.cpp:3831-3905
        inline std::size_t proof_size_bytes(const Proof& proof)
        {
            constexpr std::size_t kPrefix = 8, kField = 32, kPoint = 48;
            std::size_t total = kPrefix;
            for (const std::string* s : proof.public_metadata.fields()) total += kPrefix + s->size();
            total += kPrefix;
            for (const auto& label : proof.block_order) total += kPrefix + label.size();
            total += kPrefix + kPoint * proof.dynamic_commitments.size();
            total += kPrefix + kPoint * proof.quotient_commitments.size();
            total += kPrefix;
            for (const auto& bundle : proof.domain_openings)
            {
                total += kPrefix;
                for (const auto& row : bundle.second.values) total += kPrefix + kField * row.second.size();
                total += kPoint;
            }
            total += kPrefix + kField * proof.external_evaluations.size();
            total += kPrefix + kField * proof.witness_scalars.size();
            total += kPoint;
            return total;
        }

        namespace detail
        {
            inline void put_u64(std::vector<std::uint8_t>& out, std::uint64_t v)
            {
                for (int i = 0; i < 8; ++i) out.push_back(static_cast<std::uint8_t>(v >> (8 * i)));
            }
            template <typename Bytes>
            inline void put_bytes(std::vector<std::uint8_t>& out, const Bytes& b)
            {
                out.insert(out.end(), b.begin(), b.end());
            }
            struct Reader
            {
                const std::uint8_t* data;
                std::size_t size, at = 0;
                void need(std::size_t n) const
                {
                    if (n > size - at) throw std::runtime_error("proof stream ends early");
                }
                std::uint64_t u64()
                {
                    need(8);
                    std::uint64_t v = 0;
                    for (int i = 0; i < 8; ++i) v |= static_cast<std::uint64_t>(data[at + i]) << (8 * i);
                    at += 8;
                    return v;
                }
                std::size_t count(std::size_t item_bytes)
                {
                    const std::uint64_t n = u64();
                    if (item_bytes != 0 && n > (size - at) / item_bytes) throw std::runtime_error("proof stream: count exceeds the remaining bytes");
                    return static_cast<std::size_t>(n);
                }
                template <typename Bytes>
                Bytes bytes()
                {
                    Bytes b{};
                    need(b.size());
                    std::memcpy(b.data(), data + at, b.size());
                    at += b.size();
                    return b;
                }
                std::string text()
                {
                    const std::size_t n = count(1);
                    std::string s(reinterpret_cast<const char*>(data + at), n);
                    at += n;
                    return s;
                }
            };
            inline const std::string& name_at(const std::vector<std::string>& names, std::size_t i, const char* what)
            {
                if (i >= names.size()) throw std::runtime_error(std::string("proof stream holds more ") + what + " than the schema names");
                return names[i];
            }
        }

        inline std::vector<std::uint8_t> serialize_proof(const Proof& proof)
        {
            std::vector<std::uint8_t> out;
            out.reserve(proof_size_bytes(proof));
            detail::put_u64(out, 24);
            for (const std::string* s : proof.public_metadata.fields())
            {
                detail::put_u64(out, s->size());
                detail::put_bytes(out, *s);
            }
            detail::put_u64(out, proof.block_order.size());
            for (const auto& label : proof.block_order)
            {
                detail::put_u64(out, label.size());
                detail::put_bytes(out, label);
            }
            detail::put_u64(out, proof.dynamic_commitments.size());
            for (const auto& c : proof.dynamic_commitments) detail::put_bytes(out, c.second);
            detail::put_u64(out, proof.quotient_commitments.size());
            for (const auto& c : proof.quotient_commitments) detail::put_bytes(out, c.second);
            detail::put_u64(out, proof.domain_openings.size());
            for (const auto& bundle : proof.domain_openings)
            {
                detail::put_u64(out, bundle.second.values.size());
                for (const auto& row : bundle.second.values)
                {
                    detail::put_u64(out, row.second.size());
                    for (const auto& v : row.second) detail::put_bytes(out, v);
                }
                detail::put_bytes(out, bundle.second.witness);
            }
            detail::put_u64(out, proof.external_evaluations.size());
            for (const auto& e : proof.external_evaluations) detail::put_bytes(out, e.second);
            detail::put_u64(out, proof.witness_scalars.size());
            for (const auto& e : proof.witness_scalars) detail::put_bytes(out, e.second);
            detail::put_bytes(out, proof.external_witness);
            return out;
        }

        inline Proof deserialize_proof(const std::uint8_t* data, std::size_t size, const ProofSchema& schema)
        {
            detail::Reader in{data, size};
            Proof proof;
            if (in.u64() != 24) throw std::runtime_error("proof stream: expected 24 metadata strings");
            for (std::string* s : proof.public_metadata.fields()) *s = in.text();
            const std::size_t blocks = in.count(8);
            for (std::size_t i = 0; i < blocks; ++i) proof.block_order.push_back(in.text());
            const std::size_t dynamic = in.count(48);
            for (std::size_t i = 0; i < dynamic; ++i)
                proof.dynamic_commitments.emplace_back(detail::name_at(schema.dynamic_commitments, i, "dynamic commitments"), in.bytes<PointBytes>());
            const std::size_t quotient = in.count(48);
            for (std::size_t i = 0; i < quotient; ++i)
                proof.quotient_commitments.emplace_back(detail::name_at(schema.quotient_commitments, i, "quotient commitments"), in.bytes<PointBytes>());
            const std::size_t bundles = in.count(56);
            for (std::size_t b = 0; b < bundles; ++b)
            {
                if (b >= schema.domain_openings.size()) throw std::runtime_error("proof stream holds more opening bundles than the schema names");
                DomainOpeningBundle bundle;
                const std::size_t rows = in.count(8);
                for (std::size_t r = 0; r < rows; ++r)
                {
                    const std::string& name = detail::name_at(schema.domain_openings[b].second, r, "opened rows");
                    const std::size_t n = in.count(32);
                    std::vector<FieldBytes> values(n);
                    for (auto& v : values) v = in.bytes<FieldBytes>();
                    bundle.values.emplace_back(name, std::move(values));
                }
                bundle.witness = in.bytes<PointBytes>();
                proof.domain_openings.emplace_back(schema.domain_openings[b].first, std::move(bundle));
            }
            const std::size_t external = in.count(32);
            for (std::size_t i = 0; i < external; ++i)
                proof.external_evaluations.emplace_back(detail::name_at(schema.external_evaluations, i, "external evaluations"), in.bytes<FieldBytes>());
            const std::size_t scalars = in.count(32);
            for (std::size_t i = 0; i < scalars; ++i)
                proof.witness_scalars.emplace_back(detail::name_at(schema.witness_scalars, i, "witness scalars"), in.bytes<FieldBytes>());
            proof.external_witness = in.bytes<PointBytes>();
            if (in.at != size) throw std::runtime_error("proof stream has trailing bytes");
            return proof;
        }
    }
}
