// Host-only check of the proof byte codec: the size formula of the reference
// (src/protocol/prover.cpp:3831-3905) on a proof with the label counts of the small
// citation-graph configuration (8 hidden heads, 1 output head, 1 hidden layer), the
// round trip through bytes, and the error paths of the reader.
#include <cstdio>
#include <random>

#include "../../project_b200/host/proof_codec.hpp"

using namespace gatzk_b200::protocol;

int main()
{
    std::mt19937_64 rng(7);
    auto field = [&] {
        FieldBytes f{};
        for (auto& b : f) b = static_cast<std::uint8_t>(rng());
        f[31] &= 0x3f;
        return f;
    };
    auto point = [&] {
        PointBytes p{};
        for (auto& b : p) b = static_cast<std::uint8_t>(rng());
        return p;
    };
    const std::size_t H = 8, K = 1, L = 1;
    const std::size_t dynamic = 5 + 82 * H + 5 * L + 68 * K + (K > 1 ? 2 : 0);  // challenges.cpp:396-507
    const std::size_t bundle_labels[7] = {5, 43 * H + 36 * K, 3 * H, 15 * H, 3 * L + 3 * K, 9 * K, 18 * H + 17 * K + L};
    const char* bundle_names[7] = {"FH", "edge", "in", "d_h", "cat", "C", "N"};

    Proof proof;
    ProofSchema schema;
    std::size_t meta_bytes = 0;
    int salt = 0;
    for (std::string* s : proof.public_metadata.fields())
    {
        *s = std::string(3 + (salt * 7) % 40, static_cast<char>('a' + salt % 26));
        meta_bytes += 8 + s->size();
        ++salt;
    }
    std::size_t block_bytes = 0;
    for (int i = 0; i < 9; ++i)
    {
        proof.block_order.push_back("block_" + std::to_string(i));
        block_bytes += 8 + proof.block_order.back().size();
    }
    for (std::size_t i = 0; i < dynamic; ++i)
    {
        schema.dynamic_commitments.push_back("P_dyn_" + std::to_string(i));
        proof.dynamic_commitments.emplace_back(schema.dynamic_commitments.back(), point());
    }
    for (int i = 0; i < 7; ++i)
    {
        schema.quotient_commitments.push_back(std::string("t_") + bundle_names[i]);
        proof.quotient_commitments.emplace_back(schema.quotient_commitments.back(), point());
    }
    std::size_t rows_total = 0;
    for (int b = 0; b < 7; ++b)
    {
        DomainOpeningBundle bundle;
        std::vector<std::string> names;
        for (std::size_t r = 0; r < bundle_labels[b] + 1; ++r)  // the labels and the quotient row, two opening points each
        {
            names.push_back(std::string(bundle_names[b]) + "_row_" + std::to_string(r));
            bundle.values.emplace_back(names.back(), std::vector<FieldBytes>{field(), field()});
        }
        rows_total += names.size();
        bundle.witness = point();
        schema.domain_openings.emplace_back(bundle_names[b], names);
        proof.domain_openings.emplace_back(bundle_names[b], bundle);
    }
    const std::size_t ext = 40, scalars = 24;
    for (std::size_t i = 0; i < ext; ++i)
    {
        schema.external_evaluations.push_back("mu_" + std::to_string(i));
        proof.external_evaluations.emplace_back(schema.external_evaluations.back(), field());
    }
    for (std::size_t i = 0; i < scalars; ++i)
    {
        schema.witness_scalars.push_back("s_" + std::to_string(i));
        proof.witness_scalars.emplace_back(schema.witness_scalars.back(), field());
    }
    proof.external_witness = point();

    int failures = 0;
    auto check = [&](bool ok, const char* what) {
        if (!ok)
        {
            ++failures;
            std::printf("MISMATCH: %s\n", what);
        }
    };
    // the closed form: 8 + meta + 8 + blocks + 8 + 48*#dyn + 8 + 48*7 + 8 + sum_bundles[8 + rows*(8 + 2*32) + 48] + 8 + 32*#ext + 8 + 32*#scalars + 48
    const std::size_t closed = 8 + meta_bytes + 8 + block_bytes + 8 + 48 * dynamic + 8 + 48 * 7 + 8 + (7 * (8 + 48) + rows_total * 72) + 8 + 32 * ext + 8 +
                               32 * scalars + 48;
    check(dynamic == 734, "734 dynamic commitments for 8 hidden heads, 1 output head, 1 layer");
    check(rows_total == 706 + 7, "706 opened labels plus one quotient row per bundle");
    // everything except metadata, block labels, external evaluations and witness scalars: 87400 of the published 90755 bytes
    check(closed - meta_bytes - block_bytes - 32 * (ext + scalars) == 87400, "fixed part of the small-configuration proof is 87400 bytes");
    check(proof_size_bytes(proof) == closed, "proof_size_bytes equals the closed form");
    const std::vector<std::uint8_t> bytes = serialize_proof(proof);
    check(bytes.size() == closed, "serialised length equals proof_size_bytes");
    const Proof back = deserialize_proof(bytes.data(), bytes.size(), schema);
    check(serialize_proof(back) == bytes, "round trip is byte-identical");
    check(back.dynamic_commitments[733].first == "P_dyn_733" && back.dynamic_commitments[733].second == proof.dynamic_commitments[733].second,
          "names come back from the schema, values from the stream");
    check(back.domain_openings[1].second.values.size() == 43 * H + 36 * K + 1, "edge bundle row count");
    check(back.public_metadata.degree_bound_id == proof.public_metadata.degree_bound_id, "metadata strings");
    bool threw = false;
    try
    {
        deserialize_proof(bytes.data(), bytes.size() - 1, schema);
    }
    catch (const std::runtime_error&)
    {
        threw = true;
    }
    check(threw, "a truncated stream is rejected");
    threw = false;
    std::vector<std::uint8_t> longer = bytes;
    longer.push_back(0);
    try
    {
        deserialize_proof(longer.data(), longer.size(), schema);
    }
    catch (const std::runtime_error&)
    {
        threw = true;
    }
    check(threw, "trailing bytes are rejected");
    threw = false;
    std::vector<std::uint8_t> bad = bytes;
    bad[0] = 23;
    try
    {
        deserialize_proof(bad.data(), bad.size(), schema);
    }
    catch (const std::runtime_error&)
    {
        threw = true;
    }
    check(threw, "a wrong metadata count is rejected");
    std::printf(failures == 0 ? "OK\n" : "FAILED %d\n", failures);
    return failures == 0 ? 0 : 1;
}
