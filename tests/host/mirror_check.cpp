// Runs the C++ host mirror (project_b200/host/gatzk_b200.hpp) on a GPU and checks its
// results against the CPU oracle (test infrastructure), value for value.
#include <cmath>
#include <cstdio>
#include <random>

#include "../../project_b200/host/gatzk_b200.hpp"

extern "C"
{
    int ora_root_of_unity(std::uint64_t size, std::uint8_t* out);
    int ora_bary_weights(const std::uint8_t* x, std::uint64_t size, std::uint8_t* out);
    int ora_eval_rotations(const std::uint8_t* columns, std::size_t k, std::size_t n, const std::uint8_t* weights, const std::uint64_t* rotations,
                           std::size_t p, std::size_t threads, std::uint8_t* out);
    int ora_commit_tau_eval(const std::uint8_t* columns, std::size_t k, std::size_t valid, const std::uint8_t* weights, std::size_t threads,
                            std::uint8_t* out);
    int ora_g1_mul_same_base(const std::uint8_t* base, const std::uint8_t* scalars, std::size_t count, std::uint8_t* out);
    int ora_horner(const std::uint8_t* coefficients, std::size_t n, const std::uint8_t* x, std::uint8_t* out);
    int ora_logup_accumulator(const std::uint8_t*, const std::uint8_t*, const std::uint8_t*, const std::uint8_t*, const std::uint8_t*, std::size_t,
                              const std::uint8_t*, std::size_t, std::uint8_t*);
    int ora_gat_head_forward(const double* features, std::size_t nodes, std::size_t inner, const double* seq_kernel, std::size_t width,
                             const double* attn_src, double bias_src, const double* attn_dst, double bias_dst, const double* out_bias,
                             std::size_t out_bias_count, int has_bias, int apply_activation, const std::uint32_t* edge_src,
                             const std::uint32_t* edge_dst, std::size_t edges, double* H_prime, double* E_src, double* E_dst, double* S, double* Z,
                             double* M, double* Delta, double* U, double* Sum, double* inv, double* alpha, double* H_agg_pre, double* H_agg);
}

using namespace gatzk_b200;
using algebra::FieldElement;

static int failures = 0;
#define CHECK(cond, what)                                  \
    do                                                     \
    {                                                      \
        if (!(cond))                                       \
        {                                                  \
            ++failures;                                    \
            std::printf("MISMATCH: %s\n", what);           \
        }                                                  \
    } while (0)

static std::vector<FieldElement> random_column(std::mt19937_64& rng, std::size_t n)
{
    std::vector<FieldElement> out(n);
    for (auto& v : out)
    {
        std::uint8_t b[32];
        for (int i = 0; i < 4; ++i)
        {
            const std::uint64_t w = rng();
            std::memcpy(b + 8 * i, &w, 8);
        }
        b[31] &= 0x3f;
        v = FieldElement::from_bytes(b);
    }
    return out;
}
static std::vector<std::uint8_t> flat(const std::vector<FieldElement>& v, std::size_t pad_to = 0)
{
    std::vector<std::uint8_t> out(std::max(v.size(), pad_to) * 32, 0);
    for (std::size_t i = 0; i < v.size(); ++i) std::memcpy(&out[32 * i], v[i].bytes(), 32);
    return out;
}

int main()
{
    Context ctx(0);
    std::mt19937_64 rng(2024);
    const std::size_t n = 1024, valid = 900;
    auto domain = algebra::RootOfUnityDomain::create(ctx, "edge", n);
    std::uint8_t w_ref[32];
    ora_root_of_unity(n, w_ref);
    CHECK(std::memcmp(domain->omega.bytes(), w_ref, 32) == 0, "root of unity");

    // generator of the standard BLS12-381 G1 subgroup (little-endian x || y)
    crypto::G1Point gen;
    {
        const char* gx = "17f1d3a73197d7942695638c4fa9ac0fc3688c4f9774b905a14e3a3f171bac586c55e83ff97a1aeffb3af00adb22c6bb";
        const char* gy = "08b3f481e3aaa0f1a09e30ed741d8ae4fcf5e095d5d00af600db18cb2c04b3edd03cc744a2888ae40caa232946c5e7e1";
        for (int i = 0; i < 48; ++i)
        {
            unsigned a, b;
            std::sscanf(gx + 2 * (47 - i), "%2x", &a);
            std::sscanf(gy + 2 * (47 - i), "%2x", &b);
            gen.affine[i] = static_cast<std::uint8_t>(a);
            gen.affine[48 + i] = static_cast<std::uint8_t>(b);
        }
    }
    const auto key = crypto::KZG::setup(11, gen);

    std::vector<std::vector<FieldElement>> columns;
    std::vector<algebra::Polynomial> polys;
    for (int k = 0; k < 4; ++k)
    {
        columns.push_back(random_column(rng, valid));
        polys.push_back(algebra::Polynomial::from_evaluations(ctx, "P_col" + std::to_string(k), columns.back(), domain));
    }
    const auto coeffs = random_column(rng, 300);
    polys.push_back(algebra::Polynomial::from_coefficients(ctx, "P_H", coeffs));
    std::vector<std::pair<std::string, const algebra::Polynomial*>> named;
    for (auto& p : polys) named.emplace_back(p.name, &p);

    // KZG::commit_batch
    const auto commitments = crypto::KZG::commit_batch(ctx, named, key);
    std::vector<std::uint8_t> weights(n * 32), cols_flat;
    ora_bary_weights(key.tau.bytes(), n, weights.data());
    for (int k = 0; k < 4; ++k)
    {
        const auto f = flat(columns[k]);
        cols_flat.insert(cols_flat.end(), f.begin(), f.end());
    }
    std::vector<std::uint8_t> want_evals(5 * 32), want_points(5 * 96);
    ora_commit_tau_eval(cols_flat.data(), 4, valid, weights.data(), 1, want_evals.data());
    const auto cflat = flat(coeffs);
    ora_horner(cflat.data(), coeffs.size(), key.tau.bytes(), &want_evals[4 * 32]);
    ora_g1_mul_same_base(gen.affine.data(), want_evals.data(), 5, want_points.data());
    for (int k = 0; k < 5; ++k)
    {
        CHECK(std::memcmp(commitments[k].tau_evaluation.bytes(), &want_evals[32 * k], 32) == 0, "commit tau evaluation");
        CHECK(std::memcmp(commitments[k].point.affine.data(), &want_points[96 * k], 96) == 0, "commitment point");
    }

    // PackedEvaluationBackend at a challenge and its rotation
    std::vector<std::pair<std::string, const algebra::Polynomial*>> eval_named(named.begin(), named.begin() + 4);
    algebra::PackedEvaluationBackend backend(ctx, domain, eval_named);
    const FieldElement z(0x9e3779b97f4a7c15ULL);
    const auto wz = domain->barycentric_weights_native(z);
    const auto opened = backend.evaluate_with_native_weight_rotations({"P_col2", "P_col0", "P_col3"}, wz, {0, 1});
    ora_bary_weights(z.bytes(), n, weights.data());
    std::vector<std::uint8_t> padded;
    for (int k : {2, 0, 3})
    {
        const auto f = flat(columns[k], n);
        padded.insert(padded.end(), f.begin(), f.end());
    }
    const std::uint64_t rot[2] = {0, 1};
    std::vector<std::uint8_t> want_open(2 * 3 * 32);
    ora_eval_rotations(padded.data(), 3, n, weights.data(), rot, 2, 1, want_open.data());
    for (int p = 0; p < 2; ++p)
        for (int k = 0; k < 3; ++k) CHECK(std::memcmp(opened[p][k].bytes(), &want_open[(p * 3 + k) * 32], 32) == 0, "opened value");

    // Polynomial::evaluate: direct hit on a domain point, and the tail beyond the stored length
    const FieldElement point5 = domain->omega.pow(5), point950 = domain->omega.pow(950);
    CHECK(polys[1].evaluate(ctx, point5) == columns[1][5], "evaluate at a domain point");
    CHECK(polys[1].evaluate(ctx, point950).is_zero(), "evaluate beyond the stored length");
    std::size_t shift = 0;
    CHECK(domain->rotation_shift(point950, &shift) && shift == 950, "rotation shift");
    CHECK(!domain->rotation_shift(z, &shift), "rotation shift of a non-member");

    // a LogUp accumulator through the protocol wrapper
    {
        const auto table = random_column(rng, n), query = random_column(rng, n), mult = random_column(rng, n);
        std::vector<FieldElement> qt(n, FieldElement::zero()), qq(n, FieldElement::zero());
        for (std::size_t i = 0; i < 700; ++i) qt[i] = FieldElement::one();
        for (std::size_t i = 0; i < valid; ++i) qq[i] = FieldElement::one();
        DeviceBuffer dt(ctx, GZK_KIND_FR, n), dq(ctx, GZK_KIND_FR, n), dm(ctx, GZK_KIND_FR, n), dqt(ctx, GZK_KIND_FR, n), dqq(ctx, GZK_KIND_FR, n);
        const auto ft = flat(table), fq = flat(query), fm = flat(mult), fqt = flat(qt), fqq = flat(qq);
        dt.upload(ft.data(), n);
        dq.upload(fq.data(), n);
        dm.upload(fm.data(), n);
        dqt.upload(fqt.data(), n);
        dqq.upload(fqq.data(), n);
        const FieldElement beta(123456789);
        const auto acc = protocol::build_logup_accumulator_with_active_count(ctx, dt, dq, dm, dqt, dqq, n, beta, valid);
        std::vector<std::uint8_t> got(n * 32), want(n * 32);
        acc->download(got.data(), n);
        ora_logup_accumulator(ft.data(), fq.data(), fm.data(), fqt.data(), fqq.data(), n, beta.bytes(), valid, want.data());
        CHECK(got == want, "LogUp accumulator");
    }

    // error behaviour: the reference throws
    bool threw = false;
    try
    {
        FieldElement::zero().inv();
    }
    catch (const std::runtime_error&)
    {
        threw = true;
    }
    CHECK(threw, "inverting zero throws");

    // fp64 forward of one attention head through the mirror of the reference's types
    {
        const std::size_t nodes = 70, inner = 13, width = 8;
        std::uniform_real_distribution<double> uni(-1.0, 1.0);
        model::FloatMatrix features(nodes, std::vector<double>(inner));
        for (auto& row : features)
            for (auto& v : row) v = uni(rng);
        model::AttentionHeadParameters params;
        params.seq_kernel_fp.assign(inner, std::vector<double>(width));
        for (auto& row : params.seq_kernel_fp)
            for (auto& v : row) v = 0.4 * uni(rng);
        params.attn_src_kernel_fp.resize(width);
        params.attn_dst_kernel_fp.resize(width);
        params.output_bias_fp.resize(width);
        for (std::size_t c = 0; c < width; ++c)
        {
            params.attn_src_kernel_fp[c] = uni(rng);
            params.attn_dst_kernel_fp[c] = uni(rng);
            params.output_bias_fp[c] = 0.1 * uni(rng);
        }
        params.attn_src_bias_fp = 0.03;
        params.attn_dst_bias_fp = -0.02;
        std::vector<model::Edge> edges;
        for (std::size_t e = 0; e < 400; ++e) edges.push_back({static_cast<std::size_t>(rng() % nodes), static_cast<std::size_t>(rng() % nodes)});
        const auto trace = model::attention_head_forward(ctx, features, edges, params, true, true);
        std::vector<double> xf, wf;
        for (const auto& row : features) xf.insert(xf.end(), row.begin(), row.end());
        for (const auto& row : params.seq_kernel_fp) wf.insert(wf.end(), row.begin(), row.end());
        std::vector<std::uint32_t> es(edges.size()), ed(edges.size());
        for (std::size_t e = 0; e < edges.size(); ++e)
        {
            es[e] = static_cast<std::uint32_t>(edges[e].src);
            ed[e] = static_cast<std::uint32_t>(edges[e].dst);
        }
        std::vector<double> H(nodes * width), Es(nodes), Ed(nodes), S(edges.size()), Z(edges.size()), M(nodes), D(edges.size()), U(edges.size()), Sum(nodes),
            Inv(nodes), A(edges.size()), Pre(nodes * width), Agg(nodes * width);
        CHECK(ora_gat_head_forward(xf.data(), nodes, inner, wf.data(), width, params.attn_src_kernel_fp.data(), params.attn_src_bias_fp,
                                   params.attn_dst_kernel_fp.data(), params.attn_dst_bias_fp, params.output_bias_fp.data(), width, 1, 1, es.data(),
                                   ed.data(), edges.size(), H.data(), Es.data(), Ed.data(), S.data(), Z.data(), M.data(), D.data(), U.data(), Sum.data(),
                                   Inv.data(), A.data(), Pre.data(), Agg.data()) == 0,
              "oracle forward runs");
        bool exact = true, close = true;
        double h_max = 0.0;
        for (double v : H) h_max = std::max(h_max, std::fabs(v));
        for (std::size_t i = 0; i < nodes; ++i)
        {
            exact = exact && trace.E_src[i] == Es[i] && trace.E_dst[i] == Ed[i] && trace.M[i] == M[i];
            close = close && std::fabs(trace.Sum[i] - Sum[i]) <= 4e-15 * Sum[i] && std::fabs(trace.inv[i] - Inv[i]) <= 4e-15 * Inv[i];
            for (std::size_t c = 0; c < width; ++c)
            {
                exact = exact && trace.H_prime[i][c] == H[i * width + c];
                close = close && std::fabs(trace.H_agg[i][c] - Agg[i * width + c]) <= 4e-15 * std::max(h_max, std::fabs(Agg[i * width + c]));
            }
        }
        for (std::size_t e = 0; e < edges.size(); ++e)
        {
            exact = exact && trace.S[e] == S[e] && trace.Z[e] == Z[e] && trace.Delta[e] == D[e];
            close = close && std::fabs(trace.U[e] - U[e]) <= 4e-15 * U[e] && std::fabs(trace.alpha[e] - A[e]) <= 4e-15 * A[e];
        }
        CHECK(exact, "head forward: H', E_src, E_dst, S, Z, M, Delta bit-identical");
        CHECK(close, "head forward: U, Sum, inv, alpha, H_agg within 4e-15");
    }
    // ---- verifier side: public columns of a domain evaluated as one group per point ----------------------
    {
        const std::size_t n = 1 << 11;
        auto domain = algebra::RootOfUnityDomain::create(ctx, "N", n);
        std::map<std::string, algebra::Polynomial> publics;
        std::vector<std::vector<FieldElement>> data;
        const char* names[3] = {"P_I", "P_Q_N", "P_src"};
        for (int k = 0; k < 3; ++k)
        {
            std::vector<FieldElement> column(n - 100 * k);  // stored prefixes of different lengths
            for (std::size_t i = 0; i < column.size(); ++i) column[i] = k == 1 ? FieldElement(i < 1500 ? 1 : 0) : FieldElement(rng() % 100000);
            data.push_back(column);
            publics.emplace(names[k], algebra::Polynomial::from_evaluations(ctx, names[k], column, domain));
        }
        protocol::PublicEvaluationBackendRegistry registry(ctx, publics);
        const FieldElement z(0x51ed270b5ULL);
        std::vector<std::uint8_t> weights(n * 32);
        ora_bary_weights(z.bytes(), n, weights.data());
        bool same = true;
        for (int k = 0; k < 3; ++k)
        {
            const auto padded = flat(data[k], n);
            const std::uint64_t rot = 0;
            std::uint8_t want[32];
            ora_eval_rotations(padded.data(), 1, n, weights.data(), &rot, 1, 1, want);
            same = same && registry.eval(names[k], z) == FieldElement::from_bytes(want);
        }
        CHECK(same, "verifier public columns at a challenge point");
        CHECK(registry.group_evaluations() == 1, "one packed evaluation serves the whole domain group");
        // a point of the domain takes the direct-index branch: column value at that row, zero beyond the stored prefix
        const FieldElement on_domain = domain->omega.pow(1950);
        CHECK(registry.eval("P_I", on_domain) == data[0][1950], "direct index inside the stored prefix");
        CHECK(registry.eval("P_src", on_domain) == FieldElement::zero(), "direct index beyond the stored prefix");
    }
    std::printf(failures == 0 ? "OK\n" : "FAILED %d\n", failures);
    return failures == 0 ? 0 : 1;
}
