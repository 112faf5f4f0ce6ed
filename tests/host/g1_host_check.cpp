// Host-side check of the XYZZ point formulas used by the CUDA kernels against the
// oracle's Jacobian implementation (affine results must agree exactly).
#include <cstdio>
#include <cstring>
#include <random>

#include "../../oracle/g1.hpp"
#include "../../project_b200/csrc/g1.cuh"

static gzk::Fp to_dev(const oracle::Fp& v)
{
    gzk::Fp f;
    std::memcpy(f.l, v.v.w.data(), 48);  // both sides: Montgomery form, R = 2^384
    return f;
}
static gzk::G1Affine to_dev(const oracle::G1Affine& a)
{
    if (a.infinity) return gzk::G1Affine::infinity();
    gzk::G1Affine p;
    p.x = to_dev(a.x);
    p.y = to_dev(a.y);
    return p;
}
static bool same(const gzk::G1Affine& d, const oracle::G1Affine& o)
{
    if (o.infinity) return d.is_infinity();
    return std::memcmp(d.x.l, o.x.v.w.data(), 48) == 0 && std::memcmp(d.y.l, o.y.v.w.data(), 48) == 0;
}

int main()
{
    using namespace oracle;
    std::mt19937_64 rng(99);
    G1Affine gen;
    {
        // generator from its published coordinates, little-endian bytes built from the hex
        const char* gx = "17f1d3a73197d7942695638c4fa9ac0fc3688c4f9774b905a14e3a3f171bac586c55e83ff97a1aeffb3af00adb22c6bb";
        const char* gy = "08b3f481e3aaa0f1a09e30ed741d8ae4fcf5e095d5d00af600db18cb2c04b3edd03cc744a2888ae40caa232946c5e7e1";
        auto parse = [](const char* hex) {
            std::uint8_t le[48];
            for (int i = 0; i < 48; ++i)
            {
                unsigned v;
                std::sscanf(hex + 2 * (47 - i), "%2x", &v);
                le[i] = static_cast<std::uint8_t>(v);
            }
            return Fp::from_le_bytes(le);
        };
        gen.x = parse(gx);
        gen.y = parse(gy);
        gen.infinity = false;
    }
    if (!on_curve(gen)) { std::printf("generator not on curve\n"); return 1; }
    const G1 G = G1::from_affine(gen);
    int failures = 0;
    for (int iter = 0; iter < 60; ++iter)
    {
        const Fr k1 = Fr::from_u64(rng() | 1), k2 = Fr::from_u64(rng() | 1) * Fr::from_u64(rng());
        const G1 P = G.mul(k1), Q = G.mul(k2);
        const G1Affine pa = P.to_affine(), qa = Q.to_affine();
        const gzk::G1Affine dp = to_dev(pa), dq = to_dev(qa);
        const gzk::G1Xyzz xp = gzk::G1Xyzz::from_affine(dp), xq = gzk::G1Xyzz::from_affine(dq);
        if (!same(gzk::g1_to_affine(gzk::g1_add_mixed(xp, dq)), P.add(Q).to_affine())) { ++failures; std::printf("mixed add\n"); }
        if (!same(gzk::g1_to_affine(gzk::g1_add_mixed(xp, dq, true)), P.add(Q.neg()).to_affine())) { ++failures; std::printf("mixed sub\n"); }
        if (!same(gzk::g1_to_affine(gzk::g1_add_mixed(xp, dp)), P.dbl().to_affine())) { ++failures; std::printf("mixed add as doubling\n"); }
        if (!gzk::g1_add_mixed(xp, dp, true).is_infinity()) { ++failures; std::printf("P - P\n"); }
        // general XYZZ operands: (P+Q) + (P+P)
        const gzk::G1Xyzz s1 = gzk::g1_add_mixed(xp, dq), s2 = gzk::g1_double(xp);
        if (!same(gzk::g1_to_affine(gzk::g1_add(s1, s2)), P.add(Q).add(P.dbl()).to_affine())) { ++failures; std::printf("full add\n"); }
        if (!same(gzk::g1_to_affine(gzk::g1_add(s1, s1)), P.add(Q).dbl().to_affine())) { ++failures; std::printf("full add as doubling\n"); }
        if (!same(gzk::g1_to_affine(gzk::g1_double(s1)), P.add(Q).dbl().to_affine())) { ++failures; std::printf("doubling\n"); }
        if (!same(gzk::g1_to_affine(gzk::g1_double_affine(dq)), Q.dbl().to_affine())) { ++failures; std::printf("affine doubling\n"); }
        if (!same(gzk::g1_to_affine(gzk::g1_add(gzk::G1Xyzz::infinity(), xq)), qa)) { ++failures; std::printf("O + Q\n"); }
        if (!same(gzk::g1_to_affine(gzk::g1_add_mixed(gzk::G1Xyzz::infinity(), dq)), qa)) { ++failures; std::printf("O + q\n"); }
        if (!same(gzk::g1_to_affine(gzk::g1_add_mixed(xp, gzk::G1Affine::infinity())), pa)) { ++failures; std::printf("P + o\n"); }
        if (failures > 5) break;
    }
    std::printf(failures == 0 ? "OK\n" : "FAILED %d\n", failures);
    return failures == 0 ? 0 : 1;
}
