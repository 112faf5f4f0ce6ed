// Host-side check of the carry-chain field arithmetic used by the CUDA kernels:
// the same header compiles for the host with an emulated carry flag and is
// compared here against the 64-bit oracle implementation on random inputs.
#include <cstdio>
#include <cstring>
#include <random>

#include "../../oracle/field.hpp"
#include "../../project_b200/csrc/field.cuh"

template <typename Cfg, typename OFe, size_t N64>
int check_field(const char* name, std::mt19937_64& rng)
{
    using F = gzk::Fe<Cfg>;
    constexpr int N = Cfg::N;
    int failures = 0;
    auto random_canonical = [&](int mode) {
        oracle::BigInt<N64> b;
        for (;;)
        {
            for (auto& w : b.w) w = mode == 1 ? ~0ULL : (mode == 2 ? 0ULL : rng());
            if (mode == 1)
            {
                b = OFe::P().modulus;
                b.w[0] -= 1 + (rng() % 3);
                return b;
            }
            if (mode == 2)
            {
                b.w[0] = rng() % 3;
                return b;
            }
            b.w[N64 - 1] &= (~0ULL) >> (64 * N64 - OFe::P().modulus.bit_length());
            if (oracle::cmp(b, OFe::P().modulus) < 0) return b;
        }
    };
    auto to_dev = [&](const oracle::BigInt<N64>& b) {
        F f;
        std::memcpy(f.l, b.w.data(), 4 * N);
        return f;
    };
    auto eq = [&](const F& f, const oracle::BigInt<N64>& b) { return std::memcmp(f.l, b.w.data(), 4 * N) == 0; };
    for (int iter = 0; iter < 20000; ++iter)
    {
        const auto ca = random_canonical(iter % 7 == 0 ? 1 : (iter % 11 == 0 ? 2 : 0));
        const auto cb = random_canonical(iter % 5 == 0 ? 1 : (iter % 13 == 0 ? 2 : 0));
        const OFe oa = OFe::from_canonical(ca), ob = OFe::from_canonical(cb);
        const F a = gzk::to_mont(to_dev(ca)), b = gzk::to_mont(to_dev(cb));
        if (!eq(a, oa.v)) { ++failures; std::printf("%s to_mont mismatch\n", name); }
        if (!eq(gzk::mul(a, b), (oa * ob).v)) { ++failures; std::printf("%s mul mismatch\n", name); }
        if (!eq(gzk::add(a, b), (oa + ob).v)) { ++failures; std::printf("%s add mismatch\n", name); }
        if (!eq(gzk::sub(a, b), (oa - ob).v)) { ++failures; std::printf("%s sub mismatch\n", name); }
        if (!eq(gzk::from_mont(a), ca)) { ++failures; std::printf("%s from_mont mismatch\n", name); }
        if (iter < 6000 && !oa.is_zero())
        {
            if (!eq(gzk::inv(a), oa.inv().v)) { ++failures; std::printf("%s inv mismatch\n", name); }
            if (!eq(gzk::inv_fermat(a), oa.inv().v)) { ++failures; std::printf("%s fermat inv mismatch\n", name); }
            if (!eq(gzk::inv_binary(a), oa.inv().v)) { ++failures; std::printf("%s binary inv mismatch\n", name); }
            if (!eq(gzk::pow_u64(a, 0x123456789abcdefULL + iter), oa.pow(0x123456789abcdefULL + iter).v)) { ++failures; std::printf("%s pow mismatch\n", name); }
        }
        if (failures > 5) return failures;
    }
    // inversion of sparse values: single bits, and the modulus minus a single bit, taken as
    // Montgomery representations directly (any residue is one)
    for (int bit = 0; bit < Cfg::BITS; ++bit)
    {
        for (int variant = 0; variant < 2; ++variant)
        {
            oracle::BigInt<N64> c{};
            c.w[bit / 64] = 1ULL << (bit % 64);
            if (variant == 1)
            {
                oracle::BigInt<N64> m = OFe::P().modulus, d{};
                unsigned __int128 borrow = 0;
                for (int i = 0; i < N64; ++i)
                {
                    const unsigned __int128 w = static_cast<unsigned __int128>(m.w[i]) - c.w[i] - borrow;
                    d.w[i] = static_cast<uint64_t>(w);
                    borrow = (w >> 64) & 1;
                }
                c = d;
            }
            if (oracle::cmp(c, OFe::P().modulus) >= 0) continue;
            OFe o;
            o.v = c;
            if (o.is_zero()) continue;
            if (!eq(gzk::inv(to_dev(c)), o.inv().v)) { ++failures; std::printf("%s sparse inv mismatch (bit %d, variant %d)\n", name, bit, variant); }
        }
        if (failures > 5) return failures;
    }
    if (!eq(F::one(), OFe::one().v)) { ++failures; std::printf("%s R1 constant wrong\n", name); }
    if (!eq(F::r2(), OFe::P().r2)) { ++failures; std::printf("%s R2 constant wrong\n", name); }
    return failures;
}

int check_wide(std::mt19937_64& rng)
{
    // sum_i w_i(Montgomery) * f_i(canonical) accumulated as plain 17-limb integers,
    // reduced once: must equal the Montgomery form of the true field sum.
    using namespace gzk;
    int failures = 0;
    for (int trial = 0; trial < 600; ++trial)
    {
        uint32_t acc[17] = {};
        gzk::WideAcc wacc;
        wacc.clear();
        gzk::WideAcc64 wacc64;
        wacc64.clear();
        oracle::Fr want = oracle::Fr::zero();
        const int terms = 1 + static_cast<int>(rng() % (trial % 50 == 0 ? 5000 : 40));
        for (int t = 0; t < terms; ++t)
        {
            oracle::BigInt<4> cw, cf;
            for (;;)
            {
                for (auto& w : cw.w) w = (trial % 3 == 0) ? ~0ULL : rng();
                for (auto& w : cf.w) w = (trial % 3 == 0) ? ~0ULL : rng();
                cw.w[3] >>= 1;
                cf.w[3] >>= 1;
                if (trial % 3 == 0)
                {
                    cw = oracle::FrTag::params().modulus;
                    cw.w[0] -= 1;
                    cf = cw;
                }
                if (oracle::cmp(cw, oracle::FrTag::params().modulus) < 0 && oracle::cmp(cf, oracle::FrTag::params().modulus) < 0) break;
            }
            const oracle::Fr ow = oracle::Fr::from_canonical(cw), of = oracle::Fr::from_canonical(cf);
            want += ow * of;
            uint32_t wl[8], fl[8], prod[16];
            std::memcpy(wl, ow.v.w.data(), 32);  // Montgomery limbs
            std::memcpy(fl, cf.w.data(), 32);    // canonical limbs
            mul_wide<8>(wl, fl, prod);
            // cross-check the wide product against 128-bit schoolbook
            {
                unsigned __int128 carry = 0;
                uint32_t ref[16] = {};
                for (int k = 0; k < 16; ++k)
                {
                    unsigned __int128 s = carry;
                    carry = 0;
                    for (int i = 0; i <= k; ++i)
                    {
                        const int j = k - i;
                        if (i < 8 && j < 8)
                        {
                            s += static_cast<uint64_t>(wl[i]) * fl[j];
                        }
                    }
                    ref[k] = static_cast<uint32_t>(s);
                    carry = s >> 32;
                }
                if (std::memcmp(ref, prod, 64) != 0) { ++failures; std::printf("mul_wide mismatch\n"); }
            }
            acc_add<17, 16>(acc, prod);
            wacc.mac<8>(wl, fl);
            wacc64.mac<8>(wl, fl);
        }
        {
            uint32_t folded[17];
            wacc64.fold(folded);
            if (std::memcmp(folded, acc, sizeof(acc)) != 0) { ++failures; std::printf("WideAcc64 mismatch\n"); }
        }
        {
            uint32_t folded[17];
            wacc.fold(folded);
            if (std::memcmp(folded, acc, sizeof(acc)) != 0) { ++failures; std::printf("WideAcc mismatch\n"); }
        }
        const Fr reduced = mul(redc_wide<FrCfg, 9>(acc), fr_const_2_544());
        if (std::memcmp(reduced.l, want.v.w.data(), 32) != 0) { ++failures; std::printf("redc_wide mismatch\n"); }
        if (failures > 5) break;
    }
    return failures;
}

int main()
{
    std::mt19937_64 rng(12345);
    int failures = 0;
    failures += check_field<gzk::FrCfg, oracle::Fr, 4>("Fr", rng);
    failures += check_field<gzk::FpCfg, oracle::Fp, 6>("Fp", rng);
    failures += check_wide(rng);
    std::printf(failures == 0 ? "OK\n" : "FAILED %d\n", failures);
    return failures == 0 ? 0 : 1;
}
