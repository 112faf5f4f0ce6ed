// Montgomery prime fields on 32-bit limbs for sm_100a: BLS12-381 Fr (8 limbs)
// and Fp (12 limbs), the fields the reference prover works in
// (include/gatzk/algebra/field.hpp:19-25 initialises mcl for BLS12_381).
//
// Multiplication keeps two accumulators, one for products that land on even
// limb boundaries and one for products that land on odd boundaries, so that
// each row of the schoolbook product is a single mad.lo.cc / madc.hi.cc carry
// chain with no carry conflicts between neighbouring products.  After every
// row the value is divided by 2^32 by swapping the roles of the two
// accumulators (the odd-aligned one becomes even-aligned).
#pragma once

#include "mp.cuh"

namespace gzk
{
    struct FrCfg
    {
        static constexpr int N = 8;
        static constexpr int BITS = 255;
        static constexpr uint32_t INV = 0xffffffffu;  // -r^-1 mod 2^32
        GZK_HD static constexpr uint32_t mod(int i)
        {
            constexpr uint32_t m[8] = {0x00000001u, 0xffffffffu, 0xfffe5bfeu, 0x53bda402u,
                                       0x09a1d805u, 0x3339d808u, 0x299d7d48u, 0x73eda753u};
            return m[i];
        }
        GZK_HD static constexpr uint32_t r1(int i)  // 2^256 mod r
        {
            constexpr uint32_t m[8] = {0xfffffffeu, 0x00000001u, 0x00034802u, 0x5884b7fau,
                                       0xecbc4ff5u, 0x998c4fefu, 0xacc5056fu, 0x1824b159u};
            return m[i];
        }
        GZK_HD static constexpr uint32_t r2(int i)  // 2^512 mod r
        {
            constexpr uint32_t m[8] = {0xf3f29c6du, 0xc999e990u, 0x87925c23u, 0x2b6cedcbu,
                                       0x7254398fu, 0x05d31496u, 0x9f59ff11u, 0x0748d9d9u};
            return m[i];
        }
    };

    struct FpCfg
    {
        static constexpr int N = 12;
        static constexpr int BITS = 381;
        static constexpr uint32_t INV = 0xfffcfffdu;  // -p^-1 mod 2^32
        GZK_HD static constexpr uint32_t mod(int i)
        {
            constexpr uint32_t m[12] = {0xffffaaabu, 0xb9feffffu, 0xb153ffffu, 0x1eabfffeu, 0xf6b0f624u, 0x6730d2a0u,
                                        0xf38512bfu, 0x64774b84u, 0x434bacd7u, 0x4b1ba7b6u, 0x397fe69au, 0x1a0111eau};
            return m[i];
        }
        GZK_HD static constexpr uint32_t r1(int i)  // 2^384 mod p
        {
            constexpr uint32_t m[12] = {0x0002fffdu, 0x76090000u, 0xc40c0002u, 0xebf4000bu, 0x53c758bau, 0x5f489857u,
                                        0x70525745u, 0x77ce5853u, 0xa256ec6du, 0x5c071a97u, 0xfa80e493u, 0x15f65ec3u};
            return m[i];
        }
        GZK_HD static constexpr uint32_t r2(int i)  // 2^768 mod p
        {
            constexpr uint32_t m[12] = {0x1c341746u, 0xf4df1f34u, 0x09d104f1u, 0x0a76e6a6u, 0x4c95b6d5u, 0x8de5476cu,
                                        0x939d83c0u, 0x67eb88a9u, 0xb519952du, 0x9a793e85u, 0x92cae3aau, 0x11988fe5u};
            return m[i];
        }
    };

    template <typename Cfg>
    struct Fe
    {
        static constexpr int N = Cfg::N;
        uint32_t l[N];

        GZK_HD static Fe zero()
        {
            Fe o;
#pragma unroll
            for (int i = 0; i < N; ++i) o.l[i] = 0;
            return o;
        }
        // Montgomery form of 1.
        GZK_HD static Fe one()
        {
            Fe o;
#pragma unroll
            for (int i = 0; i < N; ++i) o.l[i] = Cfg::r1(i);
            return o;
        }
        GZK_HD static Fe r2()
        {
            Fe o;
#pragma unroll
            for (int i = 0; i < N; ++i) o.l[i] = Cfg::r2(i);
            return o;
        }
        GZK_HD static Fe modulus()
        {
            Fe o;
#pragma unroll
            for (int i = 0; i < N; ++i) o.l[i] = Cfg::mod(i);
            return o;
        }
        GZK_HD bool is_zero() const
        {
            uint32_t acc = 0;
#pragma unroll
            for (int i = 0; i < N; ++i) acc |= l[i];
            return acc == 0;
        }
        GZK_HD bool operator==(const Fe& o) const
        {
            uint32_t acc = 0;
#pragma unroll
            for (int i = 0; i < N; ++i) acc |= l[i] ^ o.l[i];
            return acc == 0;
        }
        GZK_HD bool operator!=(const Fe& o) const { return !(*this == o); }
    };

    // r = a - modulus if a >= modulus else a  (input < 2*modulus, N limbs).
    template <typename Cfg>
    GZK_HD Fe<Cfg> reduce_once(const Fe<Cfg>& a)
    {
        constexpr int N = Cfg::N;
        Fe<Cfg> t;
        t.l[0] = mp::sub_cc(a.l[0], Cfg::mod(0));
#pragma unroll
        for (int i = 1; i < N; ++i) t.l[i] = mp::subc_cc(a.l[i], Cfg::mod(i));
        const uint32_t borrow = mp::subc(0, 0);  // 0 or 0xffffffff
        Fe<Cfg> o;
#pragma unroll
        for (int i = 0; i < N; ++i) o.l[i] = borrow ? a.l[i] : t.l[i];
        return o;
    }

    template <typename Cfg>
    GZK_HD Fe<Cfg> add(const Fe<Cfg>& a, const Fe<Cfg>& b)
    {
        constexpr int N = Cfg::N;
        // Both moduli leave the top bit of the top limb free, so a+b fits N limbs.
        Fe<Cfg> s;
        s.l[0] = mp::add_cc(a.l[0], b.l[0]);
#pragma unroll
        for (int i = 1; i < N - 1; ++i) s.l[i] = mp::addc_cc(a.l[i], b.l[i]);
        s.l[N - 1] = mp::addc(a.l[N - 1], b.l[N - 1]);
        return reduce_once(s);
    }

    template <typename Cfg>
    GZK_HD Fe<Cfg> sub(const Fe<Cfg>& a, const Fe<Cfg>& b)
    {
        constexpr int N = Cfg::N;
        Fe<Cfg> d;
        d.l[0] = mp::sub_cc(a.l[0], b.l[0]);
#pragma unroll
        for (int i = 1; i < N; ++i) d.l[i] = mp::subc_cc(a.l[i], b.l[i]);
        const uint32_t borrow = mp::subc(0, 0);
        Fe<Cfg> o;
        o.l[0] = mp::add_cc(d.l[0], borrow & Cfg::mod(0));
#pragma unroll
        for (int i = 1; i < N - 1; ++i) o.l[i] = mp::addc_cc(d.l[i], borrow & Cfg::mod(i));
        o.l[N - 1] = mp::addc(d.l[N - 1], borrow & Cfg::mod(N - 1));
        return o;
    }

    template <typename Cfg>
    GZK_HD Fe<Cfg> neg(const Fe<Cfg>& a)
    {
        return sub(Fe<Cfg>::zero(), a);
    }

    namespace detail
    {
        // P (N+1 limbs, even-aligned) += sum over even j of x[j] * y * 2^(32 j);
        // the carry out of the chain is added to P[N].
        template <typename Cfg, typename X>
        GZK_HD void mad_even(uint32_t* P, X x, uint32_t y)
        {
            constexpr int N = Cfg::N;
            P[0] = mp::mad_lo_cc(x(0), y, P[0]);
            P[1] = mp::madc_hi_cc(x(0), y, P[1]);
#pragma unroll
            for (int j = 2; j < N; j += 2)
            {
                P[j] = mp::madc_lo_cc(x(j), y, P[j]);
                P[j + 1] = mp::madc_hi_cc(x(j), y, P[j + 1]);
            }
            P[N] = mp::addc(P[N], 0);
        }
        // Q (N limbs, odd-aligned) += sum over odd j of x[j] * y * 2^(32 (j-1));
        // the caller guarantees that the sum fits N limbs.
        template <typename Cfg, typename X>
        GZK_HD void mad_odd(uint32_t* Q, X x, uint32_t y)
        {
            constexpr int N = Cfg::N;
            Q[0] = mp::mad_lo_cc(x(1), y, Q[0]);
            Q[1] = mp::madc_hi_cc(x(1), y, Q[1]);
#pragma unroll
            for (int j = 3; j < N - 1; j += 2)
            {
                Q[j - 1] = mp::madc_lo_cc(x(j), y, Q[j - 1]);
                Q[j] = mp::madc_hi_cc(x(j), y, Q[j]);
            }
            Q[N - 2] = mp::madc_lo_cc(x(N - 1), y, Q[N - 2]);
            Q[N - 1] = mp::madc_hi(x(N - 1), y, Q[N - 1]);
        }

        template <typename Cfg>
        struct ModLimb
        {
            GZK_HD constexpr uint32_t operator()(int i) const { return Cfg::mod(i); }
        };
        struct ArrLimb
        {
            const uint32_t* p;
            GZK_HD uint32_t operator()(int i) const { return p[i]; }
        };

        // One Montgomery row: on entry `P` holds the previous odd-aligned
        // accumulator (N limbs) and `Q` the previous even-aligned one (N+1
        // limbs, limb 0 already zero).  The running value is divided by 2^32 by
        // swapping roles, then a*bi and m*modulus are added.
        template <typename Cfg>
        GZK_HD void mont_row(uint32_t* P, uint32_t* Q, const uint32_t* a, uint32_t bi)
        {
            constexpr int N = Cfg::N;
            // value/2^32 = (Q >> 32) + P: limb Q[1] joins P[0]; the carry of that
            // addition has weight 2^32, which is exactly limb 0 of the new
            // odd-aligned accumulator, so it feeds the next chain.
            P[0] = mp::add_cc(P[0], Q[1]);
            // new odd-aligned accumulator = (Q >> 64) + odd limbs of a times bi
#pragma unroll
            for (int j = 1; j < N - 1; j += 2)
            {
                Q[j - 1] = mp::madc_lo_cc(a[j], bi, Q[j + 1]);
                Q[j] = mp::madc_hi_cc(a[j], bi, Q[j + 2]);
            }
            Q[N - 2] = mp::madc_lo_cc(a[N - 1], bi, Q[N]);
            Q[N - 1] = mp::madc_hi(a[N - 1], bi, 0);
            Q[N] = 0;
            P[N] = 0;
            mad_even<Cfg>(P, ArrLimb{a}, bi);
            const uint32_t m = mp::mul_lo(P[0], Cfg::INV);
            mad_odd<Cfg>(Q, ModLimb<Cfg>{}, m);
            mad_even<Cfg>(P, ModLimb<Cfg>{}, m);
        }
    }

    // Montgomery product a*b*2^(-32N) mod modulus, fully reduced.
    template <typename Cfg>
    GZK_HD Fe<Cfg> mul(const Fe<Cfg>& a, const Fe<Cfg>& b)
    {
        constexpr int N = Cfg::N;
        static_assert(N % 2 == 0, "limb count must be even");
        uint32_t X[N + 1], Y[N + 1];
        // first row: plain products, no accumulation
#pragma unroll
        for (int j = 0; j < N; j += 2)
        {
            X[j] = mp::mul_lo(a.l[j], b.l[0]);
            X[j + 1] = mp::mul_hi(a.l[j], b.l[0]);
            Y[j] = mp::mul_lo(a.l[j + 1], b.l[0]);
            Y[j + 1] = mp::mul_hi(a.l[j + 1], b.l[0]);
        }
        X[N] = 0;
        Y[N] = 0;
        {
            const uint32_t m = mp::mul_lo(X[0], Cfg::INV);
            detail::mad_odd<Cfg>(Y, detail::ModLimb<Cfg>{}, m);
            detail::mad_even<Cfg>(X, detail::ModLimb<Cfg>{}, m);
        }
#pragma unroll
        for (int i = 1; i < N; i += 2)
        {
            detail::mont_row<Cfg>(Y, X, a.l, b.l[i]);
            if (i + 1 < N) detail::mont_row<Cfg>(X, Y, a.l, b.l[i + 1]);
        }
        // after an odd number of role swaps Y is even-aligned (limb 0 zero) and X
        // odd-aligned: result = (Y >> 32) + X < 2*modulus.
        Fe<Cfg> s;
        s.l[0] = mp::add_cc(Y[1], X[0]);
#pragma unroll
        for (int k = 1; k < N - 1; ++k) s.l[k] = mp::addc_cc(Y[k + 1], X[k]);
        s.l[N - 1] = mp::addc(Y[N], X[N - 1]);
        return reduce_once(s);
    }

    template <typename Cfg>
    GZK_HD Fe<Cfg> sqr(const Fe<Cfg>& a)
    {
        return mul(a, a);
    }

    template <typename Cfg>
    GZK_HD Fe<Cfg> to_mont(const Fe<Cfg>& canonical)
    {
        return mul(canonical, Fe<Cfg>::r2());
    }

    template <typename Cfg>
    GZK_HD Fe<Cfg> from_mont(const Fe<Cfg>& a)
    {
        Fe<Cfg> one_plain = Fe<Cfg>::zero();
        one_plain.l[0] = 1;
        return mul(a, one_plain);
    }

    // a^e for a 64-bit exponent (Montgomery in, Montgomery out).
    template <typename Cfg>
    GZK_HD Fe<Cfg> pow_u64(const Fe<Cfg>& a, uint64_t e)
    {
        Fe<Cfg> out = Fe<Cfg>::one();
        bool started = false;
        for (int i = 63; i >= 0; --i)
        {
            if (started) out = sqr(out);
            if ((e >> i) & 1ULL)
            {
                out = started ? mul(out, a) : a;
                started = true;
            }
        }
        return out;
    }

    // Fermat inverse a^(modulus-2); a must be non-zero (0 maps to 0).  Kept as the
    // cross-check of the binary algorithm below.
    template <typename Cfg>
    GZK_HD Fe<Cfg> inv_fermat(const Fe<Cfg>& a)
    {
        constexpr int N = Cfg::N;
        Fe<Cfg> out = Fe<Cfg>::one();
        bool started = false;
        uint32_t exponent[N];
        {
            // modulus - 2 with borrow propagation
            uint32_t borrow = 2;
#pragma unroll
            for (int i = 0; i < N; ++i)
            {
                const uint32_t m = Cfg::mod(i);
                exponent[i] = m - borrow;
                borrow = m < borrow ? 1u : 0u;
            }
        }
        for (int limb = N - 1; limb >= 0; --limb)
        {
            const uint32_t e = exponent[limb];
            for (int bit = 31; bit >= 0; --bit)
            {
                if (started) out = sqr(out);
                if ((e >> bit) & 1U)
                {
                    out = started ? mul(out, a) : a;
                    started = true;
                }
            }
        }
        return out;
    }

    namespace detail
    {
        template <int N>
        GZK_HD bool limbs_even(const uint32_t* a) { return (a[0] & 1u) == 0; }
        template <int N>
        GZK_HD bool limbs_is_one(const uint32_t* a)
        {
            uint32_t acc = a[0] ^ 1u;
#pragma unroll
            for (int i = 1; i < N; ++i) acc |= a[i];
            return acc == 0;
        }
        template <int N>
        GZK_HD void limbs_shr1(uint32_t* a)
        {
#pragma unroll
            for (int i = 0; i < N - 1; ++i) a[i] = (a[i] >> 1) | (a[i + 1] << 31);
            a[N - 1] >>= 1;
        }
        // a >= b ?
        template <int N>
        GZK_HD bool limbs_geq(const uint32_t* a, const uint32_t* b)
        {
            mp::sub_cc(a[0], b[0]);
#pragma unroll
            for (int i = 1; i < N; ++i) mp::subc_cc(a[i], b[i]);
            return mp::subc(0, 0) == 0;  // no borrow
        }
        template <int N>
        GZK_HD void limbs_sub(uint32_t* a, const uint32_t* b)
        {
            a[0] = mp::sub_cc(a[0], b[0]);
#pragma unroll
            for (int i = 1; i < N - 1; ++i) a[i] = mp::subc_cc(a[i], b[i]);
            a[N - 1] = mp::subc(a[N - 1], b[N - 1]);
        }
        // x = x / 2 mod modulus (x < modulus; modulus odd with a spare top bit)
        template <typename Cfg>
        GZK_HD void halve_mod(uint32_t* x)
        {
            constexpr int N = Cfg::N;
            if (x[0] & 1u)
            {
                x[0] = mp::add_cc(x[0], Cfg::mod(0));
#pragma unroll
                for (int i = 1; i < N - 1; ++i) x[i] = mp::addc_cc(x[i], Cfg::mod(i));
                x[N - 1] = mp::addc(x[N - 1], Cfg::mod(N - 1));
            }
            limbs_shr1<N>(x);
        }
    }

    // Inverse by the plain binary extended Euclidean algorithm (shifts and subtractions on
    // N limbs, about 2*bits short iterations) followed by one Montgomery product that
    // restores the Montgomery form.  Kept as a cross-check of inv() below.
    // a must be non-zero (0 maps to 0).
    template <typename Cfg>
    GZK_HD Fe<Cfg> inv_binary(const Fe<Cfg>& a)
    {
        constexpr int N = Cfg::N;
        if (a.is_zero()) return a;
        uint32_t u[N], v[N], x1[N], x2[N];
#pragma unroll
        for (int i = 0; i < N; ++i)
        {
            u[i] = a.l[i];
            v[i] = Cfg::mod(i);
            x1[i] = 0;
            x2[i] = 0;
        }
        x1[0] = 1;
        // every pass removes at least one bit from u or v: 2 * 32 * N passes suffice
        for (int guard = 0; guard < 64 * N + 8; ++guard)
        {
            if (detail::limbs_is_one<N>(u) || detail::limbs_is_one<N>(v)) break;
            while (detail::limbs_even<N>(u))
            {
                detail::limbs_shr1<N>(u);
                detail::halve_mod<Cfg>(x1);
            }
            while (detail::limbs_even<N>(v))
            {
                detail::limbs_shr1<N>(v);
                detail::halve_mod<Cfg>(x2);
            }
            if (detail::limbs_geq<N>(u, v))
            {
                detail::limbs_sub<N>(u, v);
                // x1 = x1 - x2 mod modulus
                if (!detail::limbs_geq<N>(x1, x2))
                {
                    x1[0] = mp::add_cc(x1[0], Cfg::mod(0));
#pragma unroll
                    for (int i = 1; i < N - 1; ++i) x1[i] = mp::addc_cc(x1[i], Cfg::mod(i));
                    x1[N - 1] = mp::addc(x1[N - 1], Cfg::mod(N - 1));
                }
                detail::limbs_sub<N>(x1, x2);
            }
            else
            {
                detail::limbs_sub<N>(v, u);
                if (!detail::limbs_geq<N>(x2, x1))
                {
                    x2[0] = mp::add_cc(x2[0], Cfg::mod(0));
#pragma unroll
                    for (int i = 1; i < N - 1; ++i) x2[i] = mp::addc_cc(x2[i], Cfg::mod(i));
                    x2[N - 1] = mp::addc(x2[N - 1], Cfg::mod(N - 1));
                }
                detail::limbs_sub<N>(x2, x1);
            }
        }
        Fe<Cfg> plain;  // (a as an integer)^-1 mod modulus
        const bool from_u = detail::limbs_is_one<N>(u);
#pragma unroll
        for (int i = 0; i < N; ++i) plain.l[i] = from_u ? x1[i] : x2[i];
        // a = A*R  =>  plain = A^-1 R^-1; Montgomery form of A^-1 is A^-1 R = plain * R^2,
        // i.e. the Montgomery product of plain with R^3.
        const Fe<Cfg> r3 = mul(Fe<Cfg>::r2(), Fe<Cfg>::r2());
        return mul(plain, r3);
    }

    namespace detail
    {
        // out[0..N] = a[0..N-1] * k
        template <int N>
        GZK_HD void limbs_mul_word(const uint32_t* a, uint32_t k, uint32_t* out)
        {
            uint64_t carry = 0;
#pragma unroll
            for (int i = 0; i < N; ++i)
            {
                const uint64_t w = static_cast<uint64_t>(a[i]) * k + carry;
                out[i] = static_cast<uint32_t>(w);
                carry = w >> 32;
            }
            out[N] = static_cast<uint32_t>(carry);
        }

        // x = |x*f + y*g| / 2^31 for N-limb x, y >= 0 and factors given as sign and
        // magnitude (magnitude <= 2^31, the division is exact); returns true when
        // x*f + y*g was negative.  Writes N limbs.
        template <int N>
        GZK_HD bool lincomb_shift31(const uint32_t* x, const uint32_t* y, uint32_t f_mag, bool f_neg, uint32_t g_mag, bool g_neg, uint32_t* out)
        {
            uint32_t p[N + 1], q[N + 1];
            limbs_mul_word<N>(x, f_mag, p);
            limbs_mul_word<N>(y, g_mag, q);
            bool negative = f_neg;
            if (f_neg == g_neg)
            {
                uint64_t carry = 0;
#pragma unroll
                for (int i = 0; i <= N; ++i)
                {
                    const uint64_t w = static_cast<uint64_t>(p[i]) + q[i] + carry;
                    p[i] = static_cast<uint32_t>(w);
                    carry = w >> 32;
                }
            }
            else
            {
                uint64_t borrow = 0;
#pragma unroll
                for (int i = 0; i <= N; ++i)
                {
                    const uint64_t w = static_cast<uint64_t>(p[i]) - q[i] - borrow;
                    p[i] = static_cast<uint32_t>(w);
                    borrow = (w >> 32) & 1u;
                }
                if (borrow)
                {
                    // |p - q| = q - p: negate the two's complement difference
                    uint64_t carry = 1;
#pragma unroll
                    for (int i = 0; i <= N; ++i)
                    {
                        const uint64_t w = static_cast<uint64_t>(~p[i]) + carry;
                        p[i] = static_cast<uint32_t>(w);
                        carry = w >> 32;
                    }
                    negative = g_neg;
                }
            }
#pragma unroll
            for (int i = 0; i < N; ++i) out[i] = (p[i] >> 31) | (p[i + 1] << 1);
            return negative;
        }

        // u = (u*f + v*g) / 2^31 mod modulus for u, v in [0, modulus]; factors as above.
        template <typename Cfg>
        GZK_HD void lincomb_mod_shift31(const uint32_t* u, const uint32_t* v, uint32_t f_mag, bool f_neg, uint32_t g_mag, bool g_neg, uint32_t* out)
        {
            constexpr int N = Cfg::N;
            uint32_t un[N], vn[N];
            // a negative factor is applied to the negated residue: -f*u = f*(modulus - u)
            {
                uint64_t borrow_u = 0, borrow_v = 0;
#pragma unroll
                for (int i = 0; i < N; ++i)
                {
                    const uint64_t wu = static_cast<uint64_t>(Cfg::mod(i)) - u[i] - borrow_u;
                    const uint64_t wv = static_cast<uint64_t>(Cfg::mod(i)) - v[i] - borrow_v;
                    un[i] = f_neg ? static_cast<uint32_t>(wu) : u[i];
                    vn[i] = g_neg ? static_cast<uint32_t>(wv) : v[i];
                    borrow_u = (wu >> 32) & 1u;
                    borrow_v = (wv >> 32) & 1u;
                }
            }
            uint32_t p[N + 1], q[N + 1];
            limbs_mul_word<N>(un, f_mag, p);
            limbs_mul_word<N>(vn, g_mag, q);
            uint64_t carry = 0;
#pragma unroll
            for (int i = 0; i <= N; ++i)
            {
                const uint64_t w = static_cast<uint64_t>(p[i]) + q[i] + carry;
                p[i] = static_cast<uint32_t>(w);
                carry = w >> 32;
            }
            // add the multiple of the modulus that clears the low 31 bits (Montgomery step with 2^31)
            const uint32_t k = (p[0] * Cfg::INV) & 0x7fffffffu;
            uint32_t km[N + 1];
            uint32_t mod[N];
#pragma unroll
            for (int i = 0; i < N; ++i) mod[i] = Cfg::mod(i);
            limbs_mul_word<N>(mod, k, km);
            carry = 0;
#pragma unroll
            for (int i = 0; i <= N; ++i)
            {
                const uint64_t w = static_cast<uint64_t>(p[i]) + km[i] + carry;
                p[i] = static_cast<uint32_t>(w);
                carry = w >> 32;
            }
            uint32_t r[N];
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = (p[i] >> 31) | (p[i + 1] << 1);
            // r < 2 * modulus: one conditional subtraction
            uint32_t d[N];
            uint64_t borrow = 0;
#pragma unroll
            for (int i = 0; i < N; ++i)
            {
                const uint64_t w = static_cast<uint64_t>(r[i]) - Cfg::mod(i) - borrow;
                d[i] = static_cast<uint32_t>(w);
                borrow = (w >> 32) & 1u;
            }
#pragma unroll
            for (int i = 0; i < N; ++i) out[i] = borrow ? r[i] : d[i];
        }
    }

    // Inverse by the binary GCD with word-sized approximations (Pornin, "Optimized Binary
    // GCD for Modular Inversion", 2020): 31 steps of the binary algorithm are run on 64-bit
    // stand-ins for a and b (their low 31 bits and the 33 bits below the longer one's top)
    // while the steps are recorded as four small factors; the factors are then applied once
    // to the full-length a, b and to the cofactors u, v.  ceil((2*bits-1)/31) such rounds
    // reach a = 0, b = 1, v = 1/value.  The cofactor update divides by 2^31 modulo the
    // modulus each round, so no correction is left at the end except the Montgomery one.
    // About four times shorter as a dependent chain than inv_binary(); every batch inversion
    // of the library ends in exactly one such serial inversion.  a must be non-zero (0 maps to 0).
    template <typename Cfg>
    GZK_HD Fe<Cfg> inv(const Fe<Cfg>& value)
    {
        constexpr int N = Cfg::N;
        constexpr int kRounds = (2 * Cfg::BITS - 1 + 30) / 31;
        if (value.is_zero()) return value;
        uint32_t a[N], b[N], u[N], v[N];
#pragma unroll
        for (int i = 0; i < N; ++i)
        {
            a[i] = value.l[i];
            b[i] = Cfg::mod(i);
            u[i] = 0;
            v[i] = 0;
        }
        u[0] = 1;
        for (int round = 0; round < kRounds; ++round)
        {
            // 64-bit stand-ins: exact when both fit 64 bits, else low 31 bits + the 33 bits under the common top
            uint32_t ah = a[1], al = a[0], bh = b[1], bl = b[0];
            bool wide = false;
#pragma unroll
            for (int i = N - 1; i >= 2; --i)
            {
                if (!wide && (a[i] | b[i]) != 0)
                {
                    ah = a[i];
                    al = a[i - 1];
                    bh = b[i];
                    bl = b[i - 1];
                    wide = true;
                }
            }
            uint64_t xa = (static_cast<uint64_t>(ah) << 32) | al;
            uint64_t xb = (static_cast<uint64_t>(bh) << 32) | bl;
            if (wide)
            {
                // leading zeros of the common top limb
#if defined(__CUDA_ARCH__)
                const int lead = __clz(static_cast<int>(ah | bh));
#else
                uint32_t top = ah | bh;
                int lead = 0;
                while ((top & 0x80000000u) == 0)
                {
                    top <<= 1;
                    ++lead;
                }
#endif
                xa = ((xa >> (31 - lead)) << 31) | (a[0] & 0x7fffffffu);
                xb = ((xb >> (31 - lead)) << 31) | (b[0] & 0x7fffffffu);
            }
            int64_t f0 = 1, g0 = 0, f1 = 0, g1 = 1;
            for (int step = 0; step < 31; ++step)
            {
                const bool odd = (xa & 1u) != 0;
                if (odd && xa < xb)
                {
                    const uint64_t tx = xa;
                    xa = xb;
                    xb = tx;
                    int64_t t = f0;
                    f0 = f1;
                    f1 = t;
                    t = g0;
                    g0 = g1;
                    g1 = t;
                }
                if (odd)
                {
                    xa -= xb;
                    f0 -= f1;
                    g0 -= g1;
                }
                xa >>= 1;
                f1 <<= 1;
                g1 <<= 1;
            }
            bool f0n = f0 < 0, g0n = g0 < 0, f1n = f1 < 0, g1n = g1 < 0;
            const uint32_t f0m = static_cast<uint32_t>(f0n ? -f0 : f0), g0m = static_cast<uint32_t>(g0n ? -g0 : g0);
            const uint32_t f1m = static_cast<uint32_t>(f1n ? -f1 : f1), g1m = static_cast<uint32_t>(g1n ? -g1 : g1);
            uint32_t na[N], nb[N];
            if (detail::lincomb_shift31<N>(a, b, f0m, f0n, g0m, g0n, na))
            {
                f0n = !f0n;
                g0n = !g0n;
            }
            if (detail::lincomb_shift31<N>(a, b, f1m, f1n, g1m, g1n, nb))
            {
                f1n = !f1n;
                g1n = !g1n;
            }
            uint32_t nu[N], nv[N];
            detail::lincomb_mod_shift31<Cfg>(u, v, f0m, f0n, g0m, g0n, nu);
            detail::lincomb_mod_shift31<Cfg>(u, v, f1m, f1n, g1m, g1n, nv);
            uint32_t a_any = 0;
#pragma unroll
            for (int i = 0; i < N; ++i)
            {
                a[i] = na[i];
                b[i] = nb[i];
                u[i] = nu[i];
                v[i] = nv[i];
                a_any |= na[i];
            }
            if (a_any == 0) break;  // b holds the gcd (1), v its cofactor
        }
        Fe<Cfg> plain;  // (value as an integer)^-1 mod modulus
#pragma unroll
        for (int i = 0; i < N; ++i) plain.l[i] = v[i];
        plain = reduce_once(plain);
        // value = A*R  =>  plain = A^-1 R^-1; the Montgomery form of A^-1 is A^-1 R = plain * R^2,
        // i.e. the Montgomery product of plain with R^3.
        const Fe<Cfg> r3 = mul(Fe<Cfg>::r2(), Fe<Cfg>::r2());
        return mul(plain, r3);
    }

    // Full 2N-limb product of two N-limb integers (no reduction).  Products whose
    // low half lands on an even limb go to E, the others to O (O is offset by one
    // limb); every carry out of a row chain lands in a limb no earlier row has
    // touched, so a single addc captures it.
    template <int N>
    GZK_HD void mul_wide(const uint32_t* a, const uint32_t* b, uint32_t* out)
    {
        static_assert(N % 2 == 0, "limb count must be even");
        uint32_t E[2 * N], O[2 * N];
#pragma unroll
        for (int k = 0; k < 2 * N; ++k)
        {
            E[k] = 0;
            O[k] = 0;
        }
#pragma unroll
        for (int j = 0; j < N; j += 2)
        {
            E[j] = mp::mul_lo(a[j], b[0]);
            E[j + 1] = mp::mul_hi(a[j], b[0]);
            O[j] = mp::mul_lo(a[j + 1], b[0]);
            O[j + 1] = mp::mul_hi(a[j + 1], b[0]);
        }
#pragma unroll
        for (int i = 1; i < N; ++i)
        {
            if (i & 1)
            {
                // odd j -> even column: E[i+j], E[i+j+1]; top pair is fresh
                E[i + 1] = mp::mad_lo_cc(a[1], b[i], E[i + 1]);
                E[i + 2] = mp::madc_hi_cc(a[1], b[i], E[i + 2]);
#pragma unroll
                for (int j = 3; j < N; j += 2)
                {
                    E[i + j] = mp::madc_lo_cc(a[j], b[i], E[i + j]);
                    E[i + j + 1] = mp::madc_hi_cc(a[j], b[i], E[i + j + 1]);
                }
                // even j -> odd column: O[i+j-1], O[i+j]; carry lands in O[i+N-1]
                O[i - 1] = mp::mad_lo_cc(a[0], b[i], O[i - 1]);
                O[i] = mp::madc_hi_cc(a[0], b[i], O[i]);
#pragma unroll
                for (int j = 2; j < N; j += 2)
                {
                    O[i + j - 1] = mp::madc_lo_cc(a[j], b[i], O[i + j - 1]);
                    O[i + j] = mp::madc_hi_cc(a[j], b[i], O[i + j]);
                }
                O[i + N - 1] = mp::addc(O[i + N - 1], 0);
            }
            else
            {
                // even j -> even column: E[i+j], E[i+j+1]; carry lands in E[i+N]
                E[i] = mp::mad_lo_cc(a[0], b[i], E[i]);
                E[i + 1] = mp::madc_hi_cc(a[0], b[i], E[i + 1]);
#pragma unroll
                for (int j = 2; j < N; j += 2)
                {
                    E[i + j] = mp::madc_lo_cc(a[j], b[i], E[i + j]);
                    E[i + j + 1] = mp::madc_hi_cc(a[j], b[i], E[i + j + 1]);
                }
                E[i + N] = mp::addc(E[i + N], 0);
                // odd j -> odd column: O[i+j-1], O[i+j]; top pair is fresh
                O[i] = mp::mad_lo_cc(a[1], b[i], O[i]);
                O[i + 1] = mp::madc_hi_cc(a[1], b[i], O[i + 1]);
#pragma unroll
                for (int j = 3; j < N; j += 2)
                {
                    O[i + j - 1] = mp::madc_lo_cc(a[j], b[i], O[i + j - 1]);
                    O[i + j] = mp::madc_hi_cc(a[j], b[i], O[i + j]);
                }
            }
        }
        out[0] = E[0];
        out[1] = mp::add_cc(E[1], O[0]);
#pragma unroll
        for (int k = 2; k < 2 * N - 1; ++k) out[k] = mp::addc_cc(E[k], O[k - 1]);
        out[2 * N - 1] = mp::addc(E[2 * N - 1], O[2 * N - 2]);
    }

    // acc (L limbs) += x (M limbs, M <= L), carries rippled to the top of acc.
    template <int L, int M>
    GZK_HD void acc_add(uint32_t* acc, const uint32_t* x)
    {
        acc[0] = mp::add_cc(acc[0], x[0]);
#pragma unroll
        for (int k = 1; k < M; ++k) acc[k] = mp::addc_cc(acc[k], x[k]);
#pragma unroll
        for (int k = M; k < L; ++k) acc[k] = mp::addc_cc(acc[k], 0);
    }

    // Montgomery reduction of a wide integer T (N + ROWS limbs, T < modulus *
    // 2^(32*ROWS)): returns T * 2^(-32*ROWS) mod modulus, fully reduced.  Used
    // once per accumulated inner product, so it favours clarity over speed.
    template <typename Cfg, int ROWS>
    GZK_HD Fe<Cfg> redc_wide(const uint32_t* T_in)
    {
        constexpr int N = Cfg::N;
        constexpr int L = N + ROWS + 1;
        uint32_t T[L];
#pragma unroll
        for (int k = 0; k < L - 1; ++k) T[k] = T_in[k];
        T[L - 1] = 0;
#pragma unroll
        for (int i = 0; i < ROWS; ++i)
        {
            const uint32_t m = mp::mul_lo(T[i], Cfg::INV);
            // low halves
            T[i] = mp::mad_lo_cc(m, Cfg::mod(0), T[i]);
#pragma unroll
            for (int j = 1; j < N; ++j) T[i + j] = mp::madc_lo_cc(m, Cfg::mod(j), T[i + j]);
#pragma unroll
            for (int k = i + N; k < L; ++k) T[k] = mp::addc_cc(T[k], 0);
            // high halves
            T[i + 1] = mp::mad_hi_cc(m, Cfg::mod(0), T[i + 1]);
#pragma unroll
            for (int j = 1; j < N; ++j) T[i + j + 1] = mp::madc_hi_cc(m, Cfg::mod(j), T[i + j + 1]);
#pragma unroll
            for (int k = i + N + 1; k < L; ++k) T[k] = mp::addc_cc(T[k], 0);
        }
        Fe<Cfg> s;
#pragma unroll
        for (int k = 0; k < N; ++k) s.l[k] = T[ROWS + k];
        return reduce_once(s);
    }

    // Unreduced accumulator for sums of 8x8-limb products (inner products of Fr
    // vectors).  Products whose low half lands on an even limb are added into E,
    // the others into O (O is offset by one limb), each row of a product as one
    // carry chain straight into the accumulator.  The carry out of a chain is not
    // rippled: it is counted in a small counter for the limb position it belongs
    // to (five positions for E, four for O).  A term therefore costs 64 wide
    // multiply-adds plus 16 carry captures and no temporaries; the pieces are
    // merged once, in fold().  Exact for up to 2^31 terms.
    struct WideAcc
    {
        uint32_t E[16];
        uint32_t O[14];
        uint32_t cE[5];  // carries into E positions 8,10,12,14,16
        uint32_t cO[4];  // carries into O positions 8,10,12,14

        GZK_HD void clear()
        {
#pragma unroll
            for (int i = 0; i < 16; ++i) E[i] = 0;
#pragma unroll
            for (int i = 0; i < 14; ++i) O[i] = 0;
#pragma unroll
            for (int i = 0; i < 5; ++i) cE[i] = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) cO[i] = 0;
        }

        template <int I>
        GZK_HD void row(const uint32_t* a, uint32_t bi)
        {
            if (I % 2 == 0)
            {
                E[I] = mp::mad_lo_cc(a[0], bi, E[I]);
                E[I + 1] = mp::madc_hi_cc(a[0], bi, E[I + 1]);
#pragma unroll
                for (int j = 2; j < 8; j += 2)
                {
                    E[I + j] = mp::madc_lo_cc(a[j], bi, E[I + j]);
                    E[I + j + 1] = mp::madc_hi_cc(a[j], bi, E[I + j + 1]);
                }
                cE[I / 2] = mp::addc(cE[I / 2], 0);
                O[I] = mp::mad_lo_cc(a[1], bi, O[I]);
                O[I + 1] = mp::madc_hi_cc(a[1], bi, O[I + 1]);
#pragma unroll
                for (int j = 3; j < 8; j += 2)
                {
                    O[I + j - 1] = mp::madc_lo_cc(a[j], bi, O[I + j - 1]);
                    O[I + j] = mp::madc_hi_cc(a[j], bi, O[I + j]);
                }
                cO[I / 2] = mp::addc(cO[I / 2], 0);
            }
            else
            {
                E[I + 1] = mp::mad_lo_cc(a[1], bi, E[I + 1]);
                E[I + 2] = mp::madc_hi_cc(a[1], bi, E[I + 2]);
#pragma unroll
                for (int j = 3; j < 8; j += 2)
                {
                    E[I + j] = mp::madc_lo_cc(a[j], bi, E[I + j]);
                    E[I + j + 1] = mp::madc_hi_cc(a[j], bi, E[I + j + 1]);
                }
                cE[(I + 1) / 2] = mp::addc(cE[(I + 1) / 2], 0);
                O[I - 1] = mp::mad_lo_cc(a[0], bi, O[I - 1]);
                O[I] = mp::madc_hi_cc(a[0], bi, O[I]);
#pragma unroll
                for (int j = 2; j < 8; j += 2)
                {
                    O[I + j - 1] = mp::madc_lo_cc(a[j], bi, O[I + j - 1]);
                    O[I + j] = mp::madc_hi_cc(a[j], bi, O[I + j]);
                }
                cO[(I - 1) / 2] = mp::addc(cO[(I - 1) / 2], 0);
            }
        }

        // acc += a * b for 8-limb a and the low ROWS limbs of b (higher limbs of b
        // are known to be zero: small-integer columns).
        template <int ROWS>
        GZK_HD void mac(const uint32_t* a, const uint32_t* b)
        {
            row<0>(a, b[0]);
            if (ROWS > 1) row<1>(a, b[1]);
            if (ROWS > 2) row<2>(a, b[2]);
            if (ROWS > 3) row<3>(a, b[3]);
            if (ROWS > 4) row<4>(a, b[4]);
            if (ROWS > 5) row<5>(a, b[5]);
            if (ROWS > 6) row<6>(a, b[6]);
            if (ROWS > 7) row<7>(a, b[7]);
        }

        // Merge into one 17-limb integer.
        GZK_HD void fold(uint32_t* out) const
        {
            uint32_t t[17];
#pragma unroll
            for (int k = 0; k < 16; ++k) out[k] = E[k];
            out[16] = 0;
#pragma unroll
            for (int k = 0; k < 17; ++k) t[k] = 0;
#pragma unroll
            for (int i = 0; i < 5; ++i) t[8 + 2 * i] = cE[i];
            acc_add<17, 17>(out, t);
            t[0] = 0;
#pragma unroll
            for (int k = 0; k < 14; ++k) t[k + 1] = O[k];
            t[15] = 0;
            t[16] = 0;
            acc_add<17, 17>(out, t);
#pragma unroll
            for (int k = 0; k < 17; ++k) t[k] = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) t[9 + 2 * i] = cO[i];
            acc_add<17, 17>(out, t);
        }
    };

    // Same accumulator with explicit wide multiplies: every limb product is one
    // mul.wide.u32 (independent of the accumulator, so the four products of a row
    // chain issue back to back) followed by a 64-bit add-with-carry into 64-bit
    // accumulator lanes.  The code generated does not depend on the assembler pairing
    // lo/hi multiply-adds.
    struct WideAcc64
    {
        uint64_t E[8];   // even-aligned lanes: E[k] holds limbs 2k, 2k+1
        uint64_t O[7];   // odd-aligned lanes, offset by one limb: O[k] holds limbs 2k+1, 2k+2
        uint32_t cE[5];  // carries out of E lanes 3..7 (limb positions 8,10,12,14,16)
        uint32_t cO[4];  // carries out of O lanes 3..6 (O limb positions 8,10,12,14)

        GZK_HD void clear()
        {
#pragma unroll
            for (int i = 0; i < 8; ++i) E[i] = 0;
#pragma unroll
            for (int i = 0; i < 7; ++i) O[i] = 0;
#pragma unroll
            for (int i = 0; i < 5; ++i) cE[i] = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) cO[i] = 0;
        }

        template <int I>
        GZK_HD void row(const uint32_t* a, uint32_t bi)
        {
            // products of this row: even j and odd j
            const uint64_t e0 = mp::mul_wide(a[(I % 2 == 0) ? 0 : 1], bi);
            const uint64_t e1 = mp::mul_wide(a[(I % 2 == 0) ? 2 : 3], bi);
            const uint64_t e2 = mp::mul_wide(a[(I % 2 == 0) ? 4 : 5], bi);
            const uint64_t e3 = mp::mul_wide(a[(I % 2 == 0) ? 6 : 7], bi);
            const uint64_t o0 = mp::mul_wide(a[(I % 2 == 0) ? 1 : 0], bi);
            const uint64_t o1 = mp::mul_wide(a[(I % 2 == 0) ? 3 : 2], bi);
            const uint64_t o2 = mp::mul_wide(a[(I % 2 == 0) ? 5 : 4], bi);
            const uint64_t o3 = mp::mul_wide(a[(I % 2 == 0) ? 7 : 6], bi);
            // E lanes: row I even starts at limb I (lane I/2); row I odd at limb I+1 (lane (I+1)/2)
            constexpr int le = (I % 2 == 0) ? I / 2 : (I + 1) / 2;
            E[le] = mp::add_cc_u64(E[le], e0);
            E[le + 1] = mp::addc_cc_u64(E[le + 1], e1);
            E[le + 2] = mp::addc_cc_u64(E[le + 2], e2);
            E[le + 3] = mp::addc_cc_u64(E[le + 3], e3);
            cE[le] = mp::addc(cE[le], 0);  // carry into limb 2*(le+4): counter index le (positions 8..16)
            // O lanes: row I even starts at O limb I (lane I/2); row I odd at O limb I-1 (lane (I-1)/2)
            constexpr int lo = (I % 2 == 0) ? I / 2 : (I - 1) / 2;
            O[lo] = mp::add_cc_u64(O[lo], o0);
            O[lo + 1] = mp::addc_cc_u64(O[lo + 1], o1);
            O[lo + 2] = mp::addc_cc_u64(O[lo + 2], o2);
            O[lo + 3] = mp::addc_cc_u64(O[lo + 3], o3);
            cO[lo] = mp::addc(cO[lo], 0);
        }

        template <int ROWS>
        GZK_HD void mac(const uint32_t* a, const uint32_t* b)
        {
            row<0>(a, b[0]);
            if (ROWS > 1) row<1>(a, b[1]);
            if (ROWS > 2) row<2>(a, b[2]);
            if (ROWS > 3) row<3>(a, b[3]);
            if (ROWS > 4) row<4>(a, b[4]);
            if (ROWS > 5) row<5>(a, b[5]);
            if (ROWS > 6) row<6>(a, b[6]);
            if (ROWS > 7) row<7>(a, b[7]);
        }

        GZK_HD void fold(uint32_t* out) const
        {
            uint32_t t[17];
#pragma unroll
            for (int k = 0; k < 8; ++k)
            {
                out[2 * k] = static_cast<uint32_t>(E[k]);
                out[2 * k + 1] = static_cast<uint32_t>(E[k] >> 32);
            }
            out[16] = 0;
#pragma unroll
            for (int k = 0; k < 17; ++k) t[k] = 0;
#pragma unroll
            for (int i = 0; i < 5; ++i) t[8 + 2 * i] = cE[i];
            acc_add<17, 17>(out, t);
            t[0] = 0;
#pragma unroll
            for (int k = 0; k < 7; ++k)
            {
                t[2 * k + 1] = static_cast<uint32_t>(O[k]);
                t[2 * k + 2] = static_cast<uint32_t>(O[k] >> 32);
            }
            t[15] = 0;
            t[16] = 0;
            acc_add<17, 17>(out, t);
#pragma unroll
            for (int k = 0; k < 17; ++k) t[k] = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) t[9 + 2 * i] = cO[i];
            acc_add<17, 17>(out, t);
        }
    };

    using Fr = Fe<FrCfg>;
    using Fp = Fe<FpCfg>;

    // 2^544 mod r: turns redc_wide<FrCfg, 9>(sum of Montgomery * canonical
    // products) back into the Montgomery form of the true sum.
    GZK_HD Fr fr_const_2_544()
    {
        constexpr uint32_t c[8] = {0xefe9ec32u, 0x0408b03au, 0x122df55fu, 0xc98a431eu,
                                   0x8277a7beu, 0xdd74d8f7u, 0x9163e436u, 0x1ef2c2b1u};
        Fr o;
#pragma unroll
        for (int i = 0; i < 8; ++i) o.l[i] = c[i];
        return o;
    }
}
