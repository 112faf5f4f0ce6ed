// TEST INFRASTRUCTURE — CPU oracle for the GAT-ZKML proving hot path.
//
// This directory restates, on the CPU, the algorithms of the reference prover
// (Solityer/project) for the data-parallel core of commit + prove.  It exists so
// that the CUDA backend can be checked bit-for-bit; it is never part of the
// product path.  Only tests, the smoke check and the CPU-baseline leg of the
// benchmark may load it.
//
// PARITY UNPINNED at the big-number boundary: the reference delegates all
// Fr/Fp/G1 arithmetic to herumi/mcl (unpinned HEAD, not vendored, absent), and
// holds no known-answer vectors for field values, roots of unity, commitments
// or transcript output.  The arithmetic here is therefore pinned against
// independent big-integer computations (Python int / pow) rather than against
// mcl output.  Field results are canonical residues, so any correct
// implementation yields the same bytes.
//
// Montgomery prime field over N 64-bit limbs.  Follows the semantics of
// include/gatzk/algebra/field.hpp:28-205 (FieldElement over mcl::Fr):
// zero(), one(), from u64, from_signed, +, -, *, inv (throws on zero), pow,
// little-endian (de)serialisation.
#pragma once

#include <array>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>

namespace oracle
{
    using u64 = std::uint64_t;
    using u128 = unsigned __int128;

    template <std::size_t N>
    struct BigInt
    {
        std::array<u64, N> w{};

        bool is_zero() const
        {
            u64 acc = 0;
            for (auto v : w) acc |= v;
            return acc == 0;
        }
        bool bit(std::size_t i) const { return (w[i / 64] >> (i % 64)) & 1U; }
        std::size_t bit_length() const
        {
            for (std::size_t i = N; i-- > 0;)
                if (w[i] != 0) return i * 64 + (64 - static_cast<std::size_t>(__builtin_clzll(w[i])));
            return 0;
        }
    };

    template <std::size_t N>
    inline int cmp(const BigInt<N>& a, const BigInt<N>& b)
    {
        for (std::size_t i = N; i-- > 0;)
        {
            if (a.w[i] < b.w[i]) return -1;
            if (a.w[i] > b.w[i]) return 1;
        }
        return 0;
    }

    template <std::size_t N>
    inline u64 add_into(BigInt<N>& a, const BigInt<N>& b)
    {
        u128 c = 0;
        for (std::size_t i = 0; i < N; ++i)
        {
            c += static_cast<u128>(a.w[i]) + b.w[i];
            a.w[i] = static_cast<u64>(c);
            c >>= 64;
        }
        return static_cast<u64>(c);
    }

    template <std::size_t N>
    inline u64 sub_into(BigInt<N>& a, const BigInt<N>& b)
    {
        u64 borrow = 0;
        for (std::size_t i = 0; i < N; ++i)
        {
            const u128 d = static_cast<u128>(a.w[i]) - b.w[i] - borrow;
            a.w[i] = static_cast<u64>(d);
            borrow = static_cast<u64>(d >> 64) & 1U;
        }
        return borrow;
    }

    // Parameters of one prime field; everything except the modulus itself is
    // derived at start-up so that no constant has to be trusted from memory.
    template <std::size_t N>
    struct FieldParams
    {
        BigInt<N> modulus;
        u64 inv = 0;            // -modulus^{-1} mod 2^64
        BigInt<N> r1;           // 2^(64N) mod modulus
        BigInt<N> r2;           // 2^(128N) mod modulus
        BigInt<N> modulus_minus_2;

        explicit FieldParams(const std::array<u64, N>& m)
        {
            modulus.w = m;
            // Newton iteration for the inverse of an odd number modulo 2^64.
            u64 x = 1;
            for (int i = 0; i < 6; ++i) x *= 2 - m[0] * x;
            inv = ~x + 1;
            // r1 = 2^(64N) mod m by doubling 1 64N times; r2 by doubling r1 64N more.
            BigInt<N> v;
            v.w[0] = 1;
            for (std::size_t i = 0; i < 128 * N; ++i)
            {
                const u64 carry = add_into(v, BigInt<N>(v));
                if (carry != 0 || cmp(v, modulus) >= 0) sub_into(v, modulus);
                if (i + 1 == 64 * N) r1 = v;
            }
            r2 = v;
            modulus_minus_2 = modulus;
            BigInt<N> two;
            two.w[0] = 2;
            sub_into(modulus_minus_2, two);
        }
    };

    // Tag supplies `static const FieldParams<N>& params()`.
    template <std::size_t N, typename Tag>
    class Fe
    {
    public:
        BigInt<N> v;  // Montgomery form

        static const FieldParams<N>& P() { return Tag::params(); }

        static Fe zero() { return Fe{}; }
        static Fe one()
        {
            Fe o;
            o.v = P().r1;
            return o;
        }
        static Fe from_u64(u64 x)
        {
            BigInt<N> b;
            b.w[0] = x;
            return from_canonical(b);
        }
        // field.hpp:71-76 (from_signed): negative values map to modulus - |x|.
        static Fe from_i64(std::int64_t x)
        {
            if (x >= 0) return from_u64(static_cast<u64>(x));
            const u64 mag = ~static_cast<u64>(x) + 1;
            return zero() - from_u64(mag);
        }
        static Fe from_canonical(const BigInt<N>& b)
        {
            Fe t;
            t.v = b;
            Fe r2;
            r2.v = P().r2;
            return t * r2;
        }
        // field.hpp:79-84 (setLittleEndianMod): interpret the bytes as an
        // integer and reduce modulo the field order.
        static Fe from_le_bytes_mod(const std::uint8_t* bytes, std::size_t size)
        {
            Fe acc = zero();
            const Fe base = from_u64(256);
            for (std::size_t i = size; i-- > 0;)
            {
                acc = acc * base + from_u64(bytes[i]);
            }
            return acc;
        }
        BigInt<N> canonical() const
        {
            // Montgomery reduction of v (multiply by 1).
            Fe o;
            o.v.w[0] = 1;
            return mont_mul(v, o.v);
        }
        // field.hpp:193-201 (write_little_endian): canonical value, LE bytes.
        void to_le_bytes(std::uint8_t* out) const
        {
            const auto c = canonical();
            std::memcpy(out, c.w.data(), 8 * N);
        }
        static Fe from_le_bytes(const std::uint8_t* in)
        {
            BigInt<N> b;
            std::memcpy(b.w.data(), in, 8 * N);
            if (cmp(b, P().modulus) >= 0) throw std::runtime_error("non-canonical field element");
            return from_canonical(b);
        }

        bool is_zero() const { return v.is_zero(); }
        bool operator==(const Fe& o) const { return cmp(v, o.v) == 0; }
        bool operator!=(const Fe& o) const { return cmp(v, o.v) != 0; }

        Fe operator+(const Fe& o) const
        {
            Fe out = *this;
            const u64 carry = add_into(out.v, o.v);
            if (carry != 0 || cmp(out.v, P().modulus) >= 0) sub_into(out.v, P().modulus);
            return out;
        }
        Fe operator-(const Fe& o) const
        {
            Fe out = *this;
            if (sub_into(out.v, o.v) != 0) add_into(out.v, P().modulus);
            return out;
        }
        Fe operator-() const { return zero() - *this; }
        Fe operator*(const Fe& o) const
        {
            Fe out;
            out.v = mont_mul(v, o.v);
            return out;
        }
        Fe& operator+=(const Fe& o) { return *this = *this + o; }
        Fe& operator-=(const Fe& o) { return *this = *this - o; }
        Fe& operator*=(const Fe& o) { return *this = *this * o; }

        template <std::size_t M>
        Fe pow(const BigInt<M>& e) const
        {
            Fe out = one();
            for (std::size_t i = e.bit_length(); i-- > 0;)
            {
                out = out * out;
                if (e.bit(i)) out = out * *this;
            }
            return out;
        }
        Fe pow(u64 e) const
        {
            BigInt<1> b;
            b.w[0] = e;
            return pow(b);
        }
        // field.hpp:169-179: inverting zero is an error.
        Fe inv() const
        {
            if (is_zero()) throw std::runtime_error("attempted to invert zero in FieldElement");
            return pow(P().modulus_minus_2);
        }

        std::string to_decimal() const
        {
            auto c = canonical();
            if (c.is_zero()) return "0";
            std::string digits;
            while (!c.is_zero())
            {
                u128 rem = 0;
                for (std::size_t i = N; i-- > 0;)
                {
                    const u128 cur = (rem << 64) | c.w[i];
                    c.w[i] = static_cast<u64>(cur / 10);
                    rem = cur % 10;
                }
                digits.push_back(static_cast<char>('0' + static_cast<int>(rem)));
            }
            return std::string(digits.rbegin(), digits.rend());
        }

    private:
        // CIOS Montgomery product a*b*2^(-64N) mod modulus, fully reduced.
        static BigInt<N> mont_mul(const BigInt<N>& a, const BigInt<N>& b)
        {
            const auto& m = P().modulus;
            u64 t[N + 2] = {};
            for (std::size_t i = 0; i < N; ++i)
            {
                u128 c = 0;
                for (std::size_t j = 0; j < N; ++j)
                {
                    c += static_cast<u128>(a.w[j]) * b.w[i] + t[j];
                    t[j] = static_cast<u64>(c);
                    c >>= 64;
                }
                c += t[N];
                t[N] = static_cast<u64>(c);
                t[N + 1] = static_cast<u64>(c >> 64);

                const u64 q = t[0] * P().inv;
                c = static_cast<u128>(q) * m.w[0] + t[0];
                c >>= 64;
                for (std::size_t j = 1; j < N; ++j)
                {
                    c += static_cast<u128>(q) * m.w[j] + t[j];
                    t[j - 1] = static_cast<u64>(c);
                    c >>= 64;
                }
                c += t[N];
                t[N - 1] = static_cast<u64>(c);
                t[N] = t[N + 1] + static_cast<u64>(c >> 64);
            }
            BigInt<N> out;
            for (std::size_t j = 0; j < N; ++j) out.w[j] = t[j];
            if (t[N] != 0 || cmp(out, m) >= 0) sub_into(out, m);
            return out;
        }
    };

    // BLS12-381 (the curve the reference initialises: field.hpp:19-25).
    struct FrTag
    {
        static const FieldParams<4>& params()
        {
            static const FieldParams<4> p({0xffffffff00000001ULL, 0x53bda402fffe5bfeULL,
                                           0x3339d80809a1d805ULL, 0x73eda753299d7d48ULL});
            return p;
        }
    };
    struct FpTag
    {
        static const FieldParams<6>& params()
        {
            static const FieldParams<6> p({0xb9feffffffffaaabULL, 0x1eabfffeb153ffffULL,
                                           0x6730d2a0f6b0f624ULL, 0x64774b84f38512bfULL,
                                           0x4b1ba7b6434bacd7ULL, 0x1a0111ea397fe69aULL});
            return p;
        }
    };
    using Fr = Fe<4, FrTag>;
    using Fp = Fe<6, FpTag>;

    // field.hpp:87-101: omega_n = 5^((r-1)/n), n a non-zero power of two.
    inline Fr root_of_unity(std::size_t size)
    {
        if (size == 0 || (size & (size - 1U)) != 0U)
            throw std::runtime_error("domain size must be a non-zero power of two");
        BigInt<4> e = FrTag::params().modulus;
        e.w[0] -= 1;  // r is odd, no borrow
        std::size_t log2n = 0;
        while ((static_cast<std::size_t>(1) << log2n) < size) ++log2n;
        if (log2n > 32) throw std::runtime_error("domain size exceeds the 2-adicity of Fr");
        for (std::size_t s = 0; s < log2n; ++s)
        {
            for (std::size_t i = 0; i < 4; ++i)
            {
                e.w[i] >>= 1;
                if (i + 1 < 4) e.w[i] |= e.w[i + 1] << 63;
            }
        }
        return Fr::from_u64(5).pow(e);
    }
}
