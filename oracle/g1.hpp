// TEST INFRASTRUCTURE — CPU oracle (see field.hpp for the full statement).
//
// BLS12-381 G1 (y^2 = x^3 + 4 over Fp) in Jacobian coordinates with the
// textbook double-and-add scalar multiplication.  Restates the *semantics* of
// src/crypto/curve.cpp:81-135 (g1_add / g1_sub / g1_mul wrappers over mcl::G1)
// and src/crypto/curve.cpp:138-238 (g1_mul_same_base_batch = K independent
// scalar multiplications of one base).  Group elements are compared and
// exported in affine form, which is representation-independent.
#pragma once

#include "field.hpp"

namespace oracle
{
    struct G1Affine
    {
        Fp x, y;
        bool infinity = true;
    };

    struct G1
    {
        Fp X, Y, Z;  // Z == 0 <=> point at infinity

        static G1 identity()
        {
            G1 o;
            o.X = Fp::one();
            o.Y = Fp::one();
            o.Z = Fp::zero();
            return o;
        }
        static G1 from_affine(const G1Affine& a)
        {
            if (a.infinity) return identity();
            G1 o;
            o.X = a.x;
            o.Y = a.y;
            o.Z = Fp::one();
            return o;
        }
        bool is_identity() const { return Z.is_zero(); }

        G1 dbl() const
        {
            if (is_identity() || Y.is_zero()) return identity();
            // a = 0 doubling.
            const Fp A = X * X;
            const Fp B = Y * Y;
            const Fp C = B * B;
            Fp D = (X + B);
            D = D * D - A - C;
            D = D + D;
            const Fp E = A + A + A;
            const Fp F = E * E;
            G1 o;
            o.X = F - D - D;
            Fp C8 = C + C;
            C8 = C8 + C8;
            C8 = C8 + C8;
            o.Y = E * (D - o.X) - C8;
            o.Z = Y * Z;
            o.Z = o.Z + o.Z;
            return o;
        }

        G1 add(const G1& q) const
        {
            if (is_identity()) return q;
            if (q.is_identity()) return *this;
            const Fp Z1Z1 = Z * Z;
            const Fp Z2Z2 = q.Z * q.Z;
            const Fp U1 = X * Z2Z2;
            const Fp U2 = q.X * Z1Z1;
            const Fp S1 = Y * q.Z * Z2Z2;
            const Fp S2 = q.Y * Z * Z1Z1;
            if (U1 == U2)
            {
                if (S1 == S2) return dbl();
                return identity();
            }
            const Fp H = U2 - U1;
            const Fp R = S2 - S1;
            const Fp HH = H * H;
            const Fp HHH = H * HH;
            const Fp V = U1 * HH;
            G1 o;
            o.X = R * R - HHH - V - V;
            o.Y = R * (V - o.X) - S1 * HHH;
            o.Z = Z * q.Z * H;
            return o;
        }

        G1 neg() const
        {
            G1 o = *this;
            o.Y = -o.Y;
            return o;
        }

        G1 mul(const Fr& scalar) const
        {
            const auto k = scalar.canonical();
            G1 acc = identity();
            for (std::size_t i = k.bit_length(); i-- > 0;)
            {
                acc = acc.dbl();
                if (k.bit(i)) acc = acc.add(*this);
            }
            return acc;
        }

        G1Affine to_affine() const
        {
            G1Affine a;
            if (is_identity()) return a;
            const Fp zi = Z.inv();
            const Fp zi2 = zi * zi;
            a.x = X * zi2;
            a.y = Y * zi2 * zi;
            a.infinity = false;
            return a;
        }
    };

    inline bool on_curve(const G1Affine& a)
    {
        if (a.infinity) return true;
        return a.y * a.y == a.x * a.x * a.x + Fp::from_u64(4);
    }

    // Wire format shared with the CUDA library: x || y, 48-byte little-endian
    // canonical each; 96 zero bytes encode the point at infinity ((0,0) is not
    // on the curve, so the encoding is unambiguous).
    inline void g1_to_bytes(const G1Affine& a, std::uint8_t* out)
    {
        std::memset(out, 0, 96);
        if (a.infinity) return;
        a.x.to_le_bytes(out);
        a.y.to_le_bytes(out + 48);
    }
    inline G1Affine g1_from_bytes(const std::uint8_t* in)
    {
        G1Affine a;
        bool all_zero = true;
        for (int i = 0; i < 96; ++i) all_zero = all_zero && in[i] == 0;
        if (all_zero) return a;
        a.x = Fp::from_le_bytes(in);
        a.y = Fp::from_le_bytes(in + 48);
        a.infinity = false;
        return a;
    }
}
