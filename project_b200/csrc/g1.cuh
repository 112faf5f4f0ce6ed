// BLS12-381 G1 (y^2 = x^3 + 4 over Fp) for the GPU: affine points and XYZZ
// accumulators (x = X/ZZ, y = Y/ZZZ, ZZ^3 = ZZZ^2; ZZ = 0 is the point at
// infinity).  Formulas are the standard XYZZ ones for a = 0 (mixed addition 8M+2S,
// full addition 12M+2S, doubling 6M+4S ... in Fp multiplications).  Everything is
// host-compilable so the formulas can be checked on the CPU.
#pragma once

#include "field.cuh"

namespace gzk
{
    struct G1Affine
    {
        Fp x, y;  // Montgomery form; (0, 0) encodes the point at infinity
        GZK_HD bool is_infinity() const { return x.is_zero() && y.is_zero(); }
        GZK_HD static G1Affine infinity()
        {
            G1Affine p;
            p.x = Fp::zero();
            p.y = Fp::zero();
            return p;
        }
    };

    struct G1Xyzz
    {
        Fp X, Y, ZZ, ZZZ;
        GZK_HD bool is_infinity() const { return ZZ.is_zero(); }
        GZK_HD static G1Xyzz infinity()
        {
            G1Xyzz p;
            p.X = Fp::zero();
            p.Y = Fp::zero();
            p.ZZ = Fp::zero();
            p.ZZZ = Fp::zero();
            return p;
        }
        GZK_HD static G1Xyzz from_affine(const G1Affine& a)
        {
            if (a.is_infinity()) return infinity();
            G1Xyzz p;
            p.X = a.x;
            p.Y = a.y;
            p.ZZ = Fp::one();
            p.ZZZ = Fp::one();
            return p;
        }
    };

    GZK_HD Fp fp_dbl(const Fp& a) { return add(a, a); }

    // 2 * (affine point)
    GZK_HD G1Xyzz g1_double_affine(const G1Affine& a)
    {
        if (a.is_infinity() || a.y.is_zero()) return G1Xyzz::infinity();
        const Fp U = fp_dbl(a.y);
        const Fp V = sqr(U);
        const Fp W = mul(U, V);
        const Fp S = mul(a.x, V);
        const Fp xx = sqr(a.x);
        const Fp M = add(fp_dbl(xx), xx);
        G1Xyzz r;
        r.X = sub(sqr(M), fp_dbl(S));
        r.Y = sub(mul(M, sub(S, r.X)), mul(W, a.y));
        r.ZZ = V;
        r.ZZZ = W;
        return r;
    }

    GZK_HD G1Xyzz g1_double(const G1Xyzz& p)
    {
        if (p.is_infinity() || p.Y.is_zero()) return G1Xyzz::infinity();
        const Fp U = fp_dbl(p.Y);
        const Fp V = sqr(U);
        const Fp W = mul(U, V);
        const Fp S = mul(p.X, V);
        const Fp xx = sqr(p.X);
        const Fp M = add(fp_dbl(xx), xx);
        G1Xyzz r;
        r.X = sub(sqr(M), fp_dbl(S));
        r.Y = sub(mul(M, sub(S, r.X)), mul(W, p.Y));
        r.ZZ = mul(V, p.ZZ);
        r.ZZZ = mul(W, p.ZZZ);
        return r;
    }

    // p + (affine q), q optionally negated
    GZK_HD G1Xyzz g1_add_mixed(const G1Xyzz& p, const G1Affine& q_in, bool negate = false)
    {
        if (q_in.is_infinity()) return p;
        G1Affine q = q_in;
        if (negate) q.y = neg(q.y);
        if (p.is_infinity()) return G1Xyzz::from_affine(q);
        const Fp U2 = mul(q.x, p.ZZ);
        const Fp S2 = mul(q.y, p.ZZZ);
        const Fp P = sub(U2, p.X);
        const Fp R = sub(S2, p.Y);
        if (P.is_zero())
        {
            if (R.is_zero()) return g1_double_affine(q);
            return G1Xyzz::infinity();
        }
        const Fp PP = sqr(P);
        const Fp PPP = mul(P, PP);
        const Fp Q = mul(p.X, PP);
        G1Xyzz r;
        r.X = sub(sub(sqr(R), PPP), fp_dbl(Q));
        r.Y = sub(mul(R, sub(Q, r.X)), mul(p.Y, PPP));
        r.ZZ = mul(p.ZZ, PP);
        r.ZZZ = mul(p.ZZZ, PPP);
        return r;
    }

    GZK_HD G1Xyzz g1_add(const G1Xyzz& p, const G1Xyzz& q)
    {
        if (p.is_infinity()) return q;
        if (q.is_infinity()) return p;
        const Fp U1 = mul(p.X, q.ZZ);
        const Fp U2 = mul(q.X, p.ZZ);
        const Fp S1 = mul(p.Y, q.ZZZ);
        const Fp S2 = mul(q.Y, p.ZZZ);
        const Fp P = sub(U2, U1);
        const Fp R = sub(S2, S1);
        if (P.is_zero())
        {
            if (R.is_zero()) return g1_double(p);
            return G1Xyzz::infinity();
        }
        const Fp PP = sqr(P);
        const Fp PPP = mul(P, PP);
        const Fp Q = mul(U1, PP);
        G1Xyzz r;
        r.X = sub(sub(sqr(R), PPP), fp_dbl(Q));
        r.Y = sub(mul(R, sub(Q, r.X)), mul(S1, PPP));
        r.ZZ = mul(mul(p.ZZ, q.ZZ), PP);
        r.ZZZ = mul(mul(p.ZZZ, q.ZZZ), PPP);
        return r;
    }

    // Affine coordinates given inv = 1/(ZZ*ZZZ): x = X * ZZZ * inv... (1/ZZ = inv*ZZZ, 1/ZZZ = inv*ZZ)
    GZK_HD G1Affine g1_to_affine_with_inverse(const G1Xyzz& p, const Fp& inv_zz_zzz)
    {
        if (p.is_infinity()) return G1Affine::infinity();
        G1Affine a;
        a.x = mul(p.X, mul(inv_zz_zzz, p.ZZZ));
        a.y = mul(p.Y, mul(inv_zz_zzz, p.ZZ));
        return a;
    }

    GZK_HD G1Affine g1_to_affine(const G1Xyzz& p)
    {
        if (p.is_infinity()) return G1Affine::infinity();
        return g1_to_affine_with_inverse(p, inv(mul(p.ZZ, p.ZZZ)));
    }

#if defined(__CUDACC__)
    __device__ __forceinline__ Fp load_fp(const Fp* p)
    {
        const uint4* q = reinterpret_cast<const uint4*>(p);
        const uint4 a = __ldg(q), b = __ldg(q + 1), c = __ldg(q + 2);
        Fp o;
        o.l[0] = a.x; o.l[1] = a.y; o.l[2] = a.z; o.l[3] = a.w;
        o.l[4] = b.x; o.l[5] = b.y; o.l[6] = b.z; o.l[7] = b.w;
        o.l[8] = c.x; o.l[9] = c.y; o.l[10] = c.z; o.l[11] = c.w;
        return o;
    }
    __device__ __forceinline__ void store_fp(Fp* p, const Fp& v)
    {
        uint4* q = reinterpret_cast<uint4*>(p);
        q[0] = make_uint4(v.l[0], v.l[1], v.l[2], v.l[3]);
        q[1] = make_uint4(v.l[4], v.l[5], v.l[6], v.l[7]);
        q[2] = make_uint4(v.l[8], v.l[9], v.l[10], v.l[11]);
    }
    __device__ __forceinline__ G1Affine load_affine(const G1Affine* p)
    {
        G1Affine a;
        a.x = load_fp(&p->x);
        a.y = load_fp(&p->y);
        return a;
    }
    __device__ __forceinline__ void store_affine(G1Affine* p, const G1Affine& a)
    {
        store_fp(&p->x, a.x);
        store_fp(&p->y, a.y);
    }
    // XYZZ accumulators are written and re-read by later kernels: plain loads
    __device__ __forceinline__ G1Xyzz load_xyzz(const G1Xyzz* p)
    {
        return *p;
    }
    __device__ __forceinline__ void store_xyzz(G1Xyzz* p, const G1Xyzz& a)
    {
        store_fp(&p->X, a.X);
        store_fp(&p->Y, a.Y);
        store_fp(&p->ZZ, a.ZZ);
        store_fp(&p->ZZZ, a.ZZZ);
    }
#endif
}
