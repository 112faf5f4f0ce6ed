// Barycentric weight vector of a root-of-unity domain at a point x:
//   w_i = (x^n - 1)/n * omega^i / (x - omega^i).
// The n field inversions are one batch inversion, organised for the GPU as
//   pass 1  per-CTA product of its 1024 denominators,
//   pass 2  one CTA inverts all CTA products (scan of products + ONE field
//           inversion for the whole vector),
//   pass 3  per-CTA: in-CTA exclusive prefix/suffix products turn the CTA inverse
//           into the 1024 element inverses; the weight is written once, coalesced.
// Denominators are regenerated from two small omega tables in pass 3 instead of
// being stored, so HBM traffic is the 32 n bytes of the output only.
//
// Whole-domain vectors use the symmetry of the domain under multiplication by the 4th
// root of unity I: the points a, -a, Ia, -Ia (a = omega^j, j < n/4) share the denominator
// D_j = x^4 - a^4, since 1/(x-a) = (x+a)(x^2+a^2)/D_j, 1/(x+a) = (x-a)(x^2+a^2)/D_j,
// 1/(x-Ia) = (x+Ia)(x^2-a^2)/D_j, 1/(x+Ia) = (x-Ia)(x^2-a^2)/D_j.  The batch inversion then
// runs over n/4 values and the whole vector costs about 6 multiplications per weight
// instead of 13.
#include "common.cuh"

namespace gzk
{
    namespace
    {
        constexpr int kThreads = 256;
        constexpr int kElems = 4;
        constexpr int kChunk = kThreads * kElems;

        struct BaryArgs
        {
            const Fr* lo;
            const Fr* hi;
            unsigned lo_bits;
            uint64_t n;      // number of weights produced by this call
            uint64_t first;  // domain index of the first one (ranges wrap around the domain)
            uint64_t mask;   // domain size - 1
            Fr x;       // Montgomery
            Fr scale;   // (x^n - 1)/n, Montgomery
            Fr x2, x4;  // x^2, x^4 (whole-domain kernels)
            Fr root4;   // I = omega^(n/4)
            uint64_t keep;  // whole-domain kernels: weights with index >= keep are not needed (except the last two, which evaluations rotated by one and by two read for rows 0 and 1)
            // fused whole-domain kernel: CTA b works on chunk b of the quartets while b < kept_blocks and on chunk
            // last_chunk otherwise (a short prefix is kept: only its chunks and the one holding the last two weights run)
            uint32_t kept_blocks, last_chunk;
        };

        __device__ __forceinline__ Fr shfl_fr(const Fr& v, int src_lane)
        {
            Fr o;
#pragma unroll
            for (int i = 0; i < 8; ++i) o.l[i] = __shfl_sync(0xffffffffu, v.l[i], src_lane);
            return o;
        }

        __global__ void __launch_bounds__(kThreads) bary_products_kernel(BaryArgs a, Fr* block_products, int* status)
        {
            __shared__ Fr warp_products[kThreads / 32];
            const uint64_t base = static_cast<uint64_t>(blockIdx.x) * kChunk;
            Fr prod = Fr::one();
#pragma unroll
            for (int j = 0; j < kElems; ++j)
            {
                const uint64_t e = base + static_cast<uint64_t>(j) * kThreads + threadIdx.x;
                if (e < a.n)
                {
                    const Fr d = sub(a.x, domain_point(a.lo, a.hi, a.lo_bits, (a.first + e) & a.mask));
                    if (d.is_zero()) raise_status(status, GZK_E_DOMAIN, 101);
                    prod = mul(prod, d);
                }
            }
            const int lane = threadIdx.x & 31;
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1)
            {
                const Fr other = shfl_fr(prod, (lane + offset) & 31);
                if (lane < offset) prod = mul(prod, other);
            }
            if (lane == 0) warp_products[threadIdx.x >> 5] = prod;
            __syncthreads();
            if (threadIdx.x == 0)
            {
                Fr total = warp_products[0];
#pragma unroll
                for (int w = 1; w < kThreads / 32; ++w) total = mul(total, warp_products[w]);
                store_fr(block_products + blockIdx.x, total);
            }
        }

        // In-place batch inversion of `count` non-zero values by ONE CTA (values are
        // Montgomery).  Each thread owns a contiguous run; run products are combined
        // with shared-memory exclusive prefix/suffix product scans.
        constexpr int kInvThreads = 512;
        __global__ void __launch_bounds__(kInvThreads) batch_invert_single_cta_kernel(Fr* values, Fr* prefix_tmp, uint32_t count)
        {
            __shared__ Fr pre[kInvThreads];
            __shared__ Fr suf[kInvThreads];
            __shared__ Fr total_inv;
            const uint32_t t = threadIdx.x;
            const uint32_t run = (count + kInvThreads - 1) / kInvThreads;
            const uint32_t begin = t * run < count ? t * run : count;
            const uint32_t end = begin + run < count ? begin + run : count;
            Fr acc = Fr::one();
            for (uint32_t i = begin; i < end; ++i)
            {
                store_fr(prefix_tmp + i, acc);
                acc = mul(acc, load_fr_plain(values + i));
            }
            pre[t] = acc;
            suf[t] = acc;
            __syncthreads();
            // inclusive scans (Hillis-Steele): pre = prod_{t' <= t}, suf = prod_{t' >= t}
            for (uint32_t offset = 1; offset < kInvThreads; offset <<= 1)
            {
                Fr p = pre[t], s = suf[t];
                const bool has_p = t >= offset, has_s = t + offset < kInvThreads;
                Fr po, so;
                if (has_p) po = pre[t - offset];
                if (has_s) so = suf[t + offset];
                __syncthreads();
                if (has_p) pre[t] = mul(p, po);
                if (has_s) suf[t] = mul(s, so);
                __syncthreads();
            }
            if (t == 0) total_inv = inv(pre[kInvThreads - 1]);
            __syncthreads();
            // 1 / (own run product) = total_inv * prod_{t' < t} * prod_{t' > t}
            Fr outer = total_inv;
            if (t > 0) outer = mul(outer, pre[t - 1]);
            if (t + 1 < kInvThreads) outer = mul(outer, suf[t + 1]);
            for (uint32_t i = end; i-- > begin;)
            {
                const Fr v = load_fr_plain(values + i);
                store_fr(values + i, mul(outer, load_fr_plain(prefix_tmp + i)));
                outer = mul(outer, v);
            }
        }

        __global__ void __launch_bounds__(kThreads) bary_finish_kernel(BaryArgs a, const Fr* block_inverses, Fr* out)
        {
            __shared__ Fr warp_incl[kThreads / 32];
            __shared__ Fr warp_pre[kThreads / 32];
            __shared__ Fr warp_suf[kThreads / 32];
            const uint64_t base = static_cast<uint64_t>(blockIdx.x) * kChunk;
            const int lane = threadIdx.x & 31;
            const int warp = threadIdx.x >> 5;

            Fr d[kElems];
#pragma unroll
            for (int j = 0; j < kElems; ++j)
            {
                const uint64_t e = base + static_cast<uint64_t>(j) * kThreads + threadIdx.x;
                d[j] = e < a.n ? sub(a.x, domain_point(a.lo, a.hi, a.lo_bits, (a.first + e) & a.mask)) : Fr::one();
            }
            // thread-local exclusive prefixes; `mine` = product of the thread's elements
            Fr pre[kElems];
            Fr mine = Fr::one();
#pragma unroll
            for (int j = 0; j < kElems; ++j)
            {
                pre[j] = mine;
                mine = mul(mine, d[j]);
            }
            // warp inclusive prefix and suffix products of `mine`
            Fr incl = mine, sufx = mine;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1)
            {
                const Fr up = shfl_fr(incl, (lane - offset) & 31);
                const Fr down = shfl_fr(sufx, (lane + offset) & 31);
                if (lane >= offset) incl = mul(incl, up);
                if (lane + offset < 32) sufx = mul(sufx, down);
            }
            Fr left = shfl_fr(incl, (lane - 1) & 31);   // exclusive prefix within the warp
            Fr right = shfl_fr(sufx, (lane + 1) & 31);  // exclusive suffix within the warp
            if (lane == 0) left = Fr::one();
            if (lane == 31) right = Fr::one();
            if (lane == 31) warp_incl[warp] = incl;
            __syncthreads();
            if (threadIdx.x == 0)
            {
                Fr run = Fr::one();
#pragma unroll
                for (int w = 0; w < kThreads / 32; ++w)
                {
                    warp_pre[w] = run;
                    run = mul(run, warp_incl[w]);
                }
                run = Fr::one();
#pragma unroll
                for (int w = kThreads / 32 - 1; w >= 0; --w)
                {
                    warp_suf[w] = run;
                    run = mul(run, warp_incl[w]);
                }
            }
            __syncthreads();
            // outer = 1 / (product of this thread's elements)
            Fr outer = mul(load_fr(block_inverses + blockIdx.x), mul(mul(left, warp_pre[warp]), mul(right, warp_suf[warp])));
            // walk the thread's elements backwards: inverse_j = outer * suffix_j * pre_j
            Fr rest = outer;  // inverse of the product of the thread's elements 0 .. j
#pragma unroll
            for (int j = kElems - 1; j >= 0; --j)
            {
                const uint64_t e = base + static_cast<uint64_t>(j) * kThreads + threadIdx.x;
                const Fr inverse = mul(rest, pre[j]);
                // omega^e = x - d_e: cheaper to rebuild than to keep in registers
                if (e < a.n) store_fr(out + e, mul(mul(a.scale, sub(a.x, d[j])), inverse));
                if (j > 0) rest = mul(rest, d[j]);
            }
        }
    }

    namespace
    {
        // a = omega^j and the shared denominator D_j = x^4 - a^4 of its four points
        __device__ __forceinline__ Fr quartet_denominator(const BaryArgs& a, uint64_t j, Fr* point, Fr* point2)
        {
            *point = domain_point(a.lo, a.hi, a.lo_bits, j);
            *point2 = sqr(*point);
            return sub(a.x4, sqr(*point2));
        }

        // a.n = n/4 here: one denominator per quartet
        __global__ void __launch_bounds__(kThreads) bary4_products_kernel(BaryArgs a, Fr* block_products, int* status)
        {
            __shared__ Fr warp_products[kThreads / 32];
            const uint64_t base = static_cast<uint64_t>(blockIdx.x) * kChunk;
            Fr prod = Fr::one();
#pragma unroll
            for (int j = 0; j < kElems; ++j)
            {
                const uint64_t e = base + static_cast<uint64_t>(j) * kThreads + threadIdx.x;
                if (e < a.n)
                {
                    Fr p1, p2;
                    const Fr d = quartet_denominator(a, e, &p1, &p2);
                    if (d.is_zero()) raise_status(status, GZK_E_DOMAIN, 102);
                    prod = mul(prod, d);
                }
            }
            const int lane = threadIdx.x & 31;
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1)
            {
                const Fr other = shfl_fr(prod, (lane + offset) & 31);
                if (lane < offset) prod = mul(prod, other);
            }
            if (lane == 0) warp_products[threadIdx.x >> 5] = prod;
            __syncthreads();
            if (threadIdx.x == 0)
            {
                Fr total = warp_products[0];
#pragma unroll
                for (int w = 1; w < kThreads / 32; ++w) total = mul(total, warp_products[w]);
                store_fr(block_products + blockIdx.x, total);
            }
        }

        __global__ void __launch_bounds__(kThreads, 2) bary4_finish_kernel(BaryArgs a, const Fr* block_inverses, Fr* out)
        {
            __shared__ Fr warp_incl[kThreads / 32];
            __shared__ Fr warp_pre[kThreads / 32];
            __shared__ Fr warp_suf[kThreads / 32];
            const uint64_t base = static_cast<uint64_t>(blockIdx.x) * kChunk;
            const int lane = threadIdx.x & 31;
            const int warp = threadIdx.x >> 5;

            Fr d[kElems], pre[kElems];
            Fr mine = Fr::one();
#pragma unroll
            for (int j = 0; j < kElems; ++j)
            {
                const uint64_t e = base + static_cast<uint64_t>(j) * kThreads + threadIdx.x;
                Fr p1, p2;
                d[j] = e < a.n ? quartet_denominator(a, e, &p1, &p2) : Fr::one();
                pre[j] = mine;
                mine = mul(mine, d[j]);
            }
            Fr incl = mine, sufx = mine;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1)
            {
                const Fr up = shfl_fr(incl, (lane - offset) & 31);
                const Fr down = shfl_fr(sufx, (lane + offset) & 31);
                if (lane >= offset) incl = mul(incl, up);
                if (lane + offset < 32) sufx = mul(sufx, down);
            }
            Fr left = shfl_fr(incl, (lane - 1) & 31);
            Fr right = shfl_fr(sufx, (lane + 1) & 31);
            if (lane == 0) left = Fr::one();
            if (lane == 31) right = Fr::one();
            if (lane == 31) warp_incl[warp] = incl;
            __syncthreads();
            if (threadIdx.x == 0)
            {
                Fr run = Fr::one();
#pragma unroll
                for (int w = 0; w < kThreads / 32; ++w)
                {
                    warp_pre[w] = run;
                    run = mul(run, warp_incl[w]);
                }
                run = Fr::one();
#pragma unroll
                for (int w = kThreads / 32 - 1; w >= 0; --w)
                {
                    warp_suf[w] = run;
                    run = mul(run, warp_incl[w]);
                }
            }
            __syncthreads();
            const Fr outer = mul(load_fr(block_inverses + blockIdx.x), mul(mul(left, warp_pre[warp]), mul(right, warp_suf[warp])));
            Fr rest = mul(a.scale, outer);  // (x^n-1)/n over the product of the thread's denominators 0 .. j
#pragma unroll
            for (int j = kElems - 1; j >= 0; --j)
            {
                const uint64_t e = base + static_cast<uint64_t>(j) * kThreads + threadIdx.x;
                const Fr scaled_inverse = mul(rest, pre[j]);  // (x^n-1)/n / D_e
                if (j > 0) rest = mul(rest, d[j]);
                if (e >= a.n) continue;
                const Fr p1 = domain_point(a.lo, a.hi, a.lo_bits, e);
                const Fr p2 = sqr(p1);
                const Fr ip1 = mul(a.root4, p1);
                const Fr plus = add(a.x2, p2), minus = sub(a.x2, p2);
                const Fr ea = mul(scaled_inverse, p1), eia = mul(scaled_inverse, ip1);
                store_fr(out + e, mul(ea, mul(add(a.x, p1), plus)));                          // point  a
                store_fr(out + e + 2 * a.n, neg(mul(ea, mul(sub(a.x, p1), plus))));           // point -a
                store_fr(out + e + a.n, mul(eia, mul(add(a.x, ip1), minus)));                 // point  Ia
                store_fr(out + e + 3 * a.n, neg(mul(eia, mul(sub(a.x, ip1), minus))));        // point -Ia
            }
        }
    }

    namespace
    {
        // Whole-domain weights in ONE launch: every CTA builds the denominators of its 1024 quartets,
        // inverts THEIR product itself (one serial inversion per CTA, all CTAs in parallel) and writes
        // its 4096 weights.  Nothing is exchanged between CTAs, so there is neither a products pass nor
        // a separate inversion pass: on a small domain (a few CTAs) the call is one short chain instead
        // of three dependent launches, on a large one the serial inversions hide behind the arithmetic
        // of the CTA that shares the SM.
        // ELEMS quartets per thread: the whole-domain call of a SMALL domain (a few thousand points, the
        // node-domain weights every binding of the flow asks for) is one dependent chain, so it takes one
        // quartet per thread and spreads over as many SMs as it has 256-quartet groups; a large domain
        // takes four and amortises the serial inversion over 1024 quartets.
        struct FusedShared
        {
            Fr warp_incl[kThreads / 32];
            Fr warp_pre[kThreads / 32];
            Fr warp_suf[kThreads / 32];
            Fr cta_inverse;
        };

        template <int ELEMS>
        __device__ __forceinline__ void bary4_fused_body(const BaryArgs& a, Fr* out, int* status, FusedShared& sh)
        {
            Fr* warp_incl = sh.warp_incl;
            Fr* warp_pre = sh.warp_pre;
            Fr* warp_suf = sh.warp_suf;
            Fr& cta_inverse = sh.cta_inverse;
            const uint32_t chunk = blockIdx.x < a.kept_blocks ? blockIdx.x : a.last_chunk;
            const uint64_t base = static_cast<uint64_t>(chunk) * (kThreads * ELEMS);
            const int lane = threadIdx.x & 31;
            const int warp = threadIdx.x >> 5;

            Fr d[ELEMS], pre[ELEMS];
            Fr mine = Fr::one();
#pragma unroll
            for (int j = 0; j < ELEMS; ++j)
            {
                const uint64_t e = base + static_cast<uint64_t>(j) * kThreads + threadIdx.x;
                Fr p1, p2;
                d[j] = e < a.n ? quartet_denominator(a, e, &p1, &p2) : Fr::one();
                pre[j] = mine;
                mine = mul(mine, d[j]);
            }
            Fr incl = mine, sufx = mine;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1)
            {
                const Fr up = shfl_fr(incl, (lane - offset) & 31);
                const Fr down = shfl_fr(sufx, (lane + offset) & 31);
                if (lane >= offset) incl = mul(incl, up);
                if (lane + offset < 32) sufx = mul(sufx, down);
            }
            Fr left = shfl_fr(incl, (lane - 1) & 31);
            Fr right = shfl_fr(sufx, (lane + 1) & 31);
            if (lane == 0) left = Fr::one();
            if (lane == 31) right = Fr::one();
            if (lane == 31) warp_incl[warp] = incl;
            __syncthreads();
            if (threadIdx.x == 0)
            {
                Fr run = Fr::one();
#pragma unroll
                for (int w = 0; w < kThreads / 32; ++w)
                {
                    warp_pre[w] = run;
                    run = mul(run, warp_incl[w]);
                }
                const Fr total = run;
                run = Fr::one();
#pragma unroll
                for (int w = kThreads / 32 - 1; w >= 0; --w)
                {
                    warp_suf[w] = run;
                    run = mul(run, warp_incl[w]);
                }
                if (total.is_zero()) raise_status(status, GZK_E_DOMAIN, 103);
                cta_inverse = inv(total);
            }
            __syncthreads();
            const Fr outer = mul(cta_inverse, mul(mul(left, warp_pre[warp]), mul(right, warp_suf[warp])));
            Fr rest = mul(a.scale, outer);  // (x^n-1)/n over the product of the thread's denominators 0 .. j
#pragma unroll
            for (int j = ELEMS - 1; j >= 0; --j)
            {
                const uint64_t e = base + static_cast<uint64_t>(j) * kThreads + threadIdx.x;
                const Fr scaled_inverse = mul(rest, pre[j]);  // (x^n-1)/n / D_e
                if (j > 0) rest = mul(rest, d[j]);
                if (e >= a.n) continue;
                const Fr p1 = domain_point(a.lo, a.hi, a.lo_bits, e);
                const Fr p2 = sqr(p1);
                const Fr ip1 = mul(a.root4, p1);
                const Fr plus = add(a.x2, p2), minus = sub(a.x2, p2);
                const uint64_t last = 4 * a.n - 1;
                auto wanted = [&](uint64_t index) { return index < a.keep || index + 1 >= last; };  // the prefix and the last two
                // the factor the two points of a pair share is formed once: three multiplications per pair, not four
                if (wanted(e) || wanted(e + 2 * a.n))
                {
                    const Fr shared = mul(mul(scaled_inverse, p1), plus);
                    if (wanted(e)) store_fr(out + e, mul(shared, add(a.x, p1)));                        // point  a
                    if (wanted(e + 2 * a.n)) store_fr(out + e + 2 * a.n, neg(mul(shared, sub(a.x, p1))));  // point -a
                }
                if (wanted(e + a.n) || wanted(e + 3 * a.n))
                {
                    const Fr shared = mul(mul(scaled_inverse, ip1), minus);
                    if (wanted(e + a.n)) store_fr(out + e + a.n, mul(shared, add(a.x, ip1)));                 // point  Ia
                    if (wanted(e + 3 * a.n)) store_fr(out + e + 3 * a.n, neg(mul(shared, sub(a.x, ip1))));   // point -Ia
                }
            }
        }

        template <int ELEMS>
        __global__ void __launch_bounds__(kThreads, 2) bary4_fused_kernel(BaryArgs a, Fr* out, int* status)
        {
            __shared__ FusedShared sh;
            bary4_fused_body<ELEMS>(a, out, status, sh);
        }

        // Several points of one small domain in one launch (blockIdx.y picks the point): the weight vectors a head
        // needs at the same Fiat-Shamir stage are independent dependent-chains, so side by side they cost one chain.
        constexpr int kMaxPoints = 4;
        struct BaryMultiArgs
        {
            BaryArgs point[kMaxPoints];
            Fr* out[kMaxPoints];
        };
        __global__ void __launch_bounds__(kThreads, 2) bary4_fused_multi_kernel(BaryMultiArgs m, int* status)
        {
            __shared__ FusedShared sh;
            bary4_fused_body<1>(m.point[blockIdx.y], m.out[blockIdx.y], status, sh);
        }
    }

    // Shared with other translation units: in-place batch inversion of a device
    // array of Montgomery values by one CTA; `tmp` must hold `count` elements.
    int launch_batch_invert_single_cta(gzk_ctx* ctx, Fr* values, Fr* tmp, uint32_t count)
    {
        if (count == 0) return GZK_OK;
        LaunchScope scope(ctx, "batch_invert_cta");
        batch_invert_single_cta_kernel<<<1, kInvThreads, 0, ctx->stream>>>(values, tmp, count);
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return GZK_OK;
    }
}

using namespace gzk;

static int bary_impl(gzk_ctx* ctx, unsigned log2n, const uint8_t x_bytes[32], uint64_t first, uint64_t count, gzk_buf* out, uint64_t keep = ~0ULL)
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (x_bytes == nullptr || out == nullptr) return fail(ctx, GZK_E_INVALID, "bary_weights: null argument");
    if (log2n > 30) return fail(ctx, GZK_E_INVALID, "bary_weights: domain too large");
    const uint64_t n = 1ULL << log2n;
    if (count > n || first >= n) return fail(ctx, GZK_E_INVALID, "bary_weights: range exceeds the domain");
    if (out->kind != GZK_KIND_FR_MONT || out->count < count)
        return fail(ctx, GZK_E_INVALID, "bary_weights: output must be a Montgomery buffer of the requested size");
    bool canonical = false;
    const Fr x_plain = host_fr_from_bytes(x_bytes, &canonical);
    if (!canonical) return fail(ctx, GZK_E_INVALID, "bary_weights: x is not a canonical field element");
    GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const DomainTables* dom = nullptr;
    int rc = get_domain(ctx, log2n, &dom);
    if (rc != GZK_OK) return rc;

    BaryArgs args;
    args.lo = dom->lo;
    args.hi = dom->hi;
    args.lo_bits = dom->lo_bits;
    args.n = count;
    args.first = first;
    args.mask = n - 1;
    args.keep = keep;
    args.kept_blocks = ~0u;
    args.last_chunk = 0;
    args.x = to_mont(x_plain);
    Fr xn = args.x;
    for (unsigned s = 0; s < log2n; ++s) xn = sqr(xn);
    const Fr zero_eval = sub(xn, Fr::one());
    if (zero_eval.is_zero()) return fail(ctx, GZK_E_DOMAIN, "bary_weights: x is a point of the domain");
    args.scale = mul(zero_eval, dom->inv_size);
    if (count == 0) return GZK_OK;

    const bool quartets = first == 0 && count == n && n >= 4;
    if (quartets)
    {
        args.n = n / 4;
        args.x2 = sqr(args.x);
        args.x4 = sqr(args.x2);
        args.root4 = host_root_of_unity(2);
    }
    // a whole small domain: one quartet per thread (see bary4_fused_kernel)
    const bool short_chain = quartets && args.n <= (1u << 16);
    const uint32_t blocks = short_chain ? static_cast<uint32_t>((args.n + kThreads - 1) / kThreads) : static_cast<uint32_t>((args.n + kChunk - 1) / kChunk);
    void* scratch = nullptr;
    if ((rc = ensure_scratch(ctx, 2, static_cast<size_t>(blocks) * 2 * sizeof(Fr), &scratch)) != GZK_OK) return rc;
    Fr* products = static_cast<Fr*>(scratch);
    Fr* tmp = products + blocks;
    if ((rc = begin_call(ctx)) != GZK_OK) return rc;
    if (quartets)
    {
        // Quartet e yields the weights e, e + n/4, e + n/2 and e + 3n/4.  When only a prefix shorter than n/4 is kept,
        // the quartets below `keep` and the last two (weights n - 1 and n - 2, both in the last chunk) are all that is needed: the work shrinks with
        // the prefix instead of staying that of the whole domain.
        args.kept_blocks = blocks;
        args.last_chunk = blocks - 1;
        uint32_t launch_blocks = blocks;
        if (keep < args.n)
        {
            const uint64_t per_block = short_chain ? kThreads : kChunk;
            const uint64_t kept = (keep + per_block - 1) / per_block;
            if (kept + 1 < blocks)
            {
                args.kept_blocks = static_cast<uint32_t>(kept);
                launch_blocks = static_cast<uint32_t>(kept) + 1;
            }
        }
        {
            LaunchScope scope(ctx, "bary_fused");
            if (short_chain)
                bary4_fused_kernel<1><<<launch_blocks, kThreads, 0, ctx->stream>>>(args, static_cast<Fr*>(out->dptr), ctx->d_status);
            else
                bary4_fused_kernel<kElems><<<launch_blocks, kThreads, 0, ctx->stream>>>(args, static_cast<Fr*>(out->dptr), ctx->d_status);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        rc = finish_call(ctx, "bary_weights: invalid input");
        if (rc == GZK_E_DOMAIN) return fail(ctx, GZK_E_DOMAIN, "bary_weights: x is a point of the domain");
        return rc;
    }
    {
        LaunchScope scope(ctx, "bary_products");
        bary_products_kernel<<<blocks, kThreads, 0, ctx->stream>>>(args, products, ctx->d_status);
    }
    GZK_CUDA_TRY(ctx, cudaGetLastError());
    if ((rc = launch_batch_invert_single_cta(ctx, products, tmp, blocks)) != GZK_OK) return rc;
    {
        LaunchScope scope(ctx, "bary_finish");
        bary_finish_kernel<<<blocks, kThreads, 0, ctx->stream>>>(args, products, static_cast<Fr*>(out->dptr));
    }
    GZK_CUDA_TRY(ctx, cudaGetLastError());
    rc = finish_call(ctx, "bary_weights: invalid input");
    if (rc == GZK_E_DOMAIN) return fail(ctx, GZK_E_DOMAIN, "bary_weights: x is a point of the domain");
    return rc;
}

// Weights of the same small domain at several points in one launch (gzk_bary_weights for each otherwise).
extern "C" int gzk_bary_weights_multi(gzk_ctx* ctx, unsigned log2n, const uint8_t* points, size_t count, gzk_buf* const* outs)
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (count == 0) return GZK_OK;
    if (points == nullptr || outs == nullptr) return fail(ctx, GZK_E_INVALID, "bary_weights_multi: null argument");
    const uint64_t n = log2n <= 30 ? (1ULL << log2n) : 0;
    const bool one_launch = count <= static_cast<size_t>(kMaxPoints) && n >= 4 && n / 4 <= (1u << 16);
    if (!one_launch)
    {
        for (size_t j = 0; j < count; ++j)
        {
            const int rc = bary_impl(ctx, log2n, points + 32 * j, 0, n, outs[j]);
            if (rc != GZK_OK) return rc;
        }
        return GZK_OK;
    }
    GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const DomainTables* dom = nullptr;
    int rc = get_domain(ctx, log2n, &dom);
    if (rc != GZK_OK) return rc;
    BaryMultiArgs m{};
    for (size_t j = 0; j < count; ++j)
    {
        if (outs[j] == nullptr || outs[j]->kind != GZK_KIND_FR_MONT || outs[j]->count < n)
            return fail(ctx, GZK_E_INVALID, "bary_weights: output must be a Montgomery buffer of the requested size");
        bool canonical = false;
        const Fr x_plain = host_fr_from_bytes(points + 32 * j, &canonical);
        if (!canonical) return fail(ctx, GZK_E_INVALID, "bary_weights: x is not a canonical field element");
        BaryArgs& a = m.point[j];
        a.lo = dom->lo;
        a.hi = dom->hi;
        a.lo_bits = dom->lo_bits;
        a.n = n / 4;
        a.first = 0;
        a.mask = n - 1;
        a.keep = ~0ULL;
        a.kept_blocks = ~0u;  // every CTA works on its own chunk
        a.last_chunk = 0;
        a.x = to_mont(x_plain);
        Fr xn = a.x;
        for (unsigned s = 0; s < log2n; ++s) xn = sqr(xn);
        const Fr zero_eval = sub(xn, Fr::one());
        if (zero_eval.is_zero()) return fail(ctx, GZK_E_DOMAIN, "bary_weights: x is a point of the domain");
        a.scale = mul(zero_eval, dom->inv_size);
        a.x2 = sqr(a.x);
        a.x4 = sqr(a.x2);
        a.root4 = host_root_of_unity(2);
        m.out[j] = static_cast<Fr*>(outs[j]->dptr);
    }
    if ((rc = begin_call(ctx)) != GZK_OK) return rc;
    {
        LaunchScope scope(ctx, "bary_fused");
        const dim3 grid(static_cast<unsigned>((n / 4 + kThreads - 1) / kThreads), static_cast<unsigned>(count));
        bary4_fused_multi_kernel<<<grid, kThreads, 0, ctx->stream>>>(m, ctx->d_status);
    }
    GZK_CUDA_TRY(ctx, cudaGetLastError());
    rc = finish_call(ctx, "bary_weights: invalid input");
    if (rc == GZK_E_DOMAIN) return fail(ctx, GZK_E_DOMAIN, "bary_weights: x is a point of the domain");
    return rc;
}

// The whole-domain weights of which only w[0 .. keep), w[n-2] and w[n-1] will be read (columns stored as prefixes
// shorter than the domain; the last weights meet rows 0 and 1 at rotations 1 and 2): the other entries of `out` are
// left as they were.
extern "C" int gzk_bary_weights_prefix(gzk_ctx* ctx, unsigned log2n, const uint8_t x_bytes[32], uint64_t keep, gzk_buf* out)
{
    return bary_impl(ctx, log2n, x_bytes, 0, log2n <= 30 ? (1ULL << log2n) : 0, out, keep);
}

extern "C" int gzk_bary_weights(gzk_ctx* ctx, unsigned log2n, const uint8_t x_bytes[32], gzk_buf* out)
{
    return bary_impl(ctx, log2n, x_bytes, 0, log2n <= 30 ? (1ULL << log2n) : 0, out);
}

// Weights first, first+1, ..., first+count-1 (indices modulo the domain size): the
// slice of the vector one GPU needs when the rows of a domain are sharded.  The
// batch inversion runs over the slice only, so no exchange between GPUs is needed.
extern "C" int gzk_bary_weights_range(gzk_ctx* ctx, unsigned log2n, const uint8_t x_bytes[32], uint64_t first, uint64_t count, gzk_buf* out)
{
    return bary_impl(ctx, log2n, x_bytes, first, count, out);
}
