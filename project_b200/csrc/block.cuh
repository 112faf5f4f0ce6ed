// CTA-level building blocks shared by the column-builder kernels: typed loads
// of column values, product scans for batch inversion, additive scans for
// running sums.  All values inside kernels are Montgomery-form Fr.
#pragma once

#include "common.cuh"

namespace gzk
{
    // A column as the kernels see it: device pointer + buffer kind.
    struct ColRef
    {
        const void* ptr;
        int kind;
    };

#if defined(__CUDACC__)
    // Value i of a column, converted to Montgomery form.
    __device__ __forceinline__ Fr col_load_mont(const ColRef& c, uint64_t i)
    {
        if (c.kind == GZK_KIND_FR_MONT) return load_fr(static_cast<const Fr*>(c.ptr) + i);
        if (c.kind == GZK_KIND_FR) return to_mont(load_fr(static_cast<const Fr*>(c.ptr) + i));
        Fr f = Fr::zero();
        if (c.kind == GZK_KIND_U32)
        {
            f.l[0] = __ldg(static_cast<const uint32_t*>(c.ptr) + i);
            return to_mont(f);
        }
        const long long v = __ldg(static_cast<const long long*>(c.ptr) + i);
        const unsigned long long mag = v < 0 ? 0ULL - static_cast<unsigned long long>(v) : static_cast<unsigned long long>(v);
        f.l[0] = static_cast<uint32_t>(mag);
        f.l[1] = static_cast<uint32_t>(mag >> 32);
        f = to_mont(f);
        return v < 0 ? neg(f) : f;
    }

    // Value i of a column as the residue it is stored as: canonical for the kinds FR, U32, I64
    // (i.e. the Montgomery representation of x / R: one factor of R short, "deficit" 1),
    // Montgomery for FR_MONT (deficit 0).
    __device__ __forceinline__ int deficit(const ColRef& c) { return c.kind == GZK_KIND_FR_MONT ? 0 : 1; }

    __device__ __forceinline__ Fr col_load_stored(const ColRef& c, uint64_t i)
    {
        if (c.kind == GZK_KIND_FR_MONT || c.kind == GZK_KIND_FR) return load_fr(static_cast<const Fr*>(c.ptr) + i);
        Fr f = Fr::zero();
        if (c.kind == GZK_KIND_U32)
        {
            f.l[0] = __ldg(static_cast<const uint32_t*>(c.ptr) + i);
            return f;
        }
        const long long v = __ldg(static_cast<const long long*>(c.ptr) + i);
        const unsigned long long mag = v < 0 ? 0ULL - static_cast<unsigned long long>(v) : static_cast<unsigned long long>(v);
        f.l[0] = static_cast<uint32_t>(mag);
        f.l[1] = static_cast<uint32_t>(mag >> 32);
        return v < 0 ? neg(f) : f;
    }


    __device__ __forceinline__ Fr shfl_fr_idx(const Fr& v, int src_lane)
    {
        Fr o;
#pragma unroll
        for (int i = 0; i < 8; ++i) o.l[i] = __shfl_sync(0xffffffffu, v.l[i], src_lane);
        return o;
    }

    // Product of `mine` over the CTA, returned to thread 0 (other threads get
    // an unspecified value).  THREADS must be a multiple of 32.
    template <int THREADS>
    __device__ __forceinline__ Fr block_product(Fr mine, Fr* warp_slots /* THREADS/32 shared */)
    {
        const int lane = threadIdx.x & 31;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1)
        {
            const Fr other = shfl_fr_idx(mine, (lane + offset) & 31);
            if (lane < offset) mine = mul(mine, other);
        }
        if (lane == 0) warp_slots[threadIdx.x >> 5] = mine;
        __syncthreads();
        Fr total = warp_slots[0];
        if (threadIdx.x == 0)
        {
#pragma unroll
            for (int w = 1; w < THREADS / 32; ++w) total = mul(total, warp_slots[w]);
        }
        __syncthreads();
        return total;
    }

    // Given each thread's product `mine` and the inverse of the product over
    // the whole CTA, returns 1/mine.  Uses 3 * THREADS/32 shared slots.
    template <int THREADS>
    __device__ __forceinline__ Fr block_invert_products(const Fr& mine, const Fr& cta_inverse, Fr* slots)
    {
        constexpr int W = THREADS / 32;
        Fr* warp_incl = slots;
        Fr* warp_pre = slots + W;
        Fr* warp_suf = slots + 2 * W;
        const int lane = threadIdx.x & 31;
        const int warp = threadIdx.x >> 5;
        Fr incl = mine, sufx = mine;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1)
        {
            const Fr up = shfl_fr_idx(incl, (lane - offset) & 31);
            const Fr down = shfl_fr_idx(sufx, (lane + offset) & 31);
            if (lane >= offset) incl = mul(incl, up);
            if (lane + offset < 32) sufx = mul(sufx, down);
        }
        Fr left = shfl_fr_idx(incl, (lane - 1) & 31);
        Fr right = shfl_fr_idx(sufx, (lane + 1) & 31);
        if (lane == 0) left = Fr::one();
        if (lane == 31) right = Fr::one();
        if (lane == 31) warp_incl[warp] = incl;
        __syncthreads();
        if (threadIdx.x == 0)
        {
            Fr run = Fr::one();
#pragma unroll
            for (int w = 0; w < W; ++w)
            {
                warp_pre[w] = run;
                run = mul(run, warp_incl[w]);
            }
            run = Fr::one();
#pragma unroll
            for (int w = W - 1; w >= 0; --w)
            {
                warp_suf[w] = run;
                run = mul(run, warp_incl[w]);
            }
        }
        __syncthreads();
        const Fr outer = mul(cta_inverse, mul(mul(left, warp_pre[warp]), mul(right, warp_suf[warp])));
        __syncthreads();
        return outer;
    }

    // Segmented additive scan element: `flag` set means "a segment starts at or
    // after the beginning of this span", value = sum since the last start.
    struct SegVal
    {
        Fr v;
        uint32_t flag;
    };
    __device__ __forceinline__ SegVal seg_combine(const SegVal& left, const SegVal& right)
    {
        SegVal o;
        o.flag = left.flag | right.flag;
        o.v = right.flag ? right.v : add(left.v, right.v);
        return o;
    }

    // Exclusive segmented scan of one SegVal per thread across the CTA; also
    // returns the CTA aggregate.  Uses THREADS/32 shared SegVal slots.
    template <int THREADS>
    __device__ __forceinline__ SegVal block_seg_exclusive_scan(const SegVal& mine, SegVal* slots, SegVal* aggregate)
    {
        constexpr int W = THREADS / 32;
        const int lane = threadIdx.x & 31;
        const int warp = threadIdx.x >> 5;
        SegVal incl = mine;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1)
        {
            SegVal up;
            up.v = shfl_fr_idx(incl.v, (lane - offset) & 31);
            up.flag = __shfl_sync(0xffffffffu, incl.flag, (lane - offset) & 31);
            if (lane >= offset) incl = seg_combine(up, incl);
        }
        SegVal excl;
        excl.v = shfl_fr_idx(incl.v, (lane - 1) & 31);
        excl.flag = __shfl_sync(0xffffffffu, incl.flag, (lane - 1) & 31);
        if (lane == 0)
        {
            excl.v = Fr::zero();
            excl.flag = 0;
        }
        if (lane == 31) slots[warp] = incl;
        __syncthreads();
        SegVal warp_offset;
        warp_offset.v = Fr::zero();
        warp_offset.flag = 0;
        SegVal total;
        total.v = Fr::zero();
        total.flag = 0;
#pragma unroll
        for (int w = 0; w < W; ++w)
        {
            if (w == warp) warp_offset = total;
            total = seg_combine(total, slots[w]);
        }
        __syncthreads();
        *aggregate = total;
        return seg_combine(warp_offset, excl);
    }
#endif
}
