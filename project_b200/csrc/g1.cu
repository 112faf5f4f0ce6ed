// G1 on the GPU: point buffers, fixed-base batch multiplication [s_k]G (the
// reference's commitment step) and XYZZ -> affine conversion with one batched
// inversion.
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "block.cuh"
#include "g1.cuh"

namespace gzk
{
    namespace
    {
        constexpr int kThreads = 128;
        constexpr int kWindowBits = 8;
        constexpr int kWindows = 32;             // 32 x 8 bits cover a 255-bit scalar
        constexpr int kEntries = 255;            // digits 1..255
        constexpr int kInvThreads = 256;

    }

    namespace
    {
        // canonical <-> Montgomery for arrays of Fp (point buffers hold 2 Fp per point)
        __global__ void convert_fp_kernel(const Fp* in, Fp* out, size_t count, int to_montgomery)
        {
            const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
            for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
            {
                const Fp v = load_fp(in + i);
                store_fp(out + i, to_montgomery ? to_mont(v) : from_mont(v));
            }
        }

        // One thread per window: table[w][d-1] = d * 2^(8w) * base, as XYZZ.
        __global__ void fixed_base_table_kernel(G1Affine base, G1Xyzz* table)
        {
            const int w = blockIdx.x * blockDim.x + threadIdx.x;
            if (w >= kWindows) return;
            G1Xyzz b = G1Xyzz::from_affine(base);
            for (int i = 0; i < w * kWindowBits; ++i) b = g1_double(b);
            G1Xyzz acc = b;
            for (int d = 1; d <= kEntries; ++d)
            {
                store_xyzz(table + w * kEntries + (d - 1), acc);
                acc = g1_add(acc, b);
            }
        }

        // z[i] = ZZ*ZZZ of point i (1 for the point at infinity, so that it can be inverted)
        __global__ void xyzz_denominators_kernel(const G1Xyzz* points, size_t count, Fp* z)
        {
            const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
            if (i >= count) return;
            const G1Xyzz p = load_xyzz(points + i);
            store_fp(z + i, p.is_infinity() ? Fp::one() : mul(p.ZZ, p.ZZZ));
        }

        // In-place batch inversion of `count` non-zero Fp values by one CTA.
        __global__ void __launch_bounds__(kInvThreads) fp_batch_invert_kernel(Fp* values, Fp* prefix_tmp, uint32_t count)
        {
            __shared__ Fp pre[kInvThreads];
            __shared__ Fp suf[kInvThreads];
            __shared__ Fp total_inv;
            const uint32_t t = threadIdx.x;
            const uint32_t run = (count + kInvThreads - 1) / kInvThreads;
            const uint32_t begin = t * run < count ? t * run : count;
            const uint32_t end = begin + run < count ? begin + run : count;
            Fp acc = Fp::one();
            for (uint32_t i = begin; i < end; ++i)
            {
                store_fp(prefix_tmp + i, acc);
                acc = mul(acc, load_fp(values + i));
            }
            pre[t] = acc;
            suf[t] = acc;
            __syncthreads();
            for (uint32_t offset = 1; offset < kInvThreads; offset <<= 1)
            {
                const Fp p = pre[t], s = suf[t];
                const bool has_p = t >= offset, has_s = t + offset < kInvThreads;
                Fp po, so;
                if (has_p) po = pre[t - offset];
                if (has_s) so = suf[t + offset];
                __syncthreads();
                if (has_p) pre[t] = mul(p, po);
                if (has_s) suf[t] = mul(s, so);
                __syncthreads();
            }
            if (t == 0) total_inv = inv(pre[kInvThreads - 1]);
            __syncthreads();
            Fp outer = total_inv;
            if (t > 0) outer = mul(outer, pre[t - 1]);
            if (t + 1 < kInvThreads) outer = mul(outer, suf[t + 1]);
            for (uint32_t i = end; i-- > begin;)
            {
                const Fp v = *(values + i);
                store_fp(values + i, mul(outer, *(prefix_tmp + i)));
                outer = mul(outer, v);
            }
        }

        // out[i] = affine(points[i]) given z_inv[i] = 1/(ZZ*ZZZ); Montgomery or canonical coordinates
        __global__ void xyzz_to_affine_kernel(const G1Xyzz* points, const Fp* z_inv, size_t count, G1Affine* out, int canonical)
        {
            const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
            if (i >= count) return;
            G1Affine a = g1_to_affine_with_inverse(load_xyzz(points + i), load_fp(z_inv + i));
            if (canonical)
            {
                a.x = from_mont(a.x);
                a.y = from_mont(a.y);
            }
            store_affine(out + i, a);
        }

        // One thread per scalar: sum over the 32 byte-windows of table[w][digit-1].
        __global__ void __launch_bounds__(kThreads) fixed_base_mul_kernel(const G1Affine* table, ColRef scalars, size_t count, G1Xyzz* out)
        {
            const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
            if (i >= count) return;
            Fr s = load_fr(static_cast<const Fr*>(scalars.ptr) + i);
            if (scalars.kind == GZK_KIND_FR_MONT) s = from_mont(s);
            G1Xyzz acc = G1Xyzz::infinity();
#pragma unroll 1
            for (int w = 0; w < kWindows; ++w)
            {
                const uint32_t digit = (s.l[w >> 2] >> ((w & 3) * 8)) & 0xffu;
                if (digit != 0) acc = g1_add_mixed(acc, load_affine(table + w * kEntries + (digit - 1)));
            }
            store_xyzz(out + i, acc);
        }

        // The same sum with the 32 windows of a scalar dealt to kLanes adjacent lanes
        // (kWindows / kLanes mixed additions each) and the lane sums combined by a shuffle
        // tree of full additions.  A batch of a few hundred scalars (the columns of one
        // commit barrier) is bound by the length of the dependent chain, not by
        // throughput: 4 mixed + 3 full additions instead of 32 mixed ones.
        constexpr int kLanes = 8;
        __device__ __forceinline__ G1Xyzz shfl_down_xyzz(const G1Xyzz& p, int offset)
        {
            G1Xyzz o;
#pragma unroll
            for (int i = 0; i < FpCfg::N; ++i)
            {
                o.X.l[i] = __shfl_down_sync(0xffffffffu, p.X.l[i], offset, kLanes);
                o.Y.l[i] = __shfl_down_sync(0xffffffffu, p.Y.l[i], offset, kLanes);
                o.ZZ.l[i] = __shfl_down_sync(0xffffffffu, p.ZZ.l[i], offset, kLanes);
                o.ZZZ.l[i] = __shfl_down_sync(0xffffffffu, p.ZZZ.l[i], offset, kLanes);
            }
            return o;
        }
        __global__ void __launch_bounds__(kThreads) fixed_base_mul_lanes_kernel(const G1Affine* table, ColRef scalars, size_t count, G1Xyzz* out)
        {
            const size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
            const size_t i = t / kLanes;
            const int part = static_cast<int>(t % kLanes);
            const size_t i_load = i < count ? i : count - 1;  // idle lanes keep the warp's shuffles whole
            Fr s = load_fr(static_cast<const Fr*>(scalars.ptr) + i_load);
            if (scalars.kind == GZK_KIND_FR_MONT) s = from_mont(s);
            G1Xyzz acc = G1Xyzz::infinity();
#pragma unroll 1
            for (int w = part * (kWindows / kLanes); w < (part + 1) * (kWindows / kLanes); ++w)
            {
                const uint32_t digit = (s.l[w >> 2] >> ((w & 3) * 8)) & 0xffu;
                if (digit != 0) acc = g1_add_mixed(acc, load_affine(table + w * kEntries + (digit - 1)));
            }
#pragma unroll 1
            for (int offset = kLanes / 2; offset > 0; offset >>= 1)
            {
                const G1Xyzz other = shfl_down_xyzz(acc, offset);
                if (part < offset) acc = g1_add(acc, other);
            }
            if (part == 0 && i < count) store_xyzz(out + i, acc);
        }

        // The lane-split sum followed, in the same launch, by the conversion to affine coordinates: each
        // point's own denominator is inverted by the lane that holds the sum.  A shared (batch) inversion
        // saves arithmetic but puts a prefix pass, one serial inversion and a suffix pass on the chain,
        // and three launches; for the few dozen points of one commit barrier every point inverting for
        // itself, all at once, is the shorter chain.
        constexpr size_t kFusedAffineLimit = 1024;
        __global__ void __launch_bounds__(128) fixed_base_mul_affine_kernel(const G1Affine* table, ColRef scalars, size_t count, G1Affine* out, int canonical)
        {
            const size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
            const size_t i = t / kLanes;
            const int part = static_cast<int>(t % kLanes);
            const size_t i_load = i < count ? i : count - 1;
            Fr s = load_fr(static_cast<const Fr*>(scalars.ptr) + i_load);
            if (scalars.kind == GZK_KIND_FR_MONT) s = from_mont(s);
            G1Xyzz acc = G1Xyzz::infinity();
#pragma unroll 1
            for (int w = part * (kWindows / kLanes); w < (part + 1) * (kWindows / kLanes); ++w)
            {
                const uint32_t digit = (s.l[w >> 2] >> ((w & 3) * 8)) & 0xffu;
                if (digit != 0) acc = g1_add_mixed(acc, load_affine(table + w * kEntries + (digit - 1)));
            }
#pragma unroll 1
            for (int offset = kLanes / 2; offset > 0; offset >>= 1)
            {
                const G1Xyzz other = shfl_down_xyzz(acc, offset);
                if (part < offset) acc = g1_add(acc, other);
            }
            if (part != 0 || i >= count) return;
            G1Affine a = g1_to_affine(acc);
            if (canonical)
            {
                a.x = from_mont(a.x);
                a.y = from_mont(a.y);
            }
            store_affine(out + i, a);
        }

        // Sum over the 32 byte-windows of every scalar: lane-split for chain-bound batch sizes.
        void launch_fixed_base_mul(gzk_ctx* ctx, const G1Affine* table, const ColRef& s, size_t count, G1Xyzz* xyzz)
        {
            static_assert(kWindows % kLanes == 0 && 32 % kLanes == 0, "lanes must divide the windows and the warp");
            if (count < 16384)
            {
                const size_t threads = count * kLanes;
                fixed_base_mul_lanes_kernel<<<static_cast<unsigned>((threads + kThreads - 1) / kThreads), kThreads, 0, ctx->stream>>>(table, s, count, xyzz);
            }
            else
            {
                fixed_base_mul_kernel<<<static_cast<unsigned>((count + kThreads - 1) / kThreads), kThreads, 0, ctx->stream>>>(table, s, count, xyzz);
            }
        }
    }

    // Converts `count` XYZZ points to affine (Montgomery coordinates in `out_mont`, or
    // canonical wire-format coordinates when `canonical`); `z_tmp` needs 2*count Fp.
    int launch_xyzz_to_affine(gzk_ctx* ctx, const G1Xyzz* points, size_t count, Fp* z_tmp, G1Affine* out, bool canonical)
    {
        if (count == 0) return GZK_OK;
        const unsigned blocks = static_cast<unsigned>((count + kThreads - 1) / kThreads);
        {
            LaunchScope scope(ctx, "g1_denominators");
            xyzz_denominators_kernel<<<blocks, kThreads, 0, ctx->stream>>>(points, count, z_tmp);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        {
            LaunchScope scope(ctx, "g1_batch_invert");
            fp_batch_invert_kernel<<<1, kInvThreads, 0, ctx->stream>>>(z_tmp, z_tmp + count, static_cast<uint32_t>(count));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        {
            LaunchScope scope(ctx, "g1_to_affine");
            xyzz_to_affine_kernel<<<blocks, kThreads, 0, ctx->stream>>>(points, z_tmp, count, out, canonical ? 1 : 0);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return GZK_OK;
    }

    int launch_convert_fp(gzk_ctx* ctx, const void* in, void* out, size_t fp_count, bool to_montgomery)
    {
        if (fp_count == 0) return GZK_OK;
        const unsigned blocks = static_cast<unsigned>((fp_count + 255) / 256 < 4096 ? (fp_count + 255) / 256 : 4096);
        LaunchScope scope(ctx, "convert_fp");
        convert_fp_kernel<<<blocks, 256, 0, ctx->stream>>>(static_cast<const Fp*>(in), static_cast<Fp*>(out), fp_count, to_montgomery ? 1 : 0);
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return GZK_OK;
    }

    namespace
    {
        struct BaseTable
        {
            G1Affine* table = nullptr;  // [kWindows][kEntries], Montgomery affine
        };
        // One table per (context, base).  Contexts live on different host threads, so the
        // container is guarded; an entry itself is only ever touched by the thread of its context.
        std::mutex& table_cache_mutex()
        {
            static std::mutex m;
            return m;
        }
        std::map<std::pair<gzk_ctx*, std::string>, BaseTable>& table_cache()
        {
            static std::map<std::pair<gzk_ctx*, std::string>, BaseTable> cache;
            return cache;
        }

        bool fp_canonical(const uint8_t* bytes)
        {
            uint32_t limbs[12];
            std::memcpy(limbs, bytes, 48);
            for (int i = 11; i >= 0; --i)
                if (limbs[i] != FpCfg::mod(i)) return limbs[i] < FpCfg::mod(i);
            return false;
        }

        int get_base_table(gzk_ctx* ctx, const uint8_t base[96], const G1Affine** out)
        {
            const std::string key(reinterpret_cast<const char*>(base), 96);
            auto& cache = table_cache();
            {
                std::lock_guard<std::mutex> lock(table_cache_mutex());
                const auto it = cache.find({ctx, key});
                if (it != cache.end())
                {
                    *out = it->second.table;
                    return GZK_OK;
                }
            }
            if (!fp_canonical(base) || !fp_canonical(base + 48)) return fail(ctx, GZK_E_INVALID, "g1: base coordinates are not canonical");
            G1Affine b;
            std::memcpy(b.x.l, base, 48);
            std::memcpy(b.y.l, base + 48, 48);
            bool is_inf = true;
            for (int i = 0; i < 96; ++i) is_inf = is_inf && base[i] == 0;
            if (is_inf) return fail(ctx, GZK_E_INVALID, "g1: the base is the point at infinity");
            b.x = to_mont(b.x);
            b.y = to_mont(b.y);
            // on-curve check y^2 = x^3 + 4 on the host
            Fp four = Fp::zero();
            four.l[0] = 4;
            if (sqr(b.y) != add(mul(sqr(b.x), b.x), to_mont(four))) return fail(ctx, GZK_E_INVALID, "g1: the base is not on the curve");
            const size_t entries = static_cast<size_t>(kWindows) * kEntries;
            G1Xyzz* xyzz = nullptr;
            Fp* z = nullptr;
            BaseTable t;
            GZK_CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void**>(&xyzz), entries * sizeof(G1Xyzz)));
            GZK_CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void**>(&z), 2 * entries * sizeof(Fp)));
            GZK_CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void**>(&t.table), entries * sizeof(G1Affine)));
            {
                LaunchScope scope(ctx, "g1_base_table");
                fixed_base_table_kernel<<<1, kWindows, 0, ctx->stream>>>(b, xyzz);
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            int rc = launch_xyzz_to_affine(ctx, xyzz, entries, z, t.table, false);
            if (rc != GZK_OK) return rc;
            GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            GZK_CUDA_TRY(ctx, cudaFree(xyzz));
            GZK_CUDA_TRY(ctx, cudaFree(z));
            {
                std::lock_guard<std::mutex> lock(table_cache_mutex());
                cache[{ctx, key}] = t;
            }
            *out = t.table;
            return GZK_OK;
        }
    }

    void g1_release_tables(gzk_ctx* ctx)
    {
        std::lock_guard<std::mutex> lock(table_cache_mutex());
        auto& cache = table_cache();
        for (auto it = cache.begin(); it != cache.end();)
        {
            if (it->first.first == ctx)
            {
                cudaFree(it->second.table);
                it = cache.erase(it);
            }
            else
            {
                ++it;
            }
        }
    }
}

using namespace gzk;

extern "C"
{
    int gzk_g1_fixed_base_mul(gzk_ctx* ctx, const uint8_t base[96], const gzk_buf* scalars, size_t count, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (count == 0) return GZK_OK;
        if (base == nullptr || scalars == nullptr || out == nullptr) return fail(ctx, GZK_E_INVALID, "g1_fixed_base_mul: null argument");
        if ((scalars->kind != GZK_KIND_FR && scalars->kind != GZK_KIND_FR_MONT) || scalars->count < count)
            return fail(ctx, GZK_E_INVALID, "g1_fixed_base_mul: scalars must be an FR or FR_MONT buffer");
        if (out->kind != GZK_KIND_G1 || out->count < count) return fail(ctx, GZK_E_INVALID, "g1_fixed_base_mul: output must be a G1 buffer");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        const G1Affine* table = nullptr;
        int rc = get_base_table(ctx, base, &table);
        if (rc != GZK_OK) return rc;
        void* scratch = nullptr;
        if ((rc = ensure_scratch(ctx, 1, count * (sizeof(G1Xyzz) + 2 * sizeof(Fp)), &scratch)) != GZK_OK) return rc;
        G1Xyzz* xyzz = static_cast<G1Xyzz*>(scratch);
        Fp* z = reinterpret_cast<Fp*>(xyzz + count);
        ColRef s;
        s.ptr = scalars->dptr;
        s.kind = scalars->kind;
        if (count <= kFusedAffineLimit)
        {
            LaunchScope scope(ctx, "g1_fixed_base_mul_affine");
            fixed_base_mul_affine_kernel<<<static_cast<unsigned>((count * kLanes + 127) / 128), 128, 0, ctx->stream>>>(table, s, count, static_cast<G1Affine*>(out->dptr), 0);
            GZK_CUDA_TRY(ctx, cudaGetLastError());
        }
        else
        {
            {
                LaunchScope scope(ctx, "g1_fixed_base_mul");
                launch_fixed_base_mul(ctx, table, s, count, xyzz);
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            if ((rc = launch_xyzz_to_affine(ctx, xyzz, count, z, static_cast<G1Affine*>(out->dptr), false)) != GZK_OK) return rc;
        }
        GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        return GZK_OK;
    }

    int gzk_g1_mul_same_base(gzk_ctx* ctx, const uint8_t base[96], const uint8_t* scalars_host, size_t count, uint8_t* points_out_host)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (count == 0) return GZK_OK;
        if (base == nullptr || scalars_host == nullptr || points_out_host == nullptr) return fail(ctx, GZK_E_INVALID, "g1_mul_same_base: null argument");
        for (size_t i = 0; i < count; ++i)
        {
            bool canonical = false;
            host_fr_from_bytes(scalars_host + 32 * i, &canonical);
            if (!canonical) return fail(ctx, GZK_E_INVALID, "g1_mul_same_base: scalar is not a canonical field element");
        }
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        const G1Affine* table = nullptr;
        int rc = get_base_table(ctx, base, &table);
        if (rc != GZK_OK) return rc;
        void* scratch = nullptr;
        const size_t bytes = count * (sizeof(Fr) + sizeof(G1Xyzz) + 2 * sizeof(Fp) + sizeof(G1Affine)) + 256;
        if ((rc = ensure_scratch(ctx, 1, bytes, &scratch)) != GZK_OK) return rc;
        G1Xyzz* xyzz = static_cast<G1Xyzz*>(scratch);
        Fp* z = reinterpret_cast<Fp*>(xyzz + count);
        G1Affine* affine = reinterpret_cast<G1Affine*>(z + 2 * count);
        Fr* d_scalars = reinterpret_cast<Fr*>(affine + count);
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(d_scalars, scalars_host, count * 32, cudaMemcpyHostToDevice, ctx->stream));
        ColRef s;
        s.ptr = d_scalars;
        s.kind = GZK_KIND_FR;
        if (count <= kFusedAffineLimit)
        {
            LaunchScope scope(ctx, "g1_fixed_base_mul_affine");
            fixed_base_mul_affine_kernel<<<static_cast<unsigned>((count * kLanes + 127) / 128), 128, 0, ctx->stream>>>(table, s, count, affine, 1);
            GZK_CUDA_TRY(ctx, cudaGetLastError());
        }
        else
        {
            {
                LaunchScope scope(ctx, "g1_fixed_base_mul");
                launch_fixed_base_mul(ctx, table, s, count, xyzz);
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            if ((rc = launch_xyzz_to_affine(ctx, xyzz, count, z, affine, true)) != GZK_OK) return rc;
        }
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(points_out_host, affine, count * 96, cudaMemcpyDeviceToHost, ctx->stream));
        GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        return GZK_OK;
    }

    // Host-side sum of a few affine points (wire format): combines the per-GPU results of
    // a point-range-sharded MSM.  Runs on the CPU; `count` is the number of GPUs.
    int gzk_g1_sum(const uint8_t* points, size_t count, uint8_t out[96])
    {
        if (points == nullptr || out == nullptr) return GZK_E_INVALID;
        G1Xyzz acc = G1Xyzz::infinity();
        for (size_t i = 0; i < count; ++i)
        {
            const uint8_t* p = points + 96 * i;
            bool is_inf = true;
            for (int b = 0; b < 96; ++b) is_inf = is_inf && p[b] == 0;
            if (is_inf) continue;
            if (!fp_canonical(p) || !fp_canonical(p + 48)) return GZK_E_INVALID;
            G1Affine a;
            std::memcpy(a.x.l, p, 48);
            std::memcpy(a.y.l, p + 48, 48);
            a.x = to_mont(a.x);
            a.y = to_mont(a.y);
            acc = g1_add_mixed(acc, a);
        }
        G1Affine r = g1_to_affine(acc);
        r.x = from_mont(r.x);
        r.y = from_mont(r.y);
        std::memcpy(out, r.x.l, 48);
        std::memcpy(out + 48, r.y.l, 48);
        return GZK_OK;
    }
}
