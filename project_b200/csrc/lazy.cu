// Public feature-domain columns that are never materialised: the reference streams
// the feature matrix against the weight vector and evaluates the generated columns
// 1, row id, column id, absolute node id and feature value on the fly.  Each sum is
// one pass over the weights with an unreduced accumulator; the generated values
// are small integers, so a term costs 8 limb products instead of 64.
#include <cstring>

#include "block.cuh"

namespace gzk
{
    int launch_eval_finish(gzk_ctx* ctx, const uint32_t* partial, int uniform_kind, uint32_t tiles, uint32_t k_count,
                           Fr* out, bool out_montgomery);

    namespace
    {
        constexpr int kThreads = 256;
        constexpr int kAccLimbs = 17;

        enum Generator
        {
            kOnes = 0,
            kRowId = 1,
            kColId = 2,
            kAbsId = 3,
            kFeature = 4,
        };

        struct LazyArgs
        {
            const Fr* weights;
            uint64_t valid;       // rows * feature_count entries carry a value
            uint32_t feature_count;
            ColRef features;      // kFeature
            ColRef abs_ids;       // kAbsId (U32 or I64, one per row)
            uint32_t* partial;    // [warp][17]
            uint64_t rotation;    // entry i meets weights[(i - rotation) & mask]
            uint64_t mask;        // domain size - 1 when rotated, all ones otherwise
        };

        template <int GEN>
        __global__ void __launch_bounds__(kThreads) lazy_dot_kernel(LazyArgs a)
        {
            const uint32_t lane = threadIdx.x & 31;
            const uint64_t warp = (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
            const uint64_t warps = (static_cast<uint64_t>(gridDim.x) * kThreads) >> 5;
            const uint64_t per_warp = ((a.valid + warps - 1) / warps + 31) & ~31ULL;
            const uint64_t begin = warp * per_warp < a.valid ? warp * per_warp : a.valid;
            const uint64_t end = begin + per_warp < a.valid ? begin + per_warp : a.valid;
            WideAcc acc;
            acc.clear();
            for (uint64_t i = begin + lane; i < end; i += 32)
            {
                Fr w = load_fr(a.weights + ((i - a.rotation) & a.mask));
                if (GEN == kOnes)
                {
                    const uint32_t one = 1;
                    acc.mac<1>(w.l, &one);
                }
                else if (GEN == kRowId || GEN == kColId)
                {
                    const uint64_t row = i / a.feature_count;
                    const uint64_t v = GEN == kRowId ? row : i - row * a.feature_count;
                    const uint32_t f[2] = {static_cast<uint32_t>(v), static_cast<uint32_t>(v >> 32)};
                    acc.mac<2>(w.l, f);
                }
                else if (GEN == kAbsId)
                {
                    const uint64_t row = i / a.feature_count;
                    const uint64_t v = a.abs_ids.kind == GZK_KIND_U32 ? __ldg(static_cast<const uint32_t*>(a.abs_ids.ptr) + row)
                                                                     : static_cast<uint64_t>(__ldg(static_cast<const long long*>(a.abs_ids.ptr) + row));
                    const uint32_t f[2] = {static_cast<uint32_t>(v), static_cast<uint32_t>(v >> 32)};
                    acc.mac<2>(w.l, f);
                }
                else if (a.features.kind == GZK_KIND_FR || a.features.kind == GZK_KIND_FR_MONT)
                {
                    const Fr f = load_fr(static_cast<const Fr*>(a.features.ptr) + i);
                    acc.mac<8>(w.l, f.l);
                }
                else if (a.features.kind == GZK_KIND_U32)
                {
                    const uint32_t f = __ldg(static_cast<const uint32_t*>(a.features.ptr) + i);
                    acc.mac<1>(w.l, &f);
                }
                else
                {
                    const long long v = __ldg(static_cast<const long long*>(a.features.ptr) + i);
                    const unsigned long long mag = v < 0 ? 0ULL - static_cast<unsigned long long>(v) : static_cast<unsigned long long>(v);
                    const uint32_t f[2] = {static_cast<uint32_t>(mag), static_cast<uint32_t>(mag >> 32)};
                    if (v < 0) w = sub(Fr::zero(), w);
                    acc.mac<2>(w.l, f);
                }
            }
            uint32_t sum[kAccLimbs];
            acc.fold(sum);
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1)
            {
                uint32_t other[kAccLimbs];
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) other[i] = __shfl_down_sync(0xffffffffu, sum[i], offset);
                acc_add<kAccLimbs, kAccLimbs>(sum, other);
            }
            if (lane == 0)
            {
                uint32_t* dst = a.partial + warp * kAccLimbs;
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) dst[i] = sum[i];
            }
        }
    }
}

using namespace gzk;

// out[0..4] = sum_{i < rows*feature_count} w[i] * {1, i / fc, i % fc, abs_ids[i / fc], features[i]}
static int fh_public_eval_impl(gzk_ctx* ctx, const gzk_buf* features, size_t rows, size_t feature_count, const gzk_buf* abs_ids,
                               const gzk_buf* weights, uint64_t rotation, uint64_t mask, uint8_t out[5 * 32]);

extern "C" int gzk_fh_public_eval(gzk_ctx* ctx, const gzk_buf* features, size_t rows, size_t feature_count, const gzk_buf* abs_ids,
                                  const gzk_buf* weights, uint8_t out[5 * 32])
{
    return fh_public_eval_impl(ctx, features, rows, feature_count, abs_ids, weights, 0, ~0ULL, out);
}

// The same sums at the rotated point omega^rotation * z from the weights at z: the weight of entry i at
// the rotated point is weights[(i - rotation) mod n] (w_i(omega z) = w_{i-1}(z)), so no second weight
// vector is needed for the {z, omega z} pairs of the prover.
extern "C" int gzk_fh_public_eval_rotated(gzk_ctx* ctx, const gzk_buf* features, size_t rows, size_t feature_count, const gzk_buf* abs_ids,
                                          const gzk_buf* weights, unsigned log2n, uint64_t rotation, uint8_t out[5 * 32])
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (log2n > 32 || weights == nullptr || weights->count < (1ULL << log2n) || rotation >= (1ULL << log2n))
        return fail(ctx, GZK_E_INVALID, "fh_public_eval_rotated: needs the weights of the whole domain and a rotation inside it");
    return fh_public_eval_impl(ctx, features, rows, feature_count, abs_ids, weights, rotation, (1ULL << log2n) - 1, out);
}

static int fh_public_eval_impl(gzk_ctx* ctx, const gzk_buf* features, size_t rows, size_t feature_count, const gzk_buf* abs_ids,
                               const gzk_buf* weights, uint64_t rotation, uint64_t mask, uint8_t out[5 * 32])
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (out == nullptr) return fail(ctx, GZK_E_INVALID, "fh_public_eval: null output");
    std::memset(out, 0, 5 * 32);
    const uint64_t valid = static_cast<uint64_t>(rows) * feature_count;
    if (valid == 0) return GZK_OK;
    if (weights == nullptr || weights->kind != GZK_KIND_FR_MONT || weights->count < valid)
        return fail(ctx, GZK_E_INVALID, "fh_public_eval: weights must be a Montgomery buffer covering rows*feature_count");
    if (feature_count > 0xffffffffull) return fail(ctx, GZK_E_INVALID, "fh_public_eval: feature_count too large");
    if (features != nullptr && (features->count < valid || features->kind == GZK_KIND_F64 || features->kind == GZK_KIND_G1))
        return fail(ctx, GZK_E_INVALID, "fh_public_eval: feature buffer too small or of the wrong kind");
    if (abs_ids != nullptr && ((abs_ids->kind != GZK_KIND_U32 && abs_ids->kind != GZK_KIND_I64) || abs_ids->count < rows))
        return fail(ctx, GZK_E_INVALID, "fh_public_eval: abs_ids must be a U32 or I64 buffer of `rows` elements");
    GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const unsigned blocks = static_cast<unsigned>(ctx->sm_count) * 2;
    const uint32_t warps = blocks * (kThreads / 32);
    void* scratch = nullptr;
    int rc = ensure_scratch(ctx, 1, static_cast<size_t>(warps) * kAccLimbs * sizeof(uint32_t) + 5 * sizeof(Fr) + 64, &scratch);
    if (rc != GZK_OK) return rc;
    LazyArgs args{};
    args.weights = static_cast<const Fr*>(weights->dptr);
    args.rotation = rotation;
    args.mask = mask;
    args.valid = valid;
    args.feature_count = static_cast<uint32_t>(feature_count);
    if (features != nullptr)
    {
        args.features.ptr = features->dptr;
        args.features.kind = features->kind;
    }
    if (abs_ids != nullptr)
    {
        args.abs_ids.ptr = abs_ids->dptr;
        args.abs_ids.kind = abs_ids->kind;
    }
    args.partial = static_cast<uint32_t*>(scratch);
    Fr* d_out = reinterpret_cast<Fr*>(static_cast<char*>(scratch) + ((static_cast<size_t>(warps) * kAccLimbs * sizeof(uint32_t) + 31) & ~static_cast<size_t>(31)));
    for (int gen = 0; gen < 5; ++gen)
    {
        if (gen == kAbsId && abs_ids == nullptr) continue;
        if (gen == kFeature && features == nullptr) continue;
        {
            LaunchScope scope(ctx, "lazy_dot");
            switch (gen)
            {
            case kOnes: lazy_dot_kernel<kOnes><<<blocks, kThreads, 0, ctx->stream>>>(args); break;
            case kRowId: lazy_dot_kernel<kRowId><<<blocks, kThreads, 0, ctx->stream>>>(args); break;
            case kColId: lazy_dot_kernel<kColId><<<blocks, kThreads, 0, ctx->stream>>>(args); break;
            case kAbsId: lazy_dot_kernel<kAbsId><<<blocks, kThreads, 0, ctx->stream>>>(args); break;
            default: lazy_dot_kernel<kFeature><<<blocks, kThreads, 0, ctx->stream>>>(args); break;
            }
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        // generated values and canonical / small-integer features are plain integers; Montgomery
        // features carry the extra factor the finish kernel divides out
        const int form = (gen == kFeature && features->kind == GZK_KIND_FR_MONT) ? GZK_KIND_FR_MONT : GZK_KIND_FR;
        if ((rc = launch_eval_finish(ctx, args.partial, form, warps, 1, d_out + gen, false)) != GZK_OK) return rc;
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(out + 32 * gen, d_out + gen, 32, cudaMemcpyDeviceToHost, ctx->stream));
    }
    GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return GZK_OK;
}
