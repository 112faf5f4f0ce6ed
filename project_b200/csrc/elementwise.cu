// Elementwise / gather / histogram leaves of witness-column construction.  All are
// HBM-bound: one coalesced pass over the inputs, one over the output.
#include <cstring>

#include "block.cuh"

namespace gzk
{
    namespace
    {
        constexpr int kThreads = 256;

        __device__ __forceinline__ uint64_t grid_stride() { return static_cast<uint64_t>(gridDim.x) * blockDim.x; }
        __device__ __forceinline__ uint64_t grid_index() { return static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; }

        // out[i] = left[i] + lambda * right[i] for i < count, zero tail.
        __global__ void weighted_sum_kernel(ColRef left, ColRef right, Fr lambda, uint64_t count, uint64_t n, Fr* out)
        {
            // canonical columns are combined as stored (lambda in Montgomery form times a canonical value
            // is the canonical product) and converted once: two multiplications per row instead of three
            const bool stored = deficit(left) == 1 && deficit(right) == 1;
            for (uint64_t i = grid_index(); i < n; i += grid_stride())
            {
                Fr v = Fr::zero();
                if (i < count)
                    v = stored ? to_mont(add(col_load_stored(left, i), mul(lambda, col_load_stored(right, i))))
                               : add(col_load_mont(left, i), mul(lambda, col_load_mont(right, i)));
                store_fr(out + i, v);
            }
        }

        // out[row*width + c] = row_id[row] + eta_i * feature_index[c] + eta_v * features[row*width + c]
        __global__ void feature_rows_kernel(ColRef row_ids, ColRef feature_indices, ColRef features, uint64_t rows, uint32_t width,
                                            Fr eta_index, Fr eta_value, Fr* out)
        {
            const uint64_t total = rows * width;
            const bool stored = deficit(row_ids) == 1 && deficit(feature_indices) == 1 && deficit(features) == 1;  // all canonical: convert once
            for (uint64_t i = grid_index(); i < total; i += grid_stride())
            {
                const uint64_t row = i / width;
                const uint32_t c = static_cast<uint32_t>(i - row * width);
                Fr v;
                if (stored)
                    v = to_mont(add(add(col_load_stored(row_ids, row), mul(eta_index, col_load_stored(feature_indices, c))),
                                    mul(eta_value, col_load_stored(features, i))));
                else
                    v = add(add(col_load_mont(row_ids, row), mul(eta_index, col_load_mont(feature_indices, c))), mul(eta_value, col_load_mont(features, i)));
                store_fr(out + i, v);
            }
        }

        __device__ __forceinline__ uint64_t index_at(const ColRef& idx, uint64_t i)
        {
            if (idx.kind == GZK_KIND_U32) return __ldg(static_cast<const uint32_t*>(idx.ptr) + i);
            return static_cast<uint64_t>(__ldg(static_cast<const long long*>(idx.ptr) + i));
        }

        // out[e] = node_values[index[e]] for e < edge_count, zero tail; element size 4, 8 or 32 bytes.
        template <typename T>
        __global__ void gather_kernel(const T* node_values, uint64_t node_count, ColRef index, uint64_t edge_count, uint64_t n, T* out,
                                      int* status)
        {
            for (uint64_t e = grid_index(); e < n; e += grid_stride())
            {
                T v{};
                if (e < edge_count)
                {
                    const uint64_t src = index_at(index, e);
                    if (src < node_count)
                        v = node_values[src];
                    else
                        raise_status(status, GZK_E_INVALID, 501);
                }
                out[e] = v;
            }
        }

        __global__ void histogram_kernel(ColRef index, uint64_t count, uint64_t domain_size, uint32_t* out, int* status)
        {
            for (uint64_t i = grid_index(); i < count; i += grid_stride())
            {
                const uint64_t b = index_at(index, i);
                if (b < domain_size)
                    atomicAdd(out + b, 1u);
                else
                    raise_status(status, GZK_E_INVALID, 502);
            }
        }

        // trace.cpp:973-976: (int64)(v >= 0 ? v*16 + 0.5 : v*16 - 0.5), no fused multiply-add
        __global__ void quantize_kernel(const double* values, uint64_t count, long long* out)
        {
            for (uint64_t i = grid_index(); i < count; i += grid_stride())
            {
                const double v = values[i];
                const double scaled = __dmul_rn(v, 16.0);
                const double shifted = v >= 0.0 ? __dadd_rn(scaled, 0.5) : __dadd_rn(scaled, -0.5);
                out[i] = static_cast<long long>(shifted);
            }
        }

        // The same rounding, and a count of the values that sit within `guard` of a rounding boundary
        // (16 |v| within guard of k + 1/2): the values whose quantised form could differ if v carried an
        // error of that size, e.g. from a last-place difference between two exp implementations.
        __global__ void quantize_guarded_kernel(const double* values, uint64_t count, double guard, long long* out, unsigned int* flagged)
        {
            unsigned int mine = 0;
            for (uint64_t i = grid_index(); i < count; i += grid_stride())
            {
                const double v = values[i];
                const double scaled = __dmul_rn(v, 16.0);
                const double shifted = v >= 0.0 ? __dadd_rn(scaled, 0.5) : __dadd_rn(scaled, -0.5);
                out[i] = static_cast<long long>(shifted);
                // distance of |16 v| + 1/2 from the nearest integer = distance of |16 v| from the nearest k + 1/2
                const double a = fabs(shifted);
                const double dist = fabs(a - rint(a));
                if (!(dist >= guard)) ++mine;  // also counts NaN
            }
            if (mine != 0) atomicAdd(flagged, mine);
        }

        // one warp per destination group: mark the first row whose delta is zero.  The lanes test 32 rows at a
        // time (a hub of a power-law graph has tens of thousands of incoming edges; one thread walking them
        // would outlast the rest of the grid).
        __global__ void first_zero_kernel(ColRef delta, ColRef group_begin, ColRef group_end, uint64_t groups, uint64_t n, uint32_t* out,
                                          int* status)
        {
            const uint32_t lane = threadIdx.x & 31;
            const uint64_t warps = grid_stride() >> 5;
            for (uint64_t g = grid_index() >> 5; g < groups; g += warps)
            {
                const uint64_t b = index_at(group_begin, g), e = index_at(group_end, g);
                if (e > n || b > e)
                {
                    if (lane == 0) raise_status(status, GZK_E_INVALID, 503);
                    continue;
                }
                for (uint64_t base = b; base < e; base += 32)
                {
                    const uint64_t k = base + lane;
                    bool zero = false;
                    if (k < e)
                    {
                        if (delta.kind == GZK_KIND_I64)
                            zero = __ldg(static_cast<const long long*>(delta.ptr) + k) == 0;
                        else if (delta.kind == GZK_KIND_U32)
                            zero = __ldg(static_cast<const uint32_t*>(delta.ptr) + k) == 0;
                        else
                            zero = load_fr(static_cast<const Fr*>(delta.ptr) + k).is_zero();
                    }
                    const uint32_t hits = __ballot_sync(0xffffffffu, zero);
                    if (hits != 0)
                    {
                        if (lane == static_cast<uint32_t>(__ffs(hits) - 1)) out[k] = 1;
                        break;
                    }
                }
            }
        }

        // generated public columns: 0 selector (1 below `valid`), 1 index i, 2 i / width, 3 i % width
        __global__ void generated_kernel(int what, uint64_t valid, uint64_t width, uint64_t n, uint32_t* out32, long long* out64)
        {
            for (uint64_t i = grid_index(); i < n; i += grid_stride())
            {
                uint64_t v = 0;
                if (i < valid)
                {
                    if (what == 0) v = 1;
                    else if (what == 1) v = i;
                    else if (what == 2) v = i / width;
                    else v = i % width;
                }
                if (out32 != nullptr) out32[i] = static_cast<uint32_t>(v);
                else out64[i] = static_cast<long long>(v);
            }
        }

        __global__ void add_scalar_kernel(Fr* data, uint64_t count, Fr scalar)
        {
            for (uint64_t i = grid_index(); i < count; i += grid_stride()) store_fr(data + i, add(load_fr_plain(data + i), scalar));
        }

        unsigned blocks_for(gzk_ctx* ctx, uint64_t n)
        {
            uint64_t b = (n + kThreads - 1) / kThreads;
            const uint64_t cap = static_cast<uint64_t>(ctx->sm_count) * 16;
            if (b > cap) b = cap;
            return b == 0 ? 1u : static_cast<unsigned>(b);
        }
        ColRef ref(const gzk_buf* b)
        {
            ColRef r;
            r.ptr = b->dptr;
            r.kind = b->kind;
            return r;
        }
        int scalar_mont(gzk_ctx* ctx, const uint8_t* bytes, Fr* out)
        {
            bool canonical = false;
            const Fr v = host_fr_from_bytes(bytes, &canonical);
            if (!canonical) return fail(ctx, GZK_E_INVALID, "scalar argument is not a canonical field element");
            *out = to_mont(v);
            return GZK_OK;
        }
        int finish_with_status(gzk_ctx* ctx, const char* message) { return finish_call(ctx, message); }
        bool index_kind_ok(const gzk_buf* b) { return b != nullptr && (b->kind == GZK_KIND_U32 || b->kind == GZK_KIND_I64); }
    }
}

using namespace gzk;

extern "C"
{
    int gzk_weighted_sum(gzk_ctx* ctx, const gzk_buf* left, const uint8_t lambda[32], const gzk_buf* right, size_t count,
                         size_t domain_size, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (domain_size == 0) return GZK_OK;
        if (left == nullptr || right == nullptr || lambda == nullptr || out == nullptr) return fail(ctx, GZK_E_INVALID, "weighted_sum: null argument");
        if (count > domain_size || left->count < count || right->count < count) return fail(ctx, GZK_E_INVALID, "weighted_sum: input size mismatch");
        if (out->kind != GZK_KIND_FR_MONT || out->count < domain_size) return fail(ctx, GZK_E_INVALID, "weighted_sum: output must be a Montgomery buffer");
        Fr l;
        int rc = scalar_mont(ctx, lambda, &l);
        if (rc != GZK_OK) return rc;
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            LaunchScope scope(ctx, "weighted_sum");
            weighted_sum_kernel<<<blocks_for(ctx, domain_size), kThreads, 0, ctx->stream>>>(ref(left), ref(right), l, count, domain_size,
                                                                                             static_cast<Fr*>(out->dptr));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }

    int gzk_feature_lookup_rows(gzk_ctx* ctx, const gzk_buf* row_ids, const gzk_buf* feature_indices, const gzk_buf* features,
                                size_t rows, size_t width, const uint8_t eta_index[32], const uint8_t eta_value[32], gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (rows == 0 || width == 0) return GZK_OK;
        if (row_ids == nullptr || feature_indices == nullptr || features == nullptr || out == nullptr || eta_index == nullptr || eta_value == nullptr)
            return fail(ctx, GZK_E_INVALID, "feature_lookup_rows: null argument");
        const uint64_t total = static_cast<uint64_t>(rows) * width;
        if (row_ids->count < rows || feature_indices->count < width || features->count < total || width > 0xffffffffu)
            return fail(ctx, GZK_E_INVALID, "feature_lookup_rows: input size mismatch");
        if (out->kind != GZK_KIND_FR_MONT || out->count < total) return fail(ctx, GZK_E_INVALID, "feature_lookup_rows: output must be a Montgomery buffer");
        Fr ei, ev;
        int rc = scalar_mont(ctx, eta_index, &ei);
        if (rc != GZK_OK) return rc;
        if ((rc = scalar_mont(ctx, eta_value, &ev)) != GZK_OK) return rc;
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            LaunchScope scope(ctx, "feature_rows");
            feature_rows_kernel<<<blocks_for(ctx, total), kThreads, 0, ctx->stream>>>(ref(row_ids), ref(feature_indices), ref(features), rows,
                                                                                       static_cast<uint32_t>(width), ei, ev,
                                                                                       static_cast<Fr*>(out->dptr));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }

    int gzk_broadcast_node_values(gzk_ctx* ctx, const gzk_buf* node_values, size_t node_count, const gzk_buf* index, size_t edge_count,
                                  size_t domain_size, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (domain_size == 0) return GZK_OK;
        if (node_values == nullptr || out == nullptr || !index_kind_ok(index)) return fail(ctx, GZK_E_INVALID, "broadcast: index must be a U32 or I64 buffer");
        if (node_values->count < node_count || index->count < edge_count || edge_count > domain_size)
            return fail(ctx, GZK_E_INVALID, "broadcast: input size mismatch");
        if (out->kind != node_values->kind || out->count < domain_size) return fail(ctx, GZK_E_INVALID, "broadcast: output must have the kind of the node values");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            const int rc_begin = begin_call(ctx);
            if (rc_begin != GZK_OK) return rc_begin;
        }
        {
            LaunchScope scope(ctx, "gather");
            const unsigned blocks = blocks_for(ctx, domain_size);
            if (node_values->elem_bytes == 32)
                gather_kernel<ulonglong4><<<blocks, kThreads, 0, ctx->stream>>>(static_cast<const ulonglong4*>(node_values->dptr), node_count, ref(index),
                                                                                 edge_count, domain_size, static_cast<ulonglong4*>(out->dptr), ctx->d_status);
            else if (node_values->elem_bytes == 8)
                gather_kernel<unsigned long long><<<blocks, kThreads, 0, ctx->stream>>>(static_cast<const unsigned long long*>(node_values->dptr), node_count,
                                                                                         ref(index), edge_count, domain_size,
                                                                                         static_cast<unsigned long long*>(out->dptr), ctx->d_status);
            else
                gather_kernel<uint32_t><<<blocks, kThreads, 0, ctx->stream>>>(static_cast<const uint32_t*>(node_values->dptr), node_count, ref(index),
                                                                               edge_count, domain_size, static_cast<uint32_t*>(out->dptr), ctx->d_status);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_with_status(ctx, "edge endpoint out of range");
    }

    int gzk_histogram(gzk_ctx* ctx, const gzk_buf* indices, size_t count, size_t domain_size, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (out == nullptr || out->kind != GZK_KIND_U32 || out->count < domain_size) return fail(ctx, GZK_E_INVALID, "histogram: output must be a U32 buffer of the domain size");
        if (count != 0 && (!index_kind_ok(indices) || indices->count < count)) return fail(ctx, GZK_E_INVALID, "histogram: indices must be a U32 or I64 buffer");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            const int rc_begin = begin_call(ctx);
            if (rc_begin != GZK_OK) return rc_begin;
        }
        GZK_CUDA_TRY(ctx, cudaMemsetAsync(out->dptr, 0, domain_size * sizeof(uint32_t), ctx->stream));
        if (count != 0)
        {
            LaunchScope scope(ctx, "histogram");
            histogram_kernel<<<blocks_for(ctx, count), kThreads, 0, ctx->stream>>>(ref(indices), count, domain_size, static_cast<uint32_t*>(out->dptr),
                                                                                    ctx->d_status);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_with_status(ctx, "lookup index out of range");
    }

    int gzk_quantize(gzk_ctx* ctx, const gzk_buf* values, size_t count, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (count == 0) return GZK_OK;
        if (values == nullptr || values->kind != GZK_KIND_F64 || values->count < count) return fail(ctx, GZK_E_INVALID, "quantize: input must be an F64 buffer");
        if (out == nullptr || out->kind != GZK_KIND_I64 || out->count < count) return fail(ctx, GZK_E_INVALID, "quantize: output must be an I64 buffer");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            LaunchScope scope(ctx, "quantize");
            quantize_kernel<<<blocks_for(ctx, count), kThreads, 0, ctx->stream>>>(static_cast<const double*>(values->dptr), count,
                                                                                   static_cast<long long*>(out->dptr));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }

    int gzk_quantize_guarded(gzk_ctx* ctx, const gzk_buf* values, size_t count, double guard, gzk_buf* out, gzk_buf* flagged)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (count == 0) return GZK_OK;
        if (values == nullptr || values->kind != GZK_KIND_F64 || values->count < count) return fail(ctx, GZK_E_INVALID, "quantize: input must be an F64 buffer");
        if (out == nullptr || out->kind != GZK_KIND_I64 || out->count < count) return fail(ctx, GZK_E_INVALID, "quantize: output must be an I64 buffer");
        if (flagged == nullptr || flagged->kind != GZK_KIND_U32 || flagged->count < 1) return fail(ctx, GZK_E_INVALID, "quantize_guarded: the counter must be a U32 buffer");
        if (!(guard >= 0.0 && guard <= 0.5)) return fail(ctx, GZK_E_INVALID, "quantize_guarded: the guard band must lie in [0, 0.5]");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            LaunchScope scope(ctx, "quantize");
            quantize_guarded_kernel<<<blocks_for(ctx, count), kThreads, 0, ctx->stream>>>(static_cast<const double*>(values->dptr), count, guard,
                                                                                           static_cast<long long*>(out->dptr),
                                                                                           static_cast<unsigned int*>(flagged->dptr));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }

    int gzk_first_zero_marker(gzk_ctx* ctx, const gzk_buf* delta, const gzk_buf* group_begin, const gzk_buf* group_end, size_t groups,
                              size_t domain_size, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (out == nullptr || out->kind != GZK_KIND_U32 || out->count < domain_size) return fail(ctx, GZK_E_INVALID, "first_zero_marker: output must be a U32 buffer of the domain size");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            const int rc_begin = begin_call(ctx);
            if (rc_begin != GZK_OK) return rc_begin;
        }
        GZK_CUDA_TRY(ctx, cudaMemsetAsync(out->dptr, 0, domain_size * sizeof(uint32_t), ctx->stream));
        if (groups != 0)
        {
            if (delta == nullptr || delta->kind == GZK_KIND_F64 || !index_kind_ok(group_begin) ||
                !index_kind_ok(group_end) || group_begin->count < groups || group_end->count < groups)
                return fail(ctx, GZK_E_INVALID, "first_zero_marker: input size mismatch");
            LaunchScope scope(ctx, "first_zero");
            first_zero_kernel<<<blocks_for(ctx, groups * 32), kThreads, 0, ctx->stream>>>(ref(delta), ref(group_begin), ref(group_end), groups,
                                                                                     delta->count < domain_size ? delta->count : domain_size,
                                                                                     static_cast<uint32_t*>(out->dptr), ctx->d_status);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_with_status(ctx, "first_zero_marker: group bounds out of range");
    }

    int gzk_generated_column(gzk_ctx* ctx, int what, size_t valid, size_t width, size_t domain_size, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (domain_size == 0) return GZK_OK;
        if (what < 0 || what > 3 || (what >= 2 && width == 0)) return fail(ctx, GZK_E_INVALID, "generated_column: unknown generator or zero width");
        if (out == nullptr || (out->kind != GZK_KIND_U32 && out->kind != GZK_KIND_I64) || out->count < domain_size)
            return fail(ctx, GZK_E_INVALID, "generated_column: output must be a U32 or I64 buffer of the domain size");
        if (valid > domain_size) valid = domain_size;
        if (out->kind == GZK_KIND_U32 && what == 1 && valid > (1ull << 32)) return fail(ctx, GZK_E_INVALID, "generated_column: indices exceed 32 bits");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            LaunchScope scope(ctx, "generated_column");
            generated_kernel<<<blocks_for(ctx, domain_size), kThreads, 0, ctx->stream>>>(
                what, valid, width == 0 ? 1 : width, domain_size, out->kind == GZK_KIND_U32 ? static_cast<uint32_t*>(out->dptr) : nullptr,
                out->kind == GZK_KIND_I64 ? static_cast<long long*>(out->dptr) : nullptr);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }

    int gzk_fr_add_scalar(gzk_ctx* ctx, gzk_buf* buf, size_t offset, size_t count, const uint8_t scalar[32])
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (count == 0) return GZK_OK;
        if (buf == nullptr || scalar == nullptr || buf->kind != GZK_KIND_FR_MONT || offset + count > buf->count)
            return fail(ctx, GZK_E_INVALID, "fr_add_scalar: needs a Montgomery buffer and a range inside it");
        Fr v;
        int rc = scalar_mont(ctx, scalar, &v);
        if (rc != GZK_OK) return rc;
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            LaunchScope scope(ctx, "add_scalar");
            add_scalar_kernel<<<blocks_for(ctx, count), kThreads, 0, ctx->stream>>>(static_cast<Fr*>(buf->dptr) + offset, count, v);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }
}
