// Column packs of the lookup and routing arguments, lookup multiplicities of the static
// tables, and small buffer utilities the prover flow needs between them.  All HBM-bound:
// one coalesced pass over the inputs, one over the output.
#include <cstring>

#include "block.cuh"

namespace gzk
{
    namespace
    {
        constexpr int kThreads = 256;
        constexpr int kMaxTerms = 8;

        __device__ __forceinline__ uint64_t grid_stride() { return static_cast<uint64_t>(gridDim.x) * blockDim.x; }
        __device__ __forceinline__ uint64_t grid_index() { return static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; }

        struct CombineArgs
        {
            ColRef cols[kMaxTerms];
            Fr k_pos[kMaxTerms];  // coefficient * 2^288 (* R for the kinds stored as plain residues), see combine_kernel
            Fr k_neg[kMaxTerms];  // r - k_pos, for negative small integers
            uint32_t terms;
        };

        // out[i] = sum_j coeff[j] * col_j[i] for i < count, zero tail.  The sum of a row is formed as ONE exact
        // integer, sum_j k_j * v_j with v_j the stored value (one or two limbs for the small-integer kinds,
        // eight for field elements), and reduced once: nine reduction rows divide by 2^288, which the
        // constants k_j = coeff_j * 2^288 (times R when the column holds plain residues) undo, so the result
        // is the Montgomery form of the sum.  A row of two small-integer terms costs 32 + 72 limb products
        // instead of the four full field multiplications (512) of converting and scaling each value.
        // SMALL: every term is a small-integer column, so the sum has at most eleven limbs and three reduction
        // rows are enough (the constants then carry 2^96 instead of 2^288).
        template <bool SMALL>
        __global__ void combine_kernel(CombineArgs a, uint64_t count, uint64_t n, Fr* out)
        {
            for (uint64_t i = grid_index(); i < n; i += grid_stride())
            {
                Fr v = Fr::zero();
                if (i < count)
                {
                    WideAcc acc;
                    acc.clear();
#pragma unroll 1
                    for (uint32_t j = 0; j < a.terms; ++j)
                    {
                        const ColRef& c = a.cols[j];
                        if (c.kind == GZK_KIND_FR || c.kind == GZK_KIND_FR_MONT)
                        {
                            const Fr x = load_fr(static_cast<const Fr*>(c.ptr) + i);
                            acc.mac<8>(a.k_pos[j].l, x.l);
                        }
                        else if (c.kind == GZK_KIND_U32)
                        {
                            const uint32_t x = __ldg(static_cast<const uint32_t*>(c.ptr) + i);
                            acc.mac<1>(a.k_pos[j].l, &x);
                        }
                        else
                        {
                            const long long x = __ldg(static_cast<const long long*>(c.ptr) + i);
                            const unsigned long long mag = x < 0 ? 0ULL - static_cast<unsigned long long>(x) : static_cast<unsigned long long>(x);
                            const uint32_t f[2] = {static_cast<uint32_t>(mag), static_cast<uint32_t>(mag >> 32)};
                            if (x < 0)
                                acc.mac<2>(a.k_neg[j].l, f);
                            else
                                acc.mac<2>(a.k_pos[j].l, f);
                        }
                    }
                    uint32_t sum[17];
                    acc.fold(sum);
                    v = SMALL ? redc_wide<FrCfg, 3>(sum) : redc_wide<FrCfg, 9>(sum);
                }
                store_fr(out + i, v);
            }
        }

        __global__ void product_kernel(ColRef left, ColRef right, uint64_t count, uint64_t n, Fr* out)
        {
            for (uint64_t i = grid_index(); i < n; i += grid_stride())
            {
                Fr v = Fr::zero();
                if (i < count)
                {
                    // stored residues: canonical * canonical is one factor of R short of the canonical
                    // product, two short of the Montgomery one
                    const Fr p = mul(col_load_stored(left, i), col_load_stored(right, i));
                    int d = deficit(left) + deficit(right);
                    v = p;
                    for (; d > 0; --d) v = to_mont(v);
                }
                store_fr(out + i, v);
            }
        }

        __device__ __forceinline__ long long int_at(const ColRef& c, uint64_t i)
        {
            if (c.kind == GZK_KIND_U32) return static_cast<long long>(__ldg(static_cast<const uint32_t*>(c.ptr) + i));
            return __ldg(static_cast<const long long*>(c.ptr) + i);
        }

        // Multiplicities of a lookup into a banded static table.  The table lists, for every
        // x in [x_min, x_min + table_size / band), `band` candidate values table_y[band * (x - x_min) + j];
        // a query (x, y) hits the first j whose candidate equals y (a table without a second
        // column, band = 1 and table_y = null, is hit by x alone).  A query outside the table
        // raises the status word.
        __global__ void banded_multiplicity_kernel(ColRef x, ColRef y, int has_y, uint64_t count, long long x_min, uint32_t band,
                                                   const long long* table_y, uint64_t table_size, uint32_t* out, int* status)
        {
            for (uint64_t i = grid_index(); i < count; i += grid_stride())
            {
                const long long xv = int_at(x, i);
                const long long rel = xv - x_min;
                bool hit = false;
                if (rel >= 0 && static_cast<uint64_t>(rel) * band + band <= table_size)
                {
                    const uint64_t base = static_cast<uint64_t>(rel) * band;
                    if (!has_y)
                    {
                        atomicAdd(out + base, 1u);
                        hit = true;
                    }
                    else
                    {
                        const long long yv = int_at(y, i);
                        for (uint32_t j = 0; j < band; ++j)
                        {
                            if (__ldg(table_y + base + j) == yv)
                            {
                                atomicAdd(out + base + j, 1u);
                                hit = true;
                                break;
                            }
                        }
                    }
                }
                if (!hit) raise_status(status, GZK_E_INVALID, 1301);
            }
        }

        // The same count with one private histogram per CTA in shared memory (tables of up to 56k entries fit).
        // Queries of a real witness pile up on a few table rows (most activations sit near zero), and
        // millions of global atomics on one address serialise; here the lanes of a warp that hit the same
        // row are counted by one of them (match.any), the CTA counts in shared memory, and only the
        // non-zero bins of each CTA reach global memory.
        constexpr int kHistThreads = 1024;
        __global__ void __launch_bounds__(kHistThreads) banded_multiplicity_shared_kernel(ColRef x, ColRef y, int has_y, uint64_t count, long long x_min,
                                                                                          uint32_t band, const long long* table_y, uint32_t table_size,
                                                                                          uint32_t* out, int* status)
        {
            extern __shared__ uint32_t hist[];
            for (uint32_t i = threadIdx.x; i < table_size; i += kHistThreads) hist[i] = 0;
            __syncthreads();
            constexpr uint32_t kNone = 0xffffffffu;
            const uint32_t lane = threadIdx.x & 31;
            const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kHistThreads;
            for (uint64_t base = static_cast<uint64_t>(blockIdx.x) * kHistThreads; base < count; base += stride)
            {
                const uint64_t i = base + threadIdx.x;  // the whole warp stays in the loop: base is uniform
                uint32_t slot = kNone;
                if (i < count)
                {
                    const long long rel = int_at(x, i) - x_min;
                    if (rel >= 0 && static_cast<uint64_t>(rel) * band + band <= table_size)
                    {
                        const uint32_t first = static_cast<uint32_t>(rel) * band;
                        if (!has_y)
                        {
                            slot = first;
                        }
                        else
                        {
                            const long long yv = int_at(y, i);
                            for (uint32_t j = 0; j < band; ++j)
                            {
                                if (__ldg(table_y + first + j) == yv)
                                {
                                    slot = first + j;
                                    break;
                                }
                            }
                        }
                    }
                    if (slot == kNone) raise_status(status, GZK_E_INVALID, 1302);
                }
                const uint32_t peers = __match_any_sync(0xffffffffu, slot);
                if (slot != kNone && lane == static_cast<uint32_t>(__ffs(peers) - 1)) atomicAdd(hist + slot, static_cast<uint32_t>(__popc(peers)));
            }
            __syncthreads();
            for (uint32_t i = threadIdx.x; i < table_size; i += kHistThreads)
            {
                const uint32_t v = hist[i];
                if (v != 0) atomicAdd(out + i, v);
            }
        }

        template <typename T>
        __global__ void copy_block_kernel(const T* src, uint64_t src_stride, T* dst, uint64_t dst_stride, uint64_t rows, uint64_t width)
        {
            const uint64_t total = rows * width;
            for (uint64_t i = grid_index(); i < total; i += grid_stride())
            {
                const uint64_t r = i / width;
                const uint64_t c = i - r * width;
                dst[r * dst_stride + c] = src[r * src_stride + c];
            }
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
        bool field_like(const gzk_buf* b)
        {
            return b != nullptr && (b->kind == GZK_KIND_FR || b->kind == GZK_KIND_FR_MONT || b->kind == GZK_KIND_I64 || b->kind == GZK_KIND_U32);
        }
        bool int_like(const gzk_buf* b) { return b != nullptr && (b->kind == GZK_KIND_I64 || b->kind == GZK_KIND_U32); }
    }
}

using namespace gzk;

extern "C"
{
    int gzk_linear_combination(gzk_ctx* ctx, const gzk_buf* const* cols, const uint8_t* coefficients, size_t terms, size_t count,
                               size_t domain_size, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (domain_size == 0) return GZK_OK;
        if (cols == nullptr || coefficients == nullptr || out == nullptr) return fail(ctx, GZK_E_INVALID, "linear_combination: null argument");
        if (terms == 0 || terms > kMaxTerms) return fail(ctx, GZK_E_INVALID, "linear_combination: between 1 and 8 terms per call");
        if (count > domain_size) return fail(ctx, GZK_E_INVALID, "linear_combination: count exceeds the domain size");
        if (out->kind != GZK_KIND_FR_MONT || out->count < domain_size) return fail(ctx, GZK_E_INVALID, "linear_combination: output must be a Montgomery buffer of the domain size");
        CombineArgs args{};
        args.terms = static_cast<uint32_t>(terms);
        bool all_small = true;
        for (size_t j = 0; j < terms; ++j) all_small = all_small && int_like(cols[j]);
        for (size_t j = 0; j < terms; ++j)
        {
            if (!field_like(cols[j]) || cols[j]->count < count) return fail(ctx, GZK_E_INVALID, "linear_combination: input size mismatch");
            bool canonical = false;
            const Fr c = host_fr_from_bytes(coefficients + 32 * j, &canonical);
            if (!canonical) return fail(ctx, GZK_E_INVALID, "scalar argument is not a canonical field element");
            args.cols[j] = ref(cols[j]);
            // 2^288 (2^96 when no term is a field-element column) in Montgomery form, by doubling
            Fr two288 = Fr::one();
            for (int d = 0; d < (all_small ? 96 : 288); ++d) two288 = add(two288, two288);
            Fr k = mul(to_mont(c), two288);  // c * R * 2^288: for columns of plain residues (FR, I64, U32)
            if (cols[j]->kind == GZK_KIND_FR_MONT) k = from_mont(k);  // the stored value already carries R
            args.k_pos[j] = k;
            args.k_neg[j] = sub(Fr::zero(), k);
        }
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            LaunchScope scope(ctx, "linear_combination");
            if (all_small)
                combine_kernel<true><<<blocks_for(ctx, domain_size), kThreads, 0, ctx->stream>>>(args, count, domain_size, static_cast<Fr*>(out->dptr));
            else
                combine_kernel<false><<<blocks_for(ctx, domain_size), kThreads, 0, ctx->stream>>>(args, count, domain_size, static_cast<Fr*>(out->dptr));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }

    int gzk_mul_columns(gzk_ctx* ctx, const gzk_buf* left, const gzk_buf* right, size_t count, size_t domain_size, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (domain_size == 0) return GZK_OK;
        if (!field_like(left) || !field_like(right) || out == nullptr) return fail(ctx, GZK_E_INVALID, "mul_columns: null argument or unsupported kind");
        if (count > domain_size || left->count < count || right->count < count) return fail(ctx, GZK_E_INVALID, "mul_columns: input size mismatch");
        if (out->kind != GZK_KIND_FR_MONT || out->count < domain_size) return fail(ctx, GZK_E_INVALID, "mul_columns: output must be a Montgomery buffer of the domain size");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            LaunchScope scope(ctx, "mul_columns");
            product_kernel<<<blocks_for(ctx, domain_size), kThreads, 0, ctx->stream>>>(ref(left), ref(right), count, domain_size,
                                                                                       static_cast<Fr*>(out->dptr));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }

    int gzk_banded_lookup_multiplicity(gzk_ctx* ctx, const gzk_buf* x, const gzk_buf* y, size_t count, int64_t x_min, size_t band,
                                       const gzk_buf* table_y, size_t table_size, size_t domain_size, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (out == nullptr || out->kind != GZK_KIND_U32 || out->count < domain_size)
            return fail(ctx, GZK_E_INVALID, "lookup multiplicity: output must be a U32 buffer of the domain size");
        if (band == 0 || band > 64 || table_size > domain_size || table_size % band != 0)
            return fail(ctx, GZK_E_INVALID, "lookup multiplicity: the table must fit the domain and hold a whole number of bands");
        const bool has_y = y != nullptr;
        if (has_y != (table_y != nullptr)) return fail(ctx, GZK_E_INVALID, "lookup multiplicity: a second query column needs the table's second column and vice versa");
        if (count != 0 && (!int_like(x) || x->count < count || (has_y && (!int_like(y) || y->count < count))))
            return fail(ctx, GZK_E_INVALID, "lookup multiplicity: queries must be I64 or U32 buffers of count elements");
        if (has_y && (table_y->kind != GZK_KIND_I64 || table_y->count < table_size))
            return fail(ctx, GZK_E_INVALID, "lookup multiplicity: the table's second column must be an I64 buffer of table_size elements");
        if (!has_y && band != 1) return fail(ctx, GZK_E_INVALID, "lookup multiplicity: a single-column table has band 1");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        int rc = begin_call(ctx);
        if (rc != GZK_OK) return rc;
        GZK_CUDA_TRY(ctx, cudaMemsetAsync(out->dptr, 0, domain_size * sizeof(uint32_t), ctx->stream));
        constexpr size_t kSharedTableLimit = 56 * 1024;  // 224 KB of counters
        if (count >= (1u << 16) && table_size <= kSharedTableLimit)
        {
            static bool opted_in[64] = {};
            if (ctx->device >= 0 && ctx->device < 64 && !opted_in[ctx->device])
            {
                GZK_CUDA_TRY(ctx, cudaFuncSetAttribute(banded_multiplicity_shared_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                       static_cast<int>(kSharedTableLimit * sizeof(uint32_t))));
                opted_in[ctx->device] = true;
            }
            // as many CTAs per SM as their histograms fit in its shared memory (two for the 24 579-row table)
            uint64_t ctas = (count + kHistThreads - 1) / kHistThreads;
            const uint64_t per_sm = table_size * sizeof(uint32_t) <= 100 * 1024 ? 2 : 1;
            if (ctas > static_cast<uint64_t>(ctx->sm_count) * per_sm) ctas = static_cast<uint64_t>(ctx->sm_count) * per_sm;
            LaunchScope scope(ctx, "lookup_multiplicity");
            banded_multiplicity_shared_kernel<<<static_cast<unsigned>(ctas), kHistThreads, table_size * sizeof(uint32_t), ctx->stream>>>(
                ref(x), has_y ? ref(y) : ref(x), has_y ? 1 : 0, count, static_cast<long long>(x_min), static_cast<uint32_t>(band),
                has_y ? static_cast<const long long*>(table_y->dptr) : nullptr, static_cast<uint32_t>(table_size), static_cast<uint32_t*>(out->dptr),
                ctx->d_status);
        }
        else if (count != 0)
        {
            LaunchScope scope(ctx, "lookup_multiplicity");
            banded_multiplicity_kernel<<<blocks_for(ctx, count), kThreads, 0, ctx->stream>>>(
                ref(x), has_y ? ref(y) : ref(x), has_y ? 1 : 0, count, static_cast<long long>(x_min), static_cast<uint32_t>(band),
                has_y ? static_cast<const long long*>(table_y->dptr) : nullptr, table_size, static_cast<uint32_t*>(out->dptr), ctx->d_status);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "lookup query escaped static table");
    }

    int gzk_buf_zero(gzk_ctx* ctx, gzk_buf* buf)
    {
        if (ctx == nullptr || buf == nullptr) return GZK_E_INVALID;
        if (buf->count == 0) return GZK_OK;
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        GZK_CUDA_TRY(ctx, cudaMemsetAsync(buf->dptr, 0, buf->count * buf->elem_bytes, ctx->stream));
        return GZK_OK;
    }

    int gzk_copy_block(gzk_ctx* ctx, const gzk_buf* src, size_t src_offset, size_t src_stride, gzk_buf* dst, size_t dst_offset,
                       size_t dst_stride, size_t rows, size_t width)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (rows == 0 || width == 0) return GZK_OK;
        if (src == nullptr || dst == nullptr) return fail(ctx, GZK_E_INVALID, "copy_block: null argument");
        if (src->kind != dst->kind)
            return fail(ctx, GZK_E_INVALID, "copy_block: source and destination must hold the same kind of element");
        if (src->kind == GZK_KIND_G1) return fail(ctx, GZK_E_INVALID, "copy_block: point buffers are not supported");
        // src_stride 0 repeats one source row (a bias vector under every row of a matrix)
        if ((src_stride != 0 && width > src_stride) || width > dst_stride || src_offset + (rows - 1) * src_stride + width > src->count ||
            dst_offset + (rows - 1) * dst_stride + width > dst->count)
            return fail(ctx, GZK_E_INVALID, "copy_block: block exceeds a buffer");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        const uint64_t total = static_cast<uint64_t>(rows) * width;
        {
            LaunchScope scope(ctx, "copy_block");
            if (src->elem_bytes == 32)
                copy_block_kernel<ulonglong4><<<blocks_for(ctx, total), kThreads, 0, ctx->stream>>>(
                    static_cast<const ulonglong4*>(src->dptr) + src_offset, src_stride, static_cast<ulonglong4*>(dst->dptr) + dst_offset, dst_stride, rows, width);
            else if (src->elem_bytes == 8)
                copy_block_kernel<unsigned long long><<<blocks_for(ctx, total), kThreads, 0, ctx->stream>>>(
                    static_cast<const unsigned long long*>(src->dptr) + src_offset, src_stride, static_cast<unsigned long long*>(dst->dptr) + dst_offset,
                    dst_stride, rows, width);
            else
                copy_block_kernel<uint32_t><<<blocks_for(ctx, total), kThreads, 0, ctx->stream>>>(
                    static_cast<const uint32_t*>(src->dptr) + src_offset, src_stride, static_cast<uint32_t*>(dst->dptr) + dst_offset, dst_stride, rows, width);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }
}
