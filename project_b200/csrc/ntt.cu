// Stand-alone Fr NTT / inverse NTT / coset variants and the multilinear fold
// (kernel sweep; the reference has no transform on its proving path).
//
// Natural order in, natural order out.  The log2(n) radix-2 stages are grouped into
// passes (10 stages in the first, up to 8 in the others); each pass loads a
// 1024-element tile into shared memory (limb-planar, conflict-free), runs its stages
// there and writes the tile back, so a 2^24-point transform touches HBM in 3 passes
// instead of 24.  Pass 0 gathers its tile through the bit-reversal permutation; later
// passes take tiles of 2^S strided rows by 2^(10-S) contiguous elements (S <= 8, at
// least one 128-byte line per row).
//
// Twiddles.  The stage-s butterfly of element pair (.., j) needs omega_(2^(s+1))^j with
// j the low s bits of the index.  Inside a pass that starts at stage s0, j splits into the
// bits below s0 ("low", constant through the pass) and the bits of the tile row that the
// pass has already combined, m: omega_(2^(s+1))^j = omega_(2^(t+1))^m * omega_(2^(s+1))^low
// with t = s - s0.  Multiplying element (row, low) ONCE, on load, by
// omega_(2^(s0+S))^(low * bitrev_S(row)) removes the second factor from every stage of the
// pass (the factor a row still carries after stage t is exactly what the remaining stages
// expect), so the stages use only the first factor: a 1024th root of unity from a
// 512-entry table, one multiplication per butterfly and none where m = 0.  The load-time
// factors come from a table per (s0, S) built once per context ([bitrev row][low], so a
// warp reads it in the same runs as the data); above 2^25 entries they are generated
// from the two-level omega tables instead (one more multiplication per element).
#include <cstring>

#include "block.cuh"

namespace gzk
{
    namespace
    {
        constexpr int kThreads = 256;
        constexpr int kTileBits = 10;
        constexpr int kTile = 1 << kTileBits;

        struct NttArgs
        {
            ColRef in;          // pass 0 only
            Fr* data;           // output / in-place working vector (Montgomery)
            const Fr* small;    // omega_1024^m (or the inverse powers), m < 512: in-pass twiddles
            const Fr* twist;    // pass > 0: load-time factors [bitrev row][low]; NULL = generate them
            const Fr* lo;       // omega^j or omega^-j (generated load-time factors)
            const Fr* hi;
            unsigned lo_bits;
            unsigned log2n;
            unsigned s0;        // first stage of this pass
            unsigned stages;    // stages in this pass
            unsigned low_bits;  // contiguous low bits in the tile (L)
            int last;           // last pass: apply the output scaling
            int scale_mode;     // 0 none, 1 multiply by `scale` (1/n), 2 also by shift^-i
            Fr scale;
            const Fr* shift_lo; // powers of the coset shift (forward: applied on load; inverse: on store)
            const Fr* shift_hi;
            unsigned shift_lo_bits;
            int pre_shift;      // pass 0: multiply input i by shift^i
        };

        __device__ __forceinline__ void smem_store(uint32_t* tile, uint32_t e, const Fr& v)
        {
#pragma unroll
            for (int i = 0; i < 8; ++i) tile[i * kTile + e] = v.l[i];
        }
        __device__ __forceinline__ Fr smem_load(const uint32_t* tile, uint32_t e)
        {
            Fr v;
#pragma unroll
            for (int i = 0; i < 8; ++i) v.l[i] = tile[i * kTile + e];
            return v;
        }
        __device__ __forceinline__ uint64_t bit_reverse(uint64_t x, unsigned bits)
        {
            return bits == 0 ? 0 : (__brevll(x) >> (64 - bits));
        }

        // global index of tile element e: [high | mid (stages bits) | lowbase | l (low_bits)]
        __device__ __forceinline__ uint64_t tile_index(const NttArgs& a, uint64_t tile_id, uint32_t e)
        {
            const uint32_t l = e & ((1u << a.low_bits) - 1u);
            const uint32_t mid = e >> a.low_bits;
            const uint64_t lows_per_group = 1ULL << (a.s0 - a.low_bits);  // lowbase values
            const uint64_t lowbase = tile_id % lows_per_group;
            const uint64_t high = tile_id / lows_per_group;
            return (high << (a.s0 + a.stages)) | (static_cast<uint64_t>(mid) << a.s0) | (lowbase << a.low_bits) | l;
        }

        __global__ void __launch_bounds__(kThreads) ntt_pass_kernel(NttArgs a)
        {
            extern __shared__ uint32_t tile[];  // [8][kTile]
            const uint64_t n = 1ULL << a.log2n;
            const uint32_t tile_elems = 1u << (a.stages + a.low_bits);
            const uint64_t vec_offset = static_cast<uint64_t>(blockIdx.y) * n;
            // Pass 0 gathers through the bit-reversal permutation: element e of tile T comes from
            // rev10(e) * n/1024 + rev(T), one 32-byte element per 128-byte line.  The four tiles T, T + Q,
            // T + 2Q, T + 3Q (Q = tiles / 4) read the four elements of the SAME lines, so they are given
            // to four consecutive CTAs: they run side by side and three of the four line reads hit L2
            // instead of DRAM.
            uint64_t tile_id = blockIdx.x;
            if (a.s0 == 0 && gridDim.x >= 4) tile_id = static_cast<uint64_t>(blockIdx.x & 3u) * (gridDim.x >> 2) + (blockIdx.x >> 2);

            for (uint32_t e = threadIdx.x; e < tile_elems; e += kThreads)
            {
                const uint64_t gi = tile_index(a, tile_id, e);
                Fr v;
                if (a.s0 == 0)
                {
                    const uint64_t src = bit_reverse(gi, a.log2n);
                    ColRef in = a.in;
                    v = col_load_mont(in, vec_offset + src);
                    if (a.pre_shift) v = mul(v, domain_point(a.shift_lo, a.shift_hi, a.shift_lo_bits, src));
                }
                else
                {
                    v = load_fr_plain(a.data + vec_offset + gi);
                    const uint32_t c = __brev(e >> a.low_bits) >> (32 - a.stages);
                    const uint64_t low = gi & ((1ULL << a.s0) - 1ULL);
                    if (c != 0 && low != 0)
                    {
                        const Fr w = a.twist != nullptr ? load_fr(a.twist + ((static_cast<uint64_t>(c) << a.s0) | low))
                                                        : domain_point(a.lo, a.hi, a.lo_bits, (low * c) << (a.log2n - a.s0 - a.stages));
                        v = mul(v, w);
                    }
                }
                smem_store(tile, e, v);
            }
            __syncthreads();

            for (unsigned t = 0; t < a.stages; ++t)
            {
                // butterflies pair rows that differ in bit t; m = the t row bits below it
                for (uint32_t b = threadIdx.x; b < tile_elems / 2; b += kThreads)
                {
                    // insert a zero at bit (t + low_bits) of b
                    const uint32_t pos = t + a.low_bits;
                    const uint32_t lower = b & ((1u << pos) - 1u);
                    const uint32_t e0 = ((b >> pos) << (pos + 1)) | lower;
                    const uint32_t e1 = e0 | (1u << pos);
                    const uint32_t m = lower >> a.low_bits;
                    const Fr u = smem_load(tile, e0);
                    Fr v = smem_load(tile, e1);
                    if (m != 0) v = mul(v, load_fr(a.small + (m << (9 - t))));
                    smem_store(tile, e0, add(u, v));
                    smem_store(tile, e1, sub(u, v));
                }
                __syncthreads();
            }

            for (uint32_t e = threadIdx.x; e < tile_elems; e += kThreads)
            {
                const uint64_t gi = tile_index(a, tile_id, e);
                Fr v = smem_load(tile, e);
                if (a.last && a.scale_mode >= 1) v = mul(v, a.scale);
                if (a.last && a.scale_mode == 2) v = mul(v, domain_point(a.shift_lo, a.shift_hi, a.shift_lo_bits, gi));
                store_fr(a.data + vec_offset + gi, v);
            }
        }

        // powers table: out[j] = base^(j << shift_bits)
        __global__ void power_table_kernel(Fr base, unsigned shift_bits, uint32_t count, Fr* out)
        {
            const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
            if (j < count) store_fr(out + j, pow_u64(base, static_cast<uint64_t>(j) << shift_bits));
        }

        // out[(c << s0) | low] = omega_(2^(s0+S))^(low * c): the load-time factors of a pass
        __global__ void twist_table_kernel(const Fr* lo, const Fr* hi, unsigned lo_bits, unsigned s0, uint64_t count, Fr* out)
        {
            const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
            if (i >= count) return;
            const uint64_t low = i & ((1ULL << s0) - 1ULL), c = i >> s0;
            store_fr(out + i, domain_point(lo, hi, lo_bits, low * c));
        }
        __global__ void small_table_kernel(const Fr* lo, const Fr* hi, unsigned lo_bits, Fr* out)
        {
            const uint32_t m = blockIdx.x * blockDim.x + threadIdx.x;
            if (m < 512) store_fr(out + m, domain_point(lo, hi, lo_bits, m));
        }

        constexpr unsigned kTwistTableMaxBits = 25;  // 1 GiB of load-time factors at most per table

        // The in-pass twiddle table (omega_1024^(+-m)) of the context, built on first use.
        int small_table(gzk_ctx* ctx, bool inverse, const Fr** out)
        {
            Fr*& slot = ctx->ntt_small[inverse ? 1 : 0];
            if (slot == nullptr)
            {
                const DomainTables* dom = nullptr;
                int rc = get_domain(ctx, 10, &dom);
                if (rc != GZK_OK) return rc;
                GZK_CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void**>(&slot), 512 * sizeof(Fr)));
                small_table_kernel<<<4, 128, 0, ctx->stream>>>(inverse ? dom->lo_inv : dom->lo, inverse ? dom->hi_inv : dom->hi, dom->lo_bits, slot);
                GZK_CUDA_TRY(ctx, cudaGetLastError());
            }
            *out = slot;
            return GZK_OK;
        }

        // The load-time factor table of a pass (s0, stages), built on first use; *out = NULL
        // when the table would exceed the size limit (the kernel then generates the factors).
        int twist_table(gzk_ctx* ctx, unsigned s0, unsigned stages, bool inverse, const Fr** out)
        {
            *out = nullptr;
            if (s0 + stages > kTwistTableMaxBits) return GZK_OK;
            for (const NttTwistTable& t : ctx->ntt_twists)
                if (t.s0 == s0 && t.stages == stages && t.inverse == inverse)
                {
                    *out = t.table;
                    return GZK_OK;
                }
            const DomainTables* dom = nullptr;
            int rc = get_domain(ctx, s0 + stages, &dom);
            if (rc != GZK_OK) return rc;
            const uint64_t count = 1ULL << (s0 + stages);
            NttTwistTable entry;
            entry.s0 = s0;
            entry.stages = stages;
            entry.inverse = inverse;
            const cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&entry.table), count * sizeof(Fr));
            if (err != cudaSuccess)
            {
                cudaGetLastError();  // no room for the table: fall back to generated factors
                return GZK_OK;
            }
            twist_table_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, ctx->stream>>>(
                inverse ? dom->lo_inv : dom->lo, inverse ? dom->hi_inv : dom->hi, dom->lo_bits, s0, count, entry.table);
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            ctx->ntt_twists.push_back(entry);
            *out = entry.table;
            return GZK_OK;
        }

        __global__ void fold_kernel(ColRef table, Fr r, uint64_t half, Fr* out, bool out_canonical)
        {
            const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
            // A canonical table enters as stored: r (Montgomery) times a canonical difference is the canonical
            // product, so lo + r (hi - lo) is formed in canonical form and converted once (two
            // multiplications per output instead of three); a Montgomery table needs one, and so does a canonical
            // table folded into a canonical (FR) output: a table that stays in one form costs one per round.
            const bool canonical = deficit(table) != 0;
            for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < half; i += stride)
            {
                const Fr lo = col_load_stored(table, 2 * i);
                const Fr hi = col_load_stored(table, 2 * i + 1);
                Fr folded = add(lo, mul(r, sub(hi, lo)));  // in the form of the table
                if (canonical && !out_canonical) folded = to_mont(folded);
                if (!canonical && out_canonical) folded = from_mont(folded);
                store_fr(out + i, folded);
            }
        }

        // Round sums of a multilinear table for one sumcheck round on a product-free claim:
        // s0 = sum t[2i], s1 = sum t[2i+1]; block partials, finished by one small block.
        __global__ void __launch_bounds__(kThreads) round_sums_kernel(ColRef table, uint64_t half, Fr* partial)
        {
            __shared__ Fr ws0[kThreads / 32], ws1[kThreads / 32];
            Fr s0 = Fr::zero(), s1 = Fr::zero();
            const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
            // sums of the stored residues; a canonical table is converted once per thread, not per element
            for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < half; i += stride)
            {
                s0 = add(s0, col_load_stored(table, 2 * i));
                s1 = add(s1, col_load_stored(table, 2 * i + 1));
            }
            if (deficit(table) != 0)
            {
                s0 = to_mont(s0);
                s1 = to_mont(s1);
            }
            const int lane = threadIdx.x & 31;
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1)
            {
                const Fr o0 = shfl_fr_idx(s0, (lane + offset) & 31);
                const Fr o1 = shfl_fr_idx(s1, (lane + offset) & 31);
                if (lane < offset)
                {
                    s0 = add(s0, o0);
                    s1 = add(s1, o1);
                }
            }
            if (lane == 0)
            {
                ws0[threadIdx.x >> 5] = s0;
                ws1[threadIdx.x >> 5] = s1;
            }
            __syncthreads();
            if (threadIdx.x == 0)
            {
                for (int w = 1; w < kThreads / 32; ++w)
                {
                    s0 = add(s0, ws0[w]);
                    s1 = add(s1, ws1[w]);
                }
                store_fr(partial + 2 * blockIdx.x, s0);
                store_fr(partial + 2 * blockIdx.x + 1, s1);
            }
        }
        __global__ void round_sums_finish_kernel(const Fr* partial, uint32_t blocks, Fr* out_canonical)
        {
            if (threadIdx.x >= 2) return;
            Fr s = Fr::zero();
            for (uint32_t b = 0; b < blocks; ++b) s = add(s, load_fr_plain(partial + 2 * b + threadIdx.x));
            store_fr(out_canonical + threadIdx.x, from_mont(s));
        }

        int scalar_mont(gzk_ctx* ctx, const uint8_t* bytes, Fr* out)
        {
            bool canonical = false;
            const Fr v = host_fr_from_bytes(bytes, &canonical);
            if (!canonical) return fail(ctx, GZK_E_INVALID, "scalar argument is not a canonical field element");
            *out = to_mont(v);
            return GZK_OK;
        }
    }
}

using namespace gzk;

extern "C"
{
    int gzk_ntt(gzk_ctx* ctx, const gzk_buf* in, gzk_buf* out, unsigned log2n, size_t batch, int inverse, const uint8_t* coset_shift)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (batch == 0) return GZK_OK;
        if (in == nullptr || out == nullptr) return fail(ctx, GZK_E_INVALID, "ntt: null argument");
        if (log2n > 30) return fail(ctx, GZK_E_INVALID, "ntt: domain too large");
        const uint64_t n = 1ULL << log2n;
        if (in->kind == GZK_KIND_F64 || in->kind == GZK_KIND_G1 || in->count < n * batch) return fail(ctx, GZK_E_INVALID, "ntt: input buffer too small or of the wrong kind");
        if (out->kind != GZK_KIND_FR_MONT || out->count < n * batch) return fail(ctx, GZK_E_INVALID, "ntt: output must be a Montgomery buffer of n*batch elements");
        if (out->dptr == in->dptr) return fail(ctx, GZK_E_INVALID, "ntt: input and output must be different buffers");
        if (batch > 65535) return fail(ctx, GZK_E_INVALID, "ntt: batch too large");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        const DomainTables* dom = nullptr;
        int rc = get_domain(ctx, log2n, &dom);
        if (rc != GZK_OK) return rc;

        NttArgs args{};
        args.in.ptr = in->dptr;
        args.in.kind = in->kind;
        args.data = static_cast<Fr*>(out->dptr);
        args.lo = inverse ? dom->lo_inv : dom->lo;
        args.hi = inverse ? dom->hi_inv : dom->hi;
        args.lo_bits = dom->lo_bits;
        if ((rc = small_table(ctx, inverse != 0, &args.small)) != GZK_OK) return rc;
        args.log2n = log2n;
        args.scale = dom->inv_size;
        args.scale_mode = inverse ? 1 : 0;

        if (coset_shift != nullptr)
        {
            Fr g;
            if ((rc = scalar_mont(ctx, coset_shift, &g)) != GZK_OK) return rc;
            if (g.is_zero()) return fail(ctx, GZK_E_INVALID, "ntt: coset shift must be non-zero");
            if (inverse) g = inv(g);
            // two-level table of powers of the shift (or its inverse)
            const unsigned lo_bits = (log2n + 1) / 2;
            const uint32_t lo_count = 1u << lo_bits, hi_count = 1u << (log2n - lo_bits);
            void* scratch = nullptr;
            if ((rc = ensure_scratch(ctx, 2, static_cast<size_t>(lo_count + hi_count) * sizeof(Fr), &scratch)) != GZK_OK) return rc;
            Fr* t_lo = static_cast<Fr*>(scratch);
            Fr* t_hi = t_lo + lo_count;
            {
                LaunchScope scope(ctx, "ntt_shift_table", 2);
                power_table_kernel<<<(lo_count + 127) / 128, 128, 0, ctx->stream>>>(g, 0, lo_count, t_lo);
                power_table_kernel<<<(hi_count + 127) / 128, 128, 0, ctx->stream>>>(g, lo_bits, hi_count, t_hi);
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            args.shift_lo = t_lo;
            args.shift_hi = t_hi;
            args.shift_lo_bits = lo_bits;
            args.pre_shift = inverse ? 0 : 1;
            if (inverse) args.scale_mode = 2;
        }

        const size_t smem = 8 * kTile * sizeof(uint32_t);
        // pass 0 takes up to 10 stages; the rest is spread evenly over passes of at most 8
        // stages, each on full 1024-element tiles (2^stages rows of 2^(10-stages) contiguous elements)
        const unsigned later = log2n > static_cast<unsigned>(kTileBits) ? log2n - kTileBits : 0;
        const unsigned later_passes = (later + 7) / 8;
        unsigned later_done = 0, pass_index = 0;
        unsigned s0 = 0;
        do
        {
            const unsigned remaining = log2n - s0;
            unsigned low_bits = 0, stages = 0;
            args.twist = nullptr;
            if (s0 == 0)
            {
                stages = remaining < static_cast<unsigned>(kTileBits) ? remaining : kTileBits;
            }
            else
            {
                // passes still to run share what is left as evenly as possible
                const unsigned passes_left = later_passes - pass_index;
                stages = (later - later_done + passes_left - 1) / passes_left;
                low_bits = kTileBits - stages;
                later_done += stages;
                ++pass_index;
                if ((rc = twist_table(ctx, s0, stages, inverse != 0, &args.twist)) != GZK_OK) return rc;
            }
            args.s0 = s0;
            args.stages = stages;
            args.low_bits = low_bits;
            args.last = (s0 + stages == log2n) ? 1 : 0;
            const uint64_t tiles = n >> (stages + low_bits);
            dim3 grid(static_cast<unsigned>(tiles), static_cast<unsigned>(batch));
            {
                LaunchScope scope(ctx, "ntt_pass");
                ntt_pass_kernel<<<grid, kThreads, smem, ctx->stream>>>(args);
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            s0 += stages;
        } while (s0 < log2n);
        return finish_call(ctx, "invalid input");
    }

    int gzk_fold(gzk_ctx* ctx, const gzk_buf* table, size_t n, const uint8_t challenge[32], gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (n < 2) return GZK_OK;
        if (table == nullptr || out == nullptr || challenge == nullptr) return fail(ctx, GZK_E_INVALID, "fold: null argument");
        if (table->kind == GZK_KIND_F64 || table->kind == GZK_KIND_G1 || table->count < n) return fail(ctx, GZK_E_INVALID, "fold: table buffer too small or of the wrong kind");
        if ((out->kind != GZK_KIND_FR_MONT && out->kind != GZK_KIND_FR) || out->count < n / 2)
            return fail(ctx, GZK_E_INVALID, "fold: output must be an FR or FR_MONT buffer of n/2 elements");
        Fr r;
        int rc = scalar_mont(ctx, challenge, &r);
        if (rc != GZK_OK) return rc;
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        ColRef t;
        t.ptr = table->dptr;
        t.kind = table->kind;
        const uint64_t half = n / 2;
        uint64_t blocks = (half + kThreads - 1) / kThreads;
        const uint64_t cap = static_cast<uint64_t>(ctx->sm_count) * 16;
        if (blocks > cap) blocks = cap;
        {
            LaunchScope scope(ctx, "fold");
            fold_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, ctx->stream>>>(t, r, half, static_cast<Fr*>(out->dptr), out->kind == GZK_KIND_FR);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }

    // out[0] = sum_i t[2i], out[1] = sum_i t[2i+1], out[2] = 2*out[1] - out[0]: the values at
    // 0, 1, 2 of the round polynomial sum_i (t[2i] + X (t[2i+1] - t[2i])) of a sumcheck round.
    // With the table split over GPUs each rank computes its three values and the ranks
    // all-gather and add them (gzk_fr_sum) before the Fiat-Shamir squeeze.
    int gzk_sumcheck_round_sums(gzk_ctx* ctx, const gzk_buf* table, size_t n, uint8_t out[3 * 32])
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (out == nullptr) return fail(ctx, GZK_E_INVALID, "sumcheck_round_sums: null output");
        std::memset(out, 0, 96);
        if (n < 2) return GZK_OK;
        if (table == nullptr || table->kind == GZK_KIND_F64 || table->kind == GZK_KIND_G1 || table->count < n)
            return fail(ctx, GZK_E_INVALID, "sumcheck_round_sums: table buffer too small or of the wrong kind");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        const uint64_t half = n / 2;
        uint64_t blocks = (half + kThreads - 1) / kThreads;
        const uint64_t cap = static_cast<uint64_t>(ctx->sm_count) * 8;
        if (blocks > cap) blocks = cap;
        void* scratch = nullptr;
        int rc = ensure_scratch(ctx, 2, (2 * blocks + 2) * sizeof(Fr), &scratch);
        if (rc != GZK_OK) return rc;
        Fr* partial = static_cast<Fr*>(scratch);
        ColRef t;
        t.ptr = table->dptr;
        t.kind = table->kind;
        {
            LaunchScope scope(ctx, "round_sums", 2);
            round_sums_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, ctx->stream>>>(t, half, partial);
            round_sums_finish_kernel<<<1, 32, 0, ctx->stream>>>(partial, static_cast<uint32_t>(blocks), partial + 2 * blocks);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(out, partial + 2 * blocks, 64, cudaMemcpyDeviceToHost, ctx->stream));
        GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        // value at 2 = s0 + 2 (s1 - s0) = 2 s1 - s0, on the host
        uint8_t twice[32];
        if (gzk_fr_op(0, out + 32, out + 32, twice) != GZK_OK || gzk_fr_op(1, twice, out, out + 64) != GZK_OK)
            return fail(ctx, GZK_E_INVALID, "sumcheck_round_sums: internal arithmetic error");
        return GZK_OK;
    }

    // Coset low-degree extension: evaluations on the 2^log2n domain -> evaluations of the
    // same polynomial on shift * (2^(log2n+log2_blowup) domain).
    int gzk_coset_lde(gzk_ctx* ctx, const gzk_buf* in, unsigned log2n, unsigned log2_blowup, const uint8_t shift[32], gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (in == nullptr || out == nullptr || shift == nullptr) return fail(ctx, GZK_E_INVALID, "coset_lde: null argument");
        if (log2n + log2_blowup > 30) return fail(ctx, GZK_E_INVALID, "coset_lde: extended domain too large");
        const size_t n = static_cast<size_t>(1) << log2n, big = n << log2_blowup;
        if (out->kind != GZK_KIND_FR_MONT || out->count < big) return fail(ctx, GZK_E_INVALID, "coset_lde: output must be a Montgomery buffer of the extended size");
        gzk_buf* coeffs = nullptr;
        int rc = gzk_buf_alloc(ctx, GZK_KIND_FR_MONT, big, &coeffs);
        if (rc != GZK_OK) return rc;
        rc = gzk_ntt(ctx, in, coeffs, log2n, 1, 1, nullptr);
        if (rc == GZK_OK && big > n)
        {
            const cudaError_t err = cudaMemsetAsync(static_cast<char*>(coeffs->dptr) + n * 32, 0, (big - n) * 32, ctx->stream);
            if (err != cudaSuccess) rc = cuda_fail(ctx, err, "cudaMemsetAsync(lde padding)");
        }
        if (rc == GZK_OK) rc = gzk_ntt(ctx, coeffs, out, log2n + log2_blowup, 1, 0, shift);
        const std::string message = ctx->last_error;
        gzk_buf_free(ctx, coeffs);
        if (rc != GZK_OK) ctx->last_error = message;
        return rc;
    }
}
