// Row-major matrix kernels of the binding / commitment path:
//   matrix_horner      the matrix read as ONE coefficient polynomial (row-major
//                      flattening) evaluated at a point;
//   fold_rows          out[c] = sum_row w[row] * M[row][c];
//   linear_form_rows   out[row] = sum_c M[row][c] * p[c];
//   powers             1, c, c^2, ...
#include <cstring>

#include "block.cuh"

namespace gzk
{
    uint32_t fold_rows_groups_tiles(gzk_ctx* ctx, size_t row_count, uint32_t cols, uint64_t* tile_rows_out);
    void launch_fold_rows_groups(gzk_ctx* ctx, const void* matrix, const Fr* weights, size_t row_count, uint32_t cols, uint64_t tile_rows, uint32_t tiles,
                                 uint32_t* partial);
    void launch_linear_form_tensor(gzk_ctx* ctx, const void* matrix, uint64_t rows, uint32_t cols, uint64_t total_entries, const Fr* powers, void* table,
                                   const Fr* bias, Fr* out);
    int launch_eval_finish(gzk_ctx* ctx, const uint32_t* partial, int uniform_kind, uint32_t tiles, uint32_t k_count,
                           Fr* out, bool out_montgomery);

    namespace
    {
        constexpr int kThreads = 256;
        constexpr int kAccLimbs = 17;

        // ---- Horner ------------------------------------------------------------------
        // CTA b owns coefficients [b*span, (b+1)*span).  Thread t runs Horner in x^T over
        // the coefficients s+t, s+t+T, ... (coalesced across the CTA), scales by x^t; the
        // CTA sum is scaled by x^s.  One Montgomery multiplication per coefficient: the coefficients
        // enter as stored (x in Montgomery form times a canonical value stays canonical), so a canonical
        // matrix gives the canonical result directly and a Montgomery one is converted at the end.
        __global__ void __launch_bounds__(kThreads) horner_kernel(ColRef coeffs, uint64_t total, uint64_t span, Fr x, Fr x_stride,
                                                                  Fr* partial)
        {
            __shared__ Fr warp_sum[kThreads / 32];
            const uint64_t s = static_cast<uint64_t>(blockIdx.x) * span;
            const uint64_t e_end = s + span < total ? s + span : total;
            Fr acc = Fr::zero();
            if (s + threadIdx.x < e_end)
            {
                const uint64_t steps = (e_end - s - threadIdx.x - 1) / kThreads;  // last index = s + t + steps*T
                for (uint64_t j = steps + 1; j-- > 0;)
                {
                    acc = mul(acc, x_stride);
                    acc = add(acc, col_load_stored(coeffs, s + threadIdx.x + j * kThreads));
                }
                acc = mul(acc, pow_u64(x, threadIdx.x));
            }
            const int lane = threadIdx.x & 31;
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1)
            {
                const Fr other = shfl_fr_idx(acc, (lane + offset) & 31);
                if (lane < offset) acc = add(acc, other);
            }
            if (lane == 0) warp_sum[threadIdx.x >> 5] = acc;
            __syncthreads();
            if (threadIdx.x == 0)
            {
                Fr sum = warp_sum[0];
#pragma unroll
                for (int w = 1; w < kThreads / 32; ++w) sum = add(sum, warp_sum[w]);
                store_fr(partial + blockIdx.x, mul(sum, pow_u64(x, s)));
            }
        }

        // Matrix entries by buffer kind, resolved at compile time so that a kernel can issue the loads of
        // several entries before the multiply-adds that consume them (a branch on the kind inside the loop
        // would pin every load behind the previous product).  acc += w * entry as an exact integer:
        // field-element entries are used as stored; a small-integer entry v enters as its magnitude (one or
        // two limbs) against w or, for v < 0, r - w (w * (r - |v|) is congruent to (r - w) * |v|): 8 x 2 limb
        // products instead of the 8 x 8 plus a conversion that widening it to a field element would cost.
        // The sum then carries the same power of R as one over canonical field elements.
        template <int KIND>
        struct Entry
        {
            using Raw = Fr;
            static __device__ __forceinline__ Raw zero() { return Fr::zero(); }
            static __device__ __forceinline__ Raw load(const void* ptr, uint64_t i) { return load_fr(static_cast<const Fr*>(ptr) + i); }
            static __device__ __forceinline__ Raw at(const Raw* p) { return load_fr(p); }
            static __device__ __forceinline__ void mac(WideAcc& acc, const Fr& w, const Raw& v) { acc.mac<8>(w.l, v.l); }
        };
        template <>
        struct Entry<GZK_KIND_U32>
        {
            using Raw = uint32_t;
            static __device__ __forceinline__ Raw zero() { return 0u; }
            static __device__ __forceinline__ Raw load(const void* ptr, uint64_t i) { return __ldg(static_cast<const uint32_t*>(ptr) + i); }
            static __device__ __forceinline__ Raw at(const Raw* p) { return __ldg(p); }
            static __device__ __forceinline__ void mac(WideAcc& acc, const Fr& w, const Raw& v) { acc.mac<1>(w.l, &v); }
        };
        template <>
        struct Entry<GZK_KIND_I64>
        {
            using Raw = long long;
            static __device__ __forceinline__ Raw zero() { return 0; }
            static __device__ __forceinline__ Raw load(const void* ptr, uint64_t i) { return __ldg(static_cast<const long long*>(ptr) + i); }
            static __device__ __forceinline__ Raw at(const Raw* p) { return __ldg(p); }
            static __device__ __forceinline__ void mac(WideAcc& acc, const Fr& w, const Raw& v)
            {
                const unsigned long long mag = v < 0 ? 0ULL - static_cast<unsigned long long>(v) : static_cast<unsigned long long>(v);
                const uint32_t f[2] = {static_cast<uint32_t>(mag), static_cast<uint32_t>(mag >> 32)};
                const Fr signed_w = v < 0 ? sub(Fr::zero(), w) : w;
                // witness values are a few dozen bits at most: the second limb is almost never set
                if (f[1] == 0)
                    acc.mac<1>(signed_w.l, f);
                else
                    acc.mac<2>(signed_w.l, f);
            }
        };
        // acc += w * (v + 2^31) for a signed 64-bit entry: the biased value is non-negative, so the sign needs no
        // negated weight; the caller subtracts 2^31 * (sum of the weights) once per sum.  v + 2^31 = u + 2^32 k with
        // u = low word of v with its top bit flipped and k = (v >> 32) + (bit 31 of v): k is 0 for |v| < 2^31, i.e.
        // for every witness value in practice, and the product is then eight limb products.
        __device__ __forceinline__ void mac_biased_i64(WideAcc& acc, const Fr& w, long long v)
        {
            const uint32_t low = static_cast<uint32_t>(static_cast<unsigned long long>(v));
            const uint32_t u = low ^ 0x80000000u;
            const long long k = (v >> 32) + static_cast<long long>(low >> 31);
            acc.mac<1>(w.l, &u);
            if (k != 0)
            {
                const unsigned long long mag = k < 0 ? 0ULL - static_cast<unsigned long long>(k) : static_cast<unsigned long long>(k);
                const Fr signed_w = k < 0 ? sub(Fr::zero(), w) : w;
                acc.row<1>(signed_w.l, static_cast<uint32_t>(mag));
                if ((mag >> 32) != 0) acc.row<2>(signed_w.l, static_cast<uint32_t>(mag >> 32));
            }
        }

        // out = scale * (v[0] + ... + v[count-1]), everything in Montgomery form; one CTA.
        __global__ void __launch_bounds__(kThreads) scaled_sum_kernel(const Fr* v, uint32_t count, Fr scale, Fr* out)
        {
            __shared__ Fr warp_sum[kThreads / 32];
            Fr acc = Fr::zero();
            for (uint32_t i = threadIdx.x; i < count; i += kThreads) acc = add(acc, load_fr(v + i));
            const int lane = threadIdx.x & 31;
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1)
            {
                const Fr other = shfl_fr_idx(acc, (lane + offset) & 31);
                if (lane < offset) acc = add(acc, other);
            }
            if (lane == 0) warp_sum[threadIdx.x >> 5] = acc;
            __syncthreads();
            if (threadIdx.x == 0)
            {
                Fr sum = warp_sum[0];
#pragma unroll
                for (int w = 1; w < kThreads / 32; ++w) sum = add(sum, warp_sum[w]);
                store_fr(out, mul(sum, scale));
            }
        }

        // FR and FR_MONT share the field-element code
        constexpr int entry_kind(int kind) { return kind == GZK_KIND_U32 || kind == GZK_KIND_I64 ? kind : GZK_KIND_FR; }

        // A table of field elements in shared memory as two arrays of 16-byte halves: lanes that read consecutive
        // elements then touch consecutive 16-byte words (no bank conflict), and a whole warp reading one element
        // is a broadcast.
        __device__ __forceinline__ void store_fr_split(uint4* lo, uint4* hi, uint32_t i, const Fr& v)
        {
            lo[i] = make_uint4(v.l[0], v.l[1], v.l[2], v.l[3]);
            hi[i] = make_uint4(v.l[4], v.l[5], v.l[6], v.l[7]);
        }
        __device__ __forceinline__ Fr load_fr_split(const uint4* lo, const uint4* hi, uint32_t i)
        {
            const uint4 a = lo[i], b = hi[i];
            Fr o;
            o.l[0] = a.x; o.l[1] = a.y; o.l[2] = a.z; o.l[3] = a.w;
            o.l[4] = b.x; o.l[5] = b.y; o.l[6] = b.z; o.l[7] = b.w;
            return o;
        }

        // Small-integer coefficients: Horner costs a full field multiplication per coefficient although the
        // coefficient itself is one or two limbs.  Cut the polynomial into blocks of 1024 coefficients,
        // r_b = sum_j c[1024 b + j] x^j as an exact 8 x 2 limb inner product against the 1024 powers of x
        // (one warp per block, 32 coefficients per lane, the powers in shared memory), and leave Horner to the
        // 1024 times shorter polynomial sum_b r_b (x^1024)^b.  out[b] is the Montgomery form of r_b.
        // The block is long because every block ends in a warp-wide exact sum, one reduction and one field
        // multiplication (some 500 instructions per lane): with 256-coefficient blocks that tail was twice the
        // cost of the products themselves.
        constexpr int kDotBlock = 1024;
        // `bias` (I64 only): 2^31 * (sum of the powers), Montgomery form; the entries then enter biased.
        template <int KIND>
        __global__ void __launch_bounds__(kThreads) block_dot_kernel(const void* coeffs, uint64_t total, const Fr* powers, uint64_t blocks, Fr* out,
                                                                     const Fr* bias)
        {
            __shared__ uint4 pw_lo[kDotBlock], pw_hi[kDotBlock];
            for (uint32_t i = threadIdx.x; i < kDotBlock; i += kThreads) store_fr_split(pw_lo, pw_hi, i, load_fr(powers + i));
            __syncthreads();
            const uint32_t lane = threadIdx.x & 31;
            const uint64_t warp = (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
            const uint64_t warps = (static_cast<uint64_t>(gridDim.x) * kThreads) >> 5;
            for (uint64_t b = warp; b < blocks; b += warps)
            {
                WideAcc acc;
                acc.clear();
                const uint64_t base = b * kDotBlock + lane;
#pragma unroll 1
                for (int k = 0; k < kDotBlock / 32; k += 4)
                {
                    typename Entry<KIND>::Raw raw[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                    {
                        const uint64_t i = base + 32ull * (k + u);
                        raw[u] = i < total ? Entry<KIND>::load(coeffs, i) : Entry<KIND>::zero();
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                    {
                        const Fr w = load_fr_split(pw_lo, pw_hi, lane + 32u * (k + u));
                        if constexpr (KIND == GZK_KIND_I64)
                            mac_biased_i64(acc, w, raw[u]);
                        else
                            Entry<KIND>::mac(acc, w, raw[u]);
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
                    Fr value = mul(redc_wide<FrCfg, 9>(sum), fr_const_2_544());
                    if constexpr (KIND == GZK_KIND_I64) value = sub(value, load_fr(bias));
                    store_fr(out + b, value);
                }
            }
        }

        // `down` > 0: that many conversions out of Montgomery form; < 0: into it.
        __global__ void sum_partials_kernel(const Fr* partial, uint32_t count, int down, Fr* out)
        {
            if (threadIdx.x != 0 || blockIdx.x != 0) return;
            Fr sum = Fr::zero();
            for (uint32_t i = 0; i < count; ++i) sum = add(sum, load_fr_plain(partial + i));
            for (; down > 0; --down) sum = from_mont(sum);
            for (; down < 0; ++down) sum = to_mont(sum);
            store_fr(out, sum);
        }

        // ---- fold rows ----------------------------------------------------------------
        // CTA (tile, column chunk): threads are laid out as (row lane, column); each
        // thread accumulates w[row] * M[row][c] unreduced over the rows of the tile that
        // fall on its row lane; row lanes are then summed through shared memory.
        // Signed 64-bit entries enter biased, as v + 2^31 >= 0 (no negated weight per negative entry); the surplus
        // 2^31 * (sum of the tile's weights) is the same for every column of the tile, so the CTA adds up its
        // weights once and every column's partial sum receives 2^31 * (r - that sum), which cancels it modulo r.
        constexpr uint32_t kFoldStage = 512;
        template <int KIND>
        __global__ void __launch_bounds__(kThreads) fold_rows_kernel(const void* matrix, const Fr* weights, uint64_t row_count, uint32_t cols,
                                                                     uint64_t tile_rows, uint32_t col_chunks, uint32_t* partial)
        {
            extern __shared__ uint32_t lanes_sum[];  // [kThreads][17]
            __shared__ Fr warp_weights[kThreads / 32];
            __shared__ uint32_t correction[9];
            __shared__ uint4 stage_lo[kFoldStage], stage_hi[kFoldStage];
            const uint32_t tile = blockIdx.x / col_chunks;
            const uint32_t chunk = blockIdx.x - tile * col_chunks;
            const uint32_t width = cols < kThreads ? cols : kThreads;   // columns handled by this CTA
            const uint32_t row_lanes = kThreads / width;
            const uint32_t c_local = threadIdx.x % width;
            const uint32_t row_lane = threadIdx.x / width;
            const uint32_t c = chunk * kThreads + c_local;
            const uint64_t r_begin = static_cast<uint64_t>(tile) * tile_rows;
            const uint64_t r_end = r_begin + tile_rows < row_count ? r_begin + tile_rows : row_count;
            if constexpr (KIND == GZK_KIND_I64)
            {
                Fr mine = Fr::zero();
                for (uint64_t row = r_begin + threadIdx.x; row < r_end; row += kThreads) mine = add(mine, load_fr(weights + row));
                const int lane = threadIdx.x & 31;
#pragma unroll
                for (int offset = 16; offset > 0; offset >>= 1) mine = add(mine, shfl_fr_idx(mine, (lane + offset) & 31));  // lane 0 ends with the warp's sum
                if (lane == 0) warp_weights[threadIdx.x >> 5] = mine;
                __syncthreads();
                if (threadIdx.x == 0)
                {
                    Fr total = warp_weights[0];
#pragma unroll
                    for (int w = 1; w < kThreads / 32; ++w) total = add(total, warp_weights[w]);
                    const Fr rest = sub(Fr::zero(), total);  // r - total (0 when total is 0)
                    correction[0] = rest.l[0] << 31;
#pragma unroll
                    for (int i = 1; i < 8; ++i) correction[i] = (rest.l[i] << 31) | (rest.l[i - 1] >> 1);
                    correction[8] = rest.l[7] >> 1;
                }
                __syncthreads();
            }
            WideAcc acc;
            acc.clear();
            auto mac = [&](const Fr& w, const typename Entry<KIND>::Raw& v) {
                if constexpr (KIND == GZK_KIND_I64)
                    mac_biased_i64(acc, w, v);
                else
                    Entry<KIND>::mac(acc, w, v);
            };
            // The weights of kFoldStage rows at a time pass through shared memory (every thread of the CTA needs the
            // same ones: a broadcast read each), and the entries are walked with a running pointer.
            using Raw = typename Entry<KIND>::Raw;
            constexpr int kAhead = KIND == GZK_KIND_FR ? 4 : 8;  // entries requested before the first product
            const bool active = row_lane < row_lanes && c < cols;
            const uint64_t stride = static_cast<uint64_t>(row_lanes) * cols;
            for (uint64_t s0 = r_begin; s0 < r_end; s0 += kFoldStage)
            {
                const uint32_t n = static_cast<uint32_t>(r_end - s0 < kFoldStage ? r_end - s0 : kFoldStage);
                for (uint32_t i = threadIdx.x; i < n; i += kThreads) store_fr_split(stage_lo, stage_hi, i, load_fr(weights + s0 + i));
                __syncthreads();
                if (active)
                {
                    const Raw* p = static_cast<const Raw*>(matrix) + (s0 + row_lane) * cols + c;
                    uint32_t j = row_lane;
                    for (; j + (kAhead - 1) * row_lanes < n; j += kAhead * row_lanes)
                    {
                        Raw raw[kAhead];
#pragma unroll
                        for (int u = 0; u < kAhead; ++u) raw[u] = Entry<KIND>::at(p + u * stride);
#pragma unroll
                        for (int u = 0; u < kAhead; ++u) mac(load_fr_split(stage_lo, stage_hi, j + u * row_lanes), raw[u]);
                        p += kAhead * stride;
                    }
                    for (; j < n; j += row_lanes)
                    {
                        mac(load_fr_split(stage_lo, stage_hi, j), Entry<KIND>::at(p));
                        p += stride;
                    }
                }
                __syncthreads();
            }
            uint32_t sum[kAccLimbs];
            acc.fold(sum);
#pragma unroll
            for (int i = 0; i < kAccLimbs; ++i) lanes_sum[threadIdx.x * kAccLimbs + i] = sum[i];
            __syncthreads();
            if (row_lane == 0 && c < cols)
            {
                for (uint32_t rl = 1; rl < row_lanes; ++rl)
                {
                    uint32_t other[kAccLimbs];
#pragma unroll
                    for (int i = 0; i < kAccLimbs; ++i) other[i] = lanes_sum[(rl * width + c_local) * kAccLimbs + i];
                    acc_add<kAccLimbs, kAccLimbs>(sum, other);
                }
                if constexpr (KIND == GZK_KIND_I64)
                {
                    uint32_t fix[9];
#pragma unroll
                    for (int i = 0; i < 9; ++i) fix[i] = correction[i];
                    acc_add<kAccLimbs, 9>(sum, fix);
                }
                uint32_t* dst = partial + (static_cast<uint64_t>(tile) * cols + c) * kAccLimbs;
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) dst[i] = sum[i];
            }
        }

        // ---- linear form over rows -------------------------------------------------------
        // One warp per row: lanes stride over the columns, exact warp sum, one reduction.
        template <int KIND>
        __global__ void __launch_bounds__(kThreads) linear_form_kernel(const void* matrix, int montgomery_entries, const Fr* powers, uint64_t rows,
                                                                       uint32_t cols, Fr* out, const Fr* bias)
        {
            const uint32_t lane = threadIdx.x & 31;
            const uint64_t row = (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
            if (row >= rows) return;
            WideAcc acc;
            acc.clear();
            uint32_t j = lane;
            for (; j + 96 < cols; j += 128)
            {
                typename Entry<KIND>::Raw raw[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) raw[u] = Entry<KIND>::load(matrix, row * cols + j + 32 * u);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                {
                    if constexpr (KIND == GZK_KIND_I64)
                        mac_biased_i64(acc, load_fr(powers + j + 32 * u), raw[u]);
                    else
                        Entry<KIND>::mac(acc, load_fr(powers + j + 32 * u), raw[u]);
                }
            }
            for (; j < cols; j += 32)
            {
                if constexpr (KIND == GZK_KIND_I64)
                    mac_biased_i64(acc, load_fr(powers + j), Entry<KIND>::load(matrix, row * cols + j));
                else
                    Entry<KIND>::mac(acc, load_fr(powers + j), Entry<KIND>::load(matrix, row * cols + j));
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
                const Fr reduced = redc_wide<FrCfg, 9>(sum);
                Fr fix;
                if (!montgomery_entries)
                {
                    fix = fr_const_2_544();  // canonical and small-integer entries: one factor of R less in the sum
                }
                else
                {
                    constexpr uint32_t c288[8] = {0xcaaf6b13u, 0x355094eau, 0x69a568efu, 0xf6b10cb3u,
                                                  0x40cc3869u, 0xe2c926a6u, 0xed269aadu, 0x736a6d3bu};
#pragma unroll
                    for (int i = 0; i < 8; ++i) fix.l[i] = c288[i];
                }
                Fr value = mul(reduced, fix);
                if constexpr (KIND == GZK_KIND_I64) value = sub(value, load_fr(bias));  // every entry entered as v + 2^31
                store_fr(out + row, value);
            }
        }

        // Small-integer matrices with many rows: one THREAD per row.  A CTA stages 128 rows x 32 columns at a time in
        // shared memory (read row-wise by the warps, so the global loads stay contiguous; rows padded by one entry
        // so that the threads' walks along their rows fall on different banks) together with the 32 powers, which
        // every thread then reads as a broadcast.  No sum crosses lanes: each thread folds and reduces its own row
        // once, which costs a few instructions per entry instead of the warp-wide exact sum per 256-entry row of
        // the warp-per-row kernel (two thirds of that kernel's instructions).
        constexpr int kRowThreads = 128, kRowChunk = 32;
        template <int KIND>
        __global__ void __launch_bounds__(kRowThreads) linear_form_by_thread_kernel(const void* matrix, const Fr* powers, uint64_t rows, uint32_t cols,
                                                                                    Fr* out, const Fr* bias)
        {
            using Raw = typename Entry<KIND>::Raw;
            __shared__ Raw tile[kRowThreads][kRowChunk + 1];
            __shared__ uint4 pw_lo[kRowChunk], pw_hi[kRowChunk];
            const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            const uint64_t row0 = static_cast<uint64_t>(blockIdx.x) * kRowThreads;
            WideAcc acc;
            acc.clear();
            for (uint32_t c0 = 0; c0 < cols; c0 += kRowChunk)
            {
                const uint32_t col = c0 + lane;
#pragma unroll 8
                for (uint32_t r = warp; r < kRowThreads; r += kRowThreads / 32)
                {
                    const uint64_t row = row0 + r;
                    tile[r][lane] = (row < rows && col < cols) ? Entry<KIND>::load(matrix, row * cols + col) : Entry<KIND>::zero();
                }
                if (threadIdx.x < kRowChunk) store_fr_split(pw_lo, pw_hi, threadIdx.x, c0 + threadIdx.x < cols ? load_fr(powers + c0 + threadIdx.x) : Fr::zero());
                __syncthreads();
                const uint32_t n = cols - c0 < kRowChunk ? cols - c0 : kRowChunk;
#pragma unroll 4
                for (uint32_t j = 0; j < n; ++j)
                {
                    const Fr w = load_fr_split(pw_lo, pw_hi, j);
                    if constexpr (KIND == GZK_KIND_I64)
                        mac_biased_i64(acc, w, tile[threadIdx.x][j]);
                    else
                        Entry<KIND>::mac(acc, w, tile[threadIdx.x][j]);
                }
                __syncthreads();
            }
            const uint64_t row = row0 + threadIdx.x;
            if (row >= rows) return;
            uint32_t sum[kAccLimbs];
            acc.fold(sum);
            Fr value = mul(redc_wide<FrCfg, 9>(sum), fr_const_2_544());  // small-integer entries: one factor of R less in the sum
            if constexpr (KIND == GZK_KIND_I64) value = sub(value, load_fr(bias));  // every entry entered as v + 2^31
            store_fr(out + row, value);
        }

        __global__ void powers_kernel(Fr c, uint64_t count, Fr* out)
        {
            const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
            if (i < count) store_fr(out + i, pow_u64(c, i));
        }

        // 2^31 in Montgomery form
        Fr mont_two_63()
        {
            Fr v = Fr::one();
            for (int d = 0; d < 63; ++d) v = add(v, v);
            return v;
        }
        Fr mont_two_31()
        {
            Fr v = Fr::one();
            for (int d = 0; d < 31; ++d) v = add(v, v);
            return v;
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
    // Shared body: the evaluation ends in dest (canonical, or Montgomery form when dest_montgomery).
    static int matrix_horner_enqueue(gzk_ctx* ctx, const gzk_buf* matrix, uint64_t total, const Fr& x, Fr* dest, bool dest_montgomery,
                                     Fr** scratch_result)
    {
        const bool small_kind = matrix->kind == GZK_KIND_I64 || matrix->kind == GZK_KIND_U32;
        const bool blocked = small_kind && total >= (1u << 16);
        const uint64_t dot_blocks = blocked ? (total + kDotBlock - 1) / kDotBlock : 0;
        const uint64_t horner_total = blocked ? dot_blocks : total;
        uint64_t ctas = (horner_total + static_cast<uint64_t>(kThreads) * 8 - 1) / (static_cast<uint64_t>(kThreads) * 8);
        const uint64_t max_ctas = static_cast<uint64_t>(ctx->sm_count) * 8;
        if (ctas > max_ctas) ctas = max_ctas;
        uint64_t span = (horner_total + ctas - 1) / ctas;
        span = (span + kThreads - 1) / kThreads * kThreads;
        ctas = (horner_total + span - 1) / span;
        void* scratch = nullptr;
        int rc = ensure_scratch(ctx, 2, (ctas + 1 + (blocked ? kDotBlock + 1 + dot_blocks : 0)) * sizeof(Fr), &scratch);
        if (rc != GZK_OK) return rc;
        Fr* partial = static_cast<Fr*>(scratch);
        ColRef m;
        m.ptr = matrix->dptr;
        m.kind = matrix->kind;
        Fr x_horner = x;
        const bool tensor_blocks = blocked && matrix->kind == GZK_KIND_I64 && dot_blocks >= static_cast<uint64_t>(ctx->sm_count) * 32;
        void* block_table = nullptr;
        if (tensor_blocks && (rc = ensure_scratch(ctx, 1, static_cast<size_t>(kDotBlock) * 256, &block_table)) != GZK_OK) return rc;
        if (blocked)
        {
            Fr* powers = partial + ctas + 1;
            Fr* bias = powers + kDotBlock;
            Fr* block_values = bias + 1;
            {
                LaunchScope scope(ctx, "powers");
                powers_kernel<<<kDotBlock / kThreads, kThreads, 0, ctx->stream>>>(x, kDotBlock, powers);
                // many blocks of I64 coefficients: the block sums are a row-wise linear form of a dot_blocks x 1024 matrix
                // and run on the tensor cores (entries biased by 2^63 there, by 2^31 in block_dot_kernel)
                if (matrix->kind == GZK_KIND_I64)
                    scaled_sum_kernel<<<1, kThreads, 0, ctx->stream>>>(powers, kDotBlock, tensor_blocks ? mont_two_63() : mont_two_31(), bias);
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            const uint64_t warps_wanted = dot_blocks < static_cast<uint64_t>(ctx->sm_count) * 64 ? dot_blocks : static_cast<uint64_t>(ctx->sm_count) * 64;
            {
                LaunchScope scope(ctx, "horner_block_dot");
                const unsigned grid = static_cast<unsigned>((warps_wanted * 32 + kThreads - 1) / kThreads);
                if (tensor_blocks)
                    launch_linear_form_tensor(ctx, m.ptr, dot_blocks, kDotBlock, total, powers, block_table, bias, block_values);
                else if (matrix->kind == GZK_KIND_I64)
                    block_dot_kernel<GZK_KIND_I64><<<grid, kThreads, 0, ctx->stream>>>(m.ptr, total, powers, dot_blocks, block_values, bias);
                else
                    block_dot_kernel<GZK_KIND_U32><<<grid, kThreads, 0, ctx->stream>>>(m.ptr, total, powers, dot_blocks, block_values, nullptr);
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            m.ptr = block_values;
            m.kind = GZK_KIND_FR_MONT;
            x_horner = pow_u64(x, kDotBlock);
        }
        {
            LaunchScope scope(ctx, "horner");
            horner_kernel<<<static_cast<unsigned>(ctas), kThreads, 0, ctx->stream>>>(m, horner_total, span, x_horner, pow_u64(x_horner, kThreads), partial);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        Fr* result = dest != nullptr ? dest : partial + ctas;
        {
            // the partial sums are Montgomery values of the canonical result (canonical entries) or of its
            // Montgomery form (Montgomery entries): one or two conversions bring them to the wanted form
            LaunchScope scope(ctx, "horner_sum");
            const int down = (m.kind == GZK_KIND_FR_MONT ? 1 : 0) - (dest_montgomery ? 1 : 0);
            sum_partials_kernel<<<1, 32, 0, ctx->stream>>>(partial, static_cast<uint32_t>(ctas), down, result);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        if (scratch_result != nullptr) *scratch_result = result;
        return GZK_OK;
    }

    int gzk_matrix_horner(gzk_ctx* ctx, const gzk_buf* matrix, size_t rows, size_t cols, const uint8_t x_bytes[32], uint8_t out[32])
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (x_bytes == nullptr || out == nullptr) return fail(ctx, GZK_E_INVALID, "matrix_horner: null argument");
        const uint64_t total = static_cast<uint64_t>(rows) * cols;
        if (total == 0)
        {
            std::memset(out, 0, 32);  // matrix_row_major_evaluation returns zero for an empty matrix
            return GZK_OK;
        }
        if (matrix == nullptr || matrix->count < total) return fail(ctx, GZK_E_INVALID, "matrix_horner: matrix buffer too small");
        Fr x;
        int rc = scalar_mont(ctx, x_bytes, &x);
        if (rc != GZK_OK) return rc;
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        Fr* result = nullptr;
        if ((rc = matrix_horner_enqueue(ctx, matrix, total, x, nullptr, false, &result)) != GZK_OK) return rc;
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(out, result, 32, cudaMemcpyDeviceToHost, ctx->stream));
        GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        return GZK_OK;
    }

    // Same evaluation, left on the device in out[out_offset] (canonical for an FR buffer, Montgomery
    // for an FR_MONT one); nothing is read back.
    int gzk_matrix_horner_device(gzk_ctx* ctx, const gzk_buf* matrix, size_t rows, size_t cols, const uint8_t x_bytes[32], gzk_buf* out,
                                 size_t out_offset)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (x_bytes == nullptr || out == nullptr) return fail(ctx, GZK_E_INVALID, "matrix_horner_device: null argument");
        if ((out->kind != GZK_KIND_FR && out->kind != GZK_KIND_FR_MONT) || out_offset >= out->count)
            return fail(ctx, GZK_E_INVALID, "matrix_horner_device: output must be an FR or FR_MONT buffer that holds out_offset");
        const uint64_t total = static_cast<uint64_t>(rows) * cols;
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        Fr* dest = static_cast<Fr*>(out->dptr) + out_offset;
        if (total == 0)
        {
            GZK_CUDA_TRY(ctx, cudaMemsetAsync(dest, 0, sizeof(Fr), ctx->stream));
            return GZK_OK;
        }
        if (matrix == nullptr || matrix->count < total) return fail(ctx, GZK_E_INVALID, "matrix_horner_device: matrix buffer too small");
        Fr x;
        int rc = scalar_mont(ctx, x_bytes, &x);
        if (rc != GZK_OK) return rc;
        if ((rc = matrix_horner_enqueue(ctx, matrix, total, x, dest, out->kind == GZK_KIND_FR_MONT, nullptr)) != GZK_OK) return rc;
        return finish_call(ctx, "invalid input");
    }

    int gzk_fold_rows(gzk_ctx* ctx, const gzk_buf* matrix, size_t rows, size_t cols, const gzk_buf* row_weights, size_t row_count,
                      gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (cols == 0 || rows == 0) return GZK_OK;  // weighted_column_sum_native returns {} for an empty matrix
        if (matrix == nullptr || row_weights == nullptr || out == nullptr) return fail(ctx, GZK_E_INVALID, "fold_rows: null argument");
        if (row_count > rows || row_count > row_weights->count || matrix->count < static_cast<uint64_t>(rows) * cols)
            return fail(ctx, GZK_E_INVALID, "weighted column sum native input size mismatch");
        if (row_weights->kind != GZK_KIND_FR_MONT) return fail(ctx, GZK_E_INVALID, "fold_rows: weights must be a Montgomery buffer");
        if (out->kind != GZK_KIND_FR || out->count < cols) return fail(ctx, GZK_E_INVALID, "fold_rows: output must be an FR buffer of cols elements");
        if (cols > (1u << 24)) return fail(ctx, GZK_E_INVALID, "fold_rows: too many columns");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        if (matrix->kind == GZK_KIND_I64 && cols % 8 == 0 && static_cast<uint64_t>(row_count) * cols >= 65536)
        {
            // small-integer entries, eight adjacent columns to a unit: the byte products on the tensor cores (eval.cu)
            uint64_t unit_rows = 0;
            const uint32_t unit_tiles = fold_rows_groups_tiles(ctx, row_count, static_cast<uint32_t>(cols), &unit_rows);
            void* sums = nullptr;
            int rc = ensure_scratch(ctx, 1, static_cast<size_t>(unit_tiles) * cols * kAccLimbs * sizeof(uint32_t), &sums);
            if (rc != GZK_OK) return rc;
            {
                LaunchScope scope(ctx, "fold_rows");
                launch_fold_rows_groups(ctx, matrix->dptr, static_cast<const Fr*>(row_weights->dptr), row_count, static_cast<uint32_t>(cols), unit_rows, unit_tiles,
                                        static_cast<uint32_t*>(sums));
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            if ((rc = launch_eval_finish(ctx, static_cast<const uint32_t*>(sums), GZK_KIND_FR, unit_tiles, static_cast<uint32_t>(cols), static_cast<Fr*>(out->dptr), false)) != GZK_OK)
                return rc;
            return finish_call(ctx, "invalid input");
        }
        const uint32_t col_chunks = static_cast<uint32_t>((cols + kThreads - 1) / kThreads);
        const uint32_t width = cols < kThreads ? static_cast<uint32_t>(cols) : kThreads;
        const uint32_t row_lanes = kThreads / width;
        // Enough tiles to fill the machine, each tile at least 8 rows per row lane: a whole number of rounds of the
        // CTAs that are resident at once (two rounds), so that the last round is not a partly filled one.
        const size_t smem = static_cast<size_t>(kThreads) * kAccLimbs * sizeof(uint32_t);
        int resident = 0;
        switch (entry_kind(matrix->kind))
        {
        case GZK_KIND_I64: cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, fold_rows_kernel<GZK_KIND_I64>, kThreads, smem); break;
        case GZK_KIND_U32: cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, fold_rows_kernel<GZK_KIND_U32>, kThreads, smem); break;
        default: cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, fold_rows_kernel<GZK_KIND_FR>, kThreads, smem); break;
        }
        if (resident < 1) resident = 2;
        uint64_t tiles = static_cast<uint64_t>(ctx->sm_count) * static_cast<uint64_t>(resident) * 2 / col_chunks;
        const uint64_t max_tiles = (row_count + 8ull * row_lanes - 1) / (8ull * row_lanes);
        if (tiles > max_tiles) tiles = max_tiles;
        if (tiles > 1024) tiles = 1024;
        if (tiles == 0) tiles = 1;
        const uint64_t tile_rows = (row_count + tiles - 1) / tiles > 0 ? (row_count + tiles - 1) / tiles : 1;
        tiles = row_count == 0 ? 1 : (row_count + tile_rows - 1) / tile_rows;
        void* scratch = nullptr;
        int rc = ensure_scratch(ctx, 1, tiles * cols * kAccLimbs * sizeof(uint32_t), &scratch);
        if (rc != GZK_OK) return rc;
        ColRef m;
        m.ptr = matrix->dptr;
        m.kind = matrix->kind;
        {
            LaunchScope scope(ctx, "fold_rows");
            const unsigned grid = static_cast<unsigned>(tiles * col_chunks);
            const Fr* w = static_cast<const Fr*>(row_weights->dptr);
            uint32_t* partial = static_cast<uint32_t*>(scratch);
            switch (entry_kind(matrix->kind))
            {
            case GZK_KIND_I64:
                fold_rows_kernel<GZK_KIND_I64><<<grid, kThreads, smem, ctx->stream>>>(m.ptr, w, row_count, static_cast<uint32_t>(cols), tile_rows, col_chunks, partial);
                break;
            case GZK_KIND_U32:
                fold_rows_kernel<GZK_KIND_U32><<<grid, kThreads, smem, ctx->stream>>>(m.ptr, w, row_count, static_cast<uint32_t>(cols), tile_rows, col_chunks, partial);
                break;
            default:
                fold_rows_kernel<GZK_KIND_FR><<<grid, kThreads, smem, ctx->stream>>>(m.ptr, w, row_count, static_cast<uint32_t>(cols), tile_rows, col_chunks, partial);
                break;
            }
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        const int form = matrix->kind == GZK_KIND_FR_MONT ? GZK_KIND_FR_MONT : GZK_KIND_FR;  // small integers count as canonical values
        if ((rc = launch_eval_finish(ctx, static_cast<const uint32_t*>(scratch), form, static_cast<uint32_t>(tiles),
                                     static_cast<uint32_t>(cols), static_cast<Fr*>(out->dptr), false)) != GZK_OK)
            return rc;
        return finish_call(ctx, "invalid input");
    }

    int gzk_linear_form_rows(gzk_ctx* ctx, const gzk_buf* matrix, size_t rows, size_t cols, const gzk_buf* column_powers, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (rows == 0) return GZK_OK;
        if (matrix == nullptr || column_powers == nullptr || out == nullptr) return fail(ctx, GZK_E_INVALID, "linear_form_rows: null argument");
        if (matrix->count < static_cast<uint64_t>(rows) * cols || column_powers->count < cols)
            return fail(ctx, GZK_E_INVALID, "linear_form_rows: input size mismatch");
        if (column_powers->kind != GZK_KIND_FR_MONT) return fail(ctx, GZK_E_INVALID, "linear_form_rows: powers must be a Montgomery buffer");
        if (out->kind != GZK_KIND_FR_MONT || out->count < rows) return fail(ctx, GZK_E_INVALID, "linear_form_rows: output must be a Montgomery buffer of rows elements");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        ColRef m;
        m.ptr = matrix->dptr;
        m.kind = matrix->kind;
        const uint64_t warps_per_cta = kThreads / 32;
        const uint64_t ctas = (rows + warps_per_cta - 1) / warps_per_cta;
        void* bias_scratch = nullptr;
        {
            const int rc_scratch = ensure_scratch(ctx, 2, 2 * sizeof(Fr), &bias_scratch);
            if (rc_scratch != GZK_OK) return rc_scratch;
        }
        Fr* bias = static_cast<Fr*>(bias_scratch);
        {
            LaunchScope scope(ctx, "linear_form");
            const unsigned grid = static_cast<unsigned>(ctas);
            const Fr* powers = static_cast<const Fr*>(column_powers->dptr);
            const int mont = matrix->kind == GZK_KIND_FR_MONT ? 1 : 0;
            Fr* dst = static_cast<Fr*>(out->dptr);
            // a thread per row once the rows fill the machine that way (a warp per row below that)
            const bool by_thread = rows >= static_cast<uint64_t>(ctx->sm_count) * kRowThreads * 2;
            const unsigned row_ctas = static_cast<unsigned>((rows + kRowThreads - 1) / kRowThreads);
            switch (entry_kind(matrix->kind))
            {
            case GZK_KIND_I64:
                if (by_thread && cols % 4 == 0 && cols <= 4096)
                {
                    // tall matrices: the byte products on the tensor cores (eval.cu); entries enter as v + 2^63
                    void* table = nullptr;
                    const int rc_table = ensure_scratch(ctx, 1, cols * 256, &table);
                    if (rc_table != GZK_OK) return rc_table;
                    scaled_sum_kernel<<<1, kThreads, 0, ctx->stream>>>(powers, static_cast<uint32_t>(cols), mont_two_63(), bias);
                    launch_linear_form_tensor(ctx, m.ptr, rows, static_cast<uint32_t>(cols), static_cast<uint64_t>(rows) * cols, powers, table, bias, dst);
                    break;
                }
                // entries enter as v + 2^31: 2^31 * (sum of the powers) is taken off every row
                scaled_sum_kernel<<<1, kThreads, 0, ctx->stream>>>(powers, static_cast<uint32_t>(cols), mont_two_31(), bias);
                if (by_thread)
                    linear_form_by_thread_kernel<GZK_KIND_I64><<<row_ctas, kRowThreads, 0, ctx->stream>>>(m.ptr, powers, rows, static_cast<uint32_t>(cols), dst, bias);
                else
                    linear_form_kernel<GZK_KIND_I64><<<grid, kThreads, 0, ctx->stream>>>(m.ptr, mont, powers, rows, static_cast<uint32_t>(cols), dst, bias);
                break;
            case GZK_KIND_U32:
                if (by_thread)
                    linear_form_by_thread_kernel<GZK_KIND_U32><<<row_ctas, kRowThreads, 0, ctx->stream>>>(m.ptr, powers, rows, static_cast<uint32_t>(cols), dst, nullptr);
                else
                    linear_form_kernel<GZK_KIND_U32><<<grid, kThreads, 0, ctx->stream>>>(m.ptr, mont, powers, rows, static_cast<uint32_t>(cols), dst, nullptr);
                break;
            default:
                linear_form_kernel<GZK_KIND_FR><<<grid, kThreads, 0, ctx->stream>>>(m.ptr, mont, powers, rows, static_cast<uint32_t>(cols), dst, nullptr);
                break;
            }
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }

    int gzk_powers(gzk_ctx* ctx, const uint8_t challenge[32], size_t count, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (count == 0) return GZK_OK;
        if (challenge == nullptr || out == nullptr || out->kind != GZK_KIND_FR_MONT || out->count < count)
            return fail(ctx, GZK_E_INVALID, "powers: output must be a Montgomery buffer of count elements");
        Fr c;
        int rc = scalar_mont(ctx, challenge, &c);
        if (rc != GZK_OK) return rc;
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        {
            LaunchScope scope(ctx, "powers");
            powers_kernel<<<static_cast<unsigned>((count + 127) / 128), 128, 0, ctx->stream>>>(c, count, static_cast<Fr*>(out->dptr));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }
}
