// G1 multi-scalar multiplication sum_i [s_i] P_i by the bucket (Pippenger) method
// with signed-digit windows and XYZZ bucket accumulators.
//
//   1. digits     every scalar is cut into W signed c-bit digits; per (window, |digit|)
//                 bucket the number of hits is counted
//   2. offsets    exclusive scan of the bucket counts (one CTA)
//   3. scatter    (point index, sign) pairs are written bucket by bucket
//   4. buckets    one thread per bucket adds its points (mixed XYZZ additions)
//   5. bits       sum_d d*B_d of a bucket set: row and column sums of the buckets laid out as a
//                 matrix, then the two small weighted sums split by the bits of the multiplier
//   6. finish     per window Horner over the bits, shift by 2^(c*w), sum, to affine
//
// With a precomputed table of the points shifted by every window (gzk_msm_precompute:
// 2^(c*w) P_i for all w, the layout for a resident SRS) the digits of all windows fall
// into ONE set of 2^(c-1) buckets: no per-window reduction and no chain of c*w doublings
// at the end (254 dependent doublings cost 2.8 ms whatever the size), and the window can
// be wider because only one window's buckets are reduced.
//
// Signed digits halve the bucket count (2^(c-1) per window): a negative digit adds
// the negated point.  Group sums do not depend on the order of additions, so the
// atomics of steps 1 and 3 leave the result bit-identical from run to run.
#include <cstdlib>
#include <cstring>

#include "block.cuh"
#include "g1.cuh"

namespace gzk
{
    namespace
    {
        constexpr int kThreads = 128;
        constexpr int kMaxWindows = 32;
        // Buckets with more entries than kBigBucket (skewed scalars: small integers, constant
        // columns, the short top window) are cut into slices of kSliceEntries entries; one CTA
        // sums a slice, one thread then adds the slices of a bucket.
        constexpr uint32_t kBigBucket = 1024;
        constexpr uint32_t kSliceEntries = 2048;

        struct BigItem
        {
            uint32_t bucket;
            uint32_t slice;
        };
        struct BigBucket
        {
            uint32_t bucket;
            uint32_t first_item;
            uint32_t slices;
        };

        struct MsmPlan
        {
            uint32_t c;        // window bits
            uint32_t windows;  // ceil(256 / c)
            uint32_t half;     // 2^(c-1) buckets per window
            uint32_t shared;   // 1: all windows share one bucket set and entries index the shifted-point table [w*n + i]
        };

        // code[w*n + i] = 0 for a zero digit, else ((|d|-1) << 1 | negative) + 1
        __global__ void __launch_bounds__(kThreads) msm_digits_kernel(ColRef scalars, uint64_t n, MsmPlan plan, uint32_t* code,
                                                                     uint32_t* bucket_count)
        {
            const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
            if (i >= n) return;
            Fr s = load_fr(static_cast<const Fr*>(scalars.ptr) + i);
            if (scalars.kind == GZK_KIND_FR_MONT) s = from_mont(s);
            uint32_t carry = 0;
            for (uint32_t w = 0; w < plan.windows; ++w)
            {
                const uint32_t bit = w * plan.c;
                uint32_t raw = 0;
                if (bit < 256)
                {
                    const uint32_t limb = bit >> 5, shift = bit & 31;
                    uint64_t two = s.l[limb];
                    if (limb + 1 < 8) two |= static_cast<uint64_t>(s.l[limb + 1]) << 32;
                    raw = static_cast<uint32_t>(two >> shift) & ((1u << plan.c) - 1u);
                }
                uint32_t d = raw + carry;
                uint32_t negative = 0;
                carry = 0;
                if (d > plan.half)
                {
                    d = (1u << plan.c) - d;
                    negative = 1;
                    carry = 1;
                }
                uint32_t out = 0;
                if (d != 0)
                {
                    out = (((d - 1) << 1) | negative) + 1;
                    atomicAdd(bucket_count + (plan.shared ? 0 : static_cast<uint64_t>(w) * plan.half) + (d - 1), 1u);
                }
                code[static_cast<uint64_t>(w) * n + i] = out;
            }
        }

        // exclusive scan of `count` uint32 values by one CTA (in place); also zeroes `cursor`
        __global__ void __launch_bounds__(1024) msm_offsets_kernel(uint32_t* values, uint32_t* cursor, uint32_t count)
        {
            __shared__ uint32_t warp_totals[32];
            __shared__ uint32_t carry_in;
            const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            if (threadIdx.x == 0) carry_in = 0;
            __syncthreads();
            for (uint32_t base = 0; base < count; base += 1024)
            {
                const uint32_t idx = base + threadIdx.x;
                const uint32_t v = idx < count ? values[idx] : 0;
                uint32_t incl = v;
#pragma unroll
                for (int offset = 1; offset < 32; offset <<= 1)
                {
                    const uint32_t up = __shfl_up_sync(0xffffffffu, incl, offset);
                    if (lane >= static_cast<uint32_t>(offset)) incl += up;
                }
                if (lane == 31) warp_totals[warp] = incl;
                __syncthreads();
                uint32_t warp_offset = 0;
                for (uint32_t w2 = 0; w2 < warp; ++w2) warp_offset += warp_totals[w2];
                const uint32_t start = carry_in;
                if (idx < count)
                {
                    values[idx] = start + warp_offset + incl - v;
                    cursor[idx] = 0;
                }
                __syncthreads();
                if (threadIdx.x == 1023) carry_in = start + warp_offset + incl;
                __syncthreads();
            }
        }

        __global__ void __launch_bounds__(kThreads) msm_scatter_kernel(const uint32_t* code, uint64_t n, MsmPlan plan,
                                                                      const uint32_t* bucket_start, uint32_t* cursor, uint32_t* entries)
        {
            const uint64_t total = n * plan.windows;
            const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
            for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride)
            {
                const uint32_t v = code[t];
                if (v == 0) continue;
                const uint64_t w = t / n;
                const uint64_t i = t - w * n;
                const uint32_t payload = v - 1;
                const uint64_t bucket = (plan.shared ? 0 : w * plan.half) + (payload >> 1);
                const uint32_t pos = atomicAdd(cursor + bucket, 1u);
                entries[bucket_start[bucket] + pos] = (static_cast<uint32_t>(plan.shared ? t : i) << 1) | (payload & 1u);
            }
        }

        __global__ void __launch_bounds__(kThreads) msm_buckets_kernel(const G1Affine* points, const uint32_t* bucket_start,
                                                                      const uint32_t* bucket_size, const uint32_t* entries,
                                                                      uint32_t buckets, G1Xyzz* out)
        {
            const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
            if (b >= buckets) return;
            const uint32_t start = bucket_start[b], size = bucket_size[b];
            if (size > kBigBucket) return;  // handled cooperatively by msm_big_slices_kernel
            G1Xyzz acc = G1Xyzz::infinity();
#pragma unroll 1
            for (uint32_t k = 0; k < size; ++k)
            {
                const uint32_t e = entries[start + k];
                acc = g1_add_mixed(acc, load_affine(points + (e >> 1)), (e & 1u) != 0);
            }
            store_xyzz(out + b, acc);
        }

        // counters[0] = number of slice items, counters[1] = number of big buckets
        __global__ void __launch_bounds__(kThreads) msm_plan_big_kernel(const uint32_t* bucket_size, uint32_t buckets, uint32_t* counters,
                                                                       BigItem* items, BigBucket* big)
        {
            const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
            if (b >= buckets) return;
            const uint32_t size = bucket_size[b];
            if (size <= kBigBucket) return;
            const uint32_t slices = (size + kSliceEntries - 1) / kSliceEntries;
            const uint32_t first = atomicAdd(counters, slices);
            const uint32_t slot = atomicAdd(counters + 1, 1u);
            BigBucket bb;
            bb.bucket = b;
            bb.first_item = first;
            bb.slices = slices;
            big[slot] = bb;
            for (uint32_t j = 0; j < slices; ++j)
            {
                BigItem it;
                it.bucket = b;
                it.slice = j;
                items[first + j] = it;
            }
        }

        // CTA per slice item: the threads stride over the slice, then a shared-memory tree
        __global__ void __launch_bounds__(kThreads) msm_big_slices_kernel(const G1Affine* points, const uint32_t* bucket_start,
                                                                         const uint32_t* bucket_size, const uint32_t* entries,
                                                                         const uint32_t* counters, const BigItem* items, G1Xyzz* partial)
        {
            __shared__ G1Xyzz slots[kThreads];
            if (blockIdx.x >= counters[0]) return;
            const BigItem it = items[blockIdx.x];
            const uint32_t start = bucket_start[it.bucket], size = bucket_size[it.bucket];
            const uint32_t begin = it.slice * kSliceEntries;
            const uint32_t end = begin + kSliceEntries < size ? begin + kSliceEntries : size;
            G1Xyzz acc = G1Xyzz::infinity();
#pragma unroll 1
            for (uint32_t k = begin + threadIdx.x; k < end; k += kThreads)
            {
                const uint32_t e = entries[start + k];
                acc = g1_add_mixed(acc, load_affine(points + (e >> 1)), (e & 1u) != 0);
            }
            slots[threadIdx.x] = acc;
            __syncthreads();
            for (uint32_t offset = kThreads / 2; offset > 0; offset >>= 1)
            {
                if (threadIdx.x < offset) slots[threadIdx.x] = g1_add(slots[threadIdx.x], slots[threadIdx.x + offset]);
                __syncthreads();
            }
            if (threadIdx.x == 0) store_xyzz(partial + blockIdx.x, slots[0]);
        }

        // CTA per big bucket: the threads stride over its slice partials, then a tree
        __global__ void __launch_bounds__(kThreads) msm_big_combine_kernel(const uint32_t* counters, const BigBucket* big, const G1Xyzz* partial,
                                                                          G1Xyzz* out)
        {
            __shared__ G1Xyzz slots[kThreads];
            if (blockIdx.x >= counters[1]) return;
            const BigBucket bb = big[blockIdx.x];
            G1Xyzz acc = G1Xyzz::infinity();
            for (uint32_t j = threadIdx.x; j < bb.slices; j += kThreads) acc = g1_add(acc, load_xyzz(partial + bb.first_item + j));
            slots[threadIdx.x] = acc;
            __syncthreads();
            for (uint32_t offset = kThreads / 2; offset > 0; offset >>= 1)
            {
                if (threadIdx.x < offset) slots[threadIdx.x] = g1_add(slots[threadIdx.x], slots[threadIdx.x + offset]);
                __syncthreads();
            }
            if (threadIdx.x == 0) store_xyzz(out + bb.bucket, slots[0]);
        }

        // one thread per window, then a tree over the windows; thread 0 converts to affine
        __global__ void __launch_bounds__(kMaxWindows) msm_finish_kernel(const G1Xyzz* bit_sums, MsmPlan plan, G1Xyzz* out_xyzz,
                                                                        G1Affine* out_canonical)
        {
            __shared__ G1Xyzz slots[kMaxWindows];
            const uint32_t w = threadIdx.x;
            G1Xyzz acc = G1Xyzz::infinity();
            if (w < plan.windows)
            {
                for (int bit = static_cast<int>(plan.c) - 1; bit >= 0; --bit)
                {
                    acc = g1_double(acc);
                    acc = g1_add(acc, load_xyzz(bit_sums + w * plan.c + bit));
                }
                for (uint32_t k = 0; k < w * plan.c; ++k) acc = g1_double(acc);
            }
            slots[w] = acc;
            __syncthreads();
            for (uint32_t offset = kMaxWindows / 2; offset > 0; offset >>= 1)
            {
                if (w < offset) slots[w] = g1_add(slots[w], slots[w + offset]);
                __syncthreads();
            }
            if (w == 0)
            {
                store_xyzz(out_xyzz, slots[0]);
                G1Affine a = g1_to_affine(slots[0]);
                a.x = from_mont(a.x);
                a.y = from_mont(a.y);
                store_affine(out_canonical, a);
            }
        }

        // ---- shared-bucket path: reduction of ONE bucket set -----------------------------------
        // sum_d d * B_d over d = 1 .. 2^(c-1) (B_d = bucket d-1).  Write d = hi * 2^h + lo and lay the
        // buckets out as a matrix [hi][lo]: with the row sums R_hi and the column sums C_lo,
        //   sum_d d * B_d = sum_lo lo * C_lo + 2^h * sum_hi hi * R_hi,
        // so the bulk of the work is 2 additions per bucket in short independent trees, and the
        // two weighted sums run over 2^h and 2^(c-1-h)+1 points only; those are split by the bits
        // of the multiplier: bit_sums[b] for b < h from the columns, for b >= h from the rows,
        // and sum_b 2^b * bit_sums[b] is the result.
        __device__ __forceinline__ G1Xyzz cta_tree_sum(G1Xyzz acc, G1Xyzz* slots)
        {
            slots[threadIdx.x] = acc;
            __syncthreads();
            for (uint32_t offset = kThreads / 2; offset > 0; offset >>= 1)
            {
                if (threadIdx.x < offset) slots[threadIdx.x] = g1_add(slots[threadIdx.x], slots[threadIdx.x + offset]);
                __syncthreads();
            }
            return slots[0];
        }
        // CTAs [0, rows): row sums; CTAs [rows, rows + cols): column sums.  rc = [rows row sums][cols column sums]
        // (blockIdx.y = window when every window has its own bucket set)
        __global__ void __launch_bounds__(kThreads) msm_rowcol_kernel(const G1Xyzz* buckets, uint32_t half, uint32_t h, uint32_t rows, G1Xyzz* rc)
        {
            __shared__ G1Xyzz slots[kThreads];
            const uint32_t cols = 1u << h;
            buckets += static_cast<uint64_t>(blockIdx.y) * half;
            rc += static_cast<uint64_t>(blockIdx.y) * (rows + cols);
            G1Xyzz acc = G1Xyzz::infinity();
            if (blockIdx.x < rows)
            {
                const uint32_t hi = blockIdx.x;
                for (uint32_t lo = threadIdx.x; lo < cols; lo += kThreads)
                {
                    const uint32_t d = (hi << h) | lo;
                    if (d >= 1 && d <= half) acc = g1_add(acc, load_xyzz(buckets + (d - 1)));
                }
            }
            else
            {
                const uint32_t lo = blockIdx.x - rows;
                for (uint32_t hi = threadIdx.x; hi < rows; hi += kThreads)
                {
                    const uint32_t d = (hi << h) | lo;
                    if (d >= 1 && d <= half) acc = g1_add(acc, load_xyzz(buckets + (d - 1)));
                }
            }
            const G1Xyzz total = cta_tree_sum(acc, slots);
            if (threadIdx.x == 0) store_xyzz(rc + blockIdx.x, total);
        }
        // CTA b < h: sum of the column sums whose lo has bit b; CTA b >= h: sum of the row sums whose hi has bit b - h
        __global__ void __launch_bounds__(kThreads) msm_rowcol_bits_kernel(const G1Xyzz* rc, uint32_t h, uint32_t rows, G1Xyzz* bit_sums)
        {
            __shared__ G1Xyzz slots[kThreads];
            const uint32_t b = blockIdx.x;
            rc += static_cast<uint64_t>(blockIdx.y) * (rows + (1u << h));
            bit_sums += static_cast<uint64_t>(blockIdx.y) * gridDim.x;
            const bool from_cols = b < h;
            const uint32_t count = from_cols ? (1u << h) : rows;
            const uint32_t bit = from_cols ? b : b - h;
            const G1Xyzz* src = from_cols ? rc + rows : rc;
            G1Xyzz acc = G1Xyzz::infinity();
            for (uint32_t j = threadIdx.x; j < count; j += kThreads)
                if ((j >> bit) & 1u) acc = g1_add(acc, load_xyzz(src + j));
            const G1Xyzz total = cta_tree_sum(acc, slots);
            if (threadIdx.x == 0) store_xyzz(bit_sums + b, total);
        }
        // thread b shifts the sum of bit b by b doublings (at most c - 1), then a tree; thread 0 converts to affine
        __global__ void __launch_bounds__(kMaxWindows) msm_finish_shared_kernel(const G1Xyzz* bit_sums, uint32_t c, G1Xyzz* out_xyzz, G1Affine* out_canonical)
        {
            __shared__ G1Xyzz slots[kMaxWindows];
            const uint32_t b = threadIdx.x;
            G1Xyzz acc = G1Xyzz::infinity();
            if (b < c)
            {
                acc = load_xyzz(bit_sums + b);
                for (uint32_t k = 0; k < b; ++k) acc = g1_double(acc);
            }
            slots[b] = acc;
            __syncthreads();
            for (uint32_t offset = kMaxWindows / 2; offset > 0; offset >>= 1)
            {
                if (b < offset) slots[b] = g1_add(slots[b], slots[b + offset]);
                __syncthreads();
            }
            if (b == 0)
            {
                store_xyzz(out_xyzz, slots[0]);
                G1Affine a = g1_to_affine(slots[0]);
                a.x = from_mont(a.x);
                a.y = from_mont(a.y);
                store_affine(out_canonical, a);
            }
        }

        // next[i] = 2^c * prev[i] (affine Montgomery in and out; one inversion per point, all in parallel)
        __global__ void __launch_bounds__(kThreads) msm_table_window_kernel(const G1Affine* prev, G1Affine* next, uint64_t n, uint32_t c)
        {
            const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
            if (i >= n) return;
            const G1Affine p = load_affine(prev + i);
            if (p.is_infinity())
            {
                store_affine(next + i, p);
                return;
            }
            G1Xyzz acc = G1Xyzz::from_affine(p);
#pragma unroll 1
            for (uint32_t k = 0; k < c; ++k) acc = g1_double(acc);
            store_affine(next + i, g1_to_affine(acc));
        }

        // Windows needed for scalars below the group order r: ceil(255 / c), plus one when the top
        // digit could still reach 2^(c-1) and push a carry out.
        uint32_t windows_for(uint32_t c)
        {
            uint32_t windows = (255 + c - 1) / c;
            const uint32_t top_shift = c * (windows - 1);
            // largest top digit = (r - 1) >> top_shift, from the modulus limbs
            uint64_t top = 0;
            for (int limb = 7; limb >= 0; --limb)
            {
                const uint32_t lo_bit = 32u * static_cast<uint32_t>(limb);
                if (lo_bit + 32 <= top_shift) break;
                const uint64_t word = FrCfg::mod(limb);
                if (lo_bit >= top_shift)
                    top |= word << (lo_bit - top_shift);
                else
                    top |= word >> (top_shift - lo_bit);
            }
            if (top + 1 > (1ULL << (c - 1))) ++windows;  // top digit + incoming carry may exceed the signed range
            return windows;
        }

        MsmPlan make_shared_plan(uint32_t c)
        {
            MsmPlan p;
            p.c = c;
            p.windows = windows_for(c);
            p.half = 1u << (c - 1);
            p.shared = 1;
            return p;
        }

        MsmPlan make_plan(uint64_t n)
        {
            uint32_t log2n = 0;
            while ((1ULL << (log2n + 1)) <= n) ++log2n;
            // larger windows mean fewer mixed additions (n per window) but 2^(c-1) * c / 2 full
            // additions per window in the bit-split reduction; log2(n) - 7 balances the two
            int c = static_cast<int>(log2n) - 6;
#ifdef GZK_BUILD_TUNING
            if (const char* forced = std::getenv("GZK_MSM_WINDOW")) c = std::atoi(forced);
#endif
            if (c < 8) c = 8;
            if (c > 16) c = 16;
            MsmPlan p;
            p.c = static_cast<uint32_t>(c);
            p.windows = (256 + p.c - 1) / p.c;
            p.half = 1u << (p.c - 1);
            p.shared = 0;
            return p;
        }
    }

    // MSM over device-resident scalars and points; the XYZZ result is left in
    // `out_xyzz` (device, optional use by multi-GPU combiners) and the canonical
    // affine result is copied to `out_host`.
    static int msm_run_plan(gzk_ctx* ctx, const gzk_buf* scalars, const gzk_buf* points, uint64_t n, const MsmPlan& plan, uint8_t out_host[96])
    {
        const uint64_t buckets = plan.shared ? plan.half : static_cast<uint64_t>(plan.windows) * plan.half;
        const size_t code_bytes = static_cast<size_t>(n) * plan.windows * sizeof(uint32_t);
        const size_t bucket_u32 = buckets * sizeof(uint32_t);
        const uint64_t total_entries = n * plan.windows;
        const uint64_t max_big = total_entries / kBigBucket + 1;          // buckets that can exceed the threshold
        const uint64_t max_items = total_entries / kSliceEntries + max_big; // sum of ceil(size / slice) over them
        const size_t big_bytes = max_items * (sizeof(BigItem) + sizeof(G1Xyzz)) + max_big * sizeof(BigBucket) + 64;
        const uint32_t split_h = (plan.c - 1) / 2;                          // low bits of the bucket multiplier
        const uint32_t split_rows = (1u << (plan.c - 1 - split_h)) + 1;     // values of the high part, 0 .. 2^(c-1-h)
        const uint32_t bucket_sets = plan.shared ? 1u : plan.windows;
        const size_t chunk_bytes = static_cast<size_t>(bucket_sets) * (static_cast<size_t>(split_rows) + (1u << split_h)) * sizeof(G1Xyzz);
        const size_t total = big_bytes + 2 * code_bytes + 3 * bucket_u32 + buckets * sizeof(G1Xyzz) + static_cast<size_t>(plan.windows) * plan.c * sizeof(G1Xyzz) +
                             chunk_bytes + sizeof(G1Xyzz) + sizeof(G1Affine) + 8192;
        void* scratch = nullptr;
        int rc = ensure_scratch(ctx, 1, total, &scratch);
        if (rc != GZK_OK) return rc;
        char* cur = static_cast<char*>(scratch);
        auto take = [&](size_t bytes) {
            char* p = cur;
            cur += (bytes + 255) & ~static_cast<size_t>(255);
            return p;
        };
        G1Xyzz* bucket_points = reinterpret_cast<G1Xyzz*>(take(buckets * sizeof(G1Xyzz)));
        G1Xyzz* bit_sums = reinterpret_cast<G1Xyzz*>(take(static_cast<size_t>(plan.windows) * plan.c * sizeof(G1Xyzz)));
        G1Xyzz* result_xyzz = reinterpret_cast<G1Xyzz*>(take(sizeof(G1Xyzz)));
        G1Affine* result_affine = reinterpret_cast<G1Affine*>(take(sizeof(G1Affine)));
        uint32_t* code = reinterpret_cast<uint32_t*>(take(code_bytes));
        uint32_t* entries = reinterpret_cast<uint32_t*>(take(code_bytes));
        uint32_t* bucket_size = reinterpret_cast<uint32_t*>(take(bucket_u32));
        uint32_t* bucket_start = reinterpret_cast<uint32_t*>(take(bucket_u32));
        uint32_t* cursor = reinterpret_cast<uint32_t*>(take(bucket_u32));
        G1Xyzz* big_partial = reinterpret_cast<G1Xyzz*>(take(max_items * sizeof(G1Xyzz)));
        BigItem* big_items = reinterpret_cast<BigItem*>(take(max_items * sizeof(BigItem)));
        BigBucket* big_buckets = reinterpret_cast<BigBucket*>(take(max_big * sizeof(BigBucket)));
        uint32_t* big_counters = reinterpret_cast<uint32_t*>(take(64));
        G1Xyzz* bit_partial = reinterpret_cast<G1Xyzz*>(take(chunk_bytes));
        if (static_cast<size_t>(cur - static_cast<char*>(scratch)) > ctx->scratch[1].bytes)
            return fail(ctx, GZK_E_INVALID, "msm: internal scratch accounting error");

        ColRef s;
        s.ptr = scalars->dptr;
        s.kind = scalars->kind;
        GZK_CUDA_TRY(ctx, cudaMemsetAsync(bucket_size, 0, bucket_u32, ctx->stream));
        {
            LaunchScope scope(ctx, "msm_digits");
            msm_digits_kernel<<<static_cast<unsigned>((n + kThreads - 1) / kThreads), kThreads, 0, ctx->stream>>>(s, n, plan, code, bucket_size);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(bucket_start, bucket_size, bucket_u32, cudaMemcpyDeviceToDevice, ctx->stream));
        {
            LaunchScope scope(ctx, "msm_offsets");
            msm_offsets_kernel<<<1, 1024, 0, ctx->stream>>>(bucket_start, cursor, static_cast<uint32_t>(buckets));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        {
            LaunchScope scope(ctx, "msm_scatter");
            const uint64_t work = n * plan.windows;
            uint64_t blocks = (work + kThreads - 1) / kThreads;
            const uint64_t cap = static_cast<uint64_t>(ctx->sm_count) * 32;
            if (blocks > cap) blocks = cap;
            msm_scatter_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, ctx->stream>>>(code, n, plan, bucket_start, cursor, entries);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        GZK_CUDA_TRY(ctx, cudaMemsetAsync(big_counters, 0, 64, ctx->stream));
        {
            LaunchScope scope(ctx, "msm_plan_big");
            msm_plan_big_kernel<<<static_cast<unsigned>((buckets + kThreads - 1) / kThreads), kThreads, 0, ctx->stream>>>(
                bucket_size, static_cast<uint32_t>(buckets), big_counters, big_items, big_buckets);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        {
            LaunchScope scope(ctx, "msm_buckets");
            msm_buckets_kernel<<<static_cast<unsigned>((buckets + kThreads - 1) / kThreads), kThreads, 0, ctx->stream>>>(
                static_cast<const G1Affine*>(points->dptr), bucket_start, bucket_size, entries, static_cast<uint32_t>(buckets), bucket_points);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        {
            // grids are upper bounds; CTAs beyond the counted work return at once
            LaunchScope scope(ctx, "msm_big_buckets", 2);
            msm_big_slices_kernel<<<static_cast<unsigned>(max_items), kThreads, 0, ctx->stream>>>(
                static_cast<const G1Affine*>(points->dptr), bucket_start, bucket_size, entries, big_counters, big_items, big_partial);
            msm_big_combine_kernel<<<static_cast<unsigned>(max_big), kThreads, 0, ctx->stream>>>(
                big_counters, big_buckets, big_partial, bucket_points);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        {
            LaunchScope scope(ctx, "msm_bits", 2);
            msm_rowcol_kernel<<<dim3(split_rows + (1u << split_h), bucket_sets), kThreads, 0, ctx->stream>>>(bucket_points, plan.half, split_h, split_rows,
                                                                                                    bit_partial);
            msm_rowcol_bits_kernel<<<dim3(plan.c, bucket_sets), kThreads, 0, ctx->stream>>>(bit_partial, split_h, split_rows, bit_sums);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        {
            LaunchScope scope(ctx, "msm_finish");
            if (plan.shared)
                msm_finish_shared_kernel<<<1, kMaxWindows, 0, ctx->stream>>>(bit_sums, plan.c, result_xyzz, result_affine);
            else
                msm_finish_kernel<<<1, kMaxWindows, 0, ctx->stream>>>(bit_sums, plan, result_xyzz, result_affine);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(out_host, result_affine, 96, cudaMemcpyDeviceToHost, ctx->stream));
        GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        return GZK_OK;
    }
}

namespace gzk
{
    int msm_run(gzk_ctx* ctx, const gzk_buf* scalars, const gzk_buf* points, uint64_t n, uint8_t out_host[96])
    {
        // Above 2^24 points the (point, window) list of one pass no longer fits the caches that the
        // counting sort and the bucket gathers live on (2^26 points in one pass run at a third of the rate
        // of 2^24): longer inputs are cut into ranges of 2^24 points and the range sums are added.
        constexpr uint64_t kRange = 1ULL << 24;
        if (n <= kRange) return msm_run_plan(ctx, scalars, points, n, make_plan(n), out_host);
        std::vector<uint8_t> partial;
        for (uint64_t first = 0; first < n; first += kRange)
        {
            const uint64_t count = n - first < kRange ? n - first : kRange;
            gzk_buf s_view = *scalars, p_view = *points;
            s_view.dptr = static_cast<char*>(scalars->dptr) + first * scalars->elem_bytes;
            s_view.count = count;
            s_view.owned = false;
            p_view.dptr = static_cast<char*>(points->dptr) + first * points->elem_bytes;
            p_view.count = count;
            p_view.owned = false;
            partial.resize(partial.size() + 96);
            const int rc = msm_run_plan(ctx, &s_view, &p_view, count, make_plan(count), partial.data() + partial.size() - 96);
            if (rc != GZK_OK) return rc;
        }
        if (gzk_g1_sum(partial.data(), partial.size() / 96, out_host) != GZK_OK) return fail(ctx, GZK_E_INVALID, "msm: range sums are not canonical points");
        return GZK_OK;
    }
}

using namespace gzk;

extern "C" unsigned gzk_msm_window_bits(size_t n)
{
    // Start from log2(n) - 3 (a few hundred entries per bucket, >= 2^15 buckets so that one bucket
    // set keeps every SM busy) and compare its neighbours by additions: n per window, 2 per bucket
    // for the reduction, and a surcharge when the top window is only a few bits wide (its handful
    // of buckets then take n / 2^bits points each and go through the slower cooperative path).
    unsigned log2n = 0;
    while ((static_cast<size_t>(1) << (log2n + 1)) <= n) ++log2n;
    int c0 = static_cast<int>(log2n) - 3;
    if (c0 < 16) c0 = 16;
    if (c0 > 23) c0 = 23;
    double best_cost = 0.0;
    unsigned best = static_cast<unsigned>(c0);
    for (int c = c0 - 1; c <= c0 + 1; ++c)
    {
        const uint32_t windows = windows_for(static_cast<uint32_t>(c));
        const uint32_t full = (255 + static_cast<uint32_t>(c) - 1) / static_cast<uint32_t>(c);
        const int top_bits = 255 - c * static_cast<int>(full - 1);
        // a window beyond ceil(255 / c) only receives the carries of the one below it: about n / 2 entries
        double cost = (static_cast<double>(full) + (windows > full ? 0.5 : 0.0)) * static_cast<double>(n) + 2.0 * static_cast<double>(1ULL << (c - 1));
        if (top_bits > 0 && top_bits < 12) cost += 1.5 * static_cast<double>(n);
        if (static_cast<double>(windows) * static_cast<double>(n) / static_cast<double>(1ULL << (c - 1)) > 768.0) cost += 4.0 * static_cast<double>(n);
        if (best_cost == 0.0 || cost < best_cost)
        {
            best_cost = cost;
            best = static_cast<unsigned>(c);
        }
    }
    return best;
}

extern "C" size_t gzk_msm_table_points(size_t n, unsigned window_bits)
{
    if (window_bits < 2 || window_bits > 24) return 0;
    return n * windows_for(window_bits);
}

extern "C" int gzk_msm_precompute(gzk_ctx* ctx, const gzk_buf* points, size_t n, unsigned window_bits, gzk_buf* table)
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (points == nullptr || table == nullptr || points->kind != GZK_KIND_G1 || table->kind != GZK_KIND_G1 || points->count < n)
        return fail(ctx, GZK_E_INVALID, "msm_precompute: points and table must be G1 buffers");
    if (window_bits < 8 || window_bits > 24) return fail(ctx, GZK_E_INVALID, "msm_precompute: window_bits must lie in [8, 24]");
    const uint32_t windows = windows_for(window_bits);
    if (table->count < n * windows || table->dptr == points->dptr) return fail(ctx, GZK_E_INVALID, "msm_precompute: table needs gzk_msm_table_points(n, window_bits) points of its own");
    if (n == 0) return GZK_OK;
    GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    G1Affine* t = static_cast<G1Affine*>(table->dptr);
    GZK_CUDA_TRY(ctx, cudaMemcpyAsync(t, points->dptr, n * sizeof(G1Affine), cudaMemcpyDeviceToDevice, ctx->stream));
    for (uint32_t w = 1; w < windows; ++w)
    {
        LaunchScope scope(ctx, "msm_table_window");
        msm_table_window_kernel<<<static_cast<unsigned>((n + kThreads - 1) / kThreads), kThreads, 0, ctx->stream>>>(t + static_cast<size_t>(w - 1) * n,
                                                                                                          t + static_cast<size_t>(w) * n, n, window_bits);
    }
    GZK_CUDA_TRY(ctx, cudaGetLastError());
    return finish_call(ctx, "invalid input");
}

extern "C" int gzk_msm_precomputed(gzk_ctx* ctx, const gzk_buf* scalars, const gzk_buf* table, size_t n, unsigned window_bits, uint8_t out[96])
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (out == nullptr) return fail(ctx, GZK_E_INVALID, "msm_precomputed: null output");
    if (n == 0)
    {
        std::memset(out, 0, 96);
        return GZK_OK;
    }
    if (scalars == nullptr || table == nullptr) return fail(ctx, GZK_E_INVALID, "msm_precomputed: null argument");
    if (window_bits < 8 || window_bits > 24) return fail(ctx, GZK_E_INVALID, "msm_precomputed: window_bits must lie in [8, 24]");
    if ((scalars->kind != GZK_KIND_FR && scalars->kind != GZK_KIND_FR_MONT) || scalars->count < n)
        return fail(ctx, GZK_E_INVALID, "msm_precomputed: scalars must be an FR or FR_MONT buffer of n elements");
    const MsmPlan plan = make_shared_plan(window_bits);
    if (table->kind != GZK_KIND_G1 || table->count < n * plan.windows) return fail(ctx, GZK_E_INVALID, "msm_precomputed: table does not hold gzk_msm_table_points(n, window_bits) points");
    if (n * plan.windows >= (1ULL << 31)) return fail(ctx, GZK_E_INVALID, "msm_precomputed: at most 2^31 - 1 table points per call");
    GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return msm_run_plan(ctx, scalars, table, n, plan, out);
}

extern "C" int gzk_msm(gzk_ctx* ctx, const gzk_buf* scalars, const gzk_buf* points, size_t n, uint8_t out[96])
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (out == nullptr) return fail(ctx, GZK_E_INVALID, "msm: null output");
    if (n == 0)
    {
        std::memset(out, 0, 96);
        return GZK_OK;
    }
    if (scalars == nullptr || points == nullptr) return fail(ctx, GZK_E_INVALID, "msm: null argument");
    if ((scalars->kind != GZK_KIND_FR && scalars->kind != GZK_KIND_FR_MONT) || scalars->count < n)
        return fail(ctx, GZK_E_INVALID, "msm: scalars must be an FR or FR_MONT buffer of n elements");
    if (points->kind != GZK_KIND_G1 || points->count < n) return fail(ctx, GZK_E_INVALID, "msm: points must be a G1 buffer of n elements");
    // the counting sort addresses n * windows (point, window) entries with 32-bit offsets
    if (n * make_plan(n).windows >= (1ULL << 31)) return fail(ctx, GZK_E_INVALID, "msm: at most 2^31 - 1 (point, window) entries per call (about 2^26 points); split the point range and add the results with gzk_g1_sum");
    GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return msm_run(ctx, scalars, points, n, out);
}
