// Running-sum column builders: LogUp accumulators, route accumulators, the
// inner-product (zkMaP / binding) accumulator and the segmented prefix states over
// the dst-sorted edge list.  All are "out = prefix sums of per-row terms"; the
// terms of the lookup arguments need one field inversion per row, done as one
// batch inversion for the whole column.
//
// Passes (no inter-CTA waiting anywhere, so nothing can spin):
//   main    per CTA of 512 rows: build the denominators, invert their product (each CTA
//           inverts its own when the whole grid is resident at once; very long columns
//           collect the CTA products in a first pass and invert them in one CTA), recover
//           each inverse from in-CTA prefix products, form the terms, scan them locally,
//           write the local running sums and the CTA aggregate
//   fix-up  elementwise: add the offset of the row's CTA (re-derived from the raw
//           aggregates by every fix-up CTA when there are at most 2048 of them, else
//           scanned by one CTA first), fill the tail with the total
// Operands enter the multiplier as they are stored (canonical or Montgomery) with the
// missing powers of R tracked per buffer kind, see "residues with a tracked power of R".
#include <cstring>

#include "block.cuh"

namespace gzk
{
    int launch_batch_invert_single_cta(gzk_ctx* ctx, Fr* values, Fr* tmp, uint32_t count);

    namespace
    {
        constexpr int kThreads = 128;
        constexpr int kElems = 4;
        constexpr int kChunk = kThreads * kElems;
        constexpr int kWarps = kThreads / 32;

        enum ScanOp
        {
            kLogup = 0,      // term = q_table*mult/(table+beta) - q_query/(query+beta)
            kRouteNode = 1,  // term = mult/(table+beta)
            kRouteEdge = 2,  // term = 1/(query+beta)
            kProduct = 3,    // term = a*b
            kSegmented = 4,  // term = value, running sum restarts where q_new = 1
            kLogupIndexed = 5,  // the LogUp term with every inverse fetched from a table of 1/(T_t+beta), see scan_main_body
            kRouteEdgeIndexed = 6,  // term = inv_table[index[e]]: the edge side of a route whose queries are gathered table rows
        };

        struct ScanArgs
        {
            ColRef c0, c1, c2, c3, c4;
            uint64_t count;  // rows that carry a term
            uint64_t n;      // length of the output column
            Fr beta;        // Montgomery form
            Fr beta_canon;  // the same challenge as a canonical residue
            Fr* out;
            Fr* cta_products;     // pass 1 -> 2 -> 3
            Fr* agg_value;        // per-CTA aggregate / exclusive offset
            uint32_t* agg_flag;
            uint32_t* agg_first;  // first row (CTA-relative) that starts a segment, kChunk if none
            Fr* total;            // grand total (Montgomery)
            int* status;
            // kLogupIndexed: c0 / c1 hold the integer query keys (x, y), c2 the multiplicities
            const Fr* inv_table;       // 1/(T_t + beta) for every table row t, Montgomery form
            const long long* table_y;  // second key column of the banded table (null: single-column table)
            uint64_t table_size;
            long long x_min;
            uint32_t band;
        };

        // ---- residues with a tracked power of R --------------------------------------------
        // A canonical residue x (kinds FR, U32, I64) is the Montgomery representation of
        // x/R, so it can enter a Montgomery product as it is stored, provided the missing
        // factors of R are counted: "deficit" below is that count (1 for canonical kinds, 0
        // for FR_MONT), a product adds the deficits of its factors, an inversion negates
        // them, and fix_scale() multiplies the remaining factors back in.  In the lookup
        // terms the deficits of numerator and denominator cancel, which saves the
        // conversion multiplication of every load.  All deficits depend only on the buffer
        // kinds, so every branch on them is uniform over the grid.
        // v carries `d` missing factors of R (d > 0) or -d surplus ones (d < 0).
        __device__ __forceinline__ Fr fix_scale(Fr v, int d)
        {
            for (; d > 0; --d) v = to_mont(v);
            for (; d < 0; ++d) v = from_mont(v);
            return v;
        }

        // the challenge in the form of column c
        __device__ __forceinline__ Fr beta_for(const ScanArgs& a, const ColRef& c) { return deficit(c) ? a.beta_canon : a.beta; }

        // 0 and 1 in the stored form of column c
        __device__ __forceinline__ bool stored_is_one(const ColRef& c, const Fr& v)
        {
            if (deficit(c) == 0) return v == Fr::one();
            return v.l[0] == 1u && (v.l[1] | v.l[2] | v.l[3] | v.l[4] | v.l[5] | v.l[6] | v.l[7]) == 0u;
        }

        // Denominator of row e in stored form; its deficit is deficit(c0) (+ deficit(c1) for LogUp).
        template <int OP>
        __device__ __forceinline__ Fr denominator(const ScanArgs& a, uint64_t e)
        {
            const Fr tb = add(col_load_stored(a.c0, e), beta_for(a, a.c0));
            if (OP == kLogup) return mul(tb, add(col_load_stored(a.c1, e), beta_for(a, a.c1)));
            return tb;
        }

        // inv_out[t] = 1/(table[t] + beta) in Montgomery form, t < count: the per-CTA batch inversion of the
        // main pass on its own (each CTA inverts the product of its 512 denominators).
        __global__ void __launch_bounds__(kThreads) shifted_inverse_kernel(ScanArgs a, Fr* inv_out)
        {
            __shared__ Fr slots[3 * kWarps];
            __shared__ Fr local_inverse;
            const uint64_t base = static_cast<uint64_t>(blockIdx.x) * kChunk + static_cast<uint64_t>(threadIdx.x) * kElems;
            Fr d[kElems], pre[kElems];
            Fr mine = Fr::one();
#pragma unroll
            for (int j = 0; j < kElems; ++j)
            {
                const uint64_t e = base + j;
                d[j] = e < a.count ? add(col_load_stored(a.c0, e), beta_for(a, a.c0)) : Fr::one();
                pre[j] = mine;
                mine = mul(mine, d[j]);
            }
            const Fr total = block_product<kThreads>(mine, slots);
            if (threadIdx.x == 0)
            {
                if (total.is_zero()) raise_status(a.status, GZK_E_DOMAIN, 1404);
                local_inverse = inv(total);
            }
            __syncthreads();
            Fr rest = block_invert_products<kThreads>(mine, local_inverse, slots);
#pragma unroll
            for (int j = kElems - 1; j >= 0; --j)
            {
                const uint64_t e = base + j;
                const Fr inverse = mul(rest, pre[j]);
                if (j > 0) rest = mul(rest, d[j]);
                if (e < a.count) store_fr(inv_out + e, fix_scale(inverse, -deficit(a.c0)));
            }
        }

        // LogUp rows with only one side switched on by its 0/1 selector (almost all of them: the table
        // fills the first rows of the column, the queries run on for millions more) need the inverse of
        // that side alone.  *side = 1 table only, 2 query only, 0 neither (denominator 1), 3 the general
        // two-sided term (also taken when a selector is neither 0 nor 1, and by the other operations).
        template <int OP>
        __device__ __forceinline__ Fr row_denominator(const ScanArgs& a, uint64_t e, int* side)
        {
            *side = 3;
            if (OP == kLogup)
            {
                const Fr sel_t = col_load_stored(a.c3, e), sel_q = col_load_stored(a.c4, e);
                const bool t_on = !sel_t.is_zero(), q_on = !sel_q.is_zero();
                const bool plain = (!t_on || stored_is_one(a.c3, sel_t)) && (!q_on || stored_is_one(a.c4, sel_q));
                if (plain) *side = (t_on ? 1 : 0) | (q_on ? 2 : 0);
                if (*side == 0) return Fr::one();
                if (*side == 1) return add(col_load_stored(a.c0, e), beta_for(a, a.c0));
                if (*side == 2) return add(col_load_stored(a.c1, e), beta_for(a, a.c1));
            }
            return denominator<OP>(a, e);
        }

        template <int OP>
        __global__ void __launch_bounds__(kThreads) scan_products_kernel(ScanArgs a)
        {
            __shared__ Fr slots[kWarps];
            const uint64_t base = static_cast<uint64_t>(blockIdx.x) * kChunk + static_cast<uint64_t>(threadIdx.x) * kElems;
            Fr prod = Fr::one();
#pragma unroll
            for (int j = 0; j < kElems; ++j)
            {
                const uint64_t e = base + j;
                if (e < a.count)
                {
                    int side;
                    const Fr d = row_denominator<OP>(a, e, &side);
                    if (d.is_zero()) raise_status(a.status, GZK_E_DOMAIN, 1401);
                    prod = mul(prod, d);
                }
            }
            const Fr total = block_product<kThreads>(prod, slots);
            if (threadIdx.x == 0) store_fr(a.cta_products + blockIdx.x, total);
        }

        // LOCAL_INV: the CTA inverts the product of its own 1024 denominators (one serial
        // inversion per CTA, all CTAs in parallel) instead of reading the result of the
        // product / single-CTA-inversion passes; used when the whole grid is resident at once.
        // Shared memory of one CTA of the main pass (the batched kernel shares one copy between its ops).
        struct MainShared
        {
            Fr slots[3 * kWarps];
            Fr local_inverse;
            SegVal seg_slots[kWarps];
            uint32_t first_flag;
        };

        // `block`: index of the CTA within its own job (blockIdx.x for a single-job launch).
        template <int OP, bool LOCAL_INV>
        __device__ __forceinline__ void scan_main_body(const ScanArgs& a, uint32_t block, MainShared& sh)
        {
            Fr* slots = sh.slots;
            Fr& local_inverse = sh.local_inverse;
            SegVal* seg_slots = sh.seg_slots;
            uint32_t& first_flag = sh.first_flag;
            const uint64_t base = static_cast<uint64_t>(block) * kChunk + static_cast<uint64_t>(threadIdx.x) * kElems;
            if (threadIdx.x == 0) first_flag = kChunk;
            __syncthreads();

            Fr term[kElems];
            uint32_t flag[kElems];
#pragma unroll
            for (int j = 0; j < kElems; ++j) flag[j] = 0;

            if (OP == kLogup || OP == kRouteNode || OP == kRouteEdge)
            {
                Fr d[kElems], pre[kElems];
                int side[kElems];
                Fr mine = Fr::one();
#pragma unroll
                for (int j = 0; j < kElems; ++j)
                {
                    const uint64_t e = base + j;
                    side[j] = 3;
                    d[j] = e < a.count ? row_denominator<OP>(a, e, &side[j]) : Fr::one();
                    pre[j] = mine;
                    mine = mul(mine, d[j]);
                }
                Fr cta_inverse;
                if (LOCAL_INV)
                {
                    const Fr total = block_product<kThreads>(mine, slots);
                    if (threadIdx.x == 0)
                    {
                        if (total.is_zero()) raise_status(a.status, GZK_E_DOMAIN, 1402);
                        local_inverse = inv(total);
                    }
                    __syncthreads();
                    cta_inverse = local_inverse;
                }
                else
                {
                    cta_inverse = load_fr(a.cta_products + block);
                }
                const Fr outer = block_invert_products<kThreads>(mine, cta_inverse, slots);
                Fr rest = outer;  // inverse of the product of the thread's rows 0 .. j
#pragma unroll
                for (int j = kElems - 1; j >= 0; --j)
                {
                    const uint64_t e = base + j;
                    const Fr inverse = mul(rest, pre[j]);
                    if (j > 0) rest = mul(rest, d[j]);
                    if (e >= a.count)
                    {
                        term[j] = Fr::zero();
                    }
                    else if (OP == kLogup && side[j] == 0)
                    {
                        term[j] = Fr::zero();
                    }
                    else if (OP == kLogup && side[j] == 1)
                    {
                        // inverse = R^d0/(T+b); the selector is one, so the weight is the multiplicity itself
                        term[j] = fix_scale(mul(col_load_stored(a.c2, e), inverse), deficit(a.c2) - deficit(a.c0));
                    }
                    else if (OP == kLogup && side[j] == 2)
                    {
                        // inverse = R^d1/(Q+b), the selector is one: the term is -1/(Q+b)
                        term[j] = sub(Fr::zero(), fix_scale(inverse, -deficit(a.c1)));
                    }
                    else if (OP == kLogup)
                    {
                        // inverse = 1/((T+b)(Q+b)) with the surplus R^(d0+d1): inverse*(Q+b) = R^d0/(T+b),
                        // inverse*(T+b) = R^d1/(Q+b)
                        const int d0 = deficit(a.c0), d1 = deficit(a.c1);
                        const Fr tb = add(col_load_stored(a.c0, e), beta_for(a, a.c0));
                        const Fr qb = add(col_load_stored(a.c1, e), beta_for(a, a.c1));
                        Fr weight = col_load_stored(a.c2, e);       // multiplicity, deficit d2
                        const Fr sel = col_load_stored(a.c3, e);    // table selector
                        if (sel.is_zero())
                            weight = Fr::zero();
                        else if (!stored_is_one(a.c3, sel))
                            weight = fix_scale(mul(weight, sel), deficit(a.c3));  // back to deficit d2
                        const Fr table_term = fix_scale(mul(weight, mul(inverse, qb)), deficit(a.c2) - d0);
                        const Fr query_term = fix_scale(mul(col_load_stored(a.c4, e), mul(inverse, tb)), deficit(a.c4) - d1);
                        term[j] = sub(table_term, query_term);
                    }
                    else if (OP == kRouteNode)
                    {
                        term[j] = fix_scale(mul(col_load_stored(a.c1, e), inverse), deficit(a.c1) - deficit(a.c0));
                    }
                    else
                    {
                        term[j] = fix_scale(inverse, -deficit(a.c0));
                    }
                }
            }
            else
            {
#pragma unroll
                for (int j = 0; j < kElems; ++j)
                {
                    const uint64_t e = base + j;
                    if (e >= a.count)
                    {
                        term[j] = Fr::zero();
                    }
                    else if (OP == kProduct)
                    {
                        term[j] = fix_scale(mul(col_load_stored(a.c0, e), col_load_stored(a.c1, e)), deficit(a.c0) + deficit(a.c1));
                    }
                    else if (OP == kRouteEdgeIndexed)
                    {
                        // the query of edge e is the table row of the node the edge points at, so 1/(Q_e + beta)
                        // is that node's entry of the inverted table
                        const uint64_t node = a.c0.kind == GZK_KIND_U32 ? static_cast<uint64_t>(__ldg(static_cast<const uint32_t*>(a.c0.ptr) + e))
                                                                        : static_cast<uint64_t>(__ldg(static_cast<const long long*>(a.c0.ptr) + e));
                        if (node < a.table_size)
                        {
                            term[j] = load_fr(a.inv_table + node);
                        }
                        else
                        {
                            raise_status(a.status, GZK_E_INVALID, 1406);
                            term[j] = Fr::zero();
                        }
                    }
                    else if (OP == kLogupIndexed)
                    {
                        // Every query equals some table row (that is what the lookup proves, and what the
                        // multiplicity pass has already checked), so 1/(Q_e + beta) IS inv_table[row hit by e]:
                        // a 32-byte fetch from a table that stays in L2 instead of a share in a batch inversion.
                        // The table side of row e < table_size is multiplicity[e] * inv_table[e].  Selectors are
                        // the prefix indicators the reference builds: table rows first, queries on rows < count.
                        Fr t = Fr::zero();
                        if (e < a.table_size)
                        {
                            const uint32_t m = __ldg(static_cast<const uint32_t*>(a.c2.ptr) + e);
                            if (m != 0)
                            {
                                Fr plain = Fr::zero();
                                plain.l[0] = m;
                                t = to_mont(mul(plain, load_fr(a.inv_table + e)));
                            }
                        }
                        const long long rel = (a.c0.kind == GZK_KIND_U32 ? static_cast<long long>(__ldg(static_cast<const uint32_t*>(a.c0.ptr) + e))
                                                                          : __ldg(static_cast<const long long*>(a.c0.ptr) + e)) - a.x_min;
                        uint64_t slot = ~0ull;
                        if (rel >= 0 && static_cast<uint64_t>(rel) * a.band + a.band <= a.table_size)
                        {
                            const uint64_t first = static_cast<uint64_t>(rel) * a.band;
                            if (a.table_y == nullptr)
                            {
                                slot = first;
                            }
                            else
                            {
                                const long long yv = a.c1.kind == GZK_KIND_U32 ? static_cast<long long>(__ldg(static_cast<const uint32_t*>(a.c1.ptr) + e))
                                                                               : __ldg(static_cast<const long long*>(a.c1.ptr) + e);
                                for (uint32_t b = 0; b < a.band; ++b)
                                {
                                    if (__ldg(a.table_y + first + b) == yv)
                                    {
                                        slot = first + b;
                                        break;
                                    }
                                }
                            }
                        }
                        if (slot == ~0ull)
                            raise_status(a.status, GZK_E_INVALID, 1405);
                        else
                            t = sub(t, load_fr(a.inv_table + slot));
                        term[j] = t;
                    }
                    else
                    {
                        term[j] = fix_scale(col_load_stored(a.c0, e), deficit(a.c0));
                        const Fr q = col_load_stored(a.c1, e);
                        if (!q.is_zero())
                        {
                            if (!stored_is_one(a.c1, q)) raise_status(a.status, GZK_E_INVALID, 1403);
                            flag[j] = 1;
                            atomicMin(&first_flag, static_cast<uint32_t>(threadIdx.x * kElems + j));
                        }
                    }
                }
            }

            // thread-local inclusive segmented scan
            SegVal local[kElems];
            SegVal run;
            run.v = Fr::zero();
            run.flag = 0;
#pragma unroll
            for (int j = 0; j < kElems; ++j)
            {
                SegVal cur;
                cur.v = term[j];
                cur.flag = flag[j];
                run = seg_combine(run, cur);
                local[j] = run;
            }
            SegVal aggregate;
            const SegVal prefix = block_seg_exclusive_scan<kThreads>(run, seg_slots, &aggregate);
#pragma unroll
            for (int j = 0; j < kElems; ++j)
            {
                const uint64_t e = base + j;
                const Fr value = seg_combine(prefix, local[j]).v;
                if (OP == kSegmented)
                {
                    if (e < a.n) store_fr(a.out + e, value);
                }
                else
                {
                    if (e < a.count && e + 1 < a.n) store_fr(a.out + e + 1, value);
                }
            }
            if (threadIdx.x == 0)
            {
                store_fr(a.agg_value + block, aggregate.v);
                a.agg_flag[block] = aggregate.flag;
                a.agg_first[block] = first_flag;
            }
        }

        template <int OP, bool LOCAL_INV>
        __global__ void __launch_bounds__(kThreads) scan_main_kernel(ScanArgs a)
        {
            __shared__ MainShared sh;
            scan_main_body<OP, LOCAL_INV>(a, blockIdx.x, sh);
        }

        // Exclusive segmented scan of the CTA aggregates (in place) by one CTA.
        // 1024 threads: the aggregates of a 2^26-row column (131072 of them) are 128 per thread instead of 1024
        constexpr int kOffsetThreads = 1024;
        __global__ void __launch_bounds__(kOffsetThreads) scan_offsets_kernel(Fr* agg_value, uint32_t* agg_flag, uint32_t ctas, Fr* total_out)
        {
            constexpr int kThreads = kOffsetThreads;
            __shared__ SegVal seg_slots[kThreads / 32];
            const uint32_t run_len = (ctas + kThreads - 1) / kThreads;
            const uint32_t begin = threadIdx.x * run_len < ctas ? threadIdx.x * run_len : ctas;
            const uint32_t end = begin + run_len < ctas ? begin + run_len : ctas;
            SegVal run;
            run.v = Fr::zero();
            run.flag = 0;
            for (uint32_t i = begin; i < end; ++i)
            {
                SegVal cur;
                cur.v = load_fr_plain(agg_value + i);
                cur.flag = agg_flag[i];
                run = seg_combine(run, cur);
            }
            SegVal total;
            SegVal prefix = block_seg_exclusive_scan<kThreads>(run, seg_slots, &total);
            for (uint32_t i = begin; i < end; ++i)
            {
                SegVal cur;
                cur.v = load_fr_plain(agg_value + i);
                cur.flag = agg_flag[i];
                store_fr(agg_value + i, prefix.v);
                agg_flag[i] = prefix.flag;
                prefix = seg_combine(prefix, cur);
            }
            if (threadIdx.x == 0) store_fr(total_out, total.v);
        }

        // The same scan in two levels for long columns (a single CTA walks 2^17 aggregates in two dependent passes of
        // 128 loads per thread: 55 us of one SM while the others wait): every group of 1024 aggregates is scanned
        // by a CTA of its own, the group totals by the kernel above, and a third kernel adds the group offsets.
        __global__ void __launch_bounds__(kOffsetThreads) scan_group_offsets_kernel(Fr* agg_value, uint32_t* agg_flag, uint32_t ctas, Fr* group_value,
                                                                                   uint32_t* group_flag)
        {
            __shared__ SegVal seg_slots[kOffsetThreads / 32];
            const uint32_t i = blockIdx.x * kOffsetThreads + threadIdx.x;
            SegVal mine;
            mine.v = Fr::zero();
            mine.flag = 0;
            if (i < ctas)
            {
                mine.v = load_fr_plain(agg_value + i);
                mine.flag = agg_flag[i];
            }
            SegVal total;
            const SegVal prefix = block_seg_exclusive_scan<kOffsetThreads>(mine, seg_slots, &total);
            if (i < ctas)
            {
                store_fr(agg_value + i, prefix.v);
                agg_flag[i] = prefix.flag;
            }
            if (threadIdx.x == 0)
            {
                store_fr(group_value + blockIdx.x, total.v);
                group_flag[blockIdx.x] = total.flag;
            }
        }
        __global__ void __launch_bounds__(kOffsetThreads) scan_apply_group_offsets_kernel(Fr* agg_value, uint32_t* agg_flag, uint32_t ctas, const Fr* group_value,
                                                                                         const uint32_t* group_flag)
        {
            const uint32_t i = blockIdx.x * kOffsetThreads + threadIdx.x;
            if (i >= ctas || blockIdx.x == 0) return;
            SegVal before, mine;
            before.v = load_fr_plain(group_value + blockIdx.x);
            before.flag = group_flag[blockIdx.x];
            mine.v = load_fr_plain(agg_value + i);
            mine.flag = agg_flag[i];
            const SegVal both = seg_combine(before, mine);
            store_fr(agg_value + i, both.v);
            agg_flag[i] = both.flag;
        }
        // the offsets pass of a column with `ctas` chunks; `groups` holds 2 * (groups + 1) spare field elements
        void launch_scan_offsets(gzk_ctx* ctx, Fr* agg_value, uint32_t* agg_flag, uint32_t ctas, Fr* total, Fr* groups)
        {
            LaunchScope scope(ctx, "scan_offsets");
            if (ctas <= 8 * kOffsetThreads)
            {
                scan_offsets_kernel<<<1, kOffsetThreads, 0, ctx->stream>>>(agg_value, agg_flag, ctas, total);
                return;
            }
            const uint32_t group_count = (ctas + kOffsetThreads - 1) / kOffsetThreads;
            uint32_t* group_flag = reinterpret_cast<uint32_t*>(groups + group_count + 1);
            scan_group_offsets_kernel<<<group_count, kOffsetThreads, 0, ctx->stream>>>(agg_value, agg_flag, ctas, groups, group_flag);
            scan_offsets_kernel<<<1, kOffsetThreads, 0, ctx->stream>>>(groups, group_flag, group_count, total);
            scan_apply_group_offsets_kernel<<<group_count, kOffsetThreads, 0, ctx->stream>>>(agg_value, agg_flag, ctas, groups, group_flag);
        }

        template <int OP>
        __global__ void __launch_bounds__(kThreads) scan_fixup_kernel(ScanArgs a)
        {
            const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
            if (idx >= a.n) return;
            if (OP == kSegmented)
            {
                const uint64_t cta = idx / kChunk;
                if (cta == 0) return;
                if (static_cast<uint32_t>(idx - cta * kChunk) < a.agg_first[cta])
                    store_fr(a.out + idx, add(load_fr_plain(a.out + idx), load_fr(a.agg_value + cta)));
                return;
            }
            if (idx == 0)
            {
                store_fr(a.out, Fr::zero());
            }
            else if (idx <= a.count)
            {
                const uint64_t cta = (idx - 1) / kChunk;
                if (cta != 0) store_fr(a.out + idx, add(load_fr_plain(a.out + idx), load_fr(a.agg_value + cta)));
            }
            else
            {
                store_fr(a.out + idx, load_fr(a.total));
            }
        }

        // Sum of one Fr per thread over the CTA, returned to every thread.
        __device__ __forceinline__ Fr cta_sum(Fr v, Fr* warp_slots)
        {
            const int lane = threadIdx.x & 31;
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1)
            {
                const Fr other = shfl_fr_idx(v, (lane + offset) & 31);
                if (lane < offset) v = add(v, other);
            }
            if (lane == 0) warp_slots[threadIdx.x >> 5] = v;
            __syncthreads();
            Fr total = warp_slots[0];
#pragma unroll
            for (int w = 1; w < kWarps; ++w) total = add(total, warp_slots[w]);
            __syncthreads();
            return total;
        }

        // Fix-up that derives the offset of its chunk from the raw CTA aggregates itself (every
        // CTA re-adds at most a few thousand 32-byte values from L2), which saves the separate
        // single-CTA scan of the aggregates when there are few of them.  A CTA covers kThreads
        // consecutive outputs, all inside one chunk of the main pass.
        struct FixupShared
        {
            Fr warp_slots[kWarps];
            int last_start;
        };

        template <int OP>
        __device__ __forceinline__ void scan_fixup_fused_body(const ScanArgs& a, uint32_t ctas, uint32_t block, FixupShared& sh)
        {
            Fr* warp_slots = sh.warp_slots;
            int& last_start = sh.last_start;
            const uint64_t first = static_cast<uint64_t>(block) * kThreads;
            const uint64_t idx = first + threadIdx.x;
            const uint32_t chunk = static_cast<uint32_t>(first / kChunk);
            if (OP == kSegmented)
            {
                if (chunk == 0) return;
                // the running segment reaches back to the last chunk in which a segment started
                if (threadIdx.x == 0) last_start = -1;
                __syncthreads();
                int mine = -1;
                for (uint32_t i = threadIdx.x; i < chunk; i += kThreads)
                    if (a.agg_flag[i] != 0) mine = static_cast<int>(i);
                if (mine >= 0) atomicMax(&last_start, mine);
                __syncthreads();
                const uint32_t from = last_start < 0 ? 0u : static_cast<uint32_t>(last_start);
                Fr part = Fr::zero();
                for (uint32_t i = from + threadIdx.x; i < chunk; i += kThreads) part = add(part, load_fr(a.agg_value + i));
                const Fr offset = cta_sum(part, warp_slots);
                if (idx < a.n && static_cast<uint32_t>(idx - static_cast<uint64_t>(chunk) * kChunk) < a.agg_first[chunk])
                    store_fr(a.out + idx, add(load_fr_plain(a.out + idx), offset));
                return;
            }
            // out[idx] for 1 <= idx <= count belongs to chunk (idx - 1) / kChunk: the CTA's first output sits
            // one chunk lower when the CTA starts on a chunk boundary
            const bool needs_total = first + kThreads > a.count + 1 || block == 0;
            Fr before = Fr::zero(), rest = Fr::zero();
            const uint32_t limit = needs_total ? ctas : chunk;
            for (uint32_t i = threadIdx.x; i < limit; i += kThreads)
            {
                const Fr v = load_fr(a.agg_value + i);
                if (i < chunk)
                    before = add(before, v);
                else
                    rest = add(rest, v);
            }
            const Fr offset = cta_sum(before, warp_slots);
            Fr total = offset;
            if (needs_total) total = add(offset, cta_sum(rest, warp_slots));
            if (block == 0 && threadIdx.x == 0) store_fr(a.total, total);
            if (idx >= a.n) return;
            if (idx == 0)
            {
                store_fr(a.out, Fr::zero());
            }
            else if (idx <= a.count)
            {
                if (idx - 1 >= static_cast<uint64_t>(chunk) * kChunk)
                {
                    if (chunk != 0) store_fr(a.out + idx, add(load_fr_plain(a.out + idx), offset));
                }
                else if (chunk >= 2)
                {
                    store_fr(a.out + idx, add(load_fr_plain(a.out + idx), sub(offset, load_fr(a.agg_value + (chunk - 1)))));
                }
            }
            else
            {
                store_fr(a.out + idx, total);
            }
        }

        template <int OP>
        __global__ void __launch_bounds__(kThreads) scan_fixup_fused_kernel(ScanArgs a, uint32_t ctas)
        {
            __shared__ FixupShared sh;
            scan_fixup_fused_body<OP>(a, ctas, blockIdx.x, sh);
        }

        // ---- several independent running sums in one pair of launches ---------------------------------
        // The column builders between two Fiat-Shamir points of one attention head (three or four lookup
        // accumulators, the node and edge sums of a routing argument, the segmented states) do not depend
        // on one another.  Each alone is a latency chain on a third of the machine (one serial inversion
        // per CTA); queued as ONE grid their chains overlap and the launch count drops from 2 J to 2.
        // A CTA finds its job from the prefix table of CTA counts and runs that job's body.
        constexpr int kMaxBatchJobs = 16;
        struct BatchJob
        {
            ScanArgs args;
            int op;
            uint32_t main_begin, main_ctas;    // CTAs of the main pass: [main_begin, main_begin + main_ctas)
            uint32_t fix_begin, fix_ctas;      // CTAs of the fix-up pass
        };
        struct BatchTable
        {
            BatchJob jobs[kMaxBatchJobs];
            uint32_t count;
        };

        __global__ void __launch_bounds__(kThreads) scan_batch_main_kernel(const BatchTable* table)
        {
            __shared__ MainShared sh;
            uint32_t j = 0;
            while (j + 1 < table->count && blockIdx.x >= table->jobs[j + 1].main_begin) ++j;
            const BatchJob& job = table->jobs[j];
            const uint32_t block = blockIdx.x - job.main_begin;
            if (block >= job.main_ctas) return;
            switch (job.op)
            {
            case kLogup: scan_main_body<kLogup, true>(job.args, block, sh); break;
            case kRouteNode: scan_main_body<kRouteNode, true>(job.args, block, sh); break;
            case kRouteEdge: scan_main_body<kRouteEdge, true>(job.args, block, sh); break;
            case kProduct: scan_main_body<kProduct, true>(job.args, block, sh); break;
            default: scan_main_body<kSegmented, true>(job.args, block, sh); break;
            }
        }

        __global__ void __launch_bounds__(kThreads) scan_batch_fixup_kernel(const BatchTable* table)
        {
            __shared__ FixupShared sh;
            uint32_t j = 0;
            while (j + 1 < table->count && blockIdx.x >= table->jobs[j + 1].fix_begin) ++j;
            const BatchJob& job = table->jobs[j];
            const uint32_t block = blockIdx.x - job.fix_begin;
            if (block >= job.fix_ctas) return;
            switch (job.op)
            {
            case kLogup: scan_fixup_fused_body<kLogup>(job.args, job.main_ctas, block, sh); break;
            case kRouteNode: scan_fixup_fused_body<kRouteNode>(job.args, job.main_ctas, block, sh); break;
            case kRouteEdge: scan_fixup_fused_body<kRouteEdge>(job.args, job.main_ctas, block, sh); break;
            case kProduct: scan_fixup_fused_body<kProduct>(job.args, job.main_ctas, block, sh); break;
            default: scan_fixup_fused_body<kSegmented>(job.args, job.main_ctas, block, sh); break;
            }
        }

        template <int OP>
        int run_scan(gzk_ctx* ctx, ScanArgs& args, bool inverting, uint8_t* total_out_host, bool call_begun = false)
        {
            GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
            const uint64_t span = OP == kSegmented ? args.n : args.count;
            const uint32_t ctas = static_cast<uint32_t>((span + kChunk - 1) / kChunk > 0 ? (span + kChunk - 1) / kChunk : 1);
            void* scratch = nullptr;
            const size_t group_count = (static_cast<size_t>(ctas) + kOffsetThreads - 1) / kOffsetThreads;
            const size_t bytes = static_cast<size_t>(ctas) * (3 * sizeof(Fr) + 2 * sizeof(uint32_t)) + 2 * sizeof(Fr) + 2 * (group_count + 1) * sizeof(Fr);
            int rc = ensure_scratch(ctx, 2, bytes, &scratch);
            if (rc != GZK_OK) return rc;
            Fr* base = static_cast<Fr*>(scratch);
            args.cta_products = base;
            Fr* tmp = base + ctas;
            args.agg_value = base + 2 * static_cast<size_t>(ctas);
            args.total = base + 3 * static_cast<size_t>(ctas);
            args.agg_flag = reinterpret_cast<uint32_t*>(base + 3 * static_cast<size_t>(ctas) + 2);
            args.agg_first = args.agg_flag + ctas;
            Fr* group_area = reinterpret_cast<Fr*>(reinterpret_cast<char*>(scratch) + ((static_cast<size_t>(ctas) * (3 * sizeof(Fr) + 2 * sizeof(uint32_t)) + 2 * sizeof(Fr) + 31) & ~static_cast<size_t>(31)));
            args.status = ctx->d_status;
            if (!call_begun && (rc = begin_call(ctx)) != GZK_OK) return rc;
            const bool local_inverse = inverting && ctas <= static_cast<uint32_t>(ctx->sm_count) * 4;
            if (inverting && !local_inverse)
            {
                {
                    LaunchScope scope(ctx, "scan_products");
                    scan_products_kernel<OP><<<ctas, kThreads, 0, ctx->stream>>>(args);
                }
                GZK_CUDA_TRY(ctx, cudaGetLastError());
                if ((rc = launch_batch_invert_single_cta(ctx, args.cta_products, tmp, ctas)) != GZK_OK) return rc;
            }
            {
                LaunchScope scope(ctx, OP == kLogup ? "scan_main_logup" : OP == kLogupIndexed ? "scan_main_logup_indexed" : OP == kRouteEdgeIndexed ? "scan_main_route_edge_indexed" : OP == kRouteNode ? "scan_main_route_node" : OP == kRouteEdge ? "scan_main_route_edge"
                                       : OP == kProduct ? "scan_main_product" : "scan_main_segmented");
                if (local_inverse)
                    scan_main_kernel<OP, true><<<ctas, kThreads, 0, ctx->stream>>>(args);
                else
                    scan_main_kernel<OP, false><<<ctas, kThreads, 0, ctx->stream>>>(args);
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            if (ctas <= 2048)
            {
                if (args.n > 0 || total_out_host != nullptr)
                {
                    LaunchScope scope(ctx, "scan_fixup");
                    const uint64_t outputs = args.n > 0 ? args.n : 1;
                    scan_fixup_fused_kernel<OP><<<static_cast<unsigned>((outputs + kThreads - 1) / kThreads), kThreads, 0, ctx->stream>>>(args, ctas);
                }
            }
            else
            {
                launch_scan_offsets(ctx, args.agg_value, args.agg_flag, ctas, args.total, group_area);
                GZK_CUDA_TRY(ctx, cudaGetLastError());
                if (args.n > 0)
                {
                    LaunchScope scope(ctx, "scan_fixup");
                    scan_fixup_kernel<OP><<<static_cast<unsigned>((args.n + kThreads - 1) / kThreads), kThreads, 0, ctx->stream>>>(args);
                }
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            if (total_out_host == nullptr) return finish_call(ctx, "q_new must hold only 0 and 1");
            struct
            {
                Fr total;
                int status;
            } host;
            GZK_CUDA_TRY(ctx, cudaMemcpyAsync(&host.total, args.total, sizeof(Fr), cudaMemcpyDeviceToHost, ctx->stream));
            GZK_CUDA_TRY(ctx, cudaMemcpyAsync(&host.status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
            GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            if (host.status == GZK_E_DOMAIN) return fail(ctx, GZK_E_DOMAIN, "batch_invert encountered zero");
            if (host.status == GZK_E_INVALID) return fail(ctx, GZK_E_INVALID, "q_new must hold only 0 and 1");
            if (total_out_host != nullptr) host_fr_to_bytes(from_mont(host.total), total_out_host);
            return GZK_OK;
        }

        bool col_ok(const gzk_buf* b, uint64_t need) { return b != nullptr && b->count >= need; }
        ColRef ref(const gzk_buf* b)
        {
            ColRef r;
            r.ptr = b->dptr;
            r.kind = b->kind;
            return r;
        }
        int load_scalar(gzk_ctx* ctx, const uint8_t* bytes, Fr* out_mont, Fr* out_canonical)
        {
            bool canonical = false;
            const Fr v = host_fr_from_bytes(bytes, &canonical);
            if (!canonical) return fail(ctx, GZK_E_INVALID, "scalar argument is not a canonical field element");
            *out_mont = to_mont(v);
            *out_canonical = v;
            return GZK_OK;
        }
        bool out_ok(const gzk_buf* out, uint64_t n) { return out != nullptr && out->kind == GZK_KIND_FR_MONT && out->count >= n; }
    }
}

using namespace gzk;

extern "C"
{
    int gzk_logup_accumulator_indexed(gzk_ctx* ctx, const gzk_buf* table, const gzk_buf* multiplicity, const gzk_buf* x, const gzk_buf* y,
                                      size_t active_count, int64_t x_min, size_t band, const gzk_buf* table_y, size_t table_size, size_t n,
                                      const uint8_t beta[32], gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (beta == nullptr || !out_ok(out, n)) return fail(ctx, GZK_E_INVALID, "logup: output must be a Montgomery buffer of n elements");
        if (n > 0 && active_count > n - 1) active_count = n - 1;  // lookup.cpp:117
        if (n == 0) return GZK_OK;
        const bool has_y = y != nullptr;
        auto keys_ok = [&](const gzk_buf* b) { return b != nullptr && (b->kind == GZK_KIND_I64 || b->kind == GZK_KIND_U32) && b->count >= active_count; };
        if (band == 0 || band > 64 || table_size == 0 || table_size % band != 0 || table_size > n || has_y != (table_y != nullptr) || (!has_y && band != 1))
            return fail(ctx, GZK_E_INVALID, "logup (indexed): the table must hold a whole number of bands and fit the column");
        if (!col_ok(table, table_size) || multiplicity == nullptr || multiplicity->kind != GZK_KIND_U32 || multiplicity->count < table_size || !keys_ok(x) ||
            (has_y && (!keys_ok(y) || table_y->kind != GZK_KIND_I64 || table_y->count < table_size)))
            return fail(ctx, GZK_E_INVALID, "lookup accumulator input size mismatch");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        ScanArgs args{};
        int rc = load_scalar(ctx, beta, &args.beta, &args.beta_canon);
        if (rc != GZK_OK) return rc;
        void* scratch = nullptr;
        if ((rc = ensure_scratch(ctx, 1, table_size * sizeof(Fr), &scratch)) != GZK_OK) return rc;
        // pass 0: the inverses of the shifted table
        args.c0 = ref(table);
        args.count = table_size;
        args.status = ctx->d_status;
        if ((rc = begin_call(ctx)) != GZK_OK) return rc;
        {
            LaunchScope scope(ctx, "logup_table_inverses");
            shifted_inverse_kernel<<<static_cast<unsigned>((table_size + kChunk - 1) / kChunk), kThreads, 0, ctx->stream>>>(args, static_cast<Fr*>(scratch));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        args.c0 = ref(x);
        args.c1 = has_y ? ref(y) : ref(x);
        args.c2 = ref(multiplicity);
        args.count = active_count;
        args.n = n;
        args.out = static_cast<Fr*>(out->dptr);
        args.inv_table = static_cast<const Fr*>(scratch);
        args.table_y = has_y ? static_cast<const long long*>(table_y->dptr) : nullptr;
        args.table_size = table_size;
        args.x_min = static_cast<long long>(x_min);
        args.band = static_cast<uint32_t>(band);
        return run_scan<kLogupIndexed>(ctx, args, false, nullptr, true);
    }

    int gzk_route_edge_accumulator_indexed(gzk_ctx* ctx, const gzk_buf* table, size_t node_count, const gzk_buf* index, size_t valid_length,
                                           size_t domain_size, const uint8_t beta[32], gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (beta == nullptr || !out_ok(out, domain_size)) return fail(ctx, GZK_E_INVALID, "route: output must be a Montgomery buffer of the domain size");
        if (domain_size == 0) return GZK_OK;
        if (valid_length > domain_size - 1) valid_length = domain_size - 1;
        if (node_count == 0 || !col_ok(table, node_count) || index == nullptr || (index->kind != GZK_KIND_I64 && index->kind != GZK_KIND_U32) ||
            index->count < valid_length)
            return fail(ctx, GZK_E_INVALID, "route accumulator input size mismatch");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        ScanArgs args{};
        int rc = load_scalar(ctx, beta, &args.beta, &args.beta_canon);
        if (rc != GZK_OK) return rc;
        void* scratch = nullptr;
        if ((rc = ensure_scratch(ctx, 1, node_count * sizeof(Fr), &scratch)) != GZK_OK) return rc;
        args.c0 = ref(table);
        args.count = node_count;
        args.status = ctx->d_status;
        if ((rc = begin_call(ctx)) != GZK_OK) return rc;
        {
            LaunchScope scope(ctx, "route_table_inverses");
            shifted_inverse_kernel<<<static_cast<unsigned>((node_count + kChunk - 1) / kChunk), kThreads, 0, ctx->stream>>>(args, static_cast<Fr*>(scratch));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        args.c0 = ref(index);
        args.count = valid_length;
        args.n = domain_size;
        args.out = static_cast<Fr*>(out->dptr);
        args.inv_table = static_cast<const Fr*>(scratch);
        args.table_size = node_count;
        return run_scan<kRouteEdgeIndexed>(ctx, args, false, nullptr, true);
    }

    int gzk_logup_accumulator(gzk_ctx* ctx, const gzk_buf* table, const gzk_buf* query, const gzk_buf* multiplicity,
                              const gzk_buf* q_table, const gzk_buf* q_query, size_t n, const uint8_t beta[32],
                              size_t active_count, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (beta == nullptr || !out_ok(out, n)) return fail(ctx, GZK_E_INVALID, "logup: output must be a Montgomery buffer of n elements");
        if (n > 0 && active_count > n - 1) active_count = n - 1;  // lookup.cpp:117
        if (n == 0) return GZK_OK;
        if (!col_ok(table, active_count) || !col_ok(query, active_count) || !col_ok(multiplicity, active_count) ||
            !col_ok(q_table, active_count) || !col_ok(q_query, active_count))
            return fail(ctx, GZK_E_INVALID, "lookup accumulator input size mismatch");
        ScanArgs args{};
        args.c0 = ref(table);
        args.c1 = ref(query);
        args.c2 = ref(multiplicity);
        args.c3 = ref(q_table);
        args.c4 = ref(q_query);
        args.count = active_count;
        args.n = n;
        args.out = static_cast<Fr*>(out->dptr);
        int rc = load_scalar(ctx, beta, &args.beta, &args.beta_canon);
        if (rc != GZK_OK) return rc;
        return run_scan<kLogup>(ctx, args, true, nullptr);
    }

    int gzk_route_node_accumulator(gzk_ctx* ctx, const gzk_buf* table, const gzk_buf* multiplicity, size_t valid_length,
                                   size_t domain_size, const uint8_t beta[32], gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (beta == nullptr || !out_ok(out, domain_size)) return fail(ctx, GZK_E_INVALID, "route node: bad output buffer");
        if (domain_size == 0) return GZK_OK;
        if (valid_length >= domain_size) return fail(ctx, GZK_E_INVALID, "route accumulator needs valid_length < domain_size");
        if (!col_ok(table, valid_length) || !col_ok(multiplicity, valid_length))
            return fail(ctx, GZK_E_INVALID, "route node accumulator input size mismatch");
        ScanArgs args{};
        args.c0 = ref(table);
        args.c1 = ref(multiplicity);
        args.count = valid_length;
        args.n = domain_size;
        args.out = static_cast<Fr*>(out->dptr);
        int rc = load_scalar(ctx, beta, &args.beta, &args.beta_canon);
        if (rc != GZK_OK) return rc;
        return run_scan<kRouteNode>(ctx, args, true, nullptr);
    }

    int gzk_route_edge_accumulator(gzk_ctx* ctx, const gzk_buf* query, size_t valid_length, size_t domain_size,
                                   const uint8_t beta[32], gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (beta == nullptr || !out_ok(out, domain_size)) return fail(ctx, GZK_E_INVALID, "route edge: bad output buffer");
        if (domain_size == 0) return GZK_OK;
        if (valid_length >= domain_size) return fail(ctx, GZK_E_INVALID, "route accumulator needs valid_length < domain_size");
        if (!col_ok(query, valid_length)) return fail(ctx, GZK_E_INVALID, "route edge accumulator input size mismatch");
        ScanArgs args{};
        args.c0 = ref(query);
        args.count = valid_length;
        args.n = domain_size;
        args.out = static_cast<Fr*>(out->dptr);
        int rc = load_scalar(ctx, beta, &args.beta, &args.beta_canon);
        if (rc != GZK_OK) return rc;
        return run_scan<kRouteEdge>(ctx, args, true, nullptr);
    }

    int gzk_zkmap_accumulator(gzk_ctx* ctx, const gzk_buf* a, const gzk_buf* b, size_t count, size_t domain_size,
                              gzk_buf* out_acc, uint8_t mu_out[32])
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (!out_ok(out_acc, domain_size)) return fail(ctx, GZK_E_INVALID, "zkmap: bad output buffer");
        if (count != 0 && count + 1 > domain_size) return fail(ctx, GZK_E_INVALID, "zkMaP accumulator exceeds its domain");
        if (!col_ok(a, count) || !col_ok(b, count)) return fail(ctx, GZK_E_INVALID, "zkMaP input size mismatch");
        if (domain_size == 0)
        {
            if (mu_out != nullptr) std::memset(mu_out, 0, 32);
            return GZK_OK;
        }
        ScanArgs args{};
        args.c0 = ref(a);
        args.c1 = ref(b);
        args.count = count;
        args.n = domain_size;
        args.beta = Fr::zero();
        args.out = static_cast<Fr*>(out_acc->dptr);
        return run_scan<kProduct>(ctx, args, false, mu_out);
    }

    int gzk_running_sums_batch(gzk_ctx* ctx, const gzk_scan_job* jobs, size_t job_count)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (job_count == 0) return GZK_OK;
        if (jobs == nullptr) return fail(ctx, GZK_E_INVALID, "running_sums_batch: null job list");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        int rc = begin_call(ctx);
        if (rc != GZK_OK) return rc;
        size_t done = 0;
        while (done < job_count)
        {
            // jobs are queued in groups of at most kMaxBatchJobs
            BatchTable table{};
            size_t scratch_frs = 0, scratch_u32 = 0;
            struct Layout
            {
                size_t fr_at, u32_at;
            } layout[kMaxBatchJobs];
            uint32_t main_total = 0, fix_total = 0;
            while (done < job_count && table.count < kMaxBatchJobs)
            {
                const gzk_scan_job& j = jobs[done];
                BatchJob& b = table.jobs[table.count];
                ScanArgs& a = b.args;
                a = ScanArgs{};
                a.beta = Fr::zero();
                size_t count = j.count;
                const size_t n = j.domain_size;
                if (!out_ok(j.out, n)) return fail(ctx, GZK_E_INVALID, "running_sums_batch: every output must be a Montgomery buffer of its domain size");
                if (n == 0)
                {
                    ++done;
                    continue;
                }
                switch (j.op)
                {
                case GZK_SCAN_LOGUP:
                    if (count > n - 1) count = n - 1;
                    if (j.beta == nullptr || !col_ok(j.c0, count) || !col_ok(j.c1, count) || !col_ok(j.c2, count) || !col_ok(j.c3, count) || !col_ok(j.c4, count))
                        return fail(ctx, GZK_E_INVALID, "lookup accumulator input size mismatch");
                    a.c0 = ref(j.c0);
                    a.c1 = ref(j.c1);
                    a.c2 = ref(j.c2);
                    a.c3 = ref(j.c3);
                    a.c4 = ref(j.c4);
                    break;
                case GZK_SCAN_ROUTE_NODE:
                    if (count >= n) return fail(ctx, GZK_E_INVALID, "route accumulator needs valid_length < domain_size");
                    if (j.beta == nullptr || !col_ok(j.c0, count) || !col_ok(j.c1, count)) return fail(ctx, GZK_E_INVALID, "route node accumulator input size mismatch");
                    a.c0 = ref(j.c0);
                    a.c1 = ref(j.c1);
                    break;
                case GZK_SCAN_ROUTE_EDGE:
                    if (count >= n) return fail(ctx, GZK_E_INVALID, "route accumulator needs valid_length < domain_size");
                    if (j.beta == nullptr || !col_ok(j.c0, count)) return fail(ctx, GZK_E_INVALID, "route edge accumulator input size mismatch");
                    a.c0 = ref(j.c0);
                    break;
                case GZK_SCAN_ZKMAP:
                    if (count != 0 && count + 1 > n) return fail(ctx, GZK_E_INVALID, "zkMaP accumulator exceeds its domain");
                    if (!col_ok(j.c0, count) || !col_ok(j.c1, count)) return fail(ctx, GZK_E_INVALID, "zkMaP input size mismatch");
                    a.c0 = ref(j.c0);
                    a.c1 = ref(j.c1);
                    break;
                case GZK_SCAN_GROUP_PREFIX:
                    count = n;
                    if (!col_ok(j.c0, n) || !col_ok(j.c1, n)) return fail(ctx, GZK_E_INVALID, "prefix state input size mismatch");
                    a.c0 = ref(j.c0);
                    a.c1 = ref(j.c1);
                    break;
                default: return fail(ctx, GZK_E_INVALID, "running_sums_batch: unknown operation");
                }
                if (j.op <= GZK_SCAN_ROUTE_EDGE && (rc = load_scalar(ctx, j.beta, &a.beta, &a.beta_canon)) != GZK_OK) return rc;
                a.count = count;
                a.n = n;
                a.out = static_cast<Fr*>(j.out->dptr);
                a.status = ctx->d_status;
                const uint64_t span = j.op == GZK_SCAN_GROUP_PREFIX ? n : count;
                const uint64_t ctas = (span + kChunk - 1) / kChunk > 0 ? (span + kChunk - 1) / kChunk : 1;
                if (ctas > 2048) return fail(ctx, GZK_E_INVALID, "running_sums_batch: at most 2^20 rows per job; use the single-column entry point for longer columns");
                b.op = j.op == GZK_SCAN_LOGUP ? kLogup : j.op == GZK_SCAN_ROUTE_NODE ? kRouteNode : j.op == GZK_SCAN_ROUTE_EDGE ? kRouteEdge
                       : j.op == GZK_SCAN_ZKMAP ? kProduct : kSegmented;
                b.main_begin = main_total;
                b.main_ctas = static_cast<uint32_t>(ctas);
                b.fix_begin = fix_total;
                b.fix_ctas = static_cast<uint32_t>((n + kThreads - 1) / kThreads);
                main_total += b.main_ctas;
                fix_total += b.fix_ctas;
                layout[table.count] = {scratch_frs, scratch_u32};
                scratch_frs += ctas + 1;       // aggregates + total
                scratch_u32 += 2 * ctas;       // flags + first-restart marks
                ++table.count;
                ++done;
            }
            if (table.count == 0) continue;
            const size_t table_bytes = (sizeof(BatchTable) + 31) & ~static_cast<size_t>(31);
            void* scratch = nullptr;
            if ((rc = ensure_scratch(ctx, 2, table_bytes + scratch_frs * sizeof(Fr) + scratch_u32 * sizeof(uint32_t), &scratch)) != GZK_OK) return rc;
            Fr* fr_base = reinterpret_cast<Fr*>(static_cast<char*>(scratch) + table_bytes);
            uint32_t* u32_base = reinterpret_cast<uint32_t*>(fr_base + scratch_frs);
            for (uint32_t t = 0; t < table.count; ++t)
            {
                ScanArgs& a = table.jobs[t].args;
                const uint32_t ctas = table.jobs[t].main_ctas;
                a.cta_products = nullptr;  // every CTA inverts its own product
                a.agg_value = fr_base + layout[t].fr_at;
                a.total = a.agg_value + ctas;
                a.agg_flag = u32_base + layout[t].u32_at;
                a.agg_first = a.agg_flag + ctas;
            }
            // the table travels from pageable memory of this call: the copy is staged before the call returns
            GZK_CUDA_TRY(ctx, cudaMemcpyAsync(scratch, &table, sizeof(BatchTable), cudaMemcpyHostToDevice, ctx->stream));
            {
                LaunchScope scope(ctx, "scan_batch_main");
                scan_batch_main_kernel<<<main_total, kThreads, 0, ctx->stream>>>(static_cast<const BatchTable*>(scratch));
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
            {
                LaunchScope scope(ctx, "scan_batch_fixup");
                scan_batch_fixup_kernel<<<fix_total, kThreads, 0, ctx->stream>>>(static_cast<const BatchTable*>(scratch));
            }
            GZK_CUDA_TRY(ctx, cudaGetLastError());
        }
        return finish_call(ctx, "q_new must hold only 0 and 1");
    }

    int gzk_group_prefix_state(gzk_ctx* ctx, const gzk_buf* values, const gzk_buf* q_new, size_t n, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (!out_ok(out, n)) return fail(ctx, GZK_E_INVALID, "prefix state: bad output buffer");
        if (!col_ok(values, n) || !col_ok(q_new, n)) return fail(ctx, GZK_E_INVALID, "prefix state input size mismatch");
        if (n == 0) return GZK_OK;
        ScanArgs args{};
        args.c0 = ref(values);
        args.c1 = ref(q_new);
        args.count = n;
        args.n = n;
        args.beta = Fr::zero();
        args.out = static_cast<Fr*>(out->dptr);
        return run_scan<kSegmented>(ctx, args, false, nullptr);
    }
}
