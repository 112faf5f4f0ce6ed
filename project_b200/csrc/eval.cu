// Packed evaluation: K columns x n rows x P rotations of Fr inner products against
// one shared weight vector.  This is the kernel behind column commitment
// (tau-evaluation of every committed column) and behind every opening / quotient
// evaluation of the prover.
//
// Arithmetic: weights are in Montgomery form, column values in canonical form.
// A unit accumulates the plain 512-bit integer products w~[c] * f[c] into a 17-limb
// sum without any modular reduction (2^32 terms fit); one reduction per (tile, column)
// pair follows in a second, tiny kernel.  Field-element columns form the products on
// the tensor cores: with the 32 bytes of w~ and of f as the two factors, the byte
// products summed over the rows are a 32 x 32 matrix product whose contraction index
// is the row (mma.sync m16n8k32, u8 x u8 -> s32; eight per 32 rows), and the sum is
// sum_ab C[a][b] 2^(8(a+b)) - the integer pipe needs 64 wide multiply-adds per row for
// the same sum and was the bound of this kernel.  Small-integer columns take the same
// route in groups of four at two evaluation points, and the integer pipe (8 products
// per row) at one.
//
// Work decomposition: the row range is cut into tiles; a unit of work is one
// (tile, column) pair, enumerated tile-major so that the warps of a CTA stream
// different columns against the SAME weight tile (served by L1/L2 after the first
// touch).  Units are dealt to warps round-robin, which balances any K and n over
// 148 SMs without atomics and keeps the tiles in flight neighbours.  Each unit produces one 17-limb partial sum in
// context-owned scratch.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace gzk
{
    namespace
    {
        constexpr int kAccLimbs = 17;
        constexpr int kThreads = 128;

        struct EvalArgs
        {
            const void* const* cols;  // K device pointers
            const int* kinds;         // K buffer kinds
            const Fr* weights;
            uint64_t len;
            uint64_t mask;
            uint64_t tile_rows;
            uint32_t tiles;
            uint32_t k_count;
            uint64_t rot[2];
            uint32_t* partial;        // [tile][p][k][17]
            int* status;              // raised when a bounded wait gives up
            uint32_t wait_limit;      // polls a wait on a chunk may take before it gives up
            uint32_t skip_copies;     // stall injection (gzk_debug_inject_eval_stall): announce the chunks but issue no copy
            const uint32_t* k_map;    // the columns this launch takes (indices into cols), or null: all k_count of them
            uint32_t k_mapped;        // entries of k_map (k_count without a map)
        };
        // Which columns a launch takes.  Field-element columns run through the shared-memory ring and the tensor
        // cores; small-integer columns in groups of four through a tensor-core kernel of their own
        // (kIntegerGroups), the ones left over through plain loads and the integer pipe (kIntegerKinds: many resident
        // warps, no shared memory).  A call launches one kernel for each kind present, over the same partial buffer.
        enum { kAllKinds = 0, kFieldKinds = 1, kIntegerKinds = 2, kIntegerGroups = 3 };

        // ---- per-warp TMA ring -------------------------------------------------------
        // Both operands of the inner product reach the arithmetic through shared memory:
        // lane 0 of each warp streams chunks (128 or 64 rows) of the column, and the
        // matching weights for every rotation, into a private ring with
        // cp.async.bulk, one chunk ahead of the arithmetic; the warp waits on the chunk's
        // mbarrier.  Column values (read once) bypass L1 entirely, the weights come from
        // L2, and the arithmetic sees only short shared-memory latencies.
        // Every wait is bounded; a wait that gives up raises the status word and the
        // kernel returns.
        constexpr int kStages = 2;
        // Rows per chunk: 128 at one evaluation point (the per-chunk bookkeeping - the wait, the next request -
        // is a sixth of the instructions at 64), 64 at two, where 128 would leave room for two CTAs per SM only and
        // the small-integer columns of the same launch need the warps.  Tiles are whole chunks of either size.
        constexpr int kChunkRows = 128;
        __host__ __device__ constexpr int chunk_rows(int p) { return p == 1 ? kChunkRows : kChunkRows / 2; }
        __host__ __device__ constexpr int chunk_bytes(int p) { return chunk_rows(p) * 32; }
        constexpr int kWarps = kThreads / 32;
        // a ring slot holds the column chunk and, behind it, one weight chunk per rotation
        __host__ __device__ constexpr size_t slot_bytes(int p) { return static_cast<size_t>(1 + p) * chunk_bytes(p); }
        __host__ __device__ constexpr size_t ring_bytes(int p) { return static_cast<size_t>(kWarps) * kStages * slot_bytes(p); }
        __host__ __device__ constexpr size_t smem_bytes(int p) { return ring_bytes(p) + static_cast<size_t>(kWarps) * kStages * sizeof(uint64_t); }
        constexpr uint32_t kWaitLimit = 1u << 22;

        __device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

        __device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
        {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
        }
        __device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
        {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        }
        __device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
        {
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                         "l"(src), "r"(bytes), "r"(bar)
                         : "memory");
        }
        __device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
        {
            uint32_t done;
            asm volatile(
                "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(done)
                : "r"(bar), "r"(parity)
                : "memory");
            return done != 0;
        }
        // Bounded wait: false when the limit ran out.
        __device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit)
        {
            for (uint32_t spin = 0; spin < limit; ++spin)
                if (mbar_try_wait(bar, parity)) return true;
            return false;
        }
        // ---- field-element columns on the tensor cores -----------------------------------
        // sum_i w_i * f_i over the rows of a unit, both factors 32 bytes: with W[i][a] and F[i][b] their bytes,
        // C[a][b] = sum_i W[i][a] * F[i][b] is a 32 x 32 matrix product with the ROWS as the contraction
        // index, and the exact integer sum is sum_ab C[a][b] * 2^(8(a+b)).  One warp-wide
        // mma.sync m16n8k32 (u8 x u8 -> s32) contracts 32 rows for a 16 x 8 block of C; eight of them cover
        // C for 32 rows - 32768 byte products where the integer pipe would issue 2048 limb products.
        // A fragment register holds ONE byte index and FOUR rows, memory holds four byte indices of one row
        // per word: every lane loads a 4 x 4 byte block (its word of four rows) and transposes it with eight
        // byte permutes.  Which rows and which bytes a lane takes is free (any permutation of the rows, the
        // same for both factors, and any numbering of the bytes): lane (g, t) = (lane / 4, lane % 4) takes word
        // g of rows t, t+4, t+8, t+12 (+16 for the second half of the contraction) - conflict-free in shared
        // memory - so that byte 4g + j of the weights is row 8*(j&1) + g of block j/2 of C, and byte
        // 4g + j of the column values is column g of block j.
        // s32 entries hold 255^2 * 32768 rows; the warp folds C into a 17-limb total before that many.
        constexpr uint32_t kStepsPerFold = 1024;  // x 32 rows

        __device__ __forceinline__ void load_rows_transposed(const unsigned char* step_base, uint32_t g, uint32_t t, uint32_t out[2][4])
        {
#pragma unroll
            for (int h = 0; h < 2; ++h)
            {
                const uint32_t* word = reinterpret_cast<const uint32_t*>(step_base + (16 * h + t) * 32) + g;
                const uint32_t x0 = word[0], x1 = word[32], x2 = word[64], x3 = word[96];  // rows t, t+4, t+8, t+12
                const uint32_t t0 = __byte_perm(x0, x1, 0x5140), t1 = __byte_perm(x2, x3, 0x5140);
                const uint32_t t2 = __byte_perm(x0, x1, 0x7362), t3 = __byte_perm(x2, x3, 0x7362);
                out[h][0] = __byte_perm(t0, t1, 0x5410);
                out[h][1] = __byte_perm(t0, t1, 0x7632);
                out[h][2] = __byte_perm(t2, t3, 0x5410);
                out[h][3] = __byte_perm(t2, t3, 0x7632);
            }
        }
        __device__ __forceinline__ void mma_u8(int32_t c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
        {
            asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                         : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
        }
        // Adds sum_ab C[a][b] 2^(8(a+b)) to `total` (17 limbs in shared memory, kept by lane 0) and clears C.
        // `scratch`: 4 KiB of this warp's shared memory that nothing else uses meanwhile.
        __device__ __forceinline__ void fold_byte_products(int32_t c[2][4][4], unsigned char* scratch, uint32_t lane, uint32_t* total)
        {
            const uint32_t g = lane >> 2, t = lane & 3;
            int32_t* matrix = reinterpret_cast<int32_t*>(scratch);
            __syncwarp();
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                    {
                        const uint32_t a = 4 * g + 2 * mt + (i >> 1);
                        const uint32_t b = 8 * t + 4 * (i & 1) + nt;
                        matrix[a * 32 + b] = c[mt][nt][i];
                        c[mt][nt][i] = 0;
                    }
            __syncwarp();
            // the two anti-diagonals a + b = lane and a + b = lane + 32
            unsigned long long low = 0, high = 0;
#pragma unroll 8
            for (uint32_t a = 0; a < 32; ++a)
            {
                const uint32_t value = static_cast<uint32_t>(matrix[31 * a + lane + (a > lane ? 32 : 0)]);
                if (a > lane)
                    high += value;
                else
                    low += value;
            }
            __syncwarp();
            unsigned long long* diagonal = reinterpret_cast<unsigned long long*>(scratch);
            diagonal[lane] = low;
            diagonal[lane + 32] = high;  // diagonal 63 does not exist: lane 31 writes 0
            __syncwarp();
            // limb j collects the diagonals 4j .. 4j+3 (each below 2^37, so the sum stays below 2^62)
            unsigned long long* limb = reinterpret_cast<unsigned long long*>(scratch + 512);  // behind the 64 diagonals
            if (lane < 16)
                limb[lane] = diagonal[4 * lane] + (diagonal[4 * lane + 1] << 8) + (diagonal[4 * lane + 2] << 16) + (diagonal[4 * lane + 3] << 24);
            __syncwarp();
            uint32_t even[kAccLimbs], odd[kAccLimbs];
#pragma unroll
            for (int k = 0; k < 8; ++k)
            {
                const unsigned long long e = limb[2 * k], o = limb[2 * k + 1];
                even[2 * k] = static_cast<uint32_t>(e);
                even[2 * k + 1] = static_cast<uint32_t>(e >> 32);
                odd[2 * k + 1] = static_cast<uint32_t>(o);
                odd[2 * k + 2] = static_cast<uint32_t>(o >> 32);
            }
            even[16] = 0;
            odd[0] = 0;
            if (lane == 0)
            {
                acc_add<kAccLimbs, kAccLimbs>(even, odd);
                uint32_t sum[kAccLimbs];
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) sum[i] = total[i];
                acc_add<kAccLimbs, kAccLimbs>(sum, even);
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) total[i] = sum[i];
            }
            // the scratch is ring memory: order these accesses before the bulk copy that refills it
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
        }

        template <int P, int MODE>
        __global__ void __launch_bounds__(kThreads, MODE == kIntegerKinds ? (P == 2 ? 4 : 5) : (P == 2 ? 4 : 3)) eval_partial_kernel(EvalArgs a)
        {
            constexpr bool kHasField = MODE != kIntegerKinds;
            extern __shared__ __align__(128) unsigned char smem[];
            __shared__ uint32_t totals[kHasField ? kWarps : 1][P][kAccLimbs];  // running sum of a field-element unit, per warp (lane 0's)
            const uint32_t lane = threadIdx.x & 31;
            const uint32_t warp_in_cta = threadIdx.x >> 5;
            unsigned char* ring = smem + static_cast<size_t>(warp_in_cta) * kStages * slot_bytes(P);
            uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ring_bytes(P)) + warp_in_cta * kStages;
            if (kHasField && lane == 0)
            {
#pragma unroll
                for (int st = 0; st < kStages; ++st) mbar_init(smem_u32(bars + st), 1);
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            __syncwarp();

            const uint64_t warp = (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
            const uint64_t warps = (static_cast<uint64_t>(gridDim.x) * kThreads) >> 5;
            const uint64_t units = static_cast<uint64_t>(a.tiles) * a.k_mapped;
            uint32_t ring_pos = 0;  // chunks this warp has pushed through the ring so far

            // Units are tile-major and dealt round-robin: at any moment the grid works on a window of
            // consecutive units, i.e. on all columns of a few hundred neighbouring tiles, so a weight tile is
            // fetched from DRAM once and served from L2 to the warps that take the other columns of that
            // tile.  (Contiguous runs per warp would put every warp on a tile of its own: the whole weight
            // vector, far larger than L2, would cycle through the cache once per column.)
            for (uint64_t u = warp; u < units; u += warps)
            {
                const uint32_t tile = static_cast<uint32_t>(u / a.k_mapped);
                const uint32_t slot_of_k = static_cast<uint32_t>(u - static_cast<uint64_t>(tile) * a.k_mapped);
                const uint32_t k = a.k_map != nullptr ? a.k_map[slot_of_k] : slot_of_k;
                const void* col = a.cols[k];
                const int kind = a.kinds[k];
                const uint64_t c_begin = static_cast<uint64_t>(tile) * a.tile_rows;
                const uint64_t c_end = c_begin + a.tile_rows < a.len ? c_begin + a.tile_rows : a.len;

                if (kHasField && (kind == GZK_KIND_FR || kind == GZK_KIND_FR_MONT))
                {
                    const unsigned char* base = static_cast<const unsigned char*>(col) + c_begin * 32;
                    const uint64_t rows = c_end > c_begin ? c_end - c_begin : 0;
                    constexpr int kRows = chunk_rows(P);
                    const uint32_t chunks = static_cast<uint32_t>((rows + kRows - 1) / kRows);
                    auto issue = [&](uint32_t j) {
                        // chunk j of this unit goes to ring slot (ring_pos + j) % kStages: the column
                        // rows, then for every rotation the weights those rows meet (the weight index
                        // wraps around the domain at most once inside a chunk)
                        const uint32_t slot = (ring_pos + j) % kStages;
                        const uint64_t row0 = static_cast<uint64_t>(j) * kRows;
                        const uint32_t rows_j = static_cast<uint32_t>(rows - row0 < kRows ? rows - row0 : kRows);
                        const uint32_t bytes = rows_j * 32;
                        const uint32_t bar = smem_u32(bars + slot);
                        unsigned char* dst = ring + static_cast<size_t>(slot) * slot_bytes(P);
                        mbar_expect_tx(bar, bytes * (1 + P));
                        if (a.skip_copies) return;  // injected stall: the barrier is armed, nothing is in flight
                        bulk_load(smem_u32(dst), base + row0 * 32, bytes, bar);
#pragma unroll
                        for (int p = 0; p < P; ++p)
                        {
                            const uint64_t w0 = (c_begin + row0 - a.rot[p]) & a.mask;
                            const uint64_t until_wrap = a.mask + 1 - w0;
                            const uint32_t first = static_cast<uint32_t>(until_wrap < rows_j ? until_wrap : rows_j);
                            unsigned char* wdst = dst + static_cast<size_t>(1 + p) * chunk_bytes(P);
                            bulk_load(smem_u32(wdst), a.weights + w0, first * 32, bar);
                            if (first < rows_j) bulk_load(smem_u32(wdst + first * 32), a.weights, (rows_j - first) * 32, bar);
                        }
                    };
                    uint32_t issued = 0;
                    if (lane == 0)
                        for (; issued < kStages - 1 && issued < chunks; ++issued) issue(issued);
                    issued = __shfl_sync(0xffffffffu, issued, 0);
                    bool ok = true;
                    const uint32_t g = lane >> 2, t = lane & 3;
                    int32_t c[P][2][4][4];
                    uint32_t(*total)[kAccLimbs] = totals[warp_in_cta];
#pragma unroll
                    for (int p = 0; p < P; ++p)
                    {
#pragma unroll
                        for (int i = 0; i < 32; ++i) (&c[p][0][0][0])[i] = 0;
                        if (lane == 0)
                        {
#pragma unroll
                            for (int i = 0; i < kAccLimbs; ++i) total[p][i] = 0;
                        }
                    }
                    uint32_t steps_unfolded = 0;
                    for (uint32_t ch = 0; ch < chunks; ++ch)
                    {
                        if (issued < chunks)
                        {
                            if (lane == 0) issue(issued);
                            ++issued;
                        }
                        const uint32_t slot = (ring_pos + ch) % kStages;
                        const uint32_t parity = ((ring_pos + ch) / kStages) & 1u;
                        ok = mbar_wait(smem_u32(bars + slot), parity, a.wait_limit);
                        if (!__all_sync(0xffffffffu, ok))
                        {
                            ok = false;
                            break;
                        }
                        unsigned char* stage = ring + static_cast<size_t>(slot) * slot_bytes(P);
                        const uint64_t row0 = static_cast<uint64_t>(ch) * kRows;
                        const uint32_t rows_here = static_cast<uint32_t>(rows - row0 < kRows ? rows - row0 : kRows);
#pragma unroll
                        for (uint32_t step = 0; step < kRows / 32; ++step)
                        {
                            if (step * 32 >= rows_here) break;
                            uint32_t fb[2][4];
                            load_rows_transposed(stage + step * 1024, g, t, fb);
                            if (rows_here < (step + 1) * 32)
                            {
                                // a ragged last chunk: the rows behind it hold older data, their bytes count as zero
#pragma unroll
                                for (int h = 0; h < 2; ++h)
                                {
                                    uint32_t keep = 0;
#pragma unroll
                                    for (int q = 0; q < 4; ++q)
                                        if (step * 32 + 16 * h + t + 4 * q < rows_here) keep |= 0xffu << (8 * q);
#pragma unroll
                                    for (int j = 0; j < 4; ++j) fb[h][j] &= keep;
                                }
                            }
#pragma unroll
                            for (int p = 0; p < P; ++p)
                            {
                                uint32_t wa[2][4];
                                load_rows_transposed(stage + static_cast<size_t>(1 + p) * chunk_bytes(P) + step * 1024, g, t, wa);
#pragma unroll
                                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                                    for (int nt = 0; nt < 4; ++nt)
                                        mma_u8(c[p][mt][nt], wa[0][2 * mt], wa[0][2 * mt + 1], wa[1][2 * mt], wa[1][2 * mt + 1], fb[0][nt], fb[1][nt]);
                            }
                            ++steps_unfolded;
                        }
                        if (steps_unfolded + kRows / 32 > kStepsPerFold || ch + 1 == chunks)
                        {
                            // the slot just read is this warp's until the next chunk is requested into it
#pragma unroll
                            for (int p = 0; p < P; ++p) fold_byte_products(c[p], stage, lane, total[p]);
                            steps_unfolded = 0;
                        }
                        __syncwarp();  // the slot may be refilled from the next iteration on
                    }
                    if (!ok)
                    {
                        // a copy never completed: flag it, give the copies still in flight a
                        // bounded chance to land, and leave
                        if (lane == 0) raise_status(a.status, GZK_E_TIMEOUT, 601);
                        for (uint32_t j = 0; j < issued && j < chunks; ++j)
                            mbar_wait(smem_u32(bars + (ring_pos + j) % kStages), ((ring_pos + j) / kStages) & 1u, a.wait_limit);
                        return;
                    }
                    ring_pos += chunks;
                    if (lane == 0)
                    {
#pragma unroll
                        for (int p = 0; p < P; ++p)
                        {
                            uint32_t* dst = a.partial + ((static_cast<uint64_t>(tile) * P + p) * a.k_count + k) * kAccLimbs;
#pragma unroll
                            for (int i = 0; i < kAccLimbs; ++i) dst[i] = total[p][i];
                        }
                    }
                    continue;
                }
                if constexpr (MODE != kFieldKinds)
                {
                if (kind == GZK_KIND_FR || kind == GZK_KIND_FR_MONT) continue;  // not this launch's
                WideAcc64 acc[P];
#pragma unroll
                for (int p = 0; p < P; ++p) acc[p].clear();
                if (kind == GZK_KIND_U32)
                {
                    const uint32_t* values = static_cast<const uint32_t*>(col);
                    for (uint64_t c = c_begin + lane; c < c_end; c += 32)
                    {
                        const uint32_t f = __ldcs(values + c);
#pragma unroll
                        for (int p = 0; p < P; ++p)
                        {
                            const Fr w = load_fr(a.weights + ((c - a.rot[p]) & a.mask));
                            acc[p].template mac<1>(w.l, &f);
                        }
                    }
                }
                else
                {
                    // I64, FieldElement::from_signed: v < 0 stands for r - |v|.  w * (r - |v|)
                    // is congruent to (r - w) * |v|, which keeps the product 8 x 2 limbs.
                    const long long* values = static_cast<const long long*>(col);
                    uint64_t c = c_begin + lane;
                    // A few rows per lane at a time: their values and weights are all requested before the first
                    // product, so the loop waits for memory once per group instead of once per row (with one row in
                    // flight per lane this path ran at a sixth of its instruction rate).
                    constexpr int kGroup = P == 1 ? 4 : 2;
                    for (; c + 32ull * (kGroup - 1) < c_end; c += 32ull * kGroup)
                    {
                        long long v[kGroup];
                        Fr w[kGroup][P];
#pragma unroll
                        for (int u = 0; u < kGroup; ++u) v[u] = __ldcs(values + c + 32ull * u);
#pragma unroll
                        for (int u = 0; u < kGroup; ++u)
#pragma unroll
                            for (int p = 0; p < P; ++p) w[u][p] = load_fr(a.weights + ((c + 32ull * u - a.rot[p]) & a.mask));
#pragma unroll
                        for (int u = 0; u < kGroup; ++u)
                        {
                            const unsigned long long mag = v[u] < 0 ? 0ULL - static_cast<unsigned long long>(v[u]) : static_cast<unsigned long long>(v[u]);
                            const uint32_t f[2] = {static_cast<uint32_t>(mag), static_cast<uint32_t>(mag >> 32)};
#pragma unroll
                            for (int p = 0; p < P; ++p)
                            {
                                const Fr signed_w = v[u] < 0 ? sub(Fr::zero(), w[u][p]) : w[u][p];
                                if (f[1] == 0)
                                    acc[p].template mac<1>(signed_w.l, f);
                                else
                                    acc[p].template mac<2>(signed_w.l, f);
                            }
                        }
                    }
                    for (; c < c_end; c += 32)
                    {
                        const long long v = __ldcs(values + c);
                        const unsigned long long mag = v < 0 ? 0ULL - static_cast<unsigned long long>(v) : static_cast<unsigned long long>(v);
                        const uint32_t f[2] = {static_cast<uint32_t>(mag), static_cast<uint32_t>(mag >> 32)};
#pragma unroll
                        for (int p = 0; p < P; ++p)
                        {
                            Fr w = load_fr(a.weights + ((c - a.rot[p]) & a.mask));
                            if (v < 0) w = sub(Fr::zero(), w);
                            if (f[1] == 0)  // witness values are a few dozen bits at most
                                acc[p].template mac<1>(w.l, f);
                            else
                                acc[p].template mac<2>(w.l, f);
                        }
                    }
                }
                // exact integer sum across the warp
#pragma unroll
                for (int p = 0; p < P; ++p)
                {
                    uint32_t sum[kAccLimbs];
                    acc[p].fold(sum);
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
                        uint32_t* dst = a.partial + ((static_cast<uint64_t>(tile) * P + p) * a.k_count + k) * kAccLimbs;
#pragma unroll
                        for (int i = 0; i < kAccLimbs; ++i) dst[i] = sum[i];
                    }
                }
                }
            }
        }

        // ---- small-integer columns on the tensor cores ----------------------------------------
        // The same byte products for I64 / U32 columns, four columns to a unit: the 4 x 8 value bytes of a row of
        // the group are the 32 columns of the product, the weights' 32 bytes its rows.  A signed value enters as
        // its two's-complement bytes u = v + 2^64 [v < 0]; a fifth block of columns holds the bit [v < 0], whose
        // products sum the weights of the negative rows, N, and the unit's sum is  sum w u - 2^64 N  (+ r 2^84, a
        // multiple of the modulus that keeps the 17-limb partial sum non-negative).  Lane (g, t) takes word g & 1
        // of column g / 2 (rows t, t+4, t+8, t+12 (+16): each load instruction reads whole 32-byte sectors of the
        // four columns) and word g of the weight rows (whole 128-byte lines), straight from global memory / L2,
        // one step (32 rows) ahead of the arithmetic.
        constexpr int kGroupColumns = 4;
        constexpr int kIntMatrixStride = 37;  // 32 value columns + 4 sign columns, odd
        struct IntegerScratch
        {
            int32_t matrix[32 * kIntMatrixStride];
            unsigned long long diagonal[kGroupColumns][40];
        };

        template <int P>
        __device__ __forceinline__ void fold_integer_group(int32_t cv[2][4][4], int32_t cs[2][4], IntegerScratch& scratch, uint32_t lane,
                                                           uint32_t (*total)[kAccLimbs])
        {
            const uint32_t g = lane >> 2, t = lane & 3;
            __syncwarp();
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i)
                {
                    const uint32_t a = 4 * g + 2 * mt + (i >> 1);
                    const uint32_t n = 2 * t + (i & 1);  // B column: column n / 2 of the group, word n & 1
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
                    {
                        scratch.matrix[a * kIntMatrixStride + (n >> 1) * 8 + 4 * (n & 1) + nt] = cv[mt][nt][i];
                        cv[mt][nt][i] = 0;
                    }
                    if (n & 1) scratch.matrix[a * kIntMatrixStride + 32 + (n >> 1)] = cs[mt][i];
                    cs[mt][i] = 0;
                }
            __syncwarp();
            {
                // lane -> column lane / 8, diagonals a + b = lane % 8 + 8 j
                const uint32_t c = lane >> 3, e = lane & 7;
#pragma unroll
                for (int j = 0; j < 5; ++j)
                {
                    const uint32_t d = e + 8 * j;
                    unsigned long long sum = 0;
#pragma unroll
                    for (uint32_t b = 0; b < 8; ++b)
                        if (d >= b && d - b < 32) sum += static_cast<uint32_t>(scratch.matrix[(d - b) * kIntMatrixStride + c * 8 + b]);
                    scratch.diagonal[c][d] = sum;  // d = 39: nothing lies on it, 0
                }
            }
            __syncwarp();
            if (lane < kGroupColumns)
            {
                const uint32_t c = lane;
                // value part: limb j collects the diagonals 4j .. 4j+3
                uint32_t value[kAccLimbs], odd[kAccLimbs], negative[kAccLimbs];
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) value[i] = odd[i] = negative[i] = 0;
#pragma unroll
                for (int j = 0; j < 10; ++j)
                {
                    const unsigned long long x = scratch.diagonal[c][4 * j] + (scratch.diagonal[c][4 * j + 1] << 8) + (scratch.diagonal[c][4 * j + 2] << 16) +
                                                 (scratch.diagonal[c][4 * j + 3] << 24);
                    uint32_t* into = (j & 1) ? odd : value;
                    into[j] = static_cast<uint32_t>(x);
                    into[j + 1] = static_cast<uint32_t>(x >> 32);
                }
                acc_add<kAccLimbs, kAccLimbs>(value, odd);
                // + r * 2^84
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) odd[i] = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                {
                    odd[i + 2] |= FrCfg::mod(i) << 20;
                    odd[i + 3] |= FrCfg::mod(i) >> 12;
                }
                acc_add<kAccLimbs, kAccLimbs>(value, odd);
                // - 2^64 * sum_a S[a] 2^(8a): limb j collects rows 4j .. 4j+3 of the sign column
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) odd[i] = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    unsigned long long y = 0;
#pragma unroll
                    for (int q = 0; q < 4; ++q) y += static_cast<unsigned long long>(static_cast<uint32_t>(scratch.matrix[(4 * j + q) * kIntMatrixStride + 32 + c])) << (8 * q);
                    uint32_t* into = (j & 1) ? odd : negative;
                    into[j + 2] = static_cast<uint32_t>(y);
                    into[j + 3] = static_cast<uint32_t>(y >> 32);
                }
                acc_add<kAccLimbs, kAccLimbs>(negative, odd);
                detail::limbs_sub<kAccLimbs>(value, negative);
                uint32_t sum[kAccLimbs];
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) sum[i] = total[c][i];
                acc_add<kAccLimbs, kAccLimbs>(sum, value);
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) total[c][i] = sum[i];
            }
            __syncwarp();
        }

        // The words reach the arithmetic through a per-warp ring in shared memory, filled by 16-byte cp.async
        // copies one or two chunks (64 rows) ahead: a copy clips itself at the end of the column and fills the
        // rest with zeros, follows the rotation and the wrap of the weight rows piece by piece, and keeps several
        // KiB per warp in flight (with plain loads one step ahead this kernel waited for memory most of the time).
        constexpr int kIntChunkRows = 64;
        constexpr int kIntColumnStride = kIntChunkRows * 8 + 32;  // + 8 words: the four columns start in different banks
        __host__ __device__ constexpr int int_stages(int) { return 2; }
        __host__ __device__ constexpr size_t int_stage_bytes(int p) { return static_cast<size_t>(kGroupColumns) * kIntColumnStride + static_cast<size_t>(p) * kIntChunkRows * 32; }
        __host__ __device__ constexpr size_t int_smem_bytes(int p) { return static_cast<size_t>(kWarps) * int_stages(p) * int_stage_bytes(p); }

        __device__ __forceinline__ void copy16(unsigned char* dst, const void* src, uint32_t src_bytes)
        {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
        }

        template <int P>
        __global__ void __launch_bounds__(kThreads, 3) eval_integers_kernel(EvalArgs a)
        {
            extern __shared__ __align__(128) unsigned char smem[];
            __shared__ IntegerScratch scratch_of[kWarps];
            __shared__ uint32_t totals[kWarps][P][kGroupColumns][kAccLimbs];
            constexpr int kStagesHere = int_stages(P);
            const uint32_t lane = threadIdx.x & 31;
            const uint32_t warp_in_cta = threadIdx.x >> 5;
            const uint32_t g = lane >> 2, t = lane & 3;
            const uint32_t my_column = g >> 1, my_word = g & 1;
            IntegerScratch& scratch = scratch_of[warp_in_cta];
            unsigned char* ring = smem + static_cast<size_t>(warp_in_cta) * kStagesHere * int_stage_bytes(P);
            const uint64_t warp = (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
            const uint64_t warps = (static_cast<uint64_t>(gridDim.x) * kThreads) >> 5;
            const uint32_t groups = (a.k_mapped + kGroupColumns - 1) / kGroupColumns;
            const uint64_t units = static_cast<uint64_t>(a.tiles) * groups;
            const unsigned char* weight_bytes = reinterpret_cast<const unsigned char*>(a.weights);
            for (uint64_t u = warp; u < units; u += warps)
            {
                const uint32_t tile = static_cast<uint32_t>(u / groups);
                const uint32_t group = static_cast<uint32_t>(u - static_cast<uint64_t>(tile) * groups);
                const uint64_t c_begin = static_cast<uint64_t>(tile) * a.tile_rows;
                const uint64_t c_end = c_begin + a.tile_rows < a.len ? c_begin + a.tile_rows : a.len;
                const uint64_t rows = c_end > c_begin ? c_end - c_begin : 0;
                const uint32_t chunks = static_cast<uint32_t>((rows + kIntChunkRows - 1) / kIntChunkRows);
                // the group's columns (the same for every lane) and this lane's own
                const unsigned char* column_of[kGroupColumns];
                bool wide_of[kGroupColumns];
#pragma unroll
                for (int c = 0; c < kGroupColumns; ++c)
                {
                    const uint32_t slot = group * kGroupColumns + c;
                    const bool there = slot < a.k_mapped;
                    const uint32_t k = there ? a.k_map[slot] : 0;
                    column_of[c] = there ? static_cast<const unsigned char*>(a.cols[k]) : nullptr;
                    wide_of[c] = there && a.kinds[k] == GZK_KIND_I64;
                }
                const bool present = group * kGroupColumns + my_column < a.k_mapped;
                bool wide = false;
#pragma unroll
                for (int c = 0; c < kGroupColumns; ++c)
                    if (c == static_cast<int>(my_column)) wide = wide_of[c];
                const bool reads = present && (wide || my_word == 0);
                if (lane < P * kGroupColumns)
                {
#pragma unroll
                    for (int i = 0; i < kAccLimbs; ++i) totals[warp_in_cta][lane / kGroupColumns][lane % kGroupColumns][i] = 0;
                }
                int32_t cv[P][2][4][4], cs[P][2][4];
#pragma unroll
                for (int p = 0; p < P; ++p)
                {
#pragma unroll
                    for (int i = 0; i < 32; ++i) (&cv[p][0][0][0])[i] = 0;
#pragma unroll
                    for (int i = 0; i < 8; ++i) (&cs[p][0][0])[i] = 0;
                }
                auto request = [&](uint32_t chunk) {
                    unsigned char* stage = ring + static_cast<size_t>(chunk % kStagesHere) * int_stage_bytes(P);
                    const uint64_t row0 = c_begin + static_cast<uint64_t>(chunk) * kIntChunkRows;
                    const uint64_t left = c_end - row0;  // rows of the column from here on (> 0)
#pragma unroll
                    for (int c = 0; c < kGroupColumns; ++c)
                    {
                        if (column_of[c] == nullptr) continue;
                        // 16 bytes = 2 rows of an I64 column (32 pieces per chunk), 4 rows of a U32 column (16 pieces)
                        const uint32_t rows_per_piece = wide_of[c] ? 2 : 4, row_bytes = wide_of[c] ? 8 : 4;
                        if (lane * rows_per_piece >= static_cast<uint32_t>(kIntChunkRows)) continue;
                        const uint64_t first = static_cast<uint64_t>(lane) * rows_per_piece;
                        const uint32_t bytes = first >= left ? 0u : static_cast<uint32_t>((left - first < rows_per_piece ? left - first : rows_per_piece) * row_bytes);
                        const unsigned char* src = bytes != 0 ? column_of[c] + (row0 + first) * row_bytes : column_of[c];
                        copy16(stage + c * kIntColumnStride + lane * 16, src, bytes);
                    }
#pragma unroll
                    for (int p = 0; p < P; ++p)
#pragma unroll
                        for (int i = 0; i < kIntChunkRows * 2 / 32; ++i)
                        {
                            const uint32_t piece = lane + 32 * i, row = piece >> 1;
                            const bool inside = row < left;
                            const unsigned char* src = inside ? weight_bytes + ((row0 + row - a.rot[p]) & a.mask) * 32 + (piece & 1) * 16 : weight_bytes;
                            copy16(stage + kGroupColumns * kIntColumnStride + p * kIntChunkRows * 32 + piece * 16, src, inside ? 16u : 0u);
                        }
                };
                // chunk ch is in flight kStagesHere - 1 iterations before it is read; one group per iteration
#pragma unroll
                for (int ahead = 0; ahead < kStagesHere - 1; ++ahead)
                {
                    if (static_cast<uint32_t>(ahead) < chunks) request(ahead);
                    asm volatile("cp.async.commit_group;" ::: "memory");
                }
                uint32_t steps_unfolded = 0;
                for (uint32_t ch = 0; ch < chunks; ++ch)
                {
                    if (ch + kStagesHere - 1 < chunks) request(ch + kStagesHere - 1);
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    asm volatile("cp.async.wait_group %0;" ::"n"(kStagesHere - 1) : "memory");
                    __syncwarp();
                    const unsigned char* stage = ring + static_cast<size_t>(ch % kStagesHere) * int_stage_bytes(P);
                    const uint64_t left = rows - static_cast<uint64_t>(ch) * kIntChunkRows;
#pragma unroll
                    for (uint32_t step = 0; step < kIntChunkRows / 32; ++step)
                    {
                        if (step * 32 >= left) break;
                        uint32_t fb[2][4], sb[2];
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                        {
                            uint32_t x[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                            {
                                const uint32_t row = step * 32 + 16 * h + t + 4 * q;
                                const uint32_t* words = reinterpret_cast<const uint32_t*>(stage + my_column * kIntColumnStride);
                                x[q] = reads ? words[wide ? 2 * row + my_word : row] : 0u;
                            }
                            const uint32_t t0 = __byte_perm(x[0], x[1], 0x5140), t1 = __byte_perm(x[2], x[3], 0x5140);
                            const uint32_t t2 = __byte_perm(x[0], x[1], 0x7362), t3 = __byte_perm(x[2], x[3], 0x7362);
                            fb[h][0] = __byte_perm(t0, t1, 0x5410);
                            fb[h][1] = __byte_perm(t0, t1, 0x7632);
                            fb[h][2] = __byte_perm(t2, t3, 0x5410);
                            fb[h][3] = __byte_perm(t2, t3, 0x7632);
                            sb[h] = (wide && my_word == 1) ? ((fb[h][3] >> 7) & 0x01010101u) : 0u;
                        }
#pragma unroll
                        for (int p = 0; p < P; ++p)
                        {
                            uint32_t wa[2][4];
                            load_rows_transposed(stage + kGroupColumns * kIntColumnStride + p * kIntChunkRows * 32 + step * 1024, g, t, wa);
#pragma unroll
                            for (int mt = 0; mt < 2; ++mt)
                            {
#pragma unroll
                                for (int nt = 0; nt < 4; ++nt)
                                    mma_u8(cv[p][mt][nt], wa[0][2 * mt], wa[0][2 * mt + 1], wa[1][2 * mt], wa[1][2 * mt + 1], fb[0][nt], fb[1][nt]);
                                mma_u8(cs[p][mt], wa[0][2 * mt], wa[0][2 * mt + 1], wa[1][2 * mt], wa[1][2 * mt + 1], sb[0], sb[1]);
                            }
                        }
                        ++steps_unfolded;
                    }
                    if (steps_unfolded + kIntChunkRows / 32 > kStepsPerFold || ch + 1 == chunks)
                    {
#pragma unroll
                        for (int p = 0; p < P; ++p) fold_integer_group<P>(cv[p], cs[p], scratch, lane, totals[warp_in_cta][p]);
                        steps_unfolded = 0;
                    }
                    __syncwarp();  // the stage is requested into again from the next iteration on
                }
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                __syncwarp();
                if (lane < kGroupColumns && group * kGroupColumns + lane < a.k_mapped)
                {
                    const uint32_t column = a.k_map[group * kGroupColumns + lane];
#pragma unroll
                    for (int p = 0; p < P; ++p)
                    {
                        uint32_t* dst = a.partial + ((static_cast<uint64_t>(tile) * P + p) * a.k_count + column) * kAccLimbs;
#pragma unroll
                        for (int i = 0; i < kAccLimbs; ++i) dst[i] = totals[warp_in_cta][p][lane][i];
                    }
                }
                __syncwarp();
            }
        }

        // ---- weighted column sums of a row-major small-integer matrix (gzk_fold_rows) -----------
        // out[j] = sum_i w[i] * M[i][j] is the packed evaluation of the matrix' columns, and four adjacent I64 columns
        // of a row are 32 contiguous bytes - the layout the group kernel wants of its four columns.  A unit is
        // (tile of rows, eight adjacent columns): two groups share one transposition of the weights.
        constexpr int kFoldGroups = 2;
        __host__ __device__ constexpr size_t fold_stage_bytes() { return static_cast<size_t>(kFoldGroups + 1) * kIntChunkRows * 32; }
        __host__ __device__ constexpr size_t fold_smem_bytes() { return static_cast<size_t>(kWarps) * 2 * fold_stage_bytes(); }

        __global__ void __launch_bounds__(kThreads, 3)
            fold_rows_groups_kernel(const unsigned char* matrix, const unsigned char* weights, uint64_t row_count, uint32_t cols, uint64_t tile_rows,
                                    uint32_t tiles, uint32_t* partial)
        {
            extern __shared__ __align__(128) unsigned char smem[];
            __shared__ IntegerScratch scratch_of[kWarps];
            __shared__ uint32_t totals[kWarps][kFoldGroups][kGroupColumns][kAccLimbs];
            const uint32_t lane = threadIdx.x & 31;
            const uint32_t warp_in_cta = threadIdx.x >> 5;
            const uint32_t g = lane >> 2, t = lane & 3;
            IntegerScratch& scratch = scratch_of[warp_in_cta];
            unsigned char* ring = smem + static_cast<size_t>(warp_in_cta) * 2 * fold_stage_bytes();
            const uint64_t warp = (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
            const uint64_t warps = (static_cast<uint64_t>(gridDim.x) * kThreads) >> 5;
            const uint32_t octets = cols / (kFoldGroups * kGroupColumns);
            const uint64_t units = static_cast<uint64_t>(tiles) * octets;
            const uint64_t row_bytes = static_cast<uint64_t>(cols) * 8;
            for (uint64_t u = warp; u < units; u += warps)
            {
                const uint32_t tile = static_cast<uint32_t>(u / octets);
                const uint32_t octet = static_cast<uint32_t>(u - static_cast<uint64_t>(tile) * octets);
                const uint64_t c_begin = static_cast<uint64_t>(tile) * tile_rows;
                const uint64_t c_end = c_begin + tile_rows < row_count ? c_begin + tile_rows : row_count;
                const uint64_t rows = c_end > c_begin ? c_end - c_begin : 0;
                const uint32_t chunks = static_cast<uint32_t>((rows + kIntChunkRows - 1) / kIntChunkRows);
                if (lane < kFoldGroups * kGroupColumns)
                {
#pragma unroll
                    for (int i = 0; i < kAccLimbs; ++i) totals[warp_in_cta][lane / kGroupColumns][lane % kGroupColumns][i] = 0;
                }
                int32_t cv[kFoldGroups][2][4][4], cs[kFoldGroups][2][4];
#pragma unroll
                for (int gi = 0; gi < kFoldGroups; ++gi)
                {
#pragma unroll
                    for (int i = 0; i < 32; ++i) (&cv[gi][0][0][0])[i] = 0;
#pragma unroll
                    for (int i = 0; i < 8; ++i) (&cs[gi][0][0])[i] = 0;
                }
                auto request = [&](uint32_t chunk) {
                    unsigned char* stage = ring + static_cast<size_t>(chunk & 1) * fold_stage_bytes();
                    const uint64_t row0 = c_begin + static_cast<uint64_t>(chunk) * kIntChunkRows;
                    const uint64_t left = c_end - row0;
                    // the eight columns of a row are 64 contiguous bytes: four pieces, two per group
#pragma unroll
                    for (int i = 0; i < kIntChunkRows * 4 / 32; ++i)
                    {
                        const uint32_t piece = lane + 32 * i, row = piece >> 2, part = piece & 3;
                        const bool inside = row < left;
                        const unsigned char* src = inside ? matrix + (row0 + row) * row_bytes + static_cast<uint64_t>(octet) * 64 + part * 16 : matrix;
                        copy16(stage + (part >> 1) * (kIntChunkRows * 32) + row * 32 + (part & 1) * 16, src, inside ? 16u : 0u);
                    }
#pragma unroll
                    for (int i = 0; i < kIntChunkRows * 2 / 32; ++i)
                    {
                        const uint32_t piece = lane + 32 * i, row = piece >> 1;
                        const bool inside = row < left;
                        const unsigned char* src = inside ? weights + (row0 + row) * 32 + (piece & 1) * 16 : weights;
                        copy16(stage + kFoldGroups * (kIntChunkRows * 32) + piece * 16, src, inside ? 16u : 0u);
                    }
                };
                if (chunks != 0) request(0);
                asm volatile("cp.async.commit_group;" ::: "memory");
                uint32_t steps_unfolded = 0;
                for (uint32_t ch = 0; ch < chunks; ++ch)
                {
                    if (ch + 1 < chunks) request(ch + 1);
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    asm volatile("cp.async.wait_group 1;" ::: "memory");
                    __syncwarp();
                    const unsigned char* stage = ring + static_cast<size_t>(ch & 1) * fold_stage_bytes();
                    const uint64_t left = rows - static_cast<uint64_t>(ch) * kIntChunkRows;
#pragma unroll
                    for (uint32_t step = 0; step < kIntChunkRows / 32; ++step)
                    {
                        if (step * 32 >= left) break;
                        uint32_t wa[2][4];
                        load_rows_transposed(stage + kFoldGroups * (kIntChunkRows * 32) + step * 1024, g, t, wa);
#pragma unroll
                        for (int gi = 0; gi < kFoldGroups; ++gi)
                        {
                            uint32_t fb[2][4], sb[2];
                            load_rows_transposed(stage + gi * (kIntChunkRows * 32) + step * 1024, g, t, fb);
                            sb[0] = (g & 1) ? ((fb[0][3] >> 7) & 0x01010101u) : 0u;  // word 1 of a column ends in its sign
                            sb[1] = (g & 1) ? ((fb[1][3] >> 7) & 0x01010101u) : 0u;
#pragma unroll
                            for (int mt = 0; mt < 2; ++mt)
                            {
#pragma unroll
                                for (int nt = 0; nt < 4; ++nt)
                                    mma_u8(cv[gi][mt][nt], wa[0][2 * mt], wa[0][2 * mt + 1], wa[1][2 * mt], wa[1][2 * mt + 1], fb[0][nt], fb[1][nt]);
                                mma_u8(cs[gi][mt], wa[0][2 * mt], wa[0][2 * mt + 1], wa[1][2 * mt], wa[1][2 * mt + 1], sb[0], sb[1]);
                            }
                        }
                        ++steps_unfolded;
                    }
                    if (steps_unfolded + kIntChunkRows / 32 > kStepsPerFold || ch + 1 == chunks)
                    {
#pragma unroll
                        for (int gi = 0; gi < kFoldGroups; ++gi) fold_integer_group<1>(cv[gi], cs[gi], scratch, lane, totals[warp_in_cta][gi]);
                        steps_unfolded = 0;
                    }
                    __syncwarp();
                }
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                __syncwarp();
                if (lane < kFoldGroups * kGroupColumns)
                {
                    uint32_t* dst = partial + (static_cast<uint64_t>(tile) * cols + octet * (kFoldGroups * kGroupColumns) + lane) * kAccLimbs;
#pragma unroll
                    for (int i = 0; i < kAccLimbs; ++i) dst[i] = totals[warp_in_cta][lane / kGroupColumns][lane % kGroupColumns][i];
                }
                __syncwarp();
            }
        }

        // ---- row-wise linear forms of a small-integer matrix (gzk_linear_form_rows) ----------------
        // out[i] = sum_j M[i][j] p_j: here the contraction runs along the contiguous bytes of a matrix row, so the
        // entries need no transposition at all - a 32-bit word of a row IS four consecutive contraction bytes of an
        // A fragment.  The other factor is a table, made once per call: P(8j + b) = p_j 2^(8b) mod r as a 32-byte
        // integer, stored in the order the B fragments want.  An entry enters as u = v + 2^63 (its top bit
        // flipped), 2^63 sum p_j is taken off every row.  A warp takes 32 rows; the 32 byte sums of a row are
        // spread over a quad of lanes, which adds them up and reduces one row per lane.
        __global__ void linear_form_table_kernel(const Fr* powers, uint32_t cols, unsigned char* table)
        {
            const uint32_t kappa = blockIdx.x * blockDim.x + threadIdx.x;  // 8j + b
            if (kappa >= cols * 8) return;
            Fr value = load_fr(powers + (kappa >> 3));
            for (uint32_t d = 0; d < 8 * (kappa & 7); ++d) value = add(value, value);
            const uint32_t step = kappa >> 5, within = kappa & 31, h = within >> 4, t = (within & 15) >> 2, q = within & 3;
#pragma unroll
            for (uint32_t n = 0; n < 32; ++n)
            {
                const uint32_t word = ((step * 4 + (n >> 3)) * 2 + h) * 32 + (n & 7) * 4 + t;
                table[word * 4 + q] = static_cast<unsigned char>(value.l[n >> 2] >> (8 * (n & 3)));
            }
        }

        // The rows reach the fragments through a per-warp ring: 32 rows x 256 bytes (8 contraction steps) per stage,
        // 16-byte cp.async copies (coalesced along the rows; a copy behind the last entry fills zeros), rows padded
        // to 272 bytes so that the eight rows a load instruction touches sit in different banks.
        constexpr int kFormStepsPerChunk = 8;
        constexpr int kFormRowStride = kFormStepsPerChunk * 32 + 16;
        __host__ __device__ constexpr size_t form_stage_bytes() { return static_cast<size_t>(32) * kFormRowStride; }
        __host__ __device__ constexpr size_t form_smem_bytes() { return static_cast<size_t>(kWarps) * 2 * form_stage_bytes(); }

        __global__ void __launch_bounds__(kThreads) linear_form_tensor_kernel(const unsigned char* matrix, uint64_t rows, uint32_t cols, uint64_t total_entries,
                                                                              const uint32_t* table, const Fr* bias, Fr* out)
        {
            extern __shared__ __align__(128) unsigned char smem[];
            const uint32_t lane = threadIdx.x & 31;
            const uint32_t warp_in_cta = threadIdx.x >> 5;
            const uint32_t g = lane >> 2, t = lane & 3;
            unsigned char* ring = smem + static_cast<size_t>(warp_in_cta) * 2 * form_stage_bytes();
            const uint64_t warp = (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
            const uint64_t warps = (static_cast<uint64_t>(gridDim.x) * kThreads) >> 5;
            const uint32_t steps = cols / 4;
            const uint32_t chunks = (steps + kFormStepsPerChunk - 1) / kFormStepsPerChunk;
            const uint64_t row_bytes = static_cast<uint64_t>(cols) * 8;
            const uint64_t total_bytes = total_entries * 8;
            const uint32_t flip = (t & 1) ? 0x80000000u : 0u;  // odd words are the upper halves of the entries
            const Fr offset = load_fr(bias);
            constexpr uint32_t c288[8] = {0xcaaf6b13u, 0x355094eau, 0x69a568efu, 0xf6b10cb3u, 0x40cc3869u, 0xe2c926a6u, 0xed269aadu, 0x736a6d3bu};  // 2^288 mod r
            const uint64_t row_blocks = (rows + 31) / 32;
            const uint64_t my_blocks = warp < row_blocks ? (row_blocks - warp + warps - 1) / warps : 0;
            const uint64_t sequence = my_blocks * chunks;  // (row block, chunk) pairs of this warp, in order
            auto request = [&](uint64_t index) {
                const uint64_t block = warp + (index / chunks) * warps;
                const uint32_t chunk = static_cast<uint32_t>(index % chunks);
                unsigned char* stage = ring + static_cast<size_t>(index & 1) * form_stage_bytes();
                const uint32_t chunk_bytes = (steps - chunk * kFormStepsPerChunk < kFormStepsPerChunk ? steps - chunk * kFormStepsPerChunk : kFormStepsPerChunk) * 32;
#pragma unroll
                for (int i = 0; i < 32 * kFormStepsPerChunk * 2 / 32; ++i)
                {
                    const uint32_t piece = lane + 32 * i, row = piece >> 4, part = piece & 15;
                    if (part * 16 >= chunk_bytes) continue;
                    const uint64_t r = block * 32 + row;
                    const uint64_t at = r * row_bytes + static_cast<uint64_t>(chunk) * (kFormStepsPerChunk * 32) + part * 16;  // two entries
                    const uint32_t bytes = (r < rows && at < total_bytes) ? static_cast<uint32_t>(total_bytes - at < 16 ? total_bytes - at : 16) : 0u;
                    copy16(stage + row * kFormRowStride + part * 16, bytes != 0 ? matrix + at : matrix, bytes);
                }
            };
            if (sequence != 0) request(0);
            asm volatile("cp.async.commit_group;" ::: "memory");
            for (uint64_t turn = 0; turn < my_blocks; ++turn)
            {
                const uint64_t block = warp + turn * warps;
                int32_t c[2][4][4];
#pragma unroll
                for (int i = 0; i < 32; ++i) (&c[0][0][0])[i] = 0;
                for (uint32_t chunk = 0; chunk < chunks; ++chunk)
                {
                    const uint64_t index = turn * chunks + chunk;
                    if (index + 1 < sequence) request(index + 1);
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    asm volatile("cp.async.wait_group 1;" ::: "memory");
                    __syncwarp();
                    const unsigned char* stage = ring + static_cast<size_t>(index & 1) * form_stage_bytes();
                    const uint32_t steps_here = steps - chunk * kFormStepsPerChunk < kFormStepsPerChunk ? steps - chunk * kFormStepsPerChunk : kFormStepsPerChunk;
#pragma unroll 4
                    for (uint32_t local = 0; local < steps_here; ++local)
                    {
                        const uint32_t s = chunk * kFormStepsPerChunk + local;
                        uint32_t a[2][4], b[4][2];
#pragma unroll
                        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                            for (int half = 0; half < 2; ++half)
#pragma unroll
                                for (int k16 = 0; k16 < 2; ++k16)
                                    a[mt][half + 2 * k16] =
                                        *reinterpret_cast<const uint32_t*>(stage + (16 * mt + 8 * half + g) * kFormRowStride + 32 * local + 16 * k16 + 4 * t) ^ flip;
                        const uint32_t* tb = table + static_cast<size_t>(s) * 256 + lane;
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt)
                        {
                            b[nt][0] = __ldg(tb + (nt * 2) * 32);
                            b[nt][1] = __ldg(tb + (nt * 2 + 1) * 32);
                        }
#pragma unroll
                        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                            for (int nt = 0; nt < 4; ++nt) mma_u8(c[mt][nt], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b[nt][0], b[nt][1]);
                    }
                    __syncwarp();  // the stage is requested into again two turns on
                }
                // row sums: byte column n = 8 nt + 2 t + e of row (mt, half) sits in c[mt][nt][2 half + e]
                uint32_t mine[10];
#pragma unroll
                for (int i = 0; i < 10; ++i) mine[i] = 0;
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int half = 0; half < 2; ++half)
                    {
                        uint32_t sum[10];
#pragma unroll
                        for (int i = 0; i < 10; ++i) sum[i] = 0;
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt)
                        {
                            const unsigned long long v = static_cast<unsigned long long>(static_cast<uint32_t>(c[mt][nt][2 * half])) +
                                                         (static_cast<unsigned long long>(static_cast<uint32_t>(c[mt][nt][2 * half + 1])) << 8);
                            const unsigned long long low = v << (16 * t);
                            const unsigned long long high = t == 0 ? 0ull : v >> (64 - 16 * t);
                            uint32_t part[10];
#pragma unroll
                            for (int i = 0; i < 10; ++i) part[i] = 0;
                            part[2 * nt] = static_cast<uint32_t>(low);
                            part[2 * nt + 1] = static_cast<uint32_t>(low >> 32);
                            part[2 * nt + 2] = static_cast<uint32_t>(high);
                            acc_add<10, 10>(sum, part);
                        }
#pragma unroll
                        for (int across = 1; across <= 2; across <<= 1)
                        {
                            uint32_t other[10];
#pragma unroll
                            for (int i = 0; i < 10; ++i) other[i] = __shfl_xor_sync(0xffffffffu, sum[i], across);
                            acc_add<10, 10>(sum, other);
                        }
                        if (static_cast<int>(t) == 2 * mt + half)
                        {
#pragma unroll
                            for (int i = 0; i < 10; ++i) mine[i] = sum[i];
                        }
                    }
                // lane t of the quad finishes row (mt, half) = (t / 2, t % 2)
                const uint64_t r = block * 32 + 16 * (t >> 1) + 8 * (t & 1) + g;
                if (r < rows)
                {
                    const Fr shifted = redc_wide<FrCfg, 1>(mine);  // the sum * 2^-32 mod r
                    Fr back;
#pragma unroll
                    for (int i = 0; i < 8; ++i) back.l[i] = c288[i];
                    store_fr(out + r, sub(mul(shifted, back), offset));
                }
            }
        }

        // Resident CTAs per SM of the two kernel variants on the CURRENT device (queried once per
        // device; also opts the kernels into their dynamic shared-memory size, which is a
        // per-device attribute).  Allocates nothing.
        constexpr int kOptInDevices = 64;
        template <int P, int MODE>
        int occupancy_of()
        {
            int nb = 0;
            cudaError_t err;
            if (MODE == kIntegerKinds)
            {
                err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, eval_partial_kernel<P, kIntegerKinds>, kThreads, 0);
            }
            else if (MODE == kIntegerGroups)
            {
                cudaFuncSetAttribute(eval_integers_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(int_smem_bytes(P)));
                err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, eval_integers_kernel<P>, kThreads, int_smem_bytes(P));
            }
            else
            {
                cudaFuncSetAttribute(eval_partial_kernel<P, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes(P)));
                err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, eval_partial_kernel<P, MODE>, kThreads, smem_bytes(P));
            }
            return (err == cudaSuccess && nb > 0) ? nb : 1;
        }
        int blocks_per_sm(int p, int mode = kAllKinds)
        {
            static std::atomic<int> per_device[kOptInDevices][3][4];  // zero-initialised; contexts on several host threads may race to fill a slot with the same value
            int device = 0;
            cudaGetDevice(&device);
            const bool cacheable = device >= 0 && device < kOptInDevices;
            std::atomic<int>& cached = per_device[cacheable ? device : 0][p][mode];
            if (!cacheable || cached.load(std::memory_order_relaxed) == 0)
            {
                int nb = 1;
                if (p == 2)
                    nb = mode == kFieldKinds ? occupancy_of<2, kFieldKinds>() : mode == kIntegerKinds ? occupancy_of<2, kIntegerKinds>() : mode == kIntegerGroups ? occupancy_of<2, kIntegerGroups>() : occupancy_of<2, kAllKinds>();
                else
                    nb = mode == kFieldKinds ? occupancy_of<1, kFieldKinds>() : mode == kIntegerKinds ? occupancy_of<1, kIntegerKinds>() : mode == kIntegerGroups ? occupancy_of<1, kIntegerGroups>() : occupancy_of<1, kAllKinds>();
                cached.store(nb, std::memory_order_relaxed);
            }
            return cached.load(std::memory_order_relaxed);
        }

        // Stall injection for tests of the bounded waits (gzk_debug_inject_eval_stall).
        std::atomic<int> g_inject_stall{0};
        constexpr uint32_t kInjectedWaitLimit = 1u << 10;

        template <int P>
        void launch_mode(cudaStream_t stream, const EvalArgs& args, int mode, unsigned blocks)
        {
            if (mode == kFieldKinds)
                eval_partial_kernel<P, kFieldKinds><<<blocks, kThreads, smem_bytes(P), stream>>>(args);
            else if (mode == kIntegerGroups)
                eval_integers_kernel<P><<<blocks, kThreads, int_smem_bytes(P), stream>>>(args);
            else if (mode == kIntegerKinds)
                eval_partial_kernel<P, kIntegerKinds><<<blocks, kThreads, 0, stream>>>(args);
            else
                eval_partial_kernel<P, kAllKinds><<<blocks, kThreads, smem_bytes(P), stream>>>(args);
        }
        // `mode` says which columns args.k_map lists (kAllKinds without a map).  Returns the CTAs launched.
        unsigned launch_eval_partial(cudaStream_t stream, EvalArgs args, int p, int sm_count, int mode = kAllKinds, unsigned blocks_per_sm_cap = 0)
        {
            const int per_sm = blocks_per_sm(p, mode);  // also makes sure the shared-memory opt-in has happened on this device
            const bool inject = g_inject_stall.load(std::memory_order_relaxed) != 0;
            args.wait_limit = inject ? kInjectedWaitLimit : kWaitLimit;
            args.skip_copies = inject ? 1u : 0u;
            if (args.k_map == nullptr) args.k_mapped = args.k_count;
            const uint64_t units = static_cast<uint64_t>(args.tiles) * (mode == kIntegerGroups ? (args.k_mapped + kGroupColumns - 1) / kGroupColumns : args.k_mapped);
            uint64_t blocks = (units + (kThreads / 32) - 1) / (kThreads / 32);
            const uint64_t max_blocks = static_cast<uint64_t>(sm_count) * (blocks_per_sm_cap != 0 && blocks_per_sm_cap < static_cast<unsigned>(per_sm) ? blocks_per_sm_cap : static_cast<unsigned>(per_sm));
            if (blocks > max_blocks) blocks = max_blocks;
            if (blocks == 0) return 0;
            if (p == 2)
                launch_mode<2>(stream, args, mode, static_cast<unsigned>(blocks));
            else
                launch_mode<1>(stream, args, mode, static_cast<unsigned>(blocks));
            return static_cast<unsigned>(blocks);
        }

        // One CTA per (rotation, column) pair: the threads sum the per-tile partials (up to 4096 of them: a
        // single warp walking them was a 40 us chain of dependent loads), four tiles requested at a time so that
        // a thread waits for memory once or twice, not once per tile; the warps and then the first warp add
        // them up exactly, thread 0 reduces once and writes the result.
        constexpr int kFinishThreads = 256;      // up to 1024 tiles
        constexpr int kFinishThreadsWide = 512;  // more
        constexpr int kFinishGroup = 4;
        inline unsigned finish_threads(uint32_t tiles) { return tiles > 1024 ? kFinishThreadsWide : kFinishThreads; }
        // `poison_status`: when given and raised (a bounded wait of the partial kernel gave up, so some
        // partial sums were never written), every output becomes 32 bytes of 0xFF - not a canonical
        // field element - instead of a sum over stale partials.
        __global__ void __launch_bounds__(kFinishThreadsWide)
            eval_finish_kernel(const uint32_t* partial, const int* kinds, uint32_t tiles, uint32_t p_count, uint32_t k_count, Fr* out_canonical,
                               int uniform_kind = -1, int out_montgomery = 0, const int* poison_status = nullptr)
        {
            __shared__ uint32_t warp_acc[kFinishThreadsWide / 32][kAccLimbs];
            const uint32_t lane = threadIdx.x & 31;
            const uint32_t threads = blockDim.x;
            const uint32_t idx = blockIdx.x;
            if (idx >= p_count * k_count) return;
            if (poison_status != nullptr && *poison_status != 0)
            {
                if (threadIdx.x == 0)
                {
                    Fr bad;
#pragma unroll
                    for (int i = 0; i < 8; ++i) bad.l[i] = 0xffffffffu;
                    store_fr(out_canonical + idx, bad);
                }
                return;
            }
            const uint32_t p = idx / k_count;
            const uint32_t k = idx - p * k_count;
            uint32_t acc[kAccLimbs];
#pragma unroll
            for (int i = 0; i < kAccLimbs; ++i) acc[i] = 0;
            const uint64_t tile_stride = static_cast<uint64_t>(p_count) * k_count * kAccLimbs;
            const uint32_t* mine = partial + (static_cast<uint64_t>(p) * k_count + k) * kAccLimbs;
            uint32_t tile = threadIdx.x;
            for (; tile + (kFinishGroup - 1) * threads < tiles; tile += kFinishGroup * threads)
            {
                uint32_t t[kFinishGroup][kAccLimbs];
#pragma unroll
                for (int g = 0; g < kFinishGroup; ++g)
                {
                    const uint32_t* src = mine + (tile + g * threads) * tile_stride;
#pragma unroll
                    for (int i = 0; i < kAccLimbs; ++i) t[g][i] = src[i];
                }
#pragma unroll
                for (int g = 0; g < kFinishGroup; ++g) acc_add<kAccLimbs, kAccLimbs>(acc, t[g]);
            }
            for (; tile < tiles; tile += threads)
            {
                const uint32_t* src = mine + tile * tile_stride;
                uint32_t t[kAccLimbs];
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) t[i] = src[i];
                acc_add<kAccLimbs, kAccLimbs>(acc, t);
            }
            auto warp_sum = [&]() {
#pragma unroll
                for (int offset = 16; offset > 0; offset >>= 1)
                {
                    uint32_t other[kAccLimbs];
#pragma unroll
                    for (int i = 0; i < kAccLimbs; ++i) other[i] = __shfl_down_sync(0xffffffffu, acc[i], offset);
                    acc_add<kAccLimbs, kAccLimbs>(acc, other);
                }
            };
            warp_sum();
            if (lane == 0)
            {
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) warp_acc[threadIdx.x >> 5][i] = acc[i];
            }
            __syncthreads();
            if (threadIdx.x >= 32) return;
            // the first warp: lane w takes the sum of warp w
#pragma unroll
            for (int i = 0; i < kAccLimbs; ++i) acc[i] = lane < (threads >> 5) ? warp_acc[lane][i] : 0u;
            warp_sum();
            if (lane != 0) return;
            // acc = 2^256 * S (canonical columns) or 2^512 * S (Montgomery columns), S the
            // true sum; 9 reduction rows divide by 2^288.
            const Fr reduced = redc_wide<FrCfg, 9>(acc);
            // reduced = S * 2^-32 (canonical columns) -> times 2^288 via Montgomery
            // product with 2^544;  S * 2^224 (Montgomery columns) -> times 2^32 via 2^288.
            Fr fix;
            if ((kinds != nullptr ? kinds[k] : uniform_kind) == GZK_KIND_FR_MONT)
            {
                constexpr uint32_t c288[8] = {0xcaaf6b13u, 0x355094eau, 0x69a568efu, 0xf6b10cb3u,
                                              0x40cc3869u, 0xe2c926a6u, 0xed269aadu, 0x736a6d3bu};
#pragma unroll
                for (int i = 0; i < 8; ++i) fix.l[i] = c288[i];
            }
            else
            {
                fix = fr_const_2_544();
            }
            const Fr mont = mul(reduced, fix);  // Montgomery form of S
            store_fr(out_canonical + idx, out_montgomery ? mont : from_mont(mont));
        }
    }
}

namespace gzk
{
    // gzk_fold_rows of an I64 matrix whose column count is a multiple of eight, on the tensor cores: chooses the
    // tiles (whole 64-row chunks; about one unit of eight columns per resident warp), returns them, and fills
    // partial[tile][column][17] (at least tiles x cols entries; at most 1024 tiles).
    uint32_t fold_rows_groups_tiles(gzk_ctx* ctx, size_t row_count, uint32_t cols, uint64_t* tile_rows_out)
    {
        int resident = 0;
        cudaFuncSetAttribute(fold_rows_groups_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(fold_smem_bytes()));
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, fold_rows_groups_kernel, kThreads, fold_smem_bytes()) != cudaSuccess || resident < 1) resident = 1;
        const uint64_t warps = static_cast<uint64_t>(ctx->sm_count) * resident * kWarps;
        const uint64_t octets = cols / (kFoldGroups * kGroupColumns);
        uint64_t tiles = warps / octets;  // rounded down: one unit for (nearly) every resident warp, no second round for a few of them
        const uint64_t max_tiles = (row_count + 4 * kIntChunkRows - 1) / (4 * kIntChunkRows);  // at least four chunks to a unit
        if (tiles > max_tiles) tiles = max_tiles;
        if (tiles > 1024) tiles = 1024;
        if (tiles == 0) tiles = 1;
        uint64_t tile_rows = (row_count + tiles - 1) / tiles;
        tile_rows = (tile_rows + kIntChunkRows - 1) / kIntChunkRows * kIntChunkRows;
        if (tile_rows == 0) tile_rows = kIntChunkRows;
        *tile_rows_out = tile_rows;
        return row_count == 0 ? 1u : static_cast<uint32_t>((row_count + tile_rows - 1) / tile_rows);
    }
    void launch_fold_rows_groups(gzk_ctx* ctx, const void* matrix, const Fr* weights, size_t row_count, uint32_t cols, uint64_t tile_rows, uint32_t tiles,
                                 uint32_t* partial)
    {
        int resident = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, fold_rows_groups_kernel, kThreads, fold_smem_bytes()) != cudaSuccess || resident < 1) resident = 1;
        const uint64_t units = static_cast<uint64_t>(tiles) * (cols / (kFoldGroups * kGroupColumns));
        uint64_t blocks = (units + kWarps - 1) / kWarps;
        const uint64_t max_blocks = static_cast<uint64_t>(ctx->sm_count) * resident;
        if (blocks > max_blocks) blocks = max_blocks;
        fold_rows_groups_kernel<<<static_cast<unsigned>(blocks), kThreads, fold_smem_bytes(), ctx->stream>>>(
            static_cast<const unsigned char*>(matrix), reinterpret_cast<const unsigned char*>(weights), row_count, cols, tile_rows, tiles, partial);
    }

    // gzk_linear_form_rows of an I64 matrix (cols a multiple of four) on the tensor cores.  `table` needs cols * 256
    // bytes; `bias` holds 2^63 * sum of the powers (Montgomery form); out receives Montgomery values.  Entries at
    // and behind total_entries count as zero.
    void launch_linear_form_tensor(gzk_ctx* ctx, const void* matrix, uint64_t rows, uint32_t cols, uint64_t total_entries, const Fr* powers, void* table,
                                   const Fr* bias, Fr* out)
    {
        linear_form_table_kernel<<<(cols * 8 + 255) / 256, 256, 0, ctx->stream>>>(powers, cols, static_cast<unsigned char*>(table));
        const uint64_t row_blocks = (rows + 31) / 32;
        uint64_t blocks = (row_blocks + kWarps - 1) / kWarps;
        const uint64_t max_blocks = static_cast<uint64_t>(ctx->sm_count) * 3;  // what the ring's shared memory lets an SM hold
        if (blocks > max_blocks) blocks = max_blocks;
        cudaFuncSetAttribute(linear_form_tensor_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(form_smem_bytes()));
        linear_form_tensor_kernel<<<static_cast<unsigned>(blocks), kThreads, form_smem_bytes(), ctx->stream>>>(static_cast<const unsigned char*>(matrix), rows, cols, total_entries,
                                                                                             static_cast<const uint32_t*>(table), bias, out);
    }

    // For the other inner-product kernels of the library, which produce partial sums
    // in the same [tile][p][k][17] layout: sum over tiles, reduce once, write results.
    int launch_eval_finish(gzk_ctx* ctx, const uint32_t* partial, int uniform_kind, uint32_t tiles, uint32_t k_count,
                           Fr* out, bool out_montgomery)
    {
        LaunchScope scope(ctx, "eval_finish");
        eval_finish_kernel<<<k_count, finish_threads(tiles), 0, ctx->stream>>>(partial, nullptr, tiles, 1, k_count, out, uniform_kind,
                                                                          out_montgomery ? 1 : 0);
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return GZK_OK;
    }
}

using namespace gzk;

// Shared body of gzk_eval_batch and gzk_eval_batch_range.  `rotations` are already the
// effective ones: row c of a column meets weights[(c - rotation) mod n] of the buffer.
// With `dest` set the results stay on the device (dest[p * k_count + k], Montgomery form when
// dest_montgomery) and the call ends like a builder call: no read-back, no synchronisation in
// deferred mode.
static int eval_batch_impl(gzk_ctx* ctx, gzk_buf* const* cols, size_t k_count, size_t len, unsigned log2n,
                           const gzk_buf* weights, const uint64_t* rotations, size_t p_count, uint8_t* out_host,
                           Fr* dest = nullptr, bool dest_montgomery = false)
{
    const uint64_t n = 1ULL << log2n;
    if (k_count > (1u << 20)) return fail(ctx, GZK_E_INVALID, "eval_batch: too many columns");
    for (size_t k = 0; k < k_count; ++k)
    {
        if (cols[k] == nullptr || cols[k]->count < len) return fail(ctx, GZK_E_INVALID, "eval_batch: column shorter than len");
    }
    for (size_t p = 0; p < p_count; ++p)
        if (rotations[p] >= n) return fail(ctx, GZK_E_INVALID, "eval_batch: rotation out of range");
    GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));

    // tile plan: enough (tile, column) units to keep every warp of the machine busy
    // several times over, but at most 256 tiles so the partial buffer stays small.
    const uint64_t resident_blocks = static_cast<uint64_t>(ctx->sm_count) * blocks_per_sm(p_count >= 2 ? 2 : 1);
    const uint64_t warps_total = resident_blocks * (kThreads / 32);
    uint64_t per_warp = 8;
#ifdef GZK_BUILD_TUNING
    if (const char* forced = std::getenv("GZK_EVAL_UNITS_PER_WARP")) per_warp = static_cast<uint64_t>(std::atoi(forced)) > 0 ? std::atoi(forced) : per_warp;
#endif
    uint64_t want_tiles = (per_warp * warps_total + k_count - 1) / k_count;
    uint64_t max_tiles = (len + 255) / 256;
    if (max_tiles == 0) max_tiles = 1;
    // the partial buffer (tiles x P x K x 68 B) is kept below 64 MiB, and below 4096 tiles
    uint64_t tile_cap = (64ull << 20) / (static_cast<uint64_t>(p_count >= 2 ? 2 : 1) * k_count * kAccLimbs * sizeof(uint32_t));
    if (tile_cap < 64) tile_cap = 64;
    if (tile_cap > 4096) tile_cap = 4096;
    if (want_tiles > tile_cap) want_tiles = tile_cap;
    if (want_tiles > max_tiles) want_tiles = max_tiles;
    if (want_tiles == 0) want_tiles = 1;
    // Every warp takes the same number of (tile, column) units, give or take one: among the tile counts close to
    // the wanted one take the one that leaves the fewest warps idle while the last units run.
    {
        uint64_t best = want_tiles;
        double best_waste = 2.0;
        for (uint64_t t = want_tiles; t >= 1 && t + want_tiles / 4 >= want_tiles; --t)
        {
            const uint64_t units = t * k_count;
            const uint64_t rounds = (units + warps_total - 1) / warps_total;
            const double waste = 1.0 - static_cast<double>(units) / static_cast<double>(rounds * warps_total);
            if (waste < best_waste - 1e-9)
            {
                best_waste = waste;
                best = t;
            }
        }
        want_tiles = best;
    }
    uint64_t tile_rows = (len + want_tiles - 1) / want_tiles;
    tile_rows = (tile_rows + kChunkRows - 1) / kChunkRows * kChunkRows;
    if (tile_rows == 0) tile_rows = kChunkRows;
    const uint32_t tiles = len == 0 ? 1 : static_cast<uint32_t>((len + tile_rows - 1) / tile_rows);

    // device-side tables and scratch
    // column pointers, kinds, and the column indices with the field-element columns first
    const size_t table_bytes = k_count * (sizeof(void*) + sizeof(int) + sizeof(uint32_t));
    const size_t table_padded = (table_bytes + 31) & ~static_cast<size_t>(31);
    // Host copy of the column table.  A call that reads results back ends with a synchronisation, so
    // it can stage through the context's pinned area; a call that leaves its results on the device
    // returns while its copy may still be queued, so its table lives in pageable memory of its own
    // (the runtime copies a pageable source to its staging area before cudaMemcpyAsync returns).
    void* h_table = nullptr;
    std::vector<unsigned char> pageable_table;
    int rc = GZK_OK;
    if (dest != nullptr)
    {
        pageable_table.resize(table_padded);
        h_table = pageable_table.data();
    }
    else if ((rc = ensure_pinned(ctx, table_padded + p_count * k_count * 32 + 64, &h_table)) != GZK_OK)
    {
        return rc;
    }
    void* d_table = nullptr;
    if ((rc = ensure_scratch(ctx, 0, table_padded + p_count * k_count * 32, &d_table)) != GZK_OK) return rc;
    const void** h_ptrs = static_cast<const void**>(h_table);
    int* h_kinds = reinterpret_cast<int*>(h_ptrs + k_count);
    uint32_t* h_map = reinterpret_cast<uint32_t*>(h_kinds + k_count);
    uint32_t field_columns = 0;
    for (size_t k = 0; k < k_count; ++k)
    {
        h_ptrs[k] = cols[k]->dptr;
        h_kinds[k] = cols[k]->kind;
        if (cols[k]->kind == GZK_KIND_FR || cols[k]->kind == GZK_KIND_FR_MONT) h_map[field_columns++] = static_cast<uint32_t>(k);
    }
    for (size_t k = 0, next = field_columns; k < k_count; ++k)
        if (cols[k]->kind != GZK_KIND_FR && cols[k]->kind != GZK_KIND_FR_MONT) h_map[next++] = static_cast<uint32_t>(k);
    GZK_CUDA_TRY(ctx, cudaMemcpyAsync(d_table, h_table, table_bytes, cudaMemcpyHostToDevice, ctx->stream));
    const void* const* d_ptrs = static_cast<const void* const*>(d_table);
    const int* d_kinds = reinterpret_cast<const int*>(static_cast<const char*>(d_table) + k_count * sizeof(void*));
    const uint32_t* d_map = reinterpret_cast<const uint32_t*>(d_kinds + k_count);
    Fr* d_out = dest != nullptr ? dest : reinterpret_cast<Fr*>(static_cast<char*>(d_table) + table_padded);
    if (dest != nullptr && (rc = begin_call(ctx)) != GZK_OK) return rc;

    uint8_t* h_out = static_cast<uint8_t*>(h_table) + table_padded;
    {
        // per launch pair: every column element once (4 / 8 / 32 bytes), the weights once per rotation
        uint64_t column_bytes = 0, limbs = 0;
        for (size_t k = 0; k < k_count; ++k)
        {
            const int kind = cols[k]->kind;
            column_bytes += len * (kind == GZK_KIND_U32 ? 4u : kind == GZK_KIND_I64 ? 8u : 32u);
            // an I64 value that fits one limb (every witness value in practice) takes the 8-product path, 16 otherwise:
            // counted at 8, so the reported integer-pipe rate is a lower bound
            limbs += len * (kind == GZK_KIND_U32 || kind == GZK_KIND_I64 ? 8u : 64u);
        }
        const uint64_t launches = (p_count + 1) / 2;
        ctx->eval_algorithmic_bytes += launches * column_bytes + p_count * len * 32;
        ctx->eval_limb_products += limbs * p_count;
        ctx->eval_terms += static_cast<uint64_t>(len) * k_count * p_count;
    }
    for (size_t p0 = 0; p0 < p_count; p0 += 2)
    {
        const uint32_t p_now = p_count - p0 >= 2 ? 2 : 1;
        void* d_partial = nullptr;
        const size_t partial_bytes = static_cast<size_t>(tiles) * p_now * k_count * kAccLimbs * sizeof(uint32_t);
        if ((rc = ensure_scratch(ctx, 1, partial_bytes, &d_partial)) != GZK_OK) return rc;
        EvalArgs args;
        args.cols = d_ptrs;
        args.kinds = d_kinds;
        args.weights = static_cast<const Fr*>(weights->dptr);
        args.len = len;
        args.mask = n - 1;
        args.tile_rows = tile_rows;
        args.tiles = tiles;
        args.k_count = static_cast<uint32_t>(k_count);
        args.rot[0] = rotations[p0];
        args.rot[1] = p_now == 2 ? rotations[p0 + 1] : 0;
        args.partial = static_cast<uint32_t*>(d_partial);
        args.status = ctx->d_status;
        {
            // one launch per kind of column present, over the same partial buffer
            if (field_columns != 0)
            {
                LaunchScope scope(ctx, p_now == 2 ? "eval_partial_p2" : "eval_partial_p1");
                args.k_map = d_map;
                args.k_mapped = field_columns;
                launch_eval_partial(ctx->stream, args, static_cast<int>(p_now), ctx->sm_count, kFieldKinds);
            }
            // Small-integer columns at two evaluation points: whole groups of four on the tensor cores, and three
            // left over too (a group costs what 2.7 columns cost on the integer pipe; 2^22 rows x 8 columns take
            // 200 us against 299 us).  At one point a group costs what 3.0 columns cost, and in the calls of a proof
            // (a handful of integer columns each, so two launches with two tails) the integer pipe alone was faster:
            // 7.0 ms against 7.6 ms per proof.
            const uint32_t integers = static_cast<uint32_t>(k_count) - field_columns;
            uint32_t grouped = 0;
            if (p_now == 2) grouped = integers % kGroupColumns == 3 ? integers : integers - integers % kGroupColumns;
            if (grouped != 0)
            {
                LaunchScope scope(ctx, p_now == 2 ? "eval_partial_integers_p2" : "eval_partial_integers_p1");
                args.k_map = d_map + field_columns;
                args.k_mapped = grouped;
                launch_eval_partial(ctx->stream, args, static_cast<int>(p_now), ctx->sm_count, kIntegerGroups);
            }
            if (grouped != integers)
            {
                LaunchScope scope(ctx, p_now == 2 ? "eval_partial_integers_p2" : "eval_partial_integers_p1");
                args.k_map = d_map + field_columns + grouped;
                args.k_mapped = integers - grouped;
                launch_eval_partial(ctx->stream, args, static_cast<int>(p_now), ctx->sm_count, kIntegerKinds);
            }
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        const uint32_t outs = p_now * static_cast<uint32_t>(k_count);
        {
            LaunchScope scope(ctx, "eval_finish");
            eval_finish_kernel<<<outs, finish_threads(tiles), 0, ctx->stream>>>(static_cast<const uint32_t*>(d_partial), d_kinds, tiles, p_now,
                                                                           static_cast<uint32_t>(k_count), d_out + p0 * k_count, -1,
                                                                           dest != nullptr && dest_montgomery ? 1 : 0);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
    }
    if (dest != nullptr) return finish_call(ctx, "eval_batch_device: invalid input");
    GZK_CUDA_TRY(ctx, cudaMemcpyAsync(h_out, d_out, p_count * k_count * 32, cudaMemcpyDeviceToHost, ctx->stream));
    int* h_status = reinterpret_cast<int*>(h_out + p_count * k_count * 32);
    GZK_CUDA_TRY(ctx, cudaMemcpyAsync(h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    if (*h_status == GZK_E_TIMEOUT)  // other codes belong to deferred calls and are reported by gzk_ctx_synchronize
    {
        GZK_CUDA_TRY(ctx, cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream));
        return fail(ctx, GZK_E_TIMEOUT, "eval_batch: a bounded wait on a bulk copy gave up");
    }
    std::memcpy(out_host, h_out, p_count * k_count * 32);
    return GZK_OK;
}


// ---------------------------------------------------------------------------------
// Packed evaluation for callers that must not allocate.
//
// gzk_eval_batch obtains its work area (the per-tile partial sums and the column
// pointer table) from the context, which grows it with cudaMalloc on demand.  Some
// users of this library cannot tolerate that: a prover host that has handed all of
// the GPU's memory to its own column pool has nothing left for cudaMalloc to give,
// and a cudaMalloc in the middle of a proof synchronises the whole device and
// stalls the other streams of the process.  For them this one entry point keeps
// its work area in a fixed array that is part of the loaded library image.
namespace
{
    constexpr size_t kStaticMaxColumns = 256;
    constexpr size_t kStaticMaxRotations = 2;
    constexpr size_t kStaticMaxTiles = 64;
    constexpr size_t kStaticTableBytes = kStaticMaxColumns * (sizeof(void*) + sizeof(int));  // 3 KiB
    constexpr size_t kStaticStatusOffset = 3584;  // one status word between the table and the partial sums
    constexpr size_t kStaticPartialOffset = 4096;
    constexpr size_t kStaticPartialBytes = kStaticMaxTiles * kStaticMaxRotations * kStaticMaxColumns * gzk::kAccLimbs * sizeof(uint32_t);
    constexpr size_t kStaticBytes = kStaticPartialOffset + kStaticPartialBytes;  // about 2.1 MiB per GPU
    static_assert(kStaticTableBytes <= kStaticStatusOffset, "pointer table must fit before the status word");

    // Held by every GPU that loads the library, until the process exits.
    static __device__ __align__(256) unsigned char g_eval_static_scratch[kStaticBytes];

    // In host code `g_eval_static_scratch` is only a handle for the runtime, not an
    // address a kernel can use; the device address is looked up once per device.
    constexpr int kMaxDevices = 64;
    void* g_static_addr[kMaxDevices] = {};
    int g_static_sms[kMaxDevices] = {};

    int static_fail(char* err, size_t cap, int code, const char* message)
    {
        if (err != nullptr && cap > 0)
        {
            std::strncpy(err, message, cap - 1);
            err[cap - 1] = '\0';
        }
        return code;
    }
}

extern "C" int gzk_eval_batch_static(int device, void* stream, const void* const* col_ptrs, const int* col_kinds,
                                     size_t k_count, size_t len, unsigned log2n, const void* weights_mont,
                                     const uint64_t* rotations, size_t p_count, void* out_device, char* err,
                                     size_t err_cap)
{
    if (k_count == 0 || p_count == 0) return GZK_OK;
    if (col_ptrs == nullptr || col_kinds == nullptr || weights_mont == nullptr || rotations == nullptr || out_device == nullptr)
        return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: null argument");
    if (device < 0 || device >= kMaxDevices) return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: device index out of range");
    if (k_count > kStaticMaxColumns)
        return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: more than 256 columns; split the batch or use gzk_eval_batch");
    if (p_count > kStaticMaxRotations)
        return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: more than 2 rotations; split the call or use gzk_eval_batch");
    if (log2n > 32) return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: domain too large");
    const uint64_t n = 1ULL << log2n;
    if (len > n) return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: len exceeds the domain size");
    for (size_t p = 0; p < p_count; ++p)
        if (rotations[p] >= n) return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: rotation out of range");
    // The kernels read field elements as 16-byte vectors and through 16-byte bulk copies: a
    // misaligned or foreign pointer would fault on the GPU, so it is refused here, before any
    // launch.  cudaPointerGetAttributes is a query; it allocates nothing.
    auto device_memory_ok = [&](const void* p, size_t align) {
        if (reinterpret_cast<uintptr_t>(p) % align != 0) return false;
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, p) != cudaSuccess)
        {
            cudaGetLastError();
            return false;
        }
        return attr.type == cudaMemoryTypeDevice && attr.device == device;
    };
    for (size_t k = 0; k < k_count; ++k)
    {
        if (col_ptrs[k] == nullptr) return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: null column pointer");
        if (col_kinds[k] < GZK_KIND_FR || col_kinds[k] > GZK_KIND_U32)
            return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: unknown column kind");
    }
    if (cudaSetDevice(device) != cudaSuccess) return static_fail(err, err_cap, GZK_E_CUDA, "eval_batch_static: cudaSetDevice failed");
    for (size_t k = 0; k < k_count; ++k)
    {
        const size_t align = col_kinds[k] == GZK_KIND_U32 ? 4 : col_kinds[k] == GZK_KIND_I64 ? 8 : 32;
        if (!device_memory_ok(col_ptrs[k], align))
            return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: a column pointer is misaligned (32 bytes for field elements, 8 for I64, 4 for U32) or is not memory of this GPU");
    }
    if (!device_memory_ok(weights_mont, 32) || !device_memory_ok(out_device, 32))
        return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: weights / output pointer is misaligned (32 bytes) or is not memory of this GPU");
    if (g_static_addr[device] == nullptr)
    {
        // one-time set-up for this device, with the device current
        void* addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_eval_static_scratch) != cudaSuccess || addr == nullptr)
            return static_fail(err, err_cap, GZK_E_CUDA, "eval_batch_static: cudaGetSymbolAddress failed");
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
            return static_fail(err, err_cap, GZK_E_CUDA, "eval_batch_static: cannot query the SM count");
        g_static_sms[device] = sms;
        g_static_addr[device] = addr;
    }
    unsigned char* scratch = static_cast<unsigned char*>(g_static_addr[device]);
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    // same tile plan as gzk_eval_batch, capped so the partial sums fit the array
    const uint64_t warps_total = static_cast<uint64_t>(g_static_sms[device]) * 2 * (kThreads / 32);
    uint64_t want_tiles = (8 * warps_total + k_count - 1) / k_count;
    uint64_t max_tiles = (len + 255) / 256;
    if (max_tiles == 0) max_tiles = 1;
    if (want_tiles > kStaticMaxTiles) want_tiles = kStaticMaxTiles;
    if (want_tiles > max_tiles) want_tiles = max_tiles;
    if (want_tiles == 0) want_tiles = 1;
    // Every warp takes the same number of (tile, column) units, give or take one: among the tile counts close to
    // the wanted one take the one that leaves the fewest warps idle while the last units run.
    {
        uint64_t best = want_tiles;
        double best_waste = 2.0;
        for (uint64_t t = want_tiles; t >= 1 && t + want_tiles / 4 >= want_tiles; --t)
        {
            const uint64_t units = t * k_count;
            const uint64_t rounds = (units + warps_total - 1) / warps_total;
            const double waste = 1.0 - static_cast<double>(units) / static_cast<double>(rounds * warps_total);
            if (waste < best_waste - 1e-9)
            {
                best_waste = waste;
                best = t;
            }
        }
        want_tiles = best;
    }
    uint64_t tile_rows = (len + want_tiles - 1) / want_tiles;
    tile_rows = (tile_rows + kChunkRows - 1) / kChunkRows * kChunkRows;
    if (tile_rows == 0) tile_rows = kChunkRows;
    const uint32_t tiles = len == 0 ? 1 : static_cast<uint32_t>((len + tile_rows - 1) / tile_rows);

    // pointer table: built on the stack, copied into the head of the array
    unsigned char table[kStaticTableBytes];
    std::memcpy(table, col_ptrs, k_count * sizeof(void*));
    std::memcpy(table + kStaticMaxColumns * sizeof(void*), col_kinds, k_count * sizeof(int));
    if (cudaMemcpyAsync(scratch, table, kStaticTableBytes, cudaMemcpyHostToDevice, s) != cudaSuccess)
        return static_fail(err, err_cap, GZK_E_CUDA, "eval_batch_static: copying the column table failed");
    // the array keeps what the previous call left: the status word must start at zero
    if (cudaMemsetAsync(scratch + kStaticStatusOffset, 0, sizeof(int), s) != cudaSuccess)
        return static_fail(err, err_cap, GZK_E_CUDA, "eval_batch_static: clearing the status word failed");

    EvalArgs args;
    args.cols = reinterpret_cast<const void* const*>(scratch);
    args.kinds = reinterpret_cast<const int*>(scratch + kStaticMaxColumns * sizeof(void*));
    args.weights = static_cast<const Fr*>(weights_mont);
    args.len = len;
    args.mask = n - 1;
    args.tile_rows = tile_rows;
    args.tiles = tiles;
    args.k_count = static_cast<uint32_t>(k_count);
    args.rot[0] = rotations[0];
    args.rot[1] = p_count == 2 ? rotations[1] : 0;
    args.partial = reinterpret_cast<uint32_t*>(scratch + kStaticPartialOffset);
    args.status = reinterpret_cast<int*>(scratch + kStaticStatusOffset);
    args.k_map = nullptr;  // at most two CTAs per SM
    launch_eval_partial(s, args, static_cast<int>(p_count), g_static_sms[device], kAllKinds, 2);
    if (cudaGetLastError() != cudaSuccess) return static_fail(err, err_cap, GZK_E_CUDA, "eval_batch_static: kernel launch failed");
    const uint32_t outs = static_cast<uint32_t>(p_count * k_count);
    eval_finish_kernel<<<outs, finish_threads(tiles), 0, s>>>(args.partial, args.kinds, tiles, static_cast<uint32_t>(p_count),
                                                         static_cast<uint32_t>(k_count), static_cast<Fr*>(out_device), -1, 0, args.status);
    if (cudaGetLastError() != cudaSuccess) return static_fail(err, err_cap, GZK_E_CUDA, "eval_batch_static: kernel launch failed");
    return GZK_OK;
}

// Test facility for the bounded waits of the packed-evaluation kernel: while switched on, every
// launch of that kernel (all contexts of the process, gzk_eval_batch_static included) arms its
// chunk barriers but issues no bulk copy and polls each barrier only a few hundred times, so the
// waits run out, the kernel raises its status word and returns with nothing in flight.
extern "C" int gzk_debug_inject_eval_stall(int on)
{
    g_inject_stall.store(on != 0 ? 1 : 0, std::memory_order_relaxed);
    return GZK_OK;
}

extern "C" int gzk_eval_batch(gzk_ctx* ctx, gzk_buf* const* cols, size_t k_count, size_t len, unsigned log2n,
                              const gzk_buf* weights, const uint64_t* rotations, size_t p_count, uint8_t* out_host)
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (k_count == 0 || p_count == 0) return GZK_OK;
    if (cols == nullptr || weights == nullptr || rotations == nullptr || out_host == nullptr)
        return fail(ctx, GZK_E_INVALID, "eval_batch: null argument");
    if (log2n > 32) return fail(ctx, GZK_E_INVALID, "eval_batch: domain too large");
    const uint64_t n = 1ULL << log2n;
    if (len > n) return fail(ctx, GZK_E_INVALID, "domain evaluation backend weight size mismatch");
    if (weights->kind != GZK_KIND_FR_MONT || weights->count < n)
        return fail(ctx, GZK_E_INVALID, "eval_batch: weights must be a Montgomery buffer of the domain size");
    return eval_batch_impl(ctx, cols, k_count, len, log2n, weights, rotations, p_count, out_host);
}

// Same sums as gzk_eval_batch, left on the device: out[out_offset + p * k_count + k], canonical for an
// FR buffer, Montgomery for an FR_MONT one.  Nothing is read back, so in deferred mode the call only
// queues kernels; the values feed device-side consumers (same-base G1 multiplication, an exchange
// between GPUs, gzk_fr_sum_device).
extern "C" int gzk_eval_batch_device(gzk_ctx* ctx, gzk_buf* const* cols, size_t k_count, size_t len, unsigned log2n,
                                     const gzk_buf* weights, const uint64_t* rotations, size_t p_count, gzk_buf* out, size_t out_offset)
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (k_count == 0 || p_count == 0) return GZK_OK;
    if (cols == nullptr || weights == nullptr || rotations == nullptr || out == nullptr)
        return fail(ctx, GZK_E_INVALID, "eval_batch_device: null argument");
    if (log2n > 32) return fail(ctx, GZK_E_INVALID, "eval_batch_device: domain too large");
    const uint64_t n = 1ULL << log2n;
    if (len > n) return fail(ctx, GZK_E_INVALID, "domain evaluation backend weight size mismatch");
    if (weights->kind != GZK_KIND_FR_MONT || weights->count < n)
        return fail(ctx, GZK_E_INVALID, "eval_batch_device: weights must be a Montgomery buffer of the domain size");
    if ((out->kind != GZK_KIND_FR && out->kind != GZK_KIND_FR_MONT) || out_offset + p_count * k_count > out->count)
        return fail(ctx, GZK_E_INVALID, "eval_batch_device: output must be an FR or FR_MONT buffer that holds p_count * k_count values at out_offset");
    return eval_batch_impl(ctx, cols, k_count, len, log2n, weights, rotations, p_count, nullptr, static_cast<Fr*>(out->dptr) + out_offset,
                           out->kind == GZK_KIND_FR_MONT);
}

// Row-sharded form with the partial sums left on the device (see gzk_eval_batch_range for the
// meaning of row_offset / weights_first).
extern "C" int gzk_eval_batch_range_device(gzk_ctx* ctx, gzk_buf* const* cols, size_t k_count, size_t len, uint64_t row_offset, unsigned log2n,
                                           const gzk_buf* weights, uint64_t weights_first, const uint64_t* rotations, size_t p_count,
                                           gzk_buf* out, size_t out_offset)
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (k_count == 0 || p_count == 0) return GZK_OK;
    if (cols == nullptr || weights == nullptr || rotations == nullptr || out == nullptr)
        return fail(ctx, GZK_E_INVALID, "eval_batch_range_device: null argument");
    if (log2n > 32) return fail(ctx, GZK_E_INVALID, "eval_batch_range_device: domain too large");
    const uint64_t n = 1ULL << log2n;
    if (len > n || row_offset >= n || weights_first >= n) return fail(ctx, GZK_E_INVALID, "eval_batch_range_device: range exceeds the domain");
    if (weights->kind != GZK_KIND_FR_MONT) return fail(ctx, GZK_E_INVALID, "eval_batch_range_device: weights must be a Montgomery buffer");
    if (p_count > 16) return fail(ctx, GZK_E_INVALID, "eval_batch_range_device: too many rotations");
    if ((out->kind != GZK_KIND_FR && out->kind != GZK_KIND_FR_MONT) || out_offset + p_count * k_count > out->count)
        return fail(ctx, GZK_E_INVALID, "eval_batch_range_device: output must be an FR or FR_MONT buffer that holds p_count * k_count values at out_offset");
    uint64_t effective[16];
    for (size_t p = 0; p < p_count; ++p)
    {
        if (rotations[p] >= n) return fail(ctx, GZK_E_INVALID, "eval_batch_range_device: rotation out of range");
        const uint64_t first_needed = (row_offset + n - rotations[p] + n - weights_first) & (n - 1);
        if (len != 0 && weights->count < n && first_needed + len > weights->count)
            return fail(ctx, GZK_E_INVALID, "eval_batch_range_device: the weight slice does not cover the rows at this rotation");
        effective[p] = (n - first_needed) & (n - 1);
    }
    return eval_batch_impl(ctx, cols, k_count, len, log2n, weights, effective, p_count, nullptr, static_cast<Fr*>(out->dptr) + out_offset,
                           out->kind == GZK_KIND_FR_MONT);
}

// Row-sharded form: this GPU holds rows [row_offset, row_offset + len) of every column
// (cols[k][0] is row row_offset) and the weights w[weights_first .. weights_first +
// weights->count) of the domain (indices modulo n, e.g. from gzk_bary_weights_range).
// Returns the PARTIAL sums over the local rows; the partials of all GPUs add up
// (gzk_fr_sum) to what gzk_eval_batch returns on the whole columns.
extern "C" int gzk_eval_batch_range(gzk_ctx* ctx, gzk_buf* const* cols, size_t k_count, size_t len, uint64_t row_offset, unsigned log2n,
                                    const gzk_buf* weights, uint64_t weights_first, const uint64_t* rotations, size_t p_count,
                                    uint8_t* out_host)
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (k_count == 0 || p_count == 0) return GZK_OK;
    if (cols == nullptr || weights == nullptr || rotations == nullptr || out_host == nullptr)
        return fail(ctx, GZK_E_INVALID, "eval_batch_range: null argument");
    if (log2n > 32) return fail(ctx, GZK_E_INVALID, "eval_batch_range: domain too large");
    const uint64_t n = 1ULL << log2n;
    if (len > n || row_offset >= n || weights_first >= n) return fail(ctx, GZK_E_INVALID, "eval_batch_range: range exceeds the domain");
    if (weights->kind != GZK_KIND_FR_MONT) return fail(ctx, GZK_E_INVALID, "eval_batch_range: weights must be a Montgomery buffer");
    if (p_count > 16) return fail(ctx, GZK_E_INVALID, "eval_batch_range: too many rotations");
    uint64_t effective[16];
    for (size_t p = 0; p < p_count; ++p)
    {
        if (rotations[p] >= n) return fail(ctx, GZK_E_INVALID, "eval_batch_range: rotation out of range");
        // local row c is global row row_offset + c and needs w[(row_offset + c - rot) mod n],
        // stored at buffer index (row_offset + c - rot - weights_first) mod n
        const uint64_t first_needed = (row_offset + n - rotations[p] + n - weights_first) & (n - 1);
        if (len != 0 && weights->count < n && first_needed + len > weights->count)
            return fail(ctx, GZK_E_INVALID, "eval_batch_range: the weight slice does not cover the rows at this rotation");
        effective[p] = (n - first_needed) & (n - 1);
    }
    return eval_batch_impl(ctx, cols, k_count, len, log2n, weights, effective, p_count, out_host);
}

// Host-side combination of per-GPU partial results: out[i] = sum_g values[g][i] (mod r).
extern "C" int gzk_fr_sum(const uint8_t* values, size_t groups, size_t count, uint8_t* out)
{
    if (values == nullptr || out == nullptr) return GZK_E_INVALID;
    for (size_t i = 0; i < count; ++i)
    {
        Fr acc = Fr::zero();
        for (size_t g = 0; g < groups; ++g)
        {
            bool canonical = false;
            const Fr v = host_fr_from_bytes(values + (g * count + i) * 32, &canonical);
            if (!canonical) return GZK_E_INVALID;
            acc = add(acc, v);  // canonical residues add like Montgomery ones
        }
        host_fr_to_bytes(acc, out + i * 32);
    }
    return GZK_OK;
}
