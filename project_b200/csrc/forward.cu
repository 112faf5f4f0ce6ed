// fp64 forward pass of one attention head (the witness the prover quantises):
//   H' = X W;  e_src = H' a_src + b_src;  e_dst = H' a_dst + b_dst;
//   per destination node over its incoming edges (in the order given):
//     M = max LeakyReLU(e_dst + e_src),  Sum = sum exp(LeakyReLU(.) - M),  inv = 1/Sum,
//     H_agg_pre = sum alpha * H'[src],  alpha = exp(LeakyReLU(.) - M) * inv;
//   per edge: S, Z = LeakyReLU(S), Delta = M - Z, U = exp(Z - M), alpha = U * inv;
//   H_agg = ELU(H_agg_pre + bias).
//
// The reference computes every sum serially in index order with separate multiply and
// add; so do these kernels (one thread owns one sum, __dmul_rn / __dadd_rn so that no
// fused multiply-add is formed), which makes H', e_src, e_dst, S, Z, M and Delta
// bit-identical to the host computation.  exp and expm1 come from the CUDA math
// library and may differ from the host's in the last unit; everything downstream of
// them (U, Sum, inv, alpha, H_agg) is equal to within a few units in the last place.
//
// Parallelism: rows x output columns for the projection, one thread per node for the
// score vectors and the softmax statistics, one thread per (node, column) for the
// aggregation, one per edge for the edge columns.  The incoming edges of a node are a
// CSR list built by the caller (the host builds it in the reference too).
#include <cmath>

#include "common.cuh"

namespace gzk
{
    namespace
    {
        constexpr int kThreads = 256;

        __device__ __forceinline__ double leaky_relu(double v) { return v >= 0.0 ? v : __dmul_rn(0.2, v); }

        // out[i][j] = sum_k x[i][k] * w[k][j], k ascending (one thread per output)
        __global__ void __launch_bounds__(kThreads) project_kernel(const double* x, const double* w, uint64_t rows, uint32_t inner, uint32_t width,
                                                                   double* out)
        {
            const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
            if (idx >= rows * width) return;
            const uint64_t i = idx / width;
            const uint32_t j = static_cast<uint32_t>(idx - i * width);
            const double* xr = x + i * inner;
            double acc = 0.0;
            for (uint32_t k = 0; k < inner; ++k) acc = __dadd_rn(acc, __dmul_rn(xr[k], __ldg(w + static_cast<uint64_t>(k) * width + j)));
            out[idx] = acc;
        }

        // The same sums for wide heads, tiled: a CTA owns 64 rows x 64 output columns, a thread 4 x 4 of them;
        // the 16-deep slices of X and W pass through shared memory, so each loaded value feeds four
        // multiply-adds instead of one.  Every output is still accumulated over k ascending with a separate
        // multiplication and addition, so the results are the one-thread-per-output kernel's bit for bit.
        constexpr int kTileM = 64, kTileN = 64, kTileK = 16;
        __global__ void __launch_bounds__(kThreads) project_tiled_kernel(const double* x, const double* w, uint64_t rows, uint32_t inner, uint32_t width,
                                                                         double* out)
        {
            // rows padded to 66 doubles: 16-byte aligned groups of four for the vector loads below, and the four
            // k-groups of a store land on different banks
            __shared__ __align__(16) double xs[kTileK][kTileM + 2];
            __shared__ __align__(16) double ws[kTileK][kTileN];
            const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
            const uint64_t i0 = static_cast<uint64_t>(blockIdx.y) * kTileM;
            const uint32_t j0 = blockIdx.x * kTileN;
            double acc[4][4];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[r][c] = 0.0;
            const uint32_t x_row = threadIdx.x >> 2, x_k = (threadIdx.x & 3) * 4;   // 64 rows x 16 k
            const uint32_t w_k = threadIdx.x >> 4, w_j = (threadIdx.x & 15) * 4;    // 16 k x 64 columns
            for (uint32_t k0 = 0; k0 < inner; k0 += kTileK)
            {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                {
                    const uint64_t row = i0 + x_row;
                    const uint32_t k = k0 + x_k + q;
                    xs[x_k + q][x_row] = (row < rows && k < inner) ? x[row * inner + k] : 0.0;
                    const uint32_t kw = k0 + w_k, j = j0 + w_j + q;
                    ws[w_k][w_j + q] = (kw < inner && j < width) ? __ldg(w + static_cast<uint64_t>(kw) * width + j) : 0.0;
                }
                __syncthreads();
                const uint32_t k_count = inner - k0 < kTileK ? inner - k0 : kTileK;
                for (uint32_t kk = 0; kk < k_count; ++kk)
                {
                    double a[4], b[4];
                    const double2 a01 = *reinterpret_cast<const double2*>(&xs[kk][ty * 4]), a23 = *reinterpret_cast<const double2*>(&xs[kk][ty * 4 + 2]);
                    const double2 b01 = *reinterpret_cast<const double2*>(&ws[kk][tx * 4]), b23 = *reinterpret_cast<const double2*>(&ws[kk][tx * 4 + 2]);
                    a[0] = a01.x; a[1] = a01.y; a[2] = a23.x; a[3] = a23.y;
                    b[0] = b01.x; b[1] = b01.y; b[2] = b23.x; b[3] = b23.y;
#pragma unroll
                    for (int r = 0; r < 4; ++r)
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[r][c] = __dadd_rn(acc[r][c], __dmul_rn(a[r], b[c]));
                }
                __syncthreads();
            }
#pragma unroll
            for (int r = 0; r < 4; ++r)
            {
                const uint64_t row = i0 + ty * 4 + r;
                if (row >= rows) continue;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                {
                    const uint32_t j = j0 + tx * 4 + c;
                    if (j < width) out[row * width + j] = acc[r][c];
                }
            }
        }

        // The same sums again for the shapes of the large models (inner a multiple of 8, width even):
        // a CTA owns 128 rows x 64 columns and a thread 8 x 4 of them (columns 2t, 2t+1, 32+2t, 32+2t+1 of the
        // tile, so that the threads of a warp read consecutive 16-byte pieces of a W row: no bank conflict; the
        // columns beyond a ragged width are computed on zeros and not stored), so an operand read from shared
        // memory feeds 5.3 multiply-adds instead of 4; the 8-deep slices are double-buffered (the next one is
        // requested from global memory before the current one is consumed) and the slice loop is unrolled.
        // Two CTAs per SM (128 registers).  Runs at about four fifths of the rate at which the fp64 pipe
        // can issue separate multiplications and additions.  Same order of operations per output, same bits.
        constexpr int kWideRows = 8, kWideCols = 4, kWideK = 8;
        constexpr int kWideM = kWideRows * 16, kWideN = kWideCols * 16;
        __global__ void __launch_bounds__(kThreads, 2) project_wide_kernel(const double* __restrict__ x, const double* __restrict__ w, uint64_t rows,
                                                                          uint32_t inner, uint32_t width, double* __restrict__ out)
        {
            __shared__ __align__(16) double xs[2][kWideK][kWideM + 2];
            __shared__ __align__(16) double ws[2][kWideK][kWideN];
            const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
            const uint64_t i0 = static_cast<uint64_t>(blockIdx.y) * kWideM;
            const uint32_t j0 = blockIdx.x * kWideN;
            double acc[kWideRows][kWideCols];
#pragma unroll
            for (int r = 0; r < kWideRows; ++r)
#pragma unroll
                for (int c = 0; c < kWideCols; ++c) acc[r][c] = 0.0;
            constexpr int kXLoads = kWideM * kWideK / 2 / kThreads;  // pairs of doubles per thread and slice
            constexpr int kWLoads = kWideK * kWideN / 2 / kThreads;
            static_assert(kXLoads * kThreads * 2 == kWideM * kWideK && kWLoads * kThreads * 2 == kWideK * kWideN, "slices must divide among the threads");
            static_assert(kWideCols == 4, "a thread owns two pairs of columns, half a tile apart");
            double2 xr[kXLoads], wr[kWLoads];
            auto request = [&](uint32_t k0) {
#pragma unroll
                for (int p = 0; p < kXLoads; ++p)
                {
                    const uint32_t id = threadIdx.x + p * kThreads;
                    const uint32_t row = id / (kWideK / 2), kq = (id % (kWideK / 2)) * 2;
                    const uint64_t gr = i0 + row;
                    xr[p] = gr < rows ? *reinterpret_cast<const double2*>(x + gr * inner + k0 + kq) : make_double2(0.0, 0.0);
                }
#pragma unroll
                for (int p = 0; p < kWLoads; ++p)
                {
                    const uint32_t id = threadIdx.x + p * kThreads;
                    const uint32_t kr = id / (kWideN / 2), jq = (id % (kWideN / 2)) * 2;
                    wr[p] = j0 + jq < width ? __ldg(reinterpret_cast<const double2*>(w + static_cast<uint64_t>(k0 + kr) * width + j0 + jq)) : make_double2(0.0, 0.0);
                }
            };
            auto stash = [&](int buf) {
#pragma unroll
                for (int p = 0; p < kXLoads; ++p)
                {
                    const uint32_t id = threadIdx.x + p * kThreads;
                    const uint32_t row = id / (kWideK / 2), kq = (id % (kWideK / 2)) * 2;
                    xs[buf][kq][row] = xr[p].x;
                    xs[buf][kq + 1][row] = xr[p].y;
                }
#pragma unroll
                for (int p = 0; p < kWLoads; ++p)
                {
                    const uint32_t id = threadIdx.x + p * kThreads;
                    const uint32_t kr = id / (kWideN / 2), jq = (id % (kWideN / 2)) * 2;
                    *reinterpret_cast<double2*>(&ws[buf][kr][jq]) = wr[p];
                }
            };
            request(0);
            stash(0);
            __syncthreads();
            int buf = 0;
            for (uint32_t k0 = 0; k0 < inner; k0 += kWideK)
            {
                const bool more = k0 + kWideK < inner;
                if (more) request(k0 + kWideK);
#pragma unroll
                for (int kk = 0; kk < kWideK; ++kk)
                {
                    double a[kWideRows], b[kWideCols];
#pragma unroll
                    for (int r = 0; r < kWideRows; r += 2)
                    {
                        const double2 v = *reinterpret_cast<const double2*>(&xs[buf][kk][ty * kWideRows + r]);
                        a[r] = v.x;
                        a[r + 1] = v.y;
                    }
#pragma unroll
                    for (int c = 0; c < kWideCols; c += 2)
                    {
                        const double2 v = *reinterpret_cast<const double2*>(&ws[buf][kk][(c / 2) * (kWideN / 2) + tx * 2]);
                        b[c] = v.x;
                        b[c + 1] = v.y;
                    }
#pragma unroll
                    for (int r = 0; r < kWideRows; ++r)
#pragma unroll
                        for (int c = 0; c < kWideCols; ++c) acc[r][c] = __dadd_rn(acc[r][c], __dmul_rn(a[r], b[c]));
                }
                if (more) stash(buf ^ 1);
                __syncthreads();
                buf ^= 1;
            }
#pragma unroll
            for (int r = 0; r < kWideRows; ++r)
            {
                const uint64_t row = i0 + ty * kWideRows + r;
                if (row >= rows) continue;
#pragma unroll
                for (int c = 0; c < kWideCols; c += 2)
                {
                    const uint32_t j = j0 + (c / 2) * (kWideN / 2) + tx * 2;
                    if (j < width) *reinterpret_cast<double2*>(out + row * width + j) = make_double2(acc[r][c], acc[r][c + 1]);
                }
            }
        }

        // e[i] = bias + sum_c h[i][c] * a[c], c ascending; both score vectors in one pass
        __global__ void __launch_bounds__(kThreads) scores_kernel(const double* h, uint64_t rows, uint32_t width, const double* a_src, double b_src,
                                                                  const double* a_dst, double b_dst, double* e_src, double* e_dst)
        {
            const uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
            if (i >= rows) return;
            const double* hr = h + i * width;
            double s = b_src, d = b_dst;
            for (uint32_t c = 0; c < width; ++c)
            {
                const double v = hr[c];
                s = __dadd_rn(s, __dmul_rn(v, __ldg(a_src + c)));
                d = __dadd_rn(d, __dmul_rn(v, __ldg(a_dst + c)));
            }
            e_src[i] = s;
            e_dst[i] = d;
        }

        // M, Sum, inv of every destination node over its incoming list
        __global__ void __launch_bounds__(kThreads) softmax_stats_kernel(const double* e_src, const double* e_dst, const uint32_t* in_ptr,
                                                                         const uint32_t* in_src, uint64_t nodes, double* m_out, double* sum_out,
                                                                         double* inv_out)
        {
            const uint64_t dst = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
            if (dst >= nodes) return;
            const uint32_t begin = in_ptr[dst], end = in_ptr[dst + 1];
            const double ed = e_dst[dst];
            double m = -INFINITY;
            for (uint32_t p = begin; p < end; ++p) m = fmax(m, leaky_relu(__dadd_rn(ed, e_src[in_src[p]])));
            double sum = 0.0;
            for (uint32_t p = begin; p < end; ++p) sum = __dadd_rn(sum, exp(__dsub_rn(leaky_relu(__dadd_rn(ed, e_src[in_src[p]])), m)));
            m_out[dst] = m;
            sum_out[dst] = sum;
            inv_out[dst] = __ddiv_rn(1.0, sum);
        }

        // The same statistics with one warp per destination node, plus the attention weight of every entry
        // of the incoming lists (alpha_in[p], p the position in in_src).  A node with tens of thousands of
        // incoming edges (the hubs of a power-law graph) would keep a single thread busy long after the rest
        // of the grid has drained; here the lanes evaluate 32 exponentials at a time and only the additions
        // stay serial - in list order, one after the other, because the reference adds them in that order
        // and floating-point addition is not associative.  (The maximum is exact in any order.)
        __global__ void __launch_bounds__(kThreads) softmax_stats_warp_kernel(const double* e_src, const double* e_dst, const uint32_t* in_ptr,
                                                                              const uint32_t* in_src, uint64_t nodes, double* m_out, double* sum_out,
                                                                              double* inv_out, double* alpha_in)
        {
            const uint64_t dst = (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
            const uint32_t lane = threadIdx.x & 31;
            if (dst >= nodes) return;
            const uint32_t begin = in_ptr[dst], end = in_ptr[dst + 1];
            const double ed = e_dst[dst];
            double m = -INFINITY;
            for (uint32_t p = begin + lane; p < end; p += 32) m = fmax(m, leaky_relu(__dadd_rn(ed, e_src[in_src[p]])));
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) m = fmax(m, __shfl_xor_sync(0xffffffffu, m, offset));
            double sum = 0.0;
            for (uint32_t base = begin; base < end; base += 32)
            {
                const uint32_t p = base + lane;
                double t = 0.0;
                if (p < end)
                {
                    t = exp(__dsub_rn(leaky_relu(__dadd_rn(ed, e_src[in_src[p]])), m));
                    alpha_in[p] = t;
                }
                const uint32_t here = end - base < 32 ? end - base : 32;
                for (uint32_t l = 0; l < here; ++l) sum = __dadd_rn(sum, __shfl_sync(0xffffffffu, t, l));
            }
            const double inv = __ddiv_rn(1.0, sum);
            if (lane == 0)
            {
                m_out[dst] = m;
                sum_out[dst] = sum;
                inv_out[dst] = inv;
            }
            for (uint32_t p = begin + lane; p < end; p += 32) alpha_in[p] = __dmul_rn(alpha_in[p], inv);  // written by this same lane above
        }

        // Aggregation with the attention weights already in alpha_in: no exponential inside the serial sum.
        __global__ void __launch_bounds__(kThreads) aggregate_alpha_kernel(const double* h, const double* alpha_in, const uint32_t* in_ptr,
                                                                           const uint32_t* in_src, uint64_t nodes, uint32_t width, const double* out_bias,
                                                                           uint32_t bias_count, int apply_activation, double* pre_out, double* agg_out,
                                                                           uint32_t heavy_above)
        {
            const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
            if (idx >= nodes * width) return;
            const uint64_t dst = idx / width;
            const uint32_t c = static_cast<uint32_t>(idx - dst * width);
            const uint32_t begin = in_ptr[dst], end = in_ptr[dst + 1];
            if (end - begin > heavy_above) return;  // aggregate_heavy_kernel owns this node
            double acc = 0.0;
            uint32_t p = begin;
            // Long lists (the hubs of a power-law graph: tens of thousands of entries for one node) would pay one
            // gather latency per entry if walked one by one.  The products are exact and independent of the
            // running sum, so sixteen of them are formed at a time (sixteen gathers in flight) and only the
            // additions stay serial, in list order.
            for (; p + 16 <= end; p += 16)
            {
                double prod[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) prod[u] = __dmul_rn(alpha_in[p + u], h[static_cast<uint64_t>(in_src[p + u]) * width + c]);
#pragma unroll
                for (int u = 0; u < 16; ++u) acc = __dadd_rn(acc, prod[u]);
            }
            for (; p + 4 <= end; p += 4)
            {
                // the four loads do not depend on acc: they are in flight together
                const double a0 = alpha_in[p], a1 = alpha_in[p + 1], a2 = alpha_in[p + 2], a3 = alpha_in[p + 3];
                const double h0 = h[static_cast<uint64_t>(in_src[p]) * width + c], h1 = h[static_cast<uint64_t>(in_src[p + 1]) * width + c];
                const double h2 = h[static_cast<uint64_t>(in_src[p + 2]) * width + c], h3 = h[static_cast<uint64_t>(in_src[p + 3]) * width + c];
                acc = __dadd_rn(acc, __dmul_rn(a0, h0));
                acc = __dadd_rn(acc, __dmul_rn(a1, h1));
                acc = __dadd_rn(acc, __dmul_rn(a2, h2));
                acc = __dadd_rn(acc, __dmul_rn(a3, h3));
            }
            for (; p < end; ++p) acc = __dadd_rn(acc, __dmul_rn(alpha_in[p], h[static_cast<uint64_t>(in_src[p]) * width + c]));
            if (pre_out != nullptr) pre_out[idx] = acc;
            double v = acc;
            if (out_bias != nullptr && c < bias_count) v = __dadd_rn(v, out_bias[c]);
            if (agg_out != nullptr) agg_out[idx] = apply_activation ? (v >= 0.0 ? v : expm1(v)) : v;
        }

        // ---- nodes with long incoming lists ------------------------------------------------------------
        // The sum over a list is serial by definition, but a thread that walks 10 000 entries and waits for a
        // gather from HBM at each of them takes milliseconds.  These nodes get a CTA each (a thread per column)
        // whose gathers run ahead of the additions as asynchronous copies into a ring of shared-memory stages:
        // sixteen entries per stage, four stages in flight, every thread copies and later reads only its own
        // column, so no barrier is needed - only cp.async.wait_group.
        constexpr uint32_t kHeavyDegree = 512;
        constexpr int kAggStages = 4, kAggChunk = 16;
        // 128 KiB of gathered values + 4 KiB of attention weights (a private copy per warp)
        constexpr size_t kAggSmemBytes = static_cast<size_t>(kAggStages) * kAggChunk * (kThreads + kThreads / 32) * sizeof(double);

        __global__ void list_heavy_nodes_kernel(const uint32_t* in_ptr, uint64_t nodes, uint32_t* heavy, uint32_t* heavy_count)
        {
            const uint64_t dst = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
            if (dst >= nodes) return;
            if (in_ptr[dst + 1] - in_ptr[dst] > kHeavyDegree) heavy[atomicAdd(heavy_count, 1u)] = static_cast<uint32_t>(dst);
        }

        __device__ __forceinline__ void cp_async_f64(double* smem_dst, const double* src)
        {
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(src) : "memory");
        }
        __device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
        template <int PENDING>
        __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

        __global__ void __launch_bounds__(kThreads) aggregate_heavy_kernel(const double* h, const double* alpha_in, const uint32_t* in_ptr,
                                                                           const uint32_t* in_src, const uint32_t* heavy, const uint32_t* heavy_count,
                                                                           uint32_t width, const double* out_bias, uint32_t bias_count,
                                                                           int apply_activation, double* pre_out, double* agg_out)
        {
            extern __shared__ double agg_stage[];  // [stage][entry][thread], then per warp [stage][entry] attention weights
            double* alpha_stage = agg_stage + static_cast<size_t>(kAggStages) * kAggChunk * kThreads + (threadIdx.x >> 5) * (kAggStages * kAggChunk);
            const uint32_t lane = threadIdx.x & 31;
            const uint32_t count = *heavy_count;
            for (uint32_t item = blockIdx.x; item < count; item += gridDim.x)
            {
                const uint64_t dst = heavy[item];
                const uint32_t begin = in_ptr[dst], end = in_ptr[dst + 1];
                const uint32_t chunks = (end - begin + kAggChunk - 1) / kAggChunk;
                for (uint32_t c0 = 0; c0 < width; c0 += kThreads)
                {
                    const uint32_t c = c0 + threadIdx.x;
                    const bool active = c < width;
                    // The source ids of a chunk are fetched by sixteen lanes (one load per warp instead of sixteen
                    // broadcast loads in a row) one chunk ahead of their use; the attention weights travel with the
                    // gathers as asynchronous copies of their own.
                    auto fetch_sources = [&](uint32_t ch) -> uint32_t {
                        const uint32_t p = begin + ch * kAggChunk + lane;
                        return (ch < chunks && lane < kAggChunk && p < end) ? in_src[p] : 0u;
                    };
                    auto issue = [&](uint32_t ch, uint32_t my_source) {
                        const uint32_t base = begin + ch * kAggChunk;
                        const uint32_t st = ch % kAggStages;
                        double* slot = agg_stage + static_cast<size_t>(st) * kAggChunk * kThreads + threadIdx.x;
                        if (lane < kAggChunk && base + lane < end) cp_async_f64(alpha_stage + st * kAggChunk + lane, alpha_in + base + lane);
#pragma unroll
                        for (int e = 0; e < kAggChunk; ++e)
                        {
                            const uint32_t source = __shfl_sync(0xffffffffu, my_source, e);
                            if (active && base + e < end) cp_async_f64(slot + e * kThreads, h + static_cast<uint64_t>(source) * width + c);
                        }
                        cp_async_commit();  // one group per step, empty or not, so that the wait below counts steps
                    };
                    uint32_t next_sources = fetch_sources(0);
                    for (uint32_t ch = 0; ch < kAggStages - 1; ++ch)
                    {
                        const uint32_t mine = next_sources;
                        next_sources = fetch_sources(ch + 1);
                        if (ch < chunks)
                            issue(ch, mine);
                        else
                            cp_async_commit();
                    }
                    double acc = 0.0;
                    for (uint32_t ch = 0; ch < chunks; ++ch)
                    {
                        const uint32_t ahead = ch + kAggStages - 1;
                        const uint32_t mine = next_sources;
                        next_sources = fetch_sources(ahead + 1);
                        if (ahead < chunks)
                            issue(ahead, mine);
                        else
                            cp_async_commit();
                        cp_async_wait<kAggStages - 1>();  // everything but the newest three groups has landed: chunk ch is in
                        __syncwarp();                       // the weights of the chunk were copied by other lanes of this warp
                        const uint32_t base = begin + ch * kAggChunk;
                        const uint32_t st = ch % kAggStages;
                        const double* slot = agg_stage + static_cast<size_t>(st) * kAggChunk * kThreads + threadIdx.x;
                        if (active)
                        {
#pragma unroll
                            for (int e = 0; e < kAggChunk; ++e)
                                if (base + e < end) acc = __dadd_rn(acc, __dmul_rn(alpha_stage[st * kAggChunk + e], slot[e * kThreads]));
                        }
                        __syncwarp();  // the stage is refilled by the copies issued in the next step
                    }
                    cp_async_wait<0>();
                    if (active)
                    {
                        const uint64_t idx = dst * width + c;
                        if (pre_out != nullptr) pre_out[idx] = acc;
                        double v = acc;
                        if (out_bias != nullptr && c < bias_count) v = __dadd_rn(v, out_bias[c]);
                        if (agg_out != nullptr) agg_out[idx] = apply_activation ? (v >= 0.0 ? v : expm1(v)) : v;
                    }
                }
            }
        }

        // H_agg_pre[dst][c] = sum over incoming src of alpha * H'[src][c]; H_agg = act(H_agg_pre + bias)
        __global__ void __launch_bounds__(kThreads) aggregate_kernel(const double* h, const double* e_src, const double* e_dst, const double* m_in,
                                                                     const double* inv_in, const uint32_t* in_ptr, const uint32_t* in_src,
                                                                     uint64_t nodes, uint32_t width, const double* out_bias, uint32_t bias_count,
                                                                     int apply_activation, double* pre_out, double* agg_out)
        {
            const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
            if (idx >= nodes * width) return;
            const uint64_t dst = idx / width;
            const uint32_t c = static_cast<uint32_t>(idx - dst * width);
            const uint32_t begin = in_ptr[dst], end = in_ptr[dst + 1];
            const double ed = e_dst[dst], m = m_in[dst], inv = inv_in[dst];
            double acc = 0.0;
            for (uint32_t p = begin; p < end; ++p)
            {
                const uint32_t src = in_src[p];
                const double alpha = __dmul_rn(exp(__dsub_rn(leaky_relu(__dadd_rn(ed, e_src[src])), m)), inv);
                acc = __dadd_rn(acc, __dmul_rn(alpha, h[static_cast<uint64_t>(src) * width + c]));
            }
            if (pre_out != nullptr) pre_out[idx] = acc;
            double v = acc;
            if (out_bias != nullptr && c < bias_count) v = __dadd_rn(v, out_bias[c]);
            if (agg_out != nullptr) agg_out[idx] = apply_activation ? (v >= 0.0 ? v : expm1(v)) : v;
        }

        __global__ void __launch_bounds__(kThreads) edge_columns_kernel(const double* e_src, const double* e_dst, const double* m_in, const double* inv_in,
                                                                        const uint32_t* src, const uint32_t* dst, uint64_t edges, uint64_t nodes,
                                                                        double* s_out, double* z_out, double* delta_out, double* u_out,
                                                                        double* alpha_out, int* status)
        {
            const uint64_t e = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
            if (e >= edges) return;
            const uint32_t a = src[e], b = dst[e];
            if (a >= nodes || b >= nodes)
            {
                raise_status(status, GZK_E_INVALID, 701);
                return;
            }
            const double s = __dadd_rn(e_dst[b], e_src[a]);
            const double z = leaky_relu(s);
            const double u = exp(__dsub_rn(z, m_in[b]));
            if (s_out != nullptr) s_out[e] = s;
            if (z_out != nullptr) z_out[e] = z;
            if (delta_out != nullptr) delta_out[e] = __dsub_rn(m_in[b], z);
            if (u_out != nullptr) u_out[e] = u;
            if (alpha_out != nullptr) alpha_out[e] = __dmul_rn(u, inv_in[b]);
        }

        __global__ void __launch_bounds__(kThreads) check_incoming_kernel(const uint32_t* in_ptr, const uint32_t* in_src, uint64_t nodes, uint64_t in_count,
                                                                          int* status)
        {
            const uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
            if (i < nodes && (in_ptr[i] > in_ptr[i + 1] || in_ptr[i + 1] > in_count)) raise_status(status, GZK_E_INVALID, 702);
            if (i == 0 && in_ptr[0] != 0) raise_status(status, GZK_E_INVALID, 703);
            if (i < in_count && in_src[i] >= nodes) raise_status(status, GZK_E_INVALID, 704);
        }

        bool f64_ok(const gzk_buf* b, uint64_t need) { return b != nullptr && b->kind == GZK_KIND_F64 && b->count >= need; }
        bool f64_opt(const gzk_buf* b, uint64_t need) { return b == nullptr || f64_ok(b, need); }
        bool u32_ok(const gzk_buf* b, uint64_t need) { return b != nullptr && b->kind == GZK_KIND_U32 && b->count >= need; }
        double* f64_ptr(const gzk_buf* b) { return b == nullptr ? nullptr : static_cast<double*>(b->dptr); }
        unsigned grid_for(uint64_t work) { return static_cast<unsigned>((work + kThreads - 1) / kThreads); }
    }
}

using namespace gzk;

extern "C" int gzk_gat_head_forward(gzk_ctx* ctx, const gzk_gat_head* head, const gzk_gat_graph* graph, const gzk_gat_trace* out)
{
    if (ctx == nullptr) return GZK_E_INVALID;
    if (head == nullptr || graph == nullptr || out == nullptr) return fail(ctx, GZK_E_INVALID, "gat_head_forward: null argument");
    const uint64_t nodes = graph->node_count, edges = graph->edge_count, in_count = graph->incoming_count;
    const uint32_t inner = head->input_width, width = head->output_width;
    if (nodes == 0) return GZK_OK;
    if (inner == 0 || width == 0) return fail(ctx, GZK_E_INVALID, "gat_head_forward: empty weight matrix");
    if (nodes > 0xfffffffeULL || in_count > 0xffffffffULL || nodes * width > (1ULL << 40)) return fail(ctx, GZK_E_INVALID, "gat_head_forward: graph too large");
    if (!f64_ok(head->features, nodes * inner) || !f64_ok(head->seq_kernel, static_cast<uint64_t>(inner) * width) ||
        !f64_ok(head->attn_src_kernel, width) || !f64_ok(head->attn_dst_kernel, width))
        return fail(ctx, GZK_E_INVALID, "gat_head_forward: feature / weight buffers must be F64 buffers of the stated shapes");
    if (head->output_bias != nullptr && !f64_ok(head->output_bias, head->output_bias_count)) return fail(ctx, GZK_E_INVALID, "gat_head_forward: bad output bias buffer");
    if ((edges != 0 && (!u32_ok(graph->edge_src, edges) || !u32_ok(graph->edge_dst, edges))) || !u32_ok(graph->incoming_ptr, nodes + 1) ||
        (in_count != 0 && !u32_ok(graph->incoming_src, in_count)))
        return fail(ctx, GZK_E_INVALID, "gat_head_forward: edge lists must be U32 buffers (incoming_ptr has node_count + 1 entries)");
    if (!f64_ok(out->H_prime, nodes * width) || !f64_ok(out->E_src, nodes) || !f64_ok(out->E_dst, nodes) || !f64_ok(out->M, nodes) ||
        !f64_ok(out->Sum, nodes) || !f64_ok(out->inv, nodes))
        return fail(ctx, GZK_E_INVALID, "gat_head_forward: H_prime, E_src, E_dst, M, Sum and inv outputs are required F64 buffers");
    if (!f64_opt(out->S, edges) || !f64_opt(out->Z, edges) || !f64_opt(out->Delta, edges) || !f64_opt(out->U, edges) || !f64_opt(out->alpha, edges) ||
        !f64_opt(out->H_agg_pre_bias, nodes * width) || !f64_opt(out->H_agg, nodes * width))
        return fail(ctx, GZK_E_INVALID, "gat_head_forward: optional outputs must be F64 buffers of the stated shapes");
    GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    int rc = begin_call(ctx);
    if (rc != GZK_OK) return rc;
    const uint32_t* in_ptr = static_cast<const uint32_t*>(graph->incoming_ptr->dptr);
    const uint32_t* in_src = in_count != 0 ? static_cast<const uint32_t*>(graph->incoming_src->dptr) : nullptr;
    {
        LaunchScope scope(ctx, "forward_check");
        check_incoming_kernel<<<grid_for(nodes > in_count ? nodes : in_count), kThreads, 0, ctx->stream>>>(in_ptr, in_src, nodes, in_count, ctx->d_status);
    }
    GZK_CUDA_TRY(ctx, cudaGetLastError());
    // the lists are read by the kernels below: settle their validity first
    {
        int status = 0;
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(&status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
        GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        if (status == GZK_E_INVALID)
        {
            GZK_CUDA_TRY(ctx, cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream));
            return fail(ctx, GZK_E_INVALID, "edge out of bounds while running attention head forward");
        }
    }
    if (width % 2 == 0 && width >= 32 && inner % kWideK == 0 && inner != 0)
    {
        LaunchScope scope(ctx, "forward_project");
        const dim3 grid((width + kWideN - 1) / kWideN, static_cast<unsigned>((nodes + kWideM - 1) / kWideM));
        project_wide_kernel<<<grid, kThreads, 0, ctx->stream>>>(f64_ptr(head->features), f64_ptr(head->seq_kernel), nodes, inner, width,
                                                                f64_ptr(out->H_prime));
    }
    else if (width >= 32)
    {
        LaunchScope scope(ctx, "forward_project");
        const dim3 grid((width + kTileN - 1) / kTileN, static_cast<unsigned>((nodes + kTileM - 1) / kTileM));
        project_tiled_kernel<<<grid, kThreads, 0, ctx->stream>>>(f64_ptr(head->features), f64_ptr(head->seq_kernel), nodes, inner, width,
                                                                 f64_ptr(out->H_prime));
    }
    else
    {
        LaunchScope scope(ctx, "forward_project");
        project_kernel<<<grid_for(nodes * width), kThreads, 0, ctx->stream>>>(f64_ptr(head->features), f64_ptr(head->seq_kernel), nodes, inner, width,
                                                                              f64_ptr(out->H_prime));
    }
    GZK_CUDA_TRY(ctx, cudaGetLastError());
    {
        LaunchScope scope(ctx, "forward_scores");
        scores_kernel<<<grid_for(nodes), kThreads, 0, ctx->stream>>>(f64_ptr(out->H_prime), nodes, width, f64_ptr(head->attn_src_kernel), head->attn_src_bias,
                                                                     f64_ptr(head->attn_dst_kernel), head->attn_dst_bias, f64_ptr(out->E_src),
                                                                     f64_ptr(out->E_dst));
    }
    GZK_CUDA_TRY(ctx, cudaGetLastError());
    // long incoming lists (an average above 4 entries, or any list above 64): one warp per node and the
    // attention weights kept per list entry; short lists keep the one-thread-per-node kernels
    const bool by_warp = in_count > 4 * nodes || in_count >= (1u << 16);
    double* alpha_in = nullptr;
    if (by_warp)
    {
        void* scratch = nullptr;
        // alpha_in, then the list of nodes with long incoming lists (at most in_count / 512 of them) and its counter
        if ((rc = ensure_scratch(ctx, 0, (in_count + 1) * sizeof(double) + (in_count / 512 + 8) * sizeof(uint32_t), &scratch)) != GZK_OK) return rc;
        alpha_in = static_cast<double*>(scratch);
        LaunchScope scope(ctx, "forward_softmax_stats");
        softmax_stats_warp_kernel<<<grid_for(nodes * 32), kThreads, 0, ctx->stream>>>(f64_ptr(out->E_src), f64_ptr(out->E_dst), in_ptr, in_src, nodes,
                                                                                      f64_ptr(out->M), f64_ptr(out->Sum), f64_ptr(out->inv), alpha_in);
    }
    else
    {
        LaunchScope scope(ctx, "forward_softmax_stats");
        softmax_stats_kernel<<<grid_for(nodes), kThreads, 0, ctx->stream>>>(f64_ptr(out->E_src), f64_ptr(out->E_dst), in_ptr, in_src, nodes, f64_ptr(out->M),
                                                                            f64_ptr(out->Sum), f64_ptr(out->inv));
    }
    GZK_CUDA_TRY(ctx, cudaGetLastError());
    if (by_warp && (out->H_agg_pre_bias != nullptr || out->H_agg != nullptr))
    {
        // the list of nodes with long incoming lists sits behind alpha_in in the same scratch area
        uint32_t* heavy_count = reinterpret_cast<uint32_t*>(alpha_in + in_count + 1);
        uint32_t* heavy = heavy_count + 2;
        static bool opted_in[64] = {};
        if (ctx->device >= 0 && ctx->device < 64 && !opted_in[ctx->device])
        {
            GZK_CUDA_TRY(ctx, cudaFuncSetAttribute(aggregate_heavy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kAggSmemBytes)));
            opted_in[ctx->device] = true;
        }
        const uint32_t bias_count = head->output_bias != nullptr ? static_cast<uint32_t>(head->output_bias_count) : 0u;
        GZK_CUDA_TRY(ctx, cudaMemsetAsync(heavy_count, 0, 2 * sizeof(uint32_t), ctx->stream));
        {
            LaunchScope scope(ctx, "forward_aggregate");
            list_heavy_nodes_kernel<<<grid_for(nodes), kThreads, 0, ctx->stream>>>(in_ptr, nodes, heavy, heavy_count);
            aggregate_alpha_kernel<<<grid_for(nodes * width), kThreads, 0, ctx->stream>>>(
                f64_ptr(out->H_prime), alpha_in, in_ptr, in_src, nodes, width, f64_ptr(head->output_bias), bias_count, head->apply_activation,
                f64_ptr(out->H_agg_pre_bias), f64_ptr(out->H_agg), kHeavyDegree);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        {
            LaunchScope scope(ctx, "forward_aggregate_heavy");
            aggregate_heavy_kernel<<<ctx->sm_count, kThreads, kAggSmemBytes, ctx->stream>>>(
                f64_ptr(out->H_prime), alpha_in, in_ptr, in_src, heavy, heavy_count, width, f64_ptr(head->output_bias), bias_count,
                head->apply_activation, f64_ptr(out->H_agg_pre_bias), f64_ptr(out->H_agg));
        }
    }
    else if (out->H_agg_pre_bias != nullptr || out->H_agg != nullptr)
    {
        LaunchScope scope(ctx, "forward_aggregate");
        aggregate_kernel<<<grid_for(nodes * width), kThreads, 0, ctx->stream>>>(
            f64_ptr(out->H_prime), f64_ptr(out->E_src), f64_ptr(out->E_dst), f64_ptr(out->M), f64_ptr(out->inv), in_ptr, in_src, nodes, width,
            f64_ptr(head->output_bias), head->output_bias != nullptr ? static_cast<uint32_t>(head->output_bias_count) : 0u, head->apply_activation,
            f64_ptr(out->H_agg_pre_bias), f64_ptr(out->H_agg));
    }
    GZK_CUDA_TRY(ctx, cudaGetLastError());
    if (edges != 0 && (out->S != nullptr || out->Z != nullptr || out->Delta != nullptr || out->U != nullptr || out->alpha != nullptr))
    {
        LaunchScope scope(ctx, "forward_edge_columns");
        edge_columns_kernel<<<grid_for(edges), kThreads, 0, ctx->stream>>>(
            f64_ptr(out->E_src), f64_ptr(out->E_dst), f64_ptr(out->M), f64_ptr(out->inv), static_cast<const uint32_t*>(graph->edge_src->dptr),
            static_cast<const uint32_t*>(graph->edge_dst->dptr), edges, nodes, f64_ptr(out->S), f64_ptr(out->Z), f64_ptr(out->Delta), f64_ptr(out->U),
            f64_ptr(out->alpha), ctx->d_status);
    }
    GZK_CUDA_TRY(ctx, cudaGetLastError());
    return finish_call(ctx, "edge out of bounds while running attention head forward");
}
