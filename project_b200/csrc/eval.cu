// Packed evaluation: K columns x n rows x P rotations of Fr inner products against
// one shared weight vector.  This is the kernel behind column commitment
// (tau-evaluation of every committed column) and behind every opening / quotient
// evaluation of the prover.
//
// Arithmetic: weights are in Montgomery form, column values in canonical form.
// Each lane accumulates the plain 512-bit integer products w~[c] * f[c] in a
// 17-limb register accumulator without any modular reduction (2^32 terms fit), so
// a term costs one 8x8-limb product (64 wide multiply-adds) instead of a full
// Montgomery multiplication (128).  One reduction per (tile, column) pair follows
// in a second, tiny kernel.
//
// Work decomposition: the row range is cut into tiles; a unit of work is one
// (tile, column) pair, enumerated tile-major so that the warps of a CTA stream
// different columns against the SAME weight tile (served by L1/L2 after the first
// touch).  Units are dealt to warps in contiguous runs, which balances any K and
// n over 148 SMs without atomics.  Each unit produces one 17-limb partial sum in
// context-owned scratch.
#include <cstring>

#include "common.cuh"

namespace gzk
{
    namespace
    {
        constexpr int kAccLimbs = 17;
        constexpr int kThreads = 256;

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
        };

        __device__ __forceinline__ Fr load_column_value(const void* col, int kind, uint64_t c)
        {
            if (kind == GZK_KIND_FR || kind == GZK_KIND_FR_MONT) return load_fr(static_cast<const Fr*>(col) + c);
            Fr f = Fr::zero();
            if (kind == GZK_KIND_U32)
            {
                f.l[0] = __ldg(static_cast<const uint32_t*>(col) + c);
                return f;
            }
            // I64: FieldElement::from_signed — negative values are r - |v|
            const long long v = __ldg(static_cast<const long long*>(col) + c);
            const unsigned long long mag = v < 0 ? 0ULL - static_cast<unsigned long long>(v) : static_cast<unsigned long long>(v);
            f.l[0] = static_cast<uint32_t>(mag);
            f.l[1] = static_cast<uint32_t>(mag >> 32);
            return v < 0 ? sub(Fr::zero(), f) : f;
        }

        template <int P>
        __global__ void __launch_bounds__(kThreads) eval_partial_kernel(EvalArgs a)
        {
            const uint32_t lane = threadIdx.x & 31;
            const uint64_t warp = (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
            const uint64_t warps = (static_cast<uint64_t>(gridDim.x) * kThreads) >> 5;
            const uint64_t units = static_cast<uint64_t>(a.tiles) * a.k_count;
            const uint64_t per_warp = (units + warps - 1) / warps;
            const uint64_t u_begin = warp * per_warp;
            const uint64_t u_end = u_begin + per_warp < units ? u_begin + per_warp : units;

            for (uint64_t u = u_begin; u < u_end; ++u)
            {
                const uint32_t tile = static_cast<uint32_t>(u / a.k_count);
                const uint32_t k = static_cast<uint32_t>(u - static_cast<uint64_t>(tile) * a.k_count);
                const void* col = a.cols[k];
                const int kind = a.kinds[k];
                const uint64_t c_begin = static_cast<uint64_t>(tile) * a.tile_rows;
                const uint64_t c_end = c_begin + a.tile_rows < a.len ? c_begin + a.tile_rows : a.len;

                uint32_t acc[P][kAccLimbs];
#pragma unroll
                for (int p = 0; p < P; ++p)
#pragma unroll
                    for (int i = 0; i < kAccLimbs; ++i) acc[p][i] = 0;

                for (uint64_t c = c_begin + lane; c < c_end; c += 32)
                {
                    const Fr f = load_column_value(col, kind, c);
#pragma unroll
                    for (int p = 0; p < P; ++p)
                    {
                        const Fr w = load_fr(a.weights + ((c - a.rot[p]) & a.mask));
                        uint32_t prod[16];
                        mul_wide<8>(w.l, f.l, prod);
                        acc_add<kAccLimbs, 16>(acc[p], prod);
                    }
                }
                // exact integer sum across the warp
#pragma unroll
                for (int p = 0; p < P; ++p)
                {
#pragma unroll
                    for (int offset = 16; offset > 0; offset >>= 1)
                    {
                        uint32_t other[kAccLimbs];
#pragma unroll
                        for (int i = 0; i < kAccLimbs; ++i) other[i] = __shfl_down_sync(0xffffffffu, acc[p][i], offset);
                        acc_add<kAccLimbs, kAccLimbs>(acc[p], other);
                    }
                    if (lane == 0)
                    {
                        uint32_t* dst = a.partial + ((static_cast<uint64_t>(tile) * P + p) * a.k_count + k) * kAccLimbs;
#pragma unroll
                        for (int i = 0; i < kAccLimbs; ++i) dst[i] = acc[p][i];
                    }
                }
            }
        }

        // Sums the per-tile partials of one (rotation, column) pair, reduces once and
        // writes the canonical result.
        __global__ void eval_finish_kernel(const uint32_t* partial, const int* kinds, uint32_t tiles, uint32_t p_count,
                                           uint32_t k_count, Fr* out_canonical)
        {
            const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
            if (idx >= p_count * k_count) return;
            const uint32_t p = idx / k_count;
            const uint32_t k = idx - p * k_count;
            uint32_t acc[kAccLimbs];
#pragma unroll
            for (int i = 0; i < kAccLimbs; ++i) acc[i] = 0;
            for (uint32_t tile = 0; tile < tiles; ++tile)
            {
                const uint32_t* src = partial + ((static_cast<uint64_t>(tile) * p_count + p) * k_count + k) * kAccLimbs;
                uint32_t t[kAccLimbs];
#pragma unroll
                for (int i = 0; i < kAccLimbs; ++i) t[i] = src[i];
                acc_add<kAccLimbs, kAccLimbs>(acc, t);
            }
            // acc = 2^256 * S (canonical columns) or 2^512 * S (Montgomery columns), S the
            // true sum; 9 reduction rows divide by 2^288.
            const Fr reduced = redc_wide<FrCfg, 9>(acc);
            // reduced = S * 2^-32 (canonical columns) -> times 2^288 via Montgomery
            // product with 2^544;  S * 2^224 (Montgomery columns) -> times 2^32 via 2^288.
            Fr fix;
            if (kinds[k] == GZK_KIND_FR_MONT)
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
            store_fr(out_canonical + idx, from_mont(mont));
        }
    }
}

using namespace gzk;

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
    const uint64_t warps_total = static_cast<uint64_t>(ctx->sm_count) * 2 * (kThreads / 32);
    uint64_t want_tiles = (8 * warps_total + k_count - 1) / k_count;
    uint64_t max_tiles = (len + 255) / 256;
    if (max_tiles == 0) max_tiles = 1;
    if (want_tiles > 256) want_tiles = 256;
    if (want_tiles > max_tiles) want_tiles = max_tiles;
    if (want_tiles == 0) want_tiles = 1;
    uint64_t tile_rows = (len + want_tiles - 1) / want_tiles;
    tile_rows = (tile_rows + 31) & ~31ULL;
    if (tile_rows == 0) tile_rows = 32;
    const uint32_t tiles = len == 0 ? 1 : static_cast<uint32_t>((len + tile_rows - 1) / tile_rows);

    // device-side tables and scratch
    const size_t table_bytes = k_count * (sizeof(void*) + sizeof(int));
    const size_t table_padded = (table_bytes + 31) & ~static_cast<size_t>(31);
    void* h_table = nullptr;
    int rc = ensure_pinned(ctx, table_padded + p_count * k_count * 32, &h_table);
    if (rc != GZK_OK) return rc;
    void* d_table = nullptr;
    if ((rc = ensure_scratch(ctx, 0, table_padded + p_count * k_count * 32, &d_table)) != GZK_OK) return rc;
    const void** h_ptrs = static_cast<const void**>(h_table);
    int* h_kinds = reinterpret_cast<int*>(h_ptrs + k_count);
    for (size_t k = 0; k < k_count; ++k)
    {
        h_ptrs[k] = cols[k]->dptr;
        h_kinds[k] = cols[k]->kind;
    }
    GZK_CUDA_TRY(ctx, cudaMemcpyAsync(d_table, h_table, table_bytes, cudaMemcpyHostToDevice, ctx->stream));
    const void* const* d_ptrs = static_cast<const void* const*>(d_table);
    const int* d_kinds = reinterpret_cast<const int*>(static_cast<const char*>(d_table) + k_count * sizeof(void*));
    Fr* d_out = reinterpret_cast<Fr*>(static_cast<char*>(d_table) + table_padded);

    uint8_t* h_out = static_cast<uint8_t*>(h_table) + table_padded;
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
        const uint64_t units = static_cast<uint64_t>(tiles) * k_count;
        uint64_t blocks = (units + (kThreads / 32) - 1) / (kThreads / 32);
        const uint64_t max_blocks = static_cast<uint64_t>(ctx->sm_count) * 2;
        if (blocks > max_blocks) blocks = max_blocks;
        {
            LaunchScope scope(ctx, p_now == 2 ? "eval_partial_p2" : "eval_partial_p1");
            if (p_now == 2)
                eval_partial_kernel<2><<<static_cast<unsigned>(blocks), kThreads, 0, ctx->stream>>>(args);
            else
                eval_partial_kernel<1><<<static_cast<unsigned>(blocks), kThreads, 0, ctx->stream>>>(args);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        const uint32_t outs = p_now * static_cast<uint32_t>(k_count);
        {
            LaunchScope scope(ctx, "eval_finish");
            eval_finish_kernel<<<(outs + 127) / 128, 128, 0, ctx->stream>>>(static_cast<const uint32_t*>(d_partial), d_kinds, tiles, p_now,
                                                                           static_cast<uint32_t>(k_count), d_out + p0 * k_count);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
    }
    GZK_CUDA_TRY(ctx, cudaMemcpyAsync(h_out, d_out, p_count * k_count * 32, cudaMemcpyDeviceToHost, ctx->stream));
    GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
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
    constexpr size_t kStaticPartialOffset = 4096;
    constexpr size_t kStaticPartialBytes = kStaticMaxTiles * kStaticMaxRotations * kStaticMaxColumns * gzk::kAccLimbs * sizeof(uint32_t);
    constexpr size_t kStaticBytes = kStaticPartialOffset + kStaticPartialBytes;  // about 2.1 MiB per GPU
    static_assert(kStaticTableBytes <= kStaticPartialOffset, "pointer table must fit before the partial sums");

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
    for (size_t k = 0; k < k_count; ++k)
    {
        if (col_ptrs[k] == nullptr) return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: null column pointer");
        if (col_kinds[k] < GZK_KIND_FR || col_kinds[k] > GZK_KIND_U32)
            return static_fail(err, err_cap, GZK_E_INVALID, "eval_batch_static: unknown column kind");
    }
    if (cudaSetDevice(device) != cudaSuccess) return static_fail(err, err_cap, GZK_E_CUDA, "eval_batch_static: cudaSetDevice failed");
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
    uint64_t tile_rows = (len + want_tiles - 1) / want_tiles;
    tile_rows = (tile_rows + 31) & ~31ULL;
    if (tile_rows == 0) tile_rows = 32;
    const uint32_t tiles = len == 0 ? 1 : static_cast<uint32_t>((len + tile_rows - 1) / tile_rows);

    // pointer table: built on the stack, copied into the head of the array
    unsigned char table[kStaticTableBytes];
    std::memcpy(table, col_ptrs, k_count * sizeof(void*));
    std::memcpy(table + kStaticMaxColumns * sizeof(void*), col_kinds, k_count * sizeof(int));
    if (cudaMemcpyAsync(scratch, table, kStaticTableBytes, cudaMemcpyHostToDevice, s) != cudaSuccess)
        return static_fail(err, err_cap, GZK_E_CUDA, "eval_batch_static: copying the column table failed");

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
    const uint64_t units = static_cast<uint64_t>(tiles) * k_count;
    uint64_t blocks = (units + (kThreads / 32) - 1) / (kThreads / 32);
    const uint64_t max_blocks = static_cast<uint64_t>(g_static_sms[device]) * 2;
    if (blocks > max_blocks) blocks = max_blocks;
    if (p_count == 2)
        eval_partial_kernel<2><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(args);
    else
        eval_partial_kernel<1><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(args);
    if (cudaGetLastError() != cudaSuccess) return static_fail(err, err_cap, GZK_E_CUDA, "eval_batch_static: kernel launch failed");
    const uint32_t outs = static_cast<uint32_t>(p_count * k_count);
    eval_finish_kernel<<<(outs + 127) / 128, 128, 0, s>>>(args.partial, args.kinds, tiles, static_cast<uint32_t>(p_count),
                                                         static_cast<uint32_t>(k_count), static_cast<Fr*>(out_device));
    if (cudaGetLastError() != cudaSuccess) return static_fail(err, err_cap, GZK_E_CUDA, "eval_batch_static: kernel launch failed");
    return GZK_OK;
}
