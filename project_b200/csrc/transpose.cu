// Data movement and twiddle kernels of the row-sharded ("four-step") transform:
//   n = n1 * n2, element i = i1 * n2 + i2; each GPU owns a block of rows i1.  The
//   transform is: exchange so that a GPU owns a block of columns i2 with every i1,
//   length-n1 transforms along i1, multiplication by omega_n^(i2*k1), a second
//   exchange so that a GPU owns a block of k1 with every i2, length-n2 transforms
//   along i2.  The exchanges themselves are the caller's (an all-to-all over NCCL);
//   the kernels here lay the chunks out so that every chunk sent to a peer is
//   contiguous, and undo that layout on arrival:
//     gzk_swap_outer   in[d0][d1][d2] -> out[d1][d0][d2]   (pack / unpack of chunks)
//     gzk_transpose    in[rows][cols] -> out[cols][rows]
//     gzk_ntt_twiddle  buf[r][c] *= omega_n^(+-(row_first + r) * c)
// Elements are 32-byte field elements; the movement kernels do not look inside them.
#include "block.cuh"

namespace gzk
{
    namespace
    {
        constexpr int kTile = 32;

        struct __align__(16) Elem32
        {
            uint4 lo, hi;
        };

        // Shared-memory tile transpose: reads and writes are both contiguous in 32-element
        // (1 KiB) runs; the padded tile keeps the 16-byte halves of a column walk on distinct
        // banks.
        __global__ void __launch_bounds__(kTile * 8) transpose_kernel(const Elem32* in, uint64_t rows, uint64_t cols, Elem32* out)
        {
            __shared__ Elem32 tile[kTile][kTile + 1];
            const uint64_t tiles_x = (cols + kTile - 1) / kTile;
            const uint64_t tile_id = blockIdx.x;
            const uint64_t r0 = (tile_id / tiles_x) * kTile, c0 = (tile_id % tiles_x) * kTile;
            const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
            for (int j = 0; j < kTile; j += 8)
            {
                const uint64_t r = r0 + ty + j, c = c0 + tx;
                if (r < rows && c < cols) tile[ty + j][tx] = in[r * cols + c];
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < kTile; j += 8)
            {
                const uint64_t c = c0 + ty + j, r = r0 + tx;
                if (r < rows && c < cols) out[c * rows + r] = tile[tx][ty + j];
            }
        }

        __global__ void __launch_bounds__(256) swap_outer_kernel(const Elem32* in, uint64_t d0, uint64_t d1, uint64_t d2, Elem32* out)
        {
            const uint64_t total = d0 * d1 * d2;
            const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
            for (uint64_t o = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; o < total; o += stride)
            {
                const uint64_t c = o % d2;
                const uint64_t a = (o / d2) % d0;
                const uint64_t b = o / (d2 * d0);
                out[o] = in[(a * d1 + b) * d2 + c];
            }
        }

        __global__ void __launch_bounds__(256) twiddle_kernel(Fr* buf, uint64_t row_first, uint64_t rows, uint64_t cols, unsigned log2n,
                                                              const Fr* lo, const Fr* hi, unsigned lo_bits)
        {
            const uint64_t total = rows * cols;
            const uint64_t mask = (1ULL << log2n) - 1ULL;
            const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
            for (uint64_t o = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; o < total; o += stride)
            {
                const uint64_t r = o / cols, c = o - r * cols;
                const uint64_t e = ((row_first + r) * c) & mask;  // both factors < 2^30: no overflow
                if (e != 0) store_fr(buf + o, mul(load_fr_plain(buf + o), domain_point(lo, hi, lo_bits, e)));
            }
        }

        bool movable(const gzk_buf* b) { return b != nullptr && (b->kind == GZK_KIND_FR || b->kind == GZK_KIND_FR_MONT); }
    }
}

using namespace gzk;

extern "C"
{
    int gzk_transpose(gzk_ctx* ctx, const gzk_buf* in, size_t rows, size_t cols, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (!movable(in) || !movable(out) || in == out || in->dptr == out->dptr) return fail(ctx, GZK_E_INVALID, "transpose: field-element buffers, out distinct from in");
        if (rows != 0 && cols > in->count / rows) return fail(ctx, GZK_E_INVALID, "transpose: input buffer too small");
        if (out->count < rows * cols || out->kind != in->kind) return fail(ctx, GZK_E_INVALID, "transpose: output must have the input's kind and rows*cols elements");
        if (rows == 0 || cols == 0) return GZK_OK;
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        const uint64_t tiles = ((rows + kTile - 1) / kTile) * ((cols + kTile - 1) / kTile);
        if (tiles > 0x7fffffffULL) return fail(ctx, GZK_E_INVALID, "transpose: matrix too large");
        {
            LaunchScope scope(ctx, "transpose");
            transpose_kernel<<<static_cast<unsigned>(tiles), kTile * 8, 0, ctx->stream>>>(static_cast<const Elem32*>(in->dptr), rows, cols,
                                                                                           static_cast<Elem32*>(out->dptr));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }

    int gzk_swap_outer(gzk_ctx* ctx, const gzk_buf* in, size_t d0, size_t d1, size_t d2, gzk_buf* out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (!movable(in) || !movable(out) || in == out || in->dptr == out->dptr) return fail(ctx, GZK_E_INVALID, "swap_outer: field-element buffers, out distinct from in");
        const size_t total = d0 * d1 * d2;
        if ((d0 != 0 && d1 != 0 && total / d0 / d1 != d2) || in->count < total || out->count < total || out->kind != in->kind)
            return fail(ctx, GZK_E_INVALID, "swap_outer: buffers must hold d0*d1*d2 elements of the same kind");
        if (total == 0) return GZK_OK;
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        uint64_t blocks = (total + 255) / 256;
        const uint64_t cap = static_cast<uint64_t>(ctx->sm_count) * 16;
        if (blocks > cap) blocks = cap;
        {
            LaunchScope scope(ctx, "swap_outer");
            swap_outer_kernel<<<static_cast<unsigned>(blocks), 256, 0, ctx->stream>>>(static_cast<const Elem32*>(in->dptr), d0, d1, d2,
                                                                                      static_cast<Elem32*>(out->dptr));
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }

    int gzk_ntt_twiddle(gzk_ctx* ctx, gzk_buf* buf, unsigned log2n, uint64_t row_first, size_t rows, size_t cols, int inverse)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (buf == nullptr || buf->kind != GZK_KIND_FR_MONT) return fail(ctx, GZK_E_INVALID, "ntt_twiddle: buffer must be a Montgomery buffer");
        if (log2n > 30) return fail(ctx, GZK_E_INVALID, "ntt_twiddle: domain too large");
        const uint64_t n = 1ULL << log2n;
        if (rows != 0 && (cols > buf->count / rows || cols > n || row_first + rows > n)) return fail(ctx, GZK_E_INVALID, "ntt_twiddle: block exceeds the buffer or the domain");
        if (rows == 0 || cols == 0) return GZK_OK;
        const DomainTables* dom = nullptr;
        int rc = get_domain(ctx, log2n, &dom);
        if (rc != GZK_OK) return rc;
        uint64_t blocks = (static_cast<uint64_t>(rows) * cols + 255) / 256;
        const uint64_t cap = static_cast<uint64_t>(ctx->sm_count) * 16;
        if (blocks > cap) blocks = cap;
        {
            LaunchScope scope(ctx, "ntt_twiddle");
            twiddle_kernel<<<static_cast<unsigned>(blocks), 256, 0, ctx->stream>>>(static_cast<Fr*>(buf->dptr), row_first, rows, cols, log2n,
                                                                                   inverse ? dom->lo_inv : dom->lo, inverse ? dom->hi_inv : dom->hi,
                                                                                   dom->lo_bits);
        }
        GZK_CUDA_TRY(ctx, cudaGetLastError());
        return finish_call(ctx, "invalid input");
    }
}
