// Multi-GPU exchange behind the C ABI: one NCCL communicator per context (one process per GPU),
// the few collectives the sharded hot path needs, and the row-sharded transform as one call.
//
//  - partial sums of a row-sharded packed evaluation: all-gather of K*P field elements per rank
//    into this GPU's own memory, then a kernel adds the ranks' contributions mod r (NCCL has no
//    reduction over a prime field);
//  - carries of sharded running sums and per-rank MSM results: plain all-gather;
//  - the two transposes of the four-step transform: all-to-all (grouped send / receive).
// Data always lands in the receiver's own HBM before one of this library's kernels reads it; no
// kernel here reads a peer's memory.
//
// Failure handling: a collective whose peer never arrives would wait on the GPU for ever.  Every
// exchange can be followed by gzk_comm_wait, which polls the stream from the host for at most
// the communicator's time limit and then aborts the communicator (ncclCommAbort ends the waiting
// kernel) and reports GZK_E_TIMEOUT; the context stays usable for local work.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy already loaded into the process if
// there is one), so the library loads on machines without NCCL; the entry points then fail
// with GZK_E_CUDA.
#include <dlfcn.h>

#include <chrono>
#include <cstring>
#include <thread>

#include "common.cuh"
#include "../host/bounded_wait.hpp"

namespace
{
    // the slice of the NCCL API used here (nccl.h; values are those of the stable ABI)
    typedef struct ncclComm* ncclComm_t;
    typedef struct
    {
        char internal[128];
    } ncclUniqueId;
    enum { ncclSuccess = 0, ncclInProgress = 7 };
    enum { ncclChar = 0 };

    struct NcclApi
    {
        int (*GetUniqueId)(ncclUniqueId*) = nullptr;
        int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
        int (*CommDestroy)(ncclComm_t) = nullptr;
        int (*CommAbort)(ncclComm_t) = nullptr;
        int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
        int (*Send)(const void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
        int (*Recv)(void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
        int (*GroupStart)() = nullptr;
        int (*GroupEnd)() = nullptr;
        const char* (*GetErrorString)(int) = nullptr;
        bool ok = false;
    };

    const NcclApi& nccl()
    {
        static NcclApi api = [] {
            NcclApi a;
            void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);  // the copy the process already uses, if any
            if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
            if (h == nullptr) return a;
            auto sym = [&](const char* name) { return dlsym(h, name); };
            a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
            a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
            a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
            a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(sym("ncclCommAbort"));
            a.AllGather = reinterpret_cast<decltype(a.AllGather)>(sym("ncclAllGather"));
            a.Send = reinterpret_cast<decltype(a.Send)>(sym("ncclSend"));
            a.Recv = reinterpret_cast<decltype(a.Recv)>(sym("ncclRecv"));
            a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(sym("ncclGroupStart"));
            a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(sym("ncclGroupEnd"));
            a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
            a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.CommAbort && a.AllGather && a.Send && a.Recv && a.GroupStart && a.GroupEnd;
            return a;
        }();
        return api;
    }
}

struct gzk_comm
{
    gzk_ctx* ctx = nullptr;
    ncclComm_t comm = nullptr;
    int nranks = 1, rank = 0;
    double timeout_seconds = 30.0;
    bool aborted = false;
    void* gather = nullptr;  // all-gather landing area in this GPU's memory
    size_t gather_bytes = 0;
};

namespace gzk
{
    namespace
    {
        constexpr int kThreads = 256;

        // out[i] = sum over ranks of gathered[rank][i]
        __global__ void sum_ranks_kernel(const Fr* gathered, uint32_t ranks, uint64_t count, Fr* out)
        {
            const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
            for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
            {
                Fr acc = load_fr_plain(gathered + i);
                for (uint32_t g = 1; g < ranks; ++g) acc = add(acc, load_fr_plain(gathered + static_cast<uint64_t>(g) * count + i));
                store_fr(out + i, acc);
            }
        }

        int nccl_fail(gzk_comm* c, int rc, const char* what)
        {
            const char* text = nccl().GetErrorString != nullptr ? nccl().GetErrorString(rc) : "?";
            return fail(c->ctx, GZK_E_CUDA, std::string("NCCL error: ") + text + " in " + what);
        }

        int ensure_gather(gzk_comm* c, size_t bytes)
        {
            if (c->gather_bytes >= bytes) return GZK_OK;
            if (c->gather != nullptr)
            {
                GZK_CUDA_TRY(c->ctx, cudaStreamSynchronize(c->ctx->stream));
                GZK_CUDA_TRY(c->ctx, cudaFree(c->gather));
                c->gather = nullptr;
                c->gather_bytes = 0;
            }
            const size_t rounded = (bytes + (1u << 20) - 1) & ~static_cast<size_t>((1u << 20) - 1);
            GZK_CUDA_TRY(c->ctx, cudaMalloc(&c->gather, rounded));
            c->gather_bytes = rounded;
            return GZK_OK;
        }

        int comm_ready(gzk_comm* c, const char* what)
        {
            if (c == nullptr) return GZK_E_INVALID;
            if (c->aborted) return fail(c->ctx, GZK_E_TIMEOUT, std::string(what) + ": the communicator was aborted after a time-out");
            return cudaSetDevice(c->ctx->device) == cudaSuccess ? GZK_OK : fail(c->ctx, GZK_E_CUDA, "cudaSetDevice failed");
        }
    }
}

using namespace gzk;

extern "C"
{
    int gzk_comm_unique_id(uint8_t out[128])
    {
        if (out == nullptr) return GZK_E_INVALID;
        if (!nccl().ok) return GZK_E_CUDA;
        ncclUniqueId id;
        if (nccl().GetUniqueId(&id) != ncclSuccess) return GZK_E_CUDA;
        std::memcpy(out, id.internal, 128);
        return GZK_OK;
    }

    int gzk_comm_create(gzk_ctx* ctx, int nranks, int rank, const uint8_t unique_id[128], gzk_comm** out)
    {
        if (ctx == nullptr || out == nullptr) return GZK_E_INVALID;
        *out = nullptr;
        if (unique_id == nullptr || nranks < 1 || rank < 0 || rank >= nranks) return fail(ctx, GZK_E_INVALID, "comm_create: bad rank or missing id");
        if (!nccl().ok) return fail(ctx, GZK_E_CUDA, "comm_create: libnccl.so.2 could not be loaded");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        gzk_comm* c = new (std::nothrow) gzk_comm();
        if (c == nullptr) return fail(ctx, GZK_E_INVALID, "out of host memory");
        c->ctx = ctx;
        c->nranks = nranks;
        c->rank = rank;
        ncclUniqueId id;
        std::memcpy(id.internal, unique_id, 128);
        const int rc = nccl().CommInitRank(&c->comm, nranks, id, rank);
        if (rc != ncclSuccess)
        {
            const int code = nccl_fail(c, rc, "ncclCommInitRank");
            delete c;
            return code;
        }
        *out = c;
        return GZK_OK;
    }

    void gzk_comm_destroy(gzk_comm* c)
    {
        if (c == nullptr) return;
        cudaSetDevice(c->ctx->device);
        if (!c->aborted)
        {
            cudaStreamSynchronize(c->ctx->stream);
            if (c->comm != nullptr) nccl().CommDestroy(c->comm);
        }
        if (c->gather != nullptr) cudaFree(c->gather);
        delete c;
    }

    int gzk_comm_set_timeout(gzk_comm* c, double seconds)
    {
        if (c == nullptr || !(seconds > 0.0)) return GZK_E_INVALID;
        c->timeout_seconds = seconds;
        return GZK_OK;
    }

    int gzk_comm_rank(const gzk_comm* c) { return c == nullptr ? -1 : c->rank; }
    int gzk_comm_size(const gzk_comm* c) { return c == nullptr ? 0 : c->nranks; }

    // Waits on the host for everything queued on the context's stream, at most the time limit: when it
    // runs out the communicator is aborted (the collective that never completed is torn down) and
    // GZK_E_TIMEOUT is returned; later exchanges on this communicator fail at once.
    int gzk_comm_wait(gzk_comm* c)
    {
        int rc = comm_ready(c, "comm_wait");
        if (rc != GZK_OK) return rc;
        cudaError_t query_error = cudaSuccess;
        const WaitResult result = bounded_wait(
            [&]() {
                const cudaError_t q = cudaStreamQuery(c->ctx->stream);
                if (q == cudaSuccess) return WaitState::Ready;
                if (q == cudaErrorNotReady) return WaitState::Pending;
                query_error = q;
                return WaitState::Failed;
            },
            [&]() {
                nccl().CommAbort(c->comm);
                c->comm = nullptr;
                c->aborted = true;
                cudaStreamSynchronize(c->ctx->stream);  // the aborted collective's kernel ends
            },
            c->timeout_seconds);
        if (result == WaitResult::Completed) return GZK_OK;
        if (result == WaitResult::QueryFailed) return cuda_fail(c->ctx, query_error, "cudaStreamQuery");
        return fail(c->ctx, GZK_E_TIMEOUT, "comm_wait: a collective did not complete within the time limit; the communicator was aborted");
    }

    int gzk_comm_allgather(gzk_comm* c, const gzk_buf* in, size_t count, gzk_buf* out)
    {
        int rc = comm_ready(c, "comm_allgather");
        if (rc != GZK_OK) return rc;
        if (count == 0) return GZK_OK;
        if (in == nullptr || out == nullptr || in->elem_bytes != out->elem_bytes || in->count < count || out->count < count * static_cast<size_t>(c->nranks))
            return fail(c->ctx, GZK_E_INVALID, "comm_allgather: the output must hold nranks * count elements of the input's kind");
        LaunchScope scope(c->ctx, "nccl_allgather");
        const int nrc = nccl().AllGather(in->dptr, out->dptr, count * in->elem_bytes, ncclChar, c->comm, c->ctx->stream);
        if (nrc != ncclSuccess) return nccl_fail(c, nrc, "ncclAllGather");
        return GZK_OK;
    }

    // out[i] = sum over all ranks of their in[i] (mod r): all-gather into this GPU's landing area, then a local sum
    int gzk_comm_allgather_fr_sum(gzk_comm* c, const gzk_buf* in, size_t count, gzk_buf* out)
    {
        int rc = comm_ready(c, "comm_allgather_fr_sum");
        if (rc != GZK_OK) return rc;
        if (count == 0) return GZK_OK;
        const bool kinds_ok = in != nullptr && out != nullptr && (in->kind == GZK_KIND_FR || in->kind == GZK_KIND_FR_MONT) && out->kind == in->kind;
        if (!kinds_ok || in->count < count || out->count < count)
            return fail(c->ctx, GZK_E_INVALID, "comm_allgather_fr_sum: input and output must be field-element buffers of one kind holding count elements");
        if ((rc = ensure_gather(c, count * sizeof(Fr) * static_cast<size_t>(c->nranks))) != GZK_OK) return rc;
        {
            LaunchScope scope(c->ctx, "nccl_allgather");
            const int nrc = nccl().AllGather(in->dptr, c->gather, count * sizeof(Fr), ncclChar, c->comm, c->ctx->stream);
            if (nrc != ncclSuccess) return nccl_fail(c, nrc, "ncclAllGather");
        }
        {
            LaunchScope scope(c->ctx, "sum_ranks");
            const unsigned blocks = static_cast<unsigned>((count + kThreads - 1) / kThreads < 1024 ? (count + kThreads - 1) / kThreads : 1024);
            sum_ranks_kernel<<<blocks, kThreads, 0, c->ctx->stream>>>(static_cast<const Fr*>(c->gather), static_cast<uint32_t>(c->nranks), count,
                                                                       static_cast<Fr*>(out->dptr));
        }
        GZK_CUDA_TRY(c->ctx, cudaGetLastError());
        return GZK_OK;
    }

    // chunk g of `in` (count_per_rank elements) goes to rank g; chunk h of `out` comes from rank h
    int gzk_comm_alltoall(gzk_comm* c, const gzk_buf* in, size_t count_per_rank, gzk_buf* out)
    {
        int rc = comm_ready(c, "comm_alltoall");
        if (rc != GZK_OK) return rc;
        if (count_per_rank == 0) return GZK_OK;
        const size_t total = count_per_rank * static_cast<size_t>(c->nranks);
        if (in == nullptr || out == nullptr || in->elem_bytes != out->elem_bytes || in->count < total || out->count < total || in->dptr == out->dptr)
            return fail(c->ctx, GZK_E_INVALID, "comm_alltoall: two different buffers of nranks * count_per_rank elements each");
        const size_t bytes = count_per_rank * in->elem_bytes;
        LaunchScope scope(c->ctx, "nccl_alltoall");
        int nrc = nccl().GroupStart();
        for (int g = 0; nrc == ncclSuccess && g < c->nranks; ++g)
        {
            nrc = nccl().Send(static_cast<const char*>(in->dptr) + static_cast<size_t>(g) * bytes, bytes, ncclChar, g, c->comm, c->ctx->stream);
            if (nrc == ncclSuccess) nrc = nccl().Recv(static_cast<char*>(out->dptr) + static_cast<size_t>(g) * bytes, bytes, ncclChar, g, c->comm, c->ctx->stream);
        }
        const int end_rc = nccl().GroupEnd();
        if (nrc != ncclSuccess) return nccl_fail(c, nrc, "ncclSend/ncclRecv");
        if (end_rc != ncclSuccess) return nccl_fail(c, end_rc, "ncclGroupEnd");
        return GZK_OK;
    }

    // Row-sharded forward transform of n = 2^log2n elements over the communicator's ranks (a power of two):
    // this rank holds rows i1 of its block of the n1 x n2 matrix (n1 = 2^(log2n / 2)) in `rows` and ends
    // with X[k1 + n1 * k2] for k1 in its block in `out` ([k1 local][k2], Montgomery form).  `work` is a
    // second buffer of the local size.  Pack -> all-to-all -> transpose -> length-n1 transforms -> twiddle ->
    // pack -> all-to-all -> transpose -> length-n2 transforms; both exchanges land in this GPU's memory.
    int gzk_ntt_sharded(gzk_comm* c, const gzk_buf* rows, unsigned log2n, gzk_buf* work, gzk_buf* out)
    {
        int rc = comm_ready(c, "ntt_sharded");
        if (rc != GZK_OK) return rc;
        gzk_ctx* ctx = c->ctx;
        const unsigned world = static_cast<unsigned>(c->nranks);
        unsigned lw = 0;
        while ((1u << lw) < world) ++lw;
        if ((1u << lw) != world) return fail(ctx, GZK_E_INVALID, "ntt_sharded: the number of ranks must be a power of two");
        const unsigned l1 = log2n / 2, l2 = log2n - l1;
        if (l1 < lw || log2n > 40) return fail(ctx, GZK_E_INVALID, "ntt_sharded: 2^log2n is too small to split over this many ranks");
        const size_t n1 = static_cast<size_t>(1) << l1, n2 = static_cast<size_t>(1) << l2;
        const size_t rows1 = n1 / world, cols2 = n2 / world, local = rows1 * n2;
        if (rows == nullptr || work == nullptr || out == nullptr || rows->count < local || work->count < local || out->count < local)
            return fail(ctx, GZK_E_INVALID, "ntt_sharded: every buffer holds n / ranks elements");
        const bool field_in = rows->kind == GZK_KIND_FR || rows->kind == GZK_KIND_FR_MONT;
        const bool field_work = work->kind == GZK_KIND_FR || work->kind == GZK_KIND_FR_MONT;
        if (!field_in || !field_work || out->kind != GZK_KIND_FR_MONT || work->dptr == out->dptr || rows->dptr == work->dptr || rows->dptr == out->dptr)
            return fail(ctx, GZK_E_INVALID, "ntt_sharded: three different field-element buffers, the output in Montgomery form");
        const int in_kind = rows->kind;
        // [dest][i1 local][i2 local] <- [i1 local][dest][i2 local]
        gzk_buf_retag(work, in_kind);
        if ((rc = gzk_swap_outer(ctx, rows, rows1, world, cols2, work)) != GZK_OK) return rc;
        gzk_buf_retag(out, in_kind);
        if ((rc = gzk_comm_alltoall(c, work, rows1 * cols2, out)) != GZK_OK) return rc;       // out: [i1][i2 local]
        if ((rc = gzk_transpose(ctx, out, n1, cols2, work)) != GZK_OK) return rc;               // work: [i2 local][i1]
        gzk_buf_retag(out, GZK_KIND_FR_MONT);
        if ((rc = gzk_ntt(ctx, work, out, l1, cols2, 0, nullptr)) != GZK_OK) return rc;         // out: [i2 local][k1]
        if ((rc = gzk_ntt_twiddle(ctx, out, log2n, static_cast<uint64_t>(c->rank) * cols2, cols2, n1, 0)) != GZK_OK) return rc;
        gzk_buf_retag(work, GZK_KIND_FR_MONT);
        if ((rc = gzk_swap_outer(ctx, out, cols2, world, rows1, work)) != GZK_OK) return rc;   // work: [dest][i2 local][k1 local]
        if ((rc = gzk_comm_alltoall(c, work, cols2 * rows1, out)) != GZK_OK) return rc;         // out: [i2][k1 local]
        if ((rc = gzk_transpose(ctx, out, n2, rows1, work)) != GZK_OK) return rc;               // work: [k1 local][i2]
        return gzk_ntt(ctx, work, out, l2, rows1, 0, nullptr);                                  // out: [k1 local][k2]
    }
}
