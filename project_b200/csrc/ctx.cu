// Context, device buffers and domain tables of libgatzk_b200.so.
#include <cstring>
#include <new>

#include "common.cuh"

namespace gzk
{
    int launch_convert_fp(gzk_ctx* ctx, const void* in, void* out, size_t fp_count, bool to_montgomery);
    void g1_release_tables(gzk_ctx* ctx);

    int fail(gzk_ctx* ctx, int code, const std::string& message)
    {
        if (ctx != nullptr) ctx->last_error = message;
        return code;
    }

    int cuda_fail(gzk_ctx* ctx, cudaError_t err, const char* what)
    {
        return fail(ctx, GZK_E_CUDA, std::string("CUDA error: ") + cudaGetErrorString(err) + " in " + what);
    }

    int ensure_scratch(gzk_ctx* ctx, int slot, size_t bytes, void** out)
    {
        Scratch& s = ctx->scratch[slot];
        if (s.bytes < bytes)
        {
            if (s.ptr != nullptr)
            {
                GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
                GZK_CUDA_TRY(ctx, cudaFree(s.ptr));
                s.ptr = nullptr;
                s.bytes = 0;
            }
            const size_t rounded = (bytes + (1u << 20) - 1) & ~static_cast<size_t>((1u << 20) - 1);
            GZK_CUDA_TRY(ctx, cudaMalloc(&s.ptr, rounded));
            s.bytes = rounded;
        }
        *out = s.ptr;
        return GZK_OK;
    }

    int ensure_pinned(gzk_ctx* ctx, size_t bytes, void** out)
    {
        if (ctx->pinned_bytes < bytes)
        {
            if (ctx->pinned != nullptr)
            {
                GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
                GZK_CUDA_TRY(ctx, cudaFreeHost(ctx->pinned));
                ctx->pinned = nullptr;
                ctx->pinned_bytes = 0;
            }
            const size_t rounded = (bytes + 65535) & ~static_cast<size_t>(65535);
            GZK_CUDA_TRY(ctx, cudaMallocHost(&ctx->pinned, rounded));
            ctx->pinned_bytes = rounded;
        }
        *out = ctx->pinned;
        return GZK_OK;
    }

    static int family_index(gzk_ctx* ctx, const char* family)
    {
        for (size_t i = 0; i < ctx->families.size(); ++i)
            if (ctx->families[i].name == family) return static_cast<int>(i);
        FamilyStat st;
        st.name = family;
        ctx->families.push_back(st);
        return static_cast<int>(ctx->families.size() - 1);
    }

    static cudaEvent_t take_event(gzk_ctx* ctx)
    {
        if (!ctx->event_pool.empty())
        {
            cudaEvent_t e = ctx->event_pool.back();
            ctx->event_pool.pop_back();
            return e;
        }
        cudaEvent_t e = nullptr;
        cudaEventCreate(&e);
        return e;
    }

    LaunchScope::LaunchScope(gzk_ctx* ctx, const char* family, unsigned launches) : ctx_(ctx), family_(family_index(ctx, family))
    {
        ctx_->families[family_].launches += launches;
        if (ctx_->timing)
        {
            start_ = take_event(ctx_);
            cudaEventRecord(start_, ctx_->stream);
        }
    }

    LaunchScope::~LaunchScope()
    {
        if (start_ != nullptr)
        {
            TimedLaunch t;
            t.family = family_;
            t.start = start_;
            t.stop = take_event(ctx_);
            cudaEventRecord(t.stop, ctx_->stream);
            ctx_->pending.push_back(t);
        }
    }

    void timing_collect(gzk_ctx* ctx)
    {
        if (ctx->pending.empty()) return;
        cudaStreamSynchronize(ctx->stream);
        for (auto& t : ctx->pending)
        {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, t.start, t.stop) == cudaSuccess) ctx->families[t.family].total_ms += ms;
            ctx->event_pool.push_back(t.start);
            ctx->event_pool.push_back(t.stop);
        }
        ctx->pending.clear();
    }

    // words[0] = status code, words[1] = the raising site (see raise_status)
    static int status_to_error(gzk_ctx* ctx, const int* words, const char* invalid_message)
    {
        const int status = words[0];
        if (status == 0) return GZK_OK;
        cudaMemsetAsync(ctx->d_status, 0, 2 * sizeof(int), ctx->stream);
        const std::string site = " [raised at site " + std::to_string(words[1]) + "]";
        if (status == GZK_E_DOMAIN) return fail(ctx, GZK_E_DOMAIN, "batch_invert encountered zero" + site);
        if (status == GZK_E_TIMEOUT) return fail(ctx, GZK_E_TIMEOUT, "a bounded wait on a bulk copy gave up" + site);
        if (status != GZK_E_INVALID) return fail(ctx, GZK_E_INVALID, std::string(invalid_message) + " [unexpected status word " + std::to_string(status) + "]" + site);
        return fail(ctx, GZK_E_INVALID, invalid_message + site);
    }

    int begin_call(gzk_ctx* ctx)
    {
        if (!ctx->deferred) GZK_CUDA_TRY(ctx, cudaMemsetAsync(ctx->d_status, 0, 2 * sizeof(int), ctx->stream));
        return GZK_OK;
    }

    int finish_call(gzk_ctx* ctx, const char* invalid_message)
    {
        if (ctx->deferred) return GZK_OK;
        int status[2] = {0, 0};
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(status, ctx->d_status, sizeof(status), cudaMemcpyDeviceToHost, ctx->stream));
        GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        return status_to_error(ctx, status, invalid_message);
    }

    Fr host_fr_from_bytes(const uint8_t* bytes, bool* canonical_ok)
    {
        Fr v;
        std::memcpy(v.l, bytes, 32);
        // canonical <=> v < r
        bool less = false;
        for (int i = 7; i >= 0; --i)
        {
            if (v.l[i] != FrCfg::mod(i))
            {
                less = v.l[i] < FrCfg::mod(i);
                break;
            }
        }
        if (canonical_ok != nullptr) *canonical_ok = less;
        return v;
    }

    void host_fr_to_bytes(const Fr& canonical, uint8_t* bytes) { std::memcpy(bytes, canonical.l, 32); }

    namespace
    {
        // 5^((r - 1) >> log2n), as FieldElement::root_of_unity divides (r-1) by n
        Fr root_of_unity_by_power(unsigned log2n)
        {
            uint32_t e[8];
            for (int i = 0; i < 8; ++i) e[i] = FrCfg::mod(i);
            e[0] -= 1;
            for (unsigned s = 0; s < log2n; ++s)
            {
                for (int i = 0; i < 8; ++i)
                {
                    e[i] >>= 1;
                    if (i + 1 < 8) e[i] |= e[i + 1] << 31;
                }
            }
            Fr five = Fr::zero();
            five.l[0] = 5;
            const Fr base = to_mont(five);
            Fr out = Fr::one();
            bool started = false;
            for (int limb = 7; limb >= 0; --limb)
            {
                for (int bit = 31; bit >= 0; --bit)
                {
                    if (started) out = sqr(out);
                    if ((e[limb] >> bit) & 1U)
                    {
                        out = started ? mul(out, base) : base;
                        started = true;
                    }
                }
            }
            return out;
        }
        struct RootTable
        {
            Fr root[33];
            // the 2^32-th root by one exponentiation, every smaller one by squaring it
            RootTable()
            {
                root[32] = root_of_unity_by_power(32);
                for (int k = 31; k >= 0; --k) root[k] = sqr(root[k + 1]);
            }
        };
    }

    // Every weight vector and every domain asks for a root; the table is built on first use.
    Fr host_root_of_unity(unsigned log2n)
    {
        static const RootTable table;
        return table.root[log2n <= 32 ? log2n : 32];
    }

    int get_domain(gzk_ctx* ctx, unsigned log2n, const DomainTables** out)
    {
        if (log2n > 32) return fail(ctx, GZK_E_INVALID, "domain size exceeds the 2-adicity of Fr");
        auto it = ctx->domains.find(log2n);
        if (it != ctx->domains.end())
        {
            *out = &it->second;
            return GZK_OK;
        }
        DomainTables t;
        t.log2n = log2n;
        t.lo_bits = log2n < 12 ? log2n : (log2n + 1) / 2 > 12 ? (log2n + 1) / 2 : 12;
        if (t.lo_bits > log2n) t.lo_bits = log2n;
        const size_t lo_count = static_cast<size_t>(1) << t.lo_bits;
        const size_t hi_count = static_cast<size_t>(1) << (log2n - t.lo_bits);
        t.omega = host_root_of_unity(log2n);
        const Fr omega_inv = inv(t.omega);
        {
            Fr n_plain = Fr::zero();
            const uint64_t n = 1ULL << log2n;
            n_plain.l[0] = static_cast<uint32_t>(n);
            n_plain.l[1] = static_cast<uint32_t>(n >> 32);
            t.inv_size = inv(to_mont(n_plain));
        }
        std::vector<Fr> host(lo_count > hi_count ? lo_count : hi_count);
        auto build = [&](const Fr& step, size_t count, Fr** dptr) -> int {
            Fr cur = Fr::one();
            for (size_t j = 0; j < count; ++j)
            {
                host[j] = cur;
                cur = mul(cur, step);
            }
            GZK_CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void**>(dptr), count * sizeof(Fr)));
            GZK_CUDA_TRY(ctx, cudaMemcpyAsync(*dptr, host.data(), count * sizeof(Fr), cudaMemcpyHostToDevice, ctx->stream));
            GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            return GZK_OK;
        };
        Fr hi_step = t.omega, hi_step_inv = omega_inv;
        for (unsigned s = 0; s < t.lo_bits; ++s)
        {
            hi_step = sqr(hi_step);
            hi_step_inv = sqr(hi_step_inv);
        }
        int rc;
        if ((rc = build(t.omega, lo_count, &t.lo)) != GZK_OK) return rc;
        if ((rc = build(hi_step, hi_count, &t.hi)) != GZK_OK) return rc;
        if ((rc = build(omega_inv, lo_count, &t.lo_inv)) != GZK_OK) return rc;
        if ((rc = build(hi_step_inv, hi_count, &t.hi_inv)) != GZK_OK) return rc;
        auto ins = ctx->domains.emplace(log2n, t);
        *out = &ins.first->second;
        return GZK_OK;
    }

    __global__ void convert_kernel(const Fr* in, Fr* out, size_t count, int to_montgomery)
    {
        const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
        for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        {
            const Fr v = load_fr(in + i);
            store_fr(out + i, to_montgomery ? to_mont(v) : from_mont(v));
        }
    }
}

using namespace gzk;

extern "C"
{
    int gzk_ctx_create(int device, gzk_ctx** out)
    {
        if (out == nullptr) return GZK_E_INVALID;
        *out = nullptr;
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0 || device < 0 || device >= count) return GZK_E_CUDA;
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return GZK_E_CUDA;
        if (prop.major != 10) return GZK_E_CUDA;  // built for sm_100a only
        if (cudaSetDevice(device) != cudaSuccess) return GZK_E_CUDA;
        gzk_ctx* ctx = new (std::nothrow) gzk_ctx();
        if (ctx == nullptr) return GZK_E_INVALID;
        ctx->device = device;
        ctx->sm_count = prop.multiProcessorCount;
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&ctx->copy_event, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&ctx->order_event, cudaEventDisableTiming) != cudaSuccess ||
            cudaMalloc(reinterpret_cast<void**>(&ctx->d_status), 64) != cudaSuccess ||
            // cleared ON THE CONTEXT'S STREAM and waited for: a cudaMemset would run on the legacy default stream, which
            // is not ordered with this non-blocking stream, so the first status read (gzk_ctx_set_deferred,
            // microseconds later) could overtake it and see whatever the memory held before - e.g. the
            // Montgomery 1 at the head of a domain table a context destroyed just before had freed
            cudaMemsetAsync(ctx->d_status, 0, 64, ctx->stream) != cudaSuccess || cudaStreamSynchronize(ctx->stream) != cudaSuccess)
        {
            delete ctx;
            return GZK_E_CUDA;
        }
        *out = ctx;
        return GZK_OK;
    }

    void gzk_ctx_destroy(gzk_ctx* ctx)
    {
        if (ctx == nullptr) return;
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);
        for (auto& kv : ctx->domains)
        {
            cudaFree(kv.second.lo);
            cudaFree(kv.second.hi);
            cudaFree(kv.second.lo_inv);
            cudaFree(kv.second.hi_inv);
        }
        for (auto& s : ctx->scratch)
            if (s.ptr != nullptr) cudaFree(s.ptr);
        for (Fr* t : ctx->ntt_small)
            if (t != nullptr) cudaFree(t);
        for (auto& t : ctx->ntt_twists) cudaFree(t.table);
        if (ctx->pinned != nullptr) cudaFreeHost(ctx->pinned);
        if (ctx->upload_ring != nullptr)
        {
            cudaFreeHost(ctx->upload_ring);
            for (auto e : ctx->upload_done) cudaEventDestroy(e);
        }
        if (ctx->d_status != nullptr) cudaFree(ctx->d_status);
        timing_collect(ctx);
        g1_release_tables(ctx);
        for (auto e : ctx->event_pool) cudaEventDestroy(e);
        cudaStreamSynchronize(ctx->copy_stream);
        cudaEventDestroy(ctx->copy_event);
        cudaEventDestroy(ctx->order_event);
        cudaStreamDestroy(ctx->copy_stream);
        cudaStreamDestroy(ctx->stream);
        delete ctx;
    }

    const char* gzk_last_error(const gzk_ctx* ctx) { return ctx == nullptr ? "no context" : ctx->last_error.c_str(); }

    int gzk_ctx_synchronize(gzk_ctx* ctx)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        int status[2] = {0, 0};
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(status, ctx->d_status, sizeof(status), cudaMemcpyDeviceToHost, ctx->stream));
        GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        return status_to_error(ctx, status, "a deferred call reported invalid input (index out of range, non-boolean selector or bad group bounds)");
    }

    int gzk_ctx_set_deferred(gzk_ctx* ctx, int on)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        const int rc = gzk_ctx_synchronize(ctx);
        ctx->deferred = on != 0;
        return rc;
    }

    void* gzk_ctx_stream(gzk_ctx* ctx) { return ctx == nullptr ? nullptr : ctx->stream; }

    // Everything queued on `ctx` from now on runs after everything queued on `other` so far (an event on the
    // one stream, a wait on the other: nothing blocks on the host).  Both contexts must be on the same GPU.
    int gzk_ctx_wait_for(gzk_ctx* ctx, gzk_ctx* other)
    {
        if (ctx == nullptr || other == nullptr) return GZK_E_INVALID;
        if (ctx == other) return GZK_OK;
        if (ctx->device != other->device) return fail(ctx, GZK_E_INVALID, "ctx_wait_for: contexts of different GPUs");
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        GZK_CUDA_TRY(ctx, cudaEventRecord(other->order_event, other->stream));
        GZK_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, other->order_event, 0));
        return GZK_OK;
    }

    int gzk_timing_enable(gzk_ctx* ctx, int on)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        timing_collect(ctx);
        ctx->timing = on != 0;
        return GZK_OK;
    }

    int gzk_timing_reset(gzk_ctx* ctx)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        timing_collect(ctx);
        for (auto& f : ctx->families)
        {
            f.launches = 0;
            f.total_ms = 0.0;
        }
        ctx->eval_algorithmic_bytes = 0;
        ctx->eval_limb_products = 0;
        ctx->eval_terms = 0;
        return GZK_OK;
    }

    int gzk_eval_work_counters(gzk_ctx* ctx, uint64_t out[3])
    {
        if (ctx == nullptr || out == nullptr) return GZK_E_INVALID;
        out[0] = ctx->eval_algorithmic_bytes;
        out[1] = ctx->eval_limb_products;
        out[2] = ctx->eval_terms;
        return GZK_OK;
    }

    int gzk_timing_family_count(gzk_ctx* ctx) { return ctx == nullptr ? 0 : static_cast<int>(ctx->families.size()); }

    int gzk_timing_get(gzk_ctx* ctx, int index, const char** name, uint64_t* launches, double* total_ms)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        timing_collect(ctx);
        if (index < 0 || index >= static_cast<int>(ctx->families.size())) return fail(ctx, GZK_E_INVALID, "timing: no such family");
        if (name != nullptr) *name = ctx->families[index].name.c_str();
        if (launches != nullptr) *launches = ctx->families[index].launches;
        if (total_ms != nullptr) *total_ms = ctx->families[index].total_ms;
        return GZK_OK;
    }

    int gzk_buf_alloc(gzk_ctx* ctx, int kind, size_t count, gzk_buf** out)
    {
        if (ctx == nullptr || out == nullptr) return GZK_E_INVALID;
        size_t elem = 0;
        switch (kind)
        {
        case GZK_KIND_FR:
        case GZK_KIND_FR_MONT: elem = 32; break;
        case GZK_KIND_I64:
        case GZK_KIND_F64: elem = 8; break;
        case GZK_KIND_U32: elem = 4; break;
        case GZK_KIND_G1: elem = 96; break;
        default: return fail(ctx, GZK_E_INVALID, "unknown buffer kind");
        }
        GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        gzk_buf* b = new (std::nothrow) gzk_buf();
        if (b == nullptr) return fail(ctx, GZK_E_INVALID, "out of host memory");
        b->count = count;
        b->kind = kind;
        b->elem_bytes = elem;
        const size_t bytes = count * elem > 0 ? count * elem : 32;
        const cudaError_t err = cudaMalloc(&b->dptr, bytes);
        if (err != cudaSuccess)
        {
            delete b;
            return cuda_fail(ctx, err, "cudaMalloc(buffer)");
        }
        *out = b;
        return GZK_OK;
    }

    int gzk_buf_free(gzk_ctx* ctx, gzk_buf* buf)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (buf == nullptr) return GZK_OK;
        GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        if (buf->owned) GZK_CUDA_TRY(ctx, cudaFree(buf->dptr));
        delete buf;
        return GZK_OK;
    }

    int gzk_buf_retag(gzk_buf* buf, int kind)
    {
        if (buf == nullptr) return GZK_E_INVALID;
        const bool field_now = buf->kind == GZK_KIND_FR || buf->kind == GZK_KIND_FR_MONT;
        const bool field_then = kind == GZK_KIND_FR || kind == GZK_KIND_FR_MONT;
        if (!field_now || !field_then) return GZK_E_INVALID;
        buf->kind = kind;
        return GZK_OK;
    }

    int gzk_buf_wrap(gzk_ctx* ctx, int kind, size_t count, void* device_ptr, gzk_buf** out)
    {
        if (ctx == nullptr || out == nullptr) return GZK_E_INVALID;
        size_t elem = 0;
        switch (kind)
        {
        case GZK_KIND_FR:
        case GZK_KIND_FR_MONT: elem = 32; break;
        case GZK_KIND_I64:
        case GZK_KIND_F64: elem = 8; break;
        case GZK_KIND_U32: elem = 4; break;
        case GZK_KIND_G1: elem = 96; break;
        default: return fail(ctx, GZK_E_INVALID, "unknown buffer kind");
        }
        if (device_ptr == nullptr || reinterpret_cast<uintptr_t>(device_ptr) % 32 != 0)
            return fail(ctx, GZK_E_INVALID, "buf_wrap: device pointer must be non-null and 32-byte aligned");
        cudaPointerAttributes attr{};
        GZK_CUDA_TRY(ctx, cudaPointerGetAttributes(&attr, device_ptr));
        if (attr.type != cudaMemoryTypeDevice || attr.device != ctx->device)
            return fail(ctx, GZK_E_INVALID, "buf_wrap: pointer is not device memory of this context's GPU");
        gzk_buf* b = new (std::nothrow) gzk_buf();
        if (b == nullptr) return fail(ctx, GZK_E_INVALID, "out of host memory");
        b->dptr = device_ptr;
        b->count = count;
        b->kind = kind;
        b->elem_bytes = elem;
        b->owned = false;
        *out = b;
        return GZK_OK;
    }

    int gzk_buf_upload(gzk_ctx* ctx, gzk_buf* buf, size_t offset, const void* host, size_t count)
    {
        if (ctx == nullptr || buf == nullptr || (host == nullptr && count != 0)) return GZK_E_INVALID;
        if (offset + count > buf->count) return fail(ctx, GZK_E_INVALID, "upload exceeds the buffer");
        if (count == 0) return GZK_OK;
        char* dst = static_cast<char*>(buf->dptr) + offset * buf->elem_bytes;
        const size_t bytes = count * buf->elem_bytes;
        // Deferred mode, small upload: stage it in a pinned slot and return without waiting, so that the
        // caller keeps queueing work behind the kernels still running (a synchronous upload in the
        // middle of a stage drains the stream and leaves the device idle while the host catches up).
        const bool staged = ctx->deferred && bytes <= gzk_ctx::kUploadSlotBytes;
        if (staged)
        {
            GZK_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
            if (ctx->upload_ring == nullptr)
            {
                GZK_CUDA_TRY(ctx, cudaHostAlloc(reinterpret_cast<void**>(&ctx->upload_ring), gzk_ctx::kUploadSlots * gzk_ctx::kUploadSlotBytes, cudaHostAllocDefault));
                for (auto& e : ctx->upload_done) GZK_CUDA_TRY(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
            }
            const int slot = ctx->upload_next;
            ctx->upload_next = (slot + 1) % gzk_ctx::kUploadSlots;
            if (ctx->upload_busy[slot]) GZK_CUDA_TRY(ctx, cudaEventSynchronize(ctx->upload_done[slot]));
            char* stage = ctx->upload_ring + static_cast<size_t>(slot) * gzk_ctx::kUploadSlotBytes;
            std::memcpy(stage, host, bytes);
            GZK_CUDA_TRY(ctx, cudaMemcpyAsync(dst, stage, bytes, cudaMemcpyHostToDevice, ctx->stream));
            GZK_CUDA_TRY(ctx, cudaEventRecord(ctx->upload_done[slot], ctx->stream));
            ctx->upload_busy[slot] = true;
        }
        else
        {
            GZK_CUDA_TRY(ctx, cudaMemcpyAsync(dst, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
        }
        if (buf->kind == GZK_KIND_FR_MONT)
        {
            Fr* p = reinterpret_cast<Fr*>(dst);
            const unsigned blocks = static_cast<unsigned>((count + 255) / 256 < 4096 ? (count + 255) / 256 : 4096);
            LaunchScope scope(ctx, "convert");
            convert_kernel<<<blocks, 256, 0, ctx->stream>>>(p, p, count, 1);
            GZK_CUDA_TRY(ctx, cudaGetLastError());
        }
        if (buf->kind == GZK_KIND_G1)
        {
            const int rc = launch_convert_fp(ctx, dst, dst, count * 2, true);
            if (rc != GZK_OK) return rc;
        }
        if (!staged) GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        return GZK_OK;
    }

    // Upload without waiting: the copy is queued on the context's copy stream and overlaps
    // with kernels already running on the compute stream.  `host` must stay valid (and
    // should be pinned) until gzk_copy_fence + a synchronisation; kernels issued after
    // gzk_copy_fence see the data.  FR / I64 / U32 / F64 buffers only (no conversion).
    int gzk_buf_upload_async(gzk_ctx* ctx, gzk_buf* buf, size_t offset, const void* host, size_t count)
    {
        if (ctx == nullptr || buf == nullptr || (host == nullptr && count != 0)) return GZK_E_INVALID;
        if (offset + count > buf->count) return fail(ctx, GZK_E_INVALID, "upload exceeds the buffer");
        if (buf->kind == GZK_KIND_FR_MONT || buf->kind == GZK_KIND_G1) return fail(ctx, GZK_E_INVALID, "upload_async: buffer kind needs conversion, use gzk_buf_upload");
        if (count == 0) return GZK_OK;
        char* dst = static_cast<char*>(buf->dptr) + offset * buf->elem_bytes;
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(dst, host, count * buf->elem_bytes, cudaMemcpyHostToDevice, ctx->copy_stream));
        return GZK_OK;
    }

    // Orders everything issued on the compute stream from now on after all uploads queued so far.
    int gzk_copy_fence(gzk_ctx* ctx)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        GZK_CUDA_TRY(ctx, cudaEventRecord(ctx->copy_event, ctx->copy_stream));
        GZK_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ctx->copy_event, 0));
        return GZK_OK;
    }

    // Pins (page-locks) a range of the caller's host memory so that uploads from it run as DMA at the
    // full host-to-device rate instead of through the runtime's staging copies.
    int gzk_host_register(void* host, size_t bytes)
    {
        if (host == nullptr || bytes == 0) return GZK_E_INVALID;
        const cudaError_t err = cudaHostRegister(host, bytes, cudaHostRegisterDefault);
        if (err != cudaSuccess)
        {
            cudaGetLastError();
            return GZK_E_CUDA;
        }
        return GZK_OK;
    }
    int gzk_host_unregister(void* host)
    {
        if (host == nullptr) return GZK_E_INVALID;
        if (cudaHostUnregister(host) != cudaSuccess)
        {
            cudaGetLastError();
            return GZK_E_CUDA;
        }
        return GZK_OK;
    }

    int gzk_buf_download(gzk_ctx* ctx, const gzk_buf* buf, size_t offset, void* host, size_t count)
    {
        if (ctx == nullptr || buf == nullptr || (host == nullptr && count != 0)) return GZK_E_INVALID;
        if (offset + count > buf->count) return fail(ctx, GZK_E_INVALID, "download exceeds the buffer");
        if (count == 0) return GZK_OK;
        const char* src = static_cast<const char*>(buf->dptr) + offset * buf->elem_bytes;
        if (buf->kind == GZK_KIND_FR_MONT)
        {
            // convert in chunks through context scratch so that the buffer itself stays Montgomery
            const size_t chunk = static_cast<size_t>(1) << 20;
            void* tmp = nullptr;
            int rc = ensure_scratch(ctx, 3, (count < chunk ? count : chunk) * 32, &tmp);
            if (rc != GZK_OK) return rc;
            for (size_t done = 0; done < count; done += chunk)
            {
                const size_t cur = count - done < chunk ? count - done : chunk;
                const unsigned blocks = static_cast<unsigned>((cur + 255) / 256 < 4096 ? (cur + 255) / 256 : 4096);
                {
                    LaunchScope scope(ctx, "convert");
                    convert_kernel<<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<const Fr*>(src) + done, static_cast<Fr*>(tmp), cur, 0);
                }
                GZK_CUDA_TRY(ctx, cudaGetLastError());
                GZK_CUDA_TRY(ctx, cudaMemcpyAsync(static_cast<char*>(host) + done * 32, tmp, cur * 32, cudaMemcpyDeviceToHost, ctx->stream));
                GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            }
            return GZK_OK;
        }
        if (buf->kind == GZK_KIND_G1)
        {
            const size_t chunk = static_cast<size_t>(1) << 18;
            void* tmp = nullptr;
            int rc = ensure_scratch(ctx, 3, (count < chunk ? count : chunk) * 96, &tmp);
            if (rc != GZK_OK) return rc;
            for (size_t done = 0; done < count; done += chunk)
            {
                const size_t cur = count - done < chunk ? count - done : chunk;
                if ((rc = launch_convert_fp(ctx, src + done * 96, tmp, cur * 2, false)) != GZK_OK) return rc;
                GZK_CUDA_TRY(ctx, cudaMemcpyAsync(static_cast<char*>(host) + done * 96, tmp, cur * 96, cudaMemcpyDeviceToHost, ctx->stream));
                GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            }
            return GZK_OK;
        }
        GZK_CUDA_TRY(ctx, cudaMemcpyAsync(host, src, count * buf->elem_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        GZK_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        return GZK_OK;
    }

    size_t gzk_buf_count(const gzk_buf* buf) { return buf == nullptr ? 0 : buf->count; }
    int gzk_buf_kind(const gzk_buf* buf) { return buf == nullptr ? -1 : buf->kind; }
    void* gzk_buf_device_ptr(gzk_buf* buf) { return buf == nullptr ? nullptr : buf->dptr; }

    int gzk_root_of_unity(gzk_ctx* ctx, uint64_t size, uint8_t out[32])
    {
        if (ctx == nullptr || out == nullptr) return GZK_E_INVALID;
        if (size == 0 || (size & (size - 1)) != 0) return fail(ctx, GZK_E_INVALID, "domain size must be a non-zero power of two");
        unsigned log2n = 0;
        while ((1ULL << log2n) < size) ++log2n;
        if (log2n > 32) return fail(ctx, GZK_E_INVALID, "domain size exceeds the 2-adicity of Fr");
        host_fr_to_bytes(from_mont(host_root_of_unity(log2n)), out);
        return GZK_OK;
    }

    namespace
    {
        // Montgomery product on four 64-bit limbs (coarsely integrated operand scanning): the host's
        // 64x64->128 multiplier does in 32 products what the kernels' 32-bit limb code does in 128.
        struct HostFr64
        {
            uint64_t modulus[4], r2[4], n0;  // n0 = -modulus^-1 mod 2^64
            HostFr64()
            {
                const Fr rr = Fr::r2();
                for (int i = 0; i < 4; ++i)
                {
                    modulus[i] = static_cast<uint64_t>(FrCfg::mod(2 * i)) | (static_cast<uint64_t>(FrCfg::mod(2 * i + 1)) << 32);
                    r2[i] = static_cast<uint64_t>(rr.l[2 * i]) | (static_cast<uint64_t>(rr.l[2 * i + 1]) << 32);
                }
                uint64_t x = 1;  // Newton: x <- x (2 - m x) doubles the correct low bits
                for (int i = 0; i < 6; ++i) x *= 2 - modulus[0] * x;
                n0 = ~x + 1;
            }
            void mul(const uint64_t a[4], const uint64_t b[4], uint64_t out[4]) const
            {
                using u128 = unsigned __int128;
                uint64_t t[6] = {0, 0, 0, 0, 0, 0};
                for (int i = 0; i < 4; ++i)
                {
                    uint64_t carry = 0;
                    for (int j = 0; j < 4; ++j)
                    {
                        const u128 w = static_cast<u128>(a[j]) * b[i] + t[j] + carry;
                        t[j] = static_cast<uint64_t>(w);
                        carry = static_cast<uint64_t>(w >> 64);
                    }
                    u128 top = static_cast<u128>(t[4]) + carry;
                    t[4] = static_cast<uint64_t>(top);
                    t[5] = static_cast<uint64_t>(top >> 64);
                    const uint64_t q = t[0] * n0;
                    u128 w = static_cast<u128>(q) * modulus[0] + t[0];
                    carry = static_cast<uint64_t>(w >> 64);
                    for (int j = 1; j < 4; ++j)
                    {
                        w = static_cast<u128>(q) * modulus[j] + t[j] + carry;
                        t[j - 1] = static_cast<uint64_t>(w);
                        carry = static_cast<uint64_t>(w >> 64);
                    }
                    top = static_cast<u128>(t[4]) + carry;
                    t[3] = static_cast<uint64_t>(top);
                    t[4] = t[5] + static_cast<uint64_t>(top >> 64);
                }
                // t < 2 * modulus: one conditional subtraction
                uint64_t d[4];
                unsigned __int128 borrow = 0;
                for (int j = 0; j < 4; ++j)
                {
                    const u128 w = static_cast<u128>(t[j]) - modulus[j] - static_cast<uint64_t>(borrow);
                    d[j] = static_cast<uint64_t>(w);
                    borrow = (w >> 64) & 1;
                }
                const bool keep = t[4] == 0 && borrow != 0;
                for (int j = 0; j < 4; ++j) out[j] = keep ? t[j] : d[j];
            }
        };
        // product of two canonical elements, canonical: (a R^2 / R) b / R
        Fr host_mul_canonical(const Fr& a, const Fr& b)
        {
            static const HostFr64 f;
            uint64_t x[4], y[4], ar[4], out[4];
            std::memcpy(x, a.l, 32);
            std::memcpy(y, b.l, 32);
            f.mul(x, f.r2, ar);
            f.mul(ar, y, out);
            Fr r;
            std::memcpy(r.l, out, 32);
            return r;
        }
    }

    // Host-side scalar arithmetic for the O(#columns) glue of a caller (same limb code as the
    // kernels, run on the CPU): op 0 add, 1 sub, 2 mul, 3 inverse of a (b ignored).
    int gzk_fr_op(int op, const uint8_t a[32], const uint8_t b[32], uint8_t out[32])
    {
        if (a == nullptr || out == nullptr || (op != 3 && b == nullptr)) return GZK_E_INVALID;
        bool ok_a = false, ok_b = true;
        const Fr x = host_fr_from_bytes(a, &ok_a);
        Fr y = Fr::zero();
        if (op != 3) y = host_fr_from_bytes(b, &ok_b);
        if (!ok_a || !ok_b) return GZK_E_INVALID;
        Fr r;
        switch (op)
        {
        case 0: r = add(x, y); break;
        case 1: r = sub(x, y); break;
        case 2: r = host_mul_canonical(x, y); break;
        case 3:
            if (x.is_zero()) return GZK_E_DOMAIN;  // FieldElement::inv throws on zero
            r = from_mont(inv(to_mont(x)));
            break;
        default: return GZK_E_INVALID;
        }
        host_fr_to_bytes(r, out);
        return GZK_OK;
    }
}
