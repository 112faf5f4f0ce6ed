// Internal declarations shared by the translation units of libgatzk_b200.so:
// the context and buffer objects behind the opaque C handles, error plumbing and
// the global-memory access helpers for 32-byte field elements.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/gatzk_b200.h"
#include "field.cuh"

struct gzk_buf
{
    void* dptr = nullptr;
    size_t count = 0;
    int kind = GZK_KIND_FR;
    size_t elem_bytes = 32;
    bool owned = true;  // false: dptr belongs to the caller (gzk_buf_wrap)
};

namespace gzk
{
    // omega powers of one domain as two small tables: omega^i = hi[i >> LO] * lo[i & mask].
    struct DomainTables
    {
        unsigned log2n = 0;
        unsigned lo_bits = 0;
        Fr* lo = nullptr;       // omega^j, j < 2^lo_bits (Montgomery)
        Fr* hi = nullptr;       // omega^(j << lo_bits), j < 2^(log2n - lo_bits)
        Fr* lo_inv = nullptr;   // omega^-j
        Fr* hi_inv = nullptr;   // omega^-(j << lo_bits)
        Fr omega;               // Montgomery
        Fr inv_size;            // 1/n, Montgomery
    };

    // Grow-only device scratch owned by the context (reused across calls, never
    // shrinks; freed with the context).
    struct Scratch
    {
        void* ptr = nullptr;
        size_t bytes = 0;
    };
}

namespace gzk
{
    // CUDA-event timing of kernel families, switched on by gzk_timing_enable.
    struct TimedLaunch
    {
        int family;
        cudaEvent_t start, stop;
    };
    struct FamilyStat
    {
        std::string name;
        uint64_t launches = 0;
        double total_ms = 0.0;
    };
}

namespace gzk
{
    // Load-time factors of one transform pass (first stage s0, `stages` stages), cached per context.
    struct NttTwistTable
    {
        unsigned s0 = 0, stages = 0;
        bool inverse = false;
        Fr* table = nullptr;
    };
}

struct gzk_ctx
{
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;  // host-to-device uploads that overlap with kernels
    cudaEvent_t copy_event = nullptr;
    cudaEvent_t order_event = nullptr;   // recorded on this stream for another context to wait on (gzk_ctx_wait_for)
    std::string last_error;
    std::unordered_map<unsigned, gzk::DomainTables> domains;
    gzk::Fr* ntt_small[2] = {nullptr, nullptr};  // omega_1024^m and omega_1024^-m, m < 512
    std::vector<gzk::NttTwistTable> ntt_twists;
    gzk::Scratch scratch[4];
    void* pinned = nullptr;  // small pinned staging area for results
    size_t pinned_bytes = 0;
    int* d_status = nullptr;  // device-side status word (zero-denominator flags etc.)
    // pinned ring for the small uploads of deferred mode: the data is copied into a slot and the
    // call returns without waiting; a slot is reused once the copy that read it has completed
    static constexpr int kUploadSlots = 16;
    static constexpr size_t kUploadSlotBytes = 256u << 10;
    char* upload_ring = nullptr;
    cudaEvent_t upload_done[kUploadSlots] = {};
    bool upload_busy[kUploadSlots] = {};
    int upload_next = 0;
    bool timing = false;
    bool deferred = false;  // builder calls return without synchronising; errors surface at gzk_ctx_synchronize
    std::vector<gzk::FamilyStat> families;
    std::vector<gzk::TimedLaunch> pending;
    std::vector<cudaEvent_t> event_pool;
    // work counters of the packed-evaluation launches since the last gzk_timing_reset
    uint64_t eval_algorithmic_bytes = 0;  // column values once per launch + the weights once per rotation
    uint64_t eval_limb_products = 0;      // 32x32-bit products of the inner loops
    uint64_t eval_terms = 0;              // (row, column, rotation) terms
};

namespace gzk
{
    int fail(gzk_ctx* ctx, int code, const std::string& message);
    int cuda_fail(gzk_ctx* ctx, cudaError_t err, const char* what);
    int ensure_scratch(gzk_ctx* ctx, int slot, size_t bytes, void** out);
    int ensure_pinned(gzk_ctx* ctx, size_t bytes, void** out);
    int get_domain(gzk_ctx* ctx, unsigned log2n, const DomainTables** out);

    // Brackets the kernel launches issued during its lifetime with CUDA events on
    // the context stream when timing is on; every launch site uses one, so the
    // per-family launch counts are maintained even when timing is off.
    class LaunchScope
    {
    public:
        LaunchScope(gzk_ctx* ctx, const char* family, unsigned launches = 1);
        ~LaunchScope();
        LaunchScope(const LaunchScope&) = delete;
        LaunchScope& operator=(const LaunchScope&) = delete;

    private:
        gzk_ctx* ctx_;
        int family_;
        cudaEvent_t start_ = nullptr;
    };
    void timing_collect(gzk_ctx* ctx);

    // End of a call whose results stay on the device: in the default mode synchronise the
    // stream and turn a raised status word into an error; in deferred mode return at once
    // (the status word stays raised until gzk_ctx_synchronize reports it).
    int finish_call(gzk_ctx* ctx, const char* invalid_message);
    // Clears the status word at the start of a call (not in deferred mode, where it is sticky).
    int begin_call(gzk_ctx* ctx);

    // Host-side scalar helpers (same arithmetic, emulated carry flag).
    Fr host_fr_from_bytes(const uint8_t* bytes, bool* canonical_ok);
    void host_fr_to_bytes(const Fr& canonical, uint8_t* bytes);
    Fr host_root_of_unity(unsigned log2n);  // Montgomery form

#define GZK_CUDA_TRY(ctx, expr)                                         \
    do                                                                  \
    {                                                                   \
        cudaError_t gzk_err_ = (expr);                                  \
        if (gzk_err_ != cudaSuccess) return gzk::cuda_fail(ctx, gzk_err_, #expr); \
    } while (0)

#if defined(__CUDACC__)
    // 32-byte element access as two 128-bit transactions.
    // Raises the context's status word from a kernel.  The word after it records where: a number that is
    // unique per raising site (file index * 100 + running number), reported with the error message.
    __device__ __forceinline__ void raise_status(int* status, int code, int site)
    {
        atomicExch(status, code);
        status[1] = site;
    }

    __device__ __forceinline__ Fr load_fr(const Fr* p)
    {
        const uint4* q = reinterpret_cast<const uint4*>(p);
        const uint4 a = __ldg(q);
        const uint4 b = __ldg(q + 1);
        Fr o;
        o.l[0] = a.x; o.l[1] = a.y; o.l[2] = a.z; o.l[3] = a.w;
        o.l[4] = b.x; o.l[5] = b.y; o.l[6] = b.z; o.l[7] = b.w;
        return o;
    }
    __device__ __forceinline__ Fr load_fr_plain(const Fr* p)
    {
        const uint4* q = reinterpret_cast<const uint4*>(p);
        const uint4 a = q[0];
        const uint4 b = q[1];
        Fr o;
        o.l[0] = a.x; o.l[1] = a.y; o.l[2] = a.z; o.l[3] = a.w;
        o.l[4] = b.x; o.l[5] = b.y; o.l[6] = b.z; o.l[7] = b.w;
        return o;
    }
    __device__ __forceinline__ void store_fr(Fr* p, const Fr& v)
    {
        uint4* q = reinterpret_cast<uint4*>(p);
        q[0] = make_uint4(v.l[0], v.l[1], v.l[2], v.l[3]);
        q[1] = make_uint4(v.l[4], v.l[5], v.l[6], v.l[7]);
    }
    // omega^i from the two-level tables.
    __device__ __forceinline__ Fr domain_point(const Fr* lo, const Fr* hi, unsigned lo_bits, uint64_t i)
    {
        const Fr a = load_fr(hi + (i >> lo_bits));
        const uint64_t j = i & ((1ULL << lo_bits) - 1ULL);
        if (j == 0) return a;
        return mul(a, load_fr(lo + j));
    }
#endif
}
