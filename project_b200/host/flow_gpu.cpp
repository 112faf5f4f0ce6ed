// libgatzk_b200_flow.so: the prover flow (prover_flow.hpp) over the C ABI of libgatzk_b200.so.
// Every Backend method is one gzk_* call; columns are gzk_buf handles that live on the GPU from
// the forward pass to the last opening.  The context runs in deferred mode: builder calls only
// queue kernels, the host reads values back once per commit barrier.
#include <algorithm>
#include <atomic>
#include <cstring>

#include "../../include/gatzk_b200.h"
#include "flow_c_impl.hpp"

namespace
{
    using namespace gatzk_flow;

    class GpuBackend;
    struct GpuCol : Col
    {
        GpuBackend* owner = nullptr;
        gzk_buf* buf = nullptr;
        ~GpuCol() override;
    };

    // test hook: fill every buffer handed out by alloc() with a byte pattern, so that a column builder that
    // reads a row nobody wrote shows up as a wrong proof instead of depending on what the memory held before
    std::atomic<int> g_poison_allocations{0};

    class GpuBackend : public Backend
    {
    public:
        explicit GpuBackend(int device) : device_(device)
        {
            if (gzk_ctx_create(device, &ctx_) != GZK_OK) throw std::runtime_error("b200 backend: no usable sm_100 GPU (there is no CPU fallback)");
            check(gzk_ctx_set_deferred(ctx_, 1));
        }
        ~GpuBackend() override
        {
            for (gzk_ctx* side : side_) gzk_ctx_synchronize(side);
            for (auto& slot : pool_)
                for (gzk_buf* b : slot.second) gzk_buf_free(ctx_, b);
            for (gzk_ctx* side : side_) gzk_ctx_destroy(side);
            gzk_ctx_destroy(ctx_);
        }
        gzk_ctx* context() const { return ctx_; }
        gzk_ctx* side_context(std::size_t i) const { return i < side_.size() ? side_[i] : nullptr; }
        // Buffers go back to a free list keyed by (kind, count) instead of to cudaFree: every proof
        // allocates the same set of columns, so from the second proof on nothing is allocated, and a
        // recycled buffer is safe to reuse at once because all work is ordered on the one stream.
        void recycle(int kind, std::size_t count, gzk_buf* buf) { pool_[{kind, count}].push_back(buf); }

        Fe fr_op(int op, const Fe& a, const Fe& b) override
        {
            Fe out{};
            if (gzk_fr_op(op, a.data(), b.data(), out.data()) != GZK_OK) throw std::runtime_error("field operation on a non-canonical or zero operand");
            return out;
        }
        Fe root_of_unity(std::uint64_t size) override
        {
            Fe out{};
            check(gzk_root_of_unity(ctx_, size, out.data()));
            return out;
        }
        ColP alloc(int kind, std::size_t count) override
        {
            auto c = std::make_shared<GpuCol>();
            c->owner = this;
            c->kind = kind;
            c->count = count;
            auto& free_list = pool_[{kind, count}];
            if (!free_list.empty())
            {
                c->buf = free_list.back();
                free_list.pop_back();
            }
            else
            {
                check(gzk_buf_alloc(ctx_, kind, count, &c->buf));
            }
            if (g_poison_allocations.load() != 0 && count != 0)
            {
                // canonical field elements for the field kinds (an upload checks nothing but converts them), 0xA5 bytes otherwise
                const std::size_t bytes = count * element_bytes(kind);
                std::vector<std::uint8_t> pattern(bytes, 0xA5);
                if (kind == kFr || kind == kFrMont || kind == kG1)
                    for (std::size_t i = 31; i < bytes; i += 32) pattern[i] = 0x05;
                check(gzk_buf_upload(ctx_, c->buf, 0, pattern.data(), count));
            }
            return c;
        }
        void upload(const ColP& col, const void* host, std::size_t count) override
        {
            check(gzk_buf_upload(ctx_, raw(col), 0, host, count));
            uploaded_bytes += count * element_bytes(col->kind);
        }
        void download(const ColP& col, std::size_t offset, std::size_t count, void* host) override
        {
            check(gzk_buf_download(ctx_, raw(col), offset, host, count));
            downloaded_bytes += count * element_bytes(col->kind);
        }
        void zero(const ColP& col) override { check(gzk_buf_zero(ctx_, raw(col))); }
        void copy_block(const ColP& src, std::size_t so, std::size_t ss, const ColP& dst, std::size_t d_o, std::size_t ds, std::size_t rows,
                        std::size_t width) override
        {
            check(gzk_copy_block(ctx_, raw(src), so, ss, raw(dst), d_o, ds, rows, width));
        }
        void head_forward(const HeadDesc& h, const GraphCols& g, const HeadTraceCols& o) override
        {
            gzk_gat_head head{};
            head.features = raw(h.features);
            head.input_width = static_cast<std::uint32_t>(h.input_width);
            head.output_width = static_cast<std::uint32_t>(h.output_width);
            head.seq_kernel = raw(h.seq_kernel);
            head.attn_src_kernel = raw(h.attn_src);
            head.attn_dst_kernel = raw(h.attn_dst);
            head.attn_src_bias = h.attn_src_bias;
            head.attn_dst_bias = h.attn_dst_bias;
            head.output_bias = h.output_bias ? raw(h.output_bias) : nullptr;
            head.output_bias_count = h.output_bias ? h.output_bias->count : 0;
            head.apply_activation = h.apply_activation ? 1 : 0;
            gzk_gat_graph graph{};
            graph.node_count = g.node_count;
            graph.edge_count = g.edge_count;
            graph.edge_src = raw(g.edge_src);
            graph.edge_dst = raw(g.edge_dst);
            graph.incoming_count = g.incoming_count;
            graph.incoming_ptr = raw(g.incoming_ptr);
            graph.incoming_src = raw(g.incoming_src);
            gzk_gat_trace tr{};
            tr.H_prime = raw(o.H_prime);
            tr.E_src = raw(o.E_src);
            tr.E_dst = raw(o.E_dst);
            tr.M = raw(o.M);
            tr.Sum = raw(o.Sum);
            tr.inv = raw(o.inv);
            tr.S = raw(o.S);
            tr.Z = raw(o.Z);
            tr.Delta = raw(o.Delta);
            tr.U = raw(o.U);
            tr.alpha = raw(o.alpha);
            tr.H_agg_pre_bias = raw(o.H_agg_pre_bias);
            tr.H_agg = raw(o.H_agg);
            check(gzk_gat_head_forward(ctx_, &head, &graph, &tr));
        }
        void quantize(const ColP& v, std::size_t count, const ColP& out) override { check(gzk_quantize(ctx_, raw(v), count, raw(out))); }
        void quantize_guarded(const ColP& v, std::size_t count, double guard, const ColP& out, const ColP& flagged) override
        {
            check(gzk_quantize_guarded(ctx_, raw(v), count, guard, raw(out), raw(flagged)));
        }
        void gather(const ColP& nv, std::size_t node_count, const ColP& index, std::size_t edge_count, std::size_t domain_size, const ColP& out) override
        {
            check(gzk_broadcast_node_values(ctx_, raw(nv), node_count, raw(index), edge_count, domain_size, raw(out)));
        }
        void linear_combination(const std::vector<ColP>& cols, const std::vector<Fe>& coefficients, std::size_t count, std::size_t domain_size,
                                const ColP& out) override
        {
            std::vector<const gzk_buf*> bufs;
            std::vector<std::uint8_t> coeff(cols.size() * 32);
            for (std::size_t j = 0; j < cols.size(); ++j)
            {
                bufs.push_back(raw(cols[j]));
                std::memcpy(&coeff[32 * j], coefficients[j].data(), 32);
            }
            check(gzk_linear_combination(ctx_, bufs.data(), coeff.data(), cols.size(), count, domain_size, raw(out)));
        }
        void mul_columns(const ColP& l, const ColP& r, std::size_t count, std::size_t domain_size, const ColP& out) override
        {
            check(gzk_mul_columns(ctx_, raw(l), raw(r), count, domain_size, raw(out)));
        }
        void linear_form_rows(const ColP& m, std::size_t rows, std::size_t cols, const ColP& powers, const ColP& out) override
        {
            check(gzk_linear_form_rows(ctx_, raw(m), rows, cols, raw(powers), raw(out)));
        }
        void powers(const Fe& c, std::size_t count, const ColP& out) override { check(gzk_powers(ctx_, c.data(), count, raw(out))); }
        void lookup_multiplicity(const ColP& x, const ColP& y, std::size_t count, std::int64_t x_min, std::size_t band, const ColP& table_y,
                                 std::size_t table_size, std::size_t domain_size, const ColP& out) override
        {
            check(gzk_banded_lookup_multiplicity(ctx_, raw(x), y ? raw(y) : nullptr, count, x_min, band, table_y ? raw(table_y) : nullptr, table_size,
                                                 domain_size, raw(out)));
        }
        void first_zero_marker(const ColP& delta, const ColP& gb, const ColP& ge, std::size_t groups, std::size_t domain_size, const ColP& out) override
        {
            check(gzk_first_zero_marker(ctx_, raw(delta), raw(gb), raw(ge), groups, domain_size, raw(out)));
        }
        void logup(const ColP& table, const ColP& query, const ColP& m, const ColP& qt, const ColP& qq, std::size_t n, const Fe& beta,
                   std::size_t active, const ColP& out) override
        {
            check(gzk_logup_accumulator(ctx_, raw(table), raw(query), raw(m), raw(qt), raw(qq), n, beta.data(), active, raw(out)));
        }
        void route_node(const ColP& table, const ColP& m, std::size_t valid, std::size_t domain_size, const Fe& beta, const ColP& out) override
        {
            check(gzk_route_node_accumulator(ctx_, raw(table), raw(m), valid, domain_size, beta.data(), raw(out)));
        }
        void route_edge(const ColP& query, std::size_t valid, std::size_t domain_size, const Fe& beta, const ColP& out) override
        {
            check(gzk_route_edge_accumulator(ctx_, raw(query), valid, domain_size, beta.data(), raw(out)));
        }
        void group_prefix_state(const ColP& values, const ColP& q_new, std::size_t n, const ColP& out) override
        {
            check(gzk_group_prefix_state(ctx_, raw(values), raw(q_new), n, raw(out)));
        }
        void zkmap(const ColP& a, const ColP& b, std::size_t count, std::size_t domain_size, const ColP& out) override
        {
            check(gzk_zkmap_accumulator(ctx_, raw(a), raw(b), count, domain_size, raw(out), nullptr));
        }
        void running_sums_batch(const std::vector<ScanJob>& jobs) override
        {
            // the batched entry point takes jobs of at most 2^20 rows; longer columns (the edge domain of the
            // large configurations) fill the machine by themselves and go through the single-column calls
            constexpr std::uint64_t kBatchRows = 1ull << 20;
            std::vector<ScanJob> small_jobs, long_jobs;
            for (const ScanJob& j : jobs)
                ((j.op == ScanJob::kGroupPrefix ? j.domain_size : j.count) > kBatchRows ? long_jobs : small_jobs).push_back(j);
            // The indexed accumulators are chains of a few kernels each, two of them short and serial (the inversion
            // of the table, the scan of the block sums).  The jobs of one barrier are independent, so they are dealt
            // over this context and two side contexts (one stream each): the short kernels of one job then run beside
            // the long ones of another.  The side streams start after everything queued here so far and this stream
            // resumes after them.
            std::vector<const ScanJob*> indexed;
            for (auto it = long_jobs.begin(); it != long_jobs.end(); ++it)
            {
                const bool logup = it->op == ScanJob::kLogup && it->key_x != nullptr && it->table_size != 0 && it->table_size <= it->count;
                const bool route = it->op == ScanJob::kRouteEdge && it->key_x != nullptr && it->table_y != nullptr && it->table_size != 0;
                if (logup || route) indexed.push_back(&*it);
            }
            if (indexed.size() > 1 && side_.empty())
            {
                for (int i = 0; i < 2; ++i)
                {
                    gzk_ctx* side = nullptr;
                    if (gzk_ctx_create(device_, &side) != GZK_OK) throw std::runtime_error("b200 backend: cannot create a side context");
                    side_.push_back(side);
                    check_on(side, gzk_ctx_set_deferred(side, 1));
                }
            }
            const bool spread = indexed.size() > 1;
            if (spread)
                for (gzk_ctx* side : side_) check_on(side, gzk_ctx_wait_for(side, ctx_));
            for (std::size_t i = 0; i < indexed.size(); ++i)
            {
                const ScanJob* it = indexed[i];
                gzk_ctx* on = spread && i % (side_.size() + 1) != 0 ? side_[i % (side_.size() + 1) - 1] : ctx_;
                // a long lookup accumulator: inverses fetched from the table (one inversion per table row, not per query)
                if (it->op == ScanJob::kLogup)
                    check_on(on, gzk_logup_accumulator_indexed(on, raw(it->c0), raw(it->c2), raw(it->key_x), it->key_y ? raw(it->key_y) : nullptr, it->count,
                                                               it->x_min, it->band, it->table_y ? raw(it->table_y) : nullptr, it->table_size,
                                                               it->domain_size, it->beta.data(), raw(it->out)));
                else
                    check_on(on, gzk_route_edge_accumulator_indexed(on, raw(it->table_y), it->table_size, raw(it->key_x), it->count, it->domain_size,
                                                                    it->beta.data(), raw(it->out)));
            }
            if (spread)
                for (gzk_ctx* side : side_) check(gzk_ctx_wait_for(ctx_, side));
            {
                std::vector<ScanJob> rest;
                for (const ScanJob& j : long_jobs)
                    if (std::find(indexed.begin(), indexed.end(), &j) == indexed.end()) rest.push_back(j);
                long_jobs.swap(rest);
            }
            if (!long_jobs.empty()) Backend::running_sums_batch(long_jobs);
            if (small_jobs.empty()) return;
            std::vector<gzk_scan_job> raw_jobs(small_jobs.size());
            for (std::size_t i = 0; i < small_jobs.size(); ++i)
            {
                const ScanJob& j = small_jobs[i];
                gzk_scan_job& r = raw_jobs[i];
                r.op = j.op;  // the numbering of ScanJob::Op is that of GZK_SCAN_*
                r.c0 = j.c0 ? raw(j.c0) : nullptr;
                r.c1 = j.c1 ? raw(j.c1) : nullptr;
                r.c2 = j.c2 ? raw(j.c2) : nullptr;
                r.c3 = j.c3 ? raw(j.c3) : nullptr;
                r.c4 = j.c4 ? raw(j.c4) : nullptr;
                r.count = j.count;
                r.domain_size = j.domain_size;
                r.beta = j.op <= ScanJob::kRouteEdge ? j.beta.data() : nullptr;
                r.out = raw(j.out);
            }
            check(gzk_running_sums_batch(ctx_, raw_jobs.data(), raw_jobs.size()));
        }
        void bary_weights(unsigned log2n, const Fe& x, const ColP& out) override { check(gzk_bary_weights(ctx_, log2n, x.data(), raw(out))); }
        void bary_weights_multi(unsigned log2n, const std::vector<Fe>& xs, const std::vector<ColP>& outs) override
        {
            std::vector<std::uint8_t> points(32 * xs.size());
            std::vector<gzk_buf*> bufs;
            for (std::size_t i = 0; i < xs.size(); ++i)
            {
                std::memcpy(points.data() + 32 * i, xs[i].data(), 32);
                bufs.push_back(raw(outs[i]));
            }
            check(gzk_bary_weights_multi(ctx_, log2n, points.data(), xs.size(), bufs.data()));
        }
        void bary_weights_prefix(unsigned log2n, const Fe& x, std::size_t keep, const ColP& out) override
        {
            check(gzk_bary_weights_prefix(ctx_, log2n, x.data(), keep, raw(out)));
        }
        void fold_rows(const ColP& m, std::size_t rows, std::size_t cols, const ColP& weights, std::size_t row_count, const ColP& out) override
        {
            check(gzk_fold_rows(ctx_, raw(m), rows, cols, raw(weights), row_count, raw(out)));
        }
        void eval_device(const std::vector<ColP>& cols, std::size_t len, unsigned log2n, const ColP& weights, const std::vector<std::uint64_t>& rotations,
                         const ColP& out, std::size_t out_offset) override
        {
            std::vector<gzk_buf*> bufs;
            for (const auto& c : cols) bufs.push_back(raw(c));
            check(gzk_eval_batch_device(ctx_, bufs.data(), bufs.size(), len, log2n, raw(weights), rotations.data(), rotations.size(), raw(out), out_offset));
        }
        void horner_device(const ColP& m, std::size_t rows, std::size_t cols, const Fe& x, const ColP& out, std::size_t out_offset) override
        {
            check(gzk_matrix_horner_device(ctx_, raw(m), rows, cols, x.data(), raw(out), out_offset));
        }
        void g1_fixed_base(const G1& base, const ColP& scalars, std::size_t count, const ColP& out_points) override
        {
            check(gzk_g1_fixed_base_mul(ctx_, base.data(), raw(scalars), count, raw(out_points)));
        }
        void fh_public_eval(const ColP& features, std::size_t rows, std::size_t fc, const ColP& abs_ids, const ColP& weights, unsigned log2n,
                            std::uint64_t rotation, Fe out[5]) override
        {
            std::uint8_t bytes[5 * 32];
            check(gzk_fh_public_eval_rotated(ctx_, raw(features), rows, fc, abs_ids ? raw(abs_ids) : nullptr, raw(weights), log2n, rotation, bytes));
            for (int i = 0; i < 5; ++i) std::memcpy(out[i].data(), bytes + 32 * i, 32);
        }
        void synchronize() override
        {
            check(gzk_ctx_synchronize(ctx_));
            for (gzk_ctx* side : side_) check_on(side, gzk_ctx_synchronize(side));  // their deferred errors
        }
        void transform(std::vector<Fe>& data, bool inverse) override
        {
            unsigned log2n = 0;
            while ((std::size_t{1} << log2n) < data.size()) ++log2n;
            if (data.empty() || (std::size_t{1} << log2n) != data.size()) throw std::runtime_error("transform: the length must be a power of two");
            const ColP in = alloc(kFr, data.size()), out = alloc(kFrMont, data.size());
            upload(in, data.data(), data.size());
            check(gzk_ntt(ctx_, raw(in), raw(out), log2n, 1, inverse ? 1 : 0, nullptr));
            download(out, 0, data.size(), data.data());
        }
        bool supports_msm() const override { return true; }
        bool supports_indexed_logup() const override { return true; }
        ColP srs_lagrange(unsigned log2n, const G1& base, const Fe& tau) override
        {
            const ColP out = alloc(kG1, static_cast<std::size_t>(1) << log2n);
            check(gzk_srs_lagrange(ctx_, log2n, base.data(), tau.data(), raw(out)));
            return out;
        }
        ColP msm_table(const ColP& points, std::size_t n, unsigned* window_bits) override
        {
            *window_bits = gzk_msm_window_bits(n);
            const ColP table = alloc(kG1, gzk_msm_table_points(n, *window_bits));
            check(gzk_msm_precompute(ctx_, raw(points), n, *window_bits, raw(table)));
            return table;
        }
        G1 msm(const ColP& scalars, const ColP& table, std::size_t n, unsigned window_bits) override
        {
            G1 out{};
            check(gzk_msm_precomputed(ctx_, raw(scalars), raw(table), n, window_bits, out.data()));
            return out;
        }

    private:
        static std::size_t element_bytes(int kind) { return kind == kU32 ? 4 : (kind == kI64 || kind == kF64) ? 8 : kind == kG1 ? 96 : 32; }
        static gzk_buf* raw(const ColP& c)
        {
            if (c == nullptr) throw std::runtime_error("flow: missing column");
            return static_cast<GpuCol*>(c.get())->buf;
        }
        void check(int rc) const
        {
            if (rc != GZK_OK) throw std::runtime_error(gzk_last_error(ctx_));
        }
        void check_on(gzk_ctx* ctx, int rc) const
        {
            if (rc != GZK_OK) throw std::runtime_error(gzk_last_error(ctx));
        }
        int device_ = 0;
        gzk_ctx* ctx_ = nullptr;
        std::vector<gzk_ctx*> side_;  // further contexts (streams) of the same GPU for independent chains of short calls
        std::map<std::pair<int, std::size_t>, std::vector<gzk_buf*>> pool_;
    };

    GpuCol::~GpuCol()
    {
        if (buf != nullptr) owner->recycle(kind, count, buf);
    }
}

struct gzk_flow : gatzk_flow::FlowHandle
{
};

extern "C"
{
    const char* gzk_flow_error(void) { return gatzk_flow::flow_error_slot().c_str(); }
    int gzk_flow_create(int device, const gzk_flow_config* config, gzk_flow** out)
    {
        gatzk_flow::FlowHandle* handle = nullptr;
        std::unique_ptr<gatzk_flow::Backend> backend;
        const int rc0 = gatzk_flow::flow_guard([&] { backend = std::make_unique<GpuBackend>(device); });
        if (rc0 != 0) return rc0;
        const int rc = gatzk_flow::flow_create_impl(std::move(backend), config, &handle);
        if (rc != 0) return rc;
        // the per-proof upload of the feature matrix comes from this copy: page-lock it (best effort)
        const auto& features = handle->flow->inputs().features;
        if (!features.empty()) gzk_host_register(const_cast<double*>(features.data()), features.size() * sizeof(double));
        *out = static_cast<gzk_flow*>(handle);
        return rc;
    }
    void gzk_flow_destroy(gzk_flow* flow)
    {
        if (flow == nullptr) return;
        if (flow->flow != nullptr && !flow->flow->inputs().features.empty())
            gzk_host_unregister(const_cast<double*>(flow->flow->inputs().features.data()));
        flow->flow.reset();  // columns go before the context
        delete static_cast<gatzk_flow::FlowHandle*>(flow);
    }
    int gzk_flow_prove(gzk_flow* flow) { return gatzk_flow::flow_prove_impl(flow, false); }
    int gzk_flow_prove_resident(gzk_flow* flow) { return gatzk_flow::flow_prove_impl(flow, true); }
    int gzk_flow_set_msm_commit(gzk_flow* flow, int on, uint64_t counts[2])
    {
        if (flow == nullptr) return 1;
        flow->flow->set_msm_commit(on != 0);
        if (counts != nullptr)
        {
            counts[0] = flow->flow->msm_commitments();
            counts[1] = flow->flow->msm_mismatches();
        }
        return 0;
    }
    size_t gzk_flow_dump(gzk_flow* flow, char* out, size_t cap) { return gatzk_flow::flow_dump_impl(flow, out, cap); }
    size_t gzk_flow_proof_bytes(gzk_flow* flow, uint8_t* out, size_t cap) { return gatzk_flow::flow_proof_bytes_impl(flow, out, cap); }
    int gzk_flow_stats(gzk_flow* flow, uint64_t out[14]) { return gatzk_flow::flow_stats_impl(flow, out); }
    int gzk_flow_column(gzk_flow* flow, const char* label, int* kind, uint64_t* length, void* out, size_t cap_elements)
    {
        return gatzk_flow::flow_column_impl(flow, label, kind, length, out, cap_elements);
    }
    int gzk_flow_constraint_violations(gzk_flow* flow, uint64_t out[7], uint64_t* failures, size_t cap, size_t* count)
    {
        return gatzk_flow::flow_constraint_violations_impl(flow, out, failures, cap, count);
    }
    int gzk_flow_honest_quotient(gzk_flow* flow, const char* domain, unsigned log2_blowup, unsigned classes, uint64_t out[6])
    {
        return gatzk_flow::flow_honest_quotient_impl(flow, domain, log2_blowup, classes, out);
    }
    size_t gzk_flow_domain_labels(gzk_flow* flow, const char* domain, char* out, size_t cap)
    {
        return gatzk_flow::flow_domain_labels_impl(flow, domain, out, cap);
    }
    void gzk_flow_debug_poison_allocations(int on) { g_poison_allocations.store(on); }
    void* gzk_flow_context(gzk_flow* flow) { return flow == nullptr ? nullptr : static_cast<GpuBackend*>(flow->backend.get())->context(); }
    void* gzk_flow_side_context(gzk_flow* flow, size_t index)
    {
        return flow == nullptr ? nullptr : static_cast<GpuBackend*>(flow->backend.get())->side_context(index);
    }
}
