// TEST INFRASTRUCTURE — the prover flow (project_b200/host/prover_flow.hpp) over a CPU backend
// built from this oracle's field and curve arithmetic.  Used only by tests (field-by-field
// comparison with the GPU run) and by the CPU-baseline / reference arm of bench.py; the product
// never links it.  "Parity unpinned" applies as stated in field.hpp.
//
// Columns are host vectors of native field elements, as the reference keeps its columns
// (std::vector<FieldElement> over mcl::Fr).  Every method restates the reference leaf it stands
// for, with the reference's loop structure and thread fan-out (std::async chunks over
// hardware_concurrency, src/algebra/eval_backend.cpp:340-390, src/algebra/polynomial.cpp:179-315;
// the column builders are serial per column, src/protocol/lookup.cpp:100-157).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../project_b200/host/flow_c_impl.hpp"
#include "field.hpp"
#include "g1.hpp"

extern "C" int ora_gat_head_forward(const double* features, std::size_t nodes, std::size_t inner, const double* seq_kernel, std::size_t width,
                                    const double* attn_src, double bias_src, const double* attn_dst, double bias_dst, const double* out_bias,
                                    std::size_t out_bias_count, int has_bias, int apply_activation, const std::uint32_t* edge_src,
                                    const std::uint32_t* edge_dst, std::size_t edges, double* H_prime, double* E_src, double* E_dst, double* S,
                                    double* Z, double* M, double* Delta, double* U, double* Sum, double* inv, double* alpha, double* H_agg_pre,
                                    double* H_agg);
extern "C" const char* ora_last_error();
extern "C" int ora_ntt(std::uint8_t* data, std::uint64_t size, int inverse, const std::uint8_t* coset_shift);

namespace
{
    using namespace gatzk_flow;
    using oracle::Fr;

    struct CpuCol : Col
    {
        std::vector<Fr> fr;            // kFr / kFrMont (both native here)
        std::vector<std::int64_t> i64;
        std::vector<std::uint32_t> u32;
        std::vector<double> f64;
        std::vector<std::array<std::uint8_t, 96>> g1;
        std::vector<Fr> widened;       // small-integer column as field elements (FieldElement::from_signed), made on first use
    };

    Fr fe_in(const Fe& a) { return Fr::from_le_bytes(a.data()); }
    Fe fe_out(const Fr& a)
    {
        Fe o;
        a.to_le_bytes(o.data());
        return o;
    }

    void parallel_chunks(std::size_t n, std::size_t threads, const std::function<void(std::size_t, std::size_t, std::size_t)>& body)
    {
        threads = std::max<std::size_t>(1, std::min(threads, n == 0 ? 1 : n));
        if (threads == 1)
        {
            body(0, 0, n);
            return;
        }
        const std::size_t chunk = (n + threads - 1) / threads;
        std::vector<std::thread> pool;
        for (std::size_t t = 0; t < threads; ++t)
        {
            const std::size_t begin = t * chunk, end = std::min(n, begin + chunk);
            if (begin >= end) break;
            pool.emplace_back(body, t, begin, end);
        }
        for (auto& th : pool) th.join();
    }

    // include/gatzk/algebra/field.hpp:221-253
    void batch_invert_in_place(std::vector<Fr>& values)
    {
        if (values.empty()) return;
        std::vector<Fr> prefixes(values.size());
        Fr acc = Fr::one();
        for (std::size_t i = 0; i < values.size(); ++i)
        {
            if (values[i].is_zero()) throw std::runtime_error("batch_invert encountered zero");
            prefixes[i] = acc;
            acc = acc * values[i];
        }
        Fr suffix_inverse = acc.inv();
        for (std::size_t i = values.size(); i-- > 0;)
        {
            const Fr v = values[i];
            values[i] = suffix_inverse * prefixes[i];
            suffix_inverse = suffix_inverse * v;
        }
    }

    class CpuBackend : public Backend
    {
    public:
        explicit CpuBackend(std::size_t threads) : threads_(std::max<std::size_t>(1, threads)) {}

        Fe fr_op(int op, const Fe& a, const Fe& b) override
        {
            const Fr x = fe_in(a);
            switch (op)
            {
            case 0: return fe_out(x + fe_in(b));
            case 1: return fe_out(x - fe_in(b));
            case 2: return fe_out(x * fe_in(b));
            case 3:
                if (x.is_zero()) throw std::runtime_error("attempted to invert zero in FieldElement");
                return fe_out(x.inv());
            default: throw std::runtime_error("unknown field operation");
            }
        }
        Fe root_of_unity(std::uint64_t size) override { return fe_out(oracle::root_of_unity(size)); }

        ColP alloc(int kind, std::size_t count) override
        {
            auto c = std::make_shared<CpuCol>();
            c->kind = kind;
            c->count = count;
            switch (kind)
            {
            case kFr:
            case kFrMont: c->fr.assign(count, Fr::zero()); break;
            case kI64: c->i64.assign(count, 0); break;
            case kU32: c->u32.assign(count, 0); break;
            case kF64: c->f64.assign(count, 0.0); break;
            case kG1: c->g1.assign(count, {}); break;
            default: throw std::runtime_error("unknown buffer kind");
            }
            return c;
        }
        void upload(const ColP& col, const void* host, std::size_t count) override
        {
            CpuCol& c = cpu(col);
            c.widened.clear();
            const auto* bytes = static_cast<const std::uint8_t*>(host);
            switch (c.kind)
            {
            case kFr:
            case kFrMont:
                for (std::size_t i = 0; i < count; ++i) c.fr[i] = Fr::from_le_bytes(bytes + 32 * i);
                break;
            case kI64: std::memcpy(c.i64.data(), host, count * 8); break;
            case kU32: std::memcpy(c.u32.data(), host, count * 4); break;
            case kF64: std::memcpy(c.f64.data(), host, count * 8); break;
            case kG1: std::memcpy(c.g1.data(), host, count * 96); break;
            }
        }
        void download(const ColP& col, std::size_t offset, std::size_t count, void* host) override
        {
            const CpuCol& c = cpu(col);
            auto* bytes = static_cast<std::uint8_t*>(host);
            switch (c.kind)
            {
            case kFr:
            case kFrMont:
                for (std::size_t i = 0; i < count; ++i) c.fr[offset + i].to_le_bytes(bytes + 32 * i);
                break;
            case kI64: std::memcpy(host, c.i64.data() + offset, count * 8); break;
            case kU32: std::memcpy(host, c.u32.data() + offset, count * 4); break;
            case kF64: std::memcpy(host, c.f64.data() + offset, count * 8); break;
            case kG1: std::memcpy(host, c.g1.data() + offset, count * 96); break;
            }
        }
        void zero(const ColP& col) override
        {
            CpuCol& c = cpu(col);
            c.widened.clear();
            std::fill(c.fr.begin(), c.fr.end(), Fr::zero());
            std::fill(c.i64.begin(), c.i64.end(), 0);
            std::fill(c.u32.begin(), c.u32.end(), 0u);
            std::fill(c.f64.begin(), c.f64.end(), 0.0);
        }
        void copy_block(const ColP& src, std::size_t so, std::size_t ss, const ColP& dst, std::size_t d_o, std::size_t ds, std::size_t rows,
                        std::size_t width) override
        {
            const CpuCol& s = cpu(src);
            CpuCol& d = cpu(dst);
            d.widened.clear();
            for (std::size_t r = 0; r < rows; ++r)
                for (std::size_t c = 0; c < width; ++c)
                {
                    const std::size_t from = so + r * ss + c, to = d_o + r * ds + c;
                    if (s.kind == kF64) d.f64[to] = s.f64[from];
                    else if (s.kind == kI64) d.i64[to] = s.i64[from];
                    else if (s.kind == kU32) d.u32[to] = s.u32[from];
                    else d.fr[to] = s.fr[from];
                }
        }

        // attention_head_forward_impl, src/model/gat.cpp:474-615 (restated in oracle.cpp)
        void head_forward(const HeadDesc& h, const GraphCols& g, const HeadTraceCols& o) override
        {
            const bool has_bias = h.output_bias != nullptr;
            const int rc = ora_gat_head_forward(
                cpu(h.features).f64.data(), g.node_count, h.input_width, cpu(h.seq_kernel).f64.data(), h.output_width, cpu(h.attn_src).f64.data(),
                h.attn_src_bias, cpu(h.attn_dst).f64.data(), h.attn_dst_bias, has_bias ? cpu(h.output_bias).f64.data() : nullptr,
                has_bias ? h.output_bias->count : 0, has_bias ? 1 : 0, h.apply_activation ? 1 : 0, cpu(g.edge_src).u32.data(), cpu(g.edge_dst).u32.data(),
                g.edge_count, cpu(o.H_prime).f64.data(), cpu(o.E_src).f64.data(), cpu(o.E_dst).f64.data(), cpu(o.S).f64.data(), cpu(o.Z).f64.data(),
                cpu(o.M).f64.data(), cpu(o.Delta).f64.data(), cpu(o.U).f64.data(), cpu(o.Sum).f64.data(), cpu(o.inv).f64.data(), cpu(o.alpha).f64.data(),
                cpu(o.H_agg_pre_bias).f64.data(), cpu(o.H_agg).f64.data());
            if (rc != 0) throw std::runtime_error(ora_last_error());
        }
        // quantize_float, src/protocol/trace.cpp:973-976
        void quantize(const ColP& v, std::size_t count, const ColP& out) override
        {
            const CpuCol& in = cpu(v);
            CpuCol& o = cpu(out);
            o.widened.clear();
            for (std::size_t i = 0; i < count; ++i)
                o.i64[i] = static_cast<std::int64_t>(in.f64[i] >= 0.0 ? in.f64[i] * 16.0 + 0.5 : in.f64[i] * 16.0 - 0.5);
        }
        // broadcast_node_values, trace.cpp:1366-1381
        void gather(const ColP& nv, std::size_t node_count, const ColP& index, std::size_t edge_count, std::size_t domain_size, const ColP& out) override
        {
            const CpuCol& n = cpu(nv);
            const CpuCol& idx = cpu(index);
            CpuCol& o = cpu(out);
            o.widened.clear();
            for (std::size_t e = 0; e < domain_size; ++e)
            {
                const bool live = e < edge_count;
                const std::size_t s = live ? (idx.kind == kU32 ? idx.u32[e] : static_cast<std::size_t>(idx.i64[e])) : 0;
                if (live && s >= node_count) throw std::runtime_error("edge endpoint out of range");
                if (n.kind == kI64) o.i64[e] = live ? n.i64[s] : 0;
                else if (n.kind == kU32) o.u32[e] = live ? n.u32[s] : 0;
                else o.fr[e] = live ? n.fr[s] : Fr::zero();
            }
        }
        void linear_combination(const std::vector<ColP>& cols, const std::vector<Fe>& coefficients, std::size_t count, std::size_t domain_size,
                                const ColP& out) override
        {
            CpuCol& o = cpu(out);
            std::vector<Fr> coeff;
            for (const auto& c : coefficients) coeff.push_back(fe_in(c));
            std::vector<const std::vector<Fr>*> values;
            for (const auto& c : cols) values.push_back(&as_field(c));
            for (std::size_t i = 0; i < domain_size; ++i)
            {
                Fr v = Fr::zero();
                if (i < count)
                    for (std::size_t j = 0; j < cols.size(); ++j) v += coeff[j] * (*values[j])[i];
                o.fr[i] = v;
            }
        }
        void mul_columns(const ColP& l, const ColP& r, std::size_t count, std::size_t domain_size, const ColP& out) override
        {
            const auto& a = as_field(l);
            const auto& b = as_field(r);
            CpuCol& o = cpu(out);
            for (std::size_t i = 0; i < domain_size; ++i) o.fr[i] = i < count ? a[i] * b[i] : Fr::zero();
        }
        // linear_form_by_powers, trace.cpp:273-296
        void linear_form_rows(const ColP& m, std::size_t rows, std::size_t cols, const ColP& powers, const ColP& out) override
        {
            const auto& matrix = as_field(m);
            const auto& p = cpu(powers).fr;
            CpuCol& o = cpu(out);
            for (std::size_t row = 0; row < rows; ++row)
            {
                Fr value = Fr::zero();
                for (std::size_t col = 0; col < cols; ++col) value += matrix[row * cols + col] * p[col];
                o.fr[row] = value;
            }
        }
        void powers(const Fe& c, std::size_t count, const ColP& out) override
        {
            CpuCol& o = cpu(out);
            const Fr base = fe_in(c);
            Fr cur = Fr::one();
            for (std::size_t i = 0; i < count; ++i)
            {
                o.fr[i] = cur;
                cur = cur * base;
            }
        }
        // build_single_lookup_artifacts / build_pair_lookup_artifacts + multiplicity_from_indices
        // (trace.cpp:1916-1933, 2011-2096): the table row of a query comes from a hash map over the
        // table entries that keeps the FIRST of equal entries (emplace), as build_value_index_map /
        // build_pair_index_map do (trace.cpp:1847-1891).
        void lookup_multiplicity(const ColP& x, const ColP& y, std::size_t count, std::int64_t x_min, std::size_t band, const ColP& table_y,
                                 std::size_t table_size, std::size_t domain_size, const ColP& out) override
        {
            CpuCol& o = cpu(out);
            o.widened.clear();
            std::fill(o.u32.begin(), o.u32.begin() + static_cast<std::ptrdiff_t>(domain_size), 0u);
            struct PairHash
            {
                std::size_t operator()(const std::pair<std::int64_t, std::int64_t>& k) const
                {
                    return std::hash<std::int64_t>{}(k.first) ^ (std::hash<std::int64_t>{}(k.second) << 1U);
                }
            };
            std::unordered_map<std::pair<std::int64_t, std::int64_t>, std::size_t, PairHash> index;
            index.reserve(table_size);
            const bool pair = y != nullptr;
            for (std::size_t i = 0; i < table_size; ++i)
                index.emplace(std::make_pair(x_min + static_cast<std::int64_t>(i / band), pair ? cpu(table_y).i64[i] : 0), i);
            auto value_at = [](const CpuCol& c, std::size_t i) { return c.kind == kU32 ? static_cast<std::int64_t>(c.u32[i]) : c.i64[i]; };
            for (std::size_t i = 0; i < count; ++i)
            {
                const auto it = index.find({value_at(cpu(x), i), pair ? value_at(cpu(y), i) : 0});
                if (it == index.end()) throw std::runtime_error("lookup query escaped static table");
                o.u32[it->second] += 1;
            }
        }
        // s_max, trace.cpp:2610-2618
        void first_zero_marker(const ColP& delta, const ColP& gb, const ColP& ge, std::size_t groups, std::size_t domain_size, const ColP& out) override
        {
            const CpuCol& d = cpu(delta);
            CpuCol& o = cpu(out);
            o.widened.clear();
            std::fill(o.u32.begin(), o.u32.begin() + static_cast<std::ptrdiff_t>(domain_size), 0u);
            for (std::size_t g = 0; g < groups; ++g)
                for (std::size_t k = cpu(gb).u32[g]; k < cpu(ge).u32[g]; ++k)
                    if ((d.kind == kI64 ? d.i64[k] == 0 : d.kind == kU32 ? d.u32[k] == 0 : d.fr[k].is_zero()))
                    {
                        o.u32[k] = 1;
                        break;
                    }
        }
        // build_logup_accumulator_with_active_count, src/protocol/lookup.cpp:100-157
        void logup(const ColP& table, const ColP& query, const ColP& mult, const ColP& qt, const ColP& qq, std::size_t n, const Fe& beta,
                   std::size_t active, const ColP& out) override
        {
            CpuCol& o = cpu(out);
            std::fill(o.fr.begin(), o.fr.begin() + static_cast<std::ptrdiff_t>(n), Fr::zero());
            if (n <= 1) return;
            active = std::min(active, n - 1);
            if (active == 0) return;
            const Fr b = fe_in(beta);
            const auto &t = as_field(table), &q = as_field(query), &m = as_field(mult), &st = as_field(qt), &sq = as_field(qq);
            std::vector<Fr> denominators(active * 2);
            for (std::size_t i = 0; i < active; ++i)
            {
                denominators[2 * i] = t[i] + b;
                denominators[2 * i + 1] = q[i] + b;
            }
            batch_invert_in_place(denominators);
            Fr running = Fr::zero();
            for (std::size_t i = 0; i < active; ++i)
            {
                running += st[i] * m[i] * denominators[2 * i];
                running = running - sq[i] * denominators[2 * i + 1];
                o.fr[i + 1] = running;
            }
            for (std::size_t i = active + 1; i < n; ++i) o.fr[i] = o.fr[active];
        }
        // build_route_node_accumulator / build_route_edge_accumulator, trace.cpp:298-361
        void route_node(const ColP& table, const ColP& mult, std::size_t valid, std::size_t domain_size, const Fe& beta, const ColP& out) override
        {
            route(as_field(table), &as_field(mult), valid, domain_size, beta, out);
        }
        void route_edge(const ColP& query, std::size_t valid, std::size_t domain_size, const Fe& beta, const ColP& out) override
        {
            route(as_field(query), nullptr, valid, domain_size, beta, out);
        }
        // build_group_prefix_state / build_max_counter_state, src/protocol/psq.cpp:7-39
        void group_prefix_state(const ColP& values, const ColP& q_new, std::size_t n, const ColP& out) override
        {
            const auto& v = as_field(values);
            const auto& q = as_field(q_new);
            CpuCol& o = cpu(out);
            if (n > 0) o.fr[0] = v[0];
            for (std::size_t i = 1; i < n; ++i) o.fr[i] = q[i] * v[i] + (Fr::one() - q[i]) * (o.fr[i - 1] + v[i]);
        }
        // accumulator of build_binding_trace (trace.cpp:1595-1621) / build_zkmap_trace (zkmap.cpp:7-32)
        void zkmap(const ColP& a, const ColP& b, std::size_t count, std::size_t domain_size, const ColP& out) override
        {
            const auto& x = as_field(a);
            const auto& y = as_field(b);
            CpuCol& o = cpu(out);
            std::fill(o.fr.begin(), o.fr.begin() + static_cast<std::ptrdiff_t>(domain_size), Fr::zero());
            Fr mu = Fr::zero();
            for (std::size_t i = 0; i < count; ++i)
            {
                mu += x[i] * y[i];
                if (i + 1 < domain_size) o.fr[i + 1] = mu;
            }
            for (std::size_t i = count + 1; i < domain_size; ++i) o.fr[i] = mu;
        }
        // barycentric_weights_native, src/algebra/polynomial.cpp:131-316: serial below 2^20, chunked batch
        // inversion over the hardware threads above (each chunk inverts its own product)
        void bary_weights(unsigned log2n, const Fe& x_bytes, const ColP& out) override
        {
            const std::size_t size = static_cast<std::size_t>(1) << log2n;
            const Fr x = fe_in(x_bytes);
            const Fr omega = oracle::root_of_unity(size);
            const Fr inv_size = Fr::from_u64(size).inv();
            const Fr zero_eval = x.pow(static_cast<oracle::u64>(size)) - Fr::one();
            if (zero_eval.is_zero()) throw std::runtime_error("barycentric point lies on the domain");
            CpuCol& o = cpu(out);
            const std::size_t used = size < (static_cast<std::size_t>(1) << 20) ? 1 : threads_;
            parallel_chunks(size, used, [&](std::size_t, std::size_t begin, std::size_t end) {
                std::vector<Fr> points(end - begin), denominators(end - begin);
                Fr point = omega.pow(static_cast<oracle::u64>(begin));
                for (std::size_t i = begin; i < end; ++i)
                {
                    points[i - begin] = point;
                    denominators[i - begin] = x - point;
                    point = point * omega;
                }
                batch_invert_in_place(denominators);
                for (std::size_t i = begin; i < end; ++i) o.fr[i] = zero_eval * (points[i - begin] * inv_size) * denominators[i - begin];
            });
        }
        // weighted_column_sum_native, trace.cpp:203-271
        void fold_rows(const ColP& m, std::size_t rows, std::size_t cols, const ColP& weights, std::size_t row_count, const ColP& out) override
        {
            (void)rows;
            const auto& matrix = as_field(m);
            const auto& w = cpu(weights).fr;
            CpuCol& o = cpu(out);
            std::vector<std::vector<Fr>> partial(threads_, std::vector<Fr>(cols, Fr::zero()));
            parallel_chunks(row_count, threads_, [&](std::size_t t, std::size_t begin, std::size_t end) {
                for (std::size_t row = begin; row < end; ++row)
                    for (std::size_t col = 0; col < cols; ++col) partial[t][col] += matrix[row * cols + col] * w[row];
            });
            for (std::size_t col = 0; col < cols; ++col)
            {
                Fr total = Fr::zero();
                for (const auto& p : partial) total += p[col];
                o.fr[col] = total;
            }
        }
        // evaluate_with_native_weight_rotations (eval_backend.cpp:309-444) / the shared-weights commit loop
        // (src/crypto/kzg.cpp:161-282): out[p][k] = sum_c w[c] * col_k[(c + rot_p) mod n], columns zero
        // beyond len; the row range is chunked over the hardware threads, partial sums added in chunk order
        void eval_device(const std::vector<ColP>& cols, std::size_t len, unsigned log2n, const ColP& weights, const std::vector<std::uint64_t>& rotations,
                         const ColP& out, std::size_t out_offset) override
        {
            const std::size_t n = static_cast<std::size_t>(1) << log2n, mask = n - 1, k_count = cols.size(), p_count = rotations.size();
            const auto& w = cpu(weights).fr;
            std::vector<const std::vector<Fr>*> values;
            for (const auto& c : cols) values.push_back(&as_field(c));
            const std::size_t used = std::max<std::size_t>(1, std::min(threads_, len / 512 == 0 ? 1 : len / 512));
            std::vector<std::vector<Fr>> partials(used, std::vector<Fr>(p_count * k_count, Fr::zero()));
            parallel_chunks(len, used, [&](std::size_t t, std::size_t begin, std::size_t end) {
                auto& partial = partials[t];
                for (std::size_t row = begin; row < end; ++row)
                    for (std::size_t p = 0; p < p_count; ++p)
                    {
                        const Fr& weight = w[(row - rotations[p]) & mask];  // row `row` of the column meets w[(row - rot) mod n]
                        for (std::size_t k = 0; k < k_count; ++k) partial[p * k_count + k] += (*values[k])[row] * weight;
                    }
            });
            CpuCol& o = cpu(out);
            for (std::size_t i = 0; i < p_count * k_count; ++i)
            {
                Fr total = Fr::zero();
                for (const auto& partial : partials) total += partial[i];
                o.fr[out_offset + i] = total;
            }
        }
        // matrix_row_major_evaluation, trace.cpp:508-573: Horner per row, rows combined with x^cols
        void horner_device(const ColP& m, std::size_t rows, std::size_t cols, const Fe& x_bytes, const ColP& out, std::size_t out_offset) override
        {
            const auto& matrix = as_field(m);
            const Fr x = fe_in(x_bytes);
            const Fr row_stride = x.pow(static_cast<oracle::u64>(cols));
            std::vector<Fr> partial(threads_, Fr::zero());
            parallel_chunks(rows, threads_, [&](std::size_t t, std::size_t begin, std::size_t end) {
                Fr acc = Fr::zero();
                for (std::size_t row = end; row-- > begin;)
                {
                    Fr row_value = Fr::zero();
                    for (std::size_t col = cols; col-- > 0;) row_value = row_value * x + matrix[row * cols + col];
                    acc = acc * row_stride + row_value;
                }
                partial[t] = acc * row_stride.pow(static_cast<oracle::u64>(begin));
            });
            Fr total = Fr::zero();
            for (const auto& p : partial) total += p;
            cpu(out).fr[out_offset] = total;
        }
        // g1_mul_same_base_batch, src/crypto/curve.cpp:138-238: K independent scalar multiplications
        void g1_fixed_base(const G1& base, const ColP& scalars, std::size_t count, const ColP& out_points) override
        {
            const oracle::G1 b = oracle::G1::from_affine(oracle::g1_from_bytes(base.data()));
            const auto& s = cpu(scalars).fr;
            CpuCol& o = cpu(out_points);
            parallel_chunks(count, threads_, [&](std::size_t, std::size_t begin, std::size_t end) {
                for (std::size_t i = begin; i < end; ++i) oracle::g1_to_bytes(b.mul(s[i]).to_affine(), o.g1[i].data());
            });
        }
        // evaluate_lazy_large_fh_public_group_points, src/protocol/prover.cpp:1205-1675: dot products of the
        // weights with generated columns {1, row, col, abs id, feature}
        void fh_public_eval(const ColP& features, std::size_t rows, std::size_t fc, const ColP& abs_ids, const ColP& weights, unsigned log2n,
                            std::uint64_t rotation, Fe out[5]) override
        {
            // the weights at the rotated point, as the reference builds them for its second opening point
            // (a rotation of the vector: w_i(omega z) = w_{i-1}(z))
            const std::size_t n = static_cast<std::size_t>(1) << log2n;
            std::vector<Fr> rotated;
            if (rotation != 0)
            {
                const auto& base = cpu(weights).fr;
                rotated.resize(n);
                for (std::size_t i = 0; i < n; ++i) rotated[i] = base[(i + n - rotation) & (n - 1)];
            }
            const auto& w = rotation != 0 ? rotated : cpu(weights).fr;
            const auto& f = as_field(features);
            const CpuCol* ids = abs_ids ? &cpu(abs_ids) : nullptr;
            const std::size_t valid = rows * fc;
            std::vector<std::array<Fr, 5>> partial(threads_);
            for (auto& p : partial) p.fill(Fr::zero());
            parallel_chunks(valid, threads_, [&](std::size_t t, std::size_t begin, std::size_t end) {
                auto& s = partial[t];
                for (std::size_t index = begin; index < end; ++index)
                {
                    const std::size_t row = index / fc;
                    s[0] += w[index];
                    s[1] += w[index] * Fr::from_u64(row);
                    s[2] += w[index] * Fr::from_u64(index % fc);
                    if (ids != nullptr) s[3] += w[index] * Fr::from_i64(ids->i64[row]);
                    s[4] += w[index] * f[index];
                }
            });
            for (int i = 0; i < 5; ++i)
            {
                Fr total = Fr::zero();
                for (const auto& p : partial) total += p[static_cast<std::size_t>(i)];
                out[i] = fe_out(total);
            }
        }
        void synchronize() override {}
        // the radix-2 transform of oracle.cpp over the same bytes
        void transform(std::vector<Fe>& data, bool inverse) override
        {
            if (ora_ntt(reinterpret_cast<std::uint8_t*>(data.data()), data.size(), inverse ? 1 : 0, nullptr) != 0)
                throw std::runtime_error("transform: the length must be a power of two");
        }
        // independent vectors on the host's threads
        void transform_many(std::vector<std::vector<Fe>>& vectors, bool inverse) override
        {
            const std::size_t workers = std::max<std::size_t>(1, std::min<std::size_t>({std::thread::hardware_concurrency(), 32, vectors.size()}));
            std::vector<std::thread> pool;
            std::vector<int> failed(workers, 0);
            for (std::size_t w = 0; w < workers; ++w)
                pool.emplace_back([&, w] {
                    for (std::size_t i = w; i < vectors.size(); i += workers)
                        if (ora_ntt(reinterpret_cast<std::uint8_t*>(vectors[i].data()), vectors[i].size(), inverse ? 1 : 0, nullptr) != 0) failed[w] = 1;
                });
            for (auto& t : pool) t.join();
            for (int f : failed)
                if (f) throw std::runtime_error("transform: the length must be a power of two");
        }

    private:
        static CpuCol& cpu(const ColP& c)
        {
            if (c == nullptr) throw std::runtime_error("flow: missing column");
            return *static_cast<CpuCol*>(c.get());
        }
        // a column as field elements; small-integer kinds are widened once (FieldElement::from_signed)
        static const std::vector<Fr>& as_field(const ColP& col)
        {
            CpuCol& c = cpu(col);
            if (c.kind == kFr || c.kind == kFrMont) return c.fr;
            const std::size_t n = c.kind == kI64 ? c.i64.size() : c.u32.size();
            if (c.widened.size() != n)
            {
                c.widened.resize(n);
                for (std::size_t i = 0; i < n; ++i) c.widened[i] = c.kind == kI64 ? Fr::from_i64(c.i64[i]) : Fr::from_u64(c.u32[i]);
            }
            return c.widened;
        }
        void route(const std::vector<Fr>& values, const std::vector<Fr>* mult, std::size_t valid, std::size_t domain_size, const Fe& beta, const ColP& out)
        {
            CpuCol& o = cpu(out);
            std::fill(o.fr.begin(), o.fr.begin() + static_cast<std::ptrdiff_t>(domain_size), Fr::zero());
            if (domain_size == 0 || valid == 0) return;
            if (valid >= domain_size) throw std::runtime_error("route accumulator needs valid_length < domain_size");
            const Fr b = fe_in(beta);
            std::vector<Fr> denominators(valid);
            for (std::size_t i = 0; i < valid; ++i) denominators[i] = values[i] + b;
            batch_invert_in_place(denominators);
            Fr running = Fr::zero();
            for (std::size_t i = 0; i < valid; ++i)
            {
                running += mult != nullptr ? (*mult)[i] * denominators[i] : denominators[i];
                o.fr[i + 1] = running;
            }
            for (std::size_t i = valid + 1; i < domain_size; ++i) o.fr[i] = o.fr[valid];
        }
        std::size_t threads_;
    };
}

struct ora_flow : gatzk_flow::FlowHandle
{
};

extern "C"
{
    const char* ora_flow_error(void) { return gatzk_flow::flow_error_slot().c_str(); }
    // `threads`: host threads for the leaves the reference fans out (0 = hardware concurrency)
    int ora_flow_create(int threads, const gzk_flow_config* config, ora_flow** out)
    {
        gatzk_flow::FlowHandle* handle = nullptr;
        const std::size_t t = threads > 0 ? static_cast<std::size_t>(threads) : std::max(1u, std::thread::hardware_concurrency());
        const int rc = gatzk_flow::flow_create_impl(std::make_unique<CpuBackend>(t), config, &handle);
        if (rc == 0) *out = static_cast<ora_flow*>(handle);
        return rc;
    }
    void ora_flow_destroy(ora_flow* flow)
    {
        if (flow == nullptr) return;
        flow->flow.reset();
        delete static_cast<gatzk_flow::FlowHandle*>(flow);
    }
    int ora_flow_prove(ora_flow* flow) { return gatzk_flow::flow_prove_impl(flow, false); }
    int ora_flow_prove_resident(ora_flow* flow) { return gatzk_flow::flow_prove_impl(flow, true); }
    size_t ora_flow_dump(ora_flow* flow, char* out, size_t cap) { return gatzk_flow::flow_dump_impl(flow, out, cap); }
    size_t ora_flow_proof_bytes(ora_flow* flow, uint8_t* out, size_t cap) { return gatzk_flow::flow_proof_bytes_impl(flow, out, cap); }
    int ora_flow_stats(ora_flow* flow, uint64_t out[14]) { return gatzk_flow::flow_stats_impl(flow, out); }
    int ora_flow_column(ora_flow* flow, const char* label, int* kind, uint64_t* length, void* out, size_t cap_elements)
    {
        return gatzk_flow::flow_column_impl(flow, label, kind, length, out, cap_elements);
    }
    int ora_flow_constraint_violations(ora_flow* flow, uint64_t out[7], uint64_t* failures, size_t cap, size_t* count)
    {
        return gatzk_flow::flow_constraint_violations_impl(flow, out, failures, cap, count);
    }
    int ora_flow_honest_quotient(ora_flow* flow, const char* domain, unsigned log2_blowup, unsigned classes, uint64_t out[6])
    {
        return gatzk_flow::flow_honest_quotient_impl(flow, domain, log2_blowup, classes, out);
    }
    size_t ora_flow_domain_labels(ora_flow* flow, const char* domain, char* out, size_t cap)
    {
        return gatzk_flow::flow_domain_labels_impl(flow, domain, out, cap);
    }
}
