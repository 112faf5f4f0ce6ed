// TEST INFRASTRUCTURE — CPU oracle (see field.hpp for the full statement,
// including "parity unpinned" at the mcl boundary).
//
// Restatement of the reference prover's data-parallel leaves with its own
// loop structure, one function per reference function, exported with C linkage
// so that tests can call them through ctypes.  All Fr values cross the
// boundary as 32-byte little-endian canonical integers (the format of
// FieldElement::write_little_endian, include/gatzk/algebra/field.hpp:193-201);
// G1 points as x||y (2 x 48 bytes LE), 96 zero bytes = infinity.
//
// Return value of every function: 0 = ok, non-zero = the reference would have
// thrown (message retrievable with ora_last_error).

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <functional>
#include <string>
#include <thread>
#include <vector>

#include "field.hpp"
#include "g1.hpp"

using namespace oracle;

namespace
{
    thread_local std::string g_error;

    using Bytes = std::uint8_t;

    std::vector<Fr> load_fr(const Bytes* in, std::size_t n)
    {
        std::vector<Fr> out(n);
        for (std::size_t i = 0; i < n; ++i) out[i] = Fr::from_le_bytes(in + 32 * i);
        return out;
    }
    void store_fr(const std::vector<Fr>& v, Bytes* out)
    {
        for (std::size_t i = 0; i < v.size(); ++i) v[i].to_le_bytes(out + 32 * i);
    }

    template <typename F>
    int guarded(F&& f)
    {
        try
        {
            f();
            return 0;
        }
        catch (const std::exception& e)
        {
            g_error = e.what();
            return 1;
        }
    }

    // The reference fans out over hardware threads with std::async in
    // contiguous chunks and adds the partial results in chunk order; field
    // addition is exact, so the chunking does not change any value.
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
            const std::size_t begin = t * chunk;
            const std::size_t end = std::min(n, begin + chunk);
            if (begin >= end) break;
            pool.emplace_back(body, t, begin, end);
        }
        for (auto& th : pool) th.join();
    }

    // include/gatzk/algebra/field.hpp:221-253 (batch_invert) and
    // src/protocol/lookup.cpp:32-58 (batch_inverse_native): prefix products,
    // one inversion, backward sweep; a zero input is an error.
    std::vector<Fr> batch_invert(const std::vector<Fr>& values)
    {
        std::vector<Fr> out(values.size());
        if (values.empty()) return out;
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
            out[i] = suffix_inverse * prefixes[i];
            suffix_inverse = suffix_inverse * values[i];
        }
        return out;
    }

    // src/algebra/polynomial.cpp:131-177 (serial branch of
    // barycentric_weights_native): w_i = (x^n - 1) * (omega^i / n) / (x - omega^i).
    // The chunk-parallel branch (:179-315) computes the same field values.
    std::vector<Fr> bary_weights(const Fr& x, std::size_t size)
    {
        const Fr omega = root_of_unity(size);
        const Fr inv_size = Fr::from_u64(size).inv();
        std::vector<Fr> denominators(size), prefixes(size), points(size);
        Fr acc = Fr::one();
        Fr point = Fr::one();
        for (std::size_t i = 0; i < size; ++i)
        {
            points[i] = point;
            denominators[i] = x - point;
            prefixes[i] = acc;
            acc = acc * denominators[i];
            point = point * omega;
        }
        if (acc.is_zero()) throw std::runtime_error("barycentric point lies on the domain");
        Fr suffix_inverse = acc.inv();
        const Fr zero_eval = x.pow(static_cast<u64>(size)) - Fr::one();
        std::vector<Fr> weights(size);
        for (std::size_t i = size; i-- > 0;)
        {
            const Fr inverse = suffix_inverse * prefixes[i];
            weights[i] = zero_eval * (points[i] * inv_size) * inverse;
            suffix_inverse = suffix_inverse * denominators[i];
        }
        return weights;
    }

    // src/algebra/polynomial.cpp:499-508.
    Fr horner(const std::vector<Fr>& coefficients, const Fr& x)
    {
        Fr out = Fr::zero();
        for (auto it = coefficients.rbegin(); it != coefficients.rend(); ++it)
        {
            out *= x;
            out += *it;
        }
        return out;
    }

    // src/crypto/transcript.cpp:10-19.
    std::uint64_t fnv1a(const std::string& data)
    {
        std::uint64_t hash = 1469598103934665603ULL;
        for (const unsigned char ch : data)
        {
            hash ^= ch;
            hash *= 1099511628211ULL;
        }
        return hash;
    }
}

extern "C"
{
    const char* ora_last_error() { return g_error.c_str(); }

    // ---- a1: field primitives (field.hpp:28-205) ---------------------------------
    int ora_fr_binop(int op, const Bytes* a, const Bytes* b, std::size_t n, Bytes* out)
    {
        return guarded([&] {
            for (std::size_t i = 0; i < n; ++i)
            {
                const Fr x = Fr::from_le_bytes(a + 32 * i);
                const Fr y = Fr::from_le_bytes(b + 32 * i);
                Fr z;
                switch (op)
                {
                case 0: z = x + y; break;
                case 1: z = x - y; break;
                case 2: z = x * y; break;
                default: throw std::runtime_error("unknown op");
                }
                z.to_le_bytes(out + 32 * i);
            }
        });
    }
    int ora_fr_inv(const Bytes* a, std::size_t n, Bytes* out)
    {
        return guarded([&] {
            for (std::size_t i = 0; i < n; ++i) Fr::from_le_bytes(a + 32 * i).inv().to_le_bytes(out + 32 * i);
        });
    }
    int ora_fr_pow_u64(const Bytes* a, std::uint64_t e, Bytes* out)
    {
        return guarded([&] { Fr::from_le_bytes(a).pow(e).to_le_bytes(out); });
    }
    int ora_fr_from_i64(const std::int64_t* in, std::size_t n, Bytes* out)
    {
        return guarded([&] {
            for (std::size_t i = 0; i < n; ++i) Fr::from_i64(in[i]).to_le_bytes(out + 32 * i);
        });
    }
    int ora_fr_from_le_mod(const Bytes* in, std::size_t size, Bytes* out)
    {
        return guarded([&] { Fr::from_le_bytes_mod(in, size).to_le_bytes(out); });
    }
    int ora_fr_to_decimal(const Bytes* a, char* out, std::size_t cap)
    {
        return guarded([&] {
            const auto s = Fr::from_le_bytes(a).to_decimal();
            if (s.size() + 1 > cap) throw std::runtime_error("buffer too small");
            std::memcpy(out, s.c_str(), s.size() + 1);
        });
    }
    int ora_fp_binop(int op, const Bytes* a, const Bytes* b, std::size_t n, Bytes* out)
    {
        return guarded([&] {
            for (std::size_t i = 0; i < n; ++i)
            {
                const Fp x = Fp::from_le_bytes(a + 48 * i);
                const Fp y = Fp::from_le_bytes(b + 48 * i);
                Fp z;
                switch (op)
                {
                case 0: z = x + y; break;
                case 1: z = x - y; break;
                case 2: z = x * y; break;
                default: throw std::runtime_error("unknown op");
                }
                z.to_le_bytes(out + 48 * i);
            }
        });
    }
    int ora_root_of_unity(std::uint64_t size, Bytes* out)
    {
        return guarded([&] { root_of_unity(size).to_le_bytes(out); });
    }
    int ora_batch_invert(const Bytes* in, std::size_t n, Bytes* out)
    {
        return guarded([&] { store_fr(batch_invert(load_fr(in, n)), out); });
    }

    // ---- a2: barycentric weights (polynomial.cpp:131-316) -------------------------
    int ora_bary_weights(const Bytes* x, std::uint64_t size, Bytes* out)
    {
        return guarded([&] { store_fr(bary_weights(Fr::from_le_bytes(x), size), out); });
    }

    // ---- a3: packed evaluation (eval_backend.cpp:191-292, 309-444) -----------------
    // columns: K column-major arrays of n elements ([k][c]); the reference's
    // interleaved [c*K+k] copy is a storage detail.  out[p][k] =
    // sum_c w[c] * col_k[(c + rot_p) mod n].
    int ora_eval_rotations(const Bytes* columns, std::size_t k_count, std::size_t n, const Bytes* weights,
                           const std::uint64_t* rotations, std::size_t p_count, std::size_t threads, Bytes* out)
    {
        return guarded([&] {
            if (n == 0 || (n & (n - 1)) != 0) throw std::runtime_error("domain size must be a non-zero power of two");
            const auto w = load_fr(weights, n);
            const std::size_t mask = n - 1;
            std::vector<std::vector<Fr>> partials;
            const std::size_t used = std::max<std::size_t>(1, std::min(threads, n / 512 == 0 ? 1 : n / 512));
            partials.assign(used, std::vector<Fr>(p_count * k_count, Fr::zero()));
            parallel_chunks(n, used, [&](std::size_t t, std::size_t begin, std::size_t end) {
                auto& partial = partials[t];
                for (std::size_t column = begin; column < end; ++column)
                {
                    for (std::size_t p = 0; p < p_count; ++p)
                    {
                        const std::size_t rotated = (column + rotations[p]) & mask;
                        for (std::size_t k = 0; k < k_count; ++k)
                        {
                            const Fr value = Fr::from_le_bytes(columns + 32 * (k * n + rotated));
                            partial[p * k_count + k] += value * w[column];
                        }
                    }
                }
            });
            std::vector<Fr> total(p_count * k_count, Fr::zero());
            for (const auto& partial : partials)
                for (std::size_t i = 0; i < total.size(); ++i) total[i] += partial[i];
            store_fr(total, out);
        });
    }

    // ---- a4: commit tau-evaluation (kzg.cpp:161-282) -------------------------------
    // K columns that share one valid length (<= n); the dot product runs over
    // the valid prefix only.
    int ora_commit_tau_eval(const Bytes* columns, std::size_t k_count, std::size_t valid, const Bytes* weights,
                            std::size_t threads, Bytes* out)
    {
        return guarded([&] {
            const auto w = load_fr(weights, valid);
            const std::size_t used = std::max<std::size_t>(1, std::min(threads, valid / 512 == 0 ? 1 : valid / 512));
            std::vector<std::vector<Fr>> partials(used, std::vector<Fr>(k_count, Fr::zero()));
            parallel_chunks(valid, used, [&](std::size_t t, std::size_t begin, std::size_t end) {
                for (std::size_t index = begin; index < end; ++index)
                    for (std::size_t k = 0; k < k_count; ++k)
                        partials[t][k] += Fr::from_le_bytes(columns + 32 * (k * valid + index)) * w[index];
            });
            std::vector<Fr> total(k_count, Fr::zero());
            for (const auto& partial : partials)
                for (std::size_t k = 0; k < k_count; ++k) total[k] += partial[k];
            store_fr(total, out);
        });
    }

    // Small-integer columns: the reference stores from_signed(v) and runs the same
    // loop; this entry point widens int64 on the fly (field.hpp:71-76).
    int ora_commit_tau_eval_i64(const std::int64_t* columns, std::size_t k_count, std::size_t valid,
                                const Bytes* weights, Bytes* out)
    {
        return guarded([&] {
            const auto w = load_fr(weights, valid);
            std::vector<Fr> total(k_count, Fr::zero());
            for (std::size_t index = 0; index < valid; ++index)
                for (std::size_t k = 0; k < k_count; ++k) total[k] += Fr::from_i64(columns[k * valid + index]) * w[index];
            store_fr(total, out);
        });
    }

    // ---- a12: Polynomial::evaluate (polynomial.cpp:415-508) ------------------------
    int ora_horner(const Bytes* coefficients, std::size_t n, const Bytes* x, Bytes* out)
    {
        return guarded([&] { horner(load_fr(coefficients, n), Fr::from_le_bytes(x)).to_le_bytes(out); });
    }
    // Evaluation-basis branch: direct hit when x is a domain point, otherwise
    // zero_eval * inv_size * sum_i v_i * omega^i / (x - omega^i) with one
    // inversion per element (polynomial.cpp:18-32, 485-495).
    int ora_poly_evaluate_barycentric(const Bytes* values, std::size_t valid, std::uint64_t size, const Bytes* x,
                                      Bytes* out)
    {
        return guarded([&] {
            const auto v = load_fr(values, valid);
            const Fr xx = Fr::from_le_bytes(x);
            const Fr omega = root_of_unity(size);
            Fr point = Fr::one();
            for (std::size_t i = 0; i < size; ++i)
            {
                if (point == xx)
                {
                    (i < valid ? v[i] : Fr::zero()).to_le_bytes(out);
                    return;
                }
                point *= omega;
            }
            const Fr zero_eval = xx.pow(size) - Fr::one();
            const Fr inv_size = Fr::from_u64(size).inv();
            Fr sum = Fr::zero();
            point = Fr::one();
            for (std::size_t i = 0; i < valid; ++i)
            {
                sum += v[i] * point * (xx - point).inv();
                point *= omega;
            }
            (zero_eval * inv_size * sum).to_le_bytes(out);
        });
    }

    // ---- a6: matrix as one coefficient polynomial (trace.cpp:508-573) ---------------
    int ora_matrix_row_major_eval(const Bytes* matrix, std::size_t rows, std::size_t cols, const Bytes* x, Bytes* out)
    {
        return guarded([&] {
            if (rows == 0 || cols == 0)
            {
                Fr::zero().to_le_bytes(out);
                return;
            }
            const Fr point = Fr::from_le_bytes(x);
            std::vector<Fr> row_evaluations(rows);
            for (std::size_t row = 0; row < rows; ++row)
            {
                Fr acc = Fr::zero();
                for (std::size_t column = cols; column-- > 0;)
                {
                    acc *= point;
                    acc += Fr::from_le_bytes(matrix + 32 * (row * cols + column));
                }
                row_evaluations[row] = acc;
            }
            const Fr row_stride = point.pow(static_cast<u64>(cols));
            Fr acc = Fr::zero();
            for (std::size_t row = rows; row-- > 0;)
            {
                acc *= row_stride;
                acc += row_evaluations[row];
            }
            acc.to_le_bytes(out);
        });
    }

    // ---- a9: bindings (trace.cpp:203-296, 1358-1364, 1595-1621; zkmap.cpp:7-32) -----
    // Fold matrix rows by weights: out[c] = sum_{row < row_count} w[row] * M[row][c].
    int ora_weighted_column_sum(const Bytes* matrix, std::size_t rows, std::size_t cols, const Bytes* row_weights,
                                std::size_t row_count, Bytes* out)
    {
        return guarded([&] {
            if (row_count > rows) throw std::runtime_error("weighted column sum native input size mismatch");
            const auto w = load_fr(row_weights, row_count);
            std::vector<Fr> total(cols, Fr::zero());
            for (std::size_t row = 0; row < row_count; ++row)
                for (std::size_t column = 0; column < cols; ++column)
                    total[column] += Fr::from_le_bytes(matrix + 32 * (row * cols + column)) * w[row];
            store_fr(total, out);
        });
    }
    // out[i] = sum_j M[i][j] * powers[j]; compress_rows_with_challenge passes
    // powers = 1, c, c^2, ...
    int ora_linear_form_by_powers(const Bytes* matrix, std::size_t rows, std::size_t cols, const Bytes* column_powers,
                                  Bytes* out)
    {
        return guarded([&] {
            const auto p = load_fr(column_powers, cols);
            for (std::size_t i = 0; i < rows; ++i)
            {
                Fr sum = Fr::zero();
                for (std::size_t j = 0; j < cols; ++j) sum += Fr::from_le_bytes(matrix + 32 * (i * cols + j)) * p[j];
                sum.to_le_bytes(out + 32 * i);
            }
        });
    }
    int ora_powers(const Bytes* challenge, std::size_t count, Bytes* out)
    {
        return guarded([&] {
            const Fr c = Fr::from_le_bytes(challenge);
            Fr cur = Fr::one();
            for (std::size_t i = 0; i < count; ++i)
            {
                cur.to_le_bytes(out + 32 * i);
                cur *= c;
            }
        });
    }
    // Running inner product: acc[0] = 0, acc[i+1] = acc[i] + a[i]*b[i] for
    // i < count, tail filled with the total; mu = total.
    int ora_zkmap_accumulator(const Bytes* a, const Bytes* b, std::size_t count, std::size_t domain_size, Bytes* acc_out,
                              Bytes* mu_out)
    {
        return guarded([&] {
            if (count + 1 > domain_size && count != 0) throw std::runtime_error("zkMaP accumulator exceeds its domain");
            const auto av = load_fr(a, count);
            const auto bv = load_fr(b, count);
            std::vector<Fr> acc(domain_size, Fr::zero());
            Fr mu = Fr::zero();
            for (std::size_t i = 0; i < count; ++i)
            {
                mu += av[i] * bv[i];
                acc[i + 1] = mu;
            }
            for (std::size_t i = count + 1; i < domain_size; ++i) acc[i] = acc[count];
            store_fr(acc, acc_out);
            mu.to_le_bytes(mu_out);
        });
    }

    // ---- a7: LogUp and route running sums (lookup.cpp:100-157; trace.cpp:298-361) ---
    int ora_logup_accumulator(const Bytes* table, const Bytes* query, const Bytes* multiplicity, const Bytes* q_table,
                              const Bytes* q_query, std::size_t n, const Bytes* beta, std::size_t active_count,
                              Bytes* out)
    {
        return guarded([&] {
            std::vector<Fr> accumulator(n, Fr::zero());
            if (n > 1)
            {
                active_count = std::min(active_count, n - 1U);
                if (active_count > 0)
                {
                    const Fr b = Fr::from_le_bytes(beta);
                    const auto t = load_fr(table, active_count);
                    const auto q = load_fr(query, active_count);
                    const auto m = load_fr(multiplicity, active_count);
                    const auto qt = load_fr(q_table, active_count);
                    const auto qq = load_fr(q_query, active_count);
                    std::vector<Fr> denominators(active_count * 2);
                    for (std::size_t i = 0; i < active_count; ++i)
                    {
                        denominators[2 * i] = t[i] + b;
                        denominators[2 * i + 1] = q[i] + b;
                    }
                    const auto inverses = batch_invert(denominators);
                    Fr running = Fr::zero();
                    for (std::size_t i = 0; i < active_count; ++i)
                    {
                        running += qt[i] * m[i] * inverses[2 * i];
                        running -= qq[i] * inverses[2 * i + 1];
                        accumulator[i + 1] = running;
                    }
                    for (std::size_t i = active_count + 1; i < n; ++i) accumulator[i] = accumulator[active_count];
                }
            }
            store_fr(accumulator, out);
        });
    }
    // lookup.cpp:12-30.
    std::uint64_t ora_active_transition_count(const Bytes* q_table, const Bytes* q_query, std::size_t n)
    {
        if (n <= 1) return 0;
        std::uint64_t active = 0;
        for (std::size_t i = 0; i + 1 < n; ++i)
        {
            bool nz = false;
            for (int b = 0; b < 32; ++b) nz = nz || q_table[32 * i + b] != 0 || q_query[32 * i + b] != 0;
            if (nz) active = i + 1;
        }
        return active;
    }
    int ora_route_node_accumulator(const Bytes* table, const Bytes* multiplicity, std::size_t valid_length,
                                   std::size_t domain_size, const Bytes* beta, Bytes* out)
    {
        return guarded([&] {
            std::vector<Fr> acc(domain_size, Fr::zero());
            if (domain_size != 0 && valid_length != 0)
            {
                if (valid_length >= domain_size) throw std::runtime_error("route accumulator needs valid_length < domain_size");
                const Fr b = Fr::from_le_bytes(beta);
                const auto t = load_fr(table, valid_length);
                const auto m = load_fr(multiplicity, valid_length);
                std::vector<Fr> denominators(valid_length);
                for (std::size_t i = 0; i < valid_length; ++i) denominators[i] = t[i] + b;
                const auto inverses = batch_invert(denominators);
                Fr running = Fr::zero();
                for (std::size_t i = 0; i < valid_length; ++i)
                {
                    running += m[i] * inverses[i];
                    acc[i + 1] = running;
                }
                for (std::size_t i = valid_length + 1; i < domain_size; ++i) acc[i] = acc[valid_length];
            }
            store_fr(acc, out);
        });
    }
    int ora_route_edge_accumulator(const Bytes* query, std::size_t valid_length, std::size_t domain_size,
                                   const Bytes* beta, Bytes* out)
    {
        return guarded([&] {
            std::vector<Fr> acc(domain_size, Fr::zero());
            if (domain_size != 0 && valid_length != 0)
            {
                if (valid_length >= domain_size) throw std::runtime_error("route accumulator needs valid_length < domain_size");
                const Fr b = Fr::from_le_bytes(beta);
                const auto q = load_fr(query, valid_length);
                std::vector<Fr> denominators(valid_length);
                for (std::size_t i = 0; i < valid_length; ++i) denominators[i] = q[i] + b;
                const auto inverses = batch_invert(denominators);
                Fr running = Fr::zero();
                for (std::size_t i = 0; i < valid_length; ++i)
                {
                    running += inverses[i];
                    acc[i + 1] = running;
                }
                for (std::size_t i = valid_length + 1; i < domain_size; ++i) acc[i] = acc[valid_length];
            }
            store_fr(acc, out);
        });
    }

    // ---- a8: segmented prefix states (psq.cpp:7-39; trace.cpp:2610-2618) -----------
    // out[0] = v[0]; out[i] = q_new[i]*v[i] + (1-q_new[i])*(out[i-1]+v[i]).  The
    // formula is evaluated literally, so q_new need not be boolean.
    int ora_group_prefix_state(const Bytes* values, const Bytes* q_new, std::size_t n, Bytes* out)
    {
        return guarded([&] {
            const auto v = load_fr(values, n);
            const auto q = load_fr(q_new, n);
            std::vector<Fr> o(n, Fr::zero());
            if (n > 0) o[0] = v[0];
            for (std::size_t i = 1; i < n; ++i) o[i] = q[i] * v[i] + (Fr::one() - q[i]) * (o[i - 1] + v[i]);
            store_fr(o, out);
        });
    }
    // s_max: for each dst group [begin,end) mark the first k with delta[k] == 0.
    int ora_first_zero_marker(const Bytes* delta, const std::uint64_t* group_begin, const std::uint64_t* group_end,
                              std::size_t groups, std::size_t domain_size, Bytes* out)
    {
        return guarded([&] {
            std::vector<Fr> s(domain_size, Fr::zero());
            for (std::size_t g = 0; g < groups; ++g)
                for (std::size_t k = group_begin[g]; k < group_end[g]; ++k)
                    if (Fr::from_le_bytes(delta + 32 * k).is_zero())
                    {
                        s[k] = Fr::one();
                        break;
                    }
            store_fr(s, out);
        });
    }

    // ---- a10: fp64 forward pass of one attention head ----------------------------------
    // gat.cpp:474-615 (attention_head_forward_impl) with matmul :366-391, matvec :394-405,
    // leaky_relu :354-357, elu :360-363.  Row-major arrays; `has_bias` mirrors
    // apply_output_bias; outputs as the fields of HeadForwardTrace.  Every loop keeps the
    // reference's order (k-ascending products, incoming sources in edge order with the node
    // itself appended when it has no self loop), so the results carry the same roundings.
    int ora_gat_head_forward(const double* features, std::size_t nodes, std::size_t inner, const double* seq_kernel, std::size_t width,
                             const double* attn_src, double bias_src, const double* attn_dst, double bias_dst, const double* out_bias,
                             std::size_t out_bias_count, int has_bias, int apply_activation, const std::uint32_t* edge_src,
                             const std::uint32_t* edge_dst, std::size_t edges, double* H_prime, double* E_src, double* E_dst, double* S, double* Z,
                             double* M, double* Delta, double* U, double* Sum, double* inv, double* alpha, double* H_agg_pre, double* H_agg)
    {
        return guarded([&] {
            auto leaky = [](double v) { return v >= 0.0 ? v : 0.2 * v; };
            for (std::size_t e = 0; e < edges; ++e)
                if (edge_src[e] >= nodes || edge_dst[e] >= nodes) throw std::runtime_error("edge out of bounds while running attention head forward");
            for (std::size_t i = 0; i < nodes * width; ++i) H_prime[i] = 0.0;
            for (std::size_t i = 0; i < nodes; ++i)
                for (std::size_t k = 0; k < inner; ++k)
                {
                    const double lhs = features[i * inner + k];
                    for (std::size_t j = 0; j < width; ++j) H_prime[i * width + j] += lhs * seq_kernel[k * width + j];
                }
            for (std::size_t i = 0; i < nodes; ++i)
            {
                E_dst[i] = bias_dst;
                E_src[i] = bias_src;
                for (std::size_t c = 0; c < width; ++c)
                {
                    E_dst[i] += H_prime[i * width + c] * attn_dst[c];
                    E_src[i] += H_prime[i * width + c] * attn_src[c];
                }
            }
            std::vector<std::vector<std::size_t>> incoming(nodes);
            for (std::size_t e = 0; e < edges; ++e) incoming[edge_dst[e]].push_back(edge_src[e]);
            for (std::size_t d = 0; d < nodes; ++d)
                if (std::find(incoming[d].begin(), incoming[d].end(), d) == incoming[d].end()) incoming[d].push_back(d);
            for (std::size_t d = 0; d < nodes; ++d)
            {
                M[d] = -std::numeric_limits<double>::infinity();
                for (const auto s : incoming[d]) M[d] = std::max(M[d], leaky(E_dst[d] + E_src[s]));
            }
            for (std::size_t d = 0; d < nodes; ++d)
            {
                Sum[d] = 0.0;
                for (const auto s : incoming[d]) Sum[d] += std::exp(leaky(E_dst[d] + E_src[s]) - M[d]);
            }
            for (std::size_t d = 0; d < nodes; ++d) inv[d] = 1.0 / Sum[d];
            for (std::size_t i = 0; i < nodes * width; ++i) H_agg_pre[i] = 0.0;
            for (std::size_t d = 0; d < nodes; ++d)
                for (const auto s : incoming[d])
                {
                    const double a = std::exp(leaky(E_dst[d] + E_src[s]) - M[d]) * inv[d];
                    for (std::size_t c = 0; c < width; ++c) H_agg_pre[d * width + c] += a * H_prime[s * width + c];
                }
            for (std::size_t e = 0; e < edges; ++e)
            {
                const std::size_t s = edge_src[e], d = edge_dst[e];
                S[e] = E_dst[d] + E_src[s];
                Z[e] = leaky(S[e]);
                Delta[e] = M[d] - Z[e];
                U[e] = std::exp(Z[e] - M[d]);
                alpha[e] = U[e] * inv[d];
            }
            for (std::size_t d = 0; d < nodes; ++d)
                for (std::size_t c = 0; c < width; ++c)
                {
                    double v = H_agg_pre[d * width + c];
                    if (has_bias && c < out_bias_count) v += out_bias[c];
                    H_agg[d * width + c] = apply_activation ? (v >= 0.0 ? v : std::expm1(v)) : v;
                }
        });
    }

    // ---- a10: witness-column leaves ---------------------------------------------------
    // trace.cpp:973-976 (quantize_float): round half away from zero at scale 16.
    int ora_quantize(const double* values, std::size_t n, std::int64_t* out)
    {
        for (std::size_t i = 0; i < n; ++i)
            out[i] = static_cast<std::int64_t>(values[i] >= 0.0 ? values[i] * 16.0 + 0.5 : values[i] * 16.0 - 0.5);
        return 0;
    }
    // trace.cpp:1366-1381 (broadcast_node_values): out[e] = node_values[idx[e]]
    // for e < edge_count, zero tail up to domain_size.
    int ora_broadcast_node_values(const Bytes* node_values, std::size_t node_count, const std::uint64_t* index,
                                  std::size_t edge_count, std::size_t domain_size, Bytes* out)
    {
        return guarded([&] {
            std::memset(out, 0, 32 * domain_size);
            for (std::size_t e = 0; e < edge_count; ++e)
            {
                if (index[e] >= node_count) throw std::runtime_error("edge endpoint out of range");
                std::memcpy(out + 32 * e, node_values + 32 * index[e], 32);
            }
        });
    }
    // trace.cpp:1916-1933 (multiplicity_from_indices).
    int ora_multiplicity_from_indices(const std::uint64_t* indices, std::size_t count, std::size_t domain_size, Bytes* out)
    {
        return guarded([&] {
            std::vector<std::uint64_t> counts(domain_size, 0);
            for (std::size_t i = 0; i < count; ++i)
            {
                if (indices[i] >= domain_size) throw std::runtime_error("lookup index out of range");
                counts[indices[i]] += 1;
            }
            for (std::size_t i = 0; i < domain_size; ++i) Fr::from_u64(counts[i]).to_le_bytes(out + 32 * i);
        });
    }
    // trace.cpp:2098-2108 (build_weighted_sum) and the query pack of
    // build_pair_lookup_artifacts (:2073): out[i] = left[i] + lambda*right[i]
    // for i < count, zero tail.
    int ora_weighted_sum(const Bytes* left, const Bytes* lambda, const Bytes* right, std::size_t count,
                         std::size_t domain_size, Bytes* out)
    {
        return guarded([&] {
            const Fr l = Fr::from_le_bytes(lambda);
            std::memset(out, 0, 32 * domain_size);
            for (std::size_t i = 0; i < count; ++i)
                (Fr::from_le_bytes(left + 32 * i) + l * Fr::from_le_bytes(right + 32 * i)).to_le_bytes(out + 32 * i);
        });
    }
    // trace.cpp:579-607 (fill_feature_lookup_rows):
    // out[row*width + c] = row_id[row] + eta_i*feature_index[c] + eta_v*features[row][c].
    int ora_feature_lookup_rows(const Bytes* row_ids, const Bytes* feature_indices, const Bytes* features,
                                std::size_t rows, std::size_t width, const Bytes* eta_index, const Bytes* eta_value,
                                Bytes* out)
    {
        return guarded([&] {
            const Fr ei = Fr::from_le_bytes(eta_index);
            const Fr ev = Fr::from_le_bytes(eta_value);
            const auto idx = load_fr(feature_indices, width);
            for (std::size_t row = 0; row < rows; ++row)
            {
                const Fr id = Fr::from_le_bytes(row_ids + 32 * row);
                for (std::size_t c = 0; c < width; ++c)
                    (id + ei * idx[c] + ev * Fr::from_le_bytes(features + 32 * (row * width + c)))
                        .to_le_bytes(out + 32 * (row * width + c));
            }
        });
    }

    // ---- a11: lazily evaluated public feature-domain columns ---------------------------
    // src/protocol/prover.cpp:224-276 (evaluate_truncated_domain_polynomial) and
    // :1341-1675 (evaluate_lazy_large_fh_public_group_points): dot products of the
    // weight vector with the generated columns 1, index / feature_count,
    // index % feature_count, absolute_ids[row], features[row][column] over the first
    // rows*feature_count entries.  out = {ones, row, col, abs, feature}.
    int ora_fh_public_eval(const Bytes* features, std::size_t rows, std::size_t feature_count, const std::uint64_t* abs_ids,
                           const Bytes* weights, Bytes* out)
    {
        return guarded([&] {
            Fr sums[5] = {Fr::zero(), Fr::zero(), Fr::zero(), Fr::zero(), Fr::zero()};
            const std::size_t valid = rows * feature_count;
            for (std::size_t index = 0; index < valid; ++index)
            {
                const Fr w = Fr::from_le_bytes(weights + 32 * index);
                const std::size_t row = index / feature_count;
                sums[0] += w;
                sums[1] += w * Fr::from_u64(row);
                sums[2] += w * Fr::from_u64(index % feature_count);
                if (abs_ids != nullptr) sums[3] += w * Fr::from_u64(abs_ids[row]);
                if (features != nullptr) sums[4] += w * Fr::from_le_bytes(features + 32 * index);
            }
            for (int i = 0; i < 5; ++i) sums[i].to_le_bytes(out + 32 * i);
        });
    }

    // ---- a5: same-base batch and group helpers (curve.cpp:81-238) -------------------
    int ora_g1_mul_same_base(const Bytes* base, const Bytes* scalars, std::size_t count, Bytes* out)
    {
        return guarded([&] {
            const G1 b = G1::from_affine(g1_from_bytes(base));
            for (std::size_t i = 0; i < count; ++i)
                g1_to_bytes(b.mul(Fr::from_le_bytes(scalars + 32 * i)).to_affine(), out + 96 * i);
        });
    }
    int ora_g1_add(const Bytes* a, const Bytes* b, Bytes* out)
    {
        return guarded([&] {
            g1_to_bytes(G1::from_affine(g1_from_bytes(a)).add(G1::from_affine(g1_from_bytes(b))).to_affine(), out);
        });
    }
    int ora_g1_on_curve(const Bytes* a)
    {
        int ok = 0;
        const int rc = guarded([&] { ok = on_curve(g1_from_bytes(a)) ? 1 : 0; });
        return rc == 0 ? ok : -1;
    }
    // Definition of an MSM: sum_i [s_i] P_i by independent scalar muls.
    int ora_g1_msm_naive(const Bytes* points, const Bytes* scalars, std::size_t count, Bytes* out)
    {
        return guarded([&] {
            G1 acc = G1::identity();
            for (std::size_t i = 0; i < count; ++i)
                acc = acc.add(G1::from_affine(g1_from_bytes(points + 96 * i)).mul(Fr::from_le_bytes(scalars + 32 * i)));
            g1_to_bytes(acc.to_affine(), out);
        });
    }

    // ---- stand-alone kernels of the sweep (no reference caller) ---------------------
    // Textbook radix-2 decimation-in-time NTT over omega_n (natural order in and out);
    // inverse uses omega^-1 and scales by 1/n; coset variants pre/post-scale by shift^i.
    int ora_ntt(Bytes* data, std::uint64_t size, int inverse, const Bytes* coset_shift)
    {
        return guarded([&] {
            auto a = load_fr(data, size);
            std::size_t log2n = 0;
            while ((1ULL << log2n) < size) ++log2n;
            if ((1ULL << log2n) != size) throw std::runtime_error("domain size must be a non-zero power of two");
            Fr shift = Fr::one();
            const bool has_shift = coset_shift != nullptr;
            if (has_shift) shift = Fr::from_le_bytes(coset_shift);
            if (has_shift && !inverse)
            {
                Fr cur = Fr::one();
                for (std::size_t i = 0; i < size; ++i)
                {
                    a[i] *= cur;
                    cur *= shift;
                }
            }
            for (std::size_t i = 0; i < size; ++i)
            {
                std::size_t j = 0;
                for (std::size_t b = 0; b < log2n; ++b) j |= ((i >> b) & 1U) << (log2n - 1 - b);
                if (i < j) std::swap(a[i], a[j]);
            }
            Fr omega = root_of_unity(size);
            if (inverse) omega = omega.inv();
            for (std::size_t len = 2; len <= size; len <<= 1)
            {
                const Fr wlen = omega.pow(static_cast<u64>(size / len));
                for (std::size_t start = 0; start < size; start += len)
                {
                    Fr w = Fr::one();
                    for (std::size_t j = 0; j < len / 2; ++j)
                    {
                        const Fr u = a[start + j];
                        const Fr v = a[start + j + len / 2] * w;
                        a[start + j] = u + v;
                        a[start + j + len / 2] = u - v;
                        w *= wlen;
                    }
                }
            }
            if (inverse)
            {
                const Fr inv_n = Fr::from_u64(size).inv();
                for (auto& v : a) v *= inv_n;
                if (has_shift)
                {
                    const Fr shift_inv = shift.inv();
                    Fr cur = Fr::one();
                    for (std::size_t i = 0; i < size; ++i)
                    {
                        a[i] *= cur;
                        cur *= shift_inv;
                    }
                }
            }
            store_fr(a, data);
        });
    }
    // Definition of the transform, O(n^2), for small sizes: out[j] = sum_i a[i] * omega^(ij).
    int ora_dft_naive(const Bytes* data, std::uint64_t size, Bytes* out)
    {
        return guarded([&] {
            const auto a = load_fr(data, size);
            const Fr omega = root_of_unity(size);
            Fr wj = Fr::one();
            for (std::size_t j = 0; j < size; ++j)
            {
                (horner(a, wj)).to_le_bytes(out + 32 * j);
                wj *= omega;
            }
        });
    }
    // Multilinear (sumcheck-style) fold of a table of 2^k entries by challenge r:
    // out[i] = t[2i] + r * (t[2i+1] - t[2i]).
    int ora_fold(const Bytes* table, std::size_t n, const Bytes* challenge, Bytes* out)
    {
        return guarded([&] {
            const Fr r = Fr::from_le_bytes(challenge);
            for (std::size_t i = 0; i < n / 2; ++i)
            {
                const Fr lo = Fr::from_le_bytes(table + 32 * (2 * i));
                const Fr hi = Fr::from_le_bytes(table + 32 * (2 * i + 1));
                (lo + r * (hi - lo)).to_le_bytes(out + 32 * i);
            }
        });
    }

    // ---- CPU baseline timing ---------------------------------------------------------
    // Times the reference's loops on values held in native (Montgomery) form, as
    // mcl::Fr holds them, so that no wire-format conversion is charged to the CPU:
    //  - packed evaluation: eval_backend.cpp:309-444 (K columns x n rows x P
    //    rotations, chunked over `threads` like its std::async fan-out);
    //  - barycentric weights: polynomial.cpp:179-315 (chunk-parallel batch inversion).
    // Inputs are seeded pseudo-random field elements generated before the clock starts.
    int ora_bench_eval(std::size_t k_count, std::size_t n, std::size_t p_count, std::size_t threads,
                       std::uint64_t seed, double* seconds, Bytes* checksum_out)
    {
        return guarded([&] {
            if (n == 0 || (n & (n - 1)) != 0) throw std::runtime_error("domain size must be a non-zero power of two");
            std::vector<Fr> values(k_count * n), w(n);
            std::uint64_t state = seed * 0x9E3779B97F4A7C15ULL + 1;
            auto next = [&]() {
                state ^= state << 13;
                state ^= state >> 7;
                state ^= state << 17;
                return state;
            };
            auto rnd = [&]() {
                Fr f;
                for (auto& limb : f.v.w) limb = next();
                f.v.w[3] >>= 2;  // < 2^254 < r: a valid residue
                return f;
            };
            for (auto& v : values) v = rnd();  // interleaved [c*K + k], as the reference packs them
            for (auto& v : w) v = rnd();
            const std::size_t mask = n - 1;
            const std::size_t used = std::max<std::size_t>(1, std::min(threads, n / 512 == 0 ? 1 : n / 512));
            std::vector<std::vector<Fr>> partials(used, std::vector<Fr>(p_count * k_count, Fr::zero()));
            const auto t0 = std::chrono::steady_clock::now();
            parallel_chunks(n, used, [&](std::size_t t, std::size_t begin, std::size_t end) {
                auto& partial = partials[t];
                for (std::size_t column = begin; column < end; ++column)
                {
                    const Fr& weight = w[column];
                    for (std::size_t p = 0; p < p_count; ++p)
                    {
                        const std::size_t rotated = (column + p) & mask;
                        const Fr* row = &values[rotated * k_count];
                        Fr* out_row = &partial[p * k_count];
                        for (std::size_t k = 0; k < k_count; ++k) out_row[k] += row[k] * weight;
                    }
                }
            });
            std::vector<Fr> total(p_count * k_count, Fr::zero());
            for (const auto& partial : partials)
                for (std::size_t i = 0; i < total.size(); ++i) total[i] += partial[i];
            const auto t1 = std::chrono::steady_clock::now();
            *seconds = std::chrono::duration<double>(t1 - t0).count();
            Fr sum = Fr::zero();
            for (const auto& v : total) sum += v;
            if (checksum_out != nullptr) sum.to_le_bytes(checksum_out);
        });
    }

    int ora_bench_bary(std::size_t n, std::size_t threads, std::uint64_t seed, double* seconds, Bytes* checksum_out)
    {
        return guarded([&] {
            const Fr x = Fr::from_u64(seed * 2654435761ULL + 12345);
            const Fr omega = root_of_unity(n);
            const Fr inv_size = Fr::from_u64(n).inv();
            std::vector<Fr> points(n);
            {
                Fr p = Fr::one();
                for (std::size_t i = 0; i < n; ++i)
                {
                    points[i] = p;
                    p *= omega;
                }
            }
            const auto t0 = std::chrono::steady_clock::now();
            const std::size_t tasks = std::max<std::size_t>(1, std::min<std::size_t>(threads, (n + (1ULL << 20) - 1) >> 20));
            std::vector<Fr> denominators(n), prefix(n), weights(n), chunk_products(tasks, Fr::one());
            const Fr zero_eval = x.pow(static_cast<u64>(n)) - Fr::one();
            parallel_chunks(n, tasks, [&](std::size_t t, std::size_t begin, std::size_t end) {
                Fr acc = Fr::one();
                for (std::size_t i = begin; i < end; ++i)
                {
                    denominators[i] = x - points[i];
                    prefix[i] = acc;
                    acc *= denominators[i];
                }
                chunk_products[t] = acc;
            });
            std::vector<Fr> cross_prefix(tasks + 1, Fr::one());
            for (std::size_t c = 0; c < tasks; ++c) cross_prefix[c + 1] = cross_prefix[c] * chunk_products[c];
            const Fr global_inv = cross_prefix[tasks].inv();
            std::vector<Fr> outer(tasks);
            Fr cross_suffix = Fr::one();
            for (std::size_t c = tasks; c-- > 0;)
            {
                outer[c] = global_inv * cross_prefix[c] * cross_suffix;
                cross_suffix *= chunk_products[c];
            }
            parallel_chunks(n, tasks, [&](std::size_t t, std::size_t begin, std::size_t end) {
                Fr running = Fr::one();
                for (std::size_t i = end; i-- > begin;)
                {
                    const Fr inv_d = outer[t] * prefix[i] * running;
                    weights[i] = zero_eval * (points[i] * inv_size) * inv_d;
                    running *= denominators[i];
                }
            });
            const auto t1 = std::chrono::steady_clock::now();
            *seconds = std::chrono::duration<double>(t1 - t0).count();
            Fr sum = Fr::zero();
            for (const auto& v : weights) sum += v;
            if (checksum_out != nullptr) sum.to_le_bytes(checksum_out);
        });
    }

    // Times one column of each builder kind on native-form values, single-threaded as the
    // reference builds them (lookup.cpp:100-157, trace.cpp:298-361, psq.cpp:7-39,
    // zkmap.cpp:7-32): seconds[0] LogUp accumulator (n rows, `valid` active), [1] route node,
    // [2] route edge, [3] segmented prefix state, [4] inner-product accumulator over `valid`
    // rows, [5] weighted column sum of a valid x 8 matrix (trace.cpp:203-271).
    int ora_bench_builders(std::size_t n, std::size_t valid, std::uint64_t seed, double* seconds, Bytes* checksum_out)
    {
        return guarded([&] {
            if (valid + 1 > n) throw std::runtime_error("valid must be below n");
            std::uint64_t state = seed * 0x9E3779B97F4A7C15ULL + 1;
            auto next = [&]() {
                state ^= state << 13;
                state ^= state >> 7;
                state ^= state << 17;
                return state;
            };
            auto rnd = [&]() {
                Fr f;
                for (auto& limb : f.v.w) limb = next();
                f.v.w[3] >>= 2;
                return f;
            };
            std::vector<Fr> table(n), query(n), mult(n), values(n), q_new(n), q_sel(n, Fr::zero());
            for (std::size_t i = 0; i < n; ++i)
            {
                table[i] = rnd();
                query[i] = rnd();
                mult[i] = Fr::from_u64(next() & 63);
                values[i] = rnd();
                q_new[i] = (next() & 7) == 0 ? Fr::one() : Fr::zero();
                if (i < valid) q_sel[i] = Fr::one();
            }
            const Fr beta = rnd();
            Fr sink = Fr::zero();
            auto clock = [] { return std::chrono::steady_clock::now(); };
            auto since = [](std::chrono::steady_clock::time_point t0) {
                return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            };
            {
                const auto t0 = clock();
                std::vector<Fr> den(2 * valid), acc(n, Fr::zero());
                for (std::size_t i = 0; i < valid; ++i)
                {
                    den[2 * i] = table[i] + beta;
                    den[2 * i + 1] = query[i] + beta;
                }
                const auto inv = batch_invert(den);
                Fr run = Fr::zero();
                for (std::size_t i = 0; i < valid; ++i)
                {
                    run += q_sel[i] * mult[i] * inv[2 * i];
                    run -= q_sel[i] * inv[2 * i + 1];
                    acc[i + 1] = run;
                }
                for (std::size_t i = valid + 1; i < n; ++i) acc[i] = acc[valid];
                seconds[0] = since(t0);
                sink += acc[n - 1];
            }
            for (int kind = 1; kind <= 2; ++kind)
            {
                const auto t0 = clock();
                std::vector<Fr> den(valid), acc(n, Fr::zero());
                for (std::size_t i = 0; i < valid; ++i) den[i] = (kind == 1 ? table[i] : query[i]) + beta;
                const auto inv = batch_invert(den);
                Fr run = Fr::zero();
                for (std::size_t i = 0; i < valid; ++i)
                {
                    run += kind == 1 ? mult[i] * inv[i] : inv[i];
                    acc[i + 1] = run;
                }
                for (std::size_t i = valid + 1; i < n; ++i) acc[i] = acc[valid];
                seconds[kind] = since(t0);
                sink += acc[n - 1];
            }
            {
                const auto t0 = clock();
                std::vector<Fr> out(n, Fr::zero());
                out[0] = values[0];
                for (std::size_t i = 1; i < n; ++i) out[i] = q_new[i] * values[i] + (Fr::one() - q_new[i]) * (out[i - 1] + values[i]);
                seconds[3] = since(t0);
                sink += out[n - 1];
            }
            {
                const auto t0 = clock();
                std::vector<Fr> acc(n, Fr::zero());
                Fr mu = Fr::zero();
                for (std::size_t i = 0; i < valid; ++i)
                {
                    mu += table[i] * query[i];
                    acc[i + 1] = mu;
                }
                for (std::size_t i = valid + 1; i < n; ++i) acc[i] = acc[valid];
                seconds[4] = since(t0);
                sink += acc[n - 1];
            }
            {
                const std::size_t rows = valid / 8 > 0 ? valid / 8 : 1;
                const auto t0 = clock();
                Fr total[8];
                for (auto& t : total) t = Fr::zero();
                for (std::size_t row = 0; row < rows; ++row)
                    for (std::size_t c = 0; c < 8; ++c) total[c] += values[row * 8 + c] * table[row];
                seconds[5] = since(t0);
                for (auto& t : total) sink += t;
            }
            if (checksum_out != nullptr) sink.to_le_bytes(checksum_out);
        });
    }

    // ---- transcript (transcript.cpp:10-55) -------------------------------------------
    std::uint64_t ora_fnv1a(const char* data, std::size_t size) { return fnv1a(std::string(data, size)); }
}
