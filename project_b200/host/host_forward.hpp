// fp64 forward pass of one attention head on the HOST, in the reference's own order of operations
// (attention_head_forward_impl, src/model/gat.cpp:474-615, with matmul :366-391, matvec :394-405,
// leaky_relu :354-357, elu :360-363): serial k-ascending products with separate multiply and add, per
// destination node its incoming sources in edge order (the node itself appended when it has no self
// loop), std::exp / std::expm1 of the host's math library.
//
// The prover flow runs the forward pass on the GPU; this restatement is its re-check: when a value of
// the GPU pass lies so close to a rounding boundary of the quantisation that a last-place difference
// of exp could flip it (gzk_quantize_guarded), the witness is recomputed here so that it is the
// reference's, bit for bit.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <limits>
#include <stdexcept>
#include <vector>

namespace gatzk_flow
{
    struct HostHeadTrace
    {
        std::vector<double> H_prime, E_src, E_dst, M, Sum, inv, S, Z, Delta, U, alpha, H_agg_pre_bias, H_agg;
    };

    inline HostHeadTrace host_head_forward(const std::vector<double>& features, std::size_t nodes, std::size_t inner,
                                           const std::vector<double>& seq_kernel, std::size_t width, const std::vector<double>& attn_src, double bias_src,
                                           const std::vector<double>& attn_dst, double bias_dst, const std::vector<double>& output_bias,
                                           bool apply_output_bias, bool apply_activation, const std::vector<std::uint32_t>& edge_src,
                                           const std::vector<std::uint32_t>& edge_dst)
    {
        const std::size_t edges = edge_src.size();
        HostHeadTrace t;
        t.H_prime.assign(nodes * width, 0.0);
        for (std::size_t i = 0; i < nodes; ++i)
            for (std::size_t k = 0; k < inner; ++k)
            {
                const double lhs = features[i * inner + k];
                for (std::size_t j = 0; j < width; ++j) t.H_prime[i * width + j] += lhs * seq_kernel[k * width + j];
            }
        t.E_src.assign(nodes, 0.0);
        t.E_dst.assign(nodes, 0.0);
        for (std::size_t i = 0; i < nodes; ++i)
        {
            double s = bias_src, d = bias_dst;  // matvec starts from the bias (gat.cpp:396-404)
            for (std::size_t c = 0; c < width; ++c)
            {
                d += t.H_prime[i * width + c] * attn_dst[c];
                s += t.H_prime[i * width + c] * attn_src[c];
            }
            t.E_src[i] = s;
            t.E_dst[i] = d;
        }
        auto leaky = [](double v) { return v >= 0.0 ? v : 0.2 * v; };
        std::vector<std::vector<std::uint32_t>> incoming(nodes);
        for (std::size_t e = 0; e < edges; ++e)
        {
            if (edge_src[e] >= nodes || edge_dst[e] >= nodes) throw std::runtime_error("edge out of bounds while running attention head forward");
            incoming[edge_dst[e]].push_back(edge_src[e]);
        }
        for (std::size_t d = 0; d < nodes; ++d)
            if (std::find(incoming[d].begin(), incoming[d].end(), static_cast<std::uint32_t>(d)) == incoming[d].end())
                incoming[d].push_back(static_cast<std::uint32_t>(d));
        t.M.assign(nodes, 0.0);
        t.Sum.assign(nodes, 0.0);
        t.inv.assign(nodes, 0.0);
        t.H_agg_pre_bias.assign(nodes * width, 0.0);
        t.H_agg.assign(nodes * width, 0.0);
        for (std::size_t d = 0; d < nodes; ++d)
        {
            double m = -std::numeric_limits<double>::infinity();
            for (const auto s : incoming[d]) m = std::max(m, leaky(t.E_dst[d] + t.E_src[s]));
            double sum = 0.0;
            for (const auto s : incoming[d]) sum += std::exp(leaky(t.E_dst[d] + t.E_src[s]) - m);
            t.M[d] = m;
            t.Sum[d] = sum;
            t.inv[d] = 1.0 / sum;
            for (const auto s : incoming[d])
            {
                const double a = std::exp(leaky(t.E_dst[d] + t.E_src[s]) - m) * t.inv[d];
                for (std::size_t c = 0; c < width; ++c) t.H_agg_pre_bias[d * width + c] += a * t.H_prime[s * width + c];
            }
        }
        t.S.assign(edges, 0.0);
        t.Z.assign(edges, 0.0);
        t.Delta.assign(edges, 0.0);
        t.U.assign(edges, 0.0);
        t.alpha.assign(edges, 0.0);
        for (std::size_t e = 0; e < edges; ++e)
        {
            const std::size_t s = edge_src[e], d = edge_dst[e];
            t.S[e] = t.E_dst[d] + t.E_src[s];
            t.Z[e] = leaky(t.S[e]);
            t.Delta[e] = t.M[d] - t.Z[e];
            t.U[e] = std::exp(t.Z[e] - t.M[d]);
            t.alpha[e] = t.U[e] * t.inv[d];
        }
        for (std::size_t d = 0; d < nodes; ++d)
            for (std::size_t c = 0; c < width; ++c)
            {
                double v = t.H_agg_pre_bias[d * width + c];
                if (apply_output_bias && c < output_bias.size()) v += output_bias[c];
                t.H_agg[d * width + c] = apply_activation ? (v >= 0.0 ? v : std::expm1(v)) : v;
            }
        return t;
    }
}
