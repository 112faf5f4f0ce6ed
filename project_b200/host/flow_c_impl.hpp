// Shared body of the C entry points of the prover flow (include/gatzk_b200_flow.h): the GPU
// build and the CPU build of the flow wrap these functions under their own symbol prefixes.
#pragma once

#include <cstdio>
#include <memory>
#include <string>

#include "../../include/gatzk_b200_flow.h"
#include "prover_flow.hpp"

namespace gatzk_flow
{
    struct FlowHandle
    {
        std::unique_ptr<Backend> backend;
        std::unique_ptr<ProverFlow> flow;
    };

    inline std::string& flow_error_slot()
    {
        thread_local std::string message;
        return message;
    }

    inline FlowInputs inputs_from_config(const gzk_flow_config& c)
    {
        FlowInputs in;
        in.node_count = c.node_count;
        in.feature_count = c.feature_count;
        in.class_count = c.class_count;
        in.features.assign(c.features, c.features + c.node_count * c.feature_count);
        in.edge_src.assign(c.edge_src, c.edge_src + c.edge_count);
        in.edge_dst.assign(c.edge_dst, c.edge_dst + c.edge_count);
        in.range_bits = c.range_bits;
        in.compact_columns = c.compact_columns != 0;
        in.seed = c.seed;
        std::memcpy(in.generator.data(), c.generator, 96);
        const double* p = c.params;
        const double* end = c.params + c.param_count;
        auto take_head = [&](std::size_t input_dim, std::size_t width) {
            if (static_cast<std::size_t>(end - p) < input_dim * width + 3 * width + 2) throw std::runtime_error("flow: parameter block too short");
            HeadParams h;
            h.seq_kernel.assign(p, p + input_dim * width);
            p += input_dim * width;
            h.attn_src.assign(p, p + width);
            p += width;
            h.attn_dst.assign(p, p + width);
            p += width;
            h.attn_src_bias = *p++;
            h.attn_dst_bias = *p++;
            h.output_bias.assign(p, p + width);
            p += width;
            return h;
        };
        std::size_t input_dim = c.feature_count;
        for (std::uint64_t l = 0; l < c.hidden_layer_count; ++l)
        {
            LayerParams layer;
            layer.input_dim = input_dim;
            layer.head_dim = c.hidden_head_dim[l];
            for (std::uint64_t h = 0; h < c.hidden_heads[l]; ++h) layer.heads.push_back(take_head(input_dim, layer.head_dim));
            input_dim = layer.head_dim * layer.heads.size();
            in.hidden_layers.push_back(std::move(layer));
        }
        in.output_layer.input_dim = input_dim;
        in.output_layer.head_dim = c.class_count;
        for (std::uint64_t h = 0; h < c.output_heads; ++h) in.output_layer.heads.push_back(take_head(input_dim, c.class_count));
        if (p != end) throw std::runtime_error("flow: parameter block longer than the model");
        return in;
    }

    template <typename Fn>
    inline int flow_guard(Fn&& fn)
    {
        try
        {
            fn();
            return 0;
        }
        catch (const std::exception& e)
        {
            flow_error_slot() = e.what();
            return 1;
        }
    }

    inline int flow_create_impl(std::unique_ptr<Backend> backend, const gzk_flow_config* config, FlowHandle** out)
    {
        return flow_guard([&] {
            if (config == nullptr || out == nullptr) throw std::runtime_error("flow: null argument");
            auto handle = std::make_unique<FlowHandle>();
            handle->backend = std::move(backend);
            handle->flow = std::make_unique<ProverFlow>(*handle->backend, inputs_from_config(*config));
            *out = handle.release();
        });
    }
    inline int flow_prove_impl(FlowHandle* h, bool inputs_resident = false)
    {
        return flow_guard([&] { h->flow->prove(inputs_resident); });
    }
    inline std::size_t copy_out(const std::string& s, char* out, std::size_t cap)
    {
        if (out != nullptr && cap > 0) std::memcpy(out, s.data(), std::min(cap, s.size()));
        return s.size();
    }
    inline std::size_t flow_dump_impl(FlowHandle* h, char* out, std::size_t cap) { return copy_out(dump_flow(*h->flow), out, cap); }
    inline std::size_t flow_proof_bytes_impl(FlowHandle* h, std::uint8_t* out, std::size_t cap)
    {
        const auto bytes = gatzk_b200::protocol::serialize_proof(h->flow->proof());
        if (out != nullptr && cap > 0) std::memcpy(out, bytes.data(), std::min(cap, bytes.size()));
        return bytes.size();
    }
    inline int flow_stats_impl(FlowHandle* h, std::uint64_t out[14])
    {
        const auto& s = h->flow->stats();
        out[0] = s.commit_barriers;
        out[1] = s.challenges;
        out[2] = s.dynamic_commitments;
        out[3] = s.opened_columns;
        static const char* names[7] = {"FH", "edge", "in", "d", "cat", "C", "N"};
        for (int i = 0; i < 7; ++i) out[4 + i] = h->flow->domain_size(names[i]);
        out[11] = h->backend->uploaded_bytes;
        out[12] = h->backend->downloaded_bytes;
        out[13] = s.guard_flags;
        return 0;
    }
    // out[0..6]: rows of each domain on which a quotient numerator does not vanish; failures (optional, up to cap
    // triples of domain index, constraint index, rows it failed on)
    inline int flow_constraint_violations_impl(FlowHandle* h, std::uint64_t out[7], std::uint64_t* failures, std::size_t cap, std::size_t* count)
    {
        return flow_guard([&] {
            std::vector<std::array<std::uint64_t, 3>> first;
            const auto bad = h->flow->constraint_violations(&first);
            for (int i = 0; i < 7; ++i) out[i] = bad[i];
            if (count != nullptr) *count = first.size();
            for (std::size_t i = 0; i < first.size() && i < cap && failures != nullptr; ++i)
                for (int j = 0; j < 3; ++j) failures[3 * i + j] = first[i][j];
        });
    }
    // the honest quotient of one domain ("FH", "edge", "in", "d", "cat", "C", "N"): see ProverFlow::honest_quotient
    inline int flow_honest_quotient_impl(FlowHandle* h, const char* domain, unsigned log2_blowup, unsigned classes, std::uint64_t out[6])
    {
        return flow_guard([&] {
            const auto report = h->flow->honest_quotient(domain, log2_blowup, classes);
            for (int i = 0; i < 6; ++i) out[i] = report[i];
        });
    }
    inline int flow_column_impl(FlowHandle* h, const char* label, int* kind, std::uint64_t* length, void* out, std::size_t cap_elements)
    {
        return flow_guard([&] {
            std::size_t len = 0;
            const ColP col = h->flow->column(label, &len);
            if (col == nullptr) throw std::runtime_error(std::string("flow: no committed column named ") + label);
            if (kind != nullptr) *kind = col->kind;
            if (length != nullptr) *length = len;
            if (out != nullptr && cap_elements > 0) h->backend->download(col, 0, std::min<std::size_t>(len, cap_elements), out);
        });
    }
    inline std::size_t flow_domain_labels_impl(FlowHandle* h, const char* domain, char* out, std::size_t cap)
    {
        std::string s;
        for (const auto& label : h->flow->domain_labels(domain)) s += label + "\n";
        return copy_out(s, out, cap);
    }
}
