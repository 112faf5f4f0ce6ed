// Second half of prover_flow.hpp (included from there): layer concatenation, output heads, the
// prove phase (quotient and opening evaluations) and the C entry points shared by the builds of the
// flow over the GPU backend and over the CPU backend.
#pragma once

namespace gatzk_flow
{
    // commit_hidden_layer_concat, trace.cpp:3076-3133
    inline void ProverFlow::commit_hidden_concat(Transcript& t, std::size_t layer_index, const ColP& concat_q, std::size_t width)
    {
        const bool final_layer = layer_index + 1 == in_.hidden_layers.size();
        const std::string suffix = final_layer ? "" : "_l" + std::to_string(layer_index);
        const std::string concat_label = "P_H_cat" + suffix, star_label = "P_H_cat_star" + suffix, cat_prefix = "P_cat" + suffix;
        const std::string xi_name = "xi_cat" + suffix, y_name = "y_cat" + suffix;
        const Domain& n = dom_.at("N");
        const Domain& cat = dom_.at("cat");
        commit_batch({matrix_item(concat_label, concat_q, n_nodes_, width)});
        absorb_dyn(t, concat_label);
        const Fe xi = challenge(t, xi_name);
        const ColP xi_powers = be_.alloc(kFrMont, cat.size);
        be_.zero(xi_powers);
        be_.powers(xi, width, xi_powers);
        const ColP star = be_.alloc(kFrMont, n_nodes_);
        be_.linear_form_rows(concat_q, n_nodes_, width, xi_powers, star);
        commit_batch({column_item(star_label, star, "N", n_nodes_)});
        absorb_dyn(t, star_label);
        const Fe y = challenge(t, y_name);
        ColP weights;
        const Binding b = build_binding(concat_q, n_nodes_, width, y, xi_powers, "cat", &weights);
        commit_batch({column_item(cat_prefix + "_a", b.a, "cat", cat.size), column_item(cat_prefix + "_b", b.b, "cat", cat.size),
                      column_item(cat_prefix + "_Acc", b.acc, "cat", cat.size)});
        const ColP out = be_.alloc(kFr, 1);
        be_.eval_device({star}, n_nodes_, n.log2n, weights, {0}, out, 0);
        Fe mu{};
        be_.download(out, 0, 1, mu.data());
        add_external(final_layer ? std::string("mu_cat") : "mu_cat_l" + std::to_string(layer_index), mu, star_label, y);
    }

    // commit_output_head, trace.cpp:3185-3650 (several output heads) / :3702-4223 (one output head, legacy labels)
    inline void ProverFlow::commit_output_head(Transcript& t, std::size_t head_index, const HeadWitness& w, const ColP& h_cat_q, std::size_t cat_width,
                                               std::vector<ColP>* y_lin_all, std::vector<ColP>* y_all)
    {
        const bool legacy = in_.output_layer.heads.size() == 1;
        const std::size_t c = in_.class_count;
        const Domain& n = dom_.at("N");
        const std::string k = std::to_string(head_index);
        const std::string base = legacy ? "P_out" : "P_out" + k, prefix = base + "_";
        const std::string y_lin_label = legacy ? "P_Y_lin" : "P_Y_lin_o" + k, y_label = legacy ? "P_Y" : "P_Y_o" + k;
        const std::string v_base = legacy ? "V_out" : "V_out" + k;
        auto cname = [&](const std::string& name) { return legacy ? name : name + "_o" + k; };

        // quantize_output_witness_cpu: y_lin = quantised pre-bias aggregate, y = y_lin + quantised bias
        const ColP y_prime = w.h_prime, y_lin = w.h_agg_pre;
        ColP y = y_lin;
        const auto& bias = in_.output_layer.heads[head_index].output_bias;
        if (!bias.empty())
        {
            // the quantised bias under every row: one row uploaded, repeated on the backend
            std::vector<std::int64_t> row(c, 0);
            for (std::size_t j = 0; j < c && j < bias.size(); ++j) row[j] = quantize_value(bias[j]);
            const ColP rep = be_.alloc(kI64, n_nodes_ * c);
            be_.copy_block(upload_i64(row), 0, 0, rep, 0, c, n_nodes_, c);
            y = be_.alloc(kFrMont, n_nodes_ * c);
            be_.linear_combination({y_lin, rep}, {fe_u64(1), fe_u64(1)}, n_nodes_ * c, n_nodes_ * c, y);
        }
        y_lin_all->push_back(y_lin);
        y_all->push_back(y);

        commit_batch({matrix_item(prefix + "Y_prime", y_prime, n_nodes_, c), column_item(prefix + "E_src", w.e_src, "N", n_nodes_),
                      column_item(prefix + "E_dst", w.e_dst, "N", n_nodes_), column_item(prefix + "S", w.s, "edge", n_edges_),
                      column_item(prefix + "Z", w.z, "edge", n_edges_), column_item(prefix + "M", w.m, "N", n_nodes_),
                      column_item(prefix + "M_edge", w.m_edge, "edge", es_), column_item(prefix + "Delta", w.delta, "edge", n_edges_),
                      column_item(prefix + "U", w.u, "edge", n_edges_), column_item(prefix + "Sum", w.sum, "N", n_nodes_),
                      column_item(prefix + "Sum_edge", w.sum_edge, "edge", es_), column_item(prefix + "inv", w.inv, "N", n_nodes_),
                      column_item(prefix + "inv_edge", w.inv_edge, "edge", es_), column_item(prefix + "alpha", w.alpha, "edge", n_edges_),
                      matrix_item(y_lin_label, y_lin, n_nodes_, c), matrix_item(y_label, y, n_nodes_, c)});

        absorb_dyn(t, "P_H_cat");
        absorb_dyn(t, prefix + "Y_prime");
        absorb_static(t, v_base + "_W");
        const Fe y_proj = challenge(t, cname("y_proj_out"));
        const Fe xi = challenge(t, cname("xi_out"));
        absorb_dyn(t, prefix + "Y_prime");
        absorb_dyn(t, prefix + "E_src");
        absorb_static(t, v_base + "_a_src");
        const Fe y_src = challenge(t, cname("y_src_out"));
        absorb_dyn(t, prefix + "Y_prime");
        absorb_dyn(t, prefix + "E_dst");
        absorb_static(t, v_base + "_a_dst");
        const Fe y_dst = challenge(t, cname("y_dst_out"));
        absorb_dyn(t, prefix + "S");
        absorb_dyn(t, prefix + "Z");
        absorb_static(t, "V_T_L_x");
        absorb_static(t, "V_T_L_y");
        const Fe eta_l = challenge(t, cname("eta_L_out"));
        const Fe beta_l = challenge(t, cname("beta_L_out"));
        absorb_dyn(t, prefix + "M");
        absorb_dyn(t, prefix + "M_edge");
        absorb_dyn(t, prefix + "Delta");
        absorb_static(t, "V_T_range");
        const Fe beta_r = challenge(t, cname("beta_R_out"));
        absorb_dyn(t, prefix + "Delta");
        absorb_dyn(t, prefix + "U");
        absorb_static(t, "V_T_exp_x");
        absorb_static(t, "V_T_exp_y");
        const Fe eta_exp = challenge(t, cname("eta_exp_out"));
        const Fe beta_exp = challenge(t, cname("beta_exp_out"));

        // cached_output_compressed_trace, trace.cpp:1694-1731
        const Domain& cd = dom_.at("C");
        const ColP xi_powers = be_.alloc(kFrMont, cd.size);
        be_.zero(xi_powers);
        be_.powers(xi, c, xi_powers);
        auto compress = [&](const ColP& matrix) {
            const ColP out = be_.alloc(kFrMont, n_nodes_);
            be_.linear_form_rows(matrix, n_nodes_, c, xi_powers, out);
            return out;
        };
        auto to_edges = [&](const ColP& node_values, const ColP& index) {
            const ColP out = be_.alloc(kFrMont, es_);
            be_.gather(node_values, n_nodes_, index, n_edges_, es_, out);
            return out;
        };
        const ColP y_prime_star = compress(y_prime), y_star = compress(y_lin);
        const ColP y_prime_star_edge = to_edges(y_prime_star, src_u32_), y_star_edge = to_edges(y_star, dst_u32_);
        const Fe eta_src = challenge(t, cname("eta_src_out"));
        const Fe beta_src = challenge(t, cname("beta_src_out"));
        const Route src_route = build_route({ids_i64_, w.e_src}, {src_i64_, y_prime_star_edge}, eta_src, src_multiplicity_, beta_src);

        const std::size_t lrelu_size = lrelu_bound_ * 2 + 1;
        const Lookup lrelu = build_pair_lookup(t_l_x_, t_l_y_, lrelu_size, -static_cast<std::int64_t>(lrelu_bound_), 1, w.s, w.z, n_edges_, eta_l,
                                               beta_l, q_tbl_l_, q_qry_l_);
        const ColP s_max = be_.alloc(kU32, es_);
        be_.first_zero_marker(w.delta, group_begin_, group_end_, groups_, es_, s_max);
        const ColP c_max = be_.alloc(kFrMont, es_);
        queue_scan(ScanJob::kGroupPrefix, s_max, q_new_, nullptr, nullptr, nullptr, es_, es_, Fe{}, c_max);
        const Lookup range = build_pair_lookup(t_range_, nullptr, range_size_, 0, 1, w.delta, nullptr, n_edges_, fe_u64(0), beta_r, q_tbl_r_, q_qry_r_);
        const Lookup exp_l = build_pair_lookup(t_exp_x_, t_exp_y_, range_size_ * 5, 0, 5, w.delta, w.u, n_edges_, eta_exp, beta_exp, q_tbl_exp_, q_qry_exp_);

        const Fe lambda = challenge(t, cname("lambda_out"));
        const ColP widehat = be_.alloc(kFrMont, es_);
        be_.mul_columns(w.alpha, y_prime_star_edge, n_edges_, es_, widehat);
        const ColP w_out = be_.alloc(kFrMont, es_);
        be_.linear_combination({w.u, widehat}, {fe_u64(1), lambda}, es_, es_, w_out);
        const ColP t_out = be_.alloc(kFrMont, n_nodes_);
        be_.linear_combination({w.sum, y_star}, {fe_u64(1), lambda}, n_nodes_, n_nodes_, t_out);
        const ColP t_out_edge = to_edges(t_out, dst_u32_);
        const ColP psq = be_.alloc(kFrMont, es_);
        queue_scan(ScanJob::kGroupPrefix, w_out, q_new_, nullptr, nullptr, nullptr, es_, es_, Fe{}, psq);

        commit_batch({column_item(prefix + "E_src_edge", w.e_src_edge, "edge", es_), column_item(prefix + "E_dst_edge", w.e_dst_edge, "edge", es_),
                      column_item(prefix + "Y_prime_star", y_prime_star, "N", n_nodes_),
                      column_item(prefix + "Y_prime_star_edge", y_prime_star_edge, "edge", es_),
                      column_item(prefix + "Table_src", src_route.table, "N", n.size), column_item(prefix + "Query_src", src_route.query, "edge", es_),
                      column_item(prefix + "m_src", src_multiplicity_, "N", n.size), column_item(prefix + "R_src_node", src_route.node_acc, "N", n.size),
                      tail_item(prefix + "R_src", src_route.edge_acc, "edge", es_), packed_item(prefix + "Table_L", lrelu.table, lrelu.table_store, lrelu, "V_T_L_x", "V_T_L_y"),
                      packed_item(prefix + "Query_L", lrelu.query, lrelu.store, lrelu, prefix + "S", prefix + "Z"), column_item(prefix + "m_L", lrelu.multiplicity, "edge", lrelu.table_store),
                      tail_item(prefix + "R_L", lrelu.acc, "edge", lrelu.store), column_item(prefix + "s_max", s_max, "edge", es_),
                      tail_item(prefix + "C_max", c_max, "edge", es_), packed_item(prefix + "Table_R", range.table, range.table_store, range, "V_T_range", ""),
                      packed_item(prefix + "Query_R", range.query, range.store, range, prefix + "Delta", ""), column_item(prefix + "m_R", range.multiplicity, "edge", range.table_store),
                      tail_item(prefix + "R_R", range.acc, "edge", range.store), packed_item(prefix + "Table_exp", exp_l.table, exp_l.table_store, exp_l, "V_T_exp_x", "V_T_exp_y"),
                      packed_item(prefix + "Query_exp", exp_l.query, exp_l.store, exp_l, prefix + "Delta", prefix + "U"), column_item(prefix + "m_exp", exp_l.multiplicity, "edge", exp_l.table_store),
                      tail_item(prefix + "R_exp", exp_l.acc, "edge", exp_l.store), column_item(prefix + "widehat_y_star", widehat, "edge", es_),
                      column_item(prefix + "w", w_out, "edge", es_), column_item(prefix + "T", t_out, "N", n_nodes_),
                      column_item(prefix + "T_edge", t_out_edge, "edge", es_), tail_item(prefix + "PSQ", psq, "edge", es_),
                      column_item(prefix + "Y_star", y_star, "N", n_nodes_), column_item(prefix + "Y_star_edge", y_star_edge, "edge", es_)});

        absorb_dyn(t, prefix + "T");
        absorb_dyn(t, prefix + "T_edge");
        const Fe eta_t = challenge(t, cname("eta_t_out"));
        const Fe beta_t = challenge(t, cname("beta_t_out"));
        const Route t_route = build_route({ids_i64_, t_out}, {dst_i64_, t_out_edge}, eta_t, dst_multiplicity_, beta_t);
        absorb_dyn(t, y_label);
        absorb_dyn(t, prefix + "Y_star");
        const Fe y_out_star = challenge(t, cname("y_out_star"));

        const ColP y_proj_powers = be_.alloc(kFrMont, std::max<std::size_t>(1, c));
        be_.powers(y_proj, c, y_proj_powers);
        const ColP proj_b = be_.alloc(kFrMont, dom_.at("cat").size);
        be_.zero(proj_b);
        be_.linear_form_rows(param_matrices_.at(v_base + "_W"), cat_width, c, y_proj_powers, proj_b);
        ColP w_src, w_dst, w_star;
        const std::vector<ColP> stage_weights = node_weights_at({y_proj, y_src, y_dst, y_out_star});
        const Binding proj = build_binding(h_cat_q, n_nodes_, cat_width, y_proj, proj_b, "cat", nullptr, stage_weights[0]);
        const Binding src_b =
            build_binding(y_prime, n_nodes_, c, y_src, upload_fe(param_vectors_.at(v_base + "_a_src"), cd.size), "C", &w_src, stage_weights[1]);
        const Binding dst_b =
            build_binding(y_prime, n_nodes_, c, y_dst, upload_fe(param_vectors_.at(v_base + "_a_dst"), cd.size), "C", &w_dst, stage_weights[2]);
        const Binding y_b = build_binding(y_lin, n_nodes_, c, y_out_star, xi_powers, "C", &w_star, stage_weights[3]);
        const Fe eta_dst = challenge(t, cname("eta_dst_out"));
        const Fe beta_dst = challenge(t, cname("beta_dst_out"));
        const Route dst_route = build_route({ids_i64_, w.e_dst, w.m, w.sum, w.inv, y_star},
                                            {dst_i64_, w.e_dst_edge, w.m_edge, w.sum_edge, w.inv_edge, y_star_edge}, eta_dst, dst_multiplicity_, beta_dst);
        const std::size_t dc = cd.size, dcat = dom_.at("cat").size;
        commit_batch({column_item(prefix + "Table_t", t_route.table, "N", n.size), column_item(prefix + "Query_t", t_route.query, "edge", es_),
                      column_item(prefix + "m_t", dst_multiplicity_, "N", n.size), column_item(prefix + "R_t_node", t_route.node_acc, "N", n.size),
                      tail_item(prefix + "R_t", t_route.edge_acc, "edge", es_), column_item(prefix + "a_proj", proj.a, "cat", dcat),
                      column_item(prefix + "b_proj", proj.b, "cat", dcat), column_item(prefix + "Acc_proj", proj.acc, "cat", dcat),
                      column_item(prefix + "a_src", src_b.a, "C", dc), column_item(prefix + "b_src", src_b.b, "C", dc),
                      column_item(prefix + "Acc_src", src_b.acc, "C", dc), column_item(prefix + "a_dst", dst_b.a, "C", dc),
                      column_item(prefix + "b_dst", dst_b.b, "C", dc), column_item(prefix + "Acc_dst", dst_b.acc, "C", dc),
                      column_item(prefix + "a_y", y_b.a, "C", dc), column_item(prefix + "b_y", y_b.b, "C", dc),
                      column_item(prefix + "Acc_y", y_b.acc, "C", dc), column_item(prefix + "Table_dst", dst_route.table, "N", n.size),
                      column_item(prefix + "Query_dst", dst_route.query, "edge", es_), column_item(prefix + "m_dst", dst_multiplicity_, "N", n.size),
                      column_item(prefix + "R_dst_node", dst_route.node_acc, "N", n.size), tail_item(prefix + "R_dst", dst_route.edge_acc, "edge", es_)});

        const std::string s_suffix = legacy ? "_out" : "_out" + k;
        pending_totals_.push_back({"S_src" + s_suffix, src_route.node_acc, n_nodes_});
        pending_totals_.push_back({"S_dst" + s_suffix, dst_route.node_acc, n_nodes_});
        pending_totals_.push_back({"S_t" + s_suffix, t_route.node_acc, n_nodes_});
        resolve_totals();
        {
            const ColP out = be_.alloc(kFr, 4);
            be_.horner_device(y_prime, n_nodes_, c, y_proj, out, 0);
            be_.eval_device({w.e_src}, n_nodes_, n.log2n, w_src, {0}, out, 1);
            be_.eval_device({w.e_dst}, n_nodes_, n.log2n, w_dst, {0}, out, 2);
            be_.eval_device({y_star}, n_nodes_, n.log2n, w_star, {0}, out, 3);
            Fe mu[4];
            be_.download(out, 0, 4, mu);
            const char* names[4] = {"proj", "src", "dst", "star"};
            const std::string labels[4] = {prefix + "Y_prime", prefix + "E_src", prefix + "E_dst", prefix + "Y_star"};
            const Fe points[4] = {y_proj, y_src, y_dst, y_out_star};
            for (int i = 0; i < 4; ++i) add_external(legacy ? std::string("mu_out_") + names[i] : "mu_out" + k + "_" + names[i], mu[i], labels[i], points[i]);
        }
    }

    // model::forward_note_style (src/model/gat.cpp:1141-1220) + the quantisation of every head
    inline void ProverFlow::forward_all(bool inputs_resident, bool on_host, std::vector<std::vector<HeadWitness>>& hidden_witness,
                                        std::vector<ColP>& concat_q, std::vector<HeadWitness>& output_witness, std::size_t& final_width)
    {
        hidden_witness.assign(in_.hidden_layers.size(), {});
        concat_q.assign(in_.hidden_layers.size(), nullptr);
        output_witness.clear();
        layer_inputs_q_.clear();
        ColP layer_input = on_host ? nullptr : (inputs_resident ? features_f64_ : upload_f64(in_.features));
        std::vector<double> host_input = on_host ? in_.features : std::vector<double>{};
        std::size_t input_dim = in_.feature_count;
        for (std::size_t li = 0; li < in_.hidden_layers.size(); ++li)
        {
            const auto& layer = in_.hidden_layers[li];
            const std::size_t width = layer.head_dim * layer.heads.size();
            const ColP concat = be_.alloc(kF64, n_nodes_ * width);
            std::vector<double> host_concat(on_host ? n_nodes_ * width : 0);
            for (std::size_t hi = 0; hi < layer.heads.size(); ++hi)
            {
                std::vector<double> head_out;
                hidden_witness[li].push_back(run_head(layer_input, input_dim, layer.head_dim, layer.heads[hi], false, on_host ? &host_input : nullptr,
                                                      on_host ? &head_out : nullptr));
                be_.copy_block(hidden_witness[li].back().h_agg_f64, 0, layer.head_dim, concat, hi * layer.head_dim, width, n_nodes_, layer.head_dim);
                if (on_host)  // concatenate_columns
                    for (std::size_t r = 0; r < n_nodes_; ++r)
                        for (std::size_t c = 0; c < layer.head_dim; ++c) host_concat[r * width + hi * layer.head_dim + c] = head_out[r * layer.head_dim + c];
            }
            concat_q[li] = be_.alloc(kI64, n_nodes_ * width);
            if (on_host)
                be_.quantize(concat, n_nodes_ * width, concat_q[li]);
            else
                be_.quantize_guarded(concat, n_nodes_ * width, kQuantizeGuard, concat_q[li], guard_counter_);
            layer_inputs_q_[li + 1] = concat_q[li];
            layer_input = concat;
            host_input.swap(host_concat);
            input_dim = width;
        }
        for (const auto& head : in_.output_layer.heads)
            output_witness.push_back(run_head(layer_input, input_dim, in_.class_count, head, true, on_host ? &host_input : nullptr, nullptr));
        final_width = input_dim;
    }

    inline void ProverFlow::prove(bool inputs_resident)
    {
        be_.uploaded_bytes = 0;
        be_.downloaded_bytes = 0;
        commitments_.clear();
        commitment_order_.clear();
        columns_.clear();
        opened_.clear();
        challenges_.clear();
        challenge_log_.clear();
        tau_eval_log_.clear();
        quotient_log_.clear();
        external_evaluations_.clear();
        external_sources_.clear();
        witness_scalars_.clear();
        layer_inputs_q_.clear();
        stats_ = FlowStats{};
        proof_ = gatzk_b200::protocol::Proof{};
        Transcript t("gatzkml");

        // ---- build_multihead_trace: P_H, metadata, feature lookup (trace.cpp:2173-2315) -------------
        commit_batch({matrix_item("P_H", features_q_, n_nodes_, in_.feature_count)});
        const std::size_t hidden_head_count = [&] {
            std::size_t c = 0;
            for (const auto& l : in_.hidden_layers) c += l.heads.size();
            return c;
        }();
        {
            auto& m = proof_.public_metadata;  // canonical_public_metadata, challenges.cpp:313-367
            std::string hidden_profile, d_in_profile;
            std::size_t d_h = 0, d_cat = 0;
            for (std::size_t i = 0; i < in_.hidden_layers.size(); ++i)
            {
                const auto& l = in_.hidden_layers[i];
                hidden_profile += (i ? "," : "") + std::to_string(l.heads.size()) + "x" + std::to_string(l.head_dim);
                d_in_profile += (i ? "," : "") + std::to_string(l.input_dim);
                d_h = std::max(d_h, l.head_dim);
                d_cat = std::max(d_cat, l.head_dim * l.heads.size());
            }
            d_in_profile += (d_in_profile.empty() ? "" : ",") + std::to_string(in_.output_layer.input_dim);
            m.protocol_id = "gatzkml";
            m.dataset_name = in_.dataset_name;
            m.task_type = "transductive_node_classification";
            m.report_unit = "node";
            m.graph_count = "1";
            m.L = std::to_string(in_.hidden_layers.size() + 1);
            m.hidden_profile = hidden_profile;
            m.d_in_profile = d_in_profile;
            m.K_out = std::to_string(in_.output_layer.heads.size());
            m.C = std::to_string(in_.class_count);
            m.batching_rule = "whole_graph_single";
            m.subgraph_rule = "whole_graph";
            m.self_loop_rule = "per_node_self_loop";
            m.edge_sort_rule = "edge_gid_then_dst_stable";
            m.chunking_rule = "none";
            m.model_arch_id = "L=" + m.L + "|hidden=" + m.hidden_profile + "|K_out=" + m.K_out + "|C=" + m.C;
            m.model_param_id = "synthetic_seed:" + std::to_string(in_.seed);
            m.static_table_id = "tables:lrelu+elu+exp+range";
            m.quant_cfg_id = "range_bits=" + std::to_string(in_.range_bits);
            auto dn = [&](const char* key, const char* name) { return std::string(key) + "=" + name + ":" + std::to_string(dom_.at(name).size); };
            m.domain_cfg = dn("FH", "FH") + "," + dn("edge", "edge") + "," + dn("in", "in") + "," + dn("d_h", "d") + "," + dn("cat", "cat") + "," + dn("C", "C") +
                           "," + dn("N", "N");
            m.dim_cfg = "N=" + std::to_string(n_nodes_) + ",E=" + std::to_string(n_edges_) + ",d_in=" + std::to_string(in_.feature_count) +
                        ",d_h=" + std::to_string(d_h) + ",d_cat=" + std::to_string(d_cat) + ",C=" + std::to_string(in_.class_count);
            m.encoding_id = "project-fixed-order-v1";
            m.padding_rule_id = "zero-pad+selector-mask";
            m.degree_bound_id = "note-target:FH,edge,in,d_h,cat,C,N";
            static const char* keys[24] = {"protocol_id",   "dataset_name",  "task_type",      "report_unit",   "graph_count",   "L",
                                           "hidden_profile", "d_in_profile", "K_out",          "C",             "batching_rule", "subgraph_rule",
                                           "self_loop_rule", "edge_sort_rule", "chunking_rule", "model_arch_id", "model_param_id", "static_table_id",
                                           "quant_cfg_id",  "domain_cfg",    "dim_cfg",        "encoding_id",   "padding_rule_id", "degree_bound_id"};
            const auto fields = m.fields();
            for (int i = 0; i < 24; ++i)  // absorb_public_metadata, challenges.cpp:369-394
            {
                const std::string label = std::string("M_pub.") + keys[i];
                t.absorb_scalar(label, fe_u64(Transcript::fnv1a(label + "=" + *fields[i])));
            }
            t.absorb_scalar("N", fe_u64(n_nodes_));
            t.absorb_scalar("E", fe_u64(n_edges_));
            t.absorb_scalar("d_in", fe_u64(in_.feature_count));
            t.absorb_scalar("d_h", fe_u64(d_h));
            t.absorb_scalar("d_cat", fe_u64(d_cat));
            t.absorb_scalar("C", fe_u64(in_.class_count));
            t.absorb_scalar("B", fe_u64(in_.range_bits));
        }
        for (const char* label : {"P_I", "P_src", "P_dst", "P_Q_new_edge", "P_Q_end_edge", "P_Q_edge_valid", "P_Q_N", "P_Q_proj_valid", "P_Q_d_valid",
                                  "P_Q_cat_valid", "P_Q_C_valid"})
            absorb_static(t, label);
        absorb_dyn(t, "P_H");
        absorb_static(t, "V_T_H");
        const Fe eta_feat = challenge(t, "eta_feat");
        challenge(t, "beta_feat");
        {
            // lazy full-feature lookup of a whole-graph run (trace.cpp:2209-2232): the four commitments are
            // combinations of public / static tau-evaluations; fh_public_tau_ = {1, row, col, abs id, feature}
            const Fe eta_i = eta_feat, eta_v = mul(eta_feat, eta_feat);
            const Fe table_tau = add(add(fh_public_tau_[1], mul(eta_i, fh_public_tau_[2])), mul(eta_v, static_commitments_.at("V_T_H").tau_evaluation));
            const Fe query_tau = add(add(fh_public_tau_[3], mul(eta_i, fh_public_tau_[2])), mul(eta_v, commitments_.at("P_H").tau_evaluation));
            const std::vector<std::pair<std::string, Fe>> lazy = {
                {"P_Table_feat", table_tau}, {"P_Query_feat", query_tau}, {"P_m_feat", fh_public_tau_[0]}, {"P_R_feat", fe_u64(0)}};
            std::vector<Fe> scalars;
            for (const auto& item : lazy) scalars.push_back(item.second);
            const ColP s = upload_fe(scalars, scalars.size());
            const ColP p = be_.alloc(kG1, scalars.size());
            be_.g1_fixed_base(in_.generator, s, scalars.size(), p);
            std::vector<G1> pts(scalars.size());
            be_.download(p, 0, scalars.size(), pts.data());
            for (std::size_t i = 0; i < lazy.size(); ++i)
            {
                commitments_[lazy[i].first] = Commitment{pts[i], lazy[i].second};
                commitment_order_.push_back(lazy[i].first);
                tau_eval_log_.push_back(lazy[i]);
            }
            stats_.dynamic_commitments += lazy.size();
        }

        // ---- forward pass + quantised witness (cached_forward_artifacts, trace.cpp:1281-1349) ------------
        // On the backend first; if any value lies within the guard band of a rounding boundary, once more on
        // the host with the reference's loop, so that the quantised witness is the reference's bit for bit.
        std::vector<std::vector<HeadWitness>> hidden_witness;
        std::vector<ColP> concat_q;
        std::vector<HeadWitness> output_witness;
        std::size_t input_dim = in_.feature_count;
        guard_counter_ = be_.alloc(kU32, 1);
        be_.zero(guard_counter_);
        forward_all(inputs_resident, false, hidden_witness, concat_q, output_witness, input_dim);
        {
            std::uint32_t flagged = 0;
            be_.download(guard_counter_, 0, 1, &flagged);
            stats_.guard_flags = flagged;
            if (flagged != 0) forward_all(inputs_resident, true, hidden_witness, concat_q, output_witness, input_dim);
        }

        // ---- commit chain: heads in transcript order -----------------------------------------------------
        std::size_t global_head = 0;
        for (std::size_t li = 0; li < in_.hidden_layers.size(); ++li)
        {
            for (std::size_t hi = 0; hi < in_.hidden_layers[li].heads.size(); ++hi, ++global_head)
                commit_hidden_head(t, global_head, li, hi, hidden_witness[li][hi]);
            commit_hidden_concat(t, li, concat_q[li], in_.hidden_layers[li].head_dim * in_.hidden_layers[li].heads.size());
        }
        (void)hidden_head_count;
        std::vector<ColP> y_lin_all, y_all;
        const std::size_t cat_width = input_dim;
        const ColP h_cat_q = concat_q.empty() ? features_q_ : concat_q.back();
        for (std::size_t k = 0; k < output_witness.size(); ++k) commit_output_head(t, k, output_witness[k], h_cat_q, cat_width, &y_lin_all, &y_all);
        const bool legacy = output_witness.size() == 1;
        const std::size_t nc = n_nodes_ * in_.class_count;
        ColP y_lin_avg = y_lin_all.front(), y_avg = y_all.front();
        if (!legacy)
        {
            // average_field_matrices (trace.cpp:994-1018): sum of the heads times 1/K in the field
            const Fe inv_k = inv(fe_u64(output_witness.size()));
            const std::vector<Fe> coeff(output_witness.size(), inv_k);
            y_lin_avg = be_.alloc(kFrMont, nc);
            y_avg = be_.alloc(kFrMont, nc);
            be_.linear_combination(y_lin_all, coeff, nc, nc, y_lin_avg);
            be_.linear_combination(y_all, coeff, nc, nc, y_avg);
            commit_batch({matrix_item("P_Y_lin", y_lin_avg, n_nodes_, in_.class_count), matrix_item("P_Y", y_avg, n_nodes_, in_.class_count)});
            for (std::size_t k = 0; k < output_witness.size(); ++k)
            {
                const std::string ks = std::to_string(k), prefix = "P_out" + ks + "_";
                absorb_dyn(t, "P_Y_lin_o" + ks);
                absorb_dyn(t, "P_Y_o" + ks);
                absorb_dyn(t, prefix + "Y_star");
                absorb_dyn(t, prefix + "Table_dst");
                absorb_dyn(t, prefix + "Query_dst");
            }
        }
        else
        {
            absorb_dyn(t, "P_out_Y_star");
            absorb_dyn(t, "P_out_Table_dst");
            absorb_dyn(t, "P_out_Query_dst");
        }
        absorb_dyn(t, "P_Y_lin");
        absorb_dyn(t, "P_Y");
        const Fe y_out = challenge(t, "y_out");
        {
            const std::size_t heads = legacy ? 0 : output_witness.size();
            const ColP out = be_.alloc(kFr, 2 * heads + 2);
            for (std::size_t k = 0; k < heads; ++k)
            {
                be_.horner_device(y_lin_all[k], n_nodes_, in_.class_count, y_out, out, 2 * k);
                be_.horner_device(y_all[k], n_nodes_, in_.class_count, y_out, out, 2 * k + 1);
            }
            be_.horner_device(y_lin_avg, n_nodes_, in_.class_count, y_out, out, 2 * heads);
            be_.horner_device(y_avg, n_nodes_, in_.class_count, y_out, out, 2 * heads + 1);
            std::vector<Fe> mu(2 * heads + 2);
            be_.download(out, 0, mu.size(), mu.data());
            for (std::size_t k = 0; k < heads; ++k)
            {
                add_external("mu_out" + std::to_string(k) + "_y_lin", mu[2 * k], "P_Y_lin_o" + std::to_string(k), y_out);
                add_external("mu_out" + std::to_string(k) + "_y", mu[2 * k + 1], "P_Y_o" + std::to_string(k), y_out);
            }
            add_external("mu_Y_lin", mu[2 * heads], "P_Y_lin", y_out);
            add_external("mu_out", mu[2 * heads + 1], "P_Y", y_out);
        }
        prove_openings(t);
    }

    // prove (multi-head branch), src/protocol/prover.cpp:3056-3398: evaluation of every opened column of
    // every domain at {tau, omega*tau}, seven quotient commitments, fresh weights at the opening
    // challenges, evaluation at {z, omega*z}, the opening witnesses (KZG::open_batch, src/crypto/kzg.cpp:544-577)
    // and the folded external opening (kzg.cpp:619-633).
    inline void ProverFlow::prove_openings(Transcript& t)
    {
        challenge(t, "alpha_quot");  // read back by name where the numerators are formed
        static const char* kDomains[7] = {"FH", "edge", "in", "d", "cat", "C", "N"};
        static const char* kBundles[7] = {"FH", "edge", "in", "d_h", "cat", "C", "N"};
        // All columns of a domain evaluated at two points (the point of `weights` and omega times it): grouped
        // by stored length, one result buffer.  With at_tau the point is tau itself: the first value of every
        // column is the evaluation its commitment was made from, and the key-dependent columns' values at
        // omega*tau are computed once per context, so only rotation 1 of the witness columns is evaluated.
        // `rotations` lists the points as powers of omega times the point of `weights` (one or two of them).
        // `only_rotated`: just the columns a quotient numerator reads at omega*x (rotated_labels) are evaluated;
        // at tau the others still get their first value, the evaluation their commitment was made from.
        auto evaluate_domain = [&](const std::string& domain, const ColP& weights, bool at_tau, const std::vector<std::uint64_t>& rotations, bool only_rotated,
                                   std::map<std::string, std::array<Fe, 2>>& out) {
            const auto it = opened_.find(domain);
            std::vector<std::string> labels = it == opened_.end() ? std::vector<std::string>{} : it->second;
            std::vector<std::string> wanted_list = only_rotated ? rotated_labels(domain) : std::vector<std::string>{};
            const std::set<std::string> wanted(wanted_list.begin(), wanted_list.end());
            if (only_rotated)
            {
                std::vector<std::string> kept;
                for (const auto& label : labels)
                {
                    if (wanted.count(label) != 0)
                        kept.push_back(label);
                    else if (at_tau)
                        out[label] = {commitments_.at(label).tau_evaluation, fe_u64(0)};
                }
                labels.swap(kept);
            }
            for (const auto& item : static_columns_)
            {
                if (item.second.domain != domain) continue;
                const auto cached = static_omega_tau_.find(item.first);
                if (only_rotated && wanted.count(item.first) == 0)
                {
                    if (at_tau) out[item.first] = {static_commitments_.at(item.first).tau_evaluation, fe_u64(0)};
                }
                else if (at_tau && cached != static_omega_tau_.end())
                    out[item.first] = {static_commitments_.at(item.first).tau_evaluation, cached->second};
                else
                    labels.push_back(item.first);
            }
            // combinations of other opened columns are not evaluated: their values follow from those
            std::vector<std::string> derived;
            {
                std::vector<std::string> evaluated;
                for (const auto& label : labels)
                {
                    const auto c = columns_.find(label);
                    (c != columns_.end() && !c->second.derived_from.empty() ? derived : evaluated).push_back(label);
                }
                labels.swap(evaluated);
            }
            auto finish_derived = [&]() {
                for (const auto& label : derived)
                {
                    std::array<Fe, 2> value = {fe_u64(0), fe_u64(0)};
                    for (const auto& term : columns_.at(label).derived_from)
                        for (int r = 0; r < 2; ++r) value[r] = add(value[r], mul(term.second, out.at(term.first)[r]));
                    out[label] = value;
                }
            };
            if (labels.empty())
            {
                finish_derived();
                return;
            }
            const Domain& d = dom_.at(domain);
            const std::size_t points = rotations.size();
            std::map<std::size_t, std::vector<std::string>> by_length;
            for (const auto& label : labels)
            {
                const auto c = columns_.find(label);
                by_length[c != columns_.end() ? c->second.length : static_columns_.at(label).length].push_back(label);
            }
            const ColP result = be_.alloc(kFr, points * labels.size());
            std::size_t offset = 0;
            struct Placed
            {
                std::size_t offset;
                const std::vector<std::string>* labels;
                std::size_t ones;  // first slot of the ones column of this length, or npos
            };
            constexpr std::size_t npos = static_cast<std::size_t>(-1);
            std::vector<Placed> placed;
            std::size_t tail_groups = 0;
            for (const auto& group : by_length)
                for (const auto& label : group.second)
                {
                    const auto c = columns_.find(label);
                    if (c != columns_.end() && c->second.const_tail)
                    {
                        ++tail_groups;
                        break;
                    }
                }
            const ColP ones_out = tail_groups == 0 ? nullptr : be_.alloc(kFr, points * tail_groups);
            std::size_t ones_next = 0;
            for (const auto& group : by_length)
            {
                std::vector<ColP> cols;
                bool has_tail = false;
                for (const auto& label : group.second)
                {
                    const auto c = columns_.find(label);
                    cols.push_back(c != columns_.end() ? c->second.col : static_columns_.at(label).col);
                    has_tail = has_tail || (c != columns_.end() && c->second.const_tail);
                }
                be_.eval_device(cols, group.first, d.log2n, weights, rotations, result, offset);
                std::size_t ones = npos;
                if (has_tail)
                {
                    ones = ones_next;
                    be_.eval_device({ones_col(group.first)}, group.first, d.log2n, weights, rotations, ones_out, ones_next);
                    ones_next += points;
                }
                placed.push_back({offset, &group.second, ones});
                offset += points * cols.size();
            }
            std::vector<Fe> host(points * labels.size()), ones_host(points * tail_groups);
            be_.download(result, 0, host.size(), host.data());
            if (tail_groups != 0) be_.download(ones_out, 0, ones_host.size(), ones_host.data());
            for (const auto& p : placed)
            {
                const std::size_t k = p.labels->size();
                for (std::size_t i = 0; i < k; ++i)
                {
                    const std::string& label = (*p.labels)[i];
                    const auto c = columns_.find(label);
                    Fe value[2];
                    for (std::size_t r = 0; r < points; ++r)
                    {
                        value[r] = host[p.offset + r * k + i];
                        // rows beyond the stored prefix hold the running sum's final value (see commit_batch)
                        if (c != columns_.end() && c->second.const_tail)
                            value[r] = add(value[r], mul(c->second.tail, sub(fe_u64(1), ones_host[p.ones + r])));
                    }
                    if (!at_tau)
                    {
                        out[label] = {value[0], points > 1 ? value[1] : fe_u64(0)};
                    }
                    else if (c != columns_.end())
                    {
                        out[label] = {commitments_.at(label).tau_evaluation, value[0]};
                    }
                    else
                    {
                        static_omega_tau_[label] = value[0];
                        out[label] = {static_commitments_.at(label).tau_evaluation, value[0]};
                    }
                }
            }
            finish_derived();
        };

        // Names the numerators use for columns this flow keeps under another label: the static tables are committed
        // as V_T_*; the feature domain has one selector for table and query rows and one column-index column.
        auto column_name = [](const std::string& label) -> std::string {
            if (label.rfind("P_T_", 0) == 0 && label != "P_T_H") return "V_T_" + label.substr(4);
            if (label == "P_Q_qry_feat") return "P_Q_tbl_feat";
            if (label == "P_Col_feat_qry") return "P_Col_feat_tbl";
            return label;
        };
        auto value_of = [&](const std::map<std::string, std::array<Fe, 2>>& values, const std::string& label, int r) -> Fe {
            const auto found = values.find(column_name(label));
            if (found == values.end()) throw std::runtime_error("flow: the quotient numerator reads " + label + ", which has no evaluation here");
            return found->second[r];
        };
        // ---- quotient scalars at tau (prover.cpp:3076-3160 with evaluate_t_* of quotients.cpp) --------------
        // Values at omega*tau are needed of the running columns only (rotated_labels); the reference precomputes
        // them for every dependency label, which changes no output.
        std::vector<Fe> quotient_values(7);
        for (int di = 0; di < 7; ++di)
        {
            const Domain& d = dom_.at(kDomains[di]);
            std::map<std::string, std::array<Fe, 2>> values;
            evaluate_domain(kDomains[di], d.w_tau, true, {1}, true, values);
            if (std::string(kDomains[di]) == "FH")
            {
                // generated public columns at tau and omega*tau (prepared with the key) and P_H
                const char* names[5] = {"P_Q_tbl_feat", "P_Row_feat_tbl", "P_Col_feat_tbl", "P_I_feat_qry", "P_T_H"};
                for (int i = 0; i < 5; ++i) values[names[i]] = {fh_public_tau_[i], fh_public_omega_tau_[i]};
                // the lazy lookup columns: the evaluations their commitments were made from (P_R_feat is identically zero)
                for (const char* label : {"P_H", "P_Table_feat", "P_Query_feat", "P_m_feat", "P_R_feat"})
                    values[label] = {commitments_.at(label).tau_evaluation, fe_u64(0)};
            }
            const auto basis = boundary_basis(d, tau_);
            const Fe numerator = quotient_numerator(
                kDomains[di], [&](const std::string& label, int r) { return value_of(values, label, r); }, basis[0], basis[1]);
            const Fe zero_eval = sub(pow(tau_, d.size), fe_u64(1));  // Z_D(tau) = tau^n - 1
            quotient_values[di] = mul(numerator, inv(zero_eval));
            quotient_log_.push_back({std::string("t_") + kBundles[di], quotient_values[di]});
            stats_.opened_columns += values.size();
        }
        // batch_quotient_commitments, prover.cpp:2220-2247
        std::vector<G1> quotient_points(7);
        {
            const ColP s = upload_fe(quotient_values, 7);
            const ColP p = be_.alloc(kG1, 7);
            be_.g1_fixed_base(in_.generator, s, 7, p);
            be_.download(p, 0, 7, quotient_points.data());
        }
        for (int di = 0; di < 7; ++di) t.absorb_commitment(std::string("t_") + kBundles[di], quotient_points[di]);
        std::map<std::string, Fe> z, v;
        for (int di = 0; di < 7; ++di) z[kDomains[di]] = challenge(t, std::string("z_") + kBundles[di]);
        for (int di = 0; di < 7; ++di) v[kDomains[di]] = challenge(t, std::string("v_") + kBundles[di]);
        const Fe rho_ext = challenge(t, "rho_ext");

        // ---- openings at {z, omega*z} -------------------------------------------------------------------
        proof_.block_order = {"M_pub", "Com_dyn", "S_route", "Eval_ext", "Eval_dom", "Com_quot", "Open_dom", "W_ext", "Pi_bind"};
        for (const auto& label : commitment_order_) proof_.dynamic_commitments.push_back({label, point_bytes(commitments_.at(label).point)});
        for (int di = 0; di < 7; ++di) proof_.quotient_commitments.push_back({std::string("t_") + kBundles[di], point_bytes(quotient_points[di])});
        std::vector<Fe> witness_scalars(7);
        for (int di = 0; di < 7; ++di)
        {
            const Domain& d = dom_.at(kDomains[di]);
            const Fe z0 = z.at(kDomains[di]), z1 = mul(z0, d.omega);
            const ColP w_z = be_.alloc(kFrMont, d.size);
            {
                // the longest stored column of the domain bounds the weights that will be read
                std::size_t keep = std::string(kDomains[di]) == "FH" ? n_nodes_ * in_.feature_count : 0;
                const auto opened = opened_.find(kDomains[di]);
                if (opened != opened_.end())
                    for (const auto& label : opened->second) keep = std::max(keep, columns_.at(label).length);
                for (const auto& item : static_columns_)
                    if (item.second.domain == kDomains[di]) keep = std::max(keep, item.second.length);
                if (compact_ && keep < d.size)
                    be_.bary_weights_prefix(d.log2n, z0, keep, w_z);
                else
                    be_.bary_weights(d.log2n, z0, w_z);
            }
            std::map<std::string, std::array<Fe, 2>> values, twice_rotated;
            evaluate_domain(kDomains[di], w_z, false, {0, 1}, false, values);
            // t_D is opened at omega*z too, and its numerator there reads the running columns at omega^2 z
            // (fh_dependency_points, prover.cpp:2294-2306)
            if (std::string(kDomains[di]) != "FH") evaluate_domain(kDomains[di], w_z, false, {2}, true, twice_rotated);
            std::vector<std::string> labels = domain_labels(kDomains[di]);
            if (std::string(kDomains[di]) == "FH")
            {
                // the feature-domain columns are never materialised: generated public columns at z and
                // omega*z (a11) and the lazy lookup columns as the same combinations as their commitments
                Fe at_z[5], at_wz[5];
                be_.fh_public_eval(features_q_, n_nodes_, in_.feature_count, ids_i64_, w_z, d.log2n, 0, at_z);
                be_.fh_public_eval(features_q_, n_nodes_, in_.feature_count, ids_i64_, w_z, d.log2n, 1, at_wz);
                const Fe eta_i = challenges_.at("eta_feat"), eta_v = mul(eta_i, eta_i);
                auto combos = [&](const Fe* p) {
                    std::array<Fe, 5> o;
                    o[0] = p[4];                                                      // P_H
                    o[1] = add(add(p[1], mul(eta_i, p[2])), mul(eta_v, p[4]));        // P_Table_feat
                    o[2] = add(add(p[3], mul(eta_i, p[2])), mul(eta_v, p[4]));        // P_Query_feat
                    o[3] = p[0];                                                      // P_m_feat
                    o[4] = fe_u64(0);                                                 // P_R_feat
                    return o;
                };
                const auto a = combos(at_z), b = combos(at_wz);
                labels = {"P_H", "P_Table_feat", "P_Query_feat", "P_m_feat", "P_R_feat"};
                for (int i = 0; i < 5; ++i) values[labels[i]] = {a[i], b[i]};
                const char* names[5] = {"P_Q_tbl_feat", "P_Row_feat_tbl", "P_Col_feat_tbl", "P_I_feat_qry", "P_T_H"};
                for (int i = 0; i < 5; ++i) values[names[i]] = {at_z[i], at_wz[i]};
                twice_rotated["P_R_feat"] = {fe_u64(0), fe_u64(0)};  // the accumulator of the feature lookup is identically zero
            }
            // the quotient's own value at the two points (make_bundle adds the t_D label, prover.cpp:3273-3274):
            // the same numerator over the opened values; Z_D(omega z) = Z_D(z)
            {
                const Fe inv_zero_eval = inv(sub(pow(z0, d.size), fe_u64(1)));
                const auto basis0 = boundary_basis(d, z0), basis1 = boundary_basis(d, z1);
                const Fe n0 = quotient_numerator(
                    kDomains[di], [&](const std::string& label, int r) { return value_of(values, label, r); }, basis0[0], basis0[1]);
                const Fe n1 = quotient_numerator(
                    kDomains[di],
                    [&](const std::string& label, int r) { return r == 0 ? value_of(values, label, 1) : value_of(twice_rotated, label, 0); },
                    basis1[0], basis1[1]);
                values[std::string("t_") + kBundles[di]] = {mul(n0, inv_zero_eval), mul(n1, inv_zero_eval)};
                labels.push_back(std::string("t_") + kBundles[di]);
            }
            gatzk_b200::protocol::DomainOpeningBundle bundle;
            // KZG::open_batch: witness scalar = sum_i v^i (p_i(tau) - I_i(tau)) / ((tau - z0)(tau - z1)),
            // I_i the line through (z0, value_0), (z1, value_1)
            const Fe dz = sub(z0, z1), inv_dz = inv(dz);
            const Fe l0 = mul(sub(tau_, z1), inv_dz), l1 = mul(sub(z0, tau_), inv_dz);  // Lagrange basis of {z0, z1} at tau
            Fe folded = fe_u64(0), power = fe_u64(1);
            for (const auto& label : labels)
            {
                const auto& val = values.at(label);
                gatzk_b200::protocol::FieldBytes b0, b1;
                std::memcpy(b0.data(), val[0].data(), 32);
                std::memcpy(b1.data(), val[1].data(), 32);
                bundle.values.push_back({label, {b0, b1}});
                Fe p_tau;
                if (label.rfind("t_", 0) == 0)
                    p_tau = quotient_values[di];
                else
                    p_tau = commitments_.at(label).tau_evaluation;
                const Fe interpolation = add(mul(val[0], l0), mul(val[1], l1));
                folded = add(folded, mul(power, sub(p_tau, interpolation)));
                power = mul(power, v.at(kDomains[di]));
            }
            witness_scalars[di] = mul(folded, inv(mul(sub(tau_, z0), sub(tau_, z1))));
            proof_.domain_openings.push_back({kBundles[di], bundle});
        }
        // external fold (KZG::open_external_fold): sum_i rho^i (p_i(tau) - mu_i) / (tau - y_i)
        Fe ext = fe_u64(0);
        {
            Fe power = fe_u64(1);
            for (std::size_t i = 0; i < external_evaluations_.size(); ++i)
            {
                const Fe p_tau = commitments_.at(external_sources_[i].first).tau_evaluation;
                const Fe quotient = mul(sub(p_tau, external_evaluations_[i].second), inv(sub(tau_, external_sources_[i].second)));
                ext = add(ext, mul(power, quotient));
                power = mul(power, rho_ext);
            }
        }
        std::vector<Fe> all = witness_scalars;
        all.push_back(ext);
        std::vector<G1> pts(all.size());
        {
            const ColP s = upload_fe(all, all.size());
            const ColP p = be_.alloc(kG1, all.size());
            be_.g1_fixed_base(in_.generator, s, all.size(), p);
            be_.download(p, 0, all.size(), pts.data());
        }
        for (int di = 0; di < 7; ++di) proof_.domain_openings[di].second.witness = point_bytes(pts[di]);
        proof_.external_witness = point_bytes(pts[7]);
        auto fb = [](const Fe& f) {
            gatzk_b200::protocol::FieldBytes b;
            std::memcpy(b.data(), f.data(), 32);
            return b;
        };
        for (const auto& item : external_evaluations_) proof_.external_evaluations.push_back({item.first, fb(item.second)});
        for (const auto& item : witness_scalars_) proof_.witness_scalars.push_back({item.first, fb(item.second)});
        be_.synchronize();
    }

    // ---- text dump of everything a proof run produced, for field-by-field comparison of two backends ----
    inline std::string dump_flow(const ProverFlow& flow)
    {
        static const char kHex[] = "0123456789abcdef";
        auto hex = [&](const std::uint8_t* p, std::size_t n) {
            std::string s;
            for (std::size_t i = 0; i < n; ++i)
            {
                s.push_back(kHex[p[i] >> 4]);
                s.push_back(kHex[p[i] & 15]);
            }
            return s;
        };
        std::string out;
        for (const auto& c : flow.challenges()) out += "challenge " + c.first + " " + hex(c.second.data(), 32) + "\n";
        for (const auto& c : flow.tau_evaluations()) out += "tau_eval " + c.first + " " + hex(c.second.data(), 32) + "\n";
        for (const auto& c : flow.quotient_scalars()) out += "quotient " + c.first + " " + hex(c.second.data(), 32) + "\n";
        const auto& p = flow.proof();
        for (const auto& c : p.dynamic_commitments) out += "commitment " + c.first + " " + hex(c.second.data(), 48) + "\n";
        for (const auto& c : p.quotient_commitments) out += "quotient_commitment " + c.first + " " + hex(c.second.data(), 48) + "\n";
        for (const auto& b : p.domain_openings)
        {
            for (const auto& row : b.second.values)
                out += "opened " + b.first + " " + row.first + " " + hex(row.second[0].data(), 32) + " " + hex(row.second[1].data(), 32) + "\n";
            out += "opening_witness " + b.first + " " + hex(b.second.witness.data(), 48) + "\n";
        }
        for (const auto& c : p.external_evaluations) out += "external " + c.first + " " + hex(c.second.data(), 32) + "\n";
        for (const auto& c : p.witness_scalars) out += "witness_scalar " + c.first + " " + hex(c.second.data(), 32) + "\n";
        out += "external_witness " + hex(p.external_witness.data(), 48) + "\n";
        return out;
    }

    // Parameter block layout of the C entry points (all little-endian, tightly packed arrays supplied by
    // the caller): see flow_c_api.h.
}
