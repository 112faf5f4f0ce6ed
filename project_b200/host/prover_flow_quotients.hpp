// Constraint numerators of the seven quotient polynomials t_FH, t_edge, t_in, t_d_h, t_cat, t_C, t_N
// (multi-head form), restated from src/protocol/quotients.cpp:311-1303.  Included by prover_flow_tail.hpp.
//
// A quotient is  t_D(x) = (sum_i alpha^i c_i(x)) / (x^n - 1),  the c_i in the fixed order of the reference
// (QuotientAccumulator, quotients.cpp:225-241: the i-th constraint ADDED gets alpha^i).  Every c_i is a
// polynomial identity in the committed columns at x and, for the running columns, at omega*x.  The code below
// states each family of constraints once (a lookup, a route, a bound inner product, ...) and lists the
// families per head in the reference's order; `at(label, r)` supplies p_label(omega^r x), r = 0 or 1.
//
// The same routine serves three callers: the quotient scalars at tau (values at tau, omega tau), the opened
// values t_D(z) and t_D(omega z) (values at z, omega z, omega^2 z), and the row check of the tests, where x is a
// point of the domain, `at` reads the columns themselves and every c_i must vanish.
#pragma once

namespace gatzk_flow
{
    // The labels a numerator reads at omega*x: the running sums and the columns their steps look ahead at.
    inline std::vector<std::string> ProverFlow::rotated_labels(const std::string& domain) const
    {
        std::vector<std::string> out;
        const bool legacy = in_.output_layer.heads.size() == 1;
        std::size_t hidden_heads = 0;
        for (const auto& layer : in_.hidden_layers) hidden_heads += layer.heads.size();
        auto output_prefix = [&](std::size_t k) { return legacy ? std::string("P_out_") : "P_out" + std::to_string(k) + "_"; };
        if (domain == "FH")
        {
            out = {"P_R_feat"};
        }
        else if (domain == "edge")
        {
            out = {"P_Q_edge_valid", "P_Q_new_edge"};
            for (std::size_t h = 0; h < hidden_heads; ++h)
                for (const char* s : {"R_src", "R_L", "s_max", "C_max", "R_R", "R_exp", "PSQ", "w_psq", "R_t", "R_ELU", "R_dst"})
                    out.push_back("P_h" + std::to_string(h) + "_" + s);
            for (std::size_t k = 0; k < in_.output_layer.heads.size(); ++k)
                for (const char* s : {"R_src", "R_L", "s_max", "C_max", "R_R", "R_exp", "PSQ", "w", "R_t", "R_dst"}) out.push_back(output_prefix(k) + s);
        }
        else if (domain == "N")
        {
            for (std::size_t h = 0; h < hidden_heads; ++h)
                for (const char* s : {"R_src_node", "R_dst_node", "R_t_node"}) out.push_back("P_h" + std::to_string(h) + "_" + s);
            for (std::size_t k = 0; k < in_.output_layer.heads.size(); ++k)
                for (const char* s : {"R_src_node", "R_dst_node", "R_t_node"}) out.push_back(output_prefix(k) + s);
        }
        else if (domain == "in")
        {
            for (std::size_t h = 0; h < hidden_heads; ++h) out.push_back("P_h" + std::to_string(h) + "_Acc_proj");
        }
        else if (domain == "d")
        {
            for (std::size_t h = 0; h < hidden_heads; ++h)
                for (const char* s : {"Acc_src", "Acc_dst", "Acc_star", "Acc_agg_pre", "Acc_agg"}) out.push_back("P_h" + std::to_string(h) + "_" + s);
        }
        else if (domain == "cat")
        {
            for (std::size_t li = 0; li < in_.hidden_layers.size(); ++li)
                out.push_back((li + 1 == in_.hidden_layers.size() ? std::string("P_cat") : "P_cat_l" + std::to_string(li)) + "_Acc");
            for (std::size_t k = 0; k < in_.output_layer.heads.size(); ++k) out.push_back(output_prefix(k) + "Acc_proj");
        }
        else if (domain == "C")
        {
            for (std::size_t k = 0; k < in_.output_layer.heads.size(); ++k)
                for (const char* s : {"Acc_src", "Acc_dst", "Acc_y"}) out.push_back(output_prefix(k) + s);
        }
        return out;
    }

    // sum_i alpha^i c_i(x) of one domain.  `first` / `last` are L_0(x) and L_{n-1}(x).
    inline Fe ProverFlow::quotient_numerator(const std::string& domain, const PointValues& at, const Fe& first, const Fe& last)
    {
        const Fe one = fe_u64(1);
        const Fe alpha = challenges_.at("alpha_quot");
        Fe sum = fe_u64(0), power = one;
        // Not every constraint of the reference holds on the witness its own builders produce.  The class of a
        // constraint says what the row check may expect of it (it does not change the numerator):
        //   kExact   vanishes on every row;
        //   kWraps   vanishes on every row but the last: a running column that ends at a non-zero total steps back
        //            to its first value across the wrap-around (the reference leaves that row to the last-row term);
        //   kLoose   need not vanish: it ties quantised values to exact sums, products or reciprocals; or it is a
        //            LogUp step of an accumulator that the builders run over the query rows only
        //            (lookup_active_transition_limit, trace.cpp:2597), so table rows behind them never enter; or it
        //            belongs to the source route, whose builder packs (id, E_src) on the node side but (src, H*)
        //            on the edge side (trace.cpp:2737-2760) while the quotient states a third packing.
        enum { kExact = 0, kWraps = 1, kLoose = 2 };
        std::size_t index = 0;
        auto push = [&](const Fe& term, int cls = kExact) {
            if (nonzero_terms_ != nullptr && term != fe_u64(0)) nonzero_terms_->push_back(index * 4 + static_cast<std::size_t>(cls));
            ++index;
            if ((term_classes_ >> cls) & 1u) sum = add(sum, mul(power, term));
            power = mul(power, alpha);
        };
        auto ch = [&](const std::string& name) {
            const auto found = challenges_.find(name);
            if (found == challenges_.end()) throw std::runtime_error("flow: the quotient numerator needs the challenge " + name);
            return found->second;
        };
        if (quotient_scalars_.size() != witness_scalars_.size() || quotient_externals_.size() != external_evaluations_.size())
        {
            quotient_scalars_ = std::map<std::string, Fe>(witness_scalars_.begin(), witness_scalars_.end());
            quotient_externals_ = std::map<std::string, Fe>(external_evaluations_.begin(), external_evaluations_.end());
        }
        const std::map<std::string, Fe>&scalars = quotient_scalars_, &externals = quotient_externals_;
        auto now = [&](const std::string& label) { return at(label, 0); };
        auto next = [&](const std::string& label) { return at(label, 1); };
        auto unselected = [&](const Fe& selector, const Fe& value) { return mul(sub(one, selector), value); };  // zero_on_unselected

        // -- constraint families ---------------------------------------------------------------------------
        // LogUp accumulator R of (table, query, multiplicity) with selectors q_tbl, q_qry (lookup_step, :281-293),
        // bracketed by R = 0 on the first and on the last row
        auto lookup = [&](const std::string& r, const Fe& table, const Fe& query, const Fe& m, const Fe& q_tbl, const Fe& q_qry, const Fe& beta) {
            push(mul(first, now(r)));
            const Fe tb = add(table, beta), qb = add(query, beta);
            push(add(sub(mul(mul(sub(next(r), now(r)), tb), qb), mul(mul(q_tbl, m), qb)), mul(q_qry, tb)), kLoose);
            push(mul(last, now(r)), kLoose);
        };
        // edge side of a route (route_edge_step, :253-260): starts at 0, one step per valid edge, ends at `total`
        auto route_edge = [&](const std::string& r, const Fe& query, const Fe& beta, const Fe& q_edge, const Fe& total, int total_class = kExact) {
            push(mul(first, now(r)));
            push(sub(mul(sub(next(r), now(r)), add(query, beta)), q_edge), kWraps);
            push(mul(last, sub(now(r), total)), total_class);
        };
        // node side (route_node_step, :243-251)
        auto route_node = [&](const std::string& r, const Fe& table, const Fe& m, const Fe& beta, const Fe& q_n, const Fe& total) {
            push(mul(first, now(r)));
            push(sub(mul(sub(next(r), now(r)), add(table, beta)), mul(q_n, m)), kWraps);
            push(mul(last, sub(now(r), total)));
        };
        // bound inner product Acc of a and b over the selected rows, ending at the externally opened value mu
        // (acc_step, :262-268)
        // `bound`: kLoose when mu is the evaluation of a QUANTISED matrix while a and b fold its exact factors
        auto inner_product = [&](const std::string& acc, const std::string& a, const std::string& b, const Fe& q_valid, const Fe& mu, int bound = kExact) {
            const Fe step = sub(next(acc), now(acc));
            push(mul(first, now(acc)));
            push(mul(q_valid, sub(step, mul(now(a), now(b)))));
            push(mul(sub(one, q_valid), step), kWraps);
            push(unselected(q_valid, now(a)));
            push(unselected(q_valid, now(b)));
            push(mul(last, sub(now(acc), mu)), bound);
        };

        if (domain == "FH")
        {
            // quotients.cpp:311-352.  The selectors, index columns and the table are generated public columns.
            const Fe beta = ch("beta_feat"), eta = ch("eta_feat"), eta2 = mul(eta, eta);
            lookup("P_R_feat", now("P_Table_feat"), now("P_Query_feat"), now("P_m_feat"), now("P_Q_tbl_feat"), now("P_Q_qry_feat"), beta);
            push(sub(now("P_Table_feat"), add(add(now("P_Row_feat_tbl"), mul(eta, now("P_Col_feat_tbl"))), mul(eta2, now("P_T_H")))));
            push(sub(now("P_Query_feat"), add(add(now("P_I_feat_qry"), mul(eta, now("P_Col_feat_qry"))), mul(eta2, now("P_H")))));
            return sum;
        }
        const bool legacy = in_.output_layer.heads.size() == 1;
        std::size_t hidden_heads = 0;
        for (const auto& layer : in_.hidden_layers) hidden_heads += layer.heads.size();
        auto output_prefix = [&](std::size_t k) { return legacy ? std::string("P_out_") : "P_out" + std::to_string(k) + "_"; };
        auto output_challenge = [&](const std::string& name, std::size_t k) { return ch(legacy ? name : name + "_o" + std::to_string(k)); };
        auto output_scalar = [&](const std::string& which, std::size_t k) { return scalars.at("S_" + which + (legacy ? "_out" : "_out" + std::to_string(k))); };
        auto output_external = [&](const std::string& which, std::size_t k) {
            return externals.at(legacy ? "mu_out_" + which : "mu_out" + std::to_string(k) + "_" + which);
        };

        if (domain == "edge")
        {
            // quotients.cpp:355-768
            const Fe q_edge = now("P_Q_edge_valid"), q_edge_next = next("P_Q_edge_valid"), q_new_next = next("P_Q_new_edge"), q_end = now("P_Q_end_edge");
            const Fe src = now("P_src"), dst = now("P_dst");
            const Fe q_tbl_l = now("P_Q_tbl_L"), q_qry_l = now("P_Q_qry_L"), q_tbl_r = now("P_Q_tbl_R"), q_qry_r = now("P_Q_qry_R");
            const Fe q_tbl_exp = now("P_Q_tbl_exp"), q_qry_exp = now("P_Q_qry_exp"), q_tbl_elu = now("P_Q_tbl_ELU"), q_qry_elu = now("P_Q_qry_ELU");
            const Fe t_l_x = now("P_T_L_x"), t_l_y = now("P_T_L_y"), t_range = now("P_T_range"), t_exp_x = now("P_T_exp_x"), t_exp_y = now("P_T_exp_y");
            const Fe t_elu_x = now("P_T_ELU_x"), t_elu_y = now("P_T_ELU_y");
            // the part of an attention head that hidden and output heads share: scores, LeakyReLU lookup, row maximum,
            // range lookup, exponential lookup
            auto scores_to_exp = [&](const std::string& p, const Fe& eta_l, const Fe& beta_l, const Fe& beta_r, const Fe& eta_exp, const Fe& beta_exp) {
                const Fe s = now(p + "S"), z = now(p + "Z"), delta = now(p + "Delta"), m_edge = now(p + "M_edge");
                push(mul(q_edge, sub(sub(s, now(p + "E_src_edge")), now(p + "E_dst_edge"))), kLoose);
                const Fe table_l = now(p + "Table_L"), query_l = now(p + "Query_L"), m_l = now(p + "m_L");
                lookup(p + "R_L", table_l, query_l, m_l, q_tbl_l, q_qry_l, beta_l);
                push(sub(table_l, add(t_l_x, mul(eta_l, t_l_y))));
                push(sub(query_l, add(s, mul(eta_l, z))));
                push(unselected(q_tbl_l, table_l));
                push(unselected(q_tbl_l, m_l));
                push(unselected(q_qry_l, query_l));
                // Delta = M_edge - Z on valid edges; s_max marks one maximal edge per destination group, C_max counts them
                const Fe s_max = now(p + "s_max"), s_max_next = next(p + "s_max"), c_max = now(p + "C_max"), c_max_next = next(p + "C_max");
                push(mul(q_edge, add(sub(delta, m_edge), z)), kLoose);
                push(mul(s_max, sub(s_max, one)));
                push(mul(s_max, delta));
                push(unselected(q_edge, s_max));
                push(mul(first, sub(c_max, s_max)));
                push(add(mul(q_edge_next, sub(sub(c_max_next, mul(q_new_next, s_max_next)), mul(sub(one, q_new_next), add(c_max, s_max_next)))),
                         mul(sub(one, q_edge_next), sub(c_max_next, c_max))));
                push(mul(q_end, sub(c_max, one)));
                const Fe table_r = now(p + "Table_R"), query_r = now(p + "Query_R"), m_r = now(p + "m_R");
                lookup(p + "R_R", table_r, query_r, m_r, q_tbl_r, q_qry_r, beta_r);
                push(sub(table_r, t_range));
                push(sub(query_r, delta));
                push(unselected(q_tbl_r, table_r));
                push(unselected(q_tbl_r, m_r));
                push(unselected(q_qry_r, query_r));
                const Fe u = now(p + "U");
                push(mul(q_edge, sub(now(p + "alpha"), mul(u, now(p + "inv_edge")))), kLoose);
                const Fe table_exp = now(p + "Table_exp"), query_exp = now(p + "Query_exp"), m_exp = now(p + "m_exp");
                lookup(p + "R_exp", table_exp, query_exp, m_exp, q_tbl_exp, q_qry_exp, beta_exp);
                push(sub(table_exp, add(t_exp_x, mul(eta_exp, t_exp_y))));
                push(sub(query_exp, add(delta, mul(eta_exp, u))));
                push(unselected(q_tbl_exp, table_exp));
                push(unselected(q_tbl_exp, m_exp));
                push(unselected(q_qry_exp, query_exp));
            };
            // grouped prefix sum PSQ of w over the edges of a destination, its group total T on the edges, routed to the nodes
            auto grouped_sum = [&](const std::string& p, const std::string& w, const std::string& t_edge, const Fe& eta_t, const Fe& beta_t, const Fe& total) {
                const Fe psq = now(p + "PSQ"), psq_next = next(p + "PSQ"), w_next = next(p + w);
                push(mul(first, sub(psq, mul(q_edge, now(p + w)))));
                // psq_step, :270-279
                push(sub(psq_next, add(mul(sub(one, q_edge_next), psq),
                                       mul(q_edge_next, add(mul(q_new_next, w_next), mul(sub(one, q_new_next), add(psq, w_next)))))));
                push(mul(q_end, sub(psq, now(p + t_edge))), kLoose);
                const Fe query_t = now(p + "Query_t");
                route_edge(p + "R_t", query_t, beta_t, q_edge, total);
                push(sub(query_t, add(dst, mul(eta_t, now(p + t_edge)))));
                push(unselected(q_edge, query_t));
            };
            auto destination_route = [&](const std::string& p, const std::string& star_edge, const Fe& eta, const Fe& beta, const Fe& total) {
                const Fe query = now(p + "Query_dst");
                route_edge(p + "R_dst", query, beta, q_edge, total);
                const Fe e2 = mul(eta, eta), e3 = mul(e2, eta), e4 = mul(e3, eta), e5 = mul(e4, eta);
                Fe packed = add(dst, mul(eta, now(p + "E_dst_edge")));
                packed = add(packed, mul(e2, now(p + "M_edge")));
                packed = add(packed, mul(e3, now(p + "Sum_edge")));
                packed = add(packed, mul(e4, now(p + "inv_edge")));
                packed = add(packed, mul(e5, now(p + star_edge)));
                push(sub(query, packed));
                push(unselected(q_edge, query));
            };
            for (std::size_t h = 0; h < hidden_heads; ++h)
            {
                const std::string hs = std::to_string(h), p = "P_h" + hs + "_";
                const Fe eta_src = ch("eta_src_h" + hs);
                const Fe query_src = now(p + "Query_src");
                route_edge(p + "R_src", query_src, ch("beta_src_h" + hs), q_edge, scalars.at("S_src_h" + hs), kLoose);
                push(sub(query_src, add(add(src, mul(eta_src, now(p + "E_src_edge"))), mul(mul(eta_src, eta_src), now(p + "H_src_star_edge")))), kLoose);
                push(unselected(q_edge, query_src));
                scores_to_exp(p, ch("eta_L_h" + hs), ch("beta_L_h" + hs), ch("beta_R_h" + hs), ch("eta_exp_h" + hs), ch("beta_exp_h" + hs));
                grouped_sum(p, "w_psq", "T_psq_edge", ch("eta_t_h" + hs), ch("beta_t_h" + hs), scalars.at("S_t_h" + hs));
                const Fe eta_elu = ch("eta_ELU_h" + hs);
                const Fe table_elu = now(p + "Table_ELU"), query_elu = now(p + "Query_ELU"), m_elu = now(p + "m_ELU");
                lookup(p + "R_ELU", table_elu, query_elu, m_elu, q_tbl_elu, q_qry_elu, ch("beta_ELU_h" + hs));
                push(sub(table_elu, add(t_elu_x, mul(eta_elu, t_elu_y))));
                push(sub(query_elu, add(now(p + "H_agg_pre_flat"), mul(eta_elu, now(p + "H_agg_flat")))));
                push(unselected(q_tbl_elu, table_elu));
                push(unselected(q_tbl_elu, m_elu));
                push(unselected(q_qry_elu, query_elu));
                destination_route(p, "H_agg_star_edge", ch("eta_dst_h" + hs), ch("beta_dst_h" + hs), scalars.at("S_dst_h" + hs));
            }
            for (std::size_t k = 0; k < in_.output_layer.heads.size(); ++k)
            {
                const std::string p = output_prefix(k);
                const Fe query_src = now(p + "Query_src");
                route_edge(p + "R_src", query_src, output_challenge("beta_src_out", k), q_edge, output_scalar("src", k), kLoose);
                push(sub(query_src, add(src, mul(output_challenge("eta_src_out", k), now(p + "E_src_edge")))), kLoose);
                push(unselected(q_edge, query_src));
                scores_to_exp(p, output_challenge("eta_L_out", k), output_challenge("beta_L_out", k), output_challenge("beta_R_out", k),
                              output_challenge("eta_exp_out", k), output_challenge("beta_exp_out", k));
                grouped_sum(p, "w", "T_edge", output_challenge("eta_t_out", k), output_challenge("beta_t_out", k), output_scalar("t", k));
                destination_route(p, "Y_star_edge", output_challenge("eta_dst_out", k), output_challenge("beta_dst_out", k), output_scalar("dst", k));
            }
            return sum;
        }
        if (domain == "N")
        {
            // quotients.cpp:887-998
            const Fe q_n = now("P_Q_N"), ids = now("P_I");
            auto node_side = [&](const std::string& p, const Fe& beta_src, const Fe& beta_dst, const Fe& beta_t, const Fe& s_src, const Fe& s_dst, const Fe& s_t) {
                route_node(p + "R_src_node", now(p + "Table_src"), now(p + "m_src"), beta_src, q_n, s_src);
                route_node(p + "R_dst_node", now(p + "Table_dst"), now(p + "m_dst"), beta_dst, q_n, s_dst);
                route_node(p + "R_t_node", now(p + "Table_t"), now(p + "m_t"), beta_t, q_n, s_t);
                push(mul(q_n, sub(mul(now(p + "Sum"), now(p + "inv")), one)), kLoose);
            };
            auto destination_table = [&](const std::string& p, const std::string& star, const Fe& eta) {
                const Fe e2 = mul(eta, eta), e3 = mul(e2, eta), e4 = mul(e3, eta), e5 = mul(e4, eta);
                Fe packed = add(ids, mul(eta, now(p + "E_dst")));
                packed = add(packed, mul(e2, now(p + "M")));
                packed = add(packed, mul(e3, now(p + "Sum")));
                packed = add(packed, mul(e4, now(p + "inv")));
                packed = add(packed, mul(e5, now(p + star)));
                push(sub(now(p + "Table_dst"), packed));
            };
            for (std::size_t h = 0; h < hidden_heads; ++h)
            {
                const std::string hs = std::to_string(h), p = "P_h" + hs + "_";
                const Fe eta_src = ch("eta_src_h" + hs);
                node_side(p, ch("beta_src_h" + hs), ch("beta_dst_h" + hs), ch("beta_t_h" + hs), scalars.at("S_src_h" + hs), scalars.at("S_dst_h" + hs),
                          scalars.at("S_t_h" + hs));
                push(mul(q_n, sub(sub(now(p + "T_psq"), now(p + "Sum")), mul(ch("lambda_psq_h" + hs), now(p + "H_agg_pre_star")))));
                push(sub(now(p + "Table_src"), add(add(ids, mul(eta_src, now(p + "E_src"))), mul(mul(eta_src, eta_src), now(p + "H_star")))), kLoose);
                destination_table(p, "H_agg_star", ch("eta_dst_h" + hs));
                push(sub(now(p + "Table_t"), add(ids, mul(ch("eta_t_h" + hs), now(p + "T_psq")))));
                for (const char* s : {"E_src", "E_dst", "M", "Sum", "inv", "H_star", "H_agg_pre_star", "H_agg_star", "Table_src", "m_src", "Table_dst", "m_dst", "T_psq",
                                      "Table_t", "m_t"})
                    push(unselected(q_n, now(p + s)));
            }
            for (std::size_t k = 0; k < in_.output_layer.heads.size(); ++k)
            {
                const std::string p = output_prefix(k);
                node_side(p, output_challenge("beta_src_out", k), output_challenge("beta_dst_out", k), output_challenge("beta_t_out", k), output_scalar("src", k),
                          output_scalar("dst", k), output_scalar("t", k));
                push(mul(q_n, sub(sub(now(p + "T"), now(p + "Sum")), mul(output_challenge("lambda_out", k), now(p + "Y_star")))));
                push(sub(now(p + "Table_src"), add(ids, mul(output_challenge("eta_src_out", k), now(p + "E_src")))));
                destination_table(p, "Y_star", output_challenge("eta_dst_out", k));
                push(sub(now(p + "Table_t"), add(ids, mul(output_challenge("eta_t_out", k), now(p + "T")))));
                for (const char* s : {"E_src", "E_dst", "M", "Sum", "inv", "Y_prime_star", "Y_star", "T", "Table_src", "m_src", "Table_dst", "m_dst", "Table_t", "m_t"})
                    push(unselected(q_n, now(p + s)));
            }
            return sum;
        }
        if (domain == "in")
        {
            // quotients.cpp:1046-1069
            const Fe q_valid = now("P_Q_proj_valid");
            for (std::size_t h = 0; h < hidden_heads; ++h)
            {
                const std::string hs = std::to_string(h), p = "P_h" + hs + "_";
                inner_product(p + "Acc_proj", p + "a_proj", p + "b_proj", q_valid, externals.at("mu_h" + hs + "_proj"), kLoose);
            }
            return sum;
        }
        if (domain == "d")
        {
            // quotients.cpp:1092-1143
            const Fe q_valid = now("P_Q_d_valid");
            for (std::size_t h = 0; h < hidden_heads; ++h)
            {
                const std::string hs = std::to_string(h), p = "P_h" + hs + "_";
                for (const char* s : {"src", "dst", "star", "agg_pre", "agg"})
                    inner_product(p + "Acc_" + s, p + "a_" + s, p + "b_" + s, q_valid, externals.at("mu_h" + hs + "_" + s),
                                  std::string(s) == "src" || std::string(s) == "dst" ? kLoose : kExact);
            }
            return sum;
        }
        if (domain == "cat")
        {
            // quotients.cpp:1190-1230
            const Fe q_valid = now("P_Q_cat_valid");
            for (std::size_t li = 0; li < in_.hidden_layers.size(); ++li)
            {
                const bool final_layer = li + 1 == in_.hidden_layers.size();
                const std::string p = final_layer ? std::string("P_cat") : "P_cat_l" + std::to_string(li);
                inner_product(p + "_Acc", p + "_a", p + "_b", q_valid, externals.at(final_layer ? std::string("mu_cat") : "mu_cat_l" + std::to_string(li)));
            }
            for (std::size_t k = 0; k < in_.output_layer.heads.size(); ++k)
            {
                const std::string p = output_prefix(k);
                inner_product(p + "Acc_proj", p + "a_proj", p + "b_proj", q_valid, output_external("proj", k), kLoose);
            }
            return sum;
        }
        if (domain == "C")
        {
            // quotients.cpp:1232-1301
            const Fe q_valid = now("P_Q_C_valid");
            const Fe y_out = ch("y_out");
            Fe summed_y_lin = fe_u64(0), summed_y = fe_u64(0);
            for (std::size_t k = 0; k < in_.output_layer.heads.size(); ++k)
            {
                const std::string p = output_prefix(k);
                inner_product(p + "Acc_src", p + "a_src", p + "b_src", q_valid, output_external("src", k), kLoose);
                inner_product(p + "Acc_dst", p + "a_dst", p + "b_dst", q_valid, output_external("dst", k), kLoose);
                inner_product(p + "Acc_y", p + "a_y", p + "b_y", q_valid, output_external("star", k));
                const Fe mu_y = legacy ? externals.at("mu_out") : output_external("y", k), mu_y_lin = legacy ? externals.at("mu_Y_lin") : output_external("y_lin", k);
                // Y = Y_lin + bias under every row, evaluated at y_out as one polynomial (bias_fold_vector, :104-127)
                const auto& bias = in_.output_layer.heads[k].output_bias;
                Fe fold = fe_u64(0);
                if (!bias.empty() && n_nodes_ != 0)
                {
                    Fe column_fold = fe_u64(0), column_power = one;
                    for (const double b : bias)
                    {
                        const double scaled = b >= 0.0 ? b * 16.0 + 0.5 : b * 16.0 - 0.5;  // quantize_bias_value, :99-102
                        column_fold = add(column_fold, mul(from_signed(static_cast<std::int64_t>(scaled)), column_power));
                        column_power = mul(column_power, y_out);
                    }
                    const Fe stride = pow(y_out, bias.size());
                    const Fe row_sum = stride == one ? fe_u64(n_nodes_) : mul(sub(pow(stride, n_nodes_), one), inv(sub(stride, one)));
                    fold = mul(column_fold, row_sum);
                }
                push(mul(first, sub(sub(mu_y, mu_y_lin), fold)));
                summed_y_lin = add(summed_y_lin, mu_y_lin);
                summed_y = add(summed_y, mu_y);
            }
            if (!legacy)
            {
                const Fe heads = fe_u64(in_.output_layer.heads.size());
                push(mul(first, sub(mul(heads, externals.at("mu_Y_lin")), summed_y_lin)));
                push(mul(first, sub(mul(heads, externals.at("mu_out")), summed_y)));
            }
            return sum;
        }
        throw std::runtime_error("flow: unknown quotient domain " + domain);
    }

    // Every column a domain's numerator reads, as n field elements on the host: committed columns (prefix-stored ones
    // filled out with their tail), derived columns summed from their sources, static columns, and for the feature
    // domain the columns the flow never stores.
    inline std::map<std::string, std::vector<Fe>> ProverFlow::domain_cells(const std::string& domain)
    {
        const Domain& d = dom_.at(domain);
        const std::size_t n = d.size;
        const Fe zero = fe_u64(0), one = fe_u64(1);
        std::map<std::string, std::vector<Fe>> cells;
        auto read_column = [&](const ColP& col, std::size_t length, bool const_tail, const Fe& tail) {
            std::vector<Fe> out(n, const_tail ? tail : zero);
            length = std::min(length, n);
            if (col->kind == kI64)
            {
                std::vector<std::int64_t> raw(length);
                be_.download(col, 0, length, raw.data());
                for (std::size_t i = 0; i < length; ++i) out[i] = from_signed(raw[i]);
            }
            else if (col->kind == kU32)
            {
                std::vector<std::uint32_t> raw(length);
                be_.download(col, 0, length, raw.data());
                for (std::size_t i = 0; i < length; ++i) out[i] = fe_u64(raw[i]);
            }
            else
            {
                be_.download(col, 0, length, out.data());
            }
            return out;
        };
        if (domain == "FH")
        {
            const std::size_t fc = in_.feature_count, valid = n_nodes_ * fc;
            std::vector<std::int64_t> ids(n_nodes_), feats(valid);
            be_.download(ids_i64_, 0, n_nodes_, ids.data());
            be_.download(features_q_, 0, valid, feats.data());
            const Fe eta = challenges_.at("eta_feat"), eta2 = mul(eta, eta);
            for (const char* label : {"P_Q_tbl_feat", "P_Row_feat_tbl", "P_Col_feat_tbl", "P_I_feat_qry", "P_T_H", "P_H", "P_Table_feat", "P_Query_feat", "P_m_feat", "P_R_feat"})
                cells[label] = std::vector<Fe>(n, zero);
            for (std::size_t i = 0; i < valid && i < n; ++i)
            {
                const Fe row = fe_u64(i / fc), column = fe_u64(i % fc), id = from_signed(ids[i / fc]), value = from_signed(feats[i]);
                cells["P_Q_tbl_feat"][i] = one;
                cells["P_Row_feat_tbl"][i] = row;
                cells["P_Col_feat_tbl"][i] = column;
                cells["P_I_feat_qry"][i] = id;
                cells["P_T_H"][i] = value;
                cells["P_H"][i] = value;
                cells["P_m_feat"][i] = one;
                cells["P_Table_feat"][i] = add(add(row, mul(eta, column)), mul(eta2, value));
                cells["P_Query_feat"][i] = add(add(id, mul(eta, column)), mul(eta2, value));
            }
        }
        else
        {
            std::vector<std::string> derived;
            const auto opened = opened_.find(domain);
            if (opened != opened_.end())
                for (const auto& label : opened->second)
                {
                    const ColumnEntry& c = columns_.at(label);
                    if (!c.derived_from.empty())
                        derived.push_back(label);
                    else
                        cells[label] = read_column(c.col, c.length, c.const_tail, c.tail);
                }
            for (const auto& item : static_columns_)
                if (item.second.domain == domain) cells[item.first] = read_column(item.second.col, item.second.length, false, zero);
            for (const auto& label : derived)
            {
                std::vector<Fe> out(n, zero);
                for (const auto& term : columns_.at(label).derived_from)
                {
                    const auto& source = cells.at(term.first);
                    for (std::size_t i = 0; i < n; ++i) out[i] = add(out[i], mul(term.second, source[i]));
                }
                cells[label] = out;
            }
        }
        return cells;
    }
    // The numerator spells a few columns differently from the committed label.
    inline std::string ProverFlow::numerator_column(const std::string& label)
    {
        if (label.rfind("P_T_", 0) == 0 && label != "P_T_H") return "V_T_" + label.substr(4);
        if (label == "P_Q_qry_feat") return "P_Q_tbl_feat";
        if (label == "P_Col_feat_qry") return "P_Col_feat_tbl";
        return label;
    }

    // Row check of the restated constraints (a diagnostic; no counterpart call in the reference, whose verifier
    // checks the same identities at the opening points): on a point omega^i of a domain the "evaluations" are the
    // column entries of rows i and i+1, L_0 and L_{n-1} are the indicators of the first and the last row, and
    // every constraint of class kExact must vanish, and every constraint of class kWraps except on the last row
    // (the classes are explained in quotient_numerator).  Returns, per domain, the number of rows on which one of
    // them does not; the offenders go to `failures` as (domain, index in the reference's order, rows it failed on).
    inline std::vector<std::uint64_t> ProverFlow::constraint_violations(std::vector<std::array<std::uint64_t, 3>>* failures)
    {
        static const char* kDomains[7] = {"FH", "edge", "in", "d", "cat", "C", "N"};
        std::vector<std::uint64_t> bad(7, 0);
        const Fe zero = fe_u64(0), one = fe_u64(1);
        for (int di = 0; di < 7; ++di)
        {
            const std::string domain = kDomains[di];
            const std::size_t n = dom_.at(domain).size;
            const std::map<std::string, std::vector<Fe>> cells = domain_cells(domain);
            auto name_of = [](const std::string& label) { return numerator_column(label); };
            std::map<std::string, const std::vector<Fe>*> by_request;  // the numerator's own spelling -> column
            std::map<std::size_t, std::uint64_t> rows_failed;           // constraint index -> rows
            for (std::size_t i = 0; i < n; ++i)
            {
                std::vector<std::size_t> failed;
                nonzero_terms_ = &failed;
                quotient_numerator(
                    domain,
                    [&](const std::string& label, int r) {
                        auto found = by_request.find(label);
                        if (found == by_request.end())
                        {
                            const auto column = cells.find(name_of(label));
                            if (column == cells.end()) throw std::runtime_error("flow: the row check finds no column " + label);
                            found = by_request.emplace(label, &column->second).first;
                        }
                        return (*found->second)[(i + static_cast<std::size_t>(r)) % n];
                    },
                    i == 0 ? one : zero, i + 1 == n ? one : zero);
                nonzero_terms_ = nullptr;
                bool strict = false;
                for (const auto tagged : failed)
                {
                    const std::size_t cls = tagged % 4;
                    if (cls == 0 || (cls == 1 && i + 1 != n))
                    {
                        strict = true;
                        ++rows_failed[tagged / 4];
                    }
                }
                if (strict) ++bad[di];
            }
            if (failures != nullptr)
                for (const auto& item : rows_failed) failures->push_back({static_cast<std::uint64_t>(di), item.first, item.second});
        }
        return bad;
    }
    // Honest quotient of one domain (a diagnostic; the reference commits t_D by the trapdoor shortcut N(tau)/Z(tau) and
    // never divides a polynomial, src/protocol/prover.cpp:3076-3160).  Every column the numerator reads goes through
    // the backend's transforms: inverse transform of its n rows, zero padding, forward transform on the domain of
    // n << log2_blowup points.  The numerator, restricted to the constraint classes in `classes` (bit c = class c of
    // quotient_numerator), is formed point by point there - a rotation by omega is a step of 1 << log2_blowup points -
    // and transformed back to coefficients, which are divided by X^n - 1:  N = t (X^n - 1) + R.
    //   out[0] n   out[1] points   out[2] degree of N (highest non-zero coefficient; 0 for the zero polynomial)
    //   out[3] rows omega^i on which R does not vanish (R(omega^i) = N(omega^i): what the row check counts)
    //   out[4] 1 when t(x) (x^n - 1) + R(x) equals the numerator formed directly from the columns' values at x and
    //          omega x (Horner on their coefficients), x a point outside the domains - this fails when the blow-up is
    //          too small for the numerator's degree
    //   out[5] degree of t
    // Host work grows with points x constraints: meant for configurations of a few thousand rows per domain.
    inline std::array<std::uint64_t, 6> ProverFlow::honest_quotient(const std::string& domain, unsigned log2_blowup, unsigned classes)
    {
        const Domain& d = dom_.at(domain);
        const std::size_t n = d.size, blowup = std::size_t{1} << log2_blowup, points = n * blowup;
        if (log2_blowup < 1 || log2_blowup > 4 || points > (std::size_t{1} << 22)) throw std::runtime_error("flow: the honest quotient takes a blow-up of 2..16 and at most 2^22 points");
        const Fe zero = fe_u64(0), one = fe_u64(1);
        std::map<std::string, std::vector<Fe>> cells = domain_cells(domain);
        cells["(first row)"] = std::vector<Fe>(n, zero);
        cells["(first row)"][0] = one;
        cells["(last row)"] = std::vector<Fe>(n, zero);
        cells["(last row)"][n - 1] = one;

        struct Extended
        {
            std::vector<Fe> coefficients, values;
        };
        std::map<std::string, Extended> extended;  // by the numerator's own spelling
        {
            // which columns the numerator reads: one pass over it with every value zero
            std::vector<std::string> labels = {"(first row)", "(last row)"};
            quotient_numerator(
                domain,
                [&](const std::string& label, int) {
                    if (std::find(labels.begin(), labels.end(), label) == labels.end()) labels.push_back(label);
                    return zero;
                },
                zero, zero);
            std::vector<std::vector<Fe>> work;
            for (const auto& label : labels)
            {
                const auto column = cells.find(numerator_column(label));
                if (column == cells.end()) throw std::runtime_error("flow: the honest quotient finds no column " + label);
                work.push_back(column->second);
            }
            be_.transform_many(work, true);
            for (std::size_t i = 0; i < labels.size(); ++i)
            {
                extended[labels[i]].coefficients = work[i];
                work[i].resize(points, zero);
            }
            be_.transform_many(work, false);
            for (std::size_t i = 0; i < labels.size(); ++i) extended[labels[i]].values = std::move(work[i]);
        }
        auto extend = [&](const std::string& label) -> const Extended& {
            const auto found = extended.find(label);
            if (found == extended.end()) throw std::runtime_error("flow: the numerator reads " + label + " on some points only");
            return found->second;
        };
        const unsigned saved = term_classes_;
        term_classes_ = classes;
        std::vector<Fe> numerator(points);
        try
        {
            const std::vector<Fe>&first = extend("(first row)").values, &last = extend("(last row)").values;
            using Requested = std::map<std::string, const std::vector<Fe>*>;
            auto at_point = [&](std::size_t j, Requested& by_request) {
                return quotient_numerator(
                    domain,
                    [&](const std::string& label, int r) {
                        auto found = by_request.find(label);
                        if (found == by_request.end()) found = by_request.emplace(label, &extend(label).values).first;
                        return (*found->second)[(j + static_cast<std::size_t>(r) * blowup) % points];
                    },
                    first[j], last[j]);
            };
            // pointwise on all host threads: the columns are only read
            const std::size_t workers = std::max<std::size_t>(1, std::min<std::size_t>({std::thread::hardware_concurrency(), 32, points / 64 + 1}));
            std::vector<std::thread> pool;
            std::vector<std::string> errors(workers);
            for (std::size_t w = 0; w < workers; ++w)
                pool.emplace_back([&, w] {
                    try
                    {
                        Requested mine;
                        for (std::size_t j = w; j < points; j += workers) numerator[j] = at_point(j, mine);
                    }
                    catch (const std::exception& e)
                    {
                        errors[w] = e.what();
                    }
                });
            for (auto& t : pool) t.join();
            for (const auto& e : errors)
                if (!e.empty()) throw std::runtime_error(e);
        }
        catch (...)
        {
            term_classes_ = saved;
            throw;
        }
        be_.transform(numerator, true);  // coefficients of N
        auto degree_of = [&](const std::vector<Fe>& c) {
            for (std::size_t i = c.size(); i-- > 0;)
                if (c[i] != zero) return static_cast<std::uint64_t>(i);
            return std::uint64_t{0};
        };
        // t's block k-1 is the sum of N's blocks k and above; R = N's block 0 + t's block 0
        std::vector<Fe> quotient(points - n, zero), remainder(n);
        for (std::size_t i = 0; i < n; ++i)
        {
            Fe running = zero;
            for (std::size_t k = blowup; k-- > 1;)
            {
                running = add(running, numerator[k * n + i]);
                quotient[(k - 1) * n + i] = running;
            }
            remainder[i] = add(numerator[i], running);
        }
        auto horner = [&](const std::vector<Fe>& c, const Fe& x) {
            Fe acc = zero;
            for (std::size_t i = c.size(); i-- > 0;) acc = add(mul(acc, x), c[i]);
            return acc;
        };
        // a point outside every domain, fixed by the transcript
        const Fe x = add(challenges_.at("alpha_quot"), fe_u64(0x9e3779b97f4a7c15ULL));
        Fe direct = zero;
        std::map<std::pair<std::string, int>, Fe> at_x;  // a column's value at x (rotation 0) or omega x (rotation 1), formed once
        try
        {
            const auto basis = boundary_basis(d, x);
            direct = quotient_numerator(
                domain,
                [&](const std::string& label, int r) {
                    const auto key = std::make_pair(label, r);
                    auto found = at_x.find(key);
                    if (found == at_x.end()) found = at_x.emplace(key, horner(extend(label).coefficients, r == 0 ? x : mul(x, pow(d.omega, static_cast<std::uint64_t>(r))))).first;
                    return found->second;
                },
                basis[0], basis[1]);
        }
        catch (...)
        {
            term_classes_ = saved;
            throw;
        }
        term_classes_ = saved;
        const Fe divided = add(mul(horner(quotient, x), sub(pow(x, n), one)), horner(remainder, x));
        std::array<std::uint64_t, 6> out{};
        out[0] = n;
        out[1] = points;
        out[2] = degree_of(numerator);
        out[5] = degree_of(quotient);
        out[4] = divided == direct ? 1 : 0;
        be_.transform(remainder, false);
        for (const Fe& value : remainder)
            if (value != zero) ++out[3];
        return out;
    }
}
