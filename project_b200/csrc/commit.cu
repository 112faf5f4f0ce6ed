// Column commitment as the reference performs it (trapdoor KZG): the tau-evaluation
// of every column by packed evaluation against w(tau), then one fixed-base
// multiplication [p_k(tau)] G per column; and the honest-prover alternative, a
// Lagrange-basis SRS [L_i(tau)] G against which a column is committed by an MSM
// (same group element, because sum_i f_i [L_i(tau)] G = [sum_i f_i L_i(tau)] G).
#include "common.cuh"

using namespace gzk;

extern "C"
{
    int gzk_commit_batch(gzk_ctx* ctx, gzk_buf* const* cols, size_t k_count, size_t len, unsigned log2n, const gzk_buf* weights_tau,
                         const uint8_t base[96], uint8_t* tau_evals_out, uint8_t* points_out)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (k_count == 0) return GZK_OK;
        if (tau_evals_out == nullptr || points_out == nullptr || base == nullptr) return fail(ctx, GZK_E_INVALID, "commit_batch: null argument");
        const uint64_t zero_rotation = 0;
        int rc = gzk_eval_batch(ctx, cols, k_count, len, log2n, weights_tau, &zero_rotation, 1, tau_evals_out);
        if (rc != GZK_OK) return rc;
        return gzk_g1_mul_same_base(ctx, base, tau_evals_out, k_count, points_out);
    }

    int gzk_srs_lagrange(gzk_ctx* ctx, unsigned log2n, const uint8_t base[96], const uint8_t tau[32], gzk_buf* out_points)
    {
        if (ctx == nullptr) return GZK_E_INVALID;
        if (log2n > 28) return fail(ctx, GZK_E_INVALID, "srs_lagrange: domain too large");
        const size_t n = static_cast<size_t>(1) << log2n;
        if (out_points == nullptr || out_points->kind != GZK_KIND_G1 || out_points->count < n)
            return fail(ctx, GZK_E_INVALID, "srs_lagrange: output must be a G1 buffer of the domain size");
        gzk_buf* weights = nullptr;
        int rc = gzk_buf_alloc(ctx, GZK_KIND_FR_MONT, n, &weights);
        if (rc != GZK_OK) return rc;
        rc = gzk_bary_weights(ctx, log2n, tau, weights);
        if (rc == GZK_OK) rc = gzk_g1_fixed_base_mul(ctx, base, weights, n, out_points);
        const std::string message = ctx->last_error;
        gzk_buf_free(ctx, weights);
        if (rc != GZK_OK) ctx->last_error = message;
        return rc;
    }
}
