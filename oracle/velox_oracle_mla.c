/*
 * velox_oracle_mla.c -- CPU statement of the multi-head latent attention (MLA) decode block (TEST INFRASTRUCTURE ONLY).
 *
 * PARITY UNPINNED beyond the single-head algebra: the reference's runtime implements only the one-head, rope-less
 * block (src/runtime.rs:944-1044, restated as vo_mla_absorbed_step_f32); the 128-head form with rope dimensions is
 * declared by its model file (examples/deepseek_v3_mla.vlx:18-45, decode scope :117-150) and by the absorption
 * identity its tests pin (src/optimizer.rs:544-585, tests/test_adversarial_step8_mla.rs:195-303).  Two statements of
 * the same block live here and are checked against each other: the explicit one (keys and values decompressed per
 * head) and the absorbed one (queries moved into the latent space, the cache never decompressed).
 *
 * Layout: every matrix is [out][in] row-major fp32 (callers round to bf16 beforehand when they model bf16 weights):
 *   w_dq [q_lora][d]   w_uq [H*dn][q_lora]   w_qr [H*dr][q_lora]   w_dkv [dc][d]   w_kr [dr][d]
 *   w_uk [H*dn][dc]    w_uv [H*dv][dc]       w_o [d][H*dv]
 * cache row = [c_kv (dc) | k_rope (dr)], fp32, [max_seq][dc + dr].
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "velox_oracle.h"

static void matvec(float* y, const float* w, const float* x, size_t out, size_t in) {
#if defined(_OPENMP)
#pragma omp parallel for schedule(static) if (out * in > 65536)
#endif
    for (size_t o = 0; o < out; ++o) {
        float acc = 0.0f;
        for (size_t k = 0; k < in; ++k) acc = fmaf(w[o * in + k], x[k], acc);
        y[o] = acc;
    }
}

static float bf16_round(float f) { return vo_bf16_to_f32(vo_f32_to_bf16(f)); }

/* Everything up to the attention core: nx, the new cache row at `pos`, q_nope [H*dn] and q_rope [H*dr] (rotated). */
static void mla_project(const vo_mla_block* m, const float* x, float* cache, size_t pos, float* q_nope, float* q_rope, int cache_bf16) {
    const size_t d = m->d_model, dc = m->kv_lora, dr = m->rope_dim, H = m->n_heads;
    float* nx = (float*)malloc(d * sizeof(float));
    float* cq = (float*)malloc(m->q_lora * sizeof(float));
    vo_rmsnorm_f32(nx, x, m->w_norm, d, m->eps);
    float* row = cache + pos * (dc + dr);
    matvec(row, m->w_dkv, nx, dc, d);
    matvec(row + dc, m->w_kr, nx, dr, d);
    vo_rope_rotate_half_f32(row + dc, 1, dr, pos, m->theta);
    if (cache_bf16)
        for (size_t i = 0; i < dc + dr; ++i) row[i] = bf16_round(row[i]);
    matvec(cq, m->w_dq, nx, m->q_lora, d);
    matvec(q_nope, m->w_uq, cq, H * m->nope_dim, m->q_lora);
    matvec(q_rope, m->w_qr, cq, H * dr, m->q_lora);
    vo_rope_rotate_half_f32(q_rope, H, dr, pos, m->theta);
    free(nx);
    free(cq);
}

static void softmax_two_pass(float* s, size_t n) {
    float mx = -INFINITY;
    for (size_t t = 0; t < n; ++t) if (s[t] > mx) mx = s[t];
    float sum = 0.0f;
    for (size_t t = 0; t < n; ++t) { s[t] = expf(s[t] - mx); sum += s[t]; }
    const float inv = 1.0f / sum;
    for (size_t t = 0; t < n; ++t) s[t] *= inv;
}

/* Absorbed form: q_abs_h = W_uk_h^T q_nope_h; scores against the latent rows; ctx_h = sum p c_kv; o_h = W_uv_h ctx_h.
 * Also returns, when asked, the concatenated queries [H][dc+dr] and the per-head latent context [H][dc] -- the inputs
 * and outputs of the attention core alone. */
void vo_mla_step_absorbed(const vo_mla_block* m, float* dst, const float* x, float* cache, size_t pos, int cache_bf16,
                          float* q_cat_out, float* ctx_out) {
    const size_t d = m->d_model, dc = m->kv_lora, dr = m->rope_dim, dn = m->nope_dim, dv = m->v_dim, H = m->n_heads, W = dc + dr;
    float* q_nope = (float*)malloc(H * dn * sizeof(float));
    float* q_rope = (float*)malloc(H * dr * sizeof(float));
    float* q_cat = (float*)malloc(H * W * sizeof(float));
    float* ctx = (float*)malloc(H * dc * sizeof(float));
    float* o = (float*)malloc(H * dv * sizeof(float));
    float* s = (float*)malloc((pos + 1) * sizeof(float));
    mla_project(m, x, cache, pos, q_nope, q_rope, cache_bf16);
    const float scale = 1.0f / sqrtf((float)(dn + dr));
    for (size_t h = 0; h < H; ++h) {
        float* q = q_cat + h * W;
        for (size_t c = 0; c < dc; ++c) {
            float acc = 0.0f;
            for (size_t k = 0; k < dn; ++k) acc = fmaf(q_nope[h * dn + k], m->w_uk[(h * dn + k) * dc + c], acc);
            q[c] = acc;
        }
        memcpy(q + dc, q_rope + h * dr, dr * sizeof(float));
    }
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (size_t h = 0; h < H; ++h) {
        float* sh = (float*)malloc((pos + 1) * sizeof(float));
        const float* q = q_cat + h * W;
        for (size_t t = 0; t <= pos; ++t) {
            float acc = 0.0f;
            for (size_t k = 0; k < W; ++k) acc = fmaf(q[k], cache[t * W + k], acc);
            sh[t] = acc * scale;
        }
        softmax_two_pass(sh, pos + 1);
        float* c = ctx + h * dc;
        memset(c, 0, dc * sizeof(float));
        for (size_t t = 0; t <= pos; ++t)
            for (size_t k = 0; k < dc; ++k) c[k] = fmaf(sh[t], cache[t * W + k], c[k]);
        matvec(o + h * dv, m->w_uv + h * dv * dc, c, dv, dc);
        free(sh);
    }
    float* y = (float*)malloc(d * sizeof(float));
    matvec(y, m->w_o, o, d, H * dv);
    for (size_t i = 0; i < d; ++i) dst[i] = x[i] + y[i];
    if (q_cat_out) memcpy(q_cat_out, q_cat, H * W * sizeof(float));
    if (ctx_out) memcpy(ctx_out, ctx, H * dc * sizeof(float));
    free(q_nope); free(q_rope); free(q_cat); free(ctx); free(o); free(s); free(y);
}

/* Explicit form: k_h(t) = [W_uk_h c_kv(t) | k_rope(t)], v_h(t) = W_uv_h c_kv(t), ordinary attention per head. */
void vo_mla_step_explicit(const vo_mla_block* m, float* dst, const float* x, float* cache, size_t pos, int cache_bf16) {
    const size_t d = m->d_model, dc = m->kv_lora, dr = m->rope_dim, dn = m->nope_dim, dv = m->v_dim, H = m->n_heads, W = dc + dr;
    float* q_nope = (float*)malloc(H * dn * sizeof(float));
    float* q_rope = (float*)malloc(H * dr * sizeof(float));
    float* o = (float*)malloc(H * dv * sizeof(float));
    mla_project(m, x, cache, pos, q_nope, q_rope, cache_bf16);
    const float scale = 1.0f / sqrtf((float)(dn + dr));
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (size_t h = 0; h < H; ++h) {
        float* s = (float*)malloc((pos + 1) * sizeof(float));
        float* kn = (float*)malloc(dn * sizeof(float));
        float* v = (float*)malloc(dv * sizeof(float));
        for (size_t t = 0; t <= pos; ++t) {
            const float* row = cache + t * W;
            matvec(kn, m->w_uk + h * dn * dc, row, dn, dc);
            float acc = 0.0f;
            for (size_t k = 0; k < dn; ++k) acc = fmaf(q_nope[h * dn + k], kn[k], acc);
            for (size_t k = 0; k < dr; ++k) acc = fmaf(q_rope[h * dr + k], row[dc + k], acc);
            s[t] = acc * scale;
        }
        softmax_two_pass(s, pos + 1);
        float* oh = o + h * dv;
        memset(oh, 0, dv * sizeof(float));
        for (size_t t = 0; t <= pos; ++t) {
            matvec(v, m->w_uv + h * dv * dc, cache + t * W, dv, dc);
            for (size_t k = 0; k < dv; ++k) oh[k] = fmaf(s[t], v[k], oh[k]);
        }
        free(s); free(kn); free(v);
    }
    float* y = (float*)malloc(d * sizeof(float));
    matvec(y, m->w_o, o, d, H * dv);
    for (size_t i = 0; i < d; ++i) dst[i] = x[i] + y[i];
    free(q_nope); free(q_rope); free(o); free(y);
}

/* The attention core alone: out[H][dc] = softmax_t(scale * q_h . row_t) weighted sum of the first dc entries of the rows. */
void vo_mla_core(float* out, const float* q_cat, const float* cache, size_t n_heads, size_t dc, size_t dr, size_t n_rows, float scale) {
    const size_t W = dc + dr;
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (size_t h = 0; h < n_heads; ++h) {
        float* s = (float*)malloc(n_rows * sizeof(float));
        for (size_t t = 0; t < n_rows; ++t) {
            float acc = 0.0f;
            for (size_t k = 0; k < W; ++k) acc = fmaf(q_cat[h * W + k], cache[t * W + k], acc);
            s[t] = acc * scale;
        }
        softmax_two_pass(s, n_rows);
        float* c = out + h * dc;
        memset(c, 0, dc * sizeof(float));
        for (size_t t = 0; t < n_rows; ++t)
            for (size_t k = 0; k < dc; ++k) c[k] = fmaf(s[t], cache[t * W + k], c[k]);
        free(s);
    }
}
