/*
 * velox_oracle.c -- CPU restatement of the Velox decode step (TEST INFRASTRUCTURE ONLY).
 *
 * The checker for the CUDA library: loaded by the tests, the smoke check and the benchmark's
 * CPU-baseline leg, never by the product path.  See velox_oracle.h for the citation of the
 * reference function each routine follows.  Build with -ffp-contract=off so that only the
 * explicit fused multiply-adds (the ones the reference's AVX2 kernel issues) are fused.
 */
#include "velox_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#define VO_AVX2 1
#endif
#if defined(_OPENMP)
#include <omp.h>
#endif

/* ------------------------------------------------------------------------------------------ */
/* scalar conversions                                                                          */
/* ------------------------------------------------------------------------------------------ */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

uint16_t vo_f32_to_f16(float f) {
    uint32_t x = f2u(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x0200u : 0u));
    }
    if (ax >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (ax < 0x33000001u) { /* below half of the smallest subnormal (2^-25) -> 0 */
        return (uint16_t)sign;
    }
    int32_t exp = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x007FFFFFu) | 0x00800000u;
    uint32_t shift, half;
    if (exp < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - exp));
        half = 0;
    } else {
        shift = 13;
        half = (uint32_t)(exp + 15) << 10;
        man &= 0x007FFFFFu;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    uint32_t r = half + q;
    if (rem > halfway || (rem == halfway && (q & 1u))) r += 1u;
    return (uint16_t)(sign | r);
}

float vo_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return u2f(sign);
        float v = (float)man * 5.9604644775390625e-8f; /* 2^-24, exact */
        return sign ? -v : v;
    }
    if (exp == 31) return u2f(sign | 0x7F800000u | (man << 13));
    return u2f(sign | ((exp + 112u) << 23) | (man << 13));
}

uint16_t vo_f32_to_bf16(float f) {
    uint32_t x = f2u(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

float vo_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* ------------------------------------------------------------------------------------------ */
/* deterministic synthetic inputs                                                              */
/* ------------------------------------------------------------------------------------------ */
static inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

static inline uint64_t stream_key(uint64_t seed, uint64_t stream) {
    return mix64(seed ^ mix64(stream + 0x9E3779B97F4A7C15ULL));
}

uint64_t vo_hash64(uint64_t seed, uint64_t stream, uint64_t counter) {
    return mix64(stream_key(seed, stream) + (counter + 1ULL) * 0x9E3779B97F4A7C15ULL);
}

static inline uint32_t lanes16_sum(uint64_t h) {
    return (uint32_t)(h & 0xFFFFu) + (uint32_t)((h >> 16) & 0xFFFFu) +
           (uint32_t)((h >> 32) & 0xFFFFu) + (uint32_t)(h >> 48);
}

void vo_fill_normal(float* dst, size_t n, uint64_t seed, uint64_t stream, float mean, float std) {
    const uint64_t key = stream_key(seed, stream);
    const float scale = std * (1.0f / 65536.0f);
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (long long ii = 0; ii < (long long)n; ++ii) {
        uint64_t i = (uint64_t)ii;
        uint32_t s = 0;
        for (uint64_t j = 0; j < 3; ++j) {
            s += lanes16_sum(mix64(key + (3ULL * i + j + 1ULL) * 0x9E3779B97F4A7C15ULL));
        }
        float v = (float)((int32_t)s - 393210) * scale;
        dst[i] = v + mean;
    }
}

void vo_fill_tokens(uint32_t* dst, size_t n, uint64_t seed, uint64_t stream, uint32_t vocab) {
    for (size_t i = 0; i < n; ++i) dst[i] = (uint32_t)(vo_hash64(seed, stream, i) % (uint64_t)vocab);
}

/* ------------------------------------------------------------------------------------------ */
/* quantizers                                                                                  */
/* ------------------------------------------------------------------------------------------ */
static inline int rn_int(float v) { return (int)lrintf(v); } /* round-half-even (default mode) */

/* 8 nibbles -> one word, element order of src/codegen.rs:2363-2364 */
static inline uint32_t pack8(const uint32_t q[8]) {
    return (q[0] << 0) | (q[2] << 4) | (q[4] << 8) | (q[6] << 12) |
           (q[1] << 16) | (q[3] << 20) | (q[5] << 24) | (q[7] << 28);
}
static inline void unpack8(uint32_t p, uint32_t q[8]) {
    q[0] = (p >> 0) & 15u;  q[2] = (p >> 4) & 15u;  q[4] = (p >> 8) & 15u;  q[6] = (p >> 12) & 15u;
    q[1] = (p >> 16) & 15u; q[3] = (p >> 20) & 15u; q[5] = (p >> 24) & 15u; q[7] = (p >> 28) & 15u;
}

void vo_quantize_q4g32(uint32_t* packed, uint16_t* scales, const float* w, size_t rows, size_t cols) {
    const size_t groups = cols / 32;
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (long long rr = 0; rr < (long long)rows; ++rr) {
        size_t r = (size_t)rr;
        for (size_t g = 0; g < groups; ++g) {
            const float* grp = w + r * cols + g * 32;
            float amax = 0.0f;
            for (int i = 0; i < 32; ++i) { float a = fabsf(grp[i]); if (a > amax) amax = a; }
            uint16_t hs = vo_f32_to_f16(amax / 7.0f);
            scales[r * groups + g] = hs;
            float s = vo_f16_to_f32(hs);
            for (int wd = 0; wd < 4; ++wd) {
                uint32_t q[8];
                for (int j = 0; j < 8; ++j) {
                    int qi = 8;
                    if (s > 0.0f) {
                        qi = rn_int(grp[wd * 8 + j] / s) + 8;
                        if (qi < 0) qi = 0;
                        if (qi > 15) qi = 15;
                    }
                    q[j] = (uint32_t)qi;
                }
                packed[(r * cols + g * 32) / 8 + (size_t)wd] = pack8(q);
            }
        }
    }
}

static void dequant_row_q4g32(float* dst, const uint32_t* packed_row, const uint16_t* scales_row, size_t cols) {
    for (size_t g = 0; g < cols / 32; ++g) {
        float s = vo_f16_to_f32(scales_row[g]);
        for (int wd = 0; wd < 4; ++wd) {
            uint32_t q[8];
            unpack8(packed_row[g * 4 + (size_t)wd], q);
            for (int j = 0; j < 8; ++j) dst[g * 32 + (size_t)wd * 8 + (size_t)j] = ((float)q[j] - 8.0f) * s;
        }
    }
}

void vo_dequant_q4g32(float* dst, const uint32_t* packed, const uint16_t* scales, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; ++r)
        dequant_row_q4g32(dst + r * cols, packed + r * (cols / 8), scales + r * (cols / 32), cols);
}

void vo_quantize_q4g64ref(uint32_t* packed, uint16_t* scale_min, const float* w, size_t rows, size_t cols) {
    const size_t n_groups = rows * cols / 64;
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (long long gg = 0; gg < (long long)n_groups; ++gg) {
        size_t g = (size_t)gg;
        const float* grp = w + g * 64;
        float fmin = grp[0], fmax = grp[0];
        for (int i = 1; i < 64; ++i) { float v = grp[i]; if (v < fmin) fmin = v; if (v > fmax) fmax = v; }
        float scale_f = (fmax > fmin) ? ((fmax - fmin) / 15.0f) : 0.0f;
        uint16_t hs = vo_f32_to_f16(scale_f), hm = vo_f32_to_f16(fmin);
        scale_min[2 * g] = hs;
        scale_min[2 * g + 1] = hm;
        float s = vo_f16_to_f32(hs), m = vo_f16_to_f32(hm);
        float inv = (s > 1.0e-12f) ? (1.0f / s) : 0.0f;
        for (int wd = 0; wd < 8; ++wd) {
            uint32_t q[8];
            for (int j = 0; j < 8; ++j) {
                int qi = rn_int((grp[wd * 8 + j] - m) * inv);
                if (qi < 0) qi = 0;
                if (qi > 15) qi = 15;
                q[j] = (uint32_t)qi;
            }
            packed[g * 8 + (size_t)wd] = pack8(q);
        }
    }
}

static void dequant_row_q4g64ref(float* dst, const uint32_t* packed_row, const uint16_t* sm_row, size_t cols) {
    for (size_t g = 0; g < cols / 64; ++g) {
        float s = vo_f16_to_f32(sm_row[2 * g]), m = vo_f16_to_f32(sm_row[2 * g + 1]);
        for (int wd = 0; wd < 8; ++wd) {
            uint32_t q[8];
            unpack8(packed_row[g * 8 + (size_t)wd], q);
            for (int j = 0; j < 8; ++j) dst[g * 64 + (size_t)wd * 8 + (size_t)j] = fmaf((float)q[j], s, m);
        }
    }
}

void vo_dequant_q4g64ref(float* dst, const uint32_t* packed, const uint16_t* scale_min, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; ++r)
        dequant_row_q4g64ref(dst + r * cols, packed + r * (cols / 8), scale_min + r * (cols / 64) * 2, cols);
}

void vo_quantize_i8pc(int8_t* q, uint16_t* scales, const float* w, size_t rows, size_t cols) {
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (long long rr = 0; rr < (long long)rows; ++rr) {
        size_t r = (size_t)rr;
        const float* row = w + r * cols;
        float amax = 0.0f;
        for (size_t i = 0; i < cols; ++i) { float a = fabsf(row[i]); if (a > amax) amax = a; }
        uint16_t hs = vo_f32_to_f16(amax / 127.0f);
        scales[r] = hs;
        float s = vo_f16_to_f32(hs);
        for (size_t i = 0; i < cols; ++i) {
            int qi = 0;
            if (s > 0.0f) {
                qi = rn_int(row[i] / s);
                if (qi < -127) qi = -127;
                if (qi > 127) qi = 127;
            }
            q[r * cols + i] = (int8_t)qi;
        }
    }
}

static void dequant_row_i8pc(float* dst, const int8_t* q_row, uint16_t hs, size_t cols) {
    float s = vo_f16_to_f32(hs);
    for (size_t i = 0; i < cols; ++i) dst[i] = (float)q_row[i] * s;
}

void vo_dequant_i8pc(float* dst, const int8_t* q, const uint16_t* scales, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; ++r) dequant_row_i8pc(dst + r * cols, q + r * cols, scales[r], cols);
}

/* ------------------------------------------------------------------------------------------ */
/* primitives                                                                                  */
/* ------------------------------------------------------------------------------------------ */
void vo_rmsnorm_f32(float* dst, const float* x, const float* w, size_t dim, float eps) {
    float ss = 0.0f;
    for (size_t i = 0; i < dim; ++i) ss += x[i] * x[i];
    float inv_rms = 1.0f / sqrtf((ss / (float)dim) + eps);
    for (size_t i = 0; i < dim; ++i) dst[i] = (x[i] * inv_rms) * w[i];
}

/* One output row: 8 FMA lanes over k, the reference's horizontal-sum tree, scalar tail. */
static inline float dot_row(const float* x, const float* w, size_t in_dim) {
    const size_t k_chunks = in_dim / 8;
#ifdef VO_AVX2
    __m256 acc = _mm256_setzero_ps();
    for (size_t c = 0; c < k_chunks; ++c)
        acc = _mm256_fmadd_ps(_mm256_loadu_ps(x + c * 8), _mm256_loadu_ps(w + c * 8), acc);
    float a[8];
    _mm256_storeu_ps(a, acc);
#else
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (size_t c = 0; c < k_chunks; ++c)
        for (int l = 0; l < 8; ++l) a[l] = fmaf(x[c * 8 + l], w[c * 8 + l], a[l]);
#endif
    float v0 = a[0] + a[4], v1 = a[1] + a[5], v2 = a[2] + a[6], v3 = a[3] + a[7];
    float s = (v0 + v1) + (v2 + v3);
    for (size_t k = k_chunks * 8; k < in_dim; ++k) s += x[k] * w[k];
    return s;
}

void vo_matmul_transposed_f32(float* dst, const float* x, const float* w, size_t in_dim, size_t out_dim) {
#if defined(_OPENMP)
#pragma omp parallel for schedule(static) if (out_dim >= 512)
#endif
    for (long long o = 0; o < (long long)out_dim; ++o) dst[o] = dot_row(x, w + (size_t)o * in_dim, in_dim);
}

static void dequant_row_any(float* dst, const void* w, const void* scales, int fmt, size_t row, size_t in_dim) {
    switch (fmt) {
    case VO_FMT_F16: {
        const uint16_t* p = (const uint16_t*)w + row * in_dim;
        for (size_t i = 0; i < in_dim; ++i) dst[i] = vo_f16_to_f32(p[i]);
    } break;
    case VO_FMT_BF16: {
        const uint16_t* p = (const uint16_t*)w + row * in_dim;
        for (size_t i = 0; i < in_dim; ++i) dst[i] = vo_bf16_to_f32(p[i]);
    } break;
    case VO_FMT_Q4G32:
        dequant_row_q4g32(dst, (const uint32_t*)w + row * (in_dim / 8), (const uint16_t*)scales + row * (in_dim / 32), in_dim);
        break;
    case VO_FMT_Q4G64REF:
        dequant_row_q4g64ref(dst, (const uint32_t*)w + row * (in_dim / 8), (const uint16_t*)scales + row * (in_dim / 64) * 2, in_dim);
        break;
    case VO_FMT_I8PC:
        dequant_row_i8pc(dst, (const int8_t*)w + row * in_dim, ((const uint16_t*)scales)[row], in_dim);
        break;
    default:
        memcpy(dst, (const float*)w + row * in_dim, in_dim * sizeof(float));
    }
}

void vo_matvec_fmt(float* dst, const float* x, const void* w, const void* scales, int fmt,
                   size_t in_dim, size_t out_dim) {
    if (fmt == VO_FMT_F32) { vo_matmul_transposed_f32(dst, x, (const float*)w, in_dim, out_dim); return; }
#if defined(_OPENMP)
#pragma omp parallel if (out_dim >= 256)
#endif
    {
        float* row = (float*)malloc(in_dim * sizeof(float));
#if defined(_OPENMP)
#pragma omp for schedule(static)
#endif
        for (long long o = 0; o < (long long)out_dim; ++o) {
            dequant_row_any(row, w, scales, fmt, (size_t)o, in_dim);
            dst[o] = dot_row(x, row, in_dim);
        }
        free(row);
    }
}

void vo_rope_rotate_half_f32(float* t, size_t n_heads, size_t head_dim, size_t pos, float theta) {
    size_t half = head_dim / 2;
    float pos_f = (float)pos;
    for (size_t h = 0; h < n_heads; ++h) {
        float* hs = t + h * head_dim;
        for (size_t j = 0; j < half; ++j) {
            float freq = 1.0f / powf(theta, (float)(2 * j) / (float)head_dim);
            float angle = pos_f * freq;
            float c = cosf(angle), s = sinf(angle);
            float x1 = hs[j], x2 = hs[j + half];
            hs[j] = x1 * c - x2 * s;
            hs[j + half] = x2 * c + x1 * s;
        }
    }
}

void vo_gqa_attention_step_f32(float* out, float* scores, const float* q, const float* k_layer,
                               const float* v_layer, size_t n_q, size_t n_kv, size_t head_dim, size_t pos) {
    size_t group = n_q / n_kv, kv_stride = n_kv * head_dim, seq_len = pos + 1;
    float scale = 1.0f / sqrtf((float)head_dim);
    for (size_t h = 0; h < n_q; ++h) {
        size_t kv_h = h / group;
        const float* qh = q + h * head_dim;
        float max_score = -INFINITY;
        for (size_t t = 0; t < seq_len; ++t) {
            const float* kh = k_layer + t * kv_stride + kv_h * head_dim;
            float dot = 0.0f;
            for (size_t d = 0; d < head_dim; ++d) dot += qh[d] * kh[d];
            float s = dot * scale;
            scores[t] = s;
            if (s > max_score) max_score = s;
        }
        float sum_exp = 0.0f;
        for (size_t t = 0; t < seq_len; ++t) { float e = expf(scores[t] - max_score); scores[t] = e; sum_exp += e; }
        float inv_sum = 1.0f / sum_exp;
        for (size_t t = 0; t < seq_len; ++t) scores[t] *= inv_sum;
        float* oh = out + h * head_dim;
        for (size_t d = 0; d < head_dim; ++d) oh[d] = 0.0f;
        for (size_t t = 0; t < seq_len; ++t) {
            float p = scores[t];
            const float* vh = v_layer + t * kv_stride + kv_h * head_dim;
            for (size_t d = 0; d < head_dim; ++d) oh[d] += p * vh[d];
        }
    }
}

void vo_swiglu_mlp_residual_f32(float* hidden, float* gate, float* up, float* down, const float* nx,
                                const float* wg, const float* wu, const float* wd, size_t d, size_t ffn) {
    vo_matmul_transposed_f32(gate, nx, wg, d, ffn);
    vo_matmul_transposed_f32(up, nx, wu, d, ffn);
    for (size_t i = 0; i < ffn; ++i) { float g = gate[i]; float silu = g / (1.0f + expf(-g)); gate[i] = silu * up[i]; }
    vo_matmul_transposed_f32(down, gate, wd, ffn, d);
    for (size_t i = 0; i < d; ++i) hidden[i] += down[i];
}

uint32_t vo_sample_argmax_f32(const float* logits, size_t n) {
    uint32_t best = 0;
    float best_val = -INFINITY;
    for (size_t i = 0; i < n; ++i) if (logits[i] > best_val) { best_val = logits[i]; best = (uint32_t)i; }
    return best;
}

void vo_mla_absorbed_step_f32(float* dst, const float* x, const float* w_norm, const float* w_dkv,
                              const float* w_absq, const float* w_abso, float* pool,
                              size_t step, size_t hidden, size_t latent, size_t max_seq, float eps) {
    float* nx = (float*)malloc(hidden * sizeof(float));
    float* q_abs = (float*)malloc(latent * sizeof(float));
    float* ctx = (float*)malloc(latent * sizeof(float));
    float* o = (float*)malloc(hidden * sizeof(float));
    vo_rmsnorm_f32(nx, x, w_norm, hidden, eps);
    size_t safe_step = (step < max_seq) ? step : (max_seq ? max_seq - 1 : 0);
    float* slot = pool + safe_step * latent;
    vo_matmul_transposed_f32(slot, nx, w_dkv, hidden, latent);
    vo_matmul_transposed_f32(q_abs, nx, w_absq, hidden, latent);
    float scale = (latent >= 128) ? (1.0f / sqrtf(128.0f)) : (1.0f / sqrtf((float)latent));
    float m = -INFINITY, l = 0.0f;
    for (size_t d = 0; d < latent; ++d) ctx[d] = 0.0f;
    for (size_t t = 0; t <= safe_step; ++t) {
        const float* k = pool + t * latent;
        float dot = 0.0f;
        for (size_t d = 0; d < latent; ++d) dot += q_abs[d] * k[d];
        float s = dot * scale;
        float new_m = (s > m) ? s : m;
        float alpha = (m == -INFINITY) ? 0.0f : expf(m - new_m);
        float beta = expf(s - new_m);
        l = l * alpha + beta;
        m = new_m;
        for (size_t d = 0; d < latent; ++d) ctx[d] = ctx[d] * alpha + beta * k[d];
    }
    if (l > 0.0f) { float inv_l = 1.0f / l; for (size_t d = 0; d < latent; ++d) ctx[d] *= inv_l; }
    vo_matmul_transposed_f32(o, ctx, w_abso, latent, hidden);
    for (size_t i = 0; i < hidden; ++i) dst[i] = x[i] + o[i];
    free(nx); free(q_abs); free(ctx); free(o);
}

/* ------------------------------------------------------------------------------------------ */
/* engine                                                                                      */
/* ------------------------------------------------------------------------------------------ */
typedef struct { const void* data; const void* scales; int fmt; } vo_tensor;

struct vo_engine {
    vo_config cfg;
    vo_tensor* t; /* [VO_ROLE_COUNT][n_layers] */
    float *k_cache, *v_cache; /* [n_seqs][L][max_seq][kv_dim] (GQA) or latent pool in k_cache (MLA) */
    float *hidden, *norm_x, *q_buf, *attn_out, *o_buf, *gate, *up, *down, *scores, *logits, *tmp_vec;
};

static vo_tensor* tensor_at(vo_engine* e, int role, int layer) {
    return &e->t[(size_t)role * e->cfg.n_layers + (size_t)layer];
}

vo_engine* vo_engine_create(const vo_config* cfg) {
    vo_engine* e = (vo_engine*)calloc(1, sizeof(vo_engine));
    if (!e) return NULL;
    e->cfg = *cfg;
    if (e->cfg.n_seqs == 0) e->cfg.n_seqs = 1;
    size_t L = cfg->n_layers ? cfg->n_layers : 1;
    e->t = (vo_tensor*)calloc((size_t)VO_ROLE_COUNT * L, sizeof(vo_tensor));
    size_t kv_dim = (size_t)cfg->n_kv_heads * cfg->head_dim;
    size_t qdim = (size_t)cfg->n_q_heads * cfg->head_dim;
    size_t per_tok = cfg->mla_latent ? cfg->mla_latent : kv_dim;
    size_t cache = (size_t)e->cfg.n_seqs * cfg->n_layers * cfg->max_seq_len * per_tok;
    e->k_cache = (float*)calloc(cache ? cache : 1, sizeof(float));
    e->v_cache = cfg->mla_latent ? NULL : (float*)calloc(cache ? cache : 1, sizeof(float));
    size_t d = cfg->d_model;
    size_t big = d > cfg->ffn_dim ? d : cfg->ffn_dim;
    if (qdim > big) big = qdim;
    e->hidden = (float*)calloc(d, 4);   e->norm_x = (float*)calloc(d, 4);
    e->q_buf = (float*)calloc(qdim ? qdim : 1, 4); e->attn_out = (float*)calloc(qdim ? qdim : 1, 4);
    e->o_buf = (float*)calloc(d, 4);
    e->gate = (float*)calloc(cfg->ffn_dim ? cfg->ffn_dim : 1, 4); e->up = (float*)calloc(cfg->ffn_dim ? cfg->ffn_dim : 1, 4);
    e->down = (float*)calloc(d, 4);
    e->scores = (float*)calloc(cfg->max_seq_len ? cfg->max_seq_len : 1, 4);
    e->logits = (float*)calloc(cfg->vocab ? cfg->vocab : 1, 4);
    e->tmp_vec = (float*)calloc(big, 4);
    return e;
}

void vo_engine_destroy(vo_engine* e) {
    if (!e) return;
    free(e->t); free(e->k_cache); free(e->v_cache); free(e->hidden); free(e->norm_x); free(e->q_buf);
    free(e->attn_out); free(e->o_buf); free(e->gate); free(e->up); free(e->down); free(e->scores);
    free(e->logits); free(e->tmp_vec); free(e);
}

int vo_engine_set_tensor(vo_engine* e, int role, int layer, const void* data, const void* scales, int fmt) {
    if (!e || role < 0 || role >= VO_ROLE_COUNT) return -1;
    if (role == VO_ROLE_EMBED || role == VO_ROLE_FINAL_NORM || role == VO_ROLE_LM_HEAD) layer = 0;
    if (layer < 0 || (uint32_t)layer >= (e->cfg.n_layers ? e->cfg.n_layers : 1)) return -1;
    vo_tensor* t = tensor_at(e, role, layer);
    t->data = data; t->scales = scales; t->fmt = fmt;
    return 0;
}

/* small vectors (norm weights, biases) are kept F32 or F16 */
static const float* vec_f32(vo_engine* e, const vo_tensor* t, size_t n, float* scratch) {
    (void)e;
    if (t->fmt == VO_FMT_F32) return (const float*)t->data;
    const uint16_t* p = (const uint16_t*)t->data;
    for (size_t i = 0; i < n; ++i) scratch[i] = (t->fmt == VO_FMT_BF16) ? vo_bf16_to_f32(p[i]) : vo_f16_to_f32(p[i]);
    return scratch;
}

static void matvec_t(float* dst, const float* x, const vo_tensor* t, size_t in_dim, size_t out_dim) {
    vo_matvec_fmt(dst, x, t->data, t->scales, t->fmt, in_dim, out_dim);
}

static void add_bias(vo_engine* e, float* dst, const vo_tensor* b, size_t n) {
    if (!b->data) return;
    const float* bv = vec_f32(e, b, n, e->tmp_vec);
    for (size_t i = 0; i < n; ++i) dst[i] = dst[i] + bv[i];
}

uint32_t vo_engine_forward_step(vo_engine* e, uint32_t seq, uint32_t token, uint32_t pos) {
    const vo_config* c = &e->cfg;
    const size_t d = c->d_model, kv_dim = (size_t)c->n_kv_heads * c->head_dim, qdim = (size_t)c->n_q_heads * c->head_dim;
    const size_t per_tok = c->mla_latent ? c->mla_latent : kv_dim;
    const size_t layer_stride = (size_t)c->max_seq_len * per_tok;
    const size_t seq_stride = (size_t)c->n_layers * layer_stride;

    /* 1. embedding row (src/runtime.rs:1335-1338) */
    dequant_row_any(e->hidden, tensor_at(e, VO_ROLE_EMBED, 0)->data, tensor_at(e, VO_ROLE_EMBED, 0)->scales,
                    tensor_at(e, VO_ROLE_EMBED, 0)->fmt, token, d);

    for (uint32_t l = 0; l < c->n_layers; ++l) {
        if (c->mla_latent) {
            /* reference absorbed-MLA block replaces norm+QKV+RoPE+attention+O-proj */
            const size_t dc = c->mla_latent;
            float* wn = (float*)malloc(d * 4);
            float* wdkv = (float*)malloc(dc * d * 4);
            float* wq = (float*)malloc(dc * d * 4);
            float* wo = (float*)malloc(dc * d * 4);
            const vo_tensor *tn = tensor_at(e, VO_ROLE_MLA_NORM, (int)l), *t1 = tensor_at(e, VO_ROLE_MLA_WDKV, (int)l),
                            *t2 = tensor_at(e, VO_ROLE_MLA_WABSQ, (int)l), *t3 = tensor_at(e, VO_ROLE_MLA_WABSO, (int)l);
            memcpy(wn, vec_f32(e, tn, d, e->tmp_vec), d * 4);
            for (size_t r = 0; r < dc; ++r) {
                dequant_row_any(wdkv + r * d, t1->data, t1->scales, t1->fmt, r, d);
                dequant_row_any(wq + r * d, t2->data, t2->scales, t2->fmt, r, d);
            }
            for (size_t r = 0; r < d; ++r) dequant_row_any(wo + r * dc, t3->data, t3->scales, t3->fmt, r, dc);
            float* pool = e->k_cache + seq * seq_stride + l * layer_stride;
            vo_mla_absorbed_step_f32(e->o_buf, e->hidden, wn, wdkv, wq, wo, pool, pos, d, dc, c->max_seq_len, c->rms_eps);
            memcpy(e->hidden, e->o_buf, d * 4);
            free(wn); free(wdkv); free(wq); free(wo);
        } else {
            /* pre-attention RMSNorm (src/runtime.rs:1356) */
            float* nw_s = (float*)malloc(d * 4);
            const float* nw = vec_f32(e, tensor_at(e, VO_ROLE_ATTN_NORM, (int)l), d, nw_s);
            vo_rmsnorm_f32(e->norm_x, e->hidden, nw, d, c->rms_eps);
            free(nw_s);
            /* Q,K,V: K and V straight into the cache slot (src/runtime.rs:1364-1370) */
            float* k_layer = e->k_cache + seq * seq_stride + l * layer_stride;
            float* v_layer = e->v_cache + seq * seq_stride + l * layer_stride;
            float* k_slot = k_layer + (size_t)pos * kv_dim;
            float* v_slot = v_layer + (size_t)pos * kv_dim;
            matvec_t(e->q_buf, e->norm_x, tensor_at(e, VO_ROLE_WQ, (int)l), d, qdim);
            matvec_t(k_slot, e->norm_x, tensor_at(e, VO_ROLE_WK, (int)l), d, kv_dim);
            matvec_t(v_slot, e->norm_x, tensor_at(e, VO_ROLE_WV, (int)l), d, kv_dim);
            if (c->qkv_bias) {
                add_bias(e, e->q_buf, tensor_at(e, VO_ROLE_BQ, (int)l), qdim);
                add_bias(e, k_slot, tensor_at(e, VO_ROLE_BK, (int)l), kv_dim);
                add_bias(e, v_slot, tensor_at(e, VO_ROLE_BV, (int)l), kv_dim);
            }
            /* RoPE on Q and on the K slot (src/runtime.rs:1373-1386) */
            vo_rope_rotate_half_f32(e->q_buf, c->n_q_heads, c->head_dim, pos, c->rope_theta);
            vo_rope_rotate_half_f32(k_slot, c->n_kv_heads, c->head_dim, pos, c->rope_theta);
            /* attention over [0..=pos] (src/runtime.rs:1391) */
            vo_gqa_attention_step_f32(e->attn_out, e->scores, e->q_buf, k_layer, v_layer, c->n_q_heads,
                                      c->n_kv_heads, c->head_dim, pos);
            /* O-proj + residual (src/runtime.rs:1404-1407) */
            matvec_t(e->o_buf, e->attn_out, tensor_at(e, VO_ROLE_WO, (int)l), qdim, d);
            for (size_t i = 0; i < d; ++i) e->hidden[i] += e->o_buf[i];
        }
        /* post-attention RMSNorm + SwiGLU + residual (src/runtime.rs:1410-1427, :1048-1073) */
        float* nw_s = (float*)malloc(d * 4);
        const float* nw = vec_f32(e, tensor_at(e, VO_ROLE_MLP_NORM, (int)l), d, nw_s);
        vo_rmsnorm_f32(e->norm_x, e->hidden, nw, d, c->rms_eps);
        free(nw_s);
        matvec_t(e->gate, e->norm_x, tensor_at(e, VO_ROLE_WGATE, (int)l), d, c->ffn_dim);
        matvec_t(e->up, e->norm_x, tensor_at(e, VO_ROLE_WUP, (int)l), d, c->ffn_dim);
        for (size_t i = 0; i < c->ffn_dim; ++i) {
            float g = e->gate[i];
            float silu = g / (1.0f + expf(-g));
            e->gate[i] = silu * e->up[i];
        }
        matvec_t(e->down, e->gate, tensor_at(e, VO_ROLE_WDOWN, (int)l), c->ffn_dim, d);
        for (size_t i = 0; i < d; ++i) e->hidden[i] += e->down[i];
    }

    /* final norm, lm_head, argmax (src/runtime.rs:1434-1448) */
    float* nw_s = (float*)malloc(d * 4);
    const float* nw = vec_f32(e, tensor_at(e, VO_ROLE_FINAL_NORM, 0), d, nw_s);
    vo_rmsnorm_f32(e->norm_x, e->hidden, nw, d, c->rms_eps);
    free(nw_s);
    const vo_tensor* head = tensor_at(e, VO_ROLE_LM_HEAD, 0);
    if (!head->data) head = tensor_at(e, VO_ROLE_EMBED, 0); /* tied embeddings */
    matvec_t(e->logits, e->norm_x, head, d, c->vocab);
    return vo_sample_argmax_f32(e->logits, c->vocab);
}

const float* vo_engine_logits(const vo_engine* e) { return e->logits; }
const float* vo_engine_hidden(const vo_engine* e) { return e->hidden; }

size_t vo_engine_generate_greedy(vo_engine* e, uint32_t seq, const uint32_t* prompt, size_t n_prompt,
                                 size_t n_new, uint32_t* out_tokens) {
    if (n_prompt == 0) return 0;
    uint32_t pos = 0, next = prompt[0];
    for (size_t i = 0; i < n_prompt; ++i) { next = vo_engine_forward_step(e, seq, prompt[i], pos); pos++; }
    if (n_new == 0) return 0;
    out_tokens[0] = next;
    for (size_t s = 1; s < n_new; ++s) { next = vo_engine_forward_step(e, seq, next, pos); pos++; out_tokens[s] = next; }
    return n_new;
}

/* Host threads the checker's matrix-vector loops may use (launchers such as torch.distributed.run export
 * OMP_NUM_THREADS=1; the timed CPU baseline states its core count and therefore sets it itself). */
void vo_set_num_threads(int n) {
#if defined(_OPENMP)
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int vo_num_threads(void) {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}
