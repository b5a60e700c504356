/*
 * velox_oracle_next.c -- CPU restatement of the rows next to the decode step (TEST INFRASTRUCTURE ONLY):
 * nucleus sampling, prompt-lookup speculative decoding and the GGUF Q4_K / Q6_K load-time unpack.
 * Declarations and reference citations are in velox_oracle.h.  Compiled with -ffp-contract=off: every fused
 * multiply-add the reference performs is written as fmaf() here.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "velox_oracle.h"

/* ------------------------------------------------------------------------------------------ */
/* sampling                                                                                    */
/* ------------------------------------------------------------------------------------------ */

/* Uniform coin in [0,1) for (seed, slot, position): the top 24 bits of the shared counter hash.  The reference
 * takes the coin from its caller (src/runtime.rs:1098 `random_coin`); this is the caller both engines use. */
float vo_sample_coin(uint64_t seed, uint32_t slot, uint32_t pos) {
    const uint64_t h = vo_hash64(seed, 0x5A4D504CULL + (uint64_t)slot, (uint64_t)pos);
    return (float)(uint32_t)(h >> 40) * (1.0f / 16777216.0f);
}

typedef struct { float p; uint32_t i; } vo_pi;
static int cmp_desc(const void* a, const void* b) {
    const vo_pi* x = (const vo_pi*)a;
    const vo_pi* y = (const vo_pi*)b;
    if (x->p > y->p) return -1;
    if (x->p < y->p) return 1;
    return x->i < y->i ? -1 : (x->i > y->i ? 1 : 0); /* equal probabilities: lower index first */
}

/* src/runtime.rs:1092-1152.  The reference sorts with sort_unstable_by, which leaves the order of equal
 * probabilities open; this restatement (and the CUDA kernel) puts the lower index first.  `margin`, when not
 * NULL, receives the smallest distance of the two threshold decisions (cumulative >= top_p, running >= target)
 * from flipping: a caller comparing against an implementation that sums in another order can tell a genuine
 * mismatch from a rounding-level one. */
uint32_t vo_sample_top_p_f32(const float* logits, size_t n, float temperature, float top_p, float random_coin,
                             float* margin) {
    if (margin) *margin = INFINITY;
    if (temperature <= 1e-5f || top_p <= 0.0f) return vo_sample_argmax_f32(logits, n);
    const float inv_temp = 1.0f / temperature;
    float max_l = -INFINITY;
    for (size_t i = 0; i < n; ++i) {
        const float s = logits[i] * inv_temp;
        if (s > max_l) max_l = s;
    }
    vo_pi* a = (vo_pi*)malloc(n * sizeof(vo_pi));
    float sum_exp = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        const float e = expf(logits[i] * inv_temp - max_l);
        a[i].p = e;
        a[i].i = (uint32_t)i;
        sum_exp += e;
    }
    const float inv_sum = 1.0f / sum_exp;
    for (size_t i = 0; i < n; ++i) a[i].p *= inv_sum;
    qsort(a, n, sizeof(vo_pi), cmp_desc);
    float cum = 0.0f, m = INFINITY;
    size_t cutoff = 1;
    for (size_t k = 0; k < n; ++k) {
        const float before = cum;
        cum += a[k].p;
        cutoff = k + 1;
        if (cum >= top_p) { m = fminf(m, fminf(cum - top_p, top_p - before)); break; }
    }
    float coin = random_coin;
    if (coin < 0.0f) coin = 0.0f;
    if (coin > 0.9999f) coin = 0.9999f;
    const float target = coin * cum;
    float running = 0.0f;
    uint32_t pick = a[0].i;
    for (size_t k = 0; k < cutoff; ++k) {
        const float before = running;
        running += a[k].p;
        if (running >= target) { pick = a[k].i; m = fminf(m, fminf(running - target, target - before)); break; }
    }
    if (margin) *margin = m;
    free(a);
    return pick;
}

/* src/runners/tinystories_smollm.c:506-529: the emitted C99 twin walks the unsorted cumulative distribution. */
uint32_t vo_sample_top_p_c99(const float* logits, size_t n, float temperature, float top_p, float random_coin,
                             float* margin) {
    if (margin) *margin = INFINITY;
    if (temperature <= 1e-5f || top_p <= 0.0f) return vo_sample_argmax_f32(logits, n);
    const float inv_temp = 1.0f / temperature;
    float max_l = logits[0] * inv_temp;
    for (size_t v = 1; v < n; ++v) {
        const float val = logits[v] * inv_temp;
        if (val > max_l) max_l = val;
    }
    float sum_exp = 0.0f;
    for (size_t v = 0; v < n; ++v) sum_exp += expf(logits[v] * inv_temp - max_l);
    const float target = random_coin * top_p * sum_exp;
    float cum = 0.0f;
    for (size_t v = 0; v < n; ++v) {
        const float before = cum;
        cum += expf(logits[v] * inv_temp - max_l);
        if (cum >= target) {
            if (margin) *margin = fminf(cum - target, target - before) / sum_exp;
            return (uint32_t)v;
        }
    }
    return 0U;
}

/* ------------------------------------------------------------------------------------------ */
/* prompt-lookup speculative decoding                                                          */
/* ------------------------------------------------------------------------------------------ */

/* src/runners/velox_cuda_runner_k2.cu:1572-1611: the most recent earlier occurrence of the last trigram,
 * bigram or unigram of the history; the tokens that followed it are the draft (a unigram match drafts at
 * most 2 tokens when more were asked for). */
int vo_prompt_lookup_draft(const uint32_t* history, size_t history_len, uint32_t* draft, int max_draft) {
    if (history_len < 2 || max_draft <= 0) return 0;
    for (int n = 3; n >= 1; --n) {
        if (history_len < (size_t)(n + 1)) continue;
        const uint32_t* needle = history + history_len - n;
        for (long long i = (long long)(history_len - n - 1); i >= 0; --i) {
            int match = 1;
            for (int k = 0; k < n; ++k)
                if (history[i + k] != needle[k]) { match = 0; break; }
            if (!match) continue;
            const size_t start = (size_t)i + n;
            if (start < history_len - n) {
                int count = (int)((history_len - n) - start);
                const int limit = (n == 1 && max_draft > 2) ? 2 : max_draft;
                if (count > limit) count = limit;
                for (int d = 0; d < count; ++d) draft[d] = history[start + d];
                return count;
            }
        }
    }
    return 0;
}

/* The adaptive policy of the reference's speculative loop (src/runners/velox_cuda_runner_k2.cu:2160-2225):
 * an EMA of the per-step draft acceptance scales the draft width and, below the floor, pauses drafting for a
 * ladder of plain steps that doubles up to 64. */
void vo_spec_policy_init(vo_spec_policy* p, int max_draft_len, float ema_floor) {
    p->max_draft_len = max_draft_len;
    p->ema_floor = ema_floor;
    p->ema = 0.70f;
    p->plain_stride = 1;
    p->plain_since_spec = 0;
}
/* K drafted tokens are on offer with `remaining` tokens still wanted: returns how many to verify (0 = plain step). */
int vo_spec_policy_width(vo_spec_policy* p, int K, size_t remaining) {
    static const float thr[5] = {0.80f, 0.60f, 0.40f, 0.20f, 0.0f};
    static const float mul[5] = {1.0f, 0.75f, 0.50f, 0.25f, 0.0f};
    if ((size_t)K > remaining) K = (int)remaining;
    if (K > 0) {
        float k_mult = 0.0f;
        for (int i = 0; i < 5; ++i)
            if (p->ema >= thr[i]) { k_mult = mul[i]; break; }
        int k_cap = (int)((float)p->max_draft_len * k_mult * (0.4f + 0.6f * fminf(p->ema, 1.0f)));
        if (k_cap < 1) k_cap = 1;
        if (K > k_cap) K = k_cap;
        if ((size_t)K > remaining) K = (int)remaining;
    }
    int use_spec;
    if (p->ema >= p->ema_floor || K <= 0) {
        use_spec = K > 0;
        p->plain_since_spec = 0;
    } else if (p->plain_since_spec >= p->plain_stride) {
        use_spec = 1;
        p->plain_since_spec = 0;
        p->plain_stride = p->plain_stride < 64 ? p->plain_stride * 2 : 64;
    } else {
        use_spec = 0;
        p->plain_since_spec++;
    }
    return use_spec ? K : 0;
}
void vo_spec_policy_update(vo_spec_policy* p, int accepted, int K) {
    const float r = (float)accepted / (float)K;
    p->ema = (1.0f - 0.35f) * p->ema + 0.35f * r;
}

/* The speculative generation loop (src/runners/velox_cuda_runner_k2.cu:2166-2310) on the CPU engine: the
 * verify pass is the per-token forward step run over the candidate rows, so the tokens are those of plain
 * greedy decoding by construction; what this pins is the draft / accept bookkeeping. */
size_t vo_engine_generate_speculative(vo_engine* e, uint32_t seq, const uint32_t* prompt, size_t n_prompt, size_t n_new,
                                      int max_draft_len, float ema_floor, uint32_t* out_tokens, vo_spec_stats* st) {
    vo_spec_stats s;
    memset(&s, 0, sizeof(s));
    if (n_prompt == 0 || n_new == 0) { if (st) *st = s; return 0; }
    uint32_t* history = (uint32_t*)malloc((n_prompt + n_new + 16) * sizeof(uint32_t));
    uint32_t next = 0, pos = 0;
    for (size_t i = 0; i < n_prompt; ++i) { next = vo_engine_forward_step(e, seq, prompt[i], pos); pos++; }
    memcpy(history, prompt, n_prompt * sizeof(uint32_t));
    history[n_prompt] = next;
    size_t hist_len = n_prompt + 1, gen = 1;
    out_tokens[0] = next;
    vo_spec_policy pol;
    vo_spec_policy_init(&pol, max_draft_len, ema_floor);
    while (gen < n_new) {
        s.steps++;
        uint32_t draft[8];
        int K = vo_prompt_lookup_draft(history, hist_len, draft, max_draft_len);
        K = vo_spec_policy_width(&pol, K, n_new - gen);
        if (K == 0) {
            s.plain_steps++;
            next = vo_engine_forward_step(e, seq, next, pos);
            pos++;
            out_tokens[gen++] = next;
            history[hist_len++] = next;
            continue;
        }
        s.drafted += (uint64_t)K;
        const int B = K + 1;
        uint32_t cand[9];
        cand[0] = next;
        for (int i = 0; i < K; ++i) cand[i + 1] = draft[i];
        int accepted = 0;
        for (int t = 0; t < B && gen < n_new; ++t) {
            /* row t of the verify pass: candidate t at position pos + t (rows past a rejection are never looked at,
             * and their cache rows are overwritten when the sequence gets there) */
            const uint32_t winner = vo_engine_forward_step(e, seq, cand[t], pos + (uint32_t)t);
            if (t < B - 1) {
                if (winner == cand[t + 1]) {
                    accepted++;
                    s.accepted++;
                    out_tokens[gen++] = cand[t + 1];
                    history[hist_len++] = cand[t + 1];
                    if (gen == n_new) { next = cand[t + 1]; pos += (uint32_t)t + 1; }
                } else {
                    out_tokens[gen++] = winner;
                    history[hist_len++] = winner;
                    next = winner;
                    pos += (uint32_t)t + 1;
                    break;
                }
            } else {
                out_tokens[gen++] = winner;
                history[hist_len++] = winner;
                next = winner;
                pos += (uint32_t)B;
            }
        }
        vo_spec_policy_update(&pol, accepted, K);
    }
    s.ema_final = pol.ema;
    s.ladder_final = (uint32_t)pol.plain_stride;
    if (st) *st = s;
    free(history);
    return n_new;
}

/* ------------------------------------------------------------------------------------------ */
/* GGUF Q4_K / Q6_K -> reference q4 group-64                                                    */
/* ------------------------------------------------------------------------------------------ */
static void get_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
    if (j < 4) {
        *d = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}
static inline int rn_i(float v) { return (int)lrintf(v); }
static inline uint32_t pack8w(const uint32_t q[8]) {
    return (q[0] << 0) | (q[2] << 4) | (q[4] << 8) | (q[6] << 12) | (q[1] << 16) | (q[3] << 20) | (q[5] << 24) | (q[7] << 28);
}
/* 64 values -> 8 packed words + half2(scale, min): the re-quantization both unpack kernels of the reference share
 * (scale and minimum are used unrounded for the integers and stored rounded to half). */
static void requant64(uint32_t* words, uint16_t* scale_min, const float* vals, float grp_min, float grp_max) {
    const float sc = (grp_max > grp_min) ? ((grp_max - grp_min) / 15.0f) : 1e-5f;
    scale_min[0] = vo_f32_to_f16(sc);
    scale_min[1] = vo_f32_to_f16(grp_min);
    const float inv_sc = 1.0f / sc;
    for (int w = 0; w < 8; ++w) {
        uint32_t q[8];
        for (int k = 0; k < 8; ++k) {
            const int qi = rn_i((vals[w * 8 + k] - grp_min) * inv_sc);
            q[k] = (uint32_t)(qi < 0 ? 0 : (qi > 15 ? 15 : qi));
        }
        words[w] = pack8w(q);
    }
}

/* src/runners/velox_cuda_runner_k2.cu:211-276 (one 144-byte Q4_K super-block = 256 weights = 4 groups of 64). */
void vo_unpack_q4_k(uint32_t* words, uint16_t* scale_min, const uint8_t* src, size_t n_blocks) {
    for (size_t b = 0; b < n_blocks; ++b) {
        const uint8_t* blk = src + b * 144;
        uint16_t dh, mh;
        memcpy(&dh, blk, 2);
        memcpy(&mh, blk + 2, 2);
        const float fd = vo_f16_to_f32(dh), fdmin = vo_f16_to_f32(mh);
        const uint8_t* scales = blk + 4;
        const uint8_t* qs = blk + 16;
        for (int g = 0; g < 4; ++g) {
            uint8_t sc0, m0, sc1, m1u;
            get_scale_min_k4(2 * g, scales, &sc0, &m0);
            get_scale_min_k4(2 * g + 1, scales, &sc1, &m1u);
            const float d1 = fd * (float)sc0, m1 = fdmin * (float)m0, d2 = fd * (float)sc1, m2 = fdmin * (float)m1u;
            const uint8_t* gq = qs + g * 32;
            float vals[64], mn = 1e30f, mx = -1e30f;
            for (int l = 0; l < 32; ++l) {
                /* d * q - m: one fused multiply-add on the GPU the reference's kernel is compiled for */
                const float v0 = fmaf(d1, (float)(gq[l] & 0x0F), -m1);
                const float v1 = fmaf(d2, (float)(gq[l] >> 4), -m2);
                vals[l] = v0;
                vals[l + 32] = v1;
                if (v0 < mn) mn = v0;
                if (v0 > mx) mx = v0;
                if (v1 < mn) mn = v1;
                if (v1 > mx) mx = v1;
            }
            requant64(words + b * 32 + (size_t)g * 8, scale_min + (b * 4 + (size_t)g) * 2, vals, mn, mx);
        }
    }
}

/* src/runners/velox_cuda_runner_k2.cu:278-347 (one 210-byte Q6_K super-block = 256 weights). */
void vo_unpack_q6_k(uint32_t* words, uint16_t* scale_min, const uint8_t* src, size_t n_blocks) {
    for (size_t b = 0; b < n_blocks; ++b) {
        const uint8_t* blk = src + b * 210;
        const uint8_t* ql = blk;
        const uint8_t* qh = blk + 128;
        const int8_t* sc = (const int8_t*)(blk + 192);
        uint16_t dh;
        memcpy(&dh, blk + 208, 2);
        const float d = vo_f16_to_f32(dh);
        for (int n = 0; n < 2; ++n) {
            const uint8_t* ql_n = ql + n * 64;
            const uint8_t* qh_n = qh + n * 32;
            const int8_t* sc_n = sc + n * 8;
            float w128[128];
            for (int l = 0; l < 32; ++l) {
                const int is = l / 16;
                const int8_t q1 = (int8_t)((int8_t)((ql_n[l] & 0xF) | (((qh_n[l] >> 0) & 3) << 4)) - 32);
                const int8_t q2 = (int8_t)((int8_t)((ql_n[l + 32] & 0xF) | (((qh_n[l] >> 2) & 3) << 4)) - 32);
                const int8_t q3 = (int8_t)((int8_t)((ql_n[l] >> 4) | (((qh_n[l] >> 4) & 3) << 4)) - 32);
                const int8_t q4 = (int8_t)((int8_t)((ql_n[l + 32] >> 4) | (((qh_n[l] >> 6) & 3) << 4)) - 32);
                w128[l] = d * (float)sc_n[is] * (float)q1;
                w128[l + 32] = d * (float)sc_n[is + 2] * (float)q2;
                w128[l + 64] = d * (float)sc_n[is + 4] * (float)q3;
                w128[l + 96] = d * (float)sc_n[is + 6] * (float)q4;
            }
            for (int sub = 0; sub < 2; ++sub) {
                const int g = n * 2 + sub;
                const float* vals = w128 + sub * 64;
                float mn = vals[0], mx = vals[0];
                for (int i = 1; i < 64; ++i) {
                    if (vals[i] < mn) mn = vals[i];
                    if (vals[i] > mx) mx = vals[i];
                }
                requant64(words + b * 32 + (size_t)g * 8, scale_min + (b * 4 + (size_t)g) * 2, vals, mn, mx);
            }
        }
    }
}
