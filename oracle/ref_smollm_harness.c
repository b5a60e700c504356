/*
 * ref_smollm_harness.c -- Linux host for the reference's own emitted C99 model
 * (TEST INFRASTRUCTURE ONLY; built into oracle/_ref/, never shipped, never copied).
 *
 * The reference's checked-in compiler output src/runners/tinystories_smollm.c is compiled
 * UNMODIFIED from where it lies: this file #includes it by the path given on the command
 * line (-DVELOX_REF_SMOLLM_C="\"...\"").  The reference's own host, velox_c99_runner.c, needs
 * <windows.h>; what it does around the model (arena allocation at the emitted sizes, weights at
 * the emitted offsets, tied head, prefill token by token then decode: velox_c99_runner.c:210-217,
 * :342-368) is restated here behind a small C ABI so that Python can drive it.
 */
#include VELOX_REF_SMOLLM_C

#include <stdlib.h>
#include <string.h>

typedef struct refsm {
    VeloxArenaContext ctx;
    uint8_t* weights;
    uint8_t* kv;
    uint8_t* act;
    uint32_t ring[1024];
} refsm;

refsm* refsm_create(void) {
    refsm* r = (refsm*)calloc(1, sizeof(refsm));
    if (!r) return NULL;
    r->weights = (uint8_t*)calloc(VELOX_WEIGHT_ARENA_BYTES, 1);
    r->kv = (uint8_t*)calloc(VELOX_KV_CACHE_POOL_BYTES, 1);
    r->act = (uint8_t*)calloc(VELOX_ACTIVATION_ARENA_BYTES, 1);
    if (!r->weights || !r->kv || !r->act) { free(r->weights); free(r->kv); free(r->act); free(r); return NULL; }
    r->ctx.weight_arena = r->weights;
    r->ctx.kv_cache_pool = r->kv;
    r->ctx.activation_arena = r->act;
    r->ctx.host_pinned_ring = r->ring;
    return r;
}

void refsm_destroy(refsm* r) {
    if (!r) return;
    free(r->weights); free(r->kv); free(r->act); free(r);
}

/* role numbering of velox_oracle.h; returns the fp32 weight slab the emitted code reads */
float* refsm_weight_ptr(refsm* r, int role) {
    uint64_t off;
    switch (role) {
    case 0: off = VELOX_W_OFFSET_W_EMBED; break;
    case 1: off = VELOX_W_OFFSET_W_ATTN_NORM; break;
    case 2: off = VELOX_W_OFFSET_W_Q; break;
    case 3: off = VELOX_W_OFFSET_W_K; break;
    case 4: off = VELOX_W_OFFSET_W_V; break;
    case 5: off = VELOX_W_OFFSET_W_OUT; break;
    case 6: off = VELOX_W_OFFSET_W_MLP_NORM; break;
    case 7: off = VELOX_W_OFFSET_W_GATE; break;
    case 8: off = VELOX_W_OFFSET_W_UP; break;
    case 9: off = VELOX_W_OFFSET_W_DOWN; break;
    case 10: off = VELOX_W_OFFSET_W_FINAL_NORM; break;
    case 11: off = VELOX_W_OFFSET_W_HEAD; break;
    default: return NULL;
    }
    return (float*)(r->weights + off);
}

uint32_t refsm_prefill(refsm* r, uint32_t token, uint64_t step) {
    return velox_SmolLM_135M_prefill(&r->ctx, token, (size_t)step, 1ULL);
}
uint32_t refsm_decode(refsm* r, uint32_t token, uint64_t step) {
    return velox_SmolLM_135M_decode(&r->ctx, token, (size_t)step, 1ULL);
}
/* logits live at activation offset 0 after either entry point (tinystories_smollm.c:596,668) */
const float* refsm_logits(const refsm* r) { return (const float*)r->act; }
void refsm_reset_kv(refsm* r) { memset(r->kv, 0, VELOX_KV_CACHE_POOL_BYTES); }

/* velox_c99_runner.c:342-368: prompt through prefill one token at a time, then decode. */
uint64_t refsm_generate(refsm* r, const uint32_t* prompt, uint64_t n_prompt, uint64_t n_new, uint32_t* out) {
    uint32_t next = 0;
    uint64_t pos = 0;
    for (uint64_t i = 0; i < n_prompt; ++i) { next = refsm_prefill(r, prompt[i], pos); pos++; }
    if (n_new == 0) return 0;
    out[0] = next;
    for (uint64_t s = 1; s < n_new; ++s) { next = refsm_decode(r, next, pos); pos++; out[s] = next; }
    return n_new;
}

/* the reference's static primitives, exported so the restatement can be checked one by one */
void refsm_rmsnorm(float* dst, const float* x, const float* w, uint64_t dim, float eps) {
    velox_c99_rmsnorm_f32(dst, x, w, (size_t)dim, eps);
}
void refsm_matmul_vec(float* dst, const float* x, const float* w, uint64_t in_dim, uint64_t out_dim) {
    velox_c99_matmul_vec_f32(dst, x, w, (size_t)in_dim, (size_t)out_dim);
}
void refsm_rope(float* t, uint64_t heads, uint64_t head_dim, uint64_t pos, float theta) {
    velox_c99_rope_rotate_half_in_place_f32(t, (size_t)heads, (size_t)head_dim, (size_t)pos, theta);
}
void refsm_gqa(float* out, float* scores, const float* q, const float* k, const float* v,
               uint64_t nq, uint64_t nkv, uint64_t hd, uint64_t pos) {
    velox_c99_gqa_attention_step_f32(out, scores, q, k, v, (size_t)nq, (size_t)nkv, (size_t)hd, (size_t)pos);
}
uint32_t refsm_argmax(const float* logits, uint64_t n) { return velox_c99_sample_argmax_f32(logits, (size_t)n); }
uint32_t refsm_sample_top_p(const float* logits, uint64_t n, float temperature, float top_p, float coin) {
    return velox_c99_sample_top_p_f32(logits, (size_t)n, temperature, top_p, coin);
}
/* hidden 576, latent 512, max_seq 2048 are compiled into the emitted function */
void refsm_mla(float* dst, const float* x, const float* w_norm, const float* w_dkv, const float* w_q,
               const float* w_o, float* pool, uint64_t layer, uint64_t step, float eps) {
    velox_c99_fused_mla_absorbed_attn(dst, x, w_norm, w_dkv, w_q, w_o, pool, (size_t)layer, (size_t)step, eps);
}
uint64_t refsm_dim(int which) {
    switch (which) {
    case 0: return VELOX_MODEL_HIDDEN_DIM;
    case 1: return VELOX_MODEL_INTERMEDIATE_DIM;
    case 2: return VELOX_MODEL_NUM_LAYERS;
    case 3: return VELOX_MODEL_NUM_HEADS;
    case 4: return VELOX_MODEL_NUM_KV_HEADS;
    case 5: return VELOX_MODEL_HEAD_DIM;
    case 6: return VELOX_MODEL_VOCAB_SIZE;
    case 7: return VELOX_MODEL_MAX_SEQ_LEN;
    default: return 0;
    }
}
int refsm_num_threads(void) {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}
