/*
 * velox_oracle.h -- CPU restatement of the Velox decode step (TEST INFRASTRUCTURE ONLY).
 *
 * This is the checker, never the product: only the test-suite, the smoke check and the
 * benchmark's CPU-baseline leg may load it.  Nothing in the shipped library links it.
 *
 * Every function restates one function of the reference's CPU runtime
 * (src/runtime.rs, and its emitted twin src/runners/tinystories_smollm.c); the
 * citation is given beside each declaration.  Arithmetic is fp32 throughout, with the
 * reference's accumulation order (8 FMA lanes + its horizontal-sum tree for matrix-vector
 * products, sequential sums elsewhere), so on SmolLM-135M shapes it reproduces the
 * compiled reference bit for bit.
 */
#ifndef VELOX_ORACLE_H
#define VELOX_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Weight storage formats (same numbering as VB_FMT_* in include/velox_b200.h). */
enum {
    VO_FMT_F32 = 0,
    VO_FMT_F16 = 1,
    VO_FMT_BF16 = 2,
    VO_FMT_Q4G32 = 3,    /* symmetric int4, groups of 32 along `in`, one fp16 scale per group */
    VO_FMT_Q4G64REF = 4, /* reference-native asymmetric int4, groups of 64, half2(scale,min)   */
    VO_FMT_I8PC = 5      /* symmetric int8, one fp16 scale per output channel                  */
};

/* Tensor roles (same numbering as VB_ROLE_* in include/velox_b200.h). */
enum {
    VO_ROLE_EMBED = 0, VO_ROLE_ATTN_NORM = 1, VO_ROLE_WQ = 2, VO_ROLE_WK = 3, VO_ROLE_WV = 4,
    VO_ROLE_WO = 5, VO_ROLE_MLP_NORM = 6, VO_ROLE_WGATE = 7, VO_ROLE_WUP = 8, VO_ROLE_WDOWN = 9,
    VO_ROLE_FINAL_NORM = 10, VO_ROLE_LM_HEAD = 11, VO_ROLE_BQ = 12, VO_ROLE_BK = 13, VO_ROLE_BV = 14,
    /* reference absorbed-MLA block (src/runtime.rs:944-1044) */
    VO_ROLE_MLA_NORM = 15, VO_ROLE_MLA_WDKV = 16, VO_ROLE_MLA_WABSQ = 17, VO_ROLE_MLA_WABSO = 18,
    VO_ROLE_COUNT = 19
};

/* ---- scalar conversions (IEEE binary16 / bfloat16, round-to-nearest-even) ---------------- */
uint16_t vo_f32_to_f16(float f);
float    vo_f16_to_f32(uint16_t h);
uint16_t vo_f32_to_bf16(float f);
float    vo_bf16_to_f32(uint16_t h);

/* ---- deterministic synthetic inputs ------------------------------------------------------ */
/* Counter-based generator shared bit-for-bit with the CUDA library (vb_fill_normal):
 * value i of (seed, stream) = (sum of twelve 16-bit hash lanes - 393210) * (std / 65536).   */
void     vo_fill_normal(float* dst, size_t n, uint64_t seed, uint64_t stream, float mean, float std);
void     vo_fill_tokens(uint32_t* dst, size_t n, uint64_t seed, uint64_t stream, uint32_t vocab);
uint64_t vo_hash64(uint64_t seed, uint64_t stream, uint64_t counter);

/* ---- quantizers / dequantizers (the "Dequant contract") ---------------------------------- */
/* Symmetric int4 g32: scale=h(max|w|/7); n=clamp(rn(w/scale)+8,0,15); value=(n-8)*scale.
 * Dequant formula pinned by tests/empirical_challenge_phase2/test3_marlin_lop3_dequant.cu:42,98-105
 * and src/codegen.rs:2778.  Nibble order per 8 elements follows src/codegen.rs:2363-2364. */
void vo_quantize_q4g32(uint32_t* packed, uint16_t* scales, const float* w, size_t rows, size_t cols);
void vo_dequant_q4g32(float* dst, const uint32_t* packed, const uint16_t* scales, size_t rows, size_t cols);
/* Reference-native q4 group-64 (src/codegen.rs:2337-2369 quantize, :2248-2265/:2381-2410 dequant). */
void vo_quantize_q4g64ref(uint32_t* packed, uint16_t* scale_min, const float* w, size_t rows, size_t cols);
void vo_dequant_q4g64ref(float* dst, const uint32_t* packed, const uint16_t* scale_min, size_t rows, size_t cols);
/* int8 per output channel: scale=h(max|w|/127); q=clamp(rn(w/scale),-127,127); value=q*scale. */
void vo_quantize_i8pc(int8_t* q, uint16_t* scales, const float* w, size_t rows, size_t cols);
void vo_dequant_i8pc(float* dst, const int8_t* q, const uint16_t* scales, size_t rows, size_t cols);

/* ---- primitives --------------------------------------------------------------------------- */
/* src/runtime.rs:588-601 */
void vo_rmsnorm_f32(float* dst, const float* x, const float* w, size_t dim, float eps);
/* src/runtime.rs:623-697,702-740 (AVX2 4-row kernel: 8 FMA lanes, hsum tree, scalar tail) */
void vo_matmul_transposed_f32(float* dst, const float* x, const float* w, size_t in_dim, size_t out_dim);
/* same product with the weight dequantized on the fly (any VO_FMT_*) */
void vo_matvec_fmt(float* dst, const float* x, const void* w, const void* scales, int fmt,
                   size_t in_dim, size_t out_dim);
/* src/runtime.rs:745-768 */
void vo_rope_rotate_half_f32(float* t, size_t n_heads, size_t head_dim, size_t pos, float theta);
/* src/runtime.rs:772-831 (two-pass softmax) */
void vo_gqa_attention_step_f32(float* out, float* scores, const float* q, const float* k_layer,
                               const float* v_layer, size_t n_q, size_t n_kv, size_t head_dim, size_t pos);
/* src/runtime.rs:1048-1073 */
void vo_swiglu_mlp_residual_f32(float* hidden, float* gate, float* up, float* down, const float* nx,
                                const float* wg, const float* wu, const float* wd, size_t d, size_t ffn);
/* src/runtime.rs:1078-1088 (strict >, start at -inf: first index wins ties, NaN never wins) */
uint32_t vo_sample_argmax_f32(const float* logits, size_t n);
/* src/runtime.rs:944-1044 (single-head latent attention, online softmax) */
void vo_mla_absorbed_step_f32(float* dst, const float* x, const float* w_norm, const float* w_dkv,
                              const float* w_absq, const float* w_abso, float* latent_pool_layer,
                              size_t step, size_t hidden, size_t latent, size_t max_seq, float eps);

/* ---- engine: src/runtime.rs:1229-1502 (forward_step :1328-1451) -------------------------- */
typedef struct vo_config {
    uint32_t vocab, d_model, n_layers, n_q_heads, n_kv_heads, head_dim, ffn_dim, max_seq_len;
    float    rms_eps, rope_theta;
    uint32_t qkv_bias;   /* q=(x.Wq)+b_q etc. before RoPE (examples/qwen2_5_7b.vlx:72-74)        */
    uint32_t n_seqs;     /* independent sequences, each with its own fp32 KV cache              */
    uint32_t mla_latent; /* >0: every layer is the reference absorbed-MLA block + SwiGLU FFN    */
} vo_config;

typedef struct vo_engine vo_engine;

vo_engine* vo_engine_create(const vo_config* cfg);
void       vo_engine_destroy(vo_engine* e);
/* Borrows the pointers; `layer` ignored for EMBED/FINAL_NORM/LM_HEAD.  Norms/biases: F32 or F16. */
int        vo_engine_set_tensor(vo_engine* e, int role, int layer, const void* data, const void* scales, int fmt);
/* One token of sequence `seq` at position `pos`; returns the greedy token, logits in vo_engine_logits. */
uint32_t   vo_engine_forward_step(vo_engine* e, uint32_t seq, uint32_t token, uint32_t pos);
const float* vo_engine_logits(const vo_engine* e);
const float* vo_engine_hidden(const vo_engine* e);
/* src/runtime.rs:1456-1490: prefill token by token, then greedy decode; returns n_new. */
size_t     vo_engine_generate_greedy(vo_engine* e, uint32_t seq, const uint32_t* prompt, size_t n_prompt,
                                     size_t n_new, uint32_t* out_tokens);
int        vo_num_threads(void);
void       vo_set_num_threads(int n);

/* ---- rows next to the decode step (velox_oracle_next.c) ----------------------------------- */
/* src/runtime.rs:1092-1152: temperature + nucleus sampling; equal probabilities sort lower index first.
 * `margin` (may be NULL): how far the two threshold decisions were from flipping. */
uint32_t vo_sample_top_p_f32(const float* logits, size_t n, float temperature, float top_p, float random_coin, float* margin);
/* src/runners/tinystories_smollm.c:506-529: the emitted C99 twin (unsorted cumulative walk). */
uint32_t vo_sample_top_p_c99(const float* logits, size_t n, float temperature, float top_p, float random_coin, float* margin);
/* The coin both engines draw for (seed, slot, position): the reference leaves the coin to its caller. */
float    vo_sample_coin(uint64_t seed, uint32_t slot, uint32_t pos);

/* src/runners/velox_cuda_runner_k2.cu:1572-1611: prompt-lookup drafting; returns the draft length. */
int      vo_prompt_lookup_draft(const uint32_t* history, size_t history_len, uint32_t* draft, int max_draft);
/* src/runners/velox_cuda_runner_k2.cu:2160-2225, :2298-2303: adaptive draft-width policy. */
typedef struct vo_spec_policy {
    int   max_draft_len;
    float ema_floor, ema;
    int   plain_stride, plain_since_spec;
} vo_spec_policy;
void     vo_spec_policy_init(vo_spec_policy* p, int max_draft_len, float ema_floor);
int      vo_spec_policy_width(vo_spec_policy* p, int K, size_t remaining);
void     vo_spec_policy_update(vo_spec_policy* p, int accepted, int K);
typedef struct vo_spec_stats {
    uint64_t steps, plain_steps, drafted, accepted;
    float    ema_final;
    uint32_t ladder_final;
} vo_spec_stats;
/* src/runners/velox_cuda_runner_k2.cu:2166-2310: the speculative generation loop over the CPU engine. */
size_t   vo_engine_generate_speculative(vo_engine* e, uint32_t seq, const uint32_t* prompt, size_t n_prompt, size_t n_new,
                                        int max_draft_len, float ema_floor, uint32_t* out_tokens, vo_spec_stats* st);

/* src/runners/velox_cuda_runner_k2.cu:200-347: GGUF Q4_K (144-byte) / Q6_K (210-byte) super-blocks of 256 weights ->
 * the reference's q4 group-64 format: 32 packed words + 4 half2(scale,min) per block. */
void     vo_unpack_q4_k(uint32_t* words, uint16_t* scale_min, const uint8_t* src, size_t n_blocks);
void     vo_unpack_q6_k(uint32_t* words, uint16_t* scale_min, const uint8_t* src, size_t n_blocks);

/* ---- multi-head latent attention, absorbed and explicit (velox_oracle_mla.c; parity unpinned beyond the
 * single-head block: see that file's header) --------------------------------------------------------------------- */
typedef struct vo_mla_block {
    uint32_t d_model, n_heads, q_lora, kv_lora, nope_dim, rope_dim, v_dim;
    float    eps, theta;
    const float *w_norm, *w_dq, *w_uq, *w_qr, *w_dkv, *w_kr, *w_uk, *w_uv, *w_o;
} vo_mla_block;
void vo_mla_step_absorbed(const vo_mla_block* m, float* dst, const float* x, float* cache, size_t pos, int cache_bf16,
                          float* q_cat_out, float* ctx_out);
void vo_mla_step_explicit(const vo_mla_block* m, float* dst, const float* x, float* cache, size_t pos, int cache_bf16);
void vo_mla_core(float* out, const float* q_cat, const float* cache, size_t n_heads, size_t dc, size_t dr, size_t n_rows, float scale);

#ifdef __cplusplus
}
#endif
#endif
