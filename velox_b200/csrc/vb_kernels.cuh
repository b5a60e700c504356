// Host-side launchers shared between the translation units of libvelox_b200.
#pragma once

#include "vb_internal.cuh"

namespace vb {

const char* last_error();
// Opt every kernel into the dynamic shared memory it may ask for (once per device, before any capture).
cudaError_t kernels_init();
cudaError_t gemv_init();
cudaError_t attn_init();

// vb_basic.cu
cudaError_t fill_normal(const LaunchCfg& lc, float* dst, uint64_t n, uint64_t seed, uint64_t stream_id, float mean, float std);
cudaError_t fill_normal_slice(const LaunchCfg& lc, float* dst, uint64_t rows, uint64_t cols, uint64_t full_cols, uint64_t r0,
                              uint64_t c0, uint64_t seed, uint64_t stream_id, float mean, float std);
cudaError_t quantize(const LaunchCfg& lc, void* data, void* scales, const float* src, int32_t fmt, uint64_t rows, uint64_t cols);
cudaError_t dequantize(const LaunchCfg& lc, float* dst, const void* data, const void* scales, int32_t fmt, uint64_t rows, uint64_t cols);
cudaError_t embed(const LaunchCfg& lc, float* dst, const uint32_t* tokens, const SeqState* state, const void* table,
                  const void* scales, int fmt, uint32_t d, uint32_t vocab, uint32_t batch);
cudaError_t rmsnorm(const LaunchCfg& lc, float* dst, const float* x, const void* w, int w_fmt, uint32_t dim, uint32_t batch, float eps);
cudaError_t rope(const LaunchCfg& lc, float* t, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta);
cudaError_t bias_rope_kv_append(const LaunchCfg& lc, float* q_out, const float* qkv, const SeqState* state, const void* bq,
                                const void* bk, const void* bv, int bias_fmt, __half* kv_layer, const int32_t* block_table,
                                uint32_t max_blocks, uint32_t Hq, uint32_t Hkv, uint32_t D, uint32_t block_tokens, float theta,
                                uint32_t batch);
cudaError_t argmax(const LaunchCfg& lc, uint32_t* out_token, const float* logits, uint32_t n, uint32_t batch, float* cand_v,
                   uint32_t* cand_i, SeqState* state, uint32_t* ring, uint32_t ring_slots);
uint32_t argmax_chunks(uint32_t n);

// vb_sample.cu: temperature + nucleus sampling, one block per sequence; `probs` = [batch][n] scratch.  The coin of a
// sequence comes from `coins[b]`, else (use_seed) from (seed, b, state[b].pos), else it is `coin`.
cudaError_t sample_top_p(const LaunchCfg& lc, uint32_t* out_token, const float* logits, float* probs, uint32_t n, uint32_t batch,
                         float temperature, float top_p, int mode, const float* coins, float coin, int use_seed, uint64_t seed,
                         SeqState* state, uint32_t* ring, uint32_t ring_slots);

// Peer-mapped receive regions of a tensor-parallel group (vb_tp.cu): base[r] is rank r's region as mapped here.
struct TpLinks {
    unsigned char* base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    uint32_t rank = 0, size = 1, max_batch = 0, max_pairs = 0;
    uint64_t epoch_off = 0, pair_off = 0, data_off = 0, bytes = 0;
    long long poll_clocks = 20000000000LL;  // limit of one poll in SM clocks (~10 s): covers host-side skew between ranks
};
void tp_links_layout(TpLinks* l, uint32_t rank, uint32_t size, uint32_t max_elems, uint32_t max_batch);
cudaError_t tp_epoch_advance(const LaunchCfg& lc, const TpLinks& l);
// `pushed`: the producing kernel already stored the partial into the peers' regions (TpPush); only poll and sum
// `state` != null: rows (of `row_elems` elements) of inactive slots take no part in the exchange
cudaError_t tp_reduce(const LaunchCfg& lc, const TpLinks& l, float* hidden, const float* partial, uint32_t n, uint32_t site,
                      uint32_t n_sites, uint32_t* err, bool pushed = false, const SeqState* state = nullptr, uint32_t row_elems = 0);
// Exchange `site` of a step: where the epilogue of a row-parallel product sends its output rows (pairs of rows,
// sequence-tagged 16-byte words, see vb_tp.cu) besides storing them locally.
struct TpPush {
    const TpLinks* links = nullptr;  // null: no push
    uint32_t site = 0, n_sites = 1;
    // != null: the product may also finish the exchange (gather the peers' rows, add everything onto this vector)
    float* reduce_hidden = nullptr;
    uint32_t* err = nullptr;
};
constexpr uint32_t TP_BUFS = 4;  // receive buffers used round-robin by consecutive exchange sites
cudaError_t tp_argmax(const LaunchCfg& lc, const TpLinks& l, const void* pairs, uint32_t batch, uint32_t site, uint32_t n_sites,
                      SeqState* state, uint32_t* ring, uint32_t ring_slots, uint32_t* err);
cudaError_t argmax_shard(const LaunchCfg& lc, void* pair_out, const float* logits, uint32_t n, uint32_t idx_offset, uint32_t batch,
                         float* cand_v, uint32_t* cand_i, SeqState* state);
cudaError_t argmax_pairs(const LaunchCfg& lc, const void* pairs, uint32_t n_ranks, uint32_t batch, SeqState* state, uint32_t* ring,
                         uint32_t ring_slots);

// vb_gemv.cu
// Epilogues of the matrix-vector kernels.
enum GemvEpilogue {
    EPI_STORE = 0,     // dst[b][o] = acc
    EPI_RESIDUAL = 1,  // dst[b][o] += acc                      (O-proj / down-proj + residual)
    EPI_SWIGLU = 2     // dst[b][o] = silu(acc_gate) * acc_up   (two matrices, same row index)
};
struct GemvArgs {
    float* dst = nullptr;            // [batch][dst_stride]
    const float* x = nullptr;        // [batch][in_dim] fp32
    WMat w;                          // [out_dim][in_dim]
    WMat w2;                         // second matrix for EPI_SWIGLU
    const void* norm_w = nullptr;    // != null: x is RMS-normalised with these weights first
    int norm_fmt = VB_FMT_F32;
    float eps = 0.0f;
    const SeqState* state = nullptr; // != null: inactive slots are skipped
    uint32_t batch = 1;
    uint32_t dst_stride = 0;         // elements between batch rows of dst (0 = out_dim)
    uint32_t dst_offset = 0;         // column offset inside dst
    int epilogue = EPI_STORE;
    uint32_t max_ring = 12;          // cap on the weight ring depth per warp
    TpPush push;                     // EPI_STORE only: also send the rows to the tensor-parallel peers
    bool* pushed = nullptr;          // out: set when the kernel that ran did send them
    bool* reduced = nullptr;         // out: set when it also finished the exchange (TpPush::reduce_hidden)
    unsigned long long* trace = nullptr;  // 3-slot timestamp record of this launch (tuned kernels only)
};
cudaError_t gemv(const LaunchCfg& lc, const GemvArgs& a, int path);

// vb_gemv_fast.cu
bool tile_q4_supported(uint32_t rows, uint32_t K);
cudaError_t tile_q4_swiglu(const LaunchCfg& lc, void* tiled, const void* canon, const void* canon_scales, uint32_t rows, uint32_t K,
                           int which);
extern bool fast_use_tma;
extern bool attn_use_mma;
extern bool attn_use_tcgen05;
cudaError_t fast_error_word(uint32_t** out);
cudaError_t fast_error_word_host(uint32_t** out);
cudaError_t tile_q4(const LaunchCfg& lc, void* tiled, void* tiled_scales, const void* canon, const void* canon_scales,
                    uint32_t rows, uint32_t K);

// vb_gemv_imma.cu
cudaError_t gemv_imma_init();
cudaError_t gemv_imma(const LaunchCfg& lc, const GemvArgs& a, bool* handled);
cudaError_t tile_i8_v3(const LaunchCfg& lc, void* blocks, void* scales, const void* canon, const void* canon_scales, uint32_t rows,
                       uint32_t K);
cudaError_t tile_i8_v3_swiglu(const LaunchCfg& lc, void* blocks, void* scales, const void* canon, const void* canon_scales, uint32_t rows,
                              uint32_t K, int which);
cudaError_t tile_q4_v3(const LaunchCfg& lc, void* tiled, const void* canon, const void* canon_scales, uint32_t rows, uint32_t K);
cudaError_t tile_q4_v3_swiglu(const LaunchCfg& lc, void* tiled, const void* canon, const void* canon_scales, uint32_t rows, uint32_t K,
                              int which);
extern bool imma_enabled;
extern bool imma_multirow;
extern int imma_pair_ring;
extern bool imma_spread;

// vb_gemm_tc.cu: multi-row products on the tcgen05 tensor cores (prefill chunks); the arguments are those of gemv(),
// `batch` = rows of x; the workspace holds the fp16 operands
cudaError_t gemm_tc_init();
extern bool gemm_tc_wide;
extern bool gemm_tc_split_k;
uint64_t gemm_tc_operand_bytes(uint32_t out_dim, uint32_t in_dim, uint32_t n_rows, bool dual);
uint64_t gemm_tc_workspace_zero_bytes();  // leading bytes of the workspace that must be zero before the first call
extern bool gemm_tc_two_per_sm;
cudaError_t weights_to_f16(const LaunchCfg& lc, void* dst, const WMat& m, void* dst_lo = nullptr);
bool gemm_tc_weights_inexact(int32_t fmt);
extern int gemm_tc_split;
bool gemm_tc_supported(const GemvArgs& a);
uint64_t gemm_tc_workspace_bytes(uint32_t out_dim, uint32_t in_dim, uint32_t n_rows, bool dual);
// counters_zeroed: the caller zeroed the head of the workspace once (allows the split-K path)
cudaError_t gemm_tc(const LaunchCfg& lc, const GemvArgs& a, void* workspace, uint64_t workspace_bytes, bool counters_zeroed = false);

// vb_gemm_i8.cu: decode batches (<= 32 rows) over int8 per-channel weights on the integer tensor cores, weights read
// where they lie (one byte per weight), exact arithmetic; workspace head (gemm_i8_workspace_zero_bytes) zero before first use
extern bool gemm_i8_enabled;
extern bool gemm_i8_tiles;
extern bool gemm_i8_half_ring;
bool gemm_i8_supported(const GemvArgs& a);
// absorbed multi-head latent attention on tcgen05 (vb_mla_tc.cu); `extra` = status word + bf16 copy of q, 16-byte aligned
extern bool mla_use_tc;
uint64_t mla_tc_extra_scratch_bytes(uint32_t batch, uint32_t n_heads);
cudaError_t mla_decode_tc(const LaunchCfg& lc, const float* q, const void* cache, const uint32_t* ctx_len, float* partial, void* extra,
                          uint32_t batch, uint32_t n_heads, uint32_t n_splits, uint32_t split_tokens, uint64_t cache_stride, float scale);
uint64_t gemm_i8_workspace_bytes(uint32_t in_dim);
// int8 [rows][K] -> tile-major copy in shared-memory order (WMat::i8_tiles); K a multiple of 128
uint64_t gemm_i8_tiles_bytes(uint32_t rows, uint32_t K);
cudaError_t gemm_i8_make_tiles(const LaunchCfg& lc, void* dst, const void* src_i8, uint32_t rows, uint32_t K);
inline uint64_t gemm_i8_workspace_zero_bytes() { return 64 * 1024; }
cudaError_t gemm_i8(const LaunchCfg& lc, const GemvArgs& a, void* workspace, uint64_t workspace_bytes, bool counters_zeroed);

// vb_attn.cu
struct AttnArgs {
    float* out = nullptr;          // [batch][Hq*D]
    const float* q = nullptr;      // [batch][Hq*D] (RoPE applied); unused when qkv_raw is given
    // fused mode (paged fp16 cache, Hq/Hkv <= 8): raw projections [batch][(Hq+2Hkv)*D]; the kernel adds the
    // biases, applies RoPE at the sequence's position and appends K/V to the cache before attending
    const float* qkv_raw = nullptr;
    const void *bq = nullptr, *bk = nullptr, *bv = nullptr;
    int bias_fmt = VB_FMT_F32;
    const float* rope_inv_freq = nullptr;  // [D/2], 1/theta^(2j/D) (device)
    const float* rope_inv_freq_host = nullptr;  // the same table on the host: travels as kernel parameters (no load)
    const void* k = nullptr;       // contiguous: [seq][Hkv*D]; paged: the layer's pool
    const void* v = nullptr;       // contiguous only
    int kv_fp16 = 0;               // element type of the cache
    const int32_t* block_table = nullptr;  // != null: paged
    uint32_t max_blocks = 0, block_tokens = 16;
    const SeqState* state = nullptr;  // paged: seq_len = state[b].pos + 1
    uint32_t pos = 0;                 // contiguous: attends [0..pos]
    uint32_t Hq = 0, Hkv = 0, D = 0, batch = 1;
    uint32_t max_splits = 1;       // grid size along the context (fixed per context so that graphs replay)
    uint32_t tokens_per_split = 32; // multiple of block_tokens
    unsigned long long* trace = nullptr;
    uint32_t* err = nullptr;       // device word that a bounded wait sets when it runs out
    float* scratch = nullptr;      // attn_scratch_floats(): partials, then the split counters (zero before the first launch)
    // paged fp16 pool as a tiled-TMA tensor map (attn_make_kv_map; a CUtensorMap on the host) and the row of that map
    // where this layer's part of the pool begins; without it the tensor-core path is not taken
    const void* kv_map = nullptr;
    uint32_t kv_map_row0 = 0;
};
// 128 bytes, 64-byte aligned: a tensor map over the whole pool as a matrix of token rows, [rows][D] fp16, boxes of
// [block_tokens = 16 rows][64 columns] with the 128-byte swizzle.  False when the driver entry point is missing.
bool attn_make_kv_map(void* map_out, const void* pool, uint64_t rows, uint32_t D);
uint64_t attn_scratch_floats(uint32_t Hq, uint32_t D, uint32_t batch, uint32_t max_splits);
uint32_t attn_pick_splits(uint32_t max_seq);
uint32_t attn_tokens_per_split(uint32_t max_seq);
cudaError_t attention(const LaunchCfg& lc, const AttnArgs& a);
cudaError_t attention_ex(const LaunchCfg& lc, const AttnArgs& a, float scale, size_t kv_batch_stride);

// vb_attn_prefill.cu: causal attention of a prefill chunk (rows = consecutive positions of one sequence)
bool attention_prefill_supported(uint32_t Hq, uint32_t Hkv, uint32_t D);
cudaError_t attention_prefill(const LaunchCfg& lc, float* out, const float* q, const __half* kv_layer, const int32_t* table_row,
                              uint32_t first, uint32_t n, uint32_t Hq, uint32_t Hkv, uint32_t D, uint32_t block_tokens);

// vb_mla.cu
cudaError_t mla_absorbed(const LaunchCfg& lc, float* dst, const float* x, const float* w_norm, const float* w_dkv,
                         const float* w_absq, const float* w_abso, float* pool, uint32_t step, uint32_t hidden,
                         uint32_t latent, uint32_t max_seq, float eps, float* scratch);
uint64_t mla_scratch_floats(uint32_t hidden, uint32_t latent);

}  // namespace vb
