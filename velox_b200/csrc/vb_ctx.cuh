// The decode context behind the C ABI (vb_ctx) and the pieces of the engine that the feature files share:
// launch sequence of a step, chunk buffers, sampling state.  Defined in vb_engine.cu.
#pragma once

#include <vector>

#include "vb_internal.cuh"
#include "vb_kernels.cuh"

namespace vb {

constexpr uint32_t RING_SLOTS = 1024;  // VELOX_HOST_RING_SLOTS (src/codegen.rs:1022)

struct Tensor {
    WMat m;
    bool loaded = false;
};

}  // namespace vb

using namespace vb;

struct vb_ctx {
    vb_model_desc d;
    int device = 0;
    cudaStream_t stream = nullptr;
    uint64_t launches = 0;
    int gemv_path = 1;
    bool use_pdl = true;
    bool fuse_append = true;
    unsigned long long* trace = nullptr;  // [TRACE_MAX][4] device timestamps when the "trace" option is on
    uint32_t trace_n = 0;
    float* rope_inv_freq = nullptr;  // [head_dim/2]
    std::vector<float> rope_inv_freq_host;

    // derived
    uint32_t qdim = 0, kvdim = 0, qkv_rows = 0, max_blocks = 0, n_blocks = 0, n_splits = 1, tokens_per_split = 32;
    // this rank's shard (tensor parallel; equal to the whole model when tp_size == 1):
    // query/KV heads, FFN columns [ffn_off, ffn_off + ffn) in whole 128-column blocks, vocabulary rows
    uint32_t hq = 0, hkv = 0, ffn = 0, ffn_off = 0, vocab = 0, vocab_off = 0;
    void* nccl = nullptr;                 // communicator of the TP group
    TpLinks links;                        // NVLink peer mappings (vb_tp_p2p_open); used instead of NCCL when open
    bool links_open = false, use_links = true, links_standin = false;
    bool tp_fused_push = true;            // row-parallel products send their rows to the peers from their own epilogue
    bool tp_fused_reduce = true;          // ... and gather the peers' copies of their own rows: no exchange kernel at all
    uint32_t ring_role[4] = {0, 0, 0, 0};   // per product (qkv, o, gate/up, down): 0 = gemv_ring
    uint32_t gemv_ring = 4, head_ring = 4;  // weight ring depth of the int4 kernel for the layers / the head (GemvArgs::max_ring)
    uint32_t* err_word = nullptr;         // device word that bounded waits set when they run out
    float* partial = nullptr;             // [max_batch][d_model] row-parallel partial sums (all-reduced in place)
    unsigned char* tp_pair = nullptr;     // [max_batch] (value, index) of this rank's best logit
    unsigned char* tp_pairs = nullptr;    // [tp_size][max_batch] gathered

    // weight arena (execution order, 256-byte aligned slabs)
    uint8_t* arena = nullptr;
    uint64_t arena_bytes = 0;
    std::vector<Tensor> t;  // [role][layer]

    // paged KV pool: per layer [block][K|V][kv_head][block_tokens][D] fp16
    __half* kv_pool = nullptr;
    uint64_t kv_layer_elems = 0;
    alignas(64) unsigned char kv_map[128] = {};  // tiled-TMA tensor map over the whole KV pool as [token rows][head_dim] (attn_make_kv_map)
    bool kv_map_ok = false;
    int32_t* block_table_dev = nullptr;
    std::vector<int32_t> block_table_host;
    std::vector<int32_t> free_blocks;
    std::vector<uint32_t> slot_blocks;  // blocks held per slot
    // host-side upper bound of every slot's device position (decode steps advance it without reading the device)
    // and whether the slot may be active: vb_decode_run refuses steps that could leave a reservation
    std::vector<uint32_t> pos_hi;
    std::vector<uint8_t> maybe_active;

    // device state
    SeqState* state = nullptr;     // decode state, one per slot
    SeqState* pf_state = nullptr;  // prefill state (only the slot being prefilled is active)
    std::vector<SeqState> state_host;
    uint32_t* ring_host = nullptr;  // mapped pinned [max_batch][RING_SLOTS]
    uint32_t* ring_dev = nullptr;
    uint32_t* pf_tokens = nullptr;  // device copy of the prompt being prefilled
    uint32_t pf_tokens_cap = 0;
    // chunked prefill: `prefill_chunk` prompt tokens go through the layers together as rows of one step (weights are
    // read once per chunk by the batched kernels); all rows live on the prefilled sequence's KV blocks
    uint32_t prefill_chunk = 16;
    SeqState* pfc_state = nullptr;        // [chunk]
    int32_t* pfc_table = nullptr;         // [chunk][max_blocks], every row = the sequence's block-table row
    float *pfc_hidden = nullptr, *pfc_qkv = nullptr, *pfc_q = nullptr, *pfc_attn = nullptr, *pfc_act = nullptr;
    uint32_t pfc_rows = 0;                // rows the buffers above hold
    // prompts of at least `prefill_gemm_min` tokens: chunks of up to `prefill_rows` tokens whose four products per layer
    // run on the tcgen05 tensor cores (vb_gemm_tc.cu); the workspace holds their fp16 operands
    bool prefill_gemm = true;
    bool decode_gemm = false;   // decode steps of wide batches through the same tensor-core GEMMs (one row per slot)
    bool decode_gemm_auto = false;  // switched on by vb_create, not by the caller: falls back silently when unsupported
    bool prefill_flash = true;  // causal tile attention for those chunks (vb_attn_prefill.cu) instead of one launch row per token
    uint32_t prefill_rows = 2048, prefill_gemm_min = 48;
    void* tc_ws = nullptr;
    uint64_t tc_ws_bytes = 0;
    void* i8_tiles_pool = nullptr;  // tile-major int8 copies of the layer matrices and the head for those products (WMat::i8_tiles)
    bool i8_tiles_tried = false;
    void* i8_ws = nullptr;      // workspace of the int8 tensor-core products of decode batches (x planes, split-K partials)
    uint64_t i8_ws_bytes = 0;
    // resident fp16 copies of the layer matrices for those products, made once when they fit `tc_resident_gb`
    // (HBM is plentiful: 14 GB for an 8B model); otherwise every call converts into the workspace
    void* f16_pool = nullptr;
    uint32_t tc_resident_gb = 40;
    bool f16_tried = false;

    // activations
    float *hidden = nullptr, *qkv = nullptr, *q = nullptr, *attn_out = nullptr, *act = nullptr, *logits = nullptr;
    float* attn_scratch = nullptr;
    float* cand_v = nullptr;
    uint32_t* cand_i = nullptr;

    // sampler: temperature <= 1e-5 or top_p <= 0 means greedy (the reference's rule, src/runtime.rs:1100)
    float sample_temperature = 0.0f, sample_top_p = 0.0f;
    int sample_mode = 0;
    uint64_t sample_seed = 0;
    float* sample_probs = nullptr;  // [max_batch][vocab] scratch of the sampling kernel

    // speculative verify pass (vb_spec.cu): logits / argmax candidates of up to 8 rows, candidate and winner tokens
    float* spec_logits = nullptr;
    float* spec_cand_v = nullptr;
    uint32_t* spec_cand_i = nullptr;
    uint32_t* spec_tokens = nullptr;

    cudaGraph_t graph = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
    uint64_t graph_nodes = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;

    Tensor& tensor(int role, int layer) { return t[(size_t)role * (d.n_layers ? d.n_layers : 1) + (size_t)layer]; }
};


namespace vb {

// Activation buffers and block table one launch sequence works on: the context's own (decode, one row per slot)
// or the prefill chunk's (one row per prompt token of the chunk, all rows on the same sequence's KV blocks).
struct StepIO {
    float *hidden, *qkv, *q, *attn_out, *act, *logits;
    const int32_t* block_table;
    uint32_t B;
    bool fused_append;  // false: K/V of all rows are appended by a kernel of their own before attention
    void* tc_ws = nullptr;  // != null: the layer products run as tensor-core GEMMs with this workspace
    uint64_t tc_ws_bytes = 0;
    void* i8_ws = nullptr;  // != null: decode batches over int8 weights take the integer tensor-core kernel
    uint64_t i8_ws_bytes = 0;
    uint32_t first = 0;     // tensor-core chunks: position of row 0 (row j is position first + j of one sequence)
    bool causal_chunk = false;  // rows are consecutive positions of one sequence (prefill chunk), not one row per slot
};

template <typename T>
inline int32_t dev_alloc(T** p, uint64_t n_elems) {
    cudaError_t e = cudaMalloc((void**)p, (n_elems ? n_elems : 1) * sizeof(T));
    if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc", __FILE__, __LINE__); return VB_ERR_OOM; }
    return VB_OK;
}

LaunchCfg lcfg(vb_ctx* c, bool pdl);
StepIO decode_io(vb_ctx* c);
// The launch sequence of one token for every active row of `state` (with_head: final norm, lm_head and sampler too).
cudaError_t enqueue_step(vb_ctx* c, SeqState* state, bool with_head, const StepIO& io);
int32_t check_ready(vb_ctx* c, const char* who);
// [rows][cols] of this rank's shard of a role, and its storage format (false: the model has no such tensor)
bool role_shape(const vb_ctx* c, int role, uint32_t* rows, uint32_t* cols, int32_t* fmt);
// vb_gguf.cu
cudaError_t unpack_gguf(const LaunchCfg& lc, void* words, void* scale_min, const void* src, int ggml_type, uint64_t n_blocks);
// Makes the chunk buffers (pfc_*) hold at least `rows` rows.
int32_t ensure_chunk_buffers(vb_ctx* c, uint32_t rows);

}  // namespace vb
