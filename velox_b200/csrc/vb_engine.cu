// The decode engine behind the C ABI: one context per GPU owning the weight arena, the paged fp16 KV pool,
// the activation buffers, the device-resident per-sequence state and the mapped token ring -- the role of
// the reference's host runner (src/runners/velox_cuda_runner.cu:417-487) plus the launch sequence its
// compiler emits per model (src/runners/tinystories_smollm.cu:2388-3249).
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>
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

    // derived
    uint32_t qdim = 0, kvdim = 0, qkv_rows = 0, max_blocks = 0, n_blocks = 0, n_splits = 1, tokens_per_split = 32;

    // weight arena (execution order, 256-byte aligned slabs)
    uint8_t* arena = nullptr;
    uint64_t arena_bytes = 0;
    std::vector<Tensor> t;  // [role][layer]

    // paged KV pool: per layer [block][K|V][kv_head][block_tokens][D] fp16
    __half* kv_pool = nullptr;
    uint64_t kv_layer_elems = 0;
    int32_t* block_table_dev = nullptr;
    std::vector<int32_t> block_table_host;
    std::vector<int32_t> free_blocks;
    std::vector<uint32_t> slot_blocks;  // blocks held per slot

    // device state
    SeqState* state = nullptr;     // decode state, one per slot
    SeqState* pf_state = nullptr;  // prefill state (only the slot being prefilled is active)
    std::vector<SeqState> state_host;
    uint32_t* ring_host = nullptr;  // mapped pinned [max_batch][RING_SLOTS]
    uint32_t* ring_dev = nullptr;
    uint32_t* pf_tokens = nullptr;  // device copy of the prompt being prefilled
    uint32_t pf_tokens_cap = 0;

    // activations
    float *hidden = nullptr, *qkv = nullptr, *q = nullptr, *attn_out = nullptr, *act = nullptr, *logits = nullptr;
    float* attn_scratch = nullptr;
    float* cand_v = nullptr;
    uint32_t* cand_i = nullptr;

    cudaGraph_t graph = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
    uint64_t graph_nodes = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;

    Tensor& tensor(int role, int layer) { return t[(size_t)role * (d.n_layers ? d.n_layers : 1) + (size_t)layer]; }
};

namespace {

inline uint64_t align256(uint64_t v) { return (v + 255) & ~255ULL; }
bool role_is_global(int role) { return role == VB_ROLE_EMBED || role == VB_ROLE_FINAL_NORM || role == VB_ROLE_LM_HEAD; }
bool role_is_vector(int role) {
    return role == VB_ROLE_ATTN_NORM || role == VB_ROLE_MLP_NORM || role == VB_ROLE_FINAL_NORM || role == VB_ROLE_BQ ||
           role == VB_ROLE_BK || role == VB_ROLE_BV;
}

// expected [rows][cols] and storage format of a role
bool role_shape(const vb_ctx* c, int role, uint32_t* rows, uint32_t* cols, int32_t* fmt) {
    const vb_model_desc& d = c->d;
    const int32_t wf = (int32_t)d.weight_fmt;
    // small vectors are kept in fp16 when the linear weights are reduced precision, else fp32
    const int32_t vf = (wf == VB_FMT_F32) ? VB_FMT_F32 : VB_FMT_F16;
    switch (role) {
    case VB_ROLE_EMBED: *rows = d.vocab; *cols = d.d_model; *fmt = (int32_t)d.embed_fmt; return true;
    case VB_ROLE_ATTN_NORM: case VB_ROLE_MLP_NORM: case VB_ROLE_FINAL_NORM: *rows = 1; *cols = d.d_model; *fmt = vf; return true;
    case VB_ROLE_WQ: *rows = c->qdim; *cols = d.d_model; *fmt = wf; return true;
    case VB_ROLE_WK: case VB_ROLE_WV: *rows = c->kvdim; *cols = d.d_model; *fmt = wf; return true;
    case VB_ROLE_WO: *rows = d.d_model; *cols = c->qdim; *fmt = wf; return true;
    case VB_ROLE_WGATE: case VB_ROLE_WUP: *rows = d.ffn_dim; *cols = d.d_model; *fmt = wf; return true;
    case VB_ROLE_WDOWN: *rows = d.d_model; *cols = d.ffn_dim; *fmt = wf; return true;
    case VB_ROLE_LM_HEAD: *rows = d.vocab; *cols = d.d_model; *fmt = (int32_t)d.head_fmt; return true;
    case VB_ROLE_BQ: *rows = 1; *cols = c->qdim; *fmt = vf; return d.qkv_bias != 0;
    case VB_ROLE_BK: case VB_ROLE_BV: *rows = 1; *cols = c->kvdim; *fmt = vf; return d.qkv_bias != 0;
    default: return false;
    }
}

// Lay the arena out in execution order.  Wq|Wk|Wv (and their scales) are adjacent so that the fused QKV
// product sees one [Hq*D + 2*Hkv*D][d] matrix.
int32_t plan_arena(vb_ctx* c) {
    uint64_t off = 0;
    // pass 1: compute offsets; pass 2 (after allocation) turns them into pointers
    struct Slot { int role, layer; uint64_t data, scales, tiled, tiled_scales, v3; bool has_tiled; };
    std::vector<Slot> slots;
    std::vector<uint64_t> swiglu_off, swiglu_v3_off;
    auto add_group = [&](std::initializer_list<int> roles, int layer) {
        // data of all members first (contiguous rows), then their scales (contiguous too)
        std::vector<Slot> g;
        for (int role : roles) {
            uint32_t rows, cols; int32_t fmt;
            if (!role_shape(c, role, &rows, &cols, &fmt)) continue;
            Tensor& t = c->tensor(role, layer);
            t.m.fmt = fmt; t.m.rows = rows; t.m.cols = cols;
            g.push_back({role, layer, off, 0, 0, 0, 0, false});
            off += wmat_data_bytes(fmt, rows, cols);
        }
        off = align256(off);
        bool tile_all = !g.empty();
        for (Slot& s : g) {
            Tensor& t = c->tensor(s.role, s.layer);
            s.scales = off;
            off += wmat_scale_bytes(t.m.fmt, t.m.rows, t.m.cols);
            if (t.m.fmt != VB_FMT_Q4G32 || !tile_q4_supported(t.m.rows, t.m.cols)) tile_all = false;
        }
        off = align256(off);
        if (tile_all) {
            // tile-major copies for the tuned kernel, members adjacent again (fused QKV = one tiled matrix)
            for (Slot& s : g) {
                Tensor& t = c->tensor(s.role, s.layer);
                s.has_tiled = true; s.tiled = off; s.tiled_scales = off;  // scales are interleaved block by block
                off += wmat_data_bytes(t.m.fmt, t.m.rows, t.m.cols) + wmat_scale_bytes(t.m.fmt, t.m.rows, t.m.cols);
            }
            off = align256(off);
            for (Slot& s : g) {  // and the integer tensor-core layout
                Tensor& t = c->tensor(s.role, s.layer);
                s.v3 = off;
                off += wmat_data_bytes(t.m.fmt, t.m.rows, t.m.cols) + wmat_scale_bytes(t.m.fmt, t.m.rows, t.m.cols);
            }
            off = align256(off);
        }
        for (Slot& s : g) slots.push_back(s);
    };
    for (uint32_t l = 0; l < c->d.n_layers; ++l) {
        add_group({VB_ROLE_ATTN_NORM}, (int)l);
        add_group({VB_ROLE_WQ, VB_ROLE_WK, VB_ROLE_WV}, (int)l);
        add_group({VB_ROLE_BQ, VB_ROLE_BK, VB_ROLE_BV}, (int)l);
        add_group({VB_ROLE_WO}, (int)l);
        add_group({VB_ROLE_MLP_NORM}, (int)l);
        add_group({VB_ROLE_WGATE}, (int)l);
        add_group({VB_ROLE_WUP}, (int)l);
        {
            // gate and up interleaved 8 rows by 8 rows for the fused SwiGLU kernel
            Tensor& tg = c->tensor(VB_ROLE_WGATE, (int)l);
            if (tg.m.fmt == VB_FMT_Q4G32 && tg.m.rows % 8 == 0 && tg.m.cols % 128 == 0) {
                swiglu_off.push_back(off);
                off += 2 * (wmat_data_bytes(tg.m.fmt, tg.m.rows, tg.m.cols) + wmat_scale_bytes(tg.m.fmt, tg.m.rows, tg.m.cols));
                off = align256(off);
                swiglu_v3_off.push_back(off);
                off += 2 * (wmat_data_bytes(tg.m.fmt, tg.m.rows, tg.m.cols) + wmat_scale_bytes(tg.m.fmt, tg.m.rows, tg.m.cols));
                off = align256(off);
            } else {
                swiglu_off.push_back(~0ULL);
                swiglu_v3_off.push_back(~0ULL);
            }
        }
        add_group({VB_ROLE_WDOWN}, (int)l);
    }
    add_group({VB_ROLE_FINAL_NORM}, 0);
    if (!c->d.tied_lm_head) add_group({VB_ROLE_LM_HEAD}, 0);
    add_group({VB_ROLE_EMBED}, 0);
    c->arena_bytes = off ? off : 256;
    cudaError_t e = cudaMalloc(&c->arena, c->arena_bytes);
    if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc(weight arena)", __FILE__, __LINE__); return VB_ERR_OOM; }
    for (const Slot& s : slots) {
        Tensor& t = c->tensor(s.role, s.layer);
        t.m.data = c->arena + s.data;
        t.m.scales = wmat_scale_bytes(t.m.fmt, t.m.rows, t.m.cols) ? c->arena + s.scales : nullptr;
        if (s.has_tiled) { t.m.tiled = c->arena + s.tiled; t.m.tiled_scales = c->arena + s.tiled_scales; t.m.v3 = c->arena + s.v3; }
    }
    for (uint32_t l = 0; l < c->d.n_layers; ++l)
        if (swiglu_off[l] != ~0ULL) {
            c->tensor(VB_ROLE_WGATE, (int)l).m.tiled_swiglu = c->arena + swiglu_off[l];
            c->tensor(VB_ROLE_WGATE, (int)l).m.v3_swiglu = c->arena + swiglu_v3_off[l];
        }
    if (c->d.tied_lm_head) {
        Tensor& h = c->tensor(VB_ROLE_LM_HEAD, 0);
        h = c->tensor(VB_ROLE_EMBED, 0);
    }
    return VB_OK;
}

template <typename T>
int32_t dev_alloc(T** p, uint64_t n_elems) {
    cudaError_t e = cudaMalloc((void**)p, (n_elems ? n_elems : 1) * sizeof(T));
    if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc", __FILE__, __LINE__); return VB_ERR_OOM; }
    return VB_OK;
}

LaunchCfg lcfg(vb_ctx* c, bool pdl) {
    LaunchCfg lc;
    lc.stream = c->stream;
    lc.pdl = pdl && c->use_pdl;
    lc.counter = &c->launches;
    return lc;
}

__global__ void k_set_state(SeqState* state, uint32_t slot, const uint32_t* tokens, uint32_t idx, uint32_t token,
                            uint32_t pos, uint32_t active) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        state[slot].token = tokens ? tokens[idx] : token;
        state[slot].pos = pos;
        state[slot].active = active;
        state[slot].pad = 0;
    }
}

bool all_loaded(vb_ctx* c, const char** missing) {
    static const char* names[] = {"embed", "attn_norm", "wq", "wk", "wv", "wo", "mlp_norm", "wgate", "wup", "wdown",
                                  "final_norm", "lm_head", "bq", "bk", "bv"};
    for (int role = 0; role <= VB_ROLE_BV; ++role) {
        uint32_t rows, cols; int32_t fmt;
        if (!role_shape(c, role, &rows, &cols, &fmt)) continue;
        const uint32_t nl = role_is_global(role) ? 1 : c->d.n_layers;
        for (uint32_t l = 0; l < nl; ++l)
            if (!c->tensor(role, (int)l).loaded) { *missing = names[role]; return false; }
    }
    return true;
}

// The launch sequence of one token for every active slot of `state`.
cudaError_t enqueue_step(vb_ctx* c, SeqState* state, bool with_head) {
    const vb_model_desc& d = c->d;
    const uint32_t B = d.max_batch;
    cudaError_t e;
    uint32_t tn = 0;
    auto next_trace = [&]() -> unsigned long long* { return (c->trace && tn < 1024) ? c->trace + 4 * (size_t)(tn++) : nullptr; };
#define VB_TRY(x) do { e = (x); if (e != cudaSuccess) return e; } while (0)
    Tensor& emb = c->tensor(VB_ROLE_EMBED, 0);
    // the first kernel of a step must not overlap the previous step's tail: launched without PDL
    VB_TRY(embed(lcfg(c, false), c->hidden, nullptr, state, emb.m.data, emb.m.scales, emb.m.fmt, d.d_model, d.vocab, B));
    for (uint32_t l = 0; l < d.n_layers; ++l) {
        const int L = (int)l;
        // RMSNorm + fused QKV projection
        GemvArgs g;
        g.state = state; g.batch = B;
        g.x = c->hidden; g.dst = c->qkv;
        g.norm_w = c->tensor(VB_ROLE_ATTN_NORM, L).m.data; g.norm_fmt = c->tensor(VB_ROLE_ATTN_NORM, L).m.fmt; g.eps = d.rms_eps;
        g.w = c->tensor(VB_ROLE_WQ, L).m; g.w.rows = c->qkv_rows;
        g.trace = next_trace();
        VB_TRY(gemv(lcfg(c, true), g, c->gemv_path));
        // bias + RoPE + KV append
        __half* kv_layer = c->kv_pool + (size_t)l * c->kv_layer_elems;
        const void *bq = nullptr, *bk = nullptr, *bv = nullptr; int bf = VB_FMT_F32;
        if (d.qkv_bias) {
            bq = c->tensor(VB_ROLE_BQ, L).m.data; bk = c->tensor(VB_ROLE_BK, L).m.data; bv = c->tensor(VB_ROLE_BV, L).m.data;
            bf = c->tensor(VB_ROLE_BQ, L).m.fmt;
        }
        const bool fused_append = (d.n_q_heads / d.n_kv_heads) <= 8 && c->fuse_append;
        if (!fused_append)
            VB_TRY(bias_rope_kv_append(lcfg(c, true), c->q, c->qkv, state, bq, bk, bv, bf, kv_layer, c->block_table_dev,
                                       c->max_blocks, d.n_q_heads, d.n_kv_heads, d.head_dim, d.kv_block_tokens, d.rope_theta, B));
        // split-K attention over the paged cache (with the bias + RoPE + KV append fused in when possible)
        AttnArgs a;
        a.out = c->attn_out; a.q = c->q; a.k = kv_layer; a.kv_fp16 = 1;
        if (fused_append) { a.qkv_raw = c->qkv; a.bq = bq; a.bk = bk; a.bv = bv; a.bias_fmt = bf; a.rope_inv_freq = c->rope_inv_freq; }
        a.block_table = c->block_table_dev; a.max_blocks = c->max_blocks; a.block_tokens = d.kv_block_tokens;
        a.state = state; a.Hq = d.n_q_heads; a.Hkv = d.n_kv_heads; a.D = d.head_dim; a.batch = B;
        a.max_splits = c->n_splits; a.tokens_per_split = c->tokens_per_split; a.scratch = c->attn_scratch;
        a.trace = next_trace();
        VB_TRY(attention(lcfg(c, true), a));
        // O-projection + residual
        GemvArgs o;
        o.state = state; o.batch = B; o.x = c->attn_out; o.dst = c->hidden; o.epilogue = EPI_RESIDUAL;
        o.w = c->tensor(VB_ROLE_WO, L).m;
        o.trace = next_trace();
        VB_TRY(gemv(lcfg(c, true), o, c->gemv_path));
        // RMSNorm + gate/up + SiLU*up
        GemvArgs gu;
        gu.state = state; gu.batch = B; gu.x = c->hidden; gu.dst = c->act; gu.epilogue = EPI_SWIGLU;
        gu.norm_w = c->tensor(VB_ROLE_MLP_NORM, L).m.data; gu.norm_fmt = c->tensor(VB_ROLE_MLP_NORM, L).m.fmt; gu.eps = d.rms_eps;
        gu.w = c->tensor(VB_ROLE_WGATE, L).m; gu.w2 = c->tensor(VB_ROLE_WUP, L).m;
        gu.trace = next_trace();
        VB_TRY(gemv(lcfg(c, true), gu, c->gemv_path));
        // down projection + residual
        GemvArgs dn;
        dn.state = state; dn.batch = B; dn.x = c->act; dn.dst = c->hidden; dn.epilogue = EPI_RESIDUAL;
        dn.w = c->tensor(VB_ROLE_WDOWN, L).m;
        dn.trace = next_trace();
        VB_TRY(gemv(lcfg(c, true), dn, c->gemv_path));
    }
    if (with_head) {
        GemvArgs h;
        h.state = state; h.batch = B; h.x = c->hidden; h.dst = c->logits;
        h.norm_w = c->tensor(VB_ROLE_FINAL_NORM, 0).m.data; h.norm_fmt = c->tensor(VB_ROLE_FINAL_NORM, 0).m.fmt; h.eps = d.rms_eps;
        h.w = c->tensor(VB_ROLE_LM_HEAD, 0).m;
        h.trace = next_trace();
        VB_TRY(gemv(lcfg(c, true), h, c->gemv_path));
        VB_TRY(argmax(lcfg(c, true), nullptr, c->logits, d.vocab, B, c->cand_v, c->cand_i, state, c->ring_dev, RING_SLOTS));
    }
#undef VB_TRY
    c->trace_n = tn;
    return cudaSuccess;
}

int32_t check_ready(vb_ctx* c, const char* who) {
    if (!c) { set_error("%s: null context", who); return VB_ERR_INVALID; }
    const char* missing = nullptr;
    if (!all_loaded(c, &missing)) { set_error("%s: tensor '%s' has not been loaded", who, missing); return VB_ERR_STATE; }
    return VB_OK;
}

}  // namespace

extern "C" {

int32_t vb_create(const vb_model_desc* desc, int32_t device, vb_ctx** out) {
    VB_REQUIRE(desc && out, "vb_create: null argument");
    VB_REQUIRE(desc->struct_bytes == sizeof(vb_model_desc), "vb_create: struct_bytes=%u, expected %u", desc->struct_bytes,
               (unsigned)sizeof(vb_model_desc));
    const vb_model_desc& d = *desc;
    VB_REQUIRE(d.vocab && d.d_model && d.n_layers && d.n_q_heads && d.n_kv_heads && d.head_dim && d.ffn_dim && d.max_seq_len,
               "vb_create: zero dimension");
    VB_REQUIRE(d.n_q_heads % d.n_kv_heads == 0, "vb_create: n_q_heads=%u not a multiple of n_kv_heads=%u", d.n_q_heads, d.n_kv_heads);
    VB_REQUIRE(d.head_dim == 32 || d.head_dim == 64 || d.head_dim == 128 || d.head_dim == 256, "vb_create: head_dim=%u unsupported", d.head_dim);
    VB_REQUIRE(d.max_batch >= 1 && d.max_batch <= 256, "vb_create: max_batch=%u out of range [1,256]", d.max_batch);
    VB_REQUIRE(d.kv_block_tokens == 16, "vb_create: kv_block_tokens must be 16");
    VB_REQUIRE(d.weight_fmt <= VB_FMT_I8PC && d.head_fmt <= VB_FMT_I8PC && d.embed_fmt <= VB_FMT_I8PC, "vb_create: unknown format");
    VB_REQUIRE(fmt_shape_ok((int32_t)d.weight_fmt, d.d_model) && fmt_shape_ok((int32_t)d.weight_fmt, d.ffn_dim) &&
               fmt_shape_ok((int32_t)d.weight_fmt, d.n_q_heads * d.head_dim) && fmt_shape_ok((int32_t)d.head_fmt, d.d_model) &&
               fmt_shape_ok((int32_t)d.embed_fmt, d.d_model) && d.d_model % 8 == 0 && d.ffn_dim % 8 == 0,
               "vb_create: dimensions not divisible by the quantization group of the chosen format");
    VB_REQUIRE(!d.tied_lm_head || d.head_fmt == d.embed_fmt, "vb_create: tied lm_head needs head_fmt == embed_fmt");
    VB_REQUIRE((uint64_t)d.ffn_dim * 4 <= 200 * 1024 && (uint64_t)d.d_model * 4 <= 200 * 1024, "vb_create: width exceeds the staging limit");
    if (d.attn_kind != VB_ATTN_GQA) { set_error("vb_create: attn_kind %u is served by vb_op_mla_absorbed only", d.attn_kind); return VB_ERR_UNSUPPORTED; }
    if (d.tp_size > 1) { set_error("vb_create: tensor parallel contexts are not available in this build"); return VB_ERR_UNSUPPORTED; }

    VB_CUDA(cudaSetDevice(device));
    VB_CUDA(kernels_init());
    vb_ctx* c = new (std::nothrow) vb_ctx();
    if (!c) { set_error("vb_create: out of host memory"); return VB_ERR_OOM; }
    c->d = d;
    c->device = device;
    c->qdim = d.n_q_heads * d.head_dim;
    c->kvdim = d.n_kv_heads * d.head_dim;
    c->qkv_rows = c->qdim + 2 * c->kvdim;
    c->max_blocks = (d.max_seq_len + d.kv_block_tokens - 1) / d.kv_block_tokens;
    c->n_blocks = d.kv_blocks_total ? d.kv_blocks_total : d.max_batch * c->max_blocks;
    c->n_splits = attn_pick_splits(d.max_seq_len);
    c->tokens_per_split = attn_tokens_per_split(d.max_seq_len);
    c->t.resize((size_t)VB_ROLE_COUNT * d.n_layers);
    int32_t rc = VB_OK;
    cudaError_t e;
#define VB_CREATE_TRY(x) do { rc = (x); if (rc != VB_OK) { vb_destroy(c); return rc; } } while (0)
#define VB_CREATE_CUDA(x) do { e = (x); if (e != cudaSuccess) { rc = cuda_fail(e, #x, __FILE__, __LINE__); vb_destroy(c); return rc; } } while (0)
    VB_CREATE_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    VB_CREATE_CUDA(cudaEventCreate(&c->ev0));
    VB_CREATE_CUDA(cudaEventCreate(&c->ev1));
    VB_CREATE_TRY(plan_arena(c));
    c->kv_layer_elems = (uint64_t)c->n_blocks * 2 * d.n_kv_heads * d.kv_block_tokens * d.head_dim;
    VB_CREATE_TRY(dev_alloc(&c->kv_pool, c->kv_layer_elems * d.n_layers));
    VB_CREATE_CUDA(cudaMemsetAsync(c->kv_pool, 0, c->kv_layer_elems * d.n_layers * sizeof(__half), c->stream));
    VB_CREATE_TRY(dev_alloc(&c->block_table_dev, (uint64_t)d.max_batch * c->max_blocks));
    c->block_table_host.assign((size_t)d.max_batch * c->max_blocks, 0);
    VB_CREATE_CUDA(cudaMemsetAsync(c->block_table_dev, 0, (size_t)d.max_batch * c->max_blocks * 4, c->stream));
    c->free_blocks.reserve(c->n_blocks);
    for (int32_t b = (int32_t)c->n_blocks - 1; b >= 0; --b) c->free_blocks.push_back(b);
    c->slot_blocks.assign(d.max_batch, 0);
    VB_CREATE_TRY(dev_alloc(&c->state, d.max_batch));
    VB_CREATE_TRY(dev_alloc(&c->pf_state, d.max_batch));
    VB_CREATE_CUDA(cudaMemsetAsync(c->state, 0, d.max_batch * sizeof(SeqState), c->stream));
    VB_CREATE_CUDA(cudaMemsetAsync(c->pf_state, 0, d.max_batch * sizeof(SeqState), c->stream));
    c->state_host.assign(d.max_batch, SeqState{0, 0, 0, 0});
    VB_CREATE_CUDA(cudaHostAlloc((void**)&c->ring_host, (size_t)d.max_batch * RING_SLOTS * 4, cudaHostAllocMapped));
    memset(c->ring_host, 0xFF, (size_t)d.max_batch * RING_SLOTS * 4);
    VB_CREATE_CUDA(cudaHostGetDevicePointer((void**)&c->ring_dev, c->ring_host, 0));
    const uint64_t B = d.max_batch;
    VB_CREATE_TRY(dev_alloc(&c->hidden, B * d.d_model));
    VB_CREATE_TRY(dev_alloc(&c->qkv, B * c->qkv_rows));
    VB_CREATE_TRY(dev_alloc(&c->q, B * c->qdim));
    VB_CREATE_TRY(dev_alloc(&c->attn_out, B * c->qdim));
    VB_CREATE_TRY(dev_alloc(&c->act, B * d.ffn_dim));
    VB_CREATE_TRY(dev_alloc(&c->logits, B * d.vocab));
    VB_CREATE_TRY(dev_alloc(&c->attn_scratch, attn_scratch_floats(d.n_q_heads, d.head_dim, d.max_batch, c->n_splits)));
    VB_CREATE_CUDA(cudaMemsetAsync(c->attn_scratch, 0, attn_scratch_floats(d.n_q_heads, d.head_dim, d.max_batch, c->n_splits) * 4, c->stream));
    VB_CREATE_TRY(dev_alloc(&c->cand_v, B * argmax_chunks(d.vocab)));
    VB_CREATE_TRY(dev_alloc(&c->cand_i, B * argmax_chunks(d.vocab)));
    {
        // RoPE frequencies exactly as the reference computes them on the host (src/runtime.rs:758)
        std::vector<float> f(d.head_dim / 2);
        for (uint32_t j = 0; j < d.head_dim / 2; ++j) f[j] = 1.0f / powf(d.rope_theta, (float)(2 * j) / (float)d.head_dim);
        VB_CREATE_TRY(dev_alloc(&c->rope_inv_freq, f.size()));
        VB_CREATE_CUDA(cudaMemcpyAsync(c->rope_inv_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice, c->stream));
        VB_CREATE_CUDA(cudaStreamSynchronize(c->stream));
    }
    VB_CREATE_CUDA(cudaStreamSynchronize(c->stream));
#undef VB_CREATE_TRY
#undef VB_CREATE_CUDA
    *out = c;
    return VB_OK;
}

int32_t vb_destroy(vb_ctx* c) {
    if (!c) return VB_OK;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->graph_exec) cudaGraphExecDestroy(c->graph_exec);
    if (c->graph) cudaGraphDestroy(c->graph);
    void* frees[] = {c->arena, c->kv_pool, c->block_table_dev, c->state, c->pf_state, c->pf_tokens, c->hidden, c->qkv, c->q,
                     c->attn_out, c->act, c->logits, c->attn_scratch, c->cand_v, c->cand_i, c->rope_inv_freq, c->trace};
    for (void* p : frees) if (p) cudaFree(p);
    if (c->ring_host) cudaFreeHost(c->ring_host);
    if (c->ev0) cudaEventDestroy(c->ev0);
    if (c->ev1) cudaEventDestroy(c->ev1);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
    return VB_OK;
}

static int32_t load_common(vb_ctx* c, int32_t role, int32_t layer, uint64_t rows, uint64_t cols, Tensor** out, const char* who) {
    VB_REQUIRE(c != nullptr, "%s: null context", who);
    VB_REQUIRE(role >= 0 && role <= VB_ROLE_BV, "%s: role %d is not an engine tensor", who, role);
    if (role_is_global(role)) layer = 0;
    VB_REQUIRE(layer >= 0 && (uint32_t)layer < c->d.n_layers, "%s: layer %d out of range", who, layer);
    uint32_t er, ec; int32_t fmt;
    VB_REQUIRE(role_shape(c, role, &er, &ec, &fmt), "%s: role %d is not part of this model", who, role);
    VB_REQUIRE(!(role == VB_ROLE_LM_HEAD && c->d.tied_lm_head), "%s: lm_head is tied to the embedding table", who);
    VB_REQUIRE(rows * cols == (uint64_t)er * ec && (rows == er || role_is_vector(role)), "%s: role %d expects [%u][%u], got [%llu][%llu]",
               who, role, er, ec, (unsigned long long)rows, (unsigned long long)cols);
    *out = &c->tensor(role, layer);
    VB_CUDA(cudaSetDevice(c->device));
    if (c->graph_exec) { cudaGraphExecDestroy(c->graph_exec); c->graph_exec = nullptr; }
    return VB_OK;
}

static int32_t finish_load(vb_ctx* c, Tensor* t, int32_t role, int32_t layer) {
    if (!t->m.tiled) return VB_OK;
    LaunchCfg lc = lcfg(c, false);
    lc.counter = nullptr;
    VB_CUDA(tile_q4(lc, const_cast<void*>(t->m.tiled), const_cast<void*>(t->m.tiled_scales), t->m.data, t->m.scales, t->m.rows, t->m.cols));
    VB_CUDA(tile_q4_v3(lc, const_cast<void*>(t->m.v3), t->m.data, t->m.scales, t->m.rows, t->m.cols));
    if (role == VB_ROLE_WGATE || role == VB_ROLE_WUP) {
        const int which = role == VB_ROLE_WUP ? 1 : 0;
        const void* il = c->tensor(VB_ROLE_WGATE, layer).m.tiled_swiglu;
        if (il) VB_CUDA(tile_q4_swiglu(lc, const_cast<void*>(il), t->m.data, t->m.scales, t->m.rows, t->m.cols, which));
        const void* il3 = c->tensor(VB_ROLE_WGATE, layer).m.v3_swiglu;
        if (il3) VB_CUDA(tile_q4_v3_swiglu(lc, const_cast<void*>(il3), t->m.data, t->m.scales, t->m.rows, t->m.cols, which));
    }
    VB_CUDA(cudaStreamSynchronize(c->stream));
    return VB_OK;
}

static void mark_loaded(vb_ctx* c, int32_t role, Tensor* t) {
    t->loaded = true;
    if (role == VB_ROLE_EMBED && c->d.tied_lm_head) c->tensor(VB_ROLE_LM_HEAD, 0) = *t;  // tied: the head reads the table
}

int32_t vb_load_tensor(vb_ctx* c, int32_t role, int32_t layer, const void* src, int32_t src_fmt, int32_t src_loc,
                       uint64_t rows, uint64_t cols) {
    Tensor* t = nullptr;
    int32_t rc = load_common(c, role, layer, rows, cols, &t, "vb_load_tensor");
    if (rc != VB_OK) return rc;
    VB_REQUIRE(src != nullptr, "vb_load_tensor: null source");
    VB_REQUIRE(src_fmt == VB_FMT_F32 || src_fmt == VB_FMT_F16 || src_fmt == VB_FMT_BF16, "vb_load_tensor: source format %d", src_fmt);
    VB_REQUIRE(src_loc == VB_LOC_HOST || src_loc == VB_LOC_DEVICE, "vb_load_tensor: source location %d", src_loc);
    const uint64_t n = rows * cols;
    const uint64_t src_bytes = n * (src_fmt == VB_FMT_F32 ? 4 : 2);
    // stage: raw source on the device, then fp32, then the storage format
    void* raw = nullptr;
    float* f32 = nullptr;
    LaunchCfg lc = lcfg(c, false);
    lc.counter = nullptr;
    cudaError_t e = cudaSuccess;
    const void* dev_src = src;
    if (src_loc == VB_LOC_HOST) {
        if ((e = cudaMalloc(&raw, src_bytes)) != cudaSuccess) { cuda_fail(e, "cudaMalloc(staging)", __FILE__, __LINE__); return VB_ERR_OOM; }
        e = cudaMemcpyAsync(raw, src, src_bytes, cudaMemcpyHostToDevice, c->stream);
        dev_src = raw;
    }
    if (e == cudaSuccess && src_fmt != VB_FMT_F32) {
        if ((e = cudaMalloc((void**)&f32, n * 4)) == cudaSuccess) e = dequantize(lc, f32, dev_src, nullptr, src_fmt, rows, cols);
        dev_src = f32;
    }
    if (e == cudaSuccess) e = quantize(lc, const_cast<void*>(t->m.data), const_cast<void*>(t->m.scales), (const float*)dev_src, t->m.fmt, t->m.rows, t->m.cols);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (raw) cudaFree(raw);
    if (f32) cudaFree(f32);
    if (e != cudaSuccess) return cuda_fail(e, "vb_load_tensor", __FILE__, __LINE__);
    if ((rc = finish_load(c, t, role, layer)) != VB_OK) return rc;
    mark_loaded(c, role, t);
    return VB_OK;
}

int32_t vb_load_tensor_packed(vb_ctx* c, int32_t role, int32_t layer, const void* data, const void* scales, int32_t src_loc,
                              uint64_t rows, uint64_t cols) {
    Tensor* t = nullptr;
    int32_t rc = load_common(c, role, layer, rows, cols, &t, "vb_load_tensor_packed");
    if (rc != VB_OK) return rc;
    const uint64_t db = wmat_data_bytes(t->m.fmt, t->m.rows, t->m.cols), sb = wmat_scale_bytes(t->m.fmt, t->m.rows, t->m.cols);
    VB_REQUIRE(data != nullptr && (sb == 0 || scales != nullptr), "vb_load_tensor_packed: null data/scales");
    const cudaMemcpyKind kind = (src_loc == VB_LOC_HOST) ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
    VB_CUDA(cudaMemcpyAsync(const_cast<void*>(t->m.data), data, db, kind, c->stream));
    if (sb) VB_CUDA(cudaMemcpyAsync(const_cast<void*>(t->m.scales), scales, sb, kind, c->stream));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    if ((rc = finish_load(c, t, role, layer)) != VB_OK) return rc;
    mark_loaded(c, role, t);
    return VB_OK;
}

int32_t vb_load_tensor_synthetic(vb_ctx* c, int32_t role, int32_t layer, uint64_t seed, uint64_t stream_id, float mean,
                                 float std, uint64_t rows, uint64_t cols) {
    Tensor* t = nullptr;
    int32_t rc = load_common(c, role, layer, rows, cols, &t, "vb_load_tensor_synthetic");
    if (rc != VB_OK) return rc;
    const uint64_t n = rows * cols;
    float* f32 = nullptr;
    cudaError_t e = cudaMalloc((void**)&f32, n * 4);
    if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc(staging)", __FILE__, __LINE__); return VB_ERR_OOM; }
    LaunchCfg lc = lcfg(c, false);
    lc.counter = nullptr;
    e = fill_normal(lc, f32, n, seed, stream_id, mean, std);
    if (e == cudaSuccess) e = quantize(lc, const_cast<void*>(t->m.data), const_cast<void*>(t->m.scales), f32, t->m.fmt, t->m.rows, t->m.cols);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    cudaFree(f32);
    if (e != cudaSuccess) return cuda_fail(e, "vb_load_tensor_synthetic", __FILE__, __LINE__);
    if ((rc = finish_load(c, t, role, layer)) != VB_OK) return rc;
    mark_loaded(c, role, t);
    return VB_OK;
}

int32_t vb_export_tensor(vb_ctx* c, int32_t role, int32_t layer, void* data, uint64_t data_bytes, void* scales, uint64_t scales_bytes) {
    VB_REQUIRE(c != nullptr, "vb_export_tensor: null context");
    VB_REQUIRE(role >= 0 && role <= VB_ROLE_BV, "vb_export_tensor: role %d", role);
    if (role_is_global(role)) layer = 0;
    VB_REQUIRE(layer >= 0 && (uint32_t)layer < c->d.n_layers, "vb_export_tensor: layer %d out of range", layer);
    Tensor& t = c->tensor(role, layer);
    if (!t.loaded) { set_error("vb_export_tensor: tensor not loaded"); return VB_ERR_STATE; }
    const uint64_t db = wmat_data_bytes(t.m.fmt, t.m.rows, t.m.cols), sb = wmat_scale_bytes(t.m.fmt, t.m.rows, t.m.cols);
    VB_REQUIRE(data && data_bytes == db, "vb_export_tensor: data buffer is %llu bytes, tensor has %llu", (unsigned long long)data_bytes, (unsigned long long)db);
    VB_REQUIRE(sb == 0 || (scales && scales_bytes == sb), "vb_export_tensor: scale buffer is %llu bytes, tensor has %llu", (unsigned long long)scales_bytes, (unsigned long long)sb);
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    VB_CUDA(cudaMemcpy(data, t.m.data, db, cudaMemcpyDeviceToHost));
    if (sb) VB_CUDA(cudaMemcpy(scales, t.m.scales, sb, cudaMemcpyDeviceToHost));
    return VB_OK;
}

int32_t vb_weight_bytes(vb_ctx* c, uint64_t* total) {
    VB_REQUIRE(c && total, "vb_weight_bytes: null argument");
    *total = c->arena_bytes;
    return VB_OK;
}

int32_t vb_seq_reserve(vb_ctx* c, int32_t slot, uint32_t n_tokens) {
    VB_REQUIRE(c != nullptr, "vb_seq_reserve: null context");
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_seq_reserve: slot %d out of range", slot);
    VB_REQUIRE(n_tokens <= c->d.max_seq_len, "vb_seq_reserve: %u tokens exceed max_seq_len=%u", n_tokens, c->d.max_seq_len);
    const uint32_t need = (n_tokens + c->d.kv_block_tokens - 1) / c->d.kv_block_tokens;
    uint32_t& have = c->slot_blocks[slot];
    if (need <= have) return VB_OK;
    if (need - have > c->free_blocks.size()) { set_error("vb_seq_reserve: KV pool exhausted (%u blocks wanted, %zu free)", need - have, c->free_blocks.size()); return VB_ERR_OOM; }
    int32_t* row = c->block_table_host.data() + (size_t)slot * c->max_blocks;
    const uint32_t first = have;
    while (have < need) { row[have++] = c->free_blocks.back(); c->free_blocks.pop_back(); }
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaMemcpyAsync(c->block_table_dev + (size_t)slot * c->max_blocks + first, row + first, (size_t)(need - first) * 4,
                            cudaMemcpyHostToDevice, c->stream));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    return VB_OK;
}

int32_t vb_seq_release(vb_ctx* c, int32_t slot) {
    VB_REQUIRE(c != nullptr, "vb_seq_release: null context");
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_seq_release: slot %d out of range", slot);
    int32_t* row = c->block_table_host.data() + (size_t)slot * c->max_blocks;
    for (uint32_t i = c->slot_blocks[slot]; i > 0; --i) c->free_blocks.push_back(row[i - 1]);
    c->slot_blocks[slot] = 0;
    return vb_seq_set(c, slot, 0, 0, 0);
}

int32_t vb_seq_set(vb_ctx* c, int32_t slot, uint32_t token, uint32_t pos, uint32_t active) {
    VB_REQUIRE(c != nullptr, "vb_seq_set: null context");
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_seq_set: slot %d out of range", slot);
    VB_REQUIRE(token < c->d.vocab, "vb_seq_set: token %u >= vocab %u", token, c->d.vocab);
    VB_REQUIRE(!active || pos < c->slot_blocks[slot] * c->d.kv_block_tokens, "vb_seq_set: position %u is beyond the slot's KV reservation (%u tokens)",
               pos, c->slot_blocks[slot] * c->d.kv_block_tokens);
    VB_CUDA(cudaSetDevice(c->device));
    LaunchCfg lc = lcfg(c, false);
    VB_CUDA(launch(lc, k_set_state, dim3(1), dim3(32), 0, c->state, (uint32_t)slot, (const uint32_t*)nullptr, 0u, token, pos, active));
    return VB_OK;
}

int32_t vb_prefill(vb_ctx* c, int32_t slot, const uint32_t* tokens, uint32_t n_tokens) {
    int32_t rc = check_ready(c, "vb_prefill");
    if (rc != VB_OK) return rc;
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_prefill: slot %d out of range", slot);
    VB_REQUIRE(tokens != nullptr && n_tokens > 0, "vb_prefill: empty prompt");
    VB_REQUIRE(n_tokens <= c->slot_blocks[slot] * c->d.kv_block_tokens,
               "vb_prefill: prompt of %u tokens exceeds the slot's KV reservation (%u tokens)", n_tokens, c->slot_blocks[slot] * c->d.kv_block_tokens);
    for (uint32_t i = 0; i < n_tokens; ++i) VB_REQUIRE(tokens[i] < c->d.vocab, "vb_prefill: token %u at %u >= vocab", tokens[i], i);
    VB_CUDA(cudaSetDevice(c->device));
    if (c->pf_tokens_cap < n_tokens) {
        if (c->pf_tokens) cudaFree(c->pf_tokens);
        c->pf_tokens = nullptr; c->pf_tokens_cap = 0;
        rc = dev_alloc(&c->pf_tokens, n_tokens);
        if (rc != VB_OK) return rc;
        c->pf_tokens_cap = n_tokens;
    }
    VB_CUDA(cudaMemcpyAsync(c->pf_tokens, tokens, (size_t)n_tokens * 4, cudaMemcpyHostToDevice, c->stream));
    VB_CUDA(cudaMemsetAsync(c->pf_state, 0, c->d.max_batch * sizeof(SeqState), c->stream));
    // the reference prefills one token per forward pass (velox_cuda_runner.cu:504-506)
    for (uint32_t i = 0; i < n_tokens; ++i) {
        VB_CUDA(launch(lcfg(c, false), k_set_state, dim3(1), dim3(32), 0, c->pf_state, (uint32_t)slot, (const uint32_t*)c->pf_tokens, i, 0u, i, 1u));
        VB_CUDA(enqueue_step(c, c->pf_state, i + 1 == n_tokens));
    }
    // hand the slot over to the decode state: first generated token at position n_tokens
    VB_CUDA(cudaMemcpyAsync(c->state + slot, c->pf_state + slot, sizeof(SeqState), cudaMemcpyDeviceToDevice, c->stream));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    return VB_OK;
}

int32_t vb_decode_step(vb_ctx* c) {
    int32_t rc = check_ready(c, "vb_decode_step");
    if (rc != VB_OK) return rc;
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(enqueue_step(c, c->state, true));
    return VB_OK;
}

int32_t vb_decode_graph_build(vb_ctx* c) {
    int32_t rc = check_ready(c, "vb_decode_graph_build");
    if (rc != VB_OK) return rc;
    VB_CUDA(cudaSetDevice(c->device));
    if (c->graph_exec) { cudaGraphExecDestroy(c->graph_exec); c->graph_exec = nullptr; }
    if (c->graph) { cudaGraphDestroy(c->graph); c->graph = nullptr; }
    for (int attempt = 0; attempt < 2; ++attempt) {
        const uint64_t before = c->launches;
        VB_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
        cudaError_t e = enqueue_step(c, c->state, true);
        cudaGraph_t g = nullptr;
        cudaError_t e2 = cudaStreamEndCapture(c->stream, &g);
        c->graph_nodes = c->launches - before;
        c->launches = before;
        cudaError_t e3 = cudaSuccess;
        if (e == cudaSuccess && e2 == cudaSuccess) {
            e3 = cudaGraphInstantiate(&c->graph_exec, g, 0);
            if (e3 == cudaSuccess) {
                c->graph = g;
                if (getenv("VELOX_B200_DEBUG")) fprintf(stderr, "[velox_b200] decode graph: %llu kernel nodes, pdl=%d\n", (unsigned long long)c->graph_nodes, (int)c->use_pdl);
                return VB_OK;
            }
        }
        if (g) cudaGraphDestroy(g);
        c->graph_exec = nullptr;
        (void)cudaGetLastError();
        if (getenv("VELOX_B200_DEBUG")) fprintf(stderr, "[velox_b200] graph capture attempt %d failed: %s / %s / %s\n", attempt,
                                                cudaGetErrorString(e), cudaGetErrorString(e2), cudaGetErrorString(e3));
        if (attempt == 0 && c->use_pdl) { c->use_pdl = false; continue; }  // capture without programmatic edges
        return cuda_fail(e != cudaSuccess ? e : (e2 != cudaSuccess ? e2 : e3), "capture(decode step)", __FILE__, __LINE__);
    }
    return VB_ERR_CUDA;
}

int32_t vb_decode_run(vb_ctx* c, uint32_t n_steps, float* elapsed_ms) {
    int32_t rc = check_ready(c, "vb_decode_run");
    if (rc != VB_OK) return rc;
    VB_CUDA(cudaSetDevice(c->device));
    if (elapsed_ms) VB_CUDA(cudaEventRecord(c->ev0, c->stream));
    for (uint32_t s = 0; s < n_steps; ++s) {
        if (c->graph_exec) {
            VB_CUDA(cudaGraphLaunch(c->graph_exec, c->stream));
            c->launches += c->graph_nodes;
        } else {
            VB_CUDA(enqueue_step(c, c->state, true));
        }
    }
    if (elapsed_ms) {
        VB_CUDA(cudaEventRecord(c->ev1, c->stream));
        VB_CUDA(cudaEventSynchronize(c->ev1));
        VB_CUDA(cudaEventElapsedTime(elapsed_ms, c->ev0, c->ev1));
    }
    return VB_OK;
}

// Reads (and clears) the device error word that bounded device-side waits set when they expire.
static int32_t check_device_error(vb_ctx* c) {
    uint32_t* w = nullptr;
    VB_CUDA(fast_error_word(&w));
    uint32_t v = 0;
    VB_CUDA(cudaMemcpy(&v, w, 4, cudaMemcpyDeviceToHost));
    if (v != 0) {
        cudaMemset(w, 0, 4);
        set_error("a bounded device-side wait expired (code 0x%x): results of the last launches are invalid", v);
        return VB_ERR_TIMEOUT;
    }
    (void)c;
    return VB_OK;
}

int32_t vb_sync(vb_ctx* c) {
    VB_REQUIRE(c != nullptr, "vb_sync: null context");
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    return check_device_error(c);
}

int32_t vb_read_tokens(vb_ctx* c, int32_t slot, uint32_t first_pos, uint32_t n, uint32_t* out) {
    VB_REQUIRE(c && out, "vb_read_tokens: null argument");
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_read_tokens: slot %d out of range", slot);
    VB_REQUIRE(n <= RING_SLOTS, "vb_read_tokens: at most %u tokens stay in the ring", RING_SLOTS);
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    { int32_t rc = check_device_error(c); if (rc != VB_OK) return rc; }
    for (uint32_t i = 0; i < n; ++i) out[i] = c->ring_host[(size_t)slot * RING_SLOTS + ((first_pos + i) % RING_SLOTS)];
    return VB_OK;
}

int32_t vb_read_logits(vb_ctx* c, int32_t slot, float* out, uint64_t n_floats) {
    VB_REQUIRE(c && out, "vb_read_logits: null argument");
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_read_logits: slot %d out of range", slot);
    VB_REQUIRE(n_floats == c->d.vocab, "vb_read_logits: buffer holds %llu floats, vocab is %u", (unsigned long long)n_floats, c->d.vocab);
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    VB_CUDA(cudaMemcpy(out, c->logits + (size_t)slot * c->d.vocab, (size_t)c->d.vocab * 4, cudaMemcpyDeviceToHost));
    return VB_OK;
}

int32_t vb_read_hidden(vb_ctx* c, int32_t slot, float* out, uint64_t n_floats) {
    VB_REQUIRE(c && out, "vb_read_hidden: null argument");
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_read_hidden: slot %d out of range", slot);
    VB_REQUIRE(n_floats == c->d.d_model, "vb_read_hidden: buffer holds %llu floats, d_model is %u", (unsigned long long)n_floats, c->d.d_model);
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    VB_CUDA(cudaMemcpy(out, c->hidden + (size_t)slot * c->d.d_model, (size_t)c->d.d_model * 4, cudaMemcpyDeviceToHost));
    return VB_OK;
}

int32_t vb_read_state(vb_ctx* c, int32_t slot, uint32_t* token, uint32_t* pos) {
    VB_REQUIRE(c != nullptr, "vb_read_state: null context");
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_read_state: slot %d out of range", slot);
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    SeqState s;
    VB_CUDA(cudaMemcpy(&s, c->state + slot, sizeof(s), cudaMemcpyDeviceToHost));
    if (token) *token = s.token;
    if (pos) *pos = s.pos;
    return VB_OK;
}

int32_t vb_launch_count(vb_ctx* c, uint64_t* out) {
    VB_REQUIRE(c && out, "vb_launch_count: null argument");
    *out = c->launches;
    return VB_OK;
}

int32_t vb_step_bytes(vb_ctx* c, uint64_t* weight_bytes, uint64_t* kv_bytes) {
    VB_REQUIRE(c != nullptr, "vb_step_bytes: null context");
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    uint64_t wb = 0;
    for (int role = 0; role <= VB_ROLE_BV; ++role) {
        if (role == VB_ROLE_EMBED) continue;
        uint32_t rows, cols; int32_t fmt;
        if (!role_shape(c, role, &rows, &cols, &fmt)) continue;
        const uint64_t one = wmat_data_bytes(fmt, rows, cols) + wmat_scale_bytes(fmt, rows, cols);
        wb += one * (role_is_global(role) ? 1 : c->d.n_layers);
    }
    std::vector<SeqState> st(c->d.max_batch);
    VB_CUDA(cudaMemcpy(st.data(), c->state, st.size() * sizeof(SeqState), cudaMemcpyDeviceToHost));
    uint64_t kb = 0, n_active = 0;
    for (const SeqState& s : st)
        if (s.active) { kb += (uint64_t)(s.pos + 1) * 2 * c->kvdim * sizeof(__half) * c->d.n_layers; ++n_active; }
    // one embedding row per active sequence
    wb += n_active * wmat_data_bytes((int32_t)c->d.embed_fmt, 1, c->d.d_model);
    if (weight_bytes) *weight_bytes = wb;
    if (kv_bytes) *kv_bytes = kb;
    return VB_OK;
}

int32_t vb_set_option(vb_ctx* c, const char* name, int64_t value) {
    VB_REQUIRE(c && name, "vb_set_option: null argument");
    if (c->graph_exec) { cudaGraphExecDestroy(c->graph_exec); c->graph_exec = nullptr; }
    if (!strcmp(name, "gemv_path")) { c->gemv_path = (int)value; return VB_OK; }
    if (!strcmp(name, "pdl")) { c->use_pdl = value != 0; return VB_OK; }
    if (!strcmp(name, "fuse_append")) { c->fuse_append = value != 0; return VB_OK; }
    if (!strcmp(name, "trace")) {
        if (value && !c->trace) {
            VB_CUDA(cudaMalloc((void**)&c->trace, 1024 * 4 * sizeof(unsigned long long)));
            VB_CUDA(cudaMemset(c->trace, 0, 1024 * 4 * sizeof(unsigned long long)));
        } else if (!value && c->trace) {
            cudaFree(c->trace);
            c->trace = nullptr;
        }
        return VB_OK;
    }
    if (!strcmp(name, "gemv_imma")) { imma_enabled = value != 0; return VB_OK; }
    if (!strcmp(name, "gemv_tma")) { fast_use_tma = value != 0; return VB_OK; }
    set_error("vb_set_option: unknown option '%s'", name);
    return VB_ERR_INVALID;
}

int32_t vb_trace_read(vb_ctx* c, uint64_t* out, uint32_t max_records, uint32_t* n_records) {
    VB_REQUIRE(c && out && n_records, "vb_trace_read: null argument");
    if (!c->trace) { set_error("vb_trace_read: enable the \"trace\" option first"); return VB_ERR_STATE; }
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    const uint32_t n = c->trace_n < max_records ? c->trace_n : max_records;
    std::vector<unsigned long long> buf((size_t)n * 4);
    VB_CUDA(cudaMemcpy(buf.data(), c->trace, buf.size() * 8, cudaMemcpyDeviceToHost));
    for (uint32_t i = 0; i < n; ++i) { out[3 * i] = buf[4 * i]; out[3 * i + 1] = buf[4 * i + 1]; out[3 * i + 2] = buf[4 * i + 2]; }
    // exit stamps are running maxima: clear them, on the context's own (non-blocking) stream
    VB_CUDA(cudaMemsetAsync(c->trace, 0, 1024 * 4 * sizeof(unsigned long long), c->stream));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    *n_records = n;
    return VB_OK;
}

int32_t vb_tp_unique_id(void* id128) {
    (void)id128;
    set_error("vb_tp_unique_id: tensor parallel contexts are not available in this build");
    return VB_ERR_UNSUPPORTED;
}
int32_t vb_tp_init(vb_ctx* c, const void* id128) {
    (void)c; (void)id128;
    set_error("vb_tp_init: tensor parallel contexts are not available in this build");
    return VB_ERR_UNSUPPORTED;
}

}  // extern "C"
