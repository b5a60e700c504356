// The decode engine behind the C ABI: one context per GPU owning the weight arena, the paged fp16 KV pool,
// the activation buffers, the device-resident per-sequence state and the mapped token ring -- the role of
// the reference's host runner (src/runners/velox_cuda_runner.cu:417-487) plus the launch sequence its
// compiler emits per model (src/runners/tinystories_smollm.cu:2388-3249).
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <new>
#include <vector>

#include "vb_ctx.cuh"
#include "vb_nccl.h"

namespace vb {

inline uint64_t align256(uint64_t v) { return (v + 255) & ~255ULL; }
bool role_is_global(int role) { return role == VB_ROLE_EMBED || role == VB_ROLE_FINAL_NORM || role == VB_ROLE_LM_HEAD; }
bool role_is_vector(int role) {
    return role == VB_ROLE_ATTN_NORM || role == VB_ROLE_MLP_NORM || role == VB_ROLE_FINAL_NORM || role == VB_ROLE_BQ ||
           role == VB_ROLE_BK || role == VB_ROLE_BV;
}

// [rows][cols] of this rank's shard of a role, and its storage format
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
    case VB_ROLE_WGATE: case VB_ROLE_WUP: *rows = c->ffn; *cols = d.d_model; *fmt = wf; return true;
    case VB_ROLE_WDOWN: *rows = d.d_model; *cols = c->ffn; *fmt = wf; return true;
    case VB_ROLE_LM_HEAD: *rows = c->vocab; *cols = d.d_model; *fmt = (int32_t)d.head_fmt; return true;
    case VB_ROLE_BQ: *rows = 1; *cols = c->qdim; *fmt = vf; return d.qkv_bias != 0;
    case VB_ROLE_BK: case VB_ROLE_BV: *rows = 1; *cols = c->kvdim; *fmt = vf; return d.qkv_bias != 0;
    default: return false;
    }
}

// Where this rank's shard sits inside the full tensor [*full_rows][*full_cols]: rows [r0, r0+rows), cols [c0, c0+cols).
void role_slice(const vb_ctx* c, int role, uint32_t* full_rows, uint32_t* full_cols, uint32_t* r0, uint32_t* c0) {
    const vb_model_desc& d = c->d;
    const uint32_t tp = d.tp_size ? d.tp_size : 1, r = d.tp_rank;
    uint32_t rows = 0, cols = 0; int32_t fmt;
    role_shape(c, role, &rows, &cols, &fmt);
    *full_rows = rows; *full_cols = cols; *r0 = 0; *c0 = 0;
    switch (role) {
    case VB_ROLE_WQ: *full_rows = rows * tp; *r0 = r * rows; break;
    case VB_ROLE_WK: case VB_ROLE_WV: *full_rows = rows * tp; *r0 = r * rows; break;
    case VB_ROLE_BQ: case VB_ROLE_BK: case VB_ROLE_BV: *full_cols = cols * tp; *c0 = r * cols; break;
    case VB_ROLE_WO: *full_cols = cols * tp; *c0 = r * cols; break;
    case VB_ROLE_WGATE: case VB_ROLE_WUP: *full_rows = d.ffn_dim; *r0 = c->ffn_off; break;
    case VB_ROLE_WDOWN: *full_cols = d.ffn_dim; *c0 = c->ffn_off; break;
    case VB_ROLE_LM_HEAD: *full_rows = d.vocab; *r0 = c->vocab_off; break;
    default: break;
    }
}

// Tied head: lm_head reads (this rank's rows of) the embedding table.
void set_tied_head(vb_ctx* c) {
    Tensor& h = c->tensor(VB_ROLE_LM_HEAD, 0);
    h = c->tensor(VB_ROLE_EMBED, 0);
    h.m.rows = c->vocab;
    h.m.data = (const unsigned char*)h.m.data + wmat_data_bytes(h.m.fmt, c->vocab_off, h.m.cols);
    if (h.m.scales) h.m.scales = (const unsigned char*)h.m.scales + wmat_scale_bytes(h.m.fmt, c->vocab_off, h.m.cols);
    h.m.tiled = h.m.tiled_scales = h.m.v3 = h.m.v3_scales = nullptr;
}

// Lay the arena out in execution order.  Wq|Wk|Wv (and their scales) are adjacent so that the fused QKV
// product sees one [Hq*D + 2*Hkv*D][d] matrix.
int32_t plan_arena(vb_ctx* c) {
    uint64_t off = 0;
    // pass 1: compute offsets; pass 2 (after allocation) turns them into pointers
    struct Slot { int role, layer; uint64_t data, scales, tiled, tiled_scales, v3; bool has_tiled; uint64_t v3_scales = ~0ULL; };
    std::vector<Slot> slots;
    std::vector<uint64_t> swiglu_off, swiglu_v3_off;
    const bool lean = (c->d.flags & VB_FLAG_LEAN_WEIGHTS) != 0;
    auto add_group = [&](std::initializer_list<int> roles, int layer) {
        std::vector<Slot> g;
        bool tile_all = true, i8_all = true;  // all members int4 g32 / all int8 per-channel, in tileable shapes
        for (int role : roles) {
            uint32_t rows, cols; int32_t fmt;
            if (!role_shape(c, role, &rows, &cols, &fmt)) continue;
            Tensor& t = c->tensor(role, layer);
            t.m.fmt = fmt; t.m.rows = rows; t.m.cols = cols;
            g.push_back({role, layer, ~0ULL, ~0ULL, 0, 0, ~0ULL, false});
            if (fmt != VB_FMT_Q4G32 || !tile_q4_supported(rows, cols)) tile_all = false;
            if (fmt != VB_FMT_I8PC || !tile_q4_supported(rows, cols)) i8_all = false;
        }
        if (g.empty()) return;
        const bool lean_group = lean && (tile_all || i8_all);  // only the integer tensor-core layout is kept
        auto packed_bytes = [&](const Slot& s) {
            const Tensor& t = c->tensor(s.role, s.layer);
            return wmat_data_bytes(t.m.fmt, t.m.rows, t.m.cols) + wmat_scale_bytes(t.m.fmt, t.m.rows, t.m.cols);
        };
        if (!lean_group) {
            // canonical layout: data of all members first (contiguous rows), then their scales (contiguous too)
            for (Slot& s : g) {
                const Tensor& t = c->tensor(s.role, s.layer);
                s.data = off;
                off += wmat_data_bytes(t.m.fmt, t.m.rows, t.m.cols);
            }
            off = align256(off);
            for (Slot& s : g) {
                const Tensor& t = c->tensor(s.role, s.layer);
                s.scales = off;
                off += wmat_scale_bytes(t.m.fmt, t.m.rows, t.m.cols);
            }
            off = align256(off);
        }
        if (tile_all) {
            if (!lean_group) {
                // tile-major copies for the fp16 tensor-core kernel, members adjacent again (fused QKV = one tiled matrix)
                for (Slot& s : g) { s.has_tiled = true; s.tiled = off; s.tiled_scales = off; off += packed_bytes(s); }
                off = align256(off);
            }
            const bool swiglu_only = lean_group && (g[0].role == VB_ROLE_WGATE || g[0].role == VB_ROLE_WUP);
            if (!swiglu_only) {
                for (Slot& s : g) { s.v3 = off; off += packed_bytes(s); }  // the integer tensor-core layout
                off = align256(off);
            }
        }
        if (i8_all) {
            // int8: the members' blocks back to back (fused QKV = one tiled matrix), then their row scales back to back
            for (Slot& s : g) { const Tensor& t = c->tensor(s.role, s.layer); s.v3 = off; off += wmat_data_bytes(t.m.fmt, t.m.rows, t.m.cols); }
            for (Slot& s : g) { const Tensor& t = c->tensor(s.role, s.layer); s.v3_scales = off; off += wmat_scale_bytes(t.m.fmt, t.m.rows, t.m.cols); }
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
                if (lean && tile_q4_supported(tg.m.rows, tg.m.cols)) {
                    swiglu_off.push_back(~0ULL);
                } else {
                    swiglu_off.push_back(off);
                    off += 2 * (wmat_data_bytes(tg.m.fmt, tg.m.rows, tg.m.cols) + wmat_scale_bytes(tg.m.fmt, tg.m.rows, tg.m.cols));
                    off = align256(off);
                }
                swiglu_v3_off.push_back(off);
                off += 2 * (wmat_data_bytes(tg.m.fmt, tg.m.rows, tg.m.cols) + wmat_scale_bytes(tg.m.fmt, tg.m.rows, tg.m.cols));
                off = align256(off);
            } else if (tg.m.fmt == VB_FMT_I8PC && tile_q4_supported(tg.m.rows, tg.m.cols)) {
                swiglu_off.push_back(~0ULL);
                swiglu_v3_off.push_back(off);  // 2*rows x cols of blocks, then 2*rows scales
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
        t.m.data = s.data != ~0ULL ? c->arena + s.data : nullptr;
        t.m.scales = (s.scales != ~0ULL && wmat_scale_bytes(t.m.fmt, t.m.rows, t.m.cols)) ? c->arena + s.scales : nullptr;
        if (s.has_tiled) { t.m.tiled = c->arena + s.tiled; t.m.tiled_scales = c->arena + s.tiled_scales; }
        if (s.v3 != ~0ULL) t.m.v3 = c->arena + s.v3;
        if (s.v3_scales != ~0ULL) t.m.v3_scales = c->arena + s.v3_scales;
    }
    for (uint32_t l = 0; l < c->d.n_layers; ++l) {
        if (swiglu_off[l] != ~0ULL) c->tensor(VB_ROLE_WGATE, (int)l).m.tiled_swiglu = c->arena + swiglu_off[l];
        if (swiglu_v3_off[l] != ~0ULL) c->tensor(VB_ROLE_WGATE, (int)l).m.v3_swiglu = c->arena + swiglu_v3_off[l];
    }
    if (c->d.tied_lm_head) set_tied_head(c);
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
                            uint32_t pos, uint32_t active, uint32_t limit) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        state[slot].token = tokens ? tokens[idx] : token;
        state[slot].pos = pos;
        state[slot].active = (limit && pos >= limit) ? 0u : active;
        state[slot].limit = limit;
    }
}
__global__ void k_set_limit(SeqState* state, uint32_t slot, uint32_t limit) {
    if (threadIdx.x == 0 && blockIdx.x == 0) state[slot].limit = limit;
}

// rows j < n of a prefill chunk: prompt token first + j at position first + j; rows beyond n inactive
__global__ void k_set_chunk_state(SeqState* state, const uint32_t* tokens, uint32_t first, uint32_t n, uint32_t rows) {
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < rows) {
        state[j].token = j < n ? tokens[first + j] : 0u;
        state[j].pos = first + j;
        state[j].active = j < n ? 1u : 0u;
        state[j].limit = 0;  // the host checked the chunk against the reservation
    }
}

// every row of the chunk's block table = the prefilled sequence's row
__global__ void k_fill_chunk_table(int32_t* dst, const int32_t* src_row, uint32_t max_blocks) {
    for (uint32_t i = threadIdx.x; i < max_blocks; i += blockDim.x) dst[(size_t)blockIdx.x * max_blocks + i] = src_row[i];
}

// The four products of a layer can run as tensor-core GEMMs when their canonical copies are resident (not with
// VB_FLAG_LEAN_WEIGHTS) in a format the conversion kernel reads.
bool tc_products_ok(vb_ctx* c) {
    const int roles[] = {VB_ROLE_WQ, VB_ROLE_WO, VB_ROLE_WGATE, VB_ROLE_WUP, VB_ROLE_WDOWN};
    for (int role : roles) {
        GemvArgs a;
        a.w = c->tensor(role, 0).m;
        if (role == VB_ROLE_WQ) a.w.rows = c->qkv_rows;
        if (!gemm_tc_supported(a)) return false;
    }
    return true;
}

// Workspace of the tensor-core products for `rows` rows of x (fp16 operands): the largest of a layer's four
// products, and of the lm_head when `with_head`.
int32_t ensure_tc_ws(vb_ctx* c, uint32_t rows, bool with_head) {
    const uint32_t dm = c->d.d_model;
    uint64_t need = gemm_tc_workspace_bytes(c->qkv_rows, dm, rows, false);
    need = std::max(need, gemm_tc_workspace_bytes(dm, c->qdim, rows, false));
    need = std::max(need, gemm_tc_workspace_bytes(c->ffn, dm, rows, true));
    need = std::max(need, gemm_tc_workspace_bytes(dm, c->ffn, rows, false));
    if (with_head) need = std::max(need, gemm_tc_workspace_bytes(c->vocab, dm, rows, false));
    if (c->tc_ws_bytes >= need) return VB_OK;
    if (c->graph_exec) { cudaGraphExecDestroy(c->graph_exec); c->graph_exec = nullptr; }  // a captured step holds the old address
    if (c->tc_ws) cudaFree(c->tc_ws);
    c->tc_ws = nullptr; c->tc_ws_bytes = 0;
    if (cudaMalloc(&c->tc_ws, need + 1024) != cudaSuccess) {  // + 1024: the swizzled operands start on a 1024-byte boundary
        cudaGetLastError();
        set_error("cannot allocate %llu bytes for the tensor-core workspace", (unsigned long long)need);
        return VB_ERR_OOM;
    }
    c->tc_ws_bytes = need;
    VB_CUDA(cudaMemsetAsync((void*)(((uintptr_t)c->tc_ws + 1023) & ~(uintptr_t)1023), 0, gemm_tc_workspace_zero_bytes(), c->stream));  // split-K tile counters
    return VB_OK;
}

// One fp16 copy of every layer matrix (QKV as one block), when they fit the budget.  Tried once per context.
int32_t ensure_f16_copies(vb_ctx* c) {
    if (c->f16_tried) return VB_OK;
    c->f16_tried = true;
    if (c->d.weight_fmt == VB_FMT_F16 || c->tc_resident_gb == 0) return VB_OK;
    const uint64_t dm = c->d.d_model;
    // weights fp16 does not hold exactly also get the part its rounding dropped (prefill chunks multiply hi + lo)
    const bool with_lo = gemm_tc_split >= 2 && gemm_tc_weights_inexact((int32_t)c->d.weight_fmt);
    const uint64_t per_layer = (((uint64_t)c->qkv_rows * dm + dm * c->qdim + 3ull * c->ffn * dm) * 2 + 5 * 1024) * (with_lo ? 2 : 1);
    Tensor& head = c->tensor(VB_ROLE_LM_HEAD, 0);
    // decode batches run the lm_head as a tensor-core product too: through a resident fp16 copy unless the integer kernel reads int8 directly
    const bool with_head = c->decode_gemm && head.m.fmt != VB_FMT_F16 && head.m.data != nullptr &&
                           !(gemm_i8_enabled && head.m.fmt == VB_FMT_I8PC && c->d.max_batch <= 32);
    const uint64_t total = per_layer * c->d.n_layers + (with_head ? (uint64_t)head.m.rows * head.m.cols * 2 + 1024 : 0);
    if (total > (uint64_t)c->tc_resident_gb << 30) return VB_OK;
    if (cudaMalloc(&c->f16_pool, total + 1024) != cudaSuccess) { cudaGetLastError(); c->f16_pool = nullptr; return VB_OK; }
    unsigned char* p = (unsigned char*)(((uintptr_t)c->f16_pool + 1023) & ~(uintptr_t)1023);
    const int roles[] = {VB_ROLE_WQ, VB_ROLE_WO, VB_ROLE_WGATE, VB_ROLE_WUP, VB_ROLE_WDOWN};
    for (uint32_t l = 0; l < c->d.n_layers; ++l)
        for (int role : roles) {
            Tensor& t = c->tensor(role, (int)l);
            WMat m = t.m;
            if (role == VB_ROLE_WQ) m.rows = c->qkv_rows;
            const uint64_t bytes = ((uint64_t)m.rows * m.cols * 2 + 1023) / 1024 * 1024;
            VB_CUDA(weights_to_f16(lcfg(c, false), p, m, with_lo ? p + bytes : nullptr));
            t.m.f16 = p;
            t.m.f16_lo = with_lo ? p + bytes : nullptr;
            p += bytes * (with_lo ? 2 : 1);
        }
    if (with_head) {
        VB_CUDA(weights_to_f16(lcfg(c, false), p, head.m));
        head.m.f16 = p;
    }
    VB_CUDA(cudaStreamSynchronize(c->stream));
    return VB_OK;
}

// Tile-major int8 copies (shared-memory order) of every layer matrix and the head for the integer tensor-core decode
// batches: one contiguous 16 KB bulk copy per tile.  Tried once per context; without them the kernel reads the canonical
// matrices through tiled TMA.
int32_t ensure_i8_tiles(vb_ctx* c) {
    if (c->i8_tiles_tried) return VB_OK;
    c->i8_tiles_tried = true;
    if (!gemm_i8_tiles) return VB_OK;
    const int roles[] = {VB_ROLE_WQ, VB_ROLE_WO, VB_ROLE_WGATE, VB_ROLE_WUP, VB_ROLE_WDOWN};
    auto rows_of = [&](int role, const Tensor& t) { return role == VB_ROLE_WQ ? c->qkv_rows : t.m.rows; };
    uint64_t total = 0;
    for (uint32_t l = 0; l < c->d.n_layers; ++l)
        for (int role : roles) {
            const Tensor& t = c->tensor(role, (int)l);
            if (t.m.fmt != VB_FMT_I8PC || !t.m.data) return VB_OK;
            total += gemm_i8_tiles_bytes(rows_of(role, t), t.m.cols);
        }
    Tensor& head = c->tensor(VB_ROLE_LM_HEAD, 0);
    const bool with_head = head.m.fmt == VB_FMT_I8PC && head.m.data != nullptr;
    if (with_head) total += gemm_i8_tiles_bytes(head.m.rows, head.m.cols);
    if (total == 0 || total > (uint64_t)c->tc_resident_gb << 30) return VB_OK;
    if (cudaMalloc(&c->i8_tiles_pool, total + 1024) != cudaSuccess) { cudaGetLastError(); c->i8_tiles_pool = nullptr; return VB_OK; }
    unsigned char* p = (unsigned char*)(((uintptr_t)c->i8_tiles_pool + 1023) & ~(uintptr_t)1023);
    LaunchCfg lc = lcfg(c, false);
    lc.counter = nullptr;
    for (uint32_t l = 0; l < c->d.n_layers; ++l)
        for (int role : roles) {
            Tensor& t = c->tensor(role, (int)l);
            const uint64_t bytes = gemm_i8_tiles_bytes(rows_of(role, t), t.m.cols);
            if (bytes == 0) continue;
            VB_CUDA(gemm_i8_make_tiles(lc, p, t.m.data, rows_of(role, t), t.m.cols));
            t.m.i8_tiles = p;
            p += bytes;
        }
    if (with_head && gemm_i8_tiles_bytes(head.m.rows, head.m.cols)) {
        VB_CUDA(gemm_i8_make_tiles(lc, p, head.m.data, head.m.rows, head.m.cols));
        head.m.i8_tiles = p;
    }
    VB_CUDA(cudaStreamSynchronize(c->stream));
    return VB_OK;
}

// decode_gemm: make sure, outside any capture, that the products can take that path and that the workspace is there
int32_t prepare_decode_gemm(vb_ctx* c) {
    if (!c->decode_gemm) return VB_OK;
    if (!tc_products_ok(c)) {
        if (c->decode_gemm_auto) { c->decode_gemm = false; return VB_OK; }
        set_error("decode_gemm needs the canonical weight copies (not VB_FLAG_LEAN_WEIGHTS) in a format the tensor-core path reads");
        return VB_ERR_UNSUPPORTED;
    }
    int32_t rc = ensure_f16_copies(c);
    if (rc != VB_OK) return rc;
    if (gemm_i8_enabled && c->d.weight_fmt == VB_FMT_I8PC && c->d.max_batch <= 32 && !c->i8_ws) {
        const uint64_t need = gemm_i8_workspace_bytes(std::max(std::max(c->d.d_model, c->ffn), c->qdim));
        if (cudaMalloc(&c->i8_ws, need + 1024) != cudaSuccess) { cudaGetLastError(); c->i8_ws = nullptr; }
        else {
            c->i8_ws_bytes = need;
            VB_CUDA(cudaMemsetAsync((void*)(((uintptr_t)c->i8_ws + 1023) & ~(uintptr_t)1023), 0, gemm_i8_workspace_zero_bytes(), c->stream));
        }
    }
    if (c->i8_ws && (rc = ensure_i8_tiles(c)) != VB_OK) return rc;
    return ensure_tc_ws(c, std::max(c->d.max_batch, c->prefill_rows), true);
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

void* tc_ws_aligned(vb_ctx* c) { return (void*)(((uintptr_t)c->tc_ws + 1023) & ~(uintptr_t)1023); }
StepIO decode_io(vb_ctx* c) {
    StepIO io{c->hidden, c->qkv, c->q, c->attn_out, c->act, c->logits, c->block_table_dev, c->d.max_batch, true};
    // wide batches: the products (lm_head included) as tensor-core GEMMs, one row of x per slot
    if (c->decode_gemm && c->tc_ws && c->d.tp_size <= 1) {
        io.tc_ws = tc_ws_aligned(c); io.tc_ws_bytes = c->tc_ws_bytes;
        if (c->i8_ws) { io.i8_ws = (void*)(((uintptr_t)c->i8_ws + 1023) & ~(uintptr_t)1023); io.i8_ws_bytes = c->i8_ws_bytes; }
    }
    return io;
}

// The launch sequence of one token for every active row of `state`.
cudaError_t enqueue_step(vb_ctx* c, SeqState* state, bool with_head, const StepIO& io) {
    const vb_model_desc& d = c->d;
    const uint32_t B = io.B;
    cudaError_t e;
    uint32_t tn = 0;
    auto next_trace = [&]() -> unsigned long long* { return (c->trace && tn < 1024) ? c->trace + 4 * (size_t)(tn++) : nullptr; };
#define VB_TRY(x) do { e = (x); if (e != cudaSuccess) return e; } while (0)
    Tensor& emb = c->tensor(VB_ROLE_EMBED, 0);
    // the first kernel of a step must not overlap the previous step's tail: launched without PDL
    VB_TRY(embed(lcfg(c, false), io.hidden, nullptr, state, emb.m.data, emb.m.scales, emb.m.fmt, d.d_model, d.vocab, B));
    // Tensor parallel: O and down are row-parallel.  Rank 0 adds its partial product onto the residual stream,
    // the other ranks overwrite theirs with the bare partial; one in-place sum all-reduce then leaves the new
    // residual stream, bit-identical, on every rank (no separate residual-add pass).
    // With NVLink peer mappings every rank instead stores its partial, pushes it to all peers and each rank
    // sums the parts onto its residual stream in rank order (tp_reduce): one small kernel, no fence, no flag.
    const bool tp = d.tp_size > 1;
    const bool p2p = tp && c->links_open && c->use_links;
    const uint32_t n_sites = 2 * d.n_layers + 1;
    const int row_epi = (!tp || (!p2p && d.tp_rank == 0)) ? EPI_RESIDUAL : EPI_STORE;
    float* row_dst = p2p ? c->partial : io.hidden;
    if (p2p) VB_TRY(tp_epoch_advance(lcfg(c, false), c->links));
    bool pushed = false;  // set by the row-parallel product when its own epilogue sent the rows to the peers
    bool reduced = false; // ... and when it also gathered the peers' rows and updated the residual stream itself
    auto exchange = [&](uint32_t site) -> cudaError_t {
        if (!tp) return cudaSuccess;
        if (p2p && reduced) return cudaSuccess;
        if (p2p) return tp_reduce(lcfg(c, true), c->links, io.hidden, c->partial, B * d.d_model, site, n_sites, c->err_word, pushed, state, d.d_model);
        return nccl_allreduce_sum_f32(c->nccl, io.hidden, (size_t)B * d.d_model, c->stream) == VB_OK ? cudaSuccess : cudaErrorUnknown;
    };
    auto product = [&](const GemvArgs& ga) -> cudaError_t {
        if (io.i8_ws && gemm_i8_supported(ga)) return gemm_i8(lcfg(c, true), ga, io.i8_ws, io.i8_ws_bytes, true);
        if (io.tc_ws) return gemm_tc(lcfg(c, true), ga, io.tc_ws, io.tc_ws_bytes, true);
        return gemv(lcfg(c, true), ga, c->gemv_path);
    };
    for (uint32_t l = 0; l < d.n_layers; ++l) {
        const int L = (int)l;
        // RMSNorm + fused QKV projection
        GemvArgs g;
        g.state = state; g.batch = B;
        g.x = io.hidden; g.dst = io.qkv;
        g.norm_w = c->tensor(VB_ROLE_ATTN_NORM, L).m.data; g.norm_fmt = c->tensor(VB_ROLE_ATTN_NORM, L).m.fmt; g.eps = d.rms_eps;
        g.w = c->tensor(VB_ROLE_WQ, L).m; g.w.rows = c->qkv_rows;
        g.trace = next_trace(); g.max_ring = c->ring_role[0] ? c->ring_role[0] : c->gemv_ring;
        VB_TRY(product(g));
        // bias + RoPE + KV append
        __half* kv_layer = c->kv_pool + (size_t)l * c->kv_layer_elems;
        const void *bq = nullptr, *bk = nullptr, *bv = nullptr; int bf = VB_FMT_F32;
        if (d.qkv_bias) {
            bq = c->tensor(VB_ROLE_BQ, L).m.data; bk = c->tensor(VB_ROLE_BK, L).m.data; bv = c->tensor(VB_ROLE_BV, L).m.data;
            bf = c->tensor(VB_ROLE_BQ, L).m.fmt;
        }
        const bool fused_append = (c->hq / c->hkv) <= 8 && c->fuse_append && io.fused_append;
        if (!fused_append)
            VB_TRY(bias_rope_kv_append(lcfg(c, true), io.q, io.qkv, state, bq, bk, bv, bf, kv_layer, io.block_table,
                                       c->max_blocks, c->hq, c->hkv, d.head_dim, d.kv_block_tokens, d.rope_theta, B));
        // split-K attention over the paged cache (with the bias + RoPE + KV append fused in when possible)
        AttnArgs a;
        a.out = io.attn_out; a.q = io.q; a.k = kv_layer; a.kv_fp16 = 1;
        if (fused_append) { a.qkv_raw = io.qkv; a.bq = bq; a.bk = bk; a.bv = bv; a.bias_fmt = bf; a.rope_inv_freq = c->rope_inv_freq; a.rope_inv_freq_host = c->rope_inv_freq_host.data(); }
        a.block_table = io.block_table; a.max_blocks = c->max_blocks; a.block_tokens = d.kv_block_tokens;
        if (c->kv_map_ok) { a.kv_map = c->kv_map; a.kv_map_row0 = (uint32_t)((uint64_t)l * (c->kv_layer_elems / d.head_dim)); }
        a.state = state; a.Hq = c->hq; a.Hkv = c->hkv; a.D = d.head_dim; a.batch = B;
        a.max_splits = c->n_splits; a.tokens_per_split = c->tokens_per_split; a.scratch = c->attn_scratch;
        a.trace = next_trace(); a.err = c->err_word;
        if (io.causal_chunk && c->prefill_flash && attention_prefill_supported(c->hq, c->hkv, d.head_dim))
            VB_TRY(attention_prefill(lcfg(c, true), io.attn_out, io.q, kv_layer, io.block_table, io.first, B, c->hq, c->hkv, d.head_dim, d.kv_block_tokens));
        else
            VB_TRY(attention(lcfg(c, true), a));
        // O-projection + residual
        GemvArgs o;
        o.state = state; o.batch = B; o.x = io.attn_out; o.dst = row_dst; o.epilogue = row_epi;
        o.w = c->tensor(VB_ROLE_WO, L).m;
        o.trace = next_trace(); o.max_ring = c->ring_role[1] ? c->ring_role[1] : c->gemv_ring;
        pushed = false; reduced = false;
        if (p2p && c->tp_fused_push) {
            o.push.links = &c->links; o.push.site = 2 * l; o.push.n_sites = n_sites; o.pushed = &pushed;
            if (c->tp_fused_reduce && B == 1) { o.push.reduce_hidden = io.hidden; o.push.err = c->err_word; o.reduced = &reduced; }
        }
        VB_TRY(product(o));
        VB_TRY(exchange(2 * l));
        // RMSNorm + gate/up + SiLU*up
        GemvArgs gu;
        gu.state = state; gu.batch = B; gu.x = io.hidden; gu.dst = io.act; gu.epilogue = EPI_SWIGLU;
        gu.norm_w = c->tensor(VB_ROLE_MLP_NORM, L).m.data; gu.norm_fmt = c->tensor(VB_ROLE_MLP_NORM, L).m.fmt; gu.eps = d.rms_eps;
        gu.w = c->tensor(VB_ROLE_WGATE, L).m; gu.w2 = c->tensor(VB_ROLE_WUP, L).m;
        gu.trace = next_trace(); gu.max_ring = c->ring_role[2] ? c->ring_role[2] : c->gemv_ring;
        VB_TRY(product(gu));
        // down projection + residual
        GemvArgs dn;
        dn.state = state; dn.batch = B; dn.x = io.act; dn.dst = row_dst; dn.epilogue = row_epi;
        dn.w = c->tensor(VB_ROLE_WDOWN, L).m;
        dn.trace = next_trace(); dn.max_ring = c->ring_role[3] ? c->ring_role[3] : c->gemv_ring;
        pushed = false; reduced = false;
        if (p2p && c->tp_fused_push) {
            dn.push.links = &c->links; dn.push.site = 2 * l + 1; dn.push.n_sites = n_sites; dn.pushed = &pushed;
            if (c->tp_fused_reduce && B == 1) { dn.push.reduce_hidden = io.hidden; dn.push.err = c->err_word; dn.reduced = &reduced; }
        }
        VB_TRY(product(dn));
        VB_TRY(exchange(2 * l + 1));
    }
    if (with_head) {
        GemvArgs h;
        h.state = state; h.batch = B; h.x = io.hidden; h.dst = io.logits;
        h.norm_w = c->tensor(VB_ROLE_FINAL_NORM, 0).m.data; h.norm_fmt = c->tensor(VB_ROLE_FINAL_NORM, 0).m.fmt; h.eps = d.rms_eps;
        h.w = c->tensor(VB_ROLE_LM_HEAD, 0).m;
        h.trace = next_trace(); h.max_ring = c->head_ring;
        if (io.i8_ws && gemm_i8_supported(h)) VB_TRY(gemm_i8(lcfg(c, true), h, io.i8_ws, io.i8_ws_bytes, true));
        else if (io.tc_ws && gemm_tc_supported(h)) VB_TRY(gemm_tc(lcfg(c, true), h, io.tc_ws, io.tc_ws_bytes, true));
        else VB_TRY(gemv(lcfg(c, true), h, c->gemv_path));
        if (!tp && c->sample_probs && c->sample_temperature > 1e-5f && c->sample_top_p > 0.0f && io.logits == c->logits) {
            VB_TRY(sample_top_p(lcfg(c, true), nullptr, io.logits, c->sample_probs, c->vocab, B, c->sample_temperature, c->sample_top_p,
                                c->sample_mode, nullptr, 0.0f, 1, c->sample_seed, state, c->ring_dev, RING_SLOTS));
        } else if (!tp) {
            VB_TRY(argmax(lcfg(c, true), nullptr, io.logits, c->vocab, B, c->cand_v, c->cand_i, state, c->ring_dev, RING_SLOTS));
        } else {
            // vocab-parallel head: best (value, global index) per rank, gathered, same tie rule over the ranks
            VB_TRY(argmax_shard(lcfg(c, true), c->tp_pair, io.logits, c->vocab, c->vocab_off, B, c->cand_v, c->cand_i, state));
            if (p2p) {
                VB_TRY(tp_argmax(lcfg(c, true), c->links, c->tp_pair, B, 2 * d.n_layers, n_sites, state, c->ring_dev, RING_SLOTS, c->err_word));
            } else {
                if (nccl_allgather_bytes(c->nccl, c->tp_pair, c->tp_pairs, (size_t)B * 8, c->stream) != VB_OK) return cudaErrorUnknown;
                VB_TRY(argmax_pairs(lcfg(c, false), c->tp_pairs, d.tp_size, B, state, c->ring_dev, RING_SLOTS));
            }
        }
    }
#undef VB_TRY
    c->trace_n = tn;
    return cudaSuccess;
}

int32_t ensure_chunk_buffers(vb_ctx* c, uint32_t cap) {
    if (c->pfc_rows >= cap) return VB_OK;
    int32_t rc;
    void* old[] = {c->pfc_state, c->pfc_table, c->pfc_hidden, c->pfc_qkv, c->pfc_q, c->pfc_attn, c->pfc_act};
    for (void* p : old) if (p) cudaFree(p);
    c->pfc_state = nullptr; c->pfc_table = nullptr; c->pfc_hidden = c->pfc_qkv = c->pfc_q = c->pfc_attn = c->pfc_act = nullptr;
    c->pfc_rows = 0;
    if ((rc = dev_alloc(&c->pfc_state, cap)) != VB_OK || (rc = dev_alloc(&c->pfc_table, (uint64_t)cap * c->max_blocks)) != VB_OK ||
        (rc = dev_alloc(&c->pfc_hidden, (uint64_t)cap * c->d.d_model)) != VB_OK || (rc = dev_alloc(&c->pfc_qkv, (uint64_t)cap * c->qkv_rows)) != VB_OK ||
        (rc = dev_alloc(&c->pfc_q, (uint64_t)cap * c->qdim)) != VB_OK || (rc = dev_alloc(&c->pfc_attn, (uint64_t)cap * c->qdim)) != VB_OK ||
        (rc = dev_alloc(&c->pfc_act, (uint64_t)cap * c->ffn)) != VB_OK)
        return rc;
    c->pfc_rows = cap;
    return VB_OK;
}

int32_t check_ready(vb_ctx* c, const char* who) {
    if (!c) { set_error("%s: null context", who); return VB_ERR_INVALID; }
    const char* missing = nullptr;
    if (!all_loaded(c, &missing)) { set_error("%s: tensor '%s' has not been loaded", who, missing); return VB_ERR_STATE; }
    if (c->d.tp_size > 1 && !c->nccl && !(c->links_open && c->use_links)) {
        set_error("%s: tensor-parallel context without a communicator (call vb_tp_init or vb_tp_p2p_open)", who);
        return VB_ERR_STATE;
    }
    return VB_OK;
}

}  // namespace vb

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
    VB_REQUIRE((d.flags & ~VB_FLAG_LEAN_WEIGHTS) == 0, "vb_create: unknown flags 0x%x", d.flags);
    VB_REQUIRE(!(d.flags & VB_FLAG_LEAN_WEIGHTS) || d.max_batch == 1, "vb_create: VB_FLAG_LEAN_WEIGHTS serves max_batch == 1 only");
    const uint32_t tp = d.tp_size ? d.tp_size : 1;
    VB_REQUIRE(tp <= 64 && d.tp_rank < tp, "vb_create: tp_rank=%u / tp_size=%u", d.tp_rank, tp);
    if (tp > 1) {
        VB_REQUIRE(d.n_kv_heads % tp == 0 && d.n_q_heads % tp == 0, "vb_create: heads (%u q, %u kv) not divisible by tp_size=%u",
                   d.n_q_heads, d.n_kv_heads, tp);
        VB_REQUIRE(d.ffn_dim % 128 == 0 && d.ffn_dim / 128 >= tp, "vb_create: tensor parallel needs ffn_dim in whole 128-column blocks");
        VB_REQUIRE(d.vocab % (16 * tp) == 0, "vb_create: vocab=%u not divisible by 16*tp_size", d.vocab);
        VB_REQUIRE(fmt_shape_ok((int32_t)d.weight_fmt, d.n_q_heads / tp * d.head_dim), "vb_create: per-rank attention width breaks the quantization group");
        // per-row scales of a column slice would differ from the whole row's: int8 per-channel stays single-GPU
        if (d.weight_fmt == VB_FMT_I8PC) { set_error("vb_create: VB_FMT_I8PC weights cannot be sharded (per-row scales)"); return VB_ERR_UNSUPPORTED; }
    }

    VB_CUDA(cudaSetDevice(device));
    VB_CUDA(kernels_init());
    vb_ctx* c = new (std::nothrow) vb_ctx();
    if (!c) { set_error("vb_create: out of host memory"); return VB_ERR_OOM; }
    c->d = d;
    c->device = device;
    c->hq = d.n_q_heads / tp;
    c->hkv = d.n_kv_heads / tp;
    c->qdim = c->hq * d.head_dim;
    c->kvdim = c->hkv * d.head_dim;
    c->qkv_rows = c->qdim + 2 * c->kvdim;
    {
        // FFN columns in whole 128-column blocks, the first (blocks % tp) ranks take one more: quantization
        // groups (32 columns) never straddle ranks, so every shard dequantizes to the same values as TP-1
        const uint32_t nb = tp > 1 ? d.ffn_dim / 128 : 0, per = tp > 1 ? nb / tp : 0, extra = tp > 1 ? nb % tp : 0;
        c->ffn = tp > 1 ? 128 * (per + (d.tp_rank < extra ? 1 : 0)) : d.ffn_dim;
        c->ffn_off = tp > 1 ? 128 * (per * d.tp_rank + (d.tp_rank < extra ? d.tp_rank : extra)) : 0;
        c->vocab = d.vocab / tp;
        c->vocab_off = c->vocab * d.tp_rank;
    }
    // wide batches of weights that fp16 holds exactly (int8 per channel, fp16): decode products as tensor-core GEMMs
    c->decode_gemm = c->decode_gemm_auto = d.max_batch >= 16 && tp <= 1 && (d.weight_fmt == VB_FMT_I8PC || d.weight_fmt == VB_FMT_F16);
    c->max_blocks = (d.max_seq_len + d.kv_block_tokens - 1) / d.kv_block_tokens;
    c->n_blocks = d.kv_blocks_total ? d.kv_blocks_total : d.max_batch * c->max_blocks;
    c->n_splits = attn_pick_splits(d.max_seq_len);
    {
        // wide batches already fill the SMs with (sequence, KV head) pairs: fewer, longer slices per pair then stream the
        // cache instead of paying a block's fixed costs (table fetch, cluster merge) for every ~150 rows
        const uint32_t g = c->hq / c->hkv, pairs = d.max_batch * c->hkv * ((g + 7) / 8);
        const uint32_t fit = pairs ? 148u / pairs : 8u;  // one block per SM: two 128-token staging buffers take most of its shared memory
        if (c->n_splits > (fit ? fit : 1u)) c->n_splits = fit ? fit : 1u;
    }
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
    c->kv_layer_elems = (uint64_t)c->n_blocks * 2 * c->hkv * d.kv_block_tokens * d.head_dim;
    VB_CREATE_TRY(dev_alloc(&c->kv_pool, c->kv_layer_elems * d.n_layers));
    VB_CREATE_CUDA(cudaMemsetAsync(c->kv_pool, 0, c->kv_layer_elems * d.n_layers * sizeof(__half), c->stream));
    // the decode attention's tensor-core path stages whole KV blocks with tiled TMA copies
    c->kv_map_ok = d.kv_block_tokens == 16 && attn_make_kv_map(c->kv_map, c->kv_pool, c->kv_layer_elems * d.n_layers / d.head_dim, d.head_dim);
    VB_CREATE_TRY(dev_alloc(&c->block_table_dev, (uint64_t)d.max_batch * c->max_blocks));
    c->block_table_host.assign((size_t)d.max_batch * c->max_blocks, 0);
    VB_CREATE_CUDA(cudaMemsetAsync(c->block_table_dev, 0, (size_t)d.max_batch * c->max_blocks * 4, c->stream));
    c->free_blocks.reserve(c->n_blocks);
    for (int32_t b = (int32_t)c->n_blocks - 1; b >= 0; --b) c->free_blocks.push_back(b);
    c->slot_blocks.assign(d.max_batch, 0);
    c->pos_hi.assign(d.max_batch, 0);
    c->maybe_active.assign(d.max_batch, 0);
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
    VB_CREATE_TRY(dev_alloc(&c->act, B * c->ffn));
    VB_CREATE_TRY(dev_alloc(&c->logits, B * c->vocab));
    if (tp > 1) {
        VB_CREATE_TRY(dev_alloc(&c->partial, B * d.d_model));
        VB_CREATE_TRY(dev_alloc(&c->tp_pair, B * 8));
        VB_CREATE_TRY(dev_alloc(&c->tp_pairs, B * 8 * tp));
    }
    VB_CREATE_TRY(dev_alloc(&c->attn_scratch, attn_scratch_floats(c->hq, d.head_dim, d.max_batch, c->n_splits)));
    VB_CREATE_CUDA(cudaMemsetAsync(c->attn_scratch, 0, attn_scratch_floats(c->hq, d.head_dim, d.max_batch, c->n_splits) * 4, c->stream));
    VB_CREATE_TRY(dev_alloc(&c->cand_v, B * argmax_chunks(c->vocab)));
    VB_CREATE_TRY(dev_alloc(&c->cand_i, B * argmax_chunks(c->vocab)));
    {
        // RoPE frequencies exactly as the reference computes them on the host (src/runtime.rs:758)
        std::vector<float> f(d.head_dim / 2);
        for (uint32_t j = 0; j < d.head_dim / 2; ++j) f[j] = 1.0f / powf(d.rope_theta, (float)(2 * j) / (float)d.head_dim);
        c->rope_inv_freq_host = f;
        VB_CREATE_TRY(dev_alloc(&c->rope_inv_freq, f.size()));
        VB_CREATE_CUDA(cudaMemcpyAsync(c->rope_inv_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice, c->stream));
        VB_CREATE_CUDA(cudaStreamSynchronize(c->stream));
    }
    VB_CREATE_CUDA(fast_error_word(&c->err_word));
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
    if (c->nccl) nccl_comm_destroy(c->nccl);
    for (uint32_t r = 0; r < 8; ++r)
        if (c->links.base[r] && r != c->links.rank) { if (c->links_standin) cudaFree(c->links.base[r]); else cudaIpcCloseMemHandle(c->links.base[r]); }
    if (c->links.base[c->links.rank]) cudaFree(c->links.base[c->links.rank]);
    void* frees[] = {c->arena, c->kv_pool, c->block_table_dev, c->state, c->pf_state, c->pf_tokens, c->hidden, c->qkv, c->q,
                     c->attn_out, c->act, c->logits, c->attn_scratch, c->cand_v, c->cand_i, c->rope_inv_freq, c->trace, c->partial, c->tp_pair, c->tp_pairs,
                     c->pfc_state, c->pfc_table, c->pfc_hidden, c->pfc_qkv, c->pfc_q, c->pfc_attn, c->pfc_act, c->tc_ws, c->f16_pool, c->i8_tiles_pool, c->sample_probs,
                     c->spec_logits, c->spec_cand_v, c->spec_cand_i, c->spec_tokens, c->i8_ws};
    for (void* p : frees) if (p) cudaFree(p);
    if (c->ring_host) cudaFreeHost(c->ring_host);
    if (c->ev0) cudaEventDestroy(c->ev0);
    if (c->ev1) cudaEventDestroy(c->ev1);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
    return VB_OK;
}

// What a loader was handed: the whole tensor (every rank passes the same checkpoint tensor and keeps its own
// rectangle) or, when `whole` is false, exactly this rank's shard.
struct LoadView {
    Tensor* t = nullptr;
    bool whole = false;
    uint32_t full_rows = 0, full_cols = 0, r0 = 0, c0 = 0;
};

static int32_t load_common(vb_ctx* c, int32_t role, int32_t layer, uint64_t rows, uint64_t cols, LoadView* out, const char* who) {
    VB_REQUIRE(c != nullptr, "%s: null context", who);
    VB_REQUIRE(role >= 0 && role <= VB_ROLE_BV, "%s: role %d is not an engine tensor", who, role);
    if (role_is_global(role)) layer = 0;
    VB_REQUIRE(layer >= 0 && (uint32_t)layer < c->d.n_layers, "%s: layer %d out of range", who, layer);
    uint32_t er, ec; int32_t fmt;
    VB_REQUIRE(role_shape(c, role, &er, &ec, &fmt), "%s: role %d is not part of this model", who, role);
    VB_REQUIRE(!(role == VB_ROLE_LM_HEAD && c->d.tied_lm_head), "%s: lm_head is tied to the embedding table", who);
    role_slice(c, role, &out->full_rows, &out->full_cols, &out->r0, &out->c0);
    const bool vec = role_is_vector(role);
    const bool is_shard = rows * cols == (uint64_t)er * ec && (rows == er || vec);
    const bool is_whole = rows * cols == (uint64_t)out->full_rows * out->full_cols && (rows == out->full_rows || vec);
    VB_REQUIRE(is_shard || is_whole, "%s: role %d expects [%u][%u] (whole tensor) or [%u][%u] (this rank's shard), got [%llu][%llu]",
               who, role, out->full_rows, out->full_cols, er, ec, (unsigned long long)rows, (unsigned long long)cols);
    out->whole = is_whole && (out->full_rows != er || out->full_cols != ec);
    out->t = &c->tensor(role, layer);
    VB_CUDA(cudaSetDevice(c->device));
    if (c->graph_exec) { cudaGraphExecDestroy(c->graph_exec); c->graph_exec = nullptr; }
    return VB_OK;
}

// Canonical (row-major packed) storage of a tensor while it is being loaded: its place in the arena, or for a
// lean context a temporary that lives until the tile-major copy has been made.
struct Canon {
    void* data = nullptr;
    void* scales = nullptr;
    void* tmp = nullptr;
    ~Canon() { if (tmp) cudaFree(tmp); }
};

static int32_t canon_begin(Tensor* t, Canon* cn) {
    const uint64_t db = wmat_data_bytes(t->m.fmt, t->m.rows, t->m.cols), sb = wmat_scale_bytes(t->m.fmt, t->m.rows, t->m.cols);
    if (t->m.data) { cn->data = const_cast<void*>(t->m.data); cn->scales = const_cast<void*>(t->m.scales); return VB_OK; }
    cudaError_t e = cudaMalloc(&cn->tmp, align256(db) + sb + 256);
    if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc(staging)", __FILE__, __LINE__); return VB_ERR_OOM; }
    cn->data = cn->tmp;
    cn->scales = sb ? (unsigned char*)cn->tmp + align256(db) : nullptr;
    return VB_OK;
}

static int32_t finish_load(vb_ctx* c, Tensor* t, int32_t role, int32_t layer, const Canon& cn) {
    LaunchCfg lc = lcfg(c, false);
    lc.counter = nullptr;
    if (t->m.tiled) VB_CUDA(tile_q4(lc, const_cast<void*>(t->m.tiled), const_cast<void*>(t->m.tiled_scales), cn.data, cn.scales, t->m.rows, t->m.cols));
    if (t->m.v3 && t->m.fmt == VB_FMT_Q4G32) VB_CUDA(tile_q4_v3(lc, const_cast<void*>(t->m.v3), cn.data, cn.scales, t->m.rows, t->m.cols));
    if (t->m.v3 && t->m.fmt == VB_FMT_I8PC)
        VB_CUDA(tile_i8_v3(lc, const_cast<void*>(t->m.v3), const_cast<void*>(t->m.v3_scales), cn.data, cn.scales, t->m.rows, t->m.cols));
    if (role == VB_ROLE_WGATE || role == VB_ROLE_WUP) {
        const int which = role == VB_ROLE_WUP ? 1 : 0;
        const void* il = c->tensor(VB_ROLE_WGATE, layer).m.tiled_swiglu;
        if (il) VB_CUDA(tile_q4_swiglu(lc, const_cast<void*>(il), cn.data, cn.scales, t->m.rows, t->m.cols, which));
        const void* il3 = c->tensor(VB_ROLE_WGATE, layer).m.v3_swiglu;
        if (il3 && t->m.fmt == VB_FMT_Q4G32) VB_CUDA(tile_q4_v3_swiglu(lc, const_cast<void*>(il3), cn.data, cn.scales, t->m.rows, t->m.cols, which));
        if (il3 && t->m.fmt == VB_FMT_I8PC) {
            unsigned char* sc = (unsigned char*)const_cast<void*>(il3) + 2 * wmat_data_bytes(t->m.fmt, t->m.rows, t->m.cols);
            VB_CUDA(tile_i8_v3_swiglu(lc, const_cast<void*>(il3), sc, cn.data, cn.scales, t->m.rows, t->m.cols, which));
        }
    }
    VB_CUDA(cudaStreamSynchronize(c->stream));
    return VB_OK;
}

// Marks the tensor loaded and brings the resident fp16 copy the tensor-core products read (made once, on first use)
// up to date with it: a tensor reloaded later must not leave those products on the old weights.  The fused QKV copy
// belongs to Wq; a tied head's copy follows the embedding table.
static int32_t mark_loaded(vb_ctx* c, int32_t role, int32_t layer, Tensor* t) {
    t->loaded = true;
    int32_t owner_role = (role == VB_ROLE_WK || role == VB_ROLE_WV) ? VB_ROLE_WQ : role;
    if (role == VB_ROLE_EMBED && c->d.tied_lm_head) {  // tied: the head reads the table
        const void* keep = c->tensor(VB_ROLE_LM_HEAD, 0).m.f16;
        const void* keep8 = c->tensor(VB_ROLE_LM_HEAD, 0).m.i8_tiles;
        set_tied_head(c);
        c->tensor(VB_ROLE_LM_HEAD, 0).m.f16 = keep;
        c->tensor(VB_ROLE_LM_HEAD, 0).m.i8_tiles = keep8;
        owner_role = VB_ROLE_LM_HEAD;
    }
    Tensor& o = c->tensor(owner_role, role_is_global(owner_role) ? 0 : layer);
    if (o.m.f16 && o.m.data) {
        WMat m = o.m;
        if (owner_role == VB_ROLE_WQ) m.rows = c->qkv_rows;
        LaunchCfg lc = lcfg(c, false);
        lc.counter = nullptr;
        VB_CUDA(weights_to_f16(lc, const_cast<void*>(o.m.f16), m, const_cast<void*>(o.m.f16_lo)));
        VB_CUDA(cudaStreamSynchronize(c->stream));
    }
    if (o.m.i8_tiles && o.m.data && o.m.fmt == VB_FMT_I8PC) {  // the tile-major int8 copy follows the canonical one too
        LaunchCfg lc = lcfg(c, false);
        lc.counter = nullptr;
        VB_CUDA(gemm_i8_make_tiles(lc, const_cast<void*>(o.m.i8_tiles), o.m.data, owner_role == VB_ROLE_WQ ? c->qkv_rows : o.m.rows, o.m.cols));
        VB_CUDA(cudaStreamSynchronize(c->stream));
    }
    return VB_OK;
}

int32_t vb_load_tensor(vb_ctx* c, int32_t role, int32_t layer, const void* src, int32_t src_fmt, int32_t src_loc,
                       uint64_t rows, uint64_t cols) {
    LoadView lv;
    int32_t rc = load_common(c, role, layer, rows, cols, &lv, "vb_load_tensor");
    if (rc != VB_OK) return rc;
    Tensor* t = lv.t;
    VB_REQUIRE(src != nullptr, "vb_load_tensor: null source");
    VB_REQUIRE(src_fmt == VB_FMT_F32 || src_fmt == VB_FMT_F16 || src_fmt == VB_FMT_BF16, "vb_load_tensor: source format %d", src_fmt);
    VB_REQUIRE(src_loc == VB_LOC_HOST || src_loc == VB_LOC_DEVICE, "vb_load_tensor: source location %d", src_loc);
    const uint64_t es = src_fmt == VB_FMT_F32 ? 4 : 2;
    const uint64_t n = (uint64_t)t->m.rows * t->m.cols;  // elements this rank keeps
    // stage: this rank's rectangle of the raw source on the device, then fp32, then the storage format
    void* raw = nullptr;
    float* f32 = nullptr;
    LaunchCfg lc = lcfg(c, false);
    lc.counter = nullptr;
    cudaError_t e = cudaSuccess;
    const void* dev_src = src;
    Canon cn;
    if ((rc = canon_begin(t, &cn)) != VB_OK) return rc;
    if (src_loc == VB_LOC_HOST || lv.whole) {
        if ((e = cudaMalloc(&raw, n * es)) != cudaSuccess) { cuda_fail(e, "cudaMalloc(staging)", __FILE__, __LINE__); return VB_ERR_OOM; }
        const cudaMemcpyKind kind = src_loc == VB_LOC_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
        if (lv.whole) {
            const char* base = (const char*)src + ((uint64_t)lv.r0 * lv.full_cols + lv.c0) * es;
            e = cudaMemcpy2DAsync(raw, (size_t)t->m.cols * es, base, (size_t)lv.full_cols * es, (size_t)t->m.cols * es, t->m.rows, kind, c->stream);
        } else {
            e = cudaMemcpyAsync(raw, src, n * es, kind, c->stream);
        }
        dev_src = raw;
    }
    if (e == cudaSuccess && src_fmt != VB_FMT_F32) {
        if ((e = cudaMalloc((void**)&f32, n * 4)) == cudaSuccess) e = dequantize(lc, f32, dev_src, nullptr, src_fmt, t->m.rows, t->m.cols);
        dev_src = f32;
    }
    if (e == cudaSuccess) e = quantize(lc, cn.data, cn.scales, (const float*)dev_src, t->m.fmt, t->m.rows, t->m.cols);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (raw) cudaFree(raw);
    if (f32) cudaFree(f32);
    if (e != cudaSuccess) return cuda_fail(e, "vb_load_tensor", __FILE__, __LINE__);
    if ((rc = finish_load(c, t, role, layer, cn)) != VB_OK) return rc;
    return mark_loaded(c, role, layer, t);
}

int32_t vb_load_tensor_packed(vb_ctx* c, int32_t role, int32_t layer, const void* data, const void* scales, int32_t src_loc,
                              uint64_t rows, uint64_t cols) {
    LoadView lv;
    int32_t rc = load_common(c, role, layer, rows, cols, &lv, "vb_load_tensor_packed");
    if (rc != VB_OK) return rc;
    Tensor* t = lv.t;
    if (lv.whole) { set_error("vb_load_tensor_packed: a sharded context takes pre-quantized tensors shard by shard"); return VB_ERR_UNSUPPORTED; }
    const uint64_t db = wmat_data_bytes(t->m.fmt, t->m.rows, t->m.cols), sb = wmat_scale_bytes(t->m.fmt, t->m.rows, t->m.cols);
    VB_REQUIRE(data != nullptr && (sb == 0 || scales != nullptr), "vb_load_tensor_packed: null data/scales");
    const cudaMemcpyKind kind = (src_loc == VB_LOC_HOST) ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
    Canon cn;
    if ((rc = canon_begin(t, &cn)) != VB_OK) return rc;
    VB_CUDA(cudaMemcpyAsync(cn.data, data, db, kind, c->stream));
    if (sb) VB_CUDA(cudaMemcpyAsync(cn.scales, scales, sb, kind, c->stream));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    if ((rc = finish_load(c, t, role, layer, cn)) != VB_OK) return rc;
    return mark_loaded(c, role, layer, t);
}

int32_t vb_load_tensor_synthetic(vb_ctx* c, int32_t role, int32_t layer, uint64_t seed, uint64_t stream_id, float mean,
                                 float std, uint64_t rows, uint64_t cols) {
    LoadView lv;
    int32_t rc = load_common(c, role, layer, rows, cols, &lv, "vb_load_tensor_synthetic");
    if (rc != VB_OK) return rc;
    Tensor* t = lv.t;
    // the generator is indexed by position in the WHOLE tensor, so a shard holds the values TP-1 holds there
    VB_REQUIRE(lv.whole || (lv.full_rows == t->m.rows && lv.full_cols == t->m.cols), "vb_load_tensor_synthetic: pass the whole tensor's shape");
    const uint64_t n = (uint64_t)t->m.rows * t->m.cols;
    float* f32 = nullptr;
    Canon cn;
    if ((rc = canon_begin(t, &cn)) != VB_OK) return rc;
    cudaError_t e = cudaMalloc((void**)&f32, n * 4);
    if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc(staging)", __FILE__, __LINE__); return VB_ERR_OOM; }
    LaunchCfg lc = lcfg(c, false);
    lc.counter = nullptr;
    e = lv.whole ? fill_normal_slice(lc, f32, t->m.rows, t->m.cols, lv.full_cols, lv.r0, lv.c0, seed, stream_id, mean, std)
                 : fill_normal(lc, f32, n, seed, stream_id, mean, std);
    if (e == cudaSuccess) e = quantize(lc, cn.data, cn.scales, f32, t->m.fmt, t->m.rows, t->m.cols);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    cudaFree(f32);
    if (e != cudaSuccess) return cuda_fail(e, "vb_load_tensor_synthetic", __FILE__, __LINE__);
    if ((rc = finish_load(c, t, role, layer, cn)) != VB_OK) return rc;
    return mark_loaded(c, role, layer, t);
}

int32_t vb_export_tensor(vb_ctx* c, int32_t role, int32_t layer, void* data, uint64_t data_bytes, void* scales, uint64_t scales_bytes) {
    VB_REQUIRE(c != nullptr, "vb_export_tensor: null context");
    VB_REQUIRE(role >= 0 && role <= VB_ROLE_BV, "vb_export_tensor: role %d", role);
    if (role_is_global(role)) layer = 0;
    VB_REQUIRE(layer >= 0 && (uint32_t)layer < c->d.n_layers, "vb_export_tensor: layer %d out of range", layer);
    Tensor& t = c->tensor(role, layer);
    if (!t.loaded) { set_error("vb_export_tensor: tensor not loaded"); return VB_ERR_STATE; }
    if (!t.m.data) { set_error("vb_export_tensor: a lean context keeps no canonical copy of this matrix"); return VB_ERR_STATE; }
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
    LaunchCfg lc = lcfg(c, false);
    lc.counter = nullptr;
    VB_CUDA(launch(lc, k_set_limit, dim3(1), dim3(32), 0, c->state, (uint32_t)slot, have * c->d.kv_block_tokens));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    return VB_OK;
}

int32_t vb_seq_release(vb_ctx* c, int32_t slot) {
    VB_REQUIRE(c != nullptr, "vb_seq_release: null context");
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_seq_release: slot %d out of range", slot);
    int32_t* row = c->block_table_host.data() + (size_t)slot * c->max_blocks;
    for (uint32_t i = c->slot_blocks[slot]; i > 0; --i) c->free_blocks.push_back(row[i - 1]);
    c->slot_blocks[slot] = 0;
    return vb_seq_set(c, slot, 0, 0, 0);  // also clears the slot's limit and host-side bound
}

int32_t vb_seq_set(vb_ctx* c, int32_t slot, uint32_t token, uint32_t pos, uint32_t active) {
    VB_REQUIRE(c != nullptr, "vb_seq_set: null context");
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_seq_set: slot %d out of range", slot);
    VB_REQUIRE(token < c->d.vocab, "vb_seq_set: token %u >= vocab %u", token, c->d.vocab);
    VB_REQUIRE(!active || pos < c->slot_blocks[slot] * c->d.kv_block_tokens, "vb_seq_set: position %u is beyond the slot's KV reservation (%u tokens)",
               pos, c->slot_blocks[slot] * c->d.kv_block_tokens);
    VB_CUDA(cudaSetDevice(c->device));
    LaunchCfg lc = lcfg(c, false);
    VB_CUDA(launch(lc, k_set_state, dim3(1), dim3(32), 0, c->state, (uint32_t)slot, (const uint32_t*)nullptr, 0u, token, pos, active,
                   c->slot_blocks[slot] * c->d.kv_block_tokens));
    c->pos_hi[slot] = pos;
    c->maybe_active[slot] = active ? 1 : 0;
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
    if ((rc = prepare_decode_gemm(c)) != VB_OK) return rc;  // the last prompt token is a decode-path step
    if (c->pf_tokens_cap < n_tokens) {
        if (c->pf_tokens) cudaFree(c->pf_tokens);
        c->pf_tokens = nullptr; c->pf_tokens_cap = 0;
        rc = dev_alloc(&c->pf_tokens, n_tokens);
        if (rc != VB_OK) return rc;
        c->pf_tokens_cap = n_tokens;
    }
    VB_CUDA(cudaMemcpyAsync(c->pf_tokens, tokens, (size_t)n_tokens * 4, cudaMemcpyHostToDevice, c->stream));
    VB_CUDA(cudaMemsetAsync(c->pf_state, 0, c->d.max_batch * sizeof(SeqState), c->stream));
    // Chunked part: all but the last token, `prefill_chunk` at a time.  Every token of a chunk is a row of one step:
    // the batched kernels read the weights once for the chunk, K/V of all rows are appended before attention and row
    // j attends positions 0..first+j, so the result is the causal one.  (The reference's batched prefill driver:
    // velox_cuda_runner_k2.cu:1614-1704.)  Sharded contexts and the last token take the per-token path below.
    uint32_t done = 0;
    const bool use_tc = c->prefill_gemm && c->d.tp_size <= 1 && n_tokens > c->prefill_gemm_min && c->prefill_rows >= 1 && tc_products_ok(c);
    const uint32_t P = use_tc ? std::min(c->prefill_rows, n_tokens - 1) : c->prefill_chunk;
    if (use_tc || (P >= 2 && P <= 32 && c->d.tp_size <= 1 && n_tokens > P)) {
        const uint32_t cap = use_tc ? c->prefill_rows : P;  // rows the chunk buffers hold
        if ((rc = ensure_chunk_buffers(c, cap)) != VB_OK) return rc;
        if (use_tc && ((rc = ensure_f16_copies(c)) != VB_OK || (rc = ensure_tc_ws(c, cap, false)) != VB_OK)) return rc;
        VB_CUDA(launch(lcfg(c, false), k_fill_chunk_table, dim3(P), dim3(128), 0, c->pfc_table,
                       (const int32_t*)(c->block_table_dev + (size_t)slot * c->max_blocks), c->max_blocks));
        StepIO io{c->pfc_hidden, c->pfc_qkv, c->pfc_q, c->pfc_attn, c->pfc_act, nullptr, c->pfc_table, P, false};
        if (use_tc) { io.tc_ws = tc_ws_aligned(c); io.tc_ws_bytes = c->tc_ws_bytes; io.causal_chunk = true; }
        // the last token always takes the per-token path below (it produces the logits); the tensor-core chunks may be
        // ragged (every row of a chunk is live), the batched-kernel chunks are whole
        while (use_tc ? done + 1 < n_tokens : done + P < n_tokens) {
            const uint32_t n = use_tc ? std::min(P, n_tokens - 1 - done) : P;
            io.B = n; io.first = done;
            VB_CUDA(launch(lcfg(c, false), k_set_chunk_state, dim3((n + 127) / 128), dim3(128), 0, c->pfc_state, (const uint32_t*)c->pf_tokens, done, n, n));
            VB_CUDA(enqueue_step(c, c->pfc_state, false, io));
            done += n;
        }
    }
    // the reference prefills one token per forward pass (velox_cuda_runner.cu:504-506)
    for (uint32_t i = done; i < n_tokens; ++i) {
        VB_CUDA(launch(lcfg(c, false), k_set_state, dim3(1), dim3(32), 0, c->pf_state, (uint32_t)slot, (const uint32_t*)c->pf_tokens, i, 0u, i, 1u,
                       c->slot_blocks[slot] * c->d.kv_block_tokens));
        VB_CUDA(enqueue_step(c, c->pf_state, i + 1 == n_tokens, decode_io(c)));
    }
    // hand the slot over to the decode state: first generated token at position n_tokens
    VB_CUDA(cudaMemcpyAsync(c->state + slot, c->pf_state + slot, sizeof(SeqState), cudaMemcpyDeviceToDevice, c->stream));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    c->pos_hi[slot] = n_tokens;
    c->maybe_active[slot] = 1;  // (a prompt that fills the reservation leaves the slot inactive on the device)
    return VB_OK;
}

// Steps that could carry a possibly-active slot past its KV reservation are refused on the host; on the device
// the sampler deactivates a slot whose next position would leave it, so no kernel ever writes outside.
static int32_t check_reservations(vb_ctx* c, uint32_t n_steps, const char* who) {
    for (uint32_t s = 0; s < c->d.max_batch; ++s) {
        if (!c->maybe_active[s]) continue;
        const uint64_t limit = (uint64_t)c->slot_blocks[s] * c->d.kv_block_tokens;
        if ((uint64_t)c->pos_hi[s] + n_steps > limit) {
            set_error("%s: %u step(s) would take slot %u from position %u past its KV reservation of %llu tokens "
                      "(reserve more with vb_seq_reserve, or release the slot)", who, n_steps, s, c->pos_hi[s], (unsigned long long)limit);
            return VB_ERR_STATE;
        }
    }
    return VB_OK;
}
static void advance_bounds(vb_ctx* c, uint32_t n_steps) {
    for (uint32_t s = 0; s < c->d.max_batch; ++s)
        if (c->maybe_active[s]) c->pos_hi[s] += n_steps;
}

int32_t vb_decode_step(vb_ctx* c) {
    int32_t rc = check_ready(c, "vb_decode_step");
    if (rc != VB_OK) return rc;
    if ((rc = check_reservations(c, 1, "vb_decode_step")) != VB_OK) return rc;
    VB_CUDA(cudaSetDevice(c->device));
    if ((rc = prepare_decode_gemm(c)) != VB_OK) return rc;
    VB_CUDA(enqueue_step(c, c->state, true, decode_io(c)));
    advance_bounds(c, 1);
    return VB_OK;
}

int32_t vb_decode_graph_build(vb_ctx* c) {
    int32_t rc = check_ready(c, "vb_decode_graph_build");
    if (rc != VB_OK) return rc;
    VB_CUDA(cudaSetDevice(c->device));
    if ((rc = prepare_decode_gemm(c)) != VB_OK) return rc;
    if (c->graph_exec) { cudaGraphExecDestroy(c->graph_exec); c->graph_exec = nullptr; }
    if (c->graph) { cudaGraphDestroy(c->graph); c->graph = nullptr; }
    for (int attempt = 0; attempt < 2; ++attempt) {
        const uint64_t before = c->launches;
        VB_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
        cudaError_t e = enqueue_step(c, c->state, true, decode_io(c));
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
    if ((rc = check_reservations(c, n_steps, "vb_decode_run")) != VB_OK) return rc;
    advance_bounds(c, n_steps);
    VB_CUDA(cudaSetDevice(c->device));
    if (elapsed_ms) VB_CUDA(cudaEventRecord(c->ev0, c->stream));
    for (uint32_t s = 0; s < n_steps; ++s) {
        if (c->graph_exec) {
            VB_CUDA(cudaGraphLaunch(c->graph_exec, c->stream));
            c->launches += c->graph_nodes;
        } else {
            VB_CUDA(enqueue_step(c, c->state, true, decode_io(c)));
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
    // callers have synchronised the stream: the mapped word is read in place
    uint32_t* w = nullptr;
    VB_CUDA(fast_error_word_host(&w));
    const uint32_t v = *reinterpret_cast<volatile uint32_t*>(w);
    if (v != 0) {
        *reinterpret_cast<volatile uint32_t*>(w) = 0;
        // a split-K product that gave up leaves its tile counters between 0 and the split count: start them over
        if (c->tc_ws) cudaMemsetAsync(tc_ws_aligned(c), 0, gemm_tc_workspace_zero_bytes(), c->stream);
        if (c->i8_ws) cudaMemsetAsync((void*)(((uintptr_t)c->i8_ws + 1023) & ~(uintptr_t)1023), 0, gemm_i8_workspace_zero_bytes(), c->stream);
        set_error("a bounded device-side wait expired (code 0x%x): results of the last launches are invalid", v);
        return VB_ERR_TIMEOUT;
    }
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
    // a tensor-parallel rank holds the logits of its own vocabulary rows [rank*vocab/tp, (rank+1)*vocab/tp)
    VB_REQUIRE(n_floats == c->vocab, "vb_read_logits: buffer holds %llu floats, this context has %u logits", (unsigned long long)n_floats, c->vocab);
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    VB_CUDA(cudaMemcpy(out, c->logits + (size_t)slot * c->vocab, (size_t)c->vocab * 4, cudaMemcpyDeviceToHost));
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

int32_t vb_read_state_ex(vb_ctx* c, int32_t slot, uint32_t* token, uint32_t* pos, uint32_t* active, uint32_t* limit) {
    VB_REQUIRE(c != nullptr, "vb_read_state_ex: null context");
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_read_state_ex: slot %d out of range", slot);
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    SeqState s;
    VB_CUDA(cudaMemcpy(&s, c->state + slot, sizeof(s), cudaMemcpyDeviceToHost));
    if (token) *token = s.token;
    if (pos) *pos = s.pos;
    if (active) *active = s.active;
    if (limit) *limit = s.limit;
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

int32_t vb_set_sampling(vb_ctx* c, float temperature, float top_p, uint64_t seed, int32_t mode) {
    VB_REQUIRE(c != nullptr, "vb_set_sampling: null context");
    VB_REQUIRE(mode == 0 || mode == 1, "vb_set_sampling: mode %d (0: runtime rule, 1: emitted C99 rule)", mode);
    VB_REQUIRE(temperature == temperature && top_p == top_p, "vb_set_sampling: NaN parameter");
    const bool on = temperature > 1e-5f && top_p > 0.0f;
    if (on && c->d.tp_size > 1) { set_error("vb_set_sampling: a sharded context holds a slice of the logits; sampling runs unsharded"); return VB_ERR_UNSUPPORTED; }
    VB_CUDA(cudaSetDevice(c->device));
    if (on && !c->sample_probs) {
        int32_t rc = dev_alloc(&c->sample_probs, (uint64_t)c->d.max_batch * c->vocab);
        if (rc != VB_OK) return rc;
    }
    if (c->graph_exec) { cudaGraphExecDestroy(c->graph_exec); c->graph_exec = nullptr; }  // the sampler is part of the captured step
    c->sample_temperature = temperature; c->sample_top_p = top_p; c->sample_seed = seed; c->sample_mode = mode;
    return VB_OK;
}

int32_t vb_set_option(vb_ctx* c, const char* name, int64_t value) {
    VB_REQUIRE(c && name, "vb_set_option: null argument");
    if (c->graph_exec) { cudaGraphExecDestroy(c->graph_exec); c->graph_exec = nullptr; }
    if (!strcmp(name, "gemv_path")) { c->gemv_path = (int)value; return VB_OK; }
    if (!strcmp(name, "pdl")) { c->use_pdl = value != 0; return VB_OK; }
    if (!strcmp(name, "fuse_append")) { c->fuse_append = value != 0; return VB_OK; }
    if (!strcmp(name, "prefill_chunk")) { c->prefill_chunk = (uint32_t)value; return VB_OK; }
    if (!strcmp(name, "prefill_gemm")) { c->prefill_gemm = value != 0; return VB_OK; }
    if (!strcmp(name, "decode_gemm")) {  // the workspace is allocated by the next vb_decode_step / vb_decode_graph_build
        VB_REQUIRE(!value || c->d.tp_size <= 1, "vb_set_option: decode_gemm is not available on a sharded context");
        c->decode_gemm = value != 0;
        c->decode_gemm_auto = false;
        return VB_OK;
    }
    if (!strcmp(name, "decode_gemm_i8")) { gemm_i8_enabled = value != 0; return VB_OK; }
    if (!strcmp(name, "i8_tiles")) { gemm_i8_tiles = value != 0; return VB_OK; }
    if (!strcmp(name, "i8_half_ring")) { gemm_i8_half_ring = value != 0; return VB_OK; }
    if (!strcmp(name, "tc_resident_gb")) { c->tc_resident_gb = (uint32_t)value; return VB_OK; }
    if (!strcmp(name, "prefill_two_per_sm")) { gemm_tc_two_per_sm = value != 0; return VB_OK; }
    if (!strcmp(name, "decode_split_k")) { gemm_tc_split_k = value != 0; return VB_OK; }
    if (!strcmp(name, "prefill_split")) {
        VB_REQUIRE(value >= 0 && value <= 2, "vb_set_option: prefill_split is 0, 1 or 2");
        VB_REQUIRE(!c->f16_tried, "vb_set_option: prefill_split must be set before the first long prefill (the resident copies are made then)");
        gemm_tc_split = (int)value;
        return VB_OK;
    }
    if (!strcmp(name, "prefill_wide")) { gemm_tc_wide = value != 0; return VB_OK; }
    if (!strcmp(name, "prefill_flash")) { c->prefill_flash = value != 0; return VB_OK; }
    if (!strcmp(name, "prefill_gemm_min")) { c->prefill_gemm_min = (uint32_t)value; return VB_OK; }
    if (!strcmp(name, "prefill_rows")) {
        VB_REQUIRE(value >= 1 && value <= 4096, "vb_set_option: prefill_rows must be in [1, 4096]");
        c->prefill_rows = (uint32_t)value;
        return VB_OK;
    }
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
    if (!strcmp(name, "attn_splits")) {
        VB_REQUIRE(value >= 1 && value <= 8, "vb_set_option: attn_splits is 1..8 (a thread-block cluster)");
        c->n_splits = (uint32_t)value;
        return VB_OK;
    }
    if (!strcmp(name, "gemv_ring")) { c->gemv_ring = (uint32_t)value; return VB_OK; }
    if (!strcmp(name, "ring_qkv")) { c->ring_role[0] = (uint32_t)value; return VB_OK; }
    if (!strcmp(name, "ring_o")) { c->ring_role[1] = (uint32_t)value; return VB_OK; }
    if (!strcmp(name, "ring_gu")) { c->ring_role[2] = (uint32_t)value; return VB_OK; }
    if (!strcmp(name, "ring_down")) { c->ring_role[3] = (uint32_t)value; return VB_OK; }
    if (!strcmp(name, "head_ring")) { c->head_ring = (uint32_t)value; return VB_OK; }
    if (!strcmp(name, "tp_p2p")) { c->use_links = value != 0; return VB_OK; }
    if (!strcmp(name, "tp_fused_push")) { c->tp_fused_push = value != 0; return VB_OK; }
    if (!strcmp(name, "tp_fused_reduce")) { c->tp_fused_reduce = value != 0; return VB_OK; }
    if (!strcmp(name, "tp_poll_ms")) {  // limit of one exchange poll (default ~10 s), at a nominal 2 GHz
        VB_REQUIRE(value > 0, "vb_set_option: tp_poll_ms must be positive");
        c->links.poll_clocks = (long long)value * 2000000LL;
        return VB_OK;
    }
    if (!strcmp(name, "tp_p2p_standin")) {
        // Diagnostic: private stand-in regions take the place of the peers', so nobody ever answers and every
        // exchange runs into its poll limit -- how the tests exercise the bounded waits without a second GPU.
        VB_REQUIRE(c->d.tp_size > 1 && c->d.tp_size <= 8 && !c->links_open, "vb_set_option: tp_p2p_standin needs a sharded context without peers");
        VB_CUDA(cudaSetDevice(c->device));
        unsigned char handle[64];
        int32_t rc = vb_tp_p2p_export(c, handle);  // allocates this rank's own region
        if (rc != VB_OK) return rc;
        for (uint32_t r = 0; r < c->d.tp_size; ++r) {
            if (r == c->d.tp_rank) continue;
            void* p = nullptr;
            VB_CUDA(cudaMalloc(&p, c->links.bytes));
            VB_CUDA(cudaMemset(p, 0, c->links.bytes));
            c->links.base[r] = (unsigned char*)p;
        }
        c->links_standin = true;
        c->links_open = true;
        return VB_OK;
    }
    if (!strcmp(name, "gemv_spread")) { imma_spread = value != 0; return VB_OK; }
    if (!strcmp(name, "gemv_pair_ring")) { imma_pair_ring = (int)value; return VB_OK; }
    if (!strcmp(name, "gemv_imma")) { imma_enabled = value != 0; return VB_OK; }
    if (!strcmp(name, "gemv_multirow")) { imma_multirow = value != 0; return VB_OK; }
    if (!strcmp(name, "attn_mma")) { attn_use_mma = value != 0; return VB_OK; }
    if (!strcmp(name, "attn_tcgen05")) { attn_use_tcgen05 = value != 0; return VB_OK; }
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
    VB_REQUIRE(id128 != nullptr, "vb_tp_unique_id: null argument");
    return nccl_unique_id((NcclUniqueId*)id128);
}
int32_t vb_tp_init(vb_ctx* c, const void* id128) {
    VB_REQUIRE(c && id128, "vb_tp_init: null argument");
    VB_REQUIRE(c->d.tp_size > 1, "vb_tp_init: the context was created with tp_size <= 1");
    VB_REQUIRE(c->nccl == nullptr, "vb_tp_init: communicator already initialised");
    VB_CUDA(cudaSetDevice(c->device));
    NcclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    return nccl_comm_init(&c->nccl, (int)c->d.tp_size, &id, (int)c->d.tp_rank);
}


// ---- NVLink peer mappings for the tensor-parallel exchange ---------------------------------------------
int32_t vb_tp_p2p_export(vb_ctx* c, void* handle64) {
    VB_REQUIRE(c && handle64, "vb_tp_p2p_export: null argument");
    VB_REQUIRE(c->d.tp_size > 1 && c->d.tp_size <= 8, "vb_tp_p2p_export: peer exchange serves 2..8 ranks (tp_size=%u)", c->d.tp_size);
    VB_CUDA(cudaSetDevice(c->device));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (!c->links.base[c->d.tp_rank]) {
        tp_links_layout(&c->links, c->d.tp_rank, c->d.tp_size, c->d.max_batch * c->d.d_model, c->d.max_batch);
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, c->links.bytes);
        if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc(peer region)", __FILE__, __LINE__); return VB_ERR_OOM; }
        VB_CUDA(cudaMemset(p, 0, c->links.bytes));
        VB_CUDA(cudaDeviceSynchronize());
        c->links.base[c->d.tp_rank] = (unsigned char*)p;
    }
    cudaIpcMemHandle_t h;
    VB_CUDA(cudaIpcGetMemHandle(&h, c->links.base[c->d.tp_rank]));
    memcpy(handle64, &h, 64);
    return VB_OK;
}

int32_t vb_tp_p2p_open(vb_ctx* c, const void* handles, uint32_t n_handles) {
    VB_REQUIRE(c && handles, "vb_tp_p2p_open: null argument");
    VB_REQUIRE(n_handles == c->d.tp_size, "vb_tp_p2p_open: %u handles for tp_size=%u", n_handles, c->d.tp_size);
    VB_REQUIRE(c->links.base[c->d.tp_rank] != nullptr, "vb_tp_p2p_open: call vb_tp_p2p_export first");
    VB_REQUIRE(!c->links_open, "vb_tp_p2p_open: already open");
    VB_CUDA(cudaSetDevice(c->device));
    for (uint32_t r = 0; r < c->d.tp_size; ++r) {
        if (r == c->d.tp_rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const unsigned char*)handles + 64 * (size_t)r, 64);
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            set_error("vb_tp_p2p_open: cannot map rank %u's region (%s); use the NCCL exchange (vb_tp_init)", r, cudaGetErrorString(e));
            return VB_ERR_COMM;
        }
        c->links.base[r] = (unsigned char*)p;
    }
    if (c->graph_exec) { cudaGraphExecDestroy(c->graph_exec); c->graph_exec = nullptr; }
    c->links_open = true;
    return VB_OK;
}


int32_t vb_tp_p2p_close(vb_ctx* c) {
    VB_REQUIRE(c != nullptr, "vb_tp_p2p_close: null context");
    VB_CUDA(cudaSetDevice(c->device));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    if (c->graph_exec) { cudaGraphExecDestroy(c->graph_exec); c->graph_exec = nullptr; }
    for (uint32_t r = 0; r < 8; ++r)
        if (c->links.base[r] && r != c->links.rank) {
            if (c->links_standin) cudaFree(c->links.base[r]); else cudaIpcCloseMemHandle(c->links.base[r]);
            c->links.base[r] = nullptr;
        }
    c->links_open = false;
    c->links_standin = false;
    return VB_OK;
}

}  // extern "C"
