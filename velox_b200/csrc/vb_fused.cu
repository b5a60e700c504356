// Per-op entry points for the two fused instructions the reference's optimizer leaves in every layer, plus the
// KVWrite and SwiGlu instructions, over caller-owned memory in the reference's own layouts.
//
// Reference: VirInst::FusedNormQkvRopeAttn / FusedOutProjResSwiGluRes (src/ir.rs:232-272), emitted as
// velox_cuda_fused_norm_qkv_rope_attn / velox_cuda_fused_out_res_swiglu_res (src/codegen.rs:1757, :1912) and as
// velox_c99_fused_norm_qkv_rope_attn / velox_c99_fused_out_res_swiglu_res (src/runners/tinystories_smollm.c:277-344);
// KVWrite src/ir.rs:83, SwiGlu src/ir.rs:158.  The reference's single-block Phase-I kernels do each instruction in
// one launch of one block; here an instruction is a short sequence of the library's kernels (row-parallel
// matrix-vector products with the norm / residual / SiLU fused in, split-K attention), which is what a
// `one call per VirInst` code generator needs.  Nothing here allocates or synchronises; with `step_dev` the position
// is read on the device, so a captured graph of these calls replays at any position.
#include "vb_ctx.cuh"

namespace vb {

namespace {

// the reference's frequency: 1 / powf(theta, 2j/D), evaluated in double and rounded once (the host's correctly
// rounded powf; the device powf can be 2 ulp off)
__device__ __forceinline__ float inv_freq(float theta, uint32_t j, uint32_t head_dim) {
    const float expo = (float)(2 * j) / (float)head_dim;
    return 1.0f / (float)pow((double)theta, (double)expo);
}

__global__ void k_make_state(SeqState* st, const uint32_t* step_dev, uint32_t step, uint32_t max_seq) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const uint32_t s = step_dev ? *step_dev : step;
        st->token = 0;
        st->pos = s < max_seq ? s : max_seq - 1;  // safe_step of the reference (tinystories_smollm.c:298)
        st->active = 1;
        st->limit = 0;
    }
}

// raw projections [(Hq+2Hkv)*D] -> q (bias, RoPE) and the cache rows of this position (K: bias + RoPE, V: bias), fp32
__global__ void k_bias_rope_kv_write_f32(float* __restrict__ q_out, float* __restrict__ k_layer, float* __restrict__ v_layer,
                                         const float* __restrict__ qkv, const SeqState* __restrict__ st, const float* __restrict__ bq,
                                         const float* __restrict__ bk, const float* __restrict__ bv, uint32_t Hq, uint32_t Hkv, uint32_t D,
                                         float theta) {
    const uint32_t pos = st->pos, half = D / 2;
    const uint32_t n_rot = (Hq + Hkv) * half, n_v = Hkv * D;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_rot) {
        const uint32_t h = i / half, j = i % half;
        const float angle = (float)pos * inv_freq(theta, j, D);
        float s, c;
        sincosf(angle, &s, &c);
        float x1 = qkv[(size_t)h * D + j], x2 = qkv[(size_t)h * D + j + half];
        if (h < Hq) {
            if (bq) { x1 += bq[h * D + j]; x2 += bq[h * D + j + half]; }
            q_out[(size_t)h * D + j] = x1 * c - x2 * s;
            q_out[(size_t)h * D + j + half] = x2 * c + x1 * s;
        } else {
            const uint32_t kh = h - Hq;
            if (bk) { x1 += bk[kh * D + j]; x2 += bk[kh * D + j + half]; }
            float* kd = k_layer + (size_t)pos * Hkv * D + (size_t)kh * D;
            kd[j] = x1 * c - x2 * s;
            kd[j + half] = x2 * c + x1 * s;
        }
    } else if (i < n_rot + n_v) {
        const uint32_t e = i - n_rot;
        float v = qkv[(size_t)(Hq + Hkv) * D + e];
        if (bv) v += bv[e];
        v_layer[(size_t)pos * Hkv * D + e] = v;
    }
}

__global__ void k_kv_write_f32(float* __restrict__ k_layer, float* __restrict__ v_layer, const float* __restrict__ k,
                               const float* __restrict__ v, const uint32_t* step_dev, uint32_t step, uint32_t kv_dim, uint32_t max_seq) {
    uint32_t s = step_dev ? *step_dev : step;
    if (s >= max_seq) s = max_seq - 1;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < kv_dim) {
        k_layer[(size_t)s * kv_dim + i] = k[i];
        v_layer[(size_t)s * kv_dim + i] = v[i];
    }
}

bool weight_ok(const vb_weight* w, uint32_t in_dim) {
    return w && w->data && w->fmt >= VB_FMT_F32 && w->fmt <= VB_FMT_I8PC && fmt_shape_ok(w->fmt, in_dim) && in_dim % 8 == 0 &&
           (wmat_scale_bytes(w->fmt, 1, in_dim) == 0 || w->scales);
}
WMat wmat(const vb_weight* w, uint32_t rows, uint32_t cols) {
    WMat m;
    m.data = w->data; m.scales = w->scales; m.fmt = w->fmt; m.rows = rows; m.cols = cols;
    return m;
}

uint64_t align16(uint64_t v) { return (v + 15) & ~15ULL; }

}  // namespace

}  // namespace vb

using namespace vb;

extern "C" {

uint64_t vb_op_fused_scratch_bytes(uint32_t d_model, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t ffn_dim, uint32_t max_seq) {
    const uint64_t qkv = (uint64_t)(n_q + 2 * n_kv) * head_dim, q = (uint64_t)n_q * head_dim;
    const uint64_t attn = attn_scratch_floats(n_q ? n_q : 1, head_dim ? head_dim : 1, 1, attn_pick_splits(max_seq ? max_seq : 1));
    const uint64_t a = 256 + align16(qkv * 4) + align16(q * 4) + align16(attn * 4);
    const uint64_t b = align16((uint64_t)ffn_dim * 4);
    (void)d_model;
    return (a > b ? a : b) + 256;
}

int32_t vb_op_fused_norm_qkv_rope_attn(float* dst_attn, const float* input_hidden, const float* w_norm, const vb_weight* w_q,
                                       const vb_weight* w_k, const vb_weight* w_v, const float* b_q, const float* b_k, const float* b_v,
                                       float* k_layer, float* v_layer, uint32_t max_seq, uint32_t step, const uint32_t* step_dev,
                                       uint32_t d_model, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, float eps, float theta,
                                       void* scratch, uint64_t scratch_bytes, void* stream) {
    VB_REQUIRE(dst_attn && input_hidden && w_norm && k_layer && v_layer && scratch, "vb_op_fused_norm_qkv_rope_attn: null pointer");
    VB_REQUIRE(weight_ok(w_q, d_model) && weight_ok(w_k, d_model) && weight_ok(w_v, d_model), "vb_op_fused_norm_qkv_rope_attn: bad weight descriptor for d_model=%u", d_model);
    VB_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "vb_op_fused_norm_qkv_rope_attn: n_q=%u not a multiple of n_kv=%u", n_q, n_kv);
    VB_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256, "vb_op_fused_norm_qkv_rope_attn: head_dim=%u", head_dim);
    VB_REQUIRE(max_seq > 0 && (step_dev || step < max_seq), "vb_op_fused_norm_qkv_rope_attn: step %u outside the cache of %u rows", step, max_seq);
    VB_REQUIRE((size_t)d_model * 4 <= 200 * 1024, "vb_op_fused_norm_qkv_rope_attn: d_model=%u exceeds the staging limit", d_model);
    VB_REQUIRE(((uintptr_t)k_layer & 15) == 0 && ((uintptr_t)v_layer & 15) == 0 && ((uintptr_t)scratch & 15) == 0, "vb_op_fused_norm_qkv_rope_attn: caches and scratch must be 16-byte aligned");
    VB_REQUIRE(scratch_bytes >= vb_op_fused_scratch_bytes(d_model, n_q, n_kv, head_dim, 0, max_seq), "vb_op_fused_norm_qkv_rope_attn: scratch of %llu bytes is too small", (unsigned long long)scratch_bytes);
    const uint32_t qdim = n_q * head_dim, kvdim = n_kv * head_dim;
    unsigned char* p = (unsigned char*)scratch;
    SeqState* st = reinterpret_cast<SeqState*>(p); p += 256;
    float* qkv = reinterpret_cast<float*>(p); p += align16((uint64_t)(qdim + 2 * kvdim) * 4);
    float* q = reinterpret_cast<float*>(p); p += align16((uint64_t)qdim * 4);
    float* attn_scratch = reinterpret_cast<float*>(p);
    LaunchCfg lc;
    lc.stream = (cudaStream_t)stream;
    VB_CUDA(kernels_init());
    VB_CUDA(launch(lc, k_make_state, dim3(1), dim3(32), 0, st, step_dev, step, max_seq));
    // RMSNorm fused into each projection's staging of x
    const vb_weight* ws[3] = {w_q, w_k, w_v};
    const uint32_t rows[3] = {qdim, kvdim, kvdim}, offs[3] = {0, qdim, qdim + kvdim};
    for (int i = 0; i < 3; ++i) {
        GemvArgs g;
        g.x = input_hidden; g.dst = qkv; g.dst_offset = offs[i]; g.dst_stride = qdim + 2 * kvdim;
        g.norm_w = w_norm; g.norm_fmt = VB_FMT_F32; g.eps = eps;
        g.w = wmat(ws[i], rows[i], d_model);
        VB_CUDA(gemv(lc, g, 0));
    }
    const uint32_t n = (n_q + n_kv) * (head_dim / 2) + kvdim;
    VB_CUDA(launch(lc, k_bias_rope_kv_write_f32, dim3((n + 127) / 128), dim3(128), 0, q, k_layer, v_layer, (const float*)qkv,
                   (const SeqState*)st, b_q, b_k, b_v, n_q, n_kv, head_dim, theta));
    AttnArgs a;
    a.out = dst_attn; a.q = q; a.k = k_layer; a.v = v_layer; a.kv_fp16 = 0;
    a.state = st; a.Hq = n_q; a.Hkv = n_kv; a.D = head_dim; a.batch = 1;
    a.max_splits = attn_pick_splits(max_seq);              // fixed by the cache size: the same launch serves every position
    a.tokens_per_split = attn_tokens_per_split(max_seq);
    a.scratch = attn_scratch;
    VB_CUDA(cudaMemsetAsync(attn_scratch, 0, attn_scratch_floats(n_q, head_dim, 1, a.max_splits) * 4, lc.stream));
    VB_CUDA(attention(lc, a));
    return VB_OK;
}

int32_t vb_op_fused_outproj_res_swiglu_res(float* dst_hidden, const float* attn_in, const float* residual_in, const vb_weight* w_out,
                                           const float* w_post_norm, const vb_weight* w_gate, const vb_weight* w_up, const vb_weight* w_down,
                                           uint32_t d_model, uint32_t attn_dim, uint32_t ffn_dim, float eps, void* scratch,
                                           uint64_t scratch_bytes, void* stream) {
    VB_REQUIRE(dst_hidden && attn_in && residual_in && w_post_norm && scratch, "vb_op_fused_outproj_res_swiglu_res: null pointer");
    VB_REQUIRE(weight_ok(w_out, attn_dim) && weight_ok(w_gate, d_model) && weight_ok(w_up, d_model) && weight_ok(w_down, ffn_dim),
               "vb_op_fused_outproj_res_swiglu_res: bad weight descriptor");
    VB_REQUIRE(w_gate->fmt == w_up->fmt, "vb_op_fused_outproj_res_swiglu_res: gate and up must share a format");
    VB_REQUIRE((size_t)ffn_dim * 4 <= 200 * 1024 && (size_t)d_model * 4 <= 200 * 1024 && (size_t)attn_dim * 4 <= 200 * 1024,
               "vb_op_fused_outproj_res_swiglu_res: a width exceeds the staging limit");
    VB_REQUIRE(scratch_bytes >= align16((uint64_t)ffn_dim * 4) && ((uintptr_t)scratch & 15) == 0, "vb_op_fused_outproj_res_swiglu_res: scratch of %llu bytes is too small or unaligned", (unsigned long long)scratch_bytes);
    float* act = (float*)scratch;
    LaunchCfg lc;
    lc.stream = (cudaStream_t)stream;
    VB_CUDA(kernels_init());
    if (dst_hidden != residual_in) VB_CUDA(cudaMemcpyAsync(dst_hidden, residual_in, (size_t)d_model * 4, cudaMemcpyDeviceToDevice, lc.stream));
    GemvArgs o;   // mid = attn . Wo^T + residual
    o.x = attn_in; o.dst = dst_hidden; o.epilogue = EPI_RESIDUAL; o.w = wmat(w_out, d_model, attn_dim);
    VB_CUDA(gemv(lc, o, 0));
    GemvArgs gu;  // act = silu(norm(mid) . Wg^T) * (norm(mid) . Wu^T)
    gu.x = dst_hidden; gu.dst = act; gu.epilogue = EPI_SWIGLU; gu.norm_w = w_post_norm; gu.norm_fmt = VB_FMT_F32; gu.eps = eps;
    gu.w = wmat(w_gate, ffn_dim, d_model); gu.w2 = wmat(w_up, ffn_dim, d_model);
    VB_CUDA(gemv(lc, gu, 0));
    GemvArgs dn;  // hidden = mid + act . Wd^T
    dn.x = act; dn.dst = dst_hidden; dn.epilogue = EPI_RESIDUAL; dn.w = wmat(w_down, d_model, ffn_dim);
    VB_CUDA(gemv(lc, dn, 0));
    return VB_OK;
}

int32_t vb_op_kv_write(float* k_layer, float* v_layer, const float* k, const float* v, uint32_t step, const uint32_t* step_dev,
                       uint32_t kv_dim, uint32_t max_seq, void* stream) {
    VB_REQUIRE(k_layer && v_layer && k && v && kv_dim > 0 && max_seq > 0, "vb_op_kv_write: null pointer or empty row");
    LaunchCfg lc;
    lc.stream = (cudaStream_t)stream;
    VB_CUDA(launch(lc, k_kv_write_f32, dim3((kv_dim + 127) / 128), dim3(128), 0, k_layer, v_layer, k, v, step_dev, step, kv_dim, max_seq));
    return VB_OK;
}

int32_t vb_op_swiglu(float* dst, const float* input, const vb_weight* w_gate, const vb_weight* w_up, const vb_weight* w_down,
                     uint32_t d_model, uint32_t ffn_dim, void* scratch, uint64_t scratch_bytes, void* stream) {
    VB_REQUIRE(dst && input && scratch, "vb_op_swiglu: null pointer");
    VB_REQUIRE(weight_ok(w_gate, d_model) && weight_ok(w_up, d_model) && weight_ok(w_down, ffn_dim) && w_gate->fmt == w_up->fmt, "vb_op_swiglu: bad weight descriptor");
    VB_REQUIRE((size_t)ffn_dim * 4 <= 200 * 1024 && (size_t)d_model * 4 <= 200 * 1024, "vb_op_swiglu: a width exceeds the staging limit");
    VB_REQUIRE(scratch_bytes >= align16((uint64_t)ffn_dim * 4) && ((uintptr_t)scratch & 15) == 0, "vb_op_swiglu: scratch too small or unaligned");
    float* act = (float*)scratch;
    LaunchCfg lc;
    lc.stream = (cudaStream_t)stream;
    VB_CUDA(kernels_init());
    GemvArgs gu;
    gu.x = input; gu.dst = act; gu.epilogue = EPI_SWIGLU;
    gu.w = wmat(w_gate, ffn_dim, d_model); gu.w2 = wmat(w_up, ffn_dim, d_model);
    VB_CUDA(gemv(lc, gu, 0));
    GemvArgs dn;
    dn.x = act; dn.dst = dst; dn.w = wmat(w_down, d_model, ffn_dim);
    VB_CUDA(gemv(lc, dn, 0));
    return VB_OK;
}

}  // extern "C"
