// The reference's absorbed-MLA block (src/runtime.rs:944-1044; emitted twin
// src/runners/tinystories_smollm.cu:945-1053): RMSNorm -> latent slot = nx.W_dkv^T written into the pool at
// `step` -> q_abs = nx.W_absq^T -> softmax over the latent history with K = V = latent (one head, no RoPE
// part, scale 1/sqrt(128) once latent >= 128) -> x + ctx.W_abso^T.  Built from the library's matrix-vector
// and split-K attention kernels instead of the reference's single 256-thread block.
#include "vb_internal.cuh"
#include "vb_kernels.cuh"

namespace vb {

cudaError_t attention_ex(const LaunchCfg& lc, const AttnArgs& a, float scale, size_t kv_batch_stride);

// scratch: q_abs [latent] | ctx [latent] | attention partials
uint64_t mla_scratch_floats(uint32_t hidden, uint32_t latent) {
    (void)hidden;
    return 2ULL * latent + attn_scratch_floats(1, latent, 1, 64) + 64;
}

cudaError_t mla_absorbed(const LaunchCfg& lc, float* dst, const float* x, const float* w_norm, const float* w_dkv,
                         const float* w_absq, const float* w_abso, float* pool, uint32_t step, uint32_t hidden,
                         uint32_t latent, uint32_t max_seq, float eps, float* scratch) {
    const uint32_t safe_step = (step < max_seq) ? step : (max_seq ? max_seq - 1 : 0);
    float* q_abs = scratch;
    float* ctx = scratch + latent;
    float* part = scratch + 2 * (size_t)latent;
    cudaError_t e;
    GemvArgs g;
    g.x = x; g.norm_w = w_norm; g.norm_fmt = VB_FMT_F32; g.eps = eps; g.batch = 1;
    g.w.fmt = VB_FMT_F32; g.w.rows = latent; g.w.cols = hidden;
    g.w.data = w_dkv; g.dst = pool + (size_t)safe_step * latent;
    if ((e = gemv(lc, g, 0)) != cudaSuccess) return e;
    g.w.data = w_absq; g.dst = q_abs;
    if ((e = gemv(lc, g, 0)) != cudaSuccess) return e;
    AttnArgs a;
    a.out = ctx; a.q = q_abs; a.k = pool; a.v = pool; a.kv_fp16 = 0; a.pos = safe_step;
    a.Hq = 1; a.Hkv = 1; a.D = latent; a.batch = 1; a.block_tokens = 16;
    a.max_splits = attn_pick_splits(safe_step + 1);
    a.tokens_per_split = attn_tokens_per_split(safe_step + 1);
    a.scratch = part;
    const float scale = (latent >= 128) ? (1.0f / sqrtf(128.0f)) : (1.0f / sqrtf((float)latent));
    if ((e = attention_ex(lc, a, scale, 0)) != cudaSuccess) return e;
    if (dst != x) {
        if ((e = cudaMemcpyAsync(dst, x, (size_t)hidden * 4, cudaMemcpyDeviceToDevice, lc.stream)) != cudaSuccess) return e;
    }
    GemvArgs o;
    o.x = ctx; o.batch = 1; o.dst = dst; o.epilogue = EPI_RESIDUAL;
    o.w.fmt = VB_FMT_F32; o.w.rows = hidden; o.w.cols = latent; o.w.data = w_abso;
    return gemv(lc, o, 0);
}

}  // namespace vb

using namespace vb;

extern "C" int32_t vb_op_mla_absorbed(float* dst, const float* x, const float* w_norm, const float* w_dkv,
                                      const float* w_absq, const float* w_abso, float* latent_pool, uint32_t step,
                                      uint32_t hidden, uint32_t latent, uint32_t max_seq, float eps, void* scratch,
                                      uint64_t scratch_bytes, void* stream) {
    VB_REQUIRE(dst && x && w_norm && w_dkv && w_absq && w_abso && latent_pool && scratch, "vb_op_mla_absorbed: null pointer");
    VB_REQUIRE(latent == 32 || latent == 64 || latent == 128 || latent == 256 || latent == 512,
               "vb_op_mla_absorbed: latent=%u (supported: 32,64,128,256,512)", latent);
    VB_REQUIRE(hidden % 8 == 0 && hidden > 0 && max_seq > 0, "vb_op_mla_absorbed: hidden must be a positive multiple of 8");
    VB_REQUIRE(scratch_bytes >= mla_scratch_floats(hidden, latent) * 4, "vb_op_mla_absorbed: scratch too small (%llu bytes needed)",
               (unsigned long long)(mla_scratch_floats(hidden, latent) * 4));
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    VB_CUDA(kernels_init());
    VB_CUDA(mla_absorbed(lc, dst, x, w_norm, w_dkv, w_absq, w_abso, latent_pool, step, hidden, latent, max_seq, eps, (float*)scratch));
    return VB_OK;
}
