// Multi-head latent attention (MLA) decode over a compressed latent KV cache: the weight-absorbed form in which
// keys and values are never decompressed.
//
// Model: the DeepSeek-V3-style stack of the reference (examples/deepseek_v3_mla.vlx:18-45, decode scope :117-150):
// per token the cache holds one latent row [c_kv (kv_lora_rank = 512) | k_rope (64)], shared by all heads; head h
// attends with q_h = [q_nope_h . W_uk_h (512) | q_rope_h (64)]:
//     s_h(t) = scale * q_h . latent(t),   p_h = softmax_t(s_h),   ctx_h = sum_t p_h(t) * c_kv(t)        (512 per head)
// The reference's runtime math for this instruction is the single-head block of src/runtime.rs:944-1044 (one head, no
// rope part, K = V = latent; served by vb_op_mla_absorbed); this kernel is the 128-head form its model file declares.
//
// Shape of the work: for one sequence all heads share every latent row, so the products are S[heads x tokens] =
// Q[heads x 576] . L^T and O[heads x 512] = P . L[:, :512] -- ~240 flop per cache byte, the one tensor-pipe-bound
// decode kernel.  One block = 64 heads of one sequence over one slice of up to `split_tokens` cache rows; 16 warps =
// 4 groups of 16 heads x 4 quarters.  Per 32-row tile (cp.async, double buffered, zero-filled past the context):
// each warp computes its group's scores for its 8 rows (bf16 mma.sync m16n8k16, fp32 accumulate), the four quarters
// exchange row maxima and the bf16 probabilities through shared memory, then each warp accumulates its 128 of the 512
// output dimensions.  Slices are merged by a second kernel (flash-decoding).  Context lengths are read on the device.
#include <cuda_bf16.h>

#include "vb_internal.cuh"
#include "vb_kernels.cuh"

namespace vb {

bool mla_use_tc = true;  // vb_op_mla_set_path(0): the mma.sync kernel of this file instead of the tcgen05 one

namespace {

constexpr int ML_LAT = 576;            // latent row: 512 + 64
constexpr int ML_V = 512;              // value part of the row
constexpr int ML_HEADS_PER_BLOCK = 64;
constexpr int ML_TILE = 32;            // cache rows per tile
constexpr int ML_THREADS = 512;
constexpr int ML_ROW = ML_LAT * 2 + 16;  // bytes per staged row: 16 bytes of padding keep ldmatrix rows on different banks
constexpr int ML_PROW = ML_TILE * 2 + 16;
constexpr size_t ML_SMEM = (size_t)ML_HEADS_PER_BLOCK * ML_ROW + 2 * (size_t)ML_TILE * ML_ROW + 2 * (size_t)ML_HEADS_PER_BLOCK * ML_PROW +
                           2 * 4 * 4 * 16 * 4 * 2;

struct MlaArgs {
    const float* q;              // [B][n_heads][576] fp32
    const __nv_bfloat16* cache;  // [B][cache_stride rows][576] bf16
    const uint32_t* ctx_len;     // [B] rows to attend (device)
    float* partial;              // [B][n_splits][n_heads][512 + 2]: unnormalised output, running max, running sum
    uint32_t n_heads, n_splits, split_tokens;
    uint64_t cache_stride;       // rows between sequences
    float scale;
};

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp16_zfill(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void group_bar(uint32_t id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

__global__ void __launch_bounds__(ML_THREADS, 1) k_mla_decode(MlaArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* q_s = smem;                                          // [64][ML_ROW]
    unsigned char* l_s = q_s + ML_HEADS_PER_BLOCK * ML_ROW;             // [2][32][ML_ROW]
    unsigned char* p_s = l_s + 2 * ML_TILE * ML_ROW;                    // [2][64][ML_PROW]
    float* pmax = reinterpret_cast<float*>(p_s + 2 * ML_HEADS_PER_BLOCK * ML_PROW);  // [2][4 groups][4 quarters][16]
    float* psum = pmax + 2 * 4 * 4 * 16;
    const uint32_t split = blockIdx.x, hb = blockIdx.y, b = blockIdx.z;
    const uint32_t ctx = a.ctx_len[b];
    const uint32_t t_lo = split * a.split_tokens;
    if (t_lo >= ctx) return;  // nothing in this slice (the merge kernel knows)
    const uint32_t t_hi = min(ctx, t_lo + a.split_tokens), n_tiles = (t_hi - t_lo + ML_TILE - 1) / ML_TILE;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, hg = warp >> 2, qt = warp & 3, g = lane >> 2, t = lane & 3;
    const __nv_bfloat16* seq = a.cache + (size_t)b * a.cache_stride * ML_LAT;
    const uint32_t l_base = (uint32_t)__cvta_generic_to_shared(l_s), q_base = (uint32_t)__cvta_generic_to_shared(q_s),
                   p_base = (uint32_t)__cvta_generic_to_shared(p_s);

    auto load_tile = [&](uint32_t tile, uint32_t buf) {
        const uint32_t row0 = t_lo + tile * ML_TILE;
        for (uint32_t i = tid; i < ML_TILE * (ML_LAT / 8); i += ML_THREADS) {
            const uint32_t r = i / (ML_LAT / 8), c = i % (ML_LAT / 8);
            const bool valid = row0 + r < t_hi;
            cp16_zfill(l_base + (buf * ML_TILE + r) * ML_ROW + c * 16, seq + (size_t)(valid ? row0 + r : t_lo) * ML_LAT + c * 8, valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_tile(0, 0);
    // this block's 64 query rows, rounded to bf16 once
    const float* qb = a.q + ((size_t)b * a.n_heads + (size_t)hb * ML_HEADS_PER_BLOCK) * ML_LAT;
    for (uint32_t i = tid; i < ML_HEADS_PER_BLOCK * (ML_LAT / 2); i += ML_THREADS) {
        const uint32_t r = i / (ML_LAT / 2), c = i % (ML_LAT / 2);
        const bool live = hb * ML_HEADS_PER_BLOCK + r < a.n_heads;
        const float2 v = live ? *reinterpret_cast<const float2*>(qb + (size_t)r * ML_LAT + 2 * c) : make_float2(0.f, 0.f);
        *reinterpret_cast<__nv_bfloat162*>(q_s + r * ML_ROW + c * 4) = __floats2bfloat162_rn(v.x, v.y);
    }

    float o[16][4];  // this warp's 16 heads x 128 output dimensions: 16 n-tiles of 8
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};  // rows g and g+8 of the head group
    const uint32_t q_lane = q_base + (hg * 16 + (lane & 15)) * ML_ROW + (lane >> 4) * 16;             // A fragments of Q
    const uint32_t k_lane_off = ((qt * 8 + (lane & 7)) * ML_ROW) + ((lane >> 3) & 3) * 16;             // B fragments of L^T: two k-steps per load
    const uint32_t v_lane_off = ((lane & 15) * ML_ROW) + (qt * 128 + (lane >> 4) * 8) * 2;            // B fragments of L[:, :512], transposed load
    const float sc = a.scale;

    for (uint32_t tile = 0; tile < n_tiles; ++tile) {
        const uint32_t buf = tile & 1;
        if (tile + 1 < n_tiles) { load_tile(tile + 1, buf ^ 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // the tile (and, the first time, Q) is in shared memory for every warp
        // ---- scores of this warp's 8 rows for its 16 heads: K = 576 in 36 steps ------------------------------------
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint32_t kb = l_base + buf * ML_TILE * ML_ROW + k_lane_off;
#pragma unroll 6
        for (int ks = 0; ks < ML_LAT / 32; ++ks) {
            uint32_t b0, b1, b2, b3, a0, a1, a2, a3;
            ldsm_x4(b0, b1, b2, b3, kb + ks * 64);
            ldsm_x4(a0, a1, a2, a3, q_lane + ks * 64);
            mma_bf16(s, a0, a1, a2, a3, b0, b1);
            ldsm_x4(a0, a1, a2, a3, q_lane + ks * 64 + 32);
            mma_bf16(s, a0, a1, a2, a3, b2, b3);
        }
        // rows past the slice end are masked; lane holds (row g | g+8) x (tokens 2t, 2t+1) of this quarter
        const uint32_t tok0 = t_lo + tile * ML_TILE + qt * 8 + 2 * t;
        const float s0 = tok0 < t_hi ? s[0] * sc : -INFINITY, s1 = tok0 + 1 < t_hi ? s[1] * sc : -INFINITY;
        const float s2 = tok0 < t_hi ? s[2] * sc : -INFINITY, s3 = tok0 + 1 < t_hi ? s[3] * sc : -INFINITY;
        float mx0 = fmaxf(s0, s1), mx1 = fmaxf(s2, s3);
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 2));
        float* pm = pmax + ((buf * 4 + hg) * 4) * 16;
        float* ps = psum + ((buf * 4 + hg) * 4) * 16;
        if (t == 0) { pm[qt * 16 + g] = mx0; pm[qt * 16 + g + 8] = mx1; }
        group_bar(1 + hg);
        const float tm0 = fmaxf(fmaxf(pm[g], pm[16 + g]), fmaxf(pm[32 + g], pm[48 + g]));
        const float tm1 = fmaxf(fmaxf(pm[g + 8], pm[16 + g + 8]), fmaxf(pm[32 + g + 8], pm[48 + g + 8]));
        const float mn0 = fmaxf(m_run[0], tm0), mn1 = fmaxf(m_run[1], tm1);  // finite: every tile has at least one live row
        const float p0 = __expf(s0 - mn0), p1 = __expf(s1 - mn0), p2 = __expf(s2 - mn1), p3 = __expf(s3 - mn1);
        // probabilities rounded to bf16 once; the row sums add the rounded values, so that numerator and denominator agree
        const __nv_bfloat162 pa = __floats2bfloat162_rn(p0, p1), pb = __floats2bfloat162_rn(p2, p3);
        unsigned char* prow = p_s + (buf * ML_HEADS_PER_BLOCK + hg * 16) * ML_PROW;
        *reinterpret_cast<__nv_bfloat162*>(prow + g * ML_PROW + (qt * 8 + 2 * t) * 2) = pa;
        *reinterpret_cast<__nv_bfloat162*>(prow + (g + 8) * ML_PROW + (qt * 8 + 2 * t) * 2) = pb;
        float sum0 = __bfloat162float(pa.x) + __bfloat162float(pa.y), sum1 = __bfloat162float(pb.x) + __bfloat162float(pb.y);
        sum0 += __shfl_xor_sync(0xFFFFFFFFu, sum0, 1); sum0 += __shfl_xor_sync(0xFFFFFFFFu, sum0, 2);
        sum1 += __shfl_xor_sync(0xFFFFFFFFu, sum1, 1); sum1 += __shfl_xor_sync(0xFFFFFFFFu, sum1, 2);
        if (t == 0) { ps[qt * 16 + g] = sum0; ps[qt * 16 + g + 8] = sum1; }
        group_bar(1 + hg);
        const float al0 = __expf(m_run[0] - mn0), al1 = __expf(m_run[1] - mn1);
        l_run[0] = l_run[0] * al0 + ((ps[g] + ps[16 + g]) + (ps[32 + g] + ps[48 + g]));
        l_run[1] = l_run[1] * al1 + ((ps[g + 8] + ps[16 + g + 8]) + (ps[32 + g + 8] + ps[48 + g + 8]));
        m_run[0] = mn0; m_run[1] = mn1;
#pragma unroll
        for (int i = 0; i < 16; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
        // ---- O[16 heads x 128 dims] += P[16 x 32] . L[32 rows][this warp's 128 dims] ----------------------------
        const uint32_t pa_addr = p_base + (buf * ML_HEADS_PER_BLOCK + hg * 16 + (lane & 15)) * ML_PROW + (lane >> 4) * 16;
        const uint32_t vb = l_base + buf * ML_TILE * ML_ROW + v_lane_off;
#pragma unroll
        for (int ks = 0; ks < ML_TILE / 16; ++ks) {
            uint32_t a0, a1, a2, a3;
            ldsm_x4(a0, a1, a2, a3, pa_addr + ks * 32);
#pragma unroll
            for (int np = 0; np < 8; ++np) {  // two n-tiles of 8 dimensions per transposed load
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(b0, b1, b2, b3, vb + ks * 16 * ML_ROW + np * 32);
                mma_bf16(o[2 * np], a0, a1, a2, a3, b0, b1);
                mma_bf16(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();  // every warp is done with this tile's buffer before the load after next overwrites it
    }
    // ---- this slice's unnormalised output, running max and sum ------------------------------------------------------
    const uint32_t head0 = hb * ML_HEADS_PER_BLOCK + hg * 16;
    float* out = a.partial + (((size_t)b * a.n_splits + split) * a.n_heads) * (ML_V + 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const uint32_t h = head0 + g + 8 * half;
        if (h >= a.n_heads) continue;
        float* row = out + (size_t)h * (ML_V + 2);
#pragma unroll
        for (int i = 0; i < 16; ++i)
            *reinterpret_cast<float2*>(row + qt * 128 + i * 8 + 2 * t) = make_float2(o[i][2 * half], o[i][2 * half + 1]);
        if (qt == 0 && t == 0) { row[ML_V] = m_run[half]; row[ML_V + 1] = l_run[half]; }
    }
}

// out[b][h][:] = sum over the live slices of partial * exp(m - M) / L; grid (n_heads, B), 128 threads x 4 dimensions
__global__ void __launch_bounds__(128) k_mla_merge(float* __restrict__ out, const float* __restrict__ partial, const uint32_t* __restrict__ ctx_len,
                                                   uint32_t n_heads, uint32_t n_splits, uint32_t split_tokens, const uint32_t* __restrict__ status) {
    const uint32_t h = blockIdx.x, b = blockIdx.y;
    if (status && *status) {
        // a wait in the tensor-core kernel ran out: the partials are not to be trusted, and the caller must see it
        float* o = out + ((size_t)b * n_heads + h) * ML_V + threadIdx.x * 4;
        o[0] = o[1] = o[2] = o[3] = __int_as_float(0x7FC00000);
        return;
    }
    const uint32_t ctx = ctx_len[b];
    const uint32_t live = ctx == 0 ? 0 : min(n_splits, (ctx + split_tokens - 1) / split_tokens);
    const float* base = partial + (((size_t)b * n_splits) * n_heads + h) * (ML_V + 2);
    const size_t stride = (size_t)n_heads * (ML_V + 2);
    float M = -INFINITY;
    for (uint32_t s = 0; s < live; ++s) M = fmaxf(M, base[s * stride + ML_V]);
    float L = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t s = 0; s < live; ++s) {
        const float w = __expf(base[s * stride + ML_V] - M);
        L += base[s * stride + ML_V + 1] * w;
        const float2 v0 = *reinterpret_cast<const float2*>(base + s * stride + threadIdx.x * 4);
        const float2 v1 = *reinterpret_cast<const float2*>(base + s * stride + threadIdx.x * 4 + 2);
        acc.x += v0.x * w; acc.y += v0.y * w; acc.z += v1.x * w; acc.w += v1.y * w;
    }
    const float inv = live ? 1.0f / L : 0.0f;
    float* o = out + ((size_t)b * n_heads + h) * ML_V + threadIdx.x * 4;
    o[0] = acc.x * inv; o[1] = acc.y * inv; o[2] = acc.z * inv; o[3] = acc.w * inv;
}

// latent rows of the step: cache[b][pos[b]][:] = bf16(row[b][:]); grid B, 288 threads (one bf16 pair each)
__global__ void k_mla_append(__nv_bfloat16* __restrict__ cache, const float* __restrict__ rows, const uint32_t* __restrict__ pos, uint64_t cache_stride) {
    const uint32_t b = blockIdx.x, i = threadIdx.x;
    if (pos[b] >= cache_stride) return;
    const float2 v = *reinterpret_cast<const float2*>(rows + (size_t)b * ML_LAT + 2 * i);
    *reinterpret_cast<__nv_bfloat162*>(cache + ((size_t)b * cache_stride + pos[b]) * ML_LAT + 2 * i) = __floats2bfloat162_rn(v.x, v.y);
}

// Per-head products of the absorbed form: dst[b][h][:n_out] = sum_k src[b][h][k] * W_h[k][n] (or W_h[n][k] when transposed),
// W bf16 [n_heads][rows_per_head][cols]; one block per (head, 16 batch rows), fp32 accumulate.
template <bool W_ROWS_ARE_OUT>
__global__ void __launch_bounds__(256) k_mla_head_product(float* __restrict__ dst, const float* __restrict__ src, const __nv_bfloat16* __restrict__ w,
                                                          uint32_t n_heads, uint32_t n_in, uint32_t n_out, uint32_t batch) {
    extern __shared__ float xs[];  // [16][n_in]
    const uint32_t h = blockIdx.x, b0 = blockIdx.y * 16;
    for (uint32_t i = threadIdx.x; i < 16 * n_in; i += 256) {
        const uint32_t r = i / n_in, k = i % n_in;
        xs[i] = b0 + r < batch ? src[((size_t)(b0 + r) * n_heads + h) * n_in + k] : 0.0f;
    }
    __syncthreads();
    // W_ROWS_ARE_OUT: W_h is [n_out][n_in] (dst = x . W_h^T); else W_h is [n_in][n_out] (dst = x . W_h)
    const __nv_bfloat16* wh = w + (size_t)h * n_in * n_out;
    for (uint32_t n = threadIdx.x; n < n_out; n += 256) {
        float acc[16];
#pragma unroll
        for (int r = 0; r < 16; ++r) acc[r] = 0.0f;
        for (uint32_t k = 0; k < n_in; ++k) {
            const float wv = __bfloat162float(W_ROWS_ARE_OUT ? wh[(size_t)n * n_in + k] : wh[(size_t)k * n_out + n]);
#pragma unroll
            for (int r = 0; r < 16; ++r) acc[r] = fmaf(xs[r * n_in + k], wv, acc[r]);
        }
        for (uint32_t r = 0; r < 16 && b0 + r < batch; ++r) dst[((size_t)(b0 + r) * n_heads + h) * n_out + n] = acc[r];
    }
}

}  // namespace

}  // namespace vb

using namespace vb;

extern "C" {

static uint64_t mla_partial_bytes(uint32_t batch, uint32_t n_heads, uint32_t max_ctx, uint32_t split_tokens) {
    const uint64_t n_splits = ((uint64_t)max_ctx + split_tokens - 1) / split_tokens;
    const uint64_t b = (uint64_t)batch * (n_splits ? n_splits : 1) * n_heads * (ML_V + 2) * 4;
    return (b + 1023) / 1024 * 1024;
}

uint64_t vb_op_mla_decode_scratch_bytes(uint32_t batch, uint32_t n_heads, uint32_t max_ctx, uint32_t split_tokens) {
    if (split_tokens == 0) split_tokens = 1024;
    // the slices' partial outputs, then the tensor-core path's status word and bf16 copy of q
    return mla_partial_bytes(batch, n_heads, max_ctx, split_tokens) + mla_tc_extra_scratch_bytes(batch, n_heads);
}

int32_t vb_op_mla_set_path(int32_t path) {
    VB_REQUIRE(path == 0 || path == 1, "vb_op_mla_set_path: 0 (mma.sync kernel) or 1 (tcgen05 kernel)");
    mla_use_tc = path == 1;
    return VB_OK;
}

int32_t vb_op_mla_decode(float* out, const float* q, const void* latent_cache, const uint32_t* ctx_len, uint32_t batch, uint32_t n_heads,
                         uint32_t max_ctx, uint64_t cache_stride_rows, float scale, uint32_t split_tokens, void* scratch, uint64_t scratch_bytes,
                         void* stream) {
    VB_REQUIRE(out && q && latent_cache && ctx_len && scratch, "vb_op_mla_decode: null pointer");
    VB_REQUIRE(batch > 0 && n_heads > 0 && max_ctx > 0 && cache_stride_rows >= max_ctx, "vb_op_mla_decode: empty problem or cache stride below max_ctx");
    if (split_tokens == 0) split_tokens = 1024;
    VB_REQUIRE(split_tokens % ML_TILE == 0, "vb_op_mla_decode: split_tokens=%u is not a multiple of %d", split_tokens, ML_TILE);
    VB_REQUIRE(((uintptr_t)latent_cache & 15) == 0 && ((uintptr_t)q & 7) == 0 && ((uintptr_t)scratch & 15) == 0, "vb_op_mla_decode: unaligned pointer");
    VB_REQUIRE(scratch_bytes >= vb_op_mla_decode_scratch_bytes(batch, n_heads, max_ctx, split_tokens), "vb_op_mla_decode: scratch of %llu bytes is too small",
               (unsigned long long)scratch_bytes);
    static bool opted = false;
    if (!opted) {
        VB_CUDA(cudaFuncSetAttribute(k_mla_decode, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ML_SMEM));
        opted = true;
    }
    MlaArgs a;
    a.q = q; a.cache = (const __nv_bfloat16*)latent_cache; a.ctx_len = ctx_len; a.partial = (float*)scratch;
    a.n_heads = n_heads; a.split_tokens = split_tokens; a.n_splits = (max_ctx + split_tokens - 1) / split_tokens;
    a.cache_stride = cache_stride_rows; a.scale = scale;
    LaunchCfg lc;
    lc.stream = (cudaStream_t)stream;
    if (mla_use_tc) {
        // tcgen05 path: both products on the 5th-generation tensor cores (vb_mla_tc.cu)
        void* extra = reinterpret_cast<unsigned char*>(scratch) + mla_partial_bytes(batch, n_heads, max_ctx, split_tokens);
        VB_CUDA(mla_decode_tc(lc, q, latent_cache, ctx_len, (float*)scratch, extra, batch, n_heads, a.n_splits, split_tokens, cache_stride_rows, scale));
        VB_CUDA(launch(lc, k_mla_merge, dim3(n_heads, batch), dim3(128), 0, out, (const float*)scratch, ctx_len, n_heads, a.n_splits, split_tokens,
                       (const uint32_t*)extra));
        return VB_OK;
    }
    const dim3 grid(a.n_splits, (n_heads + ML_HEADS_PER_BLOCK - 1) / ML_HEADS_PER_BLOCK, batch);
    VB_CUDA(launch(lc, k_mla_decode, grid, dim3(ML_THREADS), ML_SMEM, a));
    VB_CUDA(launch(lc, k_mla_merge, dim3(n_heads, batch), dim3(128), 0, out, (const float*)scratch, ctx_len, n_heads, a.n_splits, split_tokens,
                   (const uint32_t*)nullptr));
    return VB_OK;
}

int32_t vb_op_mla_latent_append(void* latent_cache, const float* rows, const uint32_t* pos, uint32_t batch, uint64_t cache_stride_rows, void* stream) {
    VB_REQUIRE(latent_cache && rows && pos && batch > 0, "vb_op_mla_latent_append: null pointer or empty batch");
    LaunchCfg lc;
    lc.stream = (cudaStream_t)stream;
    VB_CUDA(launch(lc, k_mla_append, dim3(batch), dim3(ML_LAT / 2), 0, (__nv_bfloat16*)latent_cache, rows, pos, cache_stride_rows));
    return VB_OK;
}

int32_t vb_op_mla_head_product(float* dst, const float* src, const void* w_bf16, uint32_t n_heads, uint32_t n_in, uint32_t n_out, uint32_t batch,
                               int32_t w_rows_are_out, void* stream) {
    VB_REQUIRE(dst && src && w_bf16 && n_heads > 0 && n_in > 0 && n_out > 0, "vb_op_mla_head_product: null pointer or empty shape");
    VB_REQUIRE((uint64_t)n_in * 16 * 4 <= 48 * 1024, "vb_op_mla_head_product: n_in=%u exceeds the staging limit", n_in);
    if (batch == 0) return VB_OK;
    LaunchCfg lc;
    lc.stream = (cudaStream_t)stream;
    const dim3 grid(n_heads, (batch + 15) / 16);
    const size_t smem = (size_t)16 * n_in * 4;
    if (w_rows_are_out) VB_CUDA(launch(lc, k_mla_head_product<true>, grid, dim3(256), smem, dst, src, (const __nv_bfloat16*)w_bf16, n_heads, n_in, n_out, batch));
    else VB_CUDA(launch(lc, k_mla_head_product<false>, grid, dim3(256), smem, dst, src, (const __nv_bfloat16*)w_bf16, n_heads, n_in, n_out, batch));
    return VB_OK;
}

}  // extern "C"
