// Causal attention of a prefill chunk over the paged fp16 cache: the rows of the chunk are n consecutive positions
// first..first+n-1 of ONE sequence, whose K/V (this chunk's included) are already in the cache.  Same arithmetic
// as the per-token kernel of vb_attn.cu with fp16 caches (the reference: src/runtime.rs:772-831, one query at a
// time; its batched driver: src/runners/velox_cuda_runner_k2.cu:1614-1704): scores (q.k)/sqrt(D), softmax over
// positions <= the row's own, weighted sum of V; q and the softmax weights are rounded to fp16 for the two
// products, maxima, sums and accumulators are fp32.
//
// One block = 64 consecutive rows of one query head (4 warps x 16 rows); the K/V rows of the head's KV group are
// staged 64 positions at a time with cp.async (double buffered, rows padded by 16 bytes against bank conflicts),
// both products run on mma.sync.m16n8k16 with ldmatrix / ldmatrix.trans fragments, the running maximum and sum
// are kept per row (online softmax).  KV tiles beyond a block's last row are never read.
#include "vb_kernels.cuh"

namespace vb {
namespace {

constexpr int QROWS = 64;   // query rows per block
constexpr int KTILE = 64;   // cache positions per staged tile

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int D>
__global__ void __launch_bounds__(128)
k_attn_prefill(float* __restrict__ out, const float* __restrict__ q, const __half* __restrict__ kv_layer,
               const int32_t* __restrict__ table_row, uint32_t first, uint32_t n, uint32_t Hq, uint32_t Hkv, uint32_t block_tokens,
               float scale) {
    constexpr int ROWB = (D + 8) * 2;            // bytes per staged row
    constexpr int TILEB = KTILE * ROWB;          // one K or V tile
    constexpr int CHUNKS = D / 8;                // 16-byte pieces per row
    extern __shared__ __align__(16) unsigned char smem[];  // [2 buffers][K tile | V tile]
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t h = blockIdx.y, kvh = h / (Hq / Hkv);
    const uint32_t r0 = blockIdx.x * QROWS;
    const uint32_t rows_here = min((uint32_t)QROWS, n - r0);
    const uint32_t kv_len = first + r0 + rows_here;                 // positions 0..kv_len-1 are visible to the last row
    const uint32_t n_tiles = (kv_len + KTILE - 1) / KTILE;

    pdl_wait();
    pdl_launch_dependents();

    auto stage = [&](uint32_t tile, uint32_t buf) {
        const uint32_t t0 = tile * KTILE;
        const uint32_t dstK = sbase + buf * 2 * TILEB, dstV = dstK + TILEB;
        for (uint32_t i = threadIdx.x; i < KTILE * CHUNKS; i += 128) {
            const uint32_t tok = i / CHUNKS, c = i % CHUNKS;
            const uint32_t pos = t0 + tok;
            const bool valid = pos < kv_len;
            const uint32_t p = valid ? pos : 0u;
            const int32_t blk = table_row[p / block_tokens];
            const __half* kp = kv_layer + ((((size_t)blk * 2 + 0) * Hkv + kvh) * block_tokens + p % block_tokens) * D + c * 8;
            const __half* vp = kp + (size_t)Hkv * block_tokens * D;
            cp_async16(dstK + tok * ROWB + c * 16, kp, valid);
            cp_async16(dstV + tok * ROWB + c * 16, vp, valid);
        }
        cp_async_commit();
    };

    stage(0, 0);

    // this warp's 16 rows of q as A fragments, pre-scaled by 1/sqrt(D)
    uint32_t qa[D / 16][4];
    {
        const uint32_t ra = r0 + warp * 16 + g, rb = ra + 8;
        const float* qa_row = q + ((size_t)min(ra, n - 1) * Hq + h) * D;
        const float* qb_row = q + ((size_t)min(rb, n - 1) * Hq + h) * D;
#pragma unroll
        for (int kt = 0; kt < D / 16; ++kt) {
            const float2 a0 = *reinterpret_cast<const float2*>(qa_row + kt * 16 + 2 * t);
            const float2 a1 = *reinterpret_cast<const float2*>(qb_row + kt * 16 + 2 * t);
            const float2 a2 = *reinterpret_cast<const float2*>(qa_row + kt * 16 + 8 + 2 * t);
            const float2 a3 = *reinterpret_cast<const float2*>(qb_row + kt * 16 + 8 + 2 * t);
            qa[kt][0] = pack_h2(a0.x * scale, a0.y * scale);
            qa[kt][1] = pack_h2(a1.x * scale, a1.y * scale);
            qa[kt][2] = pack_h2(a2.x * scale, a2.y * scale);
            qa[kt][3] = pack_h2(a3.x * scale, a3.y * scale);
        }
    }
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;   // rows g and g+8 of this warp
    const uint32_t pos_a = first + r0 + warp * 16 + g, pos_b = pos_a + 8;
    constexpr float LOG2E = 1.4426950408889634f;

    for (uint32_t tile = 0; tile < n_tiles; ++tile) {
        const uint32_t buf = tile & 1;
        if (tile + 1 < n_tiles) { stage(tile + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        const uint32_t sK = sbase + buf * 2 * TILEB, sV = sK + TILEB;
        const uint32_t t0 = tile * KTILE;
        // warps whose rows all lie before this tile have nothing to add (uniform per warp)
        if (t0 <= first + r0 + warp * 16 + 15) {
            float s[KTILE / 8][4];
#pragma unroll
            for (int j = 0; j < KTILE / 8; ++j) {
                s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
                for (int kt = 0; kt < D / 16; kt += 2) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(sK + (8 * j + (lane & 7)) * ROWB + (16 * kt + 8 * (lane >> 3)) * 2, b0, b1, b2, b3);
                    mma16816(s[j], qa[kt], b0, b1);
                    mma16816(s[j], qa[kt + 1], b2, b3);
                }
            }
            // causal mask, running maximum
            float mx_a = m_a, mx_b = m_b;
#pragma unroll
            for (int j = 0; j < KTILE / 8; ++j) {
                const uint32_t col = t0 + 8 * j + 2 * t;
                if (col > pos_a) s[j][0] = -INFINITY;
                if (col + 1 > pos_a) s[j][1] = -INFINITY;
                if (col > pos_b) s[j][2] = -INFINITY;
                if (col + 1 > pos_b) s[j][3] = -INFINITY;
                mx_a = fmaxf(mx_a, fmaxf(s[j][0], s[j][1]));
                mx_b = fmaxf(mx_b, fmaxf(s[j][2], s[j][3]));
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xFFFFFFFFu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xFFFFFFFFu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xFFFFFFFFu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xFFFFFFFFu, mx_b, 2));
            // position 0 is visible to every row, so the maxima are finite from the first tile on
            const float ca = exp2f((m_a - mx_a) * LOG2E), cb = exp2f((m_b - mx_b) * LOG2E);
            m_a = mx_a; m_b = mx_b;
            float sum_a = 0.0f, sum_b = 0.0f;
            uint32_t pa[KTILE / 16][4];
#pragma unroll
            for (int j = 0; j < KTILE / 8; ++j) {
                const float p0 = exp2f((s[j][0] - m_a) * LOG2E), p1 = exp2f((s[j][1] - m_a) * LOG2E);
                const float p2 = exp2f((s[j][2] - m_b) * LOG2E), p3 = exp2f((s[j][3] - m_b) * LOG2E);
                sum_a += p0 + p1; sum_b += p2 + p3;
                pa[j >> 1][(j & 1) * 2 + 0] = pack_h2(p0, p1);
                pa[j >> 1][(j & 1) * 2 + 1] = pack_h2(p2, p3);
            }
            l_a = l_a * ca + sum_a; l_b = l_b * cb + sum_b;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) { o[i][0] *= ca; o[i][1] *= ca; o[i][2] *= cb; o[i][3] *= cb; }
#pragma unroll
            for (int kk = 0; kk < KTILE / 16; ++kk) {
#pragma unroll
                for (int dn = 0; dn < D / 8; dn += 2) {
                    uint32_t b0, b1, b2, b3;
                    const uint32_t mtx = lane >> 3;
                    ldsm_x4_t(sV + (16 * kk + 8 * (mtx & 1) + (lane & 7)) * ROWB + (8 * (dn + (mtx >> 1))) * 2, b0, b1, b2, b3);
                    mma16816(o[dn], pa[kk], b0, b1);
                    mma16816(o[dn + 1], pa[kk], b2, b3);
                }
            }
        }
        __syncthreads();  // the buffer is staged again two tiles on
    }
    // row sums over the four lanes of a row, normalise, store
    l_a += __shfl_xor_sync(0xFFFFFFFFu, l_a, 1); l_a += __shfl_xor_sync(0xFFFFFFFFu, l_a, 2);
    l_b += __shfl_xor_sync(0xFFFFFFFFu, l_b, 1); l_b += __shfl_xor_sync(0xFFFFFFFFu, l_b, 2);
    const float ia = 1.0f / l_a, ib = 1.0f / l_b;
    const uint32_t ra = r0 + warp * 16 + g, rb = ra + 8;
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn) {
        if (ra < n) *reinterpret_cast<float2*>(out + ((size_t)ra * Hq + h) * D + 8 * dn + 2 * t) = make_float2(o[dn][0] * ia, o[dn][1] * ia);
        if (rb < n) *reinterpret_cast<float2*>(out + ((size_t)rb * Hq + h) * D + 8 * dn + 2 * t) = make_float2(o[dn][2] * ib, o[dn][3] * ib);
    }
}

template <int D>
cudaError_t launch_prefill(const LaunchCfg& lc, float* out, const float* q, const __half* kv_layer, const int32_t* table_row,
                           uint32_t first, uint32_t n, uint32_t Hq, uint32_t Hkv, uint32_t block_tokens) {
    constexpr int SMEM = 2 * 2 * KTILE * (D + 8) * 2;
    static bool opted = false;
    if (!opted) {
        cudaError_t e = cudaFuncSetAttribute(k_attn_prefill<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return e;
        opted = true;
    }
    const float scale = 1.0f / sqrtf((float)D);
    return launch(lc, k_attn_prefill<D>, dim3((n + QROWS - 1) / QROWS, Hq), dim3(128), SMEM, out, q, kv_layer, table_row, first, n, Hq,
                  Hkv, block_tokens, scale);
}

}  // namespace

bool attention_prefill_supported(uint32_t Hq, uint32_t Hkv, uint32_t D) {
    return (D == 64 || D == 128) && Hkv > 0 && Hq % Hkv == 0;
}

// out/q: [n][Hq*D] fp32 (q with bias and RoPE applied); rows are positions first..first+n-1 of the sequence whose
// block-table row is `table_row`
cudaError_t attention_prefill(const LaunchCfg& lc, float* out, const float* q, const __half* kv_layer, const int32_t* table_row,
                              uint32_t first, uint32_t n, uint32_t Hq, uint32_t Hkv, uint32_t D, uint32_t block_tokens) {
    if (n == 0) return cudaSuccess;
    if (!attention_prefill_supported(Hq, Hkv, D)) return cudaErrorInvalidValue;
    if (D == 64) return launch_prefill<64>(lc, out, q, kv_layer, table_row, first, n, Hq, Hkv, block_tokens);
    return launch_prefill<128>(lc, out, q, kv_layer, table_row, first, n, Hq, Hkv, block_tokens);
}

}  // namespace vb
