// Decode attention: flash-decode split-K over the KV length with grouped queries.
//
// Pass 1 (k_attn_split): grid (kv_head x q-head chunk, split, sequence).  A block owns one KV head, the
// (up to 8) query heads that share it and one slice of the context; its 4 warps walk the slice token by
// token, every K/V row is read once and used for all the query heads of the group, and each warp keeps an
// online-softmax state (m, l, acc) per query head.  The block's partial (m, l, unnormalised acc) goes to
// scratch.  Pass 2 (k_attn_combine) merges the splits.  The reference computes the same quantity with a
// two-pass softmax on the CPU (src/runtime.rs:772-831) and a sequential online softmax on the GPU
// (src/runners/tinystories_smollm.cu:321-393); its split-K test is
// tests/empirical_challenge_phase2/test2_split_k_flashdecoding_parity.cu.
//
// The cache is either the reference's contiguous fp32 layout [t][Hkv*D] or this library's paged fp16 pool,
// per layer [block][K|V][kv_head][block_tokens][D].
#include "vb_internal.cuh"
#include "vb_kernels.cuh"

namespace vb {

constexpr int ATTN_WARPS = 4;

struct AttnKArgs {
    AttnArgs a;
    float scale;
    uint32_t G;          // query heads per KV head
    uint32_t g_chunks;   // ceil(G / GM), GM = query heads a block handles at once
    uint32_t n_splits;
    size_t kv_batch_stride;  // contiguous: elements between sequences
};

template <typename KVT, int EPL>
__device__ __forceinline__ void load_row(const KVT* __restrict__ p, uint32_t lane, float out[EPL]) {
    if constexpr (sizeof(KVT) == 2) {
        if constexpr (EPL == 1) {
            out[0] = __half2float(reinterpret_cast<const __half*>(p)[lane]);
        } else if constexpr (EPL == 2) {
            float2 f = __half22float2(reinterpret_cast<const __half2*>(p)[lane]);
            out[0] = f.x; out[1] = f.y;
        } else if constexpr (EPL == 4) {
            uint2 raw = reinterpret_cast<const uint2*>(p)[lane];
            const __half2* h = reinterpret_cast<const __half2*>(&raw);
            float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
            out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
        } else {
#pragma unroll
            for (int c = 0; c < EPL / 8; ++c) {
                uint4 raw = reinterpret_cast<const uint4*>(p)[lane * (EPL / 8) + c];
                const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); out[c * 8 + 2 * i] = f.x; out[c * 8 + 2 * i + 1] = f.y; }
            }
        }
    } else {
        const float* f = reinterpret_cast<const float*>(p) + (size_t)lane * EPL;
        if constexpr (EPL % 4 == 0) {
#pragma unroll
            for (int c = 0; c < EPL / 4; ++c) {
                float4 v = reinterpret_cast<const float4*>(f)[c];
                out[4 * c] = v.x; out[4 * c + 1] = v.y; out[4 * c + 2] = v.z; out[4 * c + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < EPL; ++i) out[i] = f[i];
        }
    }
}

template <typename KVT, int EPL, int GM>
__global__ void __launch_bounds__(ATTN_WARPS * 32) k_attn_split(AttnKArgs ka) {
    const AttnArgs& a = ka.a;
    constexpr int D = EPL * 32;
    __shared__ float q_s[GM][D];
    __shared__ float part_ml[ATTN_WARPS][GM][2];
    extern __shared__ __align__(16) float part_acc[];  // [ATTN_WARPS][GM][D]

    pdl_wait();
    pdl_launch_dependents();

    const uint32_t b = blockIdx.z, split = blockIdx.y;
    const uint32_t kvh = blockIdx.x / ka.g_chunks, gc = blockIdx.x % ka.g_chunks;
    const uint32_t g0 = gc * GM;
    const uint32_t ng = min((uint32_t)GM, ka.G - g0);
    if (a.state && !a.state[b].active) return;
    const uint32_t seq_len = (a.state ? a.state[b].pos : a.pos) + 1;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // slice of the context owned by this split (whole KV blocks)
    uint32_t per = (seq_len + ka.n_splits - 1) / ka.n_splits;
    per = ((per + a.block_tokens - 1) / a.block_tokens) * a.block_tokens;
    const uint32_t t_lo = min(seq_len, split * per), t_hi = min(seq_len, t_lo + per);

    const float* qb = a.q + (size_t)b * a.Hq * D + (size_t)(kvh * ka.G + g0) * D;
    for (uint32_t i = threadIdx.x; i < ng * D; i += blockDim.x) q_s[i / D][i % D] = qb[i];
    __syncthreads();

    float m[GM], l[GM], acc[GM][EPL], qr[GM][EPL];
#pragma unroll
    for (int g = 0; g < GM; ++g) {
        m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) { acc[g][e] = 0.0f; qr[g][e] = (g < (int)ng) ? q_s[g][lane * EPL + e] : 0.0f; }
    }

    for (uint32_t t = t_lo + warp; t < t_hi; t += ATTN_WARPS) {
        const KVT *kp, *vp;
        if (a.block_table) {
            const int32_t blk = a.block_table[(size_t)b * a.max_blocks + t / a.block_tokens];
            const size_t base = (((size_t)blk * 2) * a.Hkv + kvh) * a.block_tokens * D + (size_t)(t % a.block_tokens) * D;
            kp = reinterpret_cast<const KVT*>(a.k) + base;
            vp = kp + (size_t)a.Hkv * a.block_tokens * D;
        } else {
            const size_t off = (size_t)b * ka.kv_batch_stride + (size_t)t * a.Hkv * D + (size_t)kvh * D;
            kp = reinterpret_cast<const KVT*>(a.k) + off;
            vp = reinterpret_cast<const KVT*>(a.v) + off;
        }
        float kr[EPL], vr[EPL];
        load_row<KVT, EPL>(kp, lane, kr);
        load_row<KVT, EPL>(vp, lane, vr);
#pragma unroll
        for (int g = 0; g < GM; ++g) {
            if (g < (int)ng) {
                float dot = 0.0f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) dot = fmaf(qr[g][e], kr[e], dot);
                dot = warp_sum(dot);
                const float s = dot * ka.scale;
                const float new_m = fmaxf(m[g], s);
                const float alpha = (m[g] == -INFINITY) ? 0.0f : __expf(m[g] - new_m);
                const float beta = __expf(s - new_m);
                l[g] = l[g] * alpha + beta;
                m[g] = new_m;
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[g][e] = fmaf(acc[g][e], alpha, beta * vr[e]);
            }
        }
    }

    // merge the 4 warps
#pragma unroll
    for (int g = 0; g < GM; ++g) {
        if (g < (int)ng) {
            if (lane == 0) { part_ml[warp][g][0] = m[g]; part_ml[warp][g][1] = l[g]; }
#pragma unroll
            for (int e = 0; e < EPL; ++e) part_acc[((size_t)warp * GM + g) * D + lane * EPL + e] = acc[g][e];
        }
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < ng * D; i += blockDim.x) {
        const uint32_t g = i / D, d = i % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; ++w) M = fmaxf(M, part_ml[w][g][0]);
        float L = 0.0f, A = 0.0f;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; ++w) {
            const float mw = part_ml[w][g][0];
            const float f = (mw == -INFINITY) ? 0.0f : __expf(mw - M);
            L = fmaf(part_ml[w][g][1], f, L);
            A = fmaf(part_acc[((size_t)w * GM + g) * D + d], f, A);
        }
        const uint32_t h = kvh * ka.G + g0 + g;
        float* ps = a.scratch + (((size_t)b * a.Hq + h) * ka.n_splits + split) * (D + 2);
        ps[2 + d] = A;
        if (d == 0) { ps[0] = M; ps[1] = L; }
    }
}

// grid (Hq, batch), D threads
__global__ void k_attn_combine(AttnKArgs ka, uint32_t D) {
    const AttnArgs& a = ka.a;
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t h = blockIdx.x, b = blockIdx.y;
    if (a.state && !a.state[b].active) return;
    const float* ps = a.scratch + (((size_t)b * a.Hq + h) * ka.n_splits) * (D + 2);
    float M = -INFINITY;
    for (uint32_t s = 0; s < ka.n_splits; ++s) M = fmaxf(M, ps[(size_t)s * (D + 2)]);
    for (uint32_t d = threadIdx.x; d < D; d += blockDim.x) {
        float L = 0.0f, A = 0.0f;
        for (uint32_t s = 0; s < ka.n_splits; ++s) {
            const float ms = ps[(size_t)s * (D + 2)];
            const float f = (ms == -INFINITY) ? 0.0f : __expf(ms - M);
            L = fmaf(ps[(size_t)s * (D + 2) + 1], f, L);
            A = fmaf(ps[(size_t)s * (D + 2) + 2 + d], f, A);
        }
        a.out[(size_t)b * a.Hq * D + (size_t)h * D + d] = (L > 0.0f) ? (A / L) : 0.0f;
    }
}

uint64_t attn_scratch_floats(uint32_t Hq, uint32_t D, uint32_t batch, uint32_t max_splits) {
    return (uint64_t)batch * Hq * max_splits * (D + 2);
}
uint32_t attn_pick_splits(uint32_t max_seq) {
    uint32_t s = (max_seq + 255) / 256;
    if (s < 1) s = 1;
    if (s > 32) s = 32;
    return s;
}

template <typename KVT, int EPL, int GM>
static cudaError_t launch_split_g(const LaunchCfg& lc, AttnKArgs ka) {
    ka.g_chunks = (ka.G + GM - 1) / GM;
    const size_t smem = (size_t)ATTN_WARPS * GM * EPL * 32 * sizeof(float);
    dim3 grid(ka.a.Hkv * ka.g_chunks, ka.n_splits, ka.a.batch);
    return launch(lc, k_attn_split<KVT, EPL, GM>, grid, dim3(ATTN_WARPS * 32), smem, ka);
}

template <typename KVT, int EPL>
static cudaError_t launch_split(const LaunchCfg& lc, const AttnKArgs& ka) {
    if constexpr (EPL >= 8) {
        return launch_split_g<KVT, EPL, 1>(lc, ka);  // wide heads: one query head per block keeps registers in bounds
    } else {
        if (ka.G == 1) return launch_split_g<KVT, EPL, 1>(lc, ka);
        if (ka.G <= 4) return launch_split_g<KVT, EPL, 4>(lc, ka);
        return launch_split_g<KVT, EPL, 8>(lc, ka);
    }
}

template <typename KVT>
static cudaError_t dispatch_split(const LaunchCfg& lc, const AttnKArgs& ka) {
    switch (ka.a.D) {
    case 32: return launch_split<KVT, 1>(lc, ka);
    case 64: return launch_split<KVT, 2>(lc, ka);
    case 128: return launch_split<KVT, 4>(lc, ka);
    case 256: return launch_split<KVT, 8>(lc, ka);
    case 512: return launch_split<KVT, 16>(lc, ka);
    default: return cudaErrorInvalidValue;
    }
}

template <typename KVT, int EPL, int GM>
static cudaError_t opt_in_one() {
    const size_t smem = (size_t)ATTN_WARPS * GM * EPL * 32 * sizeof(float);
    if (smem <= 32 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(k_attn_split<KVT, EPL, GM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}
template <typename KVT>
static cudaError_t opt_in_all() {
    cudaError_t e;
    if ((e = opt_in_one<KVT, 4, 8>()) != cudaSuccess) return e;
    if ((e = opt_in_one<KVT, 8, 1>()) != cudaSuccess) return e;
    return opt_in_one<KVT, 16, 1>();
}
cudaError_t attn_init() {
    cudaError_t e = opt_in_all<__half>();
    if (e != cudaSuccess) return e;
    return opt_in_all<float>();
}

cudaError_t attention_ex(const LaunchCfg& lc, const AttnArgs& a, float scale, size_t kv_batch_stride) {
    if (a.batch == 0 || a.Hq == 0) return cudaSuccess;
    if (a.Hkv == 0 || a.Hq % a.Hkv != 0) return cudaErrorInvalidValue;
    AttnKArgs ka;
    ka.a = a;
    ka.scale = (scale != 0.0f) ? scale : 1.0f / sqrtf((float)a.D);
    ka.G = a.Hq / a.Hkv;
    ka.g_chunks = 1;
    ka.n_splits = a.max_splits ? a.max_splits : 1;
    ka.kv_batch_stride = kv_batch_stride;
    cudaError_t e = a.kv_fp16 ? dispatch_split<__half>(lc, ka) : dispatch_split<float>(lc, ka);
    if (e != cudaSuccess) return e;
    return launch(lc, k_attn_combine, dim3(a.Hq, a.batch), dim3(a.D < 128 ? a.D : 128), 0, ka, a.D);
}

cudaError_t attention(const LaunchCfg& lc, const AttnArgs& a) { return attention_ex(lc, a, 0.0f, 0); }

}  // namespace vb

using namespace vb;

extern "C" int32_t vb_op_gqa_attention(float* out, const float* q, const float* k_cache, const float* v_cache,
                                       uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t pos, void* scratch,
                                       uint64_t scratch_bytes, void* stream) {
    VB_REQUIRE(out && q && k_cache && v_cache && scratch, "vb_op_gqa_attention: null pointer");
    VB_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "vb_op_gqa_attention: n_q=%u not a multiple of n_kv=%u", n_q, n_kv);
    VB_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256 || head_dim == 512,
               "vb_op_gqa_attention: head_dim=%u (supported: 32,64,128,256,512)", head_dim);
    AttnArgs a;
    a.out = out; a.q = q; a.k = k_cache; a.v = v_cache; a.kv_fp16 = 0;
    a.pos = pos; a.Hq = n_q; a.Hkv = n_kv; a.D = head_dim; a.batch = 1;
    a.max_splits = attn_pick_splits(pos + 1);
    a.scratch = (float*)scratch;
    VB_REQUIRE(scratch_bytes >= attn_scratch_floats(n_q, head_dim, 1, a.max_splits) * 4,
               "vb_op_gqa_attention: scratch too small (%llu bytes)", (unsigned long long)scratch_bytes);
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    VB_CUDA(kernels_init());
    VB_CUDA(attention(lc, a));
    return VB_OK;
}

extern "C" uint64_t vb_op_scratch_bytes(uint32_t n_q_heads, uint32_t head_dim, uint32_t max_seq, uint32_t vocab) {
    uint64_t a = attn_scratch_floats(n_q_heads ? n_q_heads : 1, head_dim, 1, attn_pick_splits(max_seq)) * 4;
    uint64_t b = (uint64_t)argmax_chunks(vocab ? vocab : 1) * 8;
    uint64_t m = (uint64_t)(head_dim > 0 ? head_dim : 1) * 16;  // q_abs + bookkeeping of the MLA op
    return a + b + m + 4096;
}
