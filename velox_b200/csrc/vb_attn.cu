// Decode attention: flash-decode split-K over the KV length with grouped queries, one kernel.
//
// Grid (kv_head x q-head chunk, split, sequence).  A block owns one KV head, the (up to 8) query heads that
// share it and one slice of the context (a whole number of 16-token KV blocks).  The kernel is latency-bound
// at decode sizes, so it makes as few dependent memory trips as it can: (1) the sequence's position, (2) the
// slice's block-table entries together with the query heads, (3) per chunk of up to 64 tokens ALL K and V
// rows at once, cp.async into shared memory, double buffered.  Each of the 4 warps then takes 4 or 8 tokens
// at a time, uses every row for all query heads of the group, reduces the per-lane partial dot products
// with a transposing butterfly (one value per lane instead of one reduction per value) and keeps an
// online-softmax state (m, l, acc) per query head.  The splits of one (sequence, head group) form a
// thread-block cluster: each block leaves its partial in its own shared memory and, after a cluster barrier,
// every block merges one slice of the head dimension by reading the others' partials through distributed
// shared memory -- no global round trip, no atomics, a fixed merge order.
// In the engine the kernel also does what the reference runs as separate kernels before attention
// (fused_rope_kernel and the KV write of fused_qkv, src/runners/tinystories_smollm.cu:189-318): bias, RoPE of
// q and of the new k at the sequence's position, and the append of K/V to the cache.
//
// The reference computes the same quantity with a two-pass softmax on the CPU (src/runtime.rs:772-831) and a
// sequential online softmax on the GPU (src/runners/tinystories_smollm.cu:321-393); its split-K test is
// tests/empirical_challenge_phase2/test2_split_k_flashdecoding_parity.cu.
//
// The cache is either the reference's contiguous fp32 layout [t][Hkv*D] or this library's paged fp16 pool,
// per layer [block][K|V][kv_head][block_tokens][D].
#include <cooperative_groups.h>
#include <stdlib.h>

#include "vb_internal.cuh"
#include "vb_kernels.cuh"

namespace cg = cooperative_groups;

namespace vb {

constexpr int ATTN_WARPS = 4;
constexpr int ATTN_MAX_SPLITS = 8;  // portable thread-block cluster size
constexpr int ATTN_MAX_BLOCKS = 1024;  // KV blocks one block's slice may span (16384 tokens)

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

__device__ __forceinline__ float bias_at(const void* w, int fmt, uint32_t i) {
    return fmt == VB_FMT_F16 ? __half2float(((const __half*)w)[i])
         : fmt == VB_FMT_BF16 ? __bfloat162float(((const __nv_bfloat16*)w)[i]) : ((const float*)w)[i];
}

// Sums NV per-lane values over the warp; afterwards v[0] of lane L is the total of value (L % NV).
template <int NV>
__device__ __forceinline__ void warp_transpose_reduce(float v[NV], uint32_t lane) {
#pragma unroll
    for (int off = 16; off >= NV; off >>= 1) {
#pragma unroll
        for (int i = 0; i < NV; ++i) v[i] += __shfl_xor_sync(0xFFFFFFFFu, v[i], off);
    }
#pragma unroll
    for (int off = (NV > 16 ? 16 : NV / 2), n = NV; off >= 1; off >>= 1, n >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float mine = upper ? v[i + n / 2] : v[i];
            const float other = upper ? v[i] : v[i + n / 2];
            v[i] = mine + __shfl_xor_sync(0xFFFFFFFFu, other, off);
        }
    }
}

__device__ __forceinline__ void attn_cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}

// Shared-memory plan of one block (dynamic): K/V staging for two chunks of CH tokens, the warp-merge buffer.
template <typename KVT, int EPL, int GM>
struct AttnSmem {
    static constexpr int D = EPL * 32;
    // tokens per staged chunk: K+V of a chunk take at most 32 KB, at most 64 tokens
    static constexpr int CH = (16384 / (D * (int)sizeof(KVT))) > 64 ? 64 : (16384 / (D * (int)sizeof(KVT)));
    static constexpr size_t kv_bytes = (size_t)2 * 2 * CH * D * sizeof(KVT);  // [buffer][K|V][CH][D]
    static constexpr size_t acc_bytes = (size_t)ATTN_WARPS * GM * D * sizeof(float);
    static constexpr size_t total = kv_bytes + acc_bytes;
};

template <typename KVT, int EPL, int GM>
__global__ void __launch_bounds__(ATTN_WARPS * 32) k_attn_split(AttnKArgs ka) {
    const AttnArgs& a = ka.a;
    using SM = AttnSmem<KVT, EPL, GM>;
    constexpr int D = EPL * 32, CH = SM::CH;
    constexpr int TCH = (EPL >= 8) ? 2 : ((GM >= 8) ? 4 : 8);  // tokens a warp handles at once
    constexpr int NV = TCH * GM;                              // partial dot products per lane (<= 32)
    constexpr int ROW16 = D * sizeof(KVT) / 16;               // 16-byte pieces per K or V row
    static_assert(NV <= 32 && (NV & (NV - 1)) == 0, "values per lane must be a power of two <= 32");
    __shared__ float q_s[GM][D];
    __shared__ float sc_s[ATTN_WARPS][32];
    __shared__ float part_ml[ATTN_WARPS][GM][2];
    __shared__ float comb[GM][D + 2];       // this block's partial, read by the whole cluster
    __shared__ int32_t blk_s[ATTN_MAX_BLOCKS];  // block-table entries of this block's slice
    __shared__ __align__(16) KVT new_kv[2][D];  // the appended token's K and V (fused mode)
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    KVT* kv_s = reinterpret_cast<KVT*>(dyn_smem);
    float* part_acc = reinterpret_cast<float*>(dyn_smem + SM::kv_bytes);  // [ATTN_WARPS][GM][D]

    trace_mark(a.trace, 0);
    pdl_wait();
    pdl_launch_dependents();
    trace_mark(a.trace, 1);

    const uint32_t b = blockIdx.z, split = blockIdx.y;
    const uint32_t kvh = blockIdx.x / ka.g_chunks, gc = blockIdx.x % ka.g_chunks;
    const uint32_t g0 = gc * GM;
    const uint32_t ng = min((uint32_t)GM, ka.G - g0);
    if (a.state && !a.state[b].active) return;
    const uint32_t seq_len = (a.state ? a.state[b].pos : a.pos) + 1;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // the context is cut into n_splits equal slices of whole KV blocks, whatever its current length
    uint32_t per = (seq_len + ka.n_splits - 1) / ka.n_splits;
    per = ((per + a.block_tokens - 1) / a.block_tokens) * a.block_tokens;
    const uint32_t t_lo = min(seq_len, split * per), t_hi = min(seq_len, t_lo + per);
    const uint32_t pos = seq_len - 1;
    const bool appender = a.qkv_raw && t_lo <= pos && pos < t_hi;

    float m[GM], l[GM], acc[GM][EPL];
#pragma unroll
    for (int g = 0; g < GM; ++g) {
        m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = 0.0f;
    }

    // One chunk = tokens [c0, c0+CH) of the slice: every 16-byte piece of its K and V rows is requested at once.
    auto stage_chunk = [&](uint32_t c0, uint32_t buf) {
        const uint32_t n_tok = min((uint32_t)CH, t_hi - c0);
        KVT* kb = kv_s + (size_t)buf * 2 * CH * D;
        for (uint32_t i = threadIdx.x; i < n_tok * 2 * ROW16; i += blockDim.x) {
            const uint32_t piece = i % ROW16, kv = (i / ROW16) & 1, tok = i / (2 * ROW16);
            const uint32_t tt = c0 + tok;
            const KVT* src;
            if (a.block_table) {
                const int32_t blk = blk_s[(tt - t_lo) / a.block_tokens];
                src = reinterpret_cast<const KVT*>(a.k) + (((size_t)blk * 2 + kv) * a.Hkv + kvh) * a.block_tokens * D +
                      (size_t)(tt % a.block_tokens) * D;
            } else {
                const size_t off = (size_t)b * ka.kv_batch_stride + (size_t)tt * a.Hkv * D + (size_t)kvh * D;
                src = reinterpret_cast<const KVT*>(kv ? a.v : a.k) + off;
            }
            attn_cp_async16((uint32_t)__cvta_generic_to_shared(kb + ((size_t)kv * CH + tok) * D) + piece * 16,
                            reinterpret_cast<const unsigned char*>(src) + piece * 16);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    if (t_lo < t_hi) {
        // ---- one trip: block-table entries of the slice, the query heads (and, fused, the new token's K/V) ----
        if (a.block_table) {
            const uint32_t nblk = (t_hi - t_lo + a.block_tokens - 1) / a.block_tokens;
            for (uint32_t i = threadIdx.x; i < nblk && i < (uint32_t)ATTN_MAX_BLOCKS; i += blockDim.x)
                blk_s[i] = a.block_table[(size_t)b * a.max_blocks + t_lo / a.block_tokens + i];
        }
        if (a.qkv_raw) {
            // fused bias + RoPE on the raw projections
            const uint32_t half = D / 2;
            const float* raw = a.qkv_raw + (size_t)b * (a.Hq + 2 * a.Hkv) * D;
            for (uint32_t i = threadIdx.x; i < GM * half; i += blockDim.x) {
                const uint32_t g = i / half, j = i % half;
                float r1 = 0.0f, r2 = 0.0f;
                if (g < ng) {
                    const uint32_t h = kvh * ka.G + g0 + g;
                    float x1 = raw[(size_t)h * D + j], x2 = raw[(size_t)h * D + j + half];
                    if (a.bq) { x1 += bias_at(a.bq, a.bias_fmt, h * D + j); x2 += bias_at(a.bq, a.bias_fmt, h * D + j + half); }
                    float sn, cs;
                    sincosf((float)pos * a.rope_inv_freq[j], &sn, &cs);
                    r1 = x1 * cs - x2 * sn;
                    r2 = x2 * cs + x1 * sn;
                }
                q_s[g][j] = r1;
                q_s[g][j + half] = r2;
            }
            if (appender) {
                const float* kr_raw = raw + (size_t)a.Hq * D + (size_t)kvh * D;
                const float* vr_raw = raw + (size_t)(a.Hq + a.Hkv) * D + (size_t)kvh * D;
                for (uint32_t j = threadIdx.x; j < half; j += blockDim.x) {
                    float x1 = kr_raw[j], x2 = kr_raw[j + half], v1 = vr_raw[j], v2 = vr_raw[j + half];
                    if (a.bk) { x1 += bias_at(a.bk, a.bias_fmt, kvh * D + j); x2 += bias_at(a.bk, a.bias_fmt, kvh * D + j + half); }
                    if (a.bv) { v1 += bias_at(a.bv, a.bias_fmt, kvh * D + j); v2 += bias_at(a.bv, a.bias_fmt, kvh * D + j + half); }
                    float sn, cs;
                    sincosf((float)pos * a.rope_inv_freq[j], &sn, &cs);
                    new_kv[0][j] = (KVT)__float2half_rn(x1 * cs - x2 * sn);
                    new_kv[0][j + half] = (KVT)__float2half_rn(x2 * cs + x1 * sn);
                    new_kv[1][j] = (KVT)__float2half_rn(v1);
                    new_kv[1][j + half] = (KVT)__float2half_rn(v2);
                }
            }
        } else {
            const float* qb = a.q + (size_t)b * a.Hq * D + (size_t)(kvh * ka.G + g0) * D;
            for (uint32_t i = threadIdx.x; i < GM * D; i += blockDim.x) q_s[i / D][i % D] = (i < ng * D) ? qb[i] : 0.0f;
        }
        __syncthreads();
        if (appender && gc == 0) {
            // the new token's row goes to the cache (16-byte stores); this block reads it from new_kv below
            const int32_t blk = blk_s[(pos - t_lo) / a.block_tokens];
            KVT* kd = reinterpret_cast<KVT*>(const_cast<void*>(a.k)) + (((size_t)blk * 2) * a.Hkv + kvh) * a.block_tokens * D +
                      (size_t)(pos % a.block_tokens) * D;
            KVT* vd = kd + (size_t)a.Hkv * a.block_tokens * D;
            for (uint32_t i = threadIdx.x; i < 2 * ROW16; i += blockDim.x) {
                const uint32_t kv = i / ROW16, piece = i % ROW16;
                reinterpret_cast<uint4*>(kv ? vd : kd)[piece] = reinterpret_cast<const uint4*>(new_kv[kv])[piece];
            }
        }

        float qr[GM][EPL];
#pragma unroll
        for (int g = 0; g < GM; ++g)
#pragma unroll
            for (int e = 0; e < EPL; ++e) qr[g][e] = q_s[g][lane * EPL + e];

        // ---- the slice, CH tokens at a time, double buffered: one memory trip per chunk ----------------------
        const uint32_t n_ch = (t_hi - t_lo + CH - 1) / CH;
        stage_chunk(t_lo, 0);
        for (uint32_t c = 0; c < n_ch; ++c) {
            const uint32_t c0 = t_lo + c * CH, buf = c & 1;
            if (c + 1 < n_ch) {
                stage_chunk(c0 + CH, buf ^ 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();
            KVT* kb = kv_s + (size_t)buf * 2 * CH * D;
            if (appender && c0 <= pos && pos < c0 + CH) {
                // overwrite the staged copy of the new token's row with the values just computed
                for (uint32_t i = threadIdx.x; i < 2 * ROW16; i += blockDim.x) {
                    const uint32_t kv = i / ROW16, piece = i % ROW16;
                    reinterpret_cast<uint4*>(kb + ((size_t)kv * CH + (pos - c0)) * D)[piece] = reinterpret_cast<const uint4*>(new_kv[kv])[piece];
                }
                __syncthreads();
            }
            const uint32_t c_hi = min(t_hi, c0 + CH);
            for (uint32_t t0 = c0 + warp * TCH; t0 < c_hi; t0 += ATTN_WARPS * TCH) {
                float kr[TCH][EPL], vr[TCH][EPL];
#pragma unroll
                for (int i = 0; i < TCH; ++i) {
                    const uint32_t tok = min(t0 + i, c_hi - 1) - c0;  // out-of-range tokens re-read the last row, masked below
                    load_row<KVT, EPL>(kb + (size_t)tok * D, lane, kr[i]);
                    load_row<KVT, EPL>(kb + ((size_t)CH + tok) * D, lane, vr[i]);
                }
                // partial dot products, value index = g * TCH + i
                float pv[NV];
#pragma unroll
                for (int g = 0; g < GM; ++g)
#pragma unroll
                    for (int i = 0; i < TCH; ++i) {
                        float d = 0.0f;
#pragma unroll
                        for (int e = 0; e < EPL; ++e) d = fmaf(qr[g][e], kr[i][e], d);
                        pv[g * TCH + i] = d;
                    }
                warp_transpose_reduce<NV>(pv, lane);
                __syncwarp();
                if (lane < NV) {
                    const uint32_t i = lane % TCH;
                    sc_s[warp][lane] = (t0 + i < c_hi) ? pv[0] * ka.scale : -INFINITY;
                }
                __syncwarp();
#pragma unroll
                for (int g = 0; g < GM; ++g) {
                    float sv[TCH];
                    float cmax = -INFINITY;
#pragma unroll
                    for (int i = 0; i < TCH; ++i) { sv[i] = sc_s[warp][g * TCH + i]; cmax = fmaxf(cmax, sv[i]); }
                    const float new_m = fmaxf(m[g], cmax);
                    if (new_m != -INFINITY) {
                        const float alpha = (m[g] == -INFINITY) ? 0.0f : __expf(m[g] - new_m);
                        float p[TCH], psum = 0.0f;
#pragma unroll
                        for (int i = 0; i < TCH; ++i) { p[i] = __expf(sv[i] - new_m); psum += p[i]; }
                        l[g] = fmaf(l[g], alpha, psum);
                        m[g] = new_m;
#pragma unroll
                        for (int e = 0; e < EPL; ++e) {
                            float v = acc[g][e] * alpha;
#pragma unroll
                            for (int i = 0; i < TCH; ++i) v = fmaf(p[i], vr[i][e], v);
                            acc[g][e] = v;
                        }
                    }
                }
            }
            __syncthreads();  // the buffer is free for the chunk after next
        }
    }

    // ---- merge the 4 warps into this block's partial (m, l, unnormalised acc), kept in shared memory --------
#pragma unroll
    for (int g = 0; g < GM; ++g) {
        if (lane == 0) { part_ml[warp][g][0] = m[g]; part_ml[warp][g][1] = l[g]; }
#pragma unroll
        for (int e = 0; e < EPL; ++e) part_acc[((size_t)warp * GM + g) * D + lane * EPL + e] = acc[g][e];
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < GM * D; i += blockDim.x) {
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
        comb[g][2 + d] = A;
        if (d == 0) { comb[g][0] = M; comb[g][1] = L; }
    }

    // ---- merge the splits: the blocks of one (sequence, head group) form a thread-block cluster and read each
    // other's partials through distributed shared memory -- no global round trip, no atomics, fixed order
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const uint32_t n = ka.n_splits;  // == cluster size along y
    const uint32_t per_d = (D + n - 1) / n;
    const uint32_t d_lo = split * per_d, d_hi = min((uint32_t)D, d_lo + per_d);
    for (uint32_t i = threadIdx.x; i < ng * per_d; i += blockDim.x) {
        const uint32_t g = i / per_d, d = d_lo + i % per_d;
        if (d < d_hi) {
            // all remote reads are issued before any is used (a remote shared-memory load costs hundreds of cycles)
            float ms[ATTN_MAX_SPLITS], ls[ATTN_MAX_SPLITS], as[ATTN_MAX_SPLITS];
#pragma unroll
            for (int r = 0; r < ATTN_MAX_SPLITS; ++r) {
                const float* rc = cluster.map_shared_rank(&comb[g][0], (uint32_t)r < n ? r : 0);
                const bool on = (uint32_t)r < n;
                ms[r] = on ? rc[0] : -INFINITY;
                ls[r] = on ? rc[1] : 0.0f;
                as[r] = on ? rc[2 + d] : 0.0f;
            }
            float M = -INFINITY;
#pragma unroll
            for (int r = 0; r < ATTN_MAX_SPLITS; ++r) M = fmaxf(M, ms[r]);
            float L = 0.0f, A = 0.0f;
#pragma unroll
            for (int r = 0; r < ATTN_MAX_SPLITS; ++r) {
                const float f = (ms[r] == -INFINITY) ? 0.0f : __expf(ms[r] - M);
                L = fmaf(ls[r], f, L);
                A = fmaf(as[r], f, A);
            }
            a.out[(size_t)b * a.Hq * D + (size_t)(kvh * ka.G + g0 + g) * D + d] = (L > 0.0f) ? (A / L) : 0.0f;
        }
    }
    cluster.sync();  // nobody leaves while its shared memory may still be read
    trace_exit(a.trace);
}

// the split partials live in shared memory now; a small scratch is still reserved for callers that pass one
uint64_t attn_scratch_floats(uint32_t Hq, uint32_t D, uint32_t batch, uint32_t max_splits) {
    (void)Hq; (void)D; (void)batch; (void)max_splits;
    return 64;
}
// kept for callers that size things per split; the kernel itself divides the current length evenly
uint32_t attn_tokens_per_split(uint32_t max_seq) {
    const uint32_t n = attn_pick_splits(max_seq);
    uint32_t tps = ((max_seq ? max_seq : 1) + n - 1) / n;
    return ((tps + 15) / 16) * 16;
}
// one split per 32 tokens of the longest context, at most a cluster's worth
uint32_t attn_pick_splits(uint32_t max_seq) {
    uint32_t s = ((max_seq ? max_seq : 1) + 31) / 32;
    if (s > (uint32_t)ATTN_MAX_SPLITS) s = ATTN_MAX_SPLITS;
    return s < 1 ? 1 : s;
}

template <typename KVT, int EPL, int GM>
static cudaError_t launch_split_g(const LaunchCfg& lc, AttnKArgs ka) {
    ka.g_chunks = (ka.G + GM - 1) / GM;
    const size_t smem = AttnSmem<KVT, EPL, GM>::total;
    dim3 grid(ka.a.Hkv * ka.g_chunks, ka.n_splits, ka.a.batch);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(ATTN_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = lc.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = ka.n_splits; attr[0].val.clusterDim.z = 1;
    cfg.numAttrs = 1;
    if (lc.pdl) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attr;
    if (lc.counter) ++*lc.counter;
    return cudaLaunchKernelEx(&cfg, k_attn_split<KVT, EPL, GM>, ka);
}

template <typename KVT, int EPL>
static cudaError_t launch_split(const LaunchCfg& lc, const AttnKArgs& ka) {
    if constexpr (EPL >= 8) {
        return launch_split_g<KVT, EPL, 1>(lc, ka);  // wide heads: one query head per block keeps registers in bounds
    } else {
        if (ka.G == 1) return launch_split_g<KVT, EPL, 1>(lc, ka);
        if (ka.G == 2) return launch_split_g<KVT, EPL, 2>(lc, ka);
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
    const size_t smem = AttnSmem<KVT, EPL, GM>::total;
    return cudaFuncSetAttribute(k_attn_split<KVT, EPL, GM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}
template <typename KVT>
static cudaError_t opt_in_all() {
    cudaError_t e;
#define VB_ATTN_OPT(E, G) if ((e = opt_in_one<KVT, E, G>()) != cudaSuccess) return e
    VB_ATTN_OPT(1, 1); VB_ATTN_OPT(1, 2); VB_ATTN_OPT(1, 4); VB_ATTN_OPT(1, 8);
    VB_ATTN_OPT(2, 1); VB_ATTN_OPT(2, 2); VB_ATTN_OPT(2, 4); VB_ATTN_OPT(2, 8);
    VB_ATTN_OPT(4, 1); VB_ATTN_OPT(4, 2); VB_ATTN_OPT(4, 4); VB_ATTN_OPT(4, 8);
    VB_ATTN_OPT(8, 1); VB_ATTN_OPT(16, 1);
#undef VB_ATTN_OPT
    return cudaSuccess;
}
cudaError_t attn_init() {
    cudaError_t e = opt_in_all<__half>();
    if (e != cudaSuccess) return e;
    return opt_in_all<float>();
}

cudaError_t attention_ex(const LaunchCfg& lc, const AttnArgs& a, float scale, size_t kv_batch_stride) {
    if (a.batch == 0 || a.Hq == 0) return cudaSuccess;
    if (a.Hkv == 0 || a.Hq % a.Hkv != 0 || a.max_splits == 0 || a.tokens_per_split == 0) return cudaErrorInvalidValue;
    AttnKArgs ka;
    ka.a = a;
    ka.scale = (scale != 0.0f) ? scale : 1.0f / sqrtf((float)a.D);
    ka.G = a.Hq / a.Hkv;
    ka.g_chunks = 1;
    ka.n_splits = a.max_splits;
    ka.kv_batch_stride = kv_batch_stride;
    return a.kv_fp16 ? dispatch_split<__half>(lc, ka) : dispatch_split<float>(lc, ka);
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
    a.tokens_per_split = attn_tokens_per_split(pos + 1);
    a.scratch = (float*)scratch;
    const uint64_t need = attn_scratch_floats(n_q, head_dim, 1, a.max_splits) * 4;
    VB_REQUIRE(scratch_bytes >= need, "vb_op_gqa_attention: scratch too small (%llu bytes, %llu needed)",
               (unsigned long long)scratch_bytes, (unsigned long long)need);
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    VB_CUDA(kernels_init());
    VB_CUDA(attention(lc, a));
    return VB_OK;
}

extern "C" uint64_t vb_op_scratch_bytes(uint32_t n_q_heads, uint32_t head_dim, uint32_t max_seq, uint32_t vocab) {
    const uint32_t hq = n_q_heads ? n_q_heads : 1, d = head_dim ? head_dim : 1;
    uint64_t a = attn_scratch_floats(hq, d, 1, attn_pick_splits(max_seq)) * 4;
    uint64_t b = (uint64_t)argmax_chunks(vocab ? vocab : 1) * 8;
    uint64_t m = mla_scratch_floats(0, d) * 4;
    return a + b + m + 4096;
}
