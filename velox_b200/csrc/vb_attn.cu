// Decode attention: flash-decode split-K over the KV length with grouped queries, one kernel.
//
// Grid (kv_head x q-head chunk, split, sequence).  A block owns one KV head, the (up to 8) query heads that
// share it and one slice of the context (a whole number of 16-token KV blocks).  The kernel is latency-bound
// at decode sizes, so it makes as few dependent memory trips as it can: (1) the sequence's position together
// with its (short) block-table row, (2) per chunk of up to 64 tokens ALL K and V rows at once, bulk copies
// (TMA) into two shared-memory buffers, requested before the grid-dependency wait because cached rows do not
// depend on this step's projections, (3) after the wait only the query heads.
// fp16 caches: the products run on the tensor cores (mma.sync m16n8k16).  A warp takes 16 tokens: S^T = K Q^T
// (tokens x heads) and O^T += V^T P^T (dims x heads) put the GROUP's query heads on the N = 8 columns, so a
// group of 8 fills the instruction and every thread's accumulator columns are the two heads whose running
// maximum it keeps; K comes in with ldmatrix, V with ldmatrix.trans, P is transposed in registers (movmatrix).
// fp32 caches (the reference's layout): each warp takes 4 or 8 tokens at a time, uses every row for all query
// heads of the group, reduces the per-lane partial dot products with a transposing butterfly (one value per
// lane instead of one reduction per value); online-softmax state (m, l, acc) per query head in fp32 throughout.
// The splits of one (sequence, head group) form a
// thread-block cluster: each block pushes slice j of its partial into block j's shared memory (distributed
// shared memory stores) and, after one cluster barrier, every block merges its slice of the head dimension
// locally -- no global round trip, no atomics, a fixed merge order.
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
#include <cuda.h>
#include <string.h>

#include "vb_kernels.cuh"
#include "vb_tma.cuh"

namespace cg = cooperative_groups;

namespace vb {

constexpr int ATTN_WARPS = 8;
// tensor-core path: probabilities as fp16 hi + lo (two products) or rounded once.  Rounded once is 1 % faster at batch 32
// (the legacy tensor path takes ~64 clocks per mma.sync per scheduler: a 16-token tile is 32 of them) and moves the
// full-depth logits from 0.0149 to 0.0160 of the checker's: the two products stay
constexpr bool ATTN_SPLIT_P = true;
constexpr int ATTN_MAX_SPLITS = 8;  // portable thread-block cluster size
constexpr int ATTN_SPEC_BLOCKS = ATTN_WARPS * 32;  // block-table rows up to this long are fetched whole, before the position is known

struct AttnKArgs {
    AttnArgs a;
    float scale;
    uint32_t G;          // query heads per KV head
    uint32_t g_chunks;   // ceil(G / GM), GM = query heads a block handles at once
    uint32_t n_splits;
    size_t kv_batch_stride;  // contiguous: elements between sequences
    uint32_t inv_freq_n;     // > 0: the rotary frequencies below are valid
    float inv_freq[256];     // [D/2], in parameter space: no memory trip before the angles can be computed
    alignas(64) CUtensorMap kv_map;  // tensor-core path: the paged pool as [token rows][D]
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


// ---- fp16 tensor-core helpers (m16n8k16) -----------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t r[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t r[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_f16_16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ float half_round(float v) { return __half2float(__float2half_rn(v)); }
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// ---- tcgen05 helpers of the head_dim-128 path (tokens are the M dimension) ---------------------------------------------
// instruction descriptors, kind::f16 with fp16 operands (format 0), fp32 accumulate, M 128 (8 << 24), N 16 (2 << 17);
// bit 15: A is MN-major (V is stored [token][dimension]: the dimensions are M, the tokens K)
constexpr uint32_t AT_IDESC_S = (1u << 4) | (2u << 17) | (8u << 24);
constexpr uint32_t AT_IDESC_O = (1u << 4) | (1u << 15) | (2u << 17) | (8u << 24);
__device__ __forceinline__ uint64_t at_desc_k_sw128(uint32_t addr) {  // K-major, rows of 128 bytes, 8-row groups 1024 bytes apart
    return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t at_desc_mn_sw128(uint32_t addr, uint32_t lbo) {  // MN-major: 64 elements of M per 128-byte row, next 64 `lbo` bytes on
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t at_desc_k_plain(uint32_t addr, uint32_t lbo, uint32_t sbo) {  // K-major core matrices of 8 rows x 16 bytes
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
__device__ __forceinline__ void at_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void at_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void at_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_ld16(uint32_t taddr, float r[16]) {
    uint32_t u[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]), "=r"(u[9]),
                   "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ __forceinline__ void at_st16(uint32_t taddr, const float r[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])), "r"(__float_as_uint(r[2])), "r"(__float_as_uint(r[3])),
                   "r"(__float_as_uint(r[4])), "r"(__float_as_uint(r[5])), "r"(__float_as_uint(r[6])), "r"(__float_as_uint(r[7])),
                   "r"(__float_as_uint(r[8])), "r"(__float_as_uint(r[9])), "r"(__float_as_uint(r[10])), "r"(__float_as_uint(r[11])),
                   "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])), "r"(__float_as_uint(r[14])), "r"(__float_as_uint(r[15]))
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Shared-memory plan of one block (dynamic): K/V staging for two chunks of CH tokens, the warp-merge buffer.
template <typename KVT, int EPL, int GM, int MMA>
struct AttnSmem {
    static constexpr int D = EPL * 32;
    // staged row stride in elements: the tensor-core path pads rows by 16 bytes so that the 8 rows of an
    // ldmatrix tile fall into different banks
    static constexpr int RS = D;
    // Tensor-core path: a staged chunk is [K|V][64-column half][CH tokens][128 bytes] with the 128-byte swizzle (what a
    // tiled TMA copy of [16 tokens][64 columns] writes): the 16-byte piece c of row r sits at piece c ^ (r & 7), so the 8
    // rows of an ldmatrix tile fall into different banks without padding, and one copy moves a KV block's 16 rows.
    static constexpr int HALVES = D / 64;
    // tokens per staged chunk: K+V of a chunk take at most 32 KB, at most 64 tokens; tensor-core path: up to 64 KB and
    // 128 tokens, a 16-token tile for each of the 8 warps (with 64 only four warps had work between two block-wide
    // barriers: batch 1 went 1.349 -> 1.300 ms per token, batch 32 3.55 -> 3.46 ms per step)
    static constexpr int CH_CAP = MMA ? 128 : 64;
    static constexpr int CH_FIT = (MMA ? 32768 : 16384) / (D * (int)sizeof(KVT));
    static constexpr int CH = CH_FIT > CH_CAP ? CH_CAP : CH_FIT;
    static constexpr size_t kv_bytes = (size_t)2 * 2 * CH * RS * sizeof(KVT);  // [buffer][K|V][CH][RS]
    static constexpr size_t acc_bytes = (size_t)ATTN_WARPS * GM * D * sizeof(float);
    // tensor-core paths: staging aligned to 1024 bytes; tcgen05 path: + the Q and P operands (4 KB each)
    static constexpr size_t total = kv_bytes + acc_bytes + (MMA ? 1024 : 0) + (MMA == 2 ? 8192 : 0);
};

template <typename KVT, int EPL, int GM, int MMA>
__global__ void __launch_bounds__(ATTN_WARPS * 32) k_attn_split(const __grid_constant__ AttnKArgs ka) {
    const AttnArgs& a = ka.a;
    using SM = AttnSmem<KVT, EPL, GM, MMA>;
    constexpr int D = EPL * 32, CH = SM::CH, RS = SM::RS;
    static_assert(!MMA || (sizeof(KVT) == 2 && D % 64 == 0), "the tensor-core path reads an fp16 cache in 64-column halves");
    constexpr int HV = MMA ? SM::HALVES : 1;
    constexpr int TCH = MMA ? 1 : ((EPL >= 8) ? 2 : ((GM >= 8) ? 4 : 8));  // scalar path: tokens a warp handles at once
    constexpr int NV = TCH * GM;                              // partial dot products per lane (<= 32)
    constexpr int ROW16 = D * sizeof(KVT) / 16;               // 16-byte pieces per K or V row
    static_assert(NV <= 32 && (NV & (NV - 1)) == 0, "values per lane must be a power of two <= 32");
    __shared__ float q_s[GM][D];
    __shared__ float sc_s[MMA ? 1 : ATTN_WARPS][32];   // scalar path: a warp's scores
    __shared__ float part_ml[ATTN_WARPS][GM][2];
    __shared__ float gath[GM * (D + 32)];   // partials of all splits for this block's slice of the head dimension
    __shared__ float rope_cs[D / 2], rope_sn[D / 2];
    __shared__ __align__(8) unsigned long long kv_bar[2];  // one transaction barrier per staging buffer
    __shared__ int32_t blk_s[ATTN_SPEC_BLOCKS];             // the sequence's block-table row (short tables only)
    __shared__ __align__(16) KVT new_kv[2][D];  // the appended token's K and V (fused mode)
    __shared__ __align__(8) unsigned long long tc_bar[2];  // tcgen05 path: S ready, P . V done (one completion per chunk each)
    __shared__ uint32_t tc_tmem_slot;
    __shared__ float tc_red[4][8];                          // per-warp maxima / sums of the 128 token rows
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    unsigned char* dyn_base = MMA ? dyn_smem + ((1024u - (smem_u32(dyn_smem) & 1023u)) & 1023u) : dyn_smem;
    KVT* kv_s = reinterpret_cast<KVT*>(dyn_base);
    float* part_acc = reinterpret_cast<float*>(dyn_base + SM::kv_bytes);  // [ATTN_WARPS][GM][D]
    // tensor-core path: until the warps' partials are written there (after the last chunk's barrier), the same bytes hold
    // the low halves of Q (q - fp16(q)) as B fragments, the same for every warp: [k step][lane], 16 * D bytes
    uint2* qlo_s = reinterpret_cast<uint2*>(part_acc);
    // tcgen05 path: the B operands, [q_hi (8 heads) | q_lo (8 heads)] as 16 rows x 128 dimensions (two 64-column halves, 128-byte
    // swizzle) and [p_hi | p_lo] as 16 rows x 128 tokens (core matrices of 8 rows x 16 bytes)
    unsigned char* qop = dyn_base + SM::kv_bytes + SM::acc_bytes;
    unsigned char* pop = qop + 4096;

    trace_mark(a.trace, 0);
    pdl_launch_dependents();

    // ---- before the wait: nothing here depends on this step's projections.  The sequence's position (written
    // by the previous step's sampler), the block table, the rotary angles and -- the long trip -- the first
    // chunk of cached K/V rows are all on their way while the QKV product is still finishing.
    const uint32_t b = blockIdx.z, split = blockIdx.y;
    const uint32_t kvh = blockIdx.x / ka.g_chunks, gc = blockIdx.x % ka.g_chunks;
    const uint32_t g0 = gc * GM;
    const uint32_t ng = min((uint32_t)GM, ka.G - g0);
    // the sequence's whole block-table row is requested together with its position when it is short enough
    const bool spec_table = a.block_table && a.max_blocks <= (uint32_t)ATTN_SPEC_BLOCKS;
    int32_t my_blk = 0;
    if (spec_table && threadIdx.x < a.max_blocks) my_blk = a.block_table[(size_t)b * a.max_blocks + threadIdx.x];
    if (a.state && !a.state[b].active) return;
    const uint32_t seq_len = (a.state ? a.state[b].pos : a.pos) + 1;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // the context is cut into n_splits equal slices of whole KV blocks, whatever its current length
    uint32_t per = (seq_len + ka.n_splits - 1) / ka.n_splits;
    per = ((per + a.block_tokens - 1) / a.block_tokens) * a.block_tokens;
    const uint32_t t_lo = min(seq_len, split * per), t_hi = min(seq_len, t_lo + per);
    const uint32_t pos = seq_len - 1;
    const bool appender = a.qkv_raw && t_lo <= pos && pos < t_hi;
    // every block of the cluster must be running before anyone writes into its shared memory: arrive now,
    // wait just before the pushes (the barrier's latency hides behind the attention itself)
    cg::cluster_group cluster = cg::this_cluster();
    cluster.barrier_arrive();
    // tensor-core path: S^T = K Q^T (16 tokens x 8 heads per mma) and O^T = V^T P^T (16 dims x 8 heads), so the
    // query heads are the N = 8 columns: no padding for a group of 8, and each thread's accumulator columns are the
    // two heads (2 * (lane & 3), +1) whose running maximum it tracks
    constexpr int MT = D / 16;
    float o_t[MMA ? MT : 1][4];
    float m2[2] = {-INFINITY, -INFINITY}, l2[2] = {0.0f, 0.0f};
    // tcgen05 path: running maximum in use and this thread's share of the sums, per head (threads 0..127 = token rows)
    float tc_m[MMA == 2 ? 8 : 1], tc_l[MMA == 2 ? 8 : 1];
#pragma unroll
    for (int h = 0; h < (MMA == 2 ? 8 : 1); ++h) { tc_m[h] = -INFINITY; tc_l[h] = 0.0f; }
#pragma unroll
    for (int i = 0; i < (MMA ? MT : 1); ++i) { o_t[i][0] = 0.0f; o_t[i][1] = 0.0f; o_t[i][2] = 0.0f; o_t[i][3] = 0.0f; }
    float m[GM], l[GM], acc[GM][EPL];
#pragma unroll
    for (int g = 0; g < GM; ++g) {
        m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = 0.0f;
    }

    // Chunk c = tokens [t_lo + c*CH, +CH) of the slice, fetched by bulk copies (TMA) into buffer c & 1 and
    // announced on that buffer's transaction barrier.  Scalar path on the paged pool: one copy moves the 16 cached
    // rows of a KV block (K or V) for this head.  Tensor-core path (rows padded in shared memory) and contiguous
    // layout: one copy per row.  Each copy is issued by a different thread of the block.
    // Called by the whole block; `rot` rotates the threads so that two chunks requested back to back use
    // different ones (their block-table reads then overlap instead of queueing behind one another).
    auto stage_chunk = [&](uint32_t c, uint32_t buf, uint32_t rot) {
        const uint32_t c0 = t_lo + c * CH;
        const uint32_t n_tok = min((uint32_t)CH, t_hi - c0);
        KVT* kb = kv_s + (size_t)buf * 2 * CH * RS;
        const uint32_t bar = smem_u32(&kv_bar[buf]);
        const uint32_t NT = ATTN_WARPS * 32;
        const uint32_t me = (threadIdx.x + NT - rot) % NT;
        const uint32_t row_bytes = D * (uint32_t)sizeof(KVT);
        if constexpr (MMA) {
            // one tiled copy per (KV block, K or V, 64-column half): 16 rows of 128 bytes, swizzled
            const uint32_t nb = (n_tok + 15u) / 16u;
            if (me == 0) mbar_expect_tx(bar, nb * 2 * HV * 2048u);
            for (uint32_t i = me; i < nb * 2 * HV; i += NT) {
                const uint32_t h = i % HV, kv = (i / HV) & 1, j = i / (2 * HV);
                const uint32_t bi = c0 / 16u + j;
                const int32_t blk = spec_table ? blk_s[bi] : a.block_table[(size_t)b * a.max_blocks + bi];
                const int y = (int)(a.kv_map_row0 + (((uint32_t)blk * 2 + kv) * a.Hkv + kvh) * 16u);
                const uint32_t dst = smem_u32(kb) + ((kv * HV + h) * CH + j * 16u) * 128u;
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                             ::"r"(dst), "l"(&ka.kv_map), "r"((int)(h * 64u)), "r"(y), "r"(bar) : "memory");
            }
        } else if (a.block_table) {
            const uint32_t nb = (n_tok + a.block_tokens - 1) / a.block_tokens;
            const uint32_t blk_bytes = a.block_tokens * row_bytes;
            if (me == 0) mbar_expect_tx(bar, nb * 2 * blk_bytes);
            for (uint32_t i = me; i < nb * 2; i += NT) {
                const uint32_t kv = i & 1, j = i >> 1;
                const uint32_t bi = c0 / a.block_tokens + j;
                const int32_t blk = spec_table ? blk_s[bi] : a.block_table[(size_t)b * a.max_blocks + bi];
                const KVT* src = reinterpret_cast<const KVT*>(a.k) + (((size_t)blk * 2 + kv) * a.Hkv + kvh) * a.block_tokens * D;
                tma_load_1d(smem_u32(kb + ((size_t)kv * CH + (size_t)j * a.block_tokens) * RS), src, blk_bytes, bar);
            }
        } else {
            // one copy per row: the contiguous layout has no larger unit
            if (me == 0) mbar_expect_tx(bar, n_tok * 2 * row_bytes);
            for (uint32_t i = me; i < n_tok * 2; i += NT) {
                const uint32_t kv = i & 1, tok = i >> 1, tt = c0 + tok;
                const KVT* src;
                if (a.block_table) {
                    const uint32_t bi = tt / a.block_tokens;
                    const int32_t blk = spec_table ? blk_s[bi] : a.block_table[(size_t)b * a.max_blocks + bi];
                    src = reinterpret_cast<const KVT*>(a.k) + (((size_t)blk * 2 + kv) * a.Hkv + kvh) * a.block_tokens * D +
                          (size_t)(tt % a.block_tokens) * D;
                } else {
                    src = reinterpret_cast<const KVT*>(kv ? a.v : a.k) + (size_t)b * ka.kv_batch_stride + (size_t)tt * a.Hkv * D + (size_t)kvh * D;
                }
                tma_load_1d(smem_u32(kb + ((size_t)kv * CH + tok) * RS), src, row_bytes, bar);
            }
        }
    };

    const bool has_tokens = t_lo < t_hi;
    const uint32_t n_ch = has_tokens ? (t_hi - t_lo + CH - 1) / CH : 0;
    // In fused mode the cached rows are older than this step (the new token's row is patched in from new_kv
    // below), so they may be fetched now; otherwise the kernel before this one wrote the newest row.
    const bool early = a.qkv_raw != nullptr;
    constexpr uint32_t half = D / 2;
    constexpr int QIT = (GM * (int)half + ATTN_WARPS * 32 - 1) / (ATTN_WARPS * 32);  // (head, pair) items per thread
    float bq1[QIT], bq2[QIT], bk1 = 0.f, bk2 = 0.f, bv1 = 0.f, bv2 = 0.f;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&kv_bar[0]), 1);
        mbar_init(smem_u32(&kv_bar[1]), 1);
        if constexpr (MMA == 2) { mbar_init(smem_u32(&tc_bar[0]), 1); mbar_init(smem_u32(&tc_bar[1]), 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if constexpr (MMA == 2) {
        if (warp == 1) {  // 32 columns of tensor memory: S^T (16) and O^T (16)
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tc_tmem_slot)), "r"(32) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        at_fence_before();
    }
    if (spec_table) blk_s[threadIdx.x] = my_blk;
    __syncthreads();  // barriers initialised, block table in place
    uint32_t tmem = 0;
    if constexpr (MMA == 2) { at_fence_after(); tmem = tc_tmem_slot; }
    if (early) {
        // the requests for the first two chunks, spread over the block (one copy per thread or fewer)
        if (n_ch > 0) stage_chunk(0, 0, 0);
        if (n_ch > 1) stage_chunk(1, 1, ATTN_WARPS * 16);
    }
    if (a.qkv_raw && warp != 0) {
        // rotary angles of this position (one sincos per frequency, shared by all heads)
        for (uint32_t j = threadIdx.x - 32; j < half; j += (ATTN_WARPS - 1) * 32) {
            float sn, cs;
            sincosf((float)pos * (ka.inv_freq_n ? ka.inv_freq[j] : a.rope_inv_freq[j]), &sn, &cs);
            rope_cs[j] = cs;
            rope_sn[j] = sn;
        }
    }
    if (a.qkv_raw) {
        // biases are weights: they can be in registers before the projections exist
#pragma unroll
        for (int it = 0; it < QIT; ++it) {
            const uint32_t i = threadIdx.x + it * ATTN_WARPS * 32, g = i / half, j = i % half;
            const uint32_t h = kvh * ka.G + g0 + g;
            const bool on = a.bq && i < GM * half && g < ng;
            bq1[it] = on ? bias_at(a.bq, a.bias_fmt, h * D + j) : 0.0f;
            bq2[it] = on ? bias_at(a.bq, a.bias_fmt, h * D + j + half) : 0.0f;
        }
        if (appender && threadIdx.x < half) {
            const uint32_t j = threadIdx.x;
            if (a.bk) { bk1 = bias_at(a.bk, a.bias_fmt, kvh * D + j); bk2 = bias_at(a.bk, a.bias_fmt, kvh * D + j + half); }
            if (a.bv) { bv1 = bias_at(a.bv, a.bias_fmt, kvh * D + j); bv2 = bias_at(a.bv, a.bias_fmt, kvh * D + j + half); }
        }
    }
    __syncthreads();

    pdl_wait();
    trace_mark(a.trace, 1);
    if (!early) {
        if (n_ch > 0) stage_chunk(0, 0, 0);
        if (n_ch > 1) stage_chunk(1, 1, ATTN_WARPS * 16);
    }

    if (has_tokens) {
        if (a.qkv_raw) {
            // fused bias + RoPE on the raw projections: all loads first, then the arithmetic
            const float* raw = a.qkv_raw + (size_t)b * (a.Hq + 2 * a.Hkv) * D;
            float x1[QIT], x2[QIT], k1 = 0.f, k2 = 0.f, v1 = 0.f, v2 = 0.f;
#pragma unroll
            for (int it = 0; it < QIT; ++it) {
                const uint32_t i = threadIdx.x + it * ATTN_WARPS * 32, g = i / half, j = i % half;
                const uint32_t h = kvh * ka.G + g0 + g;
                const bool on = i < GM * half && g < ng;
                x1[it] = on ? raw[(size_t)h * D + j] : 0.0f;
                x2[it] = on ? raw[(size_t)h * D + j + half] : 0.0f;
            }
            const bool kv_thread = appender && threadIdx.x < half;
            if (kv_thread) {
                const float* kr_raw = raw + (size_t)a.Hq * D + (size_t)kvh * D;
                const float* vr_raw = raw + (size_t)(a.Hq + a.Hkv) * D + (size_t)kvh * D;
                const uint32_t j = threadIdx.x;
                k1 = kr_raw[j]; k2 = kr_raw[j + half]; v1 = vr_raw[j]; v2 = vr_raw[j + half];
            }
#pragma unroll
            for (int it = 0; it < QIT; ++it) {
                const uint32_t i = threadIdx.x + it * ATTN_WARPS * 32, g = i / half, j = i % half;
                if (i < GM * half) {
                    const float a1 = x1[it] + bq1[it], a2 = x2[it] + bq2[it];
                    const float sn = rope_sn[j], cs = rope_cs[j];
                    const bool on = g < ng;
                    q_s[g][j] = on ? a1 * cs - a2 * sn : 0.0f;
                    q_s[g][j + half] = on ? a2 * cs + a1 * sn : 0.0f;
                }
            }
            if (kv_thread) {
                const uint32_t j = threadIdx.x;
                const float a1 = k1 + bk1, a2 = k2 + bk2;
                const float sn = rope_sn[j], cs = rope_cs[j];
                new_kv[0][j] = (KVT)__float2half_rn(a1 * cs - a2 * sn);
                new_kv[0][j + half] = (KVT)__float2half_rn(a2 * cs + a1 * sn);
                new_kv[1][j] = (KVT)__float2half_rn(v1 + bv1);
                new_kv[1][j + half] = (KVT)__float2half_rn(v2 + bv2);
            }
        } else {
            const float* qb = a.q + (size_t)b * a.Hq * D + (size_t)(kvh * ka.G + g0) * D;
            for (uint32_t i = threadIdx.x; i < GM * D; i += blockDim.x) q_s[i / D][i % D] = (i < ng * D) ? qb[i] : 0.0f;
        }
        __syncthreads();
        if (appender && gc == 0 && !(a.state && a.state[b].limit && pos >= a.state[b].limit)) {
            // the new token's row goes to the cache (16-byte stores); this block reads it from new_kv below
            // (never outside the slot's reservation: the sampler deactivates a slot before that can happen)
            const int32_t blk = spec_table ? blk_s[pos / a.block_tokens] : a.block_table[(size_t)b * a.max_blocks + pos / a.block_tokens];
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
            for (int e = 0; e < EPL; ++e) qr[g][e] = MMA ? 0.0f : q_s[g][lane * EPL + e];
        // Q^T as B fragments (k = head dimension, n = query head), fp16
        uint32_t qb[MMA == 1 ? MT : 1][2];
        if constexpr (MMA == 2) {
            // the B operand of S^T = K . Q^T: rows 0..7 = fp16(q) of the group's heads, rows 8..15 = q - fp16(q): the split of Q
            // costs no extra instruction (N = 16 is the smallest tile anyway)
            for (uint32_t i = threadIdx.x; i < 16 * (D / 2); i += blockDim.x) {
                const uint32_t n = i / (D / 2), d = 2 * (i % (D / 2)), g = n & 7;
                float v0 = 0.0f, v1 = 0.0f;
                if (g < (uint32_t)GM) {
                    v0 = q_s[g][d]; v1 = q_s[g][d + 1];
                    if (n >= 8) { v0 -= half_round(v0); v1 -= half_round(v1); }
                }
                *reinterpret_cast<uint32_t*>(qop + (d >> 6) * 2048 + n * 128 + ((((d & 63) >> 3) ^ (n & 7)) << 4) + (d & 7) * 2) = pack_half2(v0, v1);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
        }
        if constexpr (MMA == 1) {
            const uint32_t n = lane >> 2, k0 = 2 * (lane & 3);
#pragma unroll
            for (int ks = 0; ks < MT; ++ks) {
                const bool on = n < (uint32_t)GM;
                const float* qrow = q_s[on ? n : 0];
                const float q0 = on ? qrow[ks * 16 + k0] : 0.0f, q1 = on ? qrow[ks * 16 + k0 + 1] : 0.0f;
                const float q8 = on ? qrow[ks * 16 + k0 + 8] : 0.0f, q9 = on ? qrow[ks * 16 + k0 + 9] : 0.0f;
                qb[ks][0] = pack_half2(q0, q1);
                qb[ks][1] = pack_half2(q8, q9);
                // Q and the probabilities go through the fp16 tensor cores as a high and a low half each (two products
                // into the same fp32 accumulators): with one half alone their 11-bit rounding, amplified over 32 layers,
                // moved the logits as much as the fp16 cache itself does.  The low halves of Q wait in shared memory.
                if (warp == 0)
                    qlo_s[ks * 32 + lane] = make_uint2(pack_half2(q0 - half_round(q0), q1 - half_round(q1)),
                                                       pack_half2(q8 - half_round(q8), q9 - half_round(q9)));
            }
            __syncthreads();
        }

        // ---- the slice, CH tokens at a time through the two buffers (both were requested above) ----------------
        for (uint32_t c = 0; c < n_ch; ++c) {
            const uint32_t c0 = t_lo + c * CH, buf = c & 1;
            if (!mbar_wait(smem_u32(&kv_bar[buf]), (c >> 1) & 1) && a.err) atomicOr(a.err, 0x400u);
            KVT* kb = kv_s + (size_t)buf * 2 * CH * RS;
            const uint32_t c_hi = min(t_hi, c0 + CH);
            if constexpr (MMA) {
                // the copies moved whole KV blocks: rows past the context's end hold whatever the pool held (they are
                // multiplied with probability 0 and must be numbers), and the new token's row is older than this step
                const bool patch = appender && c0 <= pos && pos < c0 + CH;
                const uint32_t n_valid = c_hi - c0, n_landed = (n_valid + 15u) & ~15u;
                if (patch || n_valid != n_landed) {
                    for (uint32_t i = threadIdx.x; i < (n_landed - n_valid) * 2 * ROW16; i += blockDim.x) {
                        const uint32_t piece = i % ROW16, rowi = i / ROW16, kv = rowi & 1, r = n_valid + (rowi >> 1);
                        reinterpret_cast<uint4*>(kb + ((size_t)(kv * HV + (piece >> 3)) * CH + r) * 64)[piece & 7] = make_uint4(0, 0, 0, 0);
                    }
                    if (patch) {
                        const uint32_t r = pos - c0;
                        for (uint32_t i = threadIdx.x; i < 2 * ROW16; i += blockDim.x) {
                            const uint32_t kv = i / ROW16, piece = i % ROW16;
                            reinterpret_cast<uint4*>(kb + ((size_t)(kv * HV + (piece >> 3)) * CH + r) * 64)[(piece & 7) ^ (r & 7)] =
                                reinterpret_cast<const uint4*>(new_kv[kv])[piece];
                        }
                    }
                    if constexpr (MMA == 2) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // read by the tensor core
                    __syncthreads();
                }
            } else if (appender && c0 <= pos && pos < c0 + CH) {
                // overwrite the staged copy of the new token's row with the values just computed
                for (uint32_t i = threadIdx.x; i < 2 * ROW16; i += blockDim.x) {
                    const uint32_t kv = i / ROW16, piece = i % ROW16;
                    reinterpret_cast<uint4*>(kb + ((size_t)kv * CH + (pos - c0)) * RS)[piece] = reinterpret_cast<const uint4*>(new_kv[kv])[piece];
                }
                __syncthreads();
            }
            if constexpr (MMA == 2) {
                const uint32_t n_valid = c_hi - c0, n_landed = (n_valid + 15u) & ~15u;
                // ---- S^T[128 tokens x 16] = K . [q_hi | q_lo]^T : D / 16 instructions from one thread --------------------------
                const uint32_t s_bar = smem_u32(&tc_bar[0]), o_bar = smem_u32(&tc_bar[1]);
                if (threadIdx.x == 0) {
                    at_fence_after();
                    const uint32_t kbase = smem_u32(kb), qbase = smem_u32(qop);
#pragma unroll
                    for (int ks = 0; ks < MT; ++ks)
                        at_mma(tmem, at_desc_k_sw128(kbase + (ks >> 2) * (CH * 128u) + (ks & 3) * 32u),
                               at_desc_k_sw128(qbase + (ks >> 2) * 2048u + (ks & 3) * 32u), AT_IDESC_S, ks != 0 ? 1u : 0u);
                    at_commit(s_bar);
                }
                if (warp < 4) {
                    // ---- softmax: thread = token row = tensor-memory lane ------------------------------------------------------
                    const uint32_t lane_addr = (warp * 32u) << 16, tok = threadIdx.x;
                    const bool ok = __all_sync(0xFFFFFFFFu, mbar_wait(s_bar, c & 1));
                    if (!ok && a.err && lane == 0) atomicOr(a.err, 0x800u);
                    at_fence_after();
                    float sv[16];
                    at_ld16(tmem + lane_addr, sv);
                    const bool valid = tok < n_valid;
                    float s8[8], mx[8];
#pragma unroll
                    for (int h = 0; h < 8; ++h) { s8[h] = valid ? (sv[h] + sv[8 + h]) * ka.scale : -INFINITY; mx[h] = s8[h]; }
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1)
#pragma unroll
                        for (int h = 0; h < 8; ++h) mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xFFFFFFFFu, mx[h], off));
#pragma unroll
                    for (int h = 0; h < 8; ++h)
                        if (lane == (uint32_t)h) tc_red[warp][h] = mx[h];   // (every lane holds all eight maxima)
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    float alpha[8];
                    bool moved = false;
#pragma unroll
                    for (int h = 0; h < 8; ++h) {
                        const float cm = fmaxf(fmaxf(tc_red[0][h], tc_red[1][h]), fmaxf(tc_red[2][h], tc_red[3][h]));
                        const float mn = fmaxf(tc_m[h], cm);  // finite: every chunk has a live token
                        alpha[h] = (tc_m[h] == -INFINITY) ? 0.0f : __expf(tc_m[h] - mn);
                        moved = moved || (mn != tc_m[h]);
                        tc_m[h] = mn;
                    }
                    // [p_hi | p_lo] as the K-major B operand of O^T = V^T . P^T: row n, token k at (n / 8) * 2048 + (k / 8) * 128 +
                    // (n % 8) * 16 + (k % 8) * 2
                    unsigned char* prow = pop + (tok >> 3) * 128 + (tok & 7) * 2;
#pragma unroll
                    for (int h = 0; h < 8; ++h) {
                        const float pv_ = valid ? __expf(s8[h] - tc_m[h]) : 0.0f;
                        tc_l[h] = fmaf(tc_l[h], alpha[h], pv_);
                        const __half ph = __float2half_rn(pv_);
                        *reinterpret_cast<__half*>(prow + h * 16) = ph;
                        *reinterpret_cast<__half*>(prow + 2048 + h * 16) = __float2half_rn(pv_ - __half2float(ph));
                    }
                    if (c > 0 && moved) {
                        // the maximum in use moved (the same decision in every thread): scale O^T, this thread = dimension `tok`
                        float o[16];
                        at_ld16(tmem + lane_addr + 16, o);
#pragma unroll
                        for (int j = 0; j < 16; ++j) o[j] *= alpha[j & 7];
                        at_st16(tmem + lane_addr + 16, o);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    at_fence_before();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                }
                if (threadIdx.x == 0) {
                    // ---- O^T[128 dimensions x 16] += V^T . [p_hi | p_lo]^T : one instruction per 16 tokens ------------------------
                    at_fence_after();
                    const uint32_t vbase = smem_u32(kb) + HV * (CH * 128u), pbase = smem_u32(pop);
                    for (uint32_t kk = 0; kk < n_landed / 16u; ++kk)
                        at_mma(tmem + 16, at_desc_mn_sw128(vbase + kk * 2048u, CH * 128u), at_desc_k_plain(pbase + kk * 256u, 128u, 2048u),
                               AT_IDESC_O, (c | kk) != 0 ? 1u : 0u);
                    at_commit(o_bar);
                }
                // the staging buffer, the P operand and S^T are free again once that product is done
                if (!mbar_wait(o_bar, c & 1) && a.err) atomicOr(a.err, 0x1000u);
                at_fence_after();
            } else if constexpr (MMA) {
                const uint32_t n_tiles = (c_hi - c0 + 15) / 16;
                const uint32_t mi = lane >> 3, r8 = lane & 7;
                for (uint32_t tile = warp; tile < n_tiles; tile += ATTN_WARPS) {
                    const uint32_t tok0 = tile * 16;
                    // scores of 16 tokens x 8 heads
                    float sc4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    // row (tok0 + (mi & 1) * 8 + r8) of K, 16-byte piece q = 2 * ks + (mi >> 1) of its D / 8: half q >> 3,
                    // piece (q & 7) ^ r8 of the 128-byte row
                    const uint32_t k_row = smem_u32(kb) + (tok0 + (mi & 1) * 8 + r8) * 128u;
#pragma unroll
                    for (int ks = 0; ks < MT; ++ks) {
                        uint32_t af[4];
                        const uint32_t q = 2u * ks + (mi >> 1);
                        ldsm_x4(af, k_row + (q >> 3) * (CH * 128u) + (((q & 7u) ^ r8) << 4));
                        const uint2 ql = qlo_s[ks * 32 + lane];
                        mma_f16_16816(sc4, af, qb[ks][0], qb[ks][1]);
                        mma_f16_16816(sc4, af, ql.x, ql.y);
                    }
                    // this thread: tokens tA = lane / 4 and tA + 8 of the tile, heads 2 * (lane & 3) and + 1
                    const uint32_t tA = c0 + tok0 + (lane >> 2);
                    const bool vA = tA < c_hi, vB = tA + 8 < c_hi;
                    const float s0 = vA ? sc4[0] * ka.scale : -INFINITY, s1 = vA ? sc4[1] * ka.scale : -INFINITY;
                    const float s2 = vB ? sc4[2] * ka.scale : -INFINITY, s3 = vB ? sc4[3] * ka.scale : -INFINITY;
                    float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
#pragma unroll
                    for (int off = 4; off < 32; off <<= 1) {
                        mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, off));
                        mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, off));
                    }
                    const float nm0 = fmaxf(m2[0], mx0), nm1 = fmaxf(m2[1], mx1);
                    const float al0 = (m2[0] == -INFINITY) ? 0.0f : __expf(m2[0] - nm0);
                    const float al1 = (m2[1] == -INFINITY) ? 0.0f : __expf(m2[1] - nm1);
                    const float p0 = (nm0 == -INFINITY) ? 0.0f : __expf(s0 - nm0), p2 = (nm0 == -INFINITY) ? 0.0f : __expf(s2 - nm0);
                    const float p1 = (nm1 == -INFINITY) ? 0.0f : __expf(s1 - nm1), p3 = (nm1 == -INFINITY) ? 0.0f : __expf(s3 - nm1);
                    l2[0] = fmaf(l2[0], al0, p0 + p2);
                    l2[1] = fmaf(l2[1], al1, p1 + p3);
                    m2[0] = nm0; m2[1] = nm1;
                    // P^T as B fragments (k = token, n = head): transpose the two 8x8 halves of the score tile
                    const uint32_t pb0 = movmatrix_trans(pack_half2(p0, p1));
                    const uint32_t pb1 = movmatrix_trans(pack_half2(p2, p3));
                    const uint32_t pl0 = movmatrix_trans(pack_half2(p0 - half_round(p0), p1 - half_round(p1)));
                    const uint32_t pl1 = movmatrix_trans(pack_half2(p2 - half_round(p2), p3 - half_round(p3)));
                    const uint32_t v_row = smem_u32(kb) + HV * (CH * 128u) + (tok0 + (mi >> 1) * 8 + r8) * 128u;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        o_t[mt][0] *= al0; o_t[mt][2] *= al0; o_t[mt][1] *= al1; o_t[mt][3] *= al1;
                        uint32_t af[4];
                        const uint32_t q = 2u * mt + (mi & 1);
                        ldsm_x4_trans(af, v_row + (q >> 3) * (CH * 128u) + (((q & 7u) ^ r8) << 4));
                        mma_f16_16816(o_t[mt], af, pb0, pb1);
                        if constexpr (ATTN_SPLIT_P) mma_f16_16816(o_t[mt], af, pl0, pl1);
                    }
                }
            } else
            for (uint32_t t0 = c0 + warp * TCH; t0 < c_hi; t0 += ATTN_WARPS * TCH) {
                float kr[TCH][EPL], vr[TCH][EPL];
#pragma unroll
                for (int i = 0; i < TCH; ++i) {
                    const uint32_t tok = min(t0 + i, c_hi - 1) - c0;  // out-of-range tokens re-read the last row, masked below
                    load_row<KVT, EPL>(kb + (size_t)tok * RS, lane, kr[i]);
                    load_row<KVT, EPL>(kb + ((size_t)CH + tok) * RS, lane, vr[i]);
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
            __syncthreads();  // every warp is done with the buffer: it takes the chunk after next
            if (c + 2 < n_ch) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                stage_chunk(c + 2, buf, 0);
            }
        }
    }

    // ---- merge the warps into this block's partial (m, l, unnormalised acc) ...
    if constexpr (MMA == 2) {
        // the whole block's result sits in tensor memory: it becomes "warp 0's" partial, the other warps contribute nothing
        for (uint32_t i = threadIdx.x; i < (ATTN_WARPS - 1) * GM * D; i += blockDim.x) part_acc[(size_t)GM * D + i] = 0.0f;
        if (threadIdx.x < (ATTN_WARPS - 1) * GM) { part_ml[1 + threadIdx.x / GM][threadIdx.x % GM][0] = -INFINITY; part_ml[1 + threadIdx.x / GM][threadIdx.x % GM][1] = 0.0f; }
        if (warp < 4) {
            float o[16];
            if (has_tokens) {
                at_fence_after();
                at_ld16(tmem + ((warp * 32u) << 16) + 16, o);   // O^T: this thread's dimension, columns = [hi | lo] heads
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) o[j] = 0.0f;
            }
#pragma unroll
            for (int h = 0; h < GM; ++h) part_acc[(size_t)h * D + threadIdx.x] = o[h] + o[8 + h];
            // sums of the probabilities: every thread holds those of its own token rows
            float ls[8];
#pragma unroll
            for (int h = 0; h < 8; ++h) ls[h] = has_tokens ? tc_l[h] : 0.0f;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
#pragma unroll
                for (int h = 0; h < 8; ++h) ls[h] += __shfl_xor_sync(0xFFFFFFFFu, ls[h], off);
#pragma unroll
            for (int h = 0; h < 8; ++h)
                if (lane == (uint32_t)h) tc_red[warp][h] = ls[h];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x < (uint32_t)GM) {
                const uint32_t h = threadIdx.x;
                part_ml[0][h][0] = has_tokens ? tc_m[h] : -INFINITY;
                part_ml[0][h][1] = (tc_red[0][h] + tc_red[1][h]) + (tc_red[2][h] + tc_red[3][h]);
            }
            at_fence_before();
        }
        __syncthreads();
        if (warp == 1) {
            at_fence_after();
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32) : "memory");
        }
    } else if constexpr (MMA) {
        // the 8 lanes that share lane & 3 hold partial sums of the same two heads
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l2[0] += __shfl_xor_sync(0xFFFFFFFFu, l2[0], off);
            l2[1] += __shfl_xor_sync(0xFFFFFFFFu, l2[1], off);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t h = 2 * (lane & 3) + i;
            if (h < (uint32_t)GM) {
                if (lane < 4) { part_ml[warp][h][0] = m2[i]; part_ml[warp][h][1] = l2[i]; }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    part_acc[((size_t)warp * GM + h) * D + mt * 16 + (lane >> 2)] = o_t[mt][i];
                    part_acc[((size_t)warp * GM + h) * D + mt * 16 + (lane >> 2) + 8] = o_t[mt][2 + i];
                }
            }
        }
    } else {
#pragma unroll
        for (int g = 0; g < GM; ++g) {
            if (lane == 0) { part_ml[warp][g][0] = m[g]; part_ml[warp][g][1] = l[g]; }
#pragma unroll
            for (int e = 0; e < EPL; ++e) part_acc[((size_t)warp * GM + g) * D + lane * EPL + e] = acc[g][e];
        }
    }
    __syncthreads();
    // ---- ... and push it to the blocks of the cluster (the splits of one sequence and head group): block j
    // merges slice j of the head dimension, so every value goes to exactly one block's shared memory.  One
    // cluster barrier later each block holds all it needs locally: no global round trip, no atomics, a fixed
    // merge order, and nobody reads remote memory after the barrier (blocks may leave at once).
    cluster.barrier_wait();
    const uint32_t n = ka.n_splits;  // == cluster size along y
    const uint32_t per_d = (D + n - 1) / n;
    const uint32_t gstride = per_d + 2;  // per (source split, head): M, L, per_d accumulators
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
        if (g < ng) {
            const uint32_t owner = d / per_d, dd = d - owner * per_d;
            float* dst = cluster.map_shared_rank(gath, owner) + ((size_t)split * GM + g) * gstride;
            dst[2 + dd] = A;
            if (dd == 0) { dst[0] = M; dst[1] = L; }
        }
    }
    cluster.sync();
    const uint32_t d_lo = split * per_d, d_hi = min((uint32_t)D, d_lo + per_d);
    for (uint32_t i = threadIdx.x; i < ng * per_d; i += blockDim.x) {
        const uint32_t g = i / per_d, dd = i % per_d, d = d_lo + dd;
        if (d < d_hi) {
            float M = -INFINITY;
            for (uint32_t r = 0; r < n; ++r) M = fmaxf(M, gath[((size_t)r * GM + g) * gstride]);
            float L = 0.0f, A = 0.0f;
            for (uint32_t r = 0; r < n; ++r) {
                const float* src = gath + ((size_t)r * GM + g) * gstride;
                const float f = (src[0] == -INFINITY) ? 0.0f : __expf(src[0] - M);
                L = fmaf(src[1], f, L);
                A = fmaf(src[2 + dd], f, A);
            }
            a.out[(size_t)b * a.Hq * D + (size_t)(kvh * ka.G + g0 + g) * D + d] = (L > 0.0f) ? (A / L) : 0.0f;
        }
    }
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

// head_dim 128 on the tensor-core path as tcgen05.mma (option "attn_tcgen05"): tokens are the M dimension, [q_hi | q_lo] and
// [p_hi | p_lo] the N = 16 columns (the hi/lo halves cost no instruction), S^T and O^T in tensor memory.  It gives the same
// results and 24 instead of 256 tensor-core instructions per 128-token chunk, but a chunk is then one serial chain of
// hand-overs (commit -> barrier -> tcgen05.ld -> cross-warp maximum -> P through shared memory and a proxy fence -> commit):
// measured 1.39 instead of 1.29 ms per token at batch 1 and 4.0 instead of 3.27 ms per step at batch 32.  Off by default.
bool attn_use_tcgen05 = false;
bool attn_use_mma = true;  // fp16 caches with head_dim <= 256: QK^T and PV on the tensor cores (option "attn_mma")

template <typename KVT, int EPL, int GM, int MMA>
static cudaError_t launch_split_g(const LaunchCfg& lc, AttnKArgs ka) {
    ka.g_chunks = (ka.G + GM - 1) / GM;
    const size_t smem = AttnSmem<KVT, EPL, GM, MMA>::total;
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
    return cudaLaunchKernelEx(&cfg, k_attn_split<KVT, EPL, GM, MMA>, ka);
}

template <typename KVT, int EPL>
static cudaError_t launch_split(const LaunchCfg& lc, const AttnKArgs& ka) {
    if constexpr (sizeof(KVT) == 2 && EPL >= 2 && EPL <= 8) {
        // tensor-core path: paged pool of 16-token blocks reachable through its tensor map
        if (attn_use_mma && ka.a.kv_map && ka.a.block_table && ka.a.block_tokens == 16) {
            if constexpr (EPL == 4) {
                if (attn_use_tcgen05) {  // head_dim 128: both products as tcgen05.mma with the tokens as the M dimension
                    if (ka.G == 1) return launch_split_g<KVT, EPL, 1, 2>(lc, ka);
                    if (ka.G == 2) return launch_split_g<KVT, EPL, 2, 2>(lc, ka);
                    if (ka.G <= 4) return launch_split_g<KVT, EPL, 4, 2>(lc, ka);
                    return launch_split_g<KVT, EPL, 8, 2>(lc, ka);
                }
            }
            if (ka.G == 1) return launch_split_g<KVT, EPL, 1, 1>(lc, ka);
            if (ka.G == 2) return launch_split_g<KVT, EPL, 2, 1>(lc, ka);
            if (ka.G <= 4) return launch_split_g<KVT, EPL, 4, 1>(lc, ka);
            return launch_split_g<KVT, EPL, 8, 1>(lc, ka);
        }
    }
    if constexpr (EPL >= 8) {
        return launch_split_g<KVT, EPL, 1, 0>(lc, ka);  // wide heads: one query head per block keeps registers in bounds
    } else {
        if (ka.G == 1) return launch_split_g<KVT, EPL, 1, 0>(lc, ka);
        if (ka.G == 2) return launch_split_g<KVT, EPL, 2, 0>(lc, ka);
        if (ka.G <= 4) return launch_split_g<KVT, EPL, 4, 0>(lc, ka);
        return launch_split_g<KVT, EPL, 8, 0>(lc, ka);
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
    cudaError_t e = cudaFuncSetAttribute(k_attn_split<KVT, EPL, GM, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)AttnSmem<KVT, EPL, GM, 0>::total);
    if constexpr (sizeof(KVT) == 2 && EPL >= 2 && EPL <= 8) {
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(k_attn_split<KVT, EPL, GM, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)AttnSmem<KVT, EPL, GM, 1>::total);
        if constexpr (EPL == 4) {
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(k_attn_split<KVT, EPL, GM, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)AttnSmem<KVT, EPL, GM, 2>::total);
        }
    }
    return e;
}
template <typename KVT>
static cudaError_t opt_in_all() {
    cudaError_t e;
#define VB_ATTN_OPT(E, G) if ((e = opt_in_one<KVT, E, G>()) != cudaSuccess) return e
    VB_ATTN_OPT(1, 1); VB_ATTN_OPT(1, 2); VB_ATTN_OPT(1, 4); VB_ATTN_OPT(1, 8);
    VB_ATTN_OPT(2, 1); VB_ATTN_OPT(2, 2); VB_ATTN_OPT(2, 4); VB_ATTN_OPT(2, 8);
    VB_ATTN_OPT(4, 1); VB_ATTN_OPT(4, 2); VB_ATTN_OPT(4, 4); VB_ATTN_OPT(4, 8);
    VB_ATTN_OPT(8, 1); VB_ATTN_OPT(8, 2); VB_ATTN_OPT(8, 4); VB_ATTN_OPT(8, 8); VB_ATTN_OPT(16, 1);
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
    // bulk copies move 16-byte aligned pieces; a paged chunk holds whole KV blocks
    if ((reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v)) & 15) return cudaErrorMisalignedAddress;
    if (a.block_table) {
        const uint32_t esz = a.kv_fp16 ? 2 : 4;
        uint32_t ch = 16384 / (a.D * esz);
        if (ch > 64) ch = 64;
        if (a.block_tokens == 0 || ch % a.block_tokens != 0) return cudaErrorInvalidValue;
    }
    AttnKArgs ka;
    ka.a = a;
    if (a.kv_map) memcpy(&ka.kv_map, a.kv_map, sizeof(CUtensorMap));
    else memset(&ka.kv_map, 0, sizeof(CUtensorMap));
    ka.scale = (scale != 0.0f) ? scale : 1.0f / sqrtf((float)a.D);
    ka.G = a.Hq / a.Hkv;
    ka.g_chunks = 1;
    ka.n_splits = a.max_splits;
    ka.kv_batch_stride = kv_batch_stride;
    ka.inv_freq_n = 0;
    if (a.rope_inv_freq_host && a.D / 2 <= 256) {
        ka.inv_freq_n = a.D / 2;
        for (uint32_t j = 0; j < a.D / 2; ++j) ka.inv_freq[j] = a.rope_inv_freq_host[j];
    }
    return a.kv_fp16 ? dispatch_split<__half>(lc, ka) : dispatch_split<float>(lc, ka);
}

cudaError_t attention(const LaunchCfg& lc, const AttnArgs& a) { return attention_ex(lc, a, 0.0f, 0); }

bool attn_make_kv_map(void* map_out, const void* pool, uint64_t rows, uint32_t D) {
    typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                      const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    if (!fn || !map_out || !pool || D % 64 != 0 || rows == 0 || rows > 0x7FFFFFFFull || ((uintptr_t)pool & 15) != 0) return false;
    const cuuint64_t dims[2] = {D, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    const cuuint32_t box[2] = {64, 16};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    memcpy(map_out, &m, sizeof(m));
    return true;
}

}  // namespace vb

using namespace vb;

extern "C" int32_t vb_op_gqa_attention(float* out, const float* q, const float* k_cache, const float* v_cache,
                                       uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t pos, void* scratch,
                                       uint64_t scratch_bytes, void* stream) {
    VB_REQUIRE(out && q && k_cache && v_cache && scratch, "vb_op_gqa_attention: null pointer");
    VB_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "vb_op_gqa_attention: n_q=%u not a multiple of n_kv=%u", n_q, n_kv);
    VB_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256 || head_dim == 512,
               "vb_op_gqa_attention: head_dim=%u (supported: 32,64,128,256,512)", head_dim);
    VB_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0, "vb_op_gqa_attention: the caches must be 16-byte aligned");
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
