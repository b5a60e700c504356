// Multi-head latent attention decode on the 5th-generation tensor cores: both products of the absorbed form run as
// tcgen05.mma with their accumulators in tensor memory.
//
// Same contract as k_mla_decode (vb_mla_decode.cu; model shape examples/deepseek_v3_mla.vlx:18-45, decode scope
// :117-150): per sequence, all heads share every latent row [c_kv 512 | k_rope 64] (bf16),
//     S[heads x tokens] = Q[heads x 576] . L^T,   P = softmax rows,   O[heads x 512] = P . L[:, :512].
//
// One block = 128 heads (the tensor-memory lanes) x one slice of the context x one half of the 512 output dimensions
// (O needs 128 lanes x 512 fp32 columns = all of tensor memory, so two blocks split the columns and each computes S
// for itself).  Per 16-token tile:
//   * warp 0 (one lane): tiled TMA brings the tile in as nine [16 rows][64 columns] boxes with the 128-byte swizzle
//     (ring of four); Q, converted to bf16 once by a small kernel, came in the same way as nine [128][64] boxes;
//   * three issuing warps (one lane each): S = Q . L^T -- 36 tcgen05.mma kind::f16 (bf16 operands, M 128, N 16, K 16,
//     both operands K-major from shared memory), twelve per issuer into its own partial sum.  One thread gets about
//     64 clocks per instruction whatever its N (measured: 1.2 us for the 36 of a tile at N = 16 and at N = 32, from
//     shared or tensor memory alike), so the instructions are shared out; the first issuer also does O += P . L[:, half]
//     -- one instruction (M 128, N 256, K 16) with P read FROM TENSOR MEMORY (bf16 pairs written by the softmax warps
//     with tcgen05.st: no shared-memory round trip, no proxy fence) and the SAME staged tile as the B operand, read
//     MN-major this time (tokens are K): no transposed copy of the latent rows exists anywhere;
//   * warps 2-5 (128 threads, one head row = one tensor-memory lane each): read their S row (tcgen05.ld, the three
//     partial sums), running maximum and sum without any shuffle, probabilities to bf16 into tensor memory.  The
//     maximum is lazy: O is rescaled (tcgen05.ld / st of 256 columns) only when a tile's maximum exceeds the one in
//     use by more than 8, so that probabilities stay below e^8 and almost every tile skips the rescale.
// S of tile i+1 is issued before the softmax of tile i is done (two S and two P buffers); every hand-over is an
// mbarrier with a bounded wait and a block-wide abort flag (a wait that runs out sets a status word at the head of the
// scratch area: the merge kernel then fills the output with NaN).  Rows of the last tile past the end of the context
// are zeroed in shared memory before P . L (their probabilities are 0, but 0 x garbage must not be NaN).
// Tried on the way (same workload, 64 sequences of 1024..8192 tokens): 32-token tiles with two slots and P in shared
// memory 0.49 ms; Q in tensor memory as the A operand with a four-way split of the output columns and a five-slot
// ring 0.66 ms (the S product is no faster from tensor memory and is computed four times); one issuer 0.49, two 0.44,
// three 0.44; P in tensor memory 0.41 ms; two softmax groups of four warps taking alternate tiles (the maximum in use
// handed from tile to tile through shared memory) 0.436 ms: the softmax chain is not what bounds a tile.  What does:
// each of the 36 S instructions of a tile reads its 128 x 16 slice of Q (4 KB) from shared memory at 128 bytes a
// clock, 1152 clocks (0.6 us) per tile whatever the tile's width, so the cost per token halves only with tiles twice
// as wide, and the tile buffers that 147 KB of Q leave room for hold 64 rows in all.
// The mma.sync kernel of vb_mla_decode.cu takes 0.65 ms.
#include <cuda.h>
#include <cuda_bf16.h>

#include "vb_internal.cuh"
#include "vb_kernels.cuh"
#include "vb_tma.cuh"

namespace vb {
namespace {

constexpr int MT_LAT = 576, MT_V = 512;
constexpr int MT_M = 128;                 // heads per block = tensor-memory lanes
constexpr int MT_T = 16;                  // tokens per tile (32 with two slots measured 0.435 ms against 0.412)
constexpr int MT_NBUF = 4;                // tile buffers in flight
constexpr int MT_NP = 2;                  // probability buffers
constexpr int MT_KB = MT_LAT / 64;        // nine column blocks of 64 elements (128 bytes)
constexpr int MT_DH = 256;                // output dimensions per block
constexpr int MT_Q_BYTES = MT_KB * MT_M * 128;   // 147,456
constexpr int MT_L_BYTES = MT_KB * MT_T * 128;   // per tile buffer
constexpr int MT_P_BYTES = MT_M * MT_T * 2;      // per probability buffer
constexpr int MT_BAR_BYTES = 256;
constexpr int MT_SMEM = MT_Q_BYTES + MT_NBUF * MT_L_BYTES + MT_BAR_BYTES + 1024;
static_assert(MT_SMEM <= 232448, "shared memory of one block");
constexpr int MT_NI = 3;                  // warps that issue the S product (each its own column blocks and partial sum): one thread
                                          // gets ~64 clocks per tcgen05.mma whatever its N, so 36 of them per tile are shared out
constexpr int MT_THREADS = 192 + 32 * (MT_NI - 1);
constexpr uint32_t MT_TMEM_COLS = 512;    // S: 2 buffers x MT_NI partial sums x MT_T columns at 0, then O: 256 columns (allocation sizes are powers of two)
constexpr uint32_t MT_TM_P = 2 * MT_NI * MT_T;          // probabilities as bf16 pairs: MT_NP buffers of MT_T / 2 columns
constexpr uint32_t MT_TM_O = MT_TM_P + 32;              // (room for two buffers of 16 columns)
static_assert(MT_NP * MT_T / 2 <= 32 && (MT_T == 16 || MT_T == 32), "probability buffers in tensor memory (stores of 8 or 16 columns)");
static_assert(MT_TM_O + MT_DH <= MT_TMEM_COLS && MT_KB % MT_NI == 0, "tensor memory columns / column blocks per issuer");
constexpr int MT_KB_I = MT_KB / MT_NI;    // column blocks per issuer
constexpr float MT_LAZY = 8.0f;

// instruction descriptors, kind::f16: fp32 accumulate (bit 4), A and B bf16 (1 at bits 7 and 10), N >> 3 at bit 17,
// M >> 4 at bit 24; bit 16 = B is MN-major
constexpr uint32_t MT_IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MT_T >> 3) << 17) | ((uint32_t)(MT_M >> 4) << 24);
constexpr uint32_t MT_IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(MT_DH >> 3) << 17) | ((uint32_t)(MT_M >> 4) << 24);

// K-major operand, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t desc_k_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand, 128-byte swizzle: 64 elements of MN contiguous (one 128-byte row per K index), the next 64 elements
// of MN `lbo` bytes further, groups of 8 K indices 1024 bytes apart
__device__ __forceinline__ uint64_t desc_mn_sw128(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// K-major operand without swizzle: core matrices of 8 rows x 16 bytes; `lbo` between the two along K, `sbo` between groups of 8 rows
__device__ __forceinline__ uint64_t desc_k_plain(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma_bf16_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// A from tensor memory (lane = row, two bf16 of K per 32-bit column), B from shared memory
__device__ __forceinline__ void mma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st8u(uint32_t taddr, const uint32_t r[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tmem_st16u(uint32_t taddr, const uint32_t r[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                   "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void commit_to(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float r[32]) {
    uint32_t u[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
                   "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
                   "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
                   "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float r[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])), "r"(__float_as_uint(r[2])), "r"(__float_as_uint(r[3])),
                   "r"(__float_as_uint(r[4])), "r"(__float_as_uint(r[5])), "r"(__float_as_uint(r[6])), "r"(__float_as_uint(r[7])),
                   "r"(__float_as_uint(r[8])), "r"(__float_as_uint(r[9])), "r"(__float_as_uint(r[10])), "r"(__float_as_uint(r[11])),
                   "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])), "r"(__float_as_uint(r[14])), "r"(__float_as_uint(r[15])),
                   "r"(__float_as_uint(r[16])), "r"(__float_as_uint(r[17])), "r"(__float_as_uint(r[18])), "r"(__float_as_uint(r[19])),
                   "r"(__float_as_uint(r[20])), "r"(__float_as_uint(r[21])), "r"(__float_as_uint(r[22])), "r"(__float_as_uint(r[23])),
                   "r"(__float_as_uint(r[24])), "r"(__float_as_uint(r[25])), "r"(__float_as_uint(r[26])), "r"(__float_as_uint(r[27])),
                   "r"(__float_as_uint(r[28])), "r"(__float_as_uint(r[29])), "r"(__float_as_uint(r[30])), "r"(__float_as_uint(r[31]))
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ bool wait_abort(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 128; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > 2000000000LL) { *abort_flag = 1u; return false; }
    }
}

// the same answer in every lane of a warp (the tensor-memory loads and __syncwarp that follow need the whole warp)
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    return __all_sync(0xFFFFFFFFu, wait_abort(bar, parity, abort_flag));
}

struct MlaTcParams {
    const uint32_t* ctx_len;   // [B]
    float* partial;            // [B][n_splits][n_heads][512 + 2]
    uint32_t* status;          // one word: nonzero when a wait ran out
    uint32_t n_heads, n_splits, split_tokens, q_rows_per_seq;  // q_rows_per_seq = head blocks * 128
    uint64_t cache_stride;     // rows between sequences
    float scale;
};

__global__ void __launch_bounds__(MT_THREADS, 1)
k_mla_decode_tc(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_l, const MlaTcParams p) {
    const uint32_t split = blockIdx.x, hb = blockIdx.y >> 1, dh = blockIdx.y & 1, b = blockIdx.z;
    const uint32_t ctx = p.ctx_len[b];
    const uint32_t t_lo = split * p.split_tokens;
    if (t_lo >= ctx) return;  // nothing in this slice (the merge kernel knows); before any barrier or allocation
    const uint32_t t_hi = min(ctx, t_lo + p.split_tokens), n_tok = t_hi - t_lo, n_tiles = (n_tok + MT_T - 1) / MT_T;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
    constexpr uint32_t L_OFF = MT_Q_BYTES, BAR_OFF = L_OFF + MT_NBUF * MT_L_BYTES;
    const uint32_t q_s = base, l_s = base + L_OFF, bars = base + BAR_OFF;
    // barriers (8 bytes each)
    constexpr int B_QFULL = 0, B_LFULL = 1, B_LEMPTY = B_LFULL + MT_NBUF, B_SFULL = B_LEMPTY + MT_NBUF, B_SFREE = B_SFULL + 2,
                  B_PFULL = B_SFREE + 2, B_OFULL = B_PFULL + 2, B_COUNT = B_OFULL + 1;
    static_assert(B_COUNT * 8 + 8 <= MT_BAR_BYTES, "barrier area");
    auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + BAR_OFF + B_COUNT * 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        // s_free, p_full: the four softmax warps; s_full: the issuers of S
        for (int i = 0; i < B_COUNT; ++i) mbar_init(bar(i), (i >= B_SFREE && i < B_OFULL) ? 4 : ((i >= B_SFULL && i < B_SFREE) ? MT_NI : 1));
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(MT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_o = tmem + MT_TM_O;

    // Tile i lives in ring slot i % MT_NBUF; its S in S buffer i & 1, its probabilities in P buffer i % MT_NP.
    // Completion counts: l_full[slot] and l_empty[slot] once per MT_NBUF tiles, the others once per 2 tiles.
    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: Q once, then the latent tiles -------------------------------------------------------------
            mbar_expect_tx(bar(B_QFULL), MT_Q_BYTES);
            const int q_row = (int)(b * p.q_rows_per_seq + hb * MT_M);
            for (int kb = 0; kb < MT_KB; ++kb) tma_2d(q_s + kb * (MT_M * 128), &map_q, kb * 64, q_row, bar(B_QFULL));
            const long long row0 = (long long)b * (long long)p.cache_stride + t_lo;
            for (uint32_t i = 0; i < n_tiles; ++i) {
                const uint32_t slot = i % MT_NBUF, round = i / MT_NBUF;
                if (round >= 1 && !wait_abort(bar(B_LEMPTY + slot), (round + 1) & 1, abort_flag)) break;  // P . L of tile i - MT_NBUF is done
                mbar_expect_tx(bar(B_LFULL + slot), MT_L_BYTES);
                const int y = (int)(row0 + (long long)i * MT_T);
                for (int kb = 0; kb < MT_KB; ++kb) tma_2d(l_s + slot * MT_L_BYTES + kb * (MT_T * 128), &map_l, kb * 64, y, bar(B_LFULL + slot));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- tensor-core issue --------------------------------------------------------------------------------
            auto issue_s = [&](uint32_t i) {
                const uint32_t lt = l_s + (i % MT_NBUF) * MT_L_BYTES;
#pragma unroll 1
                for (int kb = 0; kb < MT_KB_I; ++kb) {
                    const uint64_t da = desc_k_sw128(q_s + kb * (MT_M * 128)), db = desc_k_sw128(lt + kb * (MT_T * 128));
#pragma unroll
                    for (int k = 0; k < 4; ++k) mma_bf16_ss(tmem + (i & 1) * MT_NI * MT_T, da + 2u * k, db + 2u * k, MT_IDESC_S, (kb | k) != 0 ? 1u : 0u);
                }
                commit_to(bar(B_SFULL + (i & 1)));
            };
            // may S of tile i be issued?  its rows have landed and the softmax of tile i - 2 has read the S buffer
            auto ready_s = [&](uint32_t i) {
                if (!wait_abort(bar(B_LFULL + i % MT_NBUF), (i / MT_NBUF) & 1, abort_flag)) return false;
                if (i >= 2 && !wait_abort(bar(B_SFREE + (i & 1)), ((i >> 1) + 1) & 1, abort_flag)) return false;
                fence_after();
                return true;
            };
            bool ok = wait_abort(bar(B_QFULL), 0u, abort_flag) && ready_s(0);
            if (ok) {
                issue_s(0);
                for (uint32_t i = 0; i < n_tiles; ++i) {
                    if (i + 1 < n_tiles) {
                        if (!ready_s(i + 1)) break;
                        issue_s(i + 1);
                    }
                    if (!wait_abort(bar(B_PFULL + (i & 1)), (i >> 1) & 1, abort_flag)) break;  // probabilities of tile i are in shared memory
                    fence_after();
                    const uint32_t lt = l_s + (i % MT_NBUF) * MT_L_BYTES + dh * 4 * (MT_T * 128);
#pragma unroll
                    for (int kk = 0; kk < MT_T / 16; ++kk) {
                        const uint64_t db = desc_mn_sw128(lt + kk * 2048, MT_T * 128);
                        mma_bf16_ts(tmem_o, tmem + MT_TM_P + (i % MT_NP) * (MT_T / 2) + kk * 8, db, MT_IDESC_O, (i | (uint32_t)kk) != 0 ? 1u : 0u);
                    }
                    commit_to(bar(B_LEMPTY + i % MT_NBUF));  // the slot, and the P buffer, of tile i are free
                    if (i + 1 == n_tiles) commit_to(bar(B_OFULL));
                }
            }
        }
    } else if (warp >= 6) {
        if (lane == 0) {
            // ---- further issuers: their column blocks of the S product into their own partial sums --------------------------
            const int q = (int)warp - 5;  // 1 .. MT_NI - 1
            bool ok = wait_abort(bar(B_QFULL), 0u, abort_flag);
            for (uint32_t i = 0; i < n_tiles && ok; ++i) {
                if (!wait_abort(bar(B_LFULL + i % MT_NBUF), (i / MT_NBUF) & 1, abort_flag)) break;
                if (i >= 2 && !wait_abort(bar(B_SFREE + (i & 1)), ((i >> 1) + 1) & 1, abort_flag)) break;
                fence_after();
                const uint32_t lt = l_s + (i % MT_NBUF) * MT_L_BYTES;
#pragma unroll 1
                for (int kb = q * MT_KB_I; kb < (q + 1) * MT_KB_I; ++kb) {
                    const uint64_t da = desc_k_sw128(q_s + kb * (MT_M * 128)), db = desc_k_sw128(lt + kb * (MT_T * 128));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mma_bf16_ss(tmem + ((i & 1) * MT_NI + q) * MT_T, da + 2u * k, db + 2u * k, MT_IDESC_S, (kb > q * MT_KB_I || k != 0) ? 1u : 0u);
                }
                commit_to(bar(B_SFULL + (i & 1)));
            }
        }
    } else {
        // ---- softmax: thread = head row = tensor-memory lane --------------------------------------------------------------
        const uint32_t lg = warp & 3;                    // the lanes this warp may touch: 32 * (warp % 4)
        const uint32_t row = lg * 32 + lane;             // head within the block
        const uint32_t lane_addr = (lg * 32u) << 16;
        float m_use = -INFINITY, l_run = 0.0f;
        bool ok = true;
        // has P . L of tile j completed?  (its slot's l_empty barrier; at most one completion behind or ahead of the caller)
        auto pv_done = [&](uint32_t j) { return warp_wait(bar(B_LEMPTY + j % MT_NBUF), (j / MT_NBUF) & 1, abort_flag); };
        for (uint32_t i = 0; i < n_tiles && ok; ++i) {
            ok = warp_wait(bar(B_SFULL + (i & 1)), (i >> 1) & 1, abort_flag);
            if (!ok) break;
            fence_after();
            float s[32];
            tmem_ld32(tmem + lane_addr + (i & 1) * MT_NI * MT_T, s);   // the issuers' partial sums
#pragma unroll 1
            for (int q = 1; q < MT_NI; ++q) {
                float s2[32];
                tmem_ld32(tmem + lane_addr + ((i & 1) * MT_NI + q) * MT_T, s2);
#pragma unroll
                for (int c = 0; c < 32; ++c) s[c] += s2[c];
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_SFREE + (i & 1)));
            const uint32_t valid = min((uint32_t)MT_T, n_tok - i * MT_T);
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < MT_T; ++j) {
                s[j] = (uint32_t)j < valid ? s[j] * p.scale : -INFINITY;
                mx = fmaxf(mx, s[j]);
            }
            // lazy maximum: move only when the tile's exceeds the one in use by more than MT_LAZY (always on the first tile)
            const bool move = mx > m_use + MT_LAZY || i == 0;
            const float m_new = move ? mx : m_use;
            const float alpha = move ? (i == 0 ? 0.0f : __expf(m_use - m_new)) : 1.0f;
            uint32_t packed[MT_T / 2];
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < MT_T / 2; ++j) {
                const __nv_bfloat162 pr = __floats2bfloat162_rn(__expf(s[2 * j] - m_new), __expf(s[2 * j + 1] - m_new));
                sum += __bfloat162float(pr.x) + __bfloat162float(pr.y);  // the rounded values: numerator and denominator agree
                packed[j] = *reinterpret_cast<const uint32_t*>(&pr);
            }
            l_run = l_run * alpha + sum;
            m_use = m_new;
            if (i >= 1 && __any_sync(0xFFFFFFFFu, move)) {
                // rescale this warp's 32 rows of O (256 columns) once every product issued so far is done; lanes that did
                // not move multiply by 1
                ok = pv_done(i - 1);
                if (!ok) break;
                fence_after();
#pragma unroll 1
                for (int c = 0; c < MT_DH / 32; ++c) {
                    float o[32];
                    tmem_ld32(tmem_o + lane_addr + c * 32, o);
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] *= alpha;
                    tmem_st32(tmem_o + lane_addr + c * 32, o);
                }
                tmem_st_wait();
            } else if (i >= (uint32_t)MT_NP) {
                ok = pv_done(i - MT_NP);  // the P buffer of this tile was read by the product of tile i - MT_NP
                if (!ok) break;
            }
            if (valid < (uint32_t)MT_T) {
                // the last tile: rows past the context's end hold whatever followed in the cache; zero them for P . L
                // (the tile has landed: S of this tile was computed from it)
                const uint32_t lt = L_OFF + (i % MT_NBUF) * MT_L_BYTES + dh * 4 * (MT_T * 128);
                const uint32_t n_zero = (MT_T - valid) * 4 * 8;  // (row, column block, 16-byte piece)
                for (uint32_t z = (warp - 2) * 32 + lane; z < n_zero; z += 128) {
                    const uint32_t piece = z & 7, cb = (z >> 3) & 3, r = valid + (z >> 5);
                    *reinterpret_cast<uint4*>(gen + lt + cb * (MT_T * 128) + r * 128 + piece * 16) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic stores, read by the tensor core
            }
            // P row: MT_T bf16 as pairs into this lane's columns of the probability buffer (the A operand of P . L)
            if constexpr (MT_T == 16) tmem_st8u(tmem + lane_addr + MT_TM_P + (i % MT_NP) * (MT_T / 2), packed);
            else tmem_st16u(tmem + lane_addr + MT_TM_P + (i % MT_NP) * (MT_T / 2), packed);
            tmem_st_wait();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_PFULL + (i & 1)));
        }
        // ---- this slice's unnormalised output, maximum in use and sum ------------------------------------------------
        if (ok) ok = warp_wait(bar(B_OFULL), 0u, abort_flag);
        if (ok) {
            fence_after();
            const uint32_t h = hb * MT_M + row;
            float* out = p.partial + ((((size_t)b * p.n_splits + split) * p.n_heads) + h) * (MT_V + 2);
#pragma unroll 1
            for (int c = 0; c < MT_DH / 32; ++c) {
                float o[32];
                tmem_ld32(tmem_o + lane_addr + c * 32, o);  // every lane of the warp takes part, rows past n_heads just do not store
                if (h < p.n_heads) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2)  // rows of 514 floats start on 8-byte boundaries only
                        *reinterpret_cast<float2*>(out + dh * MT_DH + c * 32 + j) = make_float2(o[j], o[j + 1]);
                }
            }
            if (dh == 0 && h < p.n_heads) { out[MT_V] = m_use; out[MT_V + 1] = l_run; }
        }
        fence_before();
    }
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicOr(p.status, 1u);
        // let copies in flight land before the block (and its shared memory) goes away
        const long long t0 = clock64();
        while (clock64() - t0 < 20000000LL) {}
        __syncthreads();
    }
    if (warp == 1) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(MT_TMEM_COLS) : "memory");
    }
}

// q fp32 [B][n_heads][576] -> bf16 [B][rows_per_seq][576], rows past n_heads zero; one block per (row, sequence), 288 threads
__global__ void __launch_bounds__(MT_LAT / 2)
k_mla_q_bf16(__nv_bfloat16* __restrict__ dst, const float* __restrict__ q, uint32_t n_heads, uint32_t rows_per_seq) {
    const uint32_t r = blockIdx.x, b = blockIdx.y, i = threadIdx.x;
    float2 v = make_float2(0.f, 0.f);
    if (r < n_heads) v = *reinterpret_cast<const float2*>(q + ((size_t)b * n_heads + r) * MT_LAT + 2 * i);
    *reinterpret_cast<__nv_bfloat162*>(dst + ((size_t)b * rows_per_seq + r) * MT_LAT + 2 * i) = __floats2bfloat162_rn(v.x, v.y);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn_mla() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}
// bf16 [rows][576] row-major, boxes of [box_rows][64 columns], 128-byte swizzle, zeros outside the matrix
bool make_map_bf16(CUtensorMap* m, const void* ptr, uint64_t rows, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn_mla();
    if (!fn) return false;
    const cuuint64_t dims[2] = {MT_LAT, rows};
    const cuuint64_t strides[1] = {MT_LAT * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

uint64_t mla_tc_extra_scratch_bytes(uint32_t batch, uint32_t n_heads) {
    const uint64_t rows = (uint64_t)((n_heads + MT_M - 1) / MT_M) * MT_M;
    return 1024 + (uint64_t)batch * rows * MT_LAT * 2;
}

// extra: the area of mla_tc_extra_scratch_bytes (16-byte aligned): a status word, then Q in bf16
cudaError_t mla_decode_tc(const LaunchCfg& lc, const float* q, const void* cache, const uint32_t* ctx_len, float* partial, void* extra,
                          uint32_t batch, uint32_t n_heads, uint32_t n_splits, uint32_t split_tokens, uint64_t cache_stride, float scale) {
    static bool opted = false;
    cudaError_t e;
    if (!opted) {
        if ((e = cudaFuncSetAttribute(k_mla_decode_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, MT_SMEM)) != cudaSuccess) return e;
        opted = true;
    }
    const uint32_t hbs = (n_heads + MT_M - 1) / MT_M, rows_per_seq = hbs * MT_M;
    uint32_t* status = reinterpret_cast<uint32_t*>(extra);
    __nv_bfloat16* q16 = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<unsigned char*>(extra) + 1024);
    CUtensorMap mq, ml;
    if (!make_map_bf16(&mq, q16, (uint64_t)batch * rows_per_seq, MT_M) || !make_map_bf16(&ml, cache, (uint64_t)batch * cache_stride, MT_T))
        return cudaErrorNotSupported;
    if ((e = cudaMemsetAsync(status, 0, 4, lc.stream)) != cudaSuccess) return e;
    if ((e = launch(lc, k_mla_q_bf16, dim3(rows_per_seq, batch), dim3(MT_LAT / 2), 0, q16, q, n_heads, rows_per_seq)) != cudaSuccess) return e;
    MlaTcParams p;
    p.ctx_len = ctx_len; p.partial = partial; p.status = status;
    p.n_heads = n_heads; p.n_splits = n_splits; p.split_tokens = split_tokens; p.q_rows_per_seq = rows_per_seq;
    p.cache_stride = cache_stride; p.scale = scale;
    return launch(lc, k_mla_decode_tc, dim3(n_splits, 2 * hbs, batch), dim3(MT_THREADS), MT_SMEM, mq, ml, p);
}

}  // namespace vb
