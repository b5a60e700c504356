// Multi-row products on the 5th-generation tensor cores (tcgen05 + tensor memory), fed by tiled TMA copies:
// the dense contraction of prefill and of wide batches,  dst[t][o] = sum_k x[t][k] * W[o][k]  for a few hundred
// rows t of x at once (the reference's multi-token register-tiled kernels, velox_cuda_runner_k2.cu:480-1085).
//
// Operands are fp16 in shared memory, accumulation is fp32 in tensor memory:
//   * x rows are converted fp32 -> fp16 (with the RMS normalisation of the reference, runtime.rs:588-601,
//     folded in) by k_rows_to_f16 into a workspace [rows][K];
//   * the weight matrix is brought to fp16 [out][K] by k_weights_to_f16 (int4 g32: the exact fp32 value
//     (q-8)*s rounded once; int8 per channel: the integer, exact, the row scale is applied to the fp32
//     accumulator in the epilogue), either once into a resident copy the engine keeps or per call into the
//     workspace; fp16 matrices are used where they lie;
//   * k_gemm_tc: one block per tile of 128 weight rows (the M of the instruction, = tensor-memory lanes) by 32,
//     128 or 256 rows of x (N, = tensor-memory columns).  Warp 0 / lane 0 issues the TMA copies of 128-byte-swizzled
//     [128][64] fp16 boxes into a ring of stages, warp 1 / lane 0 issues tcgen05.mma (four K=16 steps per
//     stage) and hands each stage back with tcgen05.commit, all four warps read the accumulator with
//     tcgen05.ld and write the epilogue (store / residual add / SiLU(gate)*up with the two accumulators of the
//     gate and up matrices side by side in tensor memory).
// Every wait is bounded; a wait that runs out sets a block-wide abort flag and the library's error word, the
// block still frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>

#include "vb_kernels.cuh"
#include "vb_tma.cuh"

namespace vb {
namespace {

constexpr int BM = 128;      // weight rows per tile (UMMA M)
                             // rows of x per tile (UMMA N): 128 or 256, a template parameter of the kernel
constexpr int BK = 64;       // K extent of a stage: 64 fp16 = one 128-byte swizzle row
constexpr int TILE_BYTES = BM * BK * 2;  // 16 KB: one box of 128 rows
// ring depth so that the stages fill 192 KB: (weight tiles + x tiles) x 16 KB per stage
__host__ __device__ constexpr int stage_bytes_for(bool dual, int bn) { return (dual ? 2 : 1) * TILE_BYTES + bn * BK * 2; }
// PER_SM = 1: the ring fills 192 KB; PER_SM = 2: 96 KB, so that two blocks share an SM and one block's prologue
// and epilogue overlap the other's main loop
__host__ __device__ constexpr int stages_for(bool dual, int bn, int per_sm = 1) { return (192 / per_sm) * 1024 / stage_bytes_for(dual, bn); }
constexpr int SMEM_BYTES_HALF = 96 * 1024 + 1024 + 256;
constexpr int SMEM_BYTES = 192 * 1024 + 1024 /* alignment slack */ + 256 /* barriers */;

// instruction descriptor of tcgen05.mma kind::f16: fp32 accumulate (bits 4-5 = 1), A and B fp16 (formats 0),
// both K-major (bits 15, 16 = 0), N >> 3 at bit 17, M >> 4 at bit 24
__host__ __device__ constexpr uint32_t idesc_for(int bn) { return (1u << 4) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24); }

// shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: start address >> 4 in bits 0-13,
// leading byte offset (unused with a swizzle; 1) in bits 16-29, stride between groups of 8 rows = 1024 bytes
// (>> 4) in bits 32-45, descriptor version 1 in bits 46-47, layout type 2 (128-byte swizzle) in bits 61-63
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t r[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                   "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                   "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Bounded wait that also gives up as soon as another thread of the block has given up.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
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

struct GemmParams {
    float* dst;                // [n_rows][dst_stride], column offset already applied
    const __half* row_scale;   // != null: accumulator of weight row o is multiplied by row_scale[o] (int8 per channel)
    const __half* row_scale2;
    const SeqState* state;     // != null: rows of inactive slots are not written
    uint32_t out_dim, n_rows, K, dst_stride;
    int epilogue;
    uint32_t* err;
    // split K (gridDim.z > 1): every block stores its fp32 partial tile, the last block to arrive at the tile's
    // counter sums the partials in split order (the same bits whoever is last) and runs the epilogue
    float* part;          // [split][tile][BN / 32][32][128]
    uint32_t* counters;   // [tile], zero between launches (the last block puts the zero back)
    // Operand splitting (prefill chunks): fp16 holds 11 significant bits, and over 32 layers and thousands of cached
    // positions that rounding reaches the logits (2.8e-2 at 2048 rows of the 8B shape).  x_parts = 2: x = x_hi + x_lo,
    // both fp16, x_lo rows lie `x_lo_row` rows below x_hi in the same tensor map; w_parts = 2: W = W_hi + W_lo likewise
    // (second tensor maps).  The products W_hi.x_hi + W_hi.x_lo + W_lo.x_hi accumulate into the same tensor-memory
    // columns, so the epilogue does not change; what is dropped (W_lo.x_lo) is 2^-22 of the result.
    uint32_t x_parts, w_parts, x_lo_row;
    uint32_t stages;      // ring depth for this operand set
};

template <bool DUAL, int BN, int PER_SM = 1>
__global__ void __launch_bounds__(128, PER_SM)
k_gemm_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
          const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wl, const __grid_constant__ CUtensorMap map_wl2,
          const GemmParams p) {
    constexpr int W_TILES = DUAL ? 2 : 1, X_TILES = BN / 128;  // BN = 32: one box of 32 rows
    constexpr int X_BYTES = BN * BK * 2;                        // one part of the x operand of a stage
    const int STAGES = (int)p.stages;
    const int WP = (int)p.w_parts, XP = (int)p.x_parts;
    const int STAGE_BYTES = W_TILES * WP * TILE_BYTES + XP * X_BYTES;  // [W hi (,W2 hi)][W lo (,W2 lo)][x hi][x lo]
    const int X_OFF = W_TILES * WP * TILE_BYTES;
    constexpr uint32_t IDESC = idesc_for(BN);
    constexpr uint32_t TMEM_COLS = DUAL ? 2 * BN : BN;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzled tiles want 1024-byte alignment
    const uint32_t bars = base + STAGES * STAGE_BYTES;            // full[STAGES], empty[STAGES], accum, then two words
    const uint32_t bar_accum = bars + 2 * STAGES * 8;
    unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + STAGES * STAGE_BYTES + (2 * STAGES + 1) * 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the tiles of x are the fastest block index: the blocks that share a weight tile run together and it comes
    // from DRAM once
    const int row0 = blockIdx.y * BM, tok0 = blockIdx.x * BN;
    const int nk_all = (int)((p.K + BK - 1) / BK);
    const int kb_first = (int)(((long long)nk_all * blockIdx.z) / gridDim.z), kb_last = (int)(((long long)nk_all * (blockIdx.z + 1)) / gridDim.z);
    const int nk = kb_last - kb_first;  // this block's share of the K blocks

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(bars + s * 8, 1); mbar_init(bars + (STAGES + s) * 8, 1); }
        mbar_init(bar_accum, 1);
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    pdl_wait();  // x (and converted weights) come from the kernels before this one
    pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---- producer: TMA copies into the ring ----
        for (int kb = 0; kb < nk; ++kb) {
            const int s = kb % STAGES;
            const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
            if (!wait_or_abort(bars + (STAGES + s) * 8, ph ^ 1u, abort_flag)) break;
            const uint32_t full = bars + s * 8, st = base + s * STAGE_BYTES;
            mbar_expect_tx(full, STAGE_BYTES);
            const int kx = (kb_first + kb) * BK;
            tma_load_2d(st, &map_w, kx, row0, full);
            if (DUAL) tma_load_2d(st + TILE_BYTES, &map_w2, kx, row0, full);
            if (WP == 2) {
                tma_load_2d(st + W_TILES * TILE_BYTES, &map_wl, kx, row0, full);
                if (DUAL) tma_load_2d(st + (W_TILES + 1) * TILE_BYTES, &map_wl2, kx, row0, full);
            }
            for (int xp = 0; xp < XP; ++xp) {
                const int xr = tok0 + xp * (int)p.x_lo_row;
                tma_load_2d(st + X_OFF + xp * X_BYTES, &map_x, kx, xr, full);
                if (X_TILES == 2) tma_load_2d(st + X_OFF + xp * X_BYTES + TILE_BYTES, &map_x, kx, xr + 128, full);  // rows 128..255: the next 16 groups of 8
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- tensor-core issue ----
        for (int kb = 0; kb < nk; ++kb) {
            const int s = kb % STAGES;
            const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
            if (!wait_or_abort(bars + s * 8, ph, abort_flag)) break;
            tc_fence_after();
            const uint32_t st = base + s * STAGE_BYTES;
            const uint64_t da = smem_desc(st), da2 = smem_desc(st + TILE_BYTES), db = smem_desc(st + X_OFF);
            const uint64_t dal = smem_desc(st + W_TILES * TILE_BYTES), dal2 = smem_desc(st + (W_TILES + 1) * TILE_BYTES), dbl = smem_desc(st + X_OFF + X_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {  // 16 fp16 = 32 bytes further along the swizzled row: +2 in the address field
                const uint32_t acc = (kb | k) != 0 ? 1u : 0u;
                mma_f16(tmem, da + 2u * k, db + 2u * k, IDESC, acc);
                if (XP == 2) mma_f16(tmem, da + 2u * k, dbl + 2u * k, IDESC, 1u);
                if (WP == 2) mma_f16(tmem, dal + 2u * k, db + 2u * k, IDESC, 1u);
                if (DUAL) {
                    mma_f16(tmem + BN, da2 + 2u * k, db + 2u * k, IDESC, acc);
                    if (XP == 2) mma_f16(tmem + BN, da2 + 2u * k, dbl + 2u * k, IDESC, 1u);
                    if (WP == 2) mma_f16(tmem + BN, dal2 + 2u * k, db + 2u * k, IDESC, 1u);
                }
            }
            mma_commit(bars + (STAGES + s) * 8);  // the stage is free again once these products have read it
        }
        mma_commit(bar_accum);
    }
    __syncwarp();

    // ---- epilogue: warp w owns tensor-memory lanes 32w..32w+31 = weight rows row0 + 32w + lane ----
    const bool ok = wait_or_abort(bar_accum, 0u, abort_flag);
    tc_fence_after();
    const bool good = __syncthreads_and(ok && !*abort_flag);
    if (good) {
        const uint32_t o = (uint32_t)row0 + warp * 32 + lane;
        const bool o_ok = o < p.out_dim;
        const float sc = (p.row_scale && o_ok) ? __half2float(p.row_scale[o]) : 1.0f;
        const float sc2 = (DUAL && p.row_scale2 && o_ok) ? __half2float(p.row_scale2[o]) : 1.0f;
        const uint32_t lane_addr = tmem + ((warp * 32u) << 16);
        const uint32_t n_split = gridDim.z, tile = blockIdx.y * gridDim.x + blockIdx.x, n_tiles = gridDim.x * gridDim.y;
        bool reduce = false;  // this block sums the partials of all splits instead of reading its accumulator
        if (!DUAL && n_split > 1) {
            __shared__ uint32_t s_last;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if ((uint32_t)(tok0 + c0) >= p.n_rows) break;
                uint32_t v[32];
                tmem_ld32(lane_addr + c0, v);
                float* pt = p.part + ((((size_t)blockIdx.z * n_tiles + tile) * (BN / 32) + c0 / 32) * 32) * 128 + threadIdx.x;
#pragma unroll
                for (int j = 0; j < 32; ++j) __stcg(pt + j * 128, __uint_as_float(v[j]));
            }
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                const uint32_t old = atomicAdd(p.counters + tile, 1u);
                s_last = old == n_split - 1 ? 1u : 0u;
                if (s_last) { p.counters[tile] = 0u; __threadfence(); }
            }
            __syncthreads();
            reduce = s_last != 0u;
        }
        if (DUAL || n_split == 1 || reduce) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            if ((uint32_t)(tok0 + c0) >= p.n_rows) break;  // uniform over the block
            // which of the 32 rows of x are written: one flag per lane, gathered once (no load between the stores below)
            const uint32_t tl = (uint32_t)(tok0 + c0) + lane;
            const bool live = tl < p.n_rows && (!p.state || p.state[tl].active);
            const uint32_t live_mask = __ballot_sync(0xFFFFFFFFu, live);
            uint32_t v[32], u[32];
            if (reduce) {
                float acc[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[j] = 0.0f;
                for (uint32_t z = 0; z < n_split; ++z) {
                    const float* pt = p.part + ((((size_t)z * n_tiles + tile) * (BN / 32) + c0 / 32) * 32) * 128 + threadIdx.x;
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[j] += __ldcg(pt + j * 128);
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(acc[j]);
            } else {
                tmem_ld32(lane_addr + c0, v);
                if (DUAL) tmem_ld32(lane_addr + BN + c0, u);
            }
            if (!o_ok) continue;
            float* d0 = p.dst + (size_t)(tok0 + c0) * p.dst_stride + o;
            if (!DUAL && p.epilogue == EPI_RESIDUAL) {
                // all 32 residual values first (independent loads), then the sums: one memory round trip, not 32
                float res[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) res[j] = ((live_mask >> j) & 1u) ? __ldcg(d0 + (size_t)j * p.dst_stride) : 0.0f;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if ((live_mask >> j) & 1u) d0[(size_t)j * p.dst_stride] = res[j] + __uint_as_float(v[j]) * sc;
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (!((live_mask >> j) & 1u)) continue;
                    const float a = __uint_as_float(v[j]) * sc;
                    if (DUAL) {
                        const float up = __uint_as_float(u[j]) * sc2;
                        d0[(size_t)j * p.dst_stride] = (a / (1.0f + expf(-a))) * up;
                    } else {
                        d0[(size_t)j * p.dst_stride] = a;
                    }
                }
            }
        }
        }
    } else {
        if (threadIdx.x == 0 && p.err) atomicOr(p.err, 0x40u);
        // let copies and products that are still in flight land before the memory they use is given back
        const long long t0 = clock64();
        while (clock64() - t0 < 20000000LL) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

// ---- operand conversion -------------------------------------------------------------------------------------
// One block per row of x: y = fp16( (x * inv_rms) * w ) (the reference's RMSNorm, runtime.rs:588-601) or fp16(x).
// Rows of inactive slots and rows beyond n_rows (up to the tile boundary) become zeros.
// dst_lo != null: the part fp16 cannot hold goes there, x = fp16 hi + fp16 lo to ~22 bits.
__global__ void __launch_bounds__(256)
k_rows_to_f16(__half* __restrict__ dst, __half* __restrict__ dst_lo, const float* __restrict__ x, const void* __restrict__ norm_w, int norm_fmt, float eps,
              const SeqState* __restrict__ state, uint32_t K, uint32_t n_rows) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t r = blockIdx.x;
    __half* out = dst + (size_t)r * K;
    const bool live = r < n_rows && (!state || state[r].active);
    if (!live) {
        for (uint32_t k = threadIdx.x; k < K; k += blockDim.x) { out[k] = __float2half_rn(0.0f); if (dst_lo) dst_lo[(size_t)r * K + k] = __float2half_rn(0.0f); }
        return;
    }
    const float4* in4 = reinterpret_cast<const float4*>(x + (size_t)r * K);  // K is a multiple of 8
    const uint32_t K4 = K / 4;
    float inv = 1.0f;
    if (norm_w) {
        __shared__ float part[8];
        float ss = 0.0f;
        for (uint32_t k = threadIdx.x; k < K4; k += blockDim.x) {
            const float4 v = in4[k];
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) tot += part[i];
        inv = 1.0f / sqrtf(tot / (float)K + eps);
    }
    uint2* out2 = reinterpret_cast<uint2*>(out);
    for (uint32_t k = threadIdx.x; k < K4; k += blockDim.x) {
        float4 v = in4[k];
        if (norm_w) {
            float4 w;
            if (norm_fmt == VB_FMT_F16) {
                const uint2 raw = reinterpret_cast<const uint2*>(norm_w)[k];
                const float2 w01 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x)), w23 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                w = make_float4(w01.x, w01.y, w23.x, w23.y);
            } else {
                w = reinterpret_cast<const float4*>(norm_w)[k];
            }
            v.x = (v.x * inv) * w.x; v.y = (v.y * inv) * w.y; v.z = (v.z * inv) * w.z; v.w = (v.w * inv) * w.w;
        }
        // un-normalised inputs (attention output, SiLU(gate) * up) may exceed fp16's range: the cast saturates instead of
        // producing infinities; with the hi + lo split the low half carries what the high half could not (exact up to 2 x 65504)
        constexpr float H_MAX = 65504.0f;
        auto sat = [](float f) { return fminf(fmaxf(f, -H_MAX), H_MAX); };
        const __half2 h01 = __floats2half2_rn(sat(v.x), sat(v.y)), h23 = __floats2half2_rn(sat(v.z), sat(v.w));
        out2[k] = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
        if (dst_lo) {
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const __half2 l01 = __floats2half2_rn(sat(v.x - f01.x), sat(v.y - f01.y)), l23 = __floats2half2_rn(sat(v.z - f23.x), sat(v.w - f23.y));
            reinterpret_cast<uint2*>(dst_lo + (size_t)r * K)[k] = make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
        }
    }
}

// Weights -> fp16 [rows][K], eight elements (one packed int4 word, one 16-byte store) per thread.
__global__ void __launch_bounds__(256)
k_weights_to_f16(uint4* __restrict__ dst, uint4* __restrict__ dst_lo, const void* __restrict__ data, const void* __restrict__ scales, int fmt, uint64_t n8, uint32_t K) {
    pdl_wait();
    pdl_launch_dependents();
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (uint64_t)gridDim.x * blockDim.x) {
        float f[8];
        const uint64_t e0 = i * 8;
        switch (fmt) {
        case VB_FMT_Q4G32: {
            unpack8_f32(reinterpret_cast<const uint32_t*>(data)[i], f);
            const float s = __half2float(reinterpret_cast<const __half*>(scales)[i >> 2]);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = __fmul_rn(__fsub_rn(f[j], 8.0f), s);
        } break;
        case VB_FMT_Q4G64REF: {
            unpack8_f32(reinterpret_cast<const uint32_t*>(data)[i], f);
            const __half2 sm = reinterpret_cast<const __half2*>(scales)[i >> 3];
            const float s = __low2float(sm), m = __high2float(sm);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = fmaf(f[j], s, m);
        } break;
        case VB_FMT_I8PC: {
            const uint2 raw = reinterpret_cast<const uint2*>(data)[i];
            const int8_t* q = reinterpret_cast<const int8_t*>(&raw);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = (float)q[j];
        } break;
        case VB_FMT_BF16: {
            const uint4 raw = reinterpret_cast<const uint4*>(data)[i];
            const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(b[j]);
        } break;
        default: {  // VB_FMT_F32
            const float4 a = reinterpret_cast<const float4*>(data)[2 * i], b = reinterpret_cast<const float4*>(data)[2 * i + 1];
            f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
        } break;
        }
        (void)e0; (void)K;
        __half2 h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
        dst[i] = *reinterpret_cast<const uint4*>(h);
        if (dst_lo) {  // what the rounding to fp16 dropped (exact as a difference of nearby floats), rounded to fp16 in turn
            __half2 l[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 hf = __half22float2(h[j]); l[j] = __floats2half2_rn(f[2 * j] - hf.x, f[2 * j + 1] - hf.y); }
            dst_lo[i] = *reinterpret_cast<const uint4*>(l);
        }
    }
}

// ---- host side --------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// fp16 [rows][K] row-major, boxes of [128 rows][64 columns], 128-byte swizzle, zeros outside the matrix
bool make_map(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t K, uint32_t box_rows = BM) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {K, rows};
    const cuuint64_t strides[1] = {K * 2};
    const cuuint32_t box[2] = {BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool g_tc_init = false;

}  // namespace

bool gemm_tc_two_per_sm = true;  // vb_set_option("prefill_two_per_sm", 0): one block of twice the ring depth per SM (measured 4 % slower)
bool gemm_tc_split_k = true;  // vb_set_option("decode_split_k", 0): one block per tile of 128 weight rows
int gemm_tc_split = 2;  // vb_set_option("prefill_split", n): prefill chunks multiply 0: fp16(x).fp16(W); 1: x as hi + lo; 2: x and W as hi + lo
bool gemm_tc_wide = false;  // vb_set_option("prefill_wide", 1): 256 rows of x per tile when a chunk has more than 128 (measured slower at 512 rows: fewer blocks than SMs)

cudaError_t gemm_tc_init() {
    if (g_tc_init) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(k_gemm_tc<false, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(k_gemm_tc<true, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(k_gemm_tc<false, 128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_HALF);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(k_gemm_tc<true, 128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_HALF);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(k_gemm_tc<false, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(k_gemm_tc<true, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(k_gemm_tc<false, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(k_gemm_tc<true, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    g_tc_init = true;
    return cudaSuccess;
}

// fp16 [rows][cols] copy of a weight matrix (int8 per channel: the integers; the row scale stays with the caller)
cudaError_t weights_to_f16(const LaunchCfg& lc, void* dst, const WMat& m, void* dst_lo) {
    const uint64_t n8 = (uint64_t)m.rows * m.cols / 8;
    uint64_t blocks = (n8 + 255) / 256;
    if (blocks > 148ull * 64) blocks = 148ull * 64;
    return launch(lc, k_weights_to_f16, dim3((unsigned)blocks), dim3(256), 0, reinterpret_cast<uint4*>(dst), reinterpret_cast<uint4*>(dst_lo), m.data,
                  m.scales, (int)m.fmt, n8, m.cols);
}
// formats whose values fp16 does not hold exactly (int8 per channel: the integers are exact, the row scale stays in fp32)
bool gemm_tc_weights_inexact(int32_t fmt) { return fmt == VB_FMT_Q4G32 || fmt == VB_FMT_Q4G64REF || fmt == VB_FMT_F32 || fmt == VB_FMT_BF16; }

bool gemm_tc_supported(const GemvArgs& a) {
    if (a.w.rows == 0 || a.w.cols == 0 || a.w.cols % 8 != 0 || !fmt_shape_ok(a.w.fmt, a.w.cols) || !a.w.data) return false;
    if (a.epilogue == EPI_SWIGLU && (a.w2.fmt != a.w.fmt || a.w2.rows != a.w.rows || a.w2.cols != a.w.cols || !a.w2.data)) return false;
    return a.push.links == nullptr;
}

uint64_t gemm_tc_rows_padded(uint32_t n_rows) { return ((uint64_t)n_rows + 127) / 128 * 128; }

// workspace: x as fp16 [rows padded to 128][K], then the weight matrix (two for gate/up) as fp16 [out][K]
// head of the workspace: the split-K tile counters (zeroed by whoever allocates the workspace) and partial tiles
constexpr uint64_t WS_COUNTER_BYTES = 64 * 1024, WS_PART_BYTES = 4 * 1024 * 1024, WS_HEAD_BYTES = WS_COUNTER_BYTES + WS_PART_BYTES;
uint64_t gemm_tc_workspace_zero_bytes() { return WS_COUNTER_BYTES; }

uint64_t gemm_tc_workspace_bytes(uint32_t out_dim, uint32_t in_dim, uint32_t n_rows, bool dual) {
    return WS_HEAD_BYTES + gemm_tc_operand_bytes(out_dim, in_dim, n_rows, dual);
}

uint64_t gemm_tc_operand_bytes(uint32_t out_dim, uint32_t in_dim, uint32_t n_rows, bool dual) {
    const uint64_t xb = (gemm_tc_rows_padded(n_rows) * in_dim * 2 + 1023) / 1024 * 1024;
    const uint64_t wb = ((uint64_t)out_dim * in_dim * 2 + 1023) / 1024 * 1024;
    return 2 * xb + (dual ? 2 : 1) * 2 * wb;  // room for the hi and lo parts of both operands
}

cudaError_t gemm_tc(const LaunchCfg& lc, const GemvArgs& a, void* workspace, uint64_t workspace_bytes, bool counters_zeroed) {
    if (!gemm_tc_supported(a)) return cudaErrorInvalidValue;
    const bool dual = a.epilogue == EPI_SWIGLU;
    const uint32_t K = a.w.cols, out_dim = a.w.rows, n_rows = a.batch;
    if (n_rows == 0) return cudaSuccess;
    if (gemm_tc_workspace_bytes(out_dim, K, n_rows, dual) > workspace_bytes || ((uintptr_t)workspace & 1023) != 0) return cudaErrorInvalidValue;
    cudaError_t e = gemm_tc_init();
    if (e != cudaSuccess) return e;
    const uint64_t rows_pad = gemm_tc_rows_padded(n_rows);
    const uint64_t xb = (rows_pad * K * 2 + 1023) / 1024 * 1024, wb = ((uint64_t)out_dim * K * 2 + 1023) / 1024 * 1024;
    const bool narrow = n_rows <= 32;  // decode batches: 32 rows of x per tile, no tensor-core work on padding
    // prefill chunks: hi + lo parts of x (and of weights fp16 does not hold exactly); decode batches keep single parts
    const uint32_t x_parts = (!narrow && gemm_tc_split >= 1) ? 2u : 1u;
    const bool w_inexact = gemm_tc_weights_inexact(a.w.fmt) || (dual && gemm_tc_weights_inexact(a.w2.fmt));
    const uint32_t w_parts = (!narrow && gemm_tc_split >= 2 && w_inexact) ? 2u : 1u;
    __half* xh = reinterpret_cast<__half*>(reinterpret_cast<unsigned char*>(workspace) + WS_HEAD_BYTES);
    __half* xl = x_parts == 2 ? xh + rows_pad * K : nullptr;  // directly below the hi rows: one tensor map covers both
    unsigned char* wbase = reinterpret_cast<unsigned char*>(workspace) + WS_HEAD_BYTES + 2 * xb;

    // decode batches (<= 32 rows, one 32-row box of x): only those 32 rows are ever read
    e = launch(lc, k_rows_to_f16, dim3(narrow ? 32u : (unsigned)rows_pad), dim3(256), 0, xh, xl, a.x, a.norm_w, a.norm_fmt, a.eps, a.state, K, n_rows);
    if (e != cudaSuccess) return e;
    const void* wh[2] = {a.w.data, a.w2.data};
    const void* wl[2] = {nullptr, nullptr};
    const WMat* mats[2] = {&a.w, &a.w2};
    for (int i = 0; i < (dual ? 2 : 1); ++i) {
        const bool need_lo = w_parts == 2;
        if (mats[i]->fmt == VB_FMT_F16) {  // used where it lies (exact)
            if (need_lo) return cudaErrorInvalidValue;  // cannot happen: fp16 weights are never inexact
            continue;
        }
        if (mats[i]->f16 && (!need_lo || mats[i]->f16_lo)) { wh[i] = mats[i]->f16; wl[i] = mats[i]->f16_lo; continue; }  // resident copies
        const uint64_t n8 = (uint64_t)out_dim * K / 8;
        uint64_t blocks = (n8 + 255) / 256;
        if (blocks > 148ull * 64) blocks = 148ull * 64;
        unsigned char* hi = wbase + (size_t)i * 2 * wb;
        unsigned char* lo = need_lo ? hi + wb : nullptr;
        e = launch(lc, k_weights_to_f16, dim3((unsigned)blocks), dim3(256), 0, reinterpret_cast<uint4*>(hi), reinterpret_cast<uint4*>(lo), mats[i]->data,
                   mats[i]->scales, (int)mats[i]->fmt, n8, K);
        if (e != cudaSuccess) return e;
        wh[i] = hi;
        wl[i] = lo;
    }
    CUtensorMap mw, mw2, mx, mwl, mwl2;
    if (!make_map(&mw, wh[0], out_dim, K) || !make_map(&mx, xh, rows_pad * x_parts, K, narrow ? 32 : BM)) return cudaErrorNotSupported;
    if (dual) { if (!make_map(&mw2, wh[1], out_dim, K)) return cudaErrorNotSupported; } else mw2 = mw;
    mwl = mw; mwl2 = mw2;
    if (w_parts == 2) {
        if (!make_map(&mwl, wl[0], out_dim, K)) return cudaErrorNotSupported;
        if (dual && !make_map(&mwl2, wl[1], out_dim, K)) return cudaErrorNotSupported;
    }
    GemmParams p;
    p.dst = a.dst + a.dst_offset;
    p.row_scale = a.w.fmt == VB_FMT_I8PC ? (const __half*)a.w.scales : nullptr;
    p.row_scale2 = (dual && a.w2.fmt == VB_FMT_I8PC) ? (const __half*)a.w2.scales : nullptr;
    p.state = a.state;
    p.out_dim = out_dim; p.n_rows = n_rows; p.K = K;
    p.dst_stride = a.dst_stride ? a.dst_stride : out_dim;
    p.epilogue = a.epilogue;
    p.err = nullptr;
    fast_error_word(&p.err);
    p.counters = reinterpret_cast<uint32_t*>(workspace);
    p.part = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + WS_COUNTER_BYTES);
    p.x_parts = x_parts; p.w_parts = w_parts; p.x_lo_row = (uint32_t)rows_pad;
    auto stages_of = [&](int bn, int ring_kb) {
        const int stage = (dual ? 2 : 1) * (int)w_parts * TILE_BYTES + (int)x_parts * bn * BK * 2;
        return ring_kb * 1024 / stage;
    };
    if (narrow) {
        // few row tiles (QKV, O, down of a decode batch: 28-36 blocks on 148 SMs): split K so that every SM streams
        const uint32_t tiles = (out_dim + BM - 1) / BM, nk = (K + BK - 1) / BK;
        uint32_t splits = 1;
        if (!dual && counters_zeroed && gemm_tc_split_k && tiles * 2 <= 148) {
            splits = std::min(std::min(148u / tiles, 8u), std::max(nk / 8u, 1u));
            if ((uint64_t)splits * tiles * 128 * 32 * 4 > WS_PART_BYTES || tiles * 4 > WS_COUNTER_BYTES) splits = 1;
        }
        const dim3 grid(1, tiles, splits);
        p.stages = (uint32_t)stages_of(32, 192);
        if (dual) return launch(lc, k_gemm_tc<true, 32>, grid, dim3(128), SMEM_BYTES, mw, mw2, mx, mwl, mwl2, p);
        return launch(lc, k_gemm_tc<false, 32>, grid, dim3(128), SMEM_BYTES, mw, mw2, mx, mwl, mwl2, p);
    }
    // 256 rows of x per tile (half the weight traffic per flop) once there are more than 128 rows
    if (n_rows > 128 && gemm_tc_wide && stages_of(256, 192) >= 2) {
        const dim3 grid((unsigned)((rows_pad + 255) / 256), (out_dim + BM - 1) / BM);
        p.stages = (uint32_t)stages_of(256, 192);
        if (dual) return launch(lc, k_gemm_tc<true, 256>, grid, dim3(128), SMEM_BYTES, mw, mw2, mx, mwl, mwl2, p);
        return launch(lc, k_gemm_tc<false, 256>, grid, dim3(128), SMEM_BYTES, mw, mw2, mx, mwl, mwl2, p);
    }
    const dim3 grid((unsigned)(rows_pad / 128), (out_dim + BM - 1) / BM);
    if (gemm_tc_two_per_sm && stages_of(128, 96) >= 2) {  // half the ring per block, two blocks per SM
        p.stages = (uint32_t)stages_of(128, 96);
        if (dual) return launch(lc, k_gemm_tc<true, 128, 2>, grid, dim3(128), SMEM_BYTES_HALF, mw, mw2, mx, mwl, mwl2, p);
        return launch(lc, k_gemm_tc<false, 128, 2>, grid, dim3(128), SMEM_BYTES_HALF, mw, mw2, mx, mwl, mwl2, p);
    }
    p.stages = (uint32_t)stages_of(128, 192);
    if (p.stages < 2) return cudaErrorInvalidConfiguration;
    if (dual) return launch(lc, k_gemm_tc<true, 128>, grid, dim3(128), SMEM_BYTES, mw, mw2, mx, mwl, mwl2, p);
    return launch(lc, k_gemm_tc<false, 128>, grid, dim3(128), SMEM_BYTES, mw, mw2, mx, mwl, mwl2, p);
}

}  // namespace vb

extern "C" uint64_t vb_op_matmul_rows_workspace_bytes(uint32_t in_dim, uint32_t out_dim, uint32_t n_rows) {
    return vb::gemm_tc_workspace_bytes(out_dim, in_dim, n_rows, false);
}

extern "C" int32_t vb_op_matmul_rows(float* dst, const float* x, const void* w, const void* scales, int32_t fmt, uint32_t in_dim,
                                     uint32_t out_dim, uint32_t n_rows, void* workspace, uint64_t workspace_bytes, void* stream) {
    using namespace vb;
    VB_REQUIRE(dst && x && w && workspace, "vb_op_matmul_rows: null pointer");
    VB_REQUIRE(fmt >= VB_FMT_F32 && fmt <= VB_FMT_I8PC, "vb_op_matmul_rows: unknown format %d", fmt);
    VB_REQUIRE(in_dim > 0 && in_dim % 8 == 0 && fmt_shape_ok(fmt, in_dim), "vb_op_matmul_rows: in_dim=%u not valid for format %d", in_dim, fmt);
    VB_REQUIRE(wmat_scale_bytes(fmt, out_dim, in_dim) == 0 || scales, "vb_op_matmul_rows: format %d needs scales", fmt);
    VB_REQUIRE(((uintptr_t)workspace & 1023) == 0, "vb_op_matmul_rows: workspace must be 1024-byte aligned");
    VB_REQUIRE(fmt != VB_FMT_F16 || ((uintptr_t)w & 15) == 0, "vb_op_matmul_rows: fp16 weights must be 16-byte aligned");
    const uint64_t need = gemm_tc_workspace_bytes(out_dim, in_dim, n_rows, false);
    VB_REQUIRE(workspace_bytes >= need, "vb_op_matmul_rows: workspace too small (%llu bytes, %llu needed)",
               (unsigned long long)workspace_bytes, (unsigned long long)need);
    if (n_rows == 0 || out_dim == 0) return VB_OK;
    GemvArgs a;
    a.dst = dst; a.x = x;
    a.w.data = w; a.w.scales = scales; a.w.fmt = fmt; a.w.rows = out_dim; a.w.cols = in_dim;
    a.batch = n_rows;
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    VB_CUDA(kernels_init());
    VB_CUDA(gemm_tc(lc, a, workspace, workspace_bytes));
    return VB_OK;
}
