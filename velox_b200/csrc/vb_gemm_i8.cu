// Decode batches over int8 per-channel weights on the integer tensor cores (tcgen05.mma kind::i8): the weights cross
// HBM as the bytes they are stored as -- no fp16 copy, one byte per weight -- and the arithmetic is exact.
//
// What it replaces: the reference's multi-token register-tiled kernels (velox_cuda_runner_k2.cu:480-1085) for the
// projections of a batched decode step, dst[t][o] = sum_k x[t][k] * q[o][k] * scale[o] for up to 32 rows t.
//
//   * x rows (with the reference's RMSNorm folded in, runtime.rs:588-601) become 16-bit fixed point per row,
//     X = rint(x * p) with p = 32000 / (the row's largest magnitude), stored as two
//     signed byte planes X = 256 * H + L (k_rows_to_i8: rows 0..31 of the operand hold H, rows 32..63 hold L);
//   * the weights are read where they lie, canonical int8 [out][K], by tiled TMA ([128 rows][128 bytes] boxes,
//     128-byte swizzle); one tcgen05.mma kind::i8 (M 128, N 64, K 32) per 32 bytes of K accumulates int32 in tensor
//     memory: columns 0..31 = sum q*H, columns 32..63 = sum q*L, both exact;
//   * the epilogue forms (256 * D_H + D_L) * scale[o] / p in fp32 and stores / adds the residual / applies
//     SiLU(gate) * up; products with few row tiles split K over several blocks, the last one to arrive sums the fp32
//     partial tiles in split order (the same bits whoever is last).
// Every wait is bounded; a wait that runs out sets a block-wide abort flag and the library's error word.
#include <cuda.h>

#include <algorithm>

#include "vb_kernels.cuh"
#include "vb_tma.cuh"

namespace vb {
namespace {

constexpr int I8_BM = 128;               // weight rows per tile (UMMA M)
constexpr int I8_BN = 64;                // operand rows of x: 32 H rows + 32 L rows (UMMA N)
constexpr int I8_BK = 128;               // bytes of K per stage: one 128-byte swizzle row
constexpr int I8_W_BYTES = I8_BM * I8_BK;  // 16 KB
constexpr int I8_X_BYTES = I8_BN * I8_BK;  // 8 KB
constexpr int I8_SMEM = 192 * 1024 + 1024 + 256;

// instruction descriptor of tcgen05.mma kind::i8: int32 accumulate (bits 4-5 = 2), A and B signed 8-bit (formats 1 at
// bits 7-9 and 10-12), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
constexpr uint32_t I8_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(I8_BN >> 3) << 17) | ((uint32_t)(I8_BM >> 4) << 24);

__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(I8_IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void commit_to(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32i(uint32_t taddr, int r[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                   "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                   "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
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

struct I8Params {
    float* dst;                 // [n_rows][dst_stride], column offset applied
    const __half* row_scale;    // [out_dim] weight row scales
    const __half* row_scale2;   // gate/up: the up matrix's
    const float* x_inv_scale;   // [32] 1 / p of every row of x
    const SeqState* state;
    uint32_t out_dim, n_rows, K, dst_stride;
    int epilogue;
    uint32_t* err;
    float* part;                // [split][tile][32 cols][128 lanes] fp32 partial tiles
    uint32_t* counters;         // [tile], zero between launches
    uint32_t stages;
    unsigned long long* trace;  // time stamps of this launch (vb_trace_read), or null
    // tile-major copies of the weights in shared-memory order (null: tiled TMA from the canonical matrices): a tile is one
    // contiguous 16 KB bulk copy -- sequential DRAM pages instead of 128 rows of 128 bytes a whole matrix row apart
    const unsigned char* w_tiles;
    const unsigned char* w2_tiles;
};

template <bool DUAL>
__global__ void __launch_bounds__(128, 1)
k_gemm_i8(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ CUtensorMap map_x,
          const I8Params p) {
    constexpr int W_TILES = DUAL ? 2 : 1;
    constexpr int STAGE_BYTES = W_TILES * I8_W_BYTES + I8_X_BYTES;
    constexpr uint32_t TMEM_COLS = DUAL ? 2 * I8_BN : I8_BN;
    const int STAGES = (int)p.stages;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES * STAGE_BYTES;  // full[STAGES], empty[STAGES], accum, then two words
    const uint32_t bar_accum = bars + 2 * STAGES * 8;
    unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + STAGES * STAGE_BYTES + (2 * STAGES + 1) * 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.y * I8_BM;
    const int nk_all = (int)((p.K + I8_BK - 1) / I8_BK);
    const int kb_first = (int)(((long long)nk_all * blockIdx.z) / gridDim.z), kb_last = (int)(((long long)nk_all * (blockIdx.z + 1)) / gridDim.z);
    const int nk = kb_last - kb_first;
    trace_mark(p.trace, 0);

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
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // weights do not depend on the kernel before this one: the whole ring of weight tiles is requested before the
        // dependency wait, the planes of x (written by the conversion kernel in front) after it
        const int pre = nk < STAGES ? nk : STAGES;
        for (int kb = 0; kb < pre; ++kb) {
            const uint32_t full = bars + kb * 8, st = base + kb * STAGE_BYTES;
            mbar_expect_tx(full, STAGE_BYTES);
            const int kx = (kb_first + kb) * I8_BK;
            if (p.w_tiles) {
                const size_t toff = ((size_t)blockIdx.y * nk_all + kb_first + kb) * I8_W_BYTES;
                tma_load_1d(st, p.w_tiles + toff, I8_W_BYTES, full);
                if (DUAL) tma_load_1d(st + I8_W_BYTES, p.w2_tiles + toff, I8_W_BYTES, full);
            } else {
                tma_2d(st, &map_w, kx, row0, full);
                if (DUAL) tma_2d(st + I8_W_BYTES, &map_w2, kx, row0, full);
            }
        }
        pdl_wait();
        trace_mark(p.trace, 1);
        for (int kb = 0; kb < pre; ++kb) tma_2d(base + kb * STAGE_BYTES + W_TILES * I8_W_BYTES, &map_x, (kb_first + kb) * I8_BK, 0, bars + kb * 8);
        for (int kb = pre; kb < nk; ++kb) {
            const int s = kb % STAGES;
            const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
            if (!wait_abort(bars + (STAGES + s) * 8, ph ^ 1u, abort_flag)) break;
            const uint32_t full = bars + s * 8, st = base + s * STAGE_BYTES;
            mbar_expect_tx(full, STAGE_BYTES);
            const int kx = (kb_first + kb) * I8_BK;
            if (p.w_tiles) {
                const size_t toff = ((size_t)blockIdx.y * nk_all + kb_first + kb) * I8_W_BYTES;
                tma_load_1d(st, p.w_tiles + toff, I8_W_BYTES, full);
                if (DUAL) tma_load_1d(st + I8_W_BYTES, p.w2_tiles + toff, I8_W_BYTES, full);
            } else {
                tma_2d(st, &map_w, kx, row0, full);
                if (DUAL) tma_2d(st + I8_W_BYTES, &map_w2, kx, row0, full);
            }
            tma_2d(st + W_TILES * I8_W_BYTES, &map_x, kx, 0, full);
        }
    } else if (warp == 1 && lane == 0) {
        for (int kb = 0; kb < nk; ++kb) {
            const int s = kb % STAGES;
            const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
            if (!wait_abort(bars + s * 8, ph, abort_flag)) break;
            fence_after();
            const uint32_t st = base + s * STAGE_BYTES;
            const uint64_t da = smem_desc_sw128(st), da2 = smem_desc_sw128(st + I8_W_BYTES), db = smem_desc_sw128(st + W_TILES * I8_W_BYTES);
#pragma unroll
            for (int k = 0; k < I8_BK / 32; ++k) {  // 32 bytes further along the swizzled row: +2 in the address field
                const uint32_t acc = (kb | k) != 0 ? 1u : 0u;
                mma_i8(tmem, da + 2u * k, db + 2u * k, acc);
                if (DUAL) mma_i8(tmem + I8_BN, da2 + 2u * k, db + 2u * k, acc);
            }
            commit_to(bars + (STAGES + s) * 8);
        }
        commit_to(bar_accum);
    }
    __syncwarp();
    pdl_wait();               // every thread: the epilogue reads the residual stream and x scales of earlier kernels
    pdl_launch_dependents();

    // the scales of x and which of its rows are live, once per block (warp 0), for every lane's 32 columns
    __shared__ float s_inv[32];
    __shared__ uint32_t s_live_mask;
    if (warp == 0) {
        s_inv[lane] = p.x_inv_scale[lane];
        const bool live = lane < p.n_rows && (!p.state || p.state[lane].active);
        const uint32_t m = __ballot_sync(0xFFFFFFFFu, live);
        if (lane == 0) s_live_mask = m;
    }
    const bool ok = wait_abort(bar_accum, 0u, abort_flag);
    fence_after();
    const bool good = __syncthreads_and(ok && !*abort_flag);
    if (good) {
        const uint32_t o = (uint32_t)row0 + warp * 32 + lane;
        const bool o_ok = o < p.out_dim;
        const float sc = o_ok ? __half2float(p.row_scale[o]) : 0.0f;
        const float sc2 = (DUAL && o_ok) ? __half2float(p.row_scale2[o]) : 0.0f;
        const uint32_t lane_addr = tmem + ((warp * 32u) << 16);
        const uint32_t n_split = gridDim.z, tile = blockIdx.y, n_tiles = gridDim.y;
        // row j of x: 256 * (sum q*H) + (sum q*L), exact in int64, to fp32 once
        int h[32], l[32];
        float v[32], u[32];
        tmem_ld32i(lane_addr, h);
        tmem_ld32i(lane_addr + 32, l);
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (float)((long long)h[j] * 256 + (long long)l[j]);
        if (DUAL) {
            tmem_ld32i(lane_addr + I8_BN, h);
            tmem_ld32i(lane_addr + I8_BN + 32, l);
#pragma unroll
            for (int j = 0; j < 32; ++j) u[j] = (float)((long long)h[j] * 256 + (long long)l[j]);
        }
        bool reduce = false;
        if (!DUAL && n_split > 1) {
            __shared__ uint32_t s_last;
            float* pt = p.part + (((size_t)blockIdx.z * n_tiles + tile) * 32) * 128 + threadIdx.x;
#pragma unroll
            for (int j = 0; j < 32; ++j) __stcg(pt + j * 128, v[j]);
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                const uint32_t old = atomicAdd(p.counters + tile, 1u);
                s_last = old == n_split - 1 ? 1u : 0u;
                if (s_last) { p.counters[tile] = 0u; __threadfence(); }
            }
            __syncthreads();
            reduce = s_last != 0u;
            if (reduce) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.0f;
                for (uint32_t z = 0; z < n_split; ++z) {
                    const float* ps = p.part + (((size_t)z * n_tiles + tile) * 32) * 128 + threadIdx.x;
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += __ldcg(ps + j * 128);
                }
            }
        }
        if ((DUAL || n_split == 1 || reduce) && o_ok) {
            const uint32_t live_mask = s_live_mask;
            float* d0 = p.dst + o;
            float res[32];
            if (!DUAL && p.epilogue == EPI_RESIDUAL) {
#pragma unroll
                for (int j = 0; j < 32; ++j) res[j] = ((live_mask >> j) & 1u) ? __ldcg(d0 + (size_t)j * p.dst_stride) : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float inv = s_inv[j];
                if (!((live_mask >> j) & 1u)) continue;
                const float a = (v[j] * inv) * sc;
                if (DUAL) {
                    const float up = (u[j] * inv) * sc2;
                    d0[(size_t)j * p.dst_stride] = (a / (1.0f + expf(-a))) * up;
                } else if (p.epilogue == EPI_RESIDUAL) {
                    d0[(size_t)j * p.dst_stride] = res[j] + a;
                } else {
                    d0[(size_t)j * p.dst_stride] = a;
                }
            }
        }
    } else {
        if (threadIdx.x == 0 && p.err) atomicOr(p.err, 0x80u);
        const long long t0 = clock64();
        while (clock64() - t0 < 20000000LL) { }
    }
    fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    trace_exit(p.trace);
}

// One block per row of x (32 blocks): planes[r][k] = H, planes[32 + r][k] = L of X = rint(norm(x) * p); inv_scale[r] = 1 / p.
// Rows of inactive slots and rows past n_rows are zeros.
__global__ void __launch_bounds__(256)
k_rows_to_i8(int8_t* __restrict__ planes, float* __restrict__ inv_scale, const float* __restrict__ x, const void* __restrict__ norm_w, int norm_fmt,
             float eps, const SeqState* __restrict__ state, uint32_t K, uint32_t n_rows) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t r = blockIdx.x;
    int8_t* hp = planes + (size_t)r * K;
    int8_t* lp = planes + (size_t)(32 + r) * K;
    const bool live = r < n_rows && (!state || state[r].active);
    const uint32_t K4 = K / 4;
    if (!live) {
        for (uint32_t k = threadIdx.x; k < K4; k += blockDim.x) { reinterpret_cast<uint32_t*>(hp)[k] = 0u; reinterpret_cast<uint32_t*>(lp)[k] = 0u; }
        if (threadIdx.x == 0) inv_scale[r] = 0.0f;
        return;
    }
    __shared__ float part[8], part_mx[8];
    const float4* in4 = reinterpret_cast<const float4*>(x + (size_t)r * K);
    float inv = 1.0f;
    if (norm_w) {
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
    auto normed = [&](uint32_t k) {
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
        return v;
    };
    float mx = 0.0f;
    for (uint32_t k = threadIdx.x; k < K4; k += blockDim.x) {
        const float4 v = normed(k);
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) part_mx[threadIdx.x >> 5] = mx;
    __syncthreads();
    float gmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) gmax = fmaxf(gmax, part_mx[i]);
    float pw = 1.0f;  // brings the row's largest magnitude to 32000; 1 for an all-zero or non-finite row
    if (gmax > 0.0f && gmax < 3.0e38f) pw = __fdividef(32000.0f, gmax);
    if (!(pw < 3.0e38f)) pw = 1.0f;
    if (threadIdx.x == 0) inv_scale[r] = 1.0f / pw;
    for (uint32_t k = threadIdx.x; k < K4; k += blockDim.x) {
        const float4 v = normed(k);
        const float e[4] = {v.x, v.y, v.z, v.w};
        uint32_t hw = 0, lw = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int X = __float2int_rn(e[i] * pw);
            X = max(-32639, min(32639, X));
            const int H = (X + 128) >> 8, L = X - (H << 8);
            hw |= (uint32_t)(H & 0xFF) << (8 * i);
            lw |= (uint32_t)(L & 0xFF) << (8 * i);
        }
        reinterpret_cast<uint32_t*>(hp)[k] = hw;
        reinterpret_cast<uint32_t*>(lp)[k] = lw;
    }
}

// The same conversion for rows of up to 4096 * XR elements in one trip through memory: 1024 threads hold the row in
// registers (XR float4 each), so the sum of squares, the largest magnitude and the two byte planes all come from one
// load; the three passes of the kernel above cost three dependent round trips per row (5-9 us, four times a layer).
template <int XR>
__global__ void __launch_bounds__(1024)
k_rows_to_i8_regs(int8_t* __restrict__ planes, float* __restrict__ inv_scale, const float* __restrict__ x, const void* __restrict__ norm_w,
                  int norm_fmt, float eps, const SeqState* __restrict__ state, uint32_t K, uint32_t n_rows) {
    pdl_launch_dependents();  // the product's set-up (tensor maps, tensor memory, its first weight tiles) runs beside this
    const uint32_t r = blockIdx.x, K4 = K / 4, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int8_t* hp = planes + (size_t)r * K;
    int8_t* lp = planes + (size_t)(32 + r) * K;
    __shared__ float red[32];
    __shared__ float bc[2];
    // norm weights are weights: on their way before the producer of x is done
    float4 w[XR];
    if (norm_w) {
#pragma unroll
        for (int i = 0; i < XR; ++i) {
            const uint32_t k = threadIdx.x + i * 1024;
            w[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k < K4) {
                if (norm_fmt == VB_FMT_F16) {
                    const uint2 raw = reinterpret_cast<const uint2*>(norm_w)[k];
                    const float2 w01 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x)), w23 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    w[i] = make_float4(w01.x, w01.y, w23.x, w23.y);
                } else {
                    w[i] = reinterpret_cast<const float4*>(norm_w)[k];
                }
            }
        }
    }
    pdl_wait();
    const bool live = r < n_rows && (!state || state[r].active);
    if (!live) {
        for (uint32_t k = threadIdx.x; k < K4; k += blockDim.x) { reinterpret_cast<uint32_t*>(hp)[k] = 0u; reinterpret_cast<uint32_t*>(lp)[k] = 0u; }
        if (threadIdx.x == 0) inv_scale[r] = 0.0f;
        return;
    }
    const float4* in4 = reinterpret_cast<const float4*>(x + (size_t)r * K);
    float4 v[XR];
#pragma unroll
    for (int i = 0; i < XR; ++i) {
        const uint32_t k = threadIdx.x + i * 1024;
        v[i] = k < K4 ? in4[k] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (norm_w) {
        // the same order of squares within a thread as the three-pass kernel would not be reproducible anyway (other
        // thread count); the checker's bound is on the product, not on these bits
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < XR; ++i) { ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss); ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss); }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (warp == 0) {
            float t = warp_sum(red[lane]);
            if (lane == 0) bc[0] = 1.0f / sqrtf(t / (float)K + eps);
        }
        __syncthreads();
        const float inv = bc[0];
#pragma unroll
        for (int i = 0; i < XR; ++i) {
            v[i].x = (v[i].x * inv) * w[i].x; v[i].y = (v[i].y * inv) * w[i].y; v[i].z = (v[i].z * inv) * w[i].z; v[i].w = (v[i].w * inv) * w[i].w;
        }
    }
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < XR; ++i) mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
    mx = warp_max(mx);
    __syncthreads();  // red[] is read no more
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (warp == 0) {
        const float g = warp_max(red[lane]);
        if (lane == 0) bc[1] = g;
    }
    __syncthreads();
    const float gmax = bc[1];
    float pw = 1.0f;  // brings the row's largest magnitude to 32000; 1 for an all-zero or non-finite row
    if (gmax > 0.0f && gmax < 3.0e38f) pw = __fdividef(32000.0f, gmax);
    if (!(pw < 3.0e38f)) pw = 1.0f;
    if (threadIdx.x == 0) inv_scale[r] = 1.0f / pw;
#pragma unroll
    for (int i = 0; i < XR; ++i) {
        const uint32_t k = threadIdx.x + i * 1024;
        if (k < K4) {
            const float e[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
            uint32_t hw = 0, lw = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int X = __float2int_rn(e[j] * pw);
                X = max(-32639, min(32639, X));
                const int H = (X + 128) >> 8, L = X - (H << 8);
                hw |= (uint32_t)(H & 0xFF) << (8 * j);
                lw |= (uint32_t)(L & 0xFF) << (8 * j);
            }
            reinterpret_cast<uint32_t*>(hp)[k] = hw;
            reinterpret_cast<uint32_t*>(lp)[k] = lw;
        }
    }
}

// dst tile (row tile rt, k block kb) at ((rt * n_kb) + kb) * 16 KB: byte b of the 16-byte piece c of row r at
// r * 128 + ((c ^ (r & 7)) << 4) + b -- what a tiled TMA copy with the 128-byte swizzle would have written; rows past the
// matrix are zeros.  One thread per 16-byte piece.
__global__ void __launch_bounds__(256)
k_tile_i8_umma(uint4* __restrict__ dst, const int8_t* __restrict__ src, uint32_t rows, uint32_t K, uint32_t n_kb, uint64_t n_pieces) {
    const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n_pieces) return;
    const uint32_t c = (uint32_t)(i & 7), r = (uint32_t)((i >> 3) & 127);
    const uint64_t tile = i >> 10;
    const uint32_t kb = (uint32_t)(tile % n_kb), rt = (uint32_t)(tile / n_kb);
    const uint32_t row = rt * 128 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows) v = *reinterpret_cast<const uint4*>(src + (size_t)row * K + (size_t)kb * 128 + c * 16);
    dst[tile * 1024 + r * 8 + (c ^ (r & 7))] = v;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn_i8() {
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
// int8 [rows][K] row-major, boxes of [box_rows][128 bytes], 128-byte swizzle, zeros outside the matrix
bool make_map_i8(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t K, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn_i8();
    if (!fn) return false;
    const cuuint64_t dims[2] = {K, rows};
    const cuuint64_t strides[1] = {K};
    const cuuint32_t box[2] = {I8_BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool g_i8_init = false;
constexpr uint64_t I8_COUNTER_BYTES = 64 * 1024, I8_PART_BYTES = 4 * 1024 * 1024;

}  // namespace

bool gemm_i8_half_ring = true;  // vb_set_option("i8_half_ring", 0): every block of k_gemm_i8 takes a whole SM's shared memory
bool gemm_i8_tiles = true;  // vb_set_option("i8_tiles", 0): weight tiles by tiled TMA from the canonical matrices instead of the tile-major copies
bool gemm_i8_enabled = true;  // vb_set_option("decode_gemm_i8", 0): decode batches over int8 weights go through the fp16 copies again

cudaError_t gemm_i8_init() {
    if (g_i8_init) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(k_gemm_i8<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, I8_SMEM);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(k_gemm_i8<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, I8_SMEM);
    if (e != cudaSuccess) return e;
    g_i8_init = true;
    return cudaSuccess;
}

bool gemm_i8_supported(const GemvArgs& a) {
    if (!gemm_i8_enabled || a.w.fmt != VB_FMT_I8PC || a.batch == 0 || a.batch > 32 || !a.w.data || !a.w.scales) return false;
    if (a.w.cols % 16 != 0 || a.w.rows == 0 || ((uintptr_t)a.w.data & 15) != 0) return false;
    if (a.epilogue == EPI_SWIGLU && (a.w2.fmt != VB_FMT_I8PC || a.w2.rows != a.w.rows || a.w2.cols != a.w.cols || !a.w2.data || !a.w2.scales ||
                                     ((uintptr_t)a.w2.data & 15) != 0))
        return false;
    return a.push.links == nullptr;
}

uint64_t gemm_i8_tiles_bytes(uint32_t rows, uint32_t K) {
    return K % I8_BK ? 0 : (uint64_t)((rows + I8_BM - 1) / I8_BM) * (K / I8_BK) * I8_W_BYTES;
}
cudaError_t gemm_i8_make_tiles(const LaunchCfg& lc, void* dst, const void* src_i8, uint32_t rows, uint32_t K) {
    if (K % I8_BK != 0 || ((uintptr_t)dst & 15) != 0 || ((uintptr_t)src_i8 & 15) != 0) return cudaErrorInvalidValue;
    const uint32_t n_kb = K / I8_BK;
    const uint64_t n_pieces = gemm_i8_tiles_bytes(rows, K) / 16;
    return launch(lc, k_tile_i8_umma, dim3((unsigned)((n_pieces + 255) / 256)), dim3(256), 0, reinterpret_cast<uint4*>(dst),
                  reinterpret_cast<const int8_t*>(src_i8), rows, K, n_kb, n_pieces);
}

// workspace head: tile counters (zero before the first call) and partial tiles, then the planes of x and their scales
uint64_t gemm_i8_workspace_bytes(uint32_t in_dim) {
    return I8_COUNTER_BYTES + I8_PART_BYTES + (((uint64_t)64 * in_dim + 1023) / 1024 * 1024) + 1024;
}

cudaError_t gemm_i8(const LaunchCfg& lc, const GemvArgs& a, void* workspace, uint64_t workspace_bytes, bool counters_zeroed) {
    if (!gemm_i8_supported(a)) return cudaErrorInvalidValue;
    const bool dual = a.epilogue == EPI_SWIGLU;
    const uint32_t K = a.w.cols, out_dim = a.w.rows, n_rows = a.batch;
    if (gemm_i8_workspace_bytes(K) > workspace_bytes || ((uintptr_t)workspace & 1023) != 0) return cudaErrorInvalidValue;
    cudaError_t e = gemm_i8_init();
    if (e != cudaSuccess) return e;
    unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
    int8_t* planes = reinterpret_cast<int8_t*>(ws + I8_COUNTER_BYTES + I8_PART_BYTES);
    float* inv_scale = reinterpret_cast<float*>(ws + I8_COUNTER_BYTES + I8_PART_BYTES + (((uint64_t)64 * K + 1023) / 1024 * 1024));
    if (K <= 4096)
        e = launch(lc, k_rows_to_i8_regs<1>, dim3(32), dim3(1024), 0, planes, inv_scale, a.x, a.norm_w, a.norm_fmt, a.eps, a.state, K, n_rows);
    else if (K <= 8192)
        e = launch(lc, k_rows_to_i8_regs<2>, dim3(32), dim3(1024), 0, planes, inv_scale, a.x, a.norm_w, a.norm_fmt, a.eps, a.state, K, n_rows);
    else if (K <= 20480)
        e = launch(lc, k_rows_to_i8_regs<5>, dim3(32), dim3(1024), 0, planes, inv_scale, a.x, a.norm_w, a.norm_fmt, a.eps, a.state, K, n_rows);
    else
        e = launch(lc, k_rows_to_i8, dim3(32), dim3(256), 0, planes, inv_scale, a.x, a.norm_w, a.norm_fmt, a.eps, a.state, K, n_rows);
    if (e != cudaSuccess) return e;
    CUtensorMap mw, mw2, mx;
    if (!make_map_i8(&mw, a.w.data, out_dim, K, I8_BM) || !make_map_i8(&mx, planes, 64, K, I8_BN)) return cudaErrorNotSupported;
    if (dual) { if (!make_map_i8(&mw2, a.w2.data, out_dim, K, I8_BM)) return cudaErrorNotSupported; } else mw2 = mw;
    I8Params p;
    p.dst = a.dst + a.dst_offset;
    p.row_scale = (const __half*)a.w.scales;
    p.row_scale2 = dual ? (const __half*)a.w2.scales : nullptr;
    p.x_inv_scale = inv_scale;
    p.state = a.state;
    p.out_dim = out_dim; p.n_rows = n_rows; p.K = K;
    p.dst_stride = a.dst_stride ? a.dst_stride : out_dim;
    p.epilogue = a.epilogue;
    p.err = nullptr;
    fast_error_word(&p.err);
    p.counters = reinterpret_cast<uint32_t*>(ws);
    p.part = reinterpret_cast<float*>(ws + I8_COUNTER_BYTES);
    const uint32_t tiles = (out_dim + I8_BM - 1) / I8_BM, nk = (K + I8_BK - 1) / I8_BK;
    uint32_t splits = 1;
    if (!dual && counters_zeroed && gemm_tc_split_k && tiles * 2 <= 148) {
        splits = std::min(std::min(148u / tiles, 8u), std::max(nk / 8u, 1u));
        if ((uint64_t)splits * tiles * 128 * 32 * 4 > I8_PART_BYTES || tiles * 4 > I8_COUNTER_BYTES) splits = 1;
    }
    // single products with more tiles than SMs (the lm_head: 1188): half the shared memory of an SM per block (4 stages),
    // two blocks per SM, so that one block's weights are on the way while the other is in its epilogue: 123 -> 94 us.
    // One-wave products measured ~1 us slower that way and keep the whole ring, as does gate/up (two weight tiles per stage).
    const uint32_t stage_bytes = (dual ? 2 : 1) * I8_W_BYTES + I8_X_BYTES;
    p.stages = (uint32_t)(192 * 1024 / stage_bytes);
    if (!dual && gemm_i8_half_ring && tiles * splits > 148) p.stages = 4;
    const size_t smem = (size_t)p.stages * stage_bytes + 1024 + 256;
    p.trace = a.trace;
    const bool use_tiles = gemm_i8_tiles && a.w.i8_tiles && (!dual || a.w2.i8_tiles) && K % I8_BK == 0;
    p.w_tiles = use_tiles ? reinterpret_cast<const unsigned char*>(a.w.i8_tiles) : nullptr;
    p.w2_tiles = (use_tiles && dual) ? reinterpret_cast<const unsigned char*>(a.w2.i8_tiles) : p.w_tiles;
    const dim3 grid(1, tiles, splits);
    if (dual) return launch(lc, k_gemm_i8<true>, grid, dim3(128), smem, mw, mw2, mx, p);
    return launch(lc, k_gemm_i8<false>, grid, dim3(128), smem, mw, mw2, mx, p);
}

}  // namespace vb
