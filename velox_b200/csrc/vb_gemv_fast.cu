// Tuned matrix-vector kernel for symmetric int4 group-32 weights (VB_FMT_Q4G32), batch 1..8 per launch row.
//
// Storage.  Besides the canonical copy, the weight arena holds a TILE-MAJOR copy of every int4 matrix:
// the matrix is cut into blocks of 16 rows x 128 columns (4 quantization groups); a block is 1 KiB and is
// laid out so that lane L = 4*g + t of a warp finds at byte 16*L the four packed words of row g that hold
// elements [8t, 8t+8) of groups 0..3, and at byte 512 + 16*L the same for row g + 8.  One warp therefore
// reads a block with two conflict-free 512-byte accesses (128 bits per lane) and what it gets IS the
// A-operand fragment layout of mma.m16n8k16: no shuffles, no transpose.  The block's 64 fp16 scales follow
// at byte 1024 (16 bytes per g: row g groups 0..3, row g+8 groups 0..3), so a block is 1152 contiguous
// bytes.  Blocks are ordered [row tile][k tile]: a row tile's whole K extent is one contiguous run, which is
// what lets a single thread move it with bulk asynchronous copies (TMA).
//
// Arithmetic.  HBM delivers ~45 int4 weights per SM per clock on B200, more than CUDA cores can multiply
// after a per-element int->float conversion.  So nibbles are turned into fp16 by OR-ing them into the
// mantissa of 1024.0 (low nibble of each byte: 1024+q; high nibble, unshifted: 1024+16q), 5 integer
// instructions per 8 weights, and the dot products run on the tensor cores (mma.sync m16n8k16, fp16
// operands, fp32 accumulate) against x staged in shared memory as fp16 (high-nibble positions pre-scaled by
// 1/16).  The constant parts, 1032*x and 72*x per element, depend only on x: they are summed once per
// group of 32 while staging (`ncorr`) and enter the accumulator as its initial value, so the accumulator
// holds sum((q-8)*x) for exactly one quantization group after two mma; it is then scaled by that group's
// fp32(scale) and added to the row's fp32 sum.  Products are exact, sums are fp32.
//
// Data movement (batch 1, k_gemv_q4_tma).  Blocks are persistent (two per SM).  A ninth, producer warp streams
// the block's row tiles through a ring of shared-memory stages with cp.async.bulk (1-D TMA) completing on
// mbarriers; the eight consumer warps wait on a stage's "full" barrier, each takes one 16x128 block of it,
// and they hand the stage back through its "empty" barrier.  The ring keeps ~70 KB per block (~140 KB per
// SM) in flight regardless of register pressure, which is what the HBM latency-bandwidth product needs.
// Every barrier wait is bounded: on expiry the thread records an error code in global memory and carries on
// (the result is then garbage but the kernel ends), and the host reports VB_ERR_TIMEOUT.
//
// Overlap.  Kernels are launched with programmatic stream serialization.  Weights never depend on the
// previous kernel, so the producer warp starts filling the ring at once, while the consumers trigger their
// own dependents and only then wait for the producer kernel's x.
#include <string.h>

#include "vb_internal.cuh"
#include "vb_kernels.cuh"
#include "vb_tma.cuh"

namespace vb {

constexpr int FAST_WARPS = 8;
constexpr int FAST_THREADS = FAST_WARPS * 32;
constexpr int FAST_PF = 2;            // blocks in flight per warp and buffer
constexpr int FAST_KC_BATCHED = 4096; // x columns staged at a time when 8 sequences share a block and the row is too long to stage whole
constexpr int FAST_XPAD = 32;         // halves of padding between staged x rows (bank spread)
constexpr int BLK_U4 = 72;            // uint4 per 16x128 block: 64 of packed weights + 8 of scales (1152 bytes)
constexpr int BLK_BYTES = BLK_U4 * 16;
constexpr int TMA_SB = 8;             // blocks per pipeline stage = one per consumer warp
constexpr int TMA_STAGE_BYTES = TMA_SB * BLK_BYTES;
constexpr int TMA_MAX_STAGES = 8;
constexpr int TMA_THREADS = FAST_THREADS + 32;  // + the producer warp

struct FastArgs {
    const uint4* w[2];     // tile-major blocks (second matrix for SwiGLU)
    uint32_t* err;         // device error word (set when a bounded wait expires)
    uint32_t n_stages;     // pipeline depth of the TMA kernel
    uint32_t rows, K;
    const float* x;        // [batch][K]
    float* dst;
    const void* norm_w; int norm_fmt; float eps;
    const SeqState* state;
    uint32_t batch, dst_stride, dst_offset;
    int epilogue;
    uint32_t kc;           // batched: x columns staged at a time (== K: staged once, persistent loop over the tiles)
};

__device__ __forceinline__ void mma16816(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1, const float c[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

__device__ __forceinline__ void prefetch_l2_bulk(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// One 16x128 block: 8 mma, accumulating scale * sum((q-8)*x) per group into acc[0..3]
// (acc[0],acc[1]: row g, columns 2t,2t+1; acc[2],acc[3]: row g+8).
template <bool BATCHED>
__device__ __forceinline__ void block_mma(const uint4& wa, const uint4& wb, const uint4& sc, const __half* __restrict__ xs_lane,
                                          const float* __restrict__ ncorr_lane, uint32_t ncorr_stride, float acc[4]) {
    const uint32_t MASK_LO = 0x000F000Fu, MASK_HI = 0x00F000F0u, MAGIC = 0x64006400u;
    const uint32_t war[4] = {wa.x, wa.y, wa.z, wa.w};
    const uint32_t wbr[4] = {wb.x, wb.y, wb.z, wb.w};
    const __half2 sg[2] = {*reinterpret_cast<const __half2*>(&sc.x), *reinterpret_cast<const __half2*>(&sc.y)};
    const __half2 sh[2] = {*reinterpret_cast<const __half2*>(&sc.z), *reinterpret_cast<const __half2*>(&sc.w)};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t a = war[j], b = wbr[j], a8 = a >> 8, b8 = b >> 8;
        const uint4 xv = *reinterpret_cast<const uint4*>(xs_lane + 32 * j);
        float c[4], d[4];
        if (BATCHED) {
            // columns 2t and 2t+1 are different sequences: each has its own correction
            c[0] = c[2] = ncorr_lane[j];
            c[1] = c[3] = ncorr_lane[j + ncorr_stride];
        } else {
            c[0] = c[1] = c[2] = c[3] = ncorr_lane[j];
        }
        mma16816(d, lop3_and_or(a, MASK_LO, MAGIC), lop3_and_or(b, MASK_LO, MAGIC), lop3_and_or(a, MASK_HI, MAGIC),
                 lop3_and_or(b, MASK_HI, MAGIC), xv.x, xv.y, c);
        mma16816(d, lop3_and_or(a8, MASK_LO, MAGIC), lop3_and_or(b8, MASK_LO, MAGIC), lop3_and_or(a8, MASK_HI, MAGIC),
                 lop3_and_or(b8, MASK_HI, MAGIC), xv.z, xv.w, d);
        const float s_g = (j & 1) ? __high2float(sg[j >> 1]) : __low2float(sg[j >> 1]);
        const float s_h = (j & 1) ? __high2float(sh[j >> 1]) : __low2float(sh[j >> 1]);
        acc[0] = fmaf(s_g, d[0], acc[0]);
        acc[2] = fmaf(s_h, d[2], acc[2]);
        if (BATCHED) {
            acc[1] = fmaf(s_g, d[1], acc[1]);
            acc[3] = fmaf(s_h, d[3], acc[3]);
        }
    }
}

__device__ __forceinline__ float norm_w_f(const void* w, int fmt, uint32_t i) {
    return fmt == VB_FMT_F16 ? __half2float(((const __half*)w)[i])
         : fmt == VB_FMT_BF16 ? __bfloat162float(((const __nv_bfloat16*)w)[i]) : ((const float*)w)[i];
}

// Stage columns [k0, k0+kc) of one x row: fp16 of x * mul (mul = RMSNorm factor times a power of two that
// brings the row's largest magnitude to [256, 512), so fp16 keeps 11 significant bits whatever the scale of
// x), with the high-nibble positions (k % 4 >= 2) scaled by 1/16, and per group of 32 the negated constant
// term -(1032*sum_low + 1152*sum_high_scaled).  All 32 lanes of a warp run every iteration (shuffles).
__device__ __forceinline__ void stage_x_row(__half* __restrict__ xs, float* __restrict__ ncorr, const float* __restrict__ x,
                                            const void* norm_w, int norm_fmt, float mul, uint32_t k0, uint32_t kc) {
    const uint32_t n = kc / 8;
    for (uint32_t c0 = 0; c0 < n; c0 += FAST_THREADS) {
        const uint32_t c = c0 + threadIdx.x;
        const bool valid = c < n;  // groups of 4 lanes are valid together (n is a multiple of 16)
        float corr = 0.0f;
        if (valid) {
            const uint32_t k = k0 + c * 8;
            const float4 v0 = *reinterpret_cast<const float4*>(x + k);
            const float4 v1 = *reinterpret_cast<const float4*>(x + k + 4);
            float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            if (norm_w) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = (v[i] * mul) * norm_w_f(norm_w, norm_fmt, k + i);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] *= mul;
            }
            __half2 h[4];
            h[0] = __floats2half2_rn(v[0], v[1]);
            h[1] = __floats2half2_rn(v[2] * 0.0625f, v[3] * 0.0625f);
            h[2] = __floats2half2_rn(v[4], v[5]);
            h[3] = __floats2half2_rn(v[6] * 0.0625f, v[7] * 0.0625f);
            const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
            corr = 1032.0f * ((f0.x + f0.y) + (f2.x + f2.y)) + 1152.0f * ((f1.x + f1.y) + (f3.x + f3.y));
            *reinterpret_cast<uint4*>(xs + c * 8) = *reinterpret_cast<const uint4*>(h);
        }
        corr += __shfl_xor_sync(0xFFFFFFFFu, corr, 1);
        corr += __shfl_xor_sync(0xFFFFFFFFu, corr, 2);
        if (valid && (threadIdx.x & 3) == 0) ncorr[c >> 2] = -corr;
    }
}

// Load this warp's next FAST_PF blocks (kt, kt+8, ...) of one row tile into registers.
__device__ __forceinline__ void load_batch(uint4 wa[FAST_PF], uint4 wb[FAST_PF], uint4 sc[FAST_PF], const uint4* __restrict__ wt,
                                           uint32_t kt, uint32_t kt_hi, uint32_t lane, uint32_t g) {
#pragma unroll
    for (int p = 0; p < FAST_PF; ++p) {
        const uint32_t kk = kt + p * FAST_WARPS;
        if (kk < kt_hi) {
            const uint4* blk = wt + (size_t)kk * BLK_U4;
            wa[p] = ldg_stream(blk + lane);
            wb[p] = ldg_stream(blk + 32 + lane);
            sc[p] = __ldg(blk + 64 + g);
        }
    }
}

// Persistent blocks: grid (min(row tiles, 2 per SM), batch groups).  A block stages x once, then walks its
// row tiles (tile = blockIdx.x, += gridDim.x); its 8 warps split the K extent of the current 16-row tile.
template <bool BATCHED, bool DUAL>
__global__ void __launch_bounds__(FAST_THREADS, 2) k_gemv_q4_mma(FastArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int NB = BATCHED ? 8 : 1;
    constexpr int NM = DUAL ? 2 : 1;
    constexpr int RED = FAST_WARPS * NM * 16 * NB;
    const uint32_t K = a.K, KT = K / 128, n_tiles = a.rows / 16;
    const uint32_t kc_max = BATCHED ? min(K, a.kc) : K;
    const bool single = (kc_max == K);  // the whole row fits the staging buffer: stage once, loop over tiles
    const uint32_t xstride = kc_max + FAST_XPAD;
    __half* xs = reinterpret_cast<__half*>(smem_raw);                         // [NB][xstride]
    float* ncorr = reinterpret_cast<float*>(xs + (size_t)NB * xstride);        // [NB][kc_max/32]
    float* red = ncorr + (size_t)NB * (kc_max / 32);                            // [2][FAST_WARPS][NM][16][NB]
    __shared__ float ssq[FAST_WARPS], smx[FAST_WARPS];
    __shared__ float mul_s[8], unscale_s[8];

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const uint32_t b0 = blockIdx.y * NB;
    uint32_t tile = blockIdx.x;

    // ---- prologue: nothing here depends on the producer kernel ---------------------------------------
    if (threadIdx.x == 0) {
        for (uint32_t tt = tile, i = 0; i < 2 && tt < n_tiles; ++i, tt += gridDim.x) {
#pragma unroll
            for (int m = 0; m < NM; ++m) prefetch_l2_bulk(a.w[m] + (size_t)tt * KT * BLK_U4, KT * BLK_BYTES);
        }
    }
    uint4 wa[FAST_PF], wb[FAST_PF], sc[FAST_PF];
    load_batch(wa, wb, sc, a.w[0] + (size_t)tile * KT * BLK_U4, warp, min(KT, kc_max / 128), lane, g);
    bool preloaded = true;
    pdl_launch_dependents();
    pdl_wait();

    // ---- activity of the sequences of this block ---------------------------------------------------------
    bool any_active = false;
    for (int i = 0; i < NB; ++i) {
        const uint32_t b = b0 + i;
        if (b < a.batch && (!a.state || a.state[b].active)) any_active = true;
    }
    if (!any_active) return;

    // ---- row statistics: sum of squares (RMSNorm) and largest magnitude (fp16 staging scale) ------------------
    for (int i = 0; i < NB; ++i) {
        const uint32_t b = min(b0 + i, a.batch - 1);
        const float* x = a.x + (size_t)b * K;
        float ss = 0.0f, mx = 0.0f;
        for (uint32_t k = threadIdx.x * 4; k < K; k += FAST_THREADS * 4) {
            const float4 v = *reinterpret_cast<const float4*>(x + k);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            if (a.norm_w) {
                mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x * norm_w_f(a.norm_w, a.norm_fmt, k)), fabsf(v.y * norm_w_f(a.norm_w, a.norm_fmt, k + 1))),
                                     fmaxf(fabsf(v.z * norm_w_f(a.norm_w, a.norm_fmt, k + 2)), fabsf(v.w * norm_w_f(a.norm_w, a.norm_fmt, k + 3)))));
            } else {
                mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
        }
        ss = warp_sum(ss);
        mx = warp_max(mx);
        if (lane == 0) { ssq[warp] = ss; smx[warp] = mx; }
        __syncthreads();
        if (threadIdx.x == 0) {
            float tot = 0.0f, m = 0.0f;
            for (int w = 0; w < FAST_WARPS; ++w) { tot += ssq[w]; m = fmaxf(m, smx[w]); }
            const float inv = a.norm_w ? 1.0f / sqrtf(tot / (float)K + a.eps) : 1.0f;
            const float amax = m * inv;
            // power of two p with amax * p in [256, 512); 1 for an all-zero or non-finite row
            float p = 1.0f;
            if (amax > 0.0f && amax < 3.0e38f) p = exp2f((float)(8 - ilogbf(amax)));
            mul_s[i] = inv * p;
            unscale_s[i] = 1.0f / p;
        }
        __syncthreads();
    }
    if (single) {
        for (int i = 0; i < NB; ++i) {
            const uint32_t b = min(b0 + i, a.batch - 1);
            stage_x_row(xs + (size_t)i * xstride, ncorr + (size_t)i * (kc_max / 32), a.x + (size_t)b * K, a.norm_w, a.norm_fmt,
                        mul_s[i], 0, K);
        }
        __syncthreads();
    }

    const uint32_t xrow = BATCHED ? g : 0;       // column n = g of the B operand is sequence b0 + g
    const uint32_t crow0 = BATCHED ? 2 * t : 0;  // accumulator columns 2t, 2t+1
    uint32_t parity = 0;
    for (; tile < n_tiles; tile += gridDim.x, parity ^= 1) {
        if (threadIdx.x == 0) {
            const uint32_t tt = tile + 2 * gridDim.x;  // keep the L2 prefetch two tiles ahead
            if (tt < n_tiles) {
#pragma unroll
                for (int m = 0; m < NM; ++m) prefetch_l2_bulk(a.w[m] + (size_t)tt * KT * BLK_U4, KT * BLK_BYTES);
            }
        }
        float acc[NM][4];
#pragma unroll
        for (int m = 0; m < NM; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.0f;

        for (uint32_t k0 = 0; k0 < K; k0 += kc_max) {
            const uint32_t kc = min(kc_max, K - k0);
            if (!single) {
                if (k0) __syncthreads();
                for (int i = 0; i < NB; ++i) {
                    const uint32_t b = min(b0 + i, a.batch - 1);
                    stage_x_row(xs + (size_t)i * xstride, ncorr + (size_t)i * (kc_max / 32), a.x + (size_t)b * K, a.norm_w,
                                a.norm_fmt, mul_s[i], k0, kc);
                }
                __syncthreads();
            }
            const uint32_t kt_lo = k0 / 128, kt_hi = (k0 + kc) / 128;
            // this warp's blocks of the chunk: kt = kt_first, kt_first + 8, ...
            const uint32_t kt_first = kt_lo + ((warp + FAST_WARPS - (kt_lo % FAST_WARPS)) % FAST_WARPS);
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                const uint4* wt = a.w[m] + (size_t)tile * KT * BLK_U4;
                uint32_t kt = kt_first;
                if (!(preloaded && k0 == 0 && m == 0)) load_batch(wa, wb, sc, wt, kt, kt_hi, lane, g);
                for (; kt < kt_hi; kt += FAST_PF * FAST_WARPS) {
                    uint4 na[FAST_PF], nb[FAST_PF], ns[FAST_PF];
                    load_batch(na, nb, ns, wt, kt + FAST_PF * FAST_WARPS, kt_hi, lane, g);  // next batch first
#pragma unroll
                    for (int p = 0; p < FAST_PF; ++p) {
                        const uint32_t kk = kt + p * FAST_WARPS;
                        if (kk < kt_hi) {
                            const uint32_t kl = kk * 128 - k0;  // column offset inside the staged chunk
                            const __half* xl = xs + (size_t)xrow * xstride + kl + 8 * t;
                            const float* nc = ncorr + (size_t)crow0 * (kc_max / 32) + kl / 32;
                            block_mma<BATCHED>(wa[p], wb[p], sc[p], xl, nc, kc_max / 32, acc[m]);
                        }
                    }
#pragma unroll
                    for (int p = 0; p < FAST_PF; ++p) { wa[p] = na[p]; wb[p] = nb[p]; sc[p] = ns[p]; }
                }
            }
        }
        // the next tile's first blocks start their trip before this tile's reduction
        preloaded = false;
        if (single && tile + gridDim.x < n_tiles) {
            const uint32_t nt = tile + gridDim.x;
            load_batch(wa, wb, sc, a.w[0] + (size_t)nt * KT * BLK_U4, warp, KT, lane, g);
            preloaded = true;
        }

        // ---- reduce the 8 warps (double-buffered by tile parity: one barrier per tile), epilogue ----------------
        float* rbuf = red + (size_t)parity * RED;  // [warp][m][row 0..15][col 0..NB-1]
        if (BATCHED) {
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                float* r = rbuf + (((size_t)warp * NM + m) * 16) * NB;
                r[(g)*NB + 2 * t] = acc[m][0];
                r[(g)*NB + 2 * t + 1] = acc[m][1];
                r[(g + 8) * NB + 2 * t] = acc[m][2];
                r[(g + 8) * NB + 2 * t + 1] = acc[m][3];
            }
        } else if (t == 0) {
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                float* r = rbuf + (((size_t)warp * NM + m) * 16);
                r[g] = acc[m][0];
                r[g + 8] = acc[m][2];
            }
        }
        __syncthreads();
        if (threadIdx.x < 16 * NB) {
            const uint32_t row = threadIdx.x / NB, col = threadIdx.x % NB;
            const uint32_t b = b0 + col;
            float v[NM];
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                float s = 0.0f;
#pragma unroll
                for (int w = 0; w < FAST_WARPS; ++w) s += rbuf[(((size_t)w * NM + m) * 16 + row) * NB + col];
                v[m] = s * unscale_s[col];
            }
            const uint32_t o = tile * 16 + row;
            if (b < a.batch && o < a.rows && (!a.state || a.state[b].active)) {
                const uint32_t stride = a.dst_stride ? a.dst_stride : a.rows;
                float* d = a.dst + (size_t)b * stride + a.dst_offset + o;
                if (DUAL) {
                    const float gate = v[0], up = v[NM - 1];
                    *d = (gate / (1.0f + expf(-gate))) * up;
                } else if (a.epilogue == EPI_RESIDUAL) {
                    *d += v[0];
                } else {
                    *d = v[0];
                }
            }
        }
    }
}

// ---- batch-1 kernel: TMA ring + warp specialization ---------------------------------------------------------
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(FAST_THREADS) : "memory"); }

constexpr uint32_t ERR_WAIT_FULL = 0x51u, ERR_WAIT_EMPTY = 0x52u;
constexpr int EPI_SWIGLU_IL = 100;  // SwiGLU over a gate/up matrix interleaved 8 rows by 8 rows

// grid: min(row tiles, 2 per SM) persistent blocks of 8 consumer warps + 1 producer warp
template <bool DUAL>
__global__ void __launch_bounds__(TMA_THREADS, 2) k_gemv_q4_tma(FastArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int NM = DUAL ? 2 : 1;
    constexpr int RED = FAST_WARPS * NM * 16;
    const uint32_t K = a.K, KT = K / 128, n_tiles = a.rows / 16, NS = a.n_stages;
    const uint32_t n_chunks = (KT + TMA_SB - 1) / TMA_SB;  // pipeline stages per (tile, matrix)
    unsigned char* ring = smem_raw;                                                // [NS][TMA_STAGE_BYTES]
    __half* xs = reinterpret_cast<__half*>(ring + (size_t)NS * TMA_STAGE_BYTES);   // [K]
    float* ncorr = reinterpret_cast<float*>(xs + K);                               // [K/32]
    float* red = ncorr + K / 32;                                                   // [2][RED]
    __shared__ __align__(8) unsigned long long bar_full[TMA_MAX_STAGES], bar_empty[TMA_MAX_STAGES];
    __shared__ float ssq[FAST_WARPS], smx[FAST_WARPS];
    __shared__ float mul_s, unscale_s;

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < NS; ++s) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), FAST_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == FAST_WARPS) {
        // ---- producer: weights do not depend on the previous kernel, so no grid-dependency wait here ----------
        if (lane == 0) {
            bool ok = true;
            uint32_t it = 0;
            for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
#pragma unroll
                for (int m = 0; m < NM; ++m) {
                    const uint4* wt = a.w[m] + (size_t)tile * KT * BLK_U4;
                    for (uint32_t c = 0; c < n_chunks; ++c, ++it) {
                        const uint32_t s = it % NS, ph = (it / NS) & 1u;
                        if (ok && !mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u)) { ok = false; atomicExch(a.err, ERR_WAIT_EMPTY); }
                        const uint32_t nblk = min((uint32_t)TMA_SB, KT - c * TMA_SB);
                        const uint32_t bytes = nblk * BLK_BYTES;
                        mbar_expect_tx(smem_u32(&bar_full[s]), bytes);
                        tma_load_1d(smem_u32(ring + (size_t)s * TMA_STAGE_BYTES), wt + (size_t)c * TMA_SB * BLK_U4, bytes,
                                    smem_u32(&bar_full[s]));
                    }
                }
            }
        }
        return;
    }

    // ---- consumers ----------------------------------------------------------------------------------------------
    pdl_wait();
    const bool active = !a.state || a.state[0].active;
    // an inactive sequence still drains the pipeline below (the producer has already started), but skips x

    // x -> shared memory.  Rows of up to 4096 elements make one trip: each thread keeps its (up to) two chunks
    // of 8 elements in registers while the block agrees on the RMSNorm factor and the fp16 staging scale.
    {
        const float* x = a.x;
        const bool in_regs = K <= 4096;
        float xr[2][8];
        float ss = 0.0f, mx = 0.0f;
        if (active && in_regs) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t c = threadIdx.x + i * FAST_THREADS;
                if (c < K / 8) {
                    const float4 v0 = *reinterpret_cast<const float4*>(x + c * 8), v1 = *reinterpret_cast<const float4*>(x + c * 8 + 4);
                    xr[i][0] = v0.x; xr[i][1] = v0.y; xr[i][2] = v0.z; xr[i][3] = v0.w;
                    xr[i][4] = v1.x; xr[i][5] = v1.y; xr[i][6] = v1.z; xr[i][7] = v1.w;
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        ss = fmaf(xr[i][e], xr[i][e], ss);
                        if (a.norm_w) xr[i][e] *= norm_w_f(a.norm_w, a.norm_fmt, c * 8 + e);  // the norm weight, applied early
                        mx = fmaxf(mx, fabsf(xr[i][e]));
                    }
                }
            }
        } else if (active) {
            for (uint32_t k = threadIdx.x * 4; k < K; k += FAST_THREADS * 4) {
                const float4 v = *reinterpret_cast<const float4*>(x + k);
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
                if (a.norm_w) {
                    mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x * norm_w_f(a.norm_w, a.norm_fmt, k)), fabsf(v.y * norm_w_f(a.norm_w, a.norm_fmt, k + 1))),
                                         fmaxf(fabsf(v.z * norm_w_f(a.norm_w, a.norm_fmt, k + 2)), fabsf(v.w * norm_w_f(a.norm_w, a.norm_fmt, k + 3)))));
                } else {
                    mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                }
            }
        }
        ss = warp_sum(ss);
        mx = warp_max(mx);
        if (lane == 0) { ssq[warp] = ss; smx[warp] = mx; }
        consumer_sync();
        {
            // every thread derives the same factors from the 8 warp partials (no second barrier needed)
            float tot = 0.0f, m = 0.0f;
#pragma unroll
            for (int w = 0; w < FAST_WARPS; ++w) { tot += ssq[w]; m = fmaxf(m, smx[w]); }
            const float inv = a.norm_w ? 1.0f / sqrtf(tot / (float)K + a.eps) : 1.0f;
            const float amax = m * inv;
            float p = 1.0f;  // power of two with amax * p in [256, 512)
            if (amax > 0.0f && amax < 3.0e38f) p = exp2f((float)(8 - ilogbf(amax)));
            if (threadIdx.x == 0) unscale_s = 1.0f / p;
            mul_s = inv * p;  // same value from every thread
        }
        if (active && in_regs) {
            const float mul = mul_s;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t c = threadIdx.x + i * FAST_THREADS;
                const bool valid = c < K / 8;  // whole warps are valid together (K is a multiple of 128)
                float corr = 0.0f;
                if (valid) {
                    __half2 h[4];
                    h[0] = __floats2half2_rn(xr[i][0] * mul, xr[i][1] * mul);
                    h[1] = __floats2half2_rn(xr[i][2] * mul * 0.0625f, xr[i][3] * mul * 0.0625f);
                    h[2] = __floats2half2_rn(xr[i][4] * mul, xr[i][5] * mul);
                    h[3] = __floats2half2_rn(xr[i][6] * mul * 0.0625f, xr[i][7] * mul * 0.0625f);
                    const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
                    corr = 1032.0f * ((f0.x + f0.y) + (f2.x + f2.y)) + 1152.0f * ((f1.x + f1.y) + (f3.x + f3.y));
                    *reinterpret_cast<uint4*>(xs + c * 8) = *reinterpret_cast<const uint4*>(h);
                }
                corr += __shfl_xor_sync(0xFFFFFFFFu, corr, 1);
                corr += __shfl_xor_sync(0xFFFFFFFFu, corr, 2);
                if (valid && (threadIdx.x & 3) == 0) ncorr[c >> 2] = -corr;
            }
        } else if (active) {
            stage_x_row(xs, ncorr, x, a.norm_w, a.norm_fmt, mul_s, 0, K);
        }
        consumer_sync();
    }

    bool ok = true;
    uint32_t it = 0, parity = 0;
    const __half* xl0 = xs + 8 * t;
    for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, parity ^= 1) {
        float acc[NM][4];
#pragma unroll
        for (int m = 0; m < NM; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.0f;
#pragma unroll
        for (int m = 0; m < NM; ++m) {
            for (uint32_t c = 0; c < n_chunks; ++c, ++it) {
                const uint32_t s = it % NS, ph = (it / NS) & 1u;
                if (ok && !mbar_wait(smem_u32(&bar_full[s]), ph)) { ok = false; atomicExch(a.err, ERR_WAIT_FULL); }
                const uint32_t kk = c * TMA_SB + warp;
                if (kk < KT && active) {
                    const uint4* blk = reinterpret_cast<const uint4*>(ring + (size_t)s * TMA_STAGE_BYTES) + (size_t)warp * BLK_U4;
                    const uint4 wa = blk[lane], wb = blk[32 + lane], sc = blk[64 + g];
                    block_mma<false>(wa, wb, sc, xl0 + kk * 128, ncorr + kk * 4, 0, acc[m]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_empty[s]));
            }
        }
        // reduce the 8 warps (double-buffered by tile parity: one barrier per tile), epilogue
        float* rbuf = red + (size_t)parity * RED;
        if (t == 0) {
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                rbuf[((size_t)warp * NM + m) * 16 + g] = acc[m][0];
                rbuf[((size_t)warp * NM + m) * 16 + g + 8] = acc[m][2];
            }
        }
        consumer_sync();
        if (a.epilogue == EPI_SWIGLU_IL) {
            // tile = 8 gate rows (mma rows 0..7) over the same 8 up rows (mma rows 8..15)
            if (threadIdx.x < 8 && active) {
                float gate = 0.0f, up = 0.0f;
#pragma unroll
                for (int w = 0; w < FAST_WARPS; ++w) { gate += rbuf[(size_t)w * NM * 16 + threadIdx.x]; up += rbuf[(size_t)w * NM * 16 + threadIdx.x + 8]; }
                gate *= unscale_s; up *= unscale_s;
                a.dst[a.dst_offset + tile * 8 + threadIdx.x] = (gate / (1.0f + expf(-gate))) * up;
            }
        } else if (threadIdx.x < 16 && active) {
            const uint32_t row = threadIdx.x;
            float v[NM];
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < FAST_WARPS; ++w) sum += rbuf[((size_t)w * NM + m) * 16 + row];
                v[m] = sum * unscale_s;
            }
            const uint32_t o = tile * 16 + row;
            float* d = a.dst + a.dst_offset + o;
            if (DUAL) {
                const float gate = v[0], up = v[NM - 1];
                *d = (gate / (1.0f + expf(-gate))) * up;
            } else if (a.epilogue == EPI_RESIDUAL) {
                *d += v[0];
            } else {
                *d = v[0];
            }
        }
    }
}


static size_t fast_smem_bytes(uint32_t K, bool batched, bool dual, uint32_t kc_batched) {
    const uint32_t nb = batched ? 8 : 1, nm = dual ? 2 : 1;
    const uint32_t kc = batched ? (K < kc_batched ? K : kc_batched) : K;
    return (size_t)nb * (kc + FAST_XPAD) * 2 + (size_t)nb * (kc / 32) * 4 + 2 * (size_t)FAST_WARPS * nm * 16 * nb * 4;
}

constexpr int FAST_MAX_SMEM = 100 * 1024;         // two blocks per SM
constexpr int FAST_MAX_SMEM_BATCHED = 200 * 1024; // batched: one block per SM may stage rows of up to ~12k elements whole
constexpr int TMA_MAX_SMEM = 112 * 1024;  // two blocks per SM

cudaError_t gemv_fast_init() {
    cudaError_t e;
#define VB_OPT_IN(B, D) if ((e = cudaFuncSetAttribute(k_gemv_q4_mma<B, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, FAST_MAX_SMEM)) != cudaSuccess) return e
    VB_OPT_IN(false, false); VB_OPT_IN(false, true);
#undef VB_OPT_IN
    if ((e = cudaFuncSetAttribute(k_gemv_q4_mma<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FAST_MAX_SMEM_BATCHED)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(k_gemv_q4_mma<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FAST_MAX_SMEM_BATCHED)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(k_gemv_q4_tma<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TMA_MAX_SMEM)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(k_gemv_q4_tma<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TMA_MAX_SMEM)) != cudaSuccess) return e;
    return cudaSuccess;
}

// Error word shared by every launch of this process on a device (bounded waits report here).  It lives in
// mapped pinned host memory: kernels only ever write it when a wait gives up, and the host reads it after a
// stream synchronisation without a copy.
static uint32_t* g_err_word[64] = {nullptr};       // device-side address
static uint32_t* g_err_word_host[64] = {nullptr};  // the same word as the host sees it
static cudaError_t err_word(uint32_t** out, uint32_t** out_host) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!g_err_word[dev]) {
        uint32_t* h = nullptr;
        if ((e = cudaHostAlloc((void**)&h, 256, cudaHostAllocMapped)) != cudaSuccess) return e;
        memset(h, 0, 256);
        if ((e = cudaHostGetDevicePointer((void**)&g_err_word[dev], h, 0)) != cudaSuccess) return e;
        g_err_word_host[dev] = h;
    }
    if (out) *out = g_err_word[dev];
    if (out_host) *out_host = g_err_word_host[dev];
    return cudaSuccess;
}
cudaError_t fast_error_word(uint32_t** out) { return err_word(out, nullptr); }
cudaError_t fast_error_word_host(uint32_t** out) { return err_word(nullptr, out); }

bool fast_use_tma = true;  // vb_set_option("gemv_tma", 0) selects the register-prefetch kernel for batch 1 too

cudaError_t gemv_fast(const LaunchCfg& lc, const GemvArgs& a, bool* handled) {
    *handled = false;
    if (a.w.fmt != VB_FMT_Q4G32 || !a.w.tiled) return cudaSuccess;
    if (a.w.rows % 16 != 0 || a.w.cols % 128 != 0) return cudaSuccess;
    const bool dual_in = a.epilogue == EPI_SWIGLU;
    const bool dual = dual_in;
    if (dual && (!a.w2.tiled || a.w2.rows != a.w.rows || a.w2.cols != a.w.cols)) return cudaSuccess;
    const bool batched = a.batch > 1;
    // batched: stage the whole row when one block per SM can hold it (then the block is persistent over its tiles)
    uint32_t kc = (uint32_t)FAST_KC_BATCHED;
    if (batched && fast_smem_bytes(a.w.cols, true, dual, a.w.cols) <= (size_t)FAST_MAX_SMEM_BATCHED) kc = a.w.cols;
    const size_t smem = fast_smem_bytes(a.w.cols, batched, dual, kc);
    FastArgs f;
    f.w[0] = (const uint4*)a.w.tiled;
    f.w[1] = dual ? (const uint4*)a.w2.tiled : f.w[0];
    f.err = nullptr; f.n_stages = 0;
    f.rows = a.w.rows; f.K = a.w.cols; f.x = a.x; f.dst = a.dst;
    f.norm_w = a.norm_w; f.norm_fmt = a.norm_fmt; f.eps = a.eps; f.state = a.state;
    f.batch = a.batch; f.dst_stride = a.dst_stride; f.dst_offset = a.dst_offset; f.epilogue = a.epilogue;
    f.kc = kc;
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
    }
    const uint32_t n_tiles = a.w.rows / 16;
    const bool single = !batched || a.w.cols <= kc;
    // persistent blocks: as many as are resident at once over all batch groups
    const uint32_t gy = batched ? (a.batch + 7) / 8 : 1;
    const uint32_t resident = (uint32_t)n_sm * (smem > (size_t)FAST_MAX_SMEM ? 1u : 2u);
    const uint32_t per_group = resident / gy ? resident / gy : 1u;
    const uint32_t gx = single ? (n_tiles < per_group ? n_tiles : per_group) : n_tiles;
    const dim3 grid(gx, gy);
    bool interleaved = false;
    if (!batched && fast_use_tma && dual && a.w.tiled_swiglu) {
        // gate and up share 16-row tiles: one matrix of 2*rows rows, half the tile size, SwiGLU in the epilogue
        interleaved = true;
        f.w[0] = f.w[1] = (const uint4*)a.w.tiled_swiglu;
        f.rows = 2 * a.w.rows;
        f.epilogue = EPI_SWIGLU_IL;
    }
    if (!batched && fast_use_tma) {
        const bool dual = dual_in && !interleaved;
        const uint32_t n_tiles = f.rows / 16;
        // ring depth: what is left of the per-block shared memory after x, its corrections and the reduction buffer
        const size_t fixed = (size_t)a.w.cols * 2 + (size_t)(a.w.cols / 32) * 4 + 2 * (size_t)FAST_WARPS * (dual ? 2 : 1) * 16 * 4 + 256;
        if (fixed + 2 * (size_t)TMA_STAGE_BYTES <= (size_t)TMA_MAX_SMEM) {
            size_t ns = ((size_t)TMA_MAX_SMEM - fixed) / TMA_STAGE_BYTES;
            if (ns > TMA_MAX_STAGES) ns = TMA_MAX_STAGES;
            f.n_stages = (uint32_t)ns;
            cudaError_t e = err_word(&f.err, nullptr);
            if (e != cudaSuccess) return e;
            *handled = true;
            const size_t tsmem = fixed + ns * TMA_STAGE_BYTES;
            const dim3 tgrid(n_tiles < 2u * n_sm ? n_tiles : 2u * n_sm);
            return dual ? launch(lc, k_gemv_q4_tma<true>, tgrid, dim3(TMA_THREADS), tsmem, f)
                        : launch(lc, k_gemv_q4_tma<false>, tgrid, dim3(TMA_THREADS), tsmem, f);
        }
    }
    if (smem > (size_t)(batched ? FAST_MAX_SMEM_BATCHED : FAST_MAX_SMEM)) return cudaSuccess;
    *handled = true;
    if (batched) {
        return dual ? launch(lc, k_gemv_q4_mma<true, true>, grid, dim3(FAST_THREADS), smem, f)
                    : launch(lc, k_gemv_q4_mma<true, false>, grid, dim3(FAST_THREADS), smem, f);
    }
    return dual ? launch(lc, k_gemv_q4_mma<false, true>, grid, dim3(FAST_THREADS), smem, f)
                : launch(lc, k_gemv_q4_mma<false, false>, grid, dim3(FAST_THREADS), smem, f);
}

// ---- canonical -> tile-major repack (load time) ------------------------------------------------------------
// block (rt, kt) = 288 words: word half*128 + L*4 + j (half 0: mma rows 0..7, half 1: rows 8..15; L = 4g+t;
// j = group), then 32 words of scales: fp16 index g*8 + half*4 + j.  One call fills one half of every block:
// source row = rt * rows_per_tile + row_off + g.  A plain matrix is two calls (16, 0, half 0) and (16, 8, half 1);
// the interleaved gate/up matrix takes gate with (8, 0, half 0) and up with (8, 0, half 1).
__global__ void k_tile_q4_words(uint32_t* __restrict__ out, const uint32_t* __restrict__ canon, uint32_t n_tiles, uint32_t K,
                                uint32_t rows_per_tile, uint32_t row_off, uint32_t half) {
    const uint32_t KT = K / 128;
    const uint64_t n = (uint64_t)n_tiles * KT * 128;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t j = i & 3, L = (i >> 2) & 31;
        const uint64_t blk = i >> 7;
        const uint32_t kt = blk % KT, rt = blk / KT, g = L >> 2, t = L & 3;
        const uint32_t row = rt * rows_per_tile + row_off + g;
        const uint32_t word = kt * 16 + 4 * j + t;  // (128*kt + 32*j + 8*t) / 8
        out[blk * (BLK_BYTES / 4) + half * 128 + (i & 127)] = canon[(uint64_t)row * (K / 8) + word];
    }
}
__global__ void k_tile_q4_scales(__half* __restrict__ out, const __half* __restrict__ canon, uint32_t n_tiles, uint32_t K,
                                 uint32_t rows_per_tile, uint32_t row_off, uint32_t half) {
    const uint32_t KT = K / 128;
    const uint64_t n = (uint64_t)n_tiles * KT * 32;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t j = i & 3, g = (i >> 2) & 7;
        const uint64_t blk = i >> 5;
        const uint32_t kt = blk % KT, rt = blk / KT;
        const uint32_t row = rt * rows_per_tile + row_off + g;
        out[blk * (BLK_BYTES / 2) + 512 + g * 8 + half * 4 + j] = canon[(uint64_t)row * (K / 32) + kt * 4 + j];
    }
}

bool tile_q4_supported(uint32_t rows, uint32_t K) { return rows % 16 == 0 && K % 128 == 0 && rows > 0 && K > 0; }

static cudaError_t tile_q4_half(const LaunchCfg& lc, void* tiled, const void* canon, const void* canon_scales, uint32_t n_tiles,
                                uint32_t K, uint32_t rows_per_tile, uint32_t row_off, uint32_t half) {
    const uint64_t nw = (uint64_t)n_tiles * (K / 128) * 128;
    unsigned blocks = (unsigned)((nw + 255) / 256 > 148 * 32 ? 148 * 32 : (nw + 255) / 256);
    cudaError_t e = launch(lc, k_tile_q4_words, dim3(blocks), dim3(256), 0, (uint32_t*)tiled, (const uint32_t*)canon, n_tiles, K,
                           rows_per_tile, row_off, half);
    if (e != cudaSuccess) return e;
    const uint64_t ns = (uint64_t)n_tiles * (K / 128) * 32;
    blocks = (unsigned)((ns + 255) / 256 > 148 * 32 ? 148 * 32 : (ns + 255) / 256);
    return launch(lc, k_tile_q4_scales, dim3(blocks), dim3(256), 0, (__half*)tiled, (const __half*)canon_scales, n_tiles, K,
                  rows_per_tile, row_off, half);
}

cudaError_t tile_q4(const LaunchCfg& lc, void* tiled, void* tiled_scales, const void* canon, const void* canon_scales,
                    uint32_t rows, uint32_t K) {
    (void)tiled_scales;  // scales live inside the blocks
    cudaError_t e = tile_q4_half(lc, tiled, canon, canon_scales, rows / 16, K, 16, 0, 0);
    if (e != cudaSuccess) return e;
    return tile_q4_half(lc, tiled, canon, canon_scales, rows / 16, K, 16, 8, 1);
}

// gate (which = 0) or up (which = 1) into the interleaved SwiGLU matrix: tile i = gate rows 8i..8i+7 | up rows 8i..8i+7
cudaError_t tile_q4_swiglu(const LaunchCfg& lc, void* tiled, const void* canon, const void* canon_scales, uint32_t rows, uint32_t K,
                           int which) {
    return tile_q4_half(lc, tiled, canon, canon_scales, rows / 8, K, 8, 0, (uint32_t)which);
}

}  // namespace vb
