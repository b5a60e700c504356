// Load-time conversion kernels (synthetic fill, quantize, dequantize), the small per-token kernels
// (embed, RMSNorm, RoPE + KV append, two-stage argmax) and their C-ABI entry points.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>

#include "vb_internal.cuh"
#include "vb_kernels.cuh"

namespace vb {

// ---- status ----------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
const char* last_error() { return g_err; }

int32_t cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
    set_error("CUDA error %d (%s) at %s:%d: %s", (int)e, cudaGetErrorString(e), file, line, what);
    return VB_ERR_CUDA;
}

// ---- synthetic fill -----------------------------------------------------------------------------
// Sum of twelve 16-bit hash lanes, centred: integer arithmetic up to one exact int->float conversion
// and two correctly rounded float operations, so the CPU checker reproduces every bit.
__global__ void k_fill_normal(float* __restrict__ dst, uint64_t n, uint64_t key, float mean, float scale) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        uint32_t s = 0;
#pragma unroll
        for (uint64_t j = 0; j < 3; ++j) s += lanes16_sum(mix64(key + (3ULL * i + j + 1ULL) * 0x9E3779B97F4A7C15ULL));
        float v = __fmul_rn((float)((int32_t)s - 393210), scale);
        dst[i] = __fadd_rn(v, mean);
    }
}

cudaError_t fill_normal(const LaunchCfg& lc, float* dst, uint64_t n, uint64_t seed, uint64_t stream_id, float mean, float std) {
    if (n == 0) return cudaSuccess;
    uint64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    return launch(lc, k_fill_normal, dim3((unsigned)blocks), dim3(256), 0, dst, n, stream_key(seed, stream_id), mean,
                  std * (1.0f / 65536.0f));
}

// The same generator restricted to the rectangle rows [r0, r0+rows) x cols [c0, c0+cols) of a [*][full_cols] tensor:
// a tensor-parallel rank fills its shard with exactly the values the whole tensor would hold there.
__global__ void k_fill_normal_slice(float* __restrict__ dst, uint64_t rows, uint64_t cols, uint64_t full_cols, uint64_t r0,
                                    uint64_t c0, uint64_t key, float mean, float scale) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, n = rows * cols;
    for (; i < n; i += stride) {
        const uint64_t r = i / cols, c = i - r * cols;
        const uint64_t g = (r0 + r) * full_cols + c0 + c;
        uint32_t s = 0;
#pragma unroll
        for (uint64_t j = 0; j < 3; ++j) s += lanes16_sum(mix64(key + (3ULL * g + j + 1ULL) * 0x9E3779B97F4A7C15ULL));
        float v = __fmul_rn((float)((int32_t)s - 393210), scale);
        dst[i] = __fadd_rn(v, mean);
    }
}

cudaError_t fill_normal_slice(const LaunchCfg& lc, float* dst, uint64_t rows, uint64_t cols, uint64_t full_cols, uint64_t r0,
                              uint64_t c0, uint64_t seed, uint64_t stream_id, float mean, float std) {
    const uint64_t n = rows * cols;
    if (n == 0) return cudaSuccess;
    uint64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    return launch(lc, k_fill_normal_slice, dim3((unsigned)blocks), dim3(256), 0, dst, rows, cols, full_cols, r0, c0,
                  stream_key(seed, stream_id), mean, std * (1.0f / 65536.0f));
}

// ---- quantizers ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack8(const uint32_t q[8]) {
    return (q[0] << 0) | (q[2] << 4) | (q[4] << 8) | (q[6] << 12) | (q[1] << 16) | (q[3] << 20) | (q[5] << 24) |
           (q[7] << 28);
}

// one thread per group of 32: scale = h(max|w|/7), n = clamp(rn(w/scale)+8, 0, 15)
__global__ void k_quantize_q4g32(uint32_t* __restrict__ packed, __half* __restrict__ scales,
                                 const float* __restrict__ src, uint64_t n_groups) {
    uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (; g < n_groups; g += stride) {
        const float4* grp = reinterpret_cast<const float4*>(src + g * 32ULL);
        float v[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) { float4 t = grp[i]; v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w; }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
        __half hs = __float2half_rn(__fdiv_rn(amax, 7.0f));
        scales[g] = hs;
        float s = __half2float(hs);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            uint32_t q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                int qi = 8;
                if (s > 0.0f) {
                    qi = __float2int_rn(__fdiv_rn(v[w * 8 + j], s)) + 8;
                    qi = max(0, min(15, qi));
                }
                q[j] = (uint32_t)qi;
            }
            packed[g * 4ULL + w] = pack8(q);
        }
    }
}

// the reference's load-time quantizer (src/codegen.rs:2337-2369), one thread per group of 64
__global__ void k_quantize_q4g64ref(uint32_t* __restrict__ packed, __half2* __restrict__ scale_min,
                                    const float* __restrict__ src, uint64_t n_groups) {
    uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (; g < n_groups; g += stride) {
        const float* grp = src + g * 64ULL;
        float fmin = grp[0], fmax = grp[0];
        for (int i = 1; i < 64; ++i) { float v = grp[i]; if (v < fmin) fmin = v; if (v > fmax) fmax = v; }
        float scale_f = (fmax > fmin) ? __fdiv_rn(__fsub_rn(fmax, fmin), 15.0f) : 0.0f;
        __half hs = __float2half_rn(scale_f), hm = __float2half_rn(fmin);
        scale_min[g] = __halves2half2(hs, hm);
        float s = __half2float(hs), m = __half2float(hm);
        float inv = (s > 1.0e-12f) ? __fdiv_rn(1.0f, s) : 0.0f;
        for (int w = 0; w < 8; ++w) {
            uint32_t q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                int qi = __float2int_rn(__fmul_rn(__fsub_rn(grp[w * 8 + j], m), inv));
                q[j] = (uint32_t)max(0, min(15, qi));
            }
            packed[g * 8ULL + w] = pack8(q);
        }
    }
}

// one block per output row: scale = h(max|w|/127), q = clamp(rn(w/scale), -127, 127)
__global__ void k_quantize_i8pc(int8_t* __restrict__ q, __half* __restrict__ scales, const float* __restrict__ src,
                                uint64_t cols) {
    const uint64_t r = blockIdx.x;
    const float* row = src + r * cols;
    __shared__ float red[32];
    float amax = 0.0f;
    for (uint64_t i = threadIdx.x; i < cols; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.0f;
        v = warp_max(v);
        if (threadIdx.x == 0) red[0] = v;
    }
    __syncthreads();
    amax = red[0];
    __half hs = __float2half_rn(__fdiv_rn(amax, 127.0f));
    if (threadIdx.x == 0) scales[r] = hs;
    float s = __half2float(hs);
    for (uint64_t i = threadIdx.x; i < cols; i += blockDim.x) {
        int qi = 0;
        if (s > 0.0f) { qi = __float2int_rn(__fdiv_rn(row[i], s)); qi = max(-127, min(127, qi)); }
        q[r * cols + i] = (int8_t)qi;
    }
}

__global__ void k_f32_to_f16(__half* __restrict__ dst, const float* __restrict__ src, uint64_t n) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i < n; i += (uint64_t)gridDim.x * blockDim.x) dst[i] = __float2half_rn(src[i]);
}
__global__ void k_f32_to_bf16(__nv_bfloat16* __restrict__ dst, const float* __restrict__ src, uint64_t n) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i < n; i += (uint64_t)gridDim.x * blockDim.x) dst[i] = __float2bfloat16_rn(src[i]);
}
__global__ void k_f16_to_f32(float* __restrict__ dst, const __half* __restrict__ src, uint64_t n) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i < n; i += (uint64_t)gridDim.x * blockDim.x) dst[i] = __half2float(src[i]);
}
__global__ void k_bf16_to_f32(float* __restrict__ dst, const __nv_bfloat16* __restrict__ src, uint64_t n) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i < n; i += (uint64_t)gridDim.x * blockDim.x) dst[i] = __bfloat162float(src[i]);
}

static inline unsigned grid_for(uint64_t n, unsigned per_block) {
    uint64_t b = (n + per_block - 1) / per_block;
    if (b > 148ULL * 64ULL) b = 148ULL * 64ULL;
    if (b == 0) b = 1;
    return (unsigned)b;
}

cudaError_t quantize(const LaunchCfg& lc, void* data, void* scales, const float* src, int32_t fmt, uint64_t rows, uint64_t cols) {
    const uint64_t n = rows * cols;
    switch (fmt) {
    case VB_FMT_F32: return cudaMemcpyAsync(data, src, n * 4, cudaMemcpyDeviceToDevice, lc.stream);
    case VB_FMT_F16: return launch(lc, k_f32_to_f16, dim3(grid_for(n, 256)), dim3(256), 0, (__half*)data, src, n);
    case VB_FMT_BF16: return launch(lc, k_f32_to_bf16, dim3(grid_for(n, 256)), dim3(256), 0, (__nv_bfloat16*)data, src, n);
    case VB_FMT_Q4G32: return launch(lc, k_quantize_q4g32, dim3(grid_for(n / 32, 128)), dim3(128), 0, (uint32_t*)data, (__half*)scales, src, n / 32);
    case VB_FMT_Q4G64REF: return launch(lc, k_quantize_q4g64ref, dim3(grid_for(n / 64, 128)), dim3(128), 0, (uint32_t*)data, (__half2*)scales, src, n / 64);
    case VB_FMT_I8PC: return launch(lc, k_quantize_i8pc, dim3((unsigned)rows), dim3(256), 0, (int8_t*)data, (__half*)scales, src, cols);
    default: return cudaErrorInvalidValue;
    }
}

// ---- dequantizers (bit-exact contract) ----------------------------------------------------------------
__global__ void k_dequant_q4(float* __restrict__ dst, const uint32_t* __restrict__ packed, const __half* __restrict__ scales,
                             uint64_t n_words, int ref_g64) {
    uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; w < n_words; w += (uint64_t)gridDim.x * blockDim.x) {
        float q[8];
        unpack8_f32(packed[w], q);
        float* out = dst + w * 8ULL;
        if (ref_g64) {
            const __half2 sm = reinterpret_cast<const __half2*>(scales)[w >> 3];
            const float s = __low2float(sm), m = __high2float(sm);
#pragma unroll
            for (int j = 0; j < 8; ++j) out[j] = fmaf(q[j], s, m);
        } else {
            const float s = __half2float(scales[w >> 2]);
#pragma unroll
            for (int j = 0; j < 8; ++j) out[j] = __fmul_rn(__fsub_rn(q[j], 8.0f), s);
        }
    }
}
__global__ void k_dequant_i8pc(float* __restrict__ dst, const int8_t* __restrict__ q, const __half* __restrict__ scales,
                               uint64_t rows, uint64_t cols) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t n = rows * cols;
    for (; i < n; i += (uint64_t)gridDim.x * blockDim.x) dst[i] = __fmul_rn((float)q[i], __half2float(scales[i / cols]));
}

cudaError_t dequantize(const LaunchCfg& lc, float* dst, const void* data, const void* scales, int32_t fmt, uint64_t rows, uint64_t cols) {
    const uint64_t n = rows * cols;
    switch (fmt) {
    case VB_FMT_F32: return cudaMemcpyAsync(dst, data, n * 4, cudaMemcpyDeviceToDevice, lc.stream);
    case VB_FMT_F16: return launch(lc, k_f16_to_f32, dim3(grid_for(n, 256)), dim3(256), 0, dst, (const __half*)data, n);
    case VB_FMT_BF16: return launch(lc, k_bf16_to_f32, dim3(grid_for(n, 256)), dim3(256), 0, dst, (const __nv_bfloat16*)data, n);
    case VB_FMT_Q4G32: return launch(lc, k_dequant_q4, dim3(grid_for(n / 8, 256)), dim3(256), 0, dst, (const uint32_t*)data, (const __half*)scales, n / 8, 0);
    case VB_FMT_Q4G64REF: return launch(lc, k_dequant_q4, dim3(grid_for(n / 8, 256)), dim3(256), 0, dst, (const uint32_t*)data, (const __half*)scales, n / 8, 1);
    case VB_FMT_I8PC: return launch(lc, k_dequant_i8pc, dim3(grid_for(n, 256)), dim3(256), 0, dst, (const int8_t*)data, (const __half*)scales, rows, cols);
    default: return cudaErrorInvalidValue;
    }
}

// ---- embed ------------------------------------------------------------------------------------------
// dst[b][:] = table[token_b][:] dequantized to fp32; grid (ceil(d/8/128), batch)
__global__ void k_embed(float* __restrict__ dst, const uint32_t* __restrict__ tokens, const SeqState* __restrict__ state,
                        const void* __restrict__ table, const void* __restrict__ scales, int fmt, uint32_t d, uint32_t vocab) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t b = blockIdx.y;
    uint32_t tok;
    if (state) { if (!state[b].active) return; tok = state[b].token; } else tok = tokens[b];
    if (tok >= vocab) tok = vocab - 1;
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;  // chunk of 8 elements
    if (c * 8 >= d) return;
    float* out = dst + (size_t)b * d + c * 8;
    const size_t e0 = (size_t)tok * d + c * 8;
    float v[8];
    switch (fmt) {
    case VB_FMT_F32: {
        const float4* p = reinterpret_cast<const float4*>((const float*)table + e0);
        float4 a = p[0], bb = p[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = bb.x; v[5] = bb.y; v[6] = bb.z; v[7] = bb.w;
    } break;
    case VB_FMT_F16: {
        uint4 raw = *reinterpret_cast<const uint4*>((const __half*)table + e0);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    } break;
    case VB_FMT_BF16: {
        uint4 raw = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)table + e0);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    } break;
    case VB_FMT_Q4G32: {
        unpack8_f32(((const uint32_t*)table)[e0 >> 3], v);
        const float s = __half2float(((const __half*)scales)[e0 >> 5]);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fsub_rn(v[i], 8.0f), s);
    } break;
    case VB_FMT_Q4G64REF: {
        unpack8_f32(((const uint32_t*)table)[e0 >> 3], v);
        const __half2 sm = ((const __half2*)scales)[e0 >> 6];
        const float s = __low2float(sm), m = __high2float(sm);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = fmaf(v[i], s, m);
    } break;
    case VB_FMT_I8PC: {
        const int8_t* p = (const int8_t*)table + e0;
        const float s = __half2float(((const __half*)scales)[tok]);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn((float)p[i], s);
    } break;
    default:
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
    reinterpret_cast<float4*>(out)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(out)[1] = make_float4(v[4], v[5], v[6], v[7]);
}

cudaError_t embed(const LaunchCfg& lc, float* dst, const uint32_t* tokens, const SeqState* state, const void* table,
                  const void* scales, int fmt, uint32_t d, uint32_t vocab, uint32_t batch) {
    dim3 grid((d / 8 + 127) / 128, batch);
    return launch(lc, k_embed, grid, dim3(128), 0, dst, tokens, state, table, scales, fmt, d, vocab);
}

// ---- RMSNorm (stand-alone op) ----------------------------------------------------------------------------
__device__ __forceinline__ float load_vec(const void* w, int fmt, uint32_t i) {
    return fmt == VB_FMT_F16 ? __half2float(((const __half*)w)[i])
         : fmt == VB_FMT_BF16 ? __bfloat162float(((const __nv_bfloat16*)w)[i]) : ((const float*)w)[i];
}

__global__ void k_rmsnorm(float* __restrict__ dst, const float* __restrict__ x, const void* __restrict__ w, int w_fmt,
                          uint32_t dim, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const float* xr = x + (size_t)blockIdx.x * dim;
    float* yr = dst + (size_t)blockIdx.x * dim;
    __shared__ float red[32];
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) { float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.0f;
        v = warp_sum(v);
        if (threadIdx.x == 0) red[0] = v;
    }
    __syncthreads();
    const float inv = 1.0f / sqrtf(red[0] / (float)dim + eps);
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) yr[i] = (xr[i] * inv) * load_vec(w, w_fmt, i);
}

cudaError_t rmsnorm(const LaunchCfg& lc, float* dst, const float* x, const void* w, int w_fmt, uint32_t dim, uint32_t batch, float eps) {
    return launch(lc, k_rmsnorm, dim3(batch), dim3(256), 0, dst, x, w, w_fmt, dim, eps);
}

// 1/theta^(2j/D) as the reference computes it in fp32 (src/runtime.rs:758).  The host libm's powf is correctly
// rounded; evaluating pow in double and rounding once gives the same fp32 value, whereas the device powf may
// be 2 ulp off, which at position 2047 already moves the angle by 1e-4 rad.
__device__ __forceinline__ float rope_inv_freq(float theta, uint32_t j, uint32_t head_dim) {
    const float expo = (float)(2 * j) / (float)head_dim;
    return 1.0f / (float)pow((double)theta, (double)expo);
}

// ---- RoPE (stand-alone op) ----------------------------------------------------------------------------------
__global__ void k_rope(float* __restrict__ t, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta) {
    const uint32_t half = head_dim / 2;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_heads * half) return;
    const uint32_t h = i / half, j = i % half;
    const float freq = rope_inv_freq(theta, j, head_dim);
    const float angle = (float)pos * freq;
    float s, c;
    sincosf(angle, &s, &c);
    float* hs = t + (size_t)h * head_dim;
    const float x1 = hs[j], x2 = hs[j + half];
    hs[j] = x1 * c - x2 * s;
    hs[j + half] = x2 * c + x1 * s;
}

cudaError_t rope(const LaunchCfg& lc, float* t, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta) {
    const uint32_t n = n_heads * (head_dim / 2);
    return launch(lc, k_rope, dim3((n + 127) / 128), dim3(128), 0, t, n_heads, head_dim, pos, theta);
}

// ---- bias + RoPE + KV append -------------------------------------------------------------------------------
// qkv [B][(Hq+2Hkv)*D] fp32 (raw projections) -> q_out [B][Hq*D] fp32 rotated; K (rotated) and V rounded
// to fp16 into the paged pool.  One thread per rotation pair / per V pair.
__global__ void k_bias_rope_kv_append(float* __restrict__ q_out, const float* __restrict__ qkv, const SeqState* __restrict__ state,
                                      const void* __restrict__ bq, const void* __restrict__ bk, const void* __restrict__ bv, int bias_fmt,
                                      __half* __restrict__ kv_layer, const int32_t* __restrict__ block_table, uint32_t max_blocks,
                                      uint32_t Hq, uint32_t Hkv, uint32_t D, uint32_t block_tokens, float theta) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t b = blockIdx.y;
    if (!state[b].active) return;
    const uint32_t pos = state[b].pos;
    if (state[b].limit && pos >= state[b].limit) return;  // never write outside the slot's reservation
    const uint32_t half = D / 2;
    const uint32_t n_rot = (Hq + Hkv) * half;  // rotation pairs of q and k
    const uint32_t n_v = Hkv * half;           // v handled as pairs too
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rot + n_v) return;
    const float* row = qkv + (size_t)b * (Hq + 2 * Hkv) * D;
    const int32_t blk = block_table[(size_t)b * max_blocks + pos / block_tokens];
    const uint32_t slot = pos % block_tokens;
    // pool layout per layer: [block][K|V][kv_head][block_tokens][D]
    if (i < n_rot) {
        const uint32_t h = i / half, j = i % half;
        const float freq = rope_inv_freq(theta, j, D);
        const float angle = (float)pos * freq;
        float s, c;
        sincosf(angle, &s, &c);
        float x1 = row[(size_t)h * D + j], x2 = row[(size_t)h * D + j + half];
        if (h < Hq) {
            if (bq) { x1 += load_vec(bq, bias_fmt, h * D + j); x2 += load_vec(bq, bias_fmt, h * D + j + half); }
            float* qo = q_out + (size_t)b * Hq * D + (size_t)h * D;
            qo[j] = x1 * c - x2 * s;
            qo[j + half] = x2 * c + x1 * s;
        } else {
            const uint32_t kh = h - Hq;
            if (bk) { x1 += load_vec(bk, bias_fmt, kh * D + j); x2 += load_vec(bk, bias_fmt, kh * D + j + half); }
            __half* kd = kv_layer + ((((size_t)blk * 2 + 0) * Hkv + kh) * block_tokens + slot) * D;
            kd[j] = __float2half_rn(x1 * c - x2 * s);
            kd[j + half] = __float2half_rn(x2 * c + x1 * s);
        }
    } else {
        const uint32_t k = i - n_rot;
        const uint32_t vh = k / half, j = k % half;
        const float* vr = row + (size_t)(Hq + Hkv) * D + (size_t)vh * D;
        float v1 = vr[j], v2 = vr[j + half];
        if (bv) { v1 += load_vec(bv, bias_fmt, vh * D + j); v2 += load_vec(bv, bias_fmt, vh * D + j + half); }
        __half* vd = kv_layer + ((((size_t)blk * 2 + 1) * Hkv + vh) * block_tokens + slot) * D;
        vd[j] = __float2half_rn(v1);
        vd[j + half] = __float2half_rn(v2);
    }
}

cudaError_t bias_rope_kv_append(const LaunchCfg& lc, float* q_out, const float* qkv, const SeqState* state, const void* bq,
                                const void* bk, const void* bv, int bias_fmt, __half* kv_layer, const int32_t* block_table,
                                uint32_t max_blocks, uint32_t Hq, uint32_t Hkv, uint32_t D, uint32_t block_tokens, float theta,
                                uint32_t batch) {
    const uint32_t n = (Hq + 2 * Hkv) * (D / 2);
    return launch(lc, k_bias_rope_kv_append, dim3((n + 127) / 128, batch), dim3(128), 0, q_out, qkv, state, bq, bk, bv,
                  bias_fmt, kv_layer, block_table, max_blocks, Hq, Hkv, D, block_tokens, theta);
}

// ---- two-stage argmax --------------------------------------------------------------------------------------
// Rule of src/runtime.rs:1078-1088: start at (-inf, index 0), replace only on strictly greater, so the
// lowest index of the maximum wins and NaN (or an all -inf row) yields index 0.
struct ArgPair { float v; uint32_t i; };
__device__ __forceinline__ ArgPair arg_merge(ArgPair a, ArgPair b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}
__device__ __forceinline__ ArgPair arg_warp(ArgPair a) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgPair b;
        b.v = __shfl_xor_sync(0xFFFFFFFFu, a.v, o);
        b.i = __shfl_xor_sync(0xFFFFFFFFu, a.i, o);
        a = arg_merge(a, b);
    }
    return a;
}
__device__ __forceinline__ ArgPair arg_block(ArgPair a, ArgPair* red) {
    a = arg_warp(a);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
    __syncthreads();
    if (threadIdx.x < 32) {
        ArgPair b = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : ArgPair{-INFINITY, 0xFFFFFFFFu};
        b = arg_warp(b);
        if (threadIdx.x == 0) red[0] = b;
    }
    __syncthreads();
    return red[0];
}

// stage 1: grid (n_chunks, batch); each block reduces `chunk` consecutive logits
__global__ void k_argmax_stage1(float* __restrict__ cand_v, uint32_t* __restrict__ cand_i, const float* __restrict__ logits,
                                uint32_t n, uint32_t chunk) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ ArgPair red[32];
    const float* row = logits + (size_t)blockIdx.y * n;
    const uint32_t lo = blockIdx.x * chunk, hi = min(n, lo + chunk);
    ArgPair best{-INFINITY, 0xFFFFFFFFu};
    for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = row[i];
        if (v > best.v) { best.v = v; best.i = i; }
    }
    best = arg_block(best, red);
    if (threadIdx.x == 0) {
        cand_v[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = best.v;
        cand_i[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = best.i;
    }
}

// stage 2: one block per sequence; writes the token, optionally advances the device state and the ring
// With `pair_out` (vocab-parallel head) it instead stores this rank's best as (value, index + idx_offset) and
// leaves the state alone: k_argmax_pairs picks the winner over all ranks.
__global__ void k_argmax_stage2(uint32_t* __restrict__ out_token, const float* __restrict__ cand_v, const uint32_t* __restrict__ cand_i,
                                uint32_t n_cand, SeqState* __restrict__ state, uint32_t* __restrict__ ring, uint32_t ring_slots,
                                ArgPair* __restrict__ pair_out, uint32_t idx_offset) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ ArgPair red[32];
    const uint32_t b = blockIdx.x;
    if (state && !state[b].active) return;
    ArgPair best{-INFINITY, 0xFFFFFFFFu};
    for (uint32_t i = threadIdx.x; i < n_cand; i += blockDim.x) {
        ArgPair c{cand_v[(size_t)b * n_cand + i], cand_i[(size_t)b * n_cand + i]};
        best = arg_merge(best, c);
    }
    best = arg_block(best, red);
    if (threadIdx.x == 0 && pair_out) {
        pair_out[b] = ArgPair{best.v, best.i == 0xFFFFFFFFu ? best.i : best.i + idx_offset};
    } else if (threadIdx.x == 0) {
        const uint32_t tok = (best.i == 0xFFFFFFFFu) ? 0u : best.i;
        if (out_token) out_token[b] = tok;
        if (state) {
            const uint32_t pos = state[b].pos;
            if (ring) ring[(size_t)b * ring_slots + (pos % ring_slots)] = tok;
            seq_advance(state + b, tok);
        }
    }
}

cudaError_t argmax(const LaunchCfg& lc, uint32_t* out_token, const float* logits, uint32_t n, uint32_t batch, float* cand_v,
                   uint32_t* cand_i, SeqState* state, uint32_t* ring, uint32_t ring_slots) {
    const uint32_t chunk = 2048;
    const uint32_t n_chunks = (n + chunk - 1) / chunk;
    cudaError_t e = launch(lc, k_argmax_stage1, dim3(n_chunks, batch), dim3(256), 0, cand_v, cand_i, logits, n, chunk);
    if (e != cudaSuccess) return e;
    return launch(lc, k_argmax_stage2, dim3(batch), dim3(256), 0, out_token, cand_v, cand_i, n_chunks, state, ring, ring_slots,
                  (ArgPair*)nullptr, 0u);
}

// Vocab-parallel head, step 1: this rank's best (value, global index) per sequence into pair_out[batch] (8 bytes each).
cudaError_t argmax_shard(const LaunchCfg& lc, void* pair_out, const float* logits, uint32_t n, uint32_t idx_offset, uint32_t batch,
                         float* cand_v, uint32_t* cand_i, SeqState* state) {
    const uint32_t chunk = 2048;
    const uint32_t n_chunks = (n + chunk - 1) / chunk;
    cudaError_t e = launch(lc, k_argmax_stage1, dim3(n_chunks, batch), dim3(256), 0, cand_v, cand_i, logits, n, chunk);
    if (e != cudaSuccess) return e;
    return launch(lc, k_argmax_stage2, dim3(batch), dim3(256), 0, (uint32_t*)nullptr, cand_v, cand_i, n_chunks, state,
                  (uint32_t*)nullptr, 0u, (ArgPair*)pair_out, idx_offset);
}

// Step 2, after the all-gather: pairs[rank][batch]; same rule (greater value, then lower index; no candidate -> 0).
__global__ void k_argmax_pairs(const ArgPair* __restrict__ pairs, uint32_t n_ranks, uint32_t batch, SeqState* __restrict__ state,
                               uint32_t* __restrict__ ring, uint32_t ring_slots) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch || !state[b].active) return;
    ArgPair best{-INFINITY, 0xFFFFFFFFu};
    for (uint32_t r = 0; r < n_ranks; ++r) best = arg_merge(best, pairs[(size_t)r * batch + b]);
    const uint32_t tok = (best.i == 0xFFFFFFFFu) ? 0u : best.i;
    const uint32_t pos = state[b].pos;
    if (ring) ring[(size_t)b * ring_slots + (pos % ring_slots)] = tok;
    seq_advance(state + b, tok);
}
cudaError_t argmax_pairs(const LaunchCfg& lc, const void* pairs, uint32_t n_ranks, uint32_t batch, SeqState* state, uint32_t* ring,
                         uint32_t ring_slots) {
    return launch(lc, k_argmax_pairs, dim3((batch + 63) / 64), dim3(64), 0, (const ArgPair*)pairs, n_ranks, batch, state, ring, ring_slots);
}
uint32_t argmax_chunks(uint32_t n) { return (n + 2047) / 2048; }

}  // namespace vb

// ---- C ABI: conversions and small ops -------------------------------------------------------------------
using namespace vb;

extern "C" {

int32_t vb_version(void) { return 1; }
const char* vb_last_error(void) { return vb::last_error(); }

int32_t vb_device_count(int32_t* out) {
    VB_REQUIRE(out != nullptr, "vb_device_count: null out");
    int n = 0;
    VB_CUDA(cudaGetDeviceCount(&n));
    *out = n;
    return VB_OK;
}

int32_t vb_op_fill_normal(float* dst, uint64_t n, uint64_t seed, uint64_t stream_id, float mean, float std, void* stream) {
    VB_REQUIRE(dst != nullptr || n == 0, "vb_op_fill_normal: null dst");
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    VB_CUDA(fill_normal(lc, dst, n, seed, stream_id, mean, std));
    return VB_OK;
}

int32_t vb_op_quantize(void* data, void* scales, const float* src, int32_t fmt, uint64_t rows, uint64_t cols, void* stream) {
    VB_REQUIRE(data && src, "vb_op_quantize: null pointer");
    VB_REQUIRE(fmt >= VB_FMT_F32 && fmt <= VB_FMT_I8PC, "vb_op_quantize: unknown format %d", fmt);
    VB_REQUIRE(fmt_shape_ok(fmt, cols), "vb_op_quantize: cols=%llu not valid for format %d", (unsigned long long)cols, fmt);
    VB_REQUIRE(wmat_scale_bytes(fmt, rows, cols) == 0 || scales, "vb_op_quantize: format %d needs a scale buffer", fmt);
    if (rows == 0) return VB_OK;
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    VB_CUDA(quantize(lc, data, scales, src, fmt, rows, cols));
    return VB_OK;
}

int32_t vb_op_dequantize(float* dst, const void* data, const void* scales, int32_t fmt, uint64_t rows, uint64_t cols, void* stream) {
    VB_REQUIRE(dst && data, "vb_op_dequantize: null pointer");
    VB_REQUIRE(fmt >= VB_FMT_F32 && fmt <= VB_FMT_I8PC, "vb_op_dequantize: unknown format %d", fmt);
    VB_REQUIRE(fmt_shape_ok(fmt, cols), "vb_op_dequantize: cols=%llu not valid for format %d", (unsigned long long)cols, fmt);
    VB_REQUIRE(wmat_scale_bytes(fmt, rows, cols) == 0 || scales, "vb_op_dequantize: format %d needs scales", fmt);
    if (rows == 0) return VB_OK;
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    VB_CUDA(dequantize(lc, dst, data, scales, fmt, rows, cols));
    return VB_OK;
}

int32_t vb_op_embed(float* dst, const uint32_t* tokens, const void* table, const void* scales, int32_t fmt,
                    uint32_t d_model, uint32_t vocab, uint32_t batch, void* stream) {
    VB_REQUIRE(dst && tokens && table, "vb_op_embed: null pointer");
    VB_REQUIRE(d_model % 8 == 0 && vocab > 0, "vb_op_embed: d_model must be a multiple of 8");
    if (batch == 0) return VB_OK;
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    VB_CUDA(embed(lc, dst, tokens, nullptr, table, scales, fmt, d_model, vocab, batch));
    return VB_OK;
}

int32_t vb_op_rmsnorm(float* dst, const float* x, const void* w, int32_t w_fmt, uint32_t dim, uint32_t batch, float eps, void* stream) {
    VB_REQUIRE(dst && x && w, "vb_op_rmsnorm: null pointer");
    VB_REQUIRE(dim > 0, "vb_op_rmsnorm: dim == 0");
    VB_REQUIRE(w_fmt == VB_FMT_F32 || w_fmt == VB_FMT_F16 || w_fmt == VB_FMT_BF16, "vb_op_rmsnorm: weight format %d", w_fmt);
    if (batch == 0) return VB_OK;
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    VB_CUDA(rmsnorm(lc, dst, x, w, w_fmt, dim, batch, eps));
    return VB_OK;
}

int32_t vb_op_rope(float* t, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta, void* stream) {
    VB_REQUIRE(t != nullptr, "vb_op_rope: null pointer");
    VB_REQUIRE(head_dim % 2 == 0, "vb_op_rope: odd head_dim");
    if (n_heads == 0 || head_dim == 0) return VB_OK;
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    VB_CUDA(rope(lc, t, n_heads, head_dim, pos, theta));
    return VB_OK;
}

int32_t vb_op_sample_argmax(uint32_t* out_token, const float* logits, uint32_t n, void* scratch, uint64_t scratch_bytes, void* stream) {
    VB_REQUIRE(out_token && logits && scratch, "vb_op_sample_argmax: null pointer");
    VB_REQUIRE(n > 0, "vb_op_sample_argmax: empty logits");
    const uint32_t nc = argmax_chunks(n);
    VB_REQUIRE(scratch_bytes >= (uint64_t)nc * 8, "vb_op_sample_argmax: scratch too small (%llu < %llu)",
               (unsigned long long)scratch_bytes, (unsigned long long)nc * 8);
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    float* cv = (float*)scratch;
    uint32_t* ci = (uint32_t*)(cv + nc);
    VB_CUDA(argmax(lc, out_token, logits, n, 1, cv, ci, nullptr, nullptr, 0));
    return VB_OK;
}

// ---- argmax without any allocation ------------------------------------------------------------------------
// Largest row the built-in scratch covers: 2^20 logits = 512 stage-1 candidates of 8 bytes.
#define VB_STATIC_ARGMAX_MAX_N (1u << 20)
static __device__ __align__(256) unsigned char g_argmax_scratch[(VB_STATIC_ARGMAX_MAX_N / 2048) * 8];
// In host code `g_argmax_scratch` is only a stand-in for the symbol; the device address is looked up once per
// device (with that device current) and kept here.
static void* g_argmax_scratch_dev[64] = {nullptr};

int32_t vb_op_sample_argmax_static(uint32_t* out_token, const float* logits, uint32_t n, void* stream) {
    VB_REQUIRE(out_token && logits, "vb_op_sample_argmax_static: null pointer");
    VB_REQUIRE(n > 0, "vb_op_sample_argmax_static: empty logits");
    VB_REQUIRE(n <= VB_STATIC_ARGMAX_MAX_N, "vb_op_sample_argmax_static: n=%u exceeds the built-in scratch (max %u logits); "
               "use vb_op_sample_argmax with your own scratch", n, (unsigned)VB_STATIC_ARGMAX_MAX_N);
    int dev = 0;
    VB_CUDA(cudaGetDevice(&dev));
    VB_REQUIRE(dev >= 0 && dev < 64, "vb_op_sample_argmax_static: device ordinal %d not supported", dev);
    if (!g_argmax_scratch_dev[dev]) {
        void* p = nullptr;
        VB_CUDA(cudaGetSymbolAddress(&p, g_argmax_scratch));  // set-up, first call on this device
        g_argmax_scratch_dev[dev] = p;
    }
    const uint32_t nc = argmax_chunks(n);
    float* cv = (float*)g_argmax_scratch_dev[dev];
    uint32_t* ci = (uint32_t*)(cv + nc);
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    // stage 1 writes every candidate slot that stage 2 reads, so nothing has to be cleared between calls
    VB_CUDA(argmax(lc, out_token, logits, n, 1, cv, ci, nullptr, nullptr, 0));
    return VB_OK;
}

int32_t vb_dev_alloc(void** out, uint64_t bytes) {
    VB_REQUIRE(out != nullptr, "vb_dev_alloc: null out");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
    if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc", __FILE__, __LINE__); return e == cudaErrorMemoryAllocation ? VB_ERR_OOM : VB_ERR_CUDA; }
    *out = p;
    return VB_OK;
}
int32_t vb_dev_free(void* p) { VB_CUDA(cudaFree(p)); return VB_OK; }
int32_t vb_dev_upload(void* dst, const void* src, uint64_t bytes) { VB_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice)); return VB_OK; }
int32_t vb_dev_download(void* dst, const void* src, uint64_t bytes) { VB_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost)); return VB_OK; }
int32_t vb_dev_sync(void) { VB_CUDA(cudaDeviceSynchronize()); return VB_OK; }

}  // extern "C"
