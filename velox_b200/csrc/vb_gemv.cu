// Matrix-vector products y = x . W^T over weights in any storage format, with the fusions the decode
// step needs (RMSNorm prologue; residual / SwiGLU epilogues).
//
// Path 0 ("exact"): fp32 activations, weights dequantized to their exact fp32 value, fp32 FMA, one warp
// per output row.  It follows the reference arithmetic (src/runtime.rs:702-740 with the dequant contract)
// up to summation order and is the precision baseline the tuned paths are checked against.
#include "vb_internal.cuh"
#include "vb_kernels.cuh"

namespace vb {

cudaError_t gemv_fast(const LaunchCfg& lc, const GemvArgs& a, bool* handled);  // vb_gemv_fast.cu

template <int FMT>
__device__ __forceinline__ float dot_chunk8(const void* __restrict__ w, const void* __restrict__ scales, size_t row,
                                            uint32_t cols, uint32_t c, const float* __restrict__ xs) {
    // chunk c = elements [8c, 8c+8) of `row`
    float wv[8];
    const size_t e0 = row * cols + (size_t)c * 8;
    if (FMT == VB_FMT_F32) {
        const float4* p = reinterpret_cast<const float4*>((const float*)w + e0);
        float4 a = __ldg(p), b = __ldg(p + 1);
        wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w; wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
    } else if (FMT == VB_FMT_F16) {
        uint4 raw = __ldg(reinterpret_cast<const uint4*>((const __half*)w + e0));
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); wv[2 * i] = f.x; wv[2 * i + 1] = f.y; }
    } else if (FMT == VB_FMT_BF16) {
        uint4 raw = __ldg(reinterpret_cast<const uint4*>((const __nv_bfloat16*)w + e0));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); wv[2 * i] = f.x; wv[2 * i + 1] = f.y; }
    } else if (FMT == VB_FMT_Q4G32) {
        unpack8_f32(__ldg((const uint32_t*)w + (e0 >> 3)), wv);
        const float s = __half2float(__ldg((const __half*)scales + (e0 >> 5)));
#pragma unroll
        for (int i = 0; i < 8; ++i) wv[i] = __fmul_rn(wv[i] - 8.0f, s);
    } else if (FMT == VB_FMT_Q4G64REF) {
        unpack8_f32(__ldg((const uint32_t*)w + (e0 >> 3)), wv);
        const __half2 sm = __ldg((const __half2*)scales + (e0 >> 6));
        const float s = __low2float(sm), m = __high2float(sm);
#pragma unroll
        for (int i = 0; i < 8; ++i) wv[i] = fmaf(wv[i], s, m);
    } else {  // I8PC: the row scale is applied by the caller
        uint2 raw = __ldg(reinterpret_cast<const uint2*>((const int8_t*)w + e0));
        const int8_t* q = reinterpret_cast<const int8_t*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) wv[i] = (float)q[i];
    }
    const float4 x0 = *reinterpret_cast<const float4*>(xs + c * 8);
    const float4 x1 = *reinterpret_cast<const float4*>(xs + c * 8 + 4);
    float acc = wv[0] * x0.x;
    acc = fmaf(wv[1], x0.y, acc); acc = fmaf(wv[2], x0.z, acc); acc = fmaf(wv[3], x0.w, acc);
    acc = fmaf(wv[4], x1.x, acc); acc = fmaf(wv[5], x1.y, acc); acc = fmaf(wv[6], x1.z, acc); acc = fmaf(wv[7], x1.w, acc);
    return acc;
}

template <int FMT>
__device__ __forceinline__ float warp_row_dot(const WMat& m, size_t row, const float* __restrict__ xs, uint32_t lane) {
    float acc = 0.0f;
    const uint32_t chunks = m.cols / 8;
    for (uint32_t c = lane; c < chunks; c += 32) acc += dot_chunk8<FMT>(m.data, m.scales, row, m.cols, c, xs);
    acc = warp_sum(acc);
    if (FMT == VB_FMT_I8PC) acc *= __half2float(__ldg((const __half*)m.scales + row));
    return acc;
}

__device__ __forceinline__ float norm_w_at(const void* w, int fmt, uint32_t i) {
    return fmt == VB_FMT_F16 ? __half2float(((const __half*)w)[i])
         : fmt == VB_FMT_BF16 ? __bfloat162float(((const __nv_bfloat16*)w)[i]) : ((const float*)w)[i];
}

// grid (ceil(out/4), batch), 128 threads = 4 warps = 4 rows; dynamic smem: in_dim floats
template <int FMT>
__global__ void __launch_bounds__(128) k_gemv_exact(GemvArgs a) {
    extern __shared__ __align__(16) float xs[];
    __shared__ float red[4];
    const uint32_t b = blockIdx.y;
    pdl_wait();
    pdl_launch_dependents();
    if (a.state && !a.state[b].active) return;
    const uint32_t K = a.w.cols, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* x = a.x + (size_t)b * K;
    if (a.norm_w) {
        float ss = 0.0f;
        for (uint32_t i = threadIdx.x; i < K; i += 128) { float v = x[i]; xs[i] = v; ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        const float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)K + a.eps);
        for (uint32_t i = threadIdx.x; i < K; i += 128) xs[i] = (xs[i] * inv) * norm_w_at(a.norm_w, a.norm_fmt, i);
    } else {
        for (uint32_t i = threadIdx.x; i < K; i += 128) xs[i] = x[i];
    }
    __syncthreads();
    const uint32_t o = blockIdx.x * 4 + warp;
    if (o >= a.w.rows) return;
    float acc = warp_row_dot<FMT>(a.w, o, xs, lane);
    const uint32_t stride = a.dst_stride ? a.dst_stride : a.w.rows;
    float* d = a.dst + (size_t)b * stride + a.dst_offset + o;
    if (a.epilogue == EPI_SWIGLU) {
        const float up = warp_row_dot<FMT>(a.w2, o, xs, lane);
        if (lane == 0) { const float silu = acc / (1.0f + expf(-acc)); *d = silu * up; }
    } else if (lane == 0) {
        if (a.epilogue == EPI_RESIDUAL) *d += acc; else *d = acc;
    }
}

constexpr int GEMV_EXACT_MAX_SMEM = 200 * 1024;

template <int FMT>
static cudaError_t launch_exact(const LaunchCfg& lc, const GemvArgs& a) {
    const size_t smem = (size_t)a.w.cols * sizeof(float);
    if (smem > (size_t)GEMV_EXACT_MAX_SMEM) return cudaErrorInvalidValue;
    return launch(lc, k_gemv_exact<FMT>, dim3((a.w.rows + 3) / 4, a.batch), dim3(128), smem, a);
}

cudaError_t gemv_fast_init();  // vb_gemv_fast.cu

cudaError_t gemv_init() {
    cudaError_t e;
#define VB_OPT_IN(F) if ((e = cudaFuncSetAttribute(k_gemv_exact<F>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_EXACT_MAX_SMEM)) != cudaSuccess) return e
    VB_OPT_IN(VB_FMT_F32); VB_OPT_IN(VB_FMT_F16); VB_OPT_IN(VB_FMT_BF16); VB_OPT_IN(VB_FMT_Q4G32); VB_OPT_IN(VB_FMT_Q4G64REF); VB_OPT_IN(VB_FMT_I8PC);
#undef VB_OPT_IN
    if ((e = gemv_imma_init()) != cudaSuccess) return e;
    return gemv_fast_init();
}

cudaError_t kernels_init() {
    cudaError_t e = gemv_init();
    if (e != cudaSuccess) return e;
    return attn_init();
}

cudaError_t gemv(const LaunchCfg& lc, const GemvArgs& a, int path) {
    if (a.batch == 0 || a.w.rows == 0) return cudaSuccess;
    if (path != 0) {
        bool handled = false;
        cudaError_t e = gemv_imma(lc, a, &handled);
        if (handled || e != cudaSuccess) return e;
        e = gemv_fast(lc, a, &handled);
        if (handled || e != cudaSuccess) return e;
    }
    if (!a.w.data) return cudaErrorInvalidValue;  // a lean context holds no canonical copy for the exact kernels
    switch (a.w.fmt) {
    case VB_FMT_F32: return launch_exact<VB_FMT_F32>(lc, a);
    case VB_FMT_F16: return launch_exact<VB_FMT_F16>(lc, a);
    case VB_FMT_BF16: return launch_exact<VB_FMT_BF16>(lc, a);
    case VB_FMT_Q4G32: return launch_exact<VB_FMT_Q4G32>(lc, a);
    case VB_FMT_Q4G64REF: return launch_exact<VB_FMT_Q4G64REF>(lc, a);
    case VB_FMT_I8PC: return launch_exact<VB_FMT_I8PC>(lc, a);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace vb

using namespace vb;

extern "C" int32_t vb_op_matmul(float* dst, const float* x, const void* w, const void* scales, int32_t fmt,
                                uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* stream) {
    VB_REQUIRE(dst && x && w, "vb_op_matmul: null pointer");
    VB_REQUIRE(fmt >= VB_FMT_F32 && fmt <= VB_FMT_I8PC, "vb_op_matmul: unknown format %d", fmt);
    VB_REQUIRE(in_dim % 8 == 0 && fmt_shape_ok(fmt, in_dim), "vb_op_matmul: in_dim=%u not valid for format %d", in_dim, fmt);
    VB_REQUIRE(wmat_scale_bytes(fmt, out_dim, in_dim) == 0 || scales, "vb_op_matmul: format %d needs scales", fmt);
    VB_REQUIRE((size_t)in_dim * 4 <= 200 * 1024, "vb_op_matmul: in_dim=%u exceeds the shared-memory staging limit", in_dim);
    if (batch == 0 || out_dim == 0) return VB_OK;
    GemvArgs a;
    a.dst = dst; a.x = x;
    a.w.data = w; a.w.scales = scales; a.w.fmt = fmt; a.w.rows = out_dim; a.w.cols = in_dim;
    a.batch = batch;
    LaunchCfg lc; lc.stream = (cudaStream_t)stream;
    VB_CUDA(kernels_init());
    VB_CUDA(gemv(lc, a, 0));
    return VB_OK;
}
