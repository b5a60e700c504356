// Load-time unpack of GGUF Q4_K / Q6_K super-blocks into the reference's q4 group-64 format.
//
// Reference: velox_cuda_unpack_q4_k_fused_kernel / velox_cuda_unpack_q6_k_fused_kernel
// (src/runners/velox_cuda_runner_k2.cu:200-347): a super-block of 256 weights is dequantized (Q4_K: 8 sub-blocks
// with 6-bit scale and minimum under fp16 d / dmin; Q6_K: 16 sub-blocks with int8 scales under fp16 d) and
// re-quantized as 4 groups of 64 with scale = (max - min) / 15 and the group minimum, both used unrounded for the
// integers and stored rounded to half2(scale, min); nibbles are packed in the interleaved word order of
// src/codegen.rs:2363-2364.  Every rounding step is spelled out so that the integers and scales equal the CPU
// checker's bit for bit (the reference's `d * q - m` is one fused multiply-add on the GPU it was written for).
#include "vb_ctx.cuh"

namespace vb {

namespace {

__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
    if (j < 4) {
        *d = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

__device__ __forceinline__ float half_at(const uint8_t* p) {
    const unsigned short bits = (unsigned short)(p[0] | (p[1] << 8));
    return __half2float(__ushort_as_half(bits));
}

// 64 dequantized values -> 8 words + half2(scale, min)
__device__ void requant64(uint32_t* __restrict__ words, __half2* __restrict__ scale_min, const float* vals, float mn, float mx) {
    const float sc = (mx > mn) ? __fdiv_rn(__fsub_rn(mx, mn), 15.0f) : 1e-5f;
    *scale_min = __halves2half2(__float2half_rn(sc), __float2half_rn(mn));
    const float inv = __fdiv_rn(1.0f, sc);
    for (int w = 0; w < 8; ++w) {
        uint32_t q[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int qi = __float2int_rn(__fmul_rn(__fsub_rn(vals[w * 8 + k], mn), inv));
            q[k] = (uint32_t)(qi < 0 ? 0 : (qi > 15 ? 15 : qi));
        }
        words[w] = (q[0] << 0) | (q[2] << 4) | (q[4] << 8) | (q[6] << 12) | (q[1] << 16) | (q[3] << 20) | (q[5] << 24) | (q[7] << 28);
    }
}

// one thread per (super-block, group of 64)
__global__ void k_unpack_q4_k(uint32_t* __restrict__ words, __half2* __restrict__ scale_min, const uint8_t* __restrict__ src, uint64_t n_groups) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_groups; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t b = i >> 2;
        const int g = (int)(i & 3);
        const uint8_t* blk = src + b * 144;
        const float fd = half_at(blk), fdmin = half_at(blk + 2);
        uint8_t sc0, m0, sc1, m1;
        scale_min_k4(2 * g, blk + 4, &sc0, &m0);
        scale_min_k4(2 * g + 1, blk + 4, &sc1, &m1);
        const float d1 = __fmul_rn(fd, (float)sc0), mm1 = __fmul_rn(fdmin, (float)m0);
        const float d2 = __fmul_rn(fd, (float)sc1), mm2 = __fmul_rn(fdmin, (float)m1);
        const uint8_t* gq = blk + 16 + g * 32;
        float vals[64], mn = 1e30f, mx = -1e30f;
        for (int l = 0; l < 32; ++l) {
            const float v0 = __fmaf_rn(d1, (float)(gq[l] & 0x0F), -mm1);
            const float v1 = __fmaf_rn(d2, (float)(gq[l] >> 4), -mm2);
            vals[l] = v0;
            vals[l + 32] = v1;
            if (v0 < mn) mn = v0;
            if (v0 > mx) mx = v0;
            if (v1 < mn) mn = v1;
            if (v1 > mx) mx = v1;
        }
        requant64(words + i * 8, scale_min + i, vals, mn, mx);
    }
}

__global__ void k_unpack_q6_k(uint32_t* __restrict__ words, __half2* __restrict__ scale_min, const uint8_t* __restrict__ src, uint64_t n_groups) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_groups; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t b = i >> 2;
        const int g = (int)(i & 3), n = g >> 1, sub = g & 1;
        const uint8_t* blk = src + b * 210;
        const uint8_t* ql = blk + n * 64;
        const uint8_t* qh = blk + 128 + n * 32;
        const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192) + n * 8;
        const float d = half_at(blk + 208);
        float vals[64];
        for (int l = 0; l < 32; ++l) {
            const int is = l / 16;
            int qa, qb;
            if (sub == 0) {
                qa = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                qb = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            } else {
                qa = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                qb = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            }
            vals[l] = __fmul_rn(__fmul_rn(d, (float)sc[is + 4 * sub]), (float)qa);
            vals[l + 32] = __fmul_rn(__fmul_rn(d, (float)sc[is + 4 * sub + 2]), (float)qb);
        }
        float mn = vals[0], mx = vals[0];
        for (int k = 1; k < 64; ++k) {
            if (vals[k] < mn) mn = vals[k];
            if (vals[k] > mx) mx = vals[k];
        }
        requant64(words + i * 8, scale_min + i, vals, mn, mx);
    }
}

}  // namespace

cudaError_t unpack_gguf(const LaunchCfg& lc, void* words, void* scale_min, const void* src, int ggml_type, uint64_t n_blocks) {
    if (n_blocks == 0) return cudaSuccess;
    const uint64_t n_groups = n_blocks * 4;
    const unsigned blocks = (unsigned)((n_groups + 127) / 128 > 148 * 16 ? 148 * 16 : (n_groups + 127) / 128);
    if (ggml_type == VB_GGML_Q4_K)
        return launch(lc, k_unpack_q4_k, dim3(blocks), dim3(128), 0, (uint32_t*)words, (__half2*)scale_min, (const uint8_t*)src, n_groups);
    if (ggml_type == VB_GGML_Q6_K)
        return launch(lc, k_unpack_q6_k, dim3(blocks), dim3(128), 0, (uint32_t*)words, (__half2*)scale_min, (const uint8_t*)src, n_groups);
    return cudaErrorInvalidValue;
}

}  // namespace vb

using namespace vb;

extern "C" {

uint64_t vb_gguf_tensor_bytes(int32_t ggml_type, uint64_t n_elems) {
    switch (ggml_type) {
    case VB_GGML_F32: return n_elems * 4;
    case VB_GGML_F16: return n_elems * 2;
    case VB_GGML_Q4_K: return n_elems % 256 ? 0 : n_elems / 256 * 144;
    case VB_GGML_Q6_K: return n_elems % 256 ? 0 : n_elems / 256 * 210;
    default: return 0;
    }
}

int32_t vb_op_unpack_gguf(void* words, void* scale_min, const void* src_blocks, int32_t ggml_type, uint64_t n_blocks, void* stream) {
    VB_REQUIRE(words && scale_min && src_blocks, "vb_op_unpack_gguf: null argument");
    VB_REQUIRE(ggml_type == VB_GGML_Q4_K || ggml_type == VB_GGML_Q6_K, "vb_op_unpack_gguf: ggml type %d (12 = Q4_K, 14 = Q6_K)", ggml_type);
    LaunchCfg lc;
    lc.stream = (cudaStream_t)stream;
    VB_CUDA(unpack_gguf(lc, words, scale_min, src_blocks, ggml_type, n_blocks));
    return VB_OK;
}

// A GGUF tensor of any supported type into the context: plain types go through vb_load_tensor; the K-quants are
// unpacked to q4 group-64 on the GPU and, when the context stores something else, converted through fp32.
int32_t vb_load_tensor_gguf(vb_ctx* c, int32_t role, int32_t layer, const void* src, int32_t ggml_type, uint64_t rows, uint64_t cols) {
    VB_REQUIRE(c && src, "vb_load_tensor_gguf: null argument");
    if (ggml_type == VB_GGML_F32) return vb_load_tensor(c, role, layer, src, VB_FMT_F32, VB_LOC_HOST, rows, cols);
    if (ggml_type == VB_GGML_F16) return vb_load_tensor(c, role, layer, src, VB_FMT_F16, VB_LOC_HOST, rows, cols);
    VB_REQUIRE(ggml_type == VB_GGML_Q4_K || ggml_type == VB_GGML_Q6_K, "vb_load_tensor_gguf: ggml type %d is not F32, F16, Q4_K or Q6_K", ggml_type);
    VB_REQUIRE(cols % 256 == 0 && rows > 0, "vb_load_tensor_gguf: K-quant rows are whole super-blocks of 256 (cols=%llu)", (unsigned long long)cols);
    if (c->d.tp_size > 1) { set_error("vb_load_tensor_gguf: sharded contexts take K-quant tensors through vb_load_tensor (fp32/fp16)"); return VB_ERR_UNSUPPORTED; }
    VB_CUDA(cudaSetDevice(c->device));
    const uint64_t n_blocks = rows * cols / 256, raw_bytes = vb_gguf_tensor_bytes(ggml_type, rows * cols);
    const uint64_t word_bytes = rows * cols / 2, scale_bytes = rows * (cols / 64) * 4;
    unsigned char *raw = nullptr, *packed = nullptr;
    float* f32 = nullptr;
    int32_t rc = VB_OK;
    cudaError_t e = cudaMalloc((void**)&raw, raw_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&packed, word_bytes + scale_bytes);
    if (e != cudaSuccess) { if (raw) cudaFree(raw); cuda_fail(e, "cudaMalloc(gguf staging)", __FILE__, __LINE__); return VB_ERR_OOM; }
    LaunchCfg lc = lcfg(c, false);
    lc.counter = nullptr;
    e = cudaMemcpyAsync(raw, src, raw_bytes, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = unpack_gguf(lc, packed, packed + word_bytes, raw, ggml_type, n_blocks);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) rc = cuda_fail(e, "vb_load_tensor_gguf", __FILE__, __LINE__);
    if (rc == VB_OK) {
        uint32_t er, ec; int32_t fmt;
        if (!role_shape(c, role, &er, &ec, &fmt)) { set_error("vb_load_tensor_gguf: role %d is not part of this model", role); rc = VB_ERR_INVALID; }
        else if (fmt == VB_FMT_Q4G64REF) {
            rc = vb_load_tensor_packed(c, role, layer, packed, packed + word_bytes, VB_LOC_DEVICE, rows, cols);
        } else {
            e = cudaMalloc((void**)&f32, rows * cols * 4);
            if (e == cudaSuccess) e = dequantize(lc, f32, packed, packed + word_bytes, VB_FMT_Q4G64REF, rows, cols);
            if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
            if (e != cudaSuccess) rc = cuda_fail(e, "vb_load_tensor_gguf(convert)", __FILE__, __LINE__);
            else rc = vb_load_tensor(c, role, layer, f32, VB_FMT_F32, VB_LOC_DEVICE, rows, cols);
        }
    }
    cudaFree(raw);
    cudaFree(packed);
    if (f32) cudaFree(f32);
    return rc;
}

}  // extern "C"
