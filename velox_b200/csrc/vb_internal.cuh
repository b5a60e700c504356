// Shared declarations of libvelox_b200: status handling, weight-matrix views, launch helpers and
// the device-side scalar routines (hashing, int4/int8 unpacking) every kernel file uses.
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/velox_b200.h"

namespace vb {

// ---- status ----------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int32_t cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define VB_CUDA(call)                                                             \
    do {                                                                          \
        cudaError_t _e = (call);                                                  \
        if (_e != cudaSuccess) return ::vb::cuda_fail(_e, #call, __FILE__, __LINE__); \
    } while (0)

#define VB_REQUIRE(cond, ...)                  \
    do {                                       \
        if (!(cond)) {                         \
            ::vb::set_error(__VA_ARGS__);      \
            return VB_ERR_INVALID;             \
        }                                      \
    } while (0)

// ---- weight matrix view ------------------------------------------------------------------------
// Canonical layout (also the exchange format of vb_load_tensor_packed / vb_export_tensor):
//   F32/F16/BF16 : [rows][cols] row-major
//   Q4G32        : data u32 [rows][cols/8], nibble order per word e0|e2<<4|e4<<8|e6<<12|e1<<16|e3<<20|e5<<24|e7<<28
//                  scales f16 [rows][cols/32]
//   Q4G64REF     : data as Q4G32, scales half2(scale,min) [rows][cols/64]
//   I8PC         : data s8 [rows][cols], scales f16 [rows]
struct WMat {
    const void* data = nullptr;
    const void* scales = nullptr;
    int32_t fmt = VB_FMT_F32;
    uint32_t rows = 0, cols = 0;
    // optional tile-major copy for the tuned int4 kernel (see vb_gemv_fast.cu); null when absent
    const void* tiled = nullptr;
    const void* tiled_scales = nullptr;
    // gate matrices only: gate and up interleaved 8 rows by 8 rows in one tile-major matrix of 2*rows rows
    const void* tiled_swiglu = nullptr;
    // the same two copies in the byte-per-nibble-pair block layout of the integer tensor-core kernel (vb_gemv_imma.cu)
    // (int8 per-channel weights: v3 = 2048-byte blocks; the row scales of the whole matrix follow its last block,
    // v3_scales points at this tensor's slice of them -- used while loading)
    const void* v3 = nullptr;
    const void* v3_scales = nullptr;
    const void* v3_swiglu = nullptr;
    // resident fp16 [rows][cols] copy for the tensor-core GEMMs (vb_gemm_tc.cu); null: converted per call.
    // f16_lo: what that copy's rounding dropped, as a second fp16 matrix (prefill chunks multiply hi + lo)
    const void* f16 = nullptr;
    const void* f16_lo = nullptr;
    // int8 per-channel weights for the integer tensor-core decode batches (vb_gemm_i8.cu): the matrix cut into
    // [128 rows][128 bytes of K] tiles, each stored as the 16 KB it occupies in shared memory (128-byte swizzle applied),
    // tiles ordered [row tile][k block]: one contiguous bulk copy per tile; null: tiled TMA from the canonical copy
    const void* i8_tiles = nullptr;
};

inline uint64_t wmat_data_bytes(int32_t fmt, uint64_t rows, uint64_t cols) {
    switch (fmt) {
    case VB_FMT_F32: return rows * cols * 4;
    case VB_FMT_F16: case VB_FMT_BF16: return rows * cols * 2;
    case VB_FMT_Q4G32: case VB_FMT_Q4G64REF: return rows * cols / 2;
    case VB_FMT_I8PC: return rows * cols;
    default: return 0;
    }
}
inline uint64_t wmat_scale_bytes(int32_t fmt, uint64_t rows, uint64_t cols) {
    switch (fmt) {
    case VB_FMT_Q4G32: return rows * (cols / 32) * 2;
    case VB_FMT_Q4G64REF: return rows * (cols / 64) * 4;
    case VB_FMT_I8PC: return rows * 2;
    default: return 0;
    }
}
inline bool fmt_shape_ok(int32_t fmt, uint64_t cols) {
    switch (fmt) {
    case VB_FMT_Q4G32: return cols % 32 == 0;
    case VB_FMT_Q4G64REF: return cols % 64 == 0;
    case VB_FMT_I8PC: return cols % 16 == 0;
    case VB_FMT_F16: case VB_FMT_BF16: return cols % 8 == 0;
    case VB_FMT_F32: return cols % 4 == 0;
    default: return false;
    }
}

// ---- per-sequence decode state (device resident; the reference's VeloxDecodeState) --------------
struct SeqState {
    uint32_t token;   // token to feed at this step
    uint32_t pos;     // its position
    uint32_t active;  // 0: slot skipped by every kernel (the reference's active_mask bit)
    uint32_t limit;   // tokens the slot's KV reservation holds (0: unchecked); positions >= limit are never written
};
// The sampler's state advance: the slot goes inactive when its next position would leave the reservation
// (the reference clamps with safe_step = min(step, S_max - 1), src/codegen.rs:1252; here the slot stops instead
// of overwriting its last row).
__host__ __device__ __forceinline__ void seq_advance(SeqState* s, uint32_t tok) {
    const uint32_t np = s->pos + 1;
    s->token = tok;
    s->pos = np;
    if (s->limit && np >= s->limit) s->active = 0;
}

// ---- launch helper: programmatic dependent launch aware -------------------------------------------
struct LaunchCfg {
    cudaStream_t stream = nullptr;
    bool pdl = false;          // launch with programmatic stream serialization
    uint64_t* counter = nullptr;
};

template <typename... KArgs, typename... Args>
inline cudaError_t launch(const LaunchCfg& lc, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = lc.stream;
    cudaLaunchAttribute attr[1];
    if (lc.pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (lc.counter) ++*lc.counter;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- device scalar helpers --------------------------------------------------------------------------
#ifdef __CUDACC__
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}
__host__ __device__ __forceinline__ uint64_t stream_key(uint64_t seed, uint64_t stream) {
    return mix64(seed ^ mix64(stream + 0x9E3779B97F4A7C15ULL));
}
__host__ __device__ __forceinline__ uint32_t lanes16_sum(uint64_t h) {
    return (uint32_t)(h & 0xFFFFu) + (uint32_t)((h >> 16) & 0xFFFFu) + (uint32_t)((h >> 32) & 0xFFFFu) +
           (uint32_t)(h >> 48);
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t bias) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(bias));
    return r;
}

// One packed word -> its 8 nibbles in element order e0..e7 as exact floats 0..15.
__device__ __forceinline__ void unpack8_f32(uint32_t p, float q[8]) {
    q[0] = (float)((p >> 0) & 15u);  q[2] = (float)((p >> 4) & 15u);
    q[4] = (float)((p >> 8) & 15u);  q[6] = (float)((p >> 12) & 15u);
    q[1] = (float)((p >> 16) & 15u); q[3] = (float)((p >> 20) & 15u);
    q[5] = (float)((p >> 24) & 15u); q[7] = (float)((p >> 28) & 15u);
}

// Grid-dependency control (programmatic dependent launch).  Both are no-ops when the kernel was
// launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

// Device-timestamp trace (profiling aid): record[0] = entry of block 0, record[1] = block 0 past the
// grid-dependency wait, record[2] = latest exit over all blocks (nanoseconds of the global timer).
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void trace_mark(unsigned long long* rec, int slot) {
    if (rec && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) rec[slot] = global_ns();
}
__device__ __forceinline__ void trace_exit(unsigned long long* rec) {
    if (rec && threadIdx.x == 0) atomicMax(rec + 2, global_ns());
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
#endif

}  // namespace vb
