// Sequence-tagged 16-byte messages of the tensor-parallel exchange (see vb_tp.cu): {payload0, seq, payload1, seq}.
// The receiver polls a slot until both sequence words carry the number of the current exchange; every poll is bounded.
#pragma once

#include "vb_internal.cuh"

namespace vb {

__device__ __forceinline__ void st_ll(uint4* p, uint32_t a, uint32_t b, uint32_t seq) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(seq), "r"(b), "r"(seq) : "memory");
}
__device__ __forceinline__ uint4 ld_ll(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// Polls one slot; false (and the error word set) when the limit is reached.
__device__ __forceinline__ bool poll_ll(const uint4* p, uint32_t seq, uint4* out, uint32_t* err, uint32_t code, long long limit) {
    uint4 v = ld_ll(p);
    if (v.y == seq && v.w == seq) { *out = v; return true; }
    const long long t0 = clock64();
    for (uint32_t spin = 0;; ++spin) {
        v = ld_ll(p);
        if (v.y == seq && v.w == seq) { *out = v; return true; }
        // give up at the limit, or at once when an earlier wait already did (the step is lost anyway)
        const bool lost = (spin & 1023u) == 1023u && *reinterpret_cast<volatile uint32_t*>(err) != 0;
        if (lost || clock64() - t0 > limit) { atomicOr(err, code); *out = make_uint4(0, 0, 0, 0); return false; }
    }
}

}  // namespace vb
