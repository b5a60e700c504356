// Temperature + nucleus (top-p) sampling on the device, one block per sequence.
//
// Reference: sample_top_p_f32 (src/runtime.rs:1092-1152) -- softmax at the given temperature, tokens sorted by
// descending probability, the shortest prefix whose mass reaches top_p, one coin scaled to that mass, the first
// token at which the running mass reaches it -- and its emitted C99 twin (src/runners/tinystories_smollm.c:506-529),
// which walks the unsorted cumulative distribution instead (`mode` 1).  Both fall back to the greedy rule when
// temperature <= 1e-5 or top_p <= 0.
//
// No sort: the two prefix decisions are thresholds on the probability value, found by bisection over the float
// bit pattern (31 passes over a row that sits in L2), and ties at a threshold are resolved in index order, the
// order the CPU checker uses for equal probabilities (the reference's unstable sort leaves it open).  Sums are
// block reductions in a fixed order: deterministic, but not the reference's sequential order, so a decision that
// sits within rounding of a threshold can go to the neighbouring token.
#include <math.h>

#include "vb_internal.cuh"
#include "vb_kernels.cuh"

namespace vb {

namespace {

constexpr int SP_THREADS = 1024;

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const uint32_t lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < SP_THREADS / 32; ++i) t += red[i];  // same order in every thread
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    const uint32_t lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = -INFINITY;
#pragma unroll
    for (int i = 0; i < SP_THREADS / 32; ++i) t = fmaxf(t, red[i]);
    return t;
}
__device__ __forceinline__ uint32_t block_sum_u32(uint32_t v, uint32_t* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    const uint32_t lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    uint32_t t = 0;
#pragma unroll
    for (int i = 0; i < SP_THREADS / 32; ++i) t += red[i];
    return t;
}

// sum of the probabilities whose bit pattern is >= t (all are positive floats: the pattern orders them)
__device__ __forceinline__ float mass_at_least(const float* __restrict__ p, uint32_t n, uint32_t t, float* red) {
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += SP_THREADS) {
        const float v = p[i];
        if (__float_as_uint(v) >= t) s += v;
    }
    return block_sum(s, red);
}

// largest pattern t in [lo, hi) with mass_at_least(t) >= want, given that lo qualifies and hi does not
__device__ uint32_t bisect_mass(const float* __restrict__ p, uint32_t n, uint32_t lo, uint32_t hi, float want, float* red) {
    while (hi - lo > 1) {
        const uint32_t mid = lo + (hi - lo) / 2;
        if (mass_at_least(p, n, mid, red) >= want) lo = mid; else hi = mid;
    }
    return lo;
}

// index of the j-th (1-based, index order) element whose pattern equals t; every thread returns it
__device__ uint32_t nth_equal(const float* __restrict__ p, uint32_t n, uint32_t t, uint32_t j, uint32_t* red_u, uint32_t* pick) {
    const uint32_t len = (n + SP_THREADS - 1) / SP_THREADS;
    const uint32_t i0 = min(n, threadIdx.x * len), i1 = min(n, i0 + len);
    uint32_t cnt = 0;
    for (uint32_t i = i0; i < i1; ++i) cnt += __float_as_uint(p[i]) == t ? 1u : 0u;
    // exclusive prefix of the per-thread counts: warp scan, then the warp totals
    const uint32_t lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    uint32_t inc = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= (uint32_t)o) inc += v;
    }
    __syncthreads();
    if (lane == 31) red_u[w] = inc;
    if (threadIdx.x == 0) *pick = 0xFFFFFFFFu;
    __syncthreads();
    uint32_t base = 0;
    for (uint32_t i = 0; i < w; ++i) base += red_u[i];
    const uint32_t before = base + inc - cnt;  // ties in earlier chunks
    if (cnt > 0 && before < j && j <= before + cnt) {
        uint32_t k = before;
        for (uint32_t i = i0; i < i1; ++i)
            if (__float_as_uint(p[i]) == t && ++k == j) { *pick = i; break; }
    }
    __syncthreads();
    return *pick;
}

struct SampleArgs {
    const float* logits;   // [batch][n]
    float* probs;          // [batch][n] scratch
    uint32_t n;
    float temperature, top_p;
    int mode;              // 0: src/runtime.rs rule, 1: the emitted C99 rule
    const float* coins;    // != null: one coin per sequence (device memory)
    float coin;            // coins == null and use_seed == 0: this coin for every sequence
    int use_seed;          // coins == null: 1 = coin drawn from (seed, sequence, position)
    uint64_t seed;
    SeqState* state;       // != null: inactive sequences are skipped, the winner is fed back and the position advances
    uint32_t* ring;
    uint32_t ring_slots;
    uint32_t* out_token;   // != null: winners [batch]
};

__device__ __forceinline__ float device_coin(uint64_t seed, uint32_t slot, uint32_t pos) {
    const uint64_t h = mix64(stream_key(seed, 0x5A4D504CULL + (uint64_t)slot) + ((uint64_t)pos + 1ULL) * 0x9E3779B97F4A7C15ULL);
    return (float)(uint32_t)(h >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(SP_THREADS) k_sample_top_p(SampleArgs a) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red[SP_THREADS / 32];
    __shared__ uint32_t red_u[SP_THREADS / 32];
    __shared__ uint32_t pick_s;
    const uint32_t b = blockIdx.x, n = a.n;
    if (a.state && !a.state[b].active) return;
    const float* lg = a.logits + (size_t)b * n;
    float* p = a.probs + (size_t)b * n;
    uint32_t tok = 0;
    if (a.temperature <= 1e-5f || a.top_p <= 0.0f) {
        // greedy rule (src/runtime.rs:1078-1088): first index of the maximum, NaN never wins, nothing above -inf -> 0
        float bv = -INFINITY;
        uint32_t bi = 0xFFFFFFFFu;
        for (uint32_t i = threadIdx.x; i < n; i += SP_THREADS) {
            const float v = lg[i];
            if (v > bv) { bv = v; bi = i; }
        }
        const float mx = block_max(bv, red);
        uint32_t cand = (bi != 0xFFFFFFFFu && bv == mx) ? bi : 0xFFFFFFFFu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xFFFFFFFFu, cand, o));
        __syncthreads();
        if ((threadIdx.x & 31) == 0) red_u[threadIdx.x >> 5] = cand;
        __syncthreads();
        uint32_t best = 0xFFFFFFFFu;
        for (int i = 0; i < SP_THREADS / 32; ++i) best = min(best, red_u[i]);
        tok = best == 0xFFFFFFFFu ? 0u : best;
    } else {
        const float coin_raw = a.coins ? a.coins[b] : (a.use_seed ? device_coin(a.seed, b, a.state ? a.state[b].pos : 0u) : a.coin);
        const float inv_temp = 1.0f / a.temperature;
        float m = -INFINITY;
        for (uint32_t i = threadIdx.x; i < n; i += SP_THREADS) m = fmaxf(m, lg[i] * inv_temp);
        const float max_l = block_max(m, red);
        float s = 0.0f;
        for (uint32_t i = threadIdx.x; i < n; i += SP_THREADS) {
            const float e = expf(__fsub_rn(__fmul_rn(lg[i], inv_temp), max_l));  // product rounded first, as the reference
            p[i] = e;
            s += e;
        }
        const float sum_exp = block_sum(s, red);
        if (a.mode == 1) {
            // unsorted walk: first index whose running sum of exp reaches coin * top_p * sum_exp
            const float target = coin_raw * a.top_p * sum_exp;
            const uint32_t len = (n + SP_THREADS - 1) / SP_THREADS;
            const uint32_t i0 = min(n, threadIdx.x * len), i1 = min(n, i0 + len);
            float part = 0.0f;
            for (uint32_t i = i0; i < i1; ++i) part += p[i];
            const uint32_t lane = threadIdx.x & 31, w = threadIdx.x >> 5;
            float inc = part;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float v = __shfl_up_sync(0xFFFFFFFFu, inc, o);
                if (lane >= (uint32_t)o) inc += v;
            }
            __syncthreads();
            if (lane == 31) red[w] = inc;
            if (threadIdx.x == 0) pick_s = 0xFFFFFFFFu;
            __syncthreads();
            float base = 0.0f;
            for (uint32_t i = 0; i < w; ++i) base += red[i];
            const float before = base + (inc - part), after = base + inc;
            // every chunk whose end reaches the target offers its first qualifying index; the lowest one wins
            if (i1 > i0 && after >= target) {
                float run = before;
                for (uint32_t i = i0; i < i1; ++i) {
                    run += p[i];
                    if (run >= target) { atomicMin(&pick_s, i); break; }
                }
            }
            __syncthreads();
            tok = pick_s == 0xFFFFFFFFu ? 0u : pick_s;
        } else {
            const float inv_sum = 1.0f / sum_exp;
            float pm = 0.0f;
            for (uint32_t i = threadIdx.x; i < n; i += SP_THREADS) {
                const float v = p[i] * inv_sum;
                p[i] = v;
                pm = fmaxf(pm, v);
            }
            __syncthreads();
            const uint32_t top_bits = __float_as_uint(block_max(pm, red));
            // nucleus: every probability above the threshold t*, plus the first `m_ties` (index order) equal to it
            const float total = mass_at_least(p, n, 0u, red);
            uint32_t t_star = 0;
            if (total >= a.top_p) t_star = bisect_mass(p, n, 0u, top_bits + 1u, a.top_p, red);
            const float tau = __uint_as_float(t_star);
            const float above = mass_at_least(p, n, t_star + 1u, red);
            uint32_t c = 0;
            for (uint32_t i = threadIdx.x; i < n; i += SP_THREADS) c += __float_as_uint(p[i]) == t_star ? 1u : 0u;
            const uint32_t n_ties = block_sum_u32(c, red_u);
            uint32_t m_ties = n_ties;
            if (total >= a.top_p && tau > 0.0f) {
                const float need = ceilf((a.top_p - above) / tau);
                m_ties = need < 1.0f ? 1u : (need > (float)n_ties ? n_ties : (uint32_t)need);
            }
            const float cum = above + (float)m_ties * tau;
            const float coin = fminf(fmaxf(coin_raw, 0.0f), 0.9999f);
            const float target = coin * cum;
            // the token at which the running mass (descending probability, ties by index) reaches the target
            const uint32_t t2 = bisect_mass(p, n, t_star, top_bits + 1u, target, red);
            const float tau2 = __uint_as_float(t2);
            const float above2 = mass_at_least(p, n, t2 + 1u, red);
            uint32_t c2 = 0;
            for (uint32_t i = threadIdx.x; i < n; i += SP_THREADS) c2 += __float_as_uint(p[i]) == t2 ? 1u : 0u;
            uint32_t n2 = block_sum_u32(c2, red_u);
            if (t2 == t_star) n2 = m_ties < n2 ? m_ties : n2;
            uint32_t j = 1;
            if (tau2 > 0.0f && target > above2) {
                const float need = ceilf((target - above2) / tau2);
                j = need < 1.0f ? 1u : (need > (float)n2 ? n2 : (uint32_t)need);
            }
            if (j < 1u) j = 1u;
            const uint32_t idx = nth_equal(p, n, t2, j, red_u, &pick_s);
            tok = idx == 0xFFFFFFFFu ? 0u : idx;
        }
    }
    if (threadIdx.x == 0) {
        if (a.out_token) a.out_token[b] = tok;
        if (a.state) {
            const uint32_t pos = a.state[b].pos;
            if (a.ring) a.ring[(size_t)b * a.ring_slots + (pos % a.ring_slots)] = tok;
            seq_advance(a.state + b, tok);
        }
    }
}

}  // namespace

cudaError_t sample_top_p(const LaunchCfg& lc, uint32_t* out_token, const float* logits, float* probs, uint32_t n, uint32_t batch,
                         float temperature, float top_p, int mode, const float* coins, float coin, int use_seed, uint64_t seed,
                         SeqState* state, uint32_t* ring, uint32_t ring_slots) {
    SampleArgs a;
    a.logits = logits; a.probs = probs; a.n = n; a.temperature = temperature; a.top_p = top_p; a.mode = mode; a.coins = coins;
    a.coin = coin; a.use_seed = use_seed; a.seed = seed; a.state = state; a.ring = ring; a.ring_slots = ring_slots; a.out_token = out_token;
    return launch(lc, k_sample_top_p, dim3(batch), dim3(SP_THREADS), 0, a);
}

}  // namespace vb

using namespace vb;

extern "C" int32_t vb_op_sample_top_p(uint32_t* out_token, const float* logits, uint32_t n, float temperature, float top_p,
                                      float random_coin, int32_t mode, void* scratch, uint64_t scratch_bytes, void* stream) {
    VB_REQUIRE(out_token && logits && n > 0, "vb_op_sample_top_p: null argument or empty row");
    VB_REQUIRE(mode == 0 || mode == 1, "vb_op_sample_top_p: mode %d (0: runtime rule, 1: emitted C99 rule)", mode);
    VB_REQUIRE(scratch && scratch_bytes >= (uint64_t)n * 4, "vb_op_sample_top_p: scratch of %llu bytes, need %llu",
               (unsigned long long)scratch_bytes, (unsigned long long)n * 4);
    LaunchCfg lc;
    lc.stream = (cudaStream_t)stream;
    VB_CUDA(sample_top_p(lc, out_token, logits, (float*)scratch, n, 1, temperature, top_p, mode, nullptr, random_coin, 0, 0, nullptr,
                         nullptr, 0));
    return VB_OK;
}
