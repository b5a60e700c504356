// Tensor-parallel exchange over NVLink peer mappings: the one-shot sum of the row-parallel partial products
// (after the O and the down projection) and the (value, index) exchange of the vocab-parallel head, written
// for the latency of a 32 KB message rather than for bandwidth.
//
// Every rank owns a receive region that all peers map (CUDA IPC).  A message element travels as a 16-byte
// store {payload0, seq, payload1, seq}: the receiver polls the slot until both sequence words carry the
// number of the current exchange, so no fence, flag or second round trip is needed (each 8-byte half is
// written atomically).  Regions are reused round-robin over four buffers; an exchange can only be one
// buffer ahead of the slowest rank because each one needs every rank's contribution to the one before.
// All polls are bounded: when one runs out the kernel records it in the error word and returns.
#include "vb_internal.cuh"
#include "vb_kernels.cuh"
#include "vb_tp_ll.cuh"

namespace vb {

namespace {


__global__ void k_tp_epoch(unsigned long long* epoch) {
    pdl_wait();
    if (threadIdx.x == 0 && blockIdx.x == 0) *epoch += 1ULL;
}

// hidden[i] += sum over ranks of partial_r[i], identical bits on every rank (fixed summation order).
// One thread per pair of elements; grid = ceil(n/2/256).
template <bool PUSHED>
__global__ void __launch_bounds__(256) k_tp_reduce_ll(TpLinks links, float* __restrict__ hidden, const float* __restrict__ partial,
                                                       uint32_t n, uint32_t site, uint32_t n_sites, uint32_t* __restrict__ err,
                                                       const SeqState* __restrict__ state, uint32_t row_elems) {
    pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;  // element pair
    // rows of inactive slots are neither sent nor awaited (activity is replicated: every rank skips the same rows)
    const bool valid = 2 * i < n && !(state && !state[(2 * i) / row_elems].active);
    const unsigned long long epoch = *reinterpret_cast<const volatile unsigned long long*>(links.base[links.rank] + links.epoch_off);
    const uint32_t seq = (uint32_t)(epoch * n_sites + site) + 1u;
    const size_t slot_elems = links.max_pairs;  // uint4 slots per (buffer, source)
    const size_t buf = site % TP_BUFS;
    float2 mine = make_float2(0.f, 0.f);
    if (valid) {
        mine = *reinterpret_cast<const float2*>(partial + 2 * (size_t)i);
        for (uint32_t p = 0; p < links.size && !PUSHED; ++p) {  // PUSHED: the product's epilogue sent them already
            if (p == links.rank) continue;
            uint4* dst = reinterpret_cast<uint4*>(links.base[p] + links.data_off) + (buf * links.size + links.rank) * slot_elems + i;
            st_ll(dst, __float_as_uint(mine.x), __float_as_uint(mine.y), seq);
        }
    }
    pdl_launch_dependents();
    if (!valid) return;
    float2 acc = *reinterpret_cast<const float2*>(hidden + 2 * (size_t)i);
    const uint4* recv = reinterpret_cast<const uint4*>(links.base[links.rank] + links.data_off) + buf * links.size * slot_elems + i;
    for (uint32_t p = 0; p < links.size; ++p) {
        float2 v = mine;
        if (p != links.rank) {
            uint4 raw;
            poll_ll(recv + p * slot_elems, seq, &raw, err, 0x100u | p, links.poll_clocks);
            v = make_float2(__uint_as_float(raw.x), __uint_as_float(raw.z));
        }
        acc.x += v.x;
        acc.y += v.y;
    }
    *reinterpret_cast<float2*>(hidden + 2 * (size_t)i) = acc;
}

// Vocab-parallel head: every rank sends (best value, global index) per sequence to all ranks; each picks the
// winner with the argmax rule (greater value, then lower index; no candidate -> token 0) and advances its state.
__global__ void k_tp_argmax_ll(TpLinks links, const uint2* __restrict__ pairs, uint32_t batch, uint32_t site, uint32_t n_sites,
                               SeqState* __restrict__ state, uint32_t* __restrict__ ring, uint32_t ring_slots, uint32_t* __restrict__ err) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch || !state[b].active) return;  // activity is replicated, so all ranks skip the same slots
    const unsigned long long epoch = *reinterpret_cast<const volatile unsigned long long*>(links.base[links.rank] + links.epoch_off);
    const uint32_t seq = (uint32_t)(epoch * n_sites + site) + 1u;
    const uint2 mine = pairs[b];
    for (uint32_t p = 0; p < links.size; ++p) {
        if (p == links.rank) continue;
        st_ll(reinterpret_cast<uint4*>(links.base[p] + links.pair_off) + (size_t)links.rank * links.max_batch + b, mine.x, mine.y, seq);
    }
    float best_v = -INFINITY;
    uint32_t best_i = 0xFFFFFFFFu;
    const uint4* recv = reinterpret_cast<const uint4*>(links.base[links.rank] + links.pair_off) + b;
    for (uint32_t p = 0; p < links.size; ++p) {
        uint2 c = mine;
        if (p != links.rank) {
            uint4 raw;
            if (!poll_ll(recv + (size_t)p * links.max_batch, seq, &raw, err, 0x200u | p, links.poll_clocks)) continue;
            c = make_uint2(raw.x, raw.z);
        }
        const float v = __uint_as_float(c.x);
        if (v > best_v || (v == best_v && c.y < best_i)) { best_v = v; best_i = c.y; }
    }
    const uint32_t tok = best_i == 0xFFFFFFFFu ? 0u : best_i;
    const uint32_t pos = state[b].pos;
    if (ring) ring[(size_t)b * ring_slots + (pos % ring_slots)] = tok;
    seq_advance(state + b, tok);
}

}  // namespace

// Layout of one rank's receive region: [epoch | pair slots [size][max_batch] | data slots [TP_BUFS][size][max_pairs]]
void tp_links_layout(TpLinks* l, uint32_t rank, uint32_t size, uint32_t max_elems, uint32_t max_batch) {
    l->rank = rank; l->size = size; l->max_batch = max_batch;
    l->max_pairs = (max_elems + 1) / 2;
    l->epoch_off = 0;
    l->pair_off = 256;
    l->data_off = (256 + (uint64_t)size * max_batch * 16 + 255) & ~255ULL;
    l->bytes = l->data_off + (uint64_t)TP_BUFS * size * l->max_pairs * 16;
}

cudaError_t tp_epoch_advance(const LaunchCfg& lc, const TpLinks& l) {
    return launch(lc, k_tp_epoch, dim3(1), dim3(32), 0, reinterpret_cast<unsigned long long*>(l.base[l.rank] + l.epoch_off));
}

cudaError_t tp_reduce(const LaunchCfg& lc, const TpLinks& l, float* hidden, const float* partial, uint32_t n, uint32_t site,
                      uint32_t n_sites, uint32_t* err, bool pushed, const SeqState* state, uint32_t row_elems) {
    if (n == 0) return cudaSuccess;
    if (n % 2 != 0 || (n + 1) / 2 > l.max_pairs || (state && (row_elems == 0 || row_elems % 2 != 0))) return cudaErrorInvalidValue;
    const uint32_t pairs = n / 2;
    if (pushed) return launch(lc, k_tp_reduce_ll<true>, dim3((pairs + 255) / 256), dim3(256), 0, l, hidden, partial, n, site, n_sites, err, state, row_elems);
    return launch(lc, k_tp_reduce_ll<false>, dim3((pairs + 255) / 256), dim3(256), 0, l, hidden, partial, n, site, n_sites, err, state, row_elems);
}

cudaError_t tp_argmax(const LaunchCfg& lc, const TpLinks& l, const void* pairs, uint32_t batch, uint32_t site, uint32_t n_sites,
                      SeqState* state, uint32_t* ring, uint32_t ring_slots, uint32_t* err) {
    if (batch > l.max_batch) return cudaErrorInvalidValue;
    return launch(lc, k_tp_argmax_ll, dim3((batch + 63) / 64), dim3(64), 0, l, (const uint2*)pairs, batch, site, n_sites, state, ring,
                  ring_slots, err);
}

}  // namespace vb
