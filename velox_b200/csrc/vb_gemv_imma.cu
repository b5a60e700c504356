// Batch-1 matrix-vector kernel for symmetric int4 group-32 weights on the integer tensor-core path.
//
// Why integers.  At HBM speed a B200 SM receives ~45 int4 weights per clock.  Turning nibbles into fp16
// costs one logic instruction per two weights on the half-rate integer/logic pipe, which measured as the
// binding limit of the fp16-mma kernel (that pipe ~47 % busy at ~33 % of DRAM bandwidth).  Here a nibble
// only has to become a byte: one AND per FOUR weights (`w & 0x0F0F0F0F`, and the same of `w >> 4`), and
// mma.sync.m16n8k32.s8 multiplies the bytes 0..15 directly.
//
// Activations.  x is staged in shared memory as 16-bit fixed point per quantization group of 32:
// X = rint(x * p_g), p_g = 32000 / (the group's largest magnitude): 16-bit fixed point,
// split into two signed bytes X = 256*H + L (L in [-128,127]).  One m16n8k32 covers exactly one group of 32
// along K for 16 rows, with H and L in two of the eight B columns; four consecutive groups use the four
// column pairs of the same accumulator, so after the four mma of a 16x128 block lane (g,t) holds, for rows
// g and g+8, the exact integers sum(q*H) and sum(q*L) of group t.  The zero point is removed with the
// group's sum(X):  sum((q-8)*X) = 256*C_H + C_L - 8*SX, an exact int32 (|.| <= 32*8*32639 < 2^23), converted once and scaled
// by fp32(scale[row][group]) / p_g.  Nothing is rounded between x's 15-bit quantization and the final fp32
// accumulation.
//
// Storage ("v3" tile-major blocks of 1152 bytes, block order [row tile][k tile]): lane L = 4g+t finds at
// byte 16*L the four words (groups 0..3) of row g and at 512+16*L those of row g+8; in a word, byte b holds
// element 4t+b of the group in its low nibble and element 16+4t+b in its high nibble -- the A fragment of
// m16n8k32 after the two ANDs.  At byte 1024 + 4*L: half2(scale[row g][group t], scale[row g+8][group t]).
//
// Data movement.  Blocks are persistent, one of 16 warps per SM: two groups of 8 warps, each group on its own
// 16-row tile whose K extent its 8 warps split; both groups share one staged copy of x.  Each warp streams ITS
// blocks through a private shared-memory ring with cp.async (16-byte asynchronous copies that bypass L1 and
// need no registers); the data path has no block-wide barrier and no spin-wait at all.  Four slots per warp
// (three blocks in flight, ~55 KB per SM) measured fastest: rings of 6 to 12 slots were each slower in the
// captured graph, 3 and 2 slower too.  (A ring fed by one producer thread with cp.async.bulk + mbarriers measured
// ~4.4 TB/s at any depth on this part and was dropped here.)  Kernels are launched with programmatic stream
// serialization: weights never depend on the previous kernel, so every warp fills its ring BEFORE the
// grid-dependency wait and only then reads x.
//
// The inner loop is instruction-bound (ALU pipe 53 % busy at 42 % of DRAM peak in isolation, ~149 warp
// instructions per 16x128 block): anything added per block shows up directly -- a generalised block cursor for
// multi-product launches or for splitting a last partial tile round cost more than it saved.
#include <type_traits>

#include "vb_internal.cuh"
#include "vb_kernels.cuh"
#include "vb_tp_ll.cuh"

namespace vb {

constexpr int IM_WARPS = 8;                              // warps that share one 16-row tile (they split its K extent)
// tile groups per block: they share the staged x, nothing else.  (Measured and dropped: 4 groups = 32 warps at 64
// registers, +4 % step time; a 64-register block of 16 warps that takes half an SM so that the next kernel's block
// moves in early: gaps between kernels shrink to ~0.6 us but the two-slot ring that fits streams at 3.9 TB/s, +28 %.)
constexpr int IM_GROUPS = 2;
constexpr int IM_CONSUMERS = IM_GROUPS * IM_WARPS * 32;  // threads per block
constexpr int IM_BLK_BYTES = 1152;     // int4: 16 rows x 128 columns of nibbles + the block's 64 fp16 scales
constexpr int IM_BLK_BYTES_I8 = 2048;  // int8 per-channel: 16 rows x 128 columns of bytes (row scales live apart)
constexpr int IM_MAX_SMEM = 216 * 1024;
// kernel flavours: int4 one block per step, int8, int4 two consecutive k-blocks per step (halves the per-step overhead)
enum { IM_Q4 = 0, IM_I8 = 1, IM_Q4X2 = 2 };
template <int W> struct ImBlk { static constexpr int bytes = W == IM_I8 ? IM_BLK_BYTES_I8 : (W == IM_Q4X2 ? 2 * IM_BLK_BYTES : IM_BLK_BYTES); };

struct ImmaArgs {
    const unsigned char* w;  // v3 tile-major blocks
    const __half* wscales;   // int8 weights: one scale per row, in tile order
    uint32_t rows, K;        // rows of the (possibly gate/up-interleaved) matrix
    const float* x;
    float* dst;
    const void* norm_w; int norm_fmt; float eps;
    const SeqState* state;
    uint32_t dst_offset;
    int epilogue;            // EPI_STORE / EPI_RESIDUAL / EPI_SWIGLU (interleaved 8+8 tiles)
    unsigned long long* trace;  // optional timestamp record
    uint32_t spread;            // tile -> (block, group) mapping, see the kernel
    uint32_t nb_rows;           // multi-row flavour: rows of x / dst / state this launch serves (1..4)
    uint32_t dst_stride;        // multi-row flavour: elements between the rows of dst
    // tensor parallel (EPI_STORE of a row-parallel product): the output rows also go to every peer's receive
    // region as sequence-tagged 16-byte words {row 2i, seq, row 2i+1, seq}; push_size == 0: no push
    unsigned char* push_base[8];
    uint32_t push_rank, push_size, push_site, push_n_sites, push_max_pairs;
    uint64_t push_epoch_off, push_data_off;
    // ... and, with reduce_hidden, each block then gathers the peers' copies of ITS OWN rows and finishes the exchange
    // itself: hidden[row] += sum over ranks (rank order) of the partial rows.  Every rank runs the same tiles at about
    // the same time, so a block waits roughly one NVLink latency after its last push instead of the exchange being a
    // kernel of its own (launch, dependency wait, poll, exit).  At most IM_RED_TILES tiles per tile group.
    float* reduce_hidden;
    uint32_t* reduce_err;
    long long reduce_poll_clocks;
};
constexpr int IM_RED_TILES = 4;

__device__ __forceinline__ void imma_16832(int d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                                           const int c[4]) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

__device__ __forceinline__ void im_consumer_sync() { __syncthreads(); }
// barrier among the 8 warps of one tile group (hardware barrier 1 + group)
__device__ __forceinline__ void im_group_sync(uint32_t group) {
    asm volatile("bar.sync %0, %1;" ::"r"(1u + group), "n"(IM_WARPS * 32) : "memory");
}

__device__ __forceinline__ float im_norm_w(const void* w, int fmt, uint32_t i) {
    return fmt == VB_FMT_F16 ? __half2float(((const __half*)w)[i])
         : fmt == VB_FMT_BF16 ? __bfloat162float(((const __nv_bfloat16*)w)[i]) : ((const float*)w)[i];
}

// One chunk of 8 consecutive elements of x (already multiplied by the RMSNorm factors) -> the staged form.
// The four lanes that share a group of 32 agree on its power-of-two scale through shuffles, so all 32
// lanes of a warp must call this together (`valid` masks the stores).
__device__ __forceinline__ void im_stage_chunk(unsigned char* __restrict__ xq, int2* __restrict__ sxp,
                                               const float v[8], uint32_t c, bool valid) {
    float gmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) gmax = fmaxf(gmax, fabsf(v[i]));
    gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, 1));
    gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, 2));
    // scale that brings the group's largest magnitude to 32000: the two signed byte planes hold X in [-32639, 32639], so
    // every group uses the full 16 bits (a power-of-two scale would leave between one and two of them unused, and at 32
    // layers that rounding alone moved the logits by ~1e-2); 1 for an all-zero or non-finite group
    float p = 1.0f;
    if (gmax > 0.0f && gmax < 3.0e38f) p = __fdividef(32000.0f, gmax);
    if (!(p < 3.0e38f)) p = 1.0f;
    int X[8], s = 0;
    uint32_t hw[2] = {0u, 0u}, lw[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        X[i] = __float2int_rn(v[i] * p);
        X[i] = max(-32639, min(32639, X[i]));
        s += X[i];
        const int H = (X[i] + 128) >> 8, L = X[i] - (H << 8);
        hw[i >> 2] |= (uint32_t)(H & 0xFF) << (8 * (i & 3));
        lw[i >> 2] |= (uint32_t)(L & 0xFF) << (8 * (i & 3));
    }
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
    if (valid) {
        // group layout: 32 H bytes then 32 L bytes, each plane ordered so that the 8 bytes lane t feeds to the mma
        // (elements 4t..4t+3 and 16+4t..16+4t+3) are adjacent: element k sits at 8*((k&15)>>2) + 4*(k>>4) + (k&3)
        const uint32_t q = c & 3;  // which 8 of the group's 32 elements
        unsigned char* gb = xq + (size_t)(c >> 2) * 64 + (q & 1) * 16 + (q >> 1) * 4;
        *reinterpret_cast<uint32_t*>(gb) = hw[0];
        *reinterpret_cast<uint32_t*>(gb + 8) = hw[1];
        *reinterpret_cast<uint32_t*>(gb + 32) = lw[0];
        *reinterpret_cast<uint32_t*>(gb + 40) = lw[1];
        if (q == 0) sxp[c >> 2] = make_int2(s, __float_as_int(1.0f / p));  // the group's sum(X) and 1/p together
    }
}

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The sequence of 16x128 blocks one warp works through: block `kk` (kk = warp, warp+8, ...) of row tile `tile`
// (tile = blockIdx.x + group * gridDim.x, += 2 * gridDim.x).
struct BlockCursor {
    uint32_t tile, kk;
    __device__ __forceinline__ bool valid(uint32_t n_tiles) const { return tile < n_tiles; }
    __device__ __forceinline__ void advance(uint32_t KT, uint32_t warp, uint32_t tile_stride) {
        kk += IM_WARPS;
        if (kk >= KT) { kk = warp; tile += tile_stride; }
    }
};

// One warp requests one block (1152 bytes) into its private ring slot: 72 asynchronous 16-byte copies.
// `KT` and `cur.kk` count steps: blocks, or pairs of blocks for IM_Q4X2 (a pair is contiguous in memory)
template <int W>
__device__ __forceinline__ void issue_block(const unsigned char* __restrict__ w, uint32_t KT, const BlockCursor& cur, uint32_t slot_smem,
                                            uint32_t lane) {
    const unsigned char* src = w + ((size_t)cur.tile * KT + cur.kk) * ImBlk<W>::bytes;
    cp_async16(slot_smem + lane * 16, src + lane * 16);
    cp_async16(slot_smem + 512 + lane * 16, src + 512 + lane * 16);
    if constexpr (W == IM_I8) {
        cp_async16(slot_smem + 1024 + lane * 16, src + 1024 + lane * 16);
        cp_async16(slot_smem + 1536 + lane * 16, src + 1536 + lane * 16);
    } else if constexpr (W == IM_Q4X2) {
        cp_async16(slot_smem + 1024 + lane * 16, src + 1024 + lane * 16);
        cp_async16(slot_smem + 1536 + lane * 16, src + 1536 + lane * 16);
        if (lane < 16) cp_async16(slot_smem + 2048 + lane * 16, src + 2048 + lane * 16);
    } else {
        if (lane < 8) cp_async16(slot_smem + 1024 + lane * 16, src + 1024 + lane * 16);
    }
}

// grid: one persistent block of 16 warps per SM.  The block stages x once (all 512 threads) and then works as
// two independent groups of 8 warps, each on its own row tile; each warp streams its own blocks through a
// private ring of NS slots with cp.async (16-byte asynchronous copies, L1 bypassed): no block-wide
// synchronisation on the data path, ring filled before the grid-dependency wait.
// (Two blocks of 8 warps per SM move the same bytes but each stages its own copy of x: twice the L2 reads
// and twice the conversion work in the serial part of the kernel.)
// I8 selects the int8 per-channel weight format: blocks of 2048 bytes whose 16-byte pieces ARE the A fragments
// (lane L of k-step j at 512*j + 16*L: rows g and g+8, columns 4t..4t+3 and 16+4t..16+4t+3 of the step), no
// unpacking and no per-group weight scale -- the row scale is applied once in the epilogue.
// NB = 4 is the multi-row flavour: up to four rows of x (sequences of a batch, or prompt tokens of a prefill
// chunk) share one pass over the weights.  The eight B columns of an mma then carry (row r, H|L) for r = 0..3 of
// ONE quantization group, so every group needs its own mma and its own rescale (the four-groups-in-one-
// accumulator trick of the single-row kernel needs the columns for itself): ~1.3-1.6x the instructions of a
// single-row pass for four times the rows.
template <int NS, int W, int NB>
__global__ void __launch_bounds__(IM_CONSUMERS, 1) k_gemv_q4_imma(ImmaArgs a) {
    constexpr int BLK = ImBlk<W>::bytes;
    constexpr bool I8 = W == IM_I8;
    constexpr int SUB = W == IM_Q4X2 ? 2 : 1;  // 16x128 blocks per ring slot / loop step
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t K = a.K, KT = K / (128 * SUB), n_tiles = a.rows / 16;  // KT: steps along K of one tile
    unsigned char* ring = smem_raw;                                              // [IM_GROUPS * IM_WARPS][NS][IM_BLK_BYTES]
    // the rows of the multi-row flavour are padded so that the four rows a warp reads together fall into different banks
    constexpr uint32_t XPAD = NB > 1 ? 64 : 0, SPAD = NB > 1 ? 4 : 0;  // bytes per row of xq, int2 per row of sxp
    const uint32_t xrow = K * 2 + XPAD, srow = K / 32 + SPAD;
    unsigned char* xq = ring + (size_t)IM_GROUPS * IM_WARPS * NS * BLK;          // [NB][K/32][64] (+ pad)
    int2* sxp = reinterpret_cast<int2*>(xq + (size_t)NB * xrow);                 // [NB][K/32] {sum(X), 1/p} (+ pad)
    float* red = reinterpret_cast<float*>(sxp + (size_t)NB * srow);              // [IM_GROUPS][2][IM_WARPS][16] ([..][64] multi-row)
    __shared__ float ssq[NB * IM_GROUPS * IM_WARPS];

    const uint32_t lane = threadIdx.x & 31, wid = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const uint32_t group = wid / IM_WARPS, warp = wid % IM_WARPS;  // tile group, warp within the group
    const uint32_t gt = threadIdx.x % (IM_WARPS * 32);            // thread within the group
    // tile t of a round belongs to block t % gridDim.x, group t / gridDim.x: a short last (or only) round spreads
    // over as many SMs as it has tiles instead of filling both groups of half as many
    const uint32_t vtile0 = a.spread ? blockIdx.x + group * gridDim.x : IM_GROUPS * blockIdx.x + group, vstride = IM_GROUPS * gridDim.x;
    trace_mark(a.trace, 0);
    pdl_launch_dependents();

    // ---- prologue: weights do not depend on the previous kernel; fill the ring before waiting for x ----------
    const unsigned char* my_ring_ptr = ring + (size_t)wid * NS * BLK;
    const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(my_ring_ptr);
    BlockCursor icur{vtile0, warp};  // next block to request
    uint32_t issued = 0;  // (slot = counter % NS measured faster than a wrapping byte offset)
    if (warp >= KT) icur.tile = n_tiles;  // fewer k-blocks than warps: this warp has no blocks at all
#pragma unroll
    for (int i = 0; i < NS - 1; ++i) {
        if (icur.valid(n_tiles)) {
            issue_block<W>(a.w, KT, icur, my_ring + (issued % NS) * BLK, lane);
            icur.advance(KT, warp, vstride);
            ++issued;
        }
        cp_async_commit();
    }

    // Norm weights are parameters too: the 16-bit ones of a row that fits in registers are fetched now.
    constexpr int XC = 4;  // chunks of 8 elements a thread holds at once (rows of up to 16384 elements in one trip)
    const uint32_t n_chunks = K / 8;
    const bool in_regs = n_chunks <= (uint32_t)XC * IM_CONSUMERS;  // rows of up to 16384 elements: one trip through registers
    const bool nw_pre = a.norm_w && in_regs && (a.norm_fmt == VB_FMT_F16 || a.norm_fmt == VB_FMT_BF16);
    uint4 nw[XC];
#pragma unroll
    for (int i = 0; i < XC; ++i) {
        const uint32_t c = threadIdx.x + i * IM_CONSUMERS;
        nw[i] = (nw_pre && c < n_chunks) ? reinterpret_cast<const uint4*>(a.norm_w)[c] : make_uint4(0, 0, 0, 0);
    }

    // ---- x: only now wait for the producer kernel ----------------------------------------------------------------
    pdl_wait();
    trace_mark(a.trace, 1);
    // An inactive row still drains the pipeline; its x is loaded all the same (the buffer always exists), so that the
    // activity flags and x travel together instead of one memory trip after the other.
    bool act[NB], row_live[NB];
    bool active = false;
#pragma unroll
    for (int r = 0; r < NB; ++r) {
        row_live[r] = NB == 1 || (uint32_t)r < a.nb_rows;
        act[r] = row_live[r] && (!a.state || a.state[r].active);
        active = active || act[r];
    }
    // the step's exchange counter (advanced once at the start of the step), for the sequence tags of pushed rows
    unsigned long long push_epoch = 0;
    if (a.push_size > 1) push_epoch = *reinterpret_cast<const volatile unsigned long long*>(a.push_base[a.push_rank] + a.push_epoch_off);

    // x -> shared memory.  All of a thread's loads of a batch are issued before any value is used: one memory
    // trip per batch of XC * 4096 elements (the whole row up to 16384 elements), not one per chunk.
    bool staged = false;
    if constexpr (NB > 1) {
        // Rows short enough that all NB of them fit a thread's registers (up to 4096 elements each, 8192 for two
        // rounds of chunks): ONE memory trip and one pair of barriers for all rows instead of one per row.
        auto stage_rows = [&](auto prs_c) {
            constexpr int PRS = decltype(prs_c)::value;  // rounds of 512 chunks per row
            constexpr int SL = NB * PRS;
            float xr[SL][8];
#pragma unroll
            for (int i = 0; i < SL; ++i) {
                const int row = i / PRS;
                const uint32_t c = threadIdx.x + (i % PRS) * IM_CONSUMERS;
                float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
                if (row_live[row] && c < n_chunks) {
                    const float* x = a.x + (size_t)row * K + c * 8;
                    v0 = *reinterpret_cast<const float4*>(x); v1 = *reinterpret_cast<const float4*>(x + 4);
                }
                xr[i][0] = v0.x; xr[i][1] = v0.y; xr[i][2] = v0.z; xr[i][3] = v0.w;
                xr[i][4] = v1.x; xr[i][5] = v1.y; xr[i][6] = v1.z; xr[i][7] = v1.w;
            }
            if (a.norm_w) {
#pragma unroll
                for (int row = 0; row < NB; ++row) {
                    float ss = 0.0f;
#pragma unroll
                    for (int sub = 0; sub < PRS; ++sub)
#pragma unroll
                        for (int e = 0; e < 8; ++e) ss = fmaf(xr[row * PRS + sub][e], xr[row * PRS + sub][e], ss);
                    ss = warp_sum(ss);
                    if (lane == 0) ssq[row * (IM_GROUPS * IM_WARPS) + wid] = ss;
                }
            }
            im_consumer_sync();
            float inv[NB];
#pragma unroll
            for (int row = 0; row < NB; ++row) {
                inv[row] = 1.0f;
                if (a.norm_w && act[row]) {
                    float tot = 0.0f;
#pragma unroll
                    for (int w = 0; w < IM_GROUPS * IM_WARPS; ++w) tot += ssq[row * (IM_GROUPS * IM_WARPS) + w];
                    inv[row] = 1.0f / sqrtf(tot / (float)K + a.eps);
                }
            }
#pragma unroll
            for (int i = 0; i < SL; ++i) {
                const int row = i / PRS, sub = i % PRS;
                const uint32_t c = threadIdx.x + sub * IM_CONSUMERS;
                if ((uint32_t)sub * IM_CONSUMERS < n_chunks) {  // uniform over the block: every lane of a warp stages together
                    const bool valid = act[row] && c < n_chunks;
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = xr[i][e];
                    if (a.norm_w && valid) {
                        if (nw_pre) {
                            const uint32_t pk[4] = {nw[sub].x, nw[sub].y, nw[sub].z, nw[sub].w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float2 f;
                                if (a.norm_fmt == VB_FMT_F16) f = __half22float2(*reinterpret_cast<const __half2*>(&pk[e]));
                                else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk[e]));
                                v[2 * e] = (v[2 * e] * inv[row]) * f.x;
                                v[2 * e + 1] = (v[2 * e + 1] * inv[row]) * f.y;
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] = (v[e] * inv[row]) * im_norm_w(a.norm_w, a.norm_fmt, c * 8 + e);
                        }
                    }
                    im_stage_chunk(xq + (size_t)row * xrow, sxp + (size_t)row * srow, v, c, valid);
                }
            }
            im_consumer_sync();
        };
        const uint32_t prs = (n_chunks + IM_CONSUMERS - 1) / IM_CONSUMERS;
        if (prs == 1) { stage_rows(std::integral_constant<int, 1>{}); staged = true; }
        else if (prs == 2 && NB * 2 <= 8) { stage_rows(std::integral_constant<int, 2>{}); staged = true; }
    }
#pragma unroll 1
    for (int row = 0; row < NB && !staged; ++row) {
        const float* x = a.x + (size_t)row * K;
        unsigned char* xq_r = xq + (size_t)row * xrow;
        int2* sxp_r = sxp + (size_t)row * srow;
        bool active_r = act[0], live_r = row_live[0];
#pragma unroll
        for (int r = 1; r < NB; ++r) if (r == row) { active_r = act[r]; live_r = row_live[r]; }
        float xr[XC][8];
        auto load_batch = [&](uint32_t it0) {
#pragma unroll
            for (int i = 0; i < XC; ++i) {
                const uint32_t c = threadIdx.x + (it0 + i) * IM_CONSUMERS;
                float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
                if (live_r && c < n_chunks) { v0 = *reinterpret_cast<const float4*>(x + c * 8); v1 = *reinterpret_cast<const float4*>(x + c * 8 + 4); }
                xr[i][0] = v0.x; xr[i][1] = v0.y; xr[i][2] = v0.z; xr[i][3] = v0.w;
                xr[i][4] = v1.x; xr[i][5] = v1.y; xr[i][6] = v1.z; xr[i][7] = v1.w;
            }
        };
        const uint32_t n_it = (n_chunks + IM_CONSUMERS - 1) / IM_CONSUMERS;  // chunk rounds of the whole block
        float ss = 0.0f;
        if (in_regs) load_batch(0);
        if (active_r && a.norm_w) {
            for (uint32_t it0 = 0; it0 < n_it; it0 += XC) {
                if (!in_regs) load_batch(it0);
#pragma unroll
                for (int i = 0; i < XC; ++i)
#pragma unroll
                    for (int e = 0; e < 8; ++e) ss = fmaf(xr[i][e], xr[i][e], ss);  // chunks past the row are zero
            }
            ss = warp_sum(ss);
            if (lane == 0) ssq[wid] = ss;
        }
        im_consumer_sync();
        float inv = 1.0f;
        if (a.norm_w && active_r) {
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w < IM_GROUPS * IM_WARPS; ++w) tot += ssq[w];
            inv = 1.0f / sqrtf(tot / (float)K + a.eps);
        }
        for (uint32_t it0 = 0; it0 < n_it; it0 += XC) {
            if (!in_regs) load_batch(it0);
#pragma unroll
            for (int i = 0; i < XC; ++i) {
                if (it0 + i < n_it) {  // uniform over the block: every lane of a warp stages together
                    const uint32_t c = threadIdx.x + (it0 + i) * IM_CONSUMERS;
                    const bool valid = active_r && c < n_chunks;  // groups of 4 lanes are valid together
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = xr[i][e];
                    if (a.norm_w && valid) {
                        if (nw_pre) {
                            const uint32_t pk[4] = {nw[i].x, nw[i].y, nw[i].z, nw[i].w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float2 f;
                                if (a.norm_fmt == VB_FMT_F16) f = __half22float2(*reinterpret_cast<const __half2*>(&pk[e]));
                                else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk[e]));
                                v[2 * e] = (v[2 * e] * inv) * f.x;
                                v[2 * e + 1] = (v[2 * e + 1] * inv) * f.y;
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] = (v[e] * inv) * im_norm_w(a.norm_w, a.norm_fmt, c * 8 + e);
                        }
                    }
                    im_stage_chunk(xq_r, sxp_r, v, c, valid);
                }
            }
        }
        im_consumer_sync();
    }

    // ---- main loop: per tile, this warp's k-blocks in order; the ring stays NS-1 blocks ahead ----------------------
    uint32_t parity = 0, consumed = 0;
    const uint32_t gj = g >> 1, plane = g & 1;  // this lane feeds column g of B: group gj of a block, H or L bytes
    // single row: column g of B is (group gj of a block, plane); multi-row: (row gj of x, plane) of one group at a time
    const unsigned char* xq_lane = NB == 1 ? xq + (size_t)gj * 64 + plane * 32 + 8 * t : xq + (size_t)(gj % NB) * xrow + plane * 32 + 8 * t;
    const int2* sxp_lane = sxp + (size_t)(t % NB) * srow;  // multi-row: lane (g,t) ends up with the sums of row t of x
    // multi-row epilogue: thread gt < 32 of a group owns mma rows e_row and e_row + 8 of row e_seq of x
    const uint32_t e_row = gt >> 2, e_seq = gt & 3;
    bool e_act = act[0];
#pragma unroll
    for (int r = 1; r < NB; ++r) if ((uint32_t)r == e_seq) e_act = act[r];
    e_act = e_act && gt < 32 && e_seq < (uint32_t)NB;  // with two rows of x, columns 4..7 of the mma repeat 0..3
    float* e_dst = a.dst + (size_t)e_seq * a.dst_stride + a.dst_offset;
    for (uint32_t tile = vtile0; tile < n_tiles; tile += vstride, parity ^= 1) {
        // residual rows fetched early so that the epilogue does not wait on them
        float resid = 0.0f, resid1 = 0.0f;
        float row_scale = 1.0f, row_scale1 = 1.0f;
        if constexpr (NB == 1) {
            if (a.epilogue == EPI_RESIDUAL && gt < 16 && active) resid = a.dst[a.dst_offset + tile * 16 + gt];
            if (I8 && gt < 16) row_scale = __half2float(a.wscales[(size_t)tile * 16 + gt]);
        } else {
            if (a.epilogue == EPI_RESIDUAL && e_act) { resid = e_dst[tile * 16 + e_row]; resid1 = e_dst[tile * 16 + e_row + 8]; }
            if (I8 && gt < 32) {
                row_scale = __half2float(a.wscales[(size_t)tile * 16 + e_row]);
                row_scale1 = __half2float(a.wscales[(size_t)tile * 16 + e_row + 8]);
            }
        }
        float acc0 = 0.0f, acc1 = 0.0f;  // rows g and g+8, this lane's groups (t of every block it sees)
        for (uint32_t kk = warp; kk < KT; kk += IM_WARPS, ++consumed) {
            // request the block NS-1 ahead (its slot was read in the previous iteration), then wait for this one
            if (icur.valid(n_tiles)) {
                issue_block<W>(a.w, KT, icur, my_ring + (issued % NS) * BLK, lane);
                icur.advance(KT, warp, vstride);
                ++issued;
            }
            cp_async_commit();
            cp_async_wait<NS - 1>();
            __syncwarp();
            if (active) {
                const unsigned char* blk = my_ring_ptr + (consumed % NS) * BLK;
                if constexpr (NB > 1) {
#pragma unroll
                    for (int sub = 0; sub < SUB; ++sub) {
                        const unsigned char* sb = blk + sub * IM_BLK_BYTES;  // SUB == 1 for int8
                        const uint32_t kb = kk * SUB + sub;                  // 16x128 block index along K
                        const unsigned char* xb = xq_lane + (size_t)kb * 256;
                        // {sum(X), 1/p} of this lane's row of x for the block's four groups
                        const int4 s01 = reinterpret_cast<const int4*>(sxp_lane + kb * 4)[0];
                        const int4 s23 = reinterpret_cast<const int4*>(sxp_lane + kb * 4)[1];
                        const int sx[4] = {s01.x, s01.z, s23.x, s23.z};
                        const float ip[4] = {__int_as_float(s01.y), __int_as_float(s01.w), __int_as_float(s23.y), __int_as_float(s23.w)};
                        if constexpr (I8) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint4 af = reinterpret_cast<const uint4*>(sb + j * 512)[lane];
                                const uint2 bx = *reinterpret_cast<const uint2*>(xb + j * 64);
                                int d[4] = {0, 0, 0, 0};
                                imma_16832(d, af.x, af.y, af.z, af.w, bx.x, bx.y, d);
                                // lane (g,t): sums of q * H and q * L of row t of x over group j, for weight rows g and g+8
                                // (replacing the two I2F by integer/float adds of 1.5 * 2^23 measured no faster)
                                acc0 = fmaf((float)(d[0] * 256 + d[1]), ip[j], acc0);
                                acc1 = fmaf((float)(d[2] * 256 + d[3]), ip[j], acc1);
                            }
                        } else {
                            const uint4 wa = reinterpret_cast<const uint4*>(sb)[lane];
                            const uint4 wb = reinterpret_cast<const uint4*>(sb + 512)[lane];
                            // scales of rows g and g+8 for the four groups: 16 consecutive bytes
                            const uint4 sq = *reinterpret_cast<const uint4*>(sb + 1024 + 16 * g);
                            const uint32_t war[4] = {wa.x, wa.y, wa.z, wa.w};
                            const uint32_t wbr[4] = {wb.x, wb.y, wb.z, wb.w};
                            const uint32_t scr[4] = {sq.x, sq.y, sq.z, sq.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint32_t msk = 0x0F0F0F0Fu;
                                const uint2 bx = *reinterpret_cast<const uint2*>(xb + j * 64);
                                int d[4] = {0, 0, 0, 0};
                                imma_16832(d, war[j] & msk, wbr[j] & msk, (war[j] >> 4) & msk, (wbr[j] >> 4) & msk, bx.x, bx.y, d);
                                const int r0 = d[0] * 256 + d[1] - 8 * sx[j];  // |r| <= 32 * 8 * 32639 < 2^23
                                const int r1 = d[2] * 256 + d[3] - 8 * sx[j];
                                const float2 s2 = __half22float2(*reinterpret_cast<const __half2*>(&scr[j]));
                                acc0 = fmaf((float)r0 * ip[j], s2.x, acc0);
                                acc1 = fmaf((float)r1 * ip[j], s2.y, acc1);
                            }
                        }
                    }
                } else if constexpr (I8) {
                    // B operand: bytes of group gj of this block (k = 4t..4t+3 and 16+4t..16+4t+3), zero for the other groups
                    const uint2 bx = *reinterpret_cast<const uint2*>(xq_lane + (size_t)kk * 256);
                    const float ip = __int_as_float(sxp[kk * 4 + t].y);
                    int d[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const uint4 af = reinterpret_cast<const uint4*>(blk + jj * 512)[lane];
                        const uint32_t b0 = (gj == (uint32_t)jj) ? bx.x : 0u, b1 = (gj == (uint32_t)jj) ? bx.y : 0u;
                        imma_16832(d, af.x, af.y, af.z, af.w, b0, b1, d);
                    }
                    // lane (g,t): exact sums of q * X over group t for rows g and g+8 (no zero point)
                    const int r0 = d[0] * 256 + d[1];
                    const int r1 = d[2] * 256 + d[3];
                    acc0 = fmaf((float)r0, ip, acc0);
                    acc1 = fmaf((float)r1, ip, acc1);
                } else {
#pragma unroll
                    for (int sub = 0; sub < SUB; ++sub) {
                        const unsigned char* sb = blk + sub * IM_BLK_BYTES;
                        const uint32_t kb = kk * SUB + sub;  // 16x128 block index along K
                        const uint2 bx = *reinterpret_cast<const uint2*>(xq_lane + (size_t)kb * 256);
                        const int2 sp = sxp[kb * 4 + t];
                        const float ip = __int_as_float(sp.y);
                        const uint4 wa = reinterpret_cast<const uint4*>(sb)[lane];
                        const uint4 wb = reinterpret_cast<const uint4*>(sb + 512)[lane];
                        const __half2 sc = reinterpret_cast<const __half2*>(sb + 1024)[lane];
                        const uint32_t war[4] = {wa.x, wa.y, wa.z, wa.w};
                        const uint32_t wbr[4] = {wb.x, wb.y, wb.z, wb.w};
                        int d[4] = {0, 0, 0, 0};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t msk = 0x0F0F0F0Fu;
                            const uint32_t b0 = (gj == (uint32_t)j) ? bx.x : 0u, b1 = (gj == (uint32_t)j) ? bx.y : 0u;
                            imma_16832(d, war[j] & msk, wbr[j] & msk, (war[j] >> 4) & msk, (wbr[j] >> 4) & msk, b0, b1, d);
                        }
                        // lane (g,t): d[0],d[1] = sums against H and L of group t for row g; d[2],d[3] for row g+8
                        const int r0 = d[0] * 256 + d[1] - 8 * sp.x;
                        const int r1 = d[2] * 256 + d[3] - 8 * sp.x;
                        const float2 s2 = __half22float2(sc);
                        acc0 = fmaf((float)r0 * ip, s2.x, acc0);
                        acc1 = fmaf((float)r1 * ip, s2.y, acc1);
                    }
                }
            }
            __syncwarp();  // every lane is done with the slot before the next iteration overwrites its predecessor
        }
        if constexpr (NB > 1) {
            // every lane holds its own (weight row, row of x): only the 8 warps remain to be added
            float* rbuf = red + ((size_t)group * 2 + parity) * (IM_WARPS * 64);
            rbuf[warp * 64 + g * 4 + t] = acc0;
            rbuf[warp * 64 + 32 + g * 4 + t] = acc1;
            im_group_sync(group);
            if (e_act) {
                float v0 = 0.0f, v1 = 0.0f;
#pragma unroll
                for (int w = 0; w < IM_WARPS; ++w) { v0 += rbuf[w * 64 + gt]; v1 += rbuf[w * 64 + 32 + gt]; }
                if constexpr (I8) { v0 *= row_scale; v1 *= row_scale1; }
                if (a.epilogue == EPI_SWIGLU) {
                    e_dst[tile * 8 + e_row] = (v0 / (1.0f + expf(-v0))) * v1;  // mma rows 0..7 gate, 8..15 up
                } else if (a.epilogue == EPI_RESIDUAL) {
                    e_dst[tile * 16 + e_row] = resid + v0;
                    e_dst[tile * 16 + e_row + 8] = resid1 + v1;
                } else {
                    e_dst[tile * 16 + e_row] = v0;
                    e_dst[tile * 16 + e_row + 8] = v1;
                }
            }
            continue;
        }
        // the four lanes of a row hold different groups: add them, then reduce the 8 warps through shared memory
        acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 1); acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 2);
        acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 1); acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 2);
        // double-buffered by tile parity: one (group) barrier per tile
        float* rbuf = red + ((size_t)group * 2 + parity) * (IM_WARPS * 16);
        if (t == 0) { rbuf[warp * 16 + g] = acc0; rbuf[warp * 16 + g + 8] = acc1; }
        im_group_sync(group);
        if (gt < 16 && active) {
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < IM_WARPS; ++w) v += rbuf[w * 16 + gt];
            if constexpr (I8) v *= row_scale;
            if (a.epilogue == EPI_SWIGLU) {
                // tile = 8 gate rows (mma rows 0..7) over the same 8 up rows (mma rows 8..15)
                const float up = __shfl_down_sync(0x0000FFFFu, v, 8);
                if (gt < 8) a.dst[a.dst_offset + tile * 8 + gt] = (v / (1.0f + expf(-v))) * up;
            } else if (a.epilogue == EPI_RESIDUAL) {
                a.dst[a.dst_offset + tile * 16 + gt] = resid + v;
            } else {
                a.dst[a.dst_offset + tile * 16 + gt] = v;
                if (a.push_size > 1) {
                    // rows 2i and 2i+1 travel together: the even thread of each pair sends to all peers
                    const float other = __shfl_xor_sync(0x0000FFFFu, v, 1);
                    if ((gt & 1) == 0) {
                        const uint32_t seq = (uint32_t)(push_epoch * a.push_n_sites + a.push_site) + 1u;
                        const size_t slot = ((size_t)(a.push_site % TP_BUFS) * a.push_size + a.push_rank) * a.push_max_pairs +
                                            ((a.dst_offset + tile * 16 + gt) >> 1);
                        for (uint32_t p = 0; p < a.push_size; ++p) {
                            // with the fused gather this rank's own pair goes through its own region too (a local store)
                            if (p == a.push_rank && !a.reduce_hidden) continue;
                            uint4* dst = reinterpret_cast<uint4*>(a.push_base[p] + a.push_data_off) + slot;
                            asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(__float_as_uint(v)), "r"(seq),
                                         "r"(__float_as_uint(other)), "r"(seq) : "memory");
                        }
                    }
                }
            }
        }
    }
    if constexpr (NB == 1) {
        // fused exchange: gather the peers' copies of the rows this thread pushed and add everything onto the residual stream
        if (a.push_size > 1 && a.reduce_hidden && gt < 16 && (gt & 1) == 0 && active) {
            const uint32_t seq = (uint32_t)(push_epoch * a.push_n_sites + a.push_site) + 1u;
            for (uint32_t tile = vtile0; tile < n_tiles; tile += vstride) {
                const uint32_t row = a.dst_offset + tile * 16 + gt;
                const size_t pair = row >> 1;
                const uint4* recv = reinterpret_cast<const uint4*>(a.push_base[a.push_rank] + a.push_data_off) +
                                    (size_t)(a.push_site % TP_BUFS) * a.push_size * a.push_max_pairs + pair;
                float2 acc = *reinterpret_cast<const float2*>(a.reduce_hidden + row);
                for (uint32_t p = 0; p < a.push_size; ++p) {
                    uint4 raw;  // p == this rank: the pair this thread stored itself, there at once
                    poll_ll(recv + (size_t)p * a.push_max_pairs, seq, &raw, a.reduce_err, 0x300u | p, a.reduce_poll_clocks);
                    acc.x += __uint_as_float(raw.x);
                    acc.y += __uint_as_float(raw.z);
                }
                *reinterpret_cast<float2*>(a.reduce_hidden + row) = acc;
            }
        }
    }
    trace_exit(a.trace);
}

// ---- canonical -> v3 repack (load time) ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t canon_nibble(const uint32_t* __restrict__ canon, uint64_t row, uint32_t K, uint32_t e) {
    const uint32_t w = canon[row * (K / 8) + (e >> 3)], r = e & 7;
    return (w >> (((r & 1) ? 16 : 0) + (r >> 1) * 4)) & 15u;
}
// one thread per output word; fills `half` (0: mma rows 0..7, 1: rows 8..15) of every block:
// source row = rt * rows_per_tile + row_off + g
__global__ void k_tile_q4_v3_words(uint32_t* __restrict__ out, const uint32_t* __restrict__ canon, uint32_t n_tiles, uint32_t K,
                                   uint32_t rows_per_tile, uint32_t row_off, uint32_t half) {
    const uint32_t KT = K / 128;
    const uint64_t n = (uint64_t)n_tiles * KT * 128;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t j = i & 3, L = (i >> 2) & 31;
        const uint64_t blk = i >> 7;
        const uint32_t kt = blk % KT, rt = blk / KT, g = L >> 2, t = L & 3;
        const uint64_t row = (uint64_t)rt * rows_per_tile + row_off + g;
        const uint32_t e0 = kt * 128 + j * 32;
        uint32_t w = 0;
#pragma unroll
        for (uint32_t b = 0; b < 4; ++b) {
            w |= canon_nibble(canon, row, K, e0 + 4 * t + b) << (8 * b);
            w |= canon_nibble(canon, row, K, e0 + 16 + 4 * t + b) << (8 * b + 4);
        }
        out[blk * (IM_BLK_BYTES / 4) + half * 128 + (i & 127)] = w;
    }
}
__global__ void k_tile_q4_v3_scales(__half* __restrict__ out, const __half* __restrict__ canon, uint32_t n_tiles, uint32_t K,
                                    uint32_t rows_per_tile, uint32_t row_off, uint32_t half) {
    const uint32_t KT = K / 128;
    const uint64_t n = (uint64_t)n_tiles * KT * 32;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t t = i & 3, g = (i >> 2) & 7;
        const uint64_t blk = i >> 5;
        const uint32_t kt = blk % KT, rt = blk / KT;
        const uint64_t row = (uint64_t)rt * rows_per_tile + row_off + g;
        out[blk * (IM_BLK_BYTES / 2) + 512 + (g * 4 + t) * 2 + half] = canon[row * (K / 32) + kt * 4 + t];
    }
}

static cudaError_t tile_v3_half(const LaunchCfg& lc, void* tiled, const void* canon, const void* canon_scales, uint32_t n_tiles,
                                uint32_t K, uint32_t rows_per_tile, uint32_t row_off, uint32_t half) {
    const uint64_t nw = (uint64_t)n_tiles * (K / 128) * 128;
    unsigned blocks = (unsigned)((nw + 255) / 256 > 148 * 32 ? 148 * 32 : (nw + 255) / 256);
    cudaError_t e = launch(lc, k_tile_q4_v3_words, dim3(blocks), dim3(256), 0, (uint32_t*)tiled, (const uint32_t*)canon, n_tiles, K,
                           rows_per_tile, row_off, half);
    if (e != cudaSuccess) return e;
    const uint64_t ns = (uint64_t)n_tiles * (K / 128) * 32;
    blocks = (unsigned)((ns + 255) / 256 > 148 * 32 ? 148 * 32 : (ns + 255) / 256);
    return launch(lc, k_tile_q4_v3_scales, dim3(blocks), dim3(256), 0, (__half*)tiled, (const __half*)canon_scales, n_tiles, K,
                  rows_per_tile, row_off, half);
}

cudaError_t tile_q4_v3(const LaunchCfg& lc, void* tiled, const void* canon, const void* canon_scales, uint32_t rows, uint32_t K) {
    cudaError_t e = tile_v3_half(lc, tiled, canon, canon_scales, rows / 16, K, 16, 0, 0);
    if (e != cudaSuccess) return e;
    return tile_v3_half(lc, tiled, canon, canon_scales, rows / 16, K, 16, 8, 1);
}
// gate (which = 0) or up (which = 1) into the interleaved SwiGLU matrix: tile i = gate rows 8i..8i+7 | up rows 8i..8i+7
cudaError_t tile_q4_v3_swiglu(const LaunchCfg& lc, void* tiled, const void* canon, const void* canon_scales, uint32_t rows, uint32_t K,
                              int which) {
    return tile_v3_half(lc, tiled, canon, canon_scales, rows / 8, K, 8, 0, (uint32_t)which);
}

constexpr int IM_NB = 4;   // rows of x per weight pass of the multi-row flavour ...
constexpr int IM_NB2 = 2;  // ... and for rows of x too long for four of them to fit beside a ring (K > ~15k)

template <int W>
static cudaError_t imma_opt_in() {
    cudaError_t e;
#define VB_OPT_IN(...) if ((e = cudaFuncSetAttribute(__VA_ARGS__, cudaFuncAttributeMaxDynamicSharedMemorySize, IM_MAX_SMEM)) != cudaSuccess) return e
    VB_OPT_IN(k_gemv_q4_imma<8, W, 1>); VB_OPT_IN(k_gemv_q4_imma<4, W, 1>); VB_OPT_IN(k_gemv_q4_imma<3, W, 1>); VB_OPT_IN(k_gemv_q4_imma<2, W, 1>);
    VB_OPT_IN(k_gemv_q4_imma<4, W, IM_NB>); VB_OPT_IN(k_gemv_q4_imma<3, W, IM_NB>); VB_OPT_IN(k_gemv_q4_imma<2, W, IM_NB>);
    VB_OPT_IN(k_gemv_q4_imma<4, W, IM_NB2>); VB_OPT_IN(k_gemv_q4_imma<3, W, IM_NB2>); VB_OPT_IN(k_gemv_q4_imma<2, W, IM_NB2>);
#undef VB_OPT_IN
    return cudaSuccess;
}
cudaError_t gemv_imma_init() {
    cudaError_t e = imma_opt_in<IM_Q4>();
    if (e == cudaSuccess) e = imma_opt_in<IM_I8>();
    return e != cudaSuccess ? e : imma_opt_in<IM_Q4X2>();
}
bool imma_spread = false;  // deal a round's tiles to blocks first, then to the second group of each block
int imma_pair_ring = 3;  // int4, even number of k-blocks: two blocks per step with this ring depth (0 = one block per step)

bool imma_enabled = true;  // vb_set_option("gemv_imma", 0) routes batch 1 to the fp16-mma kernels
bool imma_multirow = true; // vb_set_option("gemv_multirow", 0) routes batch > 1 to the fp16-mma kernels

// shared memory besides the ring: staged x (+ row padding), group sums, the reduction buffers, slack for alignment
static size_t imma_fixed_smem(uint32_t K, int nb) {
    const size_t xrow = (size_t)K * 2 + (nb > 1 ? 64 : 0), srow = (size_t)(K / 32 + (nb > 1 ? 4 : 0)) * 8;
    return (size_t)nb * (xrow + srow) + (size_t)IM_GROUPS * 2 * IM_WARPS * (nb > 1 ? 64 : 16) * 4 + 256;
}
// ring depth that fits (0: none)
static size_t imma_ring_depth(uint32_t K, int nb, size_t blk_bytes) {
    const size_t fixed = imma_fixed_smem(K, nb), stage = (size_t)IM_GROUPS * IM_WARPS * blk_bytes;
    if (fixed + 2 * stage > (size_t)IM_MAX_SMEM) return 0;
    return ((size_t)IM_MAX_SMEM - fixed) / stage;
}

static int sm_count() {
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
    }
    return n_sm;
}

template <int W, int NB>
static cudaError_t imma_launch(const LaunchCfg& lc, const ImmaArgs& f, uint32_t max_ring) {
    const size_t fixed = imma_fixed_smem(f.K, NB);
    const size_t stage = (size_t)IM_GROUPS * IM_WARPS * ImBlk<W>::bytes;  // one ring slot of every warp
    size_t ns = imma_ring_depth(f.K, NB, ImBlk<W>::bytes);
    if (ns == 0) return cudaErrorInvalidConfiguration;
    if (max_ring >= 2 && ns > max_ring) ns = max_ring;
    if (NB > 1 && ns > 4) ns = 4;
    ns = ns >= 8 ? 8 : (ns >= 4 ? 4 : (ns >= 3 ? 3 : 2));  // ring depth per warp (template parameter); 4 measured fastest
    const int n_sm = sm_count();
    const uint32_t n_tiles = f.rows / 16;
    const uint32_t want = f.spread ? n_tiles : (n_tiles + IM_GROUPS - 1) / IM_GROUPS;
    const dim3 grid(want < (uint32_t)n_sm ? want : (uint32_t)n_sm);
    const size_t smem = fixed + ns * stage;
    if constexpr (NB == 1) {
        if (ns == 8) return launch(lc, k_gemv_q4_imma<8, W, 1>, grid, dim3(IM_CONSUMERS), smem, f);
    }
    if (ns == 4) return launch(lc, k_gemv_q4_imma<4, W, NB>, grid, dim3(IM_CONSUMERS), smem, f);
    if (ns == 3) return launch(lc, k_gemv_q4_imma<3, W, NB>, grid, dim3(IM_CONSUMERS), smem, f);
    return launch(lc, k_gemv_q4_imma<2, W, NB>, grid, dim3(IM_CONSUMERS), smem, f);
}

cudaError_t gemv_imma(const LaunchCfg& lc, const GemvArgs& a, bool* handled) {
    *handled = false;
    const bool i8 = a.w.fmt == VB_FMT_I8PC;
    if (!imma_enabled || !(a.w.fmt == VB_FMT_Q4G32 || i8)) return cudaSuccess;
    const bool multi = a.batch > 1;
    if (multi && !imma_multirow) return cudaSuccess;
    const bool swiglu = a.epilogue == EPI_SWIGLU;
    const void* w = swiglu ? a.w.v3_swiglu : a.w.v3;
    if (!w || a.w.cols % 128 != 0) return cudaSuccess;
    if (swiglu && (a.w2.rows != a.w.rows || a.w2.cols != a.w.cols)) return cudaSuccess;
    const uint32_t rows = swiglu ? 2 * a.w.rows : a.w.rows;
    if (rows % 16 != 0) return cudaSuccess;
    const size_t blk_bytes = i8 ? IM_BLK_BYTES_I8 : IM_BLK_BYTES;
    // rows of x per pass: four when they fit beside a ring of two slots, else two
    const int nb = !multi ? 1 : (imma_ring_depth(a.w.cols, IM_NB, blk_bytes) >= 2 ? IM_NB : IM_NB2);
    if (imma_ring_depth(a.w.cols, nb, blk_bytes) == 0) return cudaSuccess;
    ImmaArgs f;
    f.nb_rows = 1;
    f.dst_stride = a.dst_stride ? a.dst_stride : a.w.rows;
    f.w = (const unsigned char*)w; f.rows = rows; f.K = a.w.cols; f.x = a.x; f.dst = a.dst;
    // int8: the row scales follow the blocks of the (whole, possibly fused or interleaved) matrix
    f.wscales = i8 ? reinterpret_cast<const __half*>((const unsigned char*)w + (size_t)rows * a.w.cols) : nullptr;
    f.norm_w = a.norm_w; f.norm_fmt = a.norm_fmt; f.eps = a.eps; f.state = a.state;
    f.dst_offset = a.dst_offset; f.epilogue = a.epilogue;
    f.trace = a.trace;
    f.spread = imma_spread ? 1u : 0u;
    f.push_size = 0;
    f.reduce_hidden = nullptr; f.reduce_err = nullptr; f.reduce_poll_clocks = 0;
    if (!multi && a.push.links && a.epilogue == EPI_STORE && a.push.links->size > 1 && a.dst_offset % 2 == 0) {
        const TpLinks& l = *a.push.links;
        for (int r = 0; r < 8; ++r) f.push_base[r] = l.base[r];
        f.push_rank = l.rank; f.push_size = l.size; f.push_site = a.push.site; f.push_n_sites = a.push.n_sites;
        f.push_max_pairs = l.max_pairs; f.push_epoch_off = l.epoch_off; f.push_data_off = l.data_off;
        if (a.pushed) *a.pushed = true;
        // the block finishes the exchange itself when every tile group has only a few tiles to gather (the gather is serial)
        const uint32_t n_tiles = rows / 16, want = imma_spread ? n_tiles : (n_tiles + IM_GROUPS - 1) / IM_GROUPS;
        const uint32_t blocks = want < (uint32_t)sm_count() ? want : (uint32_t)sm_count(), groups = IM_GROUPS * blocks;
        if (a.push.reduce_hidden && a.dst_offset == 0 && (n_tiles + groups - 1) / groups <= (uint32_t)IM_RED_TILES) {
            f.reduce_hidden = a.push.reduce_hidden; f.reduce_err = a.push.err; f.reduce_poll_clocks = l.poll_clocks;
            if (a.reduced) *a.reduced = true;
        }
    }
    *handled = true;
    // two blocks per step when every warp's share of a tile is a whole number of pairs
    const bool pairs = !i8 && imma_pair_ring >= 2 && (a.w.cols / 128) % (2 * IM_WARPS) == 0;
    if (!multi) {
        if (i8) return imma_launch<IM_I8, 1>(lc, f, a.max_ring);
        if (pairs) return imma_launch<IM_Q4X2, 1>(lc, f, (uint32_t)imma_pair_ring);
        return imma_launch<IM_Q4, 1>(lc, f, a.max_ring);
    }
    // batch > 1: passes of up to nb rows of x, each one trip over the weights
    const bool pairs_fit = pairs && imma_ring_depth(a.w.cols, nb, 2 * IM_BLK_BYTES) >= 3;
    for (uint32_t b0 = 0; b0 < a.batch; b0 += (uint32_t)nb) {
        ImmaArgs p = f;
        p.nb_rows = a.batch - b0 < (uint32_t)nb ? a.batch - b0 : (uint32_t)nb;
        p.x = a.x + (size_t)b0 * a.w.cols;
        p.dst = a.dst + (size_t)b0 * f.dst_stride;
        p.state = a.state ? a.state + b0 : nullptr;
        cudaError_t e;
        if (nb == IM_NB) {
            e = i8 ? imma_launch<IM_I8, IM_NB>(lc, p, a.max_ring)
              : pairs_fit ? imma_launch<IM_Q4X2, IM_NB>(lc, p, (uint32_t)imma_pair_ring) : imma_launch<IM_Q4, IM_NB>(lc, p, a.max_ring);
        } else {
            e = i8 ? imma_launch<IM_I8, IM_NB2>(lc, p, a.max_ring)
              : pairs_fit ? imma_launch<IM_Q4X2, IM_NB2>(lc, p, (uint32_t)imma_pair_ring) : imma_launch<IM_Q4, IM_NB2>(lc, p, a.max_ring);
        }
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// ---- int8 per-channel: canonical [rows][K] bytes + fp16 row scales -> tile-major blocks, then the scales ----
// one thread per output word (4 consecutive k of one row)
__global__ void k_tile_i8_v3(uint32_t* __restrict__ out, const uint32_t* __restrict__ canon, uint32_t n_tiles, uint32_t K,
                             uint32_t rows_per_tile, uint32_t row_off, uint32_t half) {
    const uint32_t KT = K / 128;
    const uint64_t n = (uint64_t)n_tiles * KT * 256;  // words of one half (8 rows) of every block
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        // i -> (block, k-step j, lane L, upper/lower column half c)
        const uint32_t c = i & 1, L = (i >> 1) & 31, j = (i >> 6) & 3;
        const uint64_t blk = i >> 8;
        const uint32_t kt = blk % KT, rt = blk / KT, g = L >> 2, t = L & 3;
        const uint64_t row = (uint64_t)rt * rows_per_tile + row_off + g;
        const uint32_t k = kt * 128 + j * 32 + c * 16 + 4 * t;
        // fragment register r = 2*c + half: rows g (half 0) / g+8 (half 1), columns 4t.. (c 0) / 16+4t.. (c 1)
        out[blk * (IM_BLK_BYTES_I8 / 4) + j * 128 + L * 4 + 2 * c + half] = canon[(row * K + k) >> 2];
    }
}
__global__ void k_tile_i8_scales(__half* __restrict__ out, const __half* __restrict__ canon, uint32_t n_tiles, uint32_t rows_per_tile,
                                 uint32_t row_off, uint32_t half) {
    const uint32_t n = n_tiles * 8;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const uint32_t g = i & 7, rt = i >> 3;
        out[(size_t)rt * 16 + half * 8 + g] = canon[(size_t)rt * rows_per_tile + row_off + g];
    }
}
static cudaError_t tile_i8_half(const LaunchCfg& lc, void* blocks, void* scales, const void* canon, const void* canon_scales,
                                uint32_t n_tiles, uint32_t K, uint32_t rows_per_tile, uint32_t row_off, uint32_t half) {
    const uint64_t nw = (uint64_t)n_tiles * (K / 128) * 256;
    unsigned nb = (unsigned)((nw + 255) / 256 > 148 * 32 ? 148 * 32 : (nw + 255) / 256);
    cudaError_t e = launch(lc, k_tile_i8_v3, dim3(nb), dim3(256), 0, (uint32_t*)blocks, (const uint32_t*)canon, n_tiles, K, rows_per_tile,
                           row_off, half);
    if (e != cudaSuccess) return e;
    nb = (n_tiles * 8 + 255) / 256;
    return launch(lc, k_tile_i8_scales, dim3(nb ? nb : 1), dim3(256), 0, (__half*)scales, (const __half*)canon_scales, n_tiles, rows_per_tile,
                  row_off, half);
}
// plain matrix: tile i = rows 16i..16i+15
cudaError_t tile_i8_v3(const LaunchCfg& lc, void* blocks, void* scales, const void* canon, const void* canon_scales, uint32_t rows,
                       uint32_t K) {
    cudaError_t e = tile_i8_half(lc, blocks, scales, canon, canon_scales, rows / 16, K, 16, 0, 0);
    if (e != cudaSuccess) return e;
    return tile_i8_half(lc, blocks, scales, canon, canon_scales, rows / 16, K, 16, 8, 1);
}
// gate (which = 0) or up (which = 1) into the interleaved SwiGLU matrix: tile i = gate rows 8i..8i+7 | up rows 8i..8i+7
cudaError_t tile_i8_v3_swiglu(const LaunchCfg& lc, void* blocks, void* scales, const void* canon, const void* canon_scales, uint32_t rows,
                              uint32_t K, int which) {
    return tile_i8_half(lc, blocks, scales, canon, canon_scales, rows / 8, K, 8, 0, (uint32_t)which);
}

}  // namespace vb
