/*
 * velox_b200.h -- C ABI of libvelox_b200, the sm_100a decode-step library for Velox.
 *
 * What this replaces.  Velox's compiler (src/codegen.rs) writes, per model, a .cu file with every
 * kernel as text plus the per-model launch sequence, exported as
 *     extern "C" void velox_<Model>_{prefill,decode}_cuda(VeloxCudaArena*, uint32_t token_in,
 *                                   size_t step, uint64_t active_mask, cudaStream_t)
 *     extern "C" void velox_<Model>_{prefill,decode}_graph_step_cuda(VeloxCudaArena*, uint64_t, cudaStream_t)
 * (src/codegen.rs:2803-2811, :3243-3253), and its host runner (src/runners/velox_cuda_runner.cu)
 * allocates the arenas, streams weights in, captures the decode step in a CUDA graph and replays it.
 * With this library the emitted file shrinks to a model description plus one call per fused IR
 * instruction (src/ir.rs:52-300), and the runner calls the engine entry points below.
 *
 * Conventions.  Plain C types only; every call returns an int32 status (VB_OK or a negative
 * VB_ERR_*) and never throws, aborts or exits; `stream` arguments are a cudaStream_t passed as
 * void* (NULL = the legacy default stream).  Device pointers are plain addresses.  A context is
 * used from one host thread at a time; tensor parallelism is one context per GPU / process.
 * After vb_decode_graph_build, vb_decode_run neither allocates nor synchronises, and the decode
 * step reads its position and input token from device memory, so one captured graph serves every
 * position (the property the reference gets from VeloxDecodeState, src/codegen.rs:1040-1050).
 */
#ifndef VELOX_B200_H
#define VELOX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VB_OK 0
#define VB_ERR_INVALID (-1)     /* bad argument / shape / format                           */
#define VB_ERR_CUDA (-2)        /* a CUDA runtime call failed (see vb_last_error)           */
#define VB_ERR_UNSUPPORTED (-3) /* valid request this build does not cover                  */
#define VB_ERR_OOM (-4)         /* device or KV-pool allocation failed                      */
#define VB_ERR_STATE (-5)       /* call order (e.g. decode before all weights are loaded)   */
#define VB_ERR_TIMEOUT (-6)     /* a bounded device-side wait ran out                       */
#define VB_ERR_COMM (-7)        /* tensor-parallel communicator failure                     */

/* Weight storage formats.  VB_FMT_Q4G64REF is the reference's own `--quantize q4_0` format
 * (src/codegen.rs:2337-2369); Q4G32 / I8PC are the symmetric formats of the benchmark configs. */
enum {
    VB_FMT_F32 = 0, VB_FMT_F16 = 1, VB_FMT_BF16 = 2,
    VB_FMT_Q4G32 = 3,    /* int4, groups of 32 along `in`, fp16 scale: (n-8)*scale              */
    VB_FMT_Q4G64REF = 4, /* int4, groups of 64, half2(scale,min): fmaf(n,scale,min)             */
    VB_FMT_I8PC = 5      /* int8, fp16 scale per output row: q*scale                            */
};

/* Tensor roles = the weight names of the .vlx models (examples/llama3_8b.vlx, qwen2_5_7b.vlx). */
enum {
    VB_ROLE_EMBED = 0,      /* [vocab][d]          */
    VB_ROLE_ATTN_NORM = 1,  /* [d]        per layer */
    VB_ROLE_WQ = 2,         /* [Hq*D][d]           */
    VB_ROLE_WK = 3,         /* [Hkv*D][d]          */
    VB_ROLE_WV = 4,         /* [Hkv*D][d]          */
    VB_ROLE_WO = 5,         /* [d][Hq*D]           */
    VB_ROLE_MLP_NORM = 6,   /* [d]                 */
    VB_ROLE_WGATE = 7,      /* [ffn][d]            */
    VB_ROLE_WUP = 8,        /* [ffn][d]            */
    VB_ROLE_WDOWN = 9,      /* [d][ffn]            */
    VB_ROLE_FINAL_NORM = 10,/* [d]                 */
    VB_ROLE_LM_HEAD = 11,   /* [vocab][d]          */
    VB_ROLE_BQ = 12, VB_ROLE_BK = 13, VB_ROLE_BV = 14, /* QKV bias, [rows]                     */
    VB_ROLE_MLA_NORM = 15, VB_ROLE_MLA_WDKV = 16, VB_ROLE_MLA_WABSQ = 17, VB_ROLE_MLA_WABSO = 18,
    VB_ROLE_COUNT = 19
};

enum { VB_LOC_HOST = 0, VB_LOC_DEVICE = 1 };
enum { VB_ATTN_GQA = 0, VB_ATTN_MLA_REF = 1 };

/* vb_model_desc.flags */
#define VB_FLAG_LEAN_WEIGHTS 1u /* keep, of each int4 g32 matrix, only the tile-major copy the batch-1 decode
                                 * kernel streams (1x the packed bytes instead of ~3-4x): for models sized to fill
                                 * the GPU.  Needs max_batch == 1; vb_export_tensor and the exact (gemv_path 0)
                                 * kernels are unavailable for those matrices. */

/* Model description: the VELOX_MODEL_* constants the compiler emits (src/codegen.rs:101-113) plus
 * the serving parameters the runner chooses.  Replaces VeloxCudaArena/TransformerConfig
 * (src/codegen.rs:1032-1043, src/runtime.rs:1160-1171). */
typedef struct vb_model_desc {
    uint32_t struct_bytes;    /* sizeof(vb_model_desc), for forward compatibility              */
    uint32_t vocab, d_model, n_layers, n_q_heads, n_kv_heads, head_dim, ffn_dim;
    uint32_t max_seq_len;     /* tokens per sequence the KV reservation may reach               */
    uint32_t max_batch;       /* sequences decoded per step (>=1)                               */
    float    rms_eps, rope_theta;
    uint32_t weight_fmt;      /* storage of the linear layers (VB_FMT_*)                        */
    uint32_t head_fmt;        /* storage of lm_head                                             */
    uint32_t embed_fmt;       /* storage of the embedding table (F32/F16/BF16/Q4G64REF)          */
    uint32_t qkv_bias;        /* 1: q=(x.Wq)+b_q ... before RoPE                                 */
    uint32_t tied_lm_head;    /* 1: lm_head reads the embedding table                           */
    uint32_t kv_block_tokens; /* paged-KV block size (16)                                       */
    uint32_t kv_blocks_total; /* pool size in blocks; 0 = max_batch*ceil(max_seq_len/block)      */
    uint32_t attn_kind;       /* VB_ATTN_*                                                      */
    uint32_t mla_latent;      /* latent width of the reference absorbed-MLA block               */
    uint32_t tp_rank, tp_size;/* tensor-parallel coordinates (tp_size 1 = single GPU)           */
    uint32_t flags;           /* VB_FLAG_* (0 = default)                                        */
    uint32_t reserved[7];
} vb_model_desc;

typedef struct vb_ctx vb_ctx;

/* ---- library ------------------------------------------------------------------------------ */
int32_t     vb_version(void);
const char* vb_last_error(void);           /* message of the last failing call on this thread  */
int32_t     vb_device_count(int32_t* out);

/* ---- engine: what velox_cuda_runner.cu:417-487 does around the emitted model --------------- */
/* Allocates weight arena, paged KV pool, activation buffers and the mapped token ring, once. */
int32_t vb_create(const vb_model_desc* desc, int32_t device, vb_ctx** out);
int32_t vb_destroy(vb_ctx* ctx);
/* Load one tensor given as [rows][cols] row-major in `src_fmt` (F32/F16/BF16) from host or device
 * memory; it is converted on the GPU to the context's storage format (quantized when that is an
 * int format), as stream_tensor_converted does (velox_cuda_runner.cu:154-199).  With tp_size>1 the
 * caller passes the FULL tensor and the context keeps its own shard. */
int32_t vb_load_tensor(vb_ctx* ctx, int32_t role, int32_t layer, const void* src, int32_t src_fmt,
                       int32_t src_loc, uint64_t rows, uint64_t cols);
/* Load a tensor that already is in the context's storage format, in the canonical layout: F32/F16/BF16
 * [rows][cols] row-major; Q4G32 / Q4G64REF u32 [rows][cols/8], a word holding elements e0..e7 as
 * e0|e2<<4|e4<<8|e6<<12|e1<<16|e3<<20|e5<<24|e7<<28 (src/codegen.rs:2363-2364), with f16 scales
 * [rows][cols/32] resp. half2(scale,min) [rows][cols/64]; I8PC s8 [rows][cols] with f16 scales [rows]. */
int32_t vb_load_tensor_packed(vb_ctx* ctx, int32_t role, int32_t layer, const void* data,
                              const void* scales, int32_t src_loc, uint64_t rows, uint64_t cols);
/* Synthetic weights: value i = mean + std * N_i(seed, stream), generated on the GPU and converted. */
int32_t vb_load_tensor_synthetic(vb_ctx* ctx, int32_t role, int32_t layer, uint64_t seed, uint64_t stream,
                                 float mean, float std, uint64_t rows, uint64_t cols);
/* Copy a stored tensor back in canonical layout (host buffers; sizes in bytes are checked). */
int32_t vb_export_tensor(vb_ctx* ctx, int32_t role, int32_t layer, void* data, uint64_t data_bytes,
                         void* scales, uint64_t scales_bytes);
int32_t vb_weight_bytes(vb_ctx* ctx, uint64_t* total_bytes);
/* GGUF tensor types this library reads (ggml type numbers), and the byte size of a tensor of n_elems elements
 * (0 for an unsupported type or a K-quant tensor that is not whole super-blocks). */
enum { VB_GGML_F32 = 0, VB_GGML_F16 = 1, VB_GGML_Q4_K = 12, VB_GGML_Q6_K = 14 };
uint64_t vb_gguf_tensor_bytes(int32_t ggml_type, uint64_t n_elems);
/* Load one tensor as it sits in a GGUF file (host memory, [rows][cols] with cols innermost): F32 / F16 as
 * vb_load_tensor; Q4_K / Q6_K are unpacked on the GPU to the reference's q4 group-64 format exactly as its loader does
 * (load_gguf_tensor_to_arena, src/runners/velox_cuda_runner_k2.cu:350-417) -- stored as is by a VB_FMT_Q4G64REF
 * context, converted through fp32 by any other. */
int32_t vb_load_tensor_gguf(vb_ctx* ctx, int32_t role, int32_t layer, const void* src, int32_t ggml_type, uint64_t rows, uint64_t cols);

/* Sequences.  A slot is one of max_batch sequences; reserve() assigns KV blocks for `n_tokens`
 * positions up front so that no decode step ever allocates. */
int32_t vb_seq_reserve(vb_ctx* ctx, int32_t slot, uint32_t n_tokens);
int32_t vb_seq_release(vb_ctx* ctx, int32_t slot);
int32_t vb_seq_set(vb_ctx* ctx, int32_t slot, uint32_t token, uint32_t pos, uint32_t active);

/* Prefill: runs the prompt of `slot` (positions 0..n-1), leaves the first generated token and
 * position n in the slot's device state (velox_cuda_runner.cu:494-520). */
int32_t vb_prefill(vb_ctx* ctx, int32_t slot, const uint32_t* tokens, uint32_t n_tokens);
/* One decode step for every active slot, launched eagerly on the context's stream
 * (velox_<Model>_decode_cuda, src/codegen.rs:3243-3253). */
int32_t vb_decode_step(vb_ctx* ctx);
/* Capture one decode step into a CUDA graph (velox_cuda_runner.cu:471-487). */
int32_t vb_decode_graph_build(vb_ctx* ctx);
/* Replay `n_steps` decode steps back to back with no host synchronisation in between
 * (velox_cuda_runner.cu:537-546).  If elapsed_ms != NULL the call brackets the replays with CUDA
 * events on the context's stream, waits for the end and returns the device time. */
int32_t vb_decode_run(vb_ctx* ctx, uint32_t n_steps, float* elapsed_ms);
/* Prompt-lookup speculative decoding of one sequence (src/runners/velox_cuda_runner_k2.cu:2127-2311; drafting
 * :1572-1611): prefill `prompt`, then generate n_new greedy tokens (the first comes from the prefill) where each
 * forward pass verifies up to max_draft_len (1..7) drafted tokens at once.  The tokens are those of plain greedy
 * decoding; `stats` (may be NULL) reports the draft bookkeeping the reference prints.  ema_floor: acceptance EMA below
 * which drafting pauses (reference default 0.20).  The slot needs n_prompt + n_new + max_draft_len reserved tokens;
 * every other slot must be inactive.  On return the slot's device state holds the next token to feed. */
typedef struct vb_spec_stats {
    uint64_t steps;        /* forward passes after the prefill                                  */
    uint64_t plain_steps;  /* of which single-token passes (no draft, or paused by the policy)   */
    uint64_t drafted, accepted;
    float    ema_final;
    uint32_t ladder_final;
} vb_spec_stats;
int32_t vb_generate_speculative(vb_ctx* ctx, int32_t slot, const uint32_t* prompt, uint32_t n_prompt, uint32_t n_new,
                                uint32_t max_draft_len, float ema_floor, uint32_t* out_tokens, vb_spec_stats* stats);
int32_t vb_sync(vb_ctx* ctx);
/* Tokens generated for `slot`: ring entries of positions [first_pos, first_pos+n). */
int32_t vb_read_tokens(vb_ctx* ctx, int32_t slot, uint32_t first_pos, uint32_t n, uint32_t* out);
int32_t vb_read_logits(vb_ctx* ctx, int32_t slot, float* out, uint64_t n_floats);
int32_t vb_read_hidden(vb_ctx* ctx, int32_t slot, float* out, uint64_t n_floats);
int32_t vb_read_state(vb_ctx* ctx, int32_t slot, uint32_t* token, uint32_t* pos);
/* The whole device state of a slot (the reference's VeloxDecodeState + its active_mask bit,
 * src/codegen.rs:1040-1050): `limit` = tokens of the slot's KV reservation.  The sampler clears `active`
 * when the next position would leave the reservation, and vb_decode_run / vb_decode_step return
 * VB_ERR_STATE instead of stepping a slot past it (the reference clamps the cache row with
 * safe_step = min(step, S_max - 1), src/runners/tinystories_smollm.cu:213). Any out pointer may be NULL. */
int32_t vb_read_state_ex(vb_ctx* ctx, int32_t slot, uint32_t* token, uint32_t* pos, uint32_t* active, uint32_t* limit);
/* Kernels launched through this context since creation (graph replays count their nodes). */
int32_t vb_launch_count(vb_ctx* ctx, uint64_t* out);
/* Algorithmic HBM bytes of one decode step at the slots' current positions (weights once + KV). */
int32_t vb_step_bytes(vb_ctx* ctx, uint64_t* weight_bytes, uint64_t* kv_bytes);
/* Device-timestamp trace of the last decode step (enable with vb_set_option(ctx, "trace", 1) before building
 * the graph).  One record of three global-timer values in ns per traced kernel, in launch order: entry of its
 * first block, that block past the grid-dependency wait, latest exit over all blocks.  The reference times
 * with host timers and cudaEvent pairs around whole phases (velox_cuda_runner.cu:39-49, :494-563); this is
 * the per-kernel view of the same thing.  Reading clears the records. */
int32_t vb_trace_read(vb_ctx* ctx, uint64_t* out, uint32_t max_records, uint32_t* n_records);
/* Tuning and diagnostic knobs (name/value); VB_ERR_INVALID for unknown names.  Changing one drops the captured
 * decode graph (build it again).  Defaults are what measured fastest.
 *   "gemv_path"      0: exact fp32 kernels for every product; 1 (default): the tuned kernels where they apply
 *   "gemv_imma"      1: integer tensor-core kernel for int4 g32 / int8 per-channel at batch 1; 0: fp16-mma kernels
 *   "gemv_tma"       with gemv_imma = 0: bulk-copy (TMA) ring instead of the register-prefetch kernel
 *   "gemv_ring", "head_ring", "ring_qkv|o|gu|down"   weight ring depth per warp (4); "gemv_pair_ring" (3, 0 = off):
 *                    ring depth when an int4 step takes two k-blocks
 *   "attn_mma"       1: tensor-core attention for the fp16 cache; 0: the scalar fp32 path
 *   "fuse_append"    1: bias + RoPE + KV append inside the attention kernel
 *   "prefill_chunk"  prompt tokens that go through the layers together in vb_prefill (16; 1 = token by token)
 *   "prefill_gemm"   1: prompts longer than "prefill_gemm_min" (48) tokens go through the layers in chunks of up to
 *                    "prefill_rows" (2048) tokens whose products run on the tcgen05 tensor cores; 0: batched kernels
 *   "prefill_split"  how those chunk products treat the 11 significant bits of fp16 operands: 2 (default): x and the
 *                    weights fp16 cannot hold exactly are multiplied as hi + lo parts (3 tensor-core products, results equal
 *                    to fp32 products to ~2^-22); 1: only x is split; 0: single fp16 operands (fastest; at 32 layers and 2048
 *                    cached rows the rounding moves the logits by up to 2.8e-2).  Set before the first long prefill.
 *   "prefill_flash"  1: those chunks use the causal tile attention kernel (head_dim 64 or 128); 0: one row per token
 *   "prefill_two_per_sm" 1 (default): 128-row tiles run two blocks per SM with half the ring depth each
 *   "prefill_wide"   1: 256 rows of x per tensor-core tile when a chunk has more than 128 rows (default 0)
 *   "decode_gemm"    1: the products of a decode step (lm_head included) run as tensor-core GEMMs, one row of x per
 *                    slot; default 1 when max_batch >= 16 and the weights are int8 per channel or fp16, else 0
 *   "decode_gemm_i8" 1 (default): those products over int8 per-channel weights (batches of up to 32) run on the integer
 *                    tensor cores straight from the stored bytes (exact arithmetic, one byte per weight from HBM); 0: through
 *                    resident fp16 copies
 *   "i8_tiles"       1 (default): those integer products stream tile-major copies of the int8 matrices (one contiguous 16 KB bulk
 *                    copy per tile, made on first use within "tc_resident_gb"); 0: tiled TMA from the canonical matrices
 *   "i8_half_ring"   1 (default): single integer products with more tiles than SMs (the lm_head) take half an SM's shared memory
 *                    per block (two blocks per SM: one block's epilogue overlaps the other's weight stream); 0: the whole ring
 *   "decode_split_k" 1 (default): decode-batch products with few 128-row tiles split K over several blocks per tile
 *                    (partials summed in a fixed order: results do not depend on scheduling)
 *   "tc_resident_gb" budget in GB for resident fp16 copies of the layer matrices used by those GEMMs (40; 0: convert
 *                    per call into the workspace)
 *   "pdl"            1: programmatic dependent launch between the kernels of a step
 *   "attn_tcgen05"   1: the decode attention of head_dim-128 models runs its two products as tcgen05.mma (tokens as the M dimension,
 *                    S^T and O^T in tensor memory); same results, measured slower than the mma.sync form (default 0)
 *   "attn_splits"    slices of the context per (sequence, KV head) in the decode attention (1..8; default: one per 32 tokens
 *                    of max_seq_len up to 8, fewer when the batch alone fills the GPU)
 *   "trace"          1: device time stamps per kernel (vb_trace_read)
 *   "tp_p2p"         1: NVLink push exchange when peer regions are open, 0: NCCL
 *   "tp_fused_push"  1: the row-parallel products send their rows to the peers from their own epilogue;
 *   "tp_fused_reduce" 1: ... and gather the peers' copies of their own rows, so the exchange needs no kernel of its own
 *   "tp_poll_ms"     limit of one exchange poll (default ~10000)
 *   "tp_p2p_standin" diagnostic: private stand-in regions instead of peers (every exchange then runs into its
 *                    poll limit; used by the time-out test) */
int32_t vb_set_option(vb_ctx* ctx, const char* name, int64_t value);
/* Sampler of the decode steps that follow: temperature <= 1e-5 or top_p <= 0 is the greedy argmax (the reference's own
 * fallback, src/runtime.rs:1100); otherwise temperature + nucleus sampling (vb_op_sample_top_p) with the coin of
 * sequence `slot` at position `pos` drawn from (seed, slot, pos) by a counter hash, so that a run is reproducible and
 * independent of batching.  mode 0: sample_top_p_f32 (src/runtime.rs:1092-1152); mode 1: the emitted C99 model's walk
 * over the unsorted distribution (src/runners/tinystories_smollm.c:506-529).  Drops the captured graph. */
int32_t vb_set_sampling(vb_ctx* ctx, float temperature, float top_p, uint64_t seed, int32_t mode);

/* Tensor parallel set-up (tp_size>1): every rank calls vb_tp_unique_id on rank 0's buffer contents
 * (128 bytes, exchanged by the host through its own channel) and then vb_tp_init. */
int32_t vb_tp_unique_id(void* id128);
int32_t vb_tp_init(vb_ctx* ctx, const void* id128);

/* Low-latency exchange over NVLink peer mappings (2..8 ranks on one node), used instead of NCCL once open:
 * each rank exports a 64-byte handle of its receive region, the host gathers all tp_size handles (rank
 * order) and every rank opens them.  The ranks' hosts must meet at a barrier after opening and before the
 * first step, and again before vb_destroy.  A rank that waits ~10 s for a peer gives up: the next
 * vb_sync / vb_read_tokens returns VB_ERR_TIMEOUT.  Option "tp_p2p" = 0 switches back to NCCL. */
int32_t vb_tp_p2p_export(vb_ctx* ctx, void* handle64);
int32_t vb_tp_p2p_open(vb_ctx* ctx, const void* handles, uint32_t n_handles);
/* Unmaps the peers' regions (this rank's own region stays until vb_destroy).  Shut-down order for a group:
 * every rank closes, the hosts meet at a barrier, then every rank destroys its context. */
int32_t vb_tp_p2p_close(vb_ctx* ctx);

/* ---- per-op entry points: one per fused IR instruction (src/ir.rs:52-300) ------------------- */
/* All pointers are device pointers; activations are fp32 as in the reference. */
/* Embed (src/runners/tinystories_smollm.cu:87): dst[b][d] = table[tokens[b]][:]. */
int32_t vb_op_embed(float* dst, const uint32_t* tokens, const void* table, const void* scales, int32_t fmt,
                    uint32_t d_model, uint32_t vocab, uint32_t batch, void* stream);
/* RmsNorm (src/runtime.rs:588-601). `w_fmt` F32 or F16. */
int32_t vb_op_rmsnorm(float* dst, const float* x, const void* w, int32_t w_fmt, uint32_t dim, uint32_t batch,
                      float eps, void* stream);
/* Matmul (src/runtime.rs:702-740): dst[b][o] = sum_k x[b][k] * W[o][k], W in canonical layout. */
int32_t vb_op_matmul(float* dst, const float* x, const void* w, const void* scales, int32_t fmt,
                     uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* stream);
/* Multi-row Matmul on the tcgen05 tensor cores (the reference's multi-token kernels for prefill chunks and
 * speculative-verify rows, src/runners/velox_cuda_runner_k2.cu:480-1085): dst[r][o] = sum_k x[r][k] * W[o][k]
 * for r < n_rows, same W layouts as vb_op_matmul.  x and W are rounded to fp16 for the product (int8 weights
 * exactly, with their row scale applied in fp32), accumulation is fp32.  `workspace`: device memory, 1024-byte
 * aligned, of at least vb_op_matmul_rows_workspace_bytes(in_dim, out_dim, n_rows) bytes; the call allocates nothing. */
uint64_t vb_op_matmul_rows_workspace_bytes(uint32_t in_dim, uint32_t out_dim, uint32_t n_rows);
int32_t vb_op_matmul_rows(float* dst, const float* x, const void* w, const void* scales, int32_t fmt,
                          uint32_t in_dim, uint32_t out_dim, uint32_t n_rows, void* workspace,
                          uint64_t workspace_bytes, void* stream);
/* RoPE, rotate-half convention (src/runtime.rs:745-768), in place on t[n_heads][head_dim]. */
int32_t vb_op_rope(float* t, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta, void* stream);
/* Decode attention over a contiguous fp32 cache laid out as the reference's
 * (src/runtime.rs:772-831): k/v [seq][n_kv*head_dim], q/out [n_q*head_dim]; split-K flash-decode. */
int32_t vb_op_gqa_attention(float* out, const float* q, const float* k_cache, const float* v_cache,
                            uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t pos,
                            void* scratch, uint64_t scratch_bytes, void* stream);
/* SampleArgmax (src/runtime.rs:1078-1088): first index of the maximum; NaN never wins. */
int32_t vb_op_sample_argmax(uint32_t* out_token, const float* logits, uint32_t n, void* scratch,
                            uint64_t scratch_bytes, void* stream);
/* SampleTopP (src/runtime.rs:1092-1152; mode 1: src/runners/tinystories_smollm.c:506-529): temperature + nucleus
 * sampling of one row of logits with the caller's coin in [0,1), as the reference takes it.  Equal probabilities
 * rank by index (the reference's unstable sort leaves their order open); sums are block reductions, so a decision
 * within rounding of a threshold may pick the neighbouring token of a sequential sum.  `scratch`: n floats. */
int32_t vb_op_sample_top_p(uint32_t* out_token, const float* logits, uint32_t n, float temperature, float top_p,
                           float random_coin, int32_t mode, void* scratch, uint64_t scratch_bytes, void* stream);
/* The same argmax for callers that must not allocate device memory and have none to spare: a runner that has
 * handed all of its memory to the arenas up front (the reference's "0 dynamic allocations" serving rule), code
 * running while a stream is being captured, or a host behind an FFI that forbids cudaMalloc.  No counterpart in
 * the reference.  The stage-1 candidates go to a scratch array built into the library (a file-scope __device__
 * array, 4 KiB, which every GPU that loads the library keeps until exit) instead of a caller buffer, so n is
 * limited to 1,048,576 logits; a larger n is refused with VB_ERR_INVALID.  The call itself allocates nothing
 * (no cudaMalloc/cudaFree, no allocating library routine).  The first call on a device looks the array's device
 * address up (cudaGetSymbolAddress): make that first call before any stream capture.  All calls on a device
 * share the one array: calls that may overlap on the GPU (different streams) race and must be serialised by
 * the caller.  Nothing in the array has to start at zero -- every slot read was written by the same call. */
int32_t vb_op_sample_argmax_static(uint32_t* out_token, const float* logits, uint32_t n, void* stream);
/* A weight matrix in caller-owned device memory: canonical layout of `fmt` (see vb_load_tensor_packed), [out][in]. */
typedef struct vb_weight {
    const void* data;
    const void* scales;  /* NULL for F32 / F16 / BF16 */
    int32_t     fmt;     /* VB_FMT_* */
} vb_weight;
/* Scratch (device bytes, 16-byte aligned) the fused ops below want for a layer shape. */
uint64_t vb_op_fused_scratch_bytes(uint32_t d_model, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t ffn_dim, uint32_t max_seq);
/* FusedNormQkvRopeAttn (src/ir.rs:232-248; emitted src/codegen.rs:1757, C99 twin src/runners/tinystories_smollm.c:277-311):
 * dst_attn[n_q*D] = GQA attention of rope(rmsnorm(x).Wq^T + b_q) over the layer's fp32 cache after K = rope(x'.Wk^T + b_k)
 * and V = x'.Wv^T + b_v were written to row `step` of k_layer / v_layer ([max_seq][n_kv*D] each, the reference's
 * contiguous layout; rows >= max_seq clamp to the last, its safe_step).  Biases are fp32 or NULL, w_norm fp32.
 * step_dev != NULL: the position is read from that device word instead of `step`, so a captured graph of this call
 * serves every position (what the reference gets from VeloxDecodeState). */
int32_t vb_op_fused_norm_qkv_rope_attn(float* dst_attn, const float* input_hidden, const float* w_norm, const vb_weight* w_q,
                                       const vb_weight* w_k, const vb_weight* w_v, const float* b_q, const float* b_k, const float* b_v,
                                       float* k_layer, float* v_layer, uint32_t max_seq, uint32_t step, const uint32_t* step_dev,
                                       uint32_t d_model, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, float eps, float theta,
                                       void* scratch, uint64_t scratch_bytes, void* stream);
/* FusedOutProjResSwiGluRes (src/ir.rs:249-272; emitted src/codegen.rs:1912, C99 twin tinystories_smollm.c:314-344):
 * mid = attn_in.Wo^T + residual_in; dst_hidden = mid + (silu(n.Wg^T) * (n.Wu^T)).Wd^T with n = rmsnorm(mid, w_post_norm).
 * dst_hidden may alias residual_in. */
int32_t vb_op_fused_outproj_res_swiglu_res(float* dst_hidden, const float* attn_in, const float* residual_in, const vb_weight* w_out,
                                           const float* w_post_norm, const vb_weight* w_gate, const vb_weight* w_up, const vb_weight* w_down,
                                           uint32_t d_model, uint32_t attn_dim, uint32_t ffn_dim, float eps, void* scratch,
                                           uint64_t scratch_bytes, void* stream);
/* KVWrite (src/ir.rs:83): k / v [kv_dim] into row `step` (or *step_dev) of the layer's fp32 cache. */
int32_t vb_op_kv_write(float* k_layer, float* v_layer, const float* k, const float* v, uint32_t step, const uint32_t* step_dev,
                       uint32_t kv_dim, uint32_t max_seq, void* stream);
/* SwiGlu (src/ir.rs:158; src/runtime.rs:1048-1073 without the residual): dst[d] = (silu(x.Wg^T) * (x.Wu^T)).Wd^T.
 * scratch: ffn_dim floats. */
int32_t vb_op_swiglu(float* dst, const float* input, const vb_weight* w_gate, const vb_weight* w_up, const vb_weight* w_down,
                     uint32_t d_model, uint32_t ffn_dim, void* scratch, uint64_t scratch_bytes, void* stream);
/* FusedMlaAbsorbedAttn (src/runtime.rs:944-1044): one layer's latent pool [max_seq][latent], fp32. */
int32_t vb_op_mla_absorbed(float* dst, const float* x, const float* w_norm, const float* w_dkv,
                           const float* w_absq, const float* w_abso, float* latent_pool, uint32_t step,
                           uint32_t hidden, uint32_t latent, uint32_t max_seq, float eps,
                           void* scratch, uint64_t scratch_bytes, void* stream);
/* Multi-head latent attention decode in the weight-absorbed form, the attention core of the DeepSeek-V3-style stack the
 * reference's model file declares (examples/deepseek_v3_mla.vlx:18-45; decode scope :117-150 `mla_decode_absorbed`); the
 * reference's runtime implements only the single-head block above.  For sequence b and head h:
 *   out[b][h][:512] = sum_t softmax_t(scale * q[b][h][:576] . cache[b][t][:576]) * cache[b][t][:512],  t < ctx_len[b]
 * q fp32 [batch][n_heads][576] = [q_nope . W_uk (512) | q_rope (64)]; latent_cache bf16 [batch][cache_stride_rows][576] =
 * [c_kv | k_rope] per token; ctx_len on the device (a captured graph serves growing contexts).  Products run in bf16 on
 * the tensor cores with fp32 accumulation; the context is cut into slices of split_tokens rows (0 = 1024) merged by a
 * second kernel.  scratch: vb_op_mla_decode_scratch_bytes, 16-byte aligned.  Default kernel: tcgen05.mma with S and O
 * in tensor memory, the latent tiles brought in by tiled TMA; vb_op_mla_set_path(0) selects the mma.sync kernel (process-wide;
 * 1 selects tcgen05 again).  A tcgen05 kernel whose bounded waits run out fills `out` with NaN. */
uint64_t vb_op_mla_decode_scratch_bytes(uint32_t batch, uint32_t n_heads, uint32_t max_ctx, uint32_t split_tokens);
int32_t vb_op_mla_decode(float* out, const float* q, const void* latent_cache, const uint32_t* ctx_len, uint32_t batch, uint32_t n_heads,
                         uint32_t max_ctx, uint64_t cache_stride_rows, float scale, uint32_t split_tokens, void* scratch, uint64_t scratch_bytes,
                         void* stream);
int32_t vb_op_mla_set_path(int32_t path);
/* LatentKVAppend (src/ir.rs:90, `kv_latent.append_latent`): cache[b][pos[b]][:] = bf16(rows[b][:576]). */
int32_t vb_op_mla_latent_append(void* latent_cache, const float* rows, const uint32_t* pos, uint32_t batch, uint64_t cache_stride_rows, void* stream);
/* The per-head products of the absorbed form: dst[b][h][:n_out] = src[b][h][:n_in] . W_h, W bf16 [n_heads][..][..] with
 * W_h stored [n_out][n_in] (w_rows_are_out = 1: ctx . W_uv_h^T) or [n_in][n_out] (0: q_nope . W_uk_h). */
int32_t vb_op_mla_head_product(float* dst, const float* src, const void* w_bf16, uint32_t n_heads, uint32_t n_in, uint32_t n_out, uint32_t batch,
                               int32_t w_rows_are_out, void* stream);
/* Load-time conversions (velox_cuda_quantize_q4_group64_kernel, src/codegen.rs:2337-2369, and the
 * symmetric formats).  `src` fp32 [rows][cols] on the device. */
int32_t vb_op_quantize(void* data, void* scales, const float* src, int32_t fmt, uint64_t rows, uint64_t cols, void* stream);
int32_t vb_op_dequantize(float* dst, const void* data, const void* scales, int32_t fmt, uint64_t rows, uint64_t cols, void* stream);
/* GGUF Q4_K (144-byte) / Q6_K (210-byte) super-blocks of 256 weights -> q4 group-64: 32 packed words and 4
 * half2(scale,min) per block (velox_cuda_unpack_q4_k_fused_kernel / _q6_k_, src/runners/velox_cuda_runner_k2.cu:211-347).
 * All pointers are device pointers. */
int32_t vb_op_unpack_gguf(void* words, void* scale_min, const void* src_blocks, int32_t ggml_type, uint64_t n_blocks, void* stream);
int32_t vb_op_fill_normal(float* dst, uint64_t n, uint64_t seed, uint64_t stream_id, float mean, float std, void* stream);
/* Bytes of scratch the ops above want for a given problem (upper bound). */
uint64_t vb_op_scratch_bytes(uint32_t n_q_heads, uint32_t head_dim, uint32_t max_seq, uint32_t vocab);

/* ---- device memory helpers for hosts without a CUDA binding (tests, FFI shims) ------------- */
int32_t vb_dev_alloc(void** out, uint64_t bytes);
int32_t vb_dev_free(void* p);
int32_t vb_dev_upload(void* dst_dev, const void* src_host, uint64_t bytes);
int32_t vb_dev_download(void* dst_host, const void* src_dev, uint64_t bytes);
int32_t vb_dev_sync(void);

#ifdef __cplusplus
}
#endif
#endif /* VELOX_B200_H */
