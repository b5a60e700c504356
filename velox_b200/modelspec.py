"""Model shapes served by the library and the synthetic-weight recipe shared by tests and benchmarks.

The shapes are the .vlx models of the reference (examples/tinystories_smollm.vlx, llama3_8b.vlx,
qwen2_5_7b.vlx, qwen2_72b.vlx); real checkpoints are not available offline, so weights are drawn from a
counter-based generator that the CUDA library (vb_load_tensor_synthetic) and the CPU checker reproduce
bit for bit: tensor (role, layer) uses stream ``role * 4096 + layer`` of the run's seed.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

from . import lib as L


@dataclass(frozen=True)
class ModelSpec:
    name: str
    vocab: int
    d_model: int
    n_layers: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    ffn_dim: int
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    weight_fmt: int = L.FMT_F32
    head_fmt: int = L.FMT_F32
    embed_fmt: int = L.FMT_F32
    qkv_bias: bool = False
    tied_lm_head: bool = False

    @property
    def qdim(self) -> int:
        return self.n_q_heads * self.head_dim

    @property
    def kvdim(self) -> int:
        return self.n_kv_heads * self.head_dim

    def scaled(self, **kw) -> "ModelSpec":
        return replace(self, **kw)

    def tensors(self):
        """(role, layer, rows, cols, mean, std) for every tensor, in load order."""
        out = []
        d, f = self.d_model, self.ffn_dim
        for l in range(self.n_layers):
            out.append((L.ROLE_ATTN_NORM, l, 1, d, 1.0, 0.02))
            out.append((L.ROLE_WQ, l, self.qdim, d, 0.0, 0.02))
            out.append((L.ROLE_WK, l, self.kvdim, d, 0.0, 0.02))
            out.append((L.ROLE_WV, l, self.kvdim, d, 0.0, 0.02))
            if self.qkv_bias:
                out.append((L.ROLE_BQ, l, 1, self.qdim, 0.0, 0.02))
                out.append((L.ROLE_BK, l, 1, self.kvdim, 0.0, 0.02))
                out.append((L.ROLE_BV, l, 1, self.kvdim, 0.0, 0.02))
            out.append((L.ROLE_WO, l, d, self.qdim, 0.0, 0.02))
            out.append((L.ROLE_MLP_NORM, l, 1, d, 1.0, 0.02))
            out.append((L.ROLE_WGATE, l, f, d, 0.0, 0.02))
            out.append((L.ROLE_WUP, l, f, d, 0.0, 0.02))
            out.append((L.ROLE_WDOWN, l, d, f, 0.0, 0.02))
        out.append((L.ROLE_FINAL_NORM, 0, 1, d, 1.0, 0.02))
        out.append((L.ROLE_EMBED, 0, self.vocab, d, 0.0, 0.02))
        if not self.tied_lm_head:
            out.append((L.ROLE_LM_HEAD, 0, self.vocab, d, 0.0, 0.02))
        return out

    def storage_fmt(self, role: int) -> int:
        if role == L.ROLE_EMBED:
            return self.embed_fmt
        if role == L.ROLE_LM_HEAD:
            return self.head_fmt
        if role in (L.ROLE_ATTN_NORM, L.ROLE_MLP_NORM, L.ROLE_FINAL_NORM, L.ROLE_BQ, L.ROLE_BK, L.ROLE_BV):
            return L.FMT_F32 if self.weight_fmt == L.FMT_F32 else L.FMT_F16
        return self.weight_fmt


@dataclass(frozen=True)
class ShardPlan:
    """One tensor-parallel rank's part of a model: heads, FFN columns [ffn_off, ffn_off+ffn), vocabulary rows."""
    q_heads: int
    kv_heads: int
    head_off: int      # first query head
    kv_head_off: int   # first KV head
    ffn: int
    ffn_off: int
    vocab: int
    vocab_off: int


def shard_plan(spec: ModelSpec, tp_rank: int, tp_size: int) -> ShardPlan:
    """The split vb_create applies: heads and vocabulary evenly; FFN columns in whole 128-column blocks with
    the first (blocks % tp) ranks taking one block more, so that 32-column quantization groups never straddle
    two ranks and every shard dequantizes to the values the unsharded tensor holds there."""
    if not (0 <= tp_rank < tp_size):
        raise ValueError(f"tp_rank {tp_rank} outside [0, {tp_size})")
    if tp_size == 1:
        return ShardPlan(spec.n_q_heads, spec.n_kv_heads, 0, 0, spec.ffn_dim, 0, spec.vocab, 0)
    if spec.n_q_heads % tp_size or spec.n_kv_heads % tp_size:
        raise ValueError("heads not divisible by tp_size")
    if spec.ffn_dim % 128 or spec.ffn_dim // 128 < tp_size:
        raise ValueError("ffn_dim must be whole 128-column blocks, at least one per rank")
    if spec.vocab % (16 * tp_size):
        raise ValueError("vocab not divisible by 16 * tp_size")
    nb = spec.ffn_dim // 128
    per, extra = divmod(nb, tp_size)
    ffn = 128 * (per + (1 if tp_rank < extra else 0))
    ffn_off = 128 * (per * tp_rank + min(tp_rank, extra))
    hq, hkv, v = spec.n_q_heads // tp_size, spec.n_kv_heads // tp_size, spec.vocab // tp_size
    return ShardPlan(hq, hkv, hq * tp_rank, hkv * tp_rank, ffn, ffn_off, v, v * tp_rank)


def stream_of(role: int, layer: int) -> int:
    return role * 4096 + layer


PROMPT_STREAM = 1 << 20  # stream id of the synthetic prompt token ids

SMOLLM_135M = ModelSpec("smollm-135m-f32", 49152, 576, 30, 9, 3, 64, 1536, 1e-5, 10000.0, tied_lm_head=True)
LLAMA3_8B_INT4 = ModelSpec("llama3-8b-int4g32", 128256, 4096, 32, 32, 8, 128, 14336, 1e-5, 500000.0,
                           weight_fmt=L.FMT_Q4G32, head_fmt=L.FMT_Q4G32, embed_fmt=L.FMT_F16)
QWEN25_7B_INT8 = ModelSpec("qwen2.5-7b-int8pc", 152064, 3584, 28, 28, 4, 128, 18944, 1e-6, 1000000.0,
                           weight_fmt=L.FMT_I8PC, head_fmt=L.FMT_I8PC, embed_fmt=L.FMT_F16, qkv_bias=True)
QWEN2_72B_INT4 = ModelSpec("qwen2-72b-int4g32", 152064, 8192, 80, 64, 8, 128, 29568, 1e-6, 1000000.0,
                           weight_fmt=L.FMT_Q4G32, head_fmt=L.FMT_Q4G32, embed_fmt=L.FMT_F16, qkv_bias=True)

SPECS = {s.name: s for s in (SMOLLM_135M, LLAMA3_8B_INT4, QWEN25_7B_INT8, QWEN2_72B_INT4)}
