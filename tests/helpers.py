"""Shared test plumbing: the same synthetic model on the CPU checker and on the CUDA engine."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O
from velox_b200 import lib as L
from velox_b200.modelspec import ModelSpec, stream_of, PROMPT_STREAM

VEC_ROLES = (L.ROLE_ATTN_NORM, L.ROLE_MLP_NORM, L.ROLE_FINAL_NORM, L.ROLE_BQ, L.ROLE_BK, L.ROLE_BV)


def host_tensor(spec: ModelSpec, seed: int, role: int, layer: int, rows: int, cols: int, mean: float, std: float):
    """fp32 source values of one tensor (bit-identical to vb_load_tensor_synthetic)."""
    return O.fill_normal(rows * cols, seed, stream_of(role, layer), std, mean).reshape(rows, cols)


def build_oracle(spec: ModelSpec, seed: int, max_seq_len: int, n_seqs: int = 1):
    """CPU checker engine holding the model in the same storage formats as the CUDA engine."""
    eng = O.Engine(vocab=spec.vocab, d_model=spec.d_model, n_layers=spec.n_layers, n_q_heads=spec.n_q_heads,
                   n_kv_heads=spec.n_kv_heads, head_dim=spec.head_dim, ffn_dim=spec.ffn_dim, max_seq_len=max_seq_len,
                   rms_eps=spec.rms_eps, rope_theta=spec.rope_theta, qkv_bias=int(spec.qkv_bias), n_seqs=n_seqs,
                   mla_latent=0)
    stored = {}
    for role, layer, rows, cols, mean, std in spec.tensors():
        w = host_tensor(spec, seed, role, layer, rows, cols, mean, std)
        fmt = spec.storage_fmt(role)
        data, scales = O.quantize(w, fmt)
        eng.set_tensor(role, layer, data, scales, fmt)
        stored[(role, layer)] = (data, scales, fmt, rows, cols)
    return eng, stored


def build_engine(spec: ModelSpec, seed: int, max_seq_len: int, max_batch: int = 1):
    from velox_b200.engine import Engine
    e = Engine(spec, max_seq_len=max_seq_len, max_batch=max_batch)
    e.load_synthetic(seed)
    return e


def prompt_tokens(spec: ModelSpec, seed: int, n: int, stream: int = PROMPT_STREAM) -> np.ndarray:
    return O.fill_tokens(n, seed, stream, spec.vocab)


TINY = ModelSpec("tiny-f32", vocab=512, d_model=128, n_layers=2, n_q_heads=4, n_kv_heads=2, head_dim=32, ffn_dim=256)
