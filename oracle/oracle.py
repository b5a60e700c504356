"""ctypes binding of the CPU checker (TEST INFRASTRUCTURE ONLY).

Loads ``libvelox_oracle.so`` (the restatement of the reference's CPU runtime, velox_oracle.c) and,
when it was built, ``_ref/libvelox_ref_smollm.so`` (the reference's own emitted C99 model).  Only the
tests, the smoke check and the benchmark's CPU-baseline leg import this module; the product package
never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

FMT_F32, FMT_F16, FMT_BF16, FMT_Q4G32, FMT_Q4G64REF, FMT_I8PC = range(6)
(ROLE_EMBED, ROLE_ATTN_NORM, ROLE_WQ, ROLE_WK, ROLE_WV, ROLE_WO, ROLE_MLP_NORM, ROLE_WGATE, ROLE_WUP,
 ROLE_WDOWN, ROLE_FINAL_NORM, ROLE_LM_HEAD, ROLE_BQ, ROLE_BK, ROLE_BV, ROLE_MLA_NORM, ROLE_MLA_WDKV,
 ROLE_MLA_WABSQ, ROLE_MLA_WABSO) = range(19)


class VoConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("vocab", "d_model", "n_layers", "n_q_heads", "n_kv_heads",
                                           "head_dim", "ffn_dim", "max_seq_len")] + \
               [("rms_eps", C.c_float), ("rope_theta", C.c_float),
                ("qkv_bias", C.c_uint32), ("n_seqs", C.c_uint32), ("mla_latent", C.c_uint32)]


def _stale(target: str) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(os.path.join(_HERE, f)) > t for f in os.listdir(_HERE) if f.endswith((".c", ".h")))


class MlaBlock(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("d_model", "n_heads", "q_lora", "kv_lora", "nope_dim", "rope_dim", "v_dim")] + \
               [("eps", C.c_float), ("theta", C.c_float)] + \
               [(n, C.c_void_p) for n in ("w_norm", "w_dq", "w_uq", "w_qr", "w_dkv", "w_kr", "w_uk", "w_uv", "w_o")]


class SpecStats(C.Structure):
    _fields_ = [("steps", C.c_uint64), ("plain_steps", C.c_uint64), ("drafted", C.c_uint64), ("accepted", C.c_uint64),
                ("ema_final", C.c_float), ("ladder_final", C.c_uint32)]


def build(force: bool = False) -> None:
    """Compile the checker with the Makefile beside this file (gcc, a few seconds)."""
    if force or _stale(os.path.join(_HERE, "libvelox_oracle.so")):
        subprocess.check_call(["make", "-C", _HERE, "libvelox_oracle.so"], stdout=subprocess.DEVNULL)
    ref_so, harness = os.path.join(_HERE, "_ref", "libvelox_ref_smollm.so"), os.path.join(_HERE, "ref_smollm_harness.c")
    # (where the reference tree is absent the recipe keeps the prebuilt file, so a newer harness is harmless there)
    if force or not os.path.exists(ref_so) or os.path.getmtime(harness) > os.path.getmtime(ref_so):
        subprocess.call(["make", "-C", _HERE, "ref"], stdout=subprocess.DEVNULL)


_lib = None
_ref = None


def _p(a, t=C.c_void_p):
    return a.ctypes.data_as(t) if a is not None else None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(os.path.join(_HERE, "libvelox_oracle.so"))
        L.vo_engine_create.restype = C.c_void_p
        L.vo_engine_create.argtypes = [C.POINTER(VoConfig)]
        L.vo_engine_destroy.argtypes = [C.c_void_p]
        L.vo_engine_set_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        L.vo_engine_forward_step.restype = C.c_uint32
        L.vo_engine_forward_step.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32]
        L.vo_engine_logits.restype = C.POINTER(C.c_float)
        L.vo_engine_logits.argtypes = [C.c_void_p]
        L.vo_engine_hidden.restype = C.POINTER(C.c_float)
        L.vo_engine_hidden.argtypes = [C.c_void_p]
        L.vo_engine_generate_greedy.restype = C.c_size_t
        L.vo_engine_generate_greedy.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]
        L.vo_fill_normal.argtypes = [C.c_void_p, C.c_size_t, C.c_uint64, C.c_uint64, C.c_float, C.c_float]
        L.vo_fill_tokens.argtypes = [C.c_void_p, C.c_size_t, C.c_uint64, C.c_uint64, C.c_uint32]
        L.vo_hash64.restype = C.c_uint64
        L.vo_hash64.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64]
        L.vo_f32_to_f16.restype = C.c_uint16
        L.vo_f32_to_f16.argtypes = [C.c_float]
        L.vo_f16_to_f32.restype = C.c_float
        L.vo_f16_to_f32.argtypes = [C.c_uint16]
        for q in ("q4g32", "q4g64ref", "i8pc"):
            getattr(L, "vo_quantize_" + q).argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t]
            getattr(L, "vo_dequant_" + q).argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t]
        L.vo_rmsnorm_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_float]
        L.vo_matmul_transposed_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t]
        L.vo_matvec_fmt.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_size_t, C.c_size_t]
        L.vo_rope_rotate_half_f32.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_float]
        L.vo_gqa_attention_step_f32.argtypes = [C.c_void_p] * 5 + [C.c_size_t] * 4
        L.vo_swiglu_mlp_residual_f32.argtypes = [C.c_void_p] * 8 + [C.c_size_t] * 2
        L.vo_sample_argmax_f32.restype = C.c_uint32
        L.vo_sample_argmax_f32.argtypes = [C.c_void_p, C.c_size_t]
        L.vo_mla_absorbed_step_f32.argtypes = [C.c_void_p] * 7 + [C.c_size_t] * 4 + [C.c_float]
        L.vo_num_threads.restype = C.c_int
        for f in ("vo_sample_top_p_f32", "vo_sample_top_p_c99"):
            getattr(L, f).restype = C.c_uint32
            getattr(L, f).argtypes = [C.c_void_p, C.c_size_t, C.c_float, C.c_float, C.c_float, C.POINTER(C.c_float)]
        L.vo_sample_coin.restype = C.c_float
        L.vo_sample_coin.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32]
        L.vo_prompt_lookup_draft.restype = C.c_int
        L.vo_prompt_lookup_draft.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_int]
        L.vo_engine_generate_speculative.restype = C.c_size_t
        L.vo_engine_generate_speculative.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_int, C.c_float,
                                                     C.c_void_p, C.POINTER(SpecStats)]
        L.vo_mla_step_absorbed.argtypes = [C.POINTER(MlaBlock), C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p]
        L.vo_mla_step_explicit.argtypes = [C.POINTER(MlaBlock), C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        L.vo_mla_core.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_float]
        L.vo_unpack_q4_k.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        L.vo_unpack_q6_k.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        L.vo_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def ref_lib():
    """The reference's own emitted C99 model (None when it was not built)."""
    global _ref
    if _ref is None:
        build()
        path = os.path.join(_HERE, "_ref", "libvelox_ref_smollm.so")
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        R.refsm_create.restype = C.c_void_p
        R.refsm_destroy.argtypes = [C.c_void_p]
        R.refsm_weight_ptr.restype = C.POINTER(C.c_float)
        R.refsm_weight_ptr.argtypes = [C.c_void_p, C.c_int]
        R.refsm_prefill.restype = C.c_uint32
        R.refsm_prefill.argtypes = [C.c_void_p, C.c_uint32, C.c_uint64]
        R.refsm_decode.restype = C.c_uint32
        R.refsm_decode.argtypes = [C.c_void_p, C.c_uint32, C.c_uint64]
        R.refsm_logits.restype = C.POINTER(C.c_float)
        R.refsm_logits.argtypes = [C.c_void_p]
        R.refsm_reset_kv.argtypes = [C.c_void_p]
        R.refsm_generate.restype = C.c_uint64
        R.refsm_generate.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p]
        R.refsm_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_float]
        R.refsm_matmul_vec.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64]
        R.refsm_rope.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float]
        R.refsm_gqa.argtypes = [C.c_void_p] * 5 + [C.c_uint64] * 4
        R.refsm_argmax.restype = C.c_uint32
        R.refsm_argmax.argtypes = [C.c_void_p, C.c_uint64]
        if hasattr(R, "refsm_sample_top_p"):
            R.refsm_sample_top_p.restype = C.c_uint32
            R.refsm_sample_top_p.argtypes = [C.c_void_p, C.c_uint64, C.c_float, C.c_float, C.c_float]
        R.refsm_mla.argtypes = [C.c_void_p] * 7 + [C.c_uint64, C.c_uint64, C.c_float]
        R.refsm_dim.restype = C.c_uint64
        R.refsm_dim.argtypes = [C.c_int]
        R.refsm_num_threads.restype = C.c_int
        _ref = R
    return _ref


# ---------------------------------------------------------------------------------------------
# numpy-facing helpers
# ---------------------------------------------------------------------------------------------
def fill_normal(n: int, seed: int, stream: int, std: float = 0.02, mean: float = 0.0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().vo_fill_normal(_p(out), n, seed, stream, mean, std)
    return out


def fill_tokens(n: int, seed: int, stream: int, vocab: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint32)
    lib().vo_fill_tokens(_p(out), n, seed, stream, vocab)
    return out


def quantize(w: np.ndarray, fmt: int):
    """fp32 [rows, cols] -> (data, scales) in storage format `fmt` (scales None for plain formats)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    L = lib()
    if fmt == FMT_F32:
        return w, None
    if fmt == FMT_F16:
        return w.astype(np.float16).view(np.uint16), None
    if fmt == FMT_BF16:
        u = w.view(np.uint32).astype(np.uint64)
        lsb = (u >> 16) & 1
        return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16), None
    if fmt == FMT_Q4G32:
        packed = np.empty((rows, cols // 8), dtype=np.uint32)
        scales = np.empty((rows, cols // 32), dtype=np.uint16)
        L.vo_quantize_q4g32(_p(packed), _p(scales), _p(w), rows, cols)
        return packed, scales
    if fmt == FMT_Q4G64REF:
        packed = np.empty((rows, cols // 8), dtype=np.uint32)
        scales = np.empty((rows, cols // 64, 2), dtype=np.uint16)
        L.vo_quantize_q4g64ref(_p(packed), _p(scales), _p(w), rows, cols)
        return packed, scales
    if fmt == FMT_I8PC:
        q = np.empty((rows, cols), dtype=np.int8)
        scales = np.empty(rows, dtype=np.uint16)
        L.vo_quantize_i8pc(_p(q), _p(scales), _p(w), rows, cols)
        return q, scales
    raise ValueError(fmt)


def dequantize(data: np.ndarray, scales, fmt: int, rows: int, cols: int) -> np.ndarray:
    L = lib()
    out = np.empty((rows, cols), dtype=np.float32)
    if fmt == FMT_F32:
        return np.asarray(data, dtype=np.float32).reshape(rows, cols)
    if fmt == FMT_F16:
        return data.view(np.float16).astype(np.float32).reshape(rows, cols)
    if fmt == FMT_BF16:
        return (data.astype(np.uint32) << 16).view(np.float32).reshape(rows, cols)
    fn = {FMT_Q4G32: L.vo_dequant_q4g32, FMT_Q4G64REF: L.vo_dequant_q4g64ref, FMT_I8PC: L.vo_dequant_i8pc}[fmt]
    fn(_p(out), _p(data), _p(scales), rows, cols)
    return out


def matvec(x: np.ndarray, data: np.ndarray, scales, fmt: int, in_dim: int, out_dim: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(out_dim, dtype=np.float32)
    lib().vo_matvec_fmt(_p(out), _p(x), _p(data), _p(scales), fmt, in_dim, out_dim)
    return out


class Engine:
    """Mirror of VeloxStaticExecutionEngine (src/runtime.rs:1229-1502) over the C restatement."""

    def __init__(self, **cfg):
        self.cfg = VoConfig(**cfg)
        self._keep = []
        self.h = lib().vo_engine_create(C.byref(self.cfg))
        if not self.h:
            raise MemoryError("vo_engine_create")

    def set_tensor(self, role: int, layer: int, data: np.ndarray, scales=None, fmt: int = FMT_F32):
        data = np.ascontiguousarray(data)
        scales = np.ascontiguousarray(scales) if scales is not None else None
        self._keep += [data, scales]
        rc = lib().vo_engine_set_tensor(self.h, role, layer, _p(data), _p(scales), fmt)
        if rc != 0:
            raise ValueError((role, layer))

    def forward_step(self, token: int, pos: int, seq: int = 0) -> int:
        return int(lib().vo_engine_forward_step(self.h, seq, int(token), int(pos)))

    @property
    def logits(self) -> np.ndarray:
        return np.ctypeslib.as_array(lib().vo_engine_logits(self.h), shape=(self.cfg.vocab,)).copy()

    @property
    def hidden(self) -> np.ndarray:
        return np.ctypeslib.as_array(lib().vo_engine_hidden(self.h), shape=(self.cfg.d_model,)).copy()

    def generate_greedy(self, prompt, n_new: int, seq: int = 0) -> np.ndarray:
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.zeros(n_new, dtype=np.uint32)
        lib().vo_engine_generate_greedy(self.h, seq, _p(prompt), len(prompt), n_new, _p(out))
        return out

    def generate_speculative(self, prompt, n_new: int, max_draft_len: int = 3, ema_floor: float = 0.20, seq: int = 0):
        """(tokens, stats) of the prompt-lookup speculative loop (velox_cuda_runner_k2.cu:2166-2310)."""
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.zeros(n_new, dtype=np.uint32)
        st = SpecStats()
        lib().vo_engine_generate_speculative(self.h, seq, _p(prompt), len(prompt), n_new, max_draft_len, ema_floor, _p(out), C.byref(st))
        return out, st

    def close(self):
        if self.h:
            lib().vo_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def sample_top_p(logits: np.ndarray, temperature: float, top_p: float, coin: float, mode: int = 0):
    """(token, margin): mode 0 = src/runtime.rs:1092-1152, mode 1 = the emitted C99 twin."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    m = C.c_float()
    fn = lib().vo_sample_top_p_f32 if mode == 0 else lib().vo_sample_top_p_c99
    tok = fn(_p(logits), logits.size, temperature, top_p, coin, C.byref(m))
    return int(tok), float(m.value)


def sample_coin(seed: int, slot: int, pos: int) -> float:
    return float(lib().vo_sample_coin(seed, slot, pos))


def prompt_lookup_draft(history, max_draft: int) -> np.ndarray:
    history = np.ascontiguousarray(history, dtype=np.uint32)
    out = np.zeros(8, dtype=np.uint32)
    n = lib().vo_prompt_lookup_draft(_p(history), len(history), _p(out), max_draft)
    return out[:n]


def unpack_gguf(blocks: np.ndarray, ggml_type: int):
    """Q4_K (type 12) / Q6_K (type 14) super-blocks -> (words [n*32] u32, scale_min [n*4][2] u16) in q4 group-64."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    bs = {12: 144, 14: 210}[ggml_type]
    n = blocks.size // bs
    words = np.empty(n * 32, dtype=np.uint32)
    sm = np.empty((n * 4, 2), dtype=np.uint16)
    (lib().vo_unpack_q4_k if ggml_type == 12 else lib().vo_unpack_q6_k)(_p(words), _p(sm), _p(blocks), n)
    return words, sm


def bf16_round(a: np.ndarray) -> np.ndarray:
    """fp32 values rounded to bfloat16 (nearest even) and widened again."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32).reshape(np.shape(a))


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16).reshape(np.shape(a))


class MlaBlockWeights:
    """One multi-head latent attention block (examples/deepseek_v3_mla.vlx:18-45) with weights rounded to bf16."""

    NAMES = ("w_norm", "w_dq", "w_uq", "w_qr", "w_dkv", "w_kr", "w_uk", "w_uv", "w_o")

    def __init__(self, rng, d_model, n_heads, q_lora, kv_lora=512, nope_dim=128, rope_dim=64, v_dim=128, eps=1e-6, theta=10000.0, std=0.02):
        self.dims = dict(d_model=d_model, n_heads=n_heads, q_lora=q_lora, kv_lora=kv_lora, nope_dim=nope_dim, rope_dim=rope_dim, v_dim=v_dim)
        H = n_heads
        shapes = {"w_norm": (d_model,), "w_dq": (q_lora, d_model), "w_uq": (H * nope_dim, q_lora), "w_qr": (H * rope_dim, q_lora),
                  "w_dkv": (kv_lora, d_model), "w_kr": (rope_dim, d_model), "w_uk": (H * nope_dim, kv_lora), "w_uv": (H * v_dim, kv_lora),
                  "w_o": (d_model, H * v_dim)}
        self.w = {}
        for n in self.NAMES:
            base = 1.0 if n == "w_norm" else 0.0
            self.w[n] = bf16_round((base + std * rng.standard_normal(shapes[n])).astype(np.float32))
        self.c = MlaBlock(eps=eps, theta=theta, **self.dims)
        for n in self.NAMES:
            setattr(self.c, n, self.w[n].ctypes.data)

    def step(self, x, cache, pos, absorbed=True, cache_bf16=False):
        x = np.ascontiguousarray(x, dtype=np.float32)
        dst = np.empty_like(x)
        H, W = self.dims["n_heads"], self.dims["kv_lora"] + self.dims["rope_dim"]
        if absorbed:
            q_cat, ctx = np.empty((H, W), np.float32), np.empty((H, self.dims["kv_lora"]), np.float32)
            lib().vo_mla_step_absorbed(C.byref(self.c), _p(dst), _p(x), _p(cache), pos, int(cache_bf16), _p(q_cat), _p(ctx))
            return dst, q_cat, ctx
        lib().vo_mla_step_explicit(C.byref(self.c), _p(dst), _p(x), _p(cache), pos, int(cache_bf16))
        return dst


def mla_core(q_cat: np.ndarray, cache_rows: np.ndarray, dc: int, scale: float) -> np.ndarray:
    q_cat = np.ascontiguousarray(q_cat, dtype=np.float32)
    cache_rows = np.ascontiguousarray(cache_rows, dtype=np.float32)
    H, W = q_cat.shape
    out = np.empty((H, dc), np.float32)
    lib().vo_mla_core(_p(out), _p(q_cat), _p(cache_rows), H, dc, W - dc, cache_rows.shape[0], scale)
    return out
