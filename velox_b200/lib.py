"""ctypes binding of libvelox_b200.so -- every symbol declared in include/velox_b200.h.

Loading never falls back to anything: a missing or stale shared object raises, and every call that
returns a negative status raises :class:`VeloxError` carrying ``vb_last_error()``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvelox_b200.so")

OK = 0
ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_OOM, ERR_STATE, ERR_TIMEOUT, ERR_COMM = -1, -2, -3, -4, -5, -6, -7
FMT_F32, FMT_F16, FMT_BF16, FMT_Q4G32, FMT_Q4G64REF, FMT_I8PC = range(6)
(ROLE_EMBED, ROLE_ATTN_NORM, ROLE_WQ, ROLE_WK, ROLE_WV, ROLE_WO, ROLE_MLP_NORM, ROLE_WGATE, ROLE_WUP,
 ROLE_WDOWN, ROLE_FINAL_NORM, ROLE_LM_HEAD, ROLE_BQ, ROLE_BK, ROLE_BV, ROLE_MLA_NORM, ROLE_MLA_WDKV,
 ROLE_MLA_WABSQ, ROLE_MLA_WABSO) = range(19)
LOC_HOST, LOC_DEVICE = 0, 1
ATTN_GQA, ATTN_MLA_REF = 0, 1
FLAG_LEAN_WEIGHTS = 1
GGML_F32, GGML_F16, GGML_Q4_K, GGML_Q6_K = 0, 1, 12, 14


class VeloxError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__("velox_b200 error %d: %s" % (code, msg))
        self.code = code


class ModelDesc(C.Structure):
    _fields_ = (
        [("struct_bytes", C.c_uint32)]
        + [(n, C.c_uint32) for n in ("vocab", "d_model", "n_layers", "n_q_heads", "n_kv_heads", "head_dim", "ffn_dim",
                                      "max_seq_len", "max_batch")]
        + [("rms_eps", C.c_float), ("rope_theta", C.c_float)]
        + [(n, C.c_uint32) for n in ("weight_fmt", "head_fmt", "embed_fmt", "qkv_bias", "tied_lm_head", "kv_block_tokens",
                                      "kv_blocks_total", "attn_kind", "mla_latent", "tp_rank", "tp_size", "flags")]
        + [("reserved", C.c_uint32 * 7)]
    )


class Weight(C.Structure):
    _fields_ = [("data", C.c_void_p), ("scales", C.c_void_p), ("fmt", C.c_int32)]


class SpecStats(C.Structure):
    _fields_ = [("steps", C.c_uint64), ("plain_steps", C.c_uint64), ("drafted", C.c_uint64), ("accepted", C.c_uint64),
                ("ema_final", C.c_float), ("ladder_final", C.c_uint32)]


# name -> (restype, argtypes); the list mirrors include/velox_b200.h one to one
_vp, _u32, _i32, _u64, _f32 = C.c_void_p, C.c_uint32, C.c_int32, C.c_uint64, C.c_float
SIGNATURES = {
    "vb_version": (_i32, []),
    "vb_last_error": (C.c_char_p, []),
    "vb_device_count": (_i32, [C.POINTER(_i32)]),
    "vb_create": (_i32, [C.POINTER(ModelDesc), _i32, C.POINTER(_vp)]),
    "vb_destroy": (_i32, [_vp]),
    "vb_load_tensor": (_i32, [_vp, _i32, _i32, _vp, _i32, _i32, _u64, _u64]),
    "vb_load_tensor_packed": (_i32, [_vp, _i32, _i32, _vp, _vp, _i32, _u64, _u64]),
    "vb_load_tensor_synthetic": (_i32, [_vp, _i32, _i32, _u64, _u64, _f32, _f32, _u64, _u64]),
    "vb_export_tensor": (_i32, [_vp, _i32, _i32, _vp, _u64, _vp, _u64]),
    "vb_weight_bytes": (_i32, [_vp, C.POINTER(_u64)]),
    "vb_gguf_tensor_bytes": (_u64, [_i32, _u64]),
    "vb_load_tensor_gguf": (_i32, [_vp, _i32, _i32, _vp, _i32, _u64, _u64]),
    "vb_seq_reserve": (_i32, [_vp, _i32, _u32]),
    "vb_seq_release": (_i32, [_vp, _i32]),
    "vb_seq_set": (_i32, [_vp, _i32, _u32, _u32, _u32]),
    "vb_prefill": (_i32, [_vp, _i32, _vp, _u32]),
    "vb_decode_step": (_i32, [_vp]),
    "vb_decode_graph_build": (_i32, [_vp]),
    "vb_decode_run": (_i32, [_vp, _u32, C.POINTER(_f32)]),
    "vb_generate_speculative": (_i32, [_vp, _i32, _vp, _u32, _u32, _u32, _f32, _vp, _vp]),
    "vb_sync": (_i32, [_vp]),
    "vb_read_tokens": (_i32, [_vp, _i32, _u32, _u32, _vp]),
    "vb_read_logits": (_i32, [_vp, _i32, _vp, _u64]),
    "vb_read_hidden": (_i32, [_vp, _i32, _vp, _u64]),
    "vb_read_state": (_i32, [_vp, _i32, C.POINTER(_u32), C.POINTER(_u32)]),
    "vb_read_state_ex": (_i32, [_vp, _i32, C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32)]),
    "vb_launch_count": (_i32, [_vp, C.POINTER(_u64)]),
    "vb_step_bytes": (_i32, [_vp, C.POINTER(_u64), C.POINTER(_u64)]),
    "vb_set_option": (_i32, [_vp, C.c_char_p, C.c_int64]),
    "vb_set_sampling": (_i32, [_vp, _f32, _f32, _u64, _i32]),
    "vb_trace_read": (_i32, [_vp, _vp, _u32, C.POINTER(_u32)]),
    "vb_tp_unique_id": (_i32, [_vp]),
    "vb_tp_init": (_i32, [_vp, _vp]),
    "vb_tp_p2p_export": (_i32, [_vp, _vp]),
    "vb_tp_p2p_open": (_i32, [_vp, _vp, _u32]),
    "vb_tp_p2p_close": (_i32, [_vp]),
    "vb_op_embed": (_i32, [_vp, _vp, _vp, _vp, _i32, _u32, _u32, _u32, _vp]),
    "vb_op_rmsnorm": (_i32, [_vp, _vp, _vp, _i32, _u32, _u32, _f32, _vp]),
    "vb_op_matmul": (_i32, [_vp, _vp, _vp, _vp, _i32, _u32, _u32, _u32, _vp]),
    "vb_op_matmul_rows_workspace_bytes": (_u64, [_u32, _u32, _u32]),
    "vb_op_matmul_rows": (_i32, [_vp, _vp, _vp, _vp, _i32, _u32, _u32, _u32, _vp, _u64, _vp]),
    "vb_op_rope": (_i32, [_vp, _u32, _u32, _u32, _f32, _vp]),
    "vb_op_gqa_attention": (_i32, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp, _u64, _vp]),
    "vb_op_sample_argmax": (_i32, [_vp, _vp, _u32, _vp, _u64, _vp]),
    "vb_op_sample_top_p": (_i32, [_vp, _vp, _u32, _f32, _f32, _f32, _i32, _vp, _u64, _vp]),
    "vb_op_sample_argmax_static": (_i32, [_vp, _vp, _u32, _vp]),
    "vb_op_fused_scratch_bytes": (_u64, [_u32] * 6),
    "vb_op_fused_norm_qkv_rope_attn": (_i32, [_vp] * 11 + [_u32, _u32, _vp] + [_u32] * 4 + [_f32, _f32, _vp, _u64, _vp]),
    "vb_op_fused_outproj_res_swiglu_res": (_i32, [_vp] * 8 + [_u32] * 3 + [_f32, _vp, _u64, _vp]),
    "vb_op_kv_write": (_i32, [_vp] * 4 + [_u32, _vp, _u32, _u32, _vp]),
    "vb_op_swiglu": (_i32, [_vp] * 5 + [_u32, _u32, _vp, _u64, _vp]),
    "vb_op_mla_absorbed": (_i32, [_vp] * 7 + [_u32] * 4 + [_f32, _vp, _u64, _vp]),
    "vb_op_mla_decode_scratch_bytes": (_u64, [_u32] * 4),
    "vb_op_mla_set_path": (_i32, [_i32]),
    "vb_op_mla_decode": (_i32, [_vp] * 4 + [_u32, _u32, _u32, _u64, _f32, _u32, _vp, _u64, _vp]),
    "vb_op_mla_latent_append": (_i32, [_vp, _vp, _vp, _u32, _u64, _vp]),
    "vb_op_mla_head_product": (_i32, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, _i32, _vp]),
    "vb_op_quantize": (_i32, [_vp, _vp, _vp, _i32, _u64, _u64, _vp]),
    "vb_op_dequantize": (_i32, [_vp, _vp, _vp, _i32, _u64, _u64, _vp]),
    "vb_op_unpack_gguf": (_i32, [_vp, _vp, _vp, _i32, _u64, _vp]),
    "vb_op_fill_normal": (_i32, [_vp, _u64, _u64, _u64, _f32, _f32, _vp]),
    "vb_op_scratch_bytes": (_u64, [_u32, _u32, _u32, _u32]),
    "vb_dev_alloc": (_i32, [C.POINTER(_vp), _u64]),
    "vb_dev_free": (_i32, [_vp]),
    "vb_dev_upload": (_i32, [_vp, _vp, _u64]),
    "vb_dev_download": (_i32, [_vp, _vp, _u64]),
    "vb_dev_sync": (_i32, []),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared object (raises if it has not been built: there is no other code path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                "%s is missing: build it with `python -m velox_b200.build` (nvcc, sm_100a)" % LIB_PATH)
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int) -> int:
    if rc < 0:
        raise VeloxError(rc, load().vb_last_error().decode("utf-8", "replace"))
    return rc
