"""Host-side mirror of the reference's engine interface over the C ABI.

``Engine`` offers what ``VeloxStaticExecutionEngine`` does (src/runtime.rs:1229-1502): load weights,
``forward_step(token, pos)``, ``generate_greedy(prompt, n_new)``, ``logits`` -- but every step runs as
CUDA kernels of libvelox_b200 (paged fp16 KV, device-resident decode state, CUDA-graph replay).  There
is no CPU path: without the shared object or a GPU these calls raise.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as L
from .modelspec import ModelSpec, stream_of


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class DeviceBuffer:
    """A device allocation owned by Python (vb_dev_alloc), with numpy upload/download."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        L.check(L.load().vb_dev_alloc(C.byref(p), self.nbytes))
        self.ptr = p

    @classmethod
    def from_numpy(cls, a: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        b = cls(a.nbytes)
        if a.nbytes:
            L.check(L.load().vb_dev_upload(b.ptr, _ptr(a), a.nbytes))
        return b

    def to_numpy(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= self.nbytes
        if out.nbytes:
            L.check(L.load().vb_dev_download(_ptr(out), self.ptr, out.nbytes))
        return out

    def free(self):
        if self.ptr:
            L.load().vb_dev_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Engine:
    def __init__(self, spec: ModelSpec, max_seq_len: int, max_batch: int = 1, device: int = 0,
                 kv_blocks_total: int = 0, tp_rank: int = 0, tp_size: int = 1, lean_weights: bool = False):
        """With tp_size > 1 this context is one rank of a tensor-parallel group: it keeps 1/tp of the heads,
        FFN columns and vocabulary rows (see modelspec.shard_plan) and needs ``tp_init`` before the first step."""
        self.spec = spec
        self.tp_rank, self.tp_size = int(tp_rank), int(tp_size)
        self.max_seq_len = int(max_seq_len)
        self.max_batch = int(max_batch)
        d = L.ModelDesc()
        d.struct_bytes = C.sizeof(L.ModelDesc)
        for k in ("vocab", "d_model", "n_layers", "n_q_heads", "n_kv_heads", "head_dim", "ffn_dim", "weight_fmt",
                  "head_fmt", "embed_fmt"):
            setattr(d, k, getattr(spec, k))
        d.max_seq_len, d.max_batch = self.max_seq_len, self.max_batch
        d.rms_eps, d.rope_theta = spec.rms_eps, spec.rope_theta
        d.qkv_bias, d.tied_lm_head = int(spec.qkv_bias), int(spec.tied_lm_head)
        d.kv_block_tokens, d.kv_blocks_total = 16, int(kv_blocks_total)
        d.attn_kind, d.tp_rank, d.tp_size = L.ATTN_GQA, self.tp_rank, self.tp_size
        d.flags = L.FLAG_LEAN_WEIGHTS if lean_weights else 0
        self._lib = L.load()
        h = C.c_void_p()
        L.check(self._lib.vb_create(C.byref(d), device, C.byref(h)))
        self.h = h

    # ---- tensor parallel ----------------------------------------------------------------------
    @staticmethod
    def tp_unique_id() -> bytes:
        """128-byte communicator id; rank 0 makes it and the host passes it to the other ranks."""
        buf = C.create_string_buffer(128)
        L.check(L.load().vb_tp_unique_id(buf))
        return buf.raw

    def tp_init(self, unique_id: bytes):
        assert len(unique_id) == 128
        L.check(self._lib.vb_tp_init(self.h, C.create_string_buffer(unique_id, 128)))

    def tp_p2p_export(self) -> bytes:
        """64-byte handle of this rank's NVLink receive region (to be gathered from all ranks, in rank order)."""
        buf = C.create_string_buffer(64)
        L.check(self._lib.vb_tp_p2p_export(self.h, buf))
        return buf.raw

    def tp_p2p_open(self, handles):
        blob = b"".join(handles)
        assert len(blob) == 64 * self.tp_size
        L.check(self._lib.vb_tp_p2p_open(self.h, C.create_string_buffer(blob, len(blob)), self.tp_size))

    def tp_p2p_close(self):
        L.check(self._lib.vb_tp_p2p_close(self.h))

    # ---- weights ----------------------------------------------------------------------------
    def load_tensor(self, role: int, layer: int, w: np.ndarray):
        """fp32/fp16 [rows][cols] host array; converted to the storage format on the GPU."""
        w = np.ascontiguousarray(w)
        fmt = {np.dtype(np.float32): L.FMT_F32, np.dtype(np.float16): L.FMT_F16}[w.dtype]
        rows, cols = (1, w.size) if w.ndim == 1 else w.shape
        L.check(self._lib.vb_load_tensor(self.h, role, layer, _ptr(w), fmt, L.LOC_HOST, rows, cols))

    def load_tensor_packed(self, role: int, layer: int, data: np.ndarray, scales, rows: int, cols: int):
        data = np.ascontiguousarray(data)
        scales = np.ascontiguousarray(scales) if scales is not None else None
        L.check(self._lib.vb_load_tensor_packed(self.h, role, layer, _ptr(data), _ptr(scales) if scales is not None else None,
                                                L.LOC_HOST, rows, cols))

    def load_synthetic(self, seed: int):
        for role, layer, rows, cols, mean, std in self.spec.tensors():
            L.check(self._lib.vb_load_tensor_synthetic(self.h, role, layer, seed, stream_of(role, layer), mean, std, rows, cols))

    def export_tensor(self, role: int, layer: int, rows: int, cols: int):
        """(data, scales) of a stored tensor in canonical layout."""
        fmt = self.spec.storage_fmt(role)
        shape, dt, sshape = {
            L.FMT_F32: ((rows, cols), np.float32, None), L.FMT_F16: ((rows, cols), np.uint16, None),
            L.FMT_BF16: ((rows, cols), np.uint16, None), L.FMT_Q4G32: ((rows, cols // 8), np.uint32, (rows, cols // 32)),
            L.FMT_Q4G64REF: ((rows, cols // 8), np.uint32, (rows, cols // 64, 2)), L.FMT_I8PC: ((rows, cols), np.int8, (rows,)),
        }[fmt]
        data = np.empty(shape, dtype=dt)
        scales = np.empty(sshape, dtype=np.uint16) if sshape is not None else None
        L.check(self._lib.vb_export_tensor(self.h, role, layer, _ptr(data), data.nbytes,
                                           _ptr(scales) if scales is not None else None,
                                           scales.nbytes if scales is not None else 0))
        return data, scales

    # ---- sequences ----------------------------------------------------------------------------
    def reserve(self, slot: int, n_tokens: int):
        L.check(self._lib.vb_seq_reserve(self.h, slot, n_tokens))

    def release(self, slot: int):
        L.check(self._lib.vb_seq_release(self.h, slot))

    def set_state(self, slot: int, token: int, pos: int, active: bool = True):
        L.check(self._lib.vb_seq_set(self.h, slot, int(token), int(pos), int(active)))

    def state(self, slot: int = 0):
        t, p = C.c_uint32(), C.c_uint32()
        L.check(self._lib.vb_read_state(self.h, slot, C.byref(t), C.byref(p)))
        return t.value, p.value

    def state_ex(self, slot: int = 0):
        """(token, pos, active, limit) of a slot; limit = tokens of its KV reservation."""
        t, p, a, l = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint32()
        L.check(self._lib.vb_read_state_ex(self.h, slot, C.byref(t), C.byref(p), C.byref(a), C.byref(l)))
        return t.value, p.value, a.value, l.value

    # ---- the reference's engine calls --------------------------------------------------------------
    def forward_step(self, token: int, pos: int, slot: int = 0) -> int:
        """src/runtime.rs:1328: one token at `pos`; returns the greedy next token."""
        self.set_state(slot, token, pos, True)
        L.check(self._lib.vb_decode_run(self.h, 1, None))  # replays the captured graph when there is one
        return int(self.read_tokens(slot, pos, 1)[0])

    def prefill(self, prompt, slot: int = 0):
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        L.check(self._lib.vb_prefill(self.h, slot, _ptr(prompt), len(prompt)))

    def prefill_lockstep(self, prompts):
        """Prefills several slots together, one decode step per prompt position (prompts right-aligned so that all
        end at the same step): slot i gets prompts[i].  The reference has no batched prefill; this is its
        token-by-token prefill run for all sequences at once."""
        prompts = [np.ascontiguousarray(p, dtype=np.uint32) for p in prompts]
        n = max(len(p) for p in prompts)
        for step in range(n):
            for slot, pr in enumerate(prompts):
                k = step - (n - len(pr))
                if k >= 0:
                    self.set_state(slot, int(pr[k]), k, True)
            L.check(self._lib.vb_decode_step(self.h))
        self.sync()

    def decode(self, n_steps: int, timed: bool = False):
        ms = C.c_float(0.0)
        L.check(self._lib.vb_decode_run(self.h, n_steps, C.byref(ms) if timed else None))
        return ms.value if timed else None

    def build_graph(self):
        L.check(self._lib.vb_decode_graph_build(self.h))

    def generate_greedy(self, prompt, n_new: int, slot: int = 0, use_graph: bool = True) -> np.ndarray:
        """src/runtime.rs:1456-1490: prefill, then n_new greedy tokens (the first comes from the prefill)."""
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        n = len(prompt)
        self.reserve(slot, n + n_new)
        self.prefill(prompt, slot)
        if n_new == 0:
            return np.zeros(0, dtype=np.uint32)
        if n_new > 1:
            if use_graph:
                self.build_graph()
            self.decode(n_new - 1)
        return self.read_tokens(slot, n - 1, n_new)

    def generate_speculative(self, prompt, n_new: int, max_draft_len: int = 3, ema_floor: float = 0.20, slot: int = 0):
        """Prompt-lookup speculative decoding (velox_cuda_runner_k2.cu:2127-2311): (tokens, stats)."""
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        self.reserve(slot, len(prompt) + n_new + max_draft_len)
        out = np.zeros(n_new, dtype=np.uint32)
        st = L.SpecStats()
        L.check(self._lib.vb_generate_speculative(self.h, slot, _ptr(prompt), len(prompt), n_new, max_draft_len, ema_floor,
                                                  _ptr(out), C.byref(st)))
        return out, st

    def read_tokens(self, slot: int, first_pos: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.uint32)
        L.check(self._lib.vb_read_tokens(self.h, slot, first_pos, n, _ptr(out)))
        return out

    def logits(self, slot: int = 0) -> np.ndarray:
        """Logits of this context's vocabulary rows (all of them unless tensor parallel)."""
        out = np.empty(self.spec.vocab // self.tp_size, dtype=np.float32)
        L.check(self._lib.vb_read_logits(self.h, slot, _ptr(out), out.size))
        return out

    def hidden(self, slot: int = 0) -> np.ndarray:
        out = np.empty(self.spec.d_model, dtype=np.float32)
        L.check(self._lib.vb_read_hidden(self.h, slot, _ptr(out), out.size))
        return out

    def sync(self):
        L.check(self._lib.vb_sync(self.h))

    def launch_count(self) -> int:
        v = C.c_uint64()
        L.check(self._lib.vb_launch_count(self.h, C.byref(v)))
        return v.value

    def step_bytes(self):
        w, k = C.c_uint64(), C.c_uint64()
        L.check(self._lib.vb_step_bytes(self.h, C.byref(w), C.byref(k)))
        return w.value, k.value

    def set_sampling(self, temperature: float, top_p: float, seed: int = 0, mode: int = 0):
        """Sampler of the following decode steps (0 / 0 = greedy); coins come from (seed, slot, position)."""
        L.check(self._lib.vb_set_sampling(self.h, float(temperature), float(top_p), int(seed), int(mode)))

    def set_option(self, name: str, value: int):
        L.check(self._lib.vb_set_option(self.h, name.encode(), int(value)))

    def close(self):
        if getattr(self, "h", None):
            self._lib.vb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
