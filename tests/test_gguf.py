"""GGUF Q4_K / Q6_K loading: the checker's unpack against the published block formulas (CPU), the CUDA unpack kernels
bit for bit against the checker and the runner reading a GGUF file written here (GPU).
Reference: src/runners/velox_cuda_runner_k2.cu:70-178 (file directory), :200-347 (unpack kernels)."""
import os
import re
import struct
import subprocess

import numpy as np
import pytest

import helpers as H
from oracle import oracle as O
from velox_b200 import lib as L
from velox_b200.modelspec import ModelSpec

Q4_K, Q6_K = 12, 14


def random_blocks(rng, ggml_type, n):
    """n random super-blocks with small positive fp16 super-scales (any bit pattern elsewhere)."""
    if ggml_type == Q4_K:
        b = rng.integers(0, 256, size=(n, 144), dtype=np.uint8)
        b[:, 0:2] = rng.uniform(1e-4, 4e-4, n).astype(np.float16).view(np.uint8).reshape(n, 2)
        b[:, 2:4] = rng.uniform(0, 4e-3, n).astype(np.float16).view(np.uint8).reshape(n, 2)
    else:
        b = rng.integers(0, 256, size=(n, 210), dtype=np.uint8)
        b[:, 208:210] = rng.uniform(2e-5, 8e-5, n).astype(np.float16).view(np.uint8).reshape(n, 2)
    return b


def dequant_q4_k(blocks):
    """Published Q4_K layout: y = d * sc_j * q - dmin * m_j for the 8 sub-blocks of 32 (fp64 here)."""
    out = np.zeros((blocks.shape[0], 256))
    for bi, b in enumerate(blocks):
        d, dmin = float(b[0:2].view(np.float16)[0]), float(b[2:4].view(np.float16)[0])
        sc, qs = b[4:16], b[16:144]
        for j in range(8):
            if j < 4:
                s, m = sc[j] & 63, sc[j + 4] & 63
            else:
                s, m = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4), (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)
            q = qs[(j // 2) * 32:(j // 2) * 32 + 32]
            q = (q & 0xF) if j % 2 == 0 else (q >> 4)
            out[bi, j * 32:(j + 1) * 32] = d * float(s) * q.astype(np.float64) - dmin * float(m)
    return out


def dequant_q6_k(blocks):
    out = np.zeros((blocks.shape[0], 256))
    for bi, b in enumerate(blocks):
        ql, qh, sc = b[0:128], b[128:192], b[192:208].view(np.int8)
        d = float(b[208:210].view(np.float16)[0])
        for n in range(2):
            for l in range(32):
                is_ = l // 16
                h = int(qh[n * 32 + l])
                q1 = int((ql[n * 64 + l] & 0xF) | (((h >> 0) & 3) << 4)) - 32
                q2 = int((ql[n * 64 + l + 32] & 0xF) | (((h >> 2) & 3) << 4)) - 32
                q3 = int((ql[n * 64 + l] >> 4) | (((h >> 4) & 3) << 4)) - 32
                q4 = int((ql[n * 64 + l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32
                base = n * 128
                out[bi, base + l] = d * float(sc[n * 8 + is_]) * q1
                out[bi, base + l + 32] = d * float(sc[n * 8 + is_ + 2]) * q2
                out[bi, base + l + 64] = d * float(sc[n * 8 + is_ + 4]) * q3
                out[bi, base + l + 96] = d * float(sc[n * 8 + is_ + 6]) * q4
    return out


def test_unpack_hand_built_q4_k_block():
    """d = 1, dmin = 0, every sub-block scale 1: the weights are the nibbles themselves; a group of 64 spanning 0..15
    re-quantizes to scale 1, minimum 0 and the same integers."""
    b = np.zeros((1, 144), dtype=np.uint8)
    b[0, 0:2] = np.array([1.0], dtype=np.float16).view(np.uint8)
    b[0, 4:8] = 1      # scales of sub-blocks 0..3
    b[0, 12:16] = 1    # low nibbles: scales of sub-blocks 4..7
    lo = np.arange(32) % 16
    hi = (np.arange(32) * 7) % 16
    b[0, 16:144] = np.tile((lo | (hi << 4)).astype(np.uint8), 4)
    words, sm = O.unpack_gguf(b, Q4_K)
    assert sm.shape == (4, 2) and np.all(sm[:, 0] == np.array([1.0], dtype=np.float16).view(np.uint16)[0]) and np.all(sm[:, 1] == 0)
    vals = O.dequantize(words.reshape(1, 32), sm.reshape(1, 4, 2), O.FMT_Q4G64REF, 1, 256)[0]
    assert np.array_equal(vals[:32], lo) and np.array_equal(vals[32:64], hi)


@pytest.mark.parametrize("ggml_type", [Q4_K, Q6_K])
def test_checker_unpack_tracks_the_published_dequantization(ggml_type):
    rng = np.random.default_rng(ggml_type)
    blocks = random_blocks(rng, ggml_type, 64)
    words, sm = O.unpack_gguf(blocks, ggml_type)
    got = O.dequantize(words.reshape(64, 32), sm.reshape(64, 4, 2), O.FMT_Q4G64REF, 64, 256)
    want = dequant_q4_k(blocks) if ggml_type == Q4_K else dequant_q6_k(blocks)
    # re-quantized to 16 levels per group of 64: within half a step (+ fp16 rounding of scale and minimum)
    for g in range(4):
        w = want[:, g * 64:(g + 1) * 64]
        step = (w.max(axis=1) - w.min(axis=1)) / 15.0
        err = np.abs(got[:, g * 64:(g + 1) * 64] - w).max(axis=1)
        assert np.all(err <= 0.5 * step * 1.02 + 16 * np.abs(w).max(axis=1) * 2.0 ** -11 + 1e-9)


def write_gguf(path, tensors):
    """tensors: list of (name, ggml_type, rows, cols, raw bytes).  GGUF v3, 32-byte alignment, a few metadata keys of
    different value types in front (the reader skips them)."""
    def s(x):
        x = x.encode()
        return struct.pack("<Q", len(x)) + x
    kv = s("general.architecture") + struct.pack("<I", 8) + s("llama")
    kv += s("llama.block_count") + struct.pack("<II", 4, 2)
    kv += s("tokenizer.ggml.tokens") + struct.pack("<IIQ", 9, 8, 3) + s("a") + s("bc") + s("def")
    kv += s("general.file_type") + struct.pack("<If", 6, 1.5)
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), 4) + kv
    infos, off, blobs = b"", 0, []
    for name, t, rows, cols, raw in tensors:
        dims = [cols] if rows == 1 else [cols, rows]
        infos += s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", t, off)
        blobs.append((off, raw))
        off += (len(raw) + 31) // 32 * 32
    body = head + infos
    body += b"\0" * ((-len(body)) % 32)
    data = bytearray(off)
    for o, raw in blobs:
        data[o:o + len(raw)] = raw
    with open(path, "wb") as f:
        f.write(body + bytes(data))


GGUF_SPEC = ModelSpec("gguf-tiny", vocab=512, d_model=256, n_layers=2, n_q_heads=4, n_kv_heads=2, head_dim=64, ffn_dim=512,
                      weight_fmt=L.FMT_Q4G64REF, head_fmt=L.FMT_Q4G64REF, embed_fmt=L.FMT_Q4G64REF)
GGUF_NAMES = {L.ROLE_EMBED: "token_embd.weight", L.ROLE_FINAL_NORM: "output_norm.weight", L.ROLE_LM_HEAD: "output.weight",
              L.ROLE_ATTN_NORM: "attn_norm.weight", L.ROLE_WQ: "attn_q.weight", L.ROLE_WK: "attn_k.weight", L.ROLE_WV: "attn_v.weight",
              L.ROLE_WO: "attn_output.weight", L.ROLE_MLP_NORM: "ffn_norm.weight", L.ROLE_WGATE: "ffn_gate.weight",
              L.ROLE_WUP: "ffn_up.weight", L.ROLE_WDOWN: "ffn_down.weight"}


def gguf_model(rng):
    """(file tensor list, {(role, layer): (data, scales, fmt)} as the checker stores them)."""
    file_tensors, stored = [], {}
    for role, layer, rows, cols, mean, std in GGUF_SPEC.tensors():
        name = GGUF_NAMES[role] if role in (L.ROLE_EMBED, L.ROLE_FINAL_NORM, L.ROLE_LM_HEAD) else "blk.%d.%s" % (layer, GGUF_NAMES[role])
        if role in H.VEC_ROLES:
            w = (1.0 + 0.02 * rng.standard_normal(cols)).astype(np.float32)
            file_tensors.append((name, 0, 1, cols, w.tobytes()))
            stored[(role, layer)] = (*O.quantize(w.reshape(1, cols), L.FMT_F16), L.FMT_F16)
            continue
        t = Q6_K if role in (L.ROLE_WV, L.ROLE_WDOWN, L.ROLE_LM_HEAD) else Q4_K   # the mix llama.cpp's Q4_K_M files use
        blocks = random_blocks(rng, t, rows * cols // 256)
        file_tensors.append((name, t, rows, cols, blocks.tobytes()))
        words, sm = O.unpack_gguf(blocks, t)
        stored[(role, layer)] = (words.reshape(rows, cols // 8), sm.reshape(rows, cols // 64, 2), L.FMT_Q4G64REF)
    return file_tensors, stored


def test_runner_refuses_a_broken_gguf(tmp_path):
    from test_runner import runner_path
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUF" + struct.pack("<IQQ", 3, 5, 0) + b"\x01" * 9)
    r = subprocess.run([runner_path(), "--weights", str(bad)], capture_output=True, text=True)
    assert r.returncode == 1 and "not a GGUF file" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("ggml_type", [Q4_K, Q6_K])
def test_cuda_unpack_is_bit_exact(vb, ggml_type):
    from velox_b200.engine import DeviceBuffer
    rng = np.random.default_rng(100 + ggml_type)
    n = 1500
    blocks = random_blocks(rng, ggml_type, n)
    want_w, want_s = O.unpack_gguf(blocks, ggml_type)
    d_src = DeviceBuffer.from_numpy(blocks)
    d_w, d_s = DeviceBuffer(n * 128), DeviceBuffer(n * 16)
    vb.check(vb.load().vb_op_unpack_gguf(d_w.ptr, d_s.ptr, d_src.ptr, ggml_type, n, None))
    vb.check(vb.load().vb_dev_sync())
    assert np.array_equal(d_w.to_numpy(np.uint32, (n * 32,)), want_w)
    assert np.array_equal(d_s.to_numpy(np.uint16, (n * 4, 2)), want_s)
    assert vb.load().vb_gguf_tensor_bytes(ggml_type, 256 * n) == blocks.nbytes
    assert vb.load().vb_gguf_tensor_bytes(ggml_type, 255) == 0


@pytest.mark.gpu
def test_runner_serves_a_gguf_file(tmp_path):
    """A GGUF file with Q4_K / Q6_K / F32 tensors through the runner (--quantize q4_0: the reference's own q4 storage)
    and through vb_load_tensor_gguf: the checker's greedy tokens and stored tensors."""
    from test_runner import runner_path
    from velox_b200.engine import Engine
    rng = np.random.default_rng(77)
    file_tensors, stored = gguf_model(rng)
    path = str(tmp_path / "tiny.gguf")
    write_gguf(path, file_tensors)
    spec = GGUF_SPEC
    ora = O.Engine(vocab=spec.vocab, d_model=spec.d_model, n_layers=spec.n_layers, n_q_heads=spec.n_q_heads, n_kv_heads=spec.n_kv_heads,
                   head_dim=spec.head_dim, ffn_dim=spec.ffn_dim, max_seq_len=64, rms_eps=spec.rms_eps, rope_theta=spec.rope_theta,
                   qkv_bias=0, n_seqs=1, mla_latent=0)
    for (role, layer), (data, scales, fmt) in stored.items():
        ora.set_tensor(role, layer, data, scales, fmt)
    prompt = np.array([5, 17, 300, 42, 7], dtype=np.uint32)
    want = ora.generate_greedy(prompt, 24)
    # the library entry point
    eng = Engine(spec, max_seq_len=64)
    by_name = {n: (t, r, c, raw) for n, t, r, c, raw in file_tensors}
    for role, layer, rows, cols, _, _ in spec.tensors():
        name = GGUF_NAMES[role] if role in (L.ROLE_EMBED, L.ROLE_FINAL_NORM, L.ROLE_LM_HEAD) else "blk.%d.%s" % (layer, GGUF_NAMES[role])
        t, r, c, raw = by_name[name]
        buf = np.frombuffer(raw, dtype=np.uint8)
        L.check(eng._lib.vb_load_tensor_gguf(eng.h, role, layer, buf.ctypes.data_as(L.C.c_void_p), t, rows, cols))
    got_d, got_s = eng.export_tensor(L.ROLE_WDOWN, 1, spec.d_model, spec.ffn_dim)
    assert np.array_equal(got_d, stored[(L.ROLE_WDOWN, 1)][0]) and np.array_equal(got_s, stored[(L.ROLE_WDOWN, 1)][1])
    got = eng.generate_greedy(prompt, 24)
    assert float(np.max(np.abs(eng.logits() - ora.logits))) <= 2e-2
    assert np.array_equal(got, want)
    eng.close()
    # the runner
    r = subprocess.run([runner_path(), "--weights", path, "--tokens", ",".join(str(int(t)) for t in prompt), "--steps", "24",
                        "--quantize", "q4_0", "--dims", "512,256,2,4,2,64,512", "--verbose"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    m = re.search(r"Generated Tokens \(24\)\s*: \[([^\]]*)\]", r.stdout)
    assert m and [int(x) for x in m.group(1).split(",")] == [int(t) for t in want]
    assert "Parity 4-token check   : SKIPPED" in r.stdout and "Parity 32-token check  : SKIPPED" in r.stdout
