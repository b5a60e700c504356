"""The CPU checker against the reference: known-answer vectors of the reference's own tests, the compiled
reference (oracle/_ref, when the reference tree is present) and the committed fixtures made from it."""
import ctypes as C
import hashlib
import json
import math
import os

import numpy as np
import pytest

import helpers as H
from velox_b200.modelspec import SMOLLM_135M

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
KA = json.load(open(os.path.join(GOLD, "known_answers.json")))


def P(a):
    return a.ctypes.data_as(C.c_void_p)


def f32(x):
    return np.ascontiguousarray(x, dtype=np.float32)


@pytest.mark.parametrize("case", KA["rmsnorm"], ids=lambda c: c["cite"])
def test_rmsnorm_known_answers(oracle, case):
    x, w = f32(case["x"]), f32(case["w"])
    out = np.ones_like(x)
    oracle.lib().vo_rmsnorm_f32(P(out), P(x), P(w), x.size, case["eps"])
    if "expect0_inv_sqrt_of" in case:
        assert abs(out[0] - 1.0 / math.sqrt(np.float32(case["expect0_inv_sqrt_of"]))) < case["tol"]
    else:
        assert np.all(np.isfinite(out))
        assert np.max(np.abs(out - f32(case["expect"]))) <= case["tol"]


def test_rope_known_answers(oracle):
    for case in KA["rope"]:
        t = f32(case["t"])
        oracle.lib().vo_rope_rotate_half_f32(P(t), case["heads"], case["head_dim"], case["pos"], case["theta"])
        assert np.max(np.abs(t - f32(case["expect"]))) < case["tol"]
    c = KA["rope_norm_preserved"]
    n = c["heads"] * c["head_dim"]
    v = f32(oracle.fill_normal(n, 1337, 0, 1.0)).clip(c["lo"], c["hi"])
    before = float(np.sqrt(np.sum(v * v)))
    oracle.lib().vo_rope_rotate_half_f32(P(v), c["heads"], c["head_dim"], c["pos"], c["theta"])
    assert abs(before - float(np.sqrt(np.sum(v * v)))) < c["tol"]


@pytest.mark.parametrize("case", KA["gqa"], ids=lambda c: c["cite"])
def test_gqa_known_answers(oracle, case):
    q, k, v = f32(case["q"]), f32(case["k"]), f32(case["v"])
    out = np.zeros(case["n_q"] * case["head_dim"], dtype=np.float32)
    scores = np.zeros(8, dtype=np.float32)
    oracle.lib().vo_gqa_attention_step_f32(P(out), P(scores), P(q), P(k), P(v), case["n_q"], case["n_kv"], case["head_dim"], case["pos"])
    assert np.array_equal(out, f32(case["expect"]))


def test_swiglu_and_matmul_known_answers(oracle):
    c = KA["swiglu"]
    hidden, nx, eye = f32(c["hidden"]), f32(c["nx"]), f32(c["eye"])
    g, u, d = (np.zeros(2, dtype=np.float32) for _ in range(3))
    oracle.lib().vo_swiglu_mlp_residual_f32(P(hidden), P(g), P(u), P(d), P(nx), P(eye), P(eye), P(eye), c["d"], c["ffn"])
    silu1 = 1.0 / (1.0 + math.exp(-1.0))
    assert abs(hidden[0] - (1.0 + silu1)) < c["tol"] and abs(hidden[1] - (2.0 + silu1)) < c["tol"]
    for m in KA["matmul"]:
        x, w = f32(m["x"]), f32(m["w"])
        out = np.zeros(m["out"], dtype=np.float32)
        oracle.lib().vo_matmul_transposed_f32(P(out), P(x), P(w), m["in"], m["out"])
        assert np.max(np.abs(out - f32(m["expect"]))) < m["tol"]


def test_argmax_known_answers(oracle):
    for c in KA["argmax"]:
        lg = f32(c["logits"])
        assert oracle.lib().vo_sample_argmax_f32(P(lg), lg.size) == c["expect"]
    # rule of src/runtime.rs:1078-1088: NaN never wins, an all -inf row gives 0
    lg = f32([np.nan, -np.inf, 1.0, np.nan, 1.0])
    assert oracle.lib().vo_sample_argmax_f32(P(lg), lg.size) == 2
    lg = f32([-np.inf, -np.inf])
    assert oracle.lib().vo_sample_argmax_f32(P(lg), lg.size) == 0


MLA_W = dict(w_norm=[1, 1, 1, 1], w_dkv=[1, 0, 0, 0, 0, 1, 0, 0], w_q=[1, 0, 0, 0, 0, 1, 0, 0], w_o=[1, 0, 0, 1, 0, 0, 0, 0])


def _mla(oracle, x, pool, step):
    dst = np.zeros(4, dtype=np.float32)
    oracle.lib().vo_mla_absorbed_step_f32(P(dst), P(f32(x)), P(f32(MLA_W["w_norm"])), P(f32(MLA_W["w_dkv"])), P(f32(MLA_W["w_q"])),
                                          P(f32(MLA_W["w_o"])), P(pool), step, 4, 2, 4, 1e-5)
    return dst


def test_mla_known_answers(oracle):
    for c in KA["mla"]:
        pool = np.zeros(8, dtype=np.float32)
        dst = _mla(oracle, c["input"], pool, 0)
        assert np.max(np.abs(dst - f32(c["expect"]))) < c["tol"]
        assert abs(pool[0] - 1.0) < 1e-4 and abs(pool[1] - 1.0) < 1e-4
    c = KA["mla_two_step"]
    pool = np.zeros(8, dtype=np.float32)
    _mla(oracle, c["input0"], pool, 0)
    dst = _mla(oracle, c["input1"], pool, 1)
    k0, k1 = pool[0:2].astype(np.float64), pool[2:4].astype(np.float64)
    scale = 1.0 / math.sqrt(2.0)
    s0, s1 = float(k1 @ k0) * scale, float(k1 @ k1) * scale
    m = max(s0, s1)
    e0, e1 = math.exp(s0 - m), math.exp(s1 - m)
    ctx = (e0 * k0 + e1 * k1) / (e0 + e1)
    want = np.array([c["input1"][0] + ctx[0], c["input1"][1] + ctx[1], c["input1"][2], c["input1"][3]])
    assert np.max(np.abs(dst - want)) < c["tol"]


def test_int4_dequant_contract(oracle):
    c = KA["int4_dequant"]
    # one row of 32 elements holding every nibble twice, scale 0.03125 (exact in fp16)
    nib = np.arange(32, dtype=np.uint32) % 16
    words = np.zeros(4, dtype=np.uint32)
    for wd in range(4):
        q = nib[wd * 8:(wd + 1) * 8]
        words[wd] = q[0] | q[2] << 4 | q[4] << 8 | q[6] << 12 | q[1] << 16 | q[3] << 20 | q[5] << 24 | q[7] << 28
    scales = np.array([oracle.lib().vo_f32_to_f16(c["scale"])], dtype=np.uint16)
    out = oracle.dequantize(words.reshape(1, 4), scales.reshape(1, 1), oracle.FMT_Q4G32, 1, 32)[0]
    want = f32(c["expect_for_nibble"])
    assert np.array_equal(out, want[nib])
    assert np.array_equal(want, (np.arange(16, dtype=np.float32) - np.float32(c["zero"])) * np.float32(c["scale"]))


def test_half_conversion_matches_numpy(oracle):
    rng = np.random.default_rng(7)
    vals = np.concatenate([rng.standard_normal(4000).astype(np.float32) * 10.0 ** rng.integers(-8, 5, 4000),
                           f32([0, -0.0, 65504, 65520, 65519.99, 1e-8, 5.96e-8, 2.98e-8, 2.99e-8, np.inf, -np.inf, 6.1e-5])])
    ours = np.array([oracle.lib().vo_f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    with np.errstate(over="ignore"):
        ref = vals.astype(np.float16).view(np.uint16)
    assert np.array_equal(ours, ref)
    back = np.array([oracle.lib().vo_f16_to_f32(int(h)) for h in ours[:2000]], dtype=np.float32)
    assert np.array_equal(back.view(np.uint32), ours[:2000].view(np.float16).astype(np.float32).view(np.uint32))


@pytest.mark.parametrize("fmt", ["q4g32", "q4g64ref", "i8pc"])
def test_quantizers_roundtrip_and_edges(oracle, fmt):
    code = {"q4g32": oracle.FMT_Q4G32, "q4g64ref": oracle.FMT_Q4G64REF, "i8pc": oracle.FMT_I8PC}[fmt]
    rows, cols = 6, 128
    w = oracle.fill_normal(rows * cols, 5, 1, 0.02).reshape(rows, cols).copy()
    w[1, :] = 0.0          # all-zero row: scale 0
    w[2, :64] = 0.0125     # constant group (max == min for the asymmetric format)
    w[3, 5] = 3.0          # outlier
    data, scales = oracle.quantize(w, code)
    deq = oracle.dequantize(data, scales, code, rows, cols)
    assert np.all(np.isfinite(deq))
    assert np.all(deq[1] == 0.0)
    # error bound: half a quantization step of the group / row (plus fp16 rounding of scale and min)
    if fmt == "q4g32":
        step = np.abs(w).reshape(rows, cols // 32, 32).max(axis=2, keepdims=True) / 7.0
        bound = np.broadcast_to(step * 0.5 * 1.01 + 1e-6, (rows, cols // 32, 32)).reshape(rows, cols)
        # the +7 end of the range clamps at 7*scale, which the fp16 rounding of the scale can move slightly
        assert np.all(np.abs(deq - w) <= bound + np.abs(w) * 2e-3)
    elif fmt == "i8pc":
        step = np.abs(w).max(axis=1, keepdims=True) / 127.0
        assert np.all(np.abs(deq - w) <= step * 0.5 * 1.01 + np.abs(w) * 2e-3 + 1e-7)
    else:
        g = w.reshape(rows, cols // 64, 64)
        step = (g.max(axis=2, keepdims=True) - g.min(axis=2, keepdims=True)) / 15.0
        bound = np.broadcast_to(step * 0.5 * 1.02 + np.abs(g).max(axis=2, keepdims=True) * 2e-3 + 1e-6, g.shape).reshape(rows, cols)
        assert np.all(np.abs(deq - w) <= bound)
    # idempotence: quantizing the dequantized values reproduces the same integers for the symmetric formats
    if fmt != "q4g64ref":
        data2, scales2 = oracle.quantize(deq, code)
        assert np.array_equal(scales2, scales) and np.array_equal(data2, data)


def test_matvec_formats_agree_with_dequantized_fp32(oracle):
    rows, cols = 40, 256
    w = oracle.fill_normal(rows * cols, 9, 3, 0.02).reshape(rows, cols)
    x = oracle.fill_normal(cols, 9, 4, 1.0)
    for code in (oracle.FMT_F16, oracle.FMT_BF16, oracle.FMT_Q4G32, oracle.FMT_Q4G64REF, oracle.FMT_I8PC):
        data, scales = oracle.quantize(w, code)
        deq = oracle.dequantize(data, scales, code, rows, cols)
        a = oracle.matvec(x, data, scales, code, cols, rows)
        b = oracle.matvec(x, deq, None, oracle.FMT_F32, cols, rows)
        assert np.array_equal(a, b)


def test_generator_statistics_and_determinism(oracle):
    a = oracle.fill_normal(200000, 11, 5, 0.02)
    b = oracle.fill_normal(200000, 11, 5, 0.02)
    assert np.array_equal(a, b)
    assert abs(float(a.mean())) < 2e-4 and abs(float(a.std()) - 0.02) < 2e-4
    assert not np.array_equal(a[:1000], oracle.fill_normal(1000, 11, 6, 0.02))
    t = oracle.fill_tokens(1000, 3, 1, 49152)
    assert t.max() < 49152 and len(np.unique(t)) > 900


# ---- the compiled reference and the fixtures made from it ----------------------------------------

def _smollm_oracle(oracle, seed, max_seq):
    eng, _ = H.build_oracle(SMOLLM_135M, seed, max_seq)
    return eng


def test_oracle_reproduces_reference_fixture(oracle):
    """Fixture = the reference's emitted C99 model run on seed weights (tests/golden/make_golden.py)."""
    g = json.load(open(os.path.join(GOLD, "smollm_ref_golden.json")))
    eng = _smollm_oracle(oracle, g["seed"], 64)
    tok, pos = 0, 0
    for t in g["prompt"]:
        tok = eng.forward_step(t, pos)
        pos += 1
    for i, st in enumerate(g["steps"]):
        lg = eng.logits
        assert tok == st["token"] == g["tokens"][i]
        assert hashlib.sha256(lg.tobytes()).hexdigest() == st["sha256"], "logits differ from the reference at step %d" % i
        assert [int(j) for j in np.argsort(-lg, kind="stable")[:5]] == st["top5_ids"]
        if i + 1 < len(g["steps"]):
            tok = eng.forward_step(tok, pos)
            pos += 1


def test_oracle_primitives_match_compiled_reference(oracle):
    R = oracle.ref_lib()
    if R is None:
        pytest.skip("oracle/_ref not built (no reference tree on this machine)")
    Lb = oracle.lib()
    for in_dim, out_dim in ((576, 1536), (1536, 576), (64, 7), (576, 512)):
        x = oracle.fill_normal(in_dim, 21, 1, 1.0)
        w = oracle.fill_normal(in_dim * out_dim, 21, 2, 0.02)
        a, b = np.zeros(out_dim, dtype=np.float32), np.zeros(out_dim, dtype=np.float32)
        Lb.vo_matmul_transposed_f32(P(a), P(x), P(w), in_dim, out_dim)
        R.refsm_matmul_vec(P(b), P(x), P(w), in_dim, out_dim)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    x = oracle.fill_normal(576, 22, 1, 1.0)
    w = oracle.fill_normal(576, 22, 2, 0.02, 1.0)
    a, b = np.zeros(576, dtype=np.float32), np.zeros(576, dtype=np.float32)
    Lb.vo_rmsnorm_f32(P(a), P(x), P(w), 576, 1e-5)
    R.refsm_rmsnorm(P(b), P(x), P(w), 576, 1e-5)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    t1 = oracle.fill_normal(9 * 64, 23, 1, 1.0)
    t2 = t1.copy()
    Lb.vo_rope_rotate_half_f32(P(t1), 9, 64, 777, 10000.0)
    R.refsm_rope(P(t2), 9, 64, 777, 10000.0)
    assert np.array_equal(t1.view(np.uint32), t2.view(np.uint32))
    S = 37
    q = oracle.fill_normal(9 * 64, 24, 1, 1.0)
    k = oracle.fill_normal(S * 3 * 64, 24, 2, 1.0)
    v = oracle.fill_normal(S * 3 * 64, 24, 3, 1.0)
    o1, o2 = np.zeros(9 * 64, dtype=np.float32), np.zeros(9 * 64, dtype=np.float32)
    sc = np.zeros(S, dtype=np.float32)
    Lb.vo_gqa_attention_step_f32(P(o1), P(sc), P(q), P(k), P(v), 9, 3, 64, S - 1)
    R.refsm_gqa(P(o2), P(sc), P(q), P(k), P(v), 9, 3, 64, S - 1)
    assert np.array_equal(o1.view(np.uint32), o2.view(np.uint32))
    # absorbed MLA: the emitted function (two-pass softmax) against the restated Rust one (online softmax)
    hid, lat, max_s = 576, 512, 2048
    wn = oracle.fill_normal(hid, 25, 1, 0.02, 1.0)
    wd = oracle.fill_normal(hid * lat, 25, 2, 0.02)
    wq = oracle.fill_normal(hid * lat, 25, 3, 0.02)
    wo = oracle.fill_normal(hid * lat, 25, 4, 0.02)
    p1, p2 = np.zeros(max_s * lat, dtype=np.float32), np.zeros(max_s * lat, dtype=np.float32)
    for step in range(6):
        xin = oracle.fill_normal(hid, 25, 10 + step, 1.0)
        d1, d2 = np.zeros(hid, dtype=np.float32), np.zeros(hid, dtype=np.float32)
        Lb.vo_mla_absorbed_step_f32(P(d1), P(xin), P(wn), P(wd), P(wq), P(wo), P(p1), step, hid, lat, max_s, 1e-5)
        R.refsm_mla(P(d2), P(xin), P(wn), P(wd), P(wq), P(wo), P(p2), 0, step, 1e-5)
        assert np.max(np.abs(d1 - d2)) < 1e-4  # bound of tests/test_adversarial_step8_mla.rs:195-303
    assert np.array_equal(p1, p2)
