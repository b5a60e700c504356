"""The per-op entry points of the fused IR instructions (FusedNormQkvRopeAttn, FusedOutProjResSwiGluRes, KVWrite, SwiGlu;
src/ir.rs:83,158,232-272) through the C ABI, against the two halves of the checker's layer step composed from its
primitives (the reference's own composition: src/runners/tinystories_smollm.c:277-344)."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
from velox_b200 import lib as L

pytestmark = pytest.mark.gpu


def P(a):
    return a.ctypes.data_as(C.c_void_p)


class DevWeight:
    """A matrix quantized by the checker, uploaded in canonical layout, with its vb_weight descriptor."""

    def __init__(self, dev, w, fmt):
        self.data_h, self.scales_h = O.quantize(w, fmt)
        self.fmt, self.rows, self.cols = fmt, w.shape[0], w.shape[1]
        self.data = dev.from_numpy(self.data_h)
        self.scales = dev.from_numpy(self.scales_h) if self.scales_h is not None else None
        self.desc = L.Weight(self.data.ptr, self.scales.ptr if self.scales is not None else None, fmt)

    def matvec(self, x):
        return O.matvec(x, self.data_h, self.scales_h, self.fmt, self.cols, self.rows)


def checker_attention_half(x, w_norm, wq, wk, wv, bq, bk, bv, k_cache, v_cache, step, n_q, n_kv, D, eps, theta):
    lib = O.lib()
    nx = np.empty_like(x)
    lib.vo_rmsnorm_f32(P(nx), P(x), P(w_norm), x.size, eps)
    q, k, v = wq.matvec(nx), wk.matvec(nx), wv.matvec(nx)
    if bq is not None:
        q, k, v = q + bq, k + bk, v + bv
    q, k = np.ascontiguousarray(q, dtype=np.float32), np.ascontiguousarray(k, dtype=np.float32)
    lib.vo_rope_rotate_half_f32(P(q), n_q, D, step, theta)
    lib.vo_rope_rotate_half_f32(P(k), n_kv, D, step, theta)
    k_cache[step], v_cache[step] = k, v
    out = np.empty(n_q * D, dtype=np.float32)
    scores = np.empty(k_cache.shape[0], dtype=np.float32)
    lib.vo_gqa_attention_step_f32(P(out), P(scores), P(q), P(k_cache), P(v_cache), n_q, n_kv, D, step)
    return out


def checker_mlp_half(attn, resid, wo, w_post, wg, wu, wd, eps):
    lib = O.lib()
    mid = (wo.matvec(attn) + resid).astype(np.float32)
    nm = np.empty_like(mid)
    lib.vo_rmsnorm_f32(P(nm), P(mid), P(w_post), mid.size, eps)
    g, u = wg.matvec(nm), wu.matvec(nm)
    act = ((g / (1.0 + np.exp(-g.astype(np.float32)))) * u).astype(np.float32)
    return (mid + wd.matvec(act)).astype(np.float32), act


CASES = [
    # d_model, n_q, n_kv, D, ffn, fmt, bias
    (576, 9, 3, 64, 1536, O.FMT_F32, False),      # the SmolLM layer the reference ships
    (512, 8, 2, 64, 1408, O.FMT_Q4G32, True),
    (512, 4, 4, 128, 1024, O.FMT_F16, False),
    (512, 8, 1, 64, 1024, O.FMT_I8PC, True),
    (512, 8, 2, 64, 1024, O.FMT_Q4G64REF, False),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "d%d-h%d/%d-f%d%s" % (c[0], c[1], c[2], c[5], "-bias" if c[6] else ""))
def test_fused_layer_halves_match_checker(vb, case):
    from velox_b200.engine import DeviceBuffer as dev
    d, n_q, n_kv, D, ffn, fmt, bias = case
    lib = vb.load()
    rng = np.random.default_rng(d + n_q + fmt)
    qd, kvd, max_seq, eps, theta = n_q * D, n_kv * D, 48, 1e-5, 10000.0

    def mat(r, c):
        return DevWeight(dev, (0.02 * rng.standard_normal((r, c))).astype(np.float32), fmt)
    wq, wk, wv, wo, wg, wu, wd = mat(qd, d), mat(kvd, d), mat(kvd, d), mat(d, qd), mat(ffn, d), mat(ffn, d), mat(d, ffn)
    w_norm = (1 + 0.02 * rng.standard_normal(d)).astype(np.float32)
    w_post = (1 + 0.02 * rng.standard_normal(d)).astype(np.float32)
    bq = (0.02 * rng.standard_normal(qd)).astype(np.float32) if bias else None
    bk = (0.02 * rng.standard_normal(kvd)).astype(np.float32) if bias else None
    bv = (0.02 * rng.standard_normal(kvd)).astype(np.float32) if bias else None
    d_norm, d_post = dev.from_numpy(w_norm), dev.from_numpy(w_post)
    d_b = [dev.from_numpy(b) if b is not None else None for b in (bq, bk, bv)]
    k_cache, v_cache = np.zeros((max_seq, kvd), np.float32), np.zeros((max_seq, kvd), np.float32)
    d_k, d_v = dev.from_numpy(k_cache), dev.from_numpy(v_cache)
    need = lib.vb_op_fused_scratch_bytes(d, n_q, n_kv, D, ffn, max_seq)
    scratch = dev(need)
    d_x, d_attn, d_hidden, d_step = dev(d * 4), dev(qd * 4), dev(d * 4), dev(4)
    x = rng.standard_normal(d).astype(np.float32)
    for step in range(0, 40):
        use_dev_step = step % 2 == 1      # alternate: position by value / read from device memory
        vb.check(lib.vb_dev_upload(d_x.ptr, P(x), d * 4))
        if use_dev_step:
            vb.check(lib.vb_dev_upload(d_step.ptr, P(np.array([step], np.uint32)), 4))
        vb.check(lib.vb_op_fused_norm_qkv_rope_attn(
            d_attn.ptr, d_x.ptr, d_norm.ptr, C.byref(wq.desc), C.byref(wk.desc), C.byref(wv.desc),
            d_b[0].ptr if bias else None, d_b[1].ptr if bias else None, d_b[2].ptr if bias else None, d_k.ptr, d_v.ptr, max_seq,
            0 if use_dev_step else step, d_step.ptr if use_dev_step else None, d, n_q, n_kv, D, eps, theta, scratch.ptr, need, None))
        vb.check(lib.vb_op_fused_outproj_res_swiglu_res(
            d_hidden.ptr, d_attn.ptr, d_x.ptr, C.byref(wo.desc), d_post.ptr, C.byref(wg.desc), C.byref(wu.desc), C.byref(wd.desc),
            d, qd, ffn, eps, scratch.ptr, need, None))
        vb.check(lib.vb_dev_sync())
        want_attn = checker_attention_half(x, w_norm, wq, wk, wv, bq, bk, bv, k_cache, v_cache, step, n_q, n_kv, D, eps, theta)
        want_hidden, _ = checker_mlp_half(want_attn, x, wo, w_post, wg, wu, wd, eps)
        got_attn, got_hidden = d_attn.to_numpy(np.float32, (qd,)), d_hidden.to_numpy(np.float32, (d,))
        assert np.max(np.abs(got_attn - want_attn)) <= 2e-4, (step, float(np.max(np.abs(got_attn - want_attn))))
        assert np.max(np.abs(got_hidden - want_hidden)) <= 1e-3 * max(1.0, float(np.max(np.abs(want_hidden)))), step
        x = want_hidden / max(1.0, float(np.max(np.abs(want_hidden))))   # next token's input, kept in range
    # the cache rows the op wrote are the checker's (fp32, RoPE applied to K)
    assert np.max(np.abs(d_k.to_numpy(np.float32, k_cache.shape) - k_cache)) <= 2e-5
    assert np.max(np.abs(d_v.to_numpy(np.float32, v_cache.shape) - v_cache)) <= 2e-5


def test_kv_write_and_swiglu_ops(vb):
    from velox_b200.engine import DeviceBuffer as dev
    lib = vb.load()
    rng = np.random.default_rng(9)
    d, ffn, kvd, max_seq = 512, 1408, 192, 16
    wg, wu, wd = (DevWeight(dev, (0.02 * rng.standard_normal(s)).astype(np.float32), O.FMT_Q4G32) for s in ((ffn, d), (ffn, d), (d, ffn)))
    x = rng.standard_normal(d).astype(np.float32)
    d_x, d_out, scratch = dev.from_numpy(x), dev(d * 4), dev(ffn * 4 + 64)
    vb.check(lib.vb_op_swiglu(d_out.ptr, d_x.ptr, C.byref(wg.desc), C.byref(wu.desc), C.byref(wd.desc), d, ffn, scratch.ptr, ffn * 4 + 64, None))
    g, u = wg.matvec(x), wu.matvec(x)
    want = wd.matvec(((g / (1.0 + np.exp(-g))) * u).astype(np.float32))
    vb.check(lib.vb_dev_sync())
    assert np.max(np.abs(d_out.to_numpy(np.float32, (d,)) - want)) <= 1e-4
    # KVWrite: rows by value, by device word, and clamped to the last row like the reference's safe_step
    d_k, d_v = dev.from_numpy(np.zeros((max_seq, kvd), np.float32)), dev.from_numpy(np.zeros((max_seq, kvd), np.float32))
    d_step = dev(4)
    want_k, want_v = np.zeros((max_seq, kvd), np.float32), np.zeros((max_seq, kvd), np.float32)
    for step, by_dev in ((0, False), (5, True), (15, False), (99, True)):
        k, v = rng.standard_normal(kvd).astype(np.float32), rng.standard_normal(kvd).astype(np.float32)
        dk, dv = dev.from_numpy(k), dev.from_numpy(v)
        if by_dev:
            vb.check(lib.vb_dev_upload(d_step.ptr, P(np.array([step], np.uint32)), 4))
        vb.check(lib.vb_op_kv_write(d_k.ptr, d_v.ptr, dk.ptr, dv.ptr, 0 if by_dev else step, d_step.ptr if by_dev else None, kvd, max_seq, None))
        vb.check(lib.vb_dev_sync())
        want_k[min(step, max_seq - 1)], want_v[min(step, max_seq - 1)] = k, v
    assert np.array_equal(d_k.to_numpy(np.float32, want_k.shape), want_k) and np.array_equal(d_v.to_numpy(np.float32, want_v.shape), want_v)
    # argument checks return status codes
    assert lib.vb_op_swiglu(None, d_x.ptr, C.byref(wg.desc), C.byref(wu.desc), C.byref(wd.desc), d, ffn, scratch.ptr, 8, None) == vb.ERR_INVALID
    assert lib.vb_op_kv_write(None, None, None, None, 0, None, 0, 0, None) == vb.ERR_INVALID
