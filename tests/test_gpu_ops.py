"""Per-op parity of the CUDA library (through the C ABI) against the CPU checker."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def P(a):
    return a.ctypes.data_as(C.c_void_p)


@pytest.fixture(scope="module")
def dev(vb):
    from velox_b200.engine import DeviceBuffer
    return DeviceBuffer


FMTS = ["f32", "f16", "bf16", "q4g32", "q4g64ref", "i8pc"]


def code(oracle, name):
    return {"f32": oracle.FMT_F32, "f16": oracle.FMT_F16, "bf16": oracle.FMT_BF16, "q4g32": oracle.FMT_Q4G32,
            "q4g64ref": oracle.FMT_Q4G64REF, "i8pc": oracle.FMT_I8PC}[name]


def test_fill_normal_bit_exact(vb, oracle, dev):
    n = 100003
    buf = dev(n * 4)
    vb.check(vb.load().vb_op_fill_normal(buf.ptr, n, 42, 7, 0.5, 0.02, None))
    got = buf.to_numpy(np.float32, (n,))
    assert np.array_equal(got.view(np.uint32), oracle.fill_normal(n, 42, 7, 0.02, 0.5).view(np.uint32))


@pytest.mark.parametrize("fmt", FMTS[1:])
def test_quantize_dequantize_bit_exact(vb, oracle, dev, fmt):
    """Quantized integers, scales and dequantized values are bit-identical to the checker's."""
    c = code(oracle, fmt)
    rows, cols = 37, 512
    w = oracle.fill_normal(rows * cols, 3, 11, 0.02).reshape(rows, cols).copy()
    w[0] = 0.0
    w[1, :64] = 0.0125
    w[2, 3] = 2.5
    w[3, :32] = np.linspace(-0.07, 0.07, 32, dtype=np.float32)  # exercises round-half-even ties
    data_ref, scales_ref = oracle.quantize(w, c)
    src = dev.from_numpy(w)
    d_data = dev(data_ref.nbytes)
    d_scales = dev(scales_ref.nbytes if scales_ref is not None else 16)
    lib = vb.load()
    vb.check(lib.vb_op_quantize(d_data.ptr, d_scales.ptr, src.ptr, c, rows, cols, None))
    got = d_data.to_numpy(data_ref.dtype, data_ref.shape)
    assert np.array_equal(got, data_ref)
    if scales_ref is not None:
        assert np.array_equal(d_scales.to_numpy(np.uint16, scales_ref.shape), scales_ref)
    out = dev(rows * cols * 4)
    vb.check(lib.vb_op_dequantize(out.ptr, d_data.ptr, d_scales.ptr, c, rows, cols, None))
    deq = out.to_numpy(np.float32, (rows, cols))
    assert np.array_equal(deq.view(np.uint32), oracle.dequantize(data_ref, scales_ref, c, rows, cols).view(np.uint32))


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("shape", [(64, 5), (576, 1536), (4096, 300), (14336, 64)])
def test_matmul_parity(vb, oracle, dev, fmt, shape):
    in_dim, out_dim = shape
    c = code(oracle, fmt)
    w = oracle.fill_normal(out_dim * in_dim, 5, 1, 0.02).reshape(out_dim, in_dim)
    data, scales = oracle.quantize(w, c)
    batch = 3
    x = oracle.fill_normal(batch * in_dim, 5, 2, 1.0).reshape(batch, in_dim)
    dw, dx, dy = dev.from_numpy(data), dev.from_numpy(x), dev(batch * out_dim * 4)
    ds = dev.from_numpy(scales) if scales is not None else None
    vb.check(vb.load().vb_op_matmul(dy.ptr, dx.ptr, dw.ptr, ds.ptr if ds else None, c, in_dim, out_dim, batch, None))
    got = dy.to_numpy(np.float32, (batch, out_dim))
    for b in range(batch):
        want = oracle.matvec(x[b], data, scales, c, in_dim, out_dim)
        scale = np.sqrt(in_dim) * 0.02
        assert np.max(np.abs(got[b] - want)) <= 1e-5 * scale + 1e-6  # fp32 summation order only


def test_matmul_empty_and_bad_shapes(vb, dev):
    lib = vb.load()
    b = dev(1024)
    assert lib.vb_op_matmul(b.ptr, b.ptr, b.ptr, None, vb.FMT_F32, 8, 0, 1, None) == vb.OK
    assert lib.vb_op_matmul(b.ptr, b.ptr, b.ptr, None, vb.FMT_F32, 8, 4, 0, None) == vb.OK
    assert lib.vb_op_matmul(b.ptr, b.ptr, b.ptr, None, vb.FMT_Q4G32, 40, 4, 1, None) == vb.ERR_INVALID  # no scales / bad group
    assert lib.vb_op_matmul(b.ptr, b.ptr, b.ptr, b.ptr, vb.FMT_Q4G32, 40, 4, 1, None) == vb.ERR_INVALID


def test_rmsnorm_rope_parity(vb, oracle, dev):
    lib = vb.load()
    for dim in (4, 576, 4096):
        x = oracle.fill_normal(2 * dim, 6, 1, 1.5).reshape(2, dim)
        w = oracle.fill_normal(dim, 6, 2, 0.02, 1.0)
        dx, dw, dy = dev.from_numpy(x), dev.from_numpy(w), dev(2 * dim * 4)
        vb.check(lib.vb_op_rmsnorm(dy.ptr, dx.ptr, dw.ptr, vb.FMT_F32, dim, 2, 1e-5, None))
        got = dy.to_numpy(np.float32, (2, dim))
        for b in range(2):
            want = np.zeros(dim, dtype=np.float32)
            oracle.lib().vo_rmsnorm_f32(P(want), P(np.ascontiguousarray(x[b])), P(w), dim, 1e-5)
            assert np.max(np.abs(got[b] - want)) < 2e-6 * max(1.0, float(np.abs(want).max()))
    z = dev.from_numpy(np.zeros(8, dtype=np.float32))
    one = dev.from_numpy(np.ones(8, dtype=np.float32))
    out = dev(32)
    vb.check(lib.vb_op_rmsnorm(out.ptr, z.ptr, one.ptr, vb.FMT_F32, 8, 1, 1e-5, None))
    assert np.all(out.to_numpy(np.float32, (8,)) == 0.0)
    for heads, hd, pos, theta in ((1, 4, 0, 10000.0), (4, 16, 47, 10000.0), (32, 128, 2047, 500000.0), (9, 64, 777, 10000.0)):
        t = oracle.fill_normal(heads * hd, 7, 1, 1.0)
        want = t.copy()
        oracle.lib().vo_rope_rotate_half_f32(P(want), heads, hd, pos, theta)
        dt = dev.from_numpy(t)
        vb.check(lib.vb_op_rope(dt.ptr, heads, hd, pos, theta, None))
        got = dt.to_numpy(np.float32, (heads * hd,))
        assert np.max(np.abs(got - want)) < 2e-5 + 2e-7 * pos  # sin/cos of an angle of up to `pos` radians
        if pos == 0:
            assert np.array_equal(got, t)


@pytest.mark.parametrize("cfg", [(2, 1, 32, 0), (9, 3, 64, 36), (32, 8, 128, 700), (28, 4, 128, 2047), (8, 8, 64, 15), (16, 1, 128, 100)])
def test_gqa_attention_parity(vb, oracle, dev, cfg):
    """Split-K flash-decode against the two-pass CPU softmax; bound 1e-4 as in the reference's split-K test."""
    nq, nkv, hd, pos = cfg
    S = pos + 1
    q = oracle.fill_normal(nq * hd, 8, 1, 1.0)
    k = oracle.fill_normal(S * nkv * hd, 8, 2, 1.0)
    v = oracle.fill_normal(S * nkv * hd, 8, 3, 1.0)
    want, sc = np.zeros(nq * hd, dtype=np.float32), np.zeros(S, dtype=np.float32)
    oracle.lib().vo_gqa_attention_step_f32(P(want), P(sc), P(q), P(k), P(v), nq, nkv, hd, pos)
    lib = vb.load()
    nbytes = lib.vb_op_scratch_bytes(nq, hd, S, 1)
    dq, dk, dv, do, ds = dev.from_numpy(q), dev.from_numpy(k), dev.from_numpy(v), dev(nq * hd * 4), dev(nbytes)
    vb.check(lib.vb_op_gqa_attention(do.ptr, dq.ptr, dk.ptr, dv.ptr, nq, nkv, hd, pos, ds.ptr, nbytes, None))
    got = do.to_numpy(np.float32, (nq * hd,))
    assert np.max(np.abs(got - want)) < 1e-4


def test_split_k_closed_form_inputs(vb, oracle, dev):
    """The closed-form inputs of tests/empirical_challenge_phase2/test2_split_k_flashdecoding_parity.cu:185-189."""
    nq, nkv, hd = 9, 3, 64
    lib = vb.load()
    for S in (64, 512, 1024, 2048):
        i = np.arange(nq * hd, dtype=np.float32)
        q = (0.1 * np.sin(i * np.float32(0.13))).astype(np.float32)
        j = np.arange(S * nkv * hd)
        k = (0.08 * np.cos((j % 23).astype(np.float32) * np.float32(0.11))).astype(np.float32)
        v = (0.06 * np.sin((j % 19).astype(np.float32) * np.float32(0.17))).astype(np.float32)
        want, sc = np.zeros(nq * hd, dtype=np.float32), np.zeros(S, dtype=np.float32)
        oracle.lib().vo_gqa_attention_step_f32(P(want), P(sc), P(q), P(k), P(v), nq, nkv, hd, S - 1)
        nbytes = lib.vb_op_scratch_bytes(nq, hd, S, 1)
        dq, dk, dv, do, ds = dev.from_numpy(q), dev.from_numpy(k), dev.from_numpy(v), dev(nq * hd * 4), dev(nbytes)
        vb.check(lib.vb_op_gqa_attention(do.ptr, dq.ptr, dk.ptr, dv.ptr, nq, nkv, hd, S - 1, ds.ptr, nbytes, None))
        assert np.max(np.abs(do.to_numpy(np.float32, (nq * hd,)) - want)) < 1e-4


def test_argmax_bit_exact(vb, oracle, dev):
    lib = vb.load()
    cases = [np.float32([-2.0, 0.5, 9.2, 3.1]), np.float32([5.0, 5.0, 5.0, 5.0]), np.float32([np.nan, -np.inf, 1.0, np.nan, 1.0]),
             np.float32([-np.inf, -np.inf]), np.float32([np.nan] * 7)]
    big = oracle.fill_normal(152064, 9, 1, 1.0)
    cases.append(big)
    tied = big.copy()
    tied[[100, 3000, 70000, 152063]] = 50.0  # ties across stage-1 blocks: the lowest index must win
    cases.append(tied)
    last = big.copy()
    last[-1] = 99.0
    cases.append(last)
    for lg in cases:
        n = lg.size
        nbytes = lib.vb_op_scratch_bytes(1, 32, 1, n)
        dl, dt, ds = dev.from_numpy(lg), dev(4), dev(nbytes)
        vb.check(lib.vb_op_sample_argmax(dt.ptr, dl.ptr, n, ds.ptr, nbytes, None))
        assert int(dt.to_numpy(np.uint32, (1,))[0]) == oracle.lib().vo_sample_argmax_f32(P(lg), n)


def test_embed_formats(vb, oracle, dev):
    lib = vb.load()
    V, d = 100, 256
    table = oracle.fill_normal(V * d, 10, 1, 0.02).reshape(V, d)
    toks = np.array([0, 99, 17, 17], dtype=np.uint32)
    for fmt in ("f32", "f16", "bf16", "q4g64ref", "q4g32"):
        c = code(oracle, fmt)
        data, scales = oracle.quantize(table, c)
        deq = oracle.dequantize(data, scales, c, V, d)
        dtab, dtok, out = dev.from_numpy(data), dev.from_numpy(toks), dev(len(toks) * d * 4)
        ds = dev.from_numpy(scales) if scales is not None else None
        vb.check(lib.vb_op_embed(out.ptr, dtok.ptr, dtab.ptr, ds.ptr if ds else None, c, d, V, len(toks), None))
        got = out.to_numpy(np.float32, (len(toks), d))
        assert np.array_equal(got.view(np.uint32), deq[toks].view(np.uint32))


def test_mla_absorbed_parity(vb, oracle, dev):
    """The reference's absorbed-MLA block: analytic two-step case, then random shapes up to (1024, 512, 128)
    with the 1e-4 bound of tests/test_adversarial_step8_mla.rs:195-303."""
    lib = vb.load()
    for hidden, latent, steps in ((64, 32, 5), (576, 512, 6), (1024, 512, 128), (256, 64, 40)):
        max_s = steps + 2
        wn = oracle.fill_normal(hidden, 12, 1, 0.02, 1.0)
        wd = oracle.fill_normal(hidden * latent, 12, 2, 0.05)
        wq = oracle.fill_normal(hidden * latent, 12, 3, 0.05)
        wo = oracle.fill_normal(hidden * latent, 12, 4, 0.05)
        pool_ref = np.zeros(max_s * latent, dtype=np.float32)
        nbytes = int(lib.vb_op_scratch_bytes(1, latent, max_s, 1)) + 64 * 1024 + 32 * (latent + 2) * 4
        dwn, dwd, dwq, dwo = (dev.from_numpy(a) for a in (wn, wd, wq, wo))
        dpool, dscr, ddst = dev.from_numpy(pool_ref), dev(nbytes), dev(hidden * 4)
        for step in range(steps):
            x = oracle.fill_normal(hidden, 12, 100 + step, 1.0)
            want = np.zeros(hidden, dtype=np.float32)
            oracle.lib().vo_mla_absorbed_step_f32(P(want), P(x), P(wn), P(wd), P(wq), P(wo), P(pool_ref), step, hidden, latent, max_s, 1e-5)
            dx = dev.from_numpy(x)
            vb.check(lib.vb_op_mla_absorbed(ddst.ptr, dx.ptr, dwn.ptr, dwd.ptr, dwq.ptr, dwo.ptr, dpool.ptr, step, hidden, latent,
                                            max_s, 1e-5, dscr.ptr, nbytes, None))
            got = ddst.to_numpy(np.float32, (hidden,))
            assert np.max(np.abs(got - want)) < 1e-4, (hidden, latent, step)
        assert np.max(np.abs(dpool.to_numpy(np.float32, (max_s * latent,)) - pool_ref)) < 1e-4
