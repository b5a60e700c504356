"""Multi-head latent attention (MLA) decode: the checker's absorbed form against its explicit form (CPU; the identity
the reference pins in src/optimizer.rs:544-585 and tests/test_adversarial_step8_mla.rs), the CUDA decode kernel and
the block built from the library's ops against the checker (GPU)."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O

DC, DR = 512, 64


def P(a):
    return a.ctypes.data_as(C.c_void_p)


def test_absorbed_equals_explicit():
    rng = np.random.default_rng(3)
    blk = O.MlaBlockWeights(rng, d_model=256, n_heads=6, q_lora=96, std=0.06)
    max_seq = 24
    ca, ce = np.zeros((max_seq, DC + DR), np.float32), np.zeros((max_seq, DC + DR), np.float32)
    x = rng.standard_normal(256).astype(np.float32)
    for pos in range(max_seq):
        ya, q_cat, ctx = blk.step(x, ca, pos, absorbed=True)
        ye = blk.step(x, ce, pos, absorbed=False)
        assert np.array_equal(ca[:pos + 1], ce[:pos + 1])                      # same cache rows
        assert np.max(np.abs(ya - ye)) <= 1e-4 * max(1.0, float(np.max(np.abs(ye))))
        # the attention core alone reproduces the block's latent context
        core = O.mla_core(q_cat, ca[:pos + 1], DC, 1.0 / np.sqrt(128 + 64))
        assert np.max(np.abs(core - ctx)) <= 1e-6
        x = (ya / np.max(np.abs(ya))).astype(np.float32)
    # position 0: one row, softmax weight 1 -> the context is the row itself for every head
    y0, q0, ctx0 = blk.step(x, np.zeros((4, DC + DR), np.float32), 0)
    assert ctx0.shape == (6, DC) and np.max(np.abs(ctx0 - ctx0[0])) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("path", [1, 0], ids=["tcgen05", "mma_sync"])
@pytest.mark.parametrize("n_heads,split", [(128, 1024), (128, 256), (40, 1024), (16, 64), (160, 512)])
def test_cuda_mla_decode_matches_checker(vb, n_heads, split, path):
    from velox_b200.engine import DeviceBuffer as dev
    lib = vb.load()
    vb.check(lib.vb_op_mla_set_path(path))
    rng = np.random.default_rng(n_heads + split)
    lens = [1, 31, 32, 33, 700, 1024, 1025, 2500] if n_heads == 128 and split == 1024 else [5, 64, 65, 900]
    B, max_ctx = len(lens), max(lens)
    stride = max_ctx + 7
    scale = 1.0 / np.sqrt(192.0)
    q = rng.standard_normal((B, n_heads, DC + DR)).astype(np.float32)
    cache = O.bf16_round(rng.standard_normal((B, stride, DC + DR)).astype(np.float32))
    # rows past a sequence's context must not matter, whatever they hold
    for b, n in enumerate(lens):
        cache[b, n:] = 1e30
    d_q, d_cache = dev.from_numpy(q), dev.from_numpy(O.to_bf16_bits(cache))
    d_len = dev.from_numpy(np.array(lens, np.uint32))
    need = lib.vb_op_mla_decode_scratch_bytes(B, n_heads, max_ctx, split)
    d_scratch, d_out = dev(need), dev(B * n_heads * DC * 4)
    vb.check(lib.vb_op_mla_decode(d_out.ptr, d_q.ptr, d_cache.ptr, d_len.ptr, B, n_heads, max_ctx, stride, scale, split, d_scratch.ptr, need, None))
    vb.check(lib.vb_dev_sync())
    got = d_out.to_numpy(np.float32, (B, n_heads, DC))
    assert np.all(np.isfinite(got))
    for b, n in enumerate(lens):
        want = O.mla_core(q[b], cache[b, :n], DC, scale)
        err = float(np.max(np.abs(got[b] - want)))
        assert err <= 1e-2 * max(1.0, float(np.max(np.abs(want)))), (b, n, err)
    # one row: every head returns that row (softmax weight 1), exactly up to bf16 -> fp32 products
    assert np.max(np.abs(got[0] - cache[0, 0, :DC])) <= 1e-6 if lens[0] == 1 else True
    assert lib.vb_op_mla_decode(d_out.ptr, d_q.ptr, d_cache.ptr, d_len.ptr, B, n_heads, max_ctx, stride, scale, 48, d_scratch.ptr, need, None) == vb.ERR_INVALID
    vb.check(lib.vb_op_mla_set_path(1))


@pytest.mark.gpu
def test_mla_block_from_library_ops_matches_checker(vb):
    """The whole block of examples/deepseek_v3_mla.vlx:117-150 composed from the C-ABI ops (bf16 weights, bf16 latent cache,
    batch of 3 sequences at different positions) against the checker's absorbed form with a bf16-rounded cache."""
    from velox_b200.engine import DeviceBuffer as dev
    lib = vb.load()
    rng = np.random.default_rng(8)
    d, H, ql, dn, dv = 512, 16, 128, 128, 128
    blk = O.MlaBlockWeights(rng, d_model=d, n_heads=H, q_lora=ql, std=0.05)
    W = {n: dev.from_numpy(O.to_bf16_bits(blk.w[n])) for n in blk.NAMES if n != "w_norm"}
    d_norm = dev.from_numpy(blk.w["w_norm"])
    B, max_seq = 3, 80
    caches = [np.zeros((max_seq, DC + DR), np.float32) for _ in range(B)]
    d_cache = dev.from_numpy(np.zeros((B, max_seq, DC + DR), np.uint16))
    xs = [rng.standard_normal(d).astype(np.float32) for _ in range(B)]
    start = [0, 7, 30]
    # sequences 1 and 2 begin with some history written by the checker and uploaded as bf16
    for b in range(B):
        for pos in range(start[b]):
            y, _, _ = blk.step(xs[b], caches[b], pos, cache_bf16=True)
            xs[b] = (y / np.max(np.abs(y))).astype(np.float32)
    hist = np.stack(caches)
    vb.check(lib.vb_dev_upload(d_cache.ptr, P(O.to_bf16_bits(hist)), hist.size * 2))
    bufs = {k: dev(B * n * 4) for k, n in (("x", d), ("nx", d), ("cq", ql), ("row", DC + DR), ("qn", H * dn), ("qr", H * DR), ("qcat", H * (DC + DR)),
                                           ("ctx", H * DC), ("o", H * dv), ("y", d))}
    d_pos, d_len = dev(B * 4), dev(B * 4)
    need = lib.vb_op_mla_decode_scratch_bytes(B, H, max_seq, 32)
    d_scratch = dev(need)
    for step in range(12):
        pos = [start[b] + step for b in range(B)]
        vb.check(lib.vb_dev_upload(bufs["x"].ptr, P(np.stack(xs)), B * d * 4))
        vb.check(lib.vb_dev_upload(d_pos.ptr, P(np.array(pos, np.uint32)), B * 4))
        vb.check(lib.vb_dev_upload(d_len.ptr, P(np.array([p + 1 for p in pos], np.uint32)), B * 4))
        vb.check(lib.vb_op_rmsnorm(bufs["nx"].ptr, bufs["x"].ptr, d_norm.ptr, vb.FMT_F32, d, B, blk.c.eps, None))
        for dst, w, rows, col0, width in (("row", "w_dkv", DC, 0, DC + DR), ("row", "w_kr", DR, DC, DC + DR), ("cq", "w_dq", ql, 0, ql)):
            # products whose rows land inside a wider row go sequence by sequence (vb_op_matmul writes dense rows)
            for b in range(B):
                vb.check(lib.vb_op_matmul(bufs[dst].ptr.value + (b * width + col0) * 4, bufs["nx"].ptr.value + b * d * 4, W[w].ptr, None, vb.FMT_BF16, d, rows, 1, None))
        vb.check(lib.vb_op_matmul(bufs["qn"].ptr, bufs["cq"].ptr, W["w_uq"].ptr, None, vb.FMT_BF16, ql, H * dn, B, None))
        vb.check(lib.vb_op_matmul(bufs["qr"].ptr, bufs["cq"].ptr, W["w_qr"].ptr, None, vb.FMT_BF16, ql, H * DR, B, None))
        for b in range(B):   # rotary part of the key row and of the queries, at each sequence's own position
            vb.check(lib.vb_op_rope(bufs["row"].ptr.value + (b * (DC + DR) + DC) * 4, 1, DR, pos[b], blk.c.theta, None))
            vb.check(lib.vb_op_rope(bufs["qr"].ptr.value + b * H * DR * 4, H, DR, pos[b], blk.c.theta, None))
        vb.check(lib.vb_op_mla_latent_append(d_cache.ptr, bufs["row"].ptr, d_pos.ptr, B, max_seq, None))
        # q_cat = [q_nope . W_uk_h | q_rope] per head
        vb.check(lib.vb_op_mla_head_product(bufs["ctx"].ptr, bufs["qn"].ptr, W["w_uk"].ptr, H, dn, DC, B, 0, None))
        vb.check(lib.vb_dev_sync())
        qa = bufs["ctx"].to_numpy(np.float32, (B, H, DC))
        qr = bufs["qr"].to_numpy(np.float32, (B, H, DR))
        vb.check(lib.vb_dev_upload(bufs["qcat"].ptr, P(np.ascontiguousarray(np.concatenate([qa, qr], axis=2))), B * H * (DC + DR) * 4))
        vb.check(lib.vb_op_mla_decode(bufs["ctx"].ptr, bufs["qcat"].ptr, d_cache.ptr, d_len.ptr, B, H, max_seq, max_seq, 1.0 / np.sqrt(dn + DR), 32,
                                      d_scratch.ptr, need, None))
        vb.check(lib.vb_op_mla_head_product(bufs["o"].ptr, bufs["ctx"].ptr, W["w_uv"].ptr, H, DC, dv, B, 1, None))
        vb.check(lib.vb_op_matmul(bufs["y"].ptr, bufs["o"].ptr, W["w_o"].ptr, None, vb.FMT_BF16, H * dv, d, B, None))
        vb.check(lib.vb_dev_sync())
        y = bufs["y"].to_numpy(np.float32, (B, d))
        for b in range(B):
            want, _, want_ctx = blk.step(xs[b], caches[b], pos[b], cache_bf16=True)
            got = xs[b] + y[b]
            assert np.max(np.abs(got - want)) <= 2e-2, (step, b, float(np.max(np.abs(got - want))))
            xs[b] = (want / np.max(np.abs(want))).astype(np.float32)
    got_cache = d_cache.to_numpy(np.uint16, (B, max_seq, DC + DR))
    for b in range(B):
        n = start[b] + 12
        diff = np.abs((got_cache[b, :n].astype(np.uint32) << 16).view(np.float32) - caches[b][:n])
        assert np.max(diff) <= 2e-2 * max(1.0, float(np.max(np.abs(caches[b][:n]))))   # a bf16 ulp where fp32 sums differ in the last bit
