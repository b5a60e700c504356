"""Nucleus sampling: the CPU checker against the reference's known answers (CPU), and the CUDA kernel against the
checker (GPU)."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O


def test_reference_known_answers():
    # src/runtime.rs:1559-1565
    logits = np.array([-1.0, 3.5, 2.1, 0.4], dtype=np.float32)
    assert O.sample_top_p(logits, 0.8, 0.9, 0.1)[0] == 1
    # tests/test_adversarial_runtime.rs:660-661, tests/test_runtime_e2e.rs:94: zero temperature / zero top_p = greedy
    lg = np.array([9.0, 1.0, 3.0], dtype=np.float32)
    assert O.sample_top_p(lg, 0.0, 0.9, 0.5)[0] == 0
    assert O.sample_top_p(lg, 0.8, 0.0, 0.5)[0] == 0
    assert O.sample_top_p(lg, 0.0, 0.9, 0.5, mode=1)[0] == 0


def test_nucleus_excludes_the_tail_and_follows_the_coin():
    # probabilities 0.5, 0.3, 0.15, 0.05 (temperature 1): top_p 0.8 keeps the first two; the coin walks them
    p = np.array([0.3, 0.05, 0.5, 0.15], dtype=np.float64)
    logits = np.log(p).astype(np.float32)
    assert O.sample_top_p(logits, 1.0, 0.8, 0.0)[0] == 2
    assert O.sample_top_p(logits, 1.0, 0.8, 0.6)[0] == 2      # target 0.48 of mass 0.8
    assert O.sample_top_p(logits, 1.0, 0.8, 0.7)[0] == 0      # target 0.56 > 0.5
    assert O.sample_top_p(logits, 1.0, 0.8, 0.9999)[0] == 0   # never index 3 or 1: outside the nucleus
    # the emitted C99 twin walks index order: cumulative 0.3, 0.35, 0.85, 1.0 against coin * top_p
    assert O.sample_top_p(logits, 1.0, 0.8, 0.3, mode=1)[0] == 0    # 0.24
    assert O.sample_top_p(logits, 1.0, 0.8, 0.42, mode=1)[0] == 1   # 0.336
    assert O.sample_top_p(logits, 1.0, 0.8, 0.5, mode=1)[0] == 2    # 0.40
    # equal probabilities rank by index
    flat = np.zeros(8, dtype=np.float32)
    assert O.sample_top_p(flat, 1.0, 0.5, 0.0)[0] == 0
    assert O.sample_top_p(flat, 1.0, 0.5, 0.9)[0] == 3              # nucleus = first 4, target 0.45 -> fourth


def test_coin_is_a_pure_function_of_seed_slot_position():
    a = [O.sample_coin(7, s, p) for s in range(3) for p in range(50)]
    assert a == [O.sample_coin(7, s, p) for s in range(3) for p in range(50)]
    assert all(0.0 <= c < 1.0 for c in a) and len(set(a)) > 140
    assert abs(np.mean([O.sample_coin(1, 0, p) for p in range(4000)]) - 0.5) < 0.03


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [0, 1])
def test_cuda_sampler_matches_checker(vb, mode):
    from velox_b200.engine import DeviceBuffer
    lib = vb.load()
    rng = np.random.default_rng(5 + mode)
    n_checked = n_close = 0
    for n in (4, 257, 4096, 50000, 128256):
        for trial in range(6):
            kind = trial % 3
            if kind == 0:
                logits = rng.normal(0, 2.0, n).astype(np.float32)            # a few dominant tokens
            elif kind == 1:
                logits = rng.normal(0, 0.05, n).astype(np.float32)           # near uniform: a nucleus of most of the row
            else:
                logits = np.round(rng.normal(0, 1.0, n)).astype(np.float32)  # many exact ties
            d_logits = DeviceBuffer.from_numpy(logits)
            d_scratch = DeviceBuffer(n * 4)
            d_out = DeviceBuffer(4)
            for temperature, top_p in ((0.8, 0.9), (1.3, 0.5), (1.0, 1.0), (0.0, 0.9), (0.7, 0.0)):
                for coin in (0.0, float(rng.random()), float(rng.random()), 0.99995):
                    want, margin = O.sample_top_p(logits, temperature, top_p, coin, mode)
                    vb.check(lib.vb_op_sample_top_p(d_out.ptr, d_logits.ptr, n, temperature, top_p, coin, mode, d_scratch.ptr, n * 4, None))
                    vb.check(lib.vb_dev_sync())
                    got = int(d_out.to_numpy(np.uint32, (1,))[0])
                    n_checked += 1
                    if got != want:
                        # only a decision within rounding of its threshold may differ: the reference sums the row
                        # sequentially in fp32 (error growing with the row length), the kernel in a fixed tree
                        assert margin < 2e-5 + 4e-9 * n, (n, trial, temperature, top_p, coin, got, want, margin)
                        n_close += 1
            for b in (d_logits, d_scratch, d_out):
                b.free()
    # near-uniform rows make every decision a close one (consecutive running sums differ by ~1/n): those may go to the
    # neighbouring token; anything else must agree, so the share of differences stays small
    assert n_close <= n_checked // 8, "%d of %d decisions differed" % (n_close, n_checked)


@pytest.mark.gpu
def test_engine_sampling_is_reproducible_and_matches_checker_coins():
    """The engine's sampler draws coin(seed, slot, position): two runs agree, and every sampled token is the checker's
    choice for the engine's own logits at that step."""
    import helpers as H
    from velox_b200.modelspec import LLAMA3_8B_INT4
    spec = LLAMA3_8B_INT4.scaled(name="llama-int4-small", d_model=512, n_layers=2, n_q_heads=8, n_kv_heads=2, head_dim=64,
                                 ffn_dim=1408, vocab=4096)
    prompt = H.prompt_tokens(spec, 3, 12)
    runs = []
    for _ in range(2):
        eng = H.build_engine(spec, 3, 64)
        eng.set_sampling(0.9, 0.95, seed=1234)
        eng.reserve(0, 64)
        eng.prefill(prompt, 0)
        toks, close = [int(eng.read_tokens(0, len(prompt) - 1, 1)[0])], 0
        for s in range(16):
            pos = len(prompt) + s
            eng.decode(1)
            tok = int(eng.read_tokens(0, pos, 1)[0])
            want, margin = O.sample_top_p(eng.logits(), 0.9, 0.95, O.sample_coin(1234, 0, pos))
            if tok != want:
                assert margin < 2e-5
                close += 1
            toks.append(tok)
        assert close <= 1
        runs.append(toks)
        eng.close()
    assert runs[0] == runs[1]
    assert len(set(runs[0])) > 4   # it does sample: greedy decoding of this model repeats far more


def test_c99_walk_twin_equals_the_compiled_reference_function():
    """The emitted C model's own velox_c99_sample_top_p_f32 (compiled in place from the reference file) against the
    restated walk, token for token, over rows of several lengths, temperatures, nucleus sizes and coins."""
    R = O.ref_lib()
    if R is None or not hasattr(R, "refsm_sample_top_p"):
        pytest.skip("compiled reference not present")
    rng = np.random.default_rng(77)
    for n in (5, 64, 1000, 49152):
        for trial in range(6):
            logits = (rng.standard_normal(n) * (0.5 + trial)).astype(np.float32)
            for temperature, top_p in ((0.8, 0.9), (1.3, 0.5), (1.0, 1.0), (0.0, 0.9), (0.7, 0.0), (1e-6, 0.5)):
                for coin in (0.0, 0.17, 0.5, 0.93, 0.99999):
                    want = R.refsm_sample_top_p(logits.ctypes.data, n, temperature, top_p, coin)
                    got, _ = O.sample_top_p(logits, temperature, top_p, coin, mode=1)
                    assert got == want, (n, trial, temperature, top_p, coin)
