"""Parity at the sizes the benchmark runs: the model shapes of the benchmark configurations at their own width (and,
for the 8B model, their own depth and vocabulary) against the CPU checker.  The checker costs ~0.75 s per 8B token on
16 cores, so prompts are short where the whole depth is run and the depth is cut where the prompt is long."""
import time

import numpy as np
import pytest

import helpers as H
from velox_b200.modelspec import LLAMA3_8B_INT4, QWEN25_7B_INT8, QWEN2_72B_INT4

pytestmark = pytest.mark.gpu
LOGIT_TOL = 2e-2  # max-abs on the logits; greedy tokens must agree for the first 32 steps


def test_llama3_8b_int4_full_model_32_steps():
    """Llama-3-8B shape, int4 g32, all 32 layers, vocabulary 128256: a 16-token prompt and 32 greedy steps, both engines fed
    the checker's token at every position (so that one near-tie cannot hide the steps after it): logits within the budget
    at every position; the greedy token equal wherever the checker's own top-two margin exceeds twice the budget (seeded
    N(0, 0.02) weights give nearly flat logits: margins below the budget do occur, and there either winner is right)."""
    spec, n_prompt, n_new = LLAMA3_8B_INT4, 16, 32
    t0 = time.time()
    ora, _ = H.build_oracle(spec, 2025, n_prompt + n_new + 1)
    eng = H.build_engine(spec, 2025, n_prompt + n_new + 16)
    eng.reserve(0, n_prompt + n_new + 16)
    prompt = H.prompt_tokens(spec, 2025, n_prompt)
    worst, near_ties, tok = 0.0, 0, None
    for pos in range(n_prompt + n_new):
        t = int(prompt[pos]) if pos < n_prompt else tok
        tok = ora.forward_step(t, pos)
        got = eng.forward_step(t, pos)
        lo = ora.logits
        worst = max(worst, float(np.max(np.abs(eng.logits() - lo))))
        if got != tok:
            top2 = np.partition(lo, -2)[-2:]
            assert float(top2[1] - top2[0]) < 2 * LOGIT_TOL, "position %d: token %d vs %d with a margin of %g" % (pos, got, tok, float(top2[1] - top2[0]))
            near_ties += 1
    eng.close()
    print("8B full depth: logits max-abs %.3g over %d positions, %d near-tie(s), %.0f s" % (worst, n_prompt + n_new, near_ties, time.time() - t0))
    assert worst <= LOGIT_TOL
    assert near_ties <= 3


def test_llama3_8b_long_prompt_through_the_tensor_core_prefill():
    """A 512-token prompt through the tcgen05 prefill (chunk rows rounded to fp16 for the products) at full width,
    6 layers: last-token logits and 8 more greedy tokens against the checker."""
    spec = LLAMA3_8B_INT4.scaled(name="llama3-8b-int4-6layers", n_layers=6)
    n_prompt, n_new = 512, 8
    ora, _ = H.build_oracle(spec, 7, n_prompt + n_new + 1)
    prompt = H.prompt_tokens(spec, 7, n_prompt)
    want = ora.generate_greedy(prompt, n_new)
    eng = H.build_engine(spec, 7, n_prompt + n_new + 16)
    got = eng.generate_greedy(prompt, n_new)
    err = float(np.max(np.abs(eng.logits() - ora.logits)))
    eng.close()
    print("8B width, 6 layers, 512-token tensor-core prefill: logits max-abs %.3g" % err)
    assert err <= LOGIT_TOL
    assert np.array_equal(got, want)


def test_llama3_8b_full_depth_prefill_paths_agree_at_2048_rows():
    """Full depth, 2048-token prompt: the tensor-core prefill (one chunk of 2047 rows) against the same engine's batched
    integer kernels (prefill_gemm = 0, which match the checker to ~3e-4): last-token logits within the budget, same
    first tokens.  What this bounds is the fp16 rounding of x and of the dequantized weights in the tensor-core products
    reaching the logits through the cached K/V of 2047 positions and 32 layers."""
    spec, n_prompt, n_new = LLAMA3_8B_INT4, 2048, 8
    prompt = H.prompt_tokens(spec, 11, n_prompt)
    outs = []
    for gemm in (1, 0):
        eng = H.build_engine(spec, 11, n_prompt + n_new + 16)
        eng.set_option("prefill_gemm", gemm)
        eng.reserve(0, n_prompt + n_new + 16)
        eng.prefill(prompt, 0)
        first = eng.logits().copy()
        eng.decode(n_new - 1)
        outs.append((first, eng.read_tokens(0, n_prompt - 1, n_new), eng.logits().copy()))
        eng.close()
    d0 = float(np.max(np.abs(outs[0][0] - outs[1][0])))
    d1 = float(np.max(np.abs(outs[0][2] - outs[1][2])))
    print("8B full depth, 2048-row tensor-core prefill vs batched kernels: last-prompt logits max-abs %.3g, after %d steps %.3g" % (d0, n_new - 1, d1))
    assert d0 <= LOGIT_TOL and d1 <= LOGIT_TOL
    assert np.array_equal(outs[0][1], outs[1][1])


def test_qwen25_7b_int8_batch32_paged_long_prompts():
    """Qwen2.5-7B shape at full width (28 q / 4 kv heads, d 3584, FFN 18944, QKV bias), int8 per channel, 2 layers,
    batch 32, prompt lengths uniform in [256, 2048] on 16-token pages, decode products on the tensor-core GEMMs:
    every slot against a single-sequence run of the exact fp32 kernels, the three shortest also against the checker."""
    spec = QWEN25_7B_INT8.scaled(name="qwen2.5-7b-int8-2layers", n_layers=2, vocab=8192)
    n_new, B = 8, 32
    lens = [int(x) for x in np.random.default_rng(31).integers(256, 2049, size=B)]
    prompts = [H.prompt_tokens(spec, 31, lens[s], stream=5000 + s) for s in range(B)]
    max_seq = max(lens) + n_new + 16
    eng = H.build_engine(spec, 31, max_seq, max_batch=B)
    for s in range(B):
        eng.reserve(s, lens[s] + n_new + 8)
        eng.prefill(prompts[s], s)
    eng.build_graph()
    eng.decode(n_new - 1)
    got = [eng.read_tokens(s, lens[s] - 1, n_new) for s in range(B)]
    got_logits = [eng.logits(s) for s in range(B)]
    eng.close()
    one = H.build_engine(spec, 31, max_seq, max_batch=1)
    one.set_option("gemv_path", 0)       # exact fp32 kernels, token by token
    one.set_option("prefill_gemm", 0)
    worst = 0.0
    for s in range(B):
        one.reserve(0, lens[s] + n_new + 8)
        one.prefill(prompts[s], 0)
        one.decode(n_new - 1)
        assert np.array_equal(got[s], one.read_tokens(0, lens[s] - 1, n_new)), "slot %d (prompt %d)" % (s, lens[s])
        worst = max(worst, float(np.max(np.abs(got_logits[s] - one.logits(0)))))
        one.release(0)
    one.close()
    print("Qwen2.5-7B width, batch 32: logits max-abs vs exact single-sequence kernels %.3g" % worst)
    assert worst <= LOGIT_TOL
    for s in sorted(range(B), key=lambda i: lens[i])[:3]:
        ora, _ = H.build_oracle(spec, 31, lens[s] + n_new + 1)
        want = ora.generate_greedy(prompts[s], n_new)
        assert np.array_equal(got[s], want), "slot %d vs checker" % s
        assert float(np.max(np.abs(got_logits[s] - ora.logits))) <= LOGIT_TOL
        ora.close()


def test_qwen2_72b_int4_full_width_two_layers():
    """Qwen2-72B shape at full width (d 8192, 64 q / 8 kv heads, FFN 29568, QKV bias, vocabulary 152064), int4 g32,
    2 layers, unsharded, both weight layouts (the lean one is what the tensor-parallel ranks and the TP-1 baseline use)."""
    spec = QWEN2_72B_INT4.scaled(name="qwen2-72b-int4-2layers", n_layers=2)
    n_prompt, n_new = 16, 32
    ora, _ = H.build_oracle(spec, 72, n_prompt + n_new + 1)
    prompt = H.prompt_tokens(spec, 72, n_prompt)
    want = ora.generate_greedy(prompt, n_new)
    from velox_b200.engine import Engine
    for lean in (False, True):
        eng = Engine(spec, max_seq_len=n_prompt + n_new + 16, lean_weights=lean)
        eng.load_synthetic(72)
        got = eng.generate_greedy(prompt, n_new)
        err = float(np.max(np.abs(eng.logits() - ora.logits)))
        eng.close()
        print("72B width, 2 layers, lean=%s: logits max-abs %.3g" % (lean, err))
        assert err <= LOGIT_TOL
        assert np.array_equal(got, want)
