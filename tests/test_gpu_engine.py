"""End-to-end parity of the decode engine (C ABI) against the CPU checker on the same seed-generated
weights: stored tensors bit-exact, logits within 2e-2 max-abs, greedy tokens identical for 32 steps."""
import json
import os

import numpy as np
import pytest

import helpers as H
from velox_b200 import lib as L
from velox_b200.modelspec import ModelSpec, SMOLLM_135M, LLAMA3_8B_INT4, QWEN25_7B_INT8

pytestmark = pytest.mark.gpu

LOGIT_TOL = 2e-2  # the tolerance the task states for fp16/bf16 compute with fp32 accumulation

SMALL_SPECS = [
    H.TINY,
    SMOLLM_135M.scaled(name="smollm-narrow", n_layers=3, vocab=2048),
    LLAMA3_8B_INT4.scaled(name="llama-int4-small", d_model=512, n_layers=3, n_q_heads=8, n_kv_heads=2, head_dim=64, ffn_dim=1408, vocab=4096),
    LLAMA3_8B_INT4.scaled(name="llama-int4-2layer-fullwidth", n_layers=2, vocab=8192),
    QWEN25_7B_INT8.scaled(name="qwen-int8-small", d_model=448, n_layers=2, n_q_heads=7, n_kv_heads=1, head_dim=64, ffn_dim=1184, vocab=3008),
    LLAMA3_8B_INT4.scaled(name="llama-q4ref-small", d_model=512, n_layers=2, n_q_heads=8, n_kv_heads=2, head_dim=64, ffn_dim=1408, vocab=4096,
                          weight_fmt=L.FMT_Q4G64REF, head_fmt=L.FMT_Q4G64REF, embed_fmt=L.FMT_Q4G64REF, tied_lm_head=True),
    LLAMA3_8B_INT4.scaled(name="llama-bf16-small", d_model=256, n_layers=2, n_q_heads=4, n_kv_heads=4, head_dim=64, ffn_dim=512, vocab=1024,
                          weight_fmt=L.FMT_BF16, head_fmt=L.FMT_BF16, embed_fmt=L.FMT_BF16),
    # a GQA group of 8 with QKV bias (the tensor-core attention's full N = 8) and a 256-wide head
    LLAMA3_8B_INT4.scaled(name="gqa8-bias-int4-small", d_model=512, n_layers=2, n_q_heads=8, n_kv_heads=1, head_dim=64, ffn_dim=1408, vocab=4096,
                          qkv_bias=True),
    LLAMA3_8B_INT4.scaled(name="head256-int4-small", d_model=512, n_layers=2, n_q_heads=2, n_kv_heads=1, head_dim=256, ffn_dim=1408, vocab=4096),
    # int8 per-channel in shapes the integer tensor-core kernel tiles (K multiples of 128, rows of 16)
    QWEN25_7B_INT8.scaled(name="qwen-int8-tiled", d_model=512, n_layers=3, n_q_heads=8, n_kv_heads=2, head_dim=64, ffn_dim=1408, vocab=4096),
    # FFN rows so long that the multi-row integer kernel stages two rows of x per weight pass instead of four
    QWEN25_7B_INT8.scaled(name="qwen-int8-longk", d_model=512, n_layers=1, n_q_heads=8, n_kv_heads=2, head_dim=64, ffn_dim=18944, vocab=2048),
    LLAMA3_8B_INT4.scaled(name="llama-int4-longk", d_model=512, n_layers=1, n_q_heads=8, n_kv_heads=2, head_dim=64, ffn_dim=20480, vocab=2048),
]


def run_parity(spec: ModelSpec, seed: int, n_prompt: int, n_new: int, path: int, check_stored: bool = True):
    max_seq = n_prompt + n_new + 1
    ora, stored = H.build_oracle(spec, seed, max_seq)
    eng = H.build_engine(spec, seed, max_seq)
    eng.set_option("gemv_path", path)
    if check_stored:
        for (role, layer), (data, scales, fmt, rows, cols) in stored.items():
            if role == L.ROLE_LM_HEAD and spec.tied_lm_head:
                continue
            got_d, got_s = eng.export_tensor(role, layer, rows, cols)
            assert np.array_equal(got_d.reshape(-1).view(np.uint8), np.ascontiguousarray(data).reshape(-1).view(np.uint8)), (role, layer)
            if scales is not None:
                assert np.array_equal(got_s.reshape(-1), scales.reshape(-1)), (role, layer)
    prompt = H.prompt_tokens(spec, seed, n_prompt)
    want = ora.generate_greedy(prompt, n_new)
    want_logits = ora.logits
    got = eng.generate_greedy(prompt, n_new)
    got_logits = eng.logits()
    err = float(np.max(np.abs(got_logits - want_logits)))
    assert err <= LOGIT_TOL, "logits max-abs %g" % err
    assert np.array_equal(got, want), "greedy tokens differ: %s vs %s" % (got, want)
    assert int(np.argmax(got_logits)) == int(np.argmax(want_logits))
    eng.close()
    return err


@pytest.mark.parametrize("spec", SMALL_SPECS, ids=lambda s: s.name)
@pytest.mark.parametrize("path", [0, 1])
def test_small_models_match_checker(spec, path):
    run_parity(spec, seed=77, n_prompt=9, n_new=32, path=path)


def test_smollm_135m_full_model_matches_reference_fixture():
    """BASELINE config 1 shape, full depth, against the committed output of the reference's emitted C99."""
    g = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "smollm_ref_golden.json")))
    eng = H.build_engine(SMOLLM_135M, g["seed"], 64)
    n_new = len(g["tokens"])
    got = eng.generate_greedy(np.array(g["prompt"], dtype=np.uint32), n_new)
    assert [int(t) for t in got] == g["tokens"]
    lg = eng.logits()
    last = g["steps"][-1]
    for tid, val in zip(last["top5_ids"], last["top5_logits"]):
        assert abs(float(lg[tid]) - val) <= LOGIT_TOL
    assert int(np.argmax(lg)) == last["top5_ids"][0]
    eng.close()


def test_smollm_135m_prompt128_32_steps():
    """BASELINE config 1: 128-token prompt, first 32 greedy tokens and final logits against the checker."""
    err = run_parity(SMOLLM_135M, seed=2024, n_prompt=128, n_new=32, path=1, check_stored=False)
    assert err <= LOGIT_TOL


@pytest.mark.parametrize("g", [4, 7])
def test_decode_attention_tcgen05_form_matches_checker(g):
    """Option "attn_tcgen05": both attention products as tcgen05.mma (head_dim 128, tokens as the M dimension) over a context
    that takes several 128-token chunks per split, group sizes that fill and do not fill the eight head columns."""
    spec = LLAMA3_8B_INT4.scaled(name="hd128-g%d-int4-small" % g, d_model=512, n_layers=2, n_q_heads=g, n_kv_heads=1, head_dim=128,
                                 ffn_dim=1408, vocab=4096)
    n_prompt, n_new = 700, 10
    max_seq = n_prompt + n_new + 1
    ora, _ = H.build_oracle(spec, 41, max_seq)
    eng = H.build_engine(spec, 41, max_seq)
    eng.set_option("attn_tcgen05", 1)
    eng.set_option("attn_splits", 2)
    prompt = H.prompt_tokens(spec, 41, n_prompt)
    try:
        want = ora.generate_greedy(prompt, n_new)
        got = eng.generate_greedy(prompt, n_new)
        err = float(np.max(np.abs(eng.logits() - ora.logits)))
    finally:
        eng.set_option("attn_tcgen05", 0)
        eng.close()
    assert err <= LOGIT_TOL, "logits max-abs %g" % err
    assert np.array_equal(got, want)


@pytest.mark.parametrize("mma", [1, 0])
def test_long_context_crosses_chunk_refills(mma):
    """A context of ~1400 tokens: every split of the attention kernel walks more than two staged chunks (the
    refill path of its two K/V buffers), on the tensor-core and on the scalar variant."""
    spec = SMALL_SPECS[2]  # int4, 8 q / 2 kv heads, head_dim 64
    n_prompt, n_new = 1390, 12
    max_seq = n_prompt + n_new + 1
    ora, _ = H.build_oracle(spec, 31, max_seq)
    eng = H.build_engine(spec, 31, max_seq)
    eng.set_option("attn_mma", mma)
    prompt = H.prompt_tokens(spec, 31, n_prompt)
    want = ora.generate_greedy(prompt, n_new)
    got = eng.generate_greedy(prompt, n_new)
    err = float(np.max(np.abs(eng.logits() - ora.logits)))
    eng.set_option("attn_mma", 1)
    eng.close()
    assert err <= LOGIT_TOL, "logits max-abs %g" % err
    assert np.array_equal(got, want)


def test_eager_graph_and_stepwise_agree():
    """Graph replay, eager launches and host-driven forward_step produce identical tokens and logits."""
    spec = SMALL_SPECS[2]
    prompt = H.prompt_tokens(spec, 5, 7)
    outs = []
    for mode in ("graph", "eager", "step"):
        eng = H.build_engine(spec, 5, 64)
        if mode == "step":
            eng.reserve(0, 40)
            tok, toks = 0, []
            for p, t in enumerate(prompt):
                tok = eng.forward_step(int(t), p)
            toks.append(tok)
            for s in range(1, 12):
                tok = eng.forward_step(tok, len(prompt) + s - 1)
                toks.append(tok)
            outs.append((np.array(toks, dtype=np.uint32), eng.logits()))
        else:
            outs.append((eng.generate_greedy(prompt, 12, use_graph=(mode == "graph")), eng.logits()))
        eng.close()
    for t, lg in outs[1:]:
        assert np.array_equal(t, outs[0][0])
        assert np.array_equal(lg, outs[0][1])


def test_lean_weight_layout_is_bit_identical_and_smaller():
    """VB_FLAG_LEAN_WEIGHTS keeps one tile-major copy per int4 matrix: same tokens and logits, less memory,
    no canonical copy to export."""
    from velox_b200.engine import Engine
    spec = SMALL_SPECS[3]
    prompt = H.prompt_tokens(spec, 9, 6)
    full = H.build_engine(spec, 9, 48)
    lean = Engine(spec, max_seq_len=48, lean_weights=True)
    lean.load_synthetic(9)
    a, b = full.generate_greedy(prompt, 10), lean.generate_greedy(prompt, 10)
    assert np.array_equal(a, b) and np.array_equal(full.logits(), lean.logits())
    wf, wl = L.C.c_uint64(), L.C.c_uint64()
    L.load().vb_weight_bytes(full.h, L.C.byref(wf))
    L.load().vb_weight_bytes(lean.h, L.C.byref(wl))
    assert wl.value * 2 < wf.value
    with pytest.raises(L.VeloxError) as ei:
        lean.export_tensor(L.ROLE_WQ, 0, spec.qdim, spec.d_model)
    assert ei.value.code == L.ERR_STATE
    with pytest.raises(L.VeloxError):
        Engine(spec, max_seq_len=48, max_batch=2, lean_weights=True)
    full.close()
    lean.close()


@pytest.mark.parametrize("spec_i", [4, 2, 9, 10, 11])
def test_batched_variable_length_sequences(spec_i):
    """Several slots with different prompt lengths decode together; each matches its own CPU run.  Six slots are
    two weight passes of the multi-row integer kernel (four rows, then one active and one inactive row)."""
    spec = SMALL_SPECS[spec_i]
    seed, n_new = 31, 10
    lens = [5, 23, 16, 1, 9]
    max_seq = max(lens) + n_new + 1
    ora, _ = H.build_oracle(spec, seed, max_seq, n_seqs=len(lens))
    eng = H.build_engine(spec, seed, max_seq, max_batch=len(lens) + 1)  # one slot stays inactive
    prompts = [H.prompt_tokens(spec, seed, n, stream=(1 << 20) + i) for i, n in enumerate(lens)]
    for i, p in enumerate(prompts):
        eng.reserve(i, len(p) + n_new)
        eng.prefill(p, i)
    eng.build_graph()
    eng.decode(n_new - 1)
    for i, p in enumerate(prompts):
        want = ora.generate_greedy(p, n_new, seq=i)
        got = eng.read_tokens(i, len(p) - 1, n_new)
        assert np.array_equal(got, want), i
        assert float(np.max(np.abs(eng.logits(i) - ora.logits))) <= LOGIT_TOL
    eng.close()


@pytest.mark.parametrize("spec_i,i8", [(2, 1), (4, 1), (4, 0), (6, 1), (7, 1), (9, 1), (9, 0), (10, 1), (11, 1)])
def test_batched_decode_on_the_tensor_core_products(spec_i, i8):
    """Option decode_gemm: the decode steps of a batch (one row per slot, one slot inactive, lm_head included) run
    their products as tcgen05 GEMMs; every sequence still matches its own CPU run (int4, int8, bf16, QKV bias; the
    long-FFN shapes split the K of the down projection over 8 blocks per tile, the others over 1 or 2).  int8 per-channel
    weights take the integer tensor-core kernel that reads the stored bytes (i8 = 1) or, with decode_gemm_i8 = 0, the
    fp16 copies."""
    spec = SMALL_SPECS[spec_i]
    seed, n_new = 33, 10
    lens = [5, 23, 16, 1, 9]
    max_seq = max(lens) + n_new + 1
    ora, _ = H.build_oracle(spec, seed, max_seq, n_seqs=len(lens))
    eng = H.build_engine(spec, seed, max_seq, max_batch=len(lens) + 1)
    eng.set_option("decode_gemm_i8", i8)   # process-wide switch: set in every case
    eng.set_option("decode_gemm", 1)
    prompts = [H.prompt_tokens(spec, seed, n, stream=(1 << 20) + i) for i, n in enumerate(lens)]
    for i, p in enumerate(prompts):
        eng.reserve(i, len(p) + n_new)
        eng.prefill(p, i)
    eng.build_graph()
    eng.decode(n_new - 1)
    for i, p in enumerate(prompts):
        want = ora.generate_greedy(p, n_new, seq=i)
        assert np.array_equal(eng.read_tokens(i, len(p) - 1, n_new), want), i
        assert float(np.max(np.abs(eng.logits(i) - ora.logits))) <= LOGIT_TOL
    eng.set_option("decode_gemm_i8", 1)
    eng.close()


def test_lockstep_prefill_matches_the_checker():
    """All slots prefilled together, one step per prompt position (right-aligned), then decoded together."""
    spec = SMALL_SPECS[2]
    seed, n_new = 17, 8
    lens = [12, 7, 12]
    max_seq = max(lens) + n_new + 1
    ora, _ = H.build_oracle(spec, seed, max_seq, n_seqs=len(lens))
    eng = H.build_engine(spec, seed, max_seq, max_batch=len(lens))
    prompts = [H.prompt_tokens(spec, seed, n, stream=(1 << 20) + i) for i, n in enumerate(lens)]
    for i, p in enumerate(prompts):
        eng.reserve(i, len(p) + n_new)
    eng.prefill_lockstep(prompts)
    eng.build_graph()
    eng.decode(n_new - 1)
    for i, p in enumerate(prompts):
        want = ora.generate_greedy(p, n_new, seq=i)
        assert np.array_equal(eng.read_tokens(i, len(p) - 1, n_new), want), i
    eng.close()


@pytest.mark.parametrize("spec_i", [0, 2, 9])
def test_chunked_prefill_agrees_with_token_by_token(spec_i):
    """Prompt tokens sent through the layers 16 (or 5) at a time by the batched kernels, or in tensor-core chunks
    (one chunk of 70 rows; ragged chunks of 32, 32, 6), give the tokens of the one-by-one prefill, and logits within
    the path's tolerance (other summation order, fp16 operands in the tensor-core products)."""
    spec = SMALL_SPECS[spec_i]
    prompt = H.prompt_tokens(spec, 3, 71)
    outs = []
    for opts in ({"prefill_gemm": 0, "prefill_chunk": 1}, {"prefill_gemm": 0, "prefill_chunk": 16}, {"prefill_gemm": 0, "prefill_chunk": 5},
                 {"prefill_rows": 512}, {"prefill_rows": 32}, {"prefill_rows": 32, "prefill_flash": 0},
                 {"prefill_rows": 512, "prefill_two_per_sm": 1}, {"prefill_rows": 512, "prefill_wide": 1}):
        eng = H.build_engine(spec, 3, 96)
        for name in ("prefill_two_per_sm", "prefill_wide"):  # process-wide switches: set in every configuration
            eng.set_option(name, opts.get(name, 0))
        for name, value in opts.items():
            eng.set_option(name, value)
        outs.append((eng.generate_greedy(prompt, 10), eng.logits()))
        eng.close()
    for toks, lg in outs[1:]:
        assert np.array_equal(toks, outs[0][0])
        assert float(np.max(np.abs(lg - outs[0][1]))) <= LOGIT_TOL


@pytest.mark.parametrize("spec_i", [0, 1, 2, 3, 4, 5, 6, 7])
def test_tensor_core_prefill_matches_checker(spec_i):
    """A 150-token prompt prefilled in tensor-core chunks (128 + 21 rows; every weight format, QKV bias, head_dim 32 /
    64 / 128, i.e. with and without the causal tile attention kernel), then 32 greedy tokens: logits within 2e-2 of
    the CPU checker, tokens identical."""
    spec = SMALL_SPECS[spec_i]
    n_prompt, n_new = 150, 32
    ora, _ = H.build_oracle(spec, 21, n_prompt + n_new + 1)
    eng = H.build_engine(spec, 21, n_prompt + n_new + 1)
    eng.set_option("prefill_rows", 128)
    prompt = H.prompt_tokens(spec, 21, n_prompt)
    want = ora.generate_greedy(prompt, n_new)
    got = eng.generate_greedy(prompt, n_new)
    err = float(np.max(np.abs(eng.logits() - ora.logits)))
    assert err <= LOGIT_TOL, "logits max-abs %g" % err
    assert np.array_equal(got, want)
    eng.close()


def test_engine_argument_errors():
    spec = H.TINY
    eng = H.build_engine(spec, 1, 32)
    with pytest.raises(L.VeloxError):
        eng.reserve(0, 33)                      # beyond max_seq_len
    with pytest.raises(L.VeloxError):
        eng.reserve(3, 4)                       # slot out of range
    eng.reserve(0, 16)
    with pytest.raises(L.VeloxError):
        eng.prefill(np.zeros(17, dtype=np.uint32))   # beyond the reservation
    with pytest.raises(L.VeloxError):
        eng.prefill(np.array([spec.vocab], dtype=np.uint32))  # token out of range
    with pytest.raises(L.VeloxError):
        eng.prefill(np.zeros(0, dtype=np.uint32))    # empty prompt
    with pytest.raises(L.VeloxError):
        eng.set_state(0, 0, 16)                 # position outside the reservation
    with pytest.raises(L.VeloxError):
        eng.set_option("no_such_option", 1)
    from velox_b200.engine import Engine
    e2 = Engine(spec, 32)
    with pytest.raises(L.VeloxError) as ei:
        e2.decode(1)                            # weights not loaded
    assert ei.value.code == L.ERR_STATE
    e2.close()
    eng.close()


def test_kv_pool_exhaustion_and_reuse():
    spec = H.TINY
    from velox_b200.engine import Engine
    eng = Engine(spec, max_seq_len=64, max_batch=2, kv_blocks_total=5)
    eng.reserve(0, 64)           # 4 blocks
    with pytest.raises(L.VeloxError) as ei:
        eng.reserve(1, 48)       # 3 more: pool has 1
    assert ei.value.code == L.ERR_OOM
    eng.release(0)
    eng.reserve(1, 48)
    eng.close()
