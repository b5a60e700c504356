"""Prompt-lookup speculative decoding: drafting and policy of the CPU checker (CPU), the CUDA engine's loop against
it (GPU).  Reference: src/runners/velox_cuda_runner_k2.cu:1572-1611 (draft), :2127-2311 (loop)."""
import numpy as np
import pytest

import helpers as H
from oracle import oracle as O
from velox_b200.modelspec import LLAMA3_8B_INT4, QWEN25_7B_INT8

SPEC = LLAMA3_8B_INT4.scaled(name="llama-int4-small", d_model=512, n_layers=2, n_q_heads=8, n_kv_heads=2, head_dim=64,
                             ffn_dim=1408, vocab=4096)


def test_prompt_lookup_draft_rules():
    # the last trigram (1,2,3) occurred at the start: what followed it, up to where the needle begins
    assert list(O.prompt_lookup_draft([1, 2, 3, 4, 1, 2, 3], 3)) == [4]
    assert list(O.prompt_lookup_draft([1, 2, 3, 4, 5, 6, 9, 1, 2, 3], 3)) == [4, 5, 6]
    assert list(O.prompt_lookup_draft([1, 2, 3, 4, 5, 6, 9, 1, 2, 3], 2)) == [4, 5]
    # the most recent earlier occurrence wins
    assert list(O.prompt_lookup_draft([7, 8, 1, 7, 8, 2, 5, 7, 8], 1)) == [2]
    # a unigram match drafts at most two tokens when more were asked for
    assert list(O.prompt_lookup_draft([5, 1, 2, 3, 4, 9, 5], 7)) == [1, 2]
    assert list(O.prompt_lookup_draft([5, 1, 2, 3, 4, 9, 5], 2)) == [1, 2]
    # nothing to copy: no earlier occurrence, or too short a history
    assert list(O.prompt_lookup_draft([1, 2, 3, 4], 3)) == []
    assert list(O.prompt_lookup_draft([1], 3)) == []
    # an occurrence that runs into the needle itself offers nothing
    assert list(O.prompt_lookup_draft([4, 4], 3)) == []


def test_checker_speculative_loop_equals_greedy():
    ora, _ = H.build_oracle(H.TINY, 4, 128)
    prompt = np.array([3, 9, 3, 9, 3, 9, 3, 9, 11, 3, 9], dtype=np.uint32)
    want = ora.generate_greedy(prompt, 40)
    ora2, _ = H.build_oracle(H.TINY, 4, 128)
    got, st = ora2.generate_speculative(prompt, 40, max_draft_len=4)
    assert np.array_equal(got, want)
    assert st.steps >= 1 and st.accepted <= st.drafted
    assert st.steps + st.accepted >= 39  # every pass yields one token plus its accepted drafts (the last may be cut short)


@pytest.mark.gpu
@pytest.mark.parametrize("spec,draft", [(SPEC, 3), (SPEC, 7), (QWEN25_7B_INT8.scaled(name="qwen-int8-tiled", d_model=512, n_layers=2, n_q_heads=8,
                                                                                     n_kv_heads=2, head_dim=64, ffn_dim=1408, vocab=4096), 4)],
                         ids=["int4-k3", "int4-k7", "int8-bias-k4"])
def test_engine_speculative_matches_checker(spec, draft):
    n_new = 64
    base = H.prompt_tokens(spec, 8, 12)
    prompt = np.concatenate([base, base[:7], base[2:9]]).astype(np.uint32)   # repeated n-grams: drafts are available at once
    ora, _ = H.build_oracle(spec, 8, 256)
    want = ora.generate_greedy(prompt, n_new)
    ora2, _ = H.build_oracle(spec, 8, 256)
    want_spec, want_st = ora2.generate_speculative(prompt, n_new, max_draft_len=draft)
    assert np.array_equal(want_spec, want)
    eng = H.build_engine(spec, 8, 256)
    got, st = eng.generate_speculative(prompt, n_new, max_draft_len=draft)
    assert np.array_equal(got, want), "speculative tokens differ from greedy decoding"
    assert (st.steps, st.plain_steps, st.drafted, st.accepted) == (want_st.steps, want_st.plain_steps, want_st.drafted, want_st.accepted)
    assert abs(st.ema_final - want_st.ema_final) < 1e-6 and st.ladder_final == want_st.ladder_final
    assert st.drafted > 0
    # the slot continues with plain decoding from where the loop stopped
    tok, pos, active, _ = eng.state_ex(0)
    assert (tok, pos, active) == (int(want[-1]), len(prompt) + n_new - 1, 1)
    eng.decode(4)
    more = eng.read_tokens(0, len(prompt) + n_new - 1, 4)
    ora3, _ = H.build_oracle(spec, 8, 256)
    assert np.array_equal(more, ora3.generate_greedy(prompt, n_new + 4)[-4:])
    eng.close()


@pytest.mark.gpu
def test_speculative_argument_checks():
    from velox_b200 import lib as L
    eng = H.build_engine(SPEC, 8, 64, max_batch=2)
    p = H.prompt_tokens(SPEC, 8, 8)
    eng.reserve(0, 20)
    out = np.zeros(32, dtype=np.uint32)
    with pytest.raises(L.VeloxError) as e:     # 32 reserved tokens (two blocks) do not hold prompt + new + draft rows
        L.check(eng._lib.vb_generate_speculative(eng.h, 0, p.ctypes.data_as(L.C.c_void_p), 8, 32, 3, 0.2, out.ctypes.data_as(L.C.c_void_p), None))
    assert e.value.code == L.ERR_INVALID
    eng.reserve(1, 32)
    eng.prefill(p, 1)
    with pytest.raises(L.VeloxError) as e:     # another slot is live
        eng.generate_speculative(p, 8)
    assert e.value.code == L.ERR_STATE
    eng.close()
