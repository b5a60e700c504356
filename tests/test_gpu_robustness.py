"""Engine behaviour at the edges of its contracts: a slot never leaves its KV reservation, reloaded weights
reach every code path that keeps a derived copy."""
import numpy as np
import pytest

import helpers as H
from oracle import oracle as O
from velox_b200 import lib as L
from velox_b200.modelspec import LLAMA3_8B_INT4, QWEN25_7B_INT8, stream_of

pytestmark = pytest.mark.gpu

LOGIT_TOL = 2e-2
SPEC = LLAMA3_8B_INT4.scaled(name="llama-int4-small", d_model=512, n_layers=2, n_q_heads=8, n_kv_heads=2, head_dim=64,
                             ffn_dim=1408, vocab=4096)


def test_decode_past_the_reservation_is_refused_on_the_host():
    eng = H.build_engine(SPEC, 3, 128)
    eng.reserve(0, 32)
    eng.prefill(H.prompt_tokens(SPEC, 3, 29), 0)
    eng.decode(3)                      # positions 29, 30, 31: the last rows of the reservation
    with pytest.raises(L.VeloxError) as e:
        eng.decode(1)
    assert e.value.code == L.ERR_STATE and "reservation" in str(e.value)
    with pytest.raises(L.VeloxError) as e:
        L.check(eng._lib.vb_decode_step(eng.h))
    assert e.value.code == L.ERR_STATE
    tok, pos, active, limit = eng.state_ex(0)
    assert (pos, active, limit) == (32, 0, 32)   # the sampler itself retired the slot
    eng.reserve(0, 48)                 # a larger reservation re-opens it
    eng.set_state(0, tok, pos, True)
    eng.decode(4)
    assert eng.state_ex(0)[1:] == (36, 1, 48)
    eng.close()


def test_exhausted_slot_goes_inactive_and_neighbours_are_untouched():
    """Two slots; slot 0 fills its reservation and is retired by the device-side sampler, slot 1 keeps decoding
    and must produce exactly the tokens of a run of its own (its KV blocks were never written by slot 0)."""
    n_new = 12
    p0, p1 = H.prompt_tokens(SPEC, 9, 15), H.prompt_tokens(SPEC, 9, 20, stream=77)
    ora, _ = H.build_oracle(SPEC, 9, 64)
    want = ora.generate_greedy(p1, n_new)
    eng = H.build_engine(SPEC, 9, 64, max_batch=2)
    eng.reserve(0, 16)
    eng.reserve(1, 64)
    eng.prefill(p0, 0)
    eng.prefill(p1, 1)
    eng.decode(1)                      # slot 0 writes its last row (position 15) and goes inactive
    assert eng.state_ex(0)[1:] == (16, 0, 16)
    with pytest.raises(L.VeloxError):  # the host still counts slot 0 as live: refuse rather than guess
        eng.decode(1)
    eng.release(0)
    eng.decode(n_new - 2)
    got = eng.read_tokens(1, len(p1) - 1, n_new)
    assert np.array_equal(got, want)
    eng.close()


@pytest.mark.parametrize("spec", [SPEC, QWEN25_7B_INT8.scaled(name="qwen-int8-tiled", d_model=512, n_layers=2, n_q_heads=8, n_kv_heads=2,
                                                                 head_dim=64, ffn_dim=1408, vocab=4096)], ids=lambda s: s.name)
def test_reloaded_tensor_reaches_the_tensor_core_copies(spec):
    """The tensor-core products read resident fp16 copies made on first use: a matrix loaded again afterwards must
    refresh them (Wk shares the fused QKV copy that hangs off Wq)."""
    n_prompt = 64
    eng = H.build_engine(spec, 21, n_prompt + 4)
    prompt = H.prompt_tokens(spec, 21, n_prompt)
    eng.reserve(0, n_prompt + 4)
    eng.prefill(prompt, 0)             # > 48 tokens: chunk rows go through the tensor-core GEMMs, copies are made
    ora, _ = H.build_oracle(spec, 21, n_prompt + 4)
    for role, rows, cols in ((L.ROLE_WK, spec.kvdim, spec.d_model), (L.ROLE_WDOWN, spec.d_model, spec.ffn_dim)):
        w = O.fill_normal(rows * cols, 4242, stream_of(role, 1), 0.02, 0.0).reshape(rows, cols)
        eng.load_tensor(role, 1, w)
        data, scales = O.quantize(w, spec.storage_fmt(role))
        ora.set_tensor(role, 1, data, scales, spec.storage_fmt(role))
    eng.prefill(prompt, 0)
    want = ora.generate_greedy(prompt, 1)
    got = eng.read_tokens(0, n_prompt - 1, 1)
    err = float(np.max(np.abs(eng.logits() - ora.logits)))
    assert err <= LOGIT_TOL, "logits max-abs %g after a reload" % err
    assert np.array_equal(got, want)
    eng.close()
