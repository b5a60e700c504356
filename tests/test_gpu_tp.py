"""Tensor-parallel decode on 2 GPUs against the unsharded engine and the CPU checker (skipped on one GPU).

The ranks run as child processes (one per GPU, torch.distributed.run); NVLS is switched off for them so a
rank that exits early cannot leave multicast bindings behind.
"""
from __future__ import annotations

import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import build_engine, build_oracle, prompt_tokens
from tp_worker import TP_SPEC
from velox_b200 import lib as L
from velox_b200.modelspec import shard_plan

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SEED, N_PROMPT, N_NEW = 11, 24, 32  # 32 steps: the logits compared below are those of step 32


def _gpu_count() -> int:
    n = L.C.c_int32(0)
    L.load().vb_device_count(L.C.byref(n))
    return n.value


def _run_group(tmp_path, world: int, extra=()):
    np.save(os.path.join(str(tmp_path), "prompt.npy"), prompt_tokens(TP_SPEC, SEED, N_PROMPT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29633", os.path.join(ROOT, "tests", "tp_worker.py"), "--out", str(tmp_path), "--seed", str(SEED),
           "--prompt", str(N_PROMPT), "--new", str(N_NEW), *extra]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=420)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return [np.load(os.path.join(str(tmp_path), f"rank{k}.npz")) for k in range(world)]


@pytest.mark.parametrize("exchange", ["p2p", "p2p-fused", "nccl"])
@pytest.mark.parametrize("graph", [True, False])
def test_tp2_matches_unsharded_and_checker(tmp_path, graph, exchange):
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    extra = ("--exchange", "p2p", "--fused-push", "1") if exchange == "p2p-fused" else ("--exchange", exchange, "--fused-push", "0")
    ranks = _run_group(tmp_path, 2, extra + (() if graph else ("--no-graph",)))
    prompt = prompt_tokens(TP_SPEC, SEED, N_PROMPT)
    # unsharded engine on this process's GPU
    eng = build_engine(TP_SPEC, SEED, N_PROMPT + N_NEW + 8)
    ref_tokens = eng.generate_greedy(prompt, N_NEW, use_graph=graph)
    ref_logits = eng.logits()
    # every rank reports the same tokens; they are the unsharded engine's
    for r in ranks:
        assert np.array_equal(r["tokens"], ranks[0]["tokens"])
    assert np.array_equal(ranks[0]["tokens"], ref_tokens)
    tp_logits = np.concatenate([r["logits"] for r in ranks])
    assert tp_logits.shape == ref_logits.shape
    assert np.max(np.abs(tp_logits - ref_logits)) < 2e-3  # only the summation order differs
    # CPU checker: logits within the path's tolerance, greedy tokens equal for the first 32 steps
    orc, stored = build_oracle(TP_SPEC, SEED, N_PROMPT + N_NEW + 8)
    o_tokens = orc.generate_greedy(prompt, N_NEW)
    assert np.array_equal(ranks[0]["tokens"], o_tokens)
    assert np.max(np.abs(tp_logits - orc.logits)) <= 2e-2
    # stored shards are the unsharded tensors' rectangles, bit for bit
    hd, d = TP_SPEC.head_dim, TP_SPEC.d_model
    for k, r in enumerate(ranks):
        p = shard_plan(TP_SPEC, k, 2)
        q0, q1 = p.head_off * hd, (p.head_off + p.q_heads) * hd
        f0, f1 = p.ffn_off, p.ffn_off + p.ffn
        data, scales = stored[(L.ROLE_WQ, 1)][:2]
        assert np.array_equal(r["wq"], data.reshape(-1, d // 8)[q0:q1]) and np.array_equal(r["wq_s"], scales.reshape(-1, d // 32)[q0:q1])
        data, scales = stored[(L.ROLE_WO, 1)][:2]
        assert np.array_equal(r["wo"], data.reshape(d, -1)[:, q0 // 8:q1 // 8]) and np.array_equal(r["wo_s"], scales.reshape(d, -1)[:, q0 // 32:q1 // 32])
        data, scales = stored[(L.ROLE_WDOWN, 2)][:2]
        assert np.array_equal(r["wd"], data.reshape(d, -1)[:, f0 // 8:f1 // 8]) and np.array_equal(r["wd_s"], scales.reshape(d, -1)[:, f0 // 32:f1 // 32])
        data, scales = stored[(L.ROLE_WGATE, 0)][:2]
        assert np.array_equal(r["wg"], data.reshape(-1, d // 8)[f0:f1]) and np.array_equal(r["wg_s"], scales.reshape(-1, d // 32)[f0:f1])
    eng.close()


def test_tp_context_needs_a_communicator():
    """A sharded context refuses to step before vb_tp_init (no hang, no launch)."""
    from velox_b200.engine import Engine
    eng = Engine(TP_SPEC, max_seq_len=64, tp_rank=1, tp_size=2)
    eng.load_synthetic(SEED)
    eng.reserve(0, 16)
    with pytest.raises(L.VeloxError) as ei:
        eng.prefill(np.array([1, 2, 3], dtype=np.uint32))
    assert ei.value.code == L.ERR_STATE
    # its logits buffer is this rank's half of the vocabulary
    assert eng.logits().shape == (TP_SPEC.vocab // 2,)
    eng.close()


def test_tp_create_rejects_unsplittable_models():
    from velox_b200.engine import Engine
    with pytest.raises(L.VeloxError):
        Engine(TP_SPEC, max_seq_len=64, tp_rank=0, tp_size=4)      # 2 KV heads over 4 ranks
    with pytest.raises(L.VeloxError):
        Engine(TP_SPEC.scaled(weight_fmt=L.FMT_I8PC), max_seq_len=64, tp_rank=0, tp_size=2)  # per-row int8 scales


def test_exchange_poll_is_bounded_and_reported():
    """A rank whose peers never answer: the exchange kernels give up at their poll limit (50 ms here), the step
    completes, the host gets VB_ERR_TIMEOUT from the next synchronisation and the context stays usable."""
    import time
    from velox_b200.engine import Engine
    eng = Engine(TP_SPEC, max_seq_len=64, tp_rank=0, tp_size=2)
    eng.load_synthetic(SEED)
    eng.set_option("tp_poll_ms", 50)
    eng.set_option("tp_p2p_standin", 1)  # stand-in regions: nobody pushes into them
    eng.reserve(0, 16)
    t0 = time.time()
    eng.prefill(np.array([1, 2, 3], dtype=np.uint32))  # three steps, 2 exchanges per layer + the argmax exchange
    with pytest.raises(L.VeloxError) as ei:
        eng.sync()
    assert ei.value.code == L.ERR_TIMEOUT
    assert time.time() - t0 < 20.0   # one poll runs out; the others see the error word and fall through
    eng.sync()                       # the error was reported once and cleared: the context still answers
    assert eng.state(0)[1] == 3      # positions advanced (with meaningless tokens)
    eng.close()
