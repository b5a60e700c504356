"""Tensor-parallel host logic on CPU: the shard plan, and a world_size-2 gloo run of the exchange steps
(row-parallel partial sums + all-reduce, vocab-parallel argmax pairs + all-gather) against the unsharded
CPU checker."""
from __future__ import annotations

import os
import subprocess
import sys

import numpy as np
import pytest

from velox_b200 import lib as L
from velox_b200.modelspec import LLAMA3_8B_INT4, QWEN2_72B_INT4, ModelSpec, shard_plan

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("spec", [QWEN2_72B_INT4, LLAMA3_8B_INT4])
@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_shard_plan_partitions_the_model(spec, tp):
    plans = [shard_plan(spec, r, tp) for r in range(tp)]
    # FFN: contiguous, whole 128-column blocks, sizes differ by at most one block, no group of 32 straddles ranks
    off = 0
    for p in plans:
        assert p.ffn_off == off and (tp == 1 or (p.ffn % 128 == 0 and p.ffn_off % 128 == 0)) and p.ffn > 0
        off += p.ffn
    assert off == spec.ffn_dim
    assert max(p.ffn for p in plans) - min(p.ffn for p in plans) <= 128
    # heads and vocabulary: even
    assert sum(p.q_heads for p in plans) == spec.n_q_heads and sum(p.kv_heads for p in plans) == spec.n_kv_heads
    assert [p.head_off for p in plans] == [r * spec.n_q_heads // tp for r in range(tp)]
    assert [p.vocab_off for p in plans] == [r * spec.vocab // tp for r in range(tp)]
    # GQA groups stay on one rank
    for p in plans:
        assert p.q_heads % p.kv_heads == 0 and p.head_off // (spec.n_q_heads // spec.n_kv_heads) == p.kv_head_off


def test_shard_plan_qwen72b_tp8_uneven_ffn():
    # 29568 = 231 blocks of 128: seven ranks hold 29 blocks, one holds 28 (an even split would cut a group of 32)
    sizes = [shard_plan(QWEN2_72B_INT4, r, 8).ffn for r in range(8)]
    assert sizes == [3712] * 7 + [3584]


def test_shard_plan_rejects_bad_splits():
    odd = ModelSpec("odd", vocab=1000, d_model=64, n_layers=1, n_q_heads=6, n_kv_heads=3, head_dim=32, ffn_dim=256)
    with pytest.raises(ValueError):
        shard_plan(odd, 0, 2)           # 3 KV heads over 2 ranks
    with pytest.raises(ValueError):
        shard_plan(QWEN2_72B_INT4, 8, 8)  # rank out of range
    small = ModelSpec("small", vocab=1024, d_model=64, n_layers=1, n_q_heads=8, n_kv_heads=8, head_dim=32, ffn_dim=256)
    with pytest.raises(ValueError):
        shard_plan(small, 0, 4)         # two FFN blocks over four ranks


def test_two_rank_gloo_exchange_matches_unsharded(tmp_path):
    """Two CPU processes over gloo: each holds its shard of a quantized block (column-parallel gate/up,
    row-parallel down, vocab-parallel head), they exchange exactly what the GPU ranks exchange, and rank 0
    compares the outcome with the unsharded computation."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29617", os.path.join(ROOT, "tests", "tp_gloo_worker.py"), "--out", str(tmp_path)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    res = np.load(os.path.join(str(tmp_path), "result.npz"))
    assert res["dequant_equal"]                      # shards dequantize to the unsharded values, bit for bit
    assert res["hidden_err"] < 1e-5                  # summation order differs, values agree
    assert int(res["token_tp"]) == int(res["token_ref"])
    assert int(res["tie_token_tp"]) == int(res["tie_token_ref"]) == int(res["tie_expected"])
    assert res["id_ok"]


def _run_membership(mode, tmp_path, port):
    import json
    procs = []
    for rank in range(2):
        env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="2",
                   PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "tp_membership_worker.py"), "--mode", mode,
                                       "--out", str(tmp_path)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for p, out in zip(procs, outs):
        assert p.returncode == 0, out[-3000:]
    return [json.load(open(os.path.join(str(tmp_path), "rank%d.json" % r))) for r in range(2)]


def test_gloo_ranks_with_different_descriptions_are_refused(tmp_path):
    """Rank 1 was started on a 3-layer description, rank 0 on 2 layers: both raise before any exchange is set up,
    naming rank 1; identical descriptions pass."""
    res = _run_membership("mismatch", tmp_path, 29621)
    for r in res:
        assert r["raised"] is not None and "[1]" in r["raised"], r
        assert r["same_ok"]


def test_gloo_rank_leaves_between_steps_and_is_noticed_on_the_host(tmp_path):
    """Rank 1 serves three steps, then leaves with nothing in flight and says so in the group's store; rank 0 learns
    of it from the store before its fourth launch (no collective is entered that nobody would answer)."""
    r0, r1 = _run_membership("leave", tmp_path, 29623)
    assert r1["done"] == 3 and r1["noticed"] is None
    assert r0["done"] == 3 and r0["failure"] is None
    assert r0["noticed"] is not None and r0["noticed"]["step"] == 3 and "[1]" in r0["noticed"]["what"]


def test_gloo_rank_that_is_simply_gone_ends_the_next_collective_with_an_error(tmp_path):
    """Rank 1 exits after three steps without a word: rank 0's next exchange fails within the group's short
    timeout (an exception on the host, not a hang) and rank 0 exits cleanly."""
    r0, r1 = _run_membership("vanish", tmp_path, 29625)
    assert r1["done"] == 3
    assert r0["done"] == 3 and r0["noticed"] is None
    assert r0["failure"] is not None and r0["failure"]["step"] == 3
