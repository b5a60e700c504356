"""One rank of the tensor-parallel parity run (started by test_gpu_tp.py through torch.distributed.run).

Every rank builds its shard of the same synthetic model, the group decodes greedily, and each rank leaves
its tokens, its slice of the final logits and a few stored shards in ``<out>/rank<r>.npz`` for the test
process to compare with the unsharded engine and the CPU checker.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from velox_b200 import lib as L  # noqa: E402
from velox_b200.modelspec import ModelSpec, shard_plan  # noqa: E402
from velox_b200.tp import create_tp_engine, env_rank, shutdown  # noqa: E402

TP_SPEC = ModelSpec("tp-tiny-q4", vocab=2048, d_model=512, n_layers=3, n_q_heads=8, n_kv_heads=2, head_dim=64,
                    ffn_dim=640, rms_eps=1e-6, rope_theta=1e6, weight_fmt=L.FMT_Q4G32, head_fmt=L.FMT_Q4G32,
                    embed_fmt=L.FMT_F16, qkv_bias=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--seed", type=int, default=11)
    ap.add_argument("--prompt", type=int, default=24)
    ap.add_argument("--new", type=int, default=40)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"])
    ap.add_argument("--fused-push", type=int, default=-1, help="0/1: override the engine's default")
    a = ap.parse_args()
    rank, world, _ = env_rank()
    import torch.distributed as dist
    eng = create_tp_engine(TP_SPEC, max_seq_len=a.prompt + a.new + 8, exchange=a.exchange)
    if a.fused_push >= 0:
        eng.set_option("tp_fused_push", a.fused_push)
    eng.load_synthetic(a.seed)
    dist.barrier()  # the exchange waits ~10 s at most for a peer: start the steps together
    prompt = np.load(os.path.join(a.out, "prompt.npy"))
    toks = eng.generate_greedy(prompt, a.new, use_graph=not a.no_graph)
    logits = eng.logits()
    plan = shard_plan(TP_SPEC, rank, world)
    hd = TP_SPEC.head_dim
    wq, wq_s = eng.export_tensor(L.ROLE_WQ, 1, plan.q_heads * hd, TP_SPEC.d_model)
    wo, wo_s = eng.export_tensor(L.ROLE_WO, 1, TP_SPEC.d_model, plan.q_heads * hd)
    wd, wd_s = eng.export_tensor(L.ROLE_WDOWN, 2, TP_SPEC.d_model, plan.ffn)
    wg, wg_s = eng.export_tensor(L.ROLE_WGATE, 0, plan.ffn, TP_SPEC.d_model)
    np.savez(os.path.join(a.out, f"rank{rank}.npz"), tokens=toks, logits=logits, launches=np.int64(eng.launch_count()),
             wq=wq, wq_s=wq_s, wo=wo, wo_s=wo_s, wd=wd, wd_s=wd_s, wg=wg, wg_s=wg_s)
    shutdown(eng)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
