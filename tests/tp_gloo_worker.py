"""One CPU rank of the gloo emulation of the tensor-parallel exchange (started by test_tp_host.py).

The arithmetic is the CPU checker's (quantize / dequantize / matvec of oracle/); the sharding is
velox_b200.modelspec.shard_plan; the exchange is what the GPU ranks do: an in-place sum all-reduce of the
residual stream where rank 0 contributes residual + partial and the others their bare partial, and an
all-gather of (best value, lowest global index) pairs for the vocab-parallel head.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from oracle import oracle as O  # noqa: E402
from velox_b200 import lib as L  # noqa: E402
from velox_b200.modelspec import ModelSpec, shard_plan  # noqa: E402
from velox_b200.tp import init_process_group, share_unique_id  # noqa: E402

SPEC = ModelSpec("gloo-q4", vocab=512, d_model=256, n_layers=1, n_q_heads=4, n_kv_heads=2, head_dim=32, ffn_dim=640,
                 weight_fmt=L.FMT_Q4G32, head_fmt=L.FMT_Q4G32, embed_fmt=L.FMT_F16)
FMT = L.FMT_Q4G32


def quant_deq(w):
    data, scales = O.quantize(w, FMT)
    return O.dequantize(data, scales, FMT, w.shape[0], w.shape[1])


def pick(pairs):
    """(value, index) rule of the argmax: greater value wins, then the lower index; no candidate -> 0."""
    best_v, best_i = -np.inf, 0xFFFFFFFF
    for v, i in pairs:
        if v > best_v or (v == best_v and i < best_i):
            best_v, best_i = v, i
    return 0 if best_i == 0xFFFFFFFF else int(best_i)


def local_best(logits, off):
    best_v, best_i = -np.inf, 0xFFFFFFFF
    for i, v in enumerate(logits):
        if v > best_v:
            best_v, best_i = float(v), i + off
    return best_v, best_i


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    plan = shard_plan(SPEC, rank, world)
    d, f, V = SPEC.d_model, SPEC.ffn_dim, SPEC.vocab
    seed = 5
    # full fp32 sources (identical on every rank: counter-based generator), then this rank's rectangles
    wg = O.fill_normal(f * d, seed, 1).reshape(f, d)
    wu = O.fill_normal(f * d, seed, 2).reshape(f, d)
    wd = O.fill_normal(d * f, seed, 3).reshape(d, f)
    wh = O.fill_normal(V * d, seed, 4).reshape(V, d)
    hidden = O.fill_normal(d, seed, 5, std=1.0)
    sl = slice(plan.ffn_off, plan.ffn_off + plan.ffn)
    vs = slice(plan.vocab_off, plan.vocab_off + plan.vocab)
    # quantizing a shard gives the values of the quantized whole at the same places (groups never straddle ranks)
    full = {k: quant_deq(w) for k, w in (("g", wg), ("u", wu), ("d", wd), ("h", wh))}
    mine = {"g": quant_deq(np.ascontiguousarray(wg[sl])), "u": quant_deq(np.ascontiguousarray(wu[sl])),
            "d": quant_deq(np.ascontiguousarray(wd[:, sl])), "h": quant_deq(np.ascontiguousarray(wh[vs]))}
    deq_equal = (np.array_equal(mine["g"], full["g"][sl]) and np.array_equal(mine["u"], full["u"][sl])
                 and np.array_equal(mine["d"], full["d"][:, sl]) and np.array_equal(mine["h"], full["h"][vs]))

    def swiglu(g, u):
        return (g / (1.0 + np.exp(-g))) * u

    # column-parallel gate/up on the replicated input, row-parallel down -> partial sums
    act = swiglu(mine["g"] @ hidden, mine["u"] @ hidden).astype(np.float32)
    partial = (mine["d"] @ act).astype(np.float32)
    buf = torch.from_numpy((hidden + partial) if rank == 0 else partial.copy())
    dist.all_reduce(buf)                                   # the one exchange of the block
    new_hidden = buf.numpy()
    ref_hidden = hidden + (full["d"] @ swiglu(full["g"] @ hidden, full["u"] @ hidden).astype(np.float32))
    # vocab-parallel head: local best, all-gather of the pairs, same rule over ranks
    logits = (mine["h"] @ new_hidden).astype(np.float32)
    pair = torch.tensor(list(local_best(logits, plan.vocab_off)), dtype=torch.float64)
    pairs = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(pairs, pair)
    token_tp = pick([(float(p[0]), int(p[1])) for p in pairs])
    token_ref = pick([local_best((full["h"] @ new_hidden).astype(np.float32), 0)])
    # a tie across ranks: both shards hold the same maximum, the lower global index must win
    tie = np.full(plan.vocab, -1.0, dtype=np.float32)
    tie[7] = 3.0
    tpair = torch.tensor(list(local_best(tie, plan.vocab_off)), dtype=torch.float64)
    tpairs = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(tpairs, tpair)
    tie_tp = pick([(float(p[0]), int(p[1])) for p in tpairs])
    tie_full = np.concatenate([tie] * world)
    tie_ref = pick([local_best(tie_full, 0)])
    # the id hand-off used for the NCCL communicator (a stand-in id: no NCCL on CPU)
    uid = share_unique_id(lambda: bytes(range(128)))
    flags = torch.tensor([int(deq_equal), int(uid == bytes(range(128)))])
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        np.savez(os.path.join(a.out, "result.npz"), dequant_equal=bool(flags[0]), id_ok=bool(flags[1]),
                 hidden_err=float(np.max(np.abs(new_hidden - ref_hidden))), token_tp=token_tp, token_ref=token_ref,
                 tie_token_tp=tie_tp, tie_token_ref=tie_ref, tie_expected=7)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
