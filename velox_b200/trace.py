"""Per-kernel device timeline of one decode step (profiling aid).

    python -m velox_b200.trace [--model llama3-8b|qwen2-72b|qwen2.5-7b] [--layers 4] [--prompt-len 512] [--batch 32]
    python -m torch.distributed.run --nproc-per-node N -m velox_b200.trace --model qwen2-72b [--exchange p2p|nccl]

Builds a Llama-3-8B- or Qwen2-72B-shape int4 model with synthetic weights (sharded over the launcher's ranks
when there are several: the gap before gate_up / the next qkv then contains the exchange), captures the decode graph with the "trace"
option on and prints, for every traced kernel of one replayed step, when its first block entered, when it got
past the grid-dependency wait and when its last block left (microseconds since the step's first kernel).
"""
from __future__ import annotations

import argparse
import ctypes as C

import numpy as np

from . import lib as L
from .engine import Engine
from .modelspec import LLAMA3_8B_INT4, PROMPT_STREAM, QWEN2_72B_INT4, QWEN25_7B_INT8
from .tp import connect, env_rank, init_process_group, shutdown


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "qwen2-72b", "qwen2.5-7b"])
    ap.add_argument("--batch", type=int, default=1, help="sequences decoding together (each prefilled with --prompt-len tokens)")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"])
    ap.add_argument("--set", action="append", default=[], metavar="NAME=VALUE", help="engine option (vb_set_option), repeatable")
    args = ap.parse_args()
    base = {"llama3-8b": LLAMA3_8B_INT4, "qwen2-72b": QWEN2_72B_INT4, "qwen2.5-7b": QWEN25_7B_INT8}[args.model]
    spec = base.scaled(name="trace", n_layers=args.layers)
    rank, world, local = env_rank()
    dist = None
    if world > 1:
        import torch.distributed as dist
        init_process_group()
        eng = Engine(spec, max_seq_len=args.prompt_len + 64, device=local, tp_rank=rank, tp_size=world)
        connect(eng, args.exchange)
    else:
        eng = Engine(spec, max_seq_len=args.prompt_len + 64, max_batch=args.batch)
    eng.load_synthetic(1)
    if dist is not None:
        dist.barrier()
    eng.set_option("trace", 1)
    for kv in args.set:
        name, _, val = kv.partition("=")
        eng.set_option(name, int(val))
    rng = np.random.default_rng(PROMPT_STREAM)
    for slot in range(args.batch):
        prompt = rng.integers(0, spec.vocab, args.prompt_len, dtype=np.uint32)
        eng.reserve(slot, args.prompt_len + 64)
        eng.prefill(prompt, slot)
    eng.build_graph()
    eng.decode(8)
    out = np.zeros(3 * 1024, dtype=np.uint64)
    n = C.c_uint32()
    lib = L.load()
    L.check(lib.vb_trace_read(eng.h, out.ctypes.data_as(C.c_void_p), 1024, C.byref(n)))  # clears
    ms = eng.decode(1, timed=True)
    L.check(lib.vb_trace_read(eng.h, out.ctypes.data_as(C.c_void_p), 1024, C.byref(n)))
    if dist is not None:
        eng.sync()
        dist.barrier()
    if rank != 0:
        shutdown(eng)
        return
    r = out[:3 * n.value].reshape(-1, 3).astype(np.int64)
    names = ["qkv", "attn", "o_proj", "gate_up", "down"]
    print("%s x%d layers, %d rank(s)%s: step %.4f ms, %d traced kernels (context %d)"
          % (args.model, args.layers, world, (" exchange=" + args.exchange) if world > 1 else "", ms, n.value, args.prompt_len + 8))
    t0, prev = r[0, 0], r[0, 0]
    for i, (a, b, c) in enumerate(r):
        nm = names[i % 5] if i < args.layers * 5 else "lm_head"
        print("%-8s enter %8.2f  past_wait %8.2f  exit %8.2f | after_wait %6.2f us  gap %5.2f us"
              % (nm, (a - t0) / 1e3, (b - t0) / 1e3, (c - t0) / 1e3, (c - b) / 1e3, (b - prev) / 1e3))
        prev = c
    shutdown(eng) if world > 1 else eng.close()


if __name__ == "__main__":
    main()
