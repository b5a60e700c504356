"""Tensor-parallel host plumbing: one process per GPU, the ranks of one model found through torch.distributed.

The reference states the intent only (examples/qwen2_72b.vlx:4, examples/nanbeige_33b.vlx:27-45:
column-parallel QKV / gate / up, row-parallel O / down, one sum all-reduce after each); the exchange itself
runs inside libvelox_b200 on its own NCCL communicator, captured into the decode graph.  torch.distributed
is used for two host-side things only: passing rank 0's 128-byte communicator id to the other ranks and
barriers / max-over-ranks of timings.
"""
from __future__ import annotations

import dataclasses
import hashlib
import os

from .engine import Engine
from .modelspec import ModelSpec


class TpConfigMismatch(RuntimeError):
    """The ranks of one group were started on different model descriptions (or group sizes)."""


class TpPeerLeft(RuntimeError):
    """A rank of the group announced that it is gone (or stopped answering) between two steps."""


def env_rank():
    """(rank, world_size, local_rank) from the launcher's environment (torchrun); (0, 1, 0) when absent."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def init_process_group(backend: str | None = None):
    """Join the launcher's group (rendezvous on 127.0.0.1 unless the launcher said otherwise)."""
    import torch
    import torch.distributed as dist
    if dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    rank, world, local = env_rank()
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local)
    dist.init_process_group(backend=backend, rank=rank, world_size=world)


def share_unique_id(make_id) -> bytes:
    """Rank 0 calls ``make_id()``; every rank returns the same 128 bytes."""
    import torch.distributed as dist
    box = [make_id() if dist.get_rank() == 0 else None]
    dist.broadcast_object_list(box, src=0)
    assert isinstance(box[0], bytes) and len(box[0]) == 128
    return box[0]


def config_fingerprint(spec: ModelSpec, tp_size: int, **extra) -> str:
    """SHA-256 over everything the ranks of one model must agree on before their kernels wait on each other:
    every field of the model description (shapes, formats, theta, eps, seed of synthetic weights), the group
    size, and whatever the caller adds (max_batch, max_seq_len, exchange kind ...)."""
    items = sorted(dataclasses.asdict(spec).items()) + [("tp_size", int(tp_size))] + sorted(extra.items())
    return hashlib.sha256(repr(items).encode()).hexdigest()


def check_same_config(fingerprint: str):
    """Every rank contributes its fingerprint; all of them raise TpConfigMismatch (naming the ranks that differ from
    rank 0) when they are not identical.  Host-side only, before any peer mapping or communicator exists: a rank
    built from another description fails here instead of inside an exchange that its peers would wait on."""
    import torch.distributed as dist
    seen = [None] * dist.get_world_size()
    dist.all_gather_object(seen, fingerprint)
    odd = [r for r, f in enumerate(seen) if f != seen[0]]
    if odd:
        raise TpConfigMismatch("ranks %s were started on a different model description than rank 0" % odd)


class Membership:
    """Who is still there, asked on the host between steps (never from a kernel).

    A rank that stops serving calls ``leave()`` once none of its kernels or collectives is in flight; it writes
    one key into the group's store.  Every other rank calls ``check()`` before its next launch: a counter read,
    no collective, no wait; it raises TpPeerLeft naming the ranks that are gone, so that no kernel is launched
    that would poll a peer region nobody writes to any more (those polls are bounded, but they take seconds)."""

    def __init__(self, store=None, rank: int | None = None, world: int | None = None, prefix: str = "vb_tp"):
        import torch.distributed as dist
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.prefix = prefix
        self.store.add(self._key("left_count"), 0)  # the key exists from now on

    def _key(self, name: str) -> str:
        return "%s/%s" % (self.prefix, name)

    def leave(self, reason: str = ""):
        self.store.set(self._key("left/%d" % self.rank), reason or "left")
        self.store.add(self._key("left_count"), 1)

    def gone(self) -> list[int]:
        if self.store.add(self._key("left_count"), 0) == 0:
            return []
        return [r for r in range(self.world) if r != self.rank and self.store.check([self._key("left/%d" % r)])]

    def check(self):
        gone = self.gone()
        if gone:
            raise TpPeerLeft("ranks %s left the group" % gone)


def connect(eng: Engine, exchange: str = "p2p"):
    """Gives a sharded engine its exchange: "nccl" (communicator inside the library) or "p2p" (NVLink peer
    mappings, 2..8 ranks; the NCCL communicator is still created so that option "tp_p2p"=0 can fall back)."""
    import torch.distributed as dist
    if exchange not in ("p2p", "nccl"):
        raise ValueError(exchange)
    check_same_config(config_fingerprint(eng.spec, eng.tp_size, max_batch=eng.max_batch, exchange=exchange))
    eng.tp_init(share_unique_id(Engine.tp_unique_id))
    if exchange == "p2p":
        handles = [None] * dist.get_world_size()
        dist.all_gather_object(handles, eng.tp_p2p_export())
        eng.tp_p2p_open(handles)
    dist.barrier()  # every region is mapped (and zeroed) before anyone steps


def create_tp_engine(spec: ModelSpec, max_seq_len: int, max_batch: int = 1, kv_blocks_total: int = 0,
                     lean_weights: bool = False, exchange: str = "p2p") -> Engine:
    """This process's rank of a tensor-parallel engine over all ranks of the default group (device = LOCAL_RANK)."""
    import torch.distributed as dist
    init_process_group()
    rank, world, local = dist.get_rank(), dist.get_world_size(), env_rank()[2]
    if world == 1:
        return Engine(spec, max_seq_len=max_seq_len, max_batch=max_batch, device=local, kv_blocks_total=kv_blocks_total,
                      lean_weights=lean_weights)
    eng = Engine(spec, max_seq_len=max_seq_len, max_batch=max_batch, device=local, kv_blocks_total=kv_blocks_total,
                 tp_rank=rank, tp_size=world, lean_weights=lean_weights)
    connect(eng, exchange)
    return eng


def shutdown(eng: Engine):
    """Closes a sharded engine in the order peer mappings need: every rank unmaps its peers, all ranks meet,
    then each frees its own region with the context."""
    import torch.distributed as dist
    eng.sync()
    if eng.tp_size > 1:
        eng.tp_p2p_close()
        dist.barrier()
    eng.close()
