"""Child process of tests/test_tp_host.py: one CPU rank of a gloo group exercising the host-side failure cases of
tensor-parallel serving (no GPU, no kernel): a description mismatch between ranks, a rank that leaves between
steps and announces it, a rank that is simply gone.  Started with RANK / WORLD_SIZE / MASTER_* in the environment."""
import argparse
import datetime
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from velox_b200 import tp  # noqa: E402
from velox_b200.modelspec import LLAMA3_8B_INT4  # noqa: E402


def step(x):
    """What one decode step exchanges: a sum over the ranks (gloo stands in for the device exchange)."""
    dist.all_reduce(x)
    return x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", required=True, choices=["mismatch", "leave", "vanish"])
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    res = {"rank": rank, "mode": args.mode}
    if args.mode == "mismatch":
        spec = LLAMA3_8B_INT4.scaled(name="m", n_layers=2 if rank == 0 else 3)
        try:
            tp.check_same_config(tp.config_fingerprint(spec, world, max_batch=1))
            res["raised"] = None
        except tp.TpConfigMismatch as e:
            res["raised"] = str(e)
        same = LLAMA3_8B_INT4.scaled(name="m", n_layers=2)
        tp.check_same_config(tp.config_fingerprint(same, world, max_batch=1))  # identical descriptions pass
        res["same_ok"] = True
    else:
        members = tp.Membership()
        dist.barrier()
        done, noticed, failure = 0, None, None
        x = torch.ones(4)
        for s in range(8):
            if rank == 1 and s == 3:
                # between steps, nothing in flight: say so (or not) and stop serving
                if args.mode == "leave":
                    members.leave("drained")
                break
            if rank == 0 and s == 3 and args.mode == "leave":
                t0 = time.time()
                while time.time() - t0 < 20.0 and not members.gone():  # the announcement is on its way
                    time.sleep(0.05)
            try:
                members.check()  # before every launch
            except tp.TpPeerLeft as e:
                noticed = {"step": s, "what": str(e)}
                break
            try:
                step(x.clone())
            except Exception as e:  # the process group's short timeout / a closed connection ends the collective
                failure = {"step": s, "what": type(e).__name__}
                break
            done += 1
        res.update(done=done, noticed=noticed, failure=failure)
    with open(os.path.join(args.out, "rank%d.json" % rank), "w") as f:
        json.dump(res, f)
    # no destroy_process_group: a rank whose peer is gone must be able to exit without another collective
    os._exit(0)


if __name__ == "__main__":
    main()
