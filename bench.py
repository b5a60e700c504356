#!/usr/bin/env python
"""Decode-throughput benchmark of libvelox_b200 (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Headline workload: Llama-3-8B-shape decoder, int4 group-32 weights + fp16 scales, fp16 embeddings, batch 1,
512-token prompt, greedy decode (seed-generated synthetic weights and token ids; no checkpoint offline).
A "step" is one decode step (one token per sequence).  `value` is decode tok/s with everything resident in
HBM, timed by CUDA events on the library's stream around K CUDA-graph replays; `e2e` is the same metric when
every step is driven from the host through the C ABI (token and position sent in, sampled token read back).
N>1 runs N independent replicas of that model (it fits one GPU): weak scaling, no data-path collective.

The same line carries three more objects:
  "tp"    at every N: ONE Qwen2-72B-shape int4-g32 model, batch 1, 1024-token prompt, sharded over the N ranks
          (tensor parallel: column-parallel QKV / gate / up, row-parallel O / down, one exchange after each; N = 1
          is the unsharded model on one GPU): per-token latency, per-GPU roofline, and at N > 1 the speed-up over
          the unsharded model measured on rank 0's GPU in the same run, plus a parity flag (a 2-layer model of the
          same width gives the same 32 greedy tokens sharded and unsharded);
  "bs32"  at N = 1: Qwen2.5-7B-shape int8 per-channel model, 32 sequences with prompt lengths uniform in
          [256, 2048], paged fp16 KV;
  "mla"   at N = 1: the absorbed multi-head latent attention decode kernel on the DeepSeek-V3-style shape (128 heads,
          latent 512 + 64, batch 64, contexts uniform in [1024, 8192]).
--workload NAME makes NAME the headline instead (the extra objects are then left out).

--impl reference times the CPU restatement of the reference runtime (oracle/, OpenMP on all host cores) on
a bounded sample of the headline workload; rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_tok_per_s"
UNIT = "tok/s"
SEED = 20250101
PROMPT_LEN = 512
TP_WORKLOAD = "qwen2-72b-int4-tp-bs1"
TP_PROMPT_LEN = 1024
BS32_WORKLOAD = "qwen2.5-7b-int8-bs32"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def is_tp(name: str) -> bool:
    return name.startswith("qwen2-72b-int4-tp")


def workload_spec(name: str):
    from velox_b200.modelspec import LLAMA3_8B_INT4, QWEN2_72B_INT4, QWEN25_7B_INT8
    if name == "llama3-8b-int4-bs1":
        return LLAMA3_8B_INT4, 1
    if name == "qwen2.5-7b-int8-bs1":  # the int8 per-channel model shape, one sequence
        return QWEN25_7B_INT8, 1
    if name == "qwen2.5-7b-int8-bs32":  # 32 sequences, prompt lengths uniform in [256, 2048]
        return QWEN25_7B_INT8, 32
    if name == "qwen2-72b-int4-tp-bs1":
        return QWEN2_72B_INT4, 1
    if name == "qwen2-72b-int4-tp-bs16":  # 16 sequences per step (sharded: the unsharded model only fits with one)
        return QWEN2_72B_INT4, 16
    if name == "qwen2-72b-int4-tp-bs1-8layers":  # quick check of the sharded path
        return QWEN2_72B_INT4.scaled(name="qwen2-72b-int4g32-8layers", n_layers=8), 1
    if name == "llama3-8b-int4-bs1-4layers":  # quick functional check of the bench itself
        return LLAMA3_8B_INT4.scaled(name="llama3-8b-int4g32-4layers", n_layers=4), 1
    raise SystemExit("unknown workload %r" % name)


def synthetic_prompt(vocab: int, n: int, stream: int = 0) -> np.ndarray:
    """Token ids uniform in [0, vocab), fixed by (SEED, stream)."""
    return np.random.default_rng([SEED, stream]).integers(0, vocab, size=n, dtype=np.int64).astype(np.uint32)


def host_cores() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_sample(spec, n_layers_sample: int, n_steps: int, warm: int):
    """Times the CPU checker on `n_layers_sample` layers + head of the workload; returns per-token seconds
    extrapolated to the full depth (weight streaming is linear in the layer count).  The thread count is set
    here, to every core this process may run on: launchers export OMP_NUM_THREADS=1."""
    os.environ["OMP_NUM_THREADS"] = str(host_cores())
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import helpers as H
    from oracle import oracle as O
    O.lib().vo_set_num_threads(host_cores())
    sub = spec.scaled(n_layers=n_layers_sample)
    eng, _ = H.build_oracle(sub, SEED, max_seq_len=warm + n_steps + 1)
    toks = H.prompt_tokens(spec, SEED, warm + n_steps)
    for i in range(warm):
        eng.forward_step(int(toks[i]), i)
    per_step = []
    head_t = None
    for i in range(warm, warm + n_steps):
        t0 = time.perf_counter()
        eng.forward_step(int(toks[i]), i)
        per_step.append(time.perf_counter() - t0)
    # separate the head (independent of depth) from the per-layer cost with a 1-layer engine
    one = spec.scaled(n_layers=1)
    e1, _ = H.build_oracle(one, SEED, max_seq_len=4)
    e1.forward_step(int(toks[0]), 0)
    t0 = time.perf_counter()
    e1.forward_step(int(toks[1]), 1)
    t1 = time.perf_counter() - t0
    t_s = float(np.median(per_step))
    per_layer = max(1e-9, (t_s - t1) / max(1, n_layers_sample - 1)) if n_layers_sample > 1 else t_s
    head_t = max(0.0, t1 - per_layer)
    full = head_t + per_layer * spec.n_layers
    return full, per_step, O.lib().vo_num_threads()


def run_reference(args, spec, batch, rank, world):
    if rank != 0:
        return
    budget_s = 150.0
    n = args.steps + args.warmup
    # pick how many layers one "step" covers so that the whole run fits the budget (calibrated on 2 layers)
    full, _, cores = cpu_sample(spec, 2, 1, 1)
    per_layer = full / spec.n_layers
    layers = int(max(2, min(spec.n_layers, budget_s / max(1e-6, n * per_layer))))
    t_wall = time.perf_counter()
    full, per_step, cores = cpu_sample(spec, layers, args.steps, args.warmup)
    value = 1.0 / full
    sample = ("each step = one decode token through %d of %d layers + lm_head on the CPU restatement of "
              "src/runtime.rs, extrapolated linearly to full depth; positions %d..%d" %
              (layers, spec.n_layers, args.warmup, args.warmup + args.steps - 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * full, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": args.workload, "model": spec.name, "batch": batch,
                                                        "prompt_len": PROMPT_LEN},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t_wall,
    }
    print(json.dumps(line), flush=True)


class Ranks:
    """The process group of this run (torch.distributed over NCCL; plumbing only: barriers, max over ranks)."""

    def __init__(self):
        import torch
        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            torch.cuda.set_device(self.local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        if self.torch.cuda.is_available():
            self.torch.cuda.synchronize()

    def max(self, v: float) -> float:
        if self.dist is None:
            return v
        t = self.torch.tensor([v], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()


def measure(args, R: Ranks, workload: str, steps: int, warmup: int, prompt_len: int, sharded: bool, solo: bool = False,
            with_e2e: bool = True, with_prefill: bool = False, layers: int = 0):
    """Builds the workload's engine(s), prefills, captures the decode graph, times `steps` replays and the same
    steps driven from the host.  sharded: one model over all ranks (else one engine per rank); solo: this rank
    alone (no barriers, no max over ranks).  Returns the figures of a bench line."""
    from velox_b200.engine import Engine
    spec, batch = workload_spec(workload)
    if layers > 0:
        spec = spec.scaled(name="%s-%dlayers" % (spec.name, layers), n_layers=layers)
    world = 1 if solo else R.world
    tp = is_tp(workload)
    prompt_lens = [prompt_len] * batch
    if workload == BS32_WORKLOAD and not args.same_prompt_len:
        prompt_lens = [int(x) for x in np.random.default_rng(SEED).integers(256, 2049, size=batch)]
    max_seq = max(prompt_lens) + warmup + 2 * steps + 16 + 512   # (512: room to keep the GPU busy for the clock sampler)

    def barrier():
        if not solo:
            R.barrier()

    if sharded and world > 1:
        # one model over all ranks; the 72B shape only fits one GPU with the single-layout arena
        from velox_b200.tp import connect
        eng = Engine(spec, max_seq_len=max_seq, max_batch=batch, device=R.local_rank, tp_rank=R.rank, tp_size=world,
                     lean_weights=batch == 1)
        connect(eng, args.tp_exchange)
    else:
        eng = Engine(spec, max_seq_len=max_seq, max_batch=batch, device=R.local_rank, lean_weights=tp and batch == 1)
    eng.set_option("gemv_path", args.gemv_path)
    for kv in args.set:
        name, _, val = kv.partition("=")
        eng.set_option(name, int(val))
    if args.no_pdl:
        eng.set_option("pdl", 0)
    t0 = time.perf_counter()
    eng.load_synthetic(SEED)
    load_s = time.perf_counter() - t0
    barrier()  # ranks of one model step together

    t0 = time.perf_counter()
    if batch == 1:
        prompt = synthetic_prompt(spec.vocab, prompt_len)
        eng.reserve(0, max_seq)
        eng.prefill(prompt, 0)
    else:
        # every slot its own prompt, prefilled slot by slot in tensor-core chunks; a sharded engine (no chunked
        # prefill) runs them in lockstep, one step per position
        for slot in range(batch):
            eng.reserve(slot, max_seq)
        prompts = [synthetic_prompt(spec.vocab, prompt_lens[slot], stream=1 + slot) for slot in range(batch)]
        if sharded and world > 1:
            eng.prefill_lockstep(prompts)
        else:
            for slot in range(batch):
                eng.prefill(prompts[slot], slot)
    eng.sync()
    ttft_s = time.perf_counter() - t0
    prefill = None
    if with_prefill and batch == 1 and not tp:
        # the same prompt once more with every buffer in place: prefill throughput.  All but the last prompt token go
        # through the layers as rows of tensor-core GEMMs (vb_gemm_tc.cu); their flops against the measured dense peak.
        t1 = time.perf_counter()
        eng.prefill(prompt, 0)
        eng.sync()
        pf_s = time.perf_counter() - t1
        qdim, kvdim = spec.n_q_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
        layer_params = spec.d_model * (qdim + 2 * kvdim) + qdim * spec.d_model + 3 * spec.ffn_dim * spec.d_model
        flops = 2.0 * layer_params * spec.n_layers * (prompt_len - 1)
        tpeak = None
        try:
            tpeak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
        except Exception:
            pass
        prefill = {"tokens": prompt_len, "ms": 1e3 * pf_s, "tok_per_s": prompt_len / pf_s,
                   "roofline": {"bound": "tensor", "achieved": flops / pf_s / 1e12, "peak": tpeak if tpeak else 1590.0, "unit": "TFLOP/s",
                                "frac": flops / pf_s / 1e12 / (tpeak if tpeak else 1590.0), "peak_kind": "measured" if tpeak else "fallback",
                                "what": "projection flops of prompt_len-1 rows / whole warm prefill time (host clock, includes attention, "
                                        "operand conversion and the last token's decode-path step)"}}
    eng.build_graph()
    qd_, kd_ = spec.n_q_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
    # decode batches over int8 weights read the stored bytes (k_gemm_i8); only with that path switched off do they read
    # resident fp16 copies of the layer matrices, 2 bytes per weight where the algorithm counts 1
    i8_off = any(kv.replace(" ", "") == "decode_gemm_i8=0" for kv in args.set)
    tc_extra_bytes = (spec.d_model * (qd_ + 2 * kd_) + qd_ * spec.d_model + 3 * spec.ffn_dim * spec.d_model) * spec.n_layers \
        if "int8" in spec.name and i8_off else 0

    sampler = ClockSampler(R.local_rank)
    sampler.start()          # nvidia-smi needs a moment to start: sample from here on, all under load
    groups = 1 if (sharded or solo) else world  # independent model instances

    # ---- end to end: every step driven from the host through the C ABI (measured first: the device-timed steps after
    # it then run on a GPU that has been under load for a while, whatever the state it was handed over in) -----------
    e2e = None
    if with_e2e:
        tok, pos = eng.state(0)
        eng_pos = [eng.state(slot)[1] for slot in range(batch)]  # position of every slot's next token
        barrier()
        t0 = time.perf_counter()
        if batch == 1:
            for _ in range(steps):
                tok = eng.forward_step(tok, pos, 0)   # sends (token,pos), replays one step, reads the token back
                pos += 1
        else:
            for _ in range(steps):               # tokens feed back on the device; the host reads every slot's token
                eng.decode(1)
                for slot in range(batch):
                    eng.read_tokens(slot, eng_pos[slot], 1)
                    eng_pos[slot] += 1
        e2e_s = time.perf_counter() - t0
        if not solo:
            e2e_s = R.max(e2e_s)
        e2e = {"value": groups * batch * steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 8 if batch == 1 else 0,
               "d2h_bytes_per_step": 4 * batch}
    # ---- device-resident timing: K graph replays between CUDA events on the library's stream ----------
    eng.decode(warmup)
    eng.sync()
    wbytes, kv0 = eng.step_bytes()
    barrier()
    l0 = eng.launch_count()
    ms = eng.decode(steps, timed=True)
    launches = eng.launch_count() - l0
    eng.sync()
    barrier()
    _, kv1 = eng.step_bytes()
    if not solo:
        ms = R.max(ms)
    ms_per_step = ms / steps
    value = groups * batch * 1e3 / ms_per_step

    # short runs: keep replaying the same step (untimed) until the sampler has three readings under load, two seconds at
    # most.  Ranks that work together decide together (a sharded step is a collective: every rank replays the same number).
    t_end = time.perf_counter() + 2.0
    spare = max_seq - max(eng.state(slot)[1] for slot in range(batch)) - 1
    while spare >= 8:
        more = 1.0 if (len(sampler.rows) < 3 and time.perf_counter() < t_end) else 0.0
        if not solo:
            more = R.max(more)
        if more == 0.0:
            break
        eng.decode(8)
        eng.sync()
        spare -= 8
    clocks = sampler.stop()

    peak, peak_kind = load_peaks()
    step_bytes = wbytes + (kv0 + kv1) // 2  # mean context over the timed region
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    out = {
        "spec": spec, "batch": batch, "ms_per_step": ms_per_step, "value": value, "e2e": e2e, "launches": int(launches),
        "clocks": clocks, "ttft_ms": 1e3 * ttft_s, "load_s": load_s, "prefill": prefill, "groups": groups,
        "config": {"workload": workload, "model": spec.name, "batch": batch,
                   "prompt_len": prompt_len if len(set(prompt_lens)) == 1 else "uniform in [256, 2048]",
                   "weights": ("int8 per output channel + fp16 scales" if "int8" in spec.name else "int4 g32 + fp16 scales") +
                              ", fp16 embeddings/norms", "kv": "paged fp16, 16-token blocks",
                   "l2_policy": "inputs larger than L2: %.2f GB of weights streamed per step" % (wbytes / 1e9),
                   "gemv_path": args.gemv_path, "replicas": groups, "tensor_parallel": world if sharded else 1,
                   "tp_exchange": (args.tp_exchange if sharded and world > 1 else None)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     # dram read+write of one step: ncu on the 4-layer case of the batch-1 workload measured 1.006x the
                     # algorithmic bytes per layer, on the 2-layer case of the batch-32 workload 1.03x (products 1.01x,
                     # attention 1.12x: block tables, queries, split partials); every layer is the same kernels, so the
                     # ratio is applied to the full depth
                     "traffic": int(step_bytes * (1.03 if batch >= 16 else 1.006)) + (tc_extra_bytes if batch >= 16 and not tp else 0),
                     "peak_kind": peak_kind,
                     "frac_of_8TBs": achieved / 8000.0,
                     "kernel": "decode step (one CUDA-graph launch = one token)" + (", per GPU" if tp else ""),
                     "bytes_per_launch": step_bytes},
    }
    if sharded and world > 1:
        from velox_b200.tp import shutdown
        shutdown(eng)
    else:
        eng.close()
    return out


def tp_parity(args, R: Ranks) -> bool:
    """A 2-layer model of the 72B width, sharded over all ranks and unsharded on rank 0: same 32 greedy tokens."""
    from velox_b200.engine import Engine
    from velox_b200.tp import connect, shutdown
    spec, _ = workload_spec(TP_WORKLOAD)
    spec = spec.scaled(name=spec.name + "-2layers", n_layers=2)
    prompt = synthetic_prompt(spec.vocab, 24, stream=99)
    eng = Engine(spec, max_seq_len=64, max_batch=1, device=R.local_rank, tp_rank=R.rank, tp_size=R.world, lean_weights=True)
    connect(eng, args.tp_exchange)
    eng.load_synthetic(SEED)
    R.barrier()
    got = eng.generate_greedy(prompt, 32)
    shutdown(eng)
    ok = 1.0
    if R.rank == 0:
        one = Engine(spec, max_seq_len=64, max_batch=1, device=R.local_rank, lean_weights=True)
        one.load_synthetic(SEED)
        want = one.generate_greedy(prompt, 32)
        one.close()
        ok = 1.0 if np.array_equal(got, want) else 0.0
    return R.max(1.0 - ok) == 0.0


def tp_object(args, R: Ranks):
    """The north-star split: Qwen2-72B shape over the N ranks of this run (see the module docstring)."""
    m = measure(args, R, TP_WORKLOAD, args.steps, args.warmup, TP_PROMPT_LEN, sharded=True, with_e2e=True)
    obj = {"workload": TP_WORKLOAD, "model": m["spec"].name, "tensor_parallel": R.world, "batch": 1, "prompt_len": TP_PROMPT_LEN,
           "ms_per_token": m["ms_per_step"], "tok_s": m["value"], "e2e_tok_s": m["e2e"]["value"], "scaling": "strong",
           "exchange": (("NVLink peer stores inside the library's kernels" if args.tp_exchange == "p2p" else "NCCL all-reduce")
                        if R.world > 1 else None),
           "roofline": dict(m["roofline"], kernel="decode step (one CUDA-graph launch = one token), per GPU"),
           "gpu_launches": m["launches"], "ttft_ms": m["ttft_ms"], "clocks": m["clocks"]}
    if R.world > 1:
        obj["parity_32_tokens_vs_unsharded"] = tp_parity(args, R)
        # the unsharded model on rank 0's GPU, same box, same run: the TP-1 latency the speed-up is quoted against
        tp1 = None
        if R.rank == 0:
            tp1 = measure(args, R, TP_WORKLOAD, args.steps, args.warmup, TP_PROMPT_LEN, sharded=False, solo=True, with_e2e=False)
        R.barrier()
        if tp1 is not None:
            obj["tp1_ms_per_token"] = tp1["ms_per_step"]
            obj["speedup_vs_tp1"] = tp1["ms_per_step"] / m["ms_per_step"]
    return obj


MLA_WORKLOAD = "deepseek-mla-bs64"


def mla_object(R: Ranks, iters: int = 20):
    """The absorbed multi-head latent attention decode kernel on the DeepSeek-V3-style shape of the benchmark
    configuration: 128 heads, latent 512 + 64, batch 64, context lengths uniform in [1024, 8192], bf16 latent cache.
    One launch = the attention of one layer for the whole batch; both bounds are reported (cache bytes against the
    copy peak, products against the dense bf16 peak)."""
    import ctypes as C
    torch = R.torch
    from velox_b200 import lib as L
    lib = L.load()
    B, H, W, DC, split = 64, 128, 576, 512, 1024
    rng = np.random.default_rng(SEED)
    lens = rng.integers(1024, 8193, size=B).astype(np.uint32)
    max_ctx = int(lens.max())
    dev = torch.device("cuda", R.local_rank)
    g = torch.Generator(device=dev).manual_seed(SEED)
    cache = torch.randn((B, max_ctx, W), device=dev, dtype=torch.float32, generator=g).to(torch.bfloat16)
    q = torch.randn((B, H, W), device=dev, dtype=torch.float32, generator=g)
    out = torch.empty((B, H, DC), device=dev, dtype=torch.float32)
    d_len = torch.from_numpy(lens.astype(np.int32)).to(dev)
    need = lib.vb_op_mla_decode_scratch_bytes(B, H, max_ctx, split)
    scratch = torch.empty(need, device=dev, dtype=torch.uint8)
    stream = torch.cuda.current_stream(dev)
    scale = 1.0 / float(np.sqrt(128 + 64))

    def launch():
        L.check(lib.vb_op_mla_decode(C.c_void_p(out.data_ptr()), C.c_void_p(q.data_ptr()), C.c_void_p(cache.data_ptr()), C.c_void_p(d_len.data_ptr()),
                                     B, H, max_ctx, max_ctx, scale, split, C.c_void_p(scratch.data_ptr()), need, C.c_void_p(stream.cuda_stream)))
    for _ in range(3):
        launch()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(iters):
        launch()
    e1.record(stream)
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / iters
    rows = int(lens.astype(np.int64).sum())
    flops = 2.0 * rows * H * (W + DC)
    nbytes = rows * W * 2 + q.numel() * 4 + out.numel() * 4
    peak, kind = load_peaks()
    try:
        tpeak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        tpeak = 1590.0
    return {"workload": MLA_WORKLOAD, "kernel": "k_mla_decode_tc (tcgen05) + k_mla_merge (one layer's attention for the batch)", "batch": B, "heads": H,
            "latent": "512 + 64 bf16", "context": "uniform in [1024, 8192], mean %d" % (rows // B), "ms_per_launch": ms, "gpu_launches": 2 * iters,
            "l2_policy": "inputs larger than L2: %.2f GB of latent cache per launch" % (rows * W * 2 / 1e9),
            "roofline_tensor": {"bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12, "peak": tpeak, "unit": "TFLOP/s",
                                "frac": flops / (ms * 1e-3) / 1e12 / tpeak, "flops_per_launch": flops},
            "roofline_hbm": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s", "frac": nbytes / (ms * 1e-3) / 1e9 / peak,
                             "bytes_per_launch": nbytes, "peak_kind": kind}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, help="headline workload (default llama3-8b-int4-bs1 plus the tp / bs32 objects)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="leave out the tp and bs32 objects")
    ap.add_argument("--gemv-path", type=int, default=1)
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--prompt-len", type=int, default=0)
    ap.add_argument("--same-prompt-len", action="store_true", help="batch workloads: every sequence gets --prompt-len tokens "
                    "instead of lengths uniform in [256, 2048] (shows what uneven lengths cost)")
    ap.add_argument("--mla-path", type=int, default=1, choices=[0, 1], help="MLA workload: 1 tcgen05 kernel (default), 0 mma.sync kernel")
    ap.add_argument("--layers", type=int, default=0, help="run the workload's shape with this many layers (quick checks)")
    ap.add_argument("--set", action="append", default=[], metavar="NAME=VALUE", help="engine option (vb_set_option), repeatable")
    ap.add_argument("--tp-exchange", default="p2p", choices=["p2p", "nccl"],
                    help="tensor-parallel workloads: NVLink peer pushes inside the library's own kernels, or NCCL")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    extras = args.workload is None and not args.no_extras and args.layers == 0
    if args.workload is None:
        args.workload = "llama3-8b-int4-bs1"
    if args.prompt_len <= 0:
        args.prompt_len = TP_PROMPT_LEN if is_tp(args.workload) else PROMPT_LEN

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload == MLA_WORKLOAD:
        # the attention kernel of the MLA configuration alone (what the "mla" object of the default line holds)
        R = Ranks()
        from velox_b200 import lib as L
        L.check(L.load().vb_op_mla_set_path(args.mla_path))
        obj = mla_object(R, iters=max(1, args.steps))
        obj["kernel_path"] = "tcgen05" if args.mla_path == 1 else "mma.sync"

        R.close()
        if rank == 0:
            print(json.dumps({"metric": "mla_attention_tflops", "value": obj["roofline_tensor"]["achieved"], "unit": "TFLOP/s", "n_gpus": 1,
                              "steps": args.steps, "warmup": 3, "ms_per_step": obj["ms_per_launch"], "higher_is_better": True,
                              "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                              "config": {"workload": MLA_WORKLOAD}, "roofline": obj["roofline_tensor"], "mla": obj,
                              "gpu_launches": obj["gpu_launches"]}), flush=True)
        return
    spec, batch = workload_spec(args.workload)
    if args.layers > 0:
        spec = spec.scaled(name="%s-%dlayers" % (spec.name, args.layers), n_layers=args.layers)

    if args.impl == "reference":
        run_reference(args, spec, batch, rank, world)
        return

    R = Ranks()
    tp = is_tp(args.workload)
    m = measure(args, R, args.workload, args.steps, args.warmup, args.prompt_len, sharded=tp, with_e2e=True, with_prefill=True,
                layers=args.layers)
    line = {
        "metric": METRIC, "value": m["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": "strong" if tp else "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic", "config": m["config"], "roofline": m["roofline"], "e2e": m["e2e"],
        "gpu_launches": m["launches"], "clocks": m["clocks"], "ttft_ms": m["ttft_ms"], "load_s": m["load_s"],
    }
    if m["prefill"] is not None:
        line["prefill"] = m["prefill"]
    if extras:
        line["tp"] = tp_object(args, R)
        if world == 1:
            b = measure(args, R, BS32_WORKLOAD, args.steps, args.warmup, 0, sharded=False, with_e2e=True)
            line["mla"] = mla_object(R)
            line["bs32"] = {"workload": BS32_WORKLOAD, "model": b["spec"].name, "batch": 32, "prompt_len": "uniform in [256, 2048]",
                            "ms_per_step": b["ms_per_step"], "tok_s": b["value"], "e2e_tok_s": b["e2e"]["value"],
                            "roofline": b["roofline"], "gpu_launches": b["launches"], "ttft_ms": b["ttft_ms"]}
    if rank == 0 and not args.no_cpu_baseline and world == 1:
        full, per_step, cores = cpu_sample(spec, 6, 6, 1)
        line["cpu_baseline"] = {"value": 1.0 / full, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": "6 decode tokens through 6 of %d layers + lm_head on the CPU restatement, "
                                          "extrapolated linearly to full depth" % spec.n_layers}
    R.close()
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
