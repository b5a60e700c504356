"""The stand-alone C++ runner (velox_b200/runner): command line, safetensors reading, and -- on a GPU -- the same
greedy tokens as the CPU checker from a checkpoint file written here."""
from __future__ import annotations

import json
import os
import re
import struct
import subprocess

import numpy as np
import pytest

import helpers as H
from velox_b200 import build
from velox_b200 import lib as L
from velox_b200.modelspec import SMOLLM_135M

HF_NAMES = {L.ROLE_EMBED: "model.embed_tokens.weight", L.ROLE_FINAL_NORM: "model.norm.weight", L.ROLE_LM_HEAD: "lm_head.weight"}
LAYER_NAMES = {L.ROLE_ATTN_NORM: "input_layernorm.weight", L.ROLE_WQ: "self_attn.q_proj.weight", L.ROLE_WK: "self_attn.k_proj.weight",
               L.ROLE_WV: "self_attn.v_proj.weight", L.ROLE_WO: "self_attn.o_proj.weight", L.ROLE_MLP_NORM: "post_attention_layernorm.weight",
               L.ROLE_WGATE: "mlp.gate_proj.weight", L.ROLE_WUP: "mlp.up_proj.weight", L.ROLE_WDOWN: "mlp.down_proj.weight",
               L.ROLE_BQ: "self_attn.q_proj.bias", L.ROLE_BK: "self_attn.k_proj.bias", L.ROLE_BV: "self_attn.v_proj.bias"}


def runner_path() -> str:
    if not os.path.exists(build.RUNNER):
        build.build_runner()
    return build.RUNNER


def write_safetensors(path, spec, seed):
    """The synthetic model as a safetensors file under the Hugging Face Llama names (fp32)."""
    header, blobs, off = {"__metadata__": {"format": "pt"}}, [], 0
    for role, layer, rows, cols, mean, std in spec.tensors():
        w = H.host_tensor(spec, seed, role, layer, rows, cols, mean, std).astype(np.float32)
        name = HF_NAMES.get(role) or "model.layers.%d.%s" % (layer, LAYER_NAMES[role])
        shape = [cols] if role in H.VEC_ROLES else [rows, cols]
        header[name] = {"dtype": "F32", "shape": shape, "data_offsets": [off, off + w.nbytes]}
        blobs.append(w.tobytes())
        off += w.nbytes
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for b in blobs:
            f.write(b)


def test_runner_rejects_bad_command_lines(tmp_path):
    exe = runner_path()
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 2 and "--weights" in r.stderr
    r = subprocess.run([exe, "--synthetic", "1", "--quantize", "nope"], capture_output=True, text=True)
    assert r.returncode == 2 and "unknown --quantize" in r.stderr
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(struct.pack("<Q", 5) + b"{oops")
    r = subprocess.run([exe, "--weights", str(bad)], capture_output=True, text=True)
    assert r.returncode == 1 and "not a safetensors file" in r.stderr
    # a well-formed file that lacks a tensor is refused by name, before any GPU work
    ok = tmp_path / "empty.safetensors"
    text = json.dumps({"__metadata__": {"a": "b"}}).encode()
    ok.write_bytes(struct.pack("<Q", len(text)) + text)
    r = subprocess.run([exe, "--weights", str(ok), "--dims", "64,32,1,2,1,16,64"], capture_output=True, text=True)
    assert r.returncode == 1  # no GPU here: vb_create fails; with a GPU: "missing model.embed_tokens.weight"
    assert "vb_create" in r.stderr or "missing model.embed_tokens.weight" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("graph", [True, False])
def test_runner_generates_the_checkers_tokens_from_a_safetensors_file(tmp_path, graph):
    spec = SMOLLM_135M.scaled(name="smollm-narrow", n_layers=3, vocab=2048)
    seed, n_new = 5, 12
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, spec, seed)
    prompt = H.prompt_tokens(spec, seed, 9)
    ora, _ = H.build_oracle(spec, seed, len(prompt) + n_new + 1)
    want = ora.generate_greedy(prompt, n_new)
    dims = "%d,%d,%d,%d,%d,%d,%d" % (spec.vocab, spec.d_model, spec.n_layers, spec.n_q_heads, spec.n_kv_heads, spec.head_dim, spec.ffn_dim)
    cmd = [runner_path(), "--weights", path, "--tokens", ",".join(str(int(t)) for t in prompt), "--steps", str(n_new), "--dims", dims,
           "--verbose"] + ([] if graph else ["--no-cuda-graph"])
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    m = re.search(r"Generated Tokens \(%d\)\s*: \[([0-9, ]*)\]" % n_new, r.stdout)
    assert m, r.stdout
    got = np.array([int(x) for x in m.group(1).split(",")], dtype=np.uint32)
    assert np.array_equal(got, want)
    assert "[Step 0] Token: %d" % want[0] in r.stdout
    assert re.search(r"TTFT \(Prefill Latency\) : [0-9.]+ ms", r.stdout) and "Final Step Top-5 Logits:" in r.stdout
    top1 = re.search(r"#1: token_id=(\d+) logit=([-0-9.]+)", r.stdout)
    assert int(top1.group(1)) == int(np.argmax(ora.logits)) and abs(float(top1.group(2)) - float(np.max(ora.logits))) <= 2e-2


@pytest.mark.gpu
def test_runner_takes_the_flags_the_compiler_driver_passes(tmp_path):
    """`veloxc --run` always passes --verbose and, when asked, --speculative / --draft-len / --spec-ema, plus --context-len
    for the K2 runner (src/cli.rs:653-683): the speculative run prints the same tokens as the plain one, the report keeps
    the lines the reference's tooling parses."""
    base = [runner_path(), "--synthetic", "3", "--dims", "4096,512,2,8,2,64,1408", "--quantize", "q4g32", "--steps", "40", "--verbose",
            "--tokens", "5,9,5,9,5,9,5,9,11,5,9"]
    plain = subprocess.run(base, capture_output=True, text=True, timeout=300)
    assert plain.returncode == 0, plain.stderr[-2000:]
    spec = subprocess.run(base + ["--speculative", "--draft-len", "4", "--spec-ema", "0.2", "--context-len", "16384"],
                          capture_output=True, text=True, timeout=300)
    assert spec.returncode == 0, spec.stderr[-2000:]
    pat = r"Generated Tokens \(40\)\s*: \[([0-9, ]*)\]"
    assert re.search(pat, plain.stdout).group(1) == re.search(pat, spec.stdout).group(1)
    steps = re.findall(r"^\[Step (\d+)\] Token: (\d+)", spec.stdout, flags=re.M)
    assert [int(s) for s, _ in steps] == list(range(40))
    assert "Decoding Mode          : Speculative Decoding (Prompt-Lookup, max draft K=4)" in spec.stdout
    assert re.search(r"Draft Acceptance Rate  : [0-9.]+% \(\d+ / \d+ draft tokens accepted\)", spec.stdout)
    assert "Parity 4-token check   : SKIPPED" in spec.stdout and "Parity 32-token check  : SKIPPED" in spec.stdout
    assert "Decoding Mode          : Autoregressive Standard (Single Token)" in plain.stdout
    # "--speculative K" carries the width itself, as the reference runner parses it
    spec2 = subprocess.run(base + ["--speculative", "2"], capture_output=True, text=True, timeout=300)
    assert spec2.returncode == 0 and "max draft K=2" in spec2.stdout
    sampled = subprocess.run(base + ["--temperature", "0.9", "--top-p", "0.9", "--seed", "4"], capture_output=True, text=True, timeout=300)
    assert sampled.returncode == 0 and "Decoding Mode          : Nucleus Sampling" in sampled.stdout
