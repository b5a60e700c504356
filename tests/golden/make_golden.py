"""Generates the committed fixtures of tests/golden/ (run in the development container only).

    python tests/golden/make_golden.py

smollm_ref_golden.json: the reference's own emitted C99 model (oracle/_ref, compiled from
src/runners/tinystories_smollm.c) run on seed-generated SmolLM-135M-shape weights: prompt, greedy
tokens, per-step top-5 logits and a SHA-256 of the full logits vector after every step.  The GPU box has
no reference tree, so the tests there compare against these numbers.
"""
import ctypes as C
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

SEED = 20240611
N_PROMPT, N_NEW = 16, 16


def main():
    R = O.ref_lib()
    if R is None:
        raise SystemExit("oracle/_ref is not built (needs the reference tree)")
    d, ffn, nl, hq, hkv, hd, V, _ = [R.refsm_dim(i) for i in range(8)]
    shapes = {0: (V, d), 1: (nl, d), 2: (nl, hq * hd, d), 3: (nl, hkv * hd, d), 4: (nl, hkv * hd, d), 5: (nl, d, hq * hd),
              6: (nl, d), 7: (nl, ffn, d), 8: (nl, ffn, d), 9: (nl, d, ffn), 10: (d,)}
    r = R.refsm_create()
    for role, shape in shapes.items():
        per_layer = role not in (0, 10)
        n_l = nl if per_layer else 1
        n = int(np.prod(shape)) // n_l
        dst = np.ctypeslib.as_array(R.refsm_weight_ptr(r, role), shape=(int(np.prod(shape)),))
        for l in range(n_l):
            mean = 1.0 if role in (1, 6, 10) else 0.0
            dst[l * n:(l + 1) * n] = O.fill_normal(n, SEED, role * 4096 + l, 0.02, mean)
    # tied head (velox_c99_runner.c:210-217)
    emb = np.ctypeslib.as_array(R.refsm_weight_ptr(r, 0), shape=(V * d,))
    np.ctypeslib.as_array(R.refsm_weight_ptr(r, 11), shape=(V * d,))[:] = emb
    prompt = O.fill_tokens(N_PROMPT, SEED, 1 << 20, V)
    steps = []
    tok, pos = 0, 0
    for t in prompt:
        tok = R.refsm_prefill(r, int(t), pos)
        pos += 1
    out = [int(tok)]
    for s in range(N_NEW):
        lg = np.ctypeslib.as_array(R.refsm_logits(r), shape=(V,)).copy()
        top = np.argsort(-lg, kind="stable")[:5]
        steps.append({"pos": pos - 1, "token": int(tok), "sha256": hashlib.sha256(lg.tobytes()).hexdigest(),
                      "top5_ids": [int(i) for i in top], "top5_logits": [float(lg[i]) for i in top]})
        if s + 1 < N_NEW:
            tok = R.refsm_decode(r, int(tok), pos)
            pos += 1
            out.append(int(tok))
    R.refsm_destroy(r)
    doc = {"source": "src/runners/tinystories_smollm.c compiled with oracle/Makefile (gcc -O2 -mavx2 -mfma -ffp-contract=off)",
           "seed": SEED, "prompt": [int(t) for t in prompt], "tokens": out, "steps": steps}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "smollm_ref_golden.json")
    with open(path, "w") as f:
        json.dump(doc, f, indent=1)
    print("wrote", path, "tokens", out)


if __name__ == "__main__":
    main()
