"""Builds libvelox_b200.so in-tree with nvcc for sm_100a (no torch, no JIT cache).

    python -m velox_b200.build [--force] [--verbose]

The shared object lands beside this file so that it travels with the source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB = os.path.join(_HERE, "libvelox_b200.so")
RUNNER = os.path.join(_HERE, "velox_b200_runner")
SOURCES = ["vb_basic.cu", "vb_gemv.cu", "vb_gemv_fast.cu", "vb_gemv_imma.cu", "vb_attn.cu", "vb_attn_prefill.cu", "vb_mla.cu", "vb_gemm_tc.cu", "vb_engine.cu", "vb_nccl.cu", "vb_tp.cu", "vb_sample.cu", "vb_spec.cu", "vb_gguf.cu", "vb_fused.cu", "vb_mla_decode.cu", "vb_gemm_i8.cu", "vb_mla_tc.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "--use_fast_math=false", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(_HERE, "..", "include", "velox_b200.h"),
                                                                  os.path.join(_HERE, "runner", "velox_b200_runner.cpp")]
    if not os.path.exists(RUNNER):
        return True
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    objs = []
    env = dict(os.environ)
    # the image exports CC/CXX pointing at a toolchain wrapper; let nvcc pick the system g++
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [_nvcc(), *[f for f in NVCC_FLAGS if f != "--use_fast_math=false"], "-ccbin", "/usr/bin/g++", "-c",
               os.path.join(CSRC, src), "-o", obj]
        procs.append((src, cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, text=True)))
    failed = False
    for src, cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write("nvcc failed for %s:\n%s\n%s\n" % (src, " ".join(cmd), out))
        elif verbose:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("nvcc failed")
    link = [_nvcc(), "-shared", "-ccbin", "/usr/bin/g++", "-o", LIB, *objs, "-lcudart", "-ldl"]
    subprocess.check_call(link, env=env)
    build_runner()
    return LIB


def build_runner() -> str:
    """The stand-alone C++ runner over the C ABI (plain g++; it links against the shared library only)."""
    src = os.path.join(_HERE, "runner", "velox_b200_runner.cpp")
    cmd = ["/usr/bin/g++", "-O2", "-std=c++17", "-Wall", "-I", os.path.join(_HERE, "..", "include"), src, "-o", RUNNER,
           "-L", _HERE, "-lvelox_b200", "-Wl,-rpath,$ORIGIN"]
    subprocess.check_call(cmd)
    return RUNNER


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
