"""In-tree build of the CUDA library (sm_100a only) and the host-only synthetic-corpus helper.

    python -m gpu_bpe_b200.build [--force]

Produces gpu_bpe_b200/libb200bpe.so (nvcc, CUDA runtime linked statically, NCCL resolved at run
time with dlopen) and gpu_bpe_b200/libb200bpe_synth.so (g++: synthetic corpora and the host
pre-tokeniser, no CUDA).  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libb200bpe.so")
SYNTH = os.path.join(PKG, "libb200bpe_synth.so")

CUDA_SOURCES = ["api.cu", "train.cu", "encode.cu", "replay.cu", "trie.cpp", "pretok.cpp", "pretok_gpu.cu", "export.cpp"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared", "-cudart", "static"]


def _newer(out: str, deps: list[str]) -> bool:
    if not os.path.exists(out):
        return False
    t = os.path.getmtime(out)
    return all(os.path.getmtime(d) <= t for d in deps)


def _deps() -> list[str]:
    d = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    d.append(os.path.join(PKG, "..", "include", "b200bpe.h"))
    return d


def build(force: bool = False, verbose: bool = False) -> tuple[str, str]:
    deps = _deps()
    if force or not _newer(LIB, deps):
        srcs = [os.path.join(CSRC, f) for f in CUDA_SOURCES if os.path.exists(os.path.join(CSRC, f))]
        cmd = ["nvcc", *NVCC_FLAGS, *( ["-Xptxas", "-v"] if verbose else []), *srcs, "-o", LIB, "-ldl"]
        subprocess.check_call(cmd)
    # host-only helpers (no CUDA): the synthetic corpora and the host pre-tokeniser, for callers that
    # must not load the CUDA library (the CPU arm of the benchmark)
    host_srcs = [os.path.join(CSRC, f) for f in ("synth.cpp", "pretok.cpp")]
    if force or not _newer(SYNTH, host_srcs + [os.path.join(CSRC, "unicode_classes.inc")]):
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-shared", "-fPIC", "-pthread", *host_srcs, "-o", SYNTH])
    return LIB, SYNTH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
