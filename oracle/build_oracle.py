"""Build recipe for the CPU oracle (test infrastructure): g++ → oracle/_build/liboracle.so.

The reference has no C/C++ sources (it is JavaScript + WGSL), so there is no `oracle/_ref`
build of the reference itself; this compiles only the restatements: bpe_oracle.cpp (the merge
loop pass by pass, the byte-class heuristic, the chunked trie encode), word_oracle.cpp (the
"fixed"-mode merge loop on the dictionary of distinct words, for full-size runs) and
replay_oracle.cpp (the merge-replay encoder).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "bpe_oracle.cpp")
SOURCES = [SRC] + [p for p in (os.path.join(HERE, "word_oracle.cpp"), os.path.join(HERE, "replay_oracle.cpp"))
                   if os.path.exists(p)]
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "liboracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(p) for p in SOURCES):
        return OUT
    cmd = ["g++", "-std=c++17", "-O3", "-march=x86-64-v3", "-shared", "-fPIC", "-pthread", *SOURCES, "-o", OUT]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
