"""Build recipe for the CPU oracle (test infrastructure): g++ → oracle/_build/liboracle.so.

The reference has no C/C++ sources (it is JavaScript + WGSL), so there is no `oracle/_ref`
build of the reference itself; this compiles only the restatement in bpe_oracle.cpp.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "bpe_oracle.cpp")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "liboracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = ["g++", "-std=c++17", "-O3", "-march=x86-64-v3", "-shared", "-fPIC", "-pthread", SRC, "-o", OUT]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
