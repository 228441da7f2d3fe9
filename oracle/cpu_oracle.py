"""ctypes front end of the C++ oracle (oracle/bpe_oracle.cpp).  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the CPU-baseline leg of bench.py may import this.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build_oracle

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = build_oracle.OUT if os.path.exists(build_oracle.OUT) and not os.path.exists(build_oracle.SRC) \
            else build_oracle.build()
        L = C.CDLL(path)
        u32p, u8p, u64p = C.POINTER(C.c_uint32), C.POINTER(C.c_uint8), C.POINTER(C.c_uint64)
        L.oracle_word_boundary.argtypes = [u32p, C.c_uint64]
        L.oracle_word_boundary.restype = None
        L.oracle_pair_counts.argtypes = [u32p, C.c_uint64, u32p, u32p, C.c_uint64]
        L.oracle_pair_counts.restype = C.c_uint64
        L.oracle_train.argtypes = [u32p, C.c_uint64, C.c_uint32, C.c_int, C.c_uint32, C.c_int, C.c_double,
                                   u32p, u32p, u32p, u32p, u64p, C.POINTER(C.c_double)]
        L.oracle_train.restype = C.c_int
        L.oracle_encode.argtypes = [u8p, C.c_uint64, u8p, C.c_uint64, C.c_uint32, C.c_int, u32p, C.c_uint64]
        L.oracle_encode.restype = C.c_uint64
        _lib = L
    return _lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def word_boundary(byte_values: np.ndarray) -> np.ndarray:
    sym = np.ascontiguousarray(byte_values, dtype=np.uint32).copy()
    lib().oracle_word_boundary(_p(sym, C.c_uint32), sym.size)
    return sym


def pair_counts(sym: np.ndarray) -> dict[int, int]:
    sym = np.ascontiguousarray(sym, dtype=np.uint32)
    cap = 1 << 16
    while True:
        k = np.empty(cap, np.uint32)
        v = np.empty(cap, np.uint32)
        n = lib().oracle_pair_counts(_p(sym, C.c_uint32), sym.size, _p(k, C.c_uint32), _p(v, C.c_uint32), cap)
        if n <= cap:
            return dict(zip(k[:n].tolist(), v[:n].tolist()))
        cap = int(n)


def train(sym: np.ndarray, max_merges: int, mode: str = "literal", first_id: int = 256, threads: int = 1,
          max_seconds: float = 0.0, want_symbols: bool = True):
    """Returns dict(merges=(M,4) u32 [a,b,id,count], early_stop, symbols, seconds)."""
    sym = np.ascontiguousarray(sym, dtype=np.uint32)
    merges = np.zeros((max(1, max_merges), 4), np.uint32)
    nm, es = C.c_uint32(0), C.c_uint32(0)
    fn, sec = C.c_uint64(0), C.c_double(0)
    final = np.empty(max(1, sym.size), np.uint32) if want_symbols else None
    lib().oracle_train(_p(sym, C.c_uint32), sym.size, max_merges, {"literal": 0, "fixed": 1}[mode], first_id,
                       threads, max_seconds, _p(merges, C.c_uint32), C.byref(nm), C.byref(es),
                       _p(final, C.c_uint32) if want_symbols else None, C.byref(fn), C.byref(sec))
    return dict(merges=merges[: nm.value].copy(), early_stop=bool(es.value),
                symbols=final[: fn.value].copy() if want_symbols else None, n=fn.value, seconds=sec.value)


def encode(data: np.ndarray, trie: bytes, chunk_size: int, threads: int = 1) -> np.ndarray:
    data = np.ascontiguousarray(data, dtype=np.uint8)
    tb = np.frombuffer(trie, dtype=np.uint8)
    cap = max(1, data.size)
    out = np.empty(cap, np.uint32)
    n = lib().oracle_encode(_p(data, C.c_uint8), data.size, _p(tb, C.c_uint8), tb.size, chunk_size, threads,
                            _p(out, C.c_uint32), cap)
    if n == 2**64 - 1:
        raise ValueError("bad trie")
    return out[:n].copy()
