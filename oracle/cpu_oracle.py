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
        L.oracle_pair_counts_mt.argtypes = [u32p, C.c_uint64, u32p, u32p, C.c_uint64, C.c_int]
        L.oracle_pair_counts_mt.restype = C.c_uint64
        L.oracle_encode_batch.argtypes = [u8p, u64p, C.c_uint32, u8p, C.c_uint64, C.c_uint32, C.c_int, u32p, C.c_uint64, u64p]
        L.oracle_encode_batch.restype = C.c_uint64
        L.oracle_train.argtypes = [u32p, C.c_uint64, C.c_uint32, C.c_int, C.c_uint32, C.c_int, C.c_double,
                                   u32p, u32p, u32p, u32p, u64p, C.POINTER(C.c_double)]
        L.oracle_train.restype = C.c_int
        L.oracle_encode.argtypes = [u8p, C.c_uint64, u8p, C.c_uint64, C.c_uint32, C.c_int, u32p, C.c_uint64]
        L.oracle_encode.restype = C.c_uint64
        L.word_oracle_train_symbols.argtypes = [u32p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_int, u32p, u32p, u32p, u64p,
                                                u64p, u64p]
        L.word_oracle_train_symbols.restype = C.c_int
        L.word_oracle_train_bytes.argtypes = [u8p, u8p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_int, u32p, u32p, u32p,
                                              u64p, u64p, u64p]
        L.word_oracle_train_bytes.restype = C.c_int
        L.oracle_replay_encode.argtypes = [u8p, C.c_uint64, u32p, C.c_uint32, u32p, C.c_uint64]
        L.oracle_replay_encode.restype = C.c_uint64
        _lib = L
    return _lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def word_boundary(byte_values: np.ndarray) -> np.ndarray:
    sym = np.ascontiguousarray(byte_values, dtype=np.uint32).copy()
    lib().oracle_word_boundary(_p(sym, C.c_uint32), sym.size)
    return sym


def pair_counts(sym: np.ndarray, threads: int = 1) -> dict[int, int]:
    sym = np.ascontiguousarray(sym, dtype=np.uint32)
    cap = 1 << 16
    while True:
        k = np.empty(cap, np.uint32)
        v = np.empty(cap, np.uint32)
        n = lib().oracle_pair_counts_mt(_p(sym, C.c_uint32), sym.size, _p(k, C.c_uint32), _p(v, C.c_uint32), cap, threads)
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


def encode_batch(data: np.ndarray, doc_offsets: np.ndarray, trie: bytes, chunk_size: int, threads: int = 1):
    """Every document encoded as its own encode() call → (tokens, token offsets per document)."""
    data = np.ascontiguousarray(data, dtype=np.uint8)
    offs = np.ascontiguousarray(doc_offsets, dtype=np.uint64)
    tb = np.frombuffer(trie, dtype=np.uint8)
    cap = max(1, int(offs[-1] - offs[0]))
    out = np.empty(cap, np.uint32)
    toff = np.zeros(offs.size, np.uint64)
    n = lib().oracle_encode_batch(_p(data, C.c_uint8), _p(offs, C.c_uint64), offs.size - 1, _p(tb, C.c_uint8), tb.size,
                                  chunk_size, threads, _p(out, C.c_uint32), cap, _p(toff, C.c_uint64))
    if n == 2**64 - 1:
        raise ValueError("bad trie")
    return out[:n].copy(), toff


def train_words(sym_or_bytes: np.ndarray, max_merges: int, word_starts: np.ndarray | None = None, first_id: int = 256,
                threads: int = 1):
    """The "fixed"-mode merge loop on the dictionary of distinct words (oracle/word_oracle.cpp): the same
    merge list as train(..., "fixed"), fast enough for full-size corpora.  Pass tagged u32 symbols, or u8
    bytes with their word-start mask.  Returns dict(merges=(M,4) u32 [a,b,id,count], early_stop, n,
    distinct_words, distinct_pairs)."""
    merges = np.zeros((max(1, max_merges), 4), np.uint32)
    nm, es = C.c_uint32(0), C.c_uint32(0)
    fn, dw, dp = C.c_uint64(0), C.c_uint64(0), C.c_uint64(0)
    if word_starts is None:
        sym = np.ascontiguousarray(sym_or_bytes, dtype=np.uint32)
        lib().word_oracle_train_symbols(_p(sym, C.c_uint32), sym.size, max_merges, first_id, threads,
                                        _p(merges, C.c_uint32), C.byref(nm), C.byref(es), C.byref(fn), C.byref(dw),
                                        C.byref(dp))
    else:
        b = np.ascontiguousarray(sym_or_bytes, dtype=np.uint8)
        w = np.ascontiguousarray(word_starts, dtype=np.uint8)
        assert b.size == w.size
        lib().word_oracle_train_bytes(_p(b, C.c_uint8), _p(w, C.c_uint8), b.size, max_merges, first_id, threads,
                                      _p(merges, C.c_uint32), C.byref(nm), C.byref(es), C.byref(fn), C.byref(dw),
                                      C.byref(dp))
    return dict(merges=merges[: nm.value].copy(), early_stop=bool(es.value), n=fn.value, distinct_words=dw.value,
                distinct_pairs=dp.value)


def replay_encode(data: np.ndarray, merges) -> np.ndarray:
    """Merge-replay encoding (oracle/replay_oracle.cpp): merges = rows [a, b, new_id] in learned order."""
    data = np.ascontiguousarray(data, dtype=np.uint8)
    m = np.ascontiguousarray(np.asarray(merges, dtype=np.uint32).reshape(-1, 3)[:, :3] if len(merges) else
                             np.zeros((0, 3), np.uint32))
    out = np.empty(max(1, data.size), np.uint32)
    n = lib().oracle_replay_encode(_p(data, C.c_uint8), data.size, _p(m, C.c_uint32), m.shape[0], _p(out, C.c_uint32),
                                   out.size)
    return out[:n].copy()
