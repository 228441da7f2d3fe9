"""Seeded synthetic corpora (host code in libb200bpe_synth.so) for tests and benchmarks."""
from __future__ import annotations

import os

import numpy as np

from . import _lib


def corpus(kind: int, seed: int, n_bytes: int, threads: int | None = None) -> np.ndarray:
    """kind 1: ASCII; 2: UTF-8 script mix; 5: heavy-tailed mix with base64-like strings."""
    out = np.empty(n_bytes, np.uint8)
    rc = _lib.synth().b200bpe_synth_corpus(kind, seed, n_bytes, out.ctypes.data, threads or os.cpu_count() or 1)
    if rc:
        raise ValueError("bad synthetic corpus arguments")
    return out


def corpus_range(kind: int, seed: int, n_bytes: int, offset: int, length: int, threads: int | None = None) -> np.ndarray:
    """Bytes [offset, offset + length) of corpus(kind, seed, n_bytes), without making the rest."""
    out = np.empty(length, np.uint8)
    rc = _lib.synth().b200bpe_synth_corpus_range(kind, seed, n_bytes, offset, length, out.ctypes.data,
                                                 threads or os.cpu_count() or 1)
    if rc:
        raise ValueError("bad synthetic corpus arguments")
    return out


def doc_offsets(seed: int, n_bytes: int, n_docs: int, sigma: float = 1.0) -> np.ndarray:
    out = np.zeros(n_docs + 1, np.uint64)
    rc = _lib.synth().b200bpe_synth_doc_offsets(seed, n_bytes, n_docs, sigma, out.ctypes.data)
    if rc:
        raise ValueError("bad document-offset arguments")
    return out
