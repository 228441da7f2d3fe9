"""Host-side sharding rules for multi-GPU jobs (one process per GPU).

Training: the corpus is cut at word starts into one contiguous span per rank, balanced by
symbol count.  Pairs never cross a word start (train.wgsl:395,483,493 of the reference), so
counting and merging a span needs nothing from its neighbours; only the per-merge count
exchange and the 24-byte all-reduce connect the ranks.

Encoding: documents are independent; a contiguous run of documents goes to each rank, balanced
by bytes, and there is no collective on the data path.

Also here: the packing of (count, pair) into one 64-bit word whose integer maximum is the
reference's arg-max order (larger count, then smaller pair id; train.wgsl:83-85).
"""
from __future__ import annotations

import numpy as np


def word_aligned_cuts(word_starts: np.ndarray, world: int) -> np.ndarray:
    """→ world + 1 offsets; cut r is the first word start at or after r * n / world."""
    n = int(word_starts.size)
    cuts = np.zeros(world + 1, np.int64)
    cuts[world] = n
    if n == 0:
        return cuts
    starts = np.flatnonzero(word_starts)
    for r in range(1, world):
        target = (n * r) // world
        k = np.searchsorted(starts, target, side="left")
        cuts[r] = int(starts[k]) if k < starts.size else n
    for r in range(1, world + 1):
        cuts[r] = max(cuts[r], cuts[r - 1])
    return cuts


def document_cuts(doc_offsets: np.ndarray, world: int) -> np.ndarray:
    """→ world + 1 document indices; rank r encodes documents [cuts[r], cuts[r + 1])."""
    offs = np.asarray(doc_offsets, np.int64)
    n_docs = offs.size - 1
    total = int(offs[-1] - offs[0])
    cuts = np.zeros(world + 1, np.int64)
    cuts[world] = n_docs
    for r in range(1, world):
        target = offs[0] + (total * r) // world
        cuts[r] = min(n_docs, int(np.searchsorted(offs, target, side="left")))
    for r in range(1, world + 1):
        cuts[r] = max(cuts[r], cuts[r - 1])
    return cuts


def pack_best(count: int, a: int, b: int) -> int:
    """(count, pair) → the word the ranks all-reduce with max."""
    pair32 = ((a & 0xFFFF) << 16) | (b & 0xFFFF)
    return ((count & 0xFFFFFFFF) << 32) | ((~pair32) & 0xFFFFFFFF)


def unpack_best(word: int) -> tuple[int, int, int]:
    count = (word >> 32) & 0xFFFFFFFF
    pair32 = (~word) & 0xFFFFFFFF
    return count, pair32 >> 16, pair32 & 0xFFFF


def owner_of_pair(a: int, b: int, world: int) -> int:
    """Rank that owns pair (a, b) in the count exchange: the hash the device code uses."""
    m = 0xFFFFFFFF
    key_lo, key_hi = b & m, a & m
    x = (key_lo ^ ((key_hi * 0x9E3779B1) & m)) & m
    x ^= x >> 16
    x = (x * 0x7FEB352D) & m
    x ^= x >> 15
    x = (x * 0x846CA68B) & m
    x ^= x >> 16
    return (((x * 0x9E3779B1) & m) * world) >> 32
