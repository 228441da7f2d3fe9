"""CPU tests of the multi-GPU host logic: sharding rules, the packed arg-max word, and the
per-merge protocol (local count → exchange by owner → all-reduce max → local merge) run as two
gloo ranks, compared with the single-process oracle."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gpu_bpe_b200.sharding import document_cuts, owner_of_pair, pack_best, unpack_best, word_aligned_cuts
from oracle import cpu_oracle as O
from tests.helpers import random_symbols, small_text

W = 0x10000


def test_word_aligned_cuts():
    mask = np.zeros(100, np.uint8)
    mask[[0, 10, 49, 51, 90]] = 1
    assert word_aligned_cuts(mask, 2).tolist() == [0, 51, 100]
    assert word_aligned_cuts(mask, 4).tolist() == [0, 49, 51, 90, 100]
    assert word_aligned_cuts(mask, 1).tolist() == [0, 100]
    one = np.zeros(10, np.uint8)
    one[0] = 1                                   # a single word cannot be cut: the other ranks get nothing
    assert word_aligned_cuts(one, 4).tolist() == [0, 10, 10, 10, 10]
    assert word_aligned_cuts(np.zeros(0, np.uint8), 3).tolist() == [0, 0, 0, 0]


def test_document_cuts():
    offs = np.array([0, 10, 10, 50, 60, 100], np.uint64)
    c = document_cuts(offs, 2)
    assert c[0] == 0 and c[-1] == 5 and 0 <= c[1] <= 5
    assert document_cuts(offs, 8)[-1] == 5 and np.all(np.diff(document_cuts(offs, 8)) >= 0)


def test_packed_argmax_order_is_the_reference_order():
    """max over the packed word == larger count first, then the smaller (a << 16 | b)."""
    rng = np.random.default_rng(0)
    cands = [(int(rng.integers(1, 5)), int(rng.integers(0, 65536)), int(rng.integers(0, 65536))) for _ in range(500)]
    best = max(cands, key=lambda t: (t[0], -((t[1] << 16) | t[2])))
    assert unpack_best(max(pack_best(*c) for c in cands)) == best
    assert unpack_best(pack_best(7, 65535, 0)) == (7, 65535, 0)
    assert unpack_best(0)[0] == 0


def test_owner_is_a_partition():
    owners = [owner_of_pair(a, b, 8) for a in range(1, 60) for b in range(1, 60)]
    assert set(owners) == set(range(8))
    assert all(owner_of_pair(a, b, 1) == 0 for a in (1, 500) for b in (2, 65535))


def apply_merge(sym: np.ndarray, a: int, b: int, new: int) -> np.ndarray:
    """One merge with snapshot semantics, compaction over every position ("fixed" mode)."""
    if sym.size < 2:
        return sym
    tok, ws = sym & 0xFFFF, (sym & W) != 0
    match = np.zeros(sym.size, bool)
    match[:-1] = (tok[:-1] == a) & (tok[1:] == b) & ~ws[1:]
    invalid = np.zeros(sym.size, bool)
    invalid[1:] = match[:-1]
    out = np.where(match, new | (sym & W), sym).astype(np.uint32)
    return out[~invalid]


def _rank_main(rank, world, port, sym, cuts, merges, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        local = sym[cuts[rank]:cuts[rank + 1]].copy()
        log, next_id = [], 256
        for _ in range(merges):
            counts = O.pair_counts(local)                      # k_pair_count
            outbox = [dict() for _ in range(world)]            # k_partition
            for k, v in counts.items():
                outbox[owner_of_pair(k >> 16, k & 0xFFFF, world)][k] = v
            gathered = [None] * world
            dist.all_gather_object(gathered, outbox)           # stands in for the all-to-all
            owned = {}
            for src in range(world):                           # k_accumulate
                for k, v in gathered[src][rank].items():
                    owned[k] = owned.get(k, 0) + v
            best = 0
            for k, v in owned.items():                         # k_argmax_setup (mode 1)
                best = max(best, pack_best(v, k >> 16, k & 0xFFFF))
            allw = [None] * world                              # gloo has no uint64 max: gather and take max
            dist.all_gather_object(allw, best)
            cnt, a, b = unpack_best(max(allw))                 # all-reduce max
            if cnt < 2 or next_id > 0xFFFF:
                break
            log.append([a, b, next_id, cnt])
            local = apply_merge(local, a, b, next_id)          # k_merge_compact
            next_id += 1
        finals = [None] * world
        dist.all_gather_object(finals, local)
        if rank == 0:
            q.put((log, np.concatenate(finals)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_protocol_matches_single_process_oracle(world):
    data, mask, sym = small_text(2, 17, 1 << 16)
    merges = 25
    cuts = word_aligned_cuts(mask, world)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000) + world
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, sym, cuts, merges, q)) for r in range(world)]
    for p in procs:
        p.start()
    log, final = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = O.train(sym, merges, "fixed")
    assert log == want["merges"].tolist()
    assert np.array_equal(final, want["symbols"])


def test_apply_merge_helper_matches_oracle():
    rng = np.random.default_rng(4)
    sym = random_symbols(rng, 5000, alphabet=3, p_ws=0.2)
    want = O.train(sym, 6, "fixed")
    cur = sym
    for a, b, nid, _c in want["merges"].tolist():
        cur = apply_merge(cur, a, b, nid)
    assert np.array_equal(cur, want["symbols"])
