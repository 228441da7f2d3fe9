"""Worker of the multi-GPU parity tests: run under torch.distributed.run, one rank per GPU.

Every rank builds the same seeded corpus, keeps its word-aligned span, trains jointly, and rank 0
checks the merge list, the gathered symbols and the exchanged pair counts against the CPU oracle.
Options come through B200BPE_TEST_* environment variables set by tests/test_multi_gpu.py.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from gpu_bpe_b200 import BPEEngine, TrainerSession, TrieTokenizer, _lib
    from gpu_bpe_b200.sharding import document_cuts, word_aligned_cuts
    from gpu_bpe_b200 import synth
    from oracle import cpu_oracle as O
    from oracle import wgsl_model as M
    from tests.helpers import small_text

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    env = os.environ.get
    merges = int(env("B200BPE_TEST_MERGES", "300"))
    exchange = env("B200BPE_TEST_EXCHANGE", "peer")
    first_cap = int(env("B200BPE_TEST_EXCHANGE_CAP", "0"))
    table_log2 = int(env("B200BPE_TEST_TABLE_LOG2", "0"))
    batch = int(env("B200BPE_TEST_BATCH", "128"))
    data, mask, sym = small_text(2, 41, int(env("B200BPE_TEST_CORPUS_KIB", "4096")) << 10)
    if env("B200BPE_TEST_ONE_WORD"):
        # one single word: every cut but the first falls at the end, so the other ranks' spans are empty
        data = np.frombuffer(b"abcabcabcabdabcabdabcabcabd" * 40, np.uint8).copy()
        mask = np.zeros(data.size, np.uint8)
        mask[0] = 1
        sym = data.astype(np.uint32) | (mask.astype(np.uint32) << 16)
    cuts = word_aligned_cuts(mask, world)
    lo, hi = int(cuts[rank]), int(cuts[rank + 1])

    uid = [BPEEngine.make_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    engine = BPEEngine(local).init_distributed(rank, world, uid[0])

    s = TrainerSession.create(engine, data[lo:hi], mask[lo:hi], target_vocab_size=256 + merges, compat_mode="fixed",
                              flags=_lib.FLAG_NCCL_EXCHANGE if exchange == "nccl" else 0, exchange_cap=first_cap,
                              table_log2=table_log2, batch_merges=batch)
    kind = s.exchange_kind()
    assert kind == exchange, f"asked for the {exchange} exchange, got {kind}"
    # exchanged counts before any merge: the union of the ranks' owned partitions is the global histogram
    # (with buckets or tables forced far too small the one-shot count exchange gives up by design; the run resizes them)
    tiny = bool(first_cap) or bool(table_log2)
    mine = {} if tiny else s.pair_counts()
    parts = [None] * world
    dist.all_gather_object(parts, mine)
    # first half, then the exchanged counts of the half-trained corpus (kept up to date by the merge
    # kernels by now; they must survive being read), then the rest
    m1, c1, _ = s.run(merges // 2)
    mid_counts = {} if tiny else s.pair_counts()
    mid_syms = s.symbols().copy()
    mids = [None] * world
    dist.all_gather_object(mids, (mid_counts, mid_syms))
    m2, c2, early = s.run()
    m, c = np.concatenate([m1, m2]), np.concatenate([c1, c2])
    final = s.symbols().copy()
    finals = [None] * world
    dist.all_gather_object(finals, final)
    lists = [None] * world
    dist.all_gather_object(lists, np.concatenate([m, c[:, None]], axis=1).tolist())
    # a reset puts everything back: the second run gives the same list
    s.reset()
    m3, c3, _ = s.run()
    assert np.array_equal(m3, m) and np.array_equal(c3, c), "a run after reset differs"
    s.destroy()

    # encoding shards documents; no collective on the data path
    vocab = M.vocab_from_merges(lists[0])
    tok = TrieTokenizer.fromVocab(engine, vocab)
    offs = synth.doc_offsets(9, data.size, 512, 1.0)
    dc = document_cuts(offs, world)
    d0, d1 = int(dc[rank]), int(dc[rank + 1])
    toks, toff = tok.encodeBatch(data[int(offs[d0]):int(offs[d1])], offs[d0:d1 + 1] - offs[d0])
    enc = [None] * world
    dist.all_gather_object(enc, (toks, toff))
    chunk = tok.chunkSize
    tok.destroy()

    if rank == 0:
        want = O.train(sym, merges, "fixed", threads=8)
        assert all(l == lists[0] for l in lists), "ranks disagree on the merge list"
        assert lists[0] == want["merges"].tolist(), "merge list differs from the oracle"
        assert np.array_equal(np.concatenate(finals), want["symbols"]), "symbols differ from the oracle"
        merged = {}
        for p in parts:
            for k, v in p.items():
                assert k not in merged, "a pair is owned by two ranks"
                merged[((k >> 32) << 16) | (k & 0xFFFF)] = v
        assert tiny or merged == O.pair_counts(sym), "exchanged pair counts differ from the oracle"
        mid = {}
        for cnts, _ in mids:
            for k, v in cnts.items():
                assert k not in mid, "a pair is owned by two ranks (mid-run)"
                mid[((k >> 32) << 16) | (k & 0xFFFF)] = v
        assert tiny or mid == O.pair_counts(np.concatenate([sy for _, sy in mids])), "mid-run exchanged pair counts differ from the oracle"
        trie = M.compile_vocab_to_trie(vocab)
        for r in range(world):
            t, to = enc[r]
            for d in range(int(dc[r]), int(dc[r + 1])):
                a, b = int(offs[d]), int(offs[d + 1])
                k = d - int(dc[r])
                ref = O.encode(data[a:b], trie, chunk) if b > a else np.zeros(0, np.uint32)
                assert np.array_equal(t[int(to[k]):int(to[k + 1])], ref), f"document {d} differs"
        print(f"multi-gpu ok: world={world} exchange={kind} merges={len(lists[0])} early={early}", flush=True)
    dist.barrier()
    engine.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
