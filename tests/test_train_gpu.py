"""GPU parity tests of the training path: libb200bpe.so through its C ABI against the CPU oracle."""
import numpy as np
import pytest

from gpu_bpe_b200 import BPETrainer, PreTokenizer, TrainerSession, _lib
from oracle import cpu_oracle as O
from oracle import wgsl_model as M
from tests.helpers import known_answers, random_symbols, small_text, tagged

pytestmark = pytest.mark.gpu


def run_gpu(engine, sym, merges, mode, **kw):
    s = TrainerSession.from_symbols(engine, sym, target_vocab_size=256 + merges, compat_mode=mode, **kw)
    try:
        m, c, early = s.run()
        final = s.symbols().copy()
    finally:
        s.destroy()
    return np.concatenate([m, c[:, None]], axis=1).tolist() if len(m) else [], early, final.tolist()


@pytest.mark.parametrize("case", known_answers(), ids=lambda c: c["input"])
@pytest.mark.parametrize("mode", ["literal", "fixed"])
def test_known_answers(engine, case, mode):
    merges, early, final = run_gpu(engine, np.array(tagged(case["input"]), np.uint32), 10, mode)
    assert merges == case[mode]["merges"]
    assert [hex(x) for x in final] == case[mode]["symbols"]
    assert early


# sizes either side of every structural edge: one 16-byte vector, one warp row (128), one span (512),
# one sub-tile (4,096), one, two and three tiles (12,288 each), the reference's workgroup (256) and its
# parallel/sequential scan switch (65,536)
@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 127, 128, 129, 255, 256, 257, 511, 513, 4095, 4096, 4097, 8191, 8193,
                               12287, 12288, 12289, 24575, 24576, 24577, 36863, 36864, 36865, 65535, 65536, 65537,
                               200_001])
@pytest.mark.parametrize("mode", ["literal", "fixed"])
def test_random_symbols_match_oracle(engine, n, mode):
    rng = np.random.default_rng(n + 17 * (mode == "fixed"))
    sym = random_symbols(rng, n, alphabet=5 if n < 70000 else 12, p_ws=0.15, p_nul=0.01)
    want = O.train(sym, 70, mode, threads=4)
    merges, early, final = run_gpu(engine, sym, 70, mode)
    assert merges == want["merges"].tolist()
    assert early == want["early_stop"]
    assert final == want["symbols"].tolist()


@pytest.mark.parametrize("drop", [0, 1, 2, 3, 4, 5, 6, 7])
def test_literal_limit_at_every_alignment(engine, drop):
    """Literal mode copies only the inputs below N - count: the first merge's count is set here so that the limit,
    and with it the end of the copy-out, lands on each of the four alignments of a 16-byte store, in the last tile
    of three."""
    n = 3 * 12288 - 5
    sym = np.full(n, 120 | 0x10000, np.uint32)  # every filler symbol starts a word: no pairs among them
    k = 40 + drop                               # k occurrences of the pair (a, b), apart from one another
    pos = np.arange(k) * 700 + 17
    sym[pos] = 97 | 0x10000
    sym[pos + 1] = 98
    want = O.train(sym, 3, "literal", threads=2)
    assert want["merges"].tolist() == [[97, 98, 256, k]] and want["early_stop"]
    merges, early, final = run_gpu(engine, sym, 3, "literal")
    assert merges == want["merges"].tolist() and final == want["symbols"].tolist() and early


@pytest.mark.parametrize("mode", ["literal", "fixed"])
def test_runs_of_equal_symbols(engine, mode):
    """a == b: a run of k equal symbols inside a word collapses to one new symbol."""
    sym = np.array(tagged("aaaaaaa|aa|aaa" * 700), np.uint32)
    want = O.train(sym, 20, mode)
    merges, early, final = run_gpu(engine, sym, 20, mode)
    assert merges == want["merges"].tolist() and final == want["symbols"].tolist() and early == want["early_stop"]


@pytest.mark.parametrize("batch,merges", [(128, 127), (128, 128), (128, 129), (128, 257), (7, 30), (1, 5)])
def test_batch_edges(engine, batch, merges):
    """Batch boundaries, odd/even merges per batch (the ping/pong parity continues across batches)."""
    rng = np.random.default_rng(batch * 1000 + merges)
    sym = random_symbols(rng, 30_000, alphabet=16, p_ws=0.1)
    for mode in ("literal", "fixed"):
        want = O.train(sym, merges, mode, threads=4)
        got = run_gpu(engine, sym, merges, mode, batch_merges=batch)
        assert got[0] == want["merges"].tolist() and got[2] == want["symbols"].tolist()


def test_graph_and_plain_launches_agree(engine):
    rng = np.random.default_rng(99)
    sym = random_symbols(rng, 100_000, alphabet=20, p_ws=0.1)
    a = run_gpu(engine, sym, 150, "literal")
    b = run_gpu(engine, sym, 150, "literal", flags=_lib.FLAG_NO_GRAPH)
    c = run_gpu(engine, sym, 150, "literal", flags=_lib.FLAG_TIME_KERNELS)
    assert a == b == c


def test_early_stop_when_best_count_drops_below_two(engine):
    sym = np.array(tagged("ab|ab|cd"), np.uint32)
    merges, early, _ = run_gpu(engine, sym, 50, "fixed")
    assert merges == [[97, 98, 256, 2]] and early


def test_id_exhaustion(engine):
    sym = np.array(tagged("abababab"), np.uint32)
    s = TrainerSession.from_symbols(engine, sym, target_vocab_size=0xFFFF + 5, first_token_id=0xFFFF, compat_mode="fixed")
    m, c, early = s.run()
    s.destroy()
    assert m.tolist() == [[97, 98, 0xFFFF]] and c.tolist() == [4] and early


def test_pair_counts_exact(engine):
    _, _, sym = small_text(2, 21, 1 << 20)
    s = TrainerSession.from_symbols(engine, sym, target_vocab_size=300)
    got = s.pair_counts()
    want = O.pair_counts(sym)
    assert {((k >> 32) << 16) | (k & 0xFFFF): v for k, v in got.items()} == want
    s.run(20)
    got2 = s.pair_counts()
    want2 = O.pair_counts(s.symbols())
    assert {((k >> 32) << 16) | (k & 0xFFFF): v for k, v in got2.items()} == want2
    s.destroy()


def test_small_table_grows(engine):
    """A table forced far too small fills up; the batch stops, the table doubles, the run resumes."""
    _, _, sym = small_text(2, 5, 1 << 19)
    want = O.train(sym, 40, "literal", threads=4)
    got = run_gpu(engine, sym, 40, "literal", table_log2=6)
    assert got[0] == want["merges"].tolist() and got[2] == want["symbols"].tolist()


@pytest.mark.parametrize("kind,seed,mb,merges", [(1, 1, 1, 1000), (2, 2, 4, 600)])
@pytest.mark.parametrize("mode", ["literal", "fixed"])
def test_text_corpus_matches_oracle(engine, kind, seed, mb, merges, mode):
    """Config-1-shaped (1 MiB ASCII, 1,000 merges) and a 4 MiB slice of the config-2 generator."""
    data, mask, sym = small_text(kind, seed, mb << 20)
    want = O.train(sym, merges, mode, threads=8)
    s = TrainerSession.create(engine, data, mask, target_vocab_size=256 + merges, compat_mode=mode)
    m, c, early = s.run()
    final = s.symbols().copy()
    # reset puts everything back: a second run gives the same list
    s.reset()
    m2, c2, early2 = s.run()
    s.destroy()
    assert np.concatenate([m, c[:, None]], axis=1).tolist() == want["merges"].tolist()
    assert early == want["early_stop"] and final.tolist() == want["symbols"].tolist()
    assert np.array_equal(m, m2) and np.array_equal(c, c2) and early == early2


def test_heuristic_boundaries_on_device(engine):
    """No mask → the byte-class heuristic runs on the device (the reference's Worker path)."""
    data, _, _ = small_text(2, 9, 1 << 18)
    sym = O.word_boundary(data)
    want = O.train(sym, 100, "literal", threads=4)
    s = TrainerSession.create(engine, data, None, target_vocab_size=356)
    first = s.symbols().copy()
    m, c, _ = s.run()
    s.destroy()
    assert np.array_equal(first, sym)
    assert np.concatenate([m, c[:, None]], axis=1).tolist() == want["merges"].tolist()


def test_trainer_api_mirror(engine):
    """BPETrainer.train: result object, vocabulary continuation, progress payload, empty-corpus error."""
    data, mask, sym = small_text(1, 3, 1 << 18)
    seen = []
    tr = BPETrainer(engine)
    res = tr.train(data, targetVocabSize=256 + 200, preTokenizer=PreTokenizer(normalize=False), onProgress=seen.append)
    want = O.train(sym, 200, "literal", threads=4)["merges"]
    assert res["merges"] == want[:, :3].tolist()
    assert res["vocabSize"] == 456 and len(res["vocab"]) == 456 and len(res["vocabStrings"]) == 456
    assert res["vocab"] == M.vocab_from_merges(want.tolist())
    assert [p["mergeIndex"] for p in seen] == [128, 200] and seen[-1]["totalMerges"] == 200
    assert seen[-1]["bestCount"] == int(want[-1, 3]) and seen[-1]["mergeString"] == res["vocabStrings"][-1]
    # a second train() on the same trainer continues the ids but starts again from the raw bytes (trainer.js:136,191,208)
    res2 = tr.train(data, targetVocabSize=456 + 10, preTokenizer=PreTokenizer(normalize=False))
    assert [m[2] for m in res2["merges"][-10:]] == list(range(456, 466))
    with pytest.raises(ValueError, match="No symbols to train on"):
        BPETrainer(engine).train(b"")
    assert "# Total tokens: 466" in tr.exportVocab()


@pytest.mark.parametrize("mode", ["literal", "fixed"])
def test_incrementally_maintained_table_stays_exact(engine, mode):
    """By default the pair table is updated in place around each merged occurrence; after any
    number of merges it must equal a fresh count of the live symbols."""
    _, _, sym = small_text(2, 23, 2 << 20)
    s = TrainerSession.from_symbols(engine, sym, target_vocab_size=256 + 400, compat_mode=mode)
    done = 0
    for step in (1, 2, 37, 128, 200):
        s.run(step - done if step > done else 0)
        done = step
        got = {((k >> 32) << 16) | (k & 0xFFFF): v for k, v in s.pair_counts().items()}
        assert got == O.pair_counts(s.symbols()), (mode, step)
    s.destroy()


@pytest.mark.parametrize("mode", ["literal", "fixed"])
def test_full_recount_and_incremental_agree(engine, mode):
    _, _, sym = small_text(1, 6, 1 << 20)
    want = O.train(sym, 300, mode, threads=8)
    a = run_gpu(engine, sym, 300, mode)
    b = run_gpu(engine, sym, 300, mode, flags=_lib.FLAG_FULL_RECOUNT)
    assert a == b
    assert a[0] == want["merges"].tolist() and a[2] == want["symbols"].tolist()


def test_incremental_with_frequent_equal_symbol_merges(engine):
    """Tiny alphabets make a == b merges common; each one forces a rebuild of the table."""
    rng = np.random.default_rng(123)
    sym = random_symbols(rng, 150_000, alphabet=3, p_ws=0.05)
    for mode in ("literal", "fixed"):
        want = O.train(sym, 120, mode, threads=4)
        got = run_gpu(engine, sym, 120, mode)
        assert got[0] == want["merges"].tolist() and got[2] == want["symbols"].tolist()


@pytest.mark.parametrize("mode", ["literal", "fixed"])
def test_long_run_candidate_list_and_batch_ends(engine, mode):
    """2,000 merges: the arg-max works from its candidate list, falls back to full scans when the
    list goes stale (the best count halves several times over such a run), and every batch still
    ends at a multiple of 128 merges."""
    _, _, sym = small_text(2, 41, 1 << 20)
    want = O.train(sym, 2000, mode, threads=8)
    s = TrainerSession.from_symbols(engine, sym, target_vocab_size=256 + 2000, compat_mode=mode)
    seen = []
    m, c, early = s.run(0, lambda p: seen.append(p.merge_index))
    final = s.symbols().copy()
    s.destroy()
    assert np.concatenate([m, c[:, None]], axis=1).tolist() == want["merges"].tolist()
    assert final.tolist() == want["symbols"].tolist()
    n = len(m)
    assert seen == [k for k in range(128, n, 128)] + [n]
