"""The word-level oracle (oracle/word_oracle.cpp) and the golden merge lists it produced.

The golden lists of the large benchmark configurations come from the word-level restatement of the
"fixed"-mode merge loop, because the pass-by-pass oracle (oracle/bpe_oracle.cpp) would take days
there.  These tests tie the two together on corpora small enough for both, cover the cases where
they could drift apart (runs of equal symbols, words of one symbol, NUL symbols, no mask at all),
and check that the committed golden lists still are what the committed generator and oracles give.
"""
import hashlib
import json
import os

import numpy as np
import pytest

from oracle import cpu_oracle as O
from tests.helpers import GOLDEN, random_symbols, small_text, tagged


def _rows(r):
    return r["merges"].tolist()


@pytest.mark.parametrize("kind,seed,n,merges", [(1, 3, 1 << 18, 400), (2, 5, 1 << 19, 500), (5, 7, 1 << 18, 300)])
def test_text_corpora(kind, seed, n, merges):
    data, mask, sym = small_text(kind, seed, n)
    want = O.train(sym, merges, "fixed", threads=4, want_symbols=False)
    got = O.train_words(sym, merges, threads=4)
    assert _rows(got) == _rows(want) and got["early_stop"] == want["early_stop"]
    # the byte + mask entry point is the same thing
    assert _rows(O.train_words(data, merges, word_starts=mask, threads=4)) == _rows(want)


@pytest.mark.parametrize("n,alphabet,p_ws,p_nul", [(1, 3, 0.5, 0.0), (2, 2, 0.0, 0.0), (5000, 2, 0.1, 0.0), (5000, 3, 0.9, 0.0),
                                                 (20000, 4, 0.2, 0.05), (20000, 5, 0.0, 0.0)])
def test_random_symbols_with_runs_and_nuls(n, alphabet, p_ws, p_nul):
    """Tiny alphabets make long runs of equal symbols (a merge of two equal symbols collapses a whole run,
    train.wgsl:482-497), high word-start rates make one-symbol words, NUL symbols never pair (train.wgsl:393-398)."""
    rng = np.random.default_rng(n * 31 + alphabet)
    sym = random_symbols(rng, n, alphabet=alphabet, p_ws=p_ws, p_nul=p_nul)
    want = O.train(sym, 60, "fixed", threads=2, want_symbols=False)
    got = O.train_words(sym, 60, threads=2)
    assert _rows(got) == _rows(want) and got["early_stop"] == want["early_stop"]


def test_hand_cases():
    for text in ("aaaa", "aaa|aaa|aa", "ab|ab|abab|b", "abcabc|abc"):
        sym = np.array(tagged(text), np.uint32)
        assert _rows(O.train_words(sym, 10)) == _rows(O.train(sym, 10, "fixed", want_symbols=False)), text


def test_golden_lists_are_intact():
    """Every committed list carries the hash of its own contents, and new ids are consecutive by construction."""
    for name in sorted(os.listdir(GOLDEN)):
        if not (name.startswith("config") and name.endswith(".npz")):
            continue
        g = np.load(os.path.join(GOLDEN, name))
        meta = json.loads(bytes(g["meta"]).decode())
        rows = np.stack([g["a"].astype(np.uint32), g["b"].astype(np.uint32), g["count"].astype(np.uint32)], axis=1)
        assert hashlib.sha256(np.ascontiguousarray(rows).tobytes()).hexdigest() == meta["sha256"], name
        assert rows.shape[0] > 0 and int(rows[:, 2].min()) >= 2, name
        # a pair only uses ids that exist when it is merged
        ids = 256 + np.arange(rows.shape[0])
        assert (rows[:, 0] < ids).all() and (rows[:, 1] < ids).all(), name


def test_config2_golden_list_from_the_committed_generator():
    """The first merges of config 2 (64 MiB), recomputed here from the committed corpus generator and host
    pre-tokeniser: 300 by the word-level oracle, 12 by the pass-by-pass oracle, both modes."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_config_merges", os.path.join(GOLDEN, "make_config_merges.py"))
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    data, mask = mk.corpus(2)
    threads = min(8, os.cpu_count() or 1)
    fixed = np.load(os.path.join(GOLDEN, "config2_fixed.npz"))
    gold = np.stack([fixed["a"], fixed["b"], 256 + np.arange(fixed["a"].size), fixed["count"]], axis=1).astype(np.uint32)
    got = O.train_words(data, 300, word_starts=mask, threads=threads)["merges"]
    assert got.tolist() == gold[:300].tolist()
    sym = data.astype(np.uint32) | (mask.astype(np.uint32) << 16)
    for mode in ("fixed", "literal"):
        g = np.load(os.path.join(GOLDEN, f"config2_{mode}.npz"))
        want = np.stack([g["a"], g["b"], 256 + np.arange(g["a"].size), g["count"]], axis=1).astype(np.uint32)[:12]
        assert O.train(sym, 12, mode, threads=threads, want_symbols=False)["merges"].tolist() == want.tolist(), mode
