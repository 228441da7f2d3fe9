"""GPU parity tests of the merge-replay encoder (b200bpe_replay_*, the reference's TokenizerManager.encode)
against the CPU oracle and the hand-derived cases."""
import json
import os

import numpy as np
import pytest

from gpu_bpe_b200 import _lib
from gpu_bpe_b200.tokenizer_manager import TokenizerManager
from oracle import cpu_oracle as O
from tests.helpers import GOLDEN, small_text

pytestmark = pytest.mark.gpu


def test_known_answers(engine):
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        cases = json.load(f)["replay"]
    for c in cases:
        tm = TokenizerManager(engine, {"merges": c["merges"], "vocab": None, "vocabStrings": None})
        r = tm.encode(c["text"])
        assert r["tokens"] == c["tokens"] and r["text"] == c["text"], c["text"]
        tm.destroy()


def test_no_model_raises(engine):
    with pytest.raises(RuntimeError, match="No trained model available"):
        TokenizerManager(engine).encode("abc")


@pytest.mark.parametrize("n", [1, 2, 3, 2047, 2048, 2049, 4097, 100_003, 1_000_000])
def test_trained_merges_on_text(engine, n):
    """Merges learned by the oracle trainer, replayed over text of sizes either side of the tile edges."""
    _, _, sym = small_text(2, 31, 1 << 20)
    merges = O.train(sym, 800, "fixed", threads=8)["merges"][:, :3]
    data, _, _ = small_text(2, 95, max(n, 1))
    data = data[:n]
    tm = TokenizerManager(engine, {"merges": merges.tolist()})
    got = tm.encodeBytes(data)
    assert np.array_equal(got, O.replay_encode(data, merges))
    assert tm.lastRounds() <= 800
    tm.destroy()


def test_runs_of_equal_tokens_pair_from_the_left(engine):
    """a == b rules on long runs, with run lengths and positions that cross thread, warp and tile edges."""
    rng = np.random.default_rng(12)
    parts = []
    for _ in range(400):
        parts.append(np.full(int(rng.integers(1, 70)), 97, np.uint8))
        parts.append(rng.integers(98, 101, int(rng.integers(1, 4)), dtype=np.uint8))
    parts.append(np.full(9000, 97, np.uint8))      # a run longer than four tiles
    parts.append(np.array([98], np.uint8))
    parts.append(np.full(4097, 97, np.uint8))
    data = np.concatenate(parts)
    merges = [[97, 97, 256], [256, 256, 257], [257, 257, 258], [98, 97, 259], [258, 258, 260], [97, 98, 261]]
    tm = TokenizerManager(engine, {"merges": merges})
    assert np.array_equal(tm.encodeBytes(data), O.replay_encode(data, merges))
    tm.destroy()


def test_random_rules_on_a_tiny_alphabet(engine):
    rng = np.random.default_rng(5)
    for trial in range(6):
        data = rng.integers(97, 100, int(rng.integers(1, 30_000)), dtype=np.uint8)
        merges, ids = [], [97, 98, 99]
        for r in range(40):
            merges.append([int(rng.choice(ids)), int(rng.choice(ids)), 256 + r])
            ids.append(256 + r)
        tm = TokenizerManager(engine, {"merges": merges})
        assert np.array_equal(tm.encodeBytes(data), O.replay_encode(data, merges)), trial
        tm.destroy()


def test_lists_no_trainer_could_produce_are_refused(engine):
    for bad in ([[97, 98, 97]],                       # makes a byte value
                [[97, 98, 256], [99, 100, 256]],      # makes the same id twice
                [[257, 98, 256], [97, 99, 257]]):     # uses an id that only a later rule makes
        with pytest.raises(_lib.B200BPEError) as ei:
            TokenizerManager(engine, {"merges": bad})
        assert ei.value.status_name == "BAD_ARG"
