"""CPU tests: the two CPU restatements against the hand-derived known answers and each other."""
import numpy as np
import pytest

from oracle import cpu_oracle as O
from oracle import wgsl_model as M
from tests.helpers import known_answers, random_symbols, tagged


@pytest.mark.parametrize("case", known_answers(), ids=lambda c: c["input"])
@pytest.mark.parametrize("mode", ["literal", "fixed"])
def test_known_answers(case, mode):
    sym = tagged(case["input"])
    want = case[mode]
    merges, early, final = M.train(sym, 10, literal=(mode == "literal"))
    assert merges == want["merges"]
    assert [hex(x) for x in final] == want["symbols"]
    assert early
    r = O.train(np.array(sym, np.uint32), 10, mode)
    assert r["merges"].tolist() == want["merges"]
    assert [hex(int(x)) for x in r["symbols"]] == want["symbols"]
    assert r["early_stop"]


@pytest.mark.parametrize("mode", ["literal", "fixed"])
@pytest.mark.parametrize("n", [1, 2, 3, 255, 256, 257, 511, 513, 1500])
def test_cpp_oracle_matches_dispatch_model(mode, n):
    rng = np.random.default_rng(n * 7 + (mode == "fixed"))
    for trial in range(3):
        sym = random_symbols(rng, n, alphabet=4 + trial, p_ws=0.15, p_nul=0.02 * trial)
        merges, early, final = M.train(sym.tolist(), 40, literal=(mode == "literal"))
        r = O.train(sym, 40, mode, threads=1 + trial)
        assert r["merges"].tolist() == merges
        assert r["symbols"].tolist() == final
        assert r["early_stop"] == early


def test_batch_edges_and_pingpong():
    """129 merges cross the 128-merge batch edge with an odd count in the second batch."""
    rng = np.random.default_rng(5)
    sym = random_symbols(rng, 6000, alphabet=12, p_ws=0.1)
    for mode in ("literal", "fixed"):
        merges, early, final = M.train(sym.tolist(), 129, literal=(mode == "literal"))
        r = O.train(sym, 129, mode, threads=2)
        assert len(merges) == 129 and not early
        assert r["merges"].tolist() == merges and r["symbols"].tolist() == final


def test_threads_do_not_change_results():
    rng = np.random.default_rng(11)
    sym = random_symbols(rng, 50_000, alphabet=20, p_ws=0.12)
    base = O.train(sym, 60, "literal", threads=1)
    for t in (2, 5, 8):
        r = O.train(sym, 60, "literal", threads=t)
        assert np.array_equal(r["merges"], base["merges"]) and np.array_equal(r["symbols"], base["symbols"])


def test_id_exhaustion_stops():
    """next_token_id > 0xFFFF stops training (train.wgsl:345)."""
    sym = np.array(tagged("abababab"), np.uint32)
    r = O.train(sym, 5, "fixed", first_id=0xFFFF)
    assert r["merges"].tolist() == [[97, 98, 0xFFFF, 4]] and r["early_stop"]
    m, e, _ = M.train(sym.tolist(), 5, first_id=0xFFFF, literal=False)
    assert m == [[97, 98, 0xFFFF, 4]] and e


def test_word_boundary_heuristic():
    text = b"Hello, world 42\nnext  line\tx"
    a = O.word_boundary(np.frombuffer(text, np.uint8)).tolist()
    assert a == M.word_boundary(list(text))
    starts = [i for i, s in enumerate(a) if s & 0x10000]
    # H | , | ' world' | ' 42' | \n | n... | ' ' (space after letter) | \t | x
    assert starts[:5] == [0, 5, 6, 12, 15]


def test_pair_counts_exact():
    sym = np.array(tagged("aaa|aa|ab"), np.uint32)
    assert O.pair_counts(sym) == {(97 << 16) | 97: 3, (97 << 16) | 98: 1}


def test_trie_and_encode_model_vs_cpp():
    rng = np.random.default_rng(3)
    sym = random_symbols(rng, 4000, alphabet=5, p_ws=0.2)
    merges = O.train(sym, 50, "fixed")["merges"].tolist()
    vocab = M.vocab_from_merges(merges)
    trie = M.compile_vocab_to_trie(vocab)
    hdr = M.parse_trie(trie)
    assert hdr["vocabSize"] == len(vocab) and hdr["nodeCount"] == hdr["edgeCount"] + 1
    data = bytes((sym & 0xFF).astype(np.uint8))
    for cs in (1, 7, 64, 512):
        want = M.encode_bytes(data, trie, cs)
        got = O.encode(np.frombuffer(data, np.uint8), trie, cs, threads=3)
        assert got.tolist() == want
        assert M.decode(want, vocab) == data


def test_trie_duplicate_and_empty_entries():
    vocab = [[97], [], [97, 98], [97]]          # id 3 repeats id 0 → last id wins; id 1 is skipped
    trie = M.compile_vocab_to_trie(vocab)
    t = M.parse_trie(trie)
    assert t["nodeCount"] == 3 and t["maxTokenLen"] == 2 and t["vocabSize"] == 4
    assert M.encode_bytes(b"aab", trie, 512) == [3, 2]
    assert M.encode_bytes(b"zab", trie, 512) == [ord("z"), 2]   # unknown byte → raw byte value


def test_trie_errors():
    trie = M.compile_vocab_to_trie([[i] for i in range(256)])
    with pytest.raises(ValueError, match="magic"):
        M.parse_trie(b"\0" * 28)
    with pytest.raises(ValueError, match="version"):
        M.parse_trie(trie[:4] + (9).to_bytes(4, "little") + trie[8:])
    with pytest.raises(ValueError, match="Truncated"):
        M.parse_trie(trie[:-1])


def test_pretokenizer_rules():
    def starts(s):
        d, m = M.pretokenize_bytes(s.encode())
        return [i for i, x in enumerate(m) if x]
    assert starts("kabul edilmek") == [0, 5]                    # space prefixes the next word
    assert starts("don't stop") == [0, 5]                       # contraction stays with its word
    assert starts("x1234567") == [0, 1, 4, 7]                   # digit runs split every 3
    assert starts("a\nb") == [0, 1, 2]                          # newline isolates
    assert starts("hi!!") == [0, 2]                             # punctuation run is one word
    assert starts("ğa“b") == [0, 3, 6]                          # multi-byte letter / punctuation by code point


def test_replay_known_answers():
    """The merge-replay oracle (oracle/replay_oracle.cpp) against the hand-derived cases and a literal Python
    transcription of the loop of src/ui/tokenizer-manager.js:45-58."""
    import json
    import os
    from tests.helpers import GOLDEN
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        cases = json.load(f)["replay"]
    for c in cases:
        data = np.frombuffer(c["text"].encode("utf-8"), np.uint8)
        assert O.replay_encode(data, c["merges"]).tolist() == c["tokens"], c["text"]

    def literal(tokens, merges):
        for a, b, new in merges:
            if len(tokens) < 2:
                break
            out, i = [], 0
            while i < len(tokens):
                if i + 1 < len(tokens) and tokens[i] == a and tokens[i + 1] == b:
                    out.append(new)
                    i += 2
                else:
                    out.append(tokens[i])
                    i += 1
            tokens = out
        return tokens

    rng = np.random.default_rng(3)
    for trial in range(20):
        data = rng.integers(97, 100, int(rng.integers(0, 200)), dtype=np.uint8)
        merges, ids = [], [97, 98, 99]
        for r in range(int(rng.integers(0, 12))):
            merges.append([int(rng.choice(ids)), int(rng.choice(ids)), 256 + r])
            ids.append(256 + r)
        assert O.replay_encode(data, merges).tolist() == literal(data.tolist(), merges), trial
