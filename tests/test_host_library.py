"""CPU tests of the shared library's host side: it loads, exports every symbol of the header,
and its host-only entry points (trie compiler, header parser, pre-tokeniser) agree with the oracle."""
import os
import re

import numpy as np
import pytest

from gpu_bpe_b200 import PreTokenizer, _lib, compileVocabToTrie, parseHeader, parseTrieBuffers, synth
from gpu_bpe_b200.vocab import Vocab, model_from_json, model_to_json
from oracle import cpu_oracle as O
from oracle import wgsl_model as M
from tests.helpers import random_symbols

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "b200bpe.h")).read()
    declared = set(re.findall(r"^(?:b200bpe_status|void|const char\*|int32_t)\s+(b200bpe_[a-z0-9_]+)\s*\(", hdr, re.M))
    assert len(declared) >= 30
    L = _lib.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} is declared in include/b200bpe.h but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes binding and header disagree"


def test_no_gpu_means_loud_failure():
    """Without a GPU the context cannot be created: there is no CPU path to fall back to."""
    L = _lib.lib()
    if L.b200bpe_device_count() > 0:
        pytest.skip("a GPU is visible")
    from gpu_bpe_b200 import BPEEngine
    with pytest.raises(_lib.B200BPEError) as ei:
        BPEEngine(0).init()
    assert ei.value.status_name == "NO_DEVICE"


def test_status_strings():
    L = _lib.lib()
    assert L.b200bpe_status_str(0) == b"ok"
    assert b"corpus is empty" in L.b200bpe_status_str(4)


def test_trie_compile_matches_oracle_bytes():
    rng = np.random.default_rng(1)
    sym = random_symbols(rng, 20000, alphabet=9, p_ws=0.15)
    vocab = M.vocab_from_merges(O.train(sym, 400, "fixed")["merges"].tolist())
    assert compileVocabToTrie(vocab) == M.compile_vocab_to_trie(vocab)
    odd = [[97], [], [97, 98], [97], [0], [255, 254, 253]]
    assert compileVocabToTrie(odd) == M.compile_vocab_to_trie(odd)
    assert compileVocabToTrie([]) == M.compile_vocab_to_trie([])


def test_trie_parse_and_errors():
    vocab = [[i] for i in range(256)] + [[104, 105]]
    trie = compileVocabToTrie(vocab)
    h = parseHeader(trie)
    assert h == {"version": 3, "nodeCount": 258, "edgeCount": 257, "maxTokenLen": 2}
    bufs = parseTrieBuffers(trie, h)
    ref = M.parse_trie(trie)
    assert bufs["nodes"].tolist() == list(ref["nodes"])
    assert bufs["edges"].reshape(-1, 2).tolist() == [list(e) for e in ref["edges"]]
    with pytest.raises(ValueError, match="Invalid trie magic"):
        parseHeader(b"\1" * 28)
    with pytest.raises(ValueError, match="Unsupported trie version"):
        parseHeader(trie[:4] + (7).to_bytes(4, "little") + trie[8:])
    with pytest.raises(ValueError, match="Truncated trie data"):
        parseTrieBuffers(trie[:-3], parseHeader(trie[:-3]))


@pytest.mark.parametrize("kind,seed", [(1, 1), (2, 2), (5, 5)])
def test_pretokenizer_matches_oracle(kind, seed):
    data = synth.corpus(kind, seed, 1 << 16).tobytes().decode("utf-8", "ignore").encode()
    want_bytes, want_mask = M.pretokenize_bytes(data)
    got = PreTokenizer().preTokenizeBytes(data)
    assert got["bytes"].tobytes() == want_bytes
    assert got["wordStarts"].tobytes() == want_mask


def test_pretokenizer_edge_text():
    text = "It's 12345678 o'clock — we'll “quote” x\r\ny\tz  a1b2 ÇA VA? fin 's"
    want_bytes, want_mask = M.pretokenize_bytes(text.encode())
    got = PreTokenizer().preTokenize(text)
    assert got["bytes"].tobytes() == want_bytes and got["wordStarts"].tobytes() == want_mask
    assert PreTokenizer().preTokenize("")["bytes"].size == 0


def test_synthetic_corpus_is_deterministic_and_valid_utf8():
    a = synth.corpus(2, 7, 3 << 20, threads=1)
    b = synth.corpus(2, 7, 3 << 20, threads=8)
    assert np.array_equal(a, b)
    text = a.tobytes().decode("utf-8")     # raises if a block cut a character
    import unicodedata
    assert unicodedata.is_normalized("NFC", text)
    frac_ascii = float((a < 0x80).mean())
    assert 0.55 < frac_ascii < 0.9
    offs = synth.doc_offsets(4, a.size, 1000, 1.0)
    assert offs[0] == 0 and offs[-1] == a.size and np.all(np.diff(offs.astype(np.int64)) >= 0)


def test_vocab_and_json_round_trip():
    v = Vocab()
    assert v.size == 256 and v.strings[0x20] == "▁" and v.strings[0x0A] == "\\n" and v.strings[0xC3] == "<0xC3>"
    nid = v.addMerge(0xC3, 0xA7)
    assert nid == 256 and v.entries[256] == [0xC3, 0xA7] and v.strings[256] == "ç"
    res = {"vocab": v.entries, "vocabStrings": v.strings, "vocabSize": v.size, "merges": [[0xC3, 0xA7, 256]]}
    back = model_from_json(model_to_json(res))
    assert back["vocab"] == v.entries and back["merges"] == [[0xC3, 0xA7, 256]] and back["vocabSize"] == 257
    assert back["vocabStrings"][256] == "ç"
    with pytest.raises(ValueError):
        model_from_json('{"vocab": []}')
    assert v.export().splitlines()[1] == "# Total tokens: 257"
