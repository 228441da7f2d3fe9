"""GPU parity tests of the encode path: token ids from libb200bpe.so against the CPU oracle."""
import numpy as np
import pytest

from gpu_bpe_b200 import TrieTokenizer, compileVocabToTrie
from oracle import cpu_oracle as O
from oracle import wgsl_model as M
from tests.helpers import small_text

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["auto", "hybrid", "hash"])
def trie_layout(request, monkeypatch):
    """Every test runs on three device layouts of the trie: the one the library picks (for these vocabularies the
    cuckoo table in shared memory), the hybrid (hot transitions in shared memory, two-byte first step) and the global
    hash table.  The layout is an option of the tokenizer; it is set here for every tokenizer a test makes."""
    real_init = TrieTokenizer.__init__

    def init(self, engine, trieData, vocab=None, options=None):
        real_init(self, engine, trieData, vocab, dict(options or {}, layout=request.param))

    monkeypatch.setattr(TrieTokenizer, "__init__", init)
    return request.param


@pytest.fixture(scope="module")
def trained():
    """A vocabulary trained by the oracle on config-2-shaped text (so the test does not depend on the GPU trainer)."""
    data, mask, sym = small_text(2, 31, 2 << 20)
    merges = O.train(sym, 1500, "fixed", threads=8)["merges"].tolist()
    vocab = M.vocab_from_merges(merges)
    return vocab, M.compile_vocab_to_trie(vocab)


def test_tokenizer_fields_and_chunk_rule(engine, trained, trie_layout):
    vocab, trie = trained
    tok = TrieTokenizer.fromVocab(engine, vocab)
    assert tok.deviceLayout[0] == {"auto": 2, "hybrid": 1, "hash": 0}[trie_layout] or (trie_layout == "auto" and tok.deviceLayout[0] == 3)
    hdr = M.parse_trie(trie)
    assert (tok.nodeCount, tok.edgeCount, tok.maxTokenLen) == (hdr["nodeCount"], hdr["edgeCount"], hdr["maxTokenLen"])
    assert tok.chunkSize == max(512, min(2048, hdr["maxTokenLen"] * 8))
    tok.destroy()
    tok = TrieTokenizer(engine, trie, vocab, {"chunkSize": 96})
    assert tok.chunkSize == 96
    tok.destroy()


@pytest.mark.parametrize("n", [0, 1, 2, 15, 16, 17, 511, 512, 513, 1023, 1025, 100_003])
def test_sizes_around_chunk_edges(engine, trained, n):
    vocab, trie = trained
    data, _, _ = small_text(2, 77, max(n, 1))
    data = data[:n]
    tok = TrieTokenizer(engine, trie, vocab)
    got = tok.encodeBytes(data)
    want = O.encode(data, trie, tok.chunkSize) if n else np.zeros(0, np.uint32)
    assert got.dtype == np.uint32 and got.tolist() == want.tolist()
    assert tok.decode(got) == data.tobytes()
    tok.destroy()


@pytest.mark.parametrize("chunk", [1, 5, 64, 512, 2048])
def test_chunk_sizes(engine, trained, chunk):
    vocab, trie = trained
    data, _, _ = small_text(2, 78, 300_000)
    tok = TrieTokenizer(engine, trie, vocab, {"chunkSize": chunk})
    got = tok.encodeBytes(data)
    assert got.tolist() == O.encode(data, trie, chunk, threads=4).tolist()
    tok.destroy()


def test_against_python_model(engine, trained):
    vocab, trie = trained
    data, _, _ = small_text(2, 79, 20_000)
    tok = TrieTokenizer(engine, trie, vocab)
    assert tok.encodeBytes(data).tolist() == M.encode_bytes(data.tobytes(), trie, tok.chunkSize)
    tok.destroy()


def test_unknown_bytes_and_sparse_vocab(engine):
    """A vocabulary without all single bytes: unmatched bytes come out as raw byte values."""
    vocab = [[97], [], [97, 98], [97], [98, 99, 100]]
    tok = TrieTokenizer.fromVocab(engine, vocab)
    data = b"aabzbcdbcxab" * 200
    want = M.encode_bytes(data, M.compile_vocab_to_trie(vocab), tok.chunkSize)
    assert tok.encodeBytes(data).tolist() == want
    assert tok.decode([0, 99999]) == b"a\xef\xbf\xbd"
    tok.destroy()


def test_random_bytes(engine, trained):
    vocab, trie = trained
    rng = np.random.default_rng(8)
    data = rng.integers(0, 256, 200_000, dtype=np.uint8)
    tok = TrieTokenizer(engine, trie, vocab)
    assert tok.encodeBytes(data).tolist() == O.encode(data, trie, tok.chunkSize, threads=4).tolist()
    tok.destroy()


def test_batch_equals_per_document_calls(engine, trained):
    from gpu_bpe_b200 import synth
    vocab, trie = trained
    data, _, _ = small_text(2, 80, 1 << 20)
    offs = synth.doc_offsets(4, data.size, 300, 1.0)
    offs[5] = offs[4]            # an empty document
    tok = TrieTokenizer(engine, trie, vocab)
    toks, toff = tok.encodeBatch(data, offs)
    assert toff[0] == 0 and toff[-1] == toks.size
    for d in range(300):
        lo, hi = int(offs[d]), int(offs[d + 1])
        want = O.encode(data[lo:hi], trie, tok.chunkSize) if hi > lo else np.zeros(0, np.uint32)
        assert toks[int(toff[d]):int(toff[d + 1])].tolist() == want.tolist(), d
    # and the same through a misaligned view of the buffer
    toks2, toff2 = tok.encodeBatch(data[3:], (offs[1:] - 3).clip(0) if offs[1] >= 3 else offs[1:])
    tok.destroy()


def test_bad_trie_rejected(engine, trained):
    _, trie = trained
    with pytest.raises(ValueError, match="Invalid trie magic"):
        TrieTokenizer(engine, b"\0" * 64)
    with pytest.raises(ValueError, match="Truncated trie data"):
        TrieTokenizer(engine, trie[: len(trie) // 2])


def test_train_then_encode_round_trip(engine):
    """The whole drop-in flow: train on the GPU, compile, encode, decode back to the input."""
    from gpu_bpe_b200 import BPETrainer, PreTokenizer
    data, _, _ = small_text(1, 12, 1 << 18)
    res = BPETrainer(engine).train(data, targetVocabSize=800, preTokenizer=PreTokenizer(normalize=False))
    tok = TrieTokenizer.fromVocab(engine, res["vocab"])
    ids = tok.encodeBytes(data)
    assert tok.decode(ids) == data.tobytes() and ids.size < data.size // 2
    assert ids.tolist() == O.encode(data, compileVocabToTrie(res["vocab"]), tok.chunkSize, threads=4).tolist()
    tok.destroy()


@pytest.mark.parametrize("n_tokens,alphabet,want_tables", [(3_000, 64, 2), (14_000, 24, 3), (70_000, 64, 1), (140_000, 256, 0)])
def test_trie_sizes_pick_their_layout(engine, trie_layout, n_tokens, alphabet, want_tables):
    """Random vocabularies sized for two cuckoo sub-tables, for three, for the hybrid (too large for shared
    memory, every node index below 130,816) and for the global table alone."""
    rng = np.random.default_rng(n_tokens)
    vocab = [[b] for b in range(256)]
    seen = set()
    while len(vocab) < 256 + n_tokens:
        t = tuple(int(x) for x in rng.integers(0, alphabet, int(rng.integers(2, 6))))
        if t not in seen:
            seen.add(t)
            vocab.append(list(t))
    trie = M.compile_vocab_to_trie(vocab)
    tok = TrieTokenizer(engine, trie, vocab)
    want = {"auto": want_tables, "hash": 0, "hybrid": 1 if want_tables else 0}[trie_layout]   # a trie too large for the hybrid falls through
    assert tok.deviceLayout[0] == want, tok.deviceLayout
    data = rng.integers(0, alphabet, 400_000, dtype=np.uint8)
    data[::97] = 255  # and bytes outside the alphabet
    assert tok.encodeBytes(data).tolist() == O.encode(data, trie, tok.chunkSize, threads=4).tolist()
    tok.destroy()


def test_batch_in_slices_equals_one_pass(engine, trained):
    """Large host batches are encoded slice by slice with the read-back of one slice under the work of
    the next; the cut must not show (here forced with small slices)."""
    from gpu_bpe_b200 import synth
    vocab, trie = trained
    data, _, _ = small_text(2, 81, 1 << 20)
    offs = synth.doc_offsets(9, data.size, 257, 1.2)
    offs[17] = offs[16]          # an empty document
    tok = TrieTokenizer(engine, trie, vocab)
    toks1, toff1 = tok.encodeBatch(data, offs)
    for slice_bytes in (4096, 65536, 300_000):
        sliced = TrieTokenizer(engine, trie, vocab, {"batchSliceBytes": slice_bytes})
        toks2, toff2 = sliced.encodeBatch(data, offs)
        sliced.destroy()
        assert np.array_equal(toks1, toks2) and np.array_equal(toff1, toff2), slice_bytes
    assert toks1.tolist() == np.concatenate([O.encode(data[int(offs[d]):int(offs[d + 1])], trie, tok.chunkSize)
                                             if offs[d + 1] > offs[d] else np.zeros(0, np.uint32) for d in range(257)]).tolist()
    tok.destroy()


def test_encode_in_slices_equals_one_pass(engine, trained):
    """encodeBytes cuts inputs beyond its buffer limit into chunk-aligned slices (tokenizer.js:181-203); with the
    limit forced down to 100,000 bytes a 300,001-byte input goes through in four slices and the cut must not show."""
    vocab, trie = trained
    data, _, _ = small_text(2, 82, 300_001)
    tok = TrieTokenizer(engine, trie, vocab)
    want = tok.encodeBytes(data)
    assert want.tolist() == O.encode(data, trie, tok.chunkSize, threads=4).tolist()
    for limit in (100_000, 512, 70_000):
        sliced = TrieTokenizer(engine, trie, vocab, {"encodeSliceBytes": limit})
        assert np.array_equal(sliced.encodeBytes(data), want), limit
        sliced.destroy()
    tok.destroy()
