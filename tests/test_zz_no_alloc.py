"""GPU test of b200bpe_encode_device_noalloc, the encode entry point for callers that cannot
allocate at encode time (its work buffers are a fixed array inside the library image).

It must give exactly the token ids of the pooled entry point b200bpe_encode_device, on two calls in
a row that share the built-in array (the second one shorter, so stale contents of the first would
show), and it must turn away inputs beyond its stated limits with a clear error.  The file name
sorts last on purpose: a run that stops at the first failure has then already run everything else.
"""
import numpy as np
import pytest
import torch

from gpu_bpe_b200 import TrieTokenizer, _lib
from oracle import cpu_oracle as O
from oracle import wgsl_model as M
from tests.helpers import small_text

pytestmark = pytest.mark.gpu


def _vocab():
    _, _, sym = small_text(2, 31, 1 << 20)
    return M.vocab_from_merges(O.train(sym, 600, "fixed", threads=8)["merges"].tolist())


def _encode_both(tok, data: np.ndarray):
    d_in = torch.from_numpy(data.copy()).cuda()
    out_a = torch.zeros(max(1, data.size), dtype=torch.int32, device="cuda")
    out_b = torch.full((max(1, data.size),), -1, dtype=torch.int32, device="cuda")
    na = tok.encodeDevice(d_in.data_ptr(), data.size, out_a.data_ptr(), out_a.numel())
    nb = tok.encodeDeviceNoAlloc(d_in.data_ptr(), data.size, out_b.data_ptr(), out_b.numel())
    return out_a[:na].cpu().numpy().astype(np.uint32), out_b[:nb].cpu().numpy().astype(np.uint32)


@pytest.mark.parametrize("layout", ["auto", "hybrid", "hash"])
def test_no_alloc_encode_matches_pooled_encode(engine, layout):
    vocab = _vocab()
    tok = TrieTokenizer.fromVocab(engine, vocab, {"layout": layout})
    trie = M.compile_vocab_to_trie(vocab)
    first, _, _ = small_text(2, 90, 1 << 20)          # the largest input the entry point takes
    second, _, _ = small_text(2, 91, 300_001)         # shorter: the array still holds the first call's data
    for data in (first, second, second[:1], first[:777]):
        a, b = _encode_both(tok, data)
        assert np.array_equal(a, b)
        assert np.array_equal(b, O.encode(data, trie, tok.chunkSize, threads=4))
    tok.destroy()


def test_no_alloc_encode_rejects_what_does_not_fit(engine):
    vocab = [[i] for i in range(256)]
    tok = TrieTokenizer.fromVocab(engine, vocab)
    too_long = torch.zeros((1 << 20) + 1, dtype=torch.uint8, device="cuda")
    out = torch.zeros(too_long.numel(), dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.B200BPEError) as ei:
        tok.encodeDeviceNoAlloc(too_long.data_ptr(), too_long.numel(), out.data_ptr(), out.numel())
    assert ei.value.status_name == "CAPACITY"
    assert b"exceeds the built-in scratch" in _lib.lib().b200bpe_last_error()
    tok.destroy()
    many_chunks = TrieTokenizer(engine, M.compile_vocab_to_trie(vocab), vocab, {"chunkSize": 16})
    with pytest.raises(_lib.B200BPEError):                      # 1 MiB / 16 = 65,536 chunks > 8,192
        many_chunks.encodeDeviceNoAlloc(too_long.data_ptr(), 1 << 20, out.data_ptr(), out.numel())
    small = torch.arange(0, 200, dtype=torch.uint8, device="cuda")
    assert many_chunks.encodeDeviceNoAlloc(small.data_ptr(), 200, out.data_ptr(), out.numel()) == 200
    assert out[:200].cpu().tolist() == list(range(200))
    many_chunks.destroy()
