"""Every device-side wait of the library is bounded: a wait that nothing can ever satisfy ends by itself,
the call returns B200BPE_ERR_LOOKBACK_TIMEOUT, and the library goes on working afterwards.

Nothing here faults, traps or hangs a GPU: the tests only make a wait run out.  Each kernel that waits on
other tiles (merge + compaction of the trainer, scan + compaction of the encoder, the device pre-tokeniser)
has a test option that starts its tile numbering at 1, so that tile 0 never publishes what every later tile
looks back for, together with a limit of a few hundred polls instead of millions.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_bpe_b200 import TrainerSession, TrieTokenizer, _lib
from oracle import cpu_oracle as O
from oracle import wgsl_model as M
from tests.helpers import random_symbols, small_text

pytestmark = pytest.mark.gpu


def test_merge_kernel_lookback_gives_up_and_the_library_recovers(engine):
    rng = np.random.default_rng(4)
    sym = random_symbols(rng, 300_000, alphabet=12, p_ws=0.1)     # some twenty tiles
    stalled = TrainerSession.from_symbols(engine, sym, target_vocab_size=256 + 5, compat_mode="fixed",
                                          test_lookback_spins=200, test_first_tile=1)
    with pytest.raises(_lib.B200BPEError) as ei:
        stalled.run()
    assert ei.value.status_name == "LOOKBACK_TIMEOUT"
    stalled.destroy()
    # the same context still trains correctly
    want = O.train(sym, 30, "fixed", threads=4)
    s = TrainerSession.from_symbols(engine, sym, target_vocab_size=256 + 30, compat_mode="fixed")
    m, c, _ = s.run()
    s.destroy()
    assert np.concatenate([m, c[:, None]], axis=1).tolist() == want["merges"].tolist()
    # a short limit alone (every tile takes part) changes nothing
    s = TrainerSession.from_symbols(engine, sym, target_vocab_size=256 + 30, compat_mode="fixed", test_lookback_spins=1 << 21)
    m2, _, _ = s.run()
    s.destroy()
    assert np.array_equal(m, m2)


def test_encode_compaction_lookback_gives_up_and_the_library_recovers(engine):
    _, _, sym = small_text(2, 31, 1 << 19)
    vocab = M.vocab_from_merges(O.train(sym, 300, "fixed", threads=8)["merges"].tolist())
    trie = M.compile_vocab_to_trie(vocab)
    data, _, _ = small_text(2, 93, 400_000)          # 782 chunks: four tiles of the compaction
    stalled = TrieTokenizer(engine, trie, vocab, {"testLookbackSpins": 300})
    with pytest.raises(_lib.B200BPEError) as ei:
        stalled.encodeBytes(data)
    assert ei.value.status_name == "LOOKBACK_TIMEOUT"
    stalled.destroy()
    tok = TrieTokenizer(engine, trie, vocab)
    assert np.array_equal(tok.encodeBytes(data), O.encode(data, trie, tok.chunkSize, threads=4))
    tok.destroy()


def test_pretokenizer_lookback_gives_up_and_the_library_recovers(engine):
    data, mask, _ = small_text(2, 94, 1 << 20)
    data = data.copy()
    data[:200_000] = ord("7")                        # one long run of digits: its count travels from tile to tile
    d_in = torch.from_numpy(data).cuda()
    d_out = torch.zeros(data.size, dtype=torch.uint8, device="cuda")
    L = _lib.lib()
    st = L.b200bpe_pretokenize_device_ex(engine.ctx, C.c_void_p(d_in.data_ptr()), data.size, C.c_void_p(d_out.data_ptr()), 300)
    assert _lib.STATUS[st] == "LOOKBACK_TIMEOUT"
    st = L.b200bpe_pretokenize_device_ex(engine.ctx, C.c_void_p(d_in.data_ptr()), data.size, C.c_void_p(d_out.data_ptr()), 0)
    assert st == 0
    want = np.zeros(data.size, np.uint8)
    assert L.b200bpe_pretokenize(data.ctypes.data, data.size, want.ctypes.data) == 0
    assert np.array_equal(d_out.cpu().numpy(), want)
