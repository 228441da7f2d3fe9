"""Full-size parity of the benchmark configurations on one GPU.

Config 2 (64 MiB, 8,000 merges): the whole merge list and its counts, in both compaction modes, against the golden
lists of tests/golden/ (made by the pass-by-pass CPU oracle; tests/golden/make_config_merges.py).
Config 3 (1 GiB, 32,000 merges) in "literal" mode, for which no oracle can produce the full list in reasonable time:
at 33 checkpoints spread over the run, the device's pair table must equal a fresh count of the live symbols by the CPU
oracle, and the merge the device applies next must be that table's arg-max under the reference's order (larger count,
then smaller pair id; train.wgsl:83-85).  ("fixed" mode of config 3 is compared entry by entry with its golden list by
bench.py on every run.)
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from gpu_bpe_b200 import TrainerSession, _lib, synth
from oracle import cpu_oracle as O
from tests.helpers import GOLDEN

pytestmark = pytest.mark.gpu
MIB = 1 << 20


def _resident_corpus(engine, kind, seed, nbytes):
    data = synth.corpus(kind, seed, nbytes)
    d_bytes = torch.from_numpy(data).cuda()
    d_mask = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    _lib.check(_lib.lib().b200bpe_pretokenize_device(engine.ctx, C.c_void_p(d_bytes.data_ptr()), nbytes, C.c_void_p(d_mask.data_ptr())))
    return d_bytes, d_mask


def _golden(cfg, mode):
    g = np.load(os.path.join(GOLDEN, f"config{cfg}_{mode}.npz"))
    return np.stack([g["a"].astype(np.uint32), g["b"].astype(np.uint32), g["count"].astype(np.uint32)], axis=1)


@pytest.mark.parametrize("mode", ["fixed", "literal"])
def test_config2_whole_merge_list(engine, mode):
    d_bytes, d_mask = _resident_corpus(engine, 2, 2, 64 * MIB)
    s = TrainerSession.create(engine, d_bytes.data_ptr(), d_mask.data_ptr(), n=64 * MIB, device_pointers=True,
                              target_vocab_size=256 + 8000, compat_mode=mode)
    m, c, early = s.run()
    s.destroy()
    gold = _golden(2, mode)
    got = np.stack([m[:, 0], m[:, 1], c], axis=1)
    assert got.shape == gold.shape and not early
    bad = np.flatnonzero((got != gold).any(axis=1))
    assert bad.size == 0, f"merge {int(bad[0])}: got {got[bad[0]].tolist()}, want {gold[bad[0]].tolist()}"


def test_config3_literal_checkpoints(engine):
    n = 1024 * MIB
    d_bytes, d_mask = _resident_corpus(engine, 2, 3, n)
    s = TrainerSession.create(engine, d_bytes.data_ptr(), d_mask.data_ptr(), n=n, device_pointers=True,
                              target_vocab_size=256 + 32000, compat_mode="literal")
    threads = os.cpu_count() or 1
    done = 0
    for k in [0] + list(range(1000, 32001, 1000)):
        if k > done:
            s.run(k - done)
            done = k
        want = O.pair_counts(s.symbols(), threads=threads)
        got = {((key >> 32) << 16) | (key & 0xFFFF): v for key, v in s.pair_counts(cap=1 << 23).items()}
        assert got == want, f"pair table differs from a fresh count after {k} merges"
        if k == 32000:
            break
        best = max(want.items(), key=lambda kv: (kv[1], -kv[0]))     # larger count, then smaller packed pair
        m, c, early = s.run(1)
        done += 1
        assert not early and (int(m[0, 0]) << 16 | int(m[0, 1]), int(c[0])) == best, f"merge {k} is not the arg-max"
    s.destroy()
