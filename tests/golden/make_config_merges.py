"""Generate the golden merge lists of the benchmark configurations (CPU only; no GPU needed).

    python tests/golden/make_config_merges.py 2        # 64 MiB / 8,000 merges: literal and fixed
    python tests/golden/make_config_merges.py 3        # 1 GiB / 32,000 merges: fixed
    python tests/golden/make_config_merges.py 5        # 8 GiB / 64,000 merges: fixed (needs ~20 GB of RAM)

Config 2 is small enough for the pass-by-pass oracle (oracle/bpe_oracle.cpp), which knows both
compaction modes; its "fixed" list is also computed with the word-level oracle
(oracle/word_oracle.cpp) and the two must agree.  Configs 3 and 5 would take that oracle days, so
their lists come from the word-level oracle alone ("fixed" mode only: the only mode that is defined
for a sharded corpus).

Output: tests/golden/config<k>_<mode>.npz with a, b (u16), count (u32); the new id of merge i is
256 + i.  Inputs are the seeded synthetic corpora of gpu_bpe_b200/csrc/synth.cpp and the host
pre-tokeniser, exactly as bench.py builds them.
"""
import hashlib
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

MIB = 1 << 20
# config → (generator kind, seed, bytes, merges)
CONFIGS = {2: (2, 2, 64 * MIB, 8000), 3: (2, 3, 1024 * MIB, 32000), 5: (5, 5, 8192 * MIB, 64000)}


def corpus(cfg: int):
    from gpu_bpe_b200 import PreTokenizer, synth
    kind, seed, nbytes, _ = CONFIGS[cfg]
    data = synth.corpus(kind, seed, nbytes)
    pt = PreTokenizer(normalize=False)
    mask = np.empty(nbytes, np.uint8)
    step = 256 * MIB   # the mask of a slice that begins at a line start equals the mask of the whole there
    lo = 0
    while lo < nbytes:
        hi = min(nbytes, lo + step)
        if hi < nbytes:
            hi = lo + int(np.flatnonzero(data[lo:hi] == 0x0A)[-1]) + 1   # cut after a newline: the rules restart there
        mask[lo:hi] = pt.preTokenizeBytes(data[lo:hi])["wordStarts"]
        lo = hi
    return data, mask


def save(cfg: int, mode: str, merges: np.ndarray, extra: dict):
    assert np.array_equal(merges[:, 2], 256 + np.arange(merges.shape[0]))
    path = os.path.join(HERE, f"config{cfg}_{mode}.npz")
    a, b, c = merges[:, 0].astype(np.uint16), merges[:, 1].astype(np.uint16), merges[:, 3].astype(np.uint32)
    sha = hashlib.sha256(np.ascontiguousarray(merges[:, [0, 1, 3]].astype(np.uint32)).tobytes()).hexdigest()
    np.savez_compressed(path, a=a, b=b, count=c, meta=np.frombuffer(json.dumps(dict(extra, sha256=sha)).encode(), np.uint8))
    print("wrote", path, merges.shape[0], "merges", sha[:16], extra, flush=True)


def main():
    from oracle import cpu_oracle as O
    cfg = int(sys.argv[1])
    kind, seed, nbytes, n_merges = CONFIGS[cfg]
    threads = os.cpu_count() or 1
    t0 = time.time()
    data, mask = corpus(cfg)
    print(f"config {cfg}: corpus + mask in {time.time() - t0:.1f} s", flush=True)
    t0 = time.time()
    w = O.train_words(data, n_merges, word_starts=mask, threads=threads)
    print(f"word-level oracle: {w['merges'].shape[0]} merges in {time.time() - t0:.1f} s, {w['distinct_words']} distinct "
          f"words, {w['distinct_pairs']} distinct pairs at merge 0, {w['n']} symbols left", flush=True)
    meta = {"config": cfg, "kind": kind, "seed": seed, "bytes": nbytes, "early_stop": w["early_stop"],
            "symbols_left": int(w["n"]), "distinct_pairs_at_merge_0": int(w["distinct_pairs"]),
            "distinct_words": int(w["distinct_words"])}
    if cfg == 2:
        sym = data.astype(np.uint32) | (mask.astype(np.uint32) << 16)
        for mode in ("fixed", "literal"):
            t0 = time.time()
            r = O.train(sym, n_merges, mode, threads=threads, want_symbols=False)
            print(f"pass-by-pass oracle, {mode}: {r['merges'].shape[0]} merges in {time.time() - t0:.1f} s", flush=True)
            if mode == "fixed":
                assert np.array_equal(r["merges"], w["merges"]), "the two oracles disagree on the fixed-mode list"
                assert r["n"] == w["n"] and r["early_stop"] == w["early_stop"]
            save(cfg, mode, r["merges"], dict(meta, oracle="bpe_oracle.cpp" + (" == word_oracle.cpp" if mode == "fixed" else ""),
                                              symbols_left=int(r["n"]), early_stop=r["early_stop"]))
    else:
        save(cfg, "fixed", w["merges"], dict(meta, oracle="word_oracle.cpp"))


if __name__ == "__main__":
    main()
