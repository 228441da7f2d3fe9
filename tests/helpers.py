"""Shared helpers of the test-suite (not collected)."""
import json
import os

import numpy as np

W = 0x10000
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def tagged(s: str) -> list[int]:
    """'ab| cd' → tagged symbols; '|' marks that the next symbol starts a word, the first always does."""
    out, ws = [], True
    for ch in s:
        if ch == "|":
            ws = True
            continue
        out.append(ord(ch) | (W if ws else 0))
        ws = False
    return out


def known_answers():
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        return json.load(f)["cases"]


def random_symbols(rng: np.random.Generator, n: int, alphabet: int = 6, p_ws: float = 0.2, p_nul: float = 0.0):
    toks = rng.integers(97, 97 + alphabet, size=n).astype(np.uint32)
    if p_nul:
        toks[rng.random(n) < p_nul] = 0
    ws = rng.random(n) < p_ws
    if n:
        ws[0] = True
    return (toks | (ws.astype(np.uint32) << 16)).astype(np.uint32)


def small_text(kind: int, seed: int, n: int):
    """Synthetic text + GPT-4-style mask + tagged symbols."""
    from gpu_bpe_b200 import PreTokenizer, synth
    data = synth.corpus(kind, seed, n)
    r = PreTokenizer(normalize=False).preTokenizeBytes(data)
    sym = data.astype(np.uint32) | (r["wordStarts"].astype(np.uint32) << 16)
    return data, r["wordStarts"], sym
