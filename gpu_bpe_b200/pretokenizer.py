"""PreTokenizer — GPT-4-style word starts (host code).

Mirrors PreTokenizer.preTokenizeBytes / preTokenize of src/wasm/pre_tokenizer.mjs:426-509.  The
reference NFC-normalises through a closed WASM library first; here Python's unicodedata does
that step and the boundary rules run in the library's host code (b200bpe_pretokenize).
"""
from __future__ import annotations

import unicodedata

import numpy as np

from . import _lib


class PreTokenizer:
    def __init__(self, normalize: bool = True, engine=None):
        """engine: a BPEEngine → the boundary rules run on its GPU (well-formed UTF-8 only: other input
        raises, and a PreTokenizer without an engine takes any bytes); None → the library's host code."""
        self.normalize = normalize
        self.engine = engine

    def preTokenizeBytes(self, raw) -> dict:
        raw = bytes(raw) if not isinstance(raw, (bytes, bytearray, np.ndarray)) else raw
        arr = np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else np.ascontiguousarray(raw, np.uint8)
        if arr.size == 0:
            return {"bytes": np.zeros(0, np.uint8), "wordStarts": np.zeros(0, np.uint8)}
        if self.normalize:
            try:
                text = arr.tobytes().decode("utf-8")
                if not unicodedata.is_normalized("NFC", text):
                    arr = np.frombuffer(unicodedata.normalize("NFC", text).encode("utf-8"), dtype=np.uint8)
            except UnicodeDecodeError:
                pass  # pre_tokenizer.mjs:466-469: on failure the raw bytes are used
        mask = np.zeros(arr.size, np.uint8)
        if self.engine is not None:
            st = _lib.lib().b200bpe_pretokenize_gpu(self.engine.ctx, arr.ctypes.data, arr.size, mask.ctypes.data)
            if st == 1:
                raise ValueError("the input is not well-formed UTF-8: the device pre-tokeniser refuses it "
                                 "(a PreTokenizer without an engine takes any bytes)")
            _lib.check(st, "b200bpe_pretokenize_gpu")
        else:
            _lib.check(_lib.lib().b200bpe_pretokenize(arr.ctypes.data, arr.size, mask.ctypes.data), "b200bpe_pretokenize")
        return {"bytes": arr, "wordStarts": mask}

    def preTokenize(self, text: str) -> dict:
        if not text:
            return {"bytes": np.zeros(0, np.uint8), "wordStarts": np.zeros(0, np.uint8)}
        return self.preTokenizeBytes(text.encode("utf-8"))
