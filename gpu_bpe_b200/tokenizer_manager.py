"""TokenizerManager — the merge-replay encoder of the reference's Tokenizer tab, on a B200.

Mirrors TokenizerManager.encode of src/ui/tokenizer-manager.js:13-61 of the reference: the text's
UTF-8 bytes become one token each, then the merge rules of the trained model are applied in the
order they were learned, each over the whole token list, left to right.  The result object has the
reference's fields {tokens, text, vocab, vocabStrings}; without a model the call raises the
reference's 'No trained model available', and a model without merges gives the bytes back.
The passes run in libb200bpe.so (b200bpe_replay_*): rounds of "smallest rule rank present" +
single-pass scan and compaction.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib


class TokenizerManager:
    def __init__(self, engine, trained_model: dict | None = None):
        """trained_model: what BPETrainer.train returns (or a loaded vocabulary JSON): needs 'merges',
        and 'vocab' / 'vocabStrings' for the result object."""
        self._engine = engine
        self._model = None
        self._h = None
        if trained_model is not None:
            self.setTrainedModel(trained_model)

    def setTrainedModel(self, model: dict):
        self.destroy()
        self._model = model
        merges = np.ascontiguousarray(np.asarray(model.get("merges") or [], np.uint32).reshape(-1, 3))
        if merges.shape[0]:
            h = C.c_void_p()
            _lib.check(_lib.lib().b200bpe_replay_create(self._engine.ctx, merges.ctypes.data, merges.shape[0], C.byref(h)),
                       "b200bpe_replay_create")
            self._h = h

    def encodeBytes(self, data) -> np.ndarray:
        arr = np.frombuffer(bytes(data), np.uint8) if not isinstance(data, np.ndarray) else np.ascontiguousarray(data, np.uint8)
        if self._model is None:
            raise RuntimeError("No trained model available")          # tokenizer-manager.js:15-17
        if self._h is None or arr.size == 0:
            return arr.astype(np.uint32)                              # no merges: byte level (tokenizer-manager.js:21-25)
        out = np.empty(arr.size, np.uint32)
        n = C.c_uint64()
        _lib.check(_lib.lib().b200bpe_replay_encode(self._h, arr.ctypes.data, arr.size, out.ctypes.data, out.size, C.byref(n)),
                   "b200bpe_replay_encode")
        return out[: n.value].copy()

    def encode(self, text: str) -> dict:
        if self._model is None:
            raise RuntimeError("No trained model available")
        tokens = self.encodeBytes(text.encode("utf-8"))
        return {"tokens": tokens.tolist(), "text": text, "vocab": self._model.get("vocab"),
                "vocabStrings": self._model.get("vocabStrings")}

    def lastRounds(self) -> int:
        r = C.c_uint32()
        if self._h is None:
            return 0
        _lib.check(_lib.lib().b200bpe_replay_last_rounds(self._h, C.byref(r)))
        return r.value

    def destroy(self):
        if self._h is not None:
            _lib.lib().b200bpe_replay_destroy(self._h)
            self._h = None
