"""The Export tab of the reference: text files → one token stream → a ".bin" file for a
Transformer trainer (src/ui/export-controller.js).  Host-side mirror over the C ABI."""
from __future__ import annotations

import ctypes as C
import json

import numpy as np

from . import _lib

MAGIC = 0x44584654  # 'DXFT' (export-controller.js:4)
SEPARATOR = b"\n\n"   # between files (export-controller.js:192)


def mergeFiles(files) -> np.ndarray:
    """All files as one byte array, two line feeds between them (export-controller.js:191-202)."""
    parts = [np.frombuffer(bytes(f), np.uint8) if not isinstance(f, np.ndarray) else f.astype(np.uint8, copy=False) for f in files]
    return np.frombuffer(SEPARATOR.join(p.tobytes() for p in parts), np.uint8)


def vocabJson(model: dict | None) -> bytes:
    """JSON.stringify({version, vocabSize, vocab, merges}) as UTF-8 (export-controller.js:224-233); b"" without a model."""
    if model is None:
        return b""
    data = {"version": 1, "vocabSize": model["vocabSize"], "vocab": [list(map(int, v)) for v in model["vocab"]],
            "merges": [list(map(int, m)) for m in model["merges"]]}
    return json.dumps(data, separators=(",", ":"), ensure_ascii=False).encode("utf-8")


def buildBin(tokens, vocabSize: int, vocabBytes: bytes = b"") -> bytes:
    """[MAGIC, vocabSize, tokenCount, vocabBytesLen, ...tokens, ...vocabJSON] (export-controller.js:235-248)."""
    tok = np.ascontiguousarray(tokens, np.uint32)
    size = C.c_uint64()
    _lib.check(_lib.lib().b200bpe_dxft_size(tok.size, len(vocabBytes), C.byref(size)), "b200bpe_dxft_size")
    out = np.empty(size.value, np.uint8)
    js = np.frombuffer(vocabBytes, np.uint8)
    _lib.check(_lib.lib().b200bpe_dxft_write(tok.ctypes.data if tok.size else None, tok.size, int(vocabSize),
                                             js.ctypes.data if js.size else None, js.size, out.ctypes.data, out.size),
               "b200bpe_dxft_write")
    return out.tobytes()


def parseBin(buf: bytes) -> dict:
    """The inverse of buildBin: {vocabSize, tokens, vocab (the embedded JSON object, or None)}."""
    arr = np.frombuffer(buf, np.uint8)
    f = (C.c_uint32 * 4)()
    t_off, j_off = C.c_uint64(), C.c_uint64()
    st = _lib.lib().b200bpe_dxft_parse(arr.ctypes.data if arr.size else None, arr.size, f, C.byref(t_off), C.byref(j_off))
    if st == 7:
        raise ValueError("Invalid .bin magic")
    if st in (1, 9):
        raise ValueError("Truncated .bin data")
    _lib.check(st, "b200bpe_dxft_parse")
    tokens = np.frombuffer(buf, np.uint32, count=f[2], offset=t_off.value).copy()
    js = bytes(buf[j_off.value:j_off.value + f[3]])
    return {"vocabSize": int(f[1]), "tokens": tokens, "vocab": json.loads(js.decode("utf-8")) if js else None}


def exportBin(tokenizer, files, model: dict | None = None) -> tuple[str, bytes]:
    """The whole Export step: join the files, encode on the GPU, write the .bin.
    → (download name "train-v{vocabSize}-{tokenCount}.bin", file bytes) (export-controller.js:179-262)."""
    merged = mergeFiles(files)
    tokens = tokenizer.encodeBytes(merged)
    vocab_size = len(model["vocab"]) if model else (len(tokenizer.vocab) if getattr(tokenizer, "vocab", None) else 256)
    data = buildBin(tokens, vocab_size, vocabJson(model))
    return f"train-v{vocab_size}-{tokens.size}.bin", data
