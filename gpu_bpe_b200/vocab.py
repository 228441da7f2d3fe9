"""Vocab — token registry of the trainer, and the JSON model format.

Mirrors src/bpe/vocab.js:92-143 of the reference (256 byte tokens, addMerge concatenates the
byte strings, display strings, text export) and the JSON written and read by
src/ui/training-manager.js:173-224: {version: 1, vocabSize, vocab: number[][], merges: [[a, b, newId], …]}.
"""
from __future__ import annotations

import json


def _fmt_hex(b: int) -> str:
    return f"<0x{b:02X}>"


def _fmt_ascii(b: int) -> str:
    if b == 0x20:
        return "▁"
    if b == 0x0A:
        return "\\n"
    if 0x21 <= b <= 0x7E:
        return chr(b)
    return _fmt_hex(b)


def bytes_to_display_string(bs) -> str:
    """vocab.js:18-53: UTF-8 where it decodes, <0xNN> for the rest, '▁' for space."""
    parts, i, n = [], 0, len(bs)
    while i < n:
        b = bs[i]
        if b < 0x80:
            parts.append(_fmt_ascii(b)); i += 1; continue
        if b < 0xC0:
            parts.append(_fmt_hex(b)); i += 1; continue
        ln = 2 if b < 0xE0 else 3 if b < 0xF0 else 4
        dec = None
        if i + ln <= n and all((bs[i + j] & 0xC0) == 0x80 for j in range(1, ln)):
            try:
                dec = bytes(bs[i:i + ln]).decode("utf-8")
            except UnicodeDecodeError:
                dec = None
        if dec is not None:
            parts.append(dec); i += ln
        else:
            parts.append(_fmt_hex(b)); i += 1
    return "".join(parts)


class Vocab:
    def __init__(self):
        self.entries: list[list[int]] = [[i] for i in range(256)]
        self.strings: list[str] = [bytes_to_display_string([i]) for i in range(256)]
        self.nextTokenId = 256

    @property
    def size(self) -> int:
        return len(self.entries)

    def addMerge(self, symbolA: int, symbolB: int) -> int:
        new_id = self.nextTokenId
        self.nextTokenId += 1
        merged = self.entries[symbolA] + self.entries[symbolB]
        self.entries.append(merged)
        self.strings.append(bytes_to_display_string(merged))
        return new_id

    def export(self) -> str:
        lines = ["# GPU BPE Vocabulary (WebGPU Trainer)", f"# Total tokens: {len(self.entries)}", ""]
        for i, e in enumerate(self.entries):
            lines.append(f"{i}\t{self.strings[i]}\t[{','.join(map(str, e))}]")
        return "\n".join(lines) + "\n"


def model_to_json(result: dict) -> str:
    """downloadModel (training-manager.js:173-192)."""
    return json.dumps({"version": 1, "vocabSize": result["vocabSize"], "vocab": result["vocab"],
                       "merges": [list(m) for m in result["merges"]]})


def model_from_json(text: str) -> dict:
    """loadFromJSON (training-manager.js:197-224): needs vocab and merges; vocabSize = len(vocab)."""
    data = json.loads(text)
    if "vocab" not in data or "merges" not in data:
        raise ValueError("Invalid model file: missing vocab or merges")
    vocab = [list(v) for v in data["vocab"]]
    return {"vocab": vocab, "vocabStrings": [bytes_to_display_string(v) for v in vocab], "vocabSize": len(vocab),
            "merges": [list(m) for m in data["merges"]], "trainingTime": "loaded"}
