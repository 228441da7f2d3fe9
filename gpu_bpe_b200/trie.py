"""compileVocabToTrie / parseHeader / parseTrieBuffers — the v3 trie binary.

Mirrors src/bpe/tokenizer/trie.js:39,110,137 of the reference; the work is done by the host
code of libb200bpe.so (b200bpe_trie_compile, b200bpe_trie_parse_header).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

HEADER_SIZE = 28


def compileVocabToTrie(vocab) -> bytes:
    flat = bytearray()
    offs = np.zeros(len(vocab) + 1, np.uint64)
    for i, e in enumerate(vocab):
        if e:
            flat += bytes(e)
        offs[i + 1] = len(flat)
    buf = np.frombuffer(bytes(flat) or b"\0", np.uint8)
    need = C.c_size_t(0)
    L = _lib.lib()
    _lib.check(L.b200bpe_trie_compile(buf.ctypes.data, offs.ctypes.data_as(_lib.u64p), len(vocab), None, C.byref(need)))
    out = np.zeros(need.value, np.uint8)
    _lib.check(L.b200bpe_trie_compile(buf.ctypes.data, offs.ctypes.data_as(_lib.u64p), len(vocab), out.ctypes.data,
                                      C.byref(need)), "b200bpe_trie_compile")
    return out.tobytes()


def parseHeader(data: bytes) -> dict:
    f = (C.c_uint32 * 5)()
    buf = np.frombuffer(data, np.uint8)
    st = _lib.lib().b200bpe_trie_parse_header(buf.ctypes.data if buf.size else None, buf.size, f)
    if st == 7:
        magic = int.from_bytes(data[:4], "little")
        raise ValueError(f"Invalid trie magic: 0x{magic:x}")       # trie.js:115-117
    if st == 8:
        raise ValueError(f"Unsupported trie version: {int.from_bytes(data[4:8], 'little')}")  # trie.js:118-120
    if st == 9 and len(data) < HEADER_SIZE:
        raise ValueError("Truncated trie data")
    if st not in (0, 9):
        _lib.check(st, "b200bpe_trie_parse_header")
    return {"version": f[0], "nodeCount": f[1], "edgeCount": f[2], "maxTokenLen": f[3]}


def parseTrieBuffers(data: bytes, header: dict) -> dict:
    """→ {nodes: u32[nodeCount*3], edges: u32[edgeCount*2]} (trie.js:137-160,209-249)."""
    v, nc, ec = header["version"], header["nodeCount"], header["edgeCount"]
    bpn, bpe = (12, 8) if v == 3 else (8, 4)
    if len(data) < HEADER_SIZE + nc * bpn + ec * bpe:
        raise ValueError("Truncated trie data")                   # trie.js:145-147
    raw = np.frombuffer(data, np.uint8)
    if v == 3:
        nodes = raw[HEADER_SIZE:HEADER_SIZE + nc * 12].view("<u4").copy()
        e = raw[HEADER_SIZE + nc * 12:HEADER_SIZE + nc * 12 + ec * 8].view("<u4").reshape(ec, 2).copy()
        e[:, 0] &= 0xFF
        return {"nodes": nodes, "edges": e.reshape(-1)}
    n16 = raw[HEADER_SIZE:HEADER_SIZE + nc * 8].view("<u2").reshape(nc, 4).astype(np.uint32)
    nodes = n16[:, :3].copy()
    nodes[nodes[:, 2] == 0xFFFF, 2] = 0xFFFFFFFF
    e16 = raw[HEADER_SIZE + nc * 8:HEADER_SIZE + nc * 8 + ec * 4].view("<u2").reshape(ec, 2).astype(np.uint32)
    e16[:, 0] &= 0xFF
    return {"nodes": nodes.reshape(-1), "edges": e16.reshape(-1)}
