"""TrieTokenizer — trie-walk encoding on a B200.

Mirrors TrieTokenizer of src/bpe/tokenizer/tokenizer.js:21-379 of the reference: constructor
(engine, trieData, vocab, {chunkSize}), fromVocab, encodeBytes → uint32 token ids, decode,
destroy, and the nodeCount / edgeCount / maxTokenLen fields.  encodeBatch is this library's
addition: many documents per call, each encoded as its own encodeBytes call would be.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .trie import compileVocabToTrie, parseHeader

UTF8_REPLACEMENT = [0xEF, 0xBF, 0xBD]  # tokenizer.js:18


class TrieTokenizer:
    def __init__(self, engine, trieData: bytes, vocab=None, options: dict | None = None):
        options = options or {}
        self._engine = engine
        self._vocab = vocab if vocab is not None else [[i] for i in range(256)]
        header = parseHeader(trieData)   # raises the reference's errors for bad magic / version / length
        buf = np.frombuffer(trieData, np.uint8)
        h = C.c_void_p()
        # chunkSize is the reference's option (tokenizer.js:67-68); layout / batchSliceBytes / encodeSliceBytes are this
        # library's (results never depend on them)
        o = _lib.TokOpts()
        o.struct_size = C.sizeof(_lib.TokOpts)
        o.chunk_size = int(options.get("chunkSize") or 0)
        o.layout = _lib.TRIE_LAYOUTS[options.get("layout") or "auto"]
        o.test_lookback_spins = int(options.get("testLookbackSpins") or 0)
        o.batch_slice_bytes = int(options.get("batchSliceBytes") or 0)
        o.encode_slice_bytes = int(options.get("encodeSliceBytes") or 0)
        st = _lib.lib().b200bpe_tokenizer_create_ex(engine.ctx, buf.ctypes.data, buf.size, C.byref(o), C.byref(h))
        if st == 9:
            raise ValueError("Truncated trie data")
        _lib.check(st, "b200bpe_tokenizer_create")
        self._h = h
        self.nodeCount, self.edgeCount, self.maxTokenLen = header["nodeCount"], header["edgeCount"], header["maxTokenLen"]
        cs = C.c_uint32()
        _lib.lib().b200bpe_tokenizer_info(h, None, None, None, C.byref(cs))
        self.chunkSize = cs.value
        d, k = C.c_uint32(), C.c_uint32()
        _lib.lib().b200bpe_tokenizer_layout(h, C.byref(d), C.byref(k))
        self.deviceLayout = (d.value, k.value)   # (2 / 3 cuckoo sub-tables, 1 hybrid, 0 global hash; log2 of the slots)

    @staticmethod
    def fromVocab(engine, vocab, options: dict | None = None) -> "TrieTokenizer":
        return TrieTokenizer(engine, compileVocabToTrie(vocab), vocab, options)

    def encodeBytes(self, data) -> np.ndarray:
        arr = np.frombuffer(bytes(data), np.uint8) if not isinstance(data, np.ndarray) else np.ascontiguousarray(data, np.uint8)
        if arr.size == 0:
            return np.zeros(0, np.uint32)
        out = np.empty(arr.size, np.uint32)
        n = C.c_uint64()
        _lib.check(_lib.lib().b200bpe_encode(self._h, arr.ctypes.data, arr.size, out.ctypes.data, out.size, C.byref(n)),
                   "b200bpe_encode")
        return out[: n.value].copy()

    def encodeBatch(self, data, doc_offsets) -> tuple[np.ndarray, np.ndarray]:
        """→ (token ids of all documents back to back, token offsets per document (n_docs + 1))."""
        arr = np.frombuffer(bytes(data), np.uint8) if not isinstance(data, np.ndarray) else np.ascontiguousarray(data, np.uint8)
        offs = np.ascontiguousarray(doc_offsets, np.uint64)
        nd = offs.size - 1
        out = np.empty(max(1, arr.size), np.uint32)
        toff = np.zeros(nd + 1, np.uint64)
        _lib.check(_lib.lib().b200bpe_encode_batch(self._h, arr.ctypes.data if arr.size else None, offs.ctypes.data, nd,
                                                  out.ctypes.data, out.size, toff.ctypes.data), "b200bpe_encode_batch")
        return out[: int(toff[nd])].copy(), toff

    def encodeDevice(self, d_bytes: int, n: int, d_tokens: int, cap: int) -> int:
        """Device pointers in, token count out; nothing but the count crosses to the host."""
        nt = C.c_uint64()
        _lib.check(_lib.lib().b200bpe_encode_device(self._h, C.c_void_p(d_bytes), n, C.c_void_p(d_tokens), cap, C.byref(nt)),
                   "b200bpe_encode_device")
        return nt.value

    def encodeDeviceNoAlloc(self, d_bytes: int, n: int, d_tokens: int, cap: int) -> int:
        """encodeDevice without any allocation inside the call: the work buffers are a fixed array
        inside the library (at most 1 MiB of input and 8,192 chunks per call).  For callers that
        cannot afford the allocator at encode time.  One call at a time per device."""
        nt = C.c_uint64()
        _lib.check(_lib.lib().b200bpe_encode_device_noalloc(self._h, C.c_void_p(d_bytes), n, C.c_void_p(d_tokens), cap,
                                                           C.byref(nt)), "b200bpe_encode_device_noalloc")
        return nt.value

    def encodeBatchDevice(self, d_bytes: int, d_doc_offsets: int, n_docs: int, n_bytes: int, d_tokens: int, cap: int,
                          d_tok_offsets: int) -> int:
        nt = C.c_uint64()
        _lib.check(_lib.lib().b200bpe_encode_batch_device(self._h, C.c_void_p(d_bytes), C.c_void_p(d_doc_offsets), n_docs,
                                                         n_bytes, C.c_void_p(d_tokens), cap, C.c_void_p(d_tok_offsets),
                                                         C.byref(nt)), "b200bpe_encode_batch_device")
        return nt.value

    def lastKernelMs(self) -> tuple[float, float]:
        a, b = C.c_double(), C.c_double()
        _lib.lib().b200bpe_tokenizer_last_ms(self._h, C.byref(a), C.byref(b))
        return a.value, b.value

    def decode(self, tokens) -> bytes:
        out = bytearray()
        for t in tokens:
            t = int(t)
            out += bytes(self._vocab[t] if t < len(self._vocab) else UTF8_REPLACEMENT)
        return bytes(out)

    def destroy(self):
        if self._h is not None:
            _lib.lib().b200bpe_tokenizer_destroy(self._h)
            self._h = None
