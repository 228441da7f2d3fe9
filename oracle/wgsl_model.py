"""Dispatch-level Python model of the reference's shaders and host rules.  TEST INFRASTRUCTURE ONLY.

A second, structurally different restatement of the hot path, used to pin the C++ oracle
(oracle/bpe_oracle.cpp) and the CUDA library on small inputs.  Where the C++ oracle works at
the level of "what a merge means", this model walks the reference's own dispatch list one
kernel at a time with the same buffers (valid_mask, block_sums, ping/pong, IterState), in the
order of src/bpe/training-pipeline.js:178-222, so that effects of kernel ORDER (the
compaction bound of train.wgsl:698,727 reading a symbol count that train.wgsl:650-651 has
already replaced) fall out of the structure instead of being coded as a rule.

PARITY UNPINNED: the reference has no tests or golden vectors and cannot run here; the
known-answer table in tests/golden/known_answers.json was derived by hand from the shader
source and is what both restatements are checked against.

Pure-Python loops: only for small cases.  Nothing outside tests/, the smoke check and the
CPU-baseline leg of bench.py may import this module.

Citations are paths inside the toprakdeviren/gpu-bpe project.
"""
from __future__ import annotations

import struct
import unicodedata

WORKGROUP_SIZE = 256           # src/bpe/engine.js:10, train.wgsl:32
WORD_START_BIT = 0x10000       # train.wgsl:36
TOKEN_MASK = 0xFFFF            # train.wgsl:37
INVALID_TOKEN = 0xFFFFFFFF
BATCH_SIZE = 128               # src/bpe/training-pipeline.js:13


# ───────────────────────── word-boundary heuristic (train.wgsl:111-186) ─────────────────────────

def char_class(tok: int) -> int:
    if tok == 0x0A:
        return 4
    if tok == 0x20:
        return 2
    if 0x30 <= tok <= 0x39:
        return 1
    if tok >= 0x80:
        return 0
    if 0x61 <= tok <= 0x7A or 0x41 <= tok <= 0x5A:
        return 0
    return 3


def word_boundary(symbols: list[int]) -> list[int]:
    """bpe_word_boundary on a snapshot of the byte values (every thread reads tokens only)."""
    toks = [s & TOKEN_MASK for s in symbols]
    out = []
    for i, tok in enumerate(toks):
        if i == 0:
            out.append(tok | WORD_START_BIT)
            continue
        c, p = char_class(tok), char_class(toks[i - 1])
        bd = c != p
        if p == 2 and c in (0, 1):
            bd = False
        if c == 2 and p != 2:
            bd = True
        if p == 4 or c == 4:
            bd = True
        out.append(tok | WORD_START_BIT if bd else tok)
    return out


# ───────────────────────── training: one kernel per function ─────────────────────────

def is_better(cn, pn, co, po):  # train.wgsl:83-85
    return cn > co or (cn == co and pn < po)


class TrainModel:
    """Buffers and dispatches of BPETrainer.train (src/bpe/trainer.js:149-335)."""

    def __init__(self, symbols: list[int], first_id: int = 256, literal: bool = True):
        n = len(symbols)
        self.bufA = list(symbols)            # symbolBuf
        self.bufB = [0] * n                  # tb.compact, zero-initialised
        self.valid_mask = [0] * n
        self.block_sums = [0] * ((n + WORKGROUP_SIZE - 1) // WORKGROUP_SIZE)
        self.literal = literal
        # IterState (train.wgsl:45-58, initial values trainer.js:187-196)
        self.state = dict(symbol_count=n, early_stop=0, next_token_id=first_id, symbol_a=0, symbol_b=0,
                          new_symbol=0, max_count=0, merges_done=0, max_symbols=n)
        self.pair_table: dict[int, int] = {}
        self.max_count = 0
        self.max_pair = 0
        self.merge_log: list[tuple[int, int, int]] = []
        self._pre_merge_count = n

    # -- Phase A --
    def clear_table(self):
        self.pair_table = {}

    def pair_count(self, sym):  # train.wgsl:376-431 (exact counting)
        st = self.state
        if st["early_stop"]:
            return
        n = st["symbol_count"]
        for i in range(n - 1):
            rb = sym[i + 1]
            if rb & WORD_START_BIT:
                continue
            a, b = sym[i] & TOKEN_MASK, rb & TOKEN_MASK
            if a == 0 or b == 0:
                continue
            k = (a << 16) | b
            self.pair_table[k] = self.pair_table.get(k, 0) + 1

    def find_max(self):  # train.wgsl:228-318, identity element (0, 0)
        bc, bp = 0, 0
        for p, c in self.pair_table.items():
            if is_better(c, p, bc, bp):
                bc, bp = c, p
        self.max_count, self.max_pair = bc, bp

    def setup_merge(self):  # train.wgsl:340-364
        st = self.state
        if st["early_stop"]:
            return
        if self.max_count < 2 or st["next_token_id"] > TOKEN_MASK:
            st["early_stop"] = 1
            return
        st["symbol_a"], st["symbol_b"] = self.max_pair >> 16, self.max_pair & 0xFFFF
        st["max_count"] = self.max_count
        st["new_symbol"] = st["next_token_id"]
        self.merge_log.append((self.max_pair, st["next_token_id"], self.max_count))
        st["next_token_id"] += 1
        st["merges_done"] += 1

    # -- Phase B --
    def merge_reduce(self, sym):  # train.wgsl:457-520, snapshot reads
        st = self.state
        if st["early_stop"]:
            return
        n, a, b, nw = st["symbol_count"], st["symbol_a"], st["symbol_b"], st["new_symbol"]
        snap = sym[:n]
        nblocks = (n + WORKGROUP_SIZE - 1) // WORKGROUP_SIZE
        sums = [0] * nblocks
        for i in range(n):
            raw = snap[i]
            raw_prev = snap[i - 1] if i > 0 else 0
            raw_next = snap[i + 1] if i + 1 < n else 0
            if (i + 1 < n and not (raw_next & WORD_START_BIT) and (raw & TOKEN_MASK) == a
                    and (raw_next & TOKEN_MASK) == b):
                sym[i] = nw | (raw & WORD_START_BIT)
            valid = 1
            if i > 0 and not (raw & WORD_START_BIT) and (raw_prev & TOKEN_MASK) == a and (raw & TOKEN_MASK) == b:
                valid = 0
            self.valid_mask[i] = valid
            sums[i // WORKGROUP_SIZE] += valid
        for blk in range(nblocks):
            self.block_sums[blk] = sums[blk]

    def scan_blocks(self):  # train.wgsl:548-618 / 636-662 — also publishes the new count
        st = self.state
        if st["early_stop"]:
            return
        self._pre_merge_count = st["symbol_count"]
        nblocks = (st["symbol_count"] + WORKGROUP_SIZE - 1) // WORKGROUP_SIZE
        s = 0
        for i in range(nblocks):
            v = self.block_sums[i]
            self.block_sums[i] = s
            s += v
        st["symbol_count"] = s

    def finalize_compact(self, src, dst, dispatched_threads):  # train.wgsl:686-731
        st = self.state
        bound = st["symbol_count"] if self.literal else self._pre_merge_count
        for blk in range((dispatched_threads + WORKGROUP_SIZE - 1) // WORKGROUP_SIZE):
            rank = 0
            for lid in range(WORKGROUP_SIZE):
                fid = blk * WORKGROUP_SIZE + lid
                v = (self.valid_mask[fid] & 1) if fid < bound else 0
                if fid < bound and v == 1:
                    dst[self.block_sums[blk] + rank] = src[fid]
                rank += v

    def run_batch(self, batch_merges: int, ping, pong):
        """encodeBatch (training-pipeline.js:178-222): 8 dispatches per merge, ping/pong by parity."""
        for i in range(batch_merges):
            a, b = (ping, pong) if i % 2 == 0 else (pong, ping)
            stopped_before = self.state["early_stop"]
            self.clear_table()
            self.pair_count(a)
            self.find_max()
            self.setup_merge()
            if self.state["early_stop"]:
                # Once stopped, merge/scan write nothing (train.wgsl:466,517,554,599,604,639);
                # the unguarded compaction only scribbles into the buffer nobody reads again.
                _ = stopped_before
                continue
            pre = self.state["symbol_count"]
            self.merge_reduce(a)
            self.scan_blocks()
            self.finalize_compact(a, b, pre)

    def train(self, merges_needed: int):
        """Host loop (trainer.js:225-335).  Returns (merges [a,b,id,count], early_stop, live symbols)."""
        ping, pong = self.bufA, self.bufB
        merges, total, early = [], 0, False
        while total < merges_needed and not early:
            batch = min(BATCH_SIZE, merges_needed - total)
            self.state["merges_done"] = 0
            self.merge_log = []
            self.run_batch(batch, ping, pong)
            done = self.state["merges_done"]
            early = self.state["early_stop"] != 0
            for pair, nid, cnt in self.merge_log[:done]:
                merges.append([pair >> 16, pair & 0xFFFF, nid, cnt])
            total += done
            if done % 2:
                ping, pong = pong, ping
        return merges, early, ping[: self.state["symbol_count"]]


def train(symbols, merges_needed, first_id=256, literal=True):
    return TrainModel(symbols, first_id, literal).train(merges_needed)


# ───────────────────────── vocabulary (src/bpe/vocab.js:92-124) ─────────────────────────

def vocab_from_merges(merges) -> list[list[int]]:
    entries = [[i] for i in range(256)]
    for m in merges:
        entries.append(entries[m[0]] + entries[m[1]])
    return entries


# ───────────────────────── trie compile (src/bpe/tokenizer/trie.js:39-98,167-206) ─────────────────────────

def compile_vocab_to_trie(vocab) -> bytes:
    root = {"children": {}, "tokenId": INVALID_TOKEN}
    max_len = 0
    for token_id, bs in enumerate(vocab):
        if not bs:
            continue
        node = root
        for byte in bs:
            nxt = node["children"].get(byte)
            if nxt is None:
                nxt = {"children": {}, "tokenId": INVALID_TOKEN}
                node["children"][byte] = nxt
            node = nxt
        node["tokenId"] = token_id          # duplicates: the last id wins
        max_len = max(max_len, len(bs))
    flat_nodes, flat_edges = [None], []
    queue, index = [root], {id(root): 0}
    head = 0
    while head < len(queue):
        tn = queue[head]
        head += 1
        my = index[id(tn)]
        entries = sorted(tn["children"].items())
        first = len(flat_edges)
        for symv, child in entries:
            ci = len(queue)
            index[id(child)] = ci
            queue.append(child)
            flat_nodes.append(None)
            flat_edges.append((symv, ci))
        flat_nodes[my] = (first, len(entries), tn["tokenId"])
    out = bytearray(struct.pack("<7I", 0x54524945, 3, len(flat_nodes), len(flat_edges), max_len, len(vocab), 0))
    for fc, nc, tid in flat_nodes:
        out += struct.pack("<3I", fc, nc, tid)
    for symv, tgt in flat_edges:
        out += struct.pack("<BBBBI", symv, 0, 0, 0, tgt)
    return bytes(out)


def parse_trie(data: bytes):
    """parseHeader + parseTrieBuffers for v3 (trie.js:110-160)."""
    if len(data) < 28:
        raise ValueError("Truncated trie data")
    magic, version, nc, ec, mtl, vs, _flags = struct.unpack_from("<7I", data, 0)
    if magic != 0x54524945:
        raise ValueError(f"Invalid trie magic: 0x{magic:x}")
    if version != 3:
        raise ValueError(f"Unsupported trie version: {version}")
    if len(data) < 28 + nc * 12 + ec * 8:
        raise ValueError("Truncated trie data")
    nodes = struct.unpack_from(f"<{nc * 3}I", data, 28)
    raw = struct.unpack_from(f"<{ec * 2}I", data, 28 + nc * 12)
    edges = [(raw[2 * i] & 0xFF, raw[2 * i + 1]) for i in range(ec)]
    return dict(nodeCount=nc, edgeCount=ec, maxTokenLen=mtl, vocabSize=vs, nodes=nodes, edges=edges)


def default_chunk_size(max_token_len: int) -> int:  # tokenizer.js:17,67-68
    return max(512, min(2048, max_token_len * 8))


def encode_bytes(data: bytes, trie: bytes, chunk_size: int | None = None) -> list[int]:
    """trie_tokenizer_chunked + prefix sum + compact (tokenize.wgsl:88-243)."""
    t = parse_trie(trie)
    nodes, edges = t["nodes"], t["edges"]
    cs = chunk_size or default_chunk_size(t["maxTokenLen"])
    out: list[int] = []
    n = len(data)
    for c0 in range(0, n, cs):
        ce = min(n, c0 + cs)
        pos = c0
        while pos < ce:
            cn, lmt, lmp, wp = 0, INVALID_TOKEN, pos, pos
            while wp < ce:
                fc, nc = nodes[cn * 3], nodes[cn * 3 + 1] & 0xFFFF
                nn = INVALID_TOKEN
                for e in range(fc, fc + nc):
                    if edges[e][0] == data[wp]:
                        nn = edges[e][1]
                        break
                if nn == INVALID_TOKEN:
                    break
                cn = nn
                wp += 1
                ti = nodes[cn * 3 + 2]
                if ti != INVALID_TOKEN:
                    lmt, lmp = ti, wp
            if lmt != INVALID_TOKEN:
                out.append(lmt)
                pos = lmp
            else:
                out.append(data[pos])
                pos += 1
    return out


def decode(tokens, vocab) -> bytes:  # tokenizer.js:344-363
    out = bytearray()
    for t in tokens:
        out += bytes(vocab[t]) if t < len(vocab) else b"\xef\xbf\xbd"
    return bytes(out)


# ───────────────────────── pre-tokenizer (src/wasm/pre_tokenizer.mjs) ─────────────────────────

LETTER, DIGIT, WHITESPACE, PUNCT, SYMBOL, NEWLINE, OTHER = range(7)
_NEWLINES = {0x0A, 0x0D, 0x85, 0x2028, 0x2029}
_APOS = {0x27, 0x2019}
_SINGLE = set(b"sStTmMdD")
_TWO = [(0x72, 0x52, 0x65, 0x45), (0x76, 0x56, 0x65, 0x45), (0x6C, 0x4C, 0x6C, 0x4C)]


def classify(cp: int) -> int:
    """pre_tokenizer.mjs:126-134 over General_Category (the predicates of decoder.mjs:244-256).

    Whitespace = Z* plus the control characters with the Unicode White_Space property (TAB, VT, FF;
    LF, CR and NEL are newlines first).
    """
    if cp in _NEWLINES:
        return NEWLINE
    cat = unicodedata.category(chr(cp))
    if cat[0] in "LM":
        return LETTER
    if cat[0] == "N":
        return DIGIT
    if cat[0] == "Z" or cp in (0x09, 0x0B, 0x0C):
        return WHITESPACE
    if cat[0] == "P":
        return PUNCT
    if cat[0] == "S":
        return SYMBOL
    return OTHER


def _match_contraction(cps, cls, i):  # pre_tokenizer.mjs:83-110
    n = len(cps)
    if i + 1 >= n:
        return 0
    nxt = cps[i + 1]
    if nxt in _SINGLE and (i + 2 >= n or cls[i + 2] != LETTER):
        return 2
    if i + 2 < n:
        nn = cps[i + 2]
        after = i + 3 >= n or cls[i + 3] != LETTER
        for lo1, hi1, lo2, hi2 in _TWO:
            if nxt in (lo1, hi1) and nn in (lo2, hi2) and after:
                return 3
    return 0


def _transition(prev, cur):  # pre_tokenizer.mjs:175-189
    ps = lambda c: c in (PUNCT, SYMBOL)
    return ((prev == LETTER and cur == DIGIT) or (prev == DIGIT and cur == LETTER)
            or (prev == LETTER and ps(cur)) or (ps(prev) and cur == LETTER)
            or (ps(prev) and cur == DIGIT) or (prev == DIGIT and ps(cur)))


def find_word_boundaries(cps, cls):  # pre_tokenizer.mjs:226-292
    n = len(cps)
    starts = [0] * n
    if n == 0:
        return starts
    starts[0] = 1
    i = 1
    while i < n:
        prev, cur = cls[i - 1], cls[i]
        if cur == NEWLINE or prev == NEWLINE:
            starts[i] = 1
            i += 1
            continue
        if cur == WHITESPACE:
            if prev != WHITESPACE:
                starts[i] = 1
            i += 1
            continue
        if prev == WHITESPACE:
            i += 1
            continue
        if prev == LETTER and cps[i] in _APOS:
            k = _match_contraction(cps, cls, i)
            if k > 0:
                i += k
                continue
        if _transition(prev, cur):
            starts[i] = 1
            i += 1
            continue
        if cur == DIGIT and prev == DIGIT:
            rs = i - 1
            while rs > 0 and cls[rs - 1] == DIGIT:
                rs -= 1
            if (i - rs) % 3 == 0:
                starts[i] = 1
        i += 1
    return starts


def pretokenize_bytes(raw: bytes, normalize: bool = True):
    """preTokenizeBytes (pre_tokenizer.mjs:459-509): NFC, classify, boundaries, byte mask."""
    text = raw.decode("utf-8")
    if normalize:
        text = unicodedata.normalize("NFC", text)
    cps = [ord(ch) for ch in text]
    cls = [classify(c) for c in cps]
    st = find_word_boundaries(cps, cls)
    data = text.encode("utf-8")
    mask = bytearray(len(data))
    pos = 0
    for c, s in zip(cps, st):
        if s:
            mask[pos] = 1
        pos += 1 if c <= 0x7F else 2 if c <= 0x7FF else 3 if c <= 0xFFFF else 4
    return data, bytes(mask)


def tag_symbols(data: bytes, mask: bytes | None) -> list[int]:
    """bytes (+mask) → tagged u32 symbols (trainer.js:76-79,115-121); heuristic when no mask."""
    if mask is None:
        return word_boundary(list(data))
    return [b | (WORD_START_BIT if m else 0) for b, m in zip(data, mask)]


# ── the Export tab's ".bin" file (src/ui/export-controller.js:4,191-202,224-248) ──
DXFT_MAGIC = 0x44584654


def merge_files(files) -> bytes:
    """Files joined by two line feeds (export-controller.js:191-202)."""
    return b"\n\n".join(bytes(f) for f in files)


def vocab_json(model) -> bytes:
    """JSON.stringify({version, vocabSize, vocab, merges}) (export-controller.js:224-233)."""
    if model is None:
        return b""
    import json
    return json.dumps({"version": 1, "vocabSize": model["vocabSize"], "vocab": model["vocab"], "merges": model["merges"]},
                      separators=(",", ":"), ensure_ascii=False).encode("utf-8")


def dxft_bytes(tokens, vocab_size: int, vocab_bytes: bytes = b"") -> bytes:
    """[MAGIC, vocabSize, tokenCount, vocabBytesLen] as u32 LE, the tokens as u32 LE, the JSON (export-controller.js:235-248)."""
    import struct
    tokens = [int(t) for t in tokens]
    return struct.pack("<4I", DXFT_MAGIC, vocab_size, len(tokens), len(vocab_bytes)) + struct.pack(f"<{len(tokens)}I", *tokens) + vocab_bytes
