// TrieTokenizer — chunk-bounded greedy longest-match encoding on a B200.
//
// Same surface as TrieTokenizer of the reference (src/bpe/tokenizer/tokenizer.js): the constructor
// (engine, trieData, vocab, {chunkSize}) :54-85, the static fromVocab :95-98, `await
// encodeBytes(Uint8Array)` → Uint32Array :173-206, decode(tokens) → Uint8Array with U+FFFD for
// unknown ids :18,344-363, destroy() :368, and the fields nodeCount / edgeCount / maxTokenLen.
// The chunk rule (:67-68) and the slicing of inputs beyond the buffer limit (:181-203) live in
// libb200bpe.so; the result depends only on (bytes, trie, chunkSize), as in the reference.
//
// NOT RUN IN THIS REPOSITORY'S TEST SUITE (Node.js is absent from the build image); the Python
// mirror gpu_bpe_b200/tokenizer.py binds the same C functions and is tested.
'use strict';

const { compileVocabToTrie, parseHeader, useAddon } = require('./trie.js');

const UTF8_REPLACEMENT = [0xEF, 0xBF, 0xBD];

class TrieTokenizer {
    #engine;
    #handle;
    #vocab;
    #chunkSize;

    constructor(engine, trieData, vocab, options = {}) {
        this.#engine = engine;
        useAddon(engine.addon);
        this.#vocab = vocab ?? Array.from({ length: 256 }, (_, b) => [b]);
        const header = parseHeader(trieData);                       // throws on a bad magic, version or length
        this.#handle = engine.addon.tokenizerCreate(engine.ctx, trieData, options.chunkSize ?? 0);
        const info = engine.addon.tokenizerInfo(this.#handle);
        this.nodeCount = header.nodeCount;
        this.edgeCount = header.edgeCount;
        this.maxTokenLen = header.maxTokenLen;
        this.#chunkSize = info.chunkSize;
    }

    static fromVocab(engine, vocab, options = {}) {
        useAddon(engine.addon);
        return new TrieTokenizer(engine, compileVocabToTrie(vocab), vocab, options);
    }

    get chunkSize() { return this.#chunkSize; }

    /** @param {Uint8Array} bytes @returns {Promise<Uint32Array>} */
    async encodeBytes(bytes) {
        if (bytes.length === 0) return new Uint32Array(0);
        return this.#engine.addon.encode(this.#handle, bytes);
    }

    /** @param {Uint32Array|number[]} tokens @returns {Uint8Array} */
    decode(tokens) {
        const parts = [];
        let total = 0;
        for (const t of tokens) {
            const id = Number(t);
            const bytes = id < this.#vocab.length ? this.#vocab[id] : UTF8_REPLACEMENT;
            parts.push(bytes);
            total += bytes.length;
        }
        const out = new Uint8Array(total);
        let at = 0;
        for (const p of parts) { out.set(p, at); at += p.length; }
        return out;
    }

    destroy() {
        if (this.#handle) this.#engine.addon.tokenizerDestroy(this.#handle);
        this.#handle = null;
    }
}

module.exports = { TrieTokenizer };
