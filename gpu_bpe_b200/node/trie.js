// Trie compiler and parsers — compileVocabToTrie, parseHeader, parseTrieBuffers.
//
// Same names, arguments, results and error texts as src/bpe/tokenizer/trie.js of the reference
// (:39 compileVocabToTrie(vocab) → ArrayBuffer in the v3 format; :110 parseHeader(data) →
// {version, nodeCount, edgeCount, maxTokenLen, vocabSize}, throwing "Invalid trie magic",
// "Unsupported trie version" or "Truncated trie data"; :137 parseTrieBuffers(data, header) →
// {nodes: Uint32Array, edges: Uint32Array}).  The compiler itself runs in libb200bpe.so
// (b200bpe_trie_compile), whose output is byte-identical to the reference's.
//
// NOT RUN IN THIS REPOSITORY'S TEST SUITE (Node.js is absent from the build image); the Python
// mirror gpu_bpe_b200/trie.py binds the same C functions and is tested.
'use strict';

const HEADER_BYTES = 28;   // magic, version, nodeCount, edgeCount, maxTokenLen, vocabSize, flags

let addon = null;
/** The addon is handed over once (by BPEEngine.init through the tokenizer module) or set by hand. */
function useAddon(a) { addon = a; }
function theAddon() {
    if (!addon) throw new Error('Engine not initialized');
    return addon;
}

/** @param {number[][]} vocab byte arrays indexed by token id; empty entries are skipped, later duplicates win @returns {ArrayBuffer} */
function compileVocabToTrie(vocab) {
    const offsets = new BigUint64Array(vocab.length + 1);
    let total = 0;
    for (let i = 0; i < vocab.length; i++) { offsets[i] = BigInt(total); total += vocab[i].length; }
    offsets[vocab.length] = BigInt(total);
    const bytes = new Uint8Array(total);
    let at = 0;
    for (const entry of vocab) { bytes.set(entry, at); at += entry.length; }
    return theAddon().trieCompile(bytes, offsets);
}

/** @param {ArrayBuffer} data */
function parseHeader(data) {
    return theAddon().trieParseHeader(data);   // throws the reference's three messages
}

/** v3: 12-byte nodes {firstChild, numChildren, tokenId}, 8-byte edges {symbol, target}; v2: the 16-bit legacy layout widened */
function parseTrieBuffers(data, header) {
    const nodeBytes = header.version === 3 ? 12 : 8, edgeBytes = header.version === 3 ? 8 : 4;
    if (data.byteLength < HEADER_BYTES + header.nodeCount * nodeBytes + header.edgeCount * edgeBytes) throw new Error('Truncated trie data');
    const nodes = new Uint32Array(header.nodeCount * 3), edges = new Uint32Array(header.edgeCount * 2);
    const view = new DataView(data);
    let at = HEADER_BYTES;
    if (header.version === 3) {
        for (let i = 0; i < nodes.length; i++, at += 4) nodes[i] = view.getUint32(at, true);
        for (let i = 0; i < header.edgeCount; i++, at += 8) {
            edges[2 * i] = view.getUint8(at);
            edges[2 * i + 1] = view.getUint32(at + 4, true);
        }
    } else {
        for (let i = 0; i < header.nodeCount; i++, at += 8) {
            nodes[3 * i] = view.getUint16(at, true);
            nodes[3 * i + 1] = view.getUint16(at + 2, true);
            const tok = view.getUint16(at + 4, true);
            nodes[3 * i + 2] = tok === 0xFFFF ? 0xFFFFFFFF : tok;
        }
        for (let i = 0; i < header.edgeCount; i++, at += 4) {
            edges[2 * i] = view.getUint16(at, true) & 0xFF;
            edges[2 * i + 1] = view.getUint16(at + 2, true);
        }
    }
    return { nodes, edges };
}

module.exports = { compileVocabToTrie, parseHeader, parseTrieBuffers, useAddon };
