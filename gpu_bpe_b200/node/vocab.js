// Vocab — the growing token registry of a training run.
//
// Same surface as Vocab of the reference (src/bpe/vocab.js:92-144): `entries` (byte arrays),
// `strings` (display forms), `nextTokenId` (256 after the single bytes, :98), `size`,
// `addMerge(a, b)` (:118-124) and `export()` with the reference's header and line format (:130-143).
// Display form (:18-88): printable ASCII as itself, space as '▁', newline as '\n', valid multi-byte
// UTF-8 decoded, everything else as <0xHH>.
//
// NOT RUN IN THIS REPOSITORY'S TEST SUITE (Node.js is absent from the build image); the Python
// mirror gpu_bpe_b200/vocab.py implements the same rules and is tested.
'use strict';

const hex = (b) => `<0x${b.toString(16).toUpperCase().padStart(2, '0')}>`;
const strictUtf8 = new TextDecoder('utf-8', { fatal: true });

function displayOfAscii(b) {
    if (b === 0x20) return '▁';
    if (b === 0x0A) return '\\n';
    return b > 0x20 && b < 0x7F ? String.fromCharCode(b) : hex(b);
}

/** @param {number[]} bytes @returns {string} */
function bytesToDisplayString(bytes) {
    let out = '';
    for (let i = 0; i < bytes.length;) {
        const lead = bytes[i];
        if (lead < 0x80) { out += displayOfAscii(lead); i += 1; continue; }
        const want = lead < 0xC0 ? 0 : lead < 0xE0 ? 2 : lead < 0xF0 ? 3 : 4;   // 0: a stray continuation byte
        let text = null;
        if (want && i + want <= bytes.length) {
            let tail = true;
            for (let k = 1; k < want; k++) tail = tail && (bytes[i + k] & 0xC0) === 0x80;
            if (tail) {
                try { text = strictUtf8.decode(Uint8Array.from(bytes.slice(i, i + want))); } catch { text = null; }
            }
        }
        if (text !== null) { out += text; i += want; } else { out += hex(lead); i += 1; }
    }
    return out;
}

class Vocab {
    constructor() {
        this.entries = [];
        this.strings = [];
        this.nextTokenId = 256;
        for (let b = 0; b < 256; b++) {
            this.entries.push([b]);
            this.strings.push(bytesToDisplayString([b]));
        }
    }

    get size() { return this.entries.length; }

    /** @returns {number} the id of the new token */
    addMerge(symbolA, symbolB) {
        const id = this.nextTokenId++;
        const bytes = this.entries[symbolA].concat(this.entries[symbolB]);
        this.entries.push(bytes);
        this.strings.push(bytesToDisplayString(bytes));
        return id;
    }

    export() {
        const rows = this.entries.map((e, i) => `${i}\t${this.strings[i]}\t[${e.join(',')}]`);
        return ['# GPU BPE Vocabulary (WebGPU Trainer)', `# Total tokens: ${this.entries.length}`, '', ...rows].join('\n') + '\n';
    }
}

module.exports = { Vocab, bytesToDisplayString };
