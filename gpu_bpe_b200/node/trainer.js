// BPETrainer — BPE vocabulary training on a B200.
//
// Same surface as BPETrainer of the reference (src/bpe/trainer.js): `new BPETrainer(engine)` :134-138,
// `await train(input, {targetVocabSize = 4096, preTokenizer = null, onProgress = null})` :149 →
// {vocab, vocabStrings, vocabSize, merges: [a, b, newId][], trainingTime} :328-334, the
// "No symbols to train on" error for an empty corpus :161-163, merges needed = targetVocabSize −
// the vocabulary's size so far :208 (a second train() continues the ids), the progress payload
// {mergeIndex, totalMerges, mergeString, bestCount, symbolCount, mergesPerSecond} :306-314 once per
// 128 merges, and exportVocab() :368.  The merge loop runs in libb200bpe.so (128 merges per CUDA
// graph launch, one read-back each); without a pre-tokeniser the word starts are tagged on the
// device with the reference's byte-class heuristic (src/bpe/train.wgsl:144-186).
//
// NOT RUN IN THIS REPOSITORY'S TEST SUITE (Node.js is absent from the build image); the Python
// mirror gpu_bpe_b200/trainer.py binds the same C functions and is tested.
'use strict';

const { Vocab } = require('./vocab.js');

const COMPAT_LITERAL = 0, COMPAT_FIXED = 1;

function formatDuration(seconds) {   // trainer.js:31-36
    if (seconds < 60) return `${seconds.toFixed(1)}s`;
    const m = Math.floor(seconds / 60), s = Math.round(seconds % 60);
    return s > 0 ? `${m}m ${s}s` : `${m}m`;
}

/** prepareInput (trainer.js:62-107): → {bytes: Uint8Array, wordStarts: Uint8Array | null} */
async function prepareInput(input, preTokenizer) {
    if (preTokenizer) {
        const r = typeof input === 'string' ? await preTokenizer.preTokenize(input) : await preTokenizer.preTokenizeBytes(input);
        if (r.bytes.length > 0) return { bytes: r.bytes, wordStarts: r.wordStarts };
        // an empty result for a non-empty input: fall back to the raw bytes (trainer.js:71-74)
    }
    const bytes = typeof input === 'string' ? new TextEncoder().encode(input) : input;
    return { bytes, wordStarts: null };
}

class BPETrainer {
    #engine;
    #vocab = new Vocab();

    /** @param {import('./engine.js').BPEEngine} engine @param {{compatMode?: 'literal' | 'fixed'}} [options] */
    constructor(engine, options = {}) {
        this.#engine = engine;
        // 'literal' reproduces the reference as shipped (the compaction bound of train.wgsl:698,727); 'fixed'
        // compacts over every pre-merge position, as the reference's comments describe
        this.compatMode = options.compatMode === 'fixed' ? COMPAT_FIXED : COMPAT_LITERAL;
    }

    async train(input, { targetVocabSize = 4096, preTokenizer = null, onProgress = null } = {}) {
        const started = performance.now();
        const { bytes, wordStarts } = await prepareInput(input, preTokenizer);
        if (bytes.length === 0) throw new Error('No symbols to train on — corpus is empty after pre-processing');
        const vocab = this.#vocab;
        const mergesNeeded = targetVocabSize - vocab.size;
        const merges = [];
        const result = (seconds) => ({
            vocab: vocab.entries, vocabStrings: vocab.strings, vocabSize: vocab.size, merges, trainingTime: formatDuration(seconds),
        });
        if (mergesNeeded <= 0) return result(0);
        const firstTokenId = vocab.nextTokenId;
        // The progress payload carries the merged string, so the vocabulary grows as the batches complete:
        // every report brings the merges finished since the last one (trainer.js:270-276 does this per batch).
        const take = (flat) => {
            for (let i = 0; i < flat.length; i += 3) merges.push([flat[i], flat[i + 1], vocab.addMerge(flat[i], flat[i + 1])]);
        };
        const progress = (p) => {
            take(p.newMerges);
            if (onProgress) {
                onProgress({
                    mergeIndex: p.mergeIndex, totalMerges: p.totalMerges,
                    mergeString: p.bestCount ? vocab.strings[vocab.strings.length - 1] : '—',
                    bestCount: p.bestCount, symbolCount: p.symbolCount, mergesPerSecond: p.mergesPerSecond,
                });
            }
        };
        const out = await this.#engine.addon.train(this.#engine.ctx, bytes, wordStarts, {
            targetVocabSize: firstTokenId + mergesNeeded, firstTokenId, compatMode: this.compatMode, batchMerges: 128,
        }, progress);
        take(out.merges.subarray(merges.length * 3));   // whatever no report has brought yet
        this.earlyStop = out.earlyStop;
        return result((performance.now() - started) / 1000);
    }

    exportVocab() { return this.#vocab.export(); }
}

module.exports = { BPETrainer, prepareInput, formatDuration };
