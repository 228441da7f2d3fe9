// BPEEngine — the B200 context behind the reference's engine object.
//
// Stands where BPEEngine of toprakdeviren/gpu-bpe stands (src/bpe/engine.js:216-244: request the
// adapter and device, compile the pipelines; `engine.device` not ready → "Engine not initialized").
// Here init() loads the N-API addon and creates one CUDA context on one B200; there is no WebGPU
// device, no shader compilation and no CPU fallback.
//
// NOT RUN IN THIS REPOSITORY'S TEST SUITE (Node.js is absent from the build image).
'use strict';

const path = require('path');

class BPEEngine {
    #addon = null;
    #ctx = null;

    /** @param {{ device?: number, addonPath?: string }} [options] */
    constructor(options = {}) {
        this.deviceIndex = options.device ?? 0;
        this.addonPath = options.addonPath ?? path.join(__dirname, 'build', 'Release', 'b200bpe.node');
    }

    /** engine.js:216-238 — async like the reference's, although nothing here needs to wait. */
    async init() {
        this.#addon = require(this.addonPath);
        this.#ctx = this.#addon.ctxCreate(this.deviceIndex);   // throws when no sm_100 GPU is visible
        return this;
    }

    get addon() {
        if (!this.#addon) throw new Error('Engine not initialized');   // engine.js:240-244
        return this.#addon;
    }

    get ctx() {
        if (!this.#ctx) throw new Error('Engine not initialized');
        return this.#ctx;
    }

    destroy() {
        if (this.#ctx) this.#addon.ctxDestroy(this.#ctx);
        this.#ctx = null;
    }
}

module.exports = { BPEEngine };
