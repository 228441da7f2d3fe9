// N-API addon: the thin bridge between the JavaScript mirrors in this directory (trainer.js,
// tokenizer.js, trie.js) and the C ABI of libb200bpe.so (include/b200bpe.h).
//
// NOT COMPILED OR RUN IN THIS REPOSITORY'S TEST SUITE: Node.js and node_api.h are absent from the
// build image.  The file is written against the stable Node-API (version 8); build it where Node is
// installed with the binding.gyp beside it (`npx node-gyp rebuild`), with libb200bpe.so on the
// linker and loader paths.
//
// Conventions kept from the reference's JavaScript surface (toprakdeviren/gpu-bpe):
//   * long-running calls return Promises (BPETrainer.train src/bpe/trainer.js:149,
//     TrieTokenizer.encodeBytes src/bpe/tokenizer/tokenizer.js:173); the work runs on the libuv pool
//   * failures reject / throw an Error whose message is the reference's text where it has one
//     (b200bpe_status_str carries those texts)
//   * inputs are borrowed typed arrays, outputs are fresh typed arrays owned by the caller
//   * one call at a time per object (the reference's pooled buffers have the same rule)
#include <node_api.h>

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/b200bpe.h"

namespace {

#define NAPI_OK(call)                                                        \
    do {                                                                     \
        if ((call) != napi_ok) {                                             \
            napi_throw_error(env, nullptr, "b200bpe addon: N-API call failed: " #call); \
            return nullptr;                                                  \
        }                                                                    \
    } while (0)

std::string status_text(b200bpe_status st) {
    std::string s = b200bpe_status_str(st);
    const char* detail = b200bpe_last_error();
    if (detail && *detail) s += std::string(" (") + detail + ")";
    return s;
}

napi_value make_error(napi_env env, const std::string& text) {
    napi_value msg, err;
    napi_create_string_utf8(env, text.c_str(), text.size(), &msg);
    napi_create_error(env, nullptr, msg, &err);
    return err;
}

template <typename T>
T* unwrap(napi_env env, napi_value v) {
    void* p = nullptr;
    if (napi_get_value_external(env, v, &p) != napi_ok) return nullptr;
    return static_cast<T*>(p);
}

bool typed_bytes(napi_env env, napi_value v, const uint8_t** data, size_t* len) {
    bool is_ta = false;
    if (napi_is_typedarray(env, v, &is_ta) != napi_ok || !is_ta) return false;
    napi_typedarray_type type;
    void* p = nullptr;
    size_t n = 0;
    if (napi_get_typedarray_info(env, v, &type, &n, &p, nullptr, nullptr) != napi_ok) return false;
    if (type != napi_uint8_array && type != napi_uint8_clamped_array) return false;
    *data = static_cast<const uint8_t*>(p);
    *len = n;
    return true;
}

uint32_t get_u32(napi_env env, napi_value obj, const char* name, uint32_t fallback) {
    napi_value v;
    bool has = false;
    if (napi_has_named_property(env, obj, name, &has) != napi_ok || !has) return fallback;
    if (napi_get_named_property(env, obj, name, &v) != napi_ok) return fallback;
    uint32_t out = fallback;
    napi_valuetype t;
    if (napi_typeof(env, v, &t) == napi_ok && t == napi_number) napi_get_value_uint32(env, v, &out);
    return out;
}

// ── context: replaces BPEEngine.init() (src/bpe/engine.js:216-238) ──
napi_value CtxCreate(napi_env env, napi_callback_info info) {
    size_t argc = 1;
    napi_value argv[1];
    NAPI_OK(napi_get_cb_info(env, info, &argc, argv, nullptr, nullptr));
    int32_t device = 0;
    if (argc >= 1) napi_get_value_int32(env, argv[0], &device);
    b200bpe_ctx* ctx = nullptr;
    const b200bpe_status st = b200bpe_ctx_create(device, &ctx);
    if (st != B200BPE_OK) { napi_throw(env, make_error(env, status_text(st))); return nullptr; }
    napi_value ext;
    NAPI_OK(napi_create_external(env, ctx, nullptr, nullptr, &ext));
    return ext;
}

napi_value CtxDestroy(napi_env env, napi_callback_info info) {
    size_t argc = 1;
    napi_value argv[1];
    NAPI_OK(napi_get_cb_info(env, info, &argc, argv, nullptr, nullptr));
    if (argc >= 1) b200bpe_ctx_destroy(unwrap<b200bpe_ctx>(env, argv[0]));
    return nullptr;
}

// ── training: BPETrainer.train (src/bpe/trainer.js:149-335) ──
struct ProgressMsg {
    b200bpe_progress p;
    std::vector<uint32_t> fresh;   // {a, b, newId} of the merges completed since the last report
};

struct TrainJob {
    napi_async_work work = nullptr;
    napi_deferred deferred = nullptr;
    napi_threadsafe_function progress = nullptr;   // may be null
    napi_ref keep_bytes = nullptr, keep_mask = nullptr;   // the borrowed inputs stay alive until the work is done
    b200bpe_ctx* ctx = nullptr;
    const uint8_t* bytes = nullptr;
    const uint8_t* mask = nullptr;
    uint64_t n = 0;
    b200bpe_train_opts opts{};
    std::vector<uint32_t> merges, counts;
    uint32_t n_merges = 0, early_stop = 0, reported = 0;
    b200bpe_status status = B200BPE_OK;
    std::string error;
};

void progress_to_js(napi_env env, napi_value js_cb, void*, void* data) {
    ProgressMsg* m = static_cast<ProgressMsg*>(data);
    if (env && js_cb) {
        // the fields of trainer.js:306-314, minus the merged string, which trainer.js (the mirror) adds
        napi_value obj, v, undefined;
        napi_create_object(env, &obj);
        napi_create_uint32(env, m->p.merge_index, &v); napi_set_named_property(env, obj, "mergeIndex", v);
        napi_create_uint32(env, m->p.total_merges, &v); napi_set_named_property(env, obj, "totalMerges", v);
        napi_create_uint32(env, m->p.last_a, &v); napi_set_named_property(env, obj, "lastA", v);
        napi_create_uint32(env, m->p.last_b, &v); napi_set_named_property(env, obj, "lastB", v);
        napi_create_uint32(env, m->p.last_count, &v); napi_set_named_property(env, obj, "bestCount", v);
        napi_create_double(env, (double)m->p.symbol_count, &v); napi_set_named_property(env, obj, "symbolCount", v);
        napi_create_double(env, m->p.merges_per_second, &v); napi_set_named_property(env, obj, "mergesPerSecond", v);
        void* dst = nullptr;
        napi_value ab;
        napi_create_arraybuffer(env, m->fresh.size() * 4, &dst, &ab);
        std::memcpy(dst, m->fresh.data(), m->fresh.size() * 4);
        napi_create_typedarray(env, napi_uint32_array, m->fresh.size(), ab, 0, &v);
        napi_set_named_property(env, obj, "newMerges", v);   // so that the caller's vocabulary can grow batch by batch
        napi_get_undefined(env, &undefined);
        napi_call_function(env, undefined, js_cb, 1, &obj, nullptr);
    }
    delete m;
}

void progress_from_library(const b200bpe_progress* p, void* user) {
    TrainJob* job = static_cast<TrainJob*>(user);
    if (!job->progress) return;
    // the library has written the merges up to merge_index into the output buffer before it reports
    ProgressMsg* m = new ProgressMsg{*p, {}};
    const uint32_t upto = p->merge_index <= (uint32_t)job->counts.size() ? p->merge_index : (uint32_t)job->counts.size();
    if (upto > job->reported) m->fresh.assign(job->merges.begin() + (size_t)job->reported * 3, job->merges.begin() + (size_t)upto * 3);
    job->reported = upto;
    if (napi_call_threadsafe_function(job->progress, m, napi_tsfn_nonblocking) != napi_ok) delete m;
}

void train_execute(napi_env, void* data) {
    TrainJob* job = static_cast<TrainJob*>(data);
    job->status = b200bpe_train(job->ctx, job->bytes, job->mask, job->n, &job->opts, job->merges.data(), job->counts.data(),
                                &job->n_merges, &job->early_stop, job->progress ? progress_from_library : nullptr, job);
    if (job->status != B200BPE_OK) job->error = status_text(job->status);
}

void train_complete(napi_env env, napi_status, void* data) {
    TrainJob* job = static_cast<TrainJob*>(data);
    if (job->status != B200BPE_OK) {
        napi_reject_deferred(env, job->deferred, make_error(env, job->error));
    } else {
        napi_value result, ab, ta, v;
        void* dst = nullptr;
        napi_create_object(env, &result);
        napi_create_arraybuffer(env, (size_t)job->n_merges * 12, &dst, &ab);
        std::memcpy(dst, job->merges.data(), (size_t)job->n_merges * 12);
        napi_create_typedarray(env, napi_uint32_array, (size_t)job->n_merges * 3, ab, 0, &ta);
        napi_set_named_property(env, result, "merges", ta);     // a, b, newId per merge (trainer.js:270-276)
        napi_create_arraybuffer(env, (size_t)job->n_merges * 4, &dst, &ab);
        std::memcpy(dst, job->counts.data(), (size_t)job->n_merges * 4);
        napi_create_typedarray(env, napi_uint32_array, job->n_merges, ab, 0, &ta);
        napi_set_named_property(env, result, "counts", ta);
        napi_get_boolean(env, job->early_stop != 0, &v);
        napi_set_named_property(env, result, "earlyStop", v);
        napi_resolve_deferred(env, job->deferred, result);
    }
    if (job->progress) napi_release_threadsafe_function(job->progress, napi_tsfn_release);
    if (job->keep_bytes) napi_delete_reference(env, job->keep_bytes);
    if (job->keep_mask) napi_delete_reference(env, job->keep_mask);
    napi_delete_async_work(env, job->work);
    delete job;
}

// train(ctx, bytes: Uint8Array, wordStarts: Uint8Array | null, {targetVocabSize, firstTokenId, compatMode, batchMerges}, onProgress | null)
napi_value Train(napi_env env, napi_callback_info info) {
    size_t argc = 5;
    napi_value argv[5];
    NAPI_OK(napi_get_cb_info(env, info, &argc, argv, nullptr, nullptr));
    if (argc < 4) { napi_throw_error(env, nullptr, "train(ctx, bytes, wordStarts, options[, onProgress])"); return nullptr; }
    TrainJob* job = new TrainJob();
    job->ctx = unwrap<b200bpe_ctx>(env, argv[0]);
    size_t nb = 0, nm = 0;
    if (!job->ctx || !typed_bytes(env, argv[1], &job->bytes, &nb)) { delete job; napi_throw_type_error(env, nullptr, "bytes must be a Uint8Array"); return nullptr; }
    napi_valuetype mt;
    napi_typeof(env, argv[2], &mt);
    if (mt != napi_null && mt != napi_undefined) {
        if (!typed_bytes(env, argv[2], &job->mask, &nm) || nm != nb) { delete job; napi_throw_type_error(env, nullptr, "wordStarts must be a Uint8Array as long as bytes"); return nullptr; }
        napi_create_reference(env, argv[2], 1, &job->keep_mask);
    }
    napi_create_reference(env, argv[1], 1, &job->keep_bytes);
    job->n = nb;
    std::memset(&job->opts, 0, sizeof(job->opts));
    job->opts.struct_size = sizeof(job->opts);
    job->opts.target_vocab_size = get_u32(env, argv[3], "targetVocabSize", 4096);   // trainer.js:149
    job->opts.first_token_id = get_u32(env, argv[3], "firstTokenId", 256);           // vocab.js:98
    job->opts.compat_mode = get_u32(env, argv[3], "compatMode", B200BPE_COMPAT_LITERAL);
    job->opts.batch_merges = get_u32(env, argv[3], "batchMerges", 128);              // training-pipeline.js:13
    const uint32_t room = job->opts.target_vocab_size > job->opts.first_token_id ? job->opts.target_vocab_size - job->opts.first_token_id : 0;
    job->merges.resize((size_t)room * 3 + 3);
    job->counts.resize((size_t)room + 1);
    if (argc >= 5) {
        napi_valuetype ft;
        napi_typeof(env, argv[4], &ft);
        if (ft == napi_function) {
            napi_value name;
            napi_create_string_utf8(env, "b200bpe progress", NAPI_AUTO_LENGTH, &name);
            napi_create_threadsafe_function(env, argv[4], nullptr, name, 0, 1, nullptr, nullptr, nullptr, progress_to_js, &job->progress);
        }
    }
    napi_value promise, name;
    NAPI_OK(napi_create_promise(env, &job->deferred, &promise));
    napi_create_string_utf8(env, "b200bpe train", NAPI_AUTO_LENGTH, &name);
    NAPI_OK(napi_create_async_work(env, nullptr, name, train_execute, train_complete, job, &job->work));
    NAPI_OK(napi_queue_async_work(env, job->work));
    return promise;
}

// ── trie: compileVocabToTrie / parseHeader (src/bpe/tokenizer/trie.js:39,110) ──
// trieCompile(vocabBytes: Uint8Array, offsets: BigUint64Array(vocabSize + 1)) → ArrayBuffer (v3 binary)
napi_value TrieCompile(napi_env env, napi_callback_info info) {
    size_t argc = 2;
    napi_value argv[2];
    NAPI_OK(napi_get_cb_info(env, info, &argc, argv, nullptr, nullptr));
    const uint8_t* bytes = nullptr;
    size_t nb = 0;
    if (argc < 2 || !typed_bytes(env, argv[0], &bytes, &nb)) { napi_throw_type_error(env, nullptr, "trieCompile(vocabBytes, offsets)"); return nullptr; }
    napi_typedarray_type type;
    void* off = nullptr;
    size_t n_off = 0;
    NAPI_OK(napi_get_typedarray_info(env, argv[1], &type, &n_off, &off, nullptr, nullptr));
    if (type != napi_biguint64_array || n_off == 0) { napi_throw_type_error(env, nullptr, "offsets must be a BigUint64Array"); return nullptr; }
    size_t len = 0;
    b200bpe_status st = b200bpe_trie_compile(bytes, static_cast<const uint64_t*>(off), (uint32_t)(n_off - 1), nullptr, &len);
    if (st != B200BPE_OK) { napi_throw(env, make_error(env, status_text(st))); return nullptr; }
    void* dst = nullptr;
    napi_value ab;
    NAPI_OK(napi_create_arraybuffer(env, len, &dst, &ab));
    st = b200bpe_trie_compile(bytes, static_cast<const uint64_t*>(off), (uint32_t)(n_off - 1), dst, &len);
    if (st != B200BPE_OK) { napi_throw(env, make_error(env, status_text(st))); return nullptr; }
    return ab;
}

// trieParseHeader(data: ArrayBuffer) → {version, nodeCount, edgeCount, maxTokenLen, vocabSize}; throws the
// reference's texts: "Invalid trie magic", "Unsupported trie version", "Truncated trie data" (trie.js:115-120,145-147)
napi_value TrieParseHeader(napi_env env, napi_callback_info info) {
    size_t argc = 1;
    napi_value argv[1];
    NAPI_OK(napi_get_cb_info(env, info, &argc, argv, nullptr, nullptr));
    void* data = nullptr;
    size_t len = 0;
    if (argc < 1 || napi_get_arraybuffer_info(env, argv[0], &data, &len) != napi_ok) { napi_throw_type_error(env, nullptr, "trieParseHeader(ArrayBuffer)"); return nullptr; }
    uint32_t f[5];
    const b200bpe_status st = b200bpe_trie_parse_header(data, len, f);
    if (st != B200BPE_OK) { napi_throw(env, make_error(env, b200bpe_status_str(st))); return nullptr; }
    static const char* names[5] = {"version", "nodeCount", "edgeCount", "maxTokenLen", "vocabSize"};
    napi_value obj, v;
    NAPI_OK(napi_create_object(env, &obj));
    for (int i = 0; i < 5; i++) { napi_create_uint32(env, f[i], &v); napi_set_named_property(env, obj, names[i], v); }
    return obj;
}

// ── tokenizer: TrieTokenizer (src/bpe/tokenizer/tokenizer.js:54-98,173-335,368) ──
napi_value TokenizerCreate(napi_env env, napi_callback_info info) {
    size_t argc = 3;
    napi_value argv[3];
    NAPI_OK(napi_get_cb_info(env, info, &argc, argv, nullptr, nullptr));
    b200bpe_ctx* ctx = argc >= 1 ? unwrap<b200bpe_ctx>(env, argv[0]) : nullptr;
    void* data = nullptr;
    size_t len = 0;
    if (!ctx || argc < 2 || napi_get_arraybuffer_info(env, argv[1], &data, &len) != napi_ok) { napi_throw_type_error(env, nullptr, "tokenizerCreate(ctx, trieData[, chunkSize])"); return nullptr; }
    uint32_t chunk = 0;
    if (argc >= 3) napi_get_value_uint32(env, argv[2], &chunk);
    b200bpe_tok* tok = nullptr;
    const b200bpe_status st = b200bpe_tokenizer_create(ctx, data, len, chunk, &tok);
    if (st != B200BPE_OK) { napi_throw(env, make_error(env, status_text(st))); return nullptr; }
    napi_value ext;
    NAPI_OK(napi_create_external(env, tok, nullptr, nullptr, &ext));
    return ext;
}

napi_value TokenizerInfo(napi_env env, napi_callback_info info) {
    size_t argc = 1;
    napi_value argv[1];
    NAPI_OK(napi_get_cb_info(env, info, &argc, argv, nullptr, nullptr));
    b200bpe_tok* tok = argc >= 1 ? unwrap<b200bpe_tok>(env, argv[0]) : nullptr;
    uint32_t f[4] = {0, 0, 0, 0};
    if (!tok || b200bpe_tokenizer_info(tok, &f[0], &f[1], &f[2], &f[3]) != B200BPE_OK) { napi_throw_error(env, nullptr, "bad tokenizer handle"); return nullptr; }
    static const char* names[4] = {"nodeCount", "edgeCount", "maxTokenLen", "chunkSize"};
    napi_value obj, v;
    NAPI_OK(napi_create_object(env, &obj));
    for (int i = 0; i < 4; i++) { napi_create_uint32(env, f[i], &v); napi_set_named_property(env, obj, names[i], v); }
    return obj;
}

napi_value TokenizerDestroy(napi_env env, napi_callback_info info) {
    size_t argc = 1;
    napi_value argv[1];
    NAPI_OK(napi_get_cb_info(env, info, &argc, argv, nullptr, nullptr));
    if (argc >= 1) b200bpe_tokenizer_destroy(unwrap<b200bpe_tok>(env, argv[0]));
    return nullptr;
}

struct EncodeJob {
    napi_async_work work = nullptr;
    napi_deferred deferred = nullptr;
    napi_ref keep = nullptr;
    b200bpe_tok* tok = nullptr;
    const uint8_t* bytes = nullptr;
    uint64_t n = 0, n_tokens = 0;
    std::vector<uint32_t> tokens;
    b200bpe_status status = B200BPE_OK;
    std::string error;
};

void encode_execute(napi_env, void* data) {
    EncodeJob* job = static_cast<EncodeJob*>(data);
    job->tokens.resize(job->n ? job->n : 1);   // one token per byte is the worst case
    job->status = b200bpe_encode(job->tok, job->bytes, job->n, job->tokens.data(), job->tokens.size(), &job->n_tokens);
    if (job->status != B200BPE_OK) job->error = status_text(job->status);
}

void encode_complete(napi_env env, napi_status, void* data) {
    EncodeJob* job = static_cast<EncodeJob*>(data);
    if (job->status != B200BPE_OK) {
        napi_reject_deferred(env, job->deferred, make_error(env, job->error));
    } else {
        void* dst = nullptr;
        napi_value ab, ta;
        napi_create_arraybuffer(env, (size_t)job->n_tokens * 4, &dst, &ab);
        std::memcpy(dst, job->tokens.data(), (size_t)job->n_tokens * 4);
        napi_create_typedarray(env, napi_uint32_array, (size_t)job->n_tokens, ab, 0, &ta);
        napi_resolve_deferred(env, job->deferred, ta);
    }
    if (job->keep) napi_delete_reference(env, job->keep);
    napi_delete_async_work(env, job->work);
    delete job;
}

// encode(tok, bytes: Uint8Array) → Promise<Uint32Array>
napi_value Encode(napi_env env, napi_callback_info info) {
    size_t argc = 2;
    napi_value argv[2];
    NAPI_OK(napi_get_cb_info(env, info, &argc, argv, nullptr, nullptr));
    EncodeJob* job = new EncodeJob();
    size_t nb = 0;
    job->tok = argc >= 1 ? unwrap<b200bpe_tok>(env, argv[0]) : nullptr;
    if (!job->tok || argc < 2 || !typed_bytes(env, argv[1], &job->bytes, &nb)) { delete job; napi_throw_type_error(env, nullptr, "encode(tokenizer, bytes: Uint8Array)"); return nullptr; }
    job->n = nb;
    napi_create_reference(env, argv[1], 1, &job->keep);
    napi_value promise, name;
    NAPI_OK(napi_create_promise(env, &job->deferred, &promise));
    napi_create_string_utf8(env, "b200bpe encode", NAPI_AUTO_LENGTH, &name);
    NAPI_OK(napi_create_async_work(env, nullptr, name, encode_execute, encode_complete, job, &job->work));
    NAPI_OK(napi_queue_async_work(env, job->work));
    return promise;
}

}  // namespace

NAPI_MODULE_INIT() {
    const napi_property_descriptor props[] = {
        {"ctxCreate", nullptr, CtxCreate, nullptr, nullptr, nullptr, napi_default, nullptr},
        {"ctxDestroy", nullptr, CtxDestroy, nullptr, nullptr, nullptr, napi_default, nullptr},
        {"train", nullptr, Train, nullptr, nullptr, nullptr, napi_default, nullptr},
        {"trieCompile", nullptr, TrieCompile, nullptr, nullptr, nullptr, napi_default, nullptr},
        {"trieParseHeader", nullptr, TrieParseHeader, nullptr, nullptr, nullptr, napi_default, nullptr},
        {"tokenizerCreate", nullptr, TokenizerCreate, nullptr, nullptr, nullptr, napi_default, nullptr},
        {"tokenizerInfo", nullptr, TokenizerInfo, nullptr, nullptr, nullptr, napi_default, nullptr},
        {"tokenizerDestroy", nullptr, TokenizerDestroy, nullptr, nullptr, nullptr, napi_default, nullptr},
        {"encode", nullptr, Encode, nullptr, nullptr, nullptr, napi_default, nullptr},
    };
    napi_define_properties(env, exports, sizeof(props) / sizeof(props[0]), props);
    return exports;
}
