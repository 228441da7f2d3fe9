/*
 * b200bpe.h — C ABI of libb200bpe.so: BPE training and trie encoding on NVIDIA B200 (sm_100a).
 *
 * This is the drop-in boundary for the two device paths of toprakdeviren/gpu-bpe.  The reference
 * has no FFI (it is browser JavaScript driving WebGPU), so each entry point cites the JavaScript
 * interface it stands behind; paths are relative to the reference project.
 *
 * Conventions: every function returns a b200bpe_status (0 = OK); no exception crosses the
 * boundary; handles are opaque; every buffer is owned by the caller; a handle is not thread-safe,
 * different handles are.  One context drives one GPU; multi-GPU jobs run one process (or thread)
 * per GPU and join their contexts with b200bpe_ctx_create_dist.
 *
 * All integers are little-endian unsigned; no floating point is computed on the path.
 */
#ifndef B200BPE_H
#define B200BPE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t b200bpe_status;

enum {
    B200BPE_OK = 0,
    B200BPE_ERR_BAD_ARG = 1,
    B200BPE_ERR_CUDA = 2,             /* a CUDA runtime call failed; see b200bpe_last_error() */
    B200BPE_ERR_NO_DEVICE = 3,        /* no usable sm_100 GPU: there is no CPU fallback */
    B200BPE_ERR_EMPTY_CORPUS = 4,     /* trainer.js:161-163 "No symbols to train on" */
    B200BPE_ERR_TABLE_FULL = 5,       /* pair table could not grow any further */
    B200BPE_ERR_LOOKBACK_TIMEOUT = 6, /* a bounded device-side wait ran out */
    B200BPE_ERR_BAD_TRIE_MAGIC = 7,   /* trie.js:115-117 */
    B200BPE_ERR_BAD_TRIE_VERSION = 8, /* trie.js:118-120 */
    B200BPE_ERR_TRUNCATED_TRIE = 9,   /* trie.js:145-147 */
    B200BPE_ERR_CAPACITY = 10,        /* caller's output buffer is too small */
    B200BPE_ERR_NCCL = 11,
    B200BPE_ERR_OOM = 12,
    B200BPE_ERR_INTERNAL = 13
};

/* compat_mode: which reference behaviour the compaction step reproduces. */
enum {
    B200BPE_COMPAT_LITERAL = 0, /* as shipped: compaction input bounded by the post-merge count
                                   (train.wgsl:698,727 after :604-606/:650-651) */
    B200BPE_COMPAT_FIXED = 1    /* compaction covers every pre-merge position */
};

enum {
    B200BPE_FLAG_NO_GRAPH = 1u,      /* launch kernels one by one instead of one CUDA graph per batch */
    B200BPE_FLAG_TIME_KERNELS = 2u,  /* bracket every kernel with CUDA events (implies NO_GRAPH) */
    B200BPE_FLAG_FULL_RECOUNT = 4u,  /* rebuild the pair table with a full count before every merge, as the
                                        reference does (train.wgsl:196-202,376-431), instead of updating it in
                                        place around the merged occurrences; the merge list is the same */
    B200BPE_FLAG_NCCL_EXCHANGE = 8u  /* sharded runs: exchange the pair counts with NCCL send/recv and all-reduce
                                        instead of this library's own kernels over NVLink peer memory (the default,
                                        which needs one process per GPU and CUDA IPC between them; the library falls
                                        back to NCCL by itself when the peers' buffers cannot be mapped) */
};

typedef struct b200bpe_ctx b200bpe_ctx;
typedef struct b200bpe_trainer b200bpe_trainer;
typedef struct b200bpe_tok b200bpe_tok;

/* Options of one training run.  Zero-initialise, set struct_size, then override. */
typedef struct {
    uint32_t struct_size;       /* sizeof(b200bpe_train_opts) */
    uint32_t target_vocab_size; /* trainer.js:149 targetVocabSize (default 4096); merges = target - first_token_id */
    uint32_t first_token_id;    /* vocab.js:98 / trainer.js:191 (default 256) */
    uint32_t batch_merges;      /* training-pipeline.js:13 BATCH_SIZE (default 128): merges per host round trip */
    uint32_t compat_mode;       /* B200BPE_COMPAT_* (default LITERAL on one GPU; FIXED is required when sharded) */
    uint32_t table_log2;        /* log2 of the pair-table capacity in slots; 0 = sized from the corpus, grows on demand */
    uint32_t flags;             /* B200BPE_FLAG_* */
    uint32_t exchange_cap;      /* tests only: first bucket size of the NCCL exchange in slots (0 = default), to reach
                                   the bucket-overflow path with a small corpus */
    /* tests only: prove that a device-side wait that can never be satisfied ends by itself.  test_lookback_spins
       (0 = default, about four million) is the number of polls after which a look-back gives up;
       test_first_tile = 1 makes the merge kernel skip tile 0, so that nobody ever publishes the count every
       other tile waits for: the run then ends with B200BPE_ERR_LOOKBACK_TIMEOUT instead of a merge list. */
    uint32_t test_lookback_spins;
    uint32_t test_first_tile;
} b200bpe_train_opts;

/* Progress payload, one call per batch: the fields of trainer.js:306-314. */
typedef struct {
    uint32_t merge_index;   /* merges completed so far */
    uint32_t total_merges;  /* merges requested */
    uint32_t last_a, last_b, last_new_id, last_count; /* last merge of the batch (count 0 = none) */
    uint64_t symbol_count;  /* live symbols after the batch (this rank) */
    double merges_per_second;
} b200bpe_progress;
typedef void (*b200bpe_progress_cb)(const b200bpe_progress*, void* user);

/* Accumulated device time and algorithmic bytes per kernel class (B200BPE_FLAG_TIME_KERNELS). */
typedef struct {
    double pair_count_ms, argmax_ms, merge_compact_ms, exchange_ms;
    uint64_t pair_count_launches, argmax_launches, merge_compact_launches, exchange_launches;
    uint64_t pair_count_bytes;    /* 4 * N_k summed over the merges that counted */
    uint64_t argmax_bytes;        /* 2 * 12 * table slots per merge (scan + clear) */
    uint64_t merge_compact_bytes; /* 4 * N_k + 4 * N_{k+1} summed over merges */
    /* launches of the count kernel that had nothing to do because the table was up to date */
    double pair_count_skipped_ms;
    uint64_t pair_count_skipped_launches;
    /* the small kernels that fold the queued pair deltas (and the literal-mode tail) into the table */
    double table_update_ms;
} b200bpe_kernel_stats;

const char* b200bpe_status_str(b200bpe_status);
/* Text of the last CUDA/NCCL failure on the calling thread ("" if none). */
const char* b200bpe_last_error(void);
/* Number of visible CUDA devices (0 when there is no driver or GPU). */
int32_t b200bpe_device_count(void);

/* ── context: replaces BPEEngine.init() (src/bpe/engine.js:216-238: adapter, device, pipelines) ── */
b200bpe_status b200bpe_ctx_create(int32_t device, b200bpe_ctx** out);
/* Join `world` contexts (one per GPU) into one sharded job.  nccl_lib is the path of the NCCL
 * shared library to use; unique_id is the 128-byte id made by b200bpe_nccl_unique_id on rank 0
 * and passed to the others by the caller.  No counterpart in the single-device reference. */
b200bpe_status b200bpe_nccl_unique_id(const char* nccl_lib, uint8_t unique_id[128]);
b200bpe_status b200bpe_ctx_create_dist(int32_t device, int32_t rank, int32_t world, const char* nccl_lib,
                                       const uint8_t unique_id[128], b200bpe_ctx** out);
void b200bpe_ctx_destroy(b200bpe_ctx*);
/* Device facts: sm_count, compute capability major*10+minor, total and free memory in bytes. */
b200bpe_status b200bpe_ctx_info(b200bpe_ctx*, int32_t* sm_count, int32_t* cc, uint64_t* total_mem, uint64_t* free_mem);
b200bpe_status b200bpe_ctx_synchronize(b200bpe_ctx*);

/* ── training: replaces BPETrainer.train (src/bpe/trainer.js:149-220, loop :225-335) ──
 * bytes[n] is the (normalised) corpus; word_starts[n] is the pre-tokeniser's mask
 * (pre_tokenizer.mjs:459-509), or NULL to tag boundaries on the device with the byte-class
 * heuristic of bpe_word_boundary (train.wgsl:144-186), as trainer.js:177-180 does.
 * merges_out gets 3 words per merge {a, b, new_id} (trainer.js:270-276), counts_out (may be NULL)
 * the winning pair's count (merge-log word 2, train.wgsl:356-360).  Both need room for
 * target_vocab_size - first_token_id merges.  *early_stop_out mirrors IterState.early_stop. */
b200bpe_status b200bpe_train(b200bpe_ctx*, const uint8_t* bytes, const uint8_t* word_starts, uint64_t n,
                             const b200bpe_train_opts*, uint32_t* merges_out, uint32_t* counts_out,
                             uint32_t* n_merges_out, uint32_t* early_stop_out, b200bpe_progress_cb, void* user);

/* The same run, split into steps so that a caller can keep the corpus resident on the device,
 * repeat runs, and inspect intermediate state.  create uploads and tags the symbols
 * (trainer.js:62-80,115-121,173-175); create_from_symbols takes already tagged u32 symbols
 * (bit 16 = word start, train.wgsl:36-37); *_device variants take device pointers. */
b200bpe_status b200bpe_trainer_create(b200bpe_ctx*, const uint8_t* bytes, const uint8_t* word_starts, uint64_t n,
                                      const b200bpe_train_opts*, b200bpe_trainer** out);
b200bpe_status b200bpe_trainer_create_device(b200bpe_ctx*, const uint8_t* d_bytes, const uint8_t* d_word_starts,
                                             uint64_t n, const b200bpe_train_opts*, b200bpe_trainer** out);
b200bpe_status b200bpe_trainer_create_from_symbols(b200bpe_ctx*, const uint32_t* symbols, uint64_t n,
                                                   const b200bpe_train_opts*, b200bpe_trainer** out);
/* Run up to max_merges more merges (0 = all that remain of the target). */
b200bpe_status b200bpe_trainer_run(b200bpe_trainer*, uint32_t max_merges, uint32_t* merges_out, uint32_t* counts_out,
                                   uint32_t* n_merges_out, uint32_t* early_stop_out, b200bpe_progress_cb, void* user);
/* Put the device state back to the freshly created one (symbols re-tagged from the resident bytes). */
b200bpe_status b200bpe_trainer_reset(b200bpe_trainer*);
/* Live symbols of this rank (device → host), for tests. */
b200bpe_status b200bpe_trainer_symbols(b200bpe_trainer*, uint32_t* out, uint64_t cap, uint64_t* n_out);
/* Run the pair-count kernel on the live symbols and return the table as (a<<32|b, count) entries,
 * unsorted (global counts when sharded); the table is left empty.  For tests. */
b200bpe_status b200bpe_trainer_pair_counts(b200bpe_trainer*, uint64_t* keys_out, uint32_t* counts_out, uint64_t cap,
                                           uint64_t* n_distinct_out);
b200bpe_status b200bpe_trainer_kernel_stats(b200bpe_trainer*, b200bpe_kernel_stats* out);
/* Kernels this trainer has launched since it was created (a graph launch counts the kernels it holds);
 * and which count exchange a sharded trainer uses: 0 none (one GPU), 1 peer memory, 2 NCCL.  Diagnostics;
 * no counterpart in the reference. */
b200bpe_status b200bpe_trainer_launches(b200bpe_trainer*, uint64_t* n_out);
b200bpe_status b200bpe_trainer_exchange_kind(b200bpe_trainer*, uint32_t* kind_out);
/* Milliseconds of device time of the last b200bpe_trainer_run, by CUDA events on the library's stream. */
b200bpe_status b200bpe_trainer_last_run_ms(b200bpe_trainer*, double* ms);
/* Milliseconds of device time of the last b200bpe_trainer_reset (symbol tagging and buffer clears). */
b200bpe_status b200bpe_trainer_last_reset_ms(b200bpe_trainer*, double* ms);
void b200bpe_trainer_destroy(b200bpe_trainer*);

/* ── trie: replaces compileVocabToTrie / parseHeader / parseTrieBuffers (src/bpe/tokenizer/trie.js:39,110,137) ──
 * vocab entry i is vocab_bytes[vocab_offsets[i] .. vocab_offsets[i+1]) (vocab_offsets has vocab_size+1
 * entries).  Call with out == NULL to get the needed size in *out_len.  The output is the reference's
 * v3 binary (28-byte header, 12-byte nodes, 8-byte edges), byte for byte. */
b200bpe_status b200bpe_trie_compile(const uint8_t* vocab_bytes, const uint64_t* vocab_offsets, uint32_t vocab_size,
                                    void* out, size_t* out_len);
/* header fields {version, nodeCount, edgeCount, maxTokenLen, vocabSize}; validates magic, version and length. */
b200bpe_status b200bpe_trie_parse_header(const void* trie, size_t len, uint32_t fields_out[5]);

/* ── encoding: replaces TrieTokenizer (src/bpe/tokenizer/tokenizer.js:54-98,173-335) ──
 * chunk_size 0 selects the reference rule max(512, min(2048, maxTokenLen*8)) (tokenizer.js:67-68). */
b200bpe_status b200bpe_tokenizer_create(b200bpe_ctx*, const void* trie_v3, size_t len, uint32_t chunk_size,
                                        b200bpe_tok** out);
/* The same with every option spelled out (zero-initialise, set struct_size; 0 = default everywhere).
 * layout picks how the trie lies on the device; the slice sizes are the points at which
 * b200bpe_encode_batch (default 32 MiB of documents) and b200bpe_encode (default 8 GiB, the analogue
 * of the buffer limit of tokenizer.js:181-203) cut their input.  Results never depend on any of them;
 * tests use them to reach every code path with small inputs. */
enum { B200BPE_TRIE_AUTO = 0, B200BPE_TRIE_CUCKOO = 1, B200BPE_TRIE_HYBRID = 2, B200BPE_TRIE_HASH = 3 };
typedef struct {
    uint32_t struct_size;        /* sizeof(b200bpe_tok_opts) */
    uint32_t chunk_size;         /* tokenizer.js:67-68 options.chunkSize; 0 = the reference rule */
    uint32_t layout;             /* B200BPE_TRIE_*; a layout the trie does not fit falls through to the next one */
    uint32_t test_lookback_spins; /* tests only: polls after which the look-back of the compaction gives up (0 = default);
                                    a value below 2^20 also makes the compaction skip tile 0, which no other tile
                                    can then get past: the call ends with B200BPE_ERR_LOOKBACK_TIMEOUT */
    uint64_t batch_slice_bytes;  /* 0 = default; at least 1024 */
    uint64_t encode_slice_bytes; /* 0 = default; at least 1024 (rounded down to whole chunks) */
} b200bpe_tok_opts;
b200bpe_status b200bpe_tokenizer_create_ex(b200bpe_ctx*, const void* trie_v3, size_t len, const b200bpe_tok_opts*,
                                           b200bpe_tok** out);
b200bpe_status b200bpe_tokenizer_info(b200bpe_tok*, uint32_t* node_count, uint32_t* edge_count,
                                      uint32_t* max_token_len, uint32_t* chunk_size);
/* How the trie lies on the device (no reference counterpart; for diagnostics and tests):
 * sub_tables 2 or 3 = cuckoo table held in shared memory, with 1 << log2_slots entries each;
 * sub_tables 1 = hybrid: the most used transitions (1 << log2_slots entries, two-byte first step) in shared
 *                memory, the rest in a global table;
 * sub_tables 0 = open-addressing table in global memory with 1 << log2_slots entries. */
b200bpe_status b200bpe_tokenizer_layout(b200bpe_tok*, uint32_t* sub_tables, uint32_t* log2_slots);
/* encodeBytes (tokenizer.js:173-206): host bytes in, host token ids out.  cap is the room in
 * tokens_out (n is always enough).  The result depends only on (bytes, trie, chunk_size). */
b200bpe_status b200bpe_encode(b200bpe_tok*, const uint8_t* bytes, uint64_t n, uint32_t* tokens_out, uint64_t cap,
                              uint64_t* n_tokens_out);
/* Many documents in one call, each encoded exactly as a separate encodeBytes call would
 * (export-controller.js:190-211 encodes one buffer; per-document calls are the sharding unit).
 * doc_offsets has n_docs+1 entries into bytes; tok_offsets_out gets n_docs+1 entries into tokens_out. */
b200bpe_status b200bpe_encode_batch(b200bpe_tok*, const uint8_t* bytes, const uint64_t* doc_offsets, uint32_t n_docs,
                                    uint32_t* tokens_out, uint64_t cap, uint64_t* tok_offsets_out);
/* Device-resident variants: d_bytes / d_doc_offsets / d_tokens_out / d_tok_offsets_out are device
 * pointers on the context's GPU; only the token total crosses to the host. */
b200bpe_status b200bpe_encode_device(b200bpe_tok*, const uint8_t* d_bytes, uint64_t n, uint32_t* d_tokens_out,
                                     uint64_t cap, uint64_t* n_tokens_out);
b200bpe_status b200bpe_encode_batch_device(b200bpe_tok*, const uint8_t* d_bytes, const uint64_t* d_doc_offsets,
                                           uint32_t n_docs, uint64_t n_bytes, uint32_t* d_tokens_out, uint64_t cap,
                                           uint64_t* d_tok_offsets_out, uint64_t* n_tokens_out);
/* b200bpe_encode_device for callers that must not allocate (no counterpart in the reference).
 * The same kernels and the same result, but the work buffers are a fixed array built into the
 * library image instead of the tokenizer's growable pool, and the call makes no cudaMalloc,
 * cudaFree or other allocating call: for encode steps inside a latency-critical or
 * memory-exhausted process, where the allocator's locks, its implicit synchronisation or its
 * failure are not acceptable.  Limits: n <= 1 MiB and at most 8,192 chunks per call; larger
 * inputs return B200BPE_ERR_CAPACITY (b200bpe_last_error() says why).  The array's device address
 * is looked up and the kernels are loaded when the tokenizer is created, not here.  With the
 * global-table trie layout this entry point does not set the persisting L2 window that the pooled
 * path asks for.  All calls on a device share the array: calls that overlap on the GPU race; one
 * at a time per device. */
b200bpe_status b200bpe_encode_device_noalloc(b200bpe_tok*, const uint8_t* d_bytes, uint64_t n, uint32_t* d_tokens_out,
                                             uint64_t cap, uint64_t* n_tokens_out);
/* Milliseconds of device time of the last encode call, split by kernel: walk, scan+compaction. */
b200bpe_status b200bpe_tokenizer_last_ms(b200bpe_tok*, double* walk_ms, double* compact_ms);
void b200bpe_tokenizer_destroy(b200bpe_tok*);

/* ── merge-replay encoding: replaces TokenizerManager.encode (src/ui/tokenizer-manager.js:13-61) ──
 * The reference's other encoder: one token per byte, then every merge rule {a, b, new_id} applied in the order
 * it was learned, each as one left-to-right pass over the whole token list (no word boundaries, no chunks; with
 * a == b a run pairs up from the left).  merges: 3 words per rule.  The list must be one a trainer could have
 * produced: every rule makes an id of its own (not a byte value) and uses only ids that earlier rules made;
 * other lists are refused with B200BPE_ERR_BAD_ARG.  No merges: the bytes are the tokens (:21-25). */
typedef struct b200bpe_replay b200bpe_replay;
b200bpe_status b200bpe_replay_create(b200bpe_ctx*, const uint32_t* merges, uint32_t n_merges, b200bpe_replay** out);
b200bpe_status b200bpe_replay_encode(b200bpe_replay*, const uint8_t* bytes, uint64_t n, uint32_t* tokens_out, uint64_t cap,
                                     uint64_t* n_tokens_out);
b200bpe_status b200bpe_replay_encode_device(b200bpe_replay*, const uint8_t* d_bytes, uint64_t n, uint32_t* d_tokens_out,
                                            uint64_t cap, uint64_t* n_tokens_out);
/* Rounds (rules that found their pair) of the last call; diagnostics. */
b200bpe_status b200bpe_replay_last_rounds(b200bpe_replay*, uint32_t* rounds_out);
void b200bpe_replay_destroy(b200bpe_replay*);

/* ── pre-tokeniser: replaces PreTokenizer.preTokenizeBytes (src/wasm/pre_tokenizer.mjs:459-509) ──
 * Host code.  GPT-4-style word starts over code-point classes; the input must already be NFC
 * (the reference normalises with a closed-source WASM library first, pre_tokenizer.mjs:465).
 * word_starts_out[n] gets 1 at the first byte of each word. */
b200bpe_status b200bpe_pretokenize(const uint8_t* bytes, uint64_t n, uint8_t* word_starts_out);
/* The same rules on the GPU, for well-formed UTF-8 (the last character may be cut short); other input is
 * refused with B200BPE_ERR_BAD_ARG and the host function above takes it.  _device: device pointers, _gpu: host
 * buffers (upload, kernel, read-back).  One kernel, one pass; the three-digit split of digit runs is carried
 * across tiles by a decoupled look-back scan. */
b200bpe_status b200bpe_pretokenize_device(b200bpe_ctx*, const uint8_t* d_bytes, uint64_t n, uint8_t* d_word_starts_out);
b200bpe_status b200bpe_pretokenize_gpu(b200bpe_ctx*, const uint8_t* bytes, uint64_t n, uint8_t* word_starts_out);
/* Tests only (no counterpart in the reference): the device function with the number of polls after which its
 * look-back gives up (0 = default).  A value below 2^20 also makes the kernel skip tile 0, whose digit count no
 * other tile can then obtain: the call ends with B200BPE_ERR_LOOKBACK_TIMEOUT, which proves that the wait is bounded. */
b200bpe_status b200bpe_pretokenize_device_ex(b200bpe_ctx*, const uint8_t* d_bytes, uint64_t n, uint8_t* d_word_starts_out,
                                             uint32_t test_lookback_spins);

/* ── token file export: replaces the ".bin" writer of the Export tab (src/ui/export-controller.js:4,235-248) ──
 * Host code.  Layout: u32 LE {0x44584654 'DXFT', vocabSize, tokenCount, vocabJsonBytes}, the tokens as u32 LE,
 * then the vocabulary JSON {version, vocabSize, vocab, merges} (JSON.stringify form; may be empty). */
b200bpe_status b200bpe_dxft_size(uint64_t n_tokens, uint64_t json_len, uint64_t* size_out);
b200bpe_status b200bpe_dxft_write(const uint32_t* tokens, uint64_t n_tokens, uint32_t vocab_size, const void* json,
                                  uint64_t json_len, void* out, uint64_t cap);
/* fields_out = {magic, vocabSize, tokenCount, vocabJsonBytes}; B200BPE_ERR_BAD_TRIE_MAGIC / _TRUNCATED_TRIE on a bad file. */
b200bpe_status b200bpe_dxft_parse(const void* buf, uint64_t len, uint32_t fields_out[4], uint64_t* tokens_offset,
                                  uint64_t* json_offset);

#ifdef __cplusplus
}
#endif
#endif /* B200BPE_H */
