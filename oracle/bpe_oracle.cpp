// CPU oracle for the BPE train / trie-encode hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file is a checker, never a product path: only tests/, the smoke check and
// the CPU-baseline leg of bench.py may load it.  It restates, on the CPU, what the
// reference's WGSL kernels and host loops compute (citations are paths inside the
// toprakdeviren/gpu-bpe project):
//
//   * training merge loop      src/bpe/train.wgsl:39-41,83-85,340-364,376-431,457-520,
//                              548-662,686-731 in the dispatch order of
//                              src/bpe/training-pipeline.js:178-222 and the host loop of
//                              src/bpe/trainer.js:187-196,235-288
//   * byte-class word heuristic src/bpe/train.wgsl:111-186
//   * chunked trie encode      src/bpe/tokenizer/tokenize.wgsl:69-175 with the host rules
//                              of src/bpe/tokenizer/tokenizer.js:67-68,181-183,218-219
//
// PARITY UNPINNED: the reference ships no tests, fixtures or golden vectors and cannot be
// executed where this oracle is built (it is browser JavaScript + WGSL).  The pins are the
// hand-derived known answers in tests/golden/ and a second, dispatch-level Python model of
// the same shaders (oracle/wgsl_model.py) that this file is cross-checked against.
//
// Defined choices where the reference's behaviour depends on GPU scheduling:
//   * the merge kernel reads a snapshot of the pre-merge buffer (train.wgsl:475-497 races
//     between one thread's in-place write and its neighbours' reads);
//   * pairs are counted exactly (the reference silently drops a pair whose 64 local or 128
//     global probes all collide, train.wgsl:401-408,422-429).
//
// Two compaction modes:
//   mode 0 "literal": as shipped.  The scan kernel publishes the post-merge symbol count
//       (train.wgsl:604-606,650-651) before the compaction kernel runs, and that kernel
//       bounds its INPUT index by it (train.wgsl:698,727): the last `count` input symbols
//       are never copied and the tail of the destination buffer keeps older contents.
//   mode 1 "fixed": compaction covers every pre-merge position (the algorithm the
//       reference's comments describe).
//
// Build: see oracle/build_oracle.py (g++ -O3 -march=native -shared -fPIC -pthread).

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

namespace {

constexpr uint32_t WORD_START_BIT = 0x10000u;  // train.wgsl:36
constexpr uint32_t TOKEN_MASK = 0xFFFFu;       // train.wgsl:37
constexpr uint32_t INVALID_TOKEN = 0xFFFFFFFFu;

inline uint32_t pack_pair(uint32_t a, uint32_t b) { return (a << 16) | b; }  // train.wgsl:39

// train.wgsl:83-85 — larger count wins, ties go to the smaller packed pair id.
inline bool is_better(uint32_t cn, uint32_t pn, uint32_t co, uint32_t po) {
    return cn > co || (cn == co && pn < po);
}

inline uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}

// Exact open-addressing counter keyed by the packed pair (never 0: a == 0 is not counted).
struct CountTable {
    std::vector<uint32_t> keys, vals;
    uint32_t mask = 0, used = 0;
    explicit CountTable(uint32_t cap_pow2 = 1u << 12) { reset(cap_pow2); }
    void reset(uint32_t cap) {
        keys.assign(cap, 0u); vals.assign(cap, 0u); mask = cap - 1; used = 0;
    }
    void clear() { std::fill(keys.begin(), keys.end(), 0u); std::fill(vals.begin(), vals.end(), 0u); used = 0; }
    void grow() {
        std::vector<uint32_t> ok, ov; ok.swap(keys); ov.swap(vals);
        reset((uint32_t)ok.size() * 2);
        for (size_t i = 0; i < ok.size(); i++) if (ok[i]) add(ok[i], ov[i]);
    }
    void add(uint32_t key, uint32_t n) {
        if ((uint64_t)used * 2 >= keys.size()) grow();
        uint32_t i = mix32(key) & mask;
        for (;;) {
            if (keys[i] == key) { vals[i] += n; return; }
            if (keys[i] == 0) { keys[i] = key; vals[i] = n; used++; return; }
            i = (i + 1) & mask;
        }
    }
};

void parallel_for(int threads, uint64_t n, const std::function<void(int, uint64_t, uint64_t)>& fn) {
    if (threads <= 1 || n < 4096) { fn(0, 0, n); return; }
    std::vector<std::thread> pool;
    uint64_t per = (n + threads - 1) / threads;
    for (int t = 0; t < threads; t++) {
        uint64_t lo = std::min<uint64_t>(n, per * t), hi = std::min<uint64_t>(n, lo + per);
        pool.emplace_back(fn, t, lo, hi);
    }
    for (auto& th : pool) th.join();
}

// train.wgsl:392-411 — one candidate pair per position id with id+1 < n.
inline bool pair_at(const uint32_t* s, uint64_t id, uint64_t n, uint32_t* key) {
    if (id + 1 >= n) return false;
    uint32_t rb = s[id + 1];
    if (rb & WORD_START_BIT) return false;
    uint32_t a = s[id] & TOKEN_MASK, b = rb & TOKEN_MASK;
    if (a == 0 || b == 0) return false;
    *key = pack_pair(a, b);
    return true;
}

struct Best { uint32_t count = 0, pair = 0; };

// Count every pair of s[0..n) and return the arg-max under is_better.
// Threads count disjoint ranges into private tables, then each thread owns the keys whose
// hash falls in its partition, sums them over all private tables and reports its own best.
Best count_and_argmax(const uint32_t* s, uint64_t n, int threads, std::vector<CountTable>& local) {
    int T = (threads <= 1 || n < 4096) ? 1 : threads;
    if ((int)local.size() < T) local.resize(T);
    parallel_for(T, n, [&](int t, uint64_t lo, uint64_t hi) {
        CountTable& tb = local[t];
        tb.clear();
        uint32_t key;
        for (uint64_t id = lo; id < hi; id++) if (pair_at(s, id, n, &key)) tb.add(key, 1);
    });
    Best best;
    if (T == 1) {
        const CountTable& tb = local[0];
        for (size_t i = 0; i < tb.keys.size(); i++)
            if (tb.keys[i] && is_better(tb.vals[i], tb.keys[i], best.count, best.pair)) {
                best.count = tb.vals[i]; best.pair = tb.keys[i];
            }
        return best;
    }
    std::vector<Best> part(T);
    std::vector<std::thread> pool;
    for (int o = 0; o < T; o++) {
        pool.emplace_back([&, o]() {
            CountTable own(1u << 12);
            for (int t = 0; t < T; t++) {
                const CountTable& tb = local[t];
                for (size_t i = 0; i < tb.keys.size(); i++) {
                    uint32_t k = tb.keys[i];
                    if (k && (int)((mix32(k) >> 20) % (uint32_t)T) == o) own.add(k, tb.vals[i]);
                }
            }
            Best b;
            for (size_t i = 0; i < own.keys.size(); i++)
                if (own.keys[i] && is_better(own.vals[i], own.keys[i], b.count, b.pair)) {
                    b.count = own.vals[i]; b.pair = own.keys[i];
                }
            part[o] = b;
        });
    }
    for (auto& th : pool) th.join();
    for (auto& b : part) if (is_better(b.count, b.pair, best.count, best.pair)) best = b;
    return best;
}

// train.wgsl:482-485 (A side) and :492-495 (B side), both on the pre-merge snapshot.
inline bool a_side(const uint32_t* s, uint64_t id, uint64_t n, uint32_t a, uint32_t b) {
    return id + 1 < n && !(s[id + 1] & WORD_START_BIT) && (s[id] & TOKEN_MASK) == a &&
           (s[id + 1] & TOKEN_MASK) == b;
}
inline bool is_valid(const uint32_t* s, uint64_t id, uint32_t a, uint32_t b) {
    return !(id > 0 && !(s[id] & WORD_START_BIT) && (s[id - 1] & TOKEN_MASK) == a &&
             (s[id] & TOKEN_MASK) == b);
}

}  // namespace

extern "C" {

// Byte-class heuristic used when the caller supplies no word mask (train.wgsl:111-186).
// sym holds raw byte values on entry; bit 16 is set on word starts on return.
void oracle_word_boundary(uint32_t* sym, uint64_t n) {
    auto cls = [](uint32_t t) -> uint32_t {
        if (t == 0x0A) return 4; if (t == 0x20) return 2; if (t - 0x30u <= 9u) return 1;
        if (t >= 0x80) return 0; if (t - 0x61u <= 25u) return 0; if (t - 0x41u <= 25u) return 0;
        return 3;
    };
    std::vector<uint8_t> flag(n, 0);
    for (uint64_t id = 0; id < n; id++) {
        uint32_t tok = sym[id] & TOKEN_MASK;
        if (id == 0) { flag[id] = 1; continue; }
        uint32_t c = cls(tok), p = cls(sym[id - 1] & TOKEN_MASK);
        bool bd = c != p;
        if (p == 2 && (c == 0 || c == 1)) bd = false;
        if (c == 2 && p != 2) bd = true;
        if (p == 4 || c == 4) bd = true;
        flag[id] = bd;
    }
    for (uint64_t id = 0; id < n; id++) sym[id] = (sym[id] & TOKEN_MASK) | (flag[id] ? WORD_START_BIT : 0);
}

// Exact pair histogram of sym[0..n): writes up to cap (key, count) entries sorted by key,
// returns the number of distinct pairs (which may exceed cap).
uint64_t oracle_pair_counts_mt(const uint32_t* sym, uint64_t n, uint32_t* keys_out, uint32_t* counts_out,
                               uint64_t cap, int threads);

uint64_t oracle_pair_counts(const uint32_t* sym, uint64_t n, uint32_t* keys_out, uint32_t* counts_out,
                            uint64_t cap) {
    return oracle_pair_counts_mt(sym, n, keys_out, counts_out, cap, 1);
}

// The same histogram with the positions split over `threads` threads (private tables, then summed).
uint64_t oracle_pair_counts_mt(const uint32_t* sym, uint64_t n, uint32_t* keys_out, uint32_t* counts_out,
                               uint64_t cap, int threads) {
    const int T = (threads <= 1 || n < 4096) ? 1 : threads;
    std::vector<CountTable> part(T, CountTable(1u << 16));
    parallel_for(T, n, [&](int t, uint64_t lo, uint64_t hi) {
        uint32_t key;
        for (uint64_t id = lo; id < hi; id++) if (pair_at(sym, id, n, &key)) part[t].add(key, 1);
    });
    CountTable& tb = part[0];
    for (int t = 1; t < T; t++)
        for (size_t i = 0; i < part[t].keys.size(); i++) if (part[t].keys[i]) tb.add(part[t].keys[i], part[t].vals[i]);
    std::vector<std::pair<uint32_t, uint32_t>> v;
    for (size_t i = 0; i < tb.keys.size(); i++) if (tb.keys[i]) v.push_back({tb.keys[i], tb.vals[i]});
    std::sort(v.begin(), v.end());
    for (size_t i = 0; i < v.size() && i < cap; i++) { keys_out[i] = v[i].first; counts_out[i] = v[i].second; }
    return v.size();
}

// The training merge loop.  sym_in holds `n` tagged symbols (bit 16 = word start).
// merges_out receives 4 words per merge: a, b, new_id, count.  final_sym (capacity n, may be
// NULL) receives the live symbol range after the last merge.  Returns 0.
// max_seconds > 0 stops after that much wall time (used only for bounded CPU-baseline samples;
// *n_merges_out then says how many merges were completed).
int oracle_train(const uint32_t* sym_in, uint64_t n, uint32_t max_merges, int mode, uint32_t first_id,
                 int threads, double max_seconds, uint32_t* merges_out, uint32_t* n_merges_out,
                 uint32_t* early_stop_out, uint32_t* final_sym, uint64_t* final_n, double* seconds_out) {
    std::vector<uint32_t> bufA(sym_in, sym_in + n), bufB(n, 0u);  // pong starts zeroed (WebGPU zero-init)
    uint32_t* ping = bufA.data();
    uint32_t* pong = bufB.data();
    uint64_t N = n;
    uint32_t next_id = first_id, done = 0, early = 0;
    int T = std::max(1, threads);
    std::vector<CountTable> local;
    auto t0 = std::chrono::steady_clock::now();

    while (done < max_merges) {
        // clear + count + two-pass arg-max (train.wgsl:196-202,376-431,228-318)
        Best best = count_and_argmax(ping, N, T, local);
        // setup (train.wgsl:340-364)
        if (best.count < 2 || next_id > TOKEN_MASK) { early = 1; break; }
        const uint32_t a = best.pair >> 16, b = best.pair & 0xFFFFu, nw = next_id;
        merges_out[done * 4 + 0] = a; merges_out[done * 4 + 1] = b;
        merges_out[done * 4 + 2] = nw; merges_out[done * 4 + 3] = best.count;
        next_id++; done++;

        // merge_reduce (train.wgsl:457-520): validity of every pre-merge position, block sums.
        int TT = (T <= 1 || N < 4096) ? 1 : T;
        std::vector<uint64_t> valid_all(TT, 0);
        parallel_for(TT, N, [&](int t, uint64_t lo, uint64_t hi) {
            uint64_t v = 0;
            for (uint64_t id = lo; id < hi; id++) v += is_valid(ping, id, a, b);
            valid_all[t] = v;
        });
        // scan_blocks (train.wgsl:636-662): the new symbol count is the total of the valid bits.
        uint64_t Nnew = 0;
        for (auto v : valid_all) Nnew += v;
        // finalize_compact (train.wgsl:686-731): stable scatter, input bounded by `limit`.
        const uint64_t limit = (mode == 0) ? Nnew : N;
        std::vector<uint64_t> cnt(TT, 0), off(TT, 0);
        std::vector<std::vector<uint64_t>> hits(TT);
        uint64_t per = (TT == 1) ? N : (N + TT - 1) / TT;
        parallel_for(TT, N, [&](int t, uint64_t lo, uint64_t hi) {
            uint64_t v = 0;
            for (uint64_t id = lo; id < hi && id < limit; id++) v += is_valid(ping, id, a, b);
            cnt[t] = v;
        });
        for (int t = 1; t < TT; t++) off[t] = off[t - 1] + cnt[t - 1];
        parallel_for(TT, N, [&](int t, uint64_t lo, uint64_t hi) {
            uint64_t d = off[t];
            for (uint64_t id = lo; id < hi; id++) {
                bool m = a_side(ping, id, N, a, b);
                if (m) hits[t].push_back(id);
                if (id < limit && is_valid(ping, id, a, b))
                    pong[d++] = m ? (nw | (ping[id] & WORD_START_BIT)) : ping[id];
            }
        });
        (void)per;
        // The A side rewrites the source buffer in place (train.wgsl:486-487); it becomes the
        // destination of the next merge, so in literal mode its contents stay observable.
        for (int t = 0; t < TT; t++)
            for (uint64_t id : hits[t]) ping[id] = nw | (ping[id] & WORD_START_BIT);
        N = Nnew;
        std::swap(ping, pong);

        if (max_seconds > 0) {
            double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            if (el > max_seconds) break;
        }
    }
    double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (seconds_out) *seconds_out = el;
    *n_merges_out = done;
    *early_stop_out = early;
    if (final_n) *final_n = N;
    if (final_sym) std::memcpy(final_sym, ping, N * sizeof(uint32_t));
    return 0;
}

// Chunk-bounded greedy longest match over a v3 trie (tokenize.wgsl:88-175).
// trie = 28-byte header, nodes {firstChild, numChildren, tokenId} u32 x3, edges {symbol, target} u32 x2.
// Chunk i covers bytes [i*cs, min((i+1)*cs, n)); a match never crosses a chunk end.
// tokens_out may be NULL (count only).  Returns the number of tokens, or UINT64_MAX on a bad trie.
uint64_t oracle_encode(const uint8_t* bytes, uint64_t n, const uint8_t* trie, uint64_t trie_len,
                       uint32_t chunk_size, int threads, uint32_t* tokens_out, uint64_t cap) {
    if (trie_len < 28) return UINT64_MAX;
    uint32_t hdr[7];
    std::memcpy(hdr, trie, 28);
    if (hdr[0] != 0x54524945u || hdr[1] != 3) return UINT64_MAX;
    const uint64_t nodeCount = hdr[2], edgeCount = hdr[3];
    if (trie_len < 28 + nodeCount * 12 + edgeCount * 8) return UINT64_MAX;
    const uint32_t* nodes = reinterpret_cast<const uint32_t*>(trie + 28);
    const uint32_t* edges = reinterpret_cast<const uint32_t*>(trie + 28 + nodeCount * 12);
    if (n == 0) return 0;

    auto find_child = [&](uint32_t first, uint32_t num, uint32_t symv) -> uint32_t {  // tokenize.wgsl:69-86
        uint32_t lo = 0, m = num;
        while (m > 0) {
            uint32_t half = m >> 1, mid = lo + half;
            bool less = (edges[(first + mid) * 2] & 0xFFu) < symv;
            lo = less ? mid + 1 : lo;
            m = less ? m - half - 1 : half;
        }
        if (lo < num) {
            uint32_t slot = (first + lo) * 2;
            if ((edges[slot] & 0xFFu) == symv) return edges[slot + 1];
        }
        return INVALID_TOKEN;
    };

    const uint64_t cs = chunk_size;
    const uint64_t chunks = (n + cs - 1) / cs;
    std::vector<uint32_t> counts(chunks, 0);
    std::vector<std::vector<uint32_t>> per_thread_tokens;
    int T = std::max(1, threads);
    if (chunks < 64) T = 1;
    // pass 1: tokenize each chunk into a private list, remember counts
    std::vector<std::vector<uint32_t>> toks(T);
    std::vector<uint64_t> first_chunk(T, 0);
    uint64_t per = (chunks + T - 1) / T;
    auto work = [&](int t) {
        uint64_t c0 = std::min(chunks, per * t), c1 = std::min(chunks, c0 + per);
        first_chunk[t] = c0;
        auto& out = toks[t];
        for (uint64_t c = c0; c < c1; c++) {
            uint64_t pos = c * cs, ce = std::min(n, pos + cs);
            uint32_t tw = 0;
            while (pos < ce && tw < chunk_size) {
                uint32_t cn = 0, lmt = INVALID_TOKEN;
                uint64_t lmp = pos, wp = pos;
                while (wp < ce) {
                    uint32_t bv = bytes[wp];
                    uint32_t nn = find_child(nodes[cn * 3], nodes[cn * 3 + 1] & 0xFFFFu, bv);
                    if (nn == INVALID_TOKEN) break;
                    cn = nn; wp++;
                    uint32_t ti = nodes[cn * 3 + 2];
                    if (ti != INVALID_TOKEN) { lmt = ti; lmp = wp; }
                }
                if (lmt != INVALID_TOKEN) { out.push_back(lmt); pos = lmp; }
                else { out.push_back(bytes[pos]); pos++; }
                tw++;
            }
            counts[c] = tw;
        }
    };
    if (T == 1) work(0);
    else {
        std::vector<std::thread> pool;
        for (int t = 0; t < T; t++) pool.emplace_back(work, t);
        for (auto& th : pool) th.join();
    }
    uint64_t total = 0;
    for (int t = 0; t < T; t++) {
        if (tokens_out)
            for (size_t i = 0; i < toks[t].size() && total + i < cap; i++) tokens_out[total + i] = toks[t][i];
        total += toks[t].size();
    }
    return total;
}

// Many documents, each encoded as a separate call of oracle_encode would encode it (chunks are
// counted from the document's first byte).  doc_offsets has n_docs + 1 entries into bytes;
// tok_offsets_out (n_docs + 1 entries) receives where each document's tokens start in tokens_out.
// Threads take contiguous runs of documents.  Returns the number of tokens, or UINT64_MAX on a bad trie.
uint64_t oracle_encode_batch(const uint8_t* bytes, const uint64_t* doc_offsets, uint32_t n_docs, const uint8_t* trie,
                             uint64_t trie_len, uint32_t chunk_size, int threads, uint32_t* tokens_out, uint64_t cap,
                             uint64_t* tok_offsets_out) {
    const int T = std::max(1, std::min<int>(threads, (int)std::max<uint32_t>(1, n_docs)));
    std::vector<std::vector<uint32_t>> toks(T);
    std::vector<std::vector<uint64_t>> lens(T);
    std::vector<uint32_t> first(T + 1, n_docs);
    const uint64_t total_bytes = doc_offsets[n_docs] - doc_offsets[0];
    first[0] = 0;
    for (int t = 1; t < T; t++) {   // balance by bytes
        const uint64_t want = doc_offsets[0] + total_bytes / T * t;
        uint32_t d = first[t - 1];
        while (d < n_docs && doc_offsets[d] < want) d++;
        first[t] = d;
    }
    std::atomic<int> bad{0};
    std::vector<std::thread> pool;
    for (int t = 0; t < T; t++) {
        pool.emplace_back([&, t]() {
            std::vector<uint32_t> tmp;
            for (uint32_t d = first[t]; d < first[t + 1]; d++) {
                const uint64_t a = doc_offsets[d], b = doc_offsets[d + 1];
                tmp.resize(std::max<uint64_t>(1, b - a));
                const uint64_t k = b > a ? oracle_encode(bytes + a, b - a, trie, trie_len, chunk_size, 1, tmp.data(), tmp.size()) : 0;
                if (k == UINT64_MAX) { bad = 1; return; }
                toks[t].insert(toks[t].end(), tmp.begin(), tmp.begin() + k);
                lens[t].push_back(k);
            }
        });
    }
    for (auto& th : pool) th.join();
    if (bad) return UINT64_MAX;
    uint64_t total = 0;
    uint32_t d = 0;
    for (int t = 0; t < T; t++) {
        uint64_t local = 0;
        for (uint64_t k : lens[t]) { tok_offsets_out[d++] = total + local; local += k; }
        if (tokens_out)
            for (size_t i = 0; i < toks[t].size() && total + i < cap; i++) tokens_out[total + i] = toks[t][i];
        total += toks[t].size();
    }
    tok_offsets_out[n_docs] = total;
    return total;
}

}  // extern "C"
