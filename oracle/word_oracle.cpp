// Word-level CPU oracle for the training merge loop in "fixed" compaction mode.
// TEST INFRASTRUCTURE ONLY: only tests/, the smoke check and bench.py's checker may load it.
//
// The direct restatement in bpe_oracle.cpp walks the whole symbol array once per merge, as the
// reference's shaders do (src/bpe/train.wgsl of toprakdeviren/gpu-bpe), which takes hours for a
// 1 GiB corpus and 32,000 merges.  This file computes the SAME merge list from the same rules by
// a different route, fast enough to check full-size runs:
//
//   * a pair is only ever counted or merged inside a word: the right symbol must not carry the
//     word-start bit (train.wgsl:393-398 count, :482-485 and :492-495 merge), and a symbol 0 never
//     pairs (train.wgsl:396-398), so it separates like a word start;
//   * in "fixed" mode the compaction keeps every surviving symbol (the documented algorithm of
//     train.wgsl:686-731 without the post-merge bound), so the corpus stays a multiset of words
//     and every merge acts on each word independently.
//
// So: split the corpus into words, keep each distinct word once with its multiplicity, and run
// the merge loop on that dictionary with exactly the reference's per-word rules:
//   count    every adjacent pair of a word, overlapping ones included (train.wgsl:392-411);
//   arg-max  larger count first, then the smaller packed pair (a << 16 | b) (train.wgsl:83-85);
//   stop     best count < 2, or the next id beyond 0xFFFF (train.wgsl:342-348);
//   merge    on the pre-merge snapshot: position i becomes the new symbol iff (s[i], s[i+1]) ==
//            (a, b); position i is dropped iff (s[i-1], s[i]) == (a, b) (train.wgsl:475-501).
//            With a == b a run of k >= 2 equal symbols therefore collapses to ONE new symbol.
// "literal" mode cannot be checked this way (it cuts symbols off the end of the array and exposes
// stale buffer contents, which breaks the word structure); bpe_oracle.cpp covers it.
//
// PARITY UNPINNED by the reference (it ships no vectors and cannot run here); this oracle is pinned
// against bpe_oracle.cpp on small corpora by tests/test_oracle.py.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <queue>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

inline uint64_t hash_bytes(const uint16_t* p, uint32_t n) {
    uint64_t h = 0x9E3779B97F4A7C15ull ^ n;
    for (uint32_t i = 0; i < n; i++) {
        h ^= p[i];
        h *= 0xff51afd7ed558ccdull;
        h ^= h >> 32;
    }
    return h;
}

// Distinct words with multiplicities: open addressing over (hash, offset, length), symbols in an arena.
struct WordSet {
    std::vector<uint64_t> hash;
    std::vector<uint64_t> off;     // into arena; UINT64_MAX = empty
    std::vector<uint32_t> len;
    std::vector<uint64_t> cnt;
    std::vector<uint16_t> arena;
    uint64_t used = 0, mask = 0;
    WordSet() { resize(1u << 16); }
    void resize(uint64_t cap) {
        hash.assign(cap, 0); off.assign(cap, UINT64_MAX); len.assign(cap, 0); cnt.assign(cap, 0);
        mask = cap - 1; used = 0;
    }
    void grow() {
        std::vector<uint64_t> h, o, c; std::vector<uint32_t> l;
        h.swap(hash); o.swap(off); c.swap(cnt); l.swap(len);
        resize(h.size() * 2);
        for (size_t i = 0; i < h.size(); i++) if (o[i] != UINT64_MAX) {
            uint64_t s = h[i] & mask;
            while (off[s] != UINT64_MAX) s = (s + 1) & mask;
            hash[s] = h[i]; off[s] = o[i]; len[s] = l[i]; cnt[s] = c[i]; used++;
        }
    }
    void add(const uint16_t* w, uint32_t n, uint64_t c) {
        if (used * 2 >= hash.size()) grow();
        const uint64_t h = hash_bytes(w, n);
        uint64_t s = h & mask;
        for (;;) {
            if (off[s] == UINT64_MAX) {
                hash[s] = h; off[s] = arena.size(); len[s] = n; cnt[s] = c; used++;
                arena.insert(arena.end(), w, w + n);
                return;
            }
            if (hash[s] == h && len[s] == n && std::memcmp(&arena[off[s]], w, n * 2ull) == 0) { cnt[s] += c; return; }
            s = (s + 1) & mask;
        }
    }
};

// Split [lo, hi) into words and add them to `ws`.  A word starts where `start(i)` says so (or at
// lo), and a symbol 0 is a word of its own.  lo must be a word start (or 0).
template <typename Tok, typename Start>
void collect(Tok tok, Start start, uint64_t lo, uint64_t hi, WordSet& ws) {
    std::vector<uint16_t> w;
    for (uint64_t i = lo; i < hi; i++) {
        const uint16_t t = tok(i);
        if (i > lo && (start(i) || t == 0 || (!w.empty() && w.back() == 0))) {
            ws.add(w.data(), (uint32_t)w.size(), 1);
            w.clear();
        }
        w.push_back(t);
    }
    if (!w.empty()) ws.add(w.data(), (uint32_t)w.size(), 1);
}

struct HeapEntry {
    uint64_t count;
    uint32_t pair;
    bool operator<(const HeapEntry& o) const {   // max-heap: larger count, then smaller pair on top
        return count < o.count || (count == o.count && pair > o.pair);
    }
};

template <typename Tok, typename Start>
int train_words(Tok tok, Start start, uint64_t n, uint32_t max_merges, uint32_t first_id, int threads,
                uint32_t* merges_out, uint32_t* n_merges_out, uint32_t* early_stop_out, uint64_t* final_n,
                uint64_t* distinct_words_out, uint64_t* distinct_pairs_out) {
    // 1. distinct words, counted in parallel over ranges that begin at word starts
    const int T = std::max(1, std::min(threads, 64));
    std::vector<uint64_t> cut(T + 1, n);
    cut[0] = 0;
    for (int t = 1; t < T; t++) {
        uint64_t c = std::max(cut[t - 1], n / T * t);
        while (c < n && !start(c)) c++;
        cut[t] = c;
    }
    std::vector<WordSet> parts(T);
    {
        std::vector<std::thread> pool;
        for (int t = 0; t < T; t++)
            pool.emplace_back([&, t]() { if (cut[t] < cut[t + 1]) collect(tok, start, cut[t], cut[t + 1], parts[t]); });
        for (auto& th : pool) th.join();
    }
    WordSet& all = parts[0];
    for (int t = 1; t < T; t++) {
        WordSet& p = parts[t];
        for (size_t i = 0; i < p.off.size(); i++)
            if (p.off[i] != UINT64_MAX) all.add(&p.arena[p.off[i]], p.len[i], p.cnt[i]);
        WordSet().hash.swap(p.hash);
        std::vector<uint16_t>().swap(p.arena);
    }
    // flat word list
    struct Word { uint64_t off; uint32_t len; uint64_t cnt; };
    std::vector<Word> words;
    words.reserve(all.used);
    for (size_t i = 0; i < all.off.size(); i++)
        if (all.off[i] != UINT64_MAX) words.push_back({all.off[i], all.len[i], all.cnt[i]});
    std::vector<uint16_t>& sym = all.arena;
    if (distinct_words_out) *distinct_words_out = words.size();

    // 2. pair counts and the words each pair occurs in (stale entries are harmless: a word is
    // re-examined when visited)
    std::unordered_map<uint32_t, uint64_t> count;
    std::unordered_map<uint32_t, std::vector<uint32_t>> where;
    count.reserve(1u << 20);
    where.reserve(1u << 20);
    auto pairs_of = [&](const Word& w, int sign, uint32_t wi, std::vector<uint32_t>* touched) {
        const uint16_t* s = &sym[w.off];
        for (uint32_t i = 0; i + 1 < w.len; i++) {
            if (s[i] == 0 || s[i + 1] == 0) continue;
            const uint32_t key = ((uint32_t)s[i] << 16) | s[i + 1];
            if (sign > 0) {
                count[key] += w.cnt;
                std::vector<uint32_t>& v = where[key];
                if (v.empty() || v.back() != wi) v.push_back(wi);
            } else {
                count[key] -= w.cnt;
            }
            if (touched) touched->push_back(key);
        }
    };
    for (uint32_t wi = 0; wi < words.size(); wi++) pairs_of(words[wi], +1, wi, nullptr);
    if (distinct_pairs_out) *distinct_pairs_out = count.size();
    std::priority_queue<HeapEntry> heap;
    for (auto& kv : count) heap.push({kv.second, kv.first});

    uint32_t next_id = first_id, done = 0, early = 0;
    std::vector<uint32_t> touched;
    while (done < max_merges) {
        // arg-max with lazy deletion: an entry is current iff it carries the pair's present count
        HeapEntry best{0, 0};
        while (!heap.empty()) {
            const HeapEntry e = heap.top();
            auto it = count.find(e.pair);
            if (it != count.end() && it->second == e.count && e.count > 0) { best = e; break; }
            heap.pop();
        }
        if (best.count < 2 || next_id > 0xFFFFu) { early = 1; break; }
        const uint32_t a = best.pair >> 16, b = best.pair & 0xFFFFu, nw = next_id;
        merges_out[done * 4 + 0] = a; merges_out[done * 4 + 1] = b;
        merges_out[done * 4 + 2] = nw; merges_out[done * 4 + 3] = (uint32_t)best.count;
        next_id++; done++;
        std::vector<uint32_t> ws;
        ws.swap(where[best.pair]);
        touched.clear();
        for (uint32_t wi : ws) {
            Word& w = words[wi];
            uint16_t* s = &sym[w.off];
            bool any = false;
            for (uint32_t i = 0; i + 1 < w.len && !any; i++) any = s[i] == a && s[i + 1] == b;
            if (!any) continue;
            pairs_of(w, -1, wi, &touched);
            // snapshot rule: keep i unless (s[i-1], s[i]) == (a, b); rewrite i iff (s[i], s[i+1]) == (a, b)
            uint32_t o = 0;
            uint16_t prev = 0;   // snapshot value of s[i-1]
            for (uint32_t i = 0; i < w.len; i++) {
                const uint16_t cur = s[i];
                const bool dropped = i > 0 && prev == a && cur == b;
                const bool rewritten = i + 1 < w.len && cur == a && s[i + 1] == b;
                prev = cur;
                if (!dropped) s[o++] = rewritten ? (uint16_t)nw : cur;
            }
            w.len = o;
            pairs_of(w, +1, wi, &touched);
        }
        std::sort(touched.begin(), touched.end());
        touched.erase(std::unique(touched.begin(), touched.end()), touched.end());
        for (uint32_t key : touched) {
            auto it = count.find(key);
            if (it == count.end()) continue;
            if (it->second == 0) { count.erase(it); where.erase(key); }
            else heap.push({it->second, key});
        }
    }
    *n_merges_out = done;
    *early_stop_out = early;
    if (final_n) {
        uint64_t N = 0;
        for (const Word& w : words) N += (uint64_t)w.len * w.cnt;
        *final_n = N;
    }
    return 0;
}

}  // namespace

extern "C" {

// Tagged u32 symbols (bit 16 = word start), as the trainer holds them.
int word_oracle_train_symbols(const uint32_t* sym, uint64_t n, uint32_t max_merges, uint32_t first_id, int threads,
                              uint32_t* merges_out, uint32_t* n_merges_out, uint32_t* early_stop_out, uint64_t* final_n,
                              uint64_t* distinct_words_out, uint64_t* distinct_pairs_out) {
    return train_words([&](uint64_t i) { return (uint16_t)(sym[i] & 0xFFFFu); },
                       [&](uint64_t i) { return (sym[i] & 0x10000u) != 0; }, n, max_merges, first_id, threads, merges_out,
                       n_merges_out, early_stop_out, final_n, distinct_words_out, distinct_pairs_out);
}

// Bytes plus the pre-tokeniser's word-start mask (one byte each), for corpora whose u32 symbols
// would not fit the host.
int word_oracle_train_bytes(const uint8_t* bytes, const uint8_t* word_starts, uint64_t n, uint32_t max_merges,
                            uint32_t first_id, int threads, uint32_t* merges_out, uint32_t* n_merges_out,
                            uint32_t* early_stop_out, uint64_t* final_n, uint64_t* distinct_words_out,
                            uint64_t* distinct_pairs_out) {
    return train_words([&](uint64_t i) { return (uint16_t)bytes[i]; }, [&](uint64_t i) { return word_starts[i] != 0; }, n,
                       max_merges, first_id, threads, merges_out, n_merges_out, early_stop_out, final_n,
                       distinct_words_out, distinct_pairs_out);
}

}  // extern "C"
