// Trie encoding on the device: chunk-bounded greedy longest match, then a single-pass
// scan + compaction of the per-chunk token runs.  Replaces trie_tokenizer_chunked,
// trie_prefix_sum and trie_tokenizer_compact (src/bpe/tokenizer/tokenize.wgsl:88-243 of the
// reference) and the host flow of TrieTokenizer.#encodeSinglePass (tokenizer.js:213-335).
//
// Device layout of the trie (built once per tokenizer from the v3 binary):
//   * nodes are renumbered: a node that ends a token gets the token id as its index, the others
//     follow after the largest id, the root comes last (or gets a reserved index)
//   * a packed child is  index | has_token | is_leaf, so a step of the walk is one lookup of
//     (parent << 8 | byte) and needs no second load to learn whether the new node ends a token
//     (and which), or whether it has children
//   * small tries (every index below 2^16, a few ten thousand transitions): a cuckoo table of
//     4-byte entries that every CTA copies into its shared memory.  The 24-bit key is permuted by
//     an odd multiplier modulo 2^24; the top bits pick the slot and only the rest is stored next to
//     the 18-bit packed child, so a lookup is two or three shared-memory loads and no branch
//   * medium tries (every index below 130,816; the 32,256-entry vocabulary of the benchmark has
//     86 K nodes): a HYBRID.  The walk's first step takes TWO bytes at once: the pairs (b0, b1)
//     that lead to a depth-2 node are keyed like transitions of a pseudo parent, and a 256-entry
//     table of the root's children says what a single byte is worth.  These and the most used of
//     the deeper transitions (ranked by the smallest token id below them: token ids are merge
//     ranks, so small means frequent) fill a bucketed cuckoo table in shared memory (two
//     sub-tables, buckets of two 4-byte entries, one 8-byte load each); the rest stay in a global
//     table, and a bit per node says whether a miss in shared memory has to look there at all
//   * larger tries: an open-addressing table of 8-byte entries in global memory, at most half
//     full, pinned in L2 with an access-policy window, behind a direct-mapped shared-memory cache
//     of recent probes (hits and misses) per CTA
#include <algorithm>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "ctx.cuh"

namespace b200bpe {

constexpr uint32_t T_MISS = 0xFFFFFFFFu;
constexpr uint32_t T_EMPTY_KEY = 0xFFFFFFFFu;
constexpr uint32_t T_HAS_TOKEN = 0x80000000u, T_LEAF = 0x40000000u, T_INDEX = 0x003FFFFFu;
constexpr uint32_t T_ROOT = 0x003FFFFEu;   // index of the root in device numbering (no flags)
constexpr uint32_t T_MAX_NODES = 0x003FFFF0u;

constexpr int TW_THREADS = 512;
constexpr int TW_CACHE_LOG2 = 13;  // 8192 entries * 8 B = 64 KB per CTA
constexpr int TW_SMEM_BYTES = (1 << TW_CACHE_LOG2) * 8;
constexpr int SC_THREADS = 256;    // scan/compaction: chunks per tile
constexpr uint32_t SC_MAX_SPINS = 1u << 22;

constexpr int CK_THREADS = 1024;   // cuckoo walk: one CTA per SM, the whole table in its shared memory
constexpr uint32_t CK_MIN_LOG2 = 11, CK_MAX_LOG2 = 14;  // slots per sub-table
constexpr uint32_t CK_HAS_TOKEN = 1u << 16, CK_LEAF = 1u << 17, CK_INDEX = 0xFFFFu, CK_VALUE = 0x3FFFFu;
constexpr uint32_t CK_EMPTY = 0xFFFFFFFFu;

// hybrid layout: 4-byte entries  remainder(13) << 19 | cold << 18 | leaf << 17 | index(17); a node ends a token iff
// its index is at most the largest token id (token nodes are numbered by their ids, the others follow);
// cold = some child of the node is in the global table only
constexpr int HY_THREADS = 512;
constexpr int HY_CTAS = 3;
constexpr uint32_t HY_BUCKET_LOG2 = 12;                       // buckets per sub-table; a bucket holds two entries
constexpr uint32_t HY_KEY_BITS = 25, HY_KEY_MASK = (1u << HY_KEY_BITS) - 1u;
constexpr uint32_t HY_REM_SHIFT = HY_KEY_BITS - HY_BUCKET_LOG2;   // 13 remainder bits
constexpr uint32_t HY_INDEX = 0x1FFFFu, HY_LEAF = 1u << 17, HY_COLD = 1u << 18;
constexpr uint32_t HY_ROOT2 = 0x1FF00u;                       // pseudo parents 0x1FF00 | b0 of the two-byte first step
constexpr uint32_t HY_MAX_INDEX = HY_ROOT2;                   // real node indices stay below
constexpr uint32_t HY_HOT_WORDS = 2u * (1u << HY_BUCKET_LOG2) * 2u;   // 16,384 entries = 64 KB
constexpr uint32_t HY_SMEM_BYTES = HY_HOT_WORDS * 4u + 256u * 4u;
constexpr double HY_MAX_LOAD = 0.86;

struct TrieHybrid {
    const uint32_t* hot;     // two sub-tables of (1 << HY_BUCKET_LOG2) buckets of two entries, then the 256 root children
    uint32_t mul[2];         // odd multipliers of the two hash functions (modulo 2^25)
    const uint2* cold;       // open addressing: {key, value in the 4-byte entry's value format}
    uint32_t cold_mask;
    uint32_t max_token;      // indices up to this one end a token
};

struct TrieDev {
    const uint2* trans;      // {parent << 8 | byte, packed child}
    uint32_t trans_mask;
    const uint32_t* cuckoo;  // D sub-tables of 1 << ck_log2 entries: remainder << 18 | packed child
    uint32_t ck_log2;
    uint32_t ck_mul[3];      // odd multipliers, one per sub-table
    uint32_t root;           // packed root
};


// Where chunk g starts and ends.  Single buffer: fixed stride.  Batch: chunks are numbered
// document by document (chunk_base = exclusive scan of per-document chunk counts) and never
// span two documents, exactly as separate encodeBytes calls would cut them.
__device__ __forceinline__ void chunk_span(uint64_t g, uint32_t cs, uint64_t n, const uint64_t* __restrict__ doc_off,
                                           const uint64_t* __restrict__ chunk_base, uint32_t n_docs, uint64_t* lo,
                                           uint64_t* hi) {
    if (!doc_off) {
        *lo = g * cs;
        *hi = min(n, *lo + cs);
        return;
    }
    uint32_t a = 0, b = n_docs;  // last d with chunk_base[d] <= g
    while (b - a > 1) {
        const uint32_t m = (a + b) >> 1;
        if (chunk_base[m] <= g) a = m; else b = m;
    }
    *lo = doc_off[a] + (g - chunk_base[a]) * cs;
    *hi = min(doc_off[a + 1], *lo + cs);
}

// One thread walks one chunk.  The walk is a flat loop: every iteration either takes one
// transition (one probe of the shared-memory cache, the root included) or ends the current token,
// with the same instructions for every lane, so the lanes of a warp stay together although their
// tokens end at different places.  Nodes that end a token are numbered by their token id, so the
// packed child says which token ends there and ending a token costs no load.  Positions are
// 32-bit offsets into the chunk; input is read one aligned 32-bit word at a time (the sector
// stays in L1 for the next seven); tokens are buffered four at a time and stored as one 16-byte word.
// D == 0: global table behind the probe cache.  D == 2 or 3: cuckoo table with D sub-tables in
// shared memory (CACHE_LOG2 unused; the dynamic shared memory holds D << ck_log2 entries).
template <int THREADS, int CACHE_LOG2, int D>
__global__ void __launch_bounds__(THREADS, D == 0 ? 3 : 1)
k_trie_walk(TrieDev t, const uint8_t* __restrict__ bytes, uint64_t n, uint32_t cs, const uint64_t* __restrict__ doc_off,
            const uint64_t* __restrict__ chunk_base, uint32_t n_docs, uint64_t n_chunks_static,
            uint32_t* __restrict__ staging, uint32_t* __restrict__ counts, uint32_t* __restrict__ ticket) {
    extern __shared__ __align__(16) unsigned char tw_smem[];
    uint2* cache = reinterpret_cast<uint2*>(tw_smem);  // {parent << 8 | byte, packed child}
    uint32_t* ck = reinterpret_cast<uint32_t*>(tw_smem);
    constexpr uint32_t HAS = D == 0 ? T_HAS_TOKEN : CK_HAS_TOKEN, LEAF = D == 0 ? T_LEAF : CK_LEAF;
    constexpr uint32_t INDEX = D == 0 ? T_INDEX : CK_INDEX;
    if constexpr (D == 0) {
        for (int i = threadIdx.x; i < (1 << CACHE_LOG2); i += THREADS) cache[i] = make_uint2(T_EMPTY_KEY, 0u);
    } else {
        const uint4* __restrict__ src = reinterpret_cast<const uint4*>(t.cuckoo);
        for (uint32_t i = threadIdx.x; i < ((uint32_t)D << t.ck_log2) / 4u; i += THREADS)
            reinterpret_cast<uint4*>(tw_smem)[i] = __ldg(src + i);
    }
    __syncthreads();
    const uint32_t ck_shift = 24u - t.ck_log2, ck_rmask = (1u << ck_shift) - 1u, ck_size = 1u << t.ck_log2;
    const uint64_t n_chunks = doc_off ? chunk_base[n_docs] : n_chunks_static;
    const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(bytes) & 3u);
    const uint32_t* __restrict__ words = reinterpret_cast<const uint32_t*>(reinterpret_cast<uintptr_t>(bytes) - shift);
    const bool vec_ok = (cs & 3u) == 0u;  // chunk staging slots are 16-byte aligned

    // Chunks are handed out 32 at a time to whichever warp is free (documents end in short chunks,
    // so a fixed assignment would leave lanes and whole warps idle at the end).
    const int lane = threadIdx.x & 31;
    for (;;) {
        uint32_t first = 0u;
        if (lane == 0) first = atomicAdd(ticket, 32u);
        first = __shfl_sync(0xFFFFFFFFu, first, 0);
        if ((uint64_t)first >= n_chunks) break;
        const uint64_t g = (uint64_t)first + lane;
        if (g >= n_chunks) continue;
        uint64_t lo, hi;
        chunk_span(g, cs, n, doc_off, chunk_base, n_docs, &lo, &hi);
        const uint32_t len = (uint32_t)(hi - lo);
        const uint32_t* __restrict__ cw = words + ((lo + shift) >> 2);  // word holding the chunk's first byte
        const uint32_t a0 = (uint32_t)((lo + shift) & 3u);              // and that byte's place in it
        uint32_t* __restrict__ out = staging + g * cs;
        uint32_t widx = 0xFFFFFFFFu, word = 0u;
        // bytes from the chunk's start to the end of the whole input: prefetches stay inside it
        const uint32_t pf_limit = (uint32_t)min((unsigned long long)(n - lo), 0xFFFFFFFFull);
        auto byte_at = [&](uint32_t r) -> uint32_t {
            const uint32_t qq = a0 + r;
            if ((qq >> 2) != widx) {
                widx = qq >> 2;
                word = __ldg(cw + widx);
                // entering a new 32-byte sector: ask for the one after it now
                if ((widx & 7u) == 0u && r + 72u < pf_limit) asm volatile("prefetch.global.L1 [%0];" ::"l"(cw + widx + 8));
            }
            return (word >> ((qq & 3u) * 8u)) & 0xFFu;
        };
        uint32_t tw = 0;
        uint4 buf = make_uint4(0u, 0u, 0u, 0u), buf_lo = make_uint4(0u, 0u, 0u, 0u);  // eight tokens = one 32-byte sector
        uint32_t p = 0, w = 0, l = 0;   // token start, walk position, end of the longest token so far
        uint32_t v = t.root;            // packed current node
        uint32_t last = 0u;
        bool have = false;              // a token ends somewhere on the walk so far
        uint32_t fb = 0u;               // the byte at p, seen by the first step of every walk
        // One iteration = one probe, then either a step or the end of a token; both outcomes are
        // computed with selects so that all lanes run the same instructions.
        while (p < len) {
            const bool can = w < len && !(v & LEAF);
            const uint32_t b = byte_at(min(w, len - 1u));
            fb = (w == p) ? b : fb;
            const uint32_t key = ((v & INDEX) << 8) | b;
            uint32_t nv;
            if constexpr (D == 0) {
                const uint32_t h = key * 0x9E3779B1u;
                const uint32_t ci = h >> (32 - CACHE_LOG2);
                const uint2 c = cache[ci];
                nv = c.y;
                if (c.x != key) {
                    nv = T_MISS;
                    uint32_t slot = (h ^ (h >> 15)) & t.trans_mask;
                    for (;;) {
                        const uint2 e = __ldg(t.trans + slot);
                        if (e.x == key) { nv = e.y; break; }
                        if (e.x == T_EMPTY_KEY) break;
                        slot = (slot + 1) & t.trans_mask;
                    }
                    cache[ci] = make_uint2(key, nv);  // misses are cached too
                }
            } else {
                nv = T_MISS;
#pragma unroll
                for (int d = D - 1; d >= 0; d--) {
                    const uint32_t h = (key * t.ck_mul[d]) & 0xFFFFFFu;
                    const uint32_t e = ck[d * ck_size + (h >> ck_shift)];
                    nv = (e >> 18) == (h & ck_rmask) ? (e & CK_VALUE) : nv;
                }
            }
            const bool step = can && nv != T_MISS;
            const bool ends = step && (nv & HAS);
            // the walk from p is over when there is no step: emit the longest token seen, or the raw byte
            const uint32_t tok = have ? last : fb;
            const uint32_t p_next = have ? l : p + 1u;
            const uint32_t k = tw & 3u;
            buf.x = (!step && k == 0u) ? tok : buf.x;
            buf.y = (!step && k == 1u) ? tok : buf.y;
            buf.z = (!step && k == 2u) ? tok : buf.z;
            buf.w = (!step && k == 3u) ? tok : buf.w;
            if (!step && k == 3u) {
                if ((tw & 4u) == 0u) {
                    buf_lo = buf;  // first half of the sector: hold it back
                } else if (vec_ok) {
                    uint4* __restrict__ o4 = reinterpret_cast<uint4*>(out + (tw & ~7u));
                    o4[0] = buf_lo;
                    o4[1] = buf;
                } else {
                    uint32_t* __restrict__ o = out + (tw & ~7u);
                    o[0] = buf_lo.x; o[1] = buf_lo.y; o[2] = buf_lo.z; o[3] = buf_lo.w;
                    o[4] = buf.x; o[5] = buf.y; o[6] = buf.z; o[7] = buf.w;
                }
            }
            tw += step ? 0u : 1u;
            p = step ? p : p_next;
            w = step ? w + 1u : p_next;
            last = ends ? (nv & INDEX) : last;
            l = ends ? w : l;
            have = step ? (have || ends) : false;
            v = step ? nv : t.root;
        }
        {   // what is left of the last sector
            uint32_t base = tw & ~7u;
            if (tw & 4u) { out[base] = buf_lo.x; out[base + 1] = buf_lo.y; out[base + 2] = buf_lo.z; out[base + 3] = buf_lo.w; base += 4u; }
            const uint32_t k = tw & 3u;
            if (k > 0u) out[base] = buf.x;
            if (k > 1u) out[base + 1] = buf.y;
            if (k > 2u) out[base + 2] = buf.z;
        }
        counts[g] = tw;
    }
}

// The hybrid walk.  One thread per chunk, one flat loop; an iteration is one probe of the shared
// table.  In the first iteration of a token the probe takes two bytes (key: pseudo parent of the
// first byte, second byte) and the root's child table gives the one-byte candidate; a miss there
// ends the token at once.  Later iterations take one byte.  Tokens are stored as they end.
__global__ void __launch_bounds__(HY_THREADS, HY_CTAS)
k_trie_walk_hybrid(TrieHybrid t, const uint8_t* __restrict__ bytes, uint64_t n, uint32_t cs, const uint64_t* __restrict__ doc_off,
                   const uint64_t* __restrict__ chunk_base, uint32_t n_docs, uint64_t n_chunks_static,
                   uint32_t* __restrict__ staging, uint32_t* __restrict__ counts, uint32_t* __restrict__ ticket) {
    extern __shared__ __align__(16) unsigned char tw_smem[];
    uint32_t* sm = reinterpret_cast<uint32_t*>(tw_smem);
    {
        const uint4* __restrict__ src = reinterpret_cast<const uint4*>(t.hot);
        for (uint32_t i = threadIdx.x; i < HY_SMEM_BYTES / 16u; i += HY_THREADS) reinterpret_cast<uint4*>(tw_smem)[i] = __ldg(src + i);
    }
    __syncthreads();
    const uint2* __restrict__ hot0 = reinterpret_cast<const uint2*>(sm);
    const uint2* __restrict__ hot1 = hot0 + (1u << HY_BUCKET_LOG2);
    const uint32_t* __restrict__ t1 = sm + HY_HOT_WORDS;
    const uint32_t mul0 = t.mul[0], mul1 = t.mul[1];
    const uint64_t n_chunks = doc_off ? chunk_base[n_docs] : n_chunks_static;
    const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(bytes) & 3u);
    const uint32_t* __restrict__ words = reinterpret_cast<const uint32_t*>(reinterpret_cast<uintptr_t>(bytes) - shift);
    const uint64_t last_word = (n + shift + 3u) / 4u;   // words [0, last_word) hold input bytes
    const int lane = threadIdx.x & 31;
    for (;;) {
        uint32_t first = 0u;
        if (lane == 0) first = atomicAdd(ticket, 32u);
        first = __shfl_sync(0xFFFFFFFFu, first, 0);
        if ((uint64_t)first >= n_chunks) break;
        const uint64_t g = (uint64_t)first + lane;
        if (g >= n_chunks) continue;
        uint64_t lo, hi;
        chunk_span(g, cs, n, doc_off, chunk_base, n_docs, &lo, &hi);
        const uint32_t len = (uint32_t)(hi - lo);
        const uint64_t w_first = (lo + shift) >> 2;                     // word holding the chunk's first byte
        const uint32_t* __restrict__ cw = words + w_first;
        const uint32_t a0 = (uint32_t)((lo + shift) & 3u);              // and that byte's place in it
        const uint32_t w_avail = (uint32_t)min((unsigned long long)(last_word - w_first), 0xFFFFFFFFull);
        uint32_t* __restrict__ out = staging + g * cs;
        // a window of two words: the bytes at q and q + 1 come out of one funnel shift
        uint32_t widx = 0u;
        uint32_t word0 = __ldg(cw), word1 = 1u < w_avail ? __ldg(cw + 1) : 0u;
        uint32_t tw = 0;
        uint32_t p = 0, w = 0, l = 0;   // token start, walk position, end of the longest token so far
        uint32_t v = 0u, last = 0u, fb = 0u;
        bool have = false;
        while (p < len) {
            const uint32_t qq = a0 + w;
            if ((qq >> 2) != widx) {   // the walk position moves by at most two bytes per iteration and never back past p
                const uint32_t nw = qq >> 2;
                if (nw == widx + 1u) { word0 = word1; }
                else { word0 = __ldg(cw + nw); }
                widx = nw;
                word1 = widx + 1u < w_avail ? __ldg(cw + widx + 1u) : 0u;
                if ((widx & 7u) == 0u && widx + 24u < w_avail) asm volatile("prefetch.global.L1 [%0];" ::"l"(cw + widx + 16));
            }
            const uint32_t two_bytes = __funnelshift_r(word0, word1, (qq & 3u) * 8u);
            const uint32_t b = two_bytes & 0xFFu, b2 = (two_bytes >> 8) & 0xFFu;
            const bool fresh = w == p;
            const bool two = fresh && (w + 1u < len);
            const uint32_t n1 = t1[b];                      // the root's child for this byte (T_MISS: none)
            fb = fresh ? b : fb;
            const uint32_t key = fresh ? (((HY_ROOT2 | b) << 8) | b2) : (((v & HY_INDEX) << 8) | b);
            const uint32_t h0 = (key * mul0) & HY_KEY_MASK, h1 = (key * mul1) & HY_KEY_MASK;
            const uint2 e0 = hot0[h0 >> HY_REM_SHIFT], e1 = hot1[h1 >> HY_REM_SHIFT];
            const uint32_t r0 = h0 & ((1u << HY_REM_SHIFT) - 1u), r1 = h1 & ((1u << HY_REM_SHIFT) - 1u);
            uint32_t nv = T_MISS;
            nv = (e0.x >> 19) == r0 ? e0.x : nv;
            nv = (e0.y >> 19) == r0 ? e0.y : nv;
            nv = (e1.x >> 19) == r1 ? e1.x : nv;
            nv = (e1.y >> 19) == r1 ? e1.y : nv;
            bool hit = (nv & HY_INDEX) != HY_INDEX && (two || !fresh);   // an empty entry is all ones
            if (!hit && !fresh && (v & HY_COLD)) {
                // some of this node's children live in the global table only
                {
                    const uint32_t hh = key * 0x9E3779B1u;
                    uint32_t slot = (hh ^ (hh >> 15)) & t.cold_mask;
                    for (;;) {
                        const uint2 e = __ldg(t.cold + slot);
                        if (e.x == key) { nv = e.y; hit = true; break; }
                        if (e.x == T_EMPTY_KEY) break;
                        slot = (slot + 1) & t.cold_mask;
                    }
                }
            }
            if (fresh) {   // what the first byte alone is worth
                have = (n1 & HY_INDEX) <= t.max_token;   // T_MISS has an index above every token id
                last = n1 & HY_INDEX;
                l = p + 1u;
            }
            if (hit) {
                v = nv;
                w = fresh ? p + 2u : w + 1u;
                if ((nv & HY_INDEX) <= t.max_token) { have = true; last = nv & HY_INDEX; l = w; }
            }
            const bool ends = !hit || (nv & HY_LEAF) != 0u || w >= len;
            if (ends) {
                out[tw++] = have ? last : fb;
                p = have ? l : p + 1u;
                w = p;
            }
        }
        counts[g] = tw;
    }
}

// Per-document chunk counts → exclusive scan (one CTA; documents are few compared with bytes).
__global__ void __launch_bounds__(1024)
k_doc_chunk_scan(const uint64_t* __restrict__ doc_off, uint32_t n_docs, uint32_t cs, uint64_t* __restrict__ chunk_base) {
    __shared__ uint64_t wsum[32];
    __shared__ uint64_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t b = 0; b < n_docs; b += 1024) {
        const uint32_t d = b + threadIdx.x;
        uint64_t c = 0;
        if (d < n_docs) c = (doc_off[d + 1] - doc_off[d] + cs - 1) / cs;
        uint64_t incl = c;
        for (int o = 1; o < 32; o <<= 1) {
            const uint64_t x = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += x;
        }
        if (lane == 31) wsum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            uint64_t w = wsum[lane], wi = w;
            for (int o = 1; o < 32; o <<= 1) {
                const uint64_t x = __shfl_up_sync(0xFFFFFFFFu, wi, o);
                if (lane >= o) wi += x;
            }
            wsum[lane] = wi - w;
        }
        __syncthreads();
        const uint64_t excl = carry + wsum[warp] + incl - c;
        if (d < n_docs) chunk_base[d] = excl;
        __syncthreads();
        if (threadIdx.x == 1023) carry = excl + c;
        __syncthreads();
    }
    if (threadIdx.x == 0) chunk_base[n_docs] = carry;
}

// Tile descriptor of the look-back: bits 63..62 = flag (1 aggregate, 2 prefix), low 62 bits = value.
__device__ __forceinline__ unsigned long long ld_d64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_d64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// One tile = SC_THREADS chunks.  Sum the tile's token counts, learn the tile's offset by
// decoupled look-back, then copy every chunk's run from its stride-`cs` staging slot to its final
// place with coalesced warp copies.  ctl[0] = tile ticket, ctl[1] = error flag; total → *total_out.
__global__ void __launch_bounds__(SC_THREADS)
k_scan_compact(const uint32_t* __restrict__ staging, const uint32_t* __restrict__ counts, uint32_t cs,
               const uint64_t* __restrict__ chunk_base, uint32_t n_docs, uint64_t n_chunks_static,
               unsigned long long* __restrict__ desc, uint32_t* __restrict__ ctl, uint64_t* __restrict__ chunk_offsets,
               uint32_t* __restrict__ out, uint64_t cap, uint64_t* __restrict__ total_out, uint32_t max_spins) {
    __shared__ uint64_t s_off[SC_THREADS];
    __shared__ uint32_t s_cnt[SC_THREADS];
    __shared__ uint32_t wsum[SC_THREADS / 32];
    __shared__ uint32_t s_tile;
    __shared__ uint64_t s_base;
    const uint64_t n_chunks = chunk_base ? chunk_base[n_docs] : n_chunks_static;
    const uint64_t ntiles = (n_chunks + SC_THREADS - 1) / SC_THREADS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (n_chunks == 0) {
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            *total_out = 0;
            if (chunk_offsets) chunk_offsets[0] = 0;
        }
        return;
    }
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) s_tile = atomicAdd(&ctl[0], 1u);
        __syncthreads();
        const uint64_t tile = s_tile;
        if (tile >= ntiles) break;
        const uint64_t g = tile * SC_THREADS + threadIdx.x;
        const uint32_t c = g < n_chunks ? counts[g] : 0u;
        uint32_t incl = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t x = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += x;
        }
        if (lane == 31) wsum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const uint32_t w = lane < SC_THREADS / 32 ? wsum[lane] : 0u;
            uint32_t wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t x = __shfl_up_sync(0xFFFFFFFFu, wi, o);
                if (lane >= o) wi += x;
            }
            if (lane < SC_THREADS / 32) wsum[lane] = wi - w;
            const unsigned long long agg = __shfl_sync(0xFFFFFFFFu, wi, SC_THREADS / 32 - 1);
            unsigned long long excl = 0ull;
            if (tile == 0) {
                if (lane == 0) st_d64(desc, (2ull << 62) | agg);
            } else {
                if (lane == 0) st_d64(desc + tile, (1ull << 62) | agg);
                long long pos = (long long)tile - 1;
                uint32_t spins = 0;
                bool timed_out = false;
                for (;;) {
                    const long long idx = pos - lane;
                    unsigned long long d = 2ull << 62;  // before tile 0: a zero prefix
                    for (;;) {
                        if (idx >= 0) d = ld_d64(desc + idx);
                        if (__all_sync(0xFFFFFFFFu, (d >> 62) != 0ull)) break;
                        if (++spins > max_spins) { timed_out = true; break; }
                        __nanosleep(40);
                    }
                    if (timed_out) break;
                    const uint32_t pmask = __ballot_sync(0xFFFFFFFFu, (d >> 62) == 2ull);
                    const int first = pmask ? (__ffs(pmask) - 1) : 32;
                    unsigned long long contrib = (lane <= first) ? (d & 0x3FFFFFFFFFFFFFFFull) : 0ull;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xFFFFFFFFu, contrib, o);
                    excl += contrib;
                    if (pmask) break;
                    pos -= 32;
                }
                if (timed_out) {
                    if (lane == 0) atomicExch(&ctl[1], 1u);
                    excl = 0ull;
                }
                if (lane == 0) st_d64(desc + tile, (2ull << 62) | (excl + agg));
            }
            if (lane == 0) {
                s_base = excl;
                if (tile == ntiles - 1) {
                    *total_out = excl + agg;
                    if (chunk_offsets) chunk_offsets[n_chunks] = excl + agg;
                }
            }
        }
        __syncthreads();
        const uint64_t off = s_base + wsum[warp] + (incl - c);
        s_off[threadIdx.x] = off;
        s_cnt[threadIdx.x] = c;
        if (chunk_offsets && g < n_chunks) chunk_offsets[g] = off;
        __syncthreads();
        for (int k = warp; k < SC_THREADS; k += SC_THREADS / 32) {
            const uint32_t cnt = s_cnt[k];
            if (cnt == 0u) continue;
            const uint64_t o = s_off[k];
            const uint32_t* __restrict__ src = staging + (tile * SC_THREADS + k) * (uint64_t)cs;
            // four loads in flight per lane before the first store: the copy is latency-bound otherwise
            for (uint32_t i = lane; i < cnt; i += 128) {
                const uint32_t v0 = src[i];
                const uint32_t v1 = i + 32 < cnt ? src[i + 32] : 0u;
                const uint32_t v2 = i + 64 < cnt ? src[i + 64] : 0u;
                const uint32_t v3 = i + 96 < cnt ? src[i + 96] : 0u;
                if (o + i < cap) out[o + i] = v0;
                if (i + 32 < cnt && o + i + 32 < cap) out[o + i + 32] = v1;
                if (i + 64 < cnt && o + i + 64 < cap) out[o + i + 64] = v2;
                if (i + 96 < cnt && o + i + 96 < cap) out[o + i + 96] = v3;
            }
        }
    }
}

__global__ void k_doc_token_offsets(const uint64_t* __restrict__ chunk_base, const uint64_t* __restrict__ chunk_offsets,
                                    uint32_t n_docs, uint64_t* __restrict__ tok_offsets) {
    for (uint32_t d = blockIdx.x * blockDim.x + threadIdx.x; d <= n_docs; d += gridDim.x * blockDim.x)
        tok_offsets[d] = chunk_offsets[chunk_base[d]];
}

struct Tokenizer {
    Ctx* ctx = nullptr;
    uint32_t node_count = 0, edge_count = 0, max_token_len = 0, chunk = 0;
    uint2* d_trans = nullptr;      // large tries: global transition table
    uint32_t trans_mask = 0;
    size_t trans_bytes = 0;
    uint32_t* d_cuckoo = nullptr;  // small tries: cuckoo table, copied into shared memory by every CTA
    int ck_d = 0;                  // its number of sub-tables (0: the global table is in use)
    uint32_t ck_log2 = 0, ck_mul[3] = {1u, 1u, 1u};
    uint32_t root = T_ROOT;
    // medium tries: the hybrid layout
    bool hybrid = false;
    uint32_t* d_hot = nullptr;       // shared-memory image: the bucketed cuckoo table, then the root's 256 children
    uint2* d_cold = nullptr;
    uint32_t hy_mul[2] = {1u, 1u}, cold_mask = 0, hot_entries = 0, max_token = 0;
    uint32_t sc_max_spins = SC_MAX_SPINS;       // polls after which the compaction's look-back gives up
    bool skip_first_tile = false;               // test of that bounded wait: tile 0 is never worked on
    uint64_t batch_slice_bytes = 32ull << 20;   // host batches above twice this are encoded slice by slice
    uint64_t encode_slice_bytes = 8ull << 30;   // b200bpe_encode: larger inputs go through in chunk-aligned slices
    // pooled work buffers (grown on demand, as tokenizer.js:108-166 does)
    uint8_t* d_in = nullptr; uint64_t in_cap = 0;
    uint32_t* d_staging = nullptr; uint64_t staging_cap = 0;   // elements
    uint32_t* d_counts = nullptr; uint64_t counts_cap = 0;
    uint64_t* d_chunk_off = nullptr; uint64_t chunk_off_cap = 0;
    uint32_t* d_out = nullptr; uint64_t out_cap = 0;           // elements
    uint64_t* d_doc_off = nullptr; uint64_t doc_off_cap = 0;
    uint64_t* d_chunk_base = nullptr; uint64_t chunk_base_cap = 0;
    uint64_t* d_tok_off = nullptr; uint64_t tok_off_cap = 0;
    unsigned long long* d_desc = nullptr; uint64_t desc_cap = 0;
    uint32_t* d_ctl = nullptr;
    uint64_t* d_total = nullptr;
    uint64_t* h_total = nullptr;  // pinned: total, error flag
    cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};
    double walk_ms = 0, compact_ms = 0;

    ~Tokenizer() {
        if (ctx) cudaSetDevice(ctx->device);
        cudaFree(d_trans); cudaFree(d_cuckoo); cudaFree(d_hot); cudaFree(d_cold); cudaFree(d_in); cudaFree(d_staging);
        cudaFree(d_counts); cudaFree(d_chunk_off); cudaFree(d_out); cudaFree(d_doc_off); cudaFree(d_chunk_base);
        cudaFree(d_tok_off); cudaFree(d_desc); cudaFree(d_ctl); cudaFree(d_total);
        if (h_total) cudaFreeHost(h_total);
        if (h_slices) cudaFreeHost(h_slices);
        for (auto e : ev) if (e) cudaEventDestroy(e);
        for (auto e : slice_ev) cudaEventDestroy(e);
        if (s_read) cudaStreamDestroy(s_read);
    }

    template <typename T>
    b200bpe_status ensure(T** p, uint64_t* cap, uint64_t need, bool grow = true) {
        if (need <= *cap) return B200BPE_OK;
        B2_CUDA(cudaStreamSynchronize(ctx->stream));
        cudaFree(*p);
        *p = nullptr;
        const uint64_t want = grow ? need + need / 2 : need;
        if (cudaMalloc(p, want * sizeof(T)) != cudaSuccess) {
            cudaGetLastError();
            B2_CUDA(cudaMalloc(p, need * sizeof(T)));
            *cap = need;
        } else {
            *cap = want;
        }
        return B200BPE_OK;
    }

    b200bpe_status ensure_work(uint64_t max_chunks) {
        b200bpe_status r;
        if ((r = ensure(&d_staging, &staging_cap, max_chunks * chunk))) return r;
        if ((r = ensure(&d_counts, &counts_cap, max_chunks + 1))) return r;
        if ((r = ensure(&d_chunk_off, &chunk_off_cap, max_chunks + 1))) return r;
        if ((r = ensure(&d_desc, &desc_cap, max_chunks / SC_THREADS + 2))) return r;
        return B200BPE_OK;
    }

    size_t walk_smem() const { return hybrid ? (size_t)HY_SMEM_BYTES : ck_d == 0 ? (size_t)TW_SMEM_BYTES : ((size_t)ck_d << ck_log2) * 4; }

    // The walk kernel for this tokenizer's trie layout; max_chunks only sizes the grid.
    void walk(const uint8_t* d_bytes, uint64_t n, const uint64_t* d_docs, const uint64_t* cb, uint32_t n_docs,
              uint64_t max_chunks, uint32_t* staging, uint32_t* counts, uint32_t* ticket) {
        cudaStream_t s = ctx->stream;
        TrieDev t{d_trans, trans_mask, d_cuckoo, ck_log2, {ck_mul[0], ck_mul[1], ck_mul[2]}, root};
        const uint64_t n_static = (n + chunk - 1) / chunk;
        if (hybrid) {
            TrieHybrid th{d_hot, {hy_mul[0], hy_mul[1]}, d_cold, cold_mask, max_token};
            const int grid = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)ctx->sm_count * HY_CTAS, (max_chunks + HY_THREADS - 1) / HY_THREADS));
            k_trie_walk_hybrid<<<grid, HY_THREADS, HY_SMEM_BYTES, s>>>(th, d_bytes, n, chunk, d_docs, cb, n_docs, n_static, staging, counts, ticket);
        } else if (ck_d == 0) {
            const int grid = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)ctx->sm_count * 3, (max_chunks + TW_THREADS - 1) / TW_THREADS));
            k_trie_walk<TW_THREADS, TW_CACHE_LOG2, 0><<<grid, TW_THREADS, walk_smem(), s>>>(
                t, d_bytes, n, chunk, d_docs, cb, n_docs, n_static, staging, counts, ticket);
        } else {
            const int grid = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)ctx->sm_count, (max_chunks + CK_THREADS - 1) / CK_THREADS));
            if (ck_d == 2)
                k_trie_walk<CK_THREADS, 0, 2><<<grid, CK_THREADS, walk_smem(), s>>>(
                    t, d_bytes, n, chunk, d_docs, cb, n_docs, n_static, staging, counts, ticket);
            else
                k_trie_walk<CK_THREADS, 0, 3><<<grid, CK_THREADS, walk_smem(), s>>>(
                    t, d_bytes, n, chunk, d_docs, cb, n_docs, n_static, staging, counts, ticket);
        }
    }

    // Walk + scan/compact on device-resident inputs.  d_docs == nullptr → one buffer.
    // h_dst / evs: where this launch's {total, error flag} and its three timing events go (default:
    // the tokenizer's own), so that several launches can be in flight on the stream.
    b200bpe_status launch(const uint8_t* d_bytes, uint64_t n, const uint64_t* d_docs, uint32_t n_docs,
                          uint32_t* d_tokens, uint64_t cap, uint64_t* d_tok_offsets, uint64_t* h_dst = nullptr,
                          cudaEvent_t* evs = nullptr) {
        cudaStream_t s = ctx->stream;
        uint64_t* hd = h_dst ? h_dst : h_total;
        cudaEvent_t* ev = evs ? evs : this->ev;
        if (ck_d == 0 && !hybrid) set_persisting_window(ctx, d_trans, trans_bytes);  // keep the transition table resident in L2
        const uint64_t max_chunks = (n + chunk - 1) / chunk + (d_docs ? n_docs : 0);
        b200bpe_status r = ensure_work(std::max<uint64_t>(1, max_chunks));
        if (r) return r;
        const uint64_t ntiles = max_chunks / SC_THREADS + 2;
        B2_CUDA(cudaMemsetAsync(d_desc, 0, ntiles * 8, s));
        B2_CUDA(cudaMemsetAsync(d_ctl, 0, 16, s));
        if (skip_first_tile) {   // the tile ticket starts at 1
            static const uint32_t one = 1u;
            B2_CUDA(cudaMemcpyAsync(d_ctl, &one, 4, cudaMemcpyHostToDevice, s));
        }
        const uint64_t* cb = nullptr;
        if (d_docs) {
            if ((r = ensure(&d_chunk_base, &chunk_base_cap, (uint64_t)n_docs + 1))) return r;
            k_doc_chunk_scan<<<1, 1024, 0, s>>>(d_docs, n_docs, chunk, d_chunk_base);
            cb = d_chunk_base;
        }
        B2_CUDA(cudaEventRecord(ev[0], s));
        walk(d_bytes, n, d_docs, cb, n_docs, max_chunks, d_staging, d_counts, d_ctl + 2);
        B2_CUDA(cudaEventRecord(ev[1], s));
        const int grid_c = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)ctx->sm_count * 8, ntiles));
        k_scan_compact<<<grid_c, SC_THREADS, 0, s>>>(d_staging, d_counts, chunk, cb, n_docs, (n + chunk - 1) / chunk, d_desc,
                                                    d_ctl, d_chunk_off, d_tokens, cap, d_total, sc_max_spins);
        B2_CUDA(cudaEventRecord(ev[2], s));
        if (d_docs && d_tok_offsets)
            k_doc_token_offsets<<<std::max(1u, std::min(1024u, (n_docs + 256) / 256)), 256, 0, s>>>(cb, d_chunk_off, n_docs, d_tok_offsets);
        B2_CUDA(cudaMemcpyAsync(hd, d_total, 8, cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaMemcpyAsync(hd + 1, d_ctl, 8, cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaGetLastError());
        return B200BPE_OK;
    }

    // Pipelined batches: a second stream for the read-back, per-slice pinned results and events.
    cudaStream_t s_read = nullptr;
    uint64_t* h_slices = nullptr; uint32_t slices_cap = 0;
    std::vector<cudaEvent_t> slice_ev;   // four per slice: three timing events, one "slice done"
    b200bpe_status ensure_slices(uint32_t n_slices) {
        if (!s_read) B2_CUDA(cudaStreamCreateWithFlags(&s_read, cudaStreamNonBlocking));
        if (n_slices > slices_cap) {
            if (h_slices) cudaFreeHost(h_slices);
            h_slices = nullptr;
            B2_CUDA(cudaMallocHost(&h_slices, (size_t)n_slices * 16));
            slices_cap = n_slices;
        }
        while (slice_ev.size() < (size_t)n_slices * 4) {
            cudaEvent_t e = nullptr;
            B2_CUDA(cudaEventCreate(&e));
            slice_ev.push_back(e);
        }
        return B200BPE_OK;
    }

    b200bpe_status finish(uint64_t cap, uint64_t* n_tokens) {
        B2_CUDA(cudaStreamSynchronize(ctx->stream));
        float a = 0, b = 0;
        cudaEventElapsedTime(&a, ev[0], ev[1]);
        cudaEventElapsedTime(&b, ev[1], ev[2]);
        walk_ms = a; compact_ms = b;
        if ((uint32_t)(h_total[1] >> 32) != 0u) return B200BPE_ERR_LOOKBACK_TIMEOUT;
        if (n_tokens) *n_tokens = h_total[0];
        return h_total[0] > cap ? B200BPE_ERR_CAPACITY : B200BPE_OK;
    }
};

}  // namespace b200bpe

struct b200bpe_tok { b200bpe::Tokenizer* t; };

using namespace b200bpe;

extern "C" {

b200bpe_status b200bpe_tokenizer_create(b200bpe_ctx* c, const void* trie, size_t len, uint32_t chunk_size,
                                        b200bpe_tok** out) {
    b200bpe_tok_opts o;
    std::memset(&o, 0, sizeof(o));
    o.struct_size = sizeof(o);
    o.chunk_size = chunk_size;
    return b200bpe_tokenizer_create_ex(c, trie, len, &o, out);
}

static b200bpe_status noalloc_scratch_for(int device, unsigned char** out);

b200bpe_status b200bpe_tokenizer_create_ex(b200bpe_ctx* c, const void* trie, size_t len, const b200bpe_tok_opts* opts,
                                           b200bpe_tok** out) {
    if (!c || !trie || !out || !opts || opts->struct_size != sizeof(b200bpe_tok_opts)) return B200BPE_ERR_BAD_ARG;
    if (opts->layout > B200BPE_TRIE_HASH) return B200BPE_ERR_BAD_ARG;
    const uint32_t chunk_size = opts->chunk_size;
    uint32_t f[5];
    b200bpe_status r = b200bpe_trie_parse_header(trie, len, f);
    if (r) return r;
    const uint32_t version = f[0], node_count = f[1], edge_count = f[2], max_len = f[3];
    if (node_count == 0 || node_count >= T_MAX_NODES) return B200BPE_ERR_BAD_ARG;  // a node index must fit 22 bits
    const uint8_t* base = static_cast<const uint8_t*>(trie) + 28;
    // unpack nodes / edges (v3: trie.js:209-249; v2 is the 16-bit legacy layout, parse-only in the reference)
    std::vector<uint32_t> nodes((size_t)node_count * 3), esym(edge_count), etgt(edge_count);
    if (version == 3) {
        std::memcpy(nodes.data(), base, (size_t)node_count * 12);
        const uint8_t* eb = base + (size_t)node_count * 12;
        for (uint32_t e = 0; e < edge_count; e++) {
            esym[e] = eb[(size_t)e * 8];
            std::memcpy(&etgt[e], eb + (size_t)e * 8 + 4, 4);
        }
    } else {
        for (uint32_t i = 0; i < node_count; i++) {
            uint16_t h[3];
            std::memcpy(h, base + (size_t)i * 8, 6);
            nodes[i * 3] = h[0]; nodes[i * 3 + 1] = h[1]; nodes[i * 3 + 2] = h[2] == 0xFFFF ? INVALID_TOKEN : h[2];
        }
        const uint8_t* eb = base + (size_t)node_count * 8;
        for (uint32_t e = 0; e < edge_count; e++) {
            uint16_t h[2];
            std::memcpy(h, eb + (size_t)e * 4, 4);
            esym[e] = h[0] & 0xFF; etgt[e] = h[1];
        }
    }
    // Device numbering: a node that ends a token is numbered by its token id, the others follow
    // after the largest id, the root comes last.
    std::vector<uint32_t> dev_index(node_count, 0u);
    uint32_t root_index = 0, max_tok = 0;
    {
        bool any = false;
        for (uint32_t i = 1; i < node_count; i++) {
            const uint32_t tk = nodes[(size_t)i * 3 + 2];
            if (tk != INVALID_TOKEN) {
                if (tk >= T_MAX_NODES) { set_last_error("token id too large for the device trie"); return B200BPE_ERR_BAD_ARG; }
                max_tok = std::max(max_tok, tk);
                any = true;
            }
        }
        std::vector<uint8_t> seen((size_t)max_tok + 1, 0);
        uint32_t next_free = any ? max_tok + 1 : 1;   // (no token at all: index 0 stays unused, so that "index <= largest token id" holds for no node)
        for (uint32_t i = 1; i < node_count; i++) {
            const uint32_t tk = nodes[(size_t)i * 3 + 2];
            if (tk != INVALID_TOKEN) {
                if (seen[tk]) { set_last_error("two trie nodes carry the same token id"); return B200BPE_ERR_BAD_ARG; }
                seen[tk] = 1;
                dev_index[i] = tk;
            } else {
                dev_index[i] = next_free++;
            }
        }
        root_index = next_free;  // the root ends no token the walk could emit
        dev_index[0] = root_index;
        if (root_index >= T_MAX_NODES) { set_last_error("trie too large for the device layout"); return B200BPE_ERR_BAD_ARG; }
    }
    // the transitions, first of equal symbols only (the reference's binary search finds that one)
    struct Transition { uint32_t key, child; };
    std::vector<Transition> edges;
    edges.reserve(edge_count);
    for (uint32_t i = 0; i < node_count; i++) {
        const uint32_t fc = nodes[(size_t)i * 3], nc = nodes[(size_t)i * 3 + 1] & 0xFFFFu;  // tokenize.wgsl:102,115
        const size_t first = edges.size();
        for (uint32_t e = fc; e < fc + nc; e++) {
            if (e >= edge_count || etgt[e] >= node_count || etgt[e] == 0) return B200BPE_ERR_TRUNCATED_TRIE;
            const uint32_t key = (dev_index[i] << 8) | (esym[e] & 0xFFu);
            bool dup = false;
            for (size_t j = first; j < edges.size() && !dup; j++) dup = edges[j].key == key;
            if (!dup) edges.push_back({key, etgt[e]});
        }
    }
    auto is_token = [&](uint32_t node) { return nodes[(size_t)node * 3 + 2] != INVALID_TOKEN; };
    auto is_leaf = [&](uint32_t node) { return (nodes[(size_t)node * 3 + 1] & 0xFFFFu) == 0; };

    // Small tries: a cuckoo table for shared memory.  Try two sub-tables (at most 42 % full), then
    // three (at most 80 % full); the environment variable B200BPE_TRIE_LAYOUT=hash forces the
    // global table (for tests of that path).
    std::vector<uint32_t> cuckoo;
    int ck_d = 0;
    uint32_t ck_log2 = 0, ck_mul[3] = {1u, 1u, 1u};
    const bool want_cuckoo = opts->layout == B200BPE_TRIE_AUTO || opts->layout == B200BPE_TRIE_CUCKOO;
    if (want_cuckoo && root_index <= CK_INDEX) {
        uint64_t rng = 0x9E3779B97F4A7C15ull ^ ((uint64_t)edges.size() << 20);
        auto next_rand = [&]() { rng ^= rng << 13; rng ^= rng >> 7; rng ^= rng << 17; return rng; };
        for (int d = 2; d <= 3 && ck_d == 0; d++) {
            const double max_load = d == 2 ? 0.42 : 0.80;
            uint32_t k = CK_MIN_LOG2;
            while (k <= CK_MAX_LOG2 && (double)edges.size() > max_load * (double)((uint64_t)d << k)) k++;
            if (k > CK_MAX_LOG2) continue;
            const uint32_t shift = 24u - k, rmask = (1u << shift) - 1u, size = 1u << k;
            for (int attempt = 0; attempt < 64 && ck_d == 0; attempt++) {
                uint32_t mul[3];
                for (int j = 0; j < 3; j++) mul[j] = ((uint32_t)(next_rand() >> 20) | 1u) & 0xFFFFFFu;
                std::vector<uint32_t> tab((size_t)d << k, CK_EMPTY), owner((size_t)d << k, 0u);  // owner: edge index
                bool ok = true;
                for (uint32_t e = 0; e < edges.size() && ok; e++) {
                    uint32_t cur = e;
                    int avoid = -1;
                    ok = false;
                    for (int kick = 0; kick < 512; kick++) {
                        const uint32_t key = edges[cur].key;
                        int placed = -1;
                        for (int j = 0; j < d && placed < 0; j++) {
                            const uint32_t h = (key * mul[j]) & 0xFFFFFFu;
                            if (tab[(size_t)j * size + (h >> shift)] == CK_EMPTY) placed = j;
                        }
                        int j = placed;
                        if (j < 0) {  // all candidate slots taken: evict one, not the one this key just left
                            do { j = (int)(next_rand() % (uint64_t)d); } while (j == avoid);
                        }
                        const uint32_t h = (key * mul[j]) & 0xFFFFFFu;
                        const size_t slot = (size_t)j * size + (h >> shift);
                        uint32_t val = dev_index[edges[cur].child];
                        if (is_token(edges[cur].child)) val |= CK_HAS_TOKEN;
                        if (is_leaf(edges[cur].child)) val |= CK_LEAF;
                        const uint32_t evicted = owner[slot];
                        const bool was_empty = tab[slot] == CK_EMPTY;
                        tab[slot] = ((h & rmask) << 18) | val;
                        owner[slot] = cur;
                        if (was_empty) { ok = true; break; }
                        cur = evicted;
                        avoid = j;
                    }
                }
                if (ok) {
                    cuckoo.swap(tab);
                    ck_d = d; ck_log2 = k;
                    for (int j = 0; j < 3; j++) ck_mul[j] = mul[j];
                }
            }
        }
    }
    // Medium tries: the hybrid layout (see the head of this file).
    std::vector<uint32_t> hot;        // the shared-memory image
    std::vector<uint2> cold;
    std::vector<uint32_t> cold_bits;
    uint32_t hy_mul[2] = {1u, 1u}, cold_mask = 0, hot_entries = 0;
    bool hybrid = false;
    const bool want_hybrid = opts->layout == B200BPE_TRIE_HYBRID || (opts->layout == B200BPE_TRIE_AUTO && ck_d == 0);
    if (want_hybrid && ck_d == 0 && root_index < HY_MAX_INDEX) {
        auto pack = [&](uint32_t node) { return dev_index[node] | (is_leaf(node) ? HY_LEAF : 0u); };   // the cold flag is added at the end
        // children of a node: first of equal symbols only, as above
        auto for_children = [&](uint32_t node, auto&& fn) {
            const uint32_t fc = nodes[(size_t)node * 3], nc = nodes[(size_t)node * 3 + 1] & 0xFFFFu;
            uint32_t seen_sym[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (uint32_t e = fc; e < fc + nc; e++) {
                const uint32_t sy = esym[e] & 0xFFu;
                if ((seen_sym[sy >> 5] >> (sy & 31u)) & 1u) continue;
                seen_sym[sy >> 5] |= 1u << (sy & 31u);
                fn(sy, etgt[e]);
            }
        };
        // depth of every node and the smallest token id at or below it (iterative, cycle-safe: a node is visited once)
        std::vector<uint32_t> depth(node_count, 0xFFFFFFFFu), best(node_count, 0xFFFFFFFFu), order;
        order.reserve(node_count);
        depth[0] = 0;
        order.push_back(0);
        for (size_t i = 0; i < order.size(); i++)
            for_children(order[i], [&](uint32_t, uint32_t ch) {
                if (depth[ch] == 0xFFFFFFFFu) { depth[ch] = depth[order[i]] + 1; order.push_back(ch); }
            });
        for (size_t i = order.size(); i-- > 0;) {
            const uint32_t nd = order[i];
            if (is_token(nd)) best[nd] = std::min(best[nd], nodes[(size_t)nd * 3 + 2]);
            for_children(nd, [&](uint32_t, uint32_t ch) { best[nd] = std::min(best[nd], best[ch]); });
        }
        struct Cand { uint32_t key, value, rank, parent; };
        std::vector<Cand> root2, deep;
        std::vector<uint32_t> t1(256, T_MISS);
        for_children(0, [&](uint32_t b0, uint32_t c1) {
            t1[b0] = pack(c1);
            for_children(c1, [&](uint32_t b1, uint32_t c2) { root2.push_back({((HY_ROOT2 | b0) << 8) | b1, pack(c2), 0u, 0u}); });
        });
        for (uint32_t nd : order)
            if (depth[nd] >= 2)
                for_children(nd, [&](uint32_t b, uint32_t ch) { deep.push_back({(dev_index[nd] << 8) | b, pack(ch), best[ch], dev_index[nd]}); });
        // Whole parents go into shared memory, most used first (rank of a parent: the smallest token id at or
        // below it): a miss under a parent that is there completely needs no look at the global table, and
        // nearly every token ends with such a miss.
        for (Cand& d : deep) d.rank = 0u;
        {
            std::vector<uint32_t> rank_of(root_index + 1, 0xFFFFFFFFu);
            for (uint32_t nd : order) if (depth[nd] >= 2) rank_of[dev_index[nd]] = best[nd];
            for (Cand& d : deep) d.rank = rank_of[d.parent];
        }
        std::stable_sort(deep.begin(), deep.end(), [](const Cand& a, const Cand& b) { return a.rank != b.rank ? a.rank < b.rank : a.parent < b.parent; });
        const uint32_t buckets = 1u << HY_BUCKET_LOG2, rem_mask = (1u << HY_REM_SHIFT) - 1u;
        const size_t hot_cap = (size_t)(HY_MAX_LOAD * (double)HY_HOT_WORDS);
        uint64_t rng = 0xD1B54A32D192ED03ull ^ ((uint64_t)deep.size() << 17);
        auto next_rand = [&]() { rng ^= rng << 13; rng ^= rng >> 7; rng ^= rng << 17; return rng; };
        for (int attempt = 0; attempt < 64 && !hybrid && root2.size() * 2 <= hot_cap; attempt++) {
            uint32_t mul[2];
            for (int j = 0; j < 2; j++) mul[j] = ((uint32_t)(next_rand() >> 20) | 1u) & HY_KEY_MASK;
            std::vector<uint32_t> tab(HY_HOT_WORDS, 0xFFFFFFFFu);
            std::vector<Cand> owner(HY_HOT_WORDS);
            // A key is never placed where a look-up could take an empty entry (remainder all ones) for it.
            auto usable = [&](uint32_t key) {
                for (int j = 0; j < 2; j++) if ((((key * mul[j]) & HY_KEY_MASK) & rem_mask) == rem_mask) return false;
                return true;
            };
            // random-walk insertion; every write is logged so that a failed insertion can be undone
            struct Undo { size_t slot; uint32_t word; Cand who; };
            std::vector<Undo> undo;
            auto insert = [&](Cand cur) -> bool {
                undo.clear();
                for (int kick = 0; kick < 500; kick++) {
                    size_t free_slot = SIZE_MAX;
                    uint32_t hj[2];
                    for (int j = 0; j < 2; j++) {
                        hj[j] = (cur.key * mul[j]) & HY_KEY_MASK;
                        const size_t base = ((size_t)j * buckets + (hj[j] >> HY_REM_SHIFT)) * 2;
                        for (int e = 0; e < 2 && free_slot == SIZE_MAX; e++) if (tab[base + e] == 0xFFFFFFFFu) free_slot = base + e;
                    }
                    if (free_slot != SIZE_MAX) {
                        const int j = (int)(free_slot / ((size_t)buckets * 2));
                        undo.push_back({free_slot, tab[free_slot], owner[free_slot]});
                        tab[free_slot] = ((hj[j] & rem_mask) << 19) | cur.value;
                        owner[free_slot] = cur;
                        return true;
                    }
                    const int j = (int)(next_rand() & 1u);
                    const size_t slot = ((size_t)j * buckets + (hj[j] >> HY_REM_SHIFT)) * 2 + (size_t)(next_rand() & 1u);
                    const Cand evicted = owner[slot];
                    undo.push_back({slot, tab[slot], evicted});
                    tab[slot] = ((hj[j] & rem_mask) << 19) | cur.value;
                    owner[slot] = cur;
                    cur = evicted;
                }
                for (size_t i = undo.size(); i-- > 0;) { tab[undo[i].slot] = undo[i].word; owner[undo[i].slot] = undo[i].who; }
                return false;
            };
            bool ok = true;
            size_t placed = 0;
            for (const Cand& r : root2) { if (!usable(r.key) || !insert(r)) { ok = false; break; } placed++; }
            if (!ok) continue;
            // the deeper transitions, most used first, while there is room
            std::vector<uint8_t> in_hot(deep.size(), 0);
            for (size_t i = 0; i < deep.size();) {
                size_t j = i;
                while (j < deep.size() && deep[j].parent == deep[i].parent) j++;   // the children of one parent
                if (placed + (j - i) <= hot_cap) {
                    for (size_t k = i; k < j; k++) {
                        if (!usable(deep[k].key) || !insert(deep[k])) break;   // a failed insertion is undone; the parent then counts as cold
                        in_hot[k] = 1;
                        placed++;
                    }
                }
                i = j;
            }
            hot.assign(tab.begin(), tab.end());
            hot.insert(hot.end(), t1.begin(), t1.end());
            hot_entries = (uint32_t)placed;
            // the rest go to the global table, and their parents are marked
            size_t n_cold = 0;
            for (size_t i = 0; i < deep.size(); i++) n_cold += in_hot[i] ? 0 : 1;
            uint32_t clog = 4;
            while ((1ull << clog) < (uint64_t)n_cold * 2 + 16) clog++;
            cold.assign((size_t)1 << clog, make_uint2(T_EMPTY_KEY, 0u));
            cold_mask = (1u << clog) - 1;
            cold_bits.assign((root_index >> 5) + 2, 0u);
            for (size_t i = 0; i < deep.size(); i++) {
                if (in_hot[i]) continue;
                const uint32_t hh = deep[i].key * 0x9E3779B1u;
                uint32_t slot = (hh ^ (hh >> 15)) & cold_mask;
                while (cold[slot].x != T_EMPTY_KEY) slot = (slot + 1) & cold_mask;
                cold[slot] = make_uint2(deep[i].key, deep[i].value);
                cold_bits[deep[i].parent >> 5] |= 1u << (deep[i].parent & 31u);
            }
            // every stored value learns whether the node it names has cold children
            auto with_cold = [&](uint32_t value) {
                const uint32_t idx = value & HY_INDEX;
                return (idx != HY_INDEX && ((cold_bits[idx >> 5] >> (idx & 31u)) & 1u)) ? (value | HY_COLD) : value;
            };
            for (uint32_t& wv : hot) if (wv != 0xFFFFFFFFu) wv = with_cold(wv);
            for (uint2& c2 : cold) if (c2.x != T_EMPTY_KEY) c2.y = with_cold(c2.y);
            hy_mul[0] = mul[0]; hy_mul[1] = mul[1];
            hybrid = true;
        }
    }
    // Larger tries (or on request): open addressing in global memory.
    std::vector<uint2> trans;
    uint32_t tmask = 0;
    if (ck_d == 0 && !hybrid) {
        uint32_t tlog = 4;
        while ((1ull << tlog) < (uint64_t)edges.size() * 2 + 16) tlog++;
        trans.assign((size_t)1 << tlog, make_uint2(T_EMPTY_KEY, 0u));
        tmask = (1u << tlog) - 1;
        for (const Transition& e : edges) {
            const uint32_t h = e.key * 0x9E3779B1u;
            uint32_t slot = (h ^ (h >> 15)) & tmask;
            while (trans[slot].x != T_EMPTY_KEY) slot = (slot + 1) & tmask;
            uint32_t v = dev_index[e.child];
            if (is_token(e.child)) v |= T_HAS_TOKEN;
            if (is_leaf(e.child)) v |= T_LEAF;
            trans[slot] = make_uint2(e.key, v);
        }
    }
    B2_CUDA(cudaSetDevice(c->c.device));
    Tokenizer* t = new Tokenizer();
    t->ctx = &c->c;
    t->node_count = node_count; t->edge_count = edge_count; t->max_token_len = max_len;
    t->chunk = chunk_size ? chunk_size : std::max(512u, std::min(2048u, max_len * 8u));  // tokenizer.js:67-68
    t->trans_mask = tmask;
    t->root = root_index;
    t->ck_d = ck_d; t->ck_log2 = ck_log2;
    for (int j = 0; j < 3; j++) t->ck_mul[j] = ck_mul[j];
    t->hybrid = hybrid;
    t->hy_mul[0] = hy_mul[0]; t->hy_mul[1] = hy_mul[1];
    t->cold_mask = cold_mask;
    t->hot_entries = hot_entries;
    t->max_token = max_tok;
    if (opts->test_lookback_spins) {
        t->sc_max_spins = opts->test_lookback_spins;
        t->skip_first_tile = opts->test_lookback_spins < (1u << 20);
    }
    if (opts->batch_slice_bytes >= 1024) t->batch_slice_bytes = opts->batch_slice_bytes;
    if (opts->encode_slice_bytes >= 1024) t->encode_slice_bytes = opts->encode_slice_bytes;
    cudaStream_t s = c->c.stream;
    auto fail = [&](b200bpe_status st) { delete t; return st; };
#define B2_TRY(expr) if ((expr) != cudaSuccess) { set_last_error(std::string(#expr) + ": " + cudaGetErrorString(cudaGetLastError())); return fail(B200BPE_ERR_CUDA); }
    if (hybrid) {
        B2_TRY(cudaMalloc(&t->d_hot, hot.size() * 4));
        B2_TRY(cudaMemcpyAsync(t->d_hot, hot.data(), hot.size() * 4, cudaMemcpyHostToDevice, s));
        B2_TRY(cudaMalloc(&t->d_cold, cold.size() * 8));
        B2_TRY(cudaMemcpyAsync(t->d_cold, cold.data(), cold.size() * 8, cudaMemcpyHostToDevice, s));
        B2_TRY(cudaFuncSetAttribute(k_trie_walk_hybrid, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)HY_SMEM_BYTES));
    } else if (ck_d == 0) {
        B2_TRY(cudaMalloc(&t->d_trans, trans.size() * 8));
        B2_TRY(cudaMemcpyAsync(t->d_trans, trans.data(), trans.size() * 8, cudaMemcpyHostToDevice, s));
        B2_TRY(cudaFuncSetAttribute(k_trie_walk<TW_THREADS, TW_CACHE_LOG2, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    TW_SMEM_BYTES));
    } else {
        B2_TRY(cudaMalloc(&t->d_cuckoo, cuckoo.size() * 4));
        B2_TRY(cudaMemcpyAsync(t->d_cuckoo, cuckoo.data(), cuckoo.size() * 4, cudaMemcpyHostToDevice, s));
        if (ck_d == 2) {
            B2_TRY(cudaFuncSetAttribute(k_trie_walk<CK_THREADS, 0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)(cuckoo.size() * 4)));
        } else {
            B2_TRY(cudaFuncSetAttribute(k_trie_walk<CK_THREADS, 0, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)(cuckoo.size() * 4)));
        }
    }
    B2_TRY(cudaMalloc(&t->d_ctl, 16));
    B2_TRY(cudaMalloc(&t->d_total, 8));
    B2_TRY(cudaMallocHost(&t->h_total, 16));
    for (auto& e : t->ev) B2_TRY(cudaEventCreate(&e));
    {
        // Whatever the driver sets up lazily for the encode kernels and for the scratch array of
        // b200bpe_encode_device_noalloc is set up here, so that that entry point finds it all in place:
        // the compaction kernel is loaded (the walk kernels were, by the attribute calls above) and
        // the array's device address is looked up.
        cudaFuncAttributes fa;
        B2_TRY(cudaFuncGetAttributes(&fa, k_scan_compact));
        unsigned char* scratch = nullptr;
        if (noalloc_scratch_for(c->c.device, &scratch) != B200BPE_OK) return fail(B200BPE_ERR_CUDA);
    }
    t->trans_bytes = trans.size() * 8;
    B2_TRY(cudaStreamSynchronize(s));
#undef B2_TRY
    *out = new b200bpe_tok{t};
    return B200BPE_OK;
}

b200bpe_status b200bpe_tokenizer_info(b200bpe_tok* h, uint32_t* node_count, uint32_t* edge_count,
                                      uint32_t* max_token_len, uint32_t* chunk_size) {
    if (!h) return B200BPE_ERR_BAD_ARG;
    if (node_count) *node_count = h->t->node_count;
    if (edge_count) *edge_count = h->t->edge_count;
    if (max_token_len) *max_token_len = h->t->max_token_len;
    if (chunk_size) *chunk_size = h->t->chunk;
    return B200BPE_OK;
}

b200bpe_status b200bpe_tokenizer_layout(b200bpe_tok* h, uint32_t* sub_tables, uint32_t* log2_slots) {
    if (!h) return B200BPE_ERR_BAD_ARG;
    const Tokenizer* t = h->t;
    if (sub_tables) *sub_tables = t->hybrid ? 1u : (uint32_t)t->ck_d;
    if (log2_slots) {
        uint32_t k = t->ck_log2;
        if (t->hybrid) k = HY_BUCKET_LOG2 + 2;
        else if (t->ck_d == 0) for (k = 0; (1u << k) <= t->trans_mask; k++) {}
        *log2_slots = k;
    }
    return B200BPE_OK;
}

b200bpe_status b200bpe_encode_device(b200bpe_tok* h, const uint8_t* d_bytes, uint64_t n, uint32_t* d_tokens_out,
                                     uint64_t cap, uint64_t* n_tokens_out) {
    if (!h || (!d_bytes && n) || (!d_tokens_out && cap)) return B200BPE_ERR_BAD_ARG;
    Tokenizer* t = h->t;
    B2_CUDA(cudaSetDevice(t->ctx->device));
    if (n == 0) { if (n_tokens_out) *n_tokens_out = 0; return B200BPE_OK; }
    b200bpe_status r = t->launch(d_bytes, n, nullptr, 0, d_tokens_out, cap, nullptr);
    if (r) return r;
    return t->finish(cap, n_tokens_out);
}

b200bpe_status b200bpe_encode_batch_device(b200bpe_tok* h, const uint8_t* d_bytes, const uint64_t* d_doc_offsets,
                                           uint32_t n_docs, uint64_t n_bytes, uint32_t* d_tokens_out, uint64_t cap,
                                           uint64_t* d_tok_offsets_out, uint64_t* n_tokens_out) {
    if (!h || !d_doc_offsets || (!d_bytes && n_bytes) || (!d_tokens_out && cap)) return B200BPE_ERR_BAD_ARG;
    Tokenizer* t = h->t;
    B2_CUDA(cudaSetDevice(t->ctx->device));
    b200bpe_status r = t->launch(d_bytes, n_bytes, d_doc_offsets, n_docs, d_tokens_out, cap, d_tok_offsets_out);
    if (r) return r;
    return t->finish(cap, n_tokens_out);
}

// encodeBytes: upload, encode, read the total, then read back exactly total*4 bytes
// (tokenizer.js:226-233,312-334).
b200bpe_status b200bpe_encode(b200bpe_tok* h, const uint8_t* bytes, uint64_t n, uint32_t* tokens_out, uint64_t cap,
                              uint64_t* n_tokens_out) {
    if (!h || (!bytes && n) || !n_tokens_out) return B200BPE_ERR_BAD_ARG;
    Tokenizer* t = h->t;
    *n_tokens_out = 0;
    if (n == 0) return B200BPE_OK;
    B2_CUDA(cudaSetDevice(t->ctx->device));
    cudaStream_t s = t->ctx->stream;
    // Inputs beyond 8 GiB go through in chunk-aligned slices, as tokenizer.js:181-203 slices to its
    // buffer limit; the result is the same as one pass because slices end on chunk boundaries.
    const uint64_t slice = std::max<uint64_t>(1, t->encode_slice_bytes / t->chunk) * t->chunk;
    uint64_t done_tokens = 0;
    for (uint64_t off = 0; off < n; off += slice) {
        const uint64_t m = std::min(slice, n - off);
        b200bpe_status r;
        if ((r = t->ensure(&t->d_in, &t->in_cap, m + 16))) return r;
        if ((r = t->ensure(&t->d_out, &t->out_cap, m))) return r;  // worst case: one token per byte
        B2_CUDA(cudaMemcpyAsync(t->d_in, bytes + off, m, cudaMemcpyHostToDevice, s));
        if ((r = t->launch(t->d_in, m, nullptr, 0, t->d_out, t->out_cap, nullptr))) return r;
        uint64_t got = 0;
        if ((r = t->finish(t->out_cap, &got))) return r;
        if (done_tokens + got > cap || !tokens_out) { *n_tokens_out = done_tokens + got; return B200BPE_ERR_CAPACITY; }
        B2_CUDA(cudaMemcpyAsync(tokens_out + done_tokens, t->d_out, got * 4, cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaStreamSynchronize(s));
        done_tokens += got;
    }
    *n_tokens_out = done_tokens;
    return B200BPE_OK;
}

b200bpe_status b200bpe_encode_batch(b200bpe_tok* h, const uint8_t* bytes, const uint64_t* doc_offsets, uint32_t n_docs,
                                    uint32_t* tokens_out, uint64_t cap, uint64_t* tok_offsets_out) {
    if (!h || !doc_offsets || !tok_offsets_out) return B200BPE_ERR_BAD_ARG;
    Tokenizer* t = h->t;
    B2_CUDA(cudaSetDevice(t->ctx->device));
    cudaStream_t s = t->ctx->stream;
    const uint64_t n = doc_offsets[n_docs] - doc_offsets[0];
    for (uint32_t d = 0; d < n_docs; d++) if (doc_offsets[d + 1] < doc_offsets[d]) return B200BPE_ERR_BAD_ARG;
    // Slices of whole documents, about BATCH_SLICE_BYTES each: the upload and the kernels of one slice
    // run while the tokens of the slices before it travel back (documents are independent, so the
    // result does not depend on the cut).
    std::vector<uint32_t> cut{0};
    const uint64_t slice_bytes = t->batch_slice_bytes;
    if (n > 2 * slice_bytes) {
        uint64_t start = doc_offsets[0];
        for (uint32_t d = 1; d < n_docs; d++)
            if (doc_offsets[d] - start >= slice_bytes) { cut.push_back(d); start = doc_offsets[d]; }
    }
    cut.push_back(n_docs);
    const uint32_t n_slices = (uint32_t)cut.size() - 1;
    b200bpe_status r;
    if ((r = t->ensure(&t->d_in, &t->in_cap, n + 16))) return r;
    if ((r = t->ensure(&t->d_out, &t->out_cap, std::max<uint64_t>(1, n)))) return r;
    if ((r = t->ensure(&t->d_doc_off, &t->doc_off_cap, (uint64_t)n_docs + n_slices + 1))) return r;
    if ((r = t->ensure(&t->d_tok_off, &t->tok_off_cap, (uint64_t)n_docs + n_slices + 1))) return r;
    // document offsets relative to the first byte of their slice, one run of (docs + 1) entries per slice
    std::vector<uint64_t> rel((size_t)n_docs + n_slices);
    uint64_t max_chunks = 1;
    uint32_t max_docs = 1;
    for (uint32_t i = 0; i < n_slices; i++) {
        const uint32_t d0 = cut[i], d1 = cut[i + 1];
        for (uint32_t d = d0; d <= d1; d++) rel[(size_t)d + i] = doc_offsets[d] - doc_offsets[d0];
        max_chunks = std::max<uint64_t>(max_chunks, (doc_offsets[d1] - doc_offsets[d0] + t->chunk - 1) / t->chunk + (d1 - d0));
        max_docs = std::max(max_docs, d1 - d0);
    }
    // every buffer a slice needs exists before the first one starts (growing one synchronises the stream)
    if ((r = t->ensure_work(max_chunks))) return r;
    if ((r = t->ensure(&t->d_chunk_base, &t->chunk_base_cap, (uint64_t)max_docs + 1))) return r;
    if ((r = t->ensure_slices(n_slices))) return r;
    B2_CUDA(cudaMemcpyAsync(t->d_doc_off, rel.data(), rel.size() * 8, cudaMemcpyHostToDevice, s));
    for (uint32_t i = 0; i < n_slices; i++) {
        const uint32_t d0 = cut[i], d1 = cut[i + 1];
        const uint64_t b0 = doc_offsets[d0] - doc_offsets[0], nb = doc_offsets[d1] - doc_offsets[d0];
        if (nb) B2_CUDA(cudaMemcpyAsync(t->d_in + b0, bytes + doc_offsets[d0], nb, cudaMemcpyHostToDevice, s));
        if ((r = t->launch(t->d_in + b0, nb, t->d_doc_off + d0 + i, d1 - d0, t->d_out + b0, std::max<uint64_t>(1, nb),
                           t->d_tok_off + d0 + i, t->h_slices + 2 * (size_t)i, &t->slice_ev[4 * (size_t)i])))
            return r;
        B2_CUDA(cudaEventRecord(t->slice_ev[4 * (size_t)i + 3], s));
    }
    // read-back on the second stream, slice by slice, as each one finishes
    uint64_t acc = 0;
    b200bpe_status result = B200BPE_OK;
    std::vector<uint64_t> base(n_slices, 0);
    t->walk_ms = t->compact_ms = 0;
    for (uint32_t i = 0; i < n_slices; i++) {
        const uint32_t d0 = cut[i], d1 = cut[i + 1];
        const uint64_t b0 = doc_offsets[d0] - doc_offsets[0];
        B2_CUDA(cudaEventSynchronize(t->slice_ev[4 * (size_t)i + 3]));
        float a = 0, b = 0;
        cudaEventElapsedTime(&a, t->slice_ev[4 * (size_t)i], t->slice_ev[4 * (size_t)i + 1]);
        cudaEventElapsedTime(&b, t->slice_ev[4 * (size_t)i + 1], t->slice_ev[4 * (size_t)i + 2]);
        t->walk_ms += a; t->compact_ms += b;
        const uint64_t got = t->h_slices[2 * (size_t)i];
        if ((uint32_t)(t->h_slices[2 * (size_t)i + 1] >> 32) != 0u) result = B200BPE_ERR_LOOKBACK_TIMEOUT;
        base[i] = acc;
        if (result == B200BPE_OK && (acc + got > cap || (!tokens_out && got))) result = B200BPE_ERR_CAPACITY;
        if (result == B200BPE_OK) {
            if (got) B2_CUDA(cudaMemcpyAsync(tokens_out + acc, t->d_out + b0, got * 4, cudaMemcpyDeviceToHost, t->s_read));
            B2_CUDA(cudaMemcpyAsync(tok_offsets_out + d0, t->d_tok_off + d0 + i, (size_t)(d1 - d0) * 8, cudaMemcpyDeviceToHost, t->s_read));
        }
        acc += got;
    }
    B2_CUDA(cudaStreamSynchronize(t->s_read));
    B2_CUDA(cudaStreamSynchronize(s));
    if (result != B200BPE_OK) return result;
    // token offsets were relative to their slice
    for (uint32_t i = 1; i < n_slices; i++)
        for (uint32_t d = cut[i]; d < cut[i + 1]; d++) tok_offsets_out[d] += base[i];
    tok_offsets_out[n_docs] = acc;
    return B200BPE_OK;
}

// ── encoding without any allocation ──
// Some callers may not allocate device memory at the moment they encode: a real-time or
// fault-tolerant loop that must not hit the allocator's locks or its out-of-memory path, code that
// runs while another library owns all remaining memory, a signal-safe or hook context.  For them
// the work buffers of one encode (per-chunk token staging, counts, offsets, look-back descriptors)
// live in one file-scope device array instead of the tokenizer's growable pool.  The array is part
// of the library image: every GPU that loads the library holds it until the process exits.
constexpr uint64_t NOALLOC_MAX_BYTES = 1ull << 20;   // largest input of one call
constexpr uint64_t NOALLOC_MAX_CHUNKS = 8192;        // largest number of chunks of one call
constexpr uint64_t NA_ALIGN = 256;
constexpr uint64_t na_up(uint64_t x) { return (x + NA_ALIGN - 1) / NA_ALIGN * NA_ALIGN; }
// Staging holds a row of chunk_size words per chunk.  A walk writes at most one word per input byte
// (the cuckoo and hash walks in whole 8-word sectors), so a call uses at most n + 8 words of it; the
// array reserves twice the largest input, and the second half is never touched.
constexpr uint64_t NA_OFF_STAGING = 0;
constexpr uint64_t NA_STAGING_BYTES = na_up((NOALLOC_MAX_BYTES + NOALLOC_MAX_BYTES) * 4);
constexpr uint64_t NA_OFF_COUNTS = NA_OFF_STAGING + NA_STAGING_BYTES;
constexpr uint64_t NA_OFF_CHUNK_OFF = NA_OFF_COUNTS + na_up((NOALLOC_MAX_CHUNKS + 1) * 4);
constexpr uint64_t NA_OFF_DESC = NA_OFF_CHUNK_OFF + na_up((NOALLOC_MAX_CHUNKS + 1) * 8);
constexpr uint64_t NA_OFF_CTL = NA_OFF_DESC + na_up((NOALLOC_MAX_CHUNKS / SC_THREADS + 2) * 8);
constexpr uint64_t NA_OFF_TOTAL = NA_OFF_CTL + NA_ALIGN;
constexpr uint64_t NOALLOC_SCRATCH_BYTES = NA_OFF_TOTAL + NA_ALIGN;

static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not an address a kernel can
// use; the device address is asked for once per device, with that device current.
static unsigned char* g_noalloc_ptr[64] = {};
static std::mutex g_noalloc_mutex;

static b200bpe_status noalloc_scratch_for(int device, unsigned char** out) {
    if (device < 0 || device >= 64) return B200BPE_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[device]) {
        void* p = nullptr;
        B2_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        g_noalloc_ptr[device] = static_cast<unsigned char*>(p);
    }
    *out = g_noalloc_ptr[device];
    return B200BPE_OK;
}

b200bpe_status b200bpe_encode_device_noalloc(b200bpe_tok* h, const uint8_t* d_bytes, uint64_t n, uint32_t* d_tokens_out,
                                             uint64_t cap, uint64_t* n_tokens_out) {
    if (!h || (!d_bytes && n) || (!d_tokens_out && cap) || !n_tokens_out) return B200BPE_ERR_BAD_ARG;
    Tokenizer* t = h->t;
    *n_tokens_out = 0;
    if (n == 0) return B200BPE_OK;
    const uint64_t chunks = (n + t->chunk - 1) / t->chunk;
    if (n > NOALLOC_MAX_BYTES || chunks > NOALLOC_MAX_CHUNKS) {
        set_last_error("b200bpe_encode_device_noalloc: input of " + std::to_string(n) + " bytes in " + std::to_string(chunks) +
                       " chunks exceeds the built-in scratch (at most " + std::to_string(NOALLOC_MAX_BYTES) + " bytes and " +
                       std::to_string(NOALLOC_MAX_CHUNKS) + " chunks per call)");
        return B200BPE_ERR_CAPACITY;
    }
    B2_CUDA(cudaSetDevice(t->ctx->device));
    unsigned char* base = nullptr;
    b200bpe_status r = noalloc_scratch_for(t->ctx->device, &base);
    if (r) return r;
    cudaStream_t s = t->ctx->stream;
    uint32_t* staging = reinterpret_cast<uint32_t*>(base + NA_OFF_STAGING);
    uint32_t* counts = reinterpret_cast<uint32_t*>(base + NA_OFF_COUNTS);
    uint64_t* chunk_off = reinterpret_cast<uint64_t*>(base + NA_OFF_CHUNK_OFF);
    unsigned long long* desc = reinterpret_cast<unsigned long long*>(base + NA_OFF_DESC);
    uint32_t* ctl = reinterpret_cast<uint32_t*>(base + NA_OFF_CTL);
    uint64_t* total = reinterpret_cast<uint64_t*>(base + NA_OFF_TOTAL);
    // The array keeps whatever the last call left: the look-back descriptors, the tile ticket and
    // the error flag must start at zero; everything else is written before it is read.
    const uint64_t ntiles = chunks / SC_THREADS + 2;
    B2_CUDA(cudaMemsetAsync(desc, 0, ntiles * 8, s));
    B2_CUDA(cudaMemsetAsync(ctl, 0, 16, s));
    t->walk(d_bytes, n, nullptr, nullptr, 0, chunks, staging, counts, ctl + 2);
    const int grid_c = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)t->ctx->sm_count * 8, ntiles));
    k_scan_compact<<<grid_c, SC_THREADS, 0, s>>>(staging, counts, t->chunk, nullptr, 0, chunks, desc, ctl, chunk_off,
                                                d_tokens_out, cap, total, t->sc_max_spins);
    B2_CUDA(cudaGetLastError());
    B2_CUDA(cudaMemcpyAsync(t->h_total, total, 8, cudaMemcpyDeviceToHost, s));
    B2_CUDA(cudaMemcpyAsync(t->h_total + 1, ctl, 8, cudaMemcpyDeviceToHost, s));
    B2_CUDA(cudaStreamSynchronize(s));
    if ((uint32_t)(t->h_total[1] >> 32) != 0u) return B200BPE_ERR_LOOKBACK_TIMEOUT;
    *n_tokens_out = t->h_total[0];
    return t->h_total[0] > cap ? B200BPE_ERR_CAPACITY : B200BPE_OK;
}

b200bpe_status b200bpe_tokenizer_last_ms(b200bpe_tok* h, double* walk_ms, double* compact_ms) {
    if (!h) return B200BPE_ERR_BAD_ARG;
    if (walk_ms) *walk_ms = h->t->walk_ms;
    if (compact_ms) *compact_ms = h->t->compact_ms;
    return B200BPE_OK;
}

void b200bpe_tokenizer_destroy(b200bpe_tok* h) {
    if (!h) return;
    delete h->t;
    delete h;
}

}  // extern "C"
