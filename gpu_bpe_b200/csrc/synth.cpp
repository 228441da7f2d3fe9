// Seeded synthetic corpora for tests and benchmarks (host code, built into libb200bpe_synth.so).
// They stand in for real text: per-script Zipf-distributed lexicons with the byte mix, line
// lengths and document lengths of the benchmark configurations.  Every code point used is
// already NFC and has had the same General_Category since long before Unicode 15, so the
// pre-tokeniser's classes do not depend on the Unicode version.
//
// The text is made in independent 1 MiB blocks, block k seeded by (seed, k), so generation is
// parallel and the bytes depend only on (kind, seed, n_bytes).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

namespace {

struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed) {}
    uint64_t next() {  // splitmix64
        uint64_t z = (s += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    double uni() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }
    uint32_t below(uint32_t n) { return (uint32_t)(((next() >> 32) * (uint64_t)n) >> 32); }
    double normal() {
        const double u1 = std::max(uni(), 1e-300), u2 = uni();
        return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2);
    }
};

void put_utf8(std::string& o, uint32_t cp) {
    if (cp <= 0x7F) o.push_back((char)cp);
    else if (cp <= 0x7FF) { o.push_back((char)(0xC0 | (cp >> 6))); o.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp <= 0xFFFF) {
        o.push_back((char)(0xE0 | (cp >> 12))); o.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
        o.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
        o.push_back((char)(0xF0 | (cp >> 18))); o.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
        o.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); o.push_back((char)(0x80 | (cp & 0x3F)));
    }
}

// Word lengths: geometric, clipped to [2, 12], mean about 6.
uint32_t word_len(Rng& r) {
    uint32_t l = 2;
    while (l < 12 && r.uni() < 0.8) l++;
    return l;
}

struct Lexicon {
    std::vector<std::string> words;
    std::vector<double> cdf;  // Zipf(s) over ranks
    void build_cdf(double s) {
        cdf.resize(words.size());
        double acc = 0;
        for (size_t i = 0; i < words.size(); i++) { acc += 1.0 / std::pow((double)(i + 1), s); cdf[i] = acc; }
        for (auto& c : cdf) c /= acc;
    }
    const std::string& draw(Rng& r) const {
        const double u = r.uni();
        size_t i = std::lower_bound(cdf.begin(), cdf.end(), u) - cdf.begin();
        if (i >= words.size()) i = words.size() - 1;
        return words[i];
    }
};

// Accented lowercase letters of Latin-1 (precomposed, two UTF-8 bytes each).
const uint32_t kAccented[] = {0xE0, 0xE1, 0xE2, 0xE4, 0xE7, 0xE8, 0xE9, 0xEA, 0xEB, 0xED, 0xEE, 0xF1, 0xF3, 0xF4, 0xF6, 0xFA, 0xFC};

Lexicon make_latin(uint64_t seed, size_t n, double zipf, double accented) {
    Lexicon L;
    Rng r(seed);
    L.words.reserve(n);
    for (size_t i = 0; i < n; i++) {
        std::string w;
        const uint32_t len = word_len(r);
        for (uint32_t k = 0; k < len; k++) {
            if (accented > 0 && r.uni() < accented) put_utf8(w, kAccented[r.below(sizeof(kAccented) / 4)]);
            else w.push_back((char)('a' + r.below(26)));
        }
        L.words.push_back(w);
    }
    L.build_cdf(zipf);
    return L;
}

Lexicon make_cyrillic(uint64_t seed, size_t n, double zipf) {
    Lexicon L;
    Rng r(seed);
    for (size_t i = 0; i < n; i++) {
        std::string w;
        const uint32_t len = word_len(r);
        for (uint32_t k = 0; k < len; k++) put_utf8(w, 0x430 + r.below(32));
        L.words.push_back(w);
    }
    L.build_cdf(zipf);
    return L;
}

Lexicon make_cjk(uint64_t seed, size_t n, double zipf) {
    Lexicon L;
    Rng r(seed);
    for (size_t i = 0; i < n; i++) {
        std::string w;
        const uint32_t len = 1 + r.below(4);
        for (uint32_t k = 0; k < len; k++) put_utf8(w, 0x4E00 + r.below(0x5000));
        L.words.push_back(w);
    }
    L.build_cdf(zipf);
    return L;
}

const char kPunct[] = {',', '.', '!', '?', '\'', '-'};
const char kB64[] = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";

void put_number(std::string& o, Rng& r) {
    const uint32_t d = 1 + r.below(4);
    for (uint32_t k = 0; k < d; k++) o.push_back((char)('0' + r.below(10)));
}

struct Plan {
    int kind;
    Lexicon latin, cyr, cjk;
};

// One block of exactly `len` bytes.
void make_block(const Plan& P, uint64_t seed, uint64_t block, uint8_t* out, size_t len) {
    Rng r(seed * 0x9E3779B97F4A7C15ull + block * 0xD1B54A32D192ED03ull + 12345);
    std::string buf;
    buf.reserve(len + 64);
    size_t line_left = 0;
    auto new_line_budget = [&]() -> size_t {
        if (P.kind == 1) return 80;
        // lognormal, mean 120 bytes: exp(mu + sigma^2/2) = 120 with sigma = 0.6
        const double v = std::exp(4.6075 + 0.6 * r.normal());
        return (size_t)std::max(8.0, std::min(4000.0, v));
    };
    line_left = new_line_budget();
    std::string tok;
    while (buf.size() + 80 < len) {
        tok.clear();
        bool spaced = true;
        const double u = r.uni();
        if (P.kind == 1) {
            if (u < 0.05) put_number(tok, r);
            else if (u < 0.08) { tok.push_back(kPunct[r.below(6)]); spaced = false; }
            else tok = P.latin.draw(r);
        } else {
            // token-level odds tuned so that the BYTE shares come out near 70 % Latin, 12 % Cyrillic,
            // 10 % CJK, 8 % digits / punctuation / emoji
            if (P.kind == 5 && u < 0.006) {
                const uint32_t l = 16 + r.below(49);
                for (uint32_t k = 0; k < l; k++) tok.push_back(kB64[r.below(64)]);
            } else if (u < 0.70) tok = P.latin.draw(r);
            else if (u < 0.765) tok = P.cyr.draw(r);
            else if (u < 0.84) { tok = P.cjk.draw(r); spaced = false; }
            else if (u < 0.90) put_number(tok, r);
            else if (u < 0.98) { tok.push_back(kPunct[r.below(6)]); spaced = false; }
            else { put_utf8(tok, 0x1F600 + r.below(0x50)); }
        }
        const size_t need = tok.size() + 1;
        if (line_left < need && !buf.empty() && buf.back() != '\n') {
            buf.push_back('\n');
            line_left = new_line_budget();
        } else if (spaced && !buf.empty() && buf.back() != '\n') {
            buf.push_back(' ');
            line_left = line_left > 1 ? line_left - 1 : 0;
        }
        buf += tok;
        line_left = line_left > tok.size() ? line_left - tok.size() : 0;
    }
    // pad to the exact block length with a plain ASCII word and a newline
    if (buf.size() < len) {
        if (!buf.empty() && buf.back() != '\n' && buf.size() + 1 < len) buf.push_back(' ');
        while (buf.size() + 1 < len) buf.push_back((char)('a' + r.below(26)));
        if (buf.size() < len) buf.push_back('\n');
    }
    std::memcpy(out, buf.data(), len);
}

}  // namespace

extern "C" {

// kind 1: ASCII (20,000-word lexicon, Zipf 1.1, numbers and punctuation, newline about every 80 bytes).
// kind 2: UTF-8 mix (50,000 words per script, Zipf 1.1, lognormal lines).
// kind 5: kind 2 with Zipf 1.0 over 500,000 words plus random base64-like strings.
// Bytes [offset, offset + len) of the corpus of n_bytes bytes: the same bytes as the whole corpus
// holds there (blocks are independent), so every rank of a sharded job can make just its span.
int b200bpe_synth_corpus_range(int kind, uint64_t seed, uint64_t n_bytes, uint64_t offset, uint64_t len, uint8_t* out,
                               int threads) {
    if ((!out && len) || (kind != 1 && kind != 2 && kind != 5) || offset > n_bytes || len > n_bytes - offset) return 1;
    if (len == 0) return 0;
    Plan P;
    P.kind = kind;
    if (kind == 1) {
        P.latin = make_latin(seed ^ 0x11, 20000, 1.1, 0.0);
    } else {
        const size_t nwords = kind == 5 ? 500000 : 50000;
        const double z = kind == 5 ? 1.0 : 1.1;
        P.latin = make_latin(seed ^ 0x11, nwords, z, 0.08);
        P.cyr = make_cyrillic(seed ^ 0x22, nwords, z);
        P.cjk = make_cjk(seed ^ 0x33, nwords, z);
    }
    const uint64_t B = 1ull << 20;
    const uint64_t b0 = offset / B, b1 = (offset + len + B - 1) / B;   // blocks [b0, b1)
    const int T = std::max(1, std::min<int>(threads, (int)(b1 - b0)));
    std::vector<std::thread> pool;
    for (int t = 0; t < T; t++) {
        pool.emplace_back([&, t]() {
            std::vector<uint8_t> tmp;
            for (uint64_t b = b0 + t; b < b1; b += T) {
                const uint64_t lo = b * B, blen = std::min(B, n_bytes - lo);
                const uint64_t from = std::max(lo, offset), to = std::min(lo + blen, offset + len);
                if (from == lo && to == lo + blen) {
                    make_block(P, seed, b, out + (lo - offset), (size_t)blen);
                } else {
                    tmp.resize(blen);
                    make_block(P, seed, b, tmp.data(), (size_t)blen);
                    std::memcpy(out + (from - offset), tmp.data() + (from - lo), (size_t)(to - from));
                }
            }
        });
    }
    for (auto& th : pool) th.join();
    return 0;
}

int b200bpe_synth_corpus(int kind, uint64_t seed, uint64_t n_bytes, uint8_t* out, int threads) {
    return b200bpe_synth_corpus_range(kind, seed, n_bytes, 0, n_bytes, out, threads);
}

// Cut n_bytes into n_docs documents with lognormal lengths (sigma given, mean n_bytes / n_docs).
// offsets_out has n_docs + 1 entries, offsets_out[n_docs] == n_bytes.
int b200bpe_synth_doc_offsets(uint64_t seed, uint64_t n_bytes, uint32_t n_docs, double sigma, uint64_t* offsets_out) {
    if (!offsets_out || n_docs == 0) return 1;
    Rng r(seed ^ 0xD0C5);
    std::vector<double> len(n_docs);
    double sum = 0;
    for (uint32_t i = 0; i < n_docs; i++) { len[i] = std::exp(sigma * r.normal()); sum += len[i]; }
    double acc = 0;
    offsets_out[0] = 0;
    for (uint32_t i = 0; i < n_docs; i++) {
        acc += len[i];
        uint64_t o = (uint64_t)std::llround(acc / sum * (double)n_bytes);
        o = std::min<uint64_t>(n_bytes, std::max<uint64_t>(o, offsets_out[i]));
        offsets_out[i + 1] = o;
    }
    offsets_out[n_docs] = n_bytes;
    return 0;
}

}  // extern "C"
