// Host pre-tokeniser: GPT-4-style word starts over code-point classes.
// Restates PreTokenizer.preTokenizeBytes (src/wasm/pre_tokenizer.mjs:459-509 of the reference):
// decode UTF-8 (:518-554), classify (:126-134), find boundaries (:226-292), map code-point starts
// to the first byte (:499-506).  The reference first NFC-normalises with a closed WASM library
// (:465); this function expects NFC input and leaves the bytes as they are.
#include <cstdint>
#include <cstring>
#include <vector>

#include "../../include/b200bpe.h"

namespace {

#include "unicode_classes.inc"

enum : uint8_t { LETTER = 0, DIGIT = 1, WHITESPACE = 2, PUNCT = 3, SYMBOL = 4, NEWLINE = 5, OTHER = 6 };

struct ClassTable {
    uint8_t low[0x3000];  // direct table for the dense low planes
    ClassTable() {
        for (const auto& r : kClassRanges)
            for (uint32_t cp = r[0]; cp <= r[1] && cp < 0x3000; cp++) low[cp] = (uint8_t)r[2];
    }
    uint8_t get(uint32_t cp) const {
        if (cp < 0x3000) return low[cp];
        size_t lo = 0, hi = sizeof(kClassRanges) / sizeof(kClassRanges[0]);
        while (hi - lo > 1) {
            const size_t mid = (lo + hi) / 2;
            if (kClassRanges[mid][0] <= cp) lo = mid; else hi = mid;
        }
        return cp <= kClassRanges[lo][1] ? (uint8_t)kClassRanges[lo][2] : (uint8_t)OTHER;
    }
};

const ClassTable& table() {
    static const ClassTable t;
    return t;
}

inline bool punct_or_symbol(uint8_t c) { return c == PUNCT || c == SYMBOL; }

inline bool transition(uint8_t p, uint8_t c) {  // pre_tokenizer.mjs:175-189
    return (p == LETTER && c == DIGIT) || (p == DIGIT && c == LETTER) || (p == LETTER && punct_or_symbol(c)) ||
           (punct_or_symbol(p) && c == LETTER) || (punct_or_symbol(p) && c == DIGIT) ||
           (p == DIGIT && punct_or_symbol(c));
}

inline bool in_set(uint32_t cp, const char* s) {
    for (; *s; s++) if (cp == (uint32_t)(uint8_t)*s) return true;
    return false;
}

// pre_tokenizer.mjs:83-110 — code points consumed by 's 't 'm 'd 're 've 'll at apostrophe i, or 0.
size_t match_contraction(const std::vector<uint32_t>& cp, const std::vector<uint8_t>& cls, size_t i) {
    const size_t n = cp.size();
    if (i + 1 >= n) return 0;
    const uint32_t nx = cp[i + 1];
    if (in_set(nx, "sStTmMdD") && (i + 2 >= n || cls[i + 2] != LETTER)) return 2;
    if (i + 2 < n) {
        const uint32_t nn = cp[i + 2];
        const bool after = i + 3 >= n || cls[i + 3] != LETTER;
        if (after && ((in_set(nx, "rR") && in_set(nn, "eE")) || (in_set(nx, "vV") && in_set(nn, "eE")) ||
                      (in_set(nx, "lL") && in_set(nn, "lL"))))
            return 3;
    }
    return 0;
}

}  // namespace

extern "C" b200bpe_status b200bpe_pretokenize(const uint8_t* bytes, uint64_t n, uint8_t* word_starts_out) {
    if ((!bytes || !word_starts_out) && n) return B200BPE_ERR_BAD_ARG;
    if (n == 0) return B200BPE_OK;
    const ClassTable& T = table();
    // decode (pre_tokenizer.mjs:518-554; lengths are taken from the lead byte, reads are clamped)
    std::vector<uint32_t> cp;
    std::vector<uint64_t> at;
    cp.reserve(n);
    at.reserve(n);
    auto b = [&](uint64_t i) -> uint32_t { return i < n ? bytes[i] : 0u; };
    for (uint64_t i = 0; i < n;) {
        const uint32_t c = bytes[i];
        uint32_t v;
        uint64_t size;
        if (c < 0x80) { v = c; size = 1; }
        else if ((c & 0xE0) == 0xC0) { v = (c & 0x1F) << 6 | (b(i + 1) & 0x3F); size = 2; }
        else if ((c & 0xF0) == 0xE0) { v = (c & 0x0F) << 12 | (b(i + 1) & 0x3F) << 6 | (b(i + 2) & 0x3F); size = 3; }
        else { v = (c & 0x07) << 18 | (b(i + 1) & 0x3F) << 12 | (b(i + 2) & 0x3F) << 6 | (b(i + 3) & 0x3F); size = 4; }
        cp.push_back(v);
        at.push_back(i);
        i += size;
    }
    const size_t m = cp.size();
    std::vector<uint8_t> cls(m);
    for (size_t i = 0; i < m; i++) cls[i] = cp[i] <= 0x10FFFF ? T.get(cp[i]) : (uint8_t)OTHER;
    std::memset(word_starts_out, 0, n);
    word_starts_out[0] = 1;
    size_t run_start = 0;  // first index of the current run of DIGIT-class code points
    for (size_t i = 1; i < m;) {
        const uint8_t p = cls[i - 1], c = cls[i];
        if (c == DIGIT && p != DIGIT) run_start = i;
        if (c == NEWLINE || p == NEWLINE) { word_starts_out[at[i]] = 1; i++; continue; }
        if (c == WHITESPACE) { if (p != WHITESPACE) word_starts_out[at[i]] = 1; i++; continue; }
        if (p == WHITESPACE) { i++; continue; }
        if (p == LETTER && (cp[i] == 0x27 || cp[i] == 0x2019)) {
            const size_t k = match_contraction(cp, cls, i);
            if (k > 0) {
                // the skipped code points may open a digit run only if they are digits, which the
                // suffix letters never are; keep run_start consistent for what follows
                i += k;
                if (i < m && cls[i] == DIGIT && cls[i - 1] == DIGIT) {
                    size_t rs = i - 1;
                    while (rs > 0 && cls[rs - 1] == DIGIT) rs--;
                    run_start = rs;
                }
                continue;
            }
        }
        if (transition(p, c)) { word_starts_out[at[i]] = 1; i++; continue; }
        if (c == DIGIT && p == DIGIT) {
            // every third digit counted from the start of the class run (pre_tokenizer.mjs:198-204)
            if ((i - run_start) % 3 == 0) word_starts_out[at[i]] = 1;
            i++;
            continue;
        }
        i++;
    }
    return B200BPE_OK;
}
