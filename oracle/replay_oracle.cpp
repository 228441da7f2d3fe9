// CPU oracle for the merge-replay encoder.  TEST INFRASTRUCTURE ONLY: only tests/ and the smoke
// check may load it.
//
// Restates TokenizerManager.encode of toprakdeviren/gpu-bpe (src/ui/tokenizer-manager.js:13-61):
// the text's UTF-8 bytes become one token each (:40-41); then every merge rule [a, b, newId] is
// applied in the order it was learned (:45), each as one left-to-right pass over the whole token
// list that replaces a matching adjacent pair and steps over both tokens (:49-58).  There are no
// word boundaries on this path, and with a == b a run of k equal tokens pairs up from the left:
// floor(k / 2) new tokens, then the odd one out.  No merges → the bytes are the tokens (:21-25).
//
// PARITY UNPINNED by the reference (no vectors, cannot run here); pinned by the hand-derived cases
// in tests/golden/known_answers.json ("replay").
#include <cstdint>
#include <vector>

extern "C" uint64_t oracle_replay_encode(const uint8_t* bytes, uint64_t n, const uint32_t* merges, uint32_t n_merges,
                                         uint32_t* tokens_out, uint64_t cap) {
    std::vector<uint32_t> tokens(bytes, bytes + n), merged;
    for (uint32_t m = 0; m < n_merges; m++) {
        if (tokens.size() < 2) break;                              // tokenizer-manager.js:46
        const uint32_t a = merges[m * 3], b = merges[m * 3 + 1], nw = merges[m * 3 + 2];
        merged.clear();
        size_t i = 0;
        while (i < tokens.size()) {
            if (i + 1 < tokens.size() && tokens[i] == a && tokens[i + 1] == b) { merged.push_back(nw); i += 2; }
            else { merged.push_back(tokens[i]); i++; }
        }
        tokens.swap(merged);
    }
    for (size_t i = 0; i < tokens.size() && i < cap; i++) tokens_out[i] = tokens[i];
    return tokens.size();
}
