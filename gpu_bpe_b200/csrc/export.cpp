// The ".bin" token file of the reference's Export tab (src/ui/export-controller.js:4,192-202,235-248):
//   u32 LE  magic 0x44584654 ('DXFT'), vocabSize, tokenCount, vocabJsonBytes
//   u32 LE  tokens[tokenCount]
//   bytes   the vocabulary JSON {version, vocabSize, vocab, merges} (may be empty)
// and the way that tab joins its input files (two line feeds between files).  Host code only.
#include <cstring>

#include "../../include/b200bpe.h"

extern "C" {

b200bpe_status b200bpe_dxft_size(uint64_t n_tokens, uint64_t json_len, uint64_t* size_out) {
    if (!size_out || n_tokens > 0xFFFFFFFFull || json_len > 0xFFFFFFFFull) return B200BPE_ERR_BAD_ARG;
    *size_out = 16 + 4 * n_tokens + json_len;
    return B200BPE_OK;
}

b200bpe_status b200bpe_dxft_write(const uint32_t* tokens, uint64_t n_tokens, uint32_t vocab_size, const void* json,
                                  uint64_t json_len, void* out, uint64_t cap) {
    uint64_t need = 0;
    b200bpe_status r = b200bpe_dxft_size(n_tokens, json_len, &need);
    if (r) return r;
    if (!out || (!tokens && n_tokens) || (!json && json_len)) return B200BPE_ERR_BAD_ARG;
    if (cap < need) return B200BPE_ERR_CAPACITY;
    const uint32_t header[4] = {0x44584654u, vocab_size, (uint32_t)n_tokens, (uint32_t)json_len};
    unsigned char* o = static_cast<unsigned char*>(out);
    std::memcpy(o, header, 16);   // little-endian host, as the typed arrays of the reference are
    if (n_tokens) std::memcpy(o + 16, tokens, 4 * n_tokens);
    if (json_len) std::memcpy(o + 16 + 4 * n_tokens, json, json_len);
    return B200BPE_OK;
}

b200bpe_status b200bpe_dxft_parse(const void* buf, uint64_t len, uint32_t fields_out[4], uint64_t* tokens_offset,
                                  uint64_t* json_offset) {
    if (!buf || !fields_out) return B200BPE_ERR_BAD_ARG;
    if (len < 16) return B200BPE_ERR_TRUNCATED_TRIE;
    uint32_t h[4];
    std::memcpy(h, buf, 16);
    if (h[0] != 0x44584654u) return B200BPE_ERR_BAD_TRIE_MAGIC;
    if (len < 16 + 4ull * h[2] + h[3]) return B200BPE_ERR_TRUNCATED_TRIE;
    for (int i = 0; i < 4; i++) fields_out[i] = h[i];
    if (tokens_offset) *tokens_offset = 16;
    if (json_offset) *json_offset = 16 + 4ull * h[2];
    return B200BPE_OK;
}

}  // extern "C"
