// Host-side trie compiler and header parser: the v3 binary of the reference
// (src/bpe/tokenizer/trie.js:39-98 compile, :110-128 header, :137-160 length check, :167-206 layout).
#include <algorithm>
#include <cstring>
#include <vector>

#include "../../include/b200bpe.h"

namespace {

constexpr uint32_t TRIE_MAGIC = 0x54524945u;  // 'TRIE'
constexpr uint32_t INVALID = 0xFFFFFFFFu;

struct BuildNode {
    uint32_t token = INVALID;
    std::vector<std::pair<uint8_t, uint32_t>> kids;  // (byte, build-node index), insertion order
};

}  // namespace

extern "C" {

b200bpe_status b200bpe_trie_compile(const uint8_t* vocab_bytes, const uint64_t* vocab_offsets, uint32_t vocab_size,
                                    void* out, size_t* out_len) {
    if (!out_len || (vocab_size && !vocab_offsets)) return B200BPE_ERR_BAD_ARG;
    // 1. insert the entries in id order; an entry that repeats an earlier byte string takes over its node
    std::vector<BuildNode> arena(1);
    uint32_t max_len = 0;
    for (uint32_t id = 0; id < vocab_size; id++) {
        const uint64_t lo = vocab_offsets[id], hi = vocab_offsets[id + 1];
        if (hi <= lo) continue;  // empty entries are skipped
        uint32_t node = 0;
        for (uint64_t p = lo; p < hi; p++) {
            const uint8_t b = vocab_bytes[p];
            uint32_t next = INVALID;
            for (auto& kv : arena[node].kids)
                if (kv.first == b) { next = kv.second; break; }
            if (next == INVALID) {
                next = (uint32_t)arena.size();
                arena[node].kids.push_back({b, next});
                arena.emplace_back();
            }
            node = next;
        }
        arena[node].token = id;
        max_len = std::max<uint32_t>(max_len, (uint32_t)(hi - lo));
    }
    // 2. breadth-first numbering, children in byte order, a node's edges contiguous
    const size_t node_count = arena.size(), edge_count = arena.size() - 1;
    const size_t need = 28 + node_count * 12 + edge_count * 8;
    if (!out) { *out_len = need; return B200BPE_OK; }
    if (*out_len < need) { *out_len = need; return B200BPE_ERR_CAPACITY; }
    *out_len = need;
    uint8_t* base = static_cast<uint8_t*>(out);
    std::memset(base, 0, need);
    const uint32_t hdr[7] = {TRIE_MAGIC, 3u, (uint32_t)node_count, (uint32_t)edge_count, max_len, vocab_size, 0u};
    std::memcpy(base, hdr, 28);
    uint32_t* nodes = reinterpret_cast<uint32_t*>(base + 28);
    uint8_t* edges = base + 28 + node_count * 12;
    std::vector<uint32_t> order;  // flat index → build index
    order.reserve(node_count);
    order.push_back(0);
    size_t edge_pos = 0;
    for (size_t head = 0; head < order.size(); head++) {
        BuildNode& bn = arena[order[head]];
        std::sort(bn.kids.begin(), bn.kids.end());
        const uint32_t first = (uint32_t)edge_pos;
        for (auto& kv : bn.kids) {
            const uint32_t child_flat = (uint32_t)order.size();
            order.push_back(kv.second);
            edges[edge_pos * 8] = kv.first;
            std::memcpy(edges + edge_pos * 8 + 4, &child_flat, 4);
            edge_pos++;
        }
        uint32_t rec[3] = {first, (uint32_t)bn.kids.size(), bn.token};
        std::memcpy(nodes + head * 3, rec, 12);
    }
    return B200BPE_OK;
}

b200bpe_status b200bpe_trie_parse_header(const void* trie, size_t len, uint32_t fields_out[5]) {
    if (!trie || !fields_out) return B200BPE_ERR_BAD_ARG;
    if (len < 28) return B200BPE_ERR_TRUNCATED_TRIE;
    uint32_t h[7];
    std::memcpy(h, trie, 28);
    if (h[0] != TRIE_MAGIC) return B200BPE_ERR_BAD_TRIE_MAGIC;
    if (h[1] != 3u && h[1] != 2u) return B200BPE_ERR_BAD_TRIE_VERSION;
    const uint64_t per_node = h[1] == 3 ? 12 : 8, per_edge = h[1] == 3 ? 8 : 4;
    fields_out[0] = h[1]; fields_out[1] = h[2]; fields_out[2] = h[3]; fields_out[3] = h[4]; fields_out[4] = h[5];
    if ((uint64_t)len < 28 + (uint64_t)h[2] * per_node + (uint64_t)h[3] * per_edge) return B200BPE_ERR_TRUNCATED_TRIE;
    return B200BPE_OK;
}

}  // extern "C"
