// Merge-replay encoding on the device: the other encode(text) of the reference, the one behind its
// Tokenizer tab (TokenizerManager.encode, src/ui/tokenizer-manager.js:13-61 of toprakdeviren/gpu-bpe).
//
// The reference starts from one token per UTF-8 byte and applies every merge rule [a, b, newId] in
// the order it was learned, each as one left-to-right pass over the WHOLE token list that replaces
// a matching adjacent pair and steps over both tokens (:45-58).  There are no word boundaries and
// no chunks on this path, and with a == b a run of k equal tokens pairs up from the left:
// floor(k / 2) new tokens, then the odd one out.  This differs from the trie encoder (greedy
// longest match) and from the trainer's merge (snapshot rule, runs collapse).
//
// Here: a rule only does anything if its pair is present, so instead of one pass per rule the
// device works in rounds.  A round (1) looks every adjacent pair of the current list up in a hash
// table pair → (rank, newId) and takes the smallest rank present, (2) applies that one rule with a
// single-pass scan + compaction (decoupled look-back, bounded waits) from the ping into the pong
// buffer.  Rounds are equivalent to the reference's rule-by-rule loop when no rule refers to an id
// that is only made by a later rule and every rule makes an id of its own (then a pair that appears
// after rule r can only match rules after r, which is all the in-order loop would still try);
// every merge list a trainer produces is like that, and b200bpe_replay_create refuses the others.
// For a == b the pairing from the left needs, per token, the parity of the run of `a` that ends
// right before it: inside a tile that is a segmented scan over (all tokens are `a`, parity of the
// trailing run); for the run that reaches the tile's first token one thread reads backwards from
// the tile's start until the run ends (runs are short in text).
#include <algorithm>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "ctx.cuh"

namespace b200bpe {

constexpr int RP_THREADS = 256;
constexpr int RP_PER_THREAD = 8;
constexpr int RP_TILE = RP_THREADS * RP_PER_THREAD;   // tokens per tile
constexpr int RP_ROUNDS_PER_GRAPH = 64;
constexpr uint32_t RP_NO_RANK = 0xFFFFFFFFu;
constexpr uint32_t RP_MAX_SPINS = 1u << 22;

struct ReplayState {
    uint32_t n[2];        // tokens in the ping / pong buffer, indexed by (epoch & 1)
    uint32_t epoch;       // rounds applied so far
    uint32_t done;        // no pair of the list has a rule any more
    uint32_t best_rank;   // smallest rank among the pairs present (RP_NO_RANK: none)
    uint32_t a, b, new_id;
    uint32_t ticket;      // next tile of the apply kernel
    uint32_t status;      // 0 ok, 2 a look-back wait ran out
    uint32_t rounds;      // statistics
    uint32_t pad;
};

struct RankSlot { unsigned long long key; uint32_t rank, new_id; };   // key 0 = empty (a pair (0, 0) is stored as ~0)

__device__ __forceinline__ uint32_t rp_hash(unsigned long long key) {
    uint32_t x = (uint32_t)key ^ ((uint32_t)(key >> 32) * 0x9E3779B1u);
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}
__device__ __forceinline__ unsigned long long rp_key(uint32_t a, uint32_t b) {
    const unsigned long long k = ((unsigned long long)a << 32) | b;
    return k ? k : ~0ull;
}

__global__ void k_replay_bytes(const uint8_t* __restrict__ bytes, uint32_t* __restrict__ tok, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) tok[i] = bytes[i];
}

// (1) the smallest rank among the adjacent pairs of the current list
__global__ void __launch_bounds__(RP_THREADS)
k_replay_rank(ReplayState* __restrict__ st, const uint32_t* buf0, const uint32_t* buf1, const RankSlot* __restrict__ table, uint32_t mask) {
    if (st->done | st->status) return;
    const uint32_t e = st->epoch, N = st->n[e & 1];
    const uint32_t* __restrict__ src = (e & 1) ? buf1 : buf0;
    uint32_t best = RP_NO_RANK;
    for (uint32_t i = blockIdx.x * RP_THREADS + threadIdx.x; i + 1 < N; i += gridDim.x * RP_THREADS) {
        const unsigned long long key = rp_key(src[i], src[i + 1]);
        uint32_t slot = rp_hash(key) & mask;
        for (;;) {
            const RankSlot s = table[slot];
            if (s.key == key) { best = min(best, s.rank); break; }
            if (s.key == 0ull) break;
            slot = (slot + 1) & mask;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xFFFFFFFFu, best, o));
    if ((threadIdx.x & 31) == 0 && best != RP_NO_RANK) atomicMin(&st->best_rank, best);
}

// between (1) and (2): the rule of this round
__global__ void k_replay_setup(ReplayState* __restrict__ st, const uint32_t* __restrict__ rules) {
    if (st->done | st->status) return;
    const uint32_t r = st->best_rank;
    if (r == RP_NO_RANK) { st->done = 1u; return; }
    st->a = rules[3 * r]; st->b = rules[3 * r + 1]; st->new_id = rules[3 * r + 2];
    st->best_rank = RP_NO_RANK;
    st->ticket = 0u;
    st->rounds += 1u;
}

// (2) apply the rule: left-to-right pairing, stable compaction ping → pong.
// desc[tile] = (tag << 34) | (flag << 32) | kept, tag = round + 1, flag 1 aggregate / 2 inclusive prefix.
__global__ void __launch_bounds__(RP_THREADS)
k_replay_apply(ReplayState* __restrict__ st, uint32_t* buf0, uint32_t* buf1, unsigned long long* __restrict__ desc) {
    __shared__ uint32_t s_tile, s_warp[RP_THREADS / 32], s_excl, s_run[RP_THREADS / 32], s_before;
    if (st->done | st->status) return;
    const uint32_t e = st->epoch, N = st->n[e & 1];
    const uint32_t* __restrict__ src = (e & 1) ? buf1 : buf0;
    uint32_t* __restrict__ dst = (e & 1) ? buf0 : buf1;
    const uint32_t A = st->a, B = st->b, NW = st->new_id;
    const uint32_t ntiles = (N + RP_TILE - 1) / RP_TILE;
    const uint32_t tag = (e + 1u) & 0x3FFFFFFFu;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) s_tile = atomicAdd(&st->ticket, 1u);
        __syncthreads();
        const uint32_t tile = s_tile;
        if (tile >= ntiles) return;
        const uint32_t i0 = tile * RP_TILE + threadIdx.x * RP_PER_THREAD;   // this thread's first token
        // a token is the second of a pair (dropped) or the first (rewritten) or neither.
        // a != b: pairs cannot overlap.  a == b: within a run of `a`, the tokens at odd distance from
        // the run's start are the second halves; the distance's parity is carried along.
        uint32_t t[RP_PER_THREAD + 1];
#pragma unroll
        for (int k = 0; k <= RP_PER_THREAD; k++) t[k] = i0 + k < N ? src[i0 + k] : 0xFFFFFFFFu;   // (0xFFFFFFFF is no token)
        uint32_t odd = 0u;   // a == b: parity of the run of `a` that ends right before this thread's first token
        const uint32_t prev = i0 > 0u && i0 <= N ? src[i0 - 1u] : 0xFFFFFFFFu;
        if (A == B) {
            // this thread's tokens as one element (bit 1: all of them are `a`, bit 0: parity of the trailing run of `a`);
            // combine(left, right) = right is all `a` ? (left.all, left.parity ^ right.parity) : right
            uint32_t tr = 0u;
#pragma unroll
            for (int k = RP_PER_THREAD - 1; k >= 0; k--) { if (t[k] == A && tr == (uint32_t)(RP_PER_THREAD - 1 - k)) tr++; }
            const uint32_t mine = (tr == (uint32_t)RP_PER_THREAD ? 2u : 0u) | (tr & 1u);
            uint32_t inc = mine;   // inclusive scan within the warp
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t left = __shfl_up_sync(0xFFFFFFFFu, inc, o);
                if (lane >= o && (inc & 2u)) inc = (left & 2u) | ((left ^ inc) & 1u);
            }
            if (lane == 31) s_run[warp] = inc;
            if (threadIdx.x == 0) {
                // the run that ends right before the tile
                uint32_t len = 0u;
                if (prev == A) { len = 1u; for (uint32_t j = i0 - 1u; j > 0u && src[j - 1u] == A; j--) len++; }
                s_before = len & 1u;
            }
            __syncthreads();
            uint32_t ex = __shfl_up_sync(0xFFFFFFFFu, inc, 1);   // exclusive: everything of the warp before this thread
            if (lane == 0) ex = 2u;                               // nothing: all `a` (vacuously), parity 0
            uint32_t pre = 2u;                                    // the warps before this one
            for (int w2 = 0; w2 < warp; w2++) { const uint32_t r = s_run[w2]; pre = (r & 2u) ? ((pre & 2u) | ((pre ^ r) & 1u)) : r; }
            const uint32_t all_before = (ex & 2u) ? ((pre & 2u) | ((pre ^ ex) & 1u)) : ex;   // the tile's tokens before this thread
            odd = (all_before & 1u) ^ ((all_before & 2u) ? s_before : 0u);
        }
        uint32_t keep = 0u, rew = 0u;
        bool prev_first = A != B ? (prev == A && t[0] == B && i0 < N) : false;   // the token before is the first of a pair that takes t[0]
        if (A == B) prev_first = odd != 0u && t[0] == A;
#pragma unroll
        for (int k = 0; k < RP_PER_THREAD; k++) {
            const bool live = i0 + k < N;
            bool first = false;
            if (!prev_first) first = live && t[k] == A && t[k + 1] == B;   // t[k + 1] is 0xFFFFFFFF beyond the end
            if (live && !prev_first) keep |= 1u << k;
            if (first) rew |= 1u << k;
            prev_first = first;
        }
        const uint32_t cnt = __popc(keep);
        uint32_t incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t x = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += x;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        uint32_t warp_off = 0u, agg = 0u;
#pragma unroll
        for (int w = 0; w < RP_THREADS / 32; w++) { if (w < warp) warp_off += s_warp[w]; agg += s_warp[w]; }
        if (warp == 0) {
            unsigned long long excl = 0ull;
            if (tile == 0u) {
                if (lane == 0)
                    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(desc), "l"(((unsigned long long)((tag << 2) | 2u) << 32) | agg) : "memory");
            } else {
                if (lane == 0) {
                    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(desc + tile), "l"(((unsigned long long)((tag << 2) | 1u) << 32) | agg) : "memory");
                }
                int pos = (int)tile - 1;
                uint32_t spins = 0u;
                bool timed_out = false;
                for (;;) {
                    const int idx = pos - lane;
                    uint32_t hi = (tag << 2) | 2u, val = 0u;   // before tile 0: a zero prefix
                    for (;;) {
                        if (idx >= 0) {
                            unsigned long long d;
                            asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(d) : "l"(desc + idx) : "memory");
                            hi = (uint32_t)(d >> 32); val = (uint32_t)d;
                        }
                        const bool ready = (hi >> 2) == tag && (hi & 3u) != 0u;
                        if (__all_sync(0xFFFFFFFFu, ready)) break;
                        if (++spins > RP_MAX_SPINS) { timed_out = true; break; }
                        __nanosleep(40);
                    }
                    if (timed_out) break;
                    const uint32_t pmask = __ballot_sync(0xFFFFFFFFu, (hi & 3u) == 2u);
                    const int first = pmask ? (__ffs(pmask) - 1) : 32;
                    uint32_t contrib = lane <= first ? val : 0u;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xFFFFFFFFu, contrib, o);
                    excl += contrib;
                    if (pmask) break;
                    pos -= 32;
                }
                if (timed_out) { if (lane == 0) atomicExch(&st->status, 2u); excl = 0ull; }
                if (lane == 0)
                    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(desc + tile), "l"(((unsigned long long)((tag << 2) | 2u) << 32) | (uint32_t)(excl + agg)) : "memory");
            }
            if (lane == 0) {
                s_excl = (uint32_t)excl;
                if (tile == ntiles - 1u) {
                    st->n[(e + 1u) & 1u] = (uint32_t)excl + agg;
                    st->epoch = e + 1u;
                }
            }
        }
        __syncthreads();
        uint32_t o = s_excl + warp_off + incl - cnt;
#pragma unroll
        for (int k = 0; k < RP_PER_THREAD; k++)
            if ((keep >> k) & 1u) dst[o++] = ((rew >> k) & 1u) ? NW : t[k];
    }
}

struct Replay {
    Ctx* ctx = nullptr;
    uint32_t n_rules = 0;
    uint32_t* d_rules = nullptr;
    RankSlot* d_table = nullptr;
    uint32_t mask = 0;
    ReplayState* d_state = nullptr;
    ReplayState* h_state = nullptr;   // pinned
    uint32_t* buf[2] = {nullptr, nullptr};
    uint8_t* d_in = nullptr;
    unsigned long long* d_desc = nullptr;
    uint64_t cap = 0;
    cudaGraphExec_t graph = nullptr;
    uint64_t graph_cap = 0;
    uint32_t last_rounds = 0;

    ~Replay() {
        if (ctx) cudaSetDevice(ctx->device);
        if (graph) cudaGraphExecDestroy(graph);
        cudaFree(d_rules); cudaFree(d_table); cudaFree(d_state); cudaFree(buf[0]); cudaFree(buf[1]); cudaFree(d_in); cudaFree(d_desc);
        if (h_state) cudaFreeHost(h_state);
    }

    b200bpe_status ensure(uint64_t n) {
        if (n <= cap) return B200BPE_OK;
        B2_CUDA(cudaStreamSynchronize(ctx->stream));
        if (graph) { cudaGraphExecDestroy(graph); graph = nullptr; }
        cudaFree(buf[0]); cudaFree(buf[1]); cudaFree(d_in); cudaFree(d_desc);
        buf[0] = buf[1] = nullptr; d_in = nullptr; d_desc = nullptr;
        cap = n + n / 2 + 16;
        B2_CUDA(cudaMalloc(&buf[0], cap * 4));
        B2_CUDA(cudaMalloc(&buf[1], cap * 4));
        B2_CUDA(cudaMalloc(&d_in, cap));
        B2_CUDA(cudaMalloc(&d_desc, (cap / RP_TILE + 2) * 8));
        B2_CUDA(cudaMemsetAsync(d_desc, 0, (cap / RP_TILE + 2) * 8, ctx->stream));
        return B200BPE_OK;
    }

    void enqueue_round(int grid_rank, int grid_apply) {
        cudaStream_t s = ctx->stream;
        k_replay_rank<<<grid_rank, RP_THREADS, 0, s>>>(d_state, buf[0], buf[1], d_table, mask);
        k_replay_setup<<<1, 1, 0, s>>>(d_state, d_rules);
        k_replay_apply<<<grid_apply, RP_THREADS, 0, s>>>(d_state, buf[0], buf[1], d_desc);
    }

    // tokens of `n` bytes (already in d_in or given as a device pointer) → buf[epoch & 1]; returns the count
    b200bpe_status run(const uint8_t* d_bytes, uint64_t n, uint64_t* n_tokens) {
        cudaStream_t s = ctx->stream;
        const int grid = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)ctx->sm_count * 8, (n + RP_TILE - 1) / RP_TILE));
        k_replay_bytes<<<grid, RP_THREADS, 0, s>>>(d_bytes, buf[0], n);
        std::memset(h_state, 0, sizeof(ReplayState));
        h_state->n[0] = (uint32_t)n;
        h_state->best_rank = RP_NO_RANK;
        h_state->done = (n_rules == 0 || n < 2) ? 1u : 0u;   // no merges: the bytes are the tokens (tokenizer-manager.js:21-25,46)
        B2_CUDA(cudaMemcpyAsync(d_state, h_state, sizeof(ReplayState), cudaMemcpyHostToDevice, s));
        // the look-back descriptors are tagged with the round number, which restarts here
        B2_CUDA(cudaMemsetAsync(d_desc, 0, (n / RP_TILE + 2) * 8, s));
        if (!graph || graph_cap != cap) {
            if (graph) { cudaGraphExecDestroy(graph); graph = nullptr; }
            const int g_all = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)ctx->sm_count * 8, (cap + RP_TILE - 1) / RP_TILE));
            cudaGraph_t g = nullptr;
            B2_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
            for (int i = 0; i < RP_ROUNDS_PER_GRAPH; i++) enqueue_round(g_all, g_all);
            B2_CUDA(cudaStreamEndCapture(s, &g));
            cudaError_t e = cudaGraphInstantiate(&graph, g, 0);
            cudaGraphDestroy(g);
            B2_CUDA(e);
            graph_cap = cap;
        }
        for (;;) {
            B2_CUDA(cudaGraphLaunch(graph, s));
            B2_CUDA(cudaMemcpyAsync(h_state, d_state, sizeof(ReplayState), cudaMemcpyDeviceToHost, s));
            B2_CUDA(cudaStreamSynchronize(s));
            if (h_state->status) return B200BPE_ERR_LOOKBACK_TIMEOUT;
            if (h_state->done) break;
        }
        last_rounds = h_state->rounds;
        *n_tokens = h_state->n[h_state->epoch & 1];
        return B200BPE_OK;
    }
};

}  // namespace b200bpe

struct b200bpe_replay { b200bpe::Replay* r; };

using namespace b200bpe;

extern "C" {

b200bpe_status b200bpe_replay_create(b200bpe_ctx* c, const uint32_t* merges, uint32_t n_merges, b200bpe_replay** out) {
    if (!c || !out || (!merges && n_merges)) return B200BPE_ERR_BAD_ARG;
    // Rounds by smallest rank equal the reference's rule-by-rule loop only for lists in which every
    // rule makes an id of its own, no byte value among them, and uses only ids made by earlier rules.
    std::unordered_map<uint32_t, uint32_t> made_at;
    for (uint32_t r = 0; r < n_merges; r++) {
        const uint32_t nw = merges[3 * r + 2];
        if (nw < 256u || made_at.count(nw)) { set_last_error("merge list: rule " + std::to_string(r) + " makes an id that is a byte value or already made"); return B200BPE_ERR_BAD_ARG; }
        made_at[nw] = r;
    }
    for (uint32_t r = 0; r < n_merges; r++)
        for (int k = 0; k < 2; k++) {
            auto it = made_at.find(merges[3 * r + k]);
            if (it != made_at.end() && it->second >= r) { set_last_error("merge list: rule " + std::to_string(r) + " uses an id that only a later rule makes"); return B200BPE_ERR_BAD_ARG; }
        }
    B2_CUDA(cudaSetDevice(c->c.device));
    Replay* rp = new Replay();
    rp->ctx = &c->c;
    rp->n_rules = n_merges;
    auto fail = [&](b200bpe_status st) { delete rp; return st; };
    uint32_t lg = 4;
    while ((1ull << lg) < (uint64_t)n_merges * 2 + 16) lg++;
    rp->mask = (1u << lg) - 1u;
    std::vector<RankSlot> table((size_t)1 << lg, RankSlot{0ull, 0u, 0u});
    for (uint32_t r = 0; r < n_merges; r++) {
        unsigned long long key = ((unsigned long long)merges[3 * r] << 32) | merges[3 * r + 1];
        if (!key) key = ~0ull;
        uint32_t x = (uint32_t)key ^ ((uint32_t)(key >> 32) * 0x9E3779B1u);
        x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
        uint32_t slot = x & rp->mask;
        bool dup = false;
        while (table[slot].key != 0ull) { if (table[slot].key == key) { dup = true; break; } slot = (slot + 1) & rp->mask; }
        if (!dup) table[slot] = RankSlot{key, r, merges[3 * r + 2]};   // the first rule of a pair wins (tokenizer-manager.js:31-33)
    }
    cudaStream_t s = c->c.stream;
    if (cudaMalloc(&rp->d_rules, std::max<size_t>(12, (size_t)n_merges * 12)) != cudaSuccess) return fail(B200BPE_ERR_OOM);
    if (cudaMalloc(&rp->d_table, table.size() * sizeof(RankSlot)) != cudaSuccess) return fail(B200BPE_ERR_OOM);
    if (cudaMalloc(&rp->d_state, sizeof(ReplayState)) != cudaSuccess) return fail(B200BPE_ERR_OOM);
    if (cudaMallocHost(&rp->h_state, sizeof(ReplayState)) != cudaSuccess) return fail(B200BPE_ERR_OOM);
    if (n_merges && cudaMemcpyAsync(rp->d_rules, merges, (size_t)n_merges * 12, cudaMemcpyHostToDevice, s) != cudaSuccess) return fail(B200BPE_ERR_CUDA);
    if (cudaMemcpyAsync(rp->d_table, table.data(), table.size() * sizeof(RankSlot), cudaMemcpyHostToDevice, s) != cudaSuccess) return fail(B200BPE_ERR_CUDA);
    if (cudaStreamSynchronize(s) != cudaSuccess) return fail(B200BPE_ERR_CUDA);
    *out = new b200bpe_replay{rp};
    return B200BPE_OK;
}

b200bpe_status b200bpe_replay_encode(b200bpe_replay* h, const uint8_t* bytes, uint64_t n, uint32_t* tokens_out, uint64_t cap,
                                     uint64_t* n_tokens_out) {
    if (!h || (!bytes && n) || !n_tokens_out) return B200BPE_ERR_BAD_ARG;
    Replay* rp = h->r;
    *n_tokens_out = 0;
    if (n == 0) return B200BPE_OK;
    if (n >= 0xFFFFFFF0ull) return B200BPE_ERR_BAD_ARG;
    B2_CUDA(cudaSetDevice(rp->ctx->device));
    b200bpe_status r = rp->ensure(n);
    if (r) return r;
    cudaStream_t s = rp->ctx->stream;
    B2_CUDA(cudaMemcpyAsync(rp->d_in, bytes, n, cudaMemcpyHostToDevice, s));
    uint64_t nt = 0;
    if ((r = rp->run(rp->d_in, n, &nt))) return r;
    *n_tokens_out = nt;
    if (nt > cap || (!tokens_out && nt)) return B200BPE_ERR_CAPACITY;
    B2_CUDA(cudaMemcpyAsync(tokens_out, rp->buf[rp->h_state->epoch & 1], nt * 4, cudaMemcpyDeviceToHost, s));
    B2_CUDA(cudaStreamSynchronize(s));
    return B200BPE_OK;
}

b200bpe_status b200bpe_replay_encode_device(b200bpe_replay* h, const uint8_t* d_bytes, uint64_t n, uint32_t* d_tokens_out,
                                            uint64_t cap, uint64_t* n_tokens_out) {
    if (!h || (!d_bytes && n) || !n_tokens_out) return B200BPE_ERR_BAD_ARG;
    Replay* rp = h->r;
    *n_tokens_out = 0;
    if (n == 0) return B200BPE_OK;
    if (n >= 0xFFFFFFF0ull) return B200BPE_ERR_BAD_ARG;
    B2_CUDA(cudaSetDevice(rp->ctx->device));
    b200bpe_status r = rp->ensure(n);
    if (r) return r;
    uint64_t nt = 0;
    if ((r = rp->run(d_bytes, n, &nt))) return r;
    *n_tokens_out = nt;
    if (nt > cap || (!d_tokens_out && nt)) return B200BPE_ERR_CAPACITY;
    B2_CUDA(cudaMemcpyAsync(d_tokens_out, rp->buf[rp->h_state->epoch & 1], nt * 4, cudaMemcpyDeviceToDevice, rp->ctx->stream));
    B2_CUDA(cudaStreamSynchronize(rp->ctx->stream));
    return B200BPE_OK;
}

b200bpe_status b200bpe_replay_last_rounds(b200bpe_replay* h, uint32_t* rounds) {
    if (!h || !rounds) return B200BPE_ERR_BAD_ARG;
    *rounds = h->r->last_rounds;
    return B200BPE_OK;
}

void b200bpe_replay_destroy(b200bpe_replay* h) {
    if (!h) return;
    delete h->r;
    delete h;
}

}  // extern "C"
