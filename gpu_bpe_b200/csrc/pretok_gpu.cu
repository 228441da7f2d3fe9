// Device pre-tokeniser: GPT-4-style word starts over code-point classes, one pass over the bytes.
// Restates PreTokenizer.preTokenizeBytes (src/wasm/pre_tokenizer.mjs:459-509 of the reference:
// decode :518-554, classify :126-134, boundaries :226-292, contractions :83-110, digit runs
// :198-204, code-point start → first byte :499-506) for input that is well-formed UTF-8 (the last
// character may be cut short); anything else is refused, b200bpe_pretokenize (host) takes any bytes.
// The reference first NFC-normalises with a closed WASM library (:465): the input must be NFC.
//
// Every rule but one looks at a few code points around a position; the exception is the split of
// digit runs every three code points counted from the start of the run, which needs the distance
// to the run's start.  That is a segmented count carried across tiles by a single-pass scan with
// decoupled look-back: a tile publishes (digit code points at its end, "all my code points are
// digits"), and a tile's carry-in is the sum over its predecessors back to the nearest one that
// is not all digits.
#include <mutex>
#include <string>

#include "ctx.cuh"

namespace b200bpe {

namespace {
#include "unicode_classes.inc"
}

enum : uint32_t { PT_LETTER = 0, PT_DIGIT = 1, PT_WS = 2, PT_PUNCT = 3, PT_SYMBOL = 4, PT_NEWLINE = 5, PT_OTHER = 6, PT_CONT = 0xFFu };

constexpr int PT_THREADS = 256;
constexpr int PT_PER = 16;                       // bytes per thread
constexpr int PT_TILE = PT_THREADS * PT_PER;     // 4,096 bytes per tile
constexpr int PT_BEFORE = 16, PT_AFTER = 16;     // halo bytes kept around a tile
constexpr uint32_t PT_LOW = 0x3000;              // code points with a direct class table
constexpr uint32_t PT_MAX_SPINS = 1u << 22;
constexpr uint32_t PT_AGG = 1u, PT_PREFIX = 2u;

struct ClassTables {
    const uint8_t* low;          // PT_LOW entries
    const uint32_t* ranges;      // {first, last, class} triples, sorted
    uint32_t n_ranges;
};

__device__ __forceinline__ uint32_t class_of(const ClassTables& t, uint32_t cp) {
    if (cp < PT_LOW) return __ldg(t.low + cp);
    if (cp > 0x10FFFFu) return PT_OTHER;
    uint32_t lo = 0, hi = t.n_ranges;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (__ldg(t.ranges + 3 * mid) <= cp) lo = mid; else hi = mid;
    }
    return cp <= __ldg(t.ranges + 3 * lo + 1) ? __ldg(t.ranges + 3 * lo + 2) : PT_OTHER;
}

__device__ __forceinline__ bool pt_punct_or_symbol(uint32_t c) { return c == PT_PUNCT || c == PT_SYMBOL; }
__device__ __forceinline__ bool pt_transition(uint32_t p, uint32_t c) {  // pre_tokenizer.mjs:175-189
    return (p == PT_LETTER && c == PT_DIGIT) || (p == PT_DIGIT && c == PT_LETTER) || (p == PT_LETTER && pt_punct_or_symbol(c)) ||
           (pt_punct_or_symbol(p) && c == PT_LETTER) || (pt_punct_or_symbol(p) && c == PT_DIGIT) ||
           (p == PT_DIGIT && pt_punct_or_symbol(c));
}
__device__ __forceinline__ bool pt_in(uint32_t b, uint32_t lower) { return (b | 0x20u) == lower && b < 0x80u; }

__device__ __forceinline__ unsigned long long pt_ld(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void pt_st(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// desc: (tag << 34) | (flag << 32) | (all_digits << 31) | digits; status[0]: 1 = malformed UTF-8, 2 = look-back timed out
__global__ void __launch_bounds__(PT_THREADS)
k_pretokenize(ClassTables tab, const uint8_t* __restrict__ bytes, uint64_t n, uint8_t* __restrict__ out,
              unsigned long long* __restrict__ desc, uint32_t* __restrict__ ticket, uint32_t* __restrict__ status,
              uint32_t tag, uint32_t max_spins) {
    __shared__ uint8_t sb[PT_BEFORE + PT_TILE + PT_AFTER];    // the bytes (0 outside the input)
    __shared__ uint8_t sc[PT_BEFORE + PT_TILE + PT_AFTER];    // class of the code point that starts here, PT_CONT on the others
    __shared__ uint32_t s_tile, s_carry, s_atr, s_aall;
    __shared__ uint32_t w_tr[PT_THREADS / 32], w_all[PT_THREADS / 32];
    const uint64_t ntiles = (n + PT_TILE - 1) / PT_TILE;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (;;) {
        if (threadIdx.x == 0) s_tile = atomicAdd(ticket, 1u);
        __syncthreads();
        const uint64_t tile = s_tile;
        if (tile >= ntiles) return;
        const long long t0 = (long long)tile * PT_TILE;   // first byte of the tile
        // bytes of the tile and its halo
        for (int i = threadIdx.x; i < PT_BEFORE + PT_TILE + PT_AFTER; i += PT_THREADS) {
            const long long g = t0 - PT_BEFORE + i;
            sb[i] = (g >= 0 && (uint64_t)g < n) ? bytes[g] : (uint8_t)0;
        }
        __syncthreads();
        // classes: decode wherever a code point starts (pre_tokenizer.mjs:518-554; bytes past the end read as 0)
        bool bad = false;
        for (int i = threadIdx.x; i < PT_BEFORE + PT_TILE + PT_AFTER; i += PT_THREADS) {
            const long long g = t0 - PT_BEFORE + i;
            uint32_t cls = PT_CONT;
            if (g >= 0 && (uint64_t)g < n) {
                const uint32_t c = sb[i];
                if ((c & 0xC0u) != 0x80u) {
                    auto at = [&](int k) -> uint32_t { return (i + k < PT_BEFORE + PT_TILE + PT_AFTER) ? sb[i + k] : 0u; };
                    uint32_t v, size;
                    if (c < 0x80u) { v = c; size = 1; }
                    else if ((c & 0xE0u) == 0xC0u) { v = (c & 0x1Fu) << 6 | (at(1) & 0x3Fu); size = 2; }
                    else if ((c & 0xF0u) == 0xE0u) { v = (c & 0x0Fu) << 12 | (at(1) & 0x3Fu) << 6 | (at(2) & 0x3Fu); size = 3; }
                    else { v = (c & 0x07u) << 18 | (at(1) & 0x3Fu) << 12 | (at(2) & 0x3Fu) << 6 | (at(3) & 0x3Fu); size = 4; }
                    // well-formed: exactly size - 1 continuation bytes follow (unless the input ends first), and no lead above F7
                    if (i >= PT_BEFORE && i < PT_BEFORE + PT_TILE) {
                        if (c >= 0xF8u) bad = true;
                        for (uint32_t k = 1; k <= size; k++) {
                            if ((uint64_t)(g + k) >= n) break;
                            const bool cont = (at((int)k) & 0xC0u) == 0x80u;
                            if (cont != (k < size)) bad = true;
                        }
                    }
                    cls = class_of(tab, v);
                } else if (g == 0) {
                    bad = true;   // the input starts inside a character
                }
            }
            sc[i] = (uint8_t)cls;
        }
        if (bad) atomicExch(status, 1u);
        __syncthreads();
        // digit runs: per thread (digits at the end of my 16 bytes, all my code points are digits)
        const int base = PT_BEFORE + threadIdx.x * PT_PER;
        uint32_t tr = 0, all = 1;
#pragma unroll
        for (int k = 0; k < PT_PER; k++) {
            const uint32_t c = sc[base + k];
            if (c == PT_DIGIT) tr++;
            else if (c != PT_CONT) { tr = 0; all = 0; }
        }
        // exclusive scan of (tr, all) over the CTA: combine(A, B) = B.all ? (A.tr + B.tr, A.all) : (B.tr, 0)
        uint32_t itr = tr, iall = all;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t ptr_ = __shfl_up_sync(0xFFFFFFFFu, itr, o), pall = __shfl_up_sync(0xFFFFFFFFu, iall, o);
            if (lane >= o) { if (iall) { itr += ptr_; iall = pall; } }
        }
        if (lane == 31) { w_tr[warp] = itr; w_all[warp] = iall; }
        __syncthreads();
        // carry into this thread from the earlier threads of the tile: (ctr, call)
        uint32_t ctr = 0, call = 1;
        for (int w = 0; w < warp; w++) {   // earlier warps, in order
            if (w_all[w]) ctr += w_tr[w]; else { ctr = w_tr[w]; call = 0; }
        }
        {
            uint32_t etr = __shfl_up_sync(0xFFFFFFFFu, itr, 1), eall = __shfl_up_sync(0xFFFFFFFFu, iall, 1);
            if (lane == 0) { etr = 0; eall = 1; }
            if (eall) { ctr += etr; } else { ctr = etr; call = 0; }
        }
        // the tile's aggregate (from the last thread) and the carry from the tiles before it
        if (threadIdx.x == PT_THREADS - 1) {
            uint32_t atr, aall;
            if (all) { atr = ctr + tr; aall = call; } else { atr = tr; aall = 0; }
            const uint32_t flag = tile == 0 ? PT_PREFIX : PT_AGG;
            pt_st(desc + tile, ((unsigned long long)((tag << 2) | flag) << 32) | ((unsigned long long)aall << 31) | atr);
            s_atr = atr; s_aall = aall;   // for the prefix published below
        }
        __syncthreads();
        if (warp == 0) {
            uint32_t in_tr = 0, in_all = 1;   // digits that end right before this tile
            bool done = tile == 0;
            long long pos = (long long)tile - 1;
            uint32_t spins = 0;
            while (!done) {
                const long long idx = pos - lane;
                uint32_t hi = (tag << 2) | PT_PREFIX, val = 0;   // before tile 0: an empty prefix that is not all digits
                for (;;) {
                    if (idx >= 0) { const unsigned long long d = pt_ld(desc + idx); hi = (uint32_t)(d >> 32); val = (uint32_t)d; }
                    const bool ready = (hi >> 2) == tag && (hi & 3u) != 0u;
                    if (__all_sync(0xFFFFFFFFu, ready)) break;
                    if (++spins > max_spins) { if (lane == 0) atomicExch(status, 2u); val = 0; hi = (tag << 2) | PT_PREFIX; break; }
                    __nanosleep(20);
                }
                // stop at the nearest predecessor that is a full prefix or is not all digits
                const bool stop = (hi & 3u) == PT_PREFIX || !(val >> 31) || idx < 0;
                const uint32_t smask = __ballot_sync(0xFFFFFFFFu, stop);
                const int first = smask ? (__ffs(smask) - 1) : 32;
                uint32_t contrib = (lane <= first && idx >= 0) ? (val & 0x7FFFFFFFu) : 0u;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xFFFFFFFFu, contrib, o);
                in_tr += contrib;
                if (smask) {
                    const uint32_t sval = __shfl_sync(0xFFFFFFFFu, val, first);
                    const long long sidx = pos - first;
                    in_all = (sidx >= 0 && (sval >> 31)) ? 1u : 0u;   // only a prefix that is itself all digits keeps the run open
                    done = true;
                } else {
                    pos -= 32;
                }
            }
            if (lane == 0) {
                s_carry = in_tr;
                if (tile != 0) {
                    const uint32_t atr = s_atr, aall = s_aall;
                    const uint32_t ptr_ = aall ? in_tr + atr : atr, pall = aall ? in_all : 0u;
                    pt_st(desc + tile, ((unsigned long long)((tag << 2) | PT_PREFIX) << 32) | ((unsigned long long)pall << 31) | ptr_);
                }
            }
        }
        __syncthreads();
        if (call) ctr += s_carry;   // the run reaches back across the tile's start
        // decisions for my 16 bytes
        uint32_t marks = 0;         // bit k: byte k starts a word
        uint32_t run = ctr;         // digit code points right before the current position
#pragma unroll 1
        for (int k = 0; k < PT_PER; k++) {
            const int i = base + k;
            const long long g = t0 + (long long)threadIdx.x * PT_PER + k;
            const uint32_t c = sc[i];
            if ((uint64_t)g >= n || c == PT_CONT) continue;
            const uint32_t run_before = run;
            run = c == PT_DIGIT ? run + 1u : 0u;
            if (g == 0) { marks |= 1u << k; continue; }
            // previous code point: the nearest start within the four bytes before
            int q = i - 1;
            while (q > i - 4 && sc[q] == PT_CONT) q--;
            const uint32_t p = sc[q];
            // is this position swallowed by a contraction that began one or two code points earlier?
            // (the swallowed code points are the ASCII letters after the apostrophe)
            auto contraction_at = [&](int a) -> int {   // a: index of an apostrophe; code points consumed, or 0
                const uint32_t b0 = sb[a];
                int la;
                if (b0 == 0x27u) la = 1;
                else if (b0 == 0xE2u && sb[a + 1] == 0x80u && sb[a + 2] == 0x99u) la = 3;
                else return 0;
                int qa = a - 1;
                while (qa > a - 4 && sc[qa] == PT_CONT) qa--;
                const long long ga = t0 - PT_BEFORE + a;
                if (ga <= 0 || sc[qa] != PT_LETTER) return 0;
                const long long g1 = ga + la;            // byte of the code point after the apostrophe
                if ((uint64_t)g1 >= n) return 0;
                const uint32_t nx = sb[a + la];
                const bool end2 = (uint64_t)(g1 + 1) >= n;
                if ((pt_in(nx, 's') || pt_in(nx, 't') || pt_in(nx, 'm') || pt_in(nx, 'd')) && (end2 || sc[a + la + 1] != PT_LETTER)) return 2;
                if (!end2 && nx < 0x80u) {
                    const uint32_t nn = sb[a + la + 1];
                    const bool end3 = (uint64_t)(g1 + 2) >= n;
                    const bool after = end3 || nn >= 0x80u || sc[a + la + 2] != PT_LETTER;
                    if (after && ((pt_in(nx, 'r') && pt_in(nn, 'e')) || (pt_in(nx, 'v') && pt_in(nn, 'e')) || (pt_in(nx, 'l') && pt_in(nn, 'l'))))
                        return 3;
                }
                return 0;
            };
            bool swallowed = false;
            if (sb[i] < 0x80u && c == PT_LETTER) {
                // one code point back
                if (sb[i - 1] == 0x27u) swallowed = contraction_at(i - 1) >= 2;
                else if (sb[i - 1] == 0x99u && i >= 3) swallowed = contraction_at(i - 3) >= 2;
                // two code points back (the one in between is an ASCII letter)
                if (!swallowed && sb[i - 1] < 0x80u && i >= 2) {
                    if (sb[i - 2] == 0x27u) swallowed = contraction_at(i - 2) == 3;
                    else if (sb[i - 2] == 0x99u && i >= 4) swallowed = contraction_at(i - 4) == 3;
                }
            }
            if (swallowed) continue;
            bool mark = false;
            if (c == PT_NEWLINE || p == PT_NEWLINE) mark = true;
            else if (c == PT_WS) mark = p != PT_WS;
            else if (p == PT_WS) mark = false;
            else if (p == PT_LETTER && contraction_at(i) > 0) mark = false;
            else if (pt_transition(p, c)) mark = true;
            else if (c == PT_DIGIT && p == PT_DIGIT) mark = run_before % 3u == 0u;
            if (mark) marks |= 1u << k;
        }
        // sixteen mask bytes per thread
        {
            const uint64_t g0 = (uint64_t)t0 + (uint64_t)threadIdx.x * PT_PER;
            if (g0 + PT_PER <= n && (reinterpret_cast<uintptr_t>(out + g0) & 15u) == 0u) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t m4 = (marks >> (4 * j)) & 15u;
                    w[j] = (m4 & 1u) | ((m4 & 2u) << 7) | ((m4 & 4u) << 14) | ((m4 & 8u) << 21);
                }
                *reinterpret_cast<uint4*>(out + g0) = make_uint4(w[0], w[1], w[2], w[3]);
            } else {
                for (int k = 0; k < PT_PER; k++) if (g0 + k < n) out[g0 + k] = (marks >> k) & 1u;
            }
        }
        __syncthreads();   // shared arrays are reused by the next tile
    }
}

// class tables on the device, once per GPU
struct DeviceTables { uint8_t* low = nullptr; uint32_t* ranges = nullptr; uint32_t n = 0; };
static DeviceTables g_tables[64];
static std::mutex g_tables_mutex;

static b200bpe_status tables_for(int device, ClassTables* out) {
    if (device < 0 || device >= 64) return B200BPE_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(g_tables_mutex);
    DeviceTables& t = g_tables[device];
    if (!t.low) {
        const uint32_t nr = (uint32_t)(sizeof(kClassRanges) / sizeof(kClassRanges[0]));
        std::string low(PT_LOW, (char)PT_OTHER);
        for (uint32_t r = 0; r < nr; r++)
            for (uint32_t cp = kClassRanges[r][0]; cp <= kClassRanges[r][1] && cp < PT_LOW; cp++) low[cp] = (char)kClassRanges[r][2];
        B2_CUDA(cudaMalloc(&t.low, PT_LOW));
        B2_CUDA(cudaMalloc(&t.ranges, sizeof(kClassRanges)));
        B2_CUDA(cudaMemcpy(t.low, low.data(), PT_LOW, cudaMemcpyHostToDevice));
        B2_CUDA(cudaMemcpy(t.ranges, kClassRanges, sizeof(kClassRanges), cudaMemcpyHostToDevice));
        t.n = nr;
    }
    out->low = t.low; out->ranges = t.ranges; out->n_ranges = t.n;
    return B200BPE_OK;
}

}  // namespace b200bpe

using namespace b200bpe;

extern "C" {

b200bpe_status b200bpe_pretokenize_device(b200bpe_ctx* c, const uint8_t* d_bytes, uint64_t n, uint8_t* d_word_starts_out) {
    return b200bpe_pretokenize_device_ex(c, d_bytes, n, d_word_starts_out, 0u);
}

b200bpe_status b200bpe_pretokenize_device_ex(b200bpe_ctx* c, const uint8_t* d_bytes, uint64_t n, uint8_t* d_word_starts_out,
                                             uint32_t test_lookback_spins) {
    if (!c || ((!d_bytes || !d_word_starts_out) && n)) return B200BPE_ERR_BAD_ARG;
    if (n == 0) return B200BPE_OK;
    B2_CUDA(cudaSetDevice(c->c.device));
    cudaStream_t s = c->c.stream;
    ClassTables tab{};
    b200bpe_status r = tables_for(c->c.device, &tab);
    if (r) return r;
    const uint64_t ntiles = (n + PT_TILE - 1) / PT_TILE;
    unsigned long long* desc = nullptr;
    uint32_t* ctl = nullptr;   // ticket, status
    B2_CUDA(cudaMalloc(&desc, ntiles * 8));
    if (cudaMalloc(&ctl, 8) != cudaSuccess) { cudaFree(desc); return B200BPE_ERR_OOM; }
    uint32_t h_ctl[2] = {0, 0};
    cudaMemsetAsync(desc, 0, ntiles * 8, s);
    cudaMemsetAsync(ctl, 0, 8, s);
    const bool stall = test_lookback_spins != 0u && test_lookback_spins < (1u << 20);
    if (stall) {   // the tile ticket starts at 1: tile 0 is never worked on and never publishes its digits
        static const uint32_t one = 1u;
        cudaMemcpyAsync(ctl, &one, 4, cudaMemcpyHostToDevice, s);
    }
    const int grid = (int)std::min<uint64_t>(ntiles, (uint64_t)c->c.sm_count * 8);
    k_pretokenize<<<grid, PT_THREADS, 0, s>>>(tab, d_bytes, n, d_word_starts_out, desc, ctl, ctl + 1, 1u,
                                              test_lookback_spins ? test_lookback_spins : PT_MAX_SPINS);
    cudaError_t e = cudaMemcpyAsync(h_ctl, ctl, 8, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFree(desc);
    cudaFree(ctl);
    if (e != cudaSuccess) { set_last_error(std::string("b200bpe_pretokenize_device: ") + cudaGetErrorString(e)); return B200BPE_ERR_CUDA; }
    if (h_ctl[1] == 2u) return B200BPE_ERR_LOOKBACK_TIMEOUT;
    if (h_ctl[1] == 1u) {
        set_last_error("b200bpe_pretokenize_device: the input is not well-formed UTF-8 (the host function b200bpe_pretokenize takes any bytes)");
        return B200BPE_ERR_BAD_ARG;
    }
    return B200BPE_OK;
}

b200bpe_status b200bpe_pretokenize_gpu(b200bpe_ctx* c, const uint8_t* bytes, uint64_t n, uint8_t* word_starts_out) {
    if (!c || ((!bytes || !word_starts_out) && n)) return B200BPE_ERR_BAD_ARG;
    if (n == 0) return B200BPE_OK;
    B2_CUDA(cudaSetDevice(c->c.device));
    cudaStream_t s = c->c.stream;
    uint8_t *d_in = nullptr, *d_out = nullptr;
    B2_CUDA(cudaMalloc(&d_in, n));
    if (cudaMalloc(&d_out, n) != cudaSuccess) { cudaFree(d_in); return B200BPE_ERR_OOM; }
    cudaMemcpyAsync(d_in, bytes, n, cudaMemcpyHostToDevice, s);
    b200bpe_status r = b200bpe_pretokenize_device(c, d_in, n, d_out);
    cudaError_t e = cudaSuccess;
    if (r == B200BPE_OK) {
        e = cudaMemcpyAsync(word_starts_out, d_out, n, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    }
    cudaFree(d_in);
    cudaFree(d_out);
    if (e != cudaSuccess) { set_last_error(std::string("b200bpe_pretokenize_gpu: ") + cudaGetErrorString(e)); return B200BPE_ERR_CUDA; }
    return r;
}

}  // extern "C"
