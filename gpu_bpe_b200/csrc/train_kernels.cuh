// Device kernels of the training merge loop.  One merge = three launches:
//
//   k_pair_count      adjacent-pair histogram of the live symbols into the open-addressing table
//                     (replaces bpe_clear_table + bpe_pair_count_b, train.wgsl:196-202,376-431)
//   k_argmax_setup    scan + clear of the table, arg-max with the reference's tie-break, and the
//                     single-thread merge set-up, all in one launch (replaces bpe_find_max_pair4,
//                     bpe_find_max_pair_final_det and bpe_setup_merge, train.wgsl:228-364)
//   k_merge_compact   snapshot merge + single-pass decoupled-look-back scan + stable compaction
//                     from the ping buffer into the pong buffer (replaces bpe_merge_reduce_b,
//                     bpe_prefix_sum_scan_blocks_* and bpe_finalize_compact_b, train.wgsl:457-731)
//
// Every kernel takes its sizes from the device control block, so a CUDA graph of many merges
// needs no host round trip; grids are persistent (a multiple of the SM count).
#pragma once

#include "common.cuh"

namespace b200bpe {

constexpr int PC_THREADS = 1024;     // pair count: threads per CTA
constexpr int PC_SLOTS_LOG2 = 13;    // pair count: shared-memory table slots per CTA (8192 * 12 B = 96 KB)
constexpr int PC_LOCAL_PROBES = 4;   // linear probes in shared memory before going to the global table
constexpr int TABLE_MAX_PROBE = 1024;
constexpr int AM_THREADS = 256;
constexpr int MC_THREADS = 256;
constexpr int MC_ROWS = 4;                               // uint4 rows per thread
constexpr int MC_TILE = MC_THREADS * 4 * MC_ROWS;        // 4096 symbols per tile
constexpr uint32_t LOOKBACK_MAX_SPINS = 1u << 22;        // bounded wait; then DS_LOOKBACK_TIMEOUT

__device__ __forceinline__ uint32_t hash_pair(unsigned long long key) {
    uint32_t x = (uint32_t)key ^ ((uint32_t)(key >> 32) * 0x9E3779B1u);
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}

// Larger count wins; equal counts go to the smaller (left, right) key — the same order as the
// reference's packed (a << 16 | b) comparison (train.wgsl:83-85).
__device__ __forceinline__ bool is_better(uint32_t cn, unsigned long long kn, uint32_t co, unsigned long long ko) {
    return cn > co || (cn == co && kn < ko);
}

// Add `c` to the count of `key` in the global table (insert on first sight).
__device__ __forceinline__ void table_add(PairSlot* __restrict__ table, uint32_t logC, unsigned long long key,
                                          uint32_t h, uint32_t c, DevState* st) {
    const uint32_t mask = (1u << logC) - 1u;
    uint32_t slot = h >> (32 - logC);
    for (int p = 0; p < TABLE_MAX_PROBE; p++) {
        unsigned long long k = __ldcg(&table[slot].key);
        if (k == 0ull) {
            k = atomicCAS(&table[slot].key, 0ull, key);
            if (k == 0ull) k = key;
        }
        if (k == key) {
            atomicAdd(&table[slot].count, c);
            return;
        }
        slot = (slot + 1) & mask;
    }
    atomicExch(&st->status, (uint32_t)DS_TABLE_FULL);
}

// ─────────────────────────────── pair count ───────────────────────────────
// Each CTA owns one contiguous span of the symbol array, reads it with 16-byte loads, and
// aggregates pairs in a shared-memory table; whatever does not fit there after a few probes
// goes straight to the global table with one atomic per distinct key per warp.  At the end the
// shared table is flushed, one global add per occupied slot.
template <int S_LOG2, int THREADS>
__global__ void __launch_bounds__(THREADS)
k_pair_count(DevState* __restrict__ st, const uint32_t* __restrict__ buf0, const uint32_t* __restrict__ buf1,
             PairSlot* __restrict__ table) {
    constexpr int S = 1 << S_LOG2;
    extern __shared__ __align__(16) unsigned char pc_smem[];
    unsigned long long* skey = reinterpret_cast<unsigned long long*>(pc_smem);
    uint32_t* scnt = reinterpret_cast<uint32_t*>(skey + S);

    // One thread reads the stop flags for the whole CTA: `status` can change while this kernel
    // runs (another CTA may find the table full), and a CTA must not split at a barrier.
    __shared__ uint32_t s_idle;
    if (threadIdx.x == 0) s_idle = st->early_stop | st->target_hit | st->status;
    for (int i = threadIdx.x; i < S; i += THREADS) { skey[i] = 0ull; scnt[i] = 0u; }
    __syncthreads();
    if (s_idle) return;
    const uint32_t e = st->epoch;
    const uint32_t N = st->n[e & 1];
    const uint32_t* __restrict__ src = (e & 1) ? buf1 : buf0;
    const uint32_t logC = st->table_log2;

    const uint32_t nvec = (N + 3u) >> 2;
    uint32_t per = (nvec + gridDim.x - 1) / gridDim.x;
    per = (per + 31u) & ~31u;
    const uint32_t v0 = min(nvec, blockIdx.x * per);
    const uint32_t v1 = min(nvec, v0 + per);
    const uint4* __restrict__ src4 = reinterpret_cast<const uint4*>(src);
    const int lane = threadIdx.x & 31;

    for (uint32_t vb = v0 + (threadIdx.x & ~31u); vb < v1; vb += THREADS) {
        const uint32_t v = vb + lane;
        const bool in = v < v1;
        uint4 q = make_uint4(WORD_START_BIT, WORD_START_BIT, WORD_START_BIT, WORD_START_BIT);
        if (in) q = __ldcs(src4 + v);
        uint32_t nx = __shfl_down_sync(0xFFFFFFFFu, q.x, 1);
        if (lane == 31 || v + 1 >= v1) {
            const uint32_t i4 = 4u * (v + 1u);
            nx = (in && i4 < N) ? __ldg(src + i4) : WORD_START_BIT;
        }
        const uint32_t rem = in ? (N - 4u * v) : 0u;  // symbols of this vector that are live
        const uint32_t s[5] = {q.x, q.y, q.z, q.w, nx};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t a = s[j] & TOKEN_MASK, rb = s[j + 1], b = rb & TOKEN_MASK;
            const bool ok = ((uint32_t)(j + 1) < rem) && !(rb & WORD_START_BIT) && a != 0u && b != 0u;
            const unsigned long long key = ((unsigned long long)a << 32) | b;
            const uint32_t h = hash_pair(key);
            bool pending = ok;
            if (ok) {
                uint32_t slot = h & (S - 1);
#pragma unroll
                for (int p = 0; p < PC_LOCAL_PROBES; p++) {
                    unsigned long long k = skey[slot];
                    if (k == 0ull) {
                        k = atomicCAS(&skey[slot], 0ull, key);
                        if (k == 0ull) k = key;
                    }
                    if (k == key) {
                        atomicAdd(&scnt[slot], 1u);
                        pending = false;
                        break;
                    }
                    slot = (slot + 1) & (S - 1);
                }
            }
            // Overflow: one global add per distinct key among the pending lanes of this warp.
            const uint32_t pend = __ballot_sync(0xFFFFFFFFu, pending);
            if (pending) {
                const uint32_t peers = __match_any_sync(pend, key);
                if (lane == __ffs(peers) - 1) table_add(table, logC, key, h, __popc(peers), st);
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < S; i += THREADS) {
        const uint32_t c = scnt[i];
        if (c) {
            const unsigned long long key = skey[i];
            table_add(table, logC, key, hash_pair(key), c, st);
        }
    }
}

// ─────────────────────────────── arg-max + clear + set-up ───────────────────────────────
__device__ __forceinline__ void warp_best(uint32_t& c, unsigned long long& k) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const uint32_t oc = __shfl_xor_sync(0xFFFFFFFFu, c, o);
        const unsigned long long ok = __shfl_xor_sync(0xFFFFFFFFu, k, o);
        if (is_better(oc, ok, c, k)) { c = oc; k = ok; }
    }
}

// The merge set-up of the reference (train.wgsl:340-364) plus this library's batch control.
__device__ __forceinline__ void setup_merge(DevState* st, uint32_t best_count, unsigned long long best_key,
                                            uint32_t* __restrict__ log) {
    if (st->status != DS_OK) { st->active = 0; return; }
    if (best_count < 2u || st->next_id > TOKEN_MASK) {
        st->early_stop = 1u;
        st->active = 0u;
        return;
    }
    const uint32_t a = (uint32_t)(best_key >> 32), b = (uint32_t)best_key;
    st->a = a; st->b = b; st->max_count = best_count; st->new_id = st->next_id;
    const uint32_t md = st->merges_done;
    log[md * 4 + 0] = a; log[md * 4 + 1] = b; log[md * 4 + 2] = st->next_id; log[md * 4 + 3] = best_count;
    st->next_id += 1u;
    st->merges_done = md + 1u;
    if (md + 1u >= st->merges_target) st->target_hit = 1u;
    st->k3_epoch = st->epoch;
    st->ticket = 0u;
    st->active = 1u;
}

// mode 0: single GPU — finish with setup_merge.
// mode 1: sharded — the last CTA only publishes this rank's best as a packed word for the
//         all-reduce (count << 32 | ~pair32); k_unpack_flags finishes after the collective.
__global__ void __launch_bounds__(AM_THREADS)
k_argmax_setup(DevState* __restrict__ st, PairSlot* __restrict__ table, CtaBest* __restrict__ cta_best,
               uint32_t* __restrict__ log, int mode) {
    __shared__ uint32_t sc[AM_THREADS / 32];
    __shared__ unsigned long long sk[AM_THREADS / 32];
    __shared__ uint32_t socc[AM_THREADS / 32];
    __shared__ bool is_last;
    // Neither flag changes before every CTA has passed this test: only the last CTA to finish
    // writes them.  Once the run has stopped, nothing is left for the merge kernel to apply.
    if (st->early_stop | st->target_hit) {
        if (blockIdx.x == 0 && threadIdx.x == 0) st->active = 0u;
        return;
    }
    const uint32_t C = 1u << st->table_log2;
    uint4* __restrict__ t4 = reinterpret_cast<uint4*>(table);
    uint32_t bc = 0, occ = 0;
    unsigned long long bk = 0ull;
    for (uint32_t i = blockIdx.x * AM_THREADS + threadIdx.x; i < C; i += gridDim.x * AM_THREADS) {
        const uint4 q = __ldcg(t4 + i);
        const unsigned long long key = ((unsigned long long)q.y << 32) | q.x;
        if (key != 0ull) {
            occ++;
            if (is_better(q.z, key, bc, bk)) { bc = q.z; bk = key; }
            __stcg(t4 + i, make_uint4(0u, 0u, 0u, 0u));
        }
    }
    warp_best(bc, bk);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) occ += __shfl_xor_sync(0xFFFFFFFFu, occ, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sc[warp] = bc; sk[warp] = bk; socc[warp] = occ; }
    __syncthreads();
    if (warp == 0) {
        bc = lane < AM_THREADS / 32 ? sc[lane] : 0u;
        bk = lane < AM_THREADS / 32 ? sk[lane] : 0ull;
        occ = lane < AM_THREADS / 32 ? socc[lane] : 0u;
        warp_best(bc, bk);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) occ += __shfl_xor_sync(0xFFFFFFFFu, occ, o);
        if (lane == 0) {
            cta_best[blockIdx.x].key = bk;
            cta_best[blockIdx.x].count = bc;
            cta_best[blockIdx.x].pad = occ;
            __threadfence();
            const uint32_t t = atomicAdd(&st->argmax_done, 1u);
            is_last = (t == gridDim.x - 1);
        }
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    bc = 0; bk = 0ull; occ = 0;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += AM_THREADS) {
        const uint32_t c = __ldcg(&cta_best[i].count);
        const unsigned long long k = __ldcg(&cta_best[i].key);
        occ += __ldcg(&cta_best[i].pad);
        if (is_better(c, k, bc, bk)) { bc = c; bk = k; }
    }
    warp_best(bc, bk);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) occ += __shfl_xor_sync(0xFFFFFFFFu, occ, o);
    __syncthreads();
    if (lane == 0) { sc[warp] = bc; sk[warp] = bk; socc[warp] = occ; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < AM_THREADS / 32; w++) {
            if (is_better(sc[w], sk[w], bc, bk)) { bc = sc[w]; bk = sk[w]; }
            occ += socc[w];
        }
        st->argmax_done = 0u;
        st->occupied = occ;
        if ((unsigned long long)occ * 2ull > (unsigned long long)C) st->want_grow = 1u;
        if (mode == 0) {
            setup_merge(st, bc, bk, log);
        } else {
            const uint32_t pair32 = ((uint32_t)(bk >> 32) << 16) | ((uint32_t)bk & 0xFFFFu);
            st->best_packed = ((unsigned long long)bc << 32) | (unsigned long long)(~pair32);
        }
    }
}

// ─────────────────────────────── merge + scan + compaction ───────────────────────────────
// Tile descriptor of the decoupled look-back: high word = (tag << 2) | flag, low word = value.
// The tag is the merge number + 1, so descriptors left by earlier merges read as "not ready"
// and the array never needs clearing.
constexpr uint32_t DESC_AGG = 1u, DESC_PREFIX = 2u;

__device__ __forceinline__ unsigned long long ld_desc(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_desc(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

template <bool LITERAL>
__global__ void __launch_bounds__(MC_THREADS)
k_merge_compact(DevState* __restrict__ st, uint32_t* buf0, uint32_t* buf1, unsigned long long* __restrict__ desc) {
    __shared__ uint32_t wsum[MC_ROWS * (MC_THREADS / 32)];
    __shared__ uint32_t s_tile, s_base;
    // `active`, `k3_epoch`, `n[k3_epoch & 1]`, `a`, `b`, `new_id` and `max_count` are written by the
    // set-up step only, so every thread of every CTA of this launch reads the same values.
    if (!st->active) return;
    const uint32_t e = st->k3_epoch;
    const uint32_t N = st->n[e & 1];
    uint32_t* src = (e & 1) ? buf1 : buf0;
    uint32_t* __restrict__ dst = (e & 1) ? buf0 : buf1;
    const uint32_t A = st->a, B = st->b, NW = st->new_id;
    const uint32_t limit = LITERAL ? (N - st->max_count) : N;
    const uint32_t ntiles = (N + MC_TILE - 1) / MC_TILE;
    const uint32_t tag = (e + 1u) & 0x3FFFFFFFu;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint4* src4 = reinterpret_cast<const uint4*>(src);

    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) s_tile = atomicAdd(&st->ticket, 1u);
        __syncthreads();
        const uint32_t tile = s_tile;
        if (tile >= ntiles) break;
        const uint32_t vbase = tile * (MC_TILE / 4);

        uint4 q[MC_ROWS];
        uint32_t pv[MC_ROWS], nx[MC_ROWS];
#pragma unroll
        for (int j = 0; j < MC_ROWS; j++) {
            const uint32_t v = vbase + j * MC_THREADS + threadIdx.x;
            const uint32_t i = 4u * v;
            q[j] = (i < N) ? src4[v] : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < MC_ROWS; j++) {
            const uint32_t v = vbase + j * MC_THREADS + threadIdx.x;
            const uint32_t i = 4u * v;
            pv[j] = __shfl_up_sync(0xFFFFFFFFu, q[j].w, 1);
            nx[j] = __shfl_down_sync(0xFFFFFFFFu, q[j].x, 1);
            if (lane == 0) pv[j] = (i > 0u && i - 1u < N) ? src[i - 1u] : 0u;
            if (lane == 31) nx[j] = (i + 4u < N) ? src[i + 4u] : 0u;
            if (LITERAL) {
                // A neighbour owned by another thread may already carry this merge's in-place
                // rewrite; the new id is fresh, so mapping it back to `a` restores the snapshot.
                if ((pv[j] & TOKEN_MASK) == NW) pv[j] = (pv[j] & WORD_START_BIT) | A;
                if ((nx[j] & TOKEN_MASK) == NW) nx[j] = (nx[j] & WORD_START_BIT) | A;
            }
        }

        uint32_t outv[MC_ROWS][4];
        uint32_t keep[MC_ROWS];  // 4 keep bits per row
        uint32_t lane_excl[MC_ROWS];
#pragma unroll
        for (int j = 0; j < MC_ROWS; j++) {
            const uint32_t i0 = 4u * (vbase + j * MC_THREADS + threadIdx.x);
            const uint32_t s[6] = {pv[j], q[j].x, q[j].y, q[j].z, q[j].w, nx[j]};
            uint32_t kb = 0u;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const uint32_t i = i0 + k;
                const uint32_t cur = s[k + 1], prv = s[k], nxt = s[k + 2];
                const bool inr = i < N;
                const bool match_a = inr && (i + 1u < N) && !(nxt & WORD_START_BIT) &&
                                     (cur & TOKEN_MASK) == A && (nxt & TOKEN_MASK) == B;
                const bool invalid = (i > 0u) && !(cur & WORD_START_BIT) && (prv & TOKEN_MASK) == A &&
                                     (cur & TOKEN_MASK) == B;
                const uint32_t ov = match_a ? (NW | (cur & WORD_START_BIT)) : cur;
                outv[j][k] = ov;
                if (inr && !invalid && i < limit) kb |= 1u << k;
                if (LITERAL && match_a) src[i] = ov;  // the reference rewrites the source in place
            }
            keep[j] = kb;
            uint32_t c = __popc(kb), incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += t;
            }
            lane_excl[j] = incl - c;
            if (lane == 31) wsum[j * (MC_THREADS / 32) + warp] = incl;
        }
        __syncthreads();
        if (warp == 0) {
            // 32 warp-row totals in index order → exclusive offsets + tile aggregate
            const uint32_t w = wsum[lane];
            uint32_t incl = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += t;
            }
            wsum[lane] = incl - w;
            const uint32_t agg = __shfl_sync(0xFFFFFFFFu, incl, 31);
            uint32_t excl = 0u;
            if (tile == 0u) {
                if (lane == 0) st_desc(desc, ((unsigned long long)((tag << 2) | DESC_PREFIX) << 32) | agg);
            } else {
                if (lane == 0) st_desc(desc + tile, ((unsigned long long)((tag << 2) | DESC_AGG) << 32) | agg);
                int pos = (int)tile - 1;
                uint32_t spins = 0;
                bool timed_out = false;
                for (;;) {
                    const int idx = pos - lane;
                    unsigned long long d = 0ull;
                    uint32_t hi = (tag << 2) | DESC_PREFIX;  // positions before tile 0 act as a zero prefix
                    uint32_t val = 0u;
                    for (;;) {
                        if (idx >= 0) {
                            d = ld_desc(desc + idx);
                            hi = (uint32_t)(d >> 32);
                            val = (uint32_t)d;
                        }
                        const bool ready = ((hi >> 2) == tag) && (hi & 3u) != 0u;
                        if (__all_sync(0xFFFFFFFFu, ready)) break;
                        if (++spins > LOOKBACK_MAX_SPINS) { timed_out = true; break; }
                        __nanosleep(40);
                    }
                    if (timed_out) break;
                    const uint32_t pmask = __ballot_sync(0xFFFFFFFFu, (hi & 3u) == DESC_PREFIX);
                    const int first = pmask ? (__ffs(pmask) - 1) : 32;  // nearest predecessor holding a full prefix
                    uint32_t contrib = (lane <= first) ? val : 0u;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xFFFFFFFFu, contrib, o);
                    excl += contrib;
                    if (pmask) break;
                    pos -= 32;
                }
                if (timed_out) {
                    if (lane == 0) atomicExch(&st->status, (uint32_t)DS_LOOKBACK_TIMEOUT);
                    excl = 0u;
                }
                if (lane == 0) st_desc(desc + tile, ((unsigned long long)((tag << 2) | DESC_PREFIX) << 32) | (excl + agg));
            }
            if (lane == 0) {
                s_base = excl;
                if (tile == ntiles - 1u) {
                    // Last tile: publish the new symbol count and advance the epoch.
                    const uint32_t total = excl + agg;
                    const uint32_t nnew = N - st->max_count;
                    if (!LITERAL && total != nnew && st->status == DS_OK && st->world == 1u)
                        atomicExch(&st->status, (uint32_t)DS_INTERNAL);
                    st->n[(e + 1u) & 1u] = LITERAL ? nnew : total;
                    st->epoch = e + 1u;
                }
            }
        }
        __syncthreads();
        const uint32_t base = s_base;
#pragma unroll
        for (int j = 0; j < MC_ROWS; j++) {
            uint32_t d = base + wsum[j * (MC_THREADS / 32) + warp] + lane_excl[j];
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (keep[j] & (1u << k)) dst[d++] = outv[j][k];
        }
    }
}

// ─────────────────────────────── symbol buffer set-up ───────────────────────────────
// bytes (+ optional word-start mask) → u32 symbols with bit 16 on word starts
// (trainer.js:76-79,115-121).  With no mask, the byte-class heuristic of bpe_word_boundary
// (train.wgsl:111-186) decides.
__device__ __forceinline__ uint32_t byte_class(uint32_t t) {
    if (t == 0x0Au) return 4u;
    if (t == 0x20u) return 2u;
    if (t - 0x30u <= 9u) return 1u;
    if (t >= 0x80u) return 0u;
    if (t - 0x61u <= 25u) return 0u;
    if (t - 0x41u <= 25u) return 0u;
    return 3u;
}

__global__ void __launch_bounds__(256)
k_tag_symbols(const uint8_t* __restrict__ bytes, const uint8_t* __restrict__ mask, uint32_t* __restrict__ sym,
              uint64_t n) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint32_t t = bytes[i];
        bool ws;
        if (mask) {
            ws = mask[i] != 0;
        } else if (i == 0) {
            ws = true;
        } else {
            const uint32_t c = byte_class(t), p = byte_class(bytes[i - 1]);
            ws = c != p;
            if (p == 2u && (c == 0u || c == 1u)) ws = false;
            if (c == 2u && p != 2u) ws = true;
            if (p == 4u || c == 4u) ws = true;
        }
        sym[i] = t | (ws ? WORD_START_BIT : 0u);
    }
}

// Copy the non-empty slots of the table out (and empty them), for tests.
__global__ void k_dump_table(PairSlot* table, uint32_t C, unsigned long long* keys, uint32_t* counts, uint32_t cap,
                             uint32_t* n_out) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < C; i += gridDim.x * blockDim.x) {
        const unsigned long long k = table[i].key;
        if (k) {
            const uint32_t d = atomicAdd(n_out, 1u);
            if (d < cap) { keys[d] = k; counts[d] = table[i].count; }
            table[i].key = 0ull; table[i].count = 0u;
        }
    }
}

}  // namespace b200bpe
