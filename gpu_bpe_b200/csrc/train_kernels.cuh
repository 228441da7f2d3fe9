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
constexpr int PC_SLOTS = 12288;      // pair count: shared-memory slots per CTA (8 B each = 96 KB: two CTAs per SM)
constexpr int PC_CTAS_PER_SM = 2;
constexpr int PC_SMEM_BYTES = PC_SLOTS * 8;
constexpr int PC_IDLE_CTAS = 64;     // pair count: CTAs that stay when there is nothing to count (literal tail fix, next merge)
constexpr int PC_LOCAL_PROBES = 2;   // linear probes in shared memory before going to the global table
constexpr int TABLE_MAX_PROBE = 1024;
constexpr int AM_THREADS = 256;
#ifndef B200BPE_MC_THREADS
#define B200BPE_MC_THREADS 256
#endif
constexpr int MC_THREADS = B200BPE_MC_THREADS;   // merge kernel: threads per CTA
#ifndef B200BPE_MC_ROWS
#define B200BPE_MC_ROWS 4
#endif
#ifndef B200BPE_MC_SUBS
#define B200BPE_MC_SUBS 3
#endif
#ifndef B200BPE_MC_NBUF
#define B200BPE_MC_NBUF 2
#endif
#ifndef B200BPE_MC_UNROLL
#define B200BPE_MC_UNROLL 0
#endif
#if B200BPE_MC_UNROLL
#define MC_UNROLL_SUBS _Pragma("unroll")
#else
#define MC_UNROLL_SUBS _Pragma("unroll 1")
#endif
#ifndef B200BPE_MC_CTAS
#define B200BPE_MC_CTAS 2
#endif
constexpr int MC_ROWS = B200BPE_MC_ROWS;                 // uint4 rows per thread per sub-tile (1..4)
constexpr int MC_SUB = MC_THREADS * 4 * MC_ROWS;         // symbols per sub-tile
constexpr int MC_SUBS = B200BPE_MC_SUBS;                 // sub-tiles per tile (1..4)
constexpr int MC_TILE = MC_SUB * MC_SUBS;                // symbols per tile: one look-back each
constexpr int MC_NBUF = B200BPE_MC_NBUF;                 // tile buffers per CTA (the pipeline needs at least two)
constexpr int MC_CTAS_PER_SM = B200BPE_MC_CTAS;
constexpr int MC_SMEM_BYTES = MC_NBUF * (MC_TILE + 8) * 4;  // the tiles and their edges (dynamic shared memory)
// Per row of a span the decisions of pass 1 take one byte of a word; these masks select the bytes of the rows in use.
constexpr uint32_t MC_ROWBYTES = MC_ROWS == 4 ? 0xFFFFFFFFu : ((1u << (8 * (MC_ROWS & 3))) - 1u);  // bytes 0..ROWS-1
constexpr uint32_t MC_KEEP_ALL = 0x0F0F0F0Fu & MC_ROWBYTES;                        // every own symbol kept
constexpr uint32_t MC_NOTLAST = MC_ROWBYTES >> 8;                                  // bytes 0..ROWS-2
constexpr int MC_LASTROW_SHIFT = 8 * (MC_ROWS - 1);                                // bit 0 of the last row's byte
static_assert(MC_NBUF >= 2 && MC_ROWS >= 1 && MC_ROWS <= 4 && MC_SUBS >= 1 && MC_SUBS <= 4, "merge kernel shape");
constexpr int MC_WARPS = MC_THREADS / 32;
constexpr uint32_t LOOKBACK_MAX_SPINS = 1u << 22;        // bounded wait; then DS_LOOKBACK_TIMEOUT
constexpr uint32_t BULK_MAX_SPINS = 1u << 20;            // bounded wait for a bulk copy; then DS_LOOKBACK_TIMEOUT

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

// Add `c` to the count of `key` in the global table (insert on first sight).  `tau` is the
// threshold of the arg-max candidate list (DevState.cand_tau, read once by the caller): an increase
// that takes a count across it appends the slot to the list.  Decreases need no answer from the
// atomic unit and are sent as reductions.
__device__ __forceinline__ void table_add(PairSlot* __restrict__ table, uint32_t logC, unsigned long long key,
                                          uint32_t h, uint32_t c, DevState* st, uint32_t tau) {
    const uint32_t mask = (1u << logC) - 1u;
    uint32_t slot = h >> (32 - logC);
    for (int p = 0; p < TABLE_MAX_PROBE; p++) {
        unsigned long long k = __ldcg(&table[slot].key);
        if (k == 0ull) {
            k = atomicCAS(&table[slot].key, 0ull, key);
            if (k == 0ull) k = key;
        }
        if (k == key) {
            if (c >= 0x80000000u || tau == 0xFFFFFFFFu) {
                atomicAdd(&table[slot].count, c);
            } else {
                const uint32_t old = atomicAdd(&table[slot].count, c);
                if (old < tau && old + c >= tau) {
                    const uint32_t i = atomicAdd(&st->cand_n, 1u);
                    if (i < CAND_CAP) st->cand[i] = slot;
                }
            }
            return;
        }
        slot = (slot + 1) & mask;
    }
    atomicExch(&st->status, (uint32_t)DS_TABLE_FULL);
}
__device__ __forceinline__ void table_add(PairSlot* __restrict__ table, uint32_t logC, unsigned long long key,
                                          uint32_t h, uint32_t c, DevState* st) {
    table_add(table, logC, key, h, c, st, c >= 0x80000000u ? 0xFFFFFFFFu : st->cand_tau);
}
// Sharded runs with the peer-memory exchange: the local table only collects the signed pair deltas
// of one merge (it is emptied when they are sent to the pairs' owners); the first entry of a slot
// appends the slot to the list of slots to send.
constexpr uint32_t DLIST_CAP = 1u << 20;
__device__ __forceinline__ void delta_add(PairSlot* __restrict__ table, uint32_t logC, unsigned long long key, uint32_t h,
                                          uint32_t c, DevState* st) {
    const uint32_t mask = (1u << logC) - 1u;
    uint32_t slot = h >> (32 - logC);
    for (int p = 0; p < TABLE_MAX_PROBE; p++) {
        unsigned long long k = __ldcg(&table[slot].key);
        if (k == 0ull) {
            k = atomicCAS(&table[slot].key, 0ull, key);
            if (k == 0ull) {
                k = key;
                const uint32_t i = atomicAdd(&st->dlist_n, 1u);
                if (i < DLIST_CAP) st->dlist[i] = slot;
                else atomicExch(&st->status, (uint32_t)DS_TABLE_FULL);
            }
        }
        if (k == key) { atomicAdd(&table[slot].count, c); return; }
        slot = (slot + 1) & mask;
    }
    atomicExch(&st->status, (uint32_t)DS_TABLE_FULL);
}

// No usable candidate list: every arg-max from iteration `from` on scans the whole table, until one
// of those scans has built a new list.
__device__ __forceinline__ void void_candidates(DevState* st, uint32_t from) {
    st->scan_from = from;
    st->cand_tau = 0xFFFFFFFFu;
    st->cand_n = 0u;
}

// Literal mode with an incrementally maintained table: k_merge_compact accounts for the merge as
// if every kept symbol had been copied; the reference, however, copies only the inputs below
// limit = N - count and leaves older contents in the rest of the destination (train.wgsl:698,727).
// This takes out the pairs of the symbols that were not copied and puts in the pairs of what the
// destination holds instead.  src = the merge's source buffer after its in-place rewrites, dst =
// its destination; V = symbols copied, N1 = the new symbol count.  Called by every thread of a
// grid after the merge kernel of that merge and before the next arg-max: by the next merge's
// count kernel (which has nothing else to do while the table is maintained incrementally), or by
// k_literal_tail at the end of a batch.  `tail_fix` is rewritten by the next set-up step, after
// every caller of the grid has read it.
__device__ __forceinline__ void literal_tail_fix(DevState* __restrict__ st, const DevState* rd, const uint32_t* buf0,
                                                 const uint32_t* buf1, PairSlot* table, uint32_t nblocks) {
    // `rd`: the control block, or the caller's copy of it (nothing read here changes meanwhile)
    if (table == nullptr) table = rd->table;
    const uint32_t e = rd->k3_epoch;   // the merge just applied; `epoch` is already one further
    const uint32_t N = rd->n[e & 1], N1 = rd->n[(e + 1u) & 1u], V = rd->v_kept;
    const uint32_t* __restrict__ src = (e & 1) ? buf1 : buf0;
    const uint32_t* __restrict__ dst = (e & 1) ? buf0 : buf1;
    const uint32_t B = rd->b, NW = rd->new_id, limit = N - rd->max_count;
    const uint32_t logC = rd->table_log2;
    const uint32_t tau = rd->cand_tau;
    auto counted = [](uint32_t l, uint32_t r) { return !(r & WORD_START_BIT) && (l & TOKEN_MASK) != 0u && (r & TOKEN_MASK) != 0u; };
    auto emit = [&](uint32_t l, uint32_t r, uint32_t delta) {
        const unsigned long long key = ((unsigned long long)(l & TOKEN_MASK) << 32) | (r & TOKEN_MASK);
        table_add(table, logC, key, hash_pair(key), delta, st, tau);
    };
    // a position of the source is dropped iff its left neighbour was rewritten to the new symbol
    auto drops = [&](uint32_t left, uint32_t cur) { return (left & TOKEN_MASK) == NW && !(cur & WORD_START_BIT) && (cur & TOKEN_MASK) == B; };
    const uint32_t gtid = blockIdx.x * blockDim.x + threadIdx.x, gstride = nblocks * blockDim.x;   // blocks 0..nblocks-1 take part
    // (1) pairs whose left symbol is a kept source position >= limit: they were counted, but never
    // copied.  The four symbols around a position are loaded together (one round trip).
    for (uint32_t i = limit + gtid; i < N; i += gstride) {
        const uint32_t sm = i > 0u ? __ldcg(src + i - 1u) : 0u, s0 = __ldcg(src + i);
        const uint32_t s1 = i + 1u < N ? __ldcg(src + i + 1u) : 0u, s2 = i + 2u < N ? __ldcg(src + i + 2u) : 0u;
        if (i > 0u && drops(sm, s0)) continue;
        const bool d1 = i + 1u < N && drops(s0, s1);
        const uint32_t r = d1 ? i + 2u : i + 1u, sr = d1 ? s2 : s1;
        if (r < N && counted(s0, sr)) emit(s0, sr, 0xFFFFFFFFu);
    }
    // (2) the pair that joined the last copied symbol to the first kept source position >= limit
    if (gtid == 0 && V > 0u && limit < N) {
        const uint32_t sm = limit > 0u ? __ldcg(src + limit - 1u) : 0u, s0 = __ldcg(src + limit);
        const uint32_t s1 = limit + 1u < N ? __ldcg(src + limit + 1u) : 0u, last = __ldcg(dst + V - 1u);
        const bool d0 = limit > 0u && drops(sm, s0);
        const uint32_t z0 = d0 ? limit + 1u : limit, sz = d0 ? s1 : s0;
        if (z0 < N && counted(last, sz)) emit(last, sz, 0xFFFFFFFFu);
    }
    // (3) the pairs of what the destination really holds from the last copied symbol on
    for (uint32_t u = (V > 0u ? V - 1u : 0u) + gtid; u + 1u < N1; u += gstride) {
        const uint32_t l = __ldcg(dst + u), r = __ldcg(dst + u + 1u);
        if (counted(l, r)) emit(l, r, 1u);
    }
}

__global__ void __launch_bounds__(256)
k_literal_tail(DevState* __restrict__ st, const uint32_t* buf0, const uint32_t* buf1, PairSlot* table) {
    if (st->tail_fix) literal_tail_fix(st, st, buf0, buf1, table, gridDim.x);
}

// ─────────────────────────────── pair count ───────────────────────────────
// Each CTA owns one contiguous span of the symbol array and reads it with 16-byte loads.
// Pairs are first aggregated in a shared-memory table: 32-bit keys (left << 16 | right) and
// 32-bit counts in two arrays, so a hit costs one 32-bit shared load and one native 32-bit shared
// atomic add.  A pair that finds no room within a few probes goes straight to the global table,
// one atomic per distinct key per warp (match-any aggregation).  At the end the shared table is
// flushed into the global table of 64-bit (left << 32 | right) keys, one add per occupied slot.
__device__ __forceinline__ uint32_t smem_slot(uint32_t key32, uint32_t nslots) {
    return __umulhi(key32 * 0x9E3779B1u, nslots);
}

__device__ __forceinline__ bool smem_count(uint32_t* __restrict__ skey, uint32_t* __restrict__ scnt, uint32_t nslots,
                                           uint32_t key32) {
    uint32_t slot = smem_slot(key32, nslots);
#pragma unroll
    for (int p = 0; p < PC_LOCAL_PROBES; p++) {
        uint32_t cur = skey[slot];
        if (cur == 0u) {
            cur = atomicCAS(&skey[slot], 0u, key32);
            if (cur == 0u) cur = key32;
        }
        if (cur == key32) {
            atomicAdd(&scnt[slot], 1u);
            return true;
        }
        slot = slot + 1 == nslots ? 0u : slot + 1;
    }
    return false;
}

__device__ __forceinline__ void warp_best(uint32_t& c, unsigned long long& k);
__device__ __forceinline__ void void_candidates(DevState* st, uint32_t from);
__device__ __forceinline__ void setup_merge(DevState* st, const DevState* rd, uint32_t best_count,
                                            unsigned long long best_key, uint32_t* __restrict__ log);

template <int S, int THREADS>
__global__ void __launch_bounds__(THREADS, PC_CTAS_PER_SM)
k_pair_count(DevState* __restrict__ st, const uint32_t* __restrict__ buf0, const uint32_t* __restrict__ buf1,
             PairSlot* table, uint32_t* __restrict__ log) {
    extern __shared__ __align__(16) unsigned char pc_smem[];
    uint32_t* skey = reinterpret_cast<uint32_t*>(pc_smem);
    uint32_t* scnt = skey + S;

    // One copy of the control block per CTA (one 16-byte load per thread, one round trip), and one
    // thread decides for the whole CTA: `status` can change while this kernel runs (another CTA may
    // find the table full), and a CTA must not split at a barrier.
    __shared__ __align__(16) DevState snap;
    __shared__ uint32_t s_idle, s_tail, s_fuse, s_last;
    __shared__ uint32_t r_c[THREADS / 32];
    __shared__ unsigned long long r_k[THREADS / 32];
    static_assert(sizeof(DevState) % 16 == 0 && sizeof(DevState) / 16 <= THREADS, "control block copy");
    if (threadIdx.x < sizeof(DevState) / 16)
        reinterpret_cast<uint4*>(&snap)[threadIdx.x] = __ldcg(reinterpret_cast<const uint4*>(st) + threadIdx.x);
    __syncthreads();
    if (threadIdx.x == 0) {
        s_idle = snap.early_stop | snap.target_hit | snap.status | (snap.incremental & (snap.recount ^ 1u));
        s_tail = snap.tail_fix;
        // Nothing to count and a usable candidate list: the last CTA of this launch to finish can
        // pick the next merge right here, and the arg-max kernel of this iteration has nothing to do.
        s_fuse = (snap.incremental != 0u && snap.world == 1u && snap.recount == 0u && snap.iter_no < snap.scan_from &&
                  snap.early_stop == 0u && snap.target_hit == 0u && snap.status == DS_OK) ? 1u : 0u;
    }
    __syncthreads();
    // literal mode, incremental table: finish the table update of the merge before this one.  When
    // there is nothing to count, a part of the grid is plenty for that (the tail is as long as the
    // merged pair's count) and the other CTAs have nothing to do.
    const uint32_t workers = s_idle ? min(gridDim.x, (uint32_t)PC_IDLE_CTAS) : gridDim.x;
    if (s_tail && blockIdx.x < workers) literal_tail_fix(st, &snap, buf0, buf1, table, workers);
    if (s_idle) {
        if (!s_fuse) return;
        // Every CTA of the launch arrives here, workers or not, and the one that arrives last picks
        // the merge: by then every CTA has taken its copy of the control block, so what the pick
        // writes cannot send a late CTA down another branch.  (k1_done is put back to zero by the
        // merge kernel of the iteration.)
        __threadfence();   // this CTA's table updates and list entries are out before it is counted as done
        __syncthreads();
        if (threadIdx.x == 0) s_last = (atomicAdd(&st->k1_done, 1u) == gridDim.x - 1u) ? 1u : 0u;
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        PairSlot* tab = table ? table : snap.table;
        const uint4* __restrict__ t4 = reinterpret_cast<const uint4*>(tab);
        const uint32_t cand_n = __ldcg(&st->cand_n);   // the tail fix may have appended
        const uint32_t n = min(cand_n, CAND_CAP);
        uint32_t bc = 0u;
        unsigned long long bk = 0ull;
        for (uint32_t i = threadIdx.x; i < n; i += THREADS) {
            const uint4 q = __ldcg(t4 + __ldcg(snap.cand + i));
            const unsigned long long key = ((unsigned long long)q.y << 32) | q.x;
            if (key != 0ull && is_better(q.z, key, bc, bk)) { bc = q.z; bk = key; }
        }
        warp_best(bc, bk);
        if ((threadIdx.x & 31) == 0) { r_c[threadIdx.x >> 5] = bc; r_k[threadIdx.x >> 5] = bk; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < THREADS / 32; w++)
                if (is_better(r_c[w], r_k[w], bc, bk)) { bc = r_c[w]; bk = r_k[w]; }
            snap.status = __ldcg(&st->status);   // the tail fix may have found the table full
            // The list decides as long as its best count is at least its threshold: everything
            // else was below the threshold at the last full scan and has not crossed it since.
            if (bc >= snap.cand_tau && cand_n < CAND_CAP && snap.since_scan < CAND_MAX_AGE) {
                st->since_scan = snap.since_scan + 1u;
                setup_merge(st, &snap, bc, bk, log);
                st->presetup_at = snap.iter_no;
            } else {
                // the arg-max kernel of this iteration scans the table
                void_candidates(st, snap.iter_no);
                st->cand_tau_next = max(2u, min(snap.cand_tau, snap.cand_tau_next) / 2u);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < 2 * S; i += THREADS) skey[i] = 0u;
    __syncthreads();
    const uint32_t e = st->epoch;
    const uint32_t N = st->n[e & 1];
    const uint32_t* __restrict__ src = (e & 1) ? buf1 : buf0;
    const uint32_t logC = st->table_log2;
    if (table == nullptr) table = st->table;

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
        uint32_t pend_mask = 0u;
        uint32_t keys[4];
        // Fast path, the same instructions for every lane: probe the home slot; a lane whose pair is
        // already there adds 1 with one predicated atomic.
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // key32 = (left token << 16) | right token; a pair needs a live right neighbour that
            // does not start a word, and neither token may be 0 (train.wgsl:393-398)
            keys[j] = __byte_perm(s[j + 1], s[j], 0x5410);
            const bool ok = ((uint32_t)(j + 1) < rem) && !(s[j + 1] & WORD_START_BIT) && (keys[j] & 0xFFFFu) != 0u &&
                            (keys[j] >> 16) != 0u;
            const uint32_t slot = smem_slot(keys[j], S);
            const bool hit = ok && skey[slot] == keys[j];
            if (hit) atomicAdd(&scnt[slot], 1u);
            if (ok && !hit) pend_mask |= 1u << j;
        }
        // Slow path, only when some lane missed: insert with compare-and-swap, probe further.
        if (__any_sync(0xFFFFFFFFu, pend_mask != 0u)) {
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (((pend_mask >> j) & 1u) && smem_count(skey, scnt, S, keys[j])) pend_mask &= ~(1u << j);
        }
        // Overflow (rare while the shared table has room): one global add per distinct key among
        // the pending lanes of this warp.
        if (__any_sync(0xFFFFFFFFu, pend_mask != 0u)) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const bool pending = (pend_mask >> j) & 1u;
                const uint32_t pend = __ballot_sync(0xFFFFFFFFu, pending);
                if (pending) {
                    const uint32_t peers = __match_any_sync(pend, keys[j]);
                    if (lane == __ffs(peers) - 1) {
                        const unsigned long long key = ((unsigned long long)(keys[j] >> 16) << 32) | (keys[j] & 0xFFFFu);
                        table_add(table, logC, key, hash_pair(key), __popc(peers), st, snap.cand_tau);
                    }
                }
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < S; i += THREADS) {
        const uint32_t k32 = skey[i];
        if (k32 != 0u) {
            const unsigned long long key = ((unsigned long long)(k32 >> 16) << 32) | (k32 & 0xFFFFu);
            table_add(table, logC, key, hash_pair(key), scnt[i], st, snap.cand_tau);
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
// `rd` is where the current values are read from: the control block itself, or a copy of it that
// the caller took at the start of its kernel (one load instead of a chain of dependent ones; no
// field read here is written by anybody else while the arg-max kernel runs).
__device__ __forceinline__ void setup_merge(DevState* st, const DevState* rd, uint32_t best_count,
                                            unsigned long long best_key, uint32_t* __restrict__ log) {
    st->tail_fix = 0u;
    if (rd->status != DS_OK) { st->active = 0u; st->recount = 1u; void_candidates(st, rd->iter_no + 1u); return; }
    const uint32_t next_id = rd->next_id;
    if (best_count < 2u || next_id > TOKEN_MASK) {
        st->early_stop = 1u;
        st->active = 0u;
        return;
    }
    const uint32_t a = (uint32_t)(best_key >> 32), b = (uint32_t)best_key;
    st->a = a; st->b = b; st->max_count = best_count; st->new_id = next_id;
    const uint32_t md = rd->merges_done;
    log[md * 4 + 0] = a; log[md * 4 + 1] = b; log[md * 4 + 2] = next_id; log[md * 4 + 3] = best_count;
    st->next_id = next_id + 1u;
    st->merges_done = md + 1u;
    if (md + 1u >= rd->merges_target) st->target_hit = 1u;
    st->k3_epoch = rd->epoch;
    st->ticket = rd->first_ticket;
    st->active = 1u;
    // Incremental table: a merge of two equal symbols collapses whole runs, which the local
    // update rule does not cover; the table is emptied and rebuilt by a full count instead.
    const uint32_t recount = rd->incremental ? (a == b ? 1u : 0u) : 1u;
    st->recount = recount;
    if (recount) void_candidates(st, rd->iter_no + 1u);   // the table is about to be rebuilt
    st->tail_fix = (rd->incremental && rd->literal && a != b) ? 1u : 0u;
}
__device__ __forceinline__ void setup_merge(DevState* st, uint32_t best_count, unsigned long long best_key,
                                            uint32_t* __restrict__ log) {
    setup_merge(st, st, best_count, best_key, log);
}

// mode 0: single GPU — finish with setup_merge.
// mode 1: sharded — the last CTA only publishes this rank's best as a packed word for the
//         all-reduce (count << 32 | ~pair32); k_unpack_flags finishes after the collective.
__global__ void __launch_bounds__(AM_THREADS)
k_argmax_setup(DevState* __restrict__ st, PairSlot* table, CtaBest* __restrict__ cta_best,
               uint32_t* __restrict__ log, int mode, uint32_t table_log2) {   // table_log2: 0 = the control block's
    __shared__ uint32_t sc[AM_THREADS / 32];
    __shared__ unsigned long long sk[AM_THREADS / 32];
    __shared__ uint32_t socc[AM_THREADS / 32];
    __shared__ bool is_last;
    // One 16-byte load per thread copies the control block into shared memory: everything the
    // kernel needs to know arrives in one round trip instead of a chain of dependent loads.
    // Whatever decides a CTA's branch is the same in every copy: the block is written by the CTA
    // that arrives last only (every CTA arrives, on every path that writes), and flags meant for
    // later kernels are stored as iteration numbers.
    __shared__ __align__(16) DevState snap;
    static_assert(sizeof(DevState) % 16 == 0 && sizeof(DevState) / 16 <= AM_THREADS, "control block copy");
    if (threadIdx.x < sizeof(DevState) / 16)
        reinterpret_cast<uint4*>(&snap)[threadIdx.x] = __ldcg(reinterpret_cast<const uint4*>(st) + threadIdx.x);
    __syncthreads();
    // The count kernel of this iteration has already chosen the merge from the candidate list.
    if (snap.presetup_at == snap.iter_no) return;
    // Once the run has stopped, nothing is left for the merge kernel to apply.
    if (snap.early_stop | snap.target_hit) {
        if (blockIdx.x == 0 && threadIdx.x == 0) { st->active = 0u; st->tail_fix = 0u; }
        return;
    }
    const uint32_t C = 1u << (table_log2 ? table_log2 : snap.table_log2);
    const bool clear = snap.incremental == 0u || mode == 1;  // an incrementally maintained table is never wiped here; a table of owned pairs always is
    if (table == nullptr) table = snap.table;
    uint4* __restrict__ t4 = reinterpret_cast<uint4*>(table);
    uint32_t bc = 0, occ = 0;
    unsigned long long bk = 0ull;
    const uint32_t stride = gridDim.x * AM_THREADS;
    // Incremental table, single GPU: most merges only look at the candidate list; a full scan is due
    // from iteration `scan_from` on.
    const bool listed = mode == 0 && snap.incremental != 0u;
    const bool use_list = listed && snap.iter_no < snap.scan_from;
    const uint32_t tau_scan = listed ? snap.cand_tau_next : 0xFFFFFFFFu;   // threshold of the list a full scan builds
    uint32_t* __restrict__ cand = snap.cand;
    if (use_list) {
        // One CTA is enough for a list of at most a few thousand slots.  The others only arrive; the
        // CTA that arrives last (nearly always CTA 0) takes CTA 0's result and sets the merge up.
        if (blockIdx.x == 0) {
            const uint32_t n = min(snap.cand_n, CAND_CAP);
            for (uint32_t i = threadIdx.x; i < n; i += AM_THREADS) {
                const uint4 q = __ldcg(t4 + cand[i]);
                const unsigned long long key = ((unsigned long long)q.y << 32) | q.x;
                if (key != 0ull && is_better(q.z, key, bc, bk)) { bc = q.z; bk = key; }
            }
            warp_best(bc, bk);
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            if (lane == 0) { sc[warp] = bc; sk[warp] = bk; }
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int w = 1; w < AM_THREADS / 32; w++)
                    if (is_better(sc[w], sk[w], bc, bk)) { bc = sc[w]; bk = sk[w]; }
                cta_best[0].key = bk;
                cta_best[0].count = bc;
            }
        }
        if (threadIdx.x == 0) {
            __threadfence();
            is_last = atomicAdd(&st->argmax_done, 1u) == gridDim.x - 1;
        }
        __syncthreads();
        if (!is_last) return;
        if (threadIdx.x == 0) {
            __threadfence();
            st->argmax_done = 0u;
            bc = __ldcg(&cta_best[0].count);
            bk = __ldcg(&cta_best[0].key);
            // The list decides as long as its best count is at least its threshold: everything
            // else was below the threshold at the last full scan and has not crossed it since.
            if (bc >= snap.cand_tau && snap.cand_n < CAND_CAP && snap.since_scan < CAND_MAX_AGE) {
                st->since_scan = snap.since_scan + 1u;
                setup_merge(st, &snap, bc, bk, log);
            } else {
                // no merge in this iteration; the next arg-max scans the table
                void_candidates(st, snap.iter_no + 1u);
                st->cand_tau_next = max(2u, min(snap.cand_tau, snap.cand_tau_next) / 2u);
                st->active = 0u;
                st->tail_fix = 0u;
            }
        }
        return;
    }
    // four independent 16-byte loads in flight per thread: the scan is latency-bound otherwise
    for (uint32_t i0 = blockIdx.x * AM_THREADS + threadIdx.x; i0 < C; i0 += 4u * stride) {
        uint4 q[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const uint32_t i = i0 + u * stride;
            q[u] = i < C ? __ldcg(t4 + i) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const unsigned long long key = ((unsigned long long)q[u].y << 32) | q[u].x;
            if (key != 0ull) {
                occ++;
                if (is_better(q[u].z, key, bc, bk)) { bc = q[u].z; bk = key; }
                if (q[u].z >= tau_scan) {
                    const uint32_t k = atomicAdd(&st->cand_n, 1u);
                    if (k < CAND_CAP) cand[k] = i0 + u * stride;
                }
                if (clear) __stcg(t4 + i0 + u * stride, make_uint4(0u, 0u, 0u, 0u));
            }
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
        st->occupied = mode == 1 ? 0u : occ;   // sharded: the word is the partition kernel's running count of the local table's fill
        if ((unsigned long long)occ * 2ull > (unsigned long long)C) st->want_grow = 1u;
        if (mode == 0) {
            if (listed) {
                st->full_scans += 1u;
                st->since_scan = 0u;
                if (tau_scan == 0xFFFFFFFFu || st->cand_n >= CAND_CAP) {
                    // no usable list yet (first scan, or too many slots above the threshold): scan again next time
                    const uint32_t over = st->cand_n >= CAND_CAP ? 1u : 0u;
                    void_candidates(st, snap.iter_no + 1u);
                    st->cand_tau_next = over ? min(0x7FFFFFFFu, tau_scan) * 2u : max(2u, bc / 2u);
                } else {
                    st->scan_from = SCAN_NEVER;
                    st->cand_tau = tau_scan;
                    st->cand_tau_next = max(2u, bc / 2u);
                }
            }
            setup_merge(st, &snap, bc, bk, log);
        } else {
            const uint32_t pair32 = ((uint32_t)(bk >> 32) << 16) | ((uint32_t)bk & 0xFFFFu);
            st->best_packed = ((unsigned long long)bc << 32) | (unsigned long long)(~pair32);
        }
    }
}

// ─────────────────────────────── merge + scan + compaction ───────────────────────────────
// Tile descriptor of the decoupled look-back: high word = (tag << 2) | flag, low word = value.
// The tag is the merge number + 1, so descriptors left by earlier merges read as "not ready"
// and the array never needs clearing between merges.
constexpr uint32_t DESC_AGG = 1u, DESC_PREFIX = 2u;

__device__ __forceinline__ unsigned long long ld_desc(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_desc(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Incremental table maintenance, the rare path of k_merge_compact: called by a whole warp for a row
// in which some pair merges.  Every lane rebuilds an 8-symbol window (left neighbour, its four
// symbols, the next three), finds which of its four (t, t+1) pairs change, and appends the old
// pair to the "minus" queue and the new one to the "plus" queue; the CTA folds its queues into the
// table when it has run out of tiles.  With a != b matches never overlap, so the symbol after a dropped one
// is always kept and this window is enough.  A full queue falls back to updating the table here.
// Each CTA of the merge kernel appends to its own segment of the queues (segment g = CTA g), so the
// reservation counters are never shared between CTAs.
struct DeltaQueues {
    uint32_t* minus;    // segments of (left << 16 | right) keys to take out once each
    uint32_t* plus;     // segments of keys to put in once each
    uint32_t* counts;   // per segment: entries reserved in minus, in plus (2 words)
    uint32_t seg_cap;   // entries per segment
    uint32_t segments;  // number of segments = CTAs of the merge kernel
};

__device__ __noinline__ void queue_deltas(DevState* st, PairSlot* __restrict__ table, DeltaQueues dq, uint32_t* qcnt, uint32_t s0, uint4 own,
                                          uint32_t s5, uint32_t y31, uint32_t z31, uint32_t i0, uint32_t N, bool interior,
                                          uint32_t A, uint32_t B, uint32_t NW, int lane, uint32_t logC, bool shard) {
    uint32_t s[8] = {s0, own.x, own.y, own.z, own.w, s5, 0u, 0u};
    s[6] = __shfl_down_sync(0xFFFFFFFFu, own.y, 1);
    s[7] = __shfl_down_sync(0xFFFFFFFFu, own.z, 1);
    if (lane == 31) { s[6] = y31; s[7] = z31; }
    uint32_t left = 0u, right = 0u, live = 0xFFu;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        left |= ((s[k] & TOKEN_MASK) == A ? 1u : 0u) << k;
        right |= ((s[k] & (TOKEN_MASK | WORD_START_BIT)) == B ? 1u : 0u) << k;
    }
    if (!interior) {
        live = (i0 >= 1u ? 1u : 0u);
#pragma unroll
        for (int k = 1; k < 8; k++) live |= (i0 + k - 1u < N ? 1u : 0u) << k;
    }
    const uint32_t m = left & (right >> 1) & live & (live >> 1);  // bit k: pair (s[k], s[k+1]) merges, k = 0..6
    const uint32_t touched = (m | (m << 1) | (m >> 1)) & 0x1Eu & live;
    uint32_t km[4], kp[4], vm = 0u, vp = 0u;
#pragma unroll
    for (int t = 1; t <= 4; t++) {
        km[t - 1] = kp[t - 1] = 0u;
        if (!((touched >> t) & 1u)) continue;
        // the old pair (s[t], s[t+1]) leaves the table if it was a counted pair
        const uint32_t lo = s[t] & TOKEN_MASK, ro = s[t + 1] & TOKEN_MASK;
        if (((live >> (t + 1)) & 1u) && !(s[t + 1] & WORD_START_BIT) && lo != 0u && ro != 0u) {
            km[t - 1] = (lo << 16) | ro;
            vm |= 1u << (t - 1);
        }
        // the new pair whose left symbol is t, unless t itself is dropped
        if (!((m >> (t - 1)) & 1u)) {
            const bool mt = (m >> t) & 1u;
            // the right symbol of a match is dropped, so the neighbour is then t + 2
            const uint32_t sr = mt ? s[t + 2] : s[t + 1];
            const bool mr = mt ? ((m >> (t + 2)) & 1u) : ((m >> (t + 1)) & 1u);
            const bool lr = mt ? ((live >> (t + 2)) & 1u) : ((live >> (t + 1)) & 1u);
            if ((mt || mr) && lr && !(sr & WORD_START_BIT)) {
                const uint32_t ln = mt ? NW : lo, rn = mr ? NW : (sr & TOKEN_MASK);
                if (ln != 0u && rn != 0u) {
                    kp[t - 1] = (ln << 16) | rn;
                    vp |= 1u << (t - 1);
                }
            }
        }
    }
    // reserve room in both queues: one atomic per queue per warp
    const uint32_t cm = __popc(vm), cp = __popc(vp);
    uint32_t im = cm, ip = cp;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t a = __shfl_up_sync(0xFFFFFFFFu, im, o), b = __shfl_up_sync(0xFFFFFFFFu, ip, o);
        if (lane >= o) { im += a; ip += b; }
    }
    uint32_t base_m = 0u, base_p = 0u;
    if (lane == 31) {
        if (im) base_m = atomicAdd(&qcnt[0], im);
        if (ip) base_p = atomicAdd(&qcnt[1], ip);
    }
    base_m = __shfl_sync(0xFFFFFFFFu, base_m, 31) + im - cm;
    base_p = __shfl_sync(0xFFFFFFFFu, base_p, 31) + ip - cp;
    uint32_t* __restrict__ seg_m = dq.minus + (size_t)blockIdx.x * dq.seg_cap;
    uint32_t* __restrict__ seg_p = dq.plus + (size_t)blockIdx.x * dq.seg_cap;
#pragma unroll
    for (int t = 0; t < 4; t++) {
        if ((vm >> t) & 1u) {
            if (base_m < dq.seg_cap) seg_m[base_m] = km[t];
            else {
                const unsigned long long key = ((unsigned long long)(km[t] >> 16) << 32) | (km[t] & 0xFFFFu);
                if (shard) delta_add(table, logC, key, hash_pair(key), 0xFFFFFFFFu, st);
                else table_add(table, logC, key, hash_pair(key), 0xFFFFFFFFu, st);
            }
            base_m++;
        }
        if ((vp >> t) & 1u) {
            if (base_p < dq.seg_cap) seg_p[base_p] = kp[t];
            else {
                const unsigned long long key = ((unsigned long long)(kp[t] >> 16) << 32) | (kp[t] & 0xFFFFu);
                if (shard) delta_add(table, logC, key, hash_pair(key), 1u, st);
                else table_add(table, logC, key, hash_pair(key), 1u, st);
            }
            base_p++;
        }
    }
}

// Fold one queue segment into the table (the whole CTA takes part).  Equal keys held by the lanes
// of a warp are combined first (match-any), so a popular neighbour pair costs one atomic per warp.
// The segment's counters are cleared at the end.
__device__ __forceinline__ void apply_segment(DevState* st, DeltaQueues dq, const uint32_t* qcnt, uint32_t g, PairSlot* __restrict__ table,
                                              uint32_t logC, bool shard) {
    const int lane = threadIdx.x & 31;
    const uint32_t nm = min(qcnt[0], dq.seg_cap), np = min(qcnt[1], dq.seg_cap);
    const uint32_t total = nm + np;
    if (total == 0u) return;
    const uint32_t tau = st->cand_tau;
    const uint32_t* __restrict__ seg_m = dq.minus + (size_t)g * dq.seg_cap;
    const uint32_t* __restrict__ seg_p = dq.plus + (size_t)g * dq.seg_cap;
    for (uint32_t base = 0; base < total; base += blockDim.x) {
        const uint32_t i = base + threadIdx.x;
        const bool on = i < total;
        const bool neg = i < nm;
        const uint32_t k32 = on ? (neg ? seg_m[i] : seg_p[i - nm]) : 0u;
        // same key and same sign within the warp → one add of the group's size
        const unsigned long long tagk = ((unsigned long long)(neg ? 1u : 0u) << 32) | k32;
        const uint32_t act = __ballot_sync(0xFFFFFFFFu, on);
        if (on) {
            const uint32_t peers = __match_any_sync(act, tagk);
            if (lane == __ffs(peers) - 1) {
                const unsigned long long key = ((unsigned long long)(k32 >> 16) << 32) | (k32 & 0xFFFFu);
                const uint32_t c = __popc(peers);
                if (shard) delta_add(table, logC, key, hash_pair(key), neg ? (0u - c) : c, st);
                else table_add(table, logC, key, hash_pair(key), neg ? (0u - c) : c, st, tau);
            }
        }
    }
}

// ── asynchronous bulk copy global → shared memory (one per tile), completion on an mbarrier ──
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}
// Orders this thread's earlier generic-proxy accesses to shared memory (and those ordered before
// it by a barrier) before later writes by the asynchronous proxy.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// The copy carries an L2 policy: a tile of the source is read once per merge and is dead afterwards
// (the next merge reads the other buffer), so its lines are marked "evict first".  What stays in L2 is
// then what the merge writes, which is what the next merge reads: a shard of up to about 100 MB is read
// from L2 instead of HBM from the second merge on.
__device__ __forceinline__ unsigned long long l2_evict_first_policy() {
    unsigned long long p;
    asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src, uint32_t bytes, unsigned long long* bar,
                                          unsigned long long policy) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(smem_u32(dst_smem)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}
// Bounded wait for the phase with the given parity; false when it never completed.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spins = 0; spins < BULK_MAX_SPINS; spins++) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// One tile = 12,288 symbols (48 KB; four CTAs of 256 threads fit an SM, which measured faster than three
// CTAs with 64 KB tiles or five with 32 KB).  One asynchronous bulk copy brings the whole tile into shared
// memory; the tile is then worked through as three sub-tiles of 4,096 symbols: in a sub-tile warp w
// owns the 512 consecutive symbols [w * 512, (w + 1) * 512), a span, as four 16-byte rows per lane,
// so a span's kept symbols are a contiguous run of the output.
//   pass 1    nothing in the buffer is written, so every neighbour read sees the snapshot.  Per span:
//             a candidate test (can any pair merge at all?), then, only where needed, the bit logic
//             that decides every symbol (kept? rewritten?), the pair deltas, the in-place rewrite of
//             the source (literal mode), and the span's kept count.  One barrier, then the tile's
//             kept count is published, long before the tile needs its own offset.
//   pass 2    every warp compacts its touched spans in place (a span belongs to one warp: no barrier).
//   look-back the whole CTA inspects 256 earlier tiles per round for the tile's global offset.
//   copy-out  every warp writes its spans with 16-byte stores whatever the alignment of the
//             destination; then the next tile's bulk copy starts.
// Tiles are handed out by an atomic ticket so that a waiting tile's predecessors are always running.
//
// Why one look-back per 48 KB: the tiles of a launch move in waves, a wave resolves its offsets
// front to back at one look-back round per L2 round trip, and that chain, not HBM, bounds the
// kernel when a tile is small.
//
// Neighbours across rows, sub-tiles and tiles are read from the shared buffer: the symbol before
// the tile sits in front of it, the three after it behind it (plain loads).  Such a symbol may
// already carry this merge's rewrite (in literal mode the source is rewritten in place by the
// tile's owner; within the tile the last symbol of a sub-tile may have been written back onto
// itself); the new id is fresh, so mapping it back to `a` restores the snapshot.
//
// INCR: the pair table is kept up to date instead of being rebuilt by a full count for the next
// merge.  Every position whose pair with its right neighbour changes takes the old pair out and
// puts the new one in (a handful of atomics per merged occurrence).  This needs `a != b` (matches
// cannot overlap, so a dropped symbol's successor is always kept and three symbols of look-ahead
// settle everything); a merge with a == b collapses whole runs (train.wgsl:482-497 on a run
// "aaaa" yields one symbol), so it empties the table here and the next merge counts from scratch.

// SHARD (sharded runs with the peer-memory exchange): the deltas go into the local delta table for
// the route kernel, and a merge of two equal symbols empties this rank's table of owned pairs.
template <bool LITERAL, bool INCR, bool SHARD = false>
__global__ void __launch_bounds__(MC_THREADS, MC_CTAS_PER_SM)
k_merge_compact(DevState* __restrict__ st, uint32_t* buf0, uint32_t* buf1, unsigned long long* __restrict__ desc,
                PairSlot* table, DeltaQueues dq) {
    // MC_NBUF tile buffers, each: 4 words (the last: left edge), the tile, 4 words (right edge)
    extern __shared__ __align__(16) uint32_t mc_smem[];
    constexpr uint32_t BUF_WORDS = MC_TILE + 8;
    __shared__ __align__(8) unsigned long long bar[MC_NBUF];
    __shared__ uint32_t span_cnt[MC_NBUF][MC_SUBS * MC_WARPS], lb_sum[MC_WARPS], lb_found[MC_WARPS];
    __shared__ uint32_t s_tid[MC_NBUF], s_fail;   // s_tid[j % MC_NBUF]: the tile of this CTA's j-th turn (>= ntiles: none)
    __shared__ uint32_t s_qcnt[2];  // entries reserved in this CTA's segments of the minus and plus queues
    // The iteration ends here: one thread advances its number and clears the arrival counters of the
    // count and arg-max kernels (nobody in this kernel reads any of the three).
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        st->iter_no = st->iter_no + 1u;
        st->k1_done = 0u;
        st->argmax_done = 0u;
    }
    // `active`, `k3_epoch`, `n[k3_epoch & 1]`, `a`, `b`, `new_id`, `max_count` and `recount` are written
    // by the set-up step only, so every thread of every CTA of this launch reads the same values.
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
    const bool deltas = INCR && st->recount == 0u;
    const uint32_t lb_max_spins = st->lb_max_spins;
    const uint32_t logC = st->table_log2;
    if (table == nullptr) table = st->table;
    auto snapshot = [&](uint32_t v) { return (v & TOKEN_MASK) == NW ? ((v & WORD_START_BIT) | A) : v; };
    const uint32_t AB = A | (B << 16);  // the low halves of a pair that may merge
    const unsigned long long src_policy = l2_evict_first_policy();


    // Start the copy of a tile into buffer b.  One bulk copy brings the tile together with the four words
    // before it (the last of them is the left edge) and the four after it (the right edge; the arrays are
    // allocated with that much room behind the last symbol, and what lies at or beyond N there is never
    // used: a span that can see it is not `interior` and masks by position).  Callers make sure (barrier)
    // that nobody still reads the buffer.
    auto fetch_tile = [&](uint32_t tile, uint32_t b) {
        uint32_t* const in = mc_smem + b * BUF_WORDS + 4;
        const uint32_t i0 = tile * MC_TILE;
        if (threadIdx.x == 0) {
            const uint32_t bytes = ((min((uint32_t)MC_TILE, N - i0) + 3u) & ~3u) * 4u + 16u;
            fence_proxy_async_smem();
            if (i0 > 0u) {
                bulk_load(in - 4, src + i0 - 4u, bytes + 16u, &bar[b], src_policy);
            } else {
                in[-1] = 0u;
                bulk_load(in, src, bytes, &bar[b], src_policy);
            }
        }
    };

    // The tiles of a CTA go through two stages, one loop iteration apart:
    //   stage 1 (turn j)      wait for the tile's bulk copy, pass 1, publish the tile's kept count, pass 2
    //   stage 2 (turn j - 1)  look-back for the tile's offset, copy-out
    // and the buffer that stage 2 frees takes the bulk copy of turn j + MC_NBUF - 1.  A tile's kept
    // count is therefore published one whole iteration before the tile needs its own offset, and the
    // time from taking a tile's ticket to publishing its count holds no wait on other tiles: a tile
    // with a smaller number always publishes earlier (give or take the jitter of a bulk copy), so the
    // look-back finds what it needs instead of waiting for the slowest of its predecessors.
    if (threadIdx.x == 0) {
#pragma unroll
        for (int b = 0; b < MC_NBUF; b++) { mbar_init(&bar[b], 1u); s_tid[b] = 0xFFFFFFFFu; }
        fence_proxy_async_smem();
        s_fail = 0u;
        s_qcnt[0] = s_qcnt[1] = 0u;
        // the first MC_NBUF - 1 tickets
#pragma unroll
        for (int b = 0; b < MC_NBUF - 1; b++) {
            const uint32_t t = atomicAdd(&st->ticket, 1u);
            s_tid[b] = t;
            if (t >= ntiles) break;
        }
    }
    __syncthreads();
#pragma unroll
    for (int b = 0; b < MC_NBUF - 1; b++)
        if (s_tid[b] < ntiles) fetch_tile(s_tid[b], b);
    uint32_t prev = 0xFFFFFFFFu;   // tile of the turn before (stage 2), if any
    bool more = true;              // tickets below ntiles may still be had
    for (uint32_t j = 0;; j++) {
        const uint32_t cb = j % MC_NBUF, pb = (j + MC_NBUF - 1u) % MC_NBUF;   // buffers of turn j and of turn j - 1
        const uint32_t tile = s_tid[cb];
        if (tile >= ntiles && prev >= ntiles) break;
        if (tile < ntiles && !mbar_wait(&bar[cb], (j / MC_NBUF) & 1u)) s_fail = 1u;
        __syncthreads();  // edges and the failure flag visible
        if (s_fail) {
            if (threadIdx.x == 0) atomicExch(&st->status, (uint32_t)DS_LOOKBACK_TIMEOUT);
            break;
        }
        uint32_t dec0 = 0u, dec1 = 0u, dec2 = 0u, dec3 = 0u;
        if (tile < ntiles) {
        uint32_t* const in = mc_smem + cb * BUF_WORDS + 4;
        const uint32_t tile0 = tile * MC_TILE;  // first symbol of the tile

        // ── pass 1: decide every symbol of the tile (kept? rewritten?) and count; nothing in the
        // buffer is written, so every neighbour read sees the snapshot.  Straight-line bit logic on
        // all four rows of a span at once: row j lives in byte j of a word,
        //   L  bit 8j + k  (k = 0..4): s[k] is `a`             (s[0] = left neighbour, s[1..4] = own)
        //   R  bit 8j + k  (k = 0..4): s[k + 1] is `b` and does not start a word   (s[5] = right neighbour)
        //   M = L & R      bit 8j + k: the pair (s[k], s[k + 1]) merges; the symbol at k + 1 is then
        //                  dropped and the one at k rewritten (train.wgsl:482-497)
        // so per row the decisions fit one byte (low nibble: own symbol kept, high nibble: own symbol
        // rewritten) and the four words of a tile stay in registers for pass 2.
        MC_UNROLL_SUBS
        for (int sub = 0; sub < MC_SUBS; sub++) {
            const uint32_t lw = sub * MC_SUB + warp * (MC_ROWS * 128);  // tile-local first symbol of the warp's span
            // a warp whose whole span (and the three symbols after it) lies below both N and the
            // compaction limit needs no bounds tests
            const bool interior = tile0 + lw + MC_ROWS * 128u + 3u < min(N, limit);
            uint4 q[MC_ROWS];
#pragma unroll
            for (int j = 0; j < MC_ROWS; j++) q[j] = reinterpret_cast<const uint4*>(in + lw)[j * 32 + lane];
            // the symbol before the span and the three after it: one load by lanes 0..3 next to the rows' loads, handed
            // round by shuffles (a load inside a one-lane branch would put a shared-memory round trip into the chain)
            uint32_t edge_sym = 0u;
            if (lane < 4) edge_sym = snapshot(lane == 0 ? in[(int)lw - 1] : in[lw + MC_ROWS * 128u + (lane - 1)]);
            const uint32_t s_prev = __shfl_sync(0xFFFFFFFFu, edge_sym, 0), s_n0 = __shfl_sync(0xFFFFFFFFu, edge_sym, 1);
            const uint32_t s_n1 = __shfl_sync(0xFFFFFFFFu, edge_sym, 2), s_n2 = __shfl_sync(0xFFFFFFFFu, edge_sym, 3);
            // Candidate test first: two neighbouring symbols can only merge if their low halves are
            // (a, b), one byte permute and one compare per pair.  Every lane tests the four pairs that
            // begin at its own symbols; lane 0 adds the pair that begins at the symbol before the span,
            // lane 31 (when deltas are queued) the two pairs that begin right after it.  A span
            // without a candidate, which is most of them, keeps everything and skips the bit logic.
            bool cand = false;
#pragma unroll
            for (int j = 0; j < MC_ROWS; j++) {
                uint32_t nx = __shfl_down_sync(0xFFFFFFFFu, q[j].x, 1);
                const uint32_t rx = __shfl_sync(0xFFFFFFFFu, q[j < MC_ROWS - 1 ? j + 1 : j].x, 0);
                if (lane == 31) nx = j < MC_ROWS - 1 ? rx : s_n0;
                cand |= __byte_perm(q[j].x, q[j].y, 0x5410) == AB || __byte_perm(q[j].y, q[j].z, 0x5410) == AB ||
                        __byte_perm(q[j].z, q[j].w, 0x5410) == AB || __byte_perm(q[j].w, nx, 0x5410) == AB;
            }
            if (lane == 0) cand |= __byte_perm(s_prev, q[0].x, 0x5410) == AB;
            if (INCR && lane == 31) {
                cand |= __byte_perm(s_n0, s_n1, 0x5410) == AB || __byte_perm(s_n1, s_n2, 0x5410) == AB;
            }
            uint32_t kb = MC_KEEP_ALL, rew = 0u;   // per row one byte: own symbol kept (low nibble), rewritten (high nibble)
            if (!interior || __any_sync(0xFFFFFFFFu, cand)) {
            uint32_t L = 0u, R = 0u;
#pragma unroll
            for (int j = 0; j < MC_ROWS; j++) {
                L |= ((q[j].x & TOKEN_MASK) == A ? 2u : 0u) << (8 * j);
                L |= ((q[j].y & TOKEN_MASK) == A ? 4u : 0u) << (8 * j);
                L |= ((q[j].z & TOKEN_MASK) == A ? 8u : 0u) << (8 * j);
                L |= ((q[j].w & TOKEN_MASK) == A ? 16u : 0u) << (8 * j);
                R |= ((q[j].x & (TOKEN_MASK | WORD_START_BIT)) == B ? 1u : 0u) << (8 * j);
                R |= ((q[j].y & (TOKEN_MASK | WORD_START_BIT)) == B ? 2u : 0u) << (8 * j);
                R |= ((q[j].z & (TOKEN_MASK | WORD_START_BIT)) == B ? 4u : 0u) << (8 * j);
                R |= ((q[j].w & (TOKEN_MASK | WORD_START_BIT)) == B ? 8u : 0u) << (8 * j);
            }
            // the symbol before the span (lane 0) and the three after it (lanes 1..3): bit 0 = is `a`, bit 1 = is a mergeable `b`
            uint32_t edge = 0u;
            if (lane < 4) {
                const uint32_t v = edge_sym;
                edge = ((v & TOKEN_MASK) == A ? 1u : 0u) | ((v & (TOKEN_MASK | WORD_START_BIT)) == B ? 2u : 0u);
            }
            const uint32_t e_prev = __shfl_sync(0xFFFFFFFFu, edge, 0), e_n0 = __shfl_sync(0xFFFFFFFFu, edge, 1);
            const uint32_t e_n1 = __shfl_sync(0xFFFFFFFFu, edge, 2), e_n2 = __shfl_sync(0xFFFFFFFFu, edge, 3);
            {
                // left neighbour is `a` → bit 8j; right neighbour is a mergeable `b` → bit 8j + 4
                const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, L, 1), dn = __shfl_down_sync(0xFFFFFFFFu, R, 1);
                const uint32_t l31 = __shfl_sync(0xFFFFFFFFu, L, 31), r0 = __shfl_sync(0xFFFFFFFFu, R, 0);
                uint32_t pa = (up >> 4) & 0x01010101u, nb = (dn << 4) & 0x10101010u;
                if (lane == 0) pa = ((l31 << 4) & 0x01010100u & MC_ROWBYTES) | (e_prev & 1u);           // the row before, or the span's left edge
                if (lane == 31) nb = ((r0 >> 4) & 0x00101010u & MC_NOTLAST) | ((e_n0 & 2u) << (MC_LASTROW_SHIFT + 3));     // the row after, or the span's right edge
                L |= pa;
                R |= nb;
            }
            uint32_t M = L & R;
            kb = ~M & MC_KEEP_ALL;                     // own symbol t (t = 1..4) is dropped iff M[t-1]
            if (!interior) {
                // live: bit 8j + k ↔ s[k] exists (k = 0: i0 >= 1; k >= 1: i0 + k - 1 < N); below: own symbol under the compaction limit
                uint32_t live = 0u, below = 0u;
#pragma unroll
                for (int j = 0; j < MC_ROWS; j++) {
                    const uint32_t i0 = tile0 + lw + 4u * (j * 32 + lane);
                    uint32_t lv = (i0 >= 1u ? 1u : 0u), bl = 0u;
#pragma unroll
                    for (int k = 1; k < 6; k++) lv |= (i0 + k - 1u < N ? 1u : 0u) << k;
#pragma unroll
                    for (int k = 0; k < 4; k++) bl |= (i0 + k < limit ? 1u : 0u) << k;
                    live |= lv << (8 * j);
                    below |= bl << (8 * j);
                }
                M &= live & (live >> 1);
                kb = ~M & MC_KEEP_ALL & (live >> 1) & below;
            }
            rew = (M >> 1) & MC_KEEP_ALL;              // and rewritten iff M[t]
            const bool any_m = __any_sync(0xFFFFFFFFu, M != 0u);
            if (INCR && deltas) {
                // The pair (t, t+1) changes iff one of the pairs at t-1, t, t+1 merges.  For lanes
                // 0..30 those are matches some lane of the row sees in its own window; lane 31 also
                // has to look at the two pairs that begin after its right neighbour: the pairs
                // (x, y) and (y, z) of the next row's lane 0, or of the symbols after the span.
                const uint32_t m0 = __shfl_sync(0xFFFFFFFFu, M, 0);
                uint32_t far = (m0 >> 8) & 0x00060606u & MC_NOTLAST;   // all rows but the last: bits 1, 2 of the next row's lane 0
                {
                    const uint32_t i5 = tile0 + lw + MC_ROWS * 128u;  // index of the symbol after the span
                    const bool p1 = (e_n0 & 1u) && (e_n1 & 2u) && (interior || i5 + 1u < N);
                    const bool p2 = (e_n1 & 1u) && (e_n2 & 2u) && (interior || i5 + 2u < N);
                    if (p1 || p2) far |= 0x02u << MC_LASTROW_SHIFT;
                }
                if (lane != 31) far = 0u;
                if (any_m || __any_sync(0xFFFFFFFFu, far != 0u)) {
#pragma unroll
                    for (int j = 0; j < MC_ROWS; j++) {
                        if (!__any_sync(0xFFFFFFFFu, ((M | far) >> (8 * j)) & 0xFFu)) continue;
                        const uint32_t l0 = lw + 4u * (j * 32 + lane);
                        uint32_t s0 = __shfl_up_sync(0xFFFFFFFFu, q[j].w, 1);
                        uint32_t s5 = __shfl_down_sync(0xFFFFFFFFu, q[j].x, 1);
                        uint32_t y = 0u, z = 0u;
                        if (lane == 0) s0 = snapshot(in[(int)l0 - 1]);
                        if (lane == 31) { s5 = snapshot(in[l0 + 4u]); y = snapshot(in[l0 + 5u]); z = snapshot(in[l0 + 6u]); }
                        queue_deltas(st, table, dq, s_qcnt, s0, q[j], s5, y, z, tile0 + l0, N, interior, A, B, NW, lane, logC, SHARD);
                    }
                }
            }
            if (LITERAL && any_m) {
                // the reference rewrites the source in place
#pragma unroll
                for (int j = 0; j < MC_ROWS; j++) {
                    const uint32_t r4 = (rew >> (8 * j)) & 15u;
                    if (r4) {
                        uint32_t* o = src + tile0 + lw + 4u * (j * 32 + lane);
                        if (r4 & 1u) o[0] = NW | (q[j].x & WORD_START_BIT);
                        if (r4 & 2u) o[1] = NW | (q[j].y & WORD_START_BIT);
                        if (r4 & 4u) o[2] = NW | (q[j].z & WORD_START_BIT);
                        if (r4 & 8u) o[3] = NW | (q[j].w & WORD_START_BIT);
                    }
                }
            }
            }
            {
                const uint32_t d = kb | (rew << 4);
                if (sub == 0) dec0 = d; else if (sub == 1) dec1 = d; else if (sub == 2) dec2 = d; else dec3 = d;
            }
            // kept symbols of the span
            uint32_t total = MC_ROWS * 128u;
            if (__any_sync(0xFFFFFFFFu, kb != MC_KEEP_ALL)) {
                uint32_t c = __popc(kb);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
                total = c;
            }
            if (lane == 0) span_cnt[cb][sub * MC_WARPS + warp] = total;
        }
        }
        __syncthreads();  // the snapshot has been read by everybody; span counts visible
        if (tile < ntiles) {
        uint32_t* const in = mc_smem + cb * BUF_WORDS + 4;
        if (threadIdx.x == 0) {
            // the tile's kept count, long before the tile needs its own offset
            uint32_t agg = 0u;
#pragma unroll
            for (int k = 0; k < MC_SUBS * MC_WARPS; k++) agg += span_cnt[cb][k];
            const uint32_t flag = tile == 0u ? DESC_PREFIX : DESC_AGG;
            st_desc(desc + tile, ((unsigned long long)((tag << 2) | flag) << 32) | agg);
        }

        // ── pass 2: every warp compacts its touched spans in place (a span belongs to one warp) ──
#pragma unroll 1
        for (int sub = 0; sub < MC_SUBS; sub++) {
            const uint32_t d = sub == 0 ? dec0 : sub == 1 ? dec1 : sub == 2 ? dec2 : dec3;
            if (__all_sync(0xFFFFFFFFu, d == MC_KEEP_ALL)) continue;
            const uint32_t lw = sub * MC_SUB + warp * (MC_ROWS * 128);
            uint4 q[MC_ROWS];
#pragma unroll
            for (int j = 0; j < MC_ROWS; j++) q[j] = reinterpret_cast<const uint4*>(in + lw)[j * 32 + lane];
            // kept counts of the four rows as four byte lanes of one word (a row keeps at most 128, so no lane overflows)
            uint32_t cnt = 0u;
#pragma unroll
            for (int j = 0; j < MC_ROWS; j++) cnt |= (uint32_t)__popc((d >> (8 * j)) & 15u) << (8 * j);
            uint32_t incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += t;
            }
            const uint32_t tot = __shfl_sync(0xFFFFFFFFu, incl, 31);
            __syncwarp();  // all lanes hold their rows: the span may be overwritten
            uint32_t run = 0u;
#pragma unroll
            for (int j = 0; j < MC_ROWS; j++) {
                const uint32_t kb = (d >> (8 * j)) & 15u, rew = (d >> (8 * j + 4)) & 15u;
                uint32_t o = lw + run + ((incl >> (8 * j)) & 0xFFu) - ((cnt >> (8 * j)) & 0xFFu);
                run += (tot >> (8 * j)) & 0xFFu;
                const uint32_t v0 = (rew & 1u) ? (NW | (q[j].x & WORD_START_BIT)) : q[j].x;
                const uint32_t v1 = (rew & 2u) ? (NW | (q[j].y & WORD_START_BIT)) : q[j].y;
                const uint32_t v2 = (rew & 4u) ? (NW | (q[j].z & WORD_START_BIT)) : q[j].z;
                const uint32_t v3 = (rew & 8u) ? (NW | (q[j].w & WORD_START_BIT)) : q[j].w;
                if (kb & 1u) in[o++] = v0;
                if (kb & 2u) in[o++] = v1;
                if (kb & 4u) in[o++] = v2;
                if (kb & 8u) in[o++] = v3;
            }
        }
        }
        uint32_t next_ticket = 0xFFFFFFFFu;
        if (prev < ntiles) {
        const uint32_t tile = prev;
        uint32_t* const in = mc_smem + pb * BUF_WORDS + 4;
        // offsets of the spans within the tile's output, and the tile's kept count
        uint32_t span_off, span_cnt_reg, agg;
        {
            const uint32_t c = lane < MC_SUBS * MC_WARPS ? span_cnt[pb][lane] : 0u;   // the spans of the tile, in tile order
            span_cnt_reg = c;
            uint32_t incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += t;
            }
            span_off = incl - c;
            agg = __shfl_sync(0xFFFFFFFFu, incl, 31);
        }

        // ── the tile's offset: look back over up to 1,024 predecessors per round: every thread reads
        // four descriptors (two 16-byte loads), nearest first, one warp per 128 ──
        uint32_t excl = 0u;
        if (tile != 0u) {
            int pos = (int)tile - 1;
            for (;;) {
                // this thread's descriptors: pos - 4 * t - k, k = 0..3, four independent loads in flight
                const int base = pos - 4 * (warp * 32 + lane);
                uint32_t hi[4], val[4];
                bool timed_out = false;
                for (uint32_t spins = 0;; spins++) {
                    bool ready = true;
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int idx = base - k;
                        hi[k] = (tag << 2) | DESC_PREFIX;   // positions before tile 0 act as a zero prefix
                        val[k] = 0u;
                        if (idx >= 0) {
                            const unsigned long long dsc = ld_desc(desc + idx);
                            hi[k] = (uint32_t)(dsc >> 32);
                            val[k] = (uint32_t)dsc;
                        }
                        ready = ready && ((hi[k] >> 2) == tag) && (hi[k] & 3u) != 0u;
                    }
                    if (__all_sync(0xFFFFFFFFu, ready)) break;
                    if (spins > lb_max_spins) { timed_out = true; break; }
                    __nanosleep(20);
                }
                // within the thread: add values, nearest first, up to and including the first full prefix
                uint32_t mine = 0u;
                bool mine_found = false;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    if (!mine_found) {
                        mine += val[k];
                        mine_found = (hi[k] & 3u) == DESC_PREFIX;
                    }
                }
                const uint32_t pmask = timed_out ? 1u : __ballot_sync(0xFFFFFFFFu, mine_found);
                const int first = pmask ? (__ffs(pmask) - 1) : 32;  // nearest lane holding a full prefix
                uint32_t contrib = (lane <= first && !timed_out) ? mine : 0u;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xFFFFFFFFu, contrib, o);
                if (lane == 0) {
                    lb_sum[warp] = contrib;
                    lb_found[warp] = pmask != 0u ? 1u : 0u;
                    if (timed_out) atomicExch(&st->status, (uint32_t)DS_LOOKBACK_TIMEOUT);
                }
                __syncthreads();
                bool found = false;
#pragma unroll
                for (int w = 0; w < MC_WARPS; w++) {
                    if (!found) {
                        excl += lb_sum[w];
                        found = lb_found[w] != 0u;
                    }
                }
                __syncthreads();  // lb_sum / lb_found may be rewritten
                if (found) break;
                pos -= 4 * MC_THREADS;
            }
        }
        if (threadIdx.x == 0) {
            if (tile != 0u) st_desc(desc + tile, ((unsigned long long)((tag << 2) | DESC_PREFIX) << 32) | (excl + agg));
            if (tile == ntiles - 1u) {
                // Last tile: publish the new symbol count and advance the epoch.
                const uint32_t total = excl + agg;
                const uint32_t nnew = N - st->max_count;
                if (!LITERAL && total != nnew && st->status == DS_OK && st->world == 1u)
                    atomicExch(&st->status, (uint32_t)DS_INTERNAL);
                st->n[(e + 1u) & 1u] = LITERAL ? nnew : total;
                st->v_kept = total;
                st->epoch = e + 1u;
            }
        }

        // ── copy-out: every warp writes its four spans, each a contiguous run, with 16-byte stores:
        // a few single symbols bring the destination to a 16-byte boundary, then every store takes
        // its four words from two neighbouring 16-byte rows of the buffer.
        __syncwarp();  // the warp's own pass-2 writes are visible to all its lanes (tile 0 passes no barrier on the way here)
        // The next tile's ticket is taken only now, one copy-out before its load starts: a tile number
        // that is reserved long before its tile is worked on makes every later tile wait in its
        // look-back for a predecessor that has not even been loaded.
        if (threadIdx.x == 0 && more) next_ticket = atomicAdd(&st->ticket, 1u);
        MC_UNROLL_SUBS
        for (int sub = 0; sub < MC_SUBS; sub++) {
            const uint32_t lw = sub * MC_SUB + warp * (MC_ROWS * 128);
            const uint32_t cnt = __shfl_sync(0xFFFFFFFFu, span_cnt_reg, sub * MC_WARPS + warp);
            const uint32_t off = excl + __shfl_sync(0xFFFFFFFFu, span_off, sub * MC_WARPS + warp);
            const uint32_t head = min(cnt, (4u - (off & 3u)) & 3u);
            const uint32_t nvec = (cnt - head) >> 2;
            const uint32_t* sp = in + lw;
            const uint4* sp4 = reinterpret_cast<const uint4*>(sp);
            uint4* __restrict__ d4 = reinterpret_cast<uint4*>(dst + off + head);
            if ((uint32_t)lane < head) dst[off + lane] = sp[lane];
            {
                // The trip count is known at compile time (a span has at most 128 * MC_ROWS / 4 vectors per lane row),
                // so all shared-memory loads of the span are in flight together; vectors beyond the span's kept count
                // are loaded (the buffer holds four more words behind every span) but not stored.
                uint4 lo[MC_ROWS], hi[MC_ROWS];
#pragma unroll
                for (int it = 0; it < MC_ROWS; it++) lo[it] = sp4[it * 32 + lane];
                if (head == 0u) {
#pragma unroll
                    for (int it = 0; it < MC_ROWS; it++)
                        if ((uint32_t)(it * 32 + lane) < nvec) d4[it * 32 + lane] = lo[it];
                } else {
#pragma unroll
                    for (int it = 0; it < MC_ROWS; it++) hi[it] = sp4[it * 32 + lane + 1];
                    if (head == 1u) {
#pragma unroll
                        for (int it = 0; it < MC_ROWS; it++)
                            if ((uint32_t)(it * 32 + lane) < nvec) d4[it * 32 + lane] = make_uint4(lo[it].y, lo[it].z, lo[it].w, hi[it].x);
                    } else if (head == 2u) {
#pragma unroll
                        for (int it = 0; it < MC_ROWS; it++)
                            if ((uint32_t)(it * 32 + lane) < nvec) d4[it * 32 + lane] = make_uint4(lo[it].z, lo[it].w, hi[it].x, hi[it].y);
                    } else {
#pragma unroll
                        for (int it = 0; it < MC_ROWS; it++)
                            if ((uint32_t)(it * 32 + lane) < nvec) d4[it * 32 + lane] = make_uint4(lo[it].w, hi[it].x, hi[it].y, hi[it].z);
                    }
                }
            }
            const uint32_t done = head + 4u * nvec;
            if (done + lane < cnt) dst[off + done + lane] = sp[done + lane];
        }
        } else if (threadIdx.x == 0 && more) {
            next_ticket = atomicAdd(&st->ticket, 1u);   // the first turn has nothing to copy out yet
        }
        // the buffer of turn j - 1 is free (or was never used): it takes the tile of turn j + MC_NBUF - 1
        if (threadIdx.x == 0) s_tid[pb] = next_ticket;
        __syncthreads();  // the buffer may be refilled; the new ticket is visible
        prev = tile;
        const uint32_t nt = s_tid[pb];
        if (nt < ntiles) fetch_tile(nt, pb); else more = false;
    }
    if (INCR && deltas) {
        // Fold this CTA's queue segment into the table.  Nobody else reads or writes the segment,
        // the updates commute with those of every other CTA, and doing it here, after the tiles,
        // keeps the scattered table traffic out of the streaming loop without another launch.
        __syncthreads();
        apply_segment(st, dq, s_qcnt, blockIdx.x, table, logC, SHARD);
    }
    if (INCR && !deltas) {
        // a == b (or a rebuild is already due): no deltas were written, so nobody else touches the
        // table during this launch; empty it for the full count that the next merge starts with.
        uint4* __restrict__ t4 = reinterpret_cast<uint4*>(SHARD ? st->owned : table);
        const uint32_t C = 1u << (SHARD ? st->owned_log2 : logC);
        for (uint32_t i = blockIdx.x * MC_THREADS + threadIdx.x; i < C; i += gridDim.x * MC_THREADS)
            t4[i] = make_uint4(0u, 0u, 0u, 0u);
        if (SHARD && blockIdx.x == 0 && threadIdx.x == 0) st->owned_inserted = 0u;
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

// Copy the pairs with a non-zero count out (and optionally empty the table), for tests.
__global__ void k_dump_table(PairSlot* table, uint32_t C, unsigned long long* keys, uint32_t* counts, uint32_t cap,
                             uint32_t* n_out, int clear) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < C; i += gridDim.x * blockDim.x) {
        const unsigned long long k = table[i].key;
        if (k) {
            if (table[i].count != 0u) {  // pairs whose count went back to 0 stay in an incremental table as dead keys
                const uint32_t d = atomicAdd(n_out, 1u);
                if (d < cap) { keys[d] = k; counts[d] = table[i].count; }
            }
            if (clear) { table[i].key = 0ull; table[i].count = 0u; }
        }
    }
}

}  // namespace b200bpe
