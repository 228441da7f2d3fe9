// Sharded training, peer-memory exchange: the per-merge count exchange written as this library's
// own kernels over NVLink peer memory (plain loads and stores, no NCCL call on the data path).
//
// The reference trains on one device; sharding is this library's addition.  The corpus is cut at
// word starts into one contiguous span per GPU (pairs never cross a word start), and every pair
// has an owner rank, owner = hash(pair) mod world, whose table holds the pair's GLOBAL count for
// the whole run.  Nothing but count CHANGES travels:
//
//   k_merge_compact   (SHARD) a merge's pair deltas (old pair -1, new pair +1) are folded into the
//                     rank's local table, which is otherwise empty; the slots that received an
//                     entry are listed
//   k_route           every listed (pair, delta) is written straight into its owner's inbox: a
//                     16-byte store into the peer's memory; the last CTA then writes one header per
//                     peer {sequence number, entries} with release semantics.  After a full count
//                     (first merge, after a merge of two equal symbols, after the table was
//                     replaced) the whole local table is routed the same way
//   k_accumulate      waits (bounded) for the headers of this round, adds the entries to the owned
//                     table, keeps the arg-max candidate list of the owned table up to date, and
//                     its last CTA picks this rank's best pair from the list
//   global pick       one warp writes {best, status} to every peer (8-byte words that carry the
//                     round's sequence number, so each is valid by itself), waits (bounded) for the
//                     words of all peers, takes the maximum, and sets up the merge.  max over
//                     (count << 32 | ~pair) is the reference's order: larger count, then the
//                     smaller pair id (train.wgsl:83-85).  Every rank computes the same winner.
//   k_argmax_peer     only when the candidate list is stale: full scan of the owned table, then
//                     the same global pick
//
// Waits on a peer are spin loops with an iteration limit; when one runs out the rank records
// DS_LOOKBACK_TIMEOUT and stops taking part, which makes its peers run into their own limits once.
// The ranks run in lockstep (the same graph on every GPU), one process per GPU; kernels of
// different ranks never share a GPU.
#pragma once

#include "ctx.cuh"
#include "train_kernels.cuh"

namespace b200bpe {

constexpr int PX_MAX_WORLD = 8;
constexpr uint32_t PX_HDR_OFF = 0;          // world x u64: (seq << 32) | entries, written by rank src at [src]
constexpr uint32_t PX_BEST_OFF = 4096;      // 2 parities x world x 4 u64 (3 used): (seq << 32) | 32 payload bits
constexpr uint32_t PX_INBOX_OFF = 16384;    // world regions of `cap` 16-byte entries
constexpr uint32_t PX_MAX_SPINS = 1u << 24; // polls of a peer's word before giving up: some ten seconds with the sleep
                                            // between them (the ranks' hosts do not start a batch at the same instant)
constexpr int PX_THREADS = 256;

struct PeerBufs {
    unsigned char* base[PX_MAX_WORLD];   // rank r's exchange buffer as this process sees it (own: local memory)
    uint32_t cap;                        // entries per (source, owner) inbox region
    uint32_t world, rank;
};

__device__ __forceinline__ uint32_t owner_of_pair(uint32_t h, uint32_t world) {
    return (uint32_t)(((unsigned long long)(h * 0x9E3779B1u) * world) >> 32);
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Add to the owned table (global counts).  Inserts are counted (the table's fill decides when it
// grows); an increase across the candidate threshold lists the slot, as table_add does.
__device__ __forceinline__ void owned_add(PairSlot* __restrict__ table, uint32_t logC, unsigned long long key, uint32_t c,
                                          DevState* st, uint32_t tau) {
    const uint32_t mask = (1u << logC) - 1u;
    uint32_t slot = (hash_pair(key) * 0x85EBCA6Bu) >> (32 - logC);   // not the owner hash again: that would fill 1/world of the table
    for (int p = 0; p < TABLE_MAX_PROBE; p++) {
        unsigned long long k = __ldcg(&table[slot].key);
        if (k == 0ull) {
            k = atomicCAS(&table[slot].key, 0ull, key);
            if (k == 0ull) { k = key; atomicAdd(&st->owned_inserted, 1u); }
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

// ── route: (pair, delta) entries of the local table → the owners' inboxes ──
__global__ void __launch_bounds__(PX_THREADS)
k_route(DevState* __restrict__ st, PairSlot* __restrict__ table, PeerBufs pb, uint32_t* __restrict__ fill) {
    __shared__ uint32_t s_last;
    // launch-invariant: written by set-up steps and by the last CTA of this kernel only
    if (st->early_stop | st->target_hit) return;
    if (st->status == DS_LOOKBACK_TIMEOUT) return;
    const bool full = st->recount != 0u;   // the count kernel of this iteration has just counted everything
    const uint32_t C = 1u << st->table_log2;
    const uint32_t n = full ? C : min(__ldcg(&st->dlist_n), DLIST_CAP);
    // A merge changes a few thousand pairs: only as many CTAs as that needs take part (and are waited for).
    // (`dlist_n` is put back to zero by the last of them, when every CTA that takes part has read it; a CTA
    // that reads the zero later has a number beyond `need` either way.)
    const uint32_t need = full ? gridDim.x : max(1u, min(gridDim.x, (n + 4u * PX_THREADS - 1u) / (4u * PX_THREADS)));
    if (blockIdx.x >= need) return;
    const uint32_t* __restrict__ dlist = st->dlist;
    uint4* __restrict__ t4 = reinterpret_cast<uint4*>(table);
    const int lane = threadIdx.x & 31;
    uint32_t live = 0u;
    bool sent = false;
    for (uint32_t i0 = blockIdx.x * PX_THREADS + (threadIdx.x & ~31u); i0 < n; i0 += need * PX_THREADS) {
        const uint32_t i = i0 + lane;
        uint32_t slot = 0u;
        uint4 q = make_uint4(0u, 0u, 0u, 0u);
        if (i < n) {
            slot = full ? i : __ldcg(dlist + i);
            q = __ldcg(t4 + slot);
        }
        const unsigned long long key = ((unsigned long long)q.y << 32) | q.x;
        if (key != 0ull) __stcg(t4 + slot, make_uint4(0u, 0u, 0u, 0u));   // the local table is empty again after this kernel
        const bool send = key != 0ull && q.z != 0u;
        live += send ? 1u : 0u;
        const uint32_t o = send ? owner_of_pair(hash_pair(key), pb.world) : 0xFFFFFFFFu;
        const uint32_t peers = __match_any_sync(0xFFFFFFFFu, o);
        if (send) {
            const int leader = __ffs(peers) - 1;
            uint32_t base = 0u;
            if (lane == leader) base = atomicAdd(&fill[o], (uint32_t)__popc(peers));
            base = __shfl_sync(peers, base, leader);
            const uint32_t d = base + (uint32_t)__popc(peers & ((1u << lane) - 1u));
            if (d < pb.cap) {
                uint4* inbox = reinterpret_cast<uint4*>(pb.base[o] + PX_INBOX_OFF) + (size_t)pb.rank * pb.cap;
                inbox[d] = make_uint4(q.x, q.y, q.z, 0u);
                sent = true;
            } else {
                atomicCAS(&st->status, (uint32_t)DS_OK, (uint32_t)DS_BUCKET_FULL);
            }
        }
    }
    if (full) {
        // the local table's fill, for the decision to grow (a table more than half full grows)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) live += __shfl_xor_sync(0xFFFFFFFFu, live, o);
        if (lane == 0 && live) atomicAdd(&st->occupied, live);
    }
    if (sent) __threadfence_system();   // this thread's entries are out before its CTA is counted as done
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(&st->xdone[0], 1u) == need - 1u) ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    const uint32_t seq = st->xseq;
    if (threadIdx.x < pb.world) {
        const uint32_t o = threadIdx.x;
        const uint32_t f = min(__ldcg(&fill[o]), pb.cap);
        fill[o] = 0u;
        unsigned long long* hdr = reinterpret_cast<unsigned long long*>(pb.base[o] + PX_HDR_OFF) + pb.rank;
        st_release_sys(hdr, ((unsigned long long)seq << 32) | f);
    }
    if (threadIdx.x == 0) {
        st->xdone[0] = 0u;
        st->dlist_n = 0u;
        if (full) {
            if ((unsigned long long)__ldcg(&st->occupied) * 2ull > (unsigned long long)C) st->want_grow = 1u;
            st->occupied = 0u;
        }
    }
}

// One warp: exchange {best, flags} with all peers, then set up the merge (or only agree on the
// status when `setup` is false).  `bc`/`bk`: this rank's best pair (0: none).  Every lane must call.
__device__ __forceinline__ void global_pick(DevState* st, DevState* snap, const PeerBufs& pb, uint32_t bc, unsigned long long bk,
                                            uint32_t* __restrict__ log, bool setup) {
    const int lane = threadIdx.x & 31;
    const uint32_t seq = snap->xseq, par = seq & 1u;
    const uint32_t pair32 = ((uint32_t)(bk >> 32) << 16) | ((uint32_t)bk & 0xFFFFu);
    const unsigned long long packed = bc ? (((unsigned long long)bc << 32) | (unsigned long long)(~pair32)) : 0ull;
    const uint32_t my_status = __ldcg(&st->status), my_grow = __ldcg(&st->want_grow);
    const unsigned long long tagv = (unsigned long long)seq << 32;
    if (lane < (int)pb.world) {
        unsigned long long* w = reinterpret_cast<unsigned long long*>(pb.base[lane] + PX_BEST_OFF) + ((size_t)(par * PX_MAX_WORLD + pb.rank) * 4);
        st_relaxed_sys(w + 0, tagv | (uint32_t)packed);
        st_relaxed_sys(w + 1, tagv | (uint32_t)(packed >> 32));
        st_relaxed_sys(w + 2, tagv | (my_status | (my_grow ? 0x100u : 0u)));
    }
    unsigned long long best = 0ull;
    uint32_t flags = 0u;
    bool timed_out = false;
    if (lane < (int)pb.world) {
        const unsigned long long* w = reinterpret_cast<const unsigned long long*>(pb.base[pb.rank] + PX_BEST_OFF) + ((size_t)(par * PX_MAX_WORLD + lane) * 4);
        unsigned long long a = 0, b = 0, c = 0;
        for (uint32_t spins = 0;; spins++) {
            a = ld_relaxed_sys(w + 0); b = ld_relaxed_sys(w + 1); c = ld_relaxed_sys(w + 2);
            if ((uint32_t)(a >> 32) == seq && (uint32_t)(b >> 32) == seq && (uint32_t)(c >> 32) == seq) break;
            if (spins > PX_MAX_SPINS || my_status == DS_LOOKBACK_TIMEOUT) { timed_out = true; break; }
            __nanosleep(400);
        }
        if (!timed_out) {
            best = ((unsigned long long)(uint32_t)b << 32) | (uint32_t)a;
            flags = (uint32_t)c;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const uint32_t of = __shfl_xor_sync(0xFFFFFFFFu, flags, o);
        best = ob > best ? ob : best;
        flags = max(flags & 0xFFu, of & 0xFFu) | ((flags | of) & 0x100u);
    }
    const bool any_timeout = __any_sync(0xFFFFFFFFu, timed_out);
    if (lane == 0) {
        uint32_t status = flags & 0xFFu;
        if (any_timeout) status = DS_LOOKBACK_TIMEOUT;
        if (status != DS_OK) st->status = status;      // every rank takes the largest status code of the job
        if (flags & 0x100u) st->want_grow = 1u;
        st->xseq = seq + 1u;
        if (setup) {
            snap->status = status;
            const uint32_t cnt = (uint32_t)(best >> 32);
            const uint32_t p32 = ~(uint32_t)best;
            const unsigned long long key = ((unsigned long long)(p32 >> 16) << 32) | (p32 & 0xFFFFu);
            setup_merge(st, snap, cnt, cnt ? key : 0ull, log);
            st->presetup_at = snap->iter_no;
        }
    }
}

// ── accumulate: the inboxes → the owned table; the last CTA picks from the candidate list ──
__global__ void __launch_bounds__(PX_THREADS)
k_accumulate(DevState* __restrict__ st, PeerBufs pb, uint32_t* __restrict__ log, int pick) {   // pick == 0: only bring the owned table up to date
    __shared__ __align__(16) DevState snap;
    __shared__ uint32_t s_fill[PX_MAX_WORLD + 1], s_last;
    __shared__ uint32_t r_c[PX_THREADS / 32];
    __shared__ unsigned long long r_k[PX_THREADS / 32];
    static_assert(sizeof(DevState) % 16 == 0 && sizeof(DevState) / 16 <= PX_THREADS, "control block copy");
    if (threadIdx.x < sizeof(DevState) / 16)
        reinterpret_cast<uint4*>(&snap)[threadIdx.x] = __ldcg(reinterpret_cast<const uint4*>(st) + threadIdx.x);
    __syncthreads();
    if (snap.early_stop | snap.target_hit) return;
    if (snap.status == DS_LOOKBACK_TIMEOUT) return;
    const uint32_t seq = snap.xseq;
    if (threadIdx.x < pb.world) {
        const unsigned long long* hdr = reinterpret_cast<const unsigned long long*>(pb.base[pb.rank] + PX_HDR_OFF) + threadIdx.x;
        unsigned long long h = 0ull;
        bool ok = false;
        for (uint32_t spins = 0; spins <= PX_MAX_SPINS; spins++) {
            h = ld_acquire_sys(hdr);
            if ((uint32_t)(h >> 32) == seq) { ok = true; break; }
            __nanosleep(400);
        }
        if (!ok) atomicExch(&st->status, (uint32_t)DS_LOOKBACK_TIMEOUT);
        s_fill[threadIdx.x + 1] = ok ? min((uint32_t)h, pb.cap) : 0u;
    }
    if (threadIdx.x == 0) s_fill[0] = 0u;
    __syncthreads();
    if (threadIdx.x == 0)
        for (uint32_t p = 0; p < pb.world; p++) s_fill[p + 1] += s_fill[p];   // exclusive offsets; s_fill[world] = total
    __syncthreads();
    const uint32_t total = s_fill[pb.world];
    PairSlot* __restrict__ owned = snap.owned;
    const uint32_t logO = snap.owned_log2, tau = snap.cand_tau;
    const uint4* __restrict__ inbox = reinterpret_cast<const uint4*>(pb.base[pb.rank] + PX_INBOX_OFF);
    for (uint32_t i = blockIdx.x * PX_THREADS + threadIdx.x; i < total; i += gridDim.x * PX_THREADS) {
        uint32_t src = 0u;
#pragma unroll
        for (int p = 1; p < PX_MAX_WORLD; p++) src += (p < (int)pb.world && i >= s_fill[p]) ? 1u : 0u;
        const uint4 q = __ldcg(inbox + (size_t)src * pb.cap + (i - s_fill[src]));
        const unsigned long long key = ((unsigned long long)q.y << 32) | q.x;
        if (key != 0ull && q.z != 0u) owned_add(owned, logO, key, q.z, st, tau);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(&st->xdone[1], 1u) == gridDim.x - 1u) ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x == 0) {
        st->xdone[1] = 0u;
        if ((unsigned long long)__ldcg(&st->owned_inserted) * 2ull > (1ull << logO)) st->want_grow = 1u;
    }
    if (!pick) return;
    // No usable list (a scan is due): the arg-max kernel of this iteration scans the owned table.
    if (!(snap.iter_no < snap.scan_from)) return;
    const uint4* __restrict__ t4 = reinterpret_cast<const uint4*>(owned);
    const uint32_t cand_n = __ldcg(&st->cand_n);
    const uint32_t n = min(cand_n, CAND_CAP);
    uint32_t bc = 0u;
    unsigned long long bk = 0ull;
    for (uint32_t i = threadIdx.x; i < n; i += PX_THREADS) {
        const uint4 q = __ldcg(t4 + __ldcg(snap.cand + i));
        const unsigned long long key = ((unsigned long long)q.y << 32) | q.x;
        if (key != 0ull && is_better(q.z, key, bc, bk)) { bc = q.z; bk = key; }
    }
    warp_best(bc, bk);
    if ((threadIdx.x & 31) == 0) { r_c[threadIdx.x >> 5] = bc; r_k[threadIdx.x >> 5] = bk; }
    __syncthreads();
    if (threadIdx.x >= 32) return;
    bc = threadIdx.x < PX_THREADS / 32 ? r_c[threadIdx.x] : 0u;
    bk = threadIdx.x < PX_THREADS / 32 ? r_k[threadIdx.x] : 0ull;
    warp_best(bc, bk);
    // The list decides as long as its best count is at least its threshold: every other owned pair
    // was below the threshold at the last full scan and has not crossed it since.  (A rank that
    // owns no pair at or above its threshold cannot tell whether it owns the global best.)
    const bool list_ok = bc >= snap.cand_tau && cand_n < CAND_CAP && snap.since_scan < CAND_MAX_AGE;
    if (!list_ok) {
        if (threadIdx.x == 0) {
            void_candidates(st, snap.iter_no);   // this iteration's arg-max kernel scans
            st->cand_tau_next = max(2u, min(snap.cand_tau, snap.cand_tau_next) / 2u);
        }
        return;
    }
    if (threadIdx.x == 0) st->since_scan = snap.since_scan + 1u;
    global_pick(st, &snap, pb, bc, bk, log, true);
}

// ── full scan of the owned table (the candidate list is stale), then the global pick ──
__global__ void __launch_bounds__(AM_THREADS)
k_argmax_peer(DevState* __restrict__ st, CtaBest* __restrict__ cta_best, PeerBufs pb, uint32_t* __restrict__ log) {
    __shared__ uint32_t sc[AM_THREADS / 32];
    __shared__ unsigned long long sk[AM_THREADS / 32];
    __shared__ bool is_last;
    __shared__ __align__(16) DevState snap;
    if (threadIdx.x < sizeof(DevState) / 16)
        reinterpret_cast<uint4*>(&snap)[threadIdx.x] = __ldcg(reinterpret_cast<const uint4*>(st) + threadIdx.x);
    __syncthreads();
    if (snap.presetup_at == snap.iter_no) return;   // the accumulate kernel has already picked
    if (snap.early_stop | snap.target_hit) {
        if (blockIdx.x == 0 && threadIdx.x == 0) { st->active = 0u; st->tail_fix = 0u; }
        return;
    }
    if (snap.status == DS_LOOKBACK_TIMEOUT) {
        if (blockIdx.x == 0 && threadIdx.x == 0) st->active = 0u;
        return;
    }
    const uint32_t C = 1u << snap.owned_log2;
    const uint4* __restrict__ t4 = reinterpret_cast<const uint4*>(snap.owned);
    uint32_t* __restrict__ cand = snap.cand;
    const uint32_t tau_scan = snap.cand_tau_next;
    uint32_t bc = 0;
    unsigned long long bk = 0ull;
    const uint32_t stride = gridDim.x * AM_THREADS;
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
                if (is_better(q[u].z, key, bc, bk)) { bc = q[u].z; bk = key; }
                if (q[u].z >= tau_scan) {
                    const uint32_t k = atomicAdd(&st->cand_n, 1u);
                    if (k < CAND_CAP) cand[k] = i0 + u * stride;
                }
            }
        }
    }
    warp_best(bc, bk);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sc[warp] = bc; sk[warp] = bk; }
    __syncthreads();
    if (warp == 0) {
        bc = lane < AM_THREADS / 32 ? sc[lane] : 0u;
        bk = lane < AM_THREADS / 32 ? sk[lane] : 0ull;
        warp_best(bc, bk);
        if (lane == 0) {
            cta_best[blockIdx.x].key = bk;
            cta_best[blockIdx.x].count = bc;
            __threadfence();
            is_last = atomicAdd(&st->argmax_done, 1u) == gridDim.x - 1;
        }
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    bc = 0; bk = 0ull;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += AM_THREADS) {
        const uint32_t c = __ldcg(&cta_best[i].count);
        const unsigned long long k = __ldcg(&cta_best[i].key);
        if (is_better(c, k, bc, bk)) { bc = c; bk = k; }
    }
    warp_best(bc, bk);
    __syncthreads();
    if (lane == 0) { sc[warp] = bc; sk[warp] = bk; }
    __syncthreads();
    if (warp != 0) return;
    bc = lane < AM_THREADS / 32 ? sc[lane] : 0u;
    bk = lane < AM_THREADS / 32 ? sk[lane] : 0ull;
    warp_best(bc, bk);
    if (lane == 0) {
        st->argmax_done = 0u;
        st->full_scans += 1u;
        st->since_scan = 0u;
        const uint32_t listed = __ldcg(&st->cand_n);
        if (tau_scan == 0xFFFFFFFFu || listed >= CAND_CAP) {
            // no usable list yet (first scan, or too many slots above the threshold): scan again next time
            const uint32_t over = listed >= CAND_CAP ? 1u : 0u;
            void_candidates(st, snap.iter_no + 1u);
            st->cand_tau_next = over ? min(0x7FFFFFFFu, tau_scan) * 2u : max(2u, bc / 2u);
        } else {
            st->scan_from = SCAN_NEVER;
            st->cand_tau = tau_scan;
            st->cand_tau_next = max(2u, bc / 2u);
        }
    }
    __syncwarp();
    global_pick(st, &snap, pb, bc, bk, log, true);
}

// End of a batch: the ranks agree on {status, want_grow} once more, so that a status raised by the
// batch's last merge kernel on one rank sends every rank down the same host-side branch.
__global__ void k_batch_sync(DevState* __restrict__ st, PeerBufs pb) {
    __shared__ __align__(16) DevState snap;
    if (threadIdx.x < sizeof(DevState) / 16)
        reinterpret_cast<uint4*>(&snap)[threadIdx.x] = __ldcg(reinterpret_cast<const uint4*>(st) + threadIdx.x);
    __syncwarp();
    global_pick(st, &snap, pb, 0u, 0ull, nullptr, false);
}

}  // namespace b200bpe
