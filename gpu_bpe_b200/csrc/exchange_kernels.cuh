// Sharded training: the count exchange between the local pair count and the merge set-up.
//
// The reference trains on one device; sharding is this library's addition.  The corpus is cut
// at word starts into one contiguous span per GPU (pairs never cross a word start, so local
// counting and local merging stay exact).  Per merge:
//
//   1. k_partition    each rank copies its local table (kept up to date by its merge kernel, or
//                     just counted and then emptied here) into one outgoing bucket per owner,
//                     owner = hash(pair) mod world
//   2. all-to-all     fixed-size NCCL send/recv of the buckets (slot 0 of a bucket is a header
//                     holding its fill, so buckets never need clearing)
//   3. k_accumulate   the owner sums what it received into its table of owned pairs
//   4. k_argmax_setup (mode 1) arg-max over the owned pairs → packed (count << 32 | ~pair)
//   5. all-reduce max of {packed best, status, want_grow, largest bucket fill} — 32 bytes
//   6. k_setup_from_packed  every rank decodes the same winner and sets up its local merge
//
// max over the packed word reproduces the reference's order exactly: larger count first, then
// the smaller pair id (train.wgsl:83-85).
#pragma once

#include "ctx.cuh"
#include "train_kernels.cuh"

namespace b200bpe {

__device__ __forceinline__ uint32_t owner_of(uint32_t h, uint32_t world) {
    return (uint32_t)(((unsigned long long)(h * 0x9E3779B1u) * world) >> 32);
}

// buckets: world consecutive regions of `cap` slots; slot 0 = header (count = fill).
__global__ void __launch_bounds__(256)
k_partition(DevState* __restrict__ st, PairSlot* __restrict__ table, PairSlot* __restrict__ buckets,
            uint32_t* __restrict__ fill, uint32_t cap, uint32_t world) {
    if (st->early_stop | st->target_hit) return;
    const uint32_t C = 1u << st->table_log2;
    const bool keep = st->incremental != 0u;   // an incrementally maintained table stays as it is (dead keys are skipped)
    uint4* __restrict__ t4 = reinterpret_cast<uint4*>(table);
    // A warp stays in the loop as a whole (the bound is tested on the warp's first slot).
    // Room in a bucket is reserved once per warp and owner (match-any), not once per entry: the
    // `world` fill counters would otherwise take one atomic for every live pair of the table.
    const int lane = threadIdx.x & 31;
    uint32_t used = 0u;   // slots that hold a key, dead or alive: the table's fill, for the decision to grow
    for (uint32_t i0 = blockIdx.x * blockDim.x + (threadIdx.x & ~31u); i0 < C; i0 += gridDim.x * blockDim.x) {
        const uint32_t i = i0 + lane;
        const uint4 q = i < C ? __ldcg(t4 + i) : make_uint4(0u, 0u, 0u, 0u);
        const unsigned long long key = ((unsigned long long)q.y << 32) | q.x;
        used += key != 0ull ? 1u : 0u;
        const bool live = key != 0ull && !(keep && q.z == 0u);
        const uint32_t o = live ? owner_of(hash_pair(key), world) : 0xFFFFFFFFu;
        const uint32_t peers = __match_any_sync(0xFFFFFFFFu, o);
        if (live) {
            const int leader = __ffs(peers) - 1;
            uint32_t base = 0u;
            if (lane == leader) base = atomicAdd(&fill[o], (uint32_t)__popc(peers));
            base = __shfl_sync(peers, base, leader);
            const uint32_t d = base + (uint32_t)__popc(peers & ((1u << lane) - 1u)) + 1u;  // slot 0 is the header
            if (d < cap) {
                reinterpret_cast<uint4*>(buckets)[(size_t)o * cap + d] = q;
            } else {
                atomicCAS(&st->status, (uint32_t)DS_OK, (uint32_t)DS_BUCKET_FULL);
            }
            if (!keep) __stcg(t4 + i, make_uint4(0u, 0u, 0u, 0u));
        }
    }
    if (keep) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) used += __shfl_xor_sync(0xFFFFFFFFu, used, o);
        if (lane == 0 && used) atomicAdd(&st->occupied, used);
    }
}

// Write the bucket headers and reset the fill counters for the next merge.
__global__ void k_seal_buckets(DevState* __restrict__ st, PairSlot* __restrict__ buckets, uint32_t* __restrict__ fill,
                               uint32_t cap, uint32_t world) {
    const uint32_t o = threadIdx.x;
    if (o >= world) return;
    if (o == 0u) {
        // a local table that is kept from merge to merge and is more than half full grows at the end of the batch
        // (without this it would only grow after a chain of 1,024 failed probes)
        if (st->incremental != 0u && (unsigned long long)st->occupied * 2ull > (1ull << st->table_log2)) st->want_grow = 1u;
        st->occupied = 0u;
    }
    const bool idle = (st->early_stop | st->target_hit) != 0u;
    const uint32_t f = idle ? 0u : min(fill[o], cap - 1u);
    buckets[(size_t)o * cap].key = 0ull;
    buckets[(size_t)o * cap].count = f;
    if (!idle) atomicMax(&st->fill_hwm, fill[o]);
    fill[o] = 0u;
}

__global__ void __launch_bounds__(256)
k_accumulate(DevState* __restrict__ st, const PairSlot* __restrict__ inbox, uint32_t cap, uint32_t world,
             PairSlot* __restrict__ owned, uint32_t owned_log2) {
    if (st->early_stop | st->target_hit) return;
    for (uint32_t p = 0; p < world; p++) {
        const PairSlot* __restrict__ b = inbox + (size_t)p * cap;
        const uint32_t f = min(b[0].count, cap - 1u);
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < f; i += gridDim.x * blockDim.x) {
            const unsigned long long key = b[1 + i].key;
            const uint32_t c = b[1 + i].count;
            if (key) table_add(owned, owned_log2, key, hash_pair(key) * 0x85EBCA6Bu, c, st, 0xFFFFFFFFu);  // no candidate list on owned tables
        }
    }
}

__global__ void k_pack_flags(DevState* __restrict__ st, unsigned long long* __restrict__ words) {
    const bool idle = (st->early_stop | st->target_hit) != 0u;
    words[0] = idle ? 0ull : st->best_packed;
    words[1] = st->status;
    words[2] = st->want_grow;
    words[3] = st->fill_hwm;
}

__global__ void k_unpack_flags(DevState* __restrict__ st, const unsigned long long* __restrict__ words,
                               uint32_t* __restrict__ log) {
    if (st->early_stop | st->target_hit) return;
    // every rank takes the largest status code: a full bucket anywhere stops all ranks alike
    if (words[1] > st->status) st->status = (uint32_t)words[1];
    if (words[2]) st->want_grow = 1u;
    st->fill_hwm = (uint32_t)words[3];
    const unsigned long long p = words[0];
    const uint32_t cnt = (uint32_t)(p >> 32);
    const uint32_t pair32 = ~(uint32_t)p;
    const unsigned long long key = ((unsigned long long)(pair32 >> 16) << 32) | (pair32 & 0xFFFFu);
    setup_merge(st, cnt, cnt ? key : 0ull, log);
}

// End of a batch: only the flags are taken over (no merge is set up).
__global__ void k_unpack_status(DevState* __restrict__ st, const unsigned long long* __restrict__ words) {
    if (words[1] > st->status) st->status = (uint32_t)words[1];
    if (words[2]) st->want_grow = 1u;
    if (words[3] > st->fill_hwm) st->fill_hwm = (uint32_t)words[3];
}
__global__ void k_pack_status(DevState* __restrict__ st, unsigned long long* __restrict__ words) {
    words[0] = 0ull;
    words[1] = st->status;
    words[2] = st->want_grow;
    words[3] = st->fill_hwm;
}

struct Exchange {
    PairSlot* send = nullptr;   // world buckets of `cap` slots
    PairSlot* recv = nullptr;   // world inboxes of `cap` slots
    PairSlot* owned = nullptr;  // pairs this rank owns
    uint32_t* fill = nullptr;
    unsigned long long* words = nullptr;      // 4 words out
    unsigned long long* words_max = nullptr;  // 4 words after the all-reduce
    uint32_t cap = 0;        // slots per bucket in use (header included); the same on every rank
    uint32_t cap_alloc = 0;  // slots per bucket allocated
    uint32_t owned_log2 = 0, local_log2 = 0;

    void release() {
        cudaFree(send); cudaFree(recv); cudaFree(owned); cudaFree(fill); cudaFree(words); cudaFree(words_max);
        send = recv = owned = nullptr; fill = nullptr; words = words_max = nullptr;
    }

    // first_cap: bucket size to start with (0 = the default); tests start small to exercise the overflow path
    b200bpe_status init(Ctx* ctx, uint32_t table_log2, uint32_t first_cap = 0) {
        const uint32_t world = (uint32_t)ctx->world;
        local_log2 = table_log2;
        owned_log2 = table_log2;
        // A local table is at most half full before it grows; spread over `world` owners that is
        // C / (2 * world) entries per bucket on average.  Twice that, plus the header.
        cap_alloc = std::max<uint32_t>(64u, (1u << table_log2) / world) + 1u;
        // What is sent per peer and merge is `cap` slots, sized to the traffic actually seen (the
        // host adapts it between batches from the all-reduced high-water mark), not to the table.
        cap = std::min<uint32_t>(cap_alloc, 32768u + 1u);
        if (first_cap >= 2 && first_cap <= cap_alloc) cap = first_cap;
        B2_CUDA(cudaMalloc(&send, sizeof(PairSlot) * (size_t)cap_alloc * world));
        B2_CUDA(cudaMalloc(&recv, sizeof(PairSlot) * (size_t)cap_alloc * world));
        B2_CUDA(cudaMalloc(&owned, sizeof(PairSlot) << owned_log2));
        B2_CUDA(cudaMalloc(&fill, sizeof(uint32_t) * world));
        B2_CUDA(cudaMalloc(&words, 32));
        B2_CUDA(cudaMalloc(&words_max, 32));
        B2_CUDA(cudaMemsetAsync(send, 0, sizeof(PairSlot) * (size_t)cap_alloc * world, ctx->stream));
        B2_CUDA(cudaMemsetAsync(recv, 0, sizeof(PairSlot) * (size_t)cap_alloc * world, ctx->stream));
        B2_CUDA(cudaMemsetAsync(owned, 0, sizeof(PairSlot) << owned_log2, ctx->stream));
        B2_CUDA(cudaMemsetAsync(fill, 0, sizeof(uint32_t) * world, ctx->stream));
        return B200BPE_OK;
    }

    b200bpe_status resize(Ctx* ctx, uint32_t table_log2, uint32_t first_cap = 0) {
        release();
        return init(ctx, table_log2, first_cap);
    }

    // After the last merge kernel of a batch: every rank takes the largest status and the other
    // flags of the job, so that all ranks grow, resize or give up together.
    b200bpe_status enqueue_status_sync(Ctx* ctx, DevState* st) {
        cudaStream_t s = ctx->stream;
        k_pack_status<<<1, 1, 0, s>>>(st, words);
        int rc = ctx->nccl.AllReduce(words, words_max, 4, /*ncclUint64*/ 5, /*ncclMax*/ 2, ctx->comm, s);
        if (rc) return nccl_fail(ctx, rc, "ncclAllReduce");
        k_unpack_status<<<1, 1, 0, s>>>(st, words_max);
        return B200BPE_OK;
    }

    // Between batches: fit the bucket size to the traffic.  Every rank sees the same all-reduced
    // numbers, so every rank takes the same decision.  Returns true if `cap` changed.
    bool adapt(bool overflowed, uint32_t fill_hwm) {
        uint32_t want = cap;
        if (overflowed) want = std::min<uint32_t>(cap_alloc, std::max<uint32_t>(cap * 4u, fill_hwm * 2u + 2u));
        else if ((uint64_t)fill_hwm * 4u < cap && cap > 4097u) want = std::max<uint32_t>(4097u, fill_hwm * 2u + 1u);
        if (want == cap) return false;
        cap = want;
        return true;
    }

    b200bpe_status nccl_fail(Ctx* ctx, int rc, const char* what) {
        set_last_error(std::string(what) + ": " + (ctx->nccl.GetErrorString ? ctx->nccl.GetErrorString(rc) : "nccl error"));
        return B200BPE_ERR_NCCL;
    }

    // Steps 1-3: after this the owned table holds the global counts of this rank's pairs.
    b200bpe_status enqueue_counts_only(Ctx* ctx, DevState* st, PairSlot* table, uint32_t table_log2) {
        cudaStream_t s = ctx->stream;
        const uint32_t world = (uint32_t)ctx->world;
        const int grid = std::max(1, std::min(ctx->sm_count * 4, (int)((1u << table_log2) / 1024)));
        k_partition<<<grid, 256, 0, s>>>(st, table, send, fill, cap, world);
        k_seal_buckets<<<1, 32, 0, s>>>(st, send, fill, cap, world);
        int rc = ctx->nccl.GroupStart();
        if (rc) return nccl_fail(ctx, rc, "ncclGroupStart");
        const size_t bytes = sizeof(PairSlot) * (size_t)cap;
        for (uint32_t p = 0; p < world; p++) {
            if ((int)p == ctx->rank) continue;
            rc = ctx->nccl.Send(send + (size_t)p * cap, bytes, /*ncclUint8*/ 1, (int)p, ctx->comm, s);
            if (rc) return nccl_fail(ctx, rc, "ncclSend");
            rc = ctx->nccl.Recv(recv + (size_t)p * cap, bytes, /*ncclUint8*/ 1, (int)p, ctx->comm, s);
            if (rc) return nccl_fail(ctx, rc, "ncclRecv");
        }
        rc = ctx->nccl.GroupEnd();
        if (rc) return nccl_fail(ctx, rc, "ncclGroupEnd");
        // This rank's own bucket needs no transfer.
        B2_CUDA(cudaMemcpyAsync(recv + (size_t)ctx->rank * cap, send + (size_t)ctx->rank * cap, bytes,
                                cudaMemcpyDeviceToDevice, s));
        k_accumulate<<<std::max(1, ctx->sm_count * 2), 256, 0, s>>>(st, recv, cap, world, owned, owned_log2);
        return B200BPE_OK;
    }

    // Steps 1-6.
    b200bpe_status enqueue(Ctx* ctx, DevState* st, PairSlot* table, uint32_t table_log2, CtaBest* cta_best,
                           uint32_t* log, int grid_am) {
        cudaStream_t s = ctx->stream;
        b200bpe_status r = enqueue_counts_only(ctx, st, table, table_log2);
        if (r) return r;
        k_argmax_setup<<<grid_am, AM_THREADS, 0, s>>>(st, owned, cta_best, log, 1, owned_log2);
        k_pack_flags<<<1, 1, 0, s>>>(st, words);
        int rc = ctx->nccl.AllReduce(words, words_max, 4, /*ncclUint64*/ 5, /*ncclMax*/ 2, ctx->comm, s);
        if (rc) return nccl_fail(ctx, rc, "ncclAllReduce");
        k_unpack_flags<<<1, 1, 0, s>>>(st, words_max, log);
        return B200BPE_OK;
    }
};

}  // namespace b200bpe
