// Host side of the training path: device buffers, the per-batch CUDA graph, the batch loop
// that mirrors BPETrainer.#runTrainingLoop (src/bpe/trainer.js:225-335 of the reference), and
// the C entry points declared in include/b200bpe.h.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "ctx.cuh"
#include "train_kernels.cuh"
#include "exchange_kernels.cuh"
#include "peer_exchange.cuh"

namespace b200bpe {

namespace {

constexpr uint32_t MAX_TABLE_LOG2 = 27;

uint32_t ceil_log2(uint64_t x) {
    uint32_t l = 0;
    while ((1ull << l) < x) l++;
    return l;
}

}  // namespace

// Host side of the peer-memory exchange: this rank's exchange buffer (headers, best words, inboxes),
// the peers' buffers mapped through CUDA IPC (one process per GPU), the table of owned pairs and
// the list of delta-table slots to send.
struct PeerExchange {
    unsigned char* xbuf = nullptr;
    size_t xbuf_bytes = 0;
    PairSlot* owned = nullptr;
    uint32_t owned_log2 = 0;
    uint32_t* dlist = nullptr;
    uint32_t* fill = nullptr;
    void* mapped[PX_MAX_WORLD] = {};
    PeerBufs pb{};
    bool ok = false;

    void release() {
        for (auto& m : mapped) { if (m) cudaIpcCloseMemHandle(m); m = nullptr; }
        cudaFree(xbuf); cudaFree(owned); cudaFree(dlist); cudaFree(fill);
        xbuf = nullptr; owned = nullptr; dlist = nullptr; fill = nullptr;
        ok = false;
    }

    // Collective over the job's ranks.  Returns OK with ok == false when some rank could not map its
    // peers (every rank then takes the NCCL exchange instead).
    b200bpe_status init(Ctx* ctx, uint32_t table_log2) {
        const uint32_t world = (uint32_t)ctx->world;
        cudaStream_t s = ctx->stream;
        if (world > PX_MAX_WORLD) return B200BPE_OK;
        owned_log2 = table_log2;
        // an inbox region holds what one rank can send one owner after a full count: a local table is
        // at most half full before it grows, and the owners share its pairs about evenly
        pb.cap = std::max<uint32_t>(4096u, (1u << table_log2) / world);
        pb.world = world;
        pb.rank = (uint32_t)ctx->rank;
        xbuf_bytes = PX_INBOX_OFF + (size_t)world * pb.cap * 16;
        B2_CUDA(cudaMalloc(&xbuf, xbuf_bytes));
        B2_CUDA(cudaMalloc(&owned, sizeof(PairSlot) << owned_log2));
        B2_CUDA(cudaMalloc(&dlist, sizeof(uint32_t) * DLIST_CAP));
        B2_CUDA(cudaMalloc(&fill, sizeof(uint32_t) * PX_MAX_WORLD));
        B2_CUDA(cudaMemsetAsync(xbuf, 0, PX_INBOX_OFF, s));
        B2_CUDA(cudaMemsetAsync(owned, 0, sizeof(PairSlot) << owned_log2, s));
        B2_CUDA(cudaMemsetAsync(fill, 0, sizeof(uint32_t) * PX_MAX_WORLD, s));
        // exchange the IPC handles of the buffers (64 bytes each) with an all-gather
        cudaIpcMemHandle_t mine{};
        unsigned long long failed = cudaIpcGetMemHandle(&mine, xbuf) != cudaSuccess ? 1ull : 0ull;
        cudaGetLastError();
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
        unsigned char* d_h = nullptr;
        B2_CUDA(cudaMalloc(&d_h, (size_t)world * 64 + 16));
        B2_CUDA(cudaMemcpyAsync(d_h + (size_t)ctx->rank * 64, &mine, 64, cudaMemcpyHostToDevice, s));
        int rc = ctx->nccl.AllGather(d_h + (size_t)ctx->rank * 64, d_h, 64, /*ncclUint8*/ 1, ctx->comm, s);
        if (rc) { cudaFree(d_h); set_last_error("ncclAllGather failed"); return B200BPE_ERR_NCCL; }
        std::vector<cudaIpcMemHandle_t> all(world);
        B2_CUDA(cudaMemcpyAsync(all.data(), d_h, (size_t)world * 64, cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaStreamSynchronize(s));
        for (uint32_t p = 0; p < world && !failed; p++) {
            if ((int)p == ctx->rank) { pb.base[p] = xbuf; continue; }
            void* ptr = nullptr;
            if (cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); failed = 1ull; break; }
            mapped[p] = ptr;
            pb.base[p] = static_cast<unsigned char*>(ptr);
        }
        // every rank learns whether every rank succeeded
        unsigned long long* d_f = reinterpret_cast<unsigned long long*>(d_h + (size_t)world * 64);
        static_assert(true, "");
        B2_CUDA(cudaMemcpyAsync(d_f, &failed, 8, cudaMemcpyHostToDevice, s));
        rc = ctx->nccl.AllReduce(d_f, d_f, 1, /*ncclUint64*/ 5, /*ncclMax*/ 2, ctx->comm, s);
        if (rc) { cudaFree(d_h); set_last_error("ncclAllReduce failed"); return B200BPE_ERR_NCCL; }
        B2_CUDA(cudaMemcpyAsync(&failed, d_f, 8, cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaStreamSynchronize(s));
        cudaFree(d_h);
        if (failed) { release(); return B200BPE_OK; }
        ok = true;
        return B200BPE_OK;
    }
};

// Collective over the job's ranks: every rank leaves with the largest v of any rank.
static b200bpe_status agree_on_max(Ctx* ctx, unsigned long long* v) {
    if (ctx->world <= 1) return B200BPE_OK;
    unsigned long long* d = nullptr;
    B2_CUDA(cudaMalloc(&d, 8));
    B2_CUDA(cudaMemcpyAsync(d, v, 8, cudaMemcpyHostToDevice, ctx->stream));
    const int rc = ctx->nccl.AllReduce(d, d, 1, /*ncclUint64*/ 5, /*ncclMax*/ 2, ctx->comm, ctx->stream);
    if (rc) { cudaFree(d); set_last_error("ncclAllReduce failed"); return B200BPE_ERR_NCCL; }
    B2_CUDA(cudaMemcpyAsync(v, d, 8, cudaMemcpyDeviceToHost, ctx->stream));
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    cudaFree(d);
    return B200BPE_OK;
}

struct Trainer {
    Ctx* ctx = nullptr;
    uint64_t n0 = 0;            // symbols at creation (this rank)
    b200bpe_train_opts opts{};
    uint32_t merges_goal = 0;   // target_vocab_size - first_token_id
    // resident inputs, to rebuild the symbols on reset
    uint8_t* d_bytes = nullptr;
    uint8_t* d_mask = nullptr;
    uint32_t* d_sym_init = nullptr;
    bool own_inputs = true;
    bool has_mask = false;
    bool incremental = false;  // local table updated in place by the merge kernel (unless FULL_RECOUNT)
    // working set
    uint32_t* buf[2] = {nullptr, nullptr};
    uint64_t cap_elems = 0;
    PairSlot* table = nullptr;
    uint32_t table_log2 = 0;
    DevState* d_state = nullptr;
    DevState* h_state = nullptr;  // pinned
    uint32_t* d_log = nullptr;
    uint32_t* h_log = nullptr;    // pinned
    CtaBest* d_cta_best = nullptr;
    uint32_t* d_cand = nullptr;   // candidate list of the arg-max (slot indices)
    unsigned long long* d_desc = nullptr;
    DeltaQueues dq{nullptr, nullptr, nullptr, 0, 0};  // incremental mode only
    Exchange xch;                 // sharded runs, NCCL exchange
    PeerExchange px;              // sharded runs, peer-memory exchange (the default)
    bool peer = false;            // which of the two is in use
    uint32_t xseq_next = 1;       // peer exchange: sequence number of the next round (continues across resets)
    uint64_t launches = 0;        // kernel launches of this trainer since creation (graph launches count their nodes)
    uint32_t graph_kernels = 0;
    cudaGraphExec_t graph = nullptr;
    uint32_t graph_iters = 0;
    int grid_pc = 1, grid_am = 1, grid_mc = 1, grid_rt = 1, grid_acc = 1;
    // host mirror
    uint32_t merges_done = 0;
    bool early_stop = false;
    uint64_t cur_n = 0;
    // timing
    cudaEvent_t ev_run0 = nullptr, ev_run1 = nullptr;
    double last_run_ms = 0, last_reset_ms = 0;
    std::vector<cudaEvent_t> kev;
    b200bpe_kernel_stats stats{};

    ~Trainer();
    b200bpe_status alloc_common();
    b200bpe_status init_state();
    b200bpe_status build_graph();
    b200bpe_status enqueue_merge(int iter, bool timed);
    b200bpe_status grow_table();
    // Kernel argument for the pair table: on one GPU the kernels take it from the control block, so a
    // captured graph survives the table being replaced; the sharded path passes pointers.
    PairSlot* ktable() const { return ctx->world > 1 ? table : nullptr; }
    // only an arg-max that works from a candidate list can use up an iteration without a merge
    uint32_t spare_iters() const { return (incremental && ctx->world == 1) ? 4u : 0u; }
    b200bpe_status run(uint32_t max_merges, uint32_t* merges_out, uint32_t* counts_out, uint32_t* n_out,
                       uint32_t* early_out, b200bpe_progress_cb cb, void* user);
};

Trainer::~Trainer() {
    if (ctx) cudaSetDevice(ctx->device);
    if (graph) cudaGraphExecDestroy(graph);
    if (own_inputs) { cudaFree(d_bytes); cudaFree(d_mask); }
    cudaFree(d_sym_init);
    cudaFree(buf[0]); cudaFree(buf[1]); cudaFree(table); cudaFree(d_state); cudaFree(d_log);
    cudaFree(d_cta_best); cudaFree(d_desc); cudaFree(d_cand); cudaFree(dq.minus); cudaFree(dq.plus); cudaFree(dq.counts);
    xch.release();
    px.release();
    if (h_state) cudaFreeHost(h_state);
    if (h_log) cudaFreeHost(h_log);
    if (ev_run0) cudaEventDestroy(ev_run0);
    if (ev_run1) cudaEventDestroy(ev_run1);
    for (auto e : kev) cudaEventDestroy(e);
}

b200bpe_status Trainer::alloc_common() {
    cap_elems = ((n0 + 3) & ~3ull) + 8;
    B2_CUDA(cudaMalloc(&buf[0], cap_elems * 4));
    B2_CUDA(cudaMalloc(&buf[1], cap_elems * 4));
    table_log2 = opts.table_log2;
    // Start small (every merge scans the whole table for the arg-max); it doubles when half full.
    // (sharded: sized for the whole corpus, because the distinct pairs of a shard, and the pairs a rank owns, do not
    // shrink in proportion to the shard; too small a start costs a chain of grow-and-recount restarts)
    if (table_log2 == 0) table_log2 = std::min<uint32_t>(21, std::max<uint32_t>(15, ceil_log2(n0 * (uint64_t)ctx->world / 128 + 1)));
    table_log2 = std::min(table_log2, MAX_TABLE_LOG2);
    if (ctx->world > 1) {
        // The ranks' spans differ by a few bytes, which can put them either side of a power of two; the exchange
        // buffers are laid out from the table size, so every rank takes the largest any rank chose.
        unsigned long long v = table_log2;
        b200bpe_status r = agree_on_max(ctx, &v);
        if (r) return r;
        table_log2 = (uint32_t)v;
    }
    B2_CUDA(cudaMalloc(&table, sizeof(PairSlot) << table_log2));
    B2_CUDA(cudaMalloc(&d_state, sizeof(DevState)));
    B2_CUDA(cudaMallocHost(&h_state, sizeof(DevState)));
    const size_t log_bytes = (size_t)std::max<uint32_t>(1, merges_goal) * 16;
    B2_CUDA(cudaMalloc(&d_log, log_bytes));
    B2_CUDA(cudaMallocHost(&h_log, log_bytes));
    const int sms = ctx->sm_count;
    const uint64_t nvec = (n0 + 3) / 4;
    grid_pc = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)sms * PC_CTAS_PER_SM, (nvec + PC_THREADS - 1) / PC_THREADS));
    grid_am = std::max(1, std::min(sms * 4, (int)((1u << table_log2) / (AM_THREADS * 4))));
    const uint64_t ntiles = (n0 + MC_TILE - 1) / MC_TILE;
    grid_mc = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)sms * MC_CTAS_PER_SM, ntiles));
    grid_rt = sms;          // route: a few thousand entries per merge, the whole local table after a full count
    grid_acc = sms / 2;     // accumulate: as many entries again, from all ranks
    B2_CUDA(cudaMalloc(&d_cta_best, sizeof(CtaBest) * (size_t)(sms * 4 + 1)));
    B2_CUDA(cudaMalloc(&d_cand, sizeof(uint32_t) * CAND_CAP));
    B2_CUDA(cudaMalloc(&d_desc, sizeof(unsigned long long) * (ntiles + 1)));
    B2_CUDA(cudaMemsetAsync(d_desc, 0, sizeof(unsigned long long) * (ntiles + 1), ctx->stream));
    if (incremental) {
        // one queue segment per CTA of the merge kernel; together about n0 / 2 entries per queue,
        // which a merge only exceeds when it rewrites a large share of the corpus (then the
        // overflow is applied to the table directly)
        dq.segments = (uint32_t)grid_mc;
        dq.seg_cap = (uint32_t)std::max<uint64_t>(1024, (n0 / 2) / dq.segments);
        B2_CUDA(cudaMalloc(&dq.minus, (size_t)dq.seg_cap * dq.segments * 4));
        B2_CUDA(cudaMalloc(&dq.plus, (size_t)dq.seg_cap * dq.segments * 4));
        B2_CUDA(cudaMalloc(&dq.counts, (size_t)dq.segments * 8));
        B2_CUDA(cudaMemsetAsync(dq.counts, 0, (size_t)dq.segments * 8, ctx->stream));
    }
    B2_CUDA(cudaEventCreate(&ev_run0));
    B2_CUDA(cudaEventCreate(&ev_run1));
    B2_CUDA(cudaFuncSetAttribute(k_pair_count<PC_SLOTS, PC_THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 PC_SMEM_BYTES));
    // The count and merge kernels need the largest shared-memory carve-out; the small kernels between them ask for
    // the same one, so that the SMs are not reconfigured from launch to launch.
    B2_CUDA(cudaFuncSetAttribute(k_argmax_setup, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    B2_CUDA(cudaFuncSetAttribute(k_literal_tail, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    B2_CUDA(cudaFuncSetAttribute(k_merge_compact<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MC_SMEM_BYTES));
    B2_CUDA(cudaFuncSetAttribute(k_merge_compact<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, MC_SMEM_BYTES));
    B2_CUDA(cudaFuncSetAttribute(k_merge_compact<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MC_SMEM_BYTES));
    B2_CUDA(cudaFuncSetAttribute(k_merge_compact<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, MC_SMEM_BYTES));
    B2_CUDA(cudaFuncSetAttribute(k_merge_compact<false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MC_SMEM_BYTES));
    if (ctx->world > 1) {
        // The peer-memory exchange needs an incrementally maintained table; FLAG_NCCL_EXCHANGE, a full
        // recount per merge, or peers that cannot be mapped select the NCCL exchange.
        if (incremental && !(opts.flags & B200BPE_FLAG_NCCL_EXCHANGE)) {
            b200bpe_status s = px.init(ctx, table_log2);
            if (s) return s;
            peer = px.ok;
        }
        if (!peer) {
            b200bpe_status s = xch.init(ctx, table_log2, opts.exchange_cap);
            if (s) return s;
        }
    }
    return B200BPE_OK;
}

// Rebuild the tagged symbols from the resident inputs and put the control block back to the
// state of a fresh BPETrainer.train call (trainer.js:187-196).
b200bpe_status Trainer::init_state() {
    cudaStream_t s = ctx->stream;
    B2_CUDA(cudaEventRecord(ev_run0, s));
    if (d_sym_init) {
        B2_CUDA(cudaMemcpyAsync(buf[0], d_sym_init, n0 * 4, cudaMemcpyDeviceToDevice, s));
    } else {
        const int grid = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)ctx->sm_count * 8, (n0 + 255) / 256));
        k_tag_symbols<<<grid, 256, 0, s>>>(d_bytes, has_mask ? d_mask : nullptr, buf[0], n0);
        launches += 1;
    }
    if (cap_elems > n0) B2_CUDA(cudaMemsetAsync(buf[0] + n0, 0, (cap_elems - n0) * 4, s));
    // The destination buffer starts zeroed, as a fresh WebGPU buffer does; in literal mode its
    // untouched tail is observable.
    B2_CUDA(cudaMemsetAsync(buf[1], 0, cap_elems * 4, s));
    B2_CUDA(cudaMemsetAsync(table, 0, sizeof(PairSlot) << table_log2, s));
    // The look-back descriptors are tagged with the merge number, which restarts here.
    B2_CUDA(cudaMemsetAsync(d_desc, 0, sizeof(unsigned long long) * ((n0 + MC_TILE - 1) / MC_TILE + 1), s));
    if (dq.counts) B2_CUDA(cudaMemsetAsync(dq.counts, 0, (size_t)dq.segments * 8, s));
    std::memset(h_state, 0, sizeof(DevState));
    if (peer) {
        B2_CUDA(cudaMemsetAsync(px.owned, 0, sizeof(PairSlot) << px.owned_log2, s));
        h_state->xseq = xseq_next;
        h_state->owned = px.owned;
        h_state->owned_log2 = px.owned_log2;
        h_state->dlist = px.dlist;
    }
    h_state->n[0] = (uint32_t)n0;
    h_state->next_id = opts.first_token_id;
    h_state->table_log2 = table_log2;
    h_state->literal = (opts.compat_mode == B200BPE_COMPAT_LITERAL) ? 1u : 0u;
    h_state->world = (uint32_t)ctx->world;
    h_state->incremental = incremental ? 1u : 0u;
    h_state->recount = 1u;
    h_state->table = table;
    h_state->lb_max_spins = opts.test_lookback_spins ? opts.test_lookback_spins : LOOKBACK_MAX_SPINS;
    h_state->first_ticket = opts.test_first_tile ? 1u : 0u;
    h_state->scan_from = 0u;            // the first arg-max scans the table
    h_state->presetup_at = 0xFFFFFFFFu;
    h_state->cand_tau = 0xFFFFFFFFu;
    h_state->cand_tau_next = 0xFFFFFFFFu;
    h_state->cand = d_cand;
    B2_CUDA(cudaMemcpyAsync(d_state, h_state, sizeof(DevState), cudaMemcpyHostToDevice, s));
    B2_CUDA(cudaEventRecord(ev_run1, s));
    B2_CUDA(cudaStreamSynchronize(s));
    {
        float ms = 0;
        cudaEventElapsedTime(&ms, ev_run0, ev_run1);
        last_reset_ms = ms;
    }
    merges_done = 0;
    early_stop = false;
    cur_n = n0;
    std::memset(&stats, 0, sizeof(stats));
    return B200BPE_OK;
}

__global__ void k_begin_batch(DevState* st, uint32_t target) {
    st->tail_fix = 0u;  // the batch before this one ended with its own k_literal_tail
    st->fill_hwm = 0u;
    st->merges_target = target;
    st->target_hit = (st->merges_done >= target) ? 1u : 0u;
}
__global__ void k_clear_status(DevState* st, uint32_t table_log2, PairSlot* table, PairSlot* owned, uint32_t owned_log2,
                               uint32_t* dlist) {
    st->status = DS_OK;
    st->want_grow = 0u;
    st->table_log2 = table_log2;
    st->table = table;
    st->owned = owned;
    st->owned_log2 = owned_log2;
    st->dlist = dlist;
    st->owned_inserted = 0u;
    st->dlist_n = 0u;
    st->occupied = 0u;
    st->recount = 1u;  // the table is new and empty
    st->scan_from = 0u;
    st->cand_tau = 0xFFFFFFFFu;
    st->cand_n = 0u;
}

// One merge iteration on the stream.  `timed` brackets each kernel with events.
b200bpe_status Trainer::enqueue_merge(int iter, bool timed) {
    cudaStream_t s = ctx->stream;
    const bool literal = opts.compat_mode == B200BPE_COMPAT_LITERAL;
    auto ev = [&](int k) -> cudaError_t {
        return timed ? cudaEventRecord(kev[(size_t)iter * 8 + k], s) : cudaSuccess;
    };
    B2_CUDA(ev(0));
    k_pair_count<PC_SLOTS, PC_THREADS><<<grid_pc, PC_THREADS, PC_SMEM_BYTES, s>>>(d_state, buf[0], buf[1], ktable(), d_log);
    B2_CUDA(ev(1));
    launches += 3;
    if (peer) {
        // deltas (or, after a full count, everything) to the owners; owners accumulate and pick; full scan only if the list is stale
        k_route<<<grid_rt, PX_THREADS, 0, s>>>(d_state, table, px.pb, px.fill);
        k_accumulate<<<grid_acc, PX_THREADS, 0, s>>>(d_state, px.pb, d_log, 1);
        B2_CUDA(ev(2));
        k_argmax_peer<<<grid_am, AM_THREADS, 0, s>>>(d_state, d_cta_best, px.pb, d_log);
        B2_CUDA(ev(3));
        k_merge_compact<false, true, true><<<grid_mc, MC_THREADS, MC_SMEM_BYTES, s>>>(d_state, buf[0], buf[1], d_desc, table, dq);
        B2_CUDA(ev(5));
        B2_CUDA(ev(4));
        launches += 2;
        B2_CUDA(cudaGetLastError());
        return B200BPE_OK;
    }
    if (ctx->world > 1) {
        b200bpe_status r = xch.enqueue(ctx, d_state, table, table_log2, d_cta_best, d_log, grid_am);
        if (r) return r;
        launches += 6;
        B2_CUDA(ev(2));
    } else {
        B2_CUDA(ev(2));
        k_argmax_setup<<<grid_am, AM_THREADS, 0, s>>>(d_state, ktable(), d_cta_best, d_log, 0, 0u);
    }
    B2_CUDA(ev(3));
    if (incremental) {
        if (literal) k_merge_compact<true, true><<<grid_mc, MC_THREADS, MC_SMEM_BYTES, s>>>(d_state, buf[0], buf[1], d_desc, ktable(), dq);
        else k_merge_compact<false, true><<<grid_mc, MC_THREADS, MC_SMEM_BYTES, s>>>(d_state, buf[0], buf[1], d_desc, ktable(), dq);
        B2_CUDA(ev(5));
    } else if (literal) {
        k_merge_compact<true, false><<<grid_mc, MC_THREADS, MC_SMEM_BYTES, s>>>(d_state, buf[0], buf[1], d_desc, ktable(), dq);
    } else {
        k_merge_compact<false, false><<<grid_mc, MC_THREADS, MC_SMEM_BYTES, s>>>(d_state, buf[0], buf[1], d_desc, ktable(), dq);
    }
    if (!incremental) B2_CUDA(ev(5));
    B2_CUDA(ev(4));
    B2_CUDA(cudaGetLastError());
    return B200BPE_OK;
}

constexpr uint32_t SPARE_ITERS = 4;   // most iterations beyond the batch size that a graph or a timed batch carries

b200bpe_status Trainer::build_graph() {
    if (graph) { cudaGraphExecDestroy(graph); graph = nullptr; }
    cudaStream_t s = ctx->stream;
    cudaGraph_t g = nullptr;
    const uint64_t launches_before = launches;
    B2_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    b200bpe_status r = B200BPE_OK;
    for (uint32_t i = 0; i < opts.batch_merges + spare_iters() && r == B200BPE_OK; i++) r = enqueue_merge((int)i, false);
    cudaError_t e = cudaStreamEndCapture(s, &g);
    graph_kernels = (uint32_t)(launches - launches_before);   // kernels per graph launch
    launches = launches_before;                                // capturing launched nothing
    if (r != B200BPE_OK) { if (g) cudaGraphDestroy(g); return r; }
    B2_CUDA(e);
    e = cudaGraphInstantiate(&graph, g, 0);
    cudaGraphDestroy(g);
    B2_CUDA(e);
    graph_iters = opts.batch_merges;
    return B200BPE_OK;
}

b200bpe_status Trainer::grow_table() {
    if (table_log2 >= MAX_TABLE_LOG2) return B200BPE_ERR_TABLE_FULL;
    cudaStream_t s = ctx->stream;
    B2_CUDA(cudaStreamSynchronize(s));
    B2_CUDA(cudaFree(table));
    table = nullptr;
    table_log2++;
    B2_CUDA(cudaMalloc(&table, sizeof(PairSlot) << table_log2));
    B2_CUDA(cudaMemsetAsync(table, 0, sizeof(PairSlot) << table_log2, s));
    grid_am = std::max(1, std::min(ctx->sm_count * 4, (int)((1u << table_log2) / (AM_THREADS * 4))));
    if (peer) {
        // the inboxes are sized from the table: new buffers, mapped again by every rank (all ranks grow together)
        px.release();
        b200bpe_status r = px.init(ctx, table_log2);
        if (r) return r;
        if (!px.ok) { set_last_error("peer buffers could not be mapped again after the table grew"); return B200BPE_ERR_CUDA; }
    } else if (ctx->world > 1) {
        b200bpe_status r = xch.resize(ctx, table_log2, opts.exchange_cap);
        if (r) return r;
    }
    k_clear_status<<<1, 1, 0, s>>>(d_state, table_log2, table, px.owned, px.owned_log2, px.dlist);
    launches += 1;
    if (graph && ctx->world > 1) { cudaGraphExecDestroy(graph); graph = nullptr; }
    return B200BPE_OK;
}

b200bpe_status Trainer::run(uint32_t max_merges, uint32_t* merges_out, uint32_t* counts_out, uint32_t* n_out,
                            uint32_t* early_out, b200bpe_progress_cb cb, void* user) {
    B2_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t s = ctx->stream;
    const bool timed = (opts.flags & B200BPE_FLAG_TIME_KERNELS) != 0;
    const bool use_graph = !timed && !(opts.flags & B200BPE_FLAG_NO_GRAPH);
    uint32_t remaining = merges_goal - merges_done;
    if (max_merges && max_merges < remaining) remaining = max_merges;
    const uint32_t start_done = merges_done;
    if (timed && kev.empty()) {
        kev.resize((size_t)(opts.batch_merges + SPARE_ITERS) * 8);
        for (auto& e : kev) B2_CUDA(cudaEventCreate(&e));
    }
    auto t0 = std::chrono::steady_clock::now();
    B2_CUDA(cudaEventRecord(ev_run0, s));
    int grow_retries = 0, idle_batches = 0;
    uint32_t full_scans_seen = 0;
    {
        B2_CUDA(cudaMemcpyAsync(h_state, d_state, sizeof(DevState), cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaStreamSynchronize(s));
        full_scans_seen = h_state->full_scans;
    }
    bool table_replaced = false;
    // A batch ends at an absolute merge index (progress is reported there, as the reference does
    // every 128 merges); an arg-max that finds its candidate list stale uses up an iteration without
    // a merge, so the graph holds a few spare iterations and a batch that still falls short is continued.
    uint32_t batch_target = merges_done;
    while (remaining > 0 && !early_stop) {
        if (merges_done >= batch_target) batch_target = merges_done + std::min(opts.batch_merges, remaining);
        const uint32_t before = merges_done;
        const uint32_t batch = batch_target - before;
        k_begin_batch<<<1, 1, 0, s>>>(d_state, batch_target);
        launches += 1;
        if (use_graph) {
            if (!graph) { b200bpe_status r = build_graph(); if (r) return r; }
            B2_CUDA(cudaGraphLaunch(graph, s));
            launches += graph_kernels;
        } else {
            for (uint32_t i = 0; i < batch + spare_iters(); i++) { b200bpe_status r = enqueue_merge((int)i, timed); if (r) return r; }
        }
        // literal mode, incremental table: inside a batch the next merge's count kernel finishes the
        // table update of a merge; the batch's last merge gets it here
        if (incremental && opts.compat_mode == B200BPE_COMPAT_LITERAL) {
            k_literal_tail<<<std::max(1, ctx->sm_count), 256, 0, s>>>(d_state, buf[0], buf[1], ktable());
            launches += 1;
        }
        // Sharded: a status that the batch's last merge kernel raised on one rank (table full, a wait
        // that ran out) reaches every rank before the host looks at it, so that all ranks grow, resize
        // or give up together.
        if (peer) {
            k_batch_sync<<<1, 32, 0, s>>>(d_state, px.pb);
            launches += 1;
        } else if (ctx->world > 1) {
            b200bpe_status r = xch.enqueue_status_sync(ctx, d_state);
            if (r) return r;
            launches += 2;
        }
        // One read-back per batch: the control block and this batch's slice of the merge log
        // (trainer.js:248-267 reads the same two things).
        B2_CUDA(cudaMemcpyAsync(h_state, d_state, sizeof(DevState), cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaMemcpyAsync(h_log + (size_t)before * 4, d_log + (size_t)before * 4, (size_t)batch * 16,
                                cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaStreamSynchronize(s));
        if (peer) xseq_next = h_state->xseq;
        const uint32_t done_now = h_state->merges_done;
        const uint32_t got = done_now - before;
        if (timed) {
            uint64_t nk = cur_n;
            for (uint32_t i = 0; i < batch + spare_iters(); i++) {   // (an iteration without a merge shifts the attribution of the ones after it: statistics only)
                float ms = 0;
                const size_t b = (size_t)i * 8;
                const bool merged = i < got;
                // In incremental mode the count kernel only works when a rebuild is due: at the very
                // first merge, after a merge of two equal symbols, and after the table was replaced.
                bool counted = true;
                if (incremental) {
                    const uint32_t g = before + i;
                    counted = (g == 0) || (i == 0 && table_replaced) ||
                              (g > 0 && i <= got && h_log[(size_t)(g - 1) * 4] == h_log[(size_t)(g - 1) * 4 + 1]);
                }
                cudaEventElapsedTime(&ms, kev[b + 0], kev[b + 1]);
                if (counted) { stats.pair_count_ms += ms; stats.pair_count_launches++; stats.pair_count_bytes += 4ull * nk; }
                else { stats.pair_count_skipped_ms += ms; stats.pair_count_skipped_launches++; }
                cudaEventElapsedTime(&ms, kev[b + 1], kev[b + 2]); stats.exchange_ms += ms;
                cudaEventElapsedTime(&ms, kev[b + 2], kev[b + 3]); stats.argmax_ms += ms;
                cudaEventElapsedTime(&ms, kev[b + 3], kev[b + 5]); stats.merge_compact_ms += ms;
                cudaEventElapsedTime(&ms, kev[b + 5], kev[b + 4]); stats.table_update_ms += ms;
                stats.argmax_launches++; stats.merge_compact_launches++;
                if (ctx->world > 1) stats.exchange_launches++;
                if (!incremental) stats.argmax_bytes += 24ull << table_log2;  // read 16 B per slot, clear the 8 B key
                if (merged) {
                    const uint64_t nn = (ctx->world > 1) ? nk : nk - h_log[(size_t)(before + i) * 4 + 3];
                    stats.merge_compact_bytes += 4ull * nk + 4ull * nn;
                    nk = nn;
                }
            }
        }
        for (uint32_t i = 0; i < got; i++) {
            const uint32_t* l = h_log + (size_t)(before + i) * 4;
            const size_t o = (size_t)(before + i - start_done);
            if (merges_out) { merges_out[o * 3 + 0] = l[0]; merges_out[o * 3 + 1] = l[1]; merges_out[o * 3 + 2] = l[2]; }
            if (counts_out) counts_out[o] = l[3];
        }
        if (got == 0 && !h_state->early_stop && h_state->status == DS_OK && !h_state->want_grow) {
            // a batch of one or two iterations can be used up by an arg-max that only found its
            // candidate list stale (the merge then follows in the next iteration)
            if (!(h_state->iter_no >= h_state->scan_from && ++idle_batches <= 4)) {
                set_last_error("a batch made no progress");
                return B200BPE_ERR_INTERNAL;
            }
        } else {
            idle_batches = 0;
        }
        if (timed && incremental) {
            // only the full scans of the table count as arg-max bytes; the other launches read a short candidate list
            stats.argmax_bytes += (16ull << table_log2) * (uint64_t)(h_state->full_scans - full_scans_seen);
        }
        full_scans_seen = h_state->full_scans;
        merges_done = done_now;
        remaining -= got;
        cur_n = h_state->n[h_state->epoch & 1];
        early_stop = h_state->early_stop != 0;
        table_replaced = false;
        if (peer && h_state->status == DS_BUCKET_FULL) h_state->status = DS_TABLE_FULL;   // an inbox too small for the table's pairs: grow both
        if (ctx->world > 1 && !peer && (h_state->status == DS_BUCKET_FULL || h_state->status == DS_OK)) {
            // sharded runs: resize the exchange buckets to the traffic seen (same decision on every rank)
            const bool over = h_state->status == DS_BUCKET_FULL;
            if (over && xch.cap >= xch.cap_alloc) { h_state->status = DS_TABLE_FULL; }
            else if (xch.adapt(over, h_state->fill_hwm) || over) {
                if (graph) { cudaGraphExecDestroy(graph); graph = nullptr; }
                if (over) {
                    // some pairs never reached their owners: count again, from an empty local table
                    B2_CUDA(cudaMemsetAsync(table, 0, sizeof(PairSlot) << table_log2, s));
                    k_clear_status<<<1, 1, 0, s>>>(d_state, table_log2, table, nullptr, 0u, nullptr);
                    h_state->status = DS_OK;
                }
            }
        }
        if (h_state->status == DS_TABLE_FULL || h_state->want_grow) {
            const bool was_full = h_state->status == DS_TABLE_FULL;
            b200bpe_status r = grow_table();
            table_replaced = true;
            if (r) return r;
            if (was_full && ++grow_retries > 16) return B200BPE_ERR_TABLE_FULL;
        } else if (h_state->status == DS_LOOKBACK_TIMEOUT) {
            return B200BPE_ERR_LOOKBACK_TIMEOUT;
        } else if (h_state->status != DS_OK) {
            return B200BPE_ERR_INTERNAL;
        }
        if (cb && (merges_done >= batch_target || early_stop || remaining == 0)) {
            b200bpe_progress p{};
            p.merge_index = merges_done;
            p.total_merges = merges_goal;
            if (got) {
                const uint32_t* l = h_log + (size_t)(merges_done - 1) * 4;
                p.last_a = l[0]; p.last_b = l[1]; p.last_new_id = l[2]; p.last_count = l[3];
            }
            p.symbol_count = cur_n;
            const double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            p.merges_per_second = el > 0 ? (merges_done - start_done) / el : 0.0;
            cb(&p, user);
        }
    }
    B2_CUDA(cudaEventRecord(ev_run1, s));
    B2_CUDA(cudaEventSynchronize(ev_run1));
    float ms = 0;
    cudaEventElapsedTime(&ms, ev_run0, ev_run1);
    last_run_ms = ms;
    if (n_out) *n_out = merges_done - start_done;
    if (early_out) *early_out = early_stop ? 1u : 0u;
    return B200BPE_OK;
}

static b200bpe_status check_opts(const Ctx* ctx, const b200bpe_train_opts* in, b200bpe_train_opts* o) {
    std::memset(o, 0, sizeof(*o));
    if (in) {
        if (in->struct_size != sizeof(b200bpe_train_opts)) return B200BPE_ERR_BAD_ARG;
        *o = *in;
    }
    if (o->target_vocab_size == 0) o->target_vocab_size = 4096;
    if (o->first_token_id == 0) o->first_token_id = 256;
    if (o->batch_merges == 0) o->batch_merges = 128;
    if (o->batch_merges > 4096) return B200BPE_ERR_BAD_ARG;
    if (o->compat_mode > B200BPE_COMPAT_FIXED) return B200BPE_ERR_BAD_ARG;
    if (o->target_vocab_size < o->first_token_id) return B200BPE_ERR_BAD_ARG;
    if (ctx->world > 1 && o->compat_mode != B200BPE_COMPAT_FIXED) return B200BPE_ERR_BAD_ARG;
    if (o->table_log2 && (o->table_log2 < 4 || o->table_log2 > MAX_TABLE_LOG2)) return B200BPE_ERR_BAD_ARG;
    return B200BPE_OK;
}

static b200bpe_status make_trainer(b200bpe_ctx* c, const uint8_t* bytes, const uint8_t* mask, const uint32_t* symbols,
                                   uint64_t n, bool device_inputs, const b200bpe_train_opts* opts, Trainer** out) {
    if (!c || !out) return B200BPE_ERR_BAD_ARG;
    // A shard of a sharded job may be empty (then without any buffer); a single-GPU corpus may not (trainer.js:161-163).
    if (n == 0 && c->c.world == 1) return (!bytes && !symbols) ? B200BPE_ERR_BAD_ARG : B200BPE_ERR_EMPTY_CORPUS;
    if (n != 0 && !bytes && !symbols) return B200BPE_ERR_BAD_ARG;
    // per-GPU symbol indices are 32-bit, and the merge kernel adds up to two tiles to an index before it tests it
    if (n >= 0xFFFFFFF0ull - 2ull * MC_TILE) return B200BPE_ERR_BAD_ARG;
    B2_CUDA(cudaSetDevice(c->c.device));
    Trainer* t = new Trainer();
    t->ctx = &c->c;
    t->n0 = n;
    b200bpe_status r = check_opts(&c->c, opts, &t->opts);
    if (r) { delete t; return r; }
    t->merges_goal = t->opts.target_vocab_size - t->opts.first_token_id;
    t->incremental = !(t->opts.flags & B200BPE_FLAG_FULL_RECOUNT);
    auto fail = [&](b200bpe_status st) { delete t; return st; };
    cudaStream_t s = c->c.stream;
    const size_t nb = std::max<uint64_t>(n, 1);
    if (symbols) {
        if (cudaMalloc(&t->d_sym_init, nb * 4) != cudaSuccess) return fail(B200BPE_ERR_OOM);
        if (n && cudaMemcpyAsync(t->d_sym_init, symbols, n * 4, device_inputs ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, s) != cudaSuccess)
            return fail(B200BPE_ERR_CUDA);
    } else if (device_inputs) {
        t->own_inputs = false;
        t->d_bytes = const_cast<uint8_t*>(bytes);
        t->d_mask = const_cast<uint8_t*>(mask);
        t->has_mask = mask != nullptr;
    } else {
        if (cudaMalloc(&t->d_bytes, nb) != cudaSuccess) return fail(B200BPE_ERR_OOM);
        if (n && cudaMemcpyAsync(t->d_bytes, bytes, n, cudaMemcpyHostToDevice, s) != cudaSuccess) return fail(B200BPE_ERR_CUDA);
        if (mask) {
            if (cudaMalloc(&t->d_mask, nb) != cudaSuccess) return fail(B200BPE_ERR_OOM);
            if (n && cudaMemcpyAsync(t->d_mask, mask, n, cudaMemcpyHostToDevice, s) != cudaSuccess) return fail(B200BPE_ERR_CUDA);
            t->has_mask = true;
        }
    }
    r = t->alloc_common();
    if (r) return fail(r);
    r = t->init_state();
    if (r) return fail(r);
    *out = t;
    return B200BPE_OK;
}

}  // namespace b200bpe

struct b200bpe_trainer { b200bpe::Trainer* t; };

using namespace b200bpe;

static b200bpe_status wrap(Trainer* t, b200bpe_trainer** out) {
    *out = new b200bpe_trainer{t};
    return B200BPE_OK;
}

extern "C" {

b200bpe_status b200bpe_trainer_create(b200bpe_ctx* c, const uint8_t* bytes, const uint8_t* word_starts, uint64_t n,
                                      const b200bpe_train_opts* opts, b200bpe_trainer** out) {
    Trainer* t = nullptr;
    b200bpe_status r = make_trainer(c, bytes, word_starts, nullptr, n, false, opts, &t);
    return r ? r : wrap(t, out);
}

b200bpe_status b200bpe_trainer_create_device(b200bpe_ctx* c, const uint8_t* d_bytes, const uint8_t* d_word_starts,
                                             uint64_t n, const b200bpe_train_opts* opts, b200bpe_trainer** out) {
    Trainer* t = nullptr;
    b200bpe_status r = make_trainer(c, d_bytes, d_word_starts, nullptr, n, true, opts, &t);
    return r ? r : wrap(t, out);
}

b200bpe_status b200bpe_trainer_create_from_symbols(b200bpe_ctx* c, const uint32_t* symbols, uint64_t n,
                                                   const b200bpe_train_opts* opts, b200bpe_trainer** out) {
    Trainer* t = nullptr;
    b200bpe_status r = make_trainer(c, nullptr, nullptr, symbols, n, false, opts, &t);
    return r ? r : wrap(t, out);
}

b200bpe_status b200bpe_trainer_run(b200bpe_trainer* h, uint32_t max_merges, uint32_t* merges_out, uint32_t* counts_out,
                                   uint32_t* n_merges_out, uint32_t* early_stop_out, b200bpe_progress_cb cb, void* user) {
    if (!h) return B200BPE_ERR_BAD_ARG;
    return h->t->run(max_merges, merges_out, counts_out, n_merges_out, early_stop_out, cb, user);
}

b200bpe_status b200bpe_trainer_reset(b200bpe_trainer* h) {
    if (!h) return B200BPE_ERR_BAD_ARG;
    B2_CUDA(cudaSetDevice(h->t->ctx->device));
    return h->t->init_state();
}

b200bpe_status b200bpe_trainer_symbols(b200bpe_trainer* h, uint32_t* out, uint64_t cap, uint64_t* n_out) {
    if (!h || !n_out) return B200BPE_ERR_BAD_ARG;
    Trainer* t = h->t;
    B2_CUDA(cudaSetDevice(t->ctx->device));
    B2_CUDA(cudaMemcpyAsync(t->h_state, t->d_state, sizeof(DevState), cudaMemcpyDeviceToHost, t->ctx->stream));
    B2_CUDA(cudaStreamSynchronize(t->ctx->stream));
    const uint32_t e = t->h_state->epoch;
    const uint64_t n = t->h_state->n[e & 1];
    *n_out = n;
    if (!out) return B200BPE_OK;
    if (cap < n) return B200BPE_ERR_CAPACITY;
    B2_CUDA(cudaMemcpy(out, t->buf[e & 1], n * 4, cudaMemcpyDeviceToHost));
    return B200BPE_OK;
}

b200bpe_status b200bpe_trainer_pair_counts(b200bpe_trainer* h, uint64_t* keys_out, uint32_t* counts_out, uint64_t cap,
                                           uint64_t* n_distinct_out) {
    if (!h || !n_distinct_out) return B200BPE_ERR_BAD_ARG;
    Trainer* t = h->t;
    B2_CUDA(cudaSetDevice(t->ctx->device));
    cudaStream_t s = t->ctx->stream;
    B2_CUDA(cudaMemcpyAsync(t->h_state, t->d_state, sizeof(DevState), cudaMemcpyDeviceToHost, s));
    B2_CUDA(cudaStreamSynchronize(s));
    // An incrementally maintained table that is up to date is read out as it stands; otherwise
    // the pairs are counted now and the table is left empty (with the rebuild still pending).
    const bool as_is = t->incremental && t->h_state->recount == 0u;
    for (int attempt = 0; attempt < 12; attempt++) {
        k_begin_batch<<<1, 1, 0, s>>>(t->d_state, 0xFFFFFFFFu);
        if (!as_is)
            k_pair_count<PC_SLOTS, PC_THREADS><<<t->grid_pc, PC_THREADS, PC_SMEM_BYTES, s>>>(
                t->d_state, t->buf[0], t->buf[1], t->table, t->d_log);
        PairSlot* tab = t->table;
        uint32_t tl2 = t->table_log2;
        if (t->peer) {
            // The owned table holds the global counts of this rank's pairs, short of what still sits in
            // the ranks' local tables: the deltas of the last merge, or (a rebuild pending) the fresh full
            // counts.  One exchange round without a pick brings it up to date (collective: every rank calls).
            k_route<<<t->grid_rt, PX_THREADS, 0, s>>>(t->d_state, t->table, t->px.pb, t->px.fill);
            k_accumulate<<<t->grid_acc, PX_THREADS, 0, s>>>(t->d_state, t->px.pb, t->d_log, 0);
            k_batch_sync<<<1, 32, 0, s>>>(t->d_state, t->px.pb);
            tab = t->px.owned;
            tl2 = t->px.owned_log2;
        } else if (t->ctx->world > 1) {
            b200bpe_status r = t->xch.enqueue_counts_only(t->ctx, t->d_state, t->table, t->table_log2);
            if (r) return r;
            tab = t->xch.owned;
            tl2 = t->xch.owned_log2;
        }
        unsigned long long* dk = nullptr;
        uint32_t *dc = nullptr, *dn = nullptr;
        const uint32_t dcap = (uint32_t)std::min<uint64_t>(cap, 1ull << tl2);
        B2_CUDA(cudaMalloc(&dk, std::max<size_t>(8, (size_t)dcap * 8)));
        B2_CUDA(cudaMalloc(&dc, std::max<size_t>(4, (size_t)dcap * 4)));
        B2_CUDA(cudaMalloc(&dn, 4));
        B2_CUDA(cudaMemsetAsync(dn, 0, 4, s));
        // A table of owned pairs is always left empty (the next merge sums into it again).  A local table
        // that is up to date stays; one that was only counted for this call is emptied, because the
        // rebuild that is still pending starts from an empty table.
        const bool owned_table = tab != t->table;
        const bool clear = t->peer ? !as_is : (owned_table || !as_is);
        k_dump_table<<<t->ctx->sm_count * 4, 256, 0, s>>>(tab, 1u << tl2, dk, dc, dcap, dn, clear ? 1 : 0);
        if (owned_table && !as_is && !t->peer) B2_CUDA(cudaMemsetAsync(t->table, 0, sizeof(PairSlot) << t->table_log2, s));
        uint32_t nd = 0;
        B2_CUDA(cudaMemcpyAsync(&nd, dn, 4, cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaMemcpyAsync(t->h_state, t->d_state, sizeof(DevState), cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaStreamSynchronize(s));
        if (t->h_state->status == DS_BUCKET_FULL) {
            // No all-reduce on this path, so the ranks cannot agree on a larger bucket here: give up.
            cudaFree(dk); cudaFree(dc); cudaFree(dn);
            // the rebuild that k_clear_status asks for starts from an empty local table
            B2_CUDA(cudaMemsetAsync(t->table, 0, sizeof(PairSlot) << t->table_log2, s));
            k_clear_status<<<1, 1, 0, s>>>(t->d_state, t->table_log2, t->table, t->px.owned, t->px.owned_log2, t->px.dlist);
            return B200BPE_ERR_CAPACITY;
        }
        if (t->peer) t->xseq_next = t->h_state->xseq;
        const bool full = t->h_state->status == DS_TABLE_FULL;
        if (!full) {
            const uint32_t m = std::min(nd, dcap);
            if (keys_out) B2_CUDA(cudaMemcpy(keys_out, dk, (size_t)m * 8, cudaMemcpyDeviceToHost));
            if (counts_out) B2_CUDA(cudaMemcpy(counts_out, dc, (size_t)m * 4, cudaMemcpyDeviceToHost));
        }
        cudaFree(dk); cudaFree(dc); cudaFree(dn);
        if (t->peer && !as_is)   // the owned table was emptied by the dump: its insert count starts over, the rebuild stays pending
            k_clear_status<<<1, 1, 0, s>>>(t->d_state, t->table_log2, t->table, t->px.owned, t->px.owned_log2, t->px.dlist);
        if (!full) {
            *n_distinct_out = nd;
            return nd > cap ? B200BPE_ERR_CAPACITY : B200BPE_OK;
        }
        // Sharded: growing is a collective step (buffers are mapped between ranks, bucket sizes must
        // agree), and this call has no way to make every rank take it: report the full table instead.
        if (t->ctx->world > 1) return B200BPE_ERR_TABLE_FULL;
        b200bpe_status r = t->grow_table();
        if (r) return r;
    }
    return B200BPE_ERR_TABLE_FULL;
}

b200bpe_status b200bpe_trainer_kernel_stats(b200bpe_trainer* h, b200bpe_kernel_stats* out) {
    if (!h || !out) return B200BPE_ERR_BAD_ARG;
    *out = h->t->stats;
    return B200BPE_OK;
}

b200bpe_status b200bpe_trainer_launches(b200bpe_trainer* h, uint64_t* n) {
    if (!h || !n) return B200BPE_ERR_BAD_ARG;
    *n = h->t->launches;
    return B200BPE_OK;
}

b200bpe_status b200bpe_trainer_exchange_kind(b200bpe_trainer* h, uint32_t* kind) {
    if (!h || !kind) return B200BPE_ERR_BAD_ARG;
    *kind = h->t->ctx->world == 1 ? 0u : (h->t->peer ? 1u : 2u);
    return B200BPE_OK;
}

b200bpe_status b200bpe_trainer_last_run_ms(b200bpe_trainer* h, double* ms) {
    if (!h || !ms) return B200BPE_ERR_BAD_ARG;
    *ms = h->t->last_run_ms;
    return B200BPE_OK;
}

b200bpe_status b200bpe_trainer_last_reset_ms(b200bpe_trainer* h, double* ms) {
    if (!h || !ms) return B200BPE_ERR_BAD_ARG;
    *ms = h->t->last_reset_ms;
    return B200BPE_OK;
}

void b200bpe_trainer_destroy(b200bpe_trainer* h) {
    if (!h) return;
    delete h->t;
    delete h;
}

b200bpe_status b200bpe_train(b200bpe_ctx* c, const uint8_t* bytes, const uint8_t* word_starts, uint64_t n,
                             const b200bpe_train_opts* opts, uint32_t* merges_out, uint32_t* counts_out,
                             uint32_t* n_merges_out, uint32_t* early_stop_out, b200bpe_progress_cb cb, void* user) {
    if (!merges_out || !n_merges_out) return B200BPE_ERR_BAD_ARG;
    b200bpe_trainer* h = nullptr;
    b200bpe_status r = b200bpe_trainer_create(c, bytes, word_starts, n, opts, &h);
    if (r) return r;
    r = b200bpe_trainer_run(h, 0, merges_out, counts_out, n_merges_out, early_stop_out, cb, user);
    b200bpe_trainer_destroy(h);
    return r;
}

}  // extern "C"


