// Shared definitions of the B200 BPE library: status helpers, the device control block and
// the layout of the pair table.  Everything here is internal; the public surface is include/b200bpe.h.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/b200bpe.h"

namespace b200bpe {

constexpr uint32_t WORD_START_BIT = 0x10000u;  // reference symbol layout: bit 16 = word start
constexpr uint32_t TOKEN_MASK = 0xFFFFu;       // low 16 bits = token id
constexpr uint32_t INVALID_TOKEN = 0xFFFFFFFFu;

// Device-side status words (DevState::status); mapped to b200bpe_status by the host.
enum DevStatus : uint32_t { DS_OK = 0, DS_TABLE_FULL = 1, DS_LOOKBACK_TIMEOUT = 2, DS_INTERNAL = 3, DS_BUCKET_FULL = 4 };

// One slot of the open-addressing pair table: 64-bit (left << 32 | right) key, 0 = empty
// (the left symbol of a counted pair is never 0), and its count.  16 bytes so that an insert
// touches one 32-byte sector and the arg-max pass reads whole uint4 words.
struct __align__(16) PairSlot {
    unsigned long long key;
    uint32_t count;
    uint32_t pad;
};

// Control block living in device memory; the kernels of a batch read and write it without any
// host round trip.  The fields up to merges_done mirror the reference's IterState.
struct DevState {
    uint32_t n[2];          // live symbol count, indexed by (epoch & 1)
    uint32_t epoch;         // merges applied to the symbol buffers so far (selects ping/pong)
    uint32_t early_stop;    // IterState.early_stop: best count < 2 or ids exhausted
    uint32_t target_hit;    // merges_done reached merges_target
    uint32_t next_id;       // IterState.next_token_id
    uint32_t a, b, new_id;  // winning pair and its new symbol
    uint32_t max_count;     // count of the winning pair
    uint32_t merges_done;   // merges logged since creation/reset
    uint32_t merges_target; // stop once merges_done reaches this
    uint32_t status;        // DevStatus
    uint32_t active;        // 1 while the merge chosen by setup still has to be applied
    uint32_t k3_epoch;      // epoch the merge/compaction kernel works on (written by setup only)
    uint32_t ticket;        // next tile of the merge/compaction kernel
    uint32_t argmax_done;   // CTAs of the arg-max kernel that have finished
    uint32_t occupied;      // non-empty table slots seen by the last arg-max pass
    uint32_t table_log2;    // log2(table capacity)
    uint32_t literal;       // 1 = compaction input bounded by the post-merge count
    uint32_t want_grow;     // arg-max saw the table more than half full
    uint32_t world;         // ranks sharing the job (1 = single GPU)
    unsigned long long best_packed;  // sharded runs: (count << 32) | ~pair32 after the all-reduce
    uint32_t incremental;   // 1 = the table is kept up to date by the merge kernel instead of being rebuilt per merge
    uint32_t recount;       // incremental mode: the next merge must start with a full count into an empty table
    uint32_t v_kept;        // symbols the last merge copied to the destination buffer
    uint32_t tail_fix;      // literal + incremental: the tail fix-up kernel has work for the merge just applied
    uint32_t fill_hwm;      // sharded runs: largest exchange-bucket fill seen on any rank since the batch began
    // Candidate list of the arg-max (incremental table only): the slots whose count was at least
    // cand_tau at the last full scan of the table, plus every slot whose count has crossed cand_tau
    // upwards since.  While the best listed count is >= cand_tau the list holds the global best.
    uint32_t scan_from;     // the arg-max scans the whole table (and rebuilds the list) in every iteration numbered >= this
    uint32_t cand_n;        // entries appended to the list (may exceed its capacity: then it is void)
    uint32_t cand_tau;      // threshold of the list; 0xFFFFFFFF = no list, nothing is appended
    uint32_t cand_tau_next; // threshold the next full scan will use
    uint32_t since_scan;    // merges since the last full scan
    uint32_t full_scans;    // full scans since creation/reset (statistics)
    uint32_t k1_done;       // CTAs of the count kernel that have arrived at its end (the last one picks the next merge)
    PairSlot* table;        // the pair table (kept here so that replacing it does not invalidate a captured graph)
    uint32_t* cand;         // the candidate list: slot indices
    // Iteration number: advanced by the merge kernel (one thread, at its entry), so it is the same for
    // every CTA of the count and arg-max kernels of an iteration whenever they read the block.  Flags
    // that one CTA of those kernels sets for a LATER kernel are stored as iteration numbers, so a CTA
    // that reads the block after that store still takes the same branch as the others.
    uint32_t iter_no;
    uint32_t presetup_at;   // iteration whose merge an earlier kernel of that iteration already chose and set up: its arg-max skips
    // sharded runs with the peer-memory exchange
    uint32_t xseq;          // sequence number of the next exchange round (the same on every rank)
    uint32_t dlist_n;       // slots of the local delta table that hold an entry (appended on first insert)
    uint32_t* dlist;        // their indices
    PairSlot* owned;        // table of the pairs this rank owns, with their global counts
    uint32_t owned_log2;
    uint32_t owned_inserted; // keys inserted into the owned table since it was last emptied
    uint32_t xdone[2];      // CTAs of the route / accumulate kernels that have arrived at their end
    uint32_t lb_max_spins;  // polls after which a look-back of the merge kernel gives up (DS_LOOKBACK_TIMEOUT)
    uint32_t first_ticket;  // first tile number the merge kernel hands out: 0, or 1 in the test of the bounded wait
    uint32_t pad[2];        // the block is copied as 16-byte words
};
constexpr uint32_t CAND_CAP = 1u << 13;      // entries of the candidate list (one CTA scans it)
constexpr uint32_t CAND_MAX_AGE = 512;       // merges after which a full scan is due anyway (refreshes the table's fill)
constexpr uint32_t SCAN_NEVER = 0xFFFFFFFFu; // DevState.scan_from: no full scan due

struct CtaBest {
    unsigned long long key;
    uint32_t count;
    uint32_t pad;
};

void set_last_error(const std::string& s);

#define B2_CUDA(expr)                                                                                   \
    do {                                                                                                \
        cudaError_t _e = (expr);                                                                        \
        if (_e != cudaSuccess) {                                                                        \
            ::b200bpe::set_last_error(std::string(#expr) + ": " + cudaGetErrorString(_e));              \
            return (_e == cudaErrorMemoryAllocation) ? B200BPE_ERR_OOM : B200BPE_ERR_CUDA;              \
        }                                                                                               \
    } while (0)

struct Ctx;  // defined in api.cu

}  // namespace b200bpe
