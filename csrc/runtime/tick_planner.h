// Continuous-batching tick planner.
//
// One tick = plan() (pure bookkeeping) -> the execution backend replays the plan ->
// ingest_prefill()/ingest_decode() feed the results back.  Policy: decode first, prefill
// piggy-backs under a token budget; admission is FIFO and pays KV pages for the suffix that
// the radix prefix cache does not cover; decode rows are physical (row r = state slot r =
// graph row r) and stay a dense prefix, so a retirement moves the highest live row into the
// hole; the decode batch is padded to a bucket of a fixed ladder so that one CUDA graph per
// bucket suffices.  Same contract as the reference's planner
// (crates/ferrite-dispatch/src/batch.rs:109-836, bucket.rs:38-108, exec.rs:57-177) and its
// older Waiting->Prefill->Decode->Finished scheduler (crates/ferrite-batch/src/lib.rs:73-254).
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "pools.h"
#include "radix.h"
#include "state_store.h"

namespace fbrt {

struct SchedConfig {
    int max_rows = 32;
    int prefill_budget = 512;
    int page_size = 16;
    int num_pages = 122880;
    int device_slots = 512, host_slots = 4096, disk_slots = 65536;
    std::vector<int> buckets = {1, 2, 4, 8, 16, 32};
    int max_ctx = 1 << 20;
    int spec_rows = 1;   // rows one decode step may append to a sequence (speculative verify width)
    // A sequence must stop while a whole step (spec_rows rows, plus the two positions the MTP cache runs
    // ahead) still fits below max_ctx: page tables and caches are sized for max_ctx positions.
    int ctx_headroom() const { return spec_rows + 2; }
};

inline int bucket_for(const std::vector<int>& ladder, int n) {
    for (int b : ladder) if (b >= n) return b;
    return ladder.empty() ? n : ladder.back();
}

enum ReqState : int { RS_QUEUED = 0, RS_PREFILL = 1, RS_DECODE = 2, RS_FINISHED = 3 };
enum EventKind : int { EV_ADMITTED = 0, EV_TOKENS = 1, EV_FINISHED = 2 };

struct Request {
    int64_t id = 0;
    std::vector<int32_t> prompt;
    int max_new = 256;
    std::set<int32_t> stop_ids;
    int state = RS_QUEUED;
    int row = -1;
    int prefilled = 0;        // prompt tokens whose KV/state exist (cached prefix included)
    int cached_tokens = 0;    // prefix served from the radix cache
    int radix_node = 0;
    int boundary_snapshot = -1;  // snapshot captured at the last block boundary of the prompt
    std::vector<int32_t> generated;
    std::vector<int> pages;   // logical page i of the sequence -> physical page
    int shared_pages = 0;     // leading pages leased from the radix cache
    std::string finish_reason;
};

struct PrefillChunk {
    int64_t req; int row; int start; int len;
    bool last;             // the chunk that ends the prompt (its last row yields the first token)
    bool snapshot_after;   // capture the recurrent state after this chunk (block boundary)
};
struct RowRestore { int row; int snapshot; int device_slot; };  // prefix hit: state <- snapshot
struct RowMove { int from_row, to_row; int64_t req; };
struct DecodeWork { std::vector<int64_t> rows; int n_live = 0; int bucket = 0; };

struct TickPlan {
    std::vector<int64_t> admitted;
    std::vector<RowMove> row_moves;
    std::vector<RowRestore> restores;
    std::vector<StateMove> state_moves;
    std::vector<PrefillChunk> prefill;
    DecodeWork decode;
    bool empty() const { return prefill.empty() && decode.n_live == 0 && row_moves.empty() && restores.empty(); }
};

struct Event {
    int64_t req; int kind;
    std::vector<int32_t> tokens;
    std::string reason;
    int prompt_tokens = 0, completion_tokens = 0, cached_tokens = 0;
    bool prefix_hit = false;
};

struct SchedStats {
    int64_t ticks = 0, tokens_committed = 0;
    int live_rows = 0, queued = 0, pages_in_use = 0, pages_free = 0;
    std::vector<int> tiers;
    RadixStats radix;
};

}  // namespace fbrt

#include "tick_planner_impl.h"
