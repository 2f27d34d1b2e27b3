// Continuous-batching planner for engines whose sequence state lives in fixed slots (no pages, no prefix tree):
// the DSV41 batched engine.  FIFO admission into free slots, chunked prefill within a per-tick token budget
// (oldest admitted first), one decode row per sequence whose prompt is in the caches, finish rules (stop id,
// output budget, context limit, cancellation).  The engine executes the plan: it runs the decode bucket and the
// prefill chunks on the device and feeds the sampled tokens back.
//
// One tick:   begin_tick()                       cancellations -> finished events, released slots
//             plan_decode()                      slots of the decoding sequences + the padded bucket
//             ingest_decode(tokens)              one token per decode row -> events
//             plan_prefill()                     admissions (slot resets) + the tick's prefill chunks
//             ingest_first(rid, token)           first token of a sequence whose last chunk just ran -> events
//
// Counterpart of the reference's batched DSV41 serving loop (crates/ferrite-dsv41/src/serve.rs) with the planning
// rules of its continuous-batching scheduler (crates/ferrite-batch/src/lib.rs: waiting -> prefill -> decode ->
// finished, chunked-prefill budget, stop / length finish).
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <map>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

namespace fbrt {

struct SlotSchedConfig {
    int max_seqs = 8;
    int prefill_rows = 64;
    int prefill_budget = 256;
    int max_ctx = 1024;
    std::vector<int> buckets;   // ascending; the last one is max_seqs
};

struct SlotEvent {
    enum Kind { ADMITTED = 0, TOKEN = 1, FINISHED = 2 };
    int64_t req = 0;
    int kind = 0;
    int32_t token = 0;
    std::string reason;
    int prompt_tokens = 0, completion_tokens = 0;
};

struct SlotChunk {
    int64_t req = 0;
    int slot = 0, start = 0, len = 0;
    bool last = false;
};

struct SlotDecodePlan {
    std::vector<int> slots;      // live decode rows, admission order
    std::vector<int64_t> reqs;   // the request of every row
    int bucket = 0;              // padded row count (0: nothing decodes this tick)
};

struct SlotPrefillPlan {
    std::vector<SlotEvent> events;   // admissions
    std::vector<int> reset_slots;    // slots handed to a new sequence: the engine clears their lengths
    std::vector<SlotChunk> chunks;   // in execution order
};

struct SlotStats {
    int64_t ticks = 0, tokens_committed = 0;
    int live = 0, queued = 0, free_slots = 0;
};

class SlotScheduler {
  public:
    explicit SlotScheduler(const SlotSchedConfig& c) : cfg_(c) {
        if (cfg_.max_seqs < 1 || cfg_.prefill_rows < 1) throw std::invalid_argument("max_seqs and prefill_rows must be positive");
        cfg_.prefill_budget = std::max(cfg_.prefill_budget, 1);
        std::vector<int> b;
        for (int x : cfg_.buckets)
            if (x >= 1 && x < cfg_.max_seqs) b.push_back(x);
        std::sort(b.begin(), b.end());
        b.erase(std::unique(b.begin(), b.end()), b.end());
        b.push_back(cfg_.max_seqs);
        cfg_.buckets = b;
        for (int s = cfg_.max_seqs - 1; s >= 0; --s) free_.push_back(s);
    }

    const std::vector<int>& buckets() const { return cfg_.buckets; }
    int max_prompt() const { return cfg_.max_ctx - 4; }

    // -1: the prompt is empty or does not fit the context limit
    int64_t submit(const std::vector<int32_t>& prompt, int max_new, const std::vector<int32_t>& stop) {
        if (prompt.empty() || (int)prompt.size() > max_prompt()) return -1;
        Seq s;
        s.rid = next_id_++;
        s.prompt_len = (int)prompt.size();
        s.max_new = std::max(1, max_new);
        s.stop.insert(stop.begin(), stop.end());
        waiting_.push_back(s);
        return s.rid;
    }
    void cancel(int64_t rid) { cancelled_.insert(rid); }
    bool idle() const { return waiting_.empty() && live_.empty(); }
    std::vector<int> free_slots() const { return free_; }

    // Cancellations of this tick; `released` gets the slots whose lengths the engine clears.
    std::vector<SlotEvent> begin_tick(std::vector<int>* released) {
        ++ticks_;
        std::vector<SlotEvent> out;
        if (cancelled_.empty()) return out;
        std::deque<Seq> keep;
        for (auto& s : waiting_)
            if (!cancelled_.count(s.rid)) keep.push_back(s);
        waiting_.swap(keep);
        std::vector<int64_t> hit;
        for (int64_t rid : order_)
            if (cancelled_.count(rid)) hit.push_back(rid);
        for (int64_t rid : hit) finish(rid, "cancelled", &out, released);
        cancelled_.clear();
        return out;
    }

    SlotDecodePlan plan_decode() {
        SlotDecodePlan p;
        for (int64_t rid : order_) {
            const Seq& s = live_.at(rid);
            if (s.filled == s.prompt_len) {
                p.slots.push_back(s.slot);
                p.reqs.push_back(rid);
            }
        }
        if (!p.slots.empty()) {
            for (int b : cfg_.buckets)
                if (b >= (int)p.slots.size()) { p.bucket = b; break; }
        }
        decode_reqs_ = p.reqs;
        return p;
    }

    // tokens[i] belongs to row i of the last plan_decode()
    std::vector<SlotEvent> ingest_decode(const std::vector<int32_t>& tokens, std::vector<int>* released) {
        if (tokens.size() < decode_reqs_.size()) throw std::invalid_argument("one token per decode row is needed");
        std::vector<SlotEvent> out;
        for (size_t i = 0; i < decode_reqs_.size(); ++i) emit(decode_reqs_[i], tokens[i], &out, released);
        decode_reqs_.clear();
        return out;
    }

    SlotPrefillPlan plan_prefill() {
        SlotPrefillPlan p;
        while (!waiting_.empty() && !free_.empty()) {
            Seq s = waiting_.front();
            waiting_.pop_front();
            s.slot = free_.back();
            free_.pop_back();
            p.reset_slots.push_back(s.slot);
            SlotEvent e;
            e.req = s.rid;
            e.kind = SlotEvent::ADMITTED;
            e.prompt_tokens = s.prompt_len;
            p.events.push_back(e);
            order_.push_back(s.rid);
            live_[s.rid] = s;
        }
        int budget = cfg_.prefill_budget;
        for (int64_t rid : order_) {
            Seq& s = live_.at(rid);
            while (budget > 0 && s.filled < s.prompt_len) {
                SlotChunk c;
                c.req = rid;
                c.slot = s.slot;
                c.start = s.filled;
                c.len = std::min({cfg_.prefill_rows, s.prompt_len - s.filled, budget});
                c.last = c.start + c.len == s.prompt_len;
                p.chunks.push_back(c);
                s.filled += c.len;
                budget -= c.len;
            }
            if (budget <= 0) break;
        }
        return p;
    }

    // First token of a sequence whose last prefill chunk ran.
    std::vector<SlotEvent> ingest_first(int64_t rid, int32_t token, std::vector<int>* released) {
        std::vector<SlotEvent> out;
        if (live_.count(rid)) emit(rid, token, &out, released);
        return out;
    }

    SlotStats stats() const {
        SlotStats s;
        s.ticks = ticks_;
        s.tokens_committed = tokens_;
        s.live = (int)live_.size();
        s.queued = (int)waiting_.size();
        s.free_slots = (int)free_.size();
        return s;
    }

  private:
    struct Seq {
        int64_t rid = 0;
        int prompt_len = 0, max_new = 1, slot = -1, filled = 0, n_out = 0;
        std::set<int32_t> stop;
    };

    void finish(int64_t rid, const std::string& reason, std::vector<SlotEvent>* out, std::vector<int>* released) {
        auto it = live_.find(rid);
        if (it == live_.end()) return;
        SlotEvent e;
        e.req = rid;
        e.kind = SlotEvent::FINISHED;
        e.reason = reason;
        e.prompt_tokens = it->second.prompt_len;
        e.completion_tokens = it->second.n_out;
        out->push_back(e);
        if (it->second.slot >= 0) {
            free_.push_back(it->second.slot);
            if (released) released->push_back(it->second.slot);
        }
        live_.erase(it);
        order_.erase(std::remove(order_.begin(), order_.end(), rid), order_.end());
    }

    // Commit one token: a stop id ends the sequence without being emitted; then the output budget, then the context limit.
    void emit(int64_t rid, int32_t tok, std::vector<SlotEvent>* out, std::vector<int>* released) {
        auto it = live_.find(rid);
        if (it == live_.end()) return;
        Seq& s = it->second;
        ++tokens_;
        if (s.stop.count(tok)) {
            finish(rid, "stop", out, released);
            return;
        }
        ++s.n_out;
        SlotEvent e;
        e.req = rid;
        e.kind = SlotEvent::TOKEN;
        e.token = tok;
        out->push_back(e);
        if (s.n_out >= s.max_new) finish(rid, "length", out, released);
        else if (s.prompt_len + s.n_out + 2 >= cfg_.max_ctx) finish(rid, "context", out, released);
    }

    SlotSchedConfig cfg_;
    std::deque<Seq> waiting_;
    std::map<int64_t, Seq> live_;
    std::vector<int64_t> order_;          // live requests in admission order
    std::vector<int> free_;               // free slots; the back is handed out next
    std::set<int64_t> cancelled_;
    std::vector<int64_t> decode_reqs_;
    int64_t next_id_ = 1, ticks_ = 0, tokens_ = 0;
};

}  // namespace fbrt
