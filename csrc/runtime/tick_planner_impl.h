// BatchScheduler: implementation of the tick planner declared in tick_planner.h.
#pragma once

namespace fbrt {

class BatchScheduler {
public:
    explicit BatchScheduler(const SchedConfig& c)
        : cfg_(c), pages_(c.num_pages), radix_(c.page_size), store_(c.device_slots, c.host_slots, c.disk_slots),
          rows_(c.max_rows, -1) {}

    // Longest prompt that can still produce a token.
    int max_prompt() const { return cfg_.max_ctx - cfg_.ctx_headroom() - 1; }

    // Returns the request id, or -1 when the prompt is empty or leaves no room below the context limit
    // (the caller answers 400; nothing is queued).
    int64_t submit(const std::vector<int32_t>& prompt, int max_new, const std::vector<int32_t>& stop_ids) {
        if (prompt.empty() || (int)prompt.size() > max_prompt()) return -1;
        Request r;
        r.id = next_id_++;
        r.prompt = prompt;
        r.max_new = std::max(1, max_new);
        r.stop_ids.insert(stop_ids.begin(), stop_ids.end());
        reqs_[r.id] = r;
        queue_.push_back(r.id);
        return r.id;
    }

    bool cancel(int64_t id) {
        auto it = reqs_.find(id);
        if (it == reqs_.end() || it->second.state == RS_FINISHED) return false;
        auto q = std::find(queue_.begin(), queue_.end(), id);
        if (q != queue_.end()) queue_.erase(q);
        finish(it->second, "cancelled", nullptr);
        return true;
    }

    TickPlan plan() {
        TickPlan p;
        ++ticks_;
        compact_rows(&p);
        // admission (FIFO): rows and pages permitting
        while (!queue_.empty()) {
            const int row = first_free_row();
            if (row < 0) break;
            Request& r = reqs_[queue_.front()];
            if (!admit(r, row, &p)) break;
            queue_.pop_front();
            p.admitted.push_back(r.id);
        }
        // decode first: every live decode row, padded to a bucket
        for (int row = 0; row < cfg_.max_rows; ++row) {
            const int64_t id = rows_[row];
            if (id >= 0 && reqs_[id].state == RS_DECODE) { p.decode.rows.push_back(id); ++p.decode.n_live; }
            else if (id >= 0) p.decode.rows.push_back(-1);
            else p.decode.rows.push_back(-1);
        }
        while (!p.decode.rows.empty() && p.decode.rows.back() < 0) p.decode.rows.pop_back();
        p.decode.bucket = p.decode.n_live ? bucket_for(cfg_.buckets, (int)p.decode.rows.size()) : 0;
        // prefill piggy-backs under the token budget, oldest request first
        int budget = cfg_.prefill_budget;
        for (int row = 0; row < cfg_.max_rows && budget > 0; ++row) {
            const int64_t id = rows_[row];
            if (id < 0) continue;
            Request& r = reqs_[id];
            if (r.state != RS_PREFILL) continue;
            const int n = (int)r.prompt.size();
            // last block boundary strictly inside the prompt: a later identical prompt can resume there
            const int boundary = ((n - 1) / cfg_.page_size) * cfg_.page_size;
            int start = r.prefilled;
            while (start < n && budget > 0) {
                int len = std::min(budget, n - start);
                bool snap = false;
                if (start < boundary && start + len >= boundary && boundary > r.cached_tokens) {
                    len = boundary - start;  // end the chunk on the boundary and capture the state there
                    snap = true;
                }
                p.prefill.push_back({id, row, start, len, start + len == n, snap});
                start += len;
                budget -= len;
                if (inflight_prefill_.count(id) == 0) inflight_prefill_[id] = r.prefilled;
            }
        }
        return p;
    }

    // The backend finished a prefill chunk of `len` tokens; `first_token` >= 0 on the last
    // chunk; `snapshot_row_captured`: the chunk asked for a snapshot and the backend took it.
    std::vector<Event> ingest_prefill(int64_t id, int len, int first_token, bool snapshot_captured,
                                      std::vector<StateMove>* moves) {
        std::vector<Event> ev;
        auto it = reqs_.find(id);
        if (it == reqs_.end() || it->second.state != RS_PREFILL) return ev;
        Request& r = it->second;
        r.prefilled += len;
        if (snapshot_captured && r.boundary_snapshot < 0) {
            std::vector<int> dropped;
            r.boundary_snapshot = store_.capture(r.row, moves, &dropped);
            for (int d : dropped) radix_.clear_snapshot(d);
        }
        if (r.prefilled >= (int)r.prompt.size() && first_token >= 0) {
            r.state = RS_DECODE;
            inflight_prefill_.erase(id);
            push_tokens(r, {first_token}, &ev);
        }
        return ev;
    }

    // tokens[i] = tokens emitted this tick by decode row i (1..n with speculative decoding).
    std::vector<Event> ingest_decode(const std::vector<std::vector<int32_t>>& tokens) {
        std::vector<Event> ev;
        for (int row = 0; row < (int)tokens.size() && row < cfg_.max_rows; ++row) {
            const int64_t id = rows_[row];
            if (id < 0 || tokens[row].empty()) continue;
            Request& r = reqs_[id];
            if (r.state != RS_DECODE) continue;
            push_tokens(r, tokens[row], &ev);
        }
        return ev;
    }

    const Request* get(int64_t id) const { auto it = reqs_.find(id); return it == reqs_.end() ? nullptr : &it->second; }
    void forget(int64_t id) { auto it = reqs_.find(id); if (it != reqs_.end() && it->second.state == RS_FINISHED) reqs_.erase(it); }
    bool idle() const {
        if (!queue_.empty()) return false;
        for (int64_t id : rows_) if (id >= 0) return false;
        return true;
    }

    SchedStats stats() const {
        SchedStats s;
        s.ticks = ticks_; s.tokens_committed = committed_; s.queued = (int)queue_.size();
        for (int64_t id : rows_) s.live_rows += id >= 0;
        s.pages_in_use = pages_.pages_in_use(); s.pages_free = pages_.free_pages();
        s.tiers = store_.census(); s.radix = radix_.stats();
        return s;
    }
    RadixCache& radix() { return radix_; }
    PagePool& pages() { return pages_; }
    TieredStore& store() { return store_; }

private:
    int first_free_row() const {
        for (int i = 0; i < cfg_.max_rows; ++i) if (rows_[i] < 0) return i;
        return -1;
    }

    bool admit(Request& r, int row, TickPlan* p) {
        const int ps = cfg_.page_size;
        RadixMatch m = radix_.match(r.prompt);
        // never serve the whole prompt from cache: the last token must run to produce logits
        while (m.tokens >= (int)r.prompt.size() && m.tokens > 0) { m = RadixMatch(); }
        const int total = std::min<int>((int)r.prompt.size() + r.max_new + 8, cfg_.max_ctx);
        const int need_pages = (total + ps - 1) / ps - (int)m.pages.size();
        if (!pages_.can_alloc(need_pages)) {
            Evicted ev = radix_.evict(need_pages - pages_.free_pages());
            for (int pg : ev.pages) pages_.release(pg);
            for (int s : ev.snapshots) store_.release(s);
            if (!pages_.can_alloc(need_pages)) return false;
            m = radix_.match(r.prompt);  // the eviction may have removed part of the match
            if (m.tokens >= (int)r.prompt.size()) m = RadixMatch();
        }
        int dev_slot = -1;
        if (m.tokens > 0) {
            std::vector<int> dropped;
            dev_slot = store_.promote(m.snapshot, &p->state_moves, &dropped);
            for (int d : dropped) radix_.clear_snapshot(d);
            if (dev_slot < 0) m = RadixMatch();
        }
        r.pages = m.pages;
        for (int pg : m.pages) pages_.retain(pg);
        r.shared_pages = (int)m.pages.size();
        std::vector<int> fresh = pages_.alloc((total + ps - 1) / ps - (int)m.pages.size());
        r.pages.insert(r.pages.end(), fresh.begin(), fresh.end());
        r.cached_tokens = m.tokens;
        r.prefilled = m.tokens;
        r.radix_node = m.node;
        if (m.node) radix_.lock(m.node);
        r.row = row;
        r.state = RS_PREFILL;
        rows_[row] = r.id;
        if (m.tokens > 0) p->restores.push_back({row, m.snapshot, dev_slot});
        pending_admit_events_.push_back(r.id);
        return true;
    }

    void push_tokens(Request& r, const std::vector<int32_t>& toks, std::vector<Event>* ev) {
        // admission event first, once
        auto pa = std::find(pending_admit_events_.begin(), pending_admit_events_.end(), r.id);
        if (pa != pending_admit_events_.end()) {
            Event a{r.id, EV_ADMITTED};
            a.prompt_tokens = (int)r.prompt.size(); a.cached_tokens = r.cached_tokens; a.prefix_hit = r.cached_tokens > 0;
            ev->push_back(a);
            pending_admit_events_.erase(pa);
        }
        Event t{r.id, EV_TOKENS};
        std::string reason;
        for (int32_t tok : toks) {
            if (r.stop_ids.count(tok)) { reason = "stop"; break; }
            r.generated.push_back(tok);
            t.tokens.push_back(tok);
            ++committed_;
            if ((int)r.generated.size() >= r.max_new) { reason = "length"; break; }
            // context limit: the next step would write positions >= max_ctx
            if ((int)(r.prompt.size() + r.generated.size()) + cfg_.ctx_headroom() >= cfg_.max_ctx) { reason = "length"; break; }
        }
        if (!t.tokens.empty()) ev->push_back(t);
        if (!reason.empty()) finish(r, reason, ev);
    }

    void finish(Request& r, const std::string& reason, std::vector<Event>* ev) {
        if (r.state == RS_FINISHED) return;
        const int ps = cfg_.page_size;
        // publish the prompt's whole blocks (with the boundary snapshot) to the prefix cache
        if (r.row >= 0 && r.prefilled >= (int)r.prompt.size()) {
            const int nblk = (int)r.prompt.size() / ps;
            std::vector<int> pg(r.pages.begin(), r.pages.begin() + std::min<int>(nblk, (int)r.pages.size()));
            std::vector<int> snaps(pg.size(), -1);
            const int sb = ((int)r.prompt.size() - 1) / ps - 1;  // block that ends on the snapshot boundary
            if (sb >= 0 && sb < (int)snaps.size() && r.boundary_snapshot >= 0) snaps[sb] = r.boundary_snapshot;
            else if (r.boundary_snapshot >= 0) store_.release(r.boundary_snapshot);
            std::vector<int> dup_pages, dup_snaps;
            for (int p : pg) pages_.retain(p);  // the tree's own reference
            radix_.insert(r.prompt, pg, snaps, &dup_pages, &dup_snaps);
            for (int p : dup_pages) pages_.release(p);
            for (int s : dup_snaps) store_.release(s);
            // pages that were already in the tree (the shared prefix) got a second tree reference above
            for (int i = 0; i < r.shared_pages && i < (int)pg.size(); ++i) pages_.release(pg[i]);
        } else if (r.boundary_snapshot >= 0) {
            store_.release(r.boundary_snapshot);
        }
        for (int p : r.pages) pages_.release(p);
        r.pages.clear();
        if (r.radix_node) radix_.unlock(r.radix_node);
        if (r.row >= 0) { rows_[r.row] = -1; r.row = -1; }
        inflight_prefill_.erase(r.id);
        r.state = RS_FINISHED;
        r.finish_reason = reason;
        if (ev) {
            Event f{r.id, EV_FINISHED};
            f.reason = reason;
            f.prompt_tokens = (int)r.prompt.size(); f.completion_tokens = (int)r.generated.size();
            f.cached_tokens = r.cached_tokens;
            ev->push_back(f);
        }
    }

    // Keep live rows a dense prefix: the highest live row moves into the lowest hole.
    void compact_rows(TickPlan* p) {
        for (;;) {
            int hole = -1, top = -1;
            for (int i = 0; i < cfg_.max_rows; ++i) if (rows_[i] < 0) { hole = i; break; }
            for (int i = cfg_.max_rows - 1; i >= 0; --i) if (rows_[i] >= 0) { top = i; break; }
            if (hole < 0 || top < 0 || top < hole) break;
            const int64_t id = rows_[top];
            rows_[hole] = id; rows_[top] = -1;
            reqs_[id].row = hole;
            p->row_moves.push_back({top, hole, id});
        }
    }

    SchedConfig cfg_;
    PagePool pages_;
    RadixCache radix_;
    TieredStore store_;
    std::vector<int64_t> rows_;
    std::map<int64_t, Request> reqs_;
    std::deque<int64_t> queue_;
    std::map<int64_t, int> inflight_prefill_;
    std::vector<int64_t> pending_admit_events_;
    int64_t next_id_ = 1, ticks_ = 0, committed_ = 0;
};

}  // namespace fbrt
