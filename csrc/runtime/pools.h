// Page allocator, state-slot pool and the CP -> DCP reshard planner.
//
// Pages hold `page_size` tokens of DSA latent KV (all DSA layers share one page id space);
// a page may be leased by several sequences through the radix prefix cache, hence the
// reference counts.  Slots hold the recurrent (GatedDeltaNet + conv) state of one
// sequence.  The reshard plan maps prefill-side pages to decode-context-parallel ranks:
// page p lives on rank p % n_dcp at local index p / n_dcp, recurrent state goes whole to
// every decode rank (reference crates/ferrite-kv/src/lib.rs:43-432, shard.rs:37-212).
#pragma once
#include <cstdint>
#include <stdexcept>
#include <utility>
#include <vector>

namespace fbrt {

class PagePool {
public:
    explicit PagePool(int num_pages) : ref_(num_pages, 0) {
        free_.reserve(num_pages);
        for (int p = num_pages - 1; p >= 0; --p) free_.push_back(p);
    }
    int num_pages() const { return (int)ref_.size(); }
    int free_pages() const { return (int)free_.size(); }
    int pages_in_use() const { return num_pages() - free_pages(); }
    bool can_alloc(int n) const { return n <= free_pages(); }
    // All-or-nothing allocation; an empty vector with n > 0 means "not enough pages".
    std::vector<int> alloc(int n) {
        std::vector<int> out;
        if (n > free_pages()) return out;
        out.reserve(n);
        for (int i = 0; i < n; ++i) {
            int p = free_.back();
            free_.pop_back();
            ref_[p] = 1;
            out.push_back(p);
        }
        return out;
    }
    void retain(int p) { check(p); if (ref_[p] <= 0) throw std::runtime_error("retain of a free page"); ++ref_[p]; }
    // Drops one reference; the page returns to the free list when nobody holds it.
    void release(int p) {
        check(p);
        if (ref_[p] <= 0) throw std::runtime_error("release of a free page");
        if (--ref_[p] == 0) free_.push_back(p);
    }
    int refcount(int p) const { return ref_.at(p); }

private:
    void check(int p) const { if (p < 0 || p >= (int)ref_.size()) throw std::out_of_range("page id"); }
    std::vector<int> ref_;
    std::vector<int> free_;
};

class SlotPool {
public:
    explicit SlotPool(int n) : used_(n, false) {}
    int capacity() const { return (int)used_.size(); }
    int in_use() const { int c = 0; for (bool u : used_) c += u; return c; }
    int alloc() {
        for (int i = 0; i < (int)used_.size(); ++i)
            if (!used_[i]) { used_[i] = true; return i; }
        return -1;
    }
    void free(int s) { used_.at(s) = false; }
    bool is_used(int s) const { return used_.at(s); }

private:
    std::vector<bool> used_;
};

// Layers [lo, hi) owned by context-parallel prefill rank r (contiguous layer split).
inline std::pair<int, int> cp_layer_range(int rank, int n_cp, int n_layers) {
    const int base = n_layers / n_cp, rem = n_layers % n_cp;
    const int lo = rank * base + (rank < rem ? rank : rem);
    return {lo, lo + base + (rank < rem ? 1 : 0)};
}

struct PageMove {
    int page;       // logical page index of the sequence
    int dst_rank;   // decode rank that owns it
    int dst_index;  // index among that rank's pages
};

struct ReshardPlan {
    int n_cp = 1, n_dcp = 1;
    std::vector<int> state_layers;  // recurrent layers: state copied whole to every decode rank
    std::vector<int> paged_layers;  // DSA layers: pages split round robin
    std::vector<int> layer_owner;   // prefill rank that produced each layer
    std::vector<PageMove> moves;

    static ReshardPlan compile(const std::vector<int>& is_dsa_layer, int n_cp, int n_dcp, int n_pages) {
        ReshardPlan p;
        p.n_cp = n_cp; p.n_dcp = n_dcp;
        const int L = (int)is_dsa_layer.size();
        p.layer_owner.resize(L);
        for (int r = 0; r < n_cp; ++r) {
            auto [lo, hi] = cp_layer_range(r, n_cp, L);
            for (int l = lo; l < hi; ++l) p.layer_owner[l] = r;
        }
        for (int l = 0; l < L; ++l) (is_dsa_layer[l] ? p.paged_layers : p.state_layers).push_back(l);
        for (int pg = 0; pg < n_pages; ++pg) p.moves.push_back({pg, pg % n_dcp, pg / n_dcp});
        return p;
    }
    std::vector<int> filter_pages(int dcp_rank) const {
        std::vector<int> out;
        for (const auto& m : moves) if (m.dst_rank == dcp_rank) out.push_back(m.page);
        return out;
    }
};

}  // namespace fbrt
