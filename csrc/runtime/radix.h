// Radix prefix cache over token blocks.
//
// A node stands for one block of `block` tokens that extends its parent's prefix; it owns
// one KV page and, optionally, a snapshot id of the recurrent state taken at the end of the
// block.  A prefix hit is only usable at a node that carries a snapshot, because the
// GatedDeltaNet state cannot be rebuilt from pages.  Nodes on the path of a running
// sequence are pinned with lock_ref; eviction removes unpinned leaves in LRU order and
// hands their pages (and snapshots) back to the caller.  Same role as the reference's
// RadixCache (crates/ferrite-dispatch/src/radix.rs:169-515).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <vector>

namespace fbrt {

struct RadixStats {
    int64_t tree_nodes = 0, tree_blocks = 0, evictable_tokens = 0, protected_tokens = 0, hits = 0, misses = 0;
};

struct RadixMatch {
    int node = 0;                  // deepest usable node (0 = root: no hit)
    int tokens = 0;                // matched tokens (multiple of block)
    std::vector<int> pages;        // pages of the matched blocks, in order
    int snapshot = -1;             // recurrent-state snapshot at the match point
};

struct Evicted {
    std::vector<int> pages;
    std::vector<int> snapshots;
};

class RadixCache {
public:
    explicit RadixCache(int block) : block_(block) { nodes_.emplace_back(); nodes_[0].alive = true; }
    int block() const { return block_; }

    // Longest cached prefix of `tokens` that ends at a node with a snapshot.
    RadixMatch match(const std::vector<int32_t>& tokens) {
        RadixMatch best;
        std::vector<int> pages;
        int cur = 0;
        const int nblk = (int)tokens.size() / block_;
        for (int b = 0; b < nblk; ++b) {
            std::vector<int32_t> key(tokens.begin() + b * block_, tokens.begin() + (b + 1) * block_);
            auto it = nodes_[cur].children.find(key);
            if (it == nodes_[cur].children.end()) break;
            cur = it->second;
            pages.push_back(nodes_[cur].page);
            nodes_[cur].last_use = ++clock_;
            if (nodes_[cur].snapshot >= 0) {
                best.node = cur; best.tokens = (b + 1) * block_; best.pages = pages; best.snapshot = nodes_[cur].snapshot;
            }
        }
        if (best.tokens > 0) ++hits_; else ++misses_;
        return best;
    }

    // Insert the blocks of `tokens` (whole blocks only).  pages[b] / snapshots[b] describe
    // block b (snapshot -1 = none).  Blocks already present keep their page: the ids of the
    // duplicates are returned so the caller can release them.  Returns the deepest node.
    int insert(const std::vector<int32_t>& tokens, const std::vector<int>& pages, const std::vector<int>& snapshots,
               std::vector<int>* duplicate_pages = nullptr, std::vector<int>* duplicate_snaps = nullptr) {
        int cur = 0;
        const int nblk = std::min<int>((int)tokens.size() / block_, (int)pages.size());
        for (int b = 0; b < nblk; ++b) {
            std::vector<int32_t> key(tokens.begin() + b * block_, tokens.begin() + (b + 1) * block_);
            auto it = nodes_[cur].children.find(key);
            const int snap = b < (int)snapshots.size() ? snapshots[b] : -1;
            if (it != nodes_[cur].children.end()) {
                cur = it->second;
                if (nodes_[cur].page != pages[b] && duplicate_pages) duplicate_pages->push_back(pages[b]);
                if (snap >= 0) {
                    if (nodes_[cur].snapshot < 0) nodes_[cur].snapshot = snap;
                    else if (nodes_[cur].snapshot != snap && duplicate_snaps) duplicate_snaps->push_back(snap);
                }
            } else {
                const int id = new_node();
                nodes_[id].parent = cur; nodes_[id].key = key; nodes_[id].page = pages[b]; nodes_[id].snapshot = snap;
                nodes_[cur].children[key] = id;
                cur = id;
            }
            nodes_[cur].last_use = ++clock_;
        }
        return cur;
    }

    void lock(int node) { for (int n = node; n > 0; n = nodes_[n].parent) ++nodes_[n].lock_ref; }
    void unlock(int node) { for (int n = node; n > 0; n = nodes_[n].parent) if (nodes_[n].lock_ref > 0) --nodes_[n].lock_ref; }

    // Evict unpinned leaves, least recently used first, until `want_pages` pages are freed.
    Evicted evict(int want_pages) {
        Evicted ev;
        while ((int)ev.pages.size() < want_pages) {
            int victim = -1;
            for (int i = 1; i < (int)nodes_.size(); ++i) {
                const Node& n = nodes_[i];
                if (!n.alive || n.lock_ref > 0 || !n.children.empty()) continue;
                if (victim < 0 || n.last_use < nodes_[victim].last_use) victim = i;
            }
            if (victim < 0) break;
            Node& v = nodes_[victim];
            ev.pages.push_back(v.page);
            if (v.snapshot >= 0) ev.snapshots.push_back(v.snapshot);
            nodes_[v.parent].children.erase(v.key);
            v.alive = false; v.children.clear(); v.key.clear();
            free_ids_.push_back(victim);
        }
        return ev;
    }

    // Drop a node's snapshot (e.g. after the tiered store demoted or lost it).
    void clear_snapshot(int snapshot) {
        for (auto& n : nodes_) if (n.alive && n.snapshot == snapshot) n.snapshot = -1;
    }

    RadixStats stats() const {
        RadixStats s;
        s.hits = hits_; s.misses = misses_;
        for (int i = 1; i < (int)nodes_.size(); ++i) {
            const Node& n = nodes_[i];
            if (!n.alive) continue;
            ++s.tree_nodes; ++s.tree_blocks;
            (n.lock_ref > 0 ? s.protected_tokens : s.evictable_tokens) += block_;
        }
        return s;
    }

private:
    struct Node {
        int parent = 0, page = -1, snapshot = -1, lock_ref = 0;
        bool alive = false;
        uint64_t last_use = 0;
        std::vector<int32_t> key;
        std::map<std::vector<int32_t>, int> children;
    };
    int new_node() {
        int id;
        if (!free_ids_.empty()) { id = free_ids_.back(); free_ids_.pop_back(); nodes_[id] = Node(); }
        else { id = (int)nodes_.size(); nodes_.emplace_back(); }
        nodes_[id].alive = true;
        return id;
    }
    int block_;
    uint64_t clock_ = 0;
    int64_t hits_ = 0, misses_ = 0;
    std::vector<Node> nodes_;
    std::vector<int> free_ids_;
};

}  // namespace fbrt
