// Three-tier store for recurrent-state snapshots: device -> host -> disk.
//
// The store only does the bookkeeping: it decides which snapshot lives in which slot of
// which tier and emits the copies ("moves") that the execution backend must perform.
// Pressure demotes before it drops: a full device tier pushes its least recently used
// snapshot to the host tier, a full host tier pushes to disk, and a snapshot is dropped only
// when every tier refuses (reference crates/ferrite-dispatch/src/state.rs:89-856).
#pragma once
#include <cstdint>
#include <map>
#include <stdexcept>
#include <vector>

namespace fbrt {

enum Tier : int { TIER_DEVICE = 0, TIER_HOST = 1, TIER_DISK = 2, TIER_NONE = 3 };

struct StateMove {
    int snapshot;
    int from_tier, from_slot;  // TIER_NONE = freshly captured from a live row (from_slot = row)
    int to_tier, to_slot;      // TIER_NONE = dropped
};

class TieredStore {
public:
    TieredStore(int device_slots, int host_slots, int disk_slots) {
        cap_[0] = device_slots; cap_[1] = host_slots; cap_[2] = disk_slots;
        for (int t = 0; t < 3; ++t) {
            free_[t].reserve(cap_[t]);
            for (int s = cap_[t] - 1; s >= 0; --s) free_[t].push_back(s);
        }
    }

    // Register a new snapshot captured from live row `row`; returns its id.  `moves` receives
    // the demotions that made room followed by the capture itself.
    int capture(int row, std::vector<StateMove>* moves, std::vector<int>* dropped) {
        const int id = next_id_++;
        const int slot = make_room(TIER_DEVICE, moves, dropped);
        if (slot < 0) { if (dropped) dropped->push_back(id); return -1; }
        entries_[id] = {TIER_DEVICE, slot, ++clock_};
        moves->push_back({id, TIER_NONE, row, TIER_DEVICE, slot});
        return id;
    }

    // Make `id` device resident (for a prefix hit); returns its device slot or -1 if unknown.
    int promote(int id, std::vector<StateMove>* moves, std::vector<int>* dropped) {
        auto it = entries_.find(id);
        if (it == entries_.end()) return -1;
        it->second.last_use = ++clock_;
        if (it->second.tier == TIER_DEVICE) return it->second.slot;
        const int from_tier = it->second.tier, from_slot = it->second.slot;
        it->second.tier = TIER_NONE;  // keep it out of the victim search
        const int slot = make_room(TIER_DEVICE, moves, dropped);
        it = entries_.find(id);
        if (slot < 0) { it->second.tier = from_tier; return -1; }
        free_[from_tier].push_back(from_slot);
        it->second.tier = TIER_DEVICE; it->second.slot = slot;
        moves->push_back({id, from_tier, from_slot, TIER_DEVICE, slot});
        return slot;
    }

    void touch(int id) { auto it = entries_.find(id); if (it != entries_.end()) it->second.last_use = ++clock_; }

    void release(int id) {
        auto it = entries_.find(id);
        if (it == entries_.end()) return;
        if (it->second.tier != TIER_NONE) free_[it->second.tier].push_back(it->second.slot);
        entries_.erase(it);
    }

    int tier_of(int id) const { auto it = entries_.find(id); return it == entries_.end() ? TIER_NONE : it->second.tier; }
    int slot_of(int id) const { auto it = entries_.find(id); return it == entries_.end() ? -1 : it->second.slot; }
    std::vector<int> census() const {
        std::vector<int> c(3, 0);
        for (const auto& kv : entries_) if (kv.second.tier < 3) ++c[kv.second.tier];
        return c;
    }

private:
    struct Entry { int tier, slot; uint64_t last_use; };

    // A free slot in `tier`, demoting that tier's LRU entry downwards when it is full.
    int make_room(int tier, std::vector<StateMove>* moves, std::vector<int>* dropped) {
        if (tier > TIER_DISK || cap_[tier] == 0) return -1;
        if (!free_[tier].empty()) { int s = free_[tier].back(); free_[tier].pop_back(); return s; }
        int victim = -1;
        for (const auto& kv : entries_)
            if (kv.second.tier == tier && (victim < 0 || kv.second.last_use < entries_[victim].last_use)) victim = kv.first;
        if (victim < 0) return -1;
        const int vslot = entries_[victim].slot;
        const int down = make_room(tier + 1, moves, dropped);
        if (down >= 0) {
            moves->push_back({victim, tier, vslot, tier + 1, down});
            entries_[victim].tier = tier + 1; entries_[victim].slot = down;
        } else {
            moves->push_back({victim, tier, vslot, TIER_NONE, -1});
            if (dropped) dropped->push_back(victim);
            entries_.erase(victim);
        }
        return vslot;
    }

    int cap_[3];
    std::vector<int> free_[3];
    std::map<int, Entry> entries_;
    int next_id_ = 1;
    uint64_t clock_ = 0;
};

}  // namespace fbrt
