// Page allocator, per-request block tables and state slots.
//
// The cache is divided into groups of layers with the same needs; each group
// has its own pages, its own free list and, for every request, its own block
// table.  A group with a window w only needs the keys of the last w positions:
// pages that every future query has passed are given back at commit time and
// their block-table entries become -1.  Beside the pages, every live request
// holds one state slot: an index into fixed-size per-request buffers, and the
// place of its RequestRecord, the one fixed-size description of a live request
// (position, lengths, sampling parameters, seed) that decode steps are packed
// from.  The reference spreads the same over Request and SamplingParams
// (crates/vllm-scheduler/src/request.rs:37-76,95-193).
//
// Policy as in the reference's BlockAllocator
// (crates/vllm-paged-attention/src/allocator.rs:57-86): FIFO free list
// (pop front, push back) so that reuse order is deterministic, a reference
// count per page, and a double free is an error.  The reference shares one
// pool between all layers (crates/vllm-paged-attention/src/block.rs:49-59);
// here a page id addresses one page in every layer of its group.
#pragma once
#include <cstdint>
#include <deque>
#include <unordered_map>
#include <vector>

namespace railgun {

enum CacheStatus : int {
    CACHE_OK = 0,
    CACHE_OUT_OF_PAGES = -1,
    CACHE_DUPLICATE = -2,
    CACHE_UNKNOWN_REQUEST = -3,
    CACHE_OUT_OF_SLOTS = -4,
    CACHE_BAD_ARGUMENT = -5,
    CACHE_CORRUPT = -6,
};

struct CacheGroup {
    int page_size = 16;
    int num_pages = 0;
    int window = 0;                 // 0: every key is kept
    std::deque<int> free_list;
    std::vector<int> refcount;
};

// One per state slot, 64 bytes, plain data: Python reads the array in place and may copy it to the device.
struct RequestRecord {
    int64_t request_id = -1;        // -1: the slot is free
    int32_t num_computed = 0;       // the request's position: tokens whose keys/state are in the cache
    int32_t prompt_len = 0;
    int32_t num_generated = 0;      // also the number of the request's next random draw
    int32_t max_new_tokens = 0;
    int32_t last_token = -1;
    int32_t top_k = 0;              // 0: no top-k filter
    float temperature = 0.f;        // 0: greedy
    float top_p = 1.f;
    uint64_t seed = 0;
    int32_t flags = 0;
    int32_t reserved[3] = {0, 0, 0};
};
static_assert(sizeof(RequestRecord) == 64, "RequestRecord is read as 16 32-bit words");

struct CacheRequest {
    int slot = -1;
    std::vector<std::vector<int>> tables;   // per group: logical page -> page id, -1 once released
};

class CacheManager {
public:
    CacheManager(int n_groups, const int* page_size, const int* num_pages, const int* window, int max_slots) {
        groups_.resize(n_groups);
        for (int g = 0; g < n_groups; ++g) {
            CacheGroup& G = groups_[g];
            G.page_size = page_size[g];
            G.num_pages = num_pages[g];
            G.window = window[g];
            G.refcount.assign(G.num_pages, 0);
            for (int p = 0; p < G.num_pages; ++p) G.free_list.push_back(p);
        }
        max_slots_ = max_slots;
        for (int s = 0; s < max_slots; ++s) free_slots_.push_back(s);
        records_.assign((size_t)(max_slots > 0 ? max_slots : 1), RequestRecord());
    }

    int num_groups() const { return (int)groups_.size(); }
    const CacheGroup& group(int g) const { return groups_[g]; }
    int free_pages(int g) const { return (int)groups_[g].free_list.size(); }
    int free_slots() const { return (int)free_slots_.size(); }
    int max_slots() const { return max_slots_; }
    int num_requests() const { return (int)reqs_.size(); }
    bool has(int64_t id) const { return reqs_.count(id) != 0; }

    // A new request: takes a state slot.  Returns the slot or a negative status.
    int add_request(int64_t id) {
        if (reqs_.count(id)) return CACHE_DUPLICATE;
        if (free_slots_.empty()) return CACHE_OUT_OF_SLOTS;
        CacheRequest r;
        r.slot = free_slots_.front();
        free_slots_.pop_front();
        r.tables.resize(groups_.size());
        records_[r.slot] = RequestRecord();
        records_[r.slot].request_id = id;
        reqs_.emplace(id, std::move(r));
        return reqs_[id].slot;
    }

    // The record of a live request (nullptr if unknown), and all of them by slot.
    RequestRecord* record(int64_t id) {
        auto it = reqs_.find(id);
        return it == reqs_.end() ? nullptr : &records_[it->second.slot];
    }
    const RequestRecord* record(int64_t id) const {
        auto it = reqs_.find(id);
        return it == reqs_.end() ? nullptr : &records_[it->second.slot];
    }
    const RequestRecord* records() const { return records_.data(); }
    int num_computed(int64_t id) const {
        const RequestRecord* r = record(id);
        return r ? r->num_computed : 0;
    }

    // Pages each group would have to add so that the request can hold new_len tokens.
    int pages_needed(int64_t id, int new_len, int* per_group) const {
        auto it = reqs_.find(id);
        for (size_t g = 0; g < groups_.size(); ++g) {
            const int have = it == reqs_.end() ? 0 : (int)it->second.tables[g].size();
            const int want = (new_len + groups_[g].page_size - 1) / groups_[g].page_size;
            per_group[g] = want > have ? want - have : 0;
        }
        return CACHE_OK;
    }

    // Could a request (live or not yet added) grow to new_len, leaving `spare` pages free in every group?
    bool can_reserve(int64_t id, int new_len, int spare = 0) const {
        std::vector<int> need(groups_.size());
        pages_needed(id, new_len, need.data());
        for (size_t g = 0; g < groups_.size(); ++g)
            if (need[g] + spare > (int)groups_[g].free_list.size() && need[g] > 0) return false;
        return true;
    }

    // Make room for tokens [0, new_len): all groups or none.
    int reserve(int64_t id, int new_len) {
        auto it = reqs_.find(id);
        if (it == reqs_.end()) return CACHE_UNKNOWN_REQUEST;
        if (new_len < 0) return CACHE_BAD_ARGUMENT;
        std::vector<int> need(groups_.size());
        pages_needed(id, new_len, need.data());
        for (size_t g = 0; g < groups_.size(); ++g)
            if (need[g] > (int)groups_[g].free_list.size()) return CACHE_OUT_OF_PAGES;
        for (size_t g = 0; g < groups_.size(); ++g) {
            CacheGroup& G = groups_[g];
            for (int k = 0; k < need[g]; ++k) {
                const int p = G.free_list.front();
                G.free_list.pop_front();
                G.refcount[p] = 1;
                it->second.tables[g].push_back(p);
            }
        }
        return CACHE_OK;
    }

    // Tokens [0, new_len) are now in the cache; windowed groups give back what every later query has passed.
    int commit(int64_t id, int new_len) {
        auto it = reqs_.find(id);
        if (it == reqs_.end()) return CACHE_UNKNOWN_REQUEST;
        CacheRequest& r = it->second;
        for (size_t g = 0; g < groups_.size(); ++g)
            if (new_len > (int)r.tables[g].size() * groups_[g].page_size) return CACHE_BAD_ARGUMENT;
        records_[r.slot].num_computed = new_len;
        for (size_t g = 0; g < groups_.size(); ++g) {
            CacheGroup& G = groups_[g];
            if (G.window <= 0) continue;
            const int first_needed = new_len - G.window + 1;     // lowest key any later query reads
            for (size_t i = 0; i < r.tables[g].size(); ++i) {
                if ((int)(i + 1) * G.page_size > first_needed) break;
                if (r.tables[g][i] >= 0) {
                    const int st = free_page(G, r.tables[g][i]);
                    if (st != CACHE_OK) return st;
                    r.tables[g][i] = -1;
                }
            }
        }
        return CACHE_OK;
    }

    // The request ends (finished, aborted or preempted): all pages and the slot come back.
    int release(int64_t id) {
        auto it = reqs_.find(id);
        if (it == reqs_.end()) return CACHE_UNKNOWN_REQUEST;
        int status = CACHE_OK;
        for (size_t g = 0; g < groups_.size(); ++g)
            for (int p : it->second.tables[g])
                if (p >= 0) {
                    const int st = free_page(groups_[g], p);
                    if (st != CACHE_OK) status = st;
                }
        free_slots_.push_back(it->second.slot);
        records_[it->second.slot] = RequestRecord();
        reqs_.erase(it);
        return status;
    }

    const CacheRequest* find(int64_t id) const {
        auto it = reqs_.find(id);
        return it == reqs_.end() ? nullptr : &it->second;
    }

    // Every page is free exactly once or held exactly once; every slot likewise.
    int check() const {
        for (size_t g = 0; g < groups_.size(); ++g) {
            const CacheGroup& G = groups_[g];
            std::vector<int> seen(G.num_pages, 0);
            for (int p : G.free_list) {
                if (p < 0 || p >= G.num_pages || seen[p]++) return CACHE_CORRUPT;
                if (G.refcount[p] != 0) return CACHE_CORRUPT;
            }
            for (const auto& kv : reqs_)
                for (int p : kv.second.tables[g]) {
                    if (p < 0) continue;
                    if (p >= G.num_pages || seen[p]++) return CACHE_CORRUPT;
                    if (G.refcount[p] != 1) return CACHE_CORRUPT;
                }
            for (int p = 0; p < G.num_pages; ++p)
                if (seen[p] != 1) return CACHE_CORRUPT;
        }
        std::vector<int> slot_seen(max_slots_, 0);
        for (int s : free_slots_)
            if (s < 0 || s >= max_slots_ || slot_seen[s]++) return CACHE_CORRUPT;
        for (const auto& kv : reqs_) {
            if (kv.second.slot < 0 || kv.second.slot >= max_slots_ || slot_seen[kv.second.slot]++) return CACHE_CORRUPT;
            if (records_[kv.second.slot].request_id != kv.first) return CACHE_CORRUPT;
        }
        for (int s : free_slots_)
            if (records_[s].request_id != -1) return CACHE_CORRUPT;
        for (int s = 0; s < max_slots_; ++s)
            if (slot_seen[s] != 1) return CACHE_CORRUPT;
        return CACHE_OK;
    }

private:
    int free_page(CacheGroup& G, int p) {
        if (p < 0 || p >= G.num_pages || G.refcount[p] <= 0) return CACHE_CORRUPT;   // double free
        if (--G.refcount[p] == 0) G.free_list.push_back(p);
        return CACHE_OK;
    }

    std::vector<CacheGroup> groups_;
    std::unordered_map<int64_t, CacheRequest> reqs_;
    std::deque<int> free_slots_;
    std::vector<RequestRecord> records_;
    int max_slots_ = 0;
};

}  // namespace railgun
