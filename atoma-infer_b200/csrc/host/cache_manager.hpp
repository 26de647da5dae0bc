// Paged cache bookkeeping (host only): page pools, block tables, state slots.
//
// The reference keeps one pool of pages shared by all layers, a LIFO free list
// (backends/vllm/src/block_allocator.rs:29-45, 59-67, 89-109) and one block table
// per sequence (backends/vllm/src/block_manager.rs:41).  It frees pages on abort
// and preemption only; a finished request's pages are never returned
// (backends/vllm/src/scheduler.rs:2203-2216).
//
// Here layers are put into groups by what they need of the cache (all keys, or a
// window of them); every group has a pool and block tables of its own.  A block
// table is indexed by absolute page number (position / page_size); entries whose
// positions have left a window are -1 and their pages are back in the pool.
// Beside the pages there are `max_seqs` slots of fixed-size per-request state.
// Page 0 of every pool is never handed out: padded batch rows write there.
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace engine {

enum CacheKind : int { kFullKeys = 0, kWindowKeys = 1 };

enum CacheStatus : int {
    kOk = 0,
    kErrNoPages = -1,       // a pool cannot cover the request now
    kErrNoSlot = -2,        // all state slots are taken
    kErrUnknownRequest = -3,// also: freed twice
    kErrDuplicate = -4,
    kErrNotReserved = -5,   // advance beyond what was reserved
    kErrNever = -6,         // would not fit an empty pool either
    kErrArgument = -7,
};

struct GroupSpec {
    int kind;       // CacheKind
    int window;     // keys a query may look back over, itself included (kWindowKeys only)
    int num_pages;  // pool size including the reserved page 0
};

class CacheManager {
public:
    CacheManager(int page_size, const std::vector<GroupSpec>& groups, int max_seqs);

    int page_size() const { return page_size_; }
    int num_groups() const { return (int)groups_.size(); }
    int max_seqs() const { return max_seqs_; }

    // Claims a state slot; the request holds no tokens yet.  Returns the slot or an error.
    int add_request(int64_t req);
    bool has_request(int64_t req) const { return reqs_.count(req) != 0; }

    // Pages this request would have to take from pool `g` so that its cache covers
    // `upto` tokens (counting from its current length; what a window has passed is not needed).
    int pages_needed(int64_t req, int g, int64_t upto) const;
    // Same for a request that is not admitted yet (length 0).
    int pages_needed_new(int g, int64_t upto) const;
    // kOk if every pool can cover `upto` tokens of this request now, kErrNoPages if
    // not now, kErrNever if not even when empty.
    int can_reserve(int64_t req, int64_t upto) const;
    // Takes the pages; all pools or none.
    int reserve(int64_t req, int64_t upto);
    // The request now holds `n` more tokens (they must be reserved).  Returns pages
    // that a window has passed to their pools.
    int advance(int64_t req, int64_t n);
    // Returns every page and the state slot.  Unknown request (or freed twice): error.
    int free_request(int64_t req);

    int64_t num_tokens(int64_t req) const;
    int state_slot(int64_t req) const;
    // Block table of `req` in group `g`: writes up to `cap` entries, returns the length.
    int table(int64_t req, int g, int32_t* out, int cap) const;
    int table_len(int64_t req, int g) const;

    int num_free_pages(int g) const { return (int)groups_[g].free_list.size(); }
    int num_usable_pages(int g) const { return groups_[g].spec.num_pages - 1; }
    int num_free_slots() const { return (int)free_slots_.size(); }
    int num_requests() const { return (int)reqs_.size(); }

    // Bookkeeping audit: every page of every pool is either free or held by exactly
    // one request, page 0 by nobody; same for slots.  Empty string = consistent.
    std::string audit() const;

private:
    struct Group {
        GroupSpec spec;
        std::vector<int32_t> free_list;  // LIFO: the back is handed out next
        std::vector<uint8_t> held;       // per page
    };
    struct Request {
        int64_t num_tokens = 0;
        int slot = -1;
        std::vector<std::vector<int32_t>> tables;  // per group, absolute page index -> page or -1
        std::vector<int64_t> first_live;           // per group, first table index that may be held
    };
    int64_t first_needed_page(const Group& g, int64_t num_tokens) const;
    int needed(const Group& g, const Request* r, int gi, int64_t upto) const;

    int page_size_;
    int max_seqs_;
    std::vector<Group> groups_;
    std::vector<int32_t> free_slots_;
    std::vector<uint8_t> slot_held_;
    std::unordered_map<int64_t, Request> reqs_;
};

}  // namespace engine
