#include "cache_manager.hpp"

#include <algorithm>
#include <sstream>

namespace engine {

CacheManager::CacheManager(int page_size, const std::vector<GroupSpec>& groups, int max_seqs)
    : page_size_(page_size), max_seqs_(max_seqs) {
    for (const GroupSpec& s : groups) {
        Group g;
        g.spec = s;
        g.held.assign(std::max(s.num_pages, 1), 0);
        // Pages 1..num_pages-1, pushed in rising order: the highest id is handed out
        // first, as the reference's allocator does (block_allocator.rs:59-67).
        for (int p = 1; p < s.num_pages; ++p) g.free_list.push_back(p);
        groups_.push_back(std::move(g));
    }
    slot_held_.assign(max_seqs, 0);
    for (int s = max_seqs - 1; s >= 0; --s) free_slots_.push_back(s);  // slot 0 first
}

int CacheManager::add_request(int64_t req) {
    if (reqs_.count(req)) return kErrDuplicate;
    if (free_slots_.empty()) return kErrNoSlot;
    Request r;
    r.slot = free_slots_.back();
    free_slots_.pop_back();
    slot_held_[r.slot] = 1;
    r.tables.resize(groups_.size());
    r.first_live.assign(groups_.size(), 0);
    int slot = r.slot;
    reqs_.emplace(req, std::move(r));
    return slot;
}

// First absolute page index that a request of `num_tokens` cached tokens still
// needs: its next query sits at position num_tokens and looks back over `window`
// keys, itself included, so the oldest key needed is num_tokens - window + 1.
int64_t CacheManager::first_needed_page(const Group& g, int64_t num_tokens) const {
    if (g.spec.kind != kWindowKeys) return 0;
    int64_t oldest = num_tokens - (int64_t)g.spec.window + 1;
    if (oldest <= 0) return 0;
    return oldest / page_size_;
}

int CacheManager::needed(const Group& g, const Request* r, int gi, int64_t upto) const {
    if (upto <= 0) return 0;
    int64_t last = (upto + page_size_ - 1) / page_size_;  // table length wanted
    int64_t first = first_needed_page(g, r ? r->num_tokens : 0);
    // Every entry between the first needed page and the table's end is held: reserve()
    // fills that whole range and the first needed page only moves forward.
    int64_t have_to = r ? std::max<int64_t>(first, (int64_t)r->tables[gi].size()) : first;
    return (int)std::max<int64_t>(0, last - have_to);
}

int CacheManager::pages_needed(int64_t req, int g, int64_t upto) const {
    auto it = reqs_.find(req);
    if (it == reqs_.end()) return kErrUnknownRequest;
    if (g < 0 || g >= num_groups()) return kErrArgument;
    return needed(groups_[g], &it->second, g, upto);
}

int CacheManager::pages_needed_new(int g, int64_t upto) const {
    if (g < 0 || g >= num_groups()) return kErrArgument;
    return needed(groups_[g], nullptr, g, upto);
}

int CacheManager::can_reserve(int64_t req, int64_t upto) const {
    auto it = reqs_.find(req);
    const Request* r = it == reqs_.end() ? nullptr : &it->second;
    int status = kOk;
    for (int g = 0; g < num_groups(); ++g) {
        int n = needed(groups_[g], r, g, upto);
        // Entries from first_live to the table's end are held, the ones before it are given back.
        int held = r ? (int)((int64_t)r->tables[g].size() - r->first_live[g]) : 0;
        if (n + held > num_usable_pages(g)) return kErrNever;
        if (n > num_free_pages(g)) status = kErrNoPages;
    }
    return status;
}

int CacheManager::reserve(int64_t req, int64_t upto) {
    auto it = reqs_.find(req);
    if (it == reqs_.end()) return kErrUnknownRequest;
    int can = can_reserve(req, upto);
    if (can != kOk) return can;
    Request& r = it->second;
    if (upto <= 0) return kOk;
    int64_t last = (upto + page_size_ - 1) / page_size_;
    for (int g = 0; g < num_groups(); ++g) {
        Group& grp = groups_[g];
        std::vector<int32_t>& t = r.tables[g];
        if ((int64_t)t.size() < last) t.resize(last, -1);
        int64_t first = first_needed_page(grp, r.num_tokens);
        for (int64_t i = first; i < last; ++i) {
            if (t[i] >= 0) continue;
            int32_t p = grp.free_list.back();
            grp.free_list.pop_back();
            grp.held[p] = 1;
            t[i] = p;
        }
    }
    return kOk;
}

int CacheManager::advance(int64_t req, int64_t n) {
    auto it = reqs_.find(req);
    if (it == reqs_.end()) return kErrUnknownRequest;
    if (n < 0) return kErrArgument;
    Request& r = it->second;
    int64_t upto = r.num_tokens + n;
    for (int g = 0; g < num_groups(); ++g) {
        int64_t last = (upto + page_size_ - 1) / page_size_;
        if ((int64_t)r.tables[g].size() < last) return kErrNotReserved;
        int64_t first = first_needed_page(groups_[g], r.num_tokens);
        for (int64_t i = first; i < last; ++i)
            if (r.tables[g][i] < 0) return kErrNotReserved;
    }
    r.num_tokens = upto;
    int released = 0;
    for (int g = 0; g < num_groups(); ++g) {
        Group& grp = groups_[g];
        int64_t first = std::min<int64_t>(first_needed_page(grp, r.num_tokens), (int64_t)r.tables[g].size());
        for (int64_t i = r.first_live[g]; i < first; ++i) {
            int32_t p = r.tables[g][i];
            if (p >= 0) {
                grp.held[p] = 0;
                grp.free_list.push_back(p);
                r.tables[g][i] = -1;
                ++released;
            }
        }
        r.first_live[g] = std::max(r.first_live[g], first);
    }
    return released;
}

int CacheManager::free_request(int64_t req) {
    auto it = reqs_.find(req);
    if (it == reqs_.end()) return kErrUnknownRequest;
    Request& r = it->second;
    int n = 0;
    for (int g = 0; g < num_groups(); ++g) {
        Group& grp = groups_[g];
        // Pages go back in table order, so the last page of the request is the next
        // one handed out: a later request sees them in another physical order.
        for (int32_t p : r.tables[g]) {
            if (p < 0) continue;
            grp.held[p] = 0;
            grp.free_list.push_back(p);
            ++n;
        }
    }
    slot_held_[r.slot] = 0;
    free_slots_.push_back(r.slot);
    reqs_.erase(it);
    return n;
}

int64_t CacheManager::num_tokens(int64_t req) const {
    auto it = reqs_.find(req);
    return it == reqs_.end() ? (int64_t)kErrUnknownRequest : it->second.num_tokens;
}

int CacheManager::state_slot(int64_t req) const {
    auto it = reqs_.find(req);
    return it == reqs_.end() ? (int)kErrUnknownRequest : it->second.slot;
}

int CacheManager::table_len(int64_t req, int g) const {
    auto it = reqs_.find(req);
    if (it == reqs_.end()) return kErrUnknownRequest;
    if (g < 0 || g >= num_groups()) return kErrArgument;
    return (int)it->second.tables[g].size();
}

int CacheManager::table(int64_t req, int g, int32_t* out, int cap) const {
    auto it = reqs_.find(req);
    if (it == reqs_.end()) return kErrUnknownRequest;
    if (g < 0 || g >= num_groups()) return kErrArgument;
    const std::vector<int32_t>& t = it->second.tables[g];
    int n = std::min<int>((int)t.size(), cap);
    for (int i = 0; i < n; ++i) out[i] = t[i];
    return (int)t.size();
}

std::string CacheManager::audit() const {
    std::ostringstream err;
    for (int g = 0; g < num_groups(); ++g) {
        const Group& grp = groups_[g];
        std::vector<int> seen(grp.spec.num_pages, 0);
        for (int32_t p : grp.free_list) {
            if (p <= 0 || p >= grp.spec.num_pages) { err << "group " << g << ": free list holds bad page " << p << "; "; continue; }
            if (grp.held[p]) err << "group " << g << ": page " << p << " is free and held; ";
            if (seen[p]++) err << "group " << g << ": page " << p << " is free twice; ";
        }
        for (const auto& kv : reqs_) {
            const std::vector<int32_t>& t = kv.second.tables[g];
            for (size_t i = 0; i < t.size(); ++i) {
                int32_t p = t[i];
                if (p < 0) continue;
                if (p == 0 || p >= grp.spec.num_pages) { err << "group " << g << ": request " << kv.first << " holds bad page " << p << "; "; continue; }
                if (!grp.held[p]) err << "group " << g << ": page " << p << " is in a table but not marked held; ";
                if (seen[p]++) err << "group " << g << ": page " << p << " is held twice; ";
            }
        }
        for (int p = 1; p < grp.spec.num_pages; ++p)
            if (!seen[p]) err << "group " << g << ": page " << p << " is lost; ";
    }
    std::vector<int> sseen(max_seqs_, 0);
    for (int32_t s : free_slots_) {
        if (s < 0 || s >= max_seqs_) { err << "bad free slot " << s << "; "; continue; }
        if (sseen[s]++) err << "slot " << s << " is free twice; ";
        if (slot_held_[s]) err << "slot " << s << " is free and held; ";
    }
    for (const auto& kv : reqs_) {
        int s = kv.second.slot;
        if (s < 0 || s >= max_seqs_) { err << "request " << kv.first << " has bad slot; "; continue; }
        if (sseen[s]++) err << "slot " << s << " is held twice; ";
    }
    for (int s = 0; s < max_seqs_; ++s)
        if (!sseen[s]) err << "slot " << s << " is lost; ";
    return err.str();
}

}  // namespace engine
