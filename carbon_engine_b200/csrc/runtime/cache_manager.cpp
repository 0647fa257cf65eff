#include "cache_manager.h"

#include <algorithm>
#include <functional>

namespace carbon {

PagePool::PagePool(int num_pages) : held_(num_pages > 0 ? num_pages : 0, 0) {
    free_.reserve(held_.size());
    for (int i = 0; i < (int)held_.size(); ++i) free_.push_back(i);
    std::make_heap(free_.begin(), free_.end(), std::greater<int>());
}

int PagePool::acquire() {
    if (free_.empty()) return -1;
    std::pop_heap(free_.begin(), free_.end(), std::greater<int>());
    int page = free_.back();
    free_.pop_back();
    held_[page] = 1;
    return page;
}

bool PagePool::release(int page) {
    if (page < 0 || page >= (int)held_.size() || !held_[page]) return false;
    held_[page] = 0;
    free_.push_back(page);
    std::push_heap(free_.begin(), free_.end(), std::greater<int>());
    return true;
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

CacheManager::CacheManager(const std::vector<GroupSpec>& groups, int max_requests, int max_pages_per_request)
    : groups_(groups), max_requests_(max_requests), max_pages_(max_pages_per_request) {
    for (const auto& g : groups_) {
        pools_.emplace_back(g.num_pages);
        tables_.emplace_back((size_t)max_requests_ * max_pages_, -1);
    }
    for (int s = max_requests_ - 1; s >= 0; --s) free_slots_.push_back(s);   // low slots go out first
}

int CacheManager::first_needed_page(int group, int length) const {
    const GroupSpec& g = groups_[group];
    if (g.window <= 0) return 0;
    int first_pos = std::max(0, length - g.window + 1);
    return first_pos / g.page_size;
}

int CacheManager::open(int64_t id) {
    if (requests_.count(id)) return CACHE_DUPLICATE;
    if (free_slots_.empty()) return CACHE_NO_SLOT;
    int slot = free_slots_.back();
    free_slots_.pop_back();
    Request r;
    r.slot = slot;
    r.length = 0;
    r.reserved = 0;
    r.first_page.assign(groups_.size(), 0);
    requests_.emplace(id, std::move(r));
    return slot;
}

int CacheManager::pages_to_reserve(int64_t id, int group, int new_len) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) return CACHE_UNKNOWN;
    const Request& r = it->second;
    const GroupSpec& g = groups_[group];
    int hi = ceil_div(new_len, g.page_size);
    if (hi > max_pages_) return CACHE_TOO_LONG;
    int lo = std::max(r.first_page[group], first_needed_page(group, r.length));
    const int32_t* row = tables_[group].data() + (size_t)r.slot * max_pages_;
    int n = 0;
    for (int i = lo; i < hi; ++i) n += row[i] < 0;
    return n;
}

int CacheManager::reserve(int64_t id, int new_len) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return CACHE_UNKNOWN;
    Request& r = it->second;
    if (new_len < r.length) return CACHE_BAD_ARG;
    // first see that every group can give what is asked, so that a refusal changes nothing
    for (int g = 0; g < (int)groups_.size(); ++g) {
        int need = pages_to_reserve(id, g, new_len);
        if (need < 0) return need;
        if (need > pools_[g].free_count()) return CACHE_NO_PAGES;
    }
    for (int g = 0; g < (int)groups_.size(); ++g) {
        int hi = ceil_div(new_len, groups_[g].page_size);
        int lo = std::max(r.first_page[g], first_needed_page(g, r.length));
        int32_t* row = table_row(g, r.slot);
        for (int i = lo; i < hi; ++i)
            if (row[i] < 0) row[i] = pools_[g].acquire();
    }
    r.reserved = std::max(r.reserved, new_len);
    return CACHE_OK;
}

int CacheManager::commit(int64_t id, int new_len) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return CACHE_UNKNOWN;
    Request& r = it->second;
    if (new_len < r.length || new_len > r.reserved) return CACHE_BAD_ARG;
    r.length = new_len;
    for (int g = 0; g < (int)groups_.size(); ++g) {
        int keep_from = first_needed_page(g, new_len);
        int32_t* row = table_row(g, r.slot);
        for (int i = r.first_page[g]; i < keep_from; ++i) {
            if (row[i] >= 0) {
                pools_[g].release(row[i]);
                row[i] = -1;
            }
        }
        r.first_page[g] = std::max(r.first_page[g], keep_from);
    }
    return CACHE_OK;
}

int CacheManager::close(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return CACHE_UNKNOWN;
    Request& r = it->second;
    for (int g = 0; g < (int)groups_.size(); ++g) {
        int32_t* row = table_row(g, r.slot);
        for (int i = 0; i < max_pages_; ++i) {
            if (row[i] >= 0) {
                pools_[g].release(row[i]);
                row[i] = -1;
            }
        }
    }
    free_slots_.push_back(r.slot);
    requests_.erase(it);
    return CACHE_OK;
}

int CacheManager::slot_of(int64_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? CACHE_UNKNOWN : it->second.slot;
}

int CacheManager::length_of(int64_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? CACHE_UNKNOWN : it->second.length;
}

int CacheManager::reserved_of(int64_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? CACHE_UNKNOWN : it->second.reserved;
}

int CacheManager::held_pages(int64_t id, int group) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) return CACHE_UNKNOWN;
    const int32_t* row = tables_[group].data() + (size_t)it->second.slot * max_pages_;
    int n = 0;
    for (int i = 0; i < max_pages_; ++i) n += row[i] >= 0;
    return n;
}

int CacheManager::pages_for_lifetime(int group, int total_len, int max_chunk) const {
    const GroupSpec& g = groups_[group];
    int all = ceil_div(total_len, g.page_size);
    if (g.window <= 0) return all;
    int span = g.window - 1 + std::max(1, max_chunk);
    return std::min(all, ceil_div(span, g.page_size) + 1);
}

int CacheManager::check() const {
    for (int g = 0; g < (int)groups_.size(); ++g) {
        std::vector<int> holders(groups_[g].num_pages, 0);
        for (const auto& kv : requests_) {
            const int32_t* row = tables_[g].data() + (size_t)kv.second.slot * max_pages_;
            for (int i = 0; i < max_pages_; ++i) {
                if (row[i] < 0) continue;
                if (row[i] >= groups_[g].num_pages) return 1;       // a page id out of range
                holders[row[i]]++;
            }
        }
        int held = 0;
        for (int p = 0; p < groups_[g].num_pages; ++p) {
            if (holders[p] > 1) return 2;                           // held twice
            if (holders[p] == 1 && !pools_[g].is_held(p)) return 3; // in a table but marked free
            if (holders[p] == 0 && pools_[g].is_held(p)) return 4;  // lost: held by nobody
            held += holders[p];
        }
        if (held + pools_[g].free_count() != groups_[g].num_pages) return 5;
        // rows of slots that no request owns must be empty
        std::vector<uint8_t> owned(max_requests_, 0);
        for (const auto& kv : requests_) owned[kv.second.slot] = 1;
        for (int s = 0; s < max_requests_; ++s) {
            if (owned[s]) continue;
            const int32_t* row = tables_[g].data() + (size_t)s * max_pages_;
            for (int i = 0; i < max_pages_; ++i)
                if (row[i] >= 0) return 6;
        }
    }
    if ((int)requests_.size() + (int)free_slots_.size() != max_requests_) return 7;
    return 0;
}

}  // namespace carbon
