// Host-side cache manager: paged key/value storage with a block table per request, and slots for
// per-request state of fixed size.
//
// The reference keeps one slot per token (page size 1) in a free list that hands out low ids
// first (src/kvcache/allocator.rs:4-44) and sends every sequence's full slot list to the device
// each step (src/batch.rs:21-23).  Here tokens live in pages of page_size tokens; a request owns
// one row of a block table per group of layers, and token p lives at
// (table[p / page_size], p % page_size).  Layers with different needs form different groups with
// pools of their own: a group that keeps all keys, or a group that keeps a window of them and
// gives pages back once the window has passed them.  Requests also own one state slot
// (src/batch.rs:18-20, src/scheduler.rs:373-379) that indexes per-request storage of fixed size.
#pragma once
#include <cstdint>
#include <unordered_map>
#include <vector>

namespace carbon {

struct GroupSpec {
    int page_size;
    int num_pages;
    int window;  // 0: all keys are kept; w > 0: a query at position p reads keys p-w+1 .. p
};

// A pool of page ids with ownership tracking: a page is either free or held by exactly one owner.
class PagePool {
  public:
    explicit PagePool(int num_pages);
    int acquire();              // a free page id (lowest first), or -1
    bool release(int page);     // false if the page was not held (double free or bad id)
    int free_count() const { return (int)free_.size(); }
    int size() const { return (int)held_.size(); }
    bool is_held(int page) const { return page >= 0 && page < (int)held_.size() && held_[page]; }

  private:
    std::vector<int> free_;     // a min-heap, so low ids go out first
    std::vector<uint8_t> held_;
};

enum CacheStatus {
    CACHE_OK = 0,
    CACHE_NO_SLOT = -1,         // every state slot is taken
    CACHE_DUPLICATE = -2,       // the request id is already open
    CACHE_UNKNOWN = -3,         // no such request
    CACHE_NO_PAGES = -4,        // a pool ran out; nothing was changed
    CACHE_TOO_LONG = -5,        // more pages than a table row holds
    CACHE_BAD_ARG = -6,
};

class CacheManager {
  public:
    CacheManager(const std::vector<GroupSpec>& groups, int max_requests, int max_pages_per_request);

    int open(int64_t id);                       // -> state slot >= 0, or a CacheStatus error
    int reserve(int64_t id, int new_len);       // pages for positions < new_len in every group
    int commit(int64_t id, int new_len);        // positions < new_len are written; windows move on
    int close(int64_t id);                      // everything the request holds goes back

    int slot_of(int64_t id) const;
    int length_of(int64_t id) const;
    int reserved_of(int64_t id) const;
    int num_groups() const { return (int)groups_.size(); }
    int free_pages(int group) const { return pools_[group].free_count(); }
    int held_pages(int64_t id, int group) const;
    int open_requests() const { return (int)requests_.size(); }
    int free_slots() const { return (int)free_slots_.size(); }
    int max_requests() const { return max_requests_; }
    int max_pages_per_request() const { return max_pages_; }
    const GroupSpec& group(int g) const { return groups_[g]; }

    // Pages a request of total_len tokens, fed at most max_chunk tokens per step, can hold at once.
    int pages_for_lifetime(int group, int total_len, int max_chunk) const;
    // Pages reserve(id, new_len) would newly take from the group's pool.
    int pages_to_reserve(int64_t id, int group, int new_len) const;

    // Block table of a group: int32 [max_requests, max_pages_per_request], -1 where no page is held.
    const int32_t* table(int group) const { return tables_[group].data(); }
    int32_t* table_row(int group, int slot) { return tables_[group].data() + (size_t)slot * max_pages_; }

    // Internal consistency: every page is free or held by exactly one table entry.  Returns 0 if so.
    int check() const;

  private:
    struct Request {
        int slot;
        int length;                       // committed tokens
        int reserved;                     // positions < reserved have pages
        std::vector<int> first_page;      // per group: first table index still held
    };
    std::vector<GroupSpec> groups_;
    std::vector<PagePool> pools_;
    std::vector<std::vector<int32_t>> tables_;
    std::vector<int> free_slots_;
    std::unordered_map<int64_t, Request> requests_;
    int max_requests_, max_pages_;

    int first_needed_page(int group, int length) const;
};

}  // namespace carbon
