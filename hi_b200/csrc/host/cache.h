// The cache manager's classes (host only): page pools, block tables, state slots.
#pragma once
#include <stdint.h>

#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "runtime.h"

namespace hbh {

// Free list of one group. Every page has at most one owner; giving back a page that is not
// held, or not held by that owner, is refused.
class PagePool {
 public:
  explicit PagePool(int num_pages);
  int total() const { return total_; }
  int free_pages() const { return (int)free_.size(); }
  int used() const { return total_ - (int)free_.size(); }
  int take(int64_t owner, int* page);
  int give(int page, int64_t owner);
  bool held(int page) const { return held_[page]; }
  int64_t owner(int page) const { return owner_[page]; }
  const std::deque<int>& free_list() const { return free_; }
  int64_t peak_used = 0, allocations = 0, failed_allocations = 0;

 private:
  int total_;
  std::deque<int> free_;
  std::vector<char> held_;
  std::vector<int64_t> owner_;
};

struct Window {
  int kind = HBH_WINDOW_NONE;
  int64_t size = 0;
  // oldest position a query at `next_position` or later can still read
  int64_t first_live(int64_t next_position) const {
    if (kind == HBH_WINDOW_CHUNK) return (next_position / size) * size;
    if (kind == HBH_WINDOW_SLIDING) return next_position - size + 1 > 0 ? next_position - size + 1 : 0;
    return 0;
  }
};

struct RequestCache {
  int slot = 0;
  int64_t length = 0;                       // tokens whose keys are in the cache
  std::vector<std::vector<int>> tables;     // per group: block -> page or HBH_FREED
  int64_t version = 0;                      // a new value whenever a table changes; no two states of any
                                            // request of a manager ever share one
};

class CacheManager {
 public:
  CacheManager(int n_groups, const int* window_kind, const int64_t* window_size, const int* pages, int page_size,
               int max_requests);
  int n_groups() const { return (int)windows_.size(); }
  int page_size() const { return page_size_; }
  int max_requests() const { return max_requests_; }
  PagePool& pool(int g) { return pools_[g]; }
  const Window& window(int g) const { return windows_[g]; }
  int free_slots() const { return (int)free_slots_.size(); }
  bool is_open(int64_t request) const { return requests_.count(request) != 0; }
  RequestCache* find(int64_t request);
  const std::unordered_map<int64_t, RequestCache>& requests() const { return requests_; }

  int open(int64_t request, int* slot);
  int close(int64_t request);
  void pages_needed(int64_t request, int n_new, int64_t length, int* out);
  // the most new pages the next n_new tokens can need at any one time when they are fed in
  // portions that may be as short as one token: a windowed group never has to hold more than its
  // window and the page being written
  void peak_pages_needed(int64_t request, int64_t n_new, int64_t length, int* out);
  bool fits(int64_t request, int n_new, int64_t length, const int* promised);
  int reserve(int64_t request, int n_new, int* fail);
  int unreserve(int64_t request, const int* table_lengths);
  int commit(int64_t request, int n_new);
  std::vector<int> returned;               // (group, page) pairs that the last commit gave back
  int check();
  std::string error;

 private:
  int64_t blocks_for(int64_t length, int n_new) const { return (length + n_new + page_size_ - 1) / page_size_; }
  int page_size_, max_requests_;
  int64_t versions_ = 0;
  std::vector<Window> windows_;
  std::vector<PagePool> pools_;
  std::deque<int> free_slots_;
  std::unordered_map<int64_t, RequestCache> requests_;
};

}  // namespace hbh
