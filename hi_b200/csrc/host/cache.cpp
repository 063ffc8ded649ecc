// The cache manager on the host: pages, block tables, state slots. No device code.
//
// Layer groups with different needs (every earlier key, or a window of them) have pools of
// their own; a request has one block table per group, indexed by position / page_size. Pages
// go back to their pool when the request ends or when the window has passed them, and are
// handed out again (the reference allocates everything at admission and frees only at
// retirement: crates/hi-cuda/src/lib.rs:641-957, 4781-4844).
#include "cache.h"

#include <algorithm>
#include <set>

namespace hbh {

PagePool::PagePool(int num_pages) : total_(num_pages), held_(num_pages, 0), owner_(num_pages, 0) {
  for (int p = 0; p < num_pages; ++p) free_.push_back(p);
}

int PagePool::take(int64_t owner, int* page) {
  if (free_.empty()) {
    ++failed_allocations;
    return HBH_ERR_NO_PAGES;
  }
  const int p = free_.front();
  free_.pop_front();
  held_[p] = 1;
  owner_[p] = owner;
  ++allocations;
  peak_used = std::max<int64_t>(peak_used, used());
  *page = p;
  return HBH_OK;
}

int PagePool::give(int page, int64_t owner) {
  if (page < 0 || page >= total_) return HBH_ERR_BAD_PAGE;
  if (!held_[page]) return HBH_ERR_DOUBLE_FREE;
  if (owner_[page] != owner) return HBH_ERR_NOT_OWNER;
  held_[page] = 0;
  free_.push_back(page);          // back of the list; it comes round again
  return HBH_OK;
}

CacheManager::CacheManager(int n_groups, const int* window_kind, const int64_t* window_size, const int* pages,
                           int page_size, int max_requests)
    : page_size_(page_size), max_requests_(max_requests) {
  for (int g = 0; g < n_groups; ++g) {
    Window w;
    w.kind = window_kind[g];
    w.size = window_size[g];
    windows_.push_back(w);
    pools_.emplace_back(pages[g]);
  }
  for (int s = 0; s < max_requests; ++s) free_slots_.push_back(s);
}

RequestCache* CacheManager::find(int64_t request) {
  auto it = requests_.find(request);
  return it == requests_.end() ? nullptr : &it->second;
}

int CacheManager::open(int64_t request, int* slot) {
  if (is_open(request)) return HBH_ERR_ALREADY_OPEN;
  if (free_slots_.empty()) return HBH_ERR_NO_SLOT;
  RequestCache rc;
  rc.slot = free_slots_.front();
  free_slots_.pop_front();
  rc.tables.resize(windows_.size());
  rc.version = ++versions_;
  *slot = rc.slot;
  requests_.emplace(request, std::move(rc));
  return HBH_OK;
}

int CacheManager::close(int64_t request) {
  auto it = requests_.find(request);
  if (it == requests_.end()) return HBH_ERR_NOT_OPEN;
  int rc = HBH_OK;
  for (size_t g = 0; g < it->second.tables.size(); ++g)
    for (int page : it->second.tables[g])
      if (page != HBH_FREED) {
        const int r = pools_[g].give(page, request);
        if (r != HBH_OK) rc = r;
      }
  free_slots_.push_back(it->second.slot);
  requests_.erase(it);
  return rc;
}

void CacheManager::pages_needed(int64_t request, int n_new, int64_t length, int* out) {
  const RequestCache* rc = request >= 0 ? find(request) : nullptr;
  if (rc) length = rc->length;
  const int64_t need_blocks = blocks_for(length, n_new);
  for (size_t g = 0; g < windows_.size(); ++g) {
    const int64_t have = rc ? (int64_t)rc->tables[g].size() : 0;
    // blocks wholly before the window of the first new token are never read
    const int64_t first_live = windows_[g].first_live(length) / page_size_;
    out[g] = (int)std::max<int64_t>(0, need_blocks - std::max(have, first_live));
  }
}

void CacheManager::peak_pages_needed(int64_t request, int64_t n_new, int64_t length, int* out) {
  const RequestCache* rc = request >= 0 ? find(request) : nullptr;
  if (rc) length = rc->length;
  const int64_t need_blocks = (length + n_new + page_size_ - 1) / page_size_;
  for (size_t g = 0; g < windows_.size(); ++g) {
    const int64_t have = rc ? (int64_t)rc->tables[g].size() : 0;
    const int64_t first_live = windows_[g].first_live(length) / page_size_;
    int64_t need = std::max<int64_t>(0, need_blocks - std::max(have, first_live));
    if (windows_[g].kind != HBH_WINDOW_NONE) {
      int64_t held = 0;
      if (rc)
        for (int page : rc->tables[g]) held += page != HBH_FREED;
      const int64_t most = (windows_[g].size + page_size_ - 1) / page_size_ + 1;
      need = std::min(need, std::max<int64_t>(0, most - held));
    }
    out[g] = (int)need;
  }
}

bool CacheManager::fits(int64_t request, int n_new, int64_t length, const int* promised) {
  std::vector<int> need(windows_.size());
  pages_needed(request, n_new, length, need.data());
  for (size_t g = 0; g < windows_.size(); ++g)
    if ((promised ? promised[g] : 0) + need[g] > pools_[g].free_pages()) return false;
  return true;
}

int CacheManager::reserve(int64_t request, int n_new, int* fail) {
  RequestCache* rc = find(request);
  if (!rc) return HBH_ERR_NOT_OPEN;
  std::vector<int> need(windows_.size());
  pages_needed(request, n_new, 0, need.data());
  for (size_t g = 0; g < windows_.size(); ++g)
    if (need[g] > pools_[g].free_pages()) {
      ++pools_[g].failed_allocations;
      if (fail) {
        fail[0] = (int)g; fail[1] = need[g]; fail[2] = pools_[g].free_pages(); fail[3] = pools_[g].total();
      }
      return HBH_ERR_NO_PAGES;
    }
  const int64_t need_blocks = blocks_for(rc->length, n_new);
  for (size_t g = 0; g < windows_.size(); ++g) {
    std::vector<int>& table = rc->tables[g];
    const int64_t first_live = windows_[g].first_live(rc->length) / page_size_;
    if ((int64_t)table.size() < need_blocks) rc->version = ++versions_;
    while ((int64_t)table.size() < need_blocks) {
      int page = HBH_FREED;
      if ((int64_t)table.size() >= first_live) {
        const int r = pools_[g].take(request, &page);
        if (r != HBH_OK) return r;      // cannot happen: the need was checked against the pool above
      }
      table.push_back(page);
    }
  }
  return HBH_OK;
}

int CacheManager::unreserve(int64_t request, const int* table_lengths) {
  RequestCache* rc = find(request);
  if (!rc) return HBH_ERR_NOT_OPEN;
  int out = HBH_OK;
  for (size_t g = 0; g < windows_.size(); ++g) {
    std::vector<int>& table = rc->tables[g];
    if (table_lengths[g] < 0 || (size_t)table_lengths[g] > table.size()) return HBH_ERR_ARG;
    if ((size_t)table_lengths[g] < table.size()) rc->version = ++versions_;
    while (table.size() > (size_t)table_lengths[g]) {
      if (table.back() != HBH_FREED) {
        const int r = pools_[g].give(table.back(), request);
        if (r != HBH_OK) out = r;
      }
      table.pop_back();
    }
  }
  return out;
}

int CacheManager::commit(int64_t request, int n_new) {
  RequestCache* rc = find(request);
  if (!rc) return HBH_ERR_NOT_OPEN;
  rc->length += n_new;
  returned.clear();
  for (size_t g = 0; g < windows_.size(); ++g) {
    const int64_t dead_blocks = windows_[g].first_live(rc->length) / page_size_;
    std::vector<int>& table = rc->tables[g];
    const int64_t upto = std::min<int64_t>(dead_blocks, (int64_t)table.size());
    for (int64_t b = 0; b < upto; ++b)
      if (table[b] != HBH_FREED) {
        const int r = pools_[g].give(table[b], request);
        if (r != HBH_OK) return r;
        returned.push_back((int)g);
        returned.push_back(table[b]);
        table[b] = HBH_FREED;
        rc->version = ++versions_;
      }
  }
  return (int)returned.size() / 2;
}

// No page lost, held twice or free while held; no slot lost or held twice.
int CacheManager::check() {
  for (size_t g = 0; g < pools_.size(); ++g) {
    PagePool& pool = pools_[g];
    std::unordered_map<int, int64_t> held;
    for (const auto& kv : requests_)
      for (int page : kv.second.tables[g]) {
        if (page == HBH_FREED) continue;
        if (held.count(page)) {
          error = "group " + std::to_string(g) + ": page " + std::to_string(page) + " held by two requests";
          return HBH_ERR_INVARIANT;
        }
        held[page] = kv.first;
        if (page < 0 || page >= pool.total() || !pool.held(page) || pool.owner(page) != kv.first) {
          error = "group " + std::to_string(g) + ": page " + std::to_string(page) + " owner mismatch";
          return HBH_ERR_INVARIANT;
        }
      }
    std::set<int> free_set(pool.free_list().begin(), pool.free_list().end());
    if (free_set.size() != pool.free_list().size()) {
      error = "group " + std::to_string(g) + ": a page is on the free list twice";
      return HBH_ERR_INVARIANT;
    }
    for (const auto& kv : held)
      if (free_set.count(kv.first)) {
        error = "group " + std::to_string(g) + ": a held page is on the free list";
        return HBH_ERR_INVARIANT;
      }
    if ((int)(free_set.size() + held.size()) != pool.total()) {
      error = "group " + std::to_string(g) + ": " + std::to_string(pool.total() - (int)free_set.size() - (int)held.size()) +
              " page(s) lost";
      return HBH_ERR_INVARIANT;
    }
  }
  std::set<int> slots(free_slots_.begin(), free_slots_.end());
  size_t taken = 0;
  for (const auto& kv : requests_) {
    if (!slots.insert(kv.second.slot).second) {
      error = "a state slot is held twice";
      return HBH_ERR_INVARIANT;
    }
    ++taken;
  }
  if (slots.size() != (size_t)max_requests_ || free_slots_.size() + taken != (size_t)max_requests_) {
    error = "a state slot is lost";
    return HBH_ERR_INVARIANT;
  }
  return HBH_OK;
}

}  // namespace hbh

// ---------------------------------------------------------------------------- C interface
using hbh::CacheManager;
using hbh::PagePool;

extern "C" {

void* hbh_pool_create(int num_pages) { return num_pages > 0 ? new PagePool(num_pages) : nullptr; }
void hbh_pool_destroy(void* pool) { delete static_cast<PagePool*>(pool); }
int hbh_pool_take(void* pool, int64_t owner, int* page) { return static_cast<PagePool*>(pool)->take(owner, page); }
int hbh_pool_give(void* pool, int page, int64_t owner) { return static_cast<PagePool*>(pool)->give(page, owner); }
int hbh_pool_owner(void* pool, int page, int64_t* owner, int* held) {
  PagePool* p = static_cast<PagePool*>(pool);
  if (page < 0 || page >= p->total()) return HBH_ERR_BAD_PAGE;
  *owner = p->owner(page);
  *held = p->held(page) ? 1 : 0;
  return HBH_OK;
}
int64_t hbh_pool_stat(void* pool, int what) {
  PagePool* p = static_cast<PagePool*>(pool);
  switch (what) {
    case 0: return p->total();
    case 1: return p->free_pages();
    case 2: return p->used();
    case 3: return p->peak_used;
    case 4: return p->allocations;
    case 5: return p->failed_allocations;
  }
  return HBH_ERR_ARG;
}

void* hbh_cache_create(int n_groups, const int* window_kind, const int64_t* window_size, const int* pages,
                       int page_size, int max_requests) {
  if (n_groups < 0 || page_size <= 0 || max_requests < 0) return nullptr;
  for (int g = 0; g < n_groups; ++g) {
    if (pages[g] <= 0) return nullptr;
    if (window_kind[g] != HBH_WINDOW_NONE && window_kind[g] != HBH_WINDOW_CHUNK && window_kind[g] != HBH_WINDOW_SLIDING)
      return nullptr;
    if (window_kind[g] != HBH_WINDOW_NONE && window_size[g] <= 0) return nullptr;
  }
  return new CacheManager(n_groups, window_kind, window_size, pages, page_size, max_requests);
}
void hbh_cache_destroy(void* cache) { delete static_cast<CacheManager*>(cache); }
const char* hbh_cache_error(void* cache) { return static_cast<CacheManager*>(cache)->error.c_str(); }
void* hbh_cache_pool(void* cache, int group) {
  CacheManager* c = static_cast<CacheManager*>(cache);
  return group >= 0 && group < c->n_groups() ? &c->pool(group) : nullptr;
}
int hbh_cache_open(void* cache, int64_t request, int* slot) { return static_cast<CacheManager*>(cache)->open(request, slot); }
int hbh_cache_close(void* cache, int64_t request) { return static_cast<CacheManager*>(cache)->close(request); }
int hbh_cache_is_open(void* cache, int64_t request) { return static_cast<CacheManager*>(cache)->is_open(request) ? 1 : 0; }
int hbh_cache_free_slots(void* cache) { return static_cast<CacheManager*>(cache)->free_slots(); }
int hbh_cache_open_requests(void* cache, int64_t* out, int cap) {
  CacheManager* c = static_cast<CacheManager*>(cache);
  int n = 0;
  for (const auto& kv : c->requests()) {
    if (out && n < cap) out[n] = kv.first;
    ++n;
  }
  return n;
}
int64_t hbh_cache_request_stat(void* cache, int64_t request, int what) {
  hbh::RequestCache* rc = static_cast<CacheManager*>(cache)->find(request);
  if (!rc) return HBH_ERR_NOT_OPEN;
  switch (what) {
    case 0: return rc->slot;
    case 1: return rc->length;
    case 2: return rc->version;
  }
  return HBH_ERR_ARG;
}
int hbh_cache_pages_needed(void* cache, int64_t request, int n_new, int64_t length, int* out) {
  static_cast<CacheManager*>(cache)->pages_needed(request, n_new, length, out);
  return HBH_OK;
}
int hbh_cache_reserve(void* cache, int64_t request, int n_new, int* fail) {
  return static_cast<CacheManager*>(cache)->reserve(request, n_new, fail);
}
int hbh_cache_unreserve(void* cache, int64_t request, const int* table_lengths) {
  return static_cast<CacheManager*>(cache)->unreserve(request, table_lengths);
}
int hbh_cache_commit(void* cache, int64_t request, int n_new) {
  return static_cast<CacheManager*>(cache)->commit(request, n_new);
}
int hbh_cache_returned(void* cache, int* out, int cap) {
  const std::vector<int>& r = static_cast<CacheManager*>(cache)->returned;
  if ((int)r.size() > 2 * cap) return HBH_ERR_CAPACITY;
  std::copy(r.begin(), r.end(), out);
  return (int)r.size() / 2;
}
int hbh_cache_table_length(void* cache, int group, int64_t request) {
  CacheManager* c = static_cast<CacheManager*>(cache);
  hbh::RequestCache* rc = c->find(request);
  if (!rc) return HBH_ERR_NOT_OPEN;
  if (group < 0 || group >= c->n_groups()) return HBH_ERR_ARG;
  return (int)rc->tables[group].size();
}
int hbh_cache_table(void* cache, int group, int64_t request, int* out, int cap) {
  CacheManager* c = static_cast<CacheManager*>(cache);
  hbh::RequestCache* rc = c->find(request);
  if (!rc) return HBH_ERR_NOT_OPEN;
  if (group < 0 || group >= c->n_groups()) return HBH_ERR_ARG;
  const std::vector<int>& t = rc->tables[group];
  if ((int)t.size() > cap) return HBH_ERR_CAPACITY;
  std::copy(t.begin(), t.end(), out);
  return (int)t.size();
}
int hbh_cache_check(void* cache) { return static_cast<CacheManager*>(cache)->check(); }

int hbh_step_widths(void* cache, int n_seqs, const int64_t* requests, int* widths) {
  CacheManager* c = static_cast<CacheManager*>(cache);
  for (int g = 0; g < c->n_groups(); ++g) widths[g] = 0;
  for (int s = 0; s < n_seqs; ++s) {
    hbh::RequestCache* rc = c->find(requests[s]);
    if (!rc) return HBH_ERR_NOT_OPEN;
    for (int g = 0; g < c->n_groups(); ++g) widths[g] = std::max(widths[g], (int)rc->tables[g].size());
  }
  return HBH_OK;
}

int hbh_pack_step(void* cache, int n_seqs, const int64_t* requests, const int* n_new, const int* tokens,
                  const int* want_counts, const int* want, const int* widths, const int64_t* offsets, int* buf,
                  int* start_pos, int* slots, int64_t* row_request, int64_t* row_version) {
  CacheManager* c = static_cast<CacheManager*>(cache);
  int* tok = buf + offsets[0];
  int* pos = buf + offsets[1];
  int* seq = buf + offsets[2];
  int* cu = buf + offsets[3];
  int* slot = buf + offsets[4];
  int* wanted = buf + offsets[5];
  int cursor = 0, want_cursor = 0;
  cu[0] = 0;
  for (int s = 0; s < n_seqs; ++s) {
    hbh::RequestCache* rc = c->find(requests[s]);
    if (!rc) return HBH_ERR_NOT_OPEN;
    const int n = n_new[s];
    for (int i = 0; i < n; ++i) {
      tok[cursor + i] = tokens[cursor + i];
      pos[cursor + i] = (int)(rc->length + i);
      seq[cursor + i] = s;
    }
    for (int w = 0; w < want_counts[s]; ++w) wanted[want_cursor + w] = cursor + want[want_cursor + w];
    want_cursor += want_counts[s];
    cursor += n;
    cu[s + 1] = cursor;
    slot[s] = rc->slot;
    start_pos[s] = (int)rc->length;
    slots[s] = rc->slot;
    // a row is rewritten only when another request sits in it or the request's tables changed
    const bool fresh = !row_request || row_request[s] != requests[s] || row_version[s] != rc->version;
    if (row_request) {
      row_request[s] = requests[s];
      row_version[s] = rc->version;
    }
    if (!fresh) continue;
    for (int g = 0; g < c->n_groups(); ++g) {
      const std::vector<int>& t = rc->tables[g];
      const int w = widths[g];
      if ((int)t.size() > w) return HBH_ERR_CAPACITY;
      int* row = buf + offsets[6 + g] + (int64_t)s * w;
      std::copy(t.begin(), t.end(), row);
      std::fill(row + t.size(), row + w, -1);
    }
  }
  return HBH_OK;
}

}  // extern "C"
