// The scheduler above the step function: admit, cut prompts into portions under a token budget,
// decode, finish and free. Host only; it decides, the engine runs. It works on counts (prompt
// length, tokens generated, tokens in the cache); the token values stay with the caller.
//
// When pages run out, in this order:
//   1. no new request is admitted; while an older request is still in its prompt a new one is
//      admitted only if the rest of every such prompt and the whole new prompt fit together;
//   2. prompt portions are shrunk to the pages that are free, or wait a step;
//   3. if a DECODE token cannot get its page, or if every running request is in its prompt and
//      none of them can get a page for even one token (no step runs, so no later step would free
//      one), the most recently admitted running request is preempted: its pages and slot go back,
//      and it returns to the head of the waiting queue with prompt + generated tokens as its prompt;
//   4. a request that could never fit is refused when it is added (insufficient_gpu_memory,
//      crates/hi-cuda/src/lib.rs:845-858).
//
// One step may be planned while the step before it still runs: a plan advances `computed` and
// counts a token "in flight" for every entry that samples, so the next plan can already hold that
// request's next decode token (its value then comes from the device, not from the host). Plans
// are committed in the order they were made, at most two are outstanding. A request that ends
// while a later plan already holds an entry of it leaves that entry void: it runs, nobody reads it.
#include <algorithm>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "cache.h"

namespace hbh {

enum Status { WAITING = 0, RUNNING = 1, FINISHED = 2 };
enum Reason { NONE = 0, LENGTH = 1, STOP = 2, ABORTED = 3, NO_MEMORY = 4 };

struct Request {
  int64_t id = 0;
  int64_t prompt_len = 0, output_len = 0, computed = 0, max_tokens = 0, preemptions = 0;
  int64_t in_flight = 0;       // tokens sampled by planned steps that are not committed yet
  int status = WAITING, reason = NONE;
  int64_t pending() const { return prompt_len + output_len + in_flight - computed; }
  bool may_sample_more() const { return output_len + in_flight < max_tokens; }
};

struct Entry {
  Request* request;
  int64_t begin, count;
  bool samples;
  bool last_in_flight;         // its last token is sampled by the step before: the host does not know it yet
  bool is_void = false;        // the request ended (or was dropped) after this entry was planned
};

struct Plan {
  int64_t id = 0;
  std::vector<Entry> entries;
};

class Scheduler {
 public:
  Scheduler(CacheManager* cache, int max_batch_size, int max_active, int max_batched_tokens, int max_prefill_portion,
            int64_t max_model_len)
      : cache_(cache), max_batch_(max_batch_size), max_active_(max_active > 0 ? max_active : max_batch_size),
        budget_(max_batched_tokens), max_portion_(max_prefill_portion), max_model_len_(max_model_len) {}

  int add(int64_t id, int64_t prompt_len, int64_t max_tokens);
  bool abort(int64_t id);
  int assume_running(int64_t id, int64_t computed);
  bool has_work() const { return !waiting_.empty() || !running_.empty(); }
  int plan();
  int commit(int64_t plan_id, const int* stop, int n_stop);
  Request* find(int64_t id) {
    auto it = requests_.find(id);
    return it == requests_.end() ? nullptr : &it->second;
  }
  void forget(int64_t id) {
    Request* r = find(id);
    if (r && r->status == FINISHED) requests_.erase(id);
  }

  std::string error;
  hbh_release_fn release_fn = nullptr;
  void* release_user = nullptr;
  std::deque<Request*> waiting_;
  std::vector<Request*> running_;          // in admission order
  std::vector<Entry> entries_;             // the plan being made / made last
  std::deque<Plan> outstanding_;           // planned, not committed yet (oldest first; at most two)
  int64_t last_plan_id = 0, current_plan_id = 0;   // ids start at 1; an empty plan has id 0 and is not kept
  std::vector<int64_t> preempted_, dropped_, finished_;   // of the last plan / the last commit (finished: id, reason)
  int64_t admitted = 0, preemptions = 0, steps = 0, shrunk = 0, stalled = 0;

 private:
  int max_active() const { return std::min(max_active_, cache_->max_requests()); }
  void release(int64_t id) {
    if (release_fn) release_fn(release_user, id);
    else if (cache_->is_open(id)) cache_->close(id);
  }
  void finish(Request* r, int reason) {
    r->status = FINISHED;
    r->reason = reason;
    running_.erase(std::remove(running_.begin(), running_.end(), r), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), r), waiting_.end());
    for (Plan& p : outstanding_)           // what later plans hold of it runs for nobody
      for (Entry& e : p.entries)
        if (e.request == r) e.is_void = true;
    release(r->id);
  }
  Entry make_entry(Request* r, int64_t count) const {
    const int64_t known = r->prompt_len + r->output_len;                 // tokens whose values the host has
    const bool samples = r->computed + count == known + r->in_flight;
    return Entry{r, r->computed, count, samples, r->computed + count > known};
  }
  void needed(const Request* r, int64_t n, std::vector<int>& out) const {
    // an open request is measured from its tables; one not yet in the cache from `computed`
    cache_->pages_needed(r->id, (int)n, r->computed, out.data());
  }
  bool fits(const Request* r, int64_t n, const std::vector<int>& promised) const {
    std::vector<int> need(promised.size());
    needed(r, n, need);
    for (size_t g = 0; g < need.size(); ++g)
      if (promised[g] + need[g] > cache_->pool((int)g).free_pages()) return false;
    return true;
  }
  void promise(const Request* r, int64_t n, std::vector<int>& promised) const {
    std::vector<int> need(promised.size());
    needed(r, n, need);
    for (size_t g = 0; g < need.size(); ++g) promised[g] += need[g];
  }
  int64_t largest_fit(const Request* r, int64_t n, const std::vector<int>& promised) const {
    if (fits(r, n, promised)) return n;
    int64_t lo = 0, hi = n;          // lo fits (0 tokens need nothing), hi does not
    while (hi - lo > 1) {
      const int64_t mid = (lo + hi) / 2;
      if (fits(r, mid, promised)) lo = mid; else hi = mid;
    }
    return lo;
  }
  int64_t planned_tokens() const {
    int64_t n = 0;
    for (const Entry& e : entries_) n += e.count;
    return n;
  }
  // pages the rest of r's tokens still needs after the first `planned` of them, fed in portions
  void add_later_need(const Request* r, int64_t planned, std::vector<int>& later) const {
    std::vector<int> all(later.size()), now(later.size());
    cache_->peak_pages_needed(r->id, r->pending(), r->computed, all.data());
    needed(r, planned, now);
    for (size_t g = 0; g < later.size(); ++g) later[g] += std::max(0, all[g] - now[g]);
  }
  void preempt(Request* victim);
  void plan_portion(Request* r, std::vector<int>& promised, int64_t budget);

  CacheManager* cache_;
  int max_batch_, max_active_, budget_, max_portion_;
  int64_t max_model_len_;
  std::unordered_map<int64_t, Request> requests_;
};

int Scheduler::add(int64_t id, int64_t prompt_len, int64_t max_tokens) {
  if (prompt_len <= 0 || max_tokens <= 0) return HBH_ERR_ARG;
  Request* old = find(id);
  if (old && old->status != FINISHED) return HBH_ERR_ALREADY_OPEN;
  const int64_t total = prompt_len + max_tokens;
  if (max_model_len_ > 0 && total > max_model_len_) {
    error = "context_length_exceeded: prompt (" + std::to_string(prompt_len) + ") + max_tokens (" +
            std::to_string(max_tokens) + ") exceeds the model's " + std::to_string(max_model_len_) + " positions";
    return HBH_ERR_CONTEXT_LENGTH;
  }
  const int64_t ps = cache_->page_size();
  for (int g = 0; g < cache_->n_groups(); ++g) {
    int64_t need = (total + ps - 1) / ps;
    const Window& w = cache_->window(g);
    // a windowed group holds at most its window plus the page being written
    if (w.kind != HBH_WINDOW_NONE) need = std::min(need, (w.size + ps - 1) / ps + 1);
    if (need > cache_->pool(g).total()) {
      error = "insufficient_gpu_memory: the request needs " + std::to_string(need) + " page(s) of group " +
              std::to_string(g) + ", the pool has " + std::to_string(cache_->pool(g).total());
      return HBH_ERR_NEVER_FITS;
    }
  }
  Request r;
  r.id = id;
  r.prompt_len = prompt_len;
  r.max_tokens = max_tokens;
  requests_[id] = r;
  waiting_.push_back(&requests_[id]);
  return HBH_OK;
}

bool Scheduler::abort(int64_t id) {
  Request* r = find(id);
  if (!r || r->status == FINISHED) return false;
  finish(r, ABORTED);
  return true;
}

// Benchmarks only: a waiting request whose first `computed` tokens the caller has put into the
// cache by other means starts running from there.
int Scheduler::assume_running(int64_t id, int64_t computed) {
  Request* r = find(id);
  if (!r || r->status != WAITING || computed < 0 || computed >= r->prompt_len + r->output_len) return HBH_ERR_ARG;
  waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), r), waiting_.end());
  r->computed = computed;
  r->status = RUNNING;
  running_.push_back(r);
  ++admitted;
  return HBH_OK;
}

void Scheduler::preempt(Request* victim) {
  running_.erase(std::remove(running_.begin(), running_.end(), victim), running_.end());
  release(victim->id);
  victim->status = WAITING;
  victim->computed = 0;
  ++victim->preemptions;
  ++preemptions;
  waiting_.push_front(victim);
  preempted_.push_back(victim->id);
  entries_.erase(std::remove_if(entries_.begin(), entries_.end(), [&](const Entry& e) { return e.request == victim; }),
                 entries_.end());
}

void Scheduler::plan_portion(Request* r, std::vector<int>& promised, int64_t budget) {
  int64_t want = std::min(r->pending(), budget);
  if (max_portion_ > 0) want = std::min<int64_t>(want, max_portion_);
  const int64_t n = largest_fit(r, want, promised);
  if (n <= 0) {
    ++stalled;
    return;
  }
  if (n < want) ++shrunk;
  promise(r, n, promised);
  entries_.push_back(make_entry(r, n));
}

int Scheduler::plan() {
  if (outstanding_.size() >= 2) {
    error = "two plans are outstanding already: commit the older one first";
    return HBH_ERR_ARG;
  }
  entries_.clear();
  preempted_.clear();
  dropped_.clear();
  int64_t budget = budget_;
  std::vector<int> promised(cache_->n_groups(), 0);

  // 1. every running request that has one token pending decodes, oldest first
  std::vector<Request*> decoding;
  for (Request* r : running_)
    if (r->pending() == 1 && r->computed >= r->prompt_len && r->may_sample_more()) decoding.push_back(r);
  std::vector<Request*> planned;           // requests with a decode entry in this plan
  size_t i = 0;
  while (i < decoding.size() && budget > 0 && (int)entries_.size() < max_batch_) {
    Request* r = decoding[i];
    if (r->status != RUNNING) {            // preempted meanwhile
      ++i;
      continue;
    }
    if (fits(r, 1, promised)) {
      promise(r, 1, promised);
      entries_.push_back(make_entry(r, 1));
      planned.push_back(r);
      --budget;
      ++i;
      continue;
    }
    Request* victim = running_.back();
    if (victim == r && running_.size() == 1) {
      finish(r, NO_MEMORY);
      dropped_.push_back(r->id);
      ++i;
      continue;
    }
    const bool was_planned = std::find(planned.begin(), planned.end(), victim) != planned.end();
    preempt(victim);
    if (was_planned) {
      // the victim's promised pages come back with it
      planned.erase(std::remove(planned.begin(), planned.end(), victim), planned.end());
      std::fill(promised.begin(), promised.end(), 0);
      budget = budget_;
      for (const Entry& e : entries_) {
        promise(e.request, e.count, promised);
        budget -= e.count;
      }
    }
    // try r again (unless it was the victim)
  }

  // 2. running requests still in their prompt get portions, oldest first
  const auto portions = [&]() {
    for (Request* r : std::vector<Request*>(running_)) {
      if (budget <= 0 || (int)entries_.size() >= max_batch_) break;
      if (std::find(planned.begin(), planned.end(), r) != planned.end() || r->pending() <= 0 || !r->may_sample_more())
        continue;                                  // planned, or only waiting for its last sample to be committed
      plan_portion(r, promised, budget);
      budget = budget_ - planned_tokens();
    }
  };
  int64_t stalled_before = stalled;
  portions();
  // every running request waits for a page and no step is in flight whose end could free one:
  // the youngest goes back to the queue until one of the older ones can move
  while (entries_.empty() && stalled > stalled_before && outstanding_.empty() && running_.size() >= 2) {
    preempt(running_.back());
    std::fill(promised.begin(), promised.end(), 0);
    budget = budget_;
    stalled_before = stalled;
    portions();
  }

  // 3. admit waiting requests into what is left
  if (preempted_.empty()) {
    // what the prompts that are under way will still ask for after this step
    std::vector<int> later(cache_->n_groups(), 0);
    bool prompt_under_way = false;
    for (Request* r : running_) {
      int64_t count = 0;
      for (const Entry& e : entries_)
        if (e.request == r) count = e.count;
      if (r->computed + count < r->prompt_len + r->output_len) {
        prompt_under_way = true;
        add_later_need(r, count, later);
      }
    }
    int slots_left = cache_->free_slots();
    while (!waiting_.empty() && budget > 0 && (int)entries_.size() < max_batch_ && (int)running_.size() < max_active() &&
           slots_left > 0) {
      Request* r = waiting_.front();
      if (prompt_under_way) {
        // both have to be able to finish their prompts: else they would fill the pool between
        // them and neither could go on
        std::vector<int> whole(later.size());
        cache_->peak_pages_needed(r->id, r->pending(), r->computed, whole.data());
        bool room = true;
        for (size_t g = 0; g < whole.size(); ++g)
          if (promised[g] + later[g] + whole[g] > cache_->pool((int)g).free_pages()) room = false;
        if (!room) break;
      }
      const size_t before = entries_.size();
      plan_portion(r, promised, budget);
      if (entries_.size() == before) break;          // no page for even one token: wait
      waiting_.pop_front();
      r->status = RUNNING;
      running_.push_back(r);
      ++admitted;
      --slots_left;
      budget = budget_ - planned_tokens();
      const int64_t count = entries_.back().count;
      if (r->computed + count < r->prompt_len + r->output_len) {
        prompt_under_way = true;
        add_later_need(r, count, later);
      }
    }
  }
  // the plan is taken as carried out: its tokens count as computed, its samples as in flight
  for (const Entry& e : entries_) {
    e.request->computed += e.count;
    if (e.samples) ++e.request->in_flight;
  }
  ++steps;
  if (entries_.empty()) {                  // nothing to run, nothing to commit
    current_plan_id = 0;
    return HBH_OK;
  }
  Plan p;
  p.id = current_plan_id = ++last_plan_id;
  p.entries = entries_;
  outstanding_.push_back(std::move(p));
  return HBH_OK;
}

int Scheduler::commit(int64_t plan_id, const int* stop, int n_stop) {
  if (outstanding_.empty() || outstanding_.front().id != plan_id) {
    error = "plans are committed in the order they were made";
    return HBH_ERR_ARG;
  }
  finished_.clear();
  Plan plan = std::move(outstanding_.front());
  outstanding_.pop_front();
  int s = 0;
  for (const Entry& e : plan.entries) {
    if (!e.samples) continue;
    if (s >= n_stop) return HBH_ERR_ARG;
    const bool stops = stop[s++] != 0;
    if (e.is_void) continue;               // the request ended before this entry's sample was read
    Request* r = e.request;
    --r->in_flight;
    int reason = NONE;
    if (stops) {
      reason = STOP;                       // the ending token is not emitted (crates/hi-mlx/src/models.rs:598-600)
    } else {
      ++r->output_len;
      if (r->output_len >= r->max_tokens) reason = LENGTH;
    }
    if (reason != NONE) {
      finish(r, reason);
      finished_.push_back(r->id);
      finished_.push_back(reason);
    }
  }
  return HBH_OK;
}

}  // namespace hbh

using hbh::Scheduler;

extern "C" {

void* hbh_sched_create(void* cache, int max_batch_size, int max_active, int max_batched_tokens,
                       int max_prefill_portion, int64_t max_model_len) {
  if (!cache || max_batch_size < 1 || max_batched_tokens < 1) return nullptr;
  return new Scheduler(static_cast<hbh::CacheManager*>(cache), max_batch_size, max_active, max_batched_tokens,
                       max_prefill_portion, max_model_len);
}
void hbh_sched_destroy(void* sched) { delete static_cast<Scheduler*>(sched); }
const char* hbh_sched_error(void* sched) { return static_cast<Scheduler*>(sched)->error.c_str(); }
void hbh_sched_set_release(void* sched, hbh_release_fn fn, void* user) {
  Scheduler* s = static_cast<Scheduler*>(sched);
  s->release_fn = fn;
  s->release_user = user;
}
int hbh_sched_add(void* sched, int64_t request, int prompt_len, int max_tokens) {
  return static_cast<Scheduler*>(sched)->add(request, prompt_len, max_tokens);
}
int hbh_sched_abort(void* sched, int64_t request) { return static_cast<Scheduler*>(sched)->abort(request) ? 1 : 0; }
int hbh_sched_assume_running(void* sched, int64_t request, int64_t computed) {
  return static_cast<Scheduler*>(sched)->assume_running(request, computed);
}
int hbh_sched_has_work(void* sched) { return static_cast<Scheduler*>(sched)->has_work() ? 1 : 0; }

int hbh_sched_plan(void* sched, int64_t* plan_id, int64_t* entries, int cap_entries, int* n_entries, int64_t* preempted,
                   int cap_preempted, int* n_preempted, int64_t* dropped, int cap_dropped, int* n_dropped) {
  Scheduler* s = static_cast<Scheduler*>(sched);
  const int rc = s->plan();
  if (rc != HBH_OK) return rc;
  *plan_id = s->current_plan_id;
  *n_entries = (int)s->entries_.size();
  *n_preempted = (int)s->preempted_.size();
  *n_dropped = (int)s->dropped_.size();
  if (*n_entries > cap_entries || *n_preempted > cap_preempted || *n_dropped > cap_dropped) return HBH_ERR_CAPACITY;
  for (int i = 0; i < *n_entries; ++i) {
    const hbh::Entry& e = s->entries_[i];
    entries[5 * i] = e.request->id;
    entries[5 * i + 1] = e.begin;
    entries[5 * i + 2] = e.count;
    entries[5 * i + 3] = e.samples ? 1 : 0;
    entries[5 * i + 4] = e.last_in_flight ? 1 : 0;
  }
  std::copy(s->preempted_.begin(), s->preempted_.end(), preempted);
  std::copy(s->dropped_.begin(), s->dropped_.end(), dropped);
  return HBH_OK;
}

int hbh_sched_commit(void* sched, int64_t plan_id, const int* stop, int n_stop, int64_t* finished, int cap,
                     int* n_finished) {
  Scheduler* s = static_cast<Scheduler*>(sched);
  const int r = s->commit(plan_id, stop, n_stop);
  if (r != HBH_OK) return r;
  *n_finished = (int)s->finished_.size() / 2;
  if (*n_finished > cap) return HBH_ERR_CAPACITY;
  std::copy(s->finished_.begin(), s->finished_.end(), finished);
  return HBH_OK;
}

int64_t hbh_sched_request_stat(void* sched, int64_t request, int what) {
  hbh::Request* r = static_cast<Scheduler*>(sched)->find(request);
  if (!r) return HBH_ERR_NOT_OPEN;
  switch (what) {
    case 0: return r->status;
    case 1: return r->computed;
    case 2: return r->preemptions;
    case 3: return r->output_len;
    case 4: return r->reason;
    case 5: return r->in_flight;
  }
  return HBH_ERR_ARG;
}

int hbh_sched_queue(void* sched, int which, int64_t* out, int cap) {
  Scheduler* s = static_cast<Scheduler*>(sched);
  int n = 0;
  if (which == 0) {
    for (hbh::Request* r : s->waiting_) {
      if (out && n < cap) out[n] = r->id;
      ++n;
    }
  } else {
    for (hbh::Request* r : s->running_) {
      if (out && n < cap) out[n] = r->id;
      ++n;
    }
  }
  return n;
}

int64_t hbh_sched_counter(void* sched, int what) {
  Scheduler* s = static_cast<Scheduler*>(sched);
  switch (what) {
    case 0: return s->admitted;
    case 1: return s->preemptions;
    case 2: return s->steps;
    case 3: return s->shrunk;
    case 4: return s->stalled;
  }
  return HBH_ERR_ARG;
}

void hbh_sched_forget(void* sched, int64_t request) { static_cast<Scheduler*>(sched)->forget(request); }

}  // extern "C"
