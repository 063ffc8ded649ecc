// C interface of the host runtime (no CUDA in here): the cache manager (page pools, block
// tables, state slots), the packing of a step's integer inputs, and the scheduler. Python
// loads the library with ctypes; every function returns HBH_OK or a negative code, and
// hbh_*_error() gives the last failure of an object in words.
//
// Compared with the reference (crates/hi-cuda/src/lib.rs:641-957 page leases, 4418-4471 and
// 5062-5298 the continuous loop): that engine leases all pages of a request at admission and
// runs prefill chunks and decode rows as separate forwards; this one takes pages step by step,
// gives windowed pages back as the window passes them, and plans decode tokens and prompt
// portions into ONE batch.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HBH_OK 0
#define HBH_ERR_ARG (-1)
#define HBH_ERR_NOT_OPEN (-2)
#define HBH_ERR_ALREADY_OPEN (-3)
#define HBH_ERR_NO_SLOT (-4)
#define HBH_ERR_NO_PAGES (-5)        // insufficient_gpu_memory (crates/hi-cuda/src/lib.rs:845-858)
#define HBH_ERR_BAD_PAGE (-6)
#define HBH_ERR_DOUBLE_FREE (-7)
#define HBH_ERR_NOT_OWNER (-8)
#define HBH_ERR_INVARIANT (-9)
#define HBH_ERR_CONTEXT_LENGTH (-10)
#define HBH_ERR_NEVER_FITS (-11)
#define HBH_ERR_CAPACITY (-12)       // an output array of the caller is too small

#define HBH_FREED (-1)               // a block whose page was given back (the window has passed it)
#define HBH_WINDOW_NONE 0            // every earlier key
#define HBH_WINDOW_CHUNK 1           // keys of the query's own block of `size` positions
#define HBH_WINDOW_SLIDING 2         // the last `size` keys

// ---- one pool of pages (the cache manager has one per layer group)
void* hbh_pool_create(int num_pages);
void hbh_pool_destroy(void* pool);
int hbh_pool_take(void* pool, int64_t owner, int* page);
int hbh_pool_give(void* pool, int page, int64_t owner);
int hbh_pool_owner(void* pool, int page, int64_t* owner, int* held);
// what: 0 total, 1 free, 2 used, 3 peak used, 4 allocations, 5 failed allocations
int64_t hbh_pool_stat(void* pool, int what);

// ---- the cache manager
void* hbh_cache_create(int n_groups, const int* window_kind, const int64_t* window_size, const int* pages,
                       int page_size, int max_requests);
void hbh_cache_destroy(void* cache);
const char* hbh_cache_error(void* cache);
void* hbh_cache_pool(void* cache, int group);                 // borrowed; lives as long as the cache
int hbh_cache_open(void* cache, int64_t request, int* slot);
int hbh_cache_close(void* cache, int64_t request);
int hbh_cache_is_open(void* cache, int64_t request);
int hbh_cache_free_slots(void* cache);
int hbh_cache_open_requests(void* cache, int64_t* out, int cap);       // returns the count
// what: 0 slot, 1 length, 2 table version
int64_t hbh_cache_request_stat(void* cache, int64_t request, int what);
// new pages per group for the next n_new tokens of an open request, or (request < 0 or not
// open) of a request that would start at `length`
int hbh_cache_pages_needed(void* cache, int64_t request, int n_new, int64_t length, int* out);
// pages for positions length .. length + n_new - 1 in every group, or none at all; on
// HBH_ERR_NO_PAGES fail[4] = group, needed, free, total
int hbh_cache_reserve(void* cache, int64_t request, int n_new, int* fail);
// take back what reserve() added: the tables shrink to table_lengths[group], their pages return
int hbh_cache_unreserve(void* cache, int64_t request, const int* table_lengths);
// the step ran: the request is n_new tokens longer; pages the window has passed go back;
// returns their number, and hbh_cache_returned() lists them as (group, page) pairs
int hbh_cache_commit(void* cache, int64_t request, int n_new);
int hbh_cache_returned(void* cache, int* out, int cap);
int hbh_cache_table_length(void* cache, int group, int64_t request);
int hbh_cache_table(void* cache, int group, int64_t request, int* out, int cap);   // returns the length
int hbh_cache_check(void* cache);                              // HBH_OK or HBH_ERR_INVARIANT (+ error text)

// ---- a step's integer inputs, packed into one buffer of the caller
// widths[group] = longest block table among the requests
int hbh_step_widths(void* cache, int n_seqs, const int64_t* requests, int* widths);
// Fills buf (int32) at offsets[]: 0 tokens, 1 positions, 2 sequence of each token, 3 cumulative
// token counts [n_seqs + 1], 4 slots, 5 wanted rows, 6 + g the block tables of group g as
// [n_seqs, widths[g]] padded with -1. start_pos / slots receive per-request values.
// row_request / row_version (or null) remember which request and table version was last written
// into each table row of a buffer that lives on between steps: rows that still hold the same
// are left alone.
int hbh_pack_step(void* cache, int n_seqs, const int64_t* requests, const int* n_new, const int* tokens,
                  const int* want_counts, const int* want, const int* widths, const int64_t* offsets, int* buf,
                  int* start_pos, int* slots, int64_t* row_request, int64_t* row_version);

// ---- the scheduler
// max_active <= 0: max_batch_size; max_prefill_portion, max_model_len <= 0: none
typedef void (*hbh_release_fn)(void* user, int64_t request);
void* hbh_sched_create(void* cache, int max_batch_size, int max_active, int max_batched_tokens,
                       int max_prefill_portion, int64_t max_model_len);
void hbh_sched_destroy(void* sched);
const char* hbh_sched_error(void* sched);
// called when a request's pages and slot must go back (preemption, finish); default: close it in the cache
void hbh_sched_set_release(void* sched, hbh_release_fn fn, void* user);
int hbh_sched_add(void* sched, int64_t request, int prompt_len, int max_tokens);
// returns 1 if the request was known (it is finished as "aborted" and released), 0 if not
int hbh_sched_abort(void* sched, int64_t request);
// benchmarks only: a waiting request whose first `computed` tokens are in the cache already runs from there
int hbh_sched_assume_running(void* sched, int64_t request, int64_t computed);
int hbh_sched_has_work(void* sched);
// Decide the next step. entries: (request, first token index, token count, samples, last token in
// flight) x n_entries: "in flight" = the entry's last token is the one the step before samples, so
// the host does not know its value yet. preempted: requests sent back to the head of the waiting
// queue (released already); dropped: requests finished as insufficient_gpu_memory (a lone decode
// that cannot get a page). The plan counts as carried out at once (tokens computed, samples in
// flight); a second plan may be made before the first is committed, not a third.
int hbh_sched_plan(void* sched, int64_t* plan_id, int64_t* entries, int cap_entries, int* n_entries, int64_t* preempted,
                   int cap_preempted, int* n_preempted, int64_t* dropped, int cap_dropped, int* n_dropped);
// The oldest outstanding plan's samples are known. stop[i] for the i-th SAMPLING entry of that
// plan: nonzero = the sampled token ends the request and is not emitted; zero = it is appended
// (flags of entries whose request has ended meanwhile are ignored). finished: (request, reason)
// pairs, reason 1 = length, 2 = stop.
int hbh_sched_commit(void* sched, int64_t plan_id, const int* stop, int n_stop, int64_t* finished, int cap,
                     int* n_finished);
// what: 0 status (0 waiting, 1 running, 2 finished), 1 computed, 2 preemptions, 3 output length,
//       4 finish reason (0 none, 1 length, 2 stop, 3 aborted, 4 insufficient_gpu_memory), 5 samples in flight
int64_t hbh_sched_request_stat(void* sched, int64_t request, int what);
int hbh_sched_queue(void* sched, int which, int64_t* out, int cap);    // 0 waiting, 1 running; returns the count
// what: 0 admitted, 1 preemptions, 2 steps, 3 shrunk portions, 4 stalled portions
int64_t hbh_sched_counter(void* sched, int what);
void hbh_sched_forget(void* sched, int64_t request);           // drop the record of a finished request

// ---- the CPU reference: a whole-sequence float32 forward in plain loops (cpu_forward.cpp)
#define HBH_CPU_ATTENTION 1
#define HBH_CPU_DENSE 1
#define HBH_CPU_EXPERTS 2
typedef struct {
  int hidden, vocab;
  float final_eps;
  const float* embedding;     // [vocab, hidden]
  const float* final_norm;    // [hidden]
  const float* head;          // [vocab, hidden] (the embedding again when the head is tied)
} hbh_cpu_model;
typedef struct {
  int mixer;                  // HBH_CPU_ATTENTION
  int heads, kv_heads, head_dim;
  int chunk, sliding;         // 0 = every earlier key
  int interleaved, qk_norm, temperature;
  float scale, qk_eps, floor_scale, attn_scale, norm_eps;
  const float* inv_freq;      // [rot_pairs] or null: no rotation
  int rot_pairs;              // the first 2 * rot_pairs dims of a head rotate
  const float *norm_mixer, *norm_feed_forward;          // [hidden]
  const float *wq, *wk, *wv, *wo, *bq, *bk, *bv, *bo;    // [out, in]; biases may be null
  int feed_forward;           // HBH_CPU_DENSE or HBH_CPU_EXPERTS
  int inter, experts, top_k, shared_inter;
  const float *w_gate, *w_up, *w_down;                  // dense: [inter, hidden] x2, [hidden, inter]; experts: stacked
  const float* router;        // [experts, hidden]
  const float *shared_gate, *shared_up, *shared_down;   // null: no shared expert
  const int* forced_ids;      // [tokens, top_k] choices to take instead of the router's own, or null
} hbh_cpu_layer;
// Logits [n_want, vocab] at positions want[] of ONE sequence of n_tokens tokens run whole through the
// layers in the order schedule[] names them. router_ids (or null) receives the experts chosen,
// [routed schedule entries, n_tokens, top_k].
int hbh_cpu_forward(const hbh_cpu_model* model, const hbh_cpu_layer* layers, const int* schedule, int n_schedule,
                    const int* tokens, int n_tokens, const int* want, int n_want, float* logits, int* router_ids);

// ---- seeded random weights (the same bits as the device kernel hb_random_normal)
// out[i] = value of element first + i of the tensor with `key`, i < n; scale = std / (sigma * 2^24)
int hbh_random_normal(float* out, int64_t n, int64_t first, uint64_t key, float scale);

#ifdef __cplusplus
}
#endif
