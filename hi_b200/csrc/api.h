// C entry points of libhi_b200_kernels.so. Every function enqueues work on `stream` and
// returns 0, a cudaError_t, or one of the HB_ERR_* codes of common.cuh; none of them
// synchronises. dtype codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int hb_feed_tokens(int* tokens, const int* dst, const int* src, const int* sampled, int n, cudaStream_t stream);
int hb_embed_gather(const void* table, int table_dtype, const int* tokens, float* out, int n, int hidden,
                    int vocab, cudaStream_t stream);
// routed_weight (or null): [n * top_k] factors of the routed rows in the sum (a score that scales the
// experts' outputs)
int hb_add_rmsnorm(float* x, const void* delta, int delta_dtype, const float* routed, const int* slot_of_entry,
                   const float* routed_weight, int top_k, const void* w, int w_dtype, void* y, int y_dtype, float* y_f32, const int* row_map,
                   int rows, int hidden, float eps, cudaStream_t stream);
int hb_swiglu(const void* in, void* out, int dtype, int rows, int inter, cudaStream_t stream);
int hb_moe_combine(const float* y, const int* slot_of_entry, const float* routed_weight, const void* shared,
                   int shared_dtype, float* out,
                   int n, int hidden, int top_k, cudaStream_t stream);

int hb_qkv_post(const void* qkv, int dtype, const float* inv_freq, int rot_pairs, int interleaved, int qk_norm,
                float qk_eps, int temp_on, float floor_scale, float attn_scale, const int* positions,
                const int* seq_of_token, const int* block_table, int table_stride, void* q_out, void* k_pages,
                void* v_pages, int page_size, int write_kv, int n_tokens, int nh, int nkv, int hd,
                cudaStream_t stream);

int hb_paged_attention(const void* q, int dtype, const void* k_pages, const void* v_pages,
                       const int* block_table, int table_stride, const int* seq_of_token, const int* positions,
                       void* out, int n_tokens, int nh, int nkv, int hd, int page_size, int chunk, int window,
                       float scale, int split_size, int max_splits, float* part_acc, float* part_ml,
                       cudaStream_t stream);

int hb_attention_merge(const float* part_acc, const float* part_ml, void* out, int dtype, int n_rows, int hd,
                       int max_splits, cudaStream_t stream);
int hb_attention_decode(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                        int table_stride, const int* seq_of_token, const int* positions, void* out, int n_tokens,
                        int nh, int nkv, int hd, int page_size, int chunk, int window, float scale, int split_size,
                        int max_splits, float* part_acc, float* part_ml, cudaStream_t stream);

int hb_attention_decode_tma(const void* q, const void* k_pages, const void* v_pages, int n_pages, const int* block_table,
                            int table_stride, const int* seq_of_token, const int* positions, void* out, int n_tokens,
                            int nh, int nkv, int hd, int page_size, int chunk, int window, float scale, int split_size,
                            int max_splits, float* part_acc, float* part_ml, int* status, cudaStream_t stream);

// hb_qkv_post, hb_attention_decode_tma and hb_attention_merge in one launch (attention_decode_tma.cu)
int hb_attention_decode_fused(const void* qkv, const float* inv_freq, int rot_pairs, int interleaved, int qk_norm,
                              float qk_eps, int temp_on, float floor_scale, float attn_scale, void* k_pages,
                              void* v_pages, int n_pages, const int* block_table, int table_stride,
                              const int* seq_of_token, const int* positions, void* out, int n_tokens, int nh, int nkv,
                              int hd, int page_size, int chunk, int window, float scale, int split_size,
                              int max_splits, float* part_acc, float* part_ml, int* counters, int* status,
                              cudaStream_t stream);

int hb_attention_prefill(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                         int table_stride, const int* cu_seqlens, const int* positions, void* out, int n_seqs,
                         int max_new, int nh, int nkv, int hd, int page_size, int chunk, int window, float scale,
                         int skip_single, cudaStream_t stream);

int hb_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                            int table_stride, const int* cu_seqlens, const int* positions, void* out, int n_tokens,
                            int n_pages, int n_seqs, int max_new, int nh, int nkv, int hd, int page_size, int chunk,
                            int window, float scale, int skip_single, int key_splits, float* part_acc, float* part_ml,
                            int* status, cudaStream_t stream);

// mode: bit 0 = scores are the softmax over all experts (clear: the sigmoid of the chosen logit),
// bit 1 = the chosen scores are divided by their sum
int hb_router_topk(const void* x, int x_dtype, const void* w, int w_dtype, int n, int hidden, int experts,
                   int top_k, int mode, float* logits_out, int* ids, float* scores, cudaStream_t stream);
int hb_moe_plan(const int* ids, int n_entries, int experts, int* offsets, int* sorted_entry,
                int* slot_of_entry, int* active, cudaStream_t stream);
int hb_router_plan(const void* x, int x_dtype, const void* w, int w_dtype, int n, int hidden, int experts, int top_k,
                   int mode, float* logits_out, int* ids, float* scores, int* offsets, int* sorted_entry, int* slot_of_entry,
                   int* active, int* counter, cudaStream_t stream);
int hb_moe_gate_up(const void* x, int dtype, const int* sorted_entry, int top_k, const void* w_gate,
                   const void* w_up, const int* offsets, const int* active, int experts, const float* scores,
                   void* act, int n_entries, int inter, int hidden, int few_rows, cudaStream_t stream);
int hb_moe_down(const void* act, int dtype, const void* w_down, const int* offsets, const int* active, int experts,
                float* y, int n_entries, int hidden, int inter, int few_rows, cudaStream_t stream);

int hb_gather_rows(const void* x, const int* sorted_entry, int top_k, void* xs, int rows, int hidden,
                   cudaStream_t stream);
int hb_moe_gate_up_tc(const void* xs, const int* sorted_entry, const void* w_gate, const void* w_up,
                      const int* offsets, int experts, const float* scores, void* act, int rows, int inter,
                      int hidden, int* status, cudaStream_t stream);
int hb_moe_down_tc(const void* act, const void* w_down, const int* offsets, int experts, float* y, int rows,
                   int hidden, int inter, float* scratch, long long scratch_floats, int* counters, int n_counters,
                   int* status, cudaStream_t stream);
long long hb_moe_down_tc_scratch_floats(int sms);

int hb_sample_rows(const float* logits, int rows, int vocab, const float* temperatures, const float* uniforms,
                   int* out, cudaStream_t stream);
int hb_sample_rows_parts(const float* logits, int rows, int vocab, int parts, const float* temperatures,
                         const float* uniforms, float* part_val, int* part_idx, float* part_max, float* part_sum,
                         int* counters, int* out, cudaStream_t stream);
int hb_ranked_rows(const float* logits, int rows, int vocab, const float* temperatures, const float* top_ps,
                   const int* top_ks, const float* uniforms, int* out, cudaStream_t stream);
int hb_argmax_rows(const float* logits, int rows, int vocab, int parts, float* part_val, int* part_idx, int* counters,
                   int* out, cudaStream_t stream);

// seeded random weights: out[i] = value of element first + i of the tensor with `key` (random_fill.cu)
int hb_random_normal(void* out, int dtype, long long n, long long first, unsigned long long key, float scale,
                     cudaStream_t stream);

#ifdef __cplusplus
}
#endif
