// hb_attention_decode_static: decode attention that allocates nothing.
//
// This entry point has no counterpart in the reference (PipeNetwork/hi); it is an addition of
// this library.
//
// Who it is for. hb_attention_decode needs scratch memory for the partial results of its
// key-range splits, and its callers get that scratch from an allocator. Some callers cannot:
// a host program that handed the whole device memory to its own arena at start-up and has
// nothing left for cudaMalloc to give; a serving loop under a no-allocation rule, because an
// allocation can stall every stream of the device while it runs. For them the scratch lives
// inside the library, in a file-scope `static __device__` array of fixed size, and this entry
// point calls no cudaMalloc, no cudaFree and no allocating library routine. The caller passes
// inputs and the output only.
//
// Limits and rules:
//   * The scratch holds HB_STATIC_SCRATCH_FLOATS floats (8 MiB + 256 KiB; every GPU that loads
//     the library holds that much until the process exits), in two parts that are checked
//     each on its own: the splits' partial outputs need
//         n_tokens * nh * max_splits * hd   <= HB_STATIC_SCRATCH_ACC_FLOATS   floats
//     and their running maxima and sums
//         n_tokens * nh * max_splits * 2    <= HB_STATIC_SCRATCH_ML_FLOATS    floats.
//     A call that breaks either bound is refused with HB_ERR_SCRATCH_CAPACITY (and a line on
//     stderr); use fewer splits, or the allocating entry point.
//     hb_attention_decode_static_fits() answers the question up front.
//   * All calls share the one array and it keeps what the last call left. Nothing in it needs
//     to start at zero: every row a call reads back it has written itself, and rows it did not
//     write (splits past a token's range) carry weight zero in the merge and are skipped.
//     Two calls that overlap on the GPU (different streams, or different host threads) race on
//     the array; run them on one stream, or order them with events.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and keeps it. Make that first call
//     before any stream capture begins.
//   * Shapes: as hb_attention_decode (bfloat16, head_dim 64 or 128, at most 16 query heads per
//     kv head, split_size a multiple of 64). max_splits == 1 is allowed and uses no scratch.
#pragma once
#include <cuda_runtime.h>

#define HB_STATIC_SCRATCH_ACC_FLOATS (1 << 21)
#define HB_STATIC_SCRATCH_ML_FLOATS (1 << 16)
#define HB_STATIC_SCRATCH_FLOATS (HB_STATIC_SCRATCH_ACC_FLOATS + HB_STATIC_SCRATCH_ML_FLOATS)
#define HB_ERR_SCRATCH_CAPACITY 1003

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as hb_attention_decode followed by hb_attention_merge, minus the
// two scratch pointers. Returns 0, a cudaError_t, HB_ERR_BAD_ARG, HB_ERR_UNSUPPORTED or
// HB_ERR_SCRATCH_CAPACITY. Enqueues on `stream`; does not synchronise.
int hb_attention_decode_static(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                               int table_stride, const int* seq_of_token, const int* positions, void* out,
                               int n_tokens, int nh, int nkv, int hd, int page_size, int chunk, int window,
                               float scale, int split_size, int max_splits, cudaStream_t stream);

// Floats of scratch a call with these sizes needs, both parts together (a total within
// HB_STATIC_SCRATCH_FLOATS does not yet mean that each part fits: ask the function below).
long long hb_attention_decode_static_need(int n_tokens, int nh, int hd, int max_splits);

// 1 if a call with these sizes fits the built-in scratch (each of the two parts within its own
// bound), 0 if it would be refused with HB_ERR_SCRATCH_CAPACITY.
int hb_attention_decode_static_fits(int n_tokens, int nh, int hd, int max_splits);

#ifdef __cplusplus
}
#endif
