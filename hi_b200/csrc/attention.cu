// Attention of new tokens over the paged cache: the general kernel.
//
// One warp per (token, query head). The keys a query at position p may read are
//   [lo, p],  lo = max(chunk ? floor(p / chunk) * chunk : 0,  window ? p - window + 1 : 0)
// (causal rule crates/hi-mlx/src/models.rs:11165-11184; the chunk rule is this engine's).
// Keys are walked 32 at a time in position order with an online softmax, so a token's
// result depends only on its own query and the keys it reads: not on how the tokens were
// cut into steps, on what else is in the batch, or on which pages hold the keys.
// Scores, max, sum and the weighted sum of values are float32 (models.rs:5963, 6024-6050).
// Query head h reads kv head h / (nh / nkv) (crates/hi-cuda/src/kernels.cu:12413-12414).
#include "api.h"
#include "common.cuh"

namespace {

constexpr int kMaxDimsPerLane = 8;  // head_dim <= 256

template <typename T>
__global__ void paged_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                                       const T* __restrict__ v_pages, const int* __restrict__ block_table,
                                       int table_stride, const int* __restrict__ seq_of_token,
                                       const int* __restrict__ positions, T* __restrict__ out, int n_tokens,
                                       int nh, int nkv, int hd, int page_size, int chunk, int window,
                                       float scale, int split_size, int max_splits,
                                       float* __restrict__ part_acc, float* __restrict__ part_ml) {
  extern __shared__ float q_smem[];  // [warps][hd]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (wid >= (long long)n_tokens * nh * max_splits) return;
  const int split = (int)(wid % max_splits);
  const long long th = wid / max_splits;
  const int t = (int)(th / nh);
  const int h = (int)(th - (long long)t * nh);
  const int kvh = h / (nh / nkv);
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * table_stride;
  int lo = 0;
  if (chunk > 0) lo = (pos / chunk) * chunk;
  if (window > 0 && pos - window + 1 > lo) lo = pos - window + 1;
  // split s of a token covers keys [lo + s*split_size, lo + (s+1)*split_size): a function of the
  // token's own visible range only, never of the batch
  int hi = pos;
  if (max_splits > 1) {
    float* ml = part_ml + ((size_t)th * max_splits + split) * 2;
    const int first = lo + split * split_size;
    if (first > pos) {
      if (lane == 0) { ml[0] = -INFINITY; ml[1] = 0.f; }
      return;
    }
    lo = first;
    hi = min(pos, first + split_size - 1);
  }

  float* qs = q_smem + warp * hd;
  const T* qrow = q + ((size_t)t * nh + h) * hd;
  for (int d = lane; d < hd; d += 32) qs[d] = hb::to_f32(qrow[d]) * scale;
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[kMaxDimsPerLane];
#pragma unroll
  for (int i = 0; i < kMaxDimsPerLane; ++i) acc[i] = 0.f;

  for (int base = lo; base <= hi; base += 32) {
    const int key = base + lane;
    const bool valid = key <= hi;
    float s = -INFINITY;
    int page = -1;
    if (valid) {
      page = table[key / page_size];
      if (page >= 0) {
        const T* krow = k_pages + (((size_t)page * nkv + kvh) * page_size + (key % page_size)) * hd;
        float dot = 0.f;
        for (int d = 0; d < hd; d += 8) {
          float kv[8];
          hb::load8(krow + d, kv);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot += qs[d + e] * kv[e];
        }
        s = dot;
      }
    }
    const float m_new = fmaxf(m, hb::warp_max(s));
    if (m_new == -INFINITY) continue;  // no readable key in this batch (a hole in the table)
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + hb::warp_sum(p);
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) acc[i] *= corr;
    const int count = min(32, hi - base + 1);
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int pg = __shfl_sync(0xffffffffu, page, j);
      if (pg < 0) continue;
      const T* vrow = v_pages + (((size_t)pg * nkv + kvh) * page_size + ((base + j) % page_size)) * hd;
#pragma unroll
      for (int i = 0; i < kMaxDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] += pj * hb::to_f32(vrow[d]);
      }
    }
    m = m_new;
  }
  if (max_splits > 1) {
    float* pa = part_acc + ((size_t)th * max_splits + split) * hd;
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) pa[d] = acc[i];
    }
    if (lane == 0) {
      float* ml = part_ml + ((size_t)th * max_splits + split) * 2;
      ml[0] = m; ml[1] = l;
    }
    return;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* orow = out + ((size_t)t * nh + h) * hd;
#pragma unroll
  for (int i = 0; i < kMaxDimsPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) orow[d] = hb::from_f32<T>(acc[i] * inv);
  }
}

// Combine the splits of each (token, head): o = sum_s acc_s e^{m_s - m} / sum_s l_s e^{m_s - m},
// in split order.
template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                       T* __restrict__ out, int hd, int max_splits) {
  extern __shared__ float wgt[];   // [max_splits] weight of each split, then 33 floats of scratch
  float* scratch = wgt + max_splits;
  const size_t th = blockIdx.x;
  const float* ml = part_ml + th * max_splits * 2;
  // The partial rows of up to MERGE_AHEAD splits are asked for before anything else, so that they
  // arrive while the weights are worked out (otherwise the merge is three trips to memory one
  // after the other). A split beyond the token's range has an unwritten row: it may be loaded,
  // but must not enter the sum (whatever the scratch holds there, even NaN); its weight is 0.
  constexpr int MERGE_AHEAD = 32;
  float ahead[MERGE_AHEAD];
  const int d0 = threadIdx.x;
  if (d0 < hd) {
#pragma unroll
    for (int s = 0; s < MERGE_AHEAD; ++s)
      if (s < max_splits) ahead[s] = part_acc[(th * max_splits + s) * hd + d0];
  }
  float m = -INFINITY;
  for (int s = threadIdx.x; s < max_splits; s += blockDim.x) m = fmaxf(m, ml[2 * s]);
  m = hb::block_max(m, scratch);
  float l = 0.f;
  for (int s = threadIdx.x; s < max_splits; s += blockDim.x) {
    const float ms = ml[2 * s];
    const float e = ms == -INFINITY ? 0.f : expf(ms - m);
    wgt[s] = e;
    l += ml[2 * s + 1] * e;
  }
  l = hb::block_sum(l, scratch);      // fixed tree order: the same inputs give the same sum
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    int s = 0;
    if (d == d0) {
#pragma unroll
      for (int q = 0; q < MERGE_AHEAD; ++q) {
        if (q < max_splits) {
          const float ws = wgt[q];
          if (ws != 0.f) o += ahead[q] * ws;
        }
      }
      s = min(max_splits, MERGE_AHEAD);
    }
#pragma unroll 8
    for (; s < max_splits; ++s) {
      const float ws = wgt[s];
      if (ws != 0.f) o += part_acc[(th * max_splits + s) * hd + d] * ws;
    }
    out[th * hd + d] = hb::from_f32<T>(o * inv);
  }
}

}  // namespace

extern "C" int hb_paged_attention(const void* q, int dtype, const void* k_pages, const void* v_pages,
                                  const int* block_table, int table_stride, const int* seq_of_token,
                                  const int* positions, void* out, int n_tokens, int nh, int nkv, int hd,
                                  int page_size, int chunk, int window, float scale, int split_size,
                                  int max_splits, float* part_acc, float* part_ml, cudaStream_t stream) {
  if (!q || !k_pages || !v_pages || !block_table || !seq_of_token || !positions || !out) return HB_ERR_BAD_ARG;
  if (max_splits < 1 || (max_splits > 1 && (split_size <= 0 || !part_acc || !part_ml))) return HB_ERR_BAD_ARG;
  if (n_tokens < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || table_stride <= 0 ||
      chunk < 0 || window < 0)
    return HB_ERR_BAD_ARG;
  if (hd <= 0 || hd % 8 != 0 || hd > 32 * kMaxDimsPerLane) return HB_ERR_UNSUPPORTED;
  if (n_tokens == 0) return HB_OK;
  const int warps_per_block = 4;
  const long long warps = (long long)n_tokens * nh * max_splits;
  const long long blocks = (warps + warps_per_block - 1) / warps_per_block;
  if (blocks > 0x7fffffffLL) return HB_ERR_UNSUPPORTED;
  const size_t smem = (size_t)warps_per_block * hd * sizeof(float);
  if (dtype == HB_DTYPE_F32)
    paged_attention_kernel<float><<<(int)blocks, warps_per_block * 32, smem, stream>>>(
        (const float*)q, (const float*)k_pages, (const float*)v_pages, block_table, table_stride, seq_of_token,
        positions, (float*)out, n_tokens, nh, nkv, hd, page_size, chunk, window, scale, split_size, max_splits,
        part_acc, part_ml);
  else if (dtype == HB_DTYPE_BF16)
    paged_attention_kernel<__nv_bfloat16><<<(int)blocks, warps_per_block * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table,
        table_stride, seq_of_token, positions, (__nv_bfloat16*)out, n_tokens, nh, nkv, hd, page_size, chunk,
        window, scale, split_size, max_splits, part_acc, part_ml);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  if (max_splits > 1) {
    if (dtype == HB_DTYPE_F32)
      attention_merge_kernel<float><<<n_tokens * nh, 128, (max_splits + 33) * sizeof(float), stream>>>(part_acc, part_ml, (float*)out, hd, max_splits);
    else
      attention_merge_kernel<__nv_bfloat16><<<n_tokens * nh, 128, (max_splits + 33) * sizeof(float), stream>>>(
          part_acc, part_ml, (__nv_bfloat16*)out, hd, max_splits);
    HB_LAUNCH_CHECK();
  }
  return HB_OK;
}

// Merge of split partials alone (the decode kernel writes the same partial layout).
extern "C" int hb_attention_merge(const float* part_acc, const float* part_ml, void* out, int dtype, int n_rows,
                                  int hd, int max_splits, cudaStream_t stream) {
  if (!part_acc || !part_ml || !out || n_rows < 0 || hd <= 0 || max_splits < 1) return HB_ERR_BAD_ARG;
  if (n_rows == 0) return HB_OK;
  if (dtype == HB_DTYPE_F32)
    attention_merge_kernel<float><<<n_rows, 128, (max_splits + 33) * sizeof(float), stream>>>(part_acc, part_ml, (float*)out, hd, max_splits);
  else if (dtype == HB_DTYPE_BF16)
    attention_merge_kernel<__nv_bfloat16><<<n_rows, 128, (max_splits + 33) * sizeof(float), stream>>>(
        part_acc, part_ml, (__nv_bfloat16*)out, hd, max_splits);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}
