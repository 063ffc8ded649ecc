// After the fused q/k/v projection: position encoding (rotary) or attention temperature,
// optional weightless L2 norm of q and k, and the append of k and v to the paged cache.
// One warp per (token, head) over the nh q heads, nkv k heads and nkv v heads; a block is one
// token and up to 16 of its heads, and computes the token's sines and cosines once for them.
// All arithmetic in float32; angles are position * inv_freq in float32 with sincosf.
//
// Formulas: rotary pairs (j, j + hd/2) or (2j, 2j+1): crates/hi-cuda/src/kernels.cu:3757-3785,
// crates/hi-mlx/src/models.rs:5997-6016; L2 norm after rotation, eps 1e-6: models.rs:6017-6021;
// page address ((page*kv_heads + head)*page_size + offset)*head_dim: kernels.cu:4214-4219.
#include "api.h"
#include "common.cuh"

namespace {

constexpr int kMaxPairsPerLane = 4;  // head_dim <= 256
constexpr int kHeadsPerBlock = 16;

template <typename T>
__global__ void qkv_post_kernel(const T* __restrict__ qkv, const float* __restrict__ inv_freq,
                                int rot_pairs, int interleaved, int qk_norm, float qk_eps, int temp_on,
                                float floor_scale, float attn_scale, const int* __restrict__ positions,
                                const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                int table_stride, T* __restrict__ q_out, T* __restrict__ k_pages,
                                T* __restrict__ v_pages, int page_size, int write_kv, int n_tokens, int nh,
                                int nkv, int hd) {
  __shared__ float cs_s[32 * kMaxPairsPerLane], sn_s[32 * kMaxPairsPerLane];
  const int lane = threadIdx.x & 31;
  const int heads_total = nh + 2 * nkv;
  const int t = blockIdx.x;
  const int head = blockIdx.y * kHeadsPerBlock + (threadIdx.x >> 5);
  const int pos = positions[t];
  if (inv_freq != nullptr && blockIdx.y * kHeadsPerBlock < nh + nkv) {   // a block of v heads alone rotates nothing
    for (int j = threadIdx.x; j < (hd >> 1); j += blockDim.x) sincosf((float)pos * inv_freq[j], &sn_s[j], &cs_s[j]);
  }
  __syncthreads();
  if (head >= heads_total) return;
  const int kind = head < nh ? 0 : (head < nh + nkv ? 1 : 2);  // q, k, v
  if (kind != 0 && !write_kv) return;
  const T* src = qkv + ((size_t)t * heads_total + head) * hd;
  const int half = hd >> 1;

  T* dst;
  if (kind == 0) {
    dst = q_out + ((size_t)t * nh + head) * hd;
  } else {
    const int seq = seq_of_token[t];
    const int page = block_table[(size_t)seq * table_stride + pos / page_size];
    if (page < 0) return;  // the host reserves pages before the step; nothing to write into
    const int kvh = kind == 1 ? head - nh : head - nh - nkv;
    T* pool = kind == 1 ? k_pages : v_pages;
    dst = pool + (((size_t)page * nkv + kvh) * page_size + (pos % page_size)) * hd;
  }

  // Each lane takes two neighbouring pairs per step (j, j+1): its loads and stores are 4 bytes
  // (bfloat16) or 8 bytes (float, or interleaved bfloat16) wide. half is even (head_dim % 16 == 0).
  float a[kMaxPairsPerLane], b[kMaxPairsPerLane];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxPairsPerLane; i += 2) {
    const int j = 2 * lane + 32 * i;            // pairs j and j + 1
    if (j < half) {
      float xa[2], xb[2];
      if (interleaved) {                        // elements 2j .. 2j+3: (a0, b0, a1, b1)
        xa[0] = hb::to_f32(src[2 * j]); xb[0] = hb::to_f32(src[2 * j + 1]);
        xa[1] = hb::to_f32(src[2 * j + 2]); xb[1] = hb::to_f32(src[2 * j + 3]);
      } else {
        xa[0] = hb::to_f32(src[j]); xa[1] = hb::to_f32(src[j + 1]);
        xb[0] = hb::to_f32(src[j + half]); xb[1] = hb::to_f32(src[j + half + 1]);
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (kind != 2 && inv_freq != nullptr) {
          const float sn = sn_s[j + e], cs = cs_s[j + e];
          const float ra = xa[e] * cs - xb[e] * sn;
          const float rb = xb[e] * cs + xa[e] * sn;
          xa[e] = ra; xb[e] = rb;
        }
        a[i + e] = xa[e]; b[i + e] = xb[e];
        ss += xa[e] * xa[e] + xb[e] * xb[e];
      }
    }
  }
  float mul = 1.f;
  if (kind != 2 && qk_norm) {
    ss = hb::warp_sum(ss);
    mul = rsqrtf(ss / (float)hd + qk_eps);
  }
  if (kind == 0 && temp_on)
    mul *= logf(floorf(((float)pos + 1.f) / floor_scale) + 1.f) * attn_scale + 1.f;
#pragma unroll
  for (int i = 0; i < kMaxPairsPerLane; i += 2) {
    const int j = 2 * lane + 32 * i;
    if (j < half) {
      if (interleaved) {
        dst[2 * j] = hb::from_f32<T>(a[i] * mul); dst[2 * j + 1] = hb::from_f32<T>(b[i] * mul);
        dst[2 * j + 2] = hb::from_f32<T>(a[i + 1] * mul); dst[2 * j + 3] = hb::from_f32<T>(b[i + 1] * mul);
      } else {
        dst[j] = hb::from_f32<T>(a[i] * mul); dst[j + 1] = hb::from_f32<T>(a[i + 1] * mul);
        dst[j + half] = hb::from_f32<T>(b[i] * mul); dst[j + half + 1] = hb::from_f32<T>(b[i + 1] * mul);
      }
    }
  }
}

}  // namespace

extern "C" int hb_qkv_post(const void* qkv, int dtype, const float* inv_freq, int rot_pairs, int interleaved,
                           int qk_norm, float qk_eps, int temp_on, float floor_scale, float attn_scale,
                           const int* positions, const int* seq_of_token, const int* block_table,
                           int table_stride, void* q_out, void* k_pages, void* v_pages, int page_size,
                           int write_kv, int n_tokens, int nh, int nkv, int hd, cudaStream_t stream) {
  if (!qkv || !positions || !q_out || n_tokens < 0 || nh <= 0 || nkv <= 0 || hd <= 0) return HB_ERR_BAD_ARG;
  if (write_kv && (!k_pages || !v_pages || !block_table || !seq_of_token || page_size <= 0 || table_stride <= 0))
    return HB_ERR_BAD_ARG;
  if (hd % 2 != 0 || hd > 64 * kMaxPairsPerLane) return HB_ERR_UNSUPPORTED;
  if (inv_freq && rot_pairs != hd / 2) return HB_ERR_UNSUPPORTED;  // all of head_dim rotates
  if (temp_on && !(floor_scale > 0.f)) return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  const int heads_total = nh + 2 * nkv;
  const dim3 grid(n_tokens, (heads_total + kHeadsPerBlock - 1) / kHeadsPerBlock);
  const int threads = 32 * (heads_total < kHeadsPerBlock ? heads_total : kHeadsPerBlock);
  if (grid.y > 65535) return HB_ERR_UNSUPPORTED;
  if (dtype == HB_DTYPE_F32)
    qkv_post_kernel<float><<<grid, threads, 0, stream>>>(
        (const float*)qkv, inv_freq, rot_pairs, interleaved, qk_norm, qk_eps, temp_on, floor_scale, attn_scale,
        positions, seq_of_token, block_table, table_stride, (float*)q_out, (float*)k_pages, (float*)v_pages,
        page_size, write_kv, n_tokens, nh, nkv, hd);
  else if (dtype == HB_DTYPE_BF16)
    qkv_post_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        (const __nv_bfloat16*)qkv, inv_freq, rot_pairs, interleaved, qk_norm, qk_eps, temp_on, floor_scale,
        attn_scale, positions, seq_of_token, block_table, table_stride, (__nv_bfloat16*)q_out,
        (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, page_size, write_kv, n_tokens, nh, nkv, hd);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}
