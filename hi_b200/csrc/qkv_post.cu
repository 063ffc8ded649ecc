// After the fused q/k/v projection: position encoding (rotary) or attention temperature,
// optional weightless L2 norm of q and k, and the append of k and v to the paged cache.
// head_dim / 16 lanes per (token, head) over the nh q heads, nkv k heads and nkv v heads; a
// block is one token and up to 8 warps of its heads, and computes the token's sines and
// cosines once for them.
// All arithmetic in float32; angles are position * inv_freq in float32 with sincosf.
//
// Formulas: rotary pairs (j, j + hd/2) or (2j, 2j+1): crates/hi-cuda/src/kernels.cu:3757-3785,
// crates/hi-mlx/src/models.rs:5997-6016; L2 norm after rotation, eps 1e-6: models.rs:6017-6021;
// page address ((page*kv_heads + head)*page_size + offset)*head_dim: kernels.cu:4214-4219.
#include "api.h"
#include "common.cuh"

namespace {

constexpr int kMaxHeadDim = 256;
constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 pack;
  uint32_t* w = reinterpret_cast<uint32_t*>(&pack);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = pack;
}

// A head is taken by head_dim / 16 neighbouring lanes (padded to `lanes_per_head`, a power of
// two): each lane owns 8 rotation pairs, which are 8 + 8 consecutive elements (pairs (j, j + rot/2))
// or 16 consecutive elements (pairs (2j, 2j + 1)), so every load and store is 16 bytes of
// bfloat16 (32 of float). Only the first rot = 2 * rot_pairs dims of a head rotate (rot a multiple
// of 16; rot = head_dim in Llama 4); the lanes past them own 16 consecutive elements that pass
// through (and count in the norm). A block is one token and up to 8 warps of its heads; it
// computes the token's sines and cosines once.
template <typename T>
__global__ void qkv_post_kernel(const T* __restrict__ qkv, const float* __restrict__ inv_freq,
                                int rot_pairs, int interleaved, int qk_norm, float qk_eps, int temp_on,
                                float floor_scale, float attn_scale, const int* __restrict__ positions,
                                const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                int table_stride, T* __restrict__ q_out, T* __restrict__ k_pages,
                                T* __restrict__ v_pages, int page_size, int write_kv, int n_tokens, int nh,
                                int nkv, int hd, int lanes_per_head) {
  __shared__ float cs_s[kMaxHeadDim / 2], sn_s[kMaxHeadDim / 2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int heads_total = nh + 2 * nkv;
  const int heads_per_warp = 32 / lanes_per_head;
  const int t = blockIdx.x;
  const int first_head = blockIdx.y * kWarpsPerBlock * heads_per_warp;
  const int head = first_head + warp * heads_per_warp + lane / lanes_per_head;
  const int sub = lane % lanes_per_head;                 // which 8 pairs of the head
  const int pos = positions[t];
  const int half = rot_pairs;                            // pairs (j, j + half) when not interleaved
  if (inv_freq != nullptr && first_head < nh + nkv) {    // a block of v heads alone rotates nothing
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf((float)pos * inv_freq[j], &sn_s[j], &cs_s[j]);
  }
  __syncthreads();
  const int kind = head < nh ? 0 : (head < nh + nkv ? 1 : 2);  // q, k, v
  bool active = head < heads_total && sub * 16 < hd && (kind == 0 || write_kv);
  T* dst = nullptr;
  if (active) {
    if (kind == 0) {
      dst = q_out + ((size_t)t * nh + head) * hd;
    } else {
      const int seq = seq_of_token[t];
      const int page = block_table[(size_t)seq * table_stride + pos / page_size];
      active = page >= 0;    // the host reserves pages before the step; without one there is nothing to write into
      const int kvh = kind == 1 ? head - nh : head - nh - nkv;
      T* pool = kind == 1 ? k_pages : v_pages;
      dst = pool + (((size_t)(active ? page : 0) * nkv + kvh) * page_size + (pos % page_size)) * hd;
    }
  }
  const int j0 = sub * 8;                                // pairs j0 .. j0 + 7
  const bool rotates = j0 < rot_pairs;                   // else: 16 elements past the rotated dims
  const bool consecutive = interleaved || !rotates;      // the lane's 16 elements lie side by side
  float a[8], b[8];
  float ss = 0.f;
  if (active) {
    const T* src = qkv + ((size_t)t * heads_total + head) * hd;
    if (consecutive) {                                   // elements 2 j0 .. 2 j0 + 15: (a0, b0, a1, b1, ...)
      float lo[8], hi[8];
      hb::load8(src + 2 * j0, lo);
      hb::load8(src + 2 * j0 + 8, hi);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = lo[2 * i]; b[i] = lo[2 * i + 1];
        a[4 + i] = hi[2 * i]; b[4 + i] = hi[2 * i + 1];
      }
    } else {
      hb::load8(src + j0, a);
      hb::load8(src + half + j0, b);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (kind != 2 && inv_freq != nullptr && rotates) {
        const float sn = sn_s[j0 + i], cs = cs_s[j0 + i];
        const float ra = a[i] * cs - b[i] * sn;
        const float rb = b[i] * cs + a[i] * sn;
        a[i] = ra; b[i] = rb;
      }
      ss += a[i] * a[i] + b[i] * b[i];
    }
  }
  // the lanes of a head add their squares (lanes that own nothing add zero)
  for (int o = lanes_per_head >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (!active) return;
  float mul = 1.f;
  if (kind != 2 && qk_norm) mul = rsqrtf(ss / (float)hd + qk_eps);
  if (kind == 0 && temp_on)
    mul *= logf(floorf(((float)pos + 1.f) / floor_scale) + 1.f) * attn_scale + 1.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) { a[i] *= mul; b[i] *= mul; }
  if (consecutive) {
    float lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo[2 * i] = a[i]; lo[2 * i + 1] = b[i];
      hi[2 * i] = a[4 + i]; hi[2 * i + 1] = b[4 + i];
    }
    store8(dst + 2 * j0, lo);
    store8(dst + 2 * j0 + 8, hi);
  } else {
    store8(dst + j0, a);
    store8(dst + half + j0, b);
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
  if (hd % 16 != 0 || hd > kMaxHeadDim) return HB_ERR_UNSUPPORTED;
  if (!inv_freq) rot_pairs = 0;
  if (rot_pairs < 0 || 2 * rot_pairs > hd || rot_pairs % 8 != 0) return HB_ERR_UNSUPPORTED;  // whole lanes rotate
  if (temp_on && !(floor_scale > 0.f)) return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  const int heads_total = nh + 2 * nkv;
  int lanes_per_head = 1;
  while (lanes_per_head * 16 < hd) lanes_per_head *= 2;
  const int heads_per_warp = 32 / lanes_per_head;
  const int warps = (heads_total + heads_per_warp - 1) / heads_per_warp;
  const dim3 grid(n_tokens, (warps + kWarpsPerBlock - 1) / kWarpsPerBlock);
  const int threads = 32 * (warps < kWarpsPerBlock ? warps : kWarpsPerBlock);
  if (grid.y > 65535) return HB_ERR_UNSUPPORTED;
  if (dtype == HB_DTYPE_F32)
    qkv_post_kernel<float><<<grid, threads, 0, stream>>>(
        (const float*)qkv, inv_freq, rot_pairs, interleaved, qk_norm, qk_eps, temp_on, floor_scale, attn_scale,
        positions, seq_of_token, block_table, table_stride, (float*)q_out, (float*)k_pages, (float*)v_pages,
        page_size, write_kv, n_tokens, nh, nkv, hd, lanes_per_head);
  else if (dtype == HB_DTYPE_BF16)
    qkv_post_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        (const __nv_bfloat16*)qkv, inv_freq, rot_pairs, interleaved, qk_norm, qk_eps, temp_on, floor_scale,
        attn_scale, positions, seq_of_token, block_table, table_stride, (__nv_bfloat16*)q_out,
        (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, page_size, write_kv, n_tokens, nh, nkv, hd, lanes_per_head);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}
