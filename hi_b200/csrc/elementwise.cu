// Embedding gather, residual-add + RMSNorm, SwiGLU, expert-output combine.
// The residual stream is float32 in every mode; statistics and sums are float32.
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
  return dtype == HB_DTYPE_F32 ? reinterpret_cast<const float*>(p)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void store_any(void* p, int dtype, size_t i, float v) {
  if (dtype == HB_DTYPE_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float4 load4_any(const void* p, int dtype, size_t i) {   // i % 4 == 0
  if (dtype == HB_DTYPE_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
  return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                     __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}
__device__ __forceinline__ void store4_any(void* p, int dtype, size_t i, float4 v) {
  if (dtype == HB_DTYPE_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = v;
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a);
    raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = raw;
  }
}

// x[t, :] = table[token[t], :]   (crates/hi-mlx/src/models.rs:6206: no multiplier)
__global__ void embed_gather_kernel(const void* table, int table_dtype, const int* tokens,
                                    float* out, int hidden, int vocab) {
  const int t = blockIdx.x;
  int id = tokens[t];
  const bool ok = id >= 0 && id < vocab;
  if ((hidden & 3) == 0) {
#pragma unroll 4
    for (int j = threadIdx.x * 4; j < hidden; j += blockDim.x * 4)
      *reinterpret_cast<float4*>(out + (size_t)t * hidden + j) =
          ok ? load4_any(table, table_dtype, (size_t)id * hidden + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    return;
  }
  for (int j = threadIdx.x; j < hidden; j += blockDim.x)
    out[(size_t)t * hidden + j] = ok ? load_any(table, table_dtype, (size_t)id * hidden + j) : 0.f;
}

// Row r of the output: src = row_map ? row_map[r] : r.
//   s = x[src] (+ delta[src]);  if no row_map: x[src] = s  (the residual sum, float32)
//   y[r] = s * rsqrt(mean(s^2) + eps) * w     (crates/hi-cuda/src/kernels.cu:61-77)
__global__ void add_rmsnorm_kernel(float* x, const void* delta, int delta_dtype, const float* routed,
                                   const int* slot_of_entry, const float* routed_weight, int top_k, const void* w,
                                   int w_dtype, void* y, int y_dtype, float* y_f32, const int* row_map,
                                   int hidden, float eps) {
  __shared__ float scratch[33];
  extern __shared__ float row[];  // hidden floats
  const int r = blockIdx.x;
  const size_t src = row_map ? (size_t)row_map[r] : (size_t)r;
  float ss = 0.f;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
    float s = x[src * hidden + j];
    if (delta) s += load_any(delta, delta_dtype, src * hidden + j);
    if (routed)
      for (int q = 0; q < top_k; ++q)
        s += routed[(size_t)slot_of_entry[src * top_k + q] * hidden + j] * (routed_weight ? routed_weight[src * top_k + q] : 1.f);
    row[j] = s;
    ss += s * s;
  }
  const float total = hb::block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
    const float s = row[j];
    if (!row_map && (delta || routed)) x[src * hidden + j] = s;
    const float wv = w ? load_any(w, w_dtype, j) : 1.f;
    store_any(y, y_dtype, (size_t)r * hidden + j, s * inv * wv);
    if (y_f32) y_f32[(size_t)r * hidden + j] = s * inv * wv;
  }
}

// The same, for hidden % 4 == 0 and hidden <= 4 * blockDim * NG: the row lives in registers, every
// load is a 16-byte (or 8-byte bfloat16) vector issued before the first use, and the sum that the
// residual takes may include the routed experts' rows:
//   s = x[src] + delta[src] + sum_j routed[slot_of_entry[src*top_k + j]]
// (the combine of crates/hi-cuda/src/kernels.cu:10661-10680, in rank order, fused into the norm).
template <int NG>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype,
                                       const float* __restrict__ routed, const int* __restrict__ slot_of_entry,
                                       const float* __restrict__ routed_weight, int top_k, const void* __restrict__ w, int w_dtype, void* __restrict__ y,
                                       int y_dtype, float* __restrict__ y_f32, const int* __restrict__ row_map,
                                       int hidden, float eps) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const size_t src = row_map ? (size_t)row_map[r] : (size_t)r;
  float4 v[NG], wv[NG];
  float ss = 0.f;
  int slots[8];
  float factor[8];
  if (routed)
    for (int j = 0; j < top_k; ++j) {
      slots[j] = slot_of_entry[src * top_k + j];
      factor[j] = routed_weight ? routed_weight[src * top_k + j] : 1.f;
    }
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    const int idx = (threadIdx.x + g * blockDim.x) * 4;
    if (idx < hidden) {
      // the norm's weight is asked for now, so that it is there when the sum of squares is
      wv[g] = w ? load4_any(w, w_dtype, idx) : make_float4(1.f, 1.f, 1.f, 1.f);
      float4 a = *reinterpret_cast<const float4*>(x + src * hidden + idx);
      if (delta) {
        const float4 d = load4_any(delta, delta_dtype, src * hidden + idx);
        a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
      }
      if (routed) {
        for (int j = 0; j < top_k; ++j) {
          const float4 d = *reinterpret_cast<const float4*>(routed + (size_t)slots[j] * hidden + idx);
          a.x += d.x * factor[j]; a.y += d.y * factor[j]; a.z += d.z * factor[j]; a.w += d.w * factor[j];
        }
      }
      v[g] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  const float total = hb::block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    const int idx = (threadIdx.x + g * blockDim.x) * 4;
    if (idx < hidden) {
      const float4 a = v[g];
      if (!row_map && (delta || routed)) *reinterpret_cast<float4*>(x + src * hidden + idx) = a;
      const float4 o = make_float4(a.x * inv * wv[g].x, a.y * inv * wv[g].y, a.z * inv * wv[g].z, a.w * inv * wv[g].w);
      store4_any(y, y_dtype, (size_t)r * hidden + idx, o);
      if (y_f32) *reinterpret_cast<float4*>(y_f32 + (size_t)r * hidden + idx) = o;
    }
  }
}

// out[t, j] = silu(in[t, j]) * in[t, inter + j]   (crates/hi-mlx/src/models.rs:2307-2312)
__global__ void swiglu_kernel(const void* in, void* out, int dtype, size_t rows, int inter) {
  const size_t total = rows * (size_t)inter;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / inter;
    const int j = (int)(i - t * inter);
    const float g = load_any(in, dtype, t * 2 * inter + j);
    const float u = load_any(in, dtype, t * 2 * inter + inter + j);
    store_any(out, dtype, i, g / (1.f + expf(-g)) * u);
  }
}

// out[t, :] = shared[t, :] + sum_j y[slot_of_entry[t*k + j], :]   in rank order, no atomics
// (crates/hi-cuda/src/kernels.cu:10661-10680; models.rs:6099 adds the shared expert).
__global__ void moe_combine_kernel(const float* y, const int* slot_of_entry, const float* routed_weight,
                                   const void* shared, int shared_dtype, float* out, int hidden, int top_k) {
  const int t = blockIdx.x;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
    float s = shared ? load_any(shared, shared_dtype, (size_t)t * hidden + j) : 0.f;
    for (int r = 0; r < top_k; ++r)
      s += y[(size_t)slot_of_entry[t * top_k + r] * hidden + j] * (routed_weight ? routed_weight[t * top_k + r] : 1.f);
    out[(size_t)t * hidden + j] = s;
  }
}

bool dtype_ok(int d) { return d == HB_DTYPE_F32 || d == HB_DTYPE_BF16; }

}  // namespace

extern "C" int hb_embed_gather(const void* table, int table_dtype, const int* tokens, float* out,
                               int n, int hidden, int vocab, cudaStream_t stream) {
  if (!table || !tokens || !out || n < 0 || hidden <= 0 || vocab <= 0 || !dtype_ok(table_dtype))
    return HB_ERR_BAD_ARG;
  if (n == 0) return HB_OK;
  embed_gather_kernel<<<n, 256, 0, stream>>>(table, table_dtype, tokens, out, hidden, vocab);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

// tokens[dst[i]] = sampled[src[i]]: the step before this one left its sampled tokens on the
// device; a step that is launched before the host has read them takes them from there.
__global__ void feed_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ dst, const int* __restrict__ src,
                                   const int* __restrict__ sampled, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) tokens[dst[i]] = sampled[src[i]];
}

extern "C" int hb_feed_tokens(int* tokens, const int* dst, const int* src, const int* sampled, int n,
                              cudaStream_t stream) {
  if (!tokens || !dst || !src || !sampled || n < 0) return HB_ERR_BAD_ARG;
  if (n == 0) return HB_OK;
  feed_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, dst, src, sampled, n);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_add_rmsnorm(float* x, const void* delta, int delta_dtype, const float* routed,
                              const int* slot_of_entry, const float* routed_weight, int top_k, const void* w, int w_dtype, void* y, int y_dtype,
                              float* y_f32, const int* row_map, int rows, int hidden, float eps,
                              cudaStream_t stream) {
  if (!x || !y || rows < 0 || hidden <= 0 || !dtype_ok(y_dtype) || (delta && !dtype_ok(delta_dtype)) ||
      (w && !dtype_ok(w_dtype)))
    return HB_ERR_BAD_ARG;
  if (routed && (!slot_of_entry || top_k < 1 || top_k > 8)) return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  if (hidden % 4 == 0 && hidden <= 4 * 512 * 8) {
    const int groups = hidden / 4;
    const int threads = groups >= 512 ? 512 : ((groups + 31) / 32) * 32;
    const int ng = (groups + threads - 1) / threads;
#define HB_NORM_LAUNCH(NG)                                                                                   \
    add_rmsnorm_vec_kernel<NG><<<rows, threads, 0, stream>>>(x, delta, delta_dtype, routed, slot_of_entry, routed_weight, top_k, \
                                                             w, w_dtype, y, y_dtype, y_f32, row_map, hidden, eps)
    if (ng <= 1) HB_NORM_LAUNCH(1);
    else if (ng <= 2) HB_NORM_LAUNCH(2);
    else if (ng <= 4) HB_NORM_LAUNCH(4);
    else HB_NORM_LAUNCH(8);
#undef HB_NORM_LAUNCH
    HB_LAUNCH_CHECK();
    return HB_OK;
  }
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return HB_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = hidden >= 2048 ? 512 : 256;
  add_rmsnorm_kernel<<<rows, threads, smem, stream>>>(x, delta, delta_dtype, routed, slot_of_entry, routed_weight, top_k, w, w_dtype,
                                                      y, y_dtype, y_f32, row_map, hidden, eps);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

// The same, 4 columns per thread with vector loads (inter % 4 == 0).
__global__ void swiglu_vec_kernel(const void* __restrict__ in, void* __restrict__ out, int dtype, size_t rows,
                                  int inter) {
  const int groups = inter / 4;
  const size_t total = rows * (size_t)groups;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / groups;
    const int j = (int)(i - t * groups) * 4;
    const float4 g = load4_any(in, dtype, t * 2 * inter + j);
    const float4 u = load4_any(in, dtype, t * 2 * inter + inter + j);
    store4_any(out, dtype, t * inter + j,
               make_float4(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y,
                           g.z / (1.f + expf(-g.z)) * u.z, g.w / (1.f + expf(-g.w)) * u.w));
  }
}

// bfloat16, 8 columns per thread (16-byte loads and stores; inter % 8 == 0), two groups in flight.
__global__ void swiglu_bf16x8_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, size_t rows, int inter) {
  const int groups = inter / 8;
  const size_t total = rows * (size_t)groups;
  auto one = [](uint32_t g2, uint32_t u2) {
    const float g0 = __uint_as_float(g2 << 16), g1 = __uint_as_float(g2 & 0xffff0000u);
    const float u0 = __uint_as_float(u2 << 16), u1 = __uint_as_float(u2 & 0xffff0000u);
    __nv_bfloat162 r = __floats2bfloat162_rn(g0 / (1.f + expf(-g0)) * u0, g1 / (1.f + expf(-g1)) * u1);
    return *reinterpret_cast<uint32_t*>(&r);
  };
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += 2 * stride) {
    const size_t i2 = i + stride;
    const size_t t = i / groups, t2 = i2 / groups;
    const int j = (int)(i - t * groups), j2 = (int)(i2 - t2 * groups);
    const uint4 g = in[t * 2 * groups + j], u = in[t * 2 * groups + groups + j];
    uint4 gb = g, ub = u;
    if (i2 < total) { gb = in[t2 * 2 * groups + j2]; ub = in[t2 * 2 * groups + groups + j2]; }
    out[i] = make_uint4(one(g.x, u.x), one(g.y, u.y), one(g.z, u.z), one(g.w, u.w));
    if (i2 < total) out[i2] = make_uint4(one(gb.x, ub.x), one(gb.y, ub.y), one(gb.z, ub.z), one(gb.w, ub.w));
  }
}

extern "C" int hb_swiglu(const void* in, void* out, int dtype, int rows, int inter, cudaStream_t stream) {
  if (!in || !out || rows < 0 || inter <= 0 || !dtype_ok(dtype)) return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  if (dtype == HB_DTYPE_BF16 && inter % 8 == 0) {
    const size_t groups = (size_t)rows * (inter / 8);
    const size_t want = (groups + 255) / 256;                       // a group per thread while the grid is small
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    swiglu_bf16x8_kernel<<<blocks, 256, 0, stream>>>((const uint4*)in, (uint4*)out, (size_t)rows, inter);
    HB_LAUNCH_CHECK();
    return HB_OK;
  }
  if (inter % 4 == 0) {
    const size_t groups = (size_t)rows * (inter / 4);
    const int blocks = (int)((groups + 255) / 256 < 148 * 32 ? (groups + 255) / 256 : 148 * 32);
    swiglu_vec_kernel<<<blocks, 256, 0, stream>>>(in, out, dtype, (size_t)rows, inter);
    HB_LAUNCH_CHECK();
    return HB_OK;
  }
  const size_t total = (size_t)rows * inter;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  swiglu_kernel<<<blocks, 256, 0, stream>>>(in, out, dtype, (size_t)rows, inter);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_moe_combine(const float* y, const int* slot_of_entry, const float* routed_weight, const void* shared,
                              int shared_dtype, float* out, int n, int hidden, int top_k,
                              cudaStream_t stream) {
  if (!y || !slot_of_entry || !out || n < 0 || hidden <= 0 || top_k <= 0 || (shared && !dtype_ok(shared_dtype)))
    return HB_ERR_BAD_ARG;
  if (n == 0) return HB_OK;
  moe_combine_kernel<<<n, 256, 0, stream>>>(y, slot_of_entry, routed_weight, shared, shared_dtype, out, hidden, top_k);
  HB_LAUNCH_CHECK();
  return HB_OK;
}
