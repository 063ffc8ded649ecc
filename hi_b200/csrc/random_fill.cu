// Seeded random weights, made where they are needed: the same bits on the device (this kernel)
// and on the host (hi_b200/weights/random_values.py, the same arithmetic in numpy).
//
// Element i of a tensor with key K (from the seed and the tensor's name) is
//     c = popcount of 256 hashed bits            (a binomial count: mean 128, variance 64)
//     u = 24 more hashed bits                    (uniform)
//     value = float32((c - 128) * 2^24 + u - 2^23) * scale
// with hashed words h(j) = mix64(K + (5 i + j + 1) * 0x9E3779B97F4A7C15), j = 0..4, and mix64 the
// 64-bit finaliser below. The count smoothed by the uniform has a piecewise-constant density
// that follows the normal curve with sigma = sqrt(64 + 1/12) steps (excess kurtosis -0.008,
// support +-16 sigma); scale = std / (sigma * 2^24) is computed by the caller. Everything before
// the one float multiplication is integer arithmetic, the conversion and the product are each
// rounded once (to nearest even), and so is the store as bfloat16: no library function of either
// side enters, which is what makes host and device agree bit for bit. The reference has no
// random-weights mode (its tests write zeros and ones: crates/hi-mlx/src/backend.rs:1299-1346).
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z;
}

__device__ __forceinline__ float random_value(unsigned long long key, unsigned long long i, float scale) {
  const unsigned long long golden = 0x9E3779B97F4A7C15ull;
  const unsigned long long base = key + (5ull * i + 1ull) * golden;
  int count = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) count += __popcll(mix64(base + (unsigned long long)j * golden));
  const long long u = (long long)(mix64(base + 4ull * golden) >> 40);
  const long long v = ((long long)count - 128) * (1ll << 24) + u - (1ll << 23);
  return __fmul_rn(__ll2float_rn(v), scale);
}

template <typename T>
__global__ void random_normal_kernel(T* out, unsigned long long n, unsigned long long first, unsigned long long key,
                                     float scale) {
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = hb::from_f32<T>(random_value(key, first + i, scale));
}

}  // namespace

// out[i] = the value of element first + i, for i < n.
extern "C" int hb_random_normal(void* out, int dtype, long long n, long long first, unsigned long long key,
                                float scale, cudaStream_t stream) {
  if (!out || n < 0 || first < 0 || (dtype != HB_DTYPE_F32 && dtype != HB_DTYPE_BF16)) return HB_ERR_BAD_ARG;
  if (n == 0) return HB_OK;
  const long long want = (n + 255) / 256;
  const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
  if (dtype == HB_DTYPE_F32)
    random_normal_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, (unsigned long long)n,
                                                            (unsigned long long)first, key, scale);
  else
    random_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, (unsigned long long)n,
                                                                    (unsigned long long)first, key, scale);
  HB_LAUNCH_CHECK();
  return HB_OK;
}
