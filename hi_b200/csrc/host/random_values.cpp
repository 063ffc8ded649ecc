// Seeded random weights on the host: the same integer arithmetic as the device kernel
// hb_random_normal (hi_b200/csrc/random_fill.cu), so a model written to a folder and a model
// generated on the GPU from the same seed hold the same bits. Element i of a tensor with key K:
//     c = popcount of 256 hashed bits,  u = 24 more hashed bits,
//     value = float32((c - 128) * 2^24 + u - 2^23) * scale,
// hashed words mix64(K + (5 i + j + 1) * 0x9E3779B97F4A7C15), j = 0..4.
#include <stdint.h>

#include "runtime.h"

namespace {

inline uint64_t mix64(uint64_t z) {
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z;
}

}  // namespace

extern "C" int hbh_random_normal(float* out, int64_t n, int64_t first, uint64_t key, float scale) {
  if (!out || n < 0 || first < 0) return HBH_ERR_ARG;
  const uint64_t golden = 0x9E3779B97F4A7C15ull;
  for (int64_t i = 0; i < n; ++i) {
    const uint64_t base = key + (5ull * (uint64_t)(first + i) + 1ull) * golden;
    int count = 0;
    for (int j = 0; j < 4; ++j) count += __builtin_popcountll(mix64(base + (uint64_t)j * golden));
    const int64_t u = (int64_t)(mix64(base + 4ull * golden) >> 40);
    const int64_t v = ((int64_t)count - 128) * (1ll << 24) + u - (1ll << 23);
    // one rounding for the conversion, one for the product; a volatile keeps the compiler from
    // fusing or reassociating them
    volatile float f = (float)v;
    out[i] = f * scale;
  }
  return HBH_OK;
}
