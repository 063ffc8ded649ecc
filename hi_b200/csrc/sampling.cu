// Per-row sampling from float32 logits: one block per row; rows may mix greedy and sampled
// requests (crates/hi-cuda/src/kernels.cu:8041-8072).
//   temperature <= 0 : argmax, the lowest id on ties (kernels.cu:7156-7186, 7225-7234)
//   temperature  > 0 : weights exp(l/T - max) walked in vocabulary order; the first id whose
//                      running sum exceeds u * total (kernels.cu:7327-7352). u is drawn by the
//                      host, one per request per step, so streams do not depend on batching.
// Ranked sampling (top-k / top-p) is done on the host, as the reference does by default.
#include "api.h"
#include "common.cuh"

namespace {

constexpr int ST = 1024;

__global__ void sample_rows_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temps,
                                   const float* __restrict__ uniforms, int* __restrict__ out) {
  __shared__ float scratch[33];
  __shared__ float sval[ST];
  __shared__ int sidx[ST];
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const float temp = temps ? temps[r] : 0.f;

  // argmax with lowest-id ties: each thread scans a strided set, keeps (value, lowest id)
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = tid; i < vocab; i += ST) {
    const float v = row[i];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  sval[tid] = bv; sidx[tid] = bi;
  __syncthreads();
  for (int s = ST / 2; s > 0; s >>= 1) {
    if (tid < s) {
      const float ov = sval[tid + s];
      const int oi = sidx[tid + s];
      if (ov > sval[tid] || (ov == sval[tid] && oi < sidx[tid])) { sval[tid] = ov; sidx[tid] = oi; }
    }
    __syncthreads();
  }
  const int arg = sidx[0] == 0x7fffffff ? 0 : sidx[0];
  const bool greedy = !(temp > 0.f) || !isfinite(temp);
  if (greedy) {
    if (tid == 0) out[r] = arg;
    return;
  }
  // max of the finite scaled logits
  float mx = -INFINITY;
  for (int i = tid; i < vocab; i += ST) {
    const float v = row[i];
    if (isfinite(v)) {
      const float sc = v / temp;
      if (isfinite(sc)) mx = fmaxf(mx, sc);
    }
  }
  mx = hb::block_max(mx, scratch);
  if (!isfinite(mx)) {
    if (tid == 0) out[r] = arg;
    return;
  }
  // contiguous chunk per thread, so the walk is in vocabulary order
  const int chunk = (vocab + ST - 1) / ST;
  const int begin = min(tid * chunk, vocab), end = min(begin + chunk, vocab);
  float local = 0.f;
  for (int i = begin; i < end; ++i) {
    const float v = row[i];
    if (isfinite(v)) local += expf(v / temp - mx);
  }
  sval[tid] = local;
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    for (int i = 0; i < ST; ++i) { const float c = sval[i]; sval[i] = run; run += c; }  // exclusive prefix
    scratch[0] = run;
  }
  __syncthreads();
  const float total = scratch[0];
  if (!(total > 0.f) || !isfinite(total)) {
    if (tid == 0) out[r] = arg;
    return;
  }
  float u = uniforms ? uniforms[r] : 0.f;
  u = isfinite(u) ? fminf(fmaxf(u, 0.f), 0.99999994f) : 0.f;
  const float target = u * total;
  // the one thread whose [prefix, prefix + local) holds the target walks its chunk
  sidx[tid] = 0x7fffffff;
  __syncthreads();
  const float prefix = sval[tid];
  if (local > 0.f && target >= prefix && target < prefix + local) {
    float cum = prefix;
    int pick = -1, last = -1;
    for (int i = begin; i < end; ++i) {
      const float v = row[i];
      if (!isfinite(v)) continue;
      const float w = expf(v / temp - mx);
      if (w <= 0.f) continue;
      last = i;
      cum += w;
      if (target < cum) { pick = i; break; }
    }
    sidx[tid] = pick >= 0 ? pick : last;
  }
  __syncthreads();
  if (tid == 0) {
    int pick = 0x7fffffff;
    for (int i = 0; i < ST; ++i) pick = min(pick, sidx[i]);
    if (pick == 0x7fffffff || pick < 0) {
      // rounding left the target past every chunk: the last id with positive weight
      pick = arg;
      for (int i = vocab - 1; i >= 0; --i) {
        const float v = row[i];
        if (isfinite(v) && expf(v / temp - mx) > 0.f) { pick = i; break; }
      }
    }
    out[r] = pick;
  }
}

// Argmax of every row with the row cut into gridDim.y parts, so that a few rows of a large
// vocabulary are read by many SMs: each block leaves (value, lowest id) of its part, and the
// block of a row that finishes last (a counter per row, zero between launches) picks among them.
__global__ void argmax_parts_kernel(const float* __restrict__ logits, int vocab, float* part_val, int* part_idx,
                                    int* counters, int* __restrict__ out) {
  __shared__ float sval[ST];
  __shared__ int sidx[ST];
  const int r = blockIdx.x, part = blockIdx.y, parts = gridDim.y, tid = threadIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const int slice = (vocab + parts - 1) / parts;
  const int begin = min(part * slice, vocab), end = min(begin + slice, vocab);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = begin + tid; i < end; i += ST) {
    const float v = row[i];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  sval[tid] = bv; sidx[tid] = bi;
  __syncthreads();
  for (int s = ST / 2; s > 0; s >>= 1) {
    if (tid < s) {
      const float ov = sval[tid + s];
      const int oi = sidx[tid + s];
      if (ov > sval[tid] || (ov == sval[tid] && oi < sidx[tid])) { sval[tid] = ov; sidx[tid] = oi; }
    }
    __syncthreads();
  }
  if (tid != 0) return;
  part_val[(size_t)r * parts + part] = sval[0];
  part_idx[(size_t)r * parts + part] = sidx[0];
  __threadfence();
  if (atomicAdd(&counters[r], 1) != parts - 1) return;
  counters[r] = 0;                 // ready for the next launch
  __threadfence();
  bv = -INFINITY; bi = 0x7fffffff;
  for (int q = 0; q < parts; ++q) {
    const float v = __ldcg(part_val + (size_t)r * parts + q);
    const int i = __ldcg(part_idx + (size_t)r * parts + q);
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  out[r] = bi == 0x7fffffff ? 0 : bi;
}

}  // namespace

// Greedy rows only, over many blocks. part_val / part_idx: [rows, parts] scratch; counters: [rows]
// ints that are zero before the first call and are left at zero.
extern "C" int hb_argmax_rows(const float* logits, int rows, int vocab, int parts, float* part_val, int* part_idx,
                              int* counters, int* out, cudaStream_t stream) {
  if (!logits || !out || !part_val || !part_idx || !counters || rows < 0 || vocab <= 0 || parts <= 0 || parts > 65535)
    return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  argmax_parts_kernel<<<dim3(rows, parts), ST, 0, stream>>>(logits, vocab, part_val, part_idx, counters, out);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_sample_rows(const float* logits, int rows, int vocab, const float* temperatures,
                              const float* uniforms, int* out, cudaStream_t stream) {
  if (!logits || !out || rows < 0 || vocab <= 0) return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  sample_rows_kernel<<<rows, ST, 0, stream>>>(logits, vocab, temperatures, uniforms, out);
  HB_LAUNCH_CHECK();
  return HB_OK;
}
