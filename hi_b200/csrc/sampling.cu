// Per-row sampling from float32 logits: one block per row; rows may mix greedy and sampled
// requests (crates/hi-cuda/src/kernels.cu:8041-8072).
//   temperature <= 0 : argmax, the lowest id on ties (kernels.cu:7156-7186, 7225-7234)
//   temperature  > 0 : weights exp(l/T - max) walked in vocabulary order; the first id whose
//                      running sum exceeds u * total (kernels.cu:7327-7352). u is drawn by the
//                      host, one per request per step, so streams do not depend on batching.
// Ranked sampling (top-k / top-p): ranked_rows_kernel below, by the host sampler's rule and in its
// order; a row with more candidates than it sorts is handed back to the host.
#include "api.h"
#include "common.cuh"

namespace {

constexpr int ST = 1024;
constexpr int SAMPLE_MAX_PARTS = 64;

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

// The same choice as sample_rows_kernel with every row cut into gridDim.y parts, so that a few rows
// of a large vocabulary are read by many SMs (one block a row reads its 800 KB three times through
// one SM: about 40 us at 202,048 words). A block leaves of its part: the largest logit and its
// lowest id, the largest finite scaled logit m_p, and the sum s_p of exp(l/T - m_p) in vocabulary
// order. The block of a row that finishes last (a counter per row, zero between launches) picks
// the part that holds u * total, where total = sum_p s_p e^(m_p - M) in part order and M = max m_p,
// and walks that part alone with the weights exp(l/T - M), as the one-block kernel walks the row.
__global__ void sample_parts_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temps,
                                    const float* __restrict__ uniforms, float* part_val, int* part_idx,
                                    float* part_max, float* part_sum, int* counters, int* __restrict__ out) {
  __shared__ float scratch[33];
  __shared__ float sval[ST];
  __shared__ int sidx[ST];
  __shared__ int s_last, s_part, s_done;
  __shared__ float s_m, s_target, s_before;
  __shared__ float p_val[SAMPLE_MAX_PARTS], p_max[SAMPLE_MAX_PARTS], p_sum[SAMPLE_MAX_PARTS];
  __shared__ int p_idx[SAMPLE_MAX_PARTS];
  const int r = blockIdx.x, part = blockIdx.y, parts = gridDim.y, tid = threadIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const float temp = temps ? temps[r] : 0.f;
  const bool greedy = !(temp > 0.f) || !isfinite(temp);
  const int slice = (vocab + parts - 1) / parts;
  const int begin = min(part * slice, vocab), end = min(begin + slice, vocab);
  const int chunk = (slice + ST - 1) / ST;          // a thread's run of consecutive words: the order of the vocabulary
  // ---- this part: argmax with lowest-id ties
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
  const float top_v = sval[0];
  const int top_i = sidx[0];
  // ---- this part: largest finite scaled logit and the sum against it
  float mp = -INFINITY, sp = 0.f;
  if (!greedy) {
    const int cb = min(begin + tid * chunk, end), ce = min(cb + chunk, end);
    float mx = -INFINITY;
    for (int i = cb; i < ce; ++i) {
      const float v = row[i];
      if (isfinite(v)) {
        const float sc = v / temp;
        if (isfinite(sc)) mx = fmaxf(mx, sc);
      }
    }
    mp = hb::block_max(mx, scratch);
    if (isfinite(mp)) {
      float local = 0.f;
      for (int i = cb; i < ce; ++i) {
        const float v = row[i];
        if (isfinite(v)) local += expf(v / temp - mp);
      }
      sp = hb::block_sum(local, scratch);             // a fixed tree: the same words give the same sum
    }
  }
  if (tid == 0) {
    const size_t at = (size_t)r * parts + part;
    part_val[at] = top_v; part_idx[at] = top_i; part_max[at] = mp; part_sum[at] = sp;
    __threadfence();
    s_last = atomicAdd(&counters[r], 1) == parts - 1;
    if (s_last) counters[r] = 0;                      // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // ---- the row's last block: which part, by one thread over the parts in order (a thread a part
  // fetches what the parts left, so the loads are in flight together)
  if (tid < parts) {
    const size_t at = (size_t)r * parts + tid;
    p_val[tid] = __ldcg(part_val + at); p_idx[tid] = __ldcg(part_idx + at);
    p_max[tid] = __ldcg(part_max + at); p_sum[tid] = __ldcg(part_sum + at);
  }
  __syncthreads();
  if (tid == 0) {
    float av = -INFINITY;
    int ai = 0x7fffffff;
    float big = -INFINITY;
    for (int q = 0; q < parts; ++q) {
      const float v = p_val[q];
      const int i = p_idx[q];
      if (v > av || (v == av && i < ai)) { av = v; ai = i; }
      big = fmaxf(big, p_max[q]);
    }
    const int arg = ai == 0x7fffffff ? 0 : ai;
    s_done = 1;
    out[r] = arg;                                     // greedy rows, and rows without a usable weight
    if (!greedy && isfinite(big)) {
      float total = 0.f;
      for (int q = 0; q < parts; ++q)
        if (isfinite(p_max[q])) total += p_sum[q] * expf(p_max[q] - big);
      if (total > 0.f && isfinite(total)) {
        float u = uniforms ? uniforms[r] : 0.f;
        u = isfinite(u) ? fminf(fmaxf(u, 0.f), 0.99999994f) : 0.f;
        const float target = u * total;
        float before = 0.f, last_before = 0.f;
        int pick = -1, last = -1;
        for (int q = 0; q < parts && pick < 0; ++q) {
          const float w = isfinite(p_max[q]) ? p_sum[q] * expf(p_max[q] - big) : 0.f;
          if (w > 0.f) {
            last = q; last_before = before;
            if (target < before + w) pick = q; else before += w;
          }
        }
        if (pick < 0) { pick = last; before = last_before; }     // rounding left the target past every part
        if (pick >= 0) { s_done = 0; s_part = pick; s_m = big; s_target = target; s_before = before; }
      }
    }
  }
  __syncthreads();
  if (s_done) return;
  // ---- walk the chosen part with the row's weights
  const int pb = min(s_part * slice, vocab), pe = min(pb + slice, vocab);
  const int cb = min(pb + tid * chunk, pe), ce = min(cb + chunk, pe);
  const float mx = s_m, target = s_target;
  float local = 0.f;
  int last_pos = -1;                                  // this thread's last word with a positive weight
  for (int i = cb; i < ce; ++i) {
    const float v = row[i];
    if (isfinite(v)) {
      const float w = expf(v / temp - mx);
      local += w;
      if (w > 0.f) last_pos = i;
    }
  }
  // Exclusive prefix of the threads' sums, in thread order (warp scans, then the warps' totals), and
  // the part's last word with a weight. Thread t owns the targets in [prefix_t, prefix_(t+1)): the
  // bounds are the same numbers for both neighbours, so every target has exactly one owner.
  const int lane = tid & 31, warp = tid >> 5;
  float incl = local;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += up;
  }
  int last_any = last_pos;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) last_any = max(last_any, __shfl_xor_sync(0xffffffffu, last_any, d));
  if (lane == 31) scratch[warp] = incl;
  if (lane == 0) sidx[warp] = last_any;
  __syncthreads();
  if (warp == 0) {
    float t = scratch[lane];                          // ST / 32 = 32 warps
    float ti = t;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, ti, d);
      if (lane >= d) ti += up;
    }
    scratch[lane] = ti - t;                           // exclusive: what the warps before this one hold
    int la = sidx[lane];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) la = max(la, __shfl_xor_sync(0xffffffffu, la, d));
    if (lane == 0) s_part = la;
  }
  __syncthreads();
  const float prefix = s_before + scratch[warp] + (incl - local);
  const int fallback = s_part;
  sval[tid] = prefix;
  __syncthreads();
  const float upper = tid + 1 < ST ? sval[tid + 1] : INFINITY;
  __syncthreads();
  sidx[tid] = 0x7fffffff;
  if (target >= prefix && target < upper) {
    float cum = prefix;
    int pick = -1, last = -1;
    for (int i = cb; i < ce; ++i) {
      const float v = row[i];
      if (!isfinite(v)) continue;
      const float w = expf(v / temp - mx);
      if (w <= 0.f) continue;
      last = i;
      cum += w;
      if (target < cum) { pick = i; break; }
    }
    sidx[tid] = pick >= 0 ? pick : last;              // (-1: no word with a weight here; the fallback below)
  }
  __syncthreads();
  // at most one thread owned the target
  int mine = sidx[tid];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) mine = min(mine, __shfl_xor_sync(0xffffffffu, mine, d));
  __syncthreads();
  if (lane == 0) sidx[warp] = mine;
  __syncthreads();
  if (tid == 0) {
    int pick = 0x7fffffff;
    for (int i = 0; i < ST / 32; ++i) pick = min(pick, sidx[i]);
    if (pick == 0x7fffffff || pick < 0) pick = fallback;          // rounding: the part's last word with a weight
    if (pick >= 0) out[r] = pick;
  }
}

// ---------------------------------------------------------------- ranked rows (top-k / top-p)
// One block per row, for rows with a temperature and a top-k below the vocabulary or a top-p
// inside (0, 1); other rows are left as they are. The rule is the host sampler's
// (crates/hi-cuda/src/qwen_cpu.rs:3692-3704, crates/hi-mlx/src/generate.rs:86-108):
//   p = exp(l/T - max) / sum; order by p descending, ties by id; keep the first k; of those the
//   shortest prefix whose running sum reaches top_p; draw = u * (sum of the kept); walk.
// The kept ids are a prefix of that order, so the kernel first finds a boundary value t: the
// largest p bit pattern such that the words with p >= t number at least k or hold at least top_p
// of the mass (slightly more, so that rounding cannot leave one out). It finds t four bits at a
// time, counting for fifteen thresholds in one pass over the row, with sums in a fixed order (no
// atomics: the same row gives the same t). The words with p >= t are sorted in shared memory and
// one thread applies the rule to them in the host's order. More than RANK_CAP such words (a nearly
// flat distribution with a wide top-p), or logits that are not finite: out[r] = -1, and the caller
// ranks that row on the host.
constexpr int RANK_THREADS = 1024;
constexpr int RANK_CAP = 4096;
constexpr int RANK_WAYS = 15;

__global__ void __launch_bounds__(RANK_THREADS)
ranked_rows_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temps,
                   const float* __restrict__ top_ps, const int* __restrict__ top_ks,
                   const float* __restrict__ uniforms, int* __restrict__ out) {
  __shared__ float scratch[33];
  __shared__ float red_mass[32][RANK_WAYS];
  __shared__ int red_cnt[32][RANK_WAYS];
  __shared__ float cand_p[RANK_CAP];
  __shared__ int cand_id[RANK_CAP];
  __shared__ unsigned s_prefix;
  __shared__ int s_count;
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float temp = temps[r];
  const int k_in = top_ks[r];
  const bool has_k = k_in > 0 && k_in < vocab;
  const float cutoff = fminf(fmaxf(top_ps[r], 0.f), 1.f);
  const bool has_p = cutoff > 0.f && cutoff < 1.f;
  if (!(temp > 0.f) || !isfinite(temp) || (!has_k && !has_p)) return;     // not a ranked row
  const int k_eff = has_k ? k_in : vocab;
  const float* row = logits + (size_t)r * vocab;

  float mx = -INFINITY;
  bool finite = true;
  for (int i = tid; i < vocab; i += RANK_THREADS) {
    const float z = row[i] / temp;
    finite &= isfinite(z);
    mx = fmaxf(mx, z);
  }
  mx = hb::block_max(mx, scratch);
  const float bad = hb::block_sum(finite ? 0.f : 1.f, scratch);
  if (bad > 0.f || !isfinite(mx)) {
    if (tid == 0) out[r] = -1;
    return;
  }
  float local = 0.f;
  for (int i = tid; i < vocab; i += RANK_THREADS) local += expf(row[i] / temp - mx);
  const float total = hb::block_sum(local, scratch);
  // p of word i, the same expression wherever it is needed
  auto prob = [&](int i) { return expf(row[i] / temp - mx) / total; };

  // ---- the boundary, four bits at a time from the top
  const float cut_mass = has_p ? cutoff * 1.0005f + 1e-6f : INFINITY;
  if (tid == 0) { s_prefix = 0u; s_count = vocab; }
  __syncthreads();
  for (int shift = 28; shift >= 0; shift -= 4) {
    const unsigned prefix = s_prefix;
    int cnt[RANK_WAYS];
    float mass[RANK_WAYS];
#pragma unroll
    for (int j = 0; j < RANK_WAYS; ++j) { cnt[j] = 0; mass[j] = 0.f; }
    for (int i = tid; i < vocab; i += RANK_THREADS) {
      const float p = prob(i);
      const unsigned key = __float_as_uint(p);
      if (key < prefix) continue;                       // below every threshold of this round
#pragma unroll
      for (int j = 0; j < RANK_WAYS; ++j)
        if (key >= (prefix | ((unsigned)(j + 1) << shift))) { cnt[j] += 1; mass[j] += p; }
    }
#pragma unroll
    for (int j = 0; j < RANK_WAYS; ++j) {
      int c = cnt[j];
      float m = mass[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) { c += __shfl_xor_sync(0xffffffffu, c, o); m += __shfl_xor_sync(0xffffffffu, m, o); }
      if (lane == 0) { red_cnt[warp][j] = c; red_mass[warp][j] = m; }
    }
    __syncthreads();
    if (tid == 0) {
      int best = 0, best_count = s_count;
      for (int j = RANK_WAYS - 1; j >= 0; --j) {        // the largest threshold that still holds enough
        int c = 0;
        float m = 0.f;
        for (int w = 0; w < RANK_THREADS / 32; ++w) { c += red_cnt[w][j]; m += red_mass[w][j]; }
        if (c >= k_eff || m >= cut_mass) { best = j + 1; best_count = c; break; }
      }
      s_prefix = prefix | ((unsigned)best << shift);
      s_count = best_count;
    }
    __syncthreads();
  }
  const unsigned boundary = s_prefix;
  const int n_cand = s_count;                           // words with p >= boundary
  if (n_cand > RANK_CAP || n_cand < 1) {
    if (tid == 0) out[r] = -1;
    return;
  }
  // ---- gather the candidates, sort them by (p descending, id ascending)
  if (tid == 0) s_count = 0;
  __syncthreads();
  for (int i = tid; i < vocab; i += RANK_THREADS) {
    const float p = prob(i);
    if (__float_as_uint(p) >= boundary) {
      const int at = atomicAdd(&s_count, 1);
      if (at < RANK_CAP) { cand_p[at] = p; cand_id[at] = i; }
    }
  }
  __syncthreads();
  int size = 1;
  while (size < n_cand) size <<= 1;
  for (int i = n_cand + tid; i < size; i += RANK_THREADS) { cand_p[i] = -1.f; cand_id[i] = 0x7fffffff; }   // padding sorts last
  __syncthreads();
  for (int span = 2; span <= size; span <<= 1) {
    for (int step = span >> 1; step > 0; step >>= 1) {
      for (int i = tid; i < size; i += RANK_THREADS) {
        const int other = i ^ step;
        if (other > i) {
          const bool ascending_block = (i & span) != 0;     // blocks alternate so that the whole ends in order
          const float pa = cand_p[i], pb = cand_p[other];
          const int ia = cand_id[i], ib = cand_id[other];
          const bool a_first = pa > pb || (pa == pb && ia < ib);  // a belongs before b in the wanted order
          if (a_first == ascending_block) {
            cand_p[i] = pb; cand_p[other] = pa;
            cand_id[i] = ib; cand_id[other] = ia;
          }
        }
      }
      __syncthreads();
    }
  }
  // ---- the host's rule on the sorted candidates, by one thread in the host's order
  if (tid == 0) {
    int n = min(n_cand, k_eff);
    if (has_p) {
      float cum = 0.f;
      int keep = -1;
      for (int i = 0; i < n; ++i) {
        cum += cand_p[i];
        if (cum >= cutoff) { keep = i + 1; break; }
      }
      if (keep < 0 && n < k_eff) {      // the running sum fell short of top_p within the candidates (rounding of
        out[r] = -1;                    // a long sum): the host's prefix is longer than what was gathered
        return;
      }
      n = keep < 0 ? n : keep;
    }
    float kept = 0.f;
    for (int i = 0; i < n; ++i) kept += cand_p[i];
    float draw = uniforms[r] * kept;
    int pick = cand_id[0];
    for (int i = 0; i < n; ++i) {
      if (draw <= cand_p[i]) { pick = cand_id[i]; break; }
      draw -= cand_p[i];
    }
    out[r] = pick;
  }
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

// Rows with top-k / top-p, after hb_sample_rows has filled the others: see ranked_rows_kernel.
// top_ks <= 0 or >= vocab means no top-k; out[r] = -1 asks the caller to rank row r on the host.
extern "C" int hb_ranked_rows(const float* logits, int rows, int vocab, const float* temperatures, const float* top_ps,
                              const int* top_ks, const float* uniforms, int* out, cudaStream_t stream) {
  if (!logits || !temperatures || !top_ps || !top_ks || !uniforms || !out || rows < 0 || vocab <= 0) return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  ranked_rows_kernel<<<rows, RANK_THREADS, 0, stream>>>(logits, vocab, temperatures, top_ps, top_ks, uniforms, out);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

// hb_sample_rows with every row cut into `parts` blocks; part_val, part_idx, part_max, part_sum hold
// rows * parts entries each, counters rows ints that are zero between launches.
extern "C" int hb_sample_rows_parts(const float* logits, int rows, int vocab, int parts, const float* temperatures,
                                    const float* uniforms, float* part_val, int* part_idx, float* part_max,
                                    float* part_sum, int* counters, int* out, cudaStream_t stream) {
  if (!logits || !out || !part_val || !part_idx || !part_max || !part_sum || !counters || rows < 0 || vocab <= 0 ||
      parts <= 0 || parts > SAMPLE_MAX_PARTS)
    return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  sample_parts_kernel<<<dim3(rows, parts), ST, 0, stream>>>(logits, vocab, temperatures, uniforms, part_val, part_idx,
                                                            part_max, part_sum, counters, out);
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
