// Routed experts: router top-k, the device-side plan (rows grouped by expert), and the
// general grouped matrix products with the SwiGLU epilogue. No step here returns to the host
// (the reference syncs per layer to pick the expert: crates/hi-mlx/src/models.rs:6081-6084).
//
// Formulas (models.rs:6086-6100): score = sigmoid(selected router logit); the score scales the
// expert INPUT: act = silu(s * (x Wg^T)) * (s * (x Wu^T)) — by linearity equal to feeding s*x —
// and y = act Wd^T. Ties between equal logits go to the lower expert id
// (crates/hi-cuda/src/kernels.cu:578-580). All accumulation, the sigmoid and SwiGLU are float32.
#include <type_traits>

#include "api.h"
#include "common.cuh"

namespace {

// ------------------------------------------------------------------ the plan, by one block
// Stable counting sort of the n = tokens*top_k routing entries by expert:
// offsets[e]..offsets[e+1] are the sorted slots of expert e, in entry order.
// active[0] = number of experts with at least one row, active[1..] = their ids in order.
// `ids` is read past L1 (other blocks may have written it), or lies in shared memory (IDS_SHARED).
// `sm` holds 2 * experts ints.
template <bool IDS_SHARED = false>
__device__ __forceinline__ void plan_block(const int* ids, int n, int experts, int* __restrict__ offsets,
                                           int* __restrict__ sorted_entry, int* __restrict__ slot_of_entry,
                                           int* __restrict__ active, int* sm) {
  int* cnt = sm;
  int* base = sm + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = IDS_SHARED ? ids[i] : __ldcg(ids + i);
    if (e >= 0 && e < experts) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, n_active = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = run;
      base[e] = run;
      run += cnt[e];
      if (cnt[e] > 0) active[1 + n_active++] = e;
    }
    offsets[experts] = run;
    active[0] = n_active;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    for (int start = 0; start < n; start += 32) {
      const int i = start + lane;
      int e = i < n ? (IDS_SHARED ? ids[i] : __ldcg(ids + i)) : -1;
      if (e >= experts) e = -1;
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      if (e >= 0) {
        const int slot = base[e] + rank;
        sorted_entry[slot] = i;
        slot_of_entry[i] = slot;
      }
      __syncwarp();
      if (e >= 0 && rank == 0) base[e] += __popc(peers);
      __syncwarp();
    }
  }
}

// The same plan with every warp of the block at work, for the many entries of a prompt portion
// (plan_block ranks with one warp, whose loads of `ids` follow one another: 20 us for 2,048
// entries). Warp w takes the w-th run of entries: it counts its run's entries per expert, the runs'
// counts are scanned per expert (a run's entries follow those of the runs before it: the sort
// stays stable), and the warp then places its entries. `sm` holds (warps + 2) * experts ints.
__device__ __forceinline__ void plan_block_wide(const int* __restrict__ ids, int n, int experts,
                                                int* __restrict__ offsets, int* __restrict__ sorted_entry,
                                                int* __restrict__ slot_of_entry, int* __restrict__ active, int* sm) {
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* total = sm;                         // [experts] entries of each expert
  int* first = sm + experts;               // [experts] its first slot
  int* hist = sm + 2 * experts;            // [warps][experts] entries of the expert in a warp's run, then its next slot
  for (int i = threadIdx.x; i < warps * experts; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  const int run = ((n + warps - 1) / warps + 31) / 32 * 32;      // whole groups of 32 entries to a warp
  const int begin = warp * run, end = min(n, begin + run);
  int* mine = hist + warp * experts;
  auto walk = [&](bool place) {
    for (int start = begin; start < end; start += 64) {           // two groups' loads in flight
      int e2[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int i = start + 32 * q + lane;
        e2[q] = i < end ? ids[i] : -1;
        if (e2[q] >= experts) e2[q] = -1;
      }
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int i = start + 32 * q + lane, e = e2[q];
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        if (place && e >= 0) {
          const int slot = mine[e] + rank;
          sorted_entry[slot] = i;
          slot_of_entry[i] = slot;
        }
        __syncwarp();
        if (e >= 0 && rank == 0) mine[e] += __popc(peers);
        __syncwarp();
      }
    }
  };
  walk(false);
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int sum = 0;
    for (int w = 0; w < warps; ++w) sum += hist[w * experts + e];
    total[e] = sum;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, n_active = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = at;
      first[e] = at;
      at += total[e];
      if (total[e] > 0) active[1 + n_active++] = e;
    }
    offsets[experts] = at;
    active[0] = n_active;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {       // counts -> first slot of each warp's run
    int at = first[e];
    for (int w = 0; w < warps; ++w) {
      const int c = hist[w * experts + e];
      hist[w * experts + e] = at;
      at += c;
    }
  }
  __syncthreads();
  walk(true);
}

// ------------------------------------------------------------------ router
// logit[t, e] = sum_k x[t, k] * w[e, k] in float32. x may be float32 while the weights are
// bfloat16: the router reads the float32 output of the norm, so its logits carry no activation
// rounding of their own.
//
// Both kernels below take the sum in the SAME order, so a token's routing does not depend on
// which of them ran (how many tokens the step had): K is cut into runs of 256 elements; the runs
// form ROUTER_KPARTS consecutive parts; inside a part lane l adds elements 8l .. 8l+7 of every run
// in ascending order into one accumulator; each part is reduced over the lanes by the xor tree
// (offsets 16, 8, 4, 2, 1); the parts are added in ascending order.
constexpr int ROUTER_KPARTS = 4;

__device__ __forceinline__ void router_part_range(int hidden, int part, int& run_begin, int& run_end) {
  const int runs = (hidden + 255) / 256, per = (runs + ROUTER_KPARTS - 1) / ROUTER_KPARTS;
  run_begin = part * per;
  run_end = min(runs, run_begin + per);
}

// The k largest of a row of logits (ties to the lower id) and their scores. THROUGH_L2: the row
// was written by other blocks of this launch and is read past L1. `mode`: bit 0 clear = the sigmoid
// of the chosen logit (crates/hi-mlx/src/models.rs:6090), set = its softmax over all experts
// (the donor kernel's two scoring rules: crates/hi-cuda/src/kernels.cu:536-546); bit 1 = the chosen
// scores are divided by their sum.
constexpr int ROUTER_SOFTMAX = 1, ROUTER_RENORMALIZE = 2;

template <bool THROUGH_L2 = false>
__device__ __forceinline__ void router_select(const float* row, int experts, int top_k, int mode, int* ids,
                                              float* scores) {
  float mx = -INFINITY, denom = 1.f;
  if (mode & ROUTER_SOFTMAX) {
    for (int e = 0; e < experts; ++e) mx = fmaxf(mx, THROUGH_L2 ? __ldcg(row + e) : row[e]);
    denom = 0.f;
    for (int e = 0; e < experts; ++e) denom += expf((THROUGH_L2 ? __ldcg(row + e) : row[e]) - mx);
  }
  float chosen = 0.f;
  for (int r = 0; r < top_k; ++r) {
    int best = -1;
    float bv = 0.f;
    for (int e = 0; e < experts; ++e) {
      bool taken = false;
      for (int q = 0; q < r; ++q) taken |= (ids[q] == e);
      if (taken) continue;
      const float v = THROUGH_L2 ? __ldcg(row + e) : row[e];
      if (best < 0 || v > bv) { best = e; bv = v; }  // strict '>' keeps the lowest id on ties
    }
    ids[r] = best;
    scores[r] = (mode & ROUTER_SOFTMAX) ? expf(bv - mx) / denom : 1.f / (1.f + expf(-bv));
    chosen += scores[r];
  }
  if (mode & ROUTER_RENORMALIZE)
    for (int r = 0; r < top_k; ++r) scores[r] /= chosen;
}

// Few tokens: a block takes one token and ROUTER_FEW_EXP experts, a warp one part of K of one
// expert with up to four runs' loads in flight, so that a single token's router still spreads over
// experts / ROUTER_FEW_EXP blocks and a handful of memory round trips (it runs beside kernels that
// keep the memory system busy). With `counter` (zero between launches) the block that finishes
// last selects for every token and makes the plan; without it router_select_kernel follows.
constexpr int ROUTER_FEW_EXP = 4;

template <typename TX, typename TW>
__global__ void __launch_bounds__(ROUTER_FEW_EXP * ROUTER_KPARTS * 32)
router_few_kernel(const TX* __restrict__ x, const TW* __restrict__ w, int n, int hidden, int experts, int top_k,
                  int mode, float* logits, int* ids, float* scores, int* __restrict__ offsets,
                  int* __restrict__ sorted_entry, int* __restrict__ slot_of_entry, int* __restrict__ active,
                  int* counter) {
  __shared__ float partial[ROUTER_FEW_EXP][ROUTER_KPARTS];
  __shared__ int is_last;
  extern __shared__ int plan_scratch[];  // 2 * experts + n * top_k ints, for the block that makes the plan
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = warp % ROUTER_KPARTS, local = warp / ROUTER_KPARTS;
  const int e = blockIdx.y * ROUTER_FEW_EXP + local;
  int run_begin, run_end;
  router_part_range(hidden, part, run_begin, run_end);
  float s = 0.f;
  if (e < experts) {
    const TX* xr = x + (size_t)t * hidden;
    const TW* wr = w + (size_t)e * hidden;
    if ((hidden & 7) == 0) {   // rows are 16-byte aligned: 8 elements per load
      constexpr int U = 4;
      for (int run = run_begin; run < run_end; run += U) {
        float xv[U][8], wv[U][8];
        bool on[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = (run + u) * 256 + lane * 8;
          on[u] = run + u < run_end && j < hidden;
          if (on[u]) {
            hb::load8(xr + j, xv[u]);
            hb::load8(wr + j, wv[u]);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (on[u])
#pragma unroll
            for (int i = 0; i < 8; ++i) s += xv[u][i] * wv[u][i];
      }
    } else {                   // any width: the same order, element by element
      for (int run = run_begin; run < run_end; ++run)
        for (int i = 0; i < 8; ++i) {
          const int j = run * 256 + lane * 8 + i;
          if (j < hidden) s += hb::to_f32(xr[j]) * hb::to_f32(wr[j]);
        }
    }
  }
  s = hb::warp_sum(s);
  if (lane == 0) partial[local][part] = s;
  __syncthreads();
  if (threadIdx.x < ROUTER_FEW_EXP) {
    const int mine = blockIdx.y * ROUTER_FEW_EXP + threadIdx.x;
    if (mine < experts) {
      float total = partial[threadIdx.x][0];
#pragma unroll
      for (int q = 1; q < ROUTER_KPARTS; ++q) total += partial[threadIdx.x][q];
      logits[(size_t)t * experts + mine] = total;
    }
    __threadfence();
  }
  if (!counter) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    const int blocks = (int)(gridDim.x * gridDim.y);
    is_last = atomicAdd(counter, 1) == blocks - 1;
    if (is_last) *counter = 0;     // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // the choices go to global memory for the kernels that follow and stay in shared memory for the plan
  int* s_ids = plan_scratch + 2 * experts;          // [n * top_k]
  for (int tok = threadIdx.x; tok < n; tok += blockDim.x) {
    int* mine = s_ids + tok * top_k;
    router_select<true>(logits + (size_t)tok * experts, experts, top_k, mode, mine, scores + (size_t)tok * top_k);
    for (int r = 0; r < top_k; ++r) ids[(size_t)tok * top_k + r] = mine[r];
  }
  __syncthreads();
  plan_block<true>(s_ids, n * top_k, experts, offsets, sorted_entry, slot_of_entry, active, plan_scratch);
}

// Many tokens: a block takes ROUTER_TOK tokens x ROUTER_EXP experts with one warp per part of K;
// a lane holds its 8 elements of the four token rows in registers and walks the expert rows past
// them, four at a time, so every load is used 4 (weights) or 16 (activations) times from
// registers and nothing waits on shared memory. Needs hidden % 8 == 0. The partial sums meet in
// shared memory and are added in part order. With one block column (experts <= ROUTER_EXP) the
// block also selects; otherwise router_select_kernel does.
constexpr int ROUTER_TOK = 4, ROUTER_EXP = 16;

template <typename TW>
__global__ void __launch_bounds__(ROUTER_KPARTS * 32)
router_logits_tiled_kernel(const float* __restrict__ x, const TW* __restrict__ w, int n, int hidden, int experts,
                           int top_k, int mode, float* __restrict__ logits, int* __restrict__ ids,
                           float* __restrict__ scores) {
  __shared__ float partial[ROUTER_KPARTS][ROUTER_TOK][ROUTER_EXP];
  __shared__ float lg[ROUTER_TOK][ROUTER_EXP];
  const int lane = threadIdx.x & 31, part = threadIdx.x >> 5;
  const int t0 = blockIdx.x * ROUTER_TOK, e0 = blockIdx.y * ROUTER_EXP;
  int run_begin, run_end;
  router_part_range(hidden, part, run_begin, run_end);
  float acc[ROUTER_TOK][ROUTER_EXP];
#pragma unroll
  for (int tt = 0; tt < ROUTER_TOK; ++tt)
#pragma unroll
    for (int e = 0; e < ROUTER_EXP; ++e) acc[tt][e] = 0.f;
  for (int run = run_begin; run < run_end; ++run) {
    const int j = run * 256 + lane * 8;
    if (j >= hidden) continue;
    float xv[ROUTER_TOK][8];
#pragma unroll
    for (int tt = 0; tt < ROUTER_TOK; ++tt) {
      if (t0 + tt < n) {
        hb::load8(x + (size_t)(t0 + tt) * hidden + j, xv[tt]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) xv[tt][i] = 0.f;
      }
    }
#pragma unroll
    for (int es = 0; es < ROUTER_EXP; es += 4) {
      float wv[4][8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int e = min(e0 + es + q, experts - 1);         // rows past the last expert: computed, not used
        hb::load8(w + (size_t)e * hidden + j, wv[q]);
      }
      // two experts an instruction (fma on a pair of floats): each logit still adds its products in
      // the same order, so the sums are the ones the single fma gives
#pragma unroll
      for (int q = 0; q < 4; q += 2)
#pragma unroll
        for (int tt = 0; tt < ROUTER_TOK; ++tt) {
          float2 a2 = make_float2(acc[tt][es + q], acc[tt][es + q + 1]);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            a2 = __ffma2_rn(make_float2(xv[tt][i], xv[tt][i]), make_float2(wv[q][i], wv[q + 1][i]), a2);
          acc[tt][es + q] = a2.x;
          acc[tt][es + q + 1] = a2.y;
        }
    }
  }
#pragma unroll
  for (int tt = 0; tt < ROUTER_TOK; ++tt)
#pragma unroll
    for (int e = 0; e < ROUTER_EXP; ++e) {
      const float v = hb::warp_sum(acc[tt][e]);
      if (lane == 0) partial[part][tt][e] = v;
    }
  __syncthreads();
  if (threadIdx.x < ROUTER_TOK * ROUTER_EXP) {
    const int tt = threadIdx.x / ROUTER_EXP, e = threadIdx.x % ROUTER_EXP;
    float total = partial[0][tt][e];
#pragma unroll
    for (int q = 1; q < ROUTER_KPARTS; ++q) total += partial[q][tt][e];
    lg[tt][e] = total;
    if (logits && t0 + tt < n && e0 + e < experts) logits[(size_t)(t0 + tt) * experts + e0 + e] = total;
  }
  if (gridDim.y > 1) return;
  __syncthreads();
  if (threadIdx.x < ROUTER_TOK && t0 + threadIdx.x < n) {
    const size_t t = t0 + threadIdx.x;
    router_select(lg[threadIdx.x], experts, top_k, mode, ids + t * top_k, scores + t * top_k);
  }
}

// Selection from stored logits, one thread per token (more experts than one block column holds).
__global__ void router_select_kernel(const float* __restrict__ logits, int n, int experts, int top_k, int mode,
                                     int* __restrict__ ids, float* __restrict__ scores) {
  const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t < (size_t)n) router_select(logits + t * experts, experts, top_k, mode, ids + t * top_k, scores + t * top_k);
}

// ------------------------------------------------------------------ plan
__global__ void moe_plan_kernel(const int* ids, int n, int experts, int* __restrict__ offsets,
                                int* __restrict__ sorted_entry, int* __restrict__ slot_of_entry,
                                int* __restrict__ active, int wide) {
  extern __shared__ int plan_sm[];  // cnt[experts], base[experts]; wide: (warps + 2) * experts
  if (wide) plan_block_wide(ids, n, experts, offsets, sorted_entry, slot_of_entry, active, plan_sm);
  else plan_block(ids, n, experts, offsets, sorted_entry, slot_of_entry, active, plan_sm);
}

// One block of 1,024 threads; every warp ranks where the per-warp counts fit shared memory and there
// are entries enough for it to pay.
int launch_plan(const int* ids, int n, int experts, int* offsets, int* sorted_entry, int* slot_of_entry, int* active,
                cudaStream_t stream) {
  const size_t wide_smem = (size_t)(32 + 2) * experts * sizeof(int);
  const int wide = n >= 256 && wide_smem <= 40 * 1024;
  moe_plan_kernel<<<1, 1024, wide ? wide_smem : 2 * (size_t)experts * sizeof(int), stream>>>(
      ids, n, experts, offsets, sorted_entry, slot_of_entry, active, wide);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

// ------------------------------------------------------------------ grouped products, general form
// C[r, n] = sum_k A[row(r), k] * W[e(r), n, k] for the sorted slots r of every expert e.
// DUAL: two weight stacks (gate, up); out = silu(s*g) * (s*u) in the engine dtype.
// else: out = float32 product (the down projection).
// Tiles BM x BN over (expert, rows of that expert) x columns; any K, any number of columns.
constexpr int BM = 32, BN = 64, BK = 16, GT = 256;

template <typename T, bool DUAL>
__global__ void grouped_gemm_kernel(const T* __restrict__ A, int lda, const int* __restrict__ sorted_entry,
                                    int top_k, const T* __restrict__ W0, const T* __restrict__ W1,
                                    const int* __restrict__ offsets, int experts,
                                    const float* __restrict__ scores, void* __restrict__ out, int n_out,
                                    int K) {
  __shared__ float As[BK][BM + 1];
  __shared__ float Bs0[BK][BN + 1];
  __shared__ float Bs1[DUAL ? BK : 1][BN + 1];
  __shared__ int tile_expert, tile_row0, tile_rows;
  if (threadIdx.x == 0) {
    // blockIdx.y-th row tile in expert order
    int want = blockIdx.y, e = 0, found = -1, r0 = 0, rows = 0;
    for (; e < experts; ++e) {
      const int c = offsets[e + 1] - offsets[e];
      const int tiles = (c + BM - 1) / BM;
      if (want < tiles) {
        found = e;
        r0 = offsets[e] + want * BM;
        rows = min(BM, offsets[e + 1] - r0);
        break;
      }
      want -= tiles;
    }
    tile_expert = found; tile_row0 = r0; tile_rows = rows;
  }
  __syncthreads();
  const int e = tile_expert;
  if (e < 0) return;
  const int row0 = tile_row0, rows = tile_rows;
  const int col0 = blockIdx.x * BN;
  const T* w0 = W0 + (size_t)e * n_out * K;
  const T* w1 = DUAL ? W1 + (size_t)e * n_out * K : nullptr;

  const int tm = threadIdx.x / 16;  // 0..15 -> rows tm*2, tm*2+1
  const int tn = threadIdx.x % 16;  // 0..15 -> cols tn*4 .. tn*4+3
  float acc0[2][4] = {}, acc1[2][4] = {};

  for (int k0 = 0; k0 < K; k0 += BK) {
    // A tile: BM x BK
    for (int i = threadIdx.x; i < BM * BK; i += GT) {
      const int r = i / BK, k = i % BK;
      float v = 0.f;
      if (r < rows && k0 + k < K) {
        const int slot = row0 + r;
        const size_t arow = sorted_entry ? (size_t)(sorted_entry[slot] / top_k) : (size_t)slot;
        v = hb::to_f32(A[arow * lda + k0 + k]);
      }
      As[k][r] = v;
    }
    for (int i = threadIdx.x; i < BN * BK; i += GT) {
      const int n = i / BK, k = i % BK;
      const bool ok = col0 + n < n_out && k0 + k < K;
      Bs0[k][n] = ok ? hb::to_f32(w0[(size_t)(col0 + n) * K + k0 + k]) : 0.f;
      if (DUAL) Bs1[k][n] = ok ? hb::to_f32(w1[(size_t)(col0 + n) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float a0 = As[k][tm * 2], a1 = As[k][tm * 2 + 1];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float b = Bs0[k][tn * 4 + c];
        acc0[0][c] += a0 * b;
        acc0[1][c] += a1 * b;
        if (DUAL) {
          const float b1 = Bs1[k][tn * 4 + c];
          acc1[0][c] += a0 * b1;
          acc1[1][c] += a1 * b1;
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = tm * 2 + rr;
    if (r >= rows) continue;
    const int slot = row0 + r;
    float s = 1.f;
    if (DUAL) s = scores[sorted_entry ? sorted_entry[slot] : slot];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int n = col0 + tn * 4 + c;
      if (n >= n_out) continue;
      if (DUAL) {
        const float g = s * acc0[rr][c], u = s * acc1[rr][c];
        reinterpret_cast<T*>(out)[(size_t)slot * n_out + n] = hb::from_f32<T>(g / (1.f + expf(-g)) * u);
      } else {
        reinterpret_cast<float*>(out)[(size_t)slot * n_out + n] = acc0[rr][c];
      }
    }
  }
}

// ------------------------------------------------------------------ grouped products, few rows per expert
// Decode shape: the weights are streamed once. One warp per output column (and per pair of
// gate/up rows when DUAL), lanes stride K with 16-byte loads, UNROLL independent loads in flight
// per lane; up to RMAX rows of A share each weight load. Needs K % 8 == 0.
constexpr int RMAX = 8;
constexpr int GEMV_WARPS = 8;

template <typename T, bool DUAL, int R>
__device__ __forceinline__ void gemv_rows(const T* __restrict__ A, int lda, const int* __restrict__ sorted_entry,
                                          int top_k, const T* __restrict__ w0, const T* __restrict__ w1,
                                          const float* __restrict__ scores, void* __restrict__ out, int n_out,
                                          int K, int n, int r0, int lane) {
  // gate/up streams two weight rows per lane; the down projection has one, and needs twice the
  // unroll for as many bytes in flight (measured at three blocks per SM: 4 and 8 beat 2, 3 or 8 and 4 or 16)
  constexpr int GEMV_UNROLL = DUAL ? 4 : 8;
  const T* arow[R];
  float sc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int slot = r0 + r;
    const size_t ar = sorted_entry ? (size_t)(sorted_entry[slot] / top_k) : (size_t)slot;
    arow[r] = A + ar * lda;
    sc[r] = DUAL ? scores[sorted_entry ? sorted_entry[slot] : slot] : 1.f;
  }
  float g[R], u[R];
#pragma unroll
  for (int r = 0; r < R; ++r) { g[r] = 0.f; u[r] = 0.f; }
  // U chunks of 256 elements with all their weight loads in flight; the sums run over the
  // chunks in ascending order whatever U is
  auto chunks = [&](int k, auto unroll) {
    constexpr int U = decltype(unroll)::value;
    float wv[U][8], wu[DUAL ? U : 1][8];
#pragma unroll
    for (int q = 0; q < U; ++q) {
      hb::load8(w0 + k + 256 * q, wv[q]);
      if (DUAL) hb::load8(w1 + k + 256 * q, wu[q]);
    }
#pragma unroll
    for (int q = 0; q < U; ++q) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float av[8];
        hb::load8(arow[r] + k + 256 * q, av);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          g[r] += av[i] * wv[q][i];
          if (DUAL) u[r] += av[i] * wu[q][i];
        }
      }
    }
  };
  int k = lane * 8;
  for (; k + 256 * (GEMV_UNROLL - 1) < K; k += 256 * GEMV_UNROLL) chunks(k, std::integral_constant<int, GEMV_UNROLL>{});
  if (GEMV_UNROLL > 4)
    for (; k + 256 * 3 < K; k += 256 * 4) chunks(k, std::integral_constant<int, 4>{});
  for (; k < K; k += 256) chunks(k, std::integral_constant<int, 1>{});
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const float gs = hb::warp_sum(g[r]);
    const float us = DUAL ? hb::warp_sum(u[r]) : 0.f;
    if (lane == 0) {
      const size_t o = (size_t)(r0 + r) * n_out + n;
      if (DUAL) {
        const float gg = sc[r] * gs, uu = sc[r] * us;
        reinterpret_cast<T*>(out)[o] = hb::from_f32<T>(gg / (1.f + expf(-gg)) * uu);
      } else {
        reinterpret_cast<float*>(out)[o] = gs;
      }
    }
  }
}

template <typename T, bool DUAL>
__global__ void __launch_bounds__(GEMV_WARPS * 32, 3)   // three blocks per SM (measured: +5 % on the batch-8 step over two)
grouped_gemv_kernel(const T* __restrict__ A, int lda, const int* __restrict__ sorted_entry, int top_k,
                    const T* __restrict__ W0, const T* __restrict__ W1, const int* __restrict__ offsets,
                    const int* __restrict__ active, const float* __restrict__ scores, void* __restrict__ out,
                    int n_out, int K) {
  // blockIdx.y counts the experts that have rows; the grid has min(experts, entries) of them
  if ((int)blockIdx.y >= active[0]) return;
  const int e = active[1 + blockIdx.y];
  const int begin = offsets[e], end = offsets[e + 1];
  if (begin == end) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * GEMV_WARPS + warp;
  if (n >= n_out) return;
  const T* w0 = W0 + ((size_t)e * n_out + n) * K;
  const T* w1 = DUAL ? W1 + ((size_t)e * n_out + n) * K : nullptr;
  int r0 = begin;
  // rows in runs of 8, 4, 2, 1: every row count is covered, each weight element is reused by
  // the whole run
  for (; r0 + 8 <= end; r0 += 8)
    gemv_rows<T, DUAL, 8>(A, lda, sorted_entry, top_k, w0, w1, scores, out, n_out, K, n, r0, lane);
  if (r0 + 4 <= end) {
    gemv_rows<T, DUAL, 4>(A, lda, sorted_entry, top_k, w0, w1, scores, out, n_out, K, n, r0, lane);
    r0 += 4;
  }
  if (r0 + 2 <= end) {
    gemv_rows<T, DUAL, 2>(A, lda, sorted_entry, top_k, w0, w1, scores, out, n_out, K, n, r0, lane);
    r0 += 2;
  }
  if (r0 < end) gemv_rows<T, DUAL, 1>(A, lda, sorted_entry, top_k, w0, w1, scores, out, n_out, K, n, r0, lane);
}

template <typename T>
int launch_grouped(bool dual, const void* A, int lda, const int* sorted_entry, int top_k, const void* W0,
                   const void* W1, const int* offsets, const int* active, int experts, const float* scores, void* out,
                   int n_entries, int n_out, int K, int few_rows, cudaStream_t stream) {
  if (few_rows && K % 8 == 0 && lda % 8 == 0) {
    dim3 grid((n_out + GEMV_WARPS - 1) / GEMV_WARPS, experts < n_entries ? experts : n_entries);
    if (dual)
      grouped_gemv_kernel<T, true><<<grid, GEMV_WARPS * 32, 0, stream>>>(
          (const T*)A, lda, sorted_entry, top_k, (const T*)W0, (const T*)W1, offsets, active, scores, out, n_out, K);
    else
      grouped_gemv_kernel<T, false><<<grid, GEMV_WARPS * 32, 0, stream>>>(
          (const T*)A, lda, sorted_entry, top_k, (const T*)W0, nullptr, offsets, active, scores, out, n_out, K);
  } else {
    const int max_tiles = (n_entries + BM - 1) / BM + (experts < n_entries ? experts : n_entries);
    dim3 grid((n_out + BN - 1) / BN, max_tiles);
    if (grid.y > 65535) return HB_ERR_UNSUPPORTED;
    if (dual)
      grouped_gemm_kernel<T, true><<<grid, GT, 0, stream>>>((const T*)A, lda, sorted_entry, top_k, (const T*)W0,
                                                            (const T*)W1, offsets, experts, scores, out, n_out, K);
    else
      grouped_gemm_kernel<T, false><<<grid, GT, 0, stream>>>((const T*)A, lda, sorted_entry, top_k, (const T*)W0,
                                                             nullptr, offsets, experts, scores, out, n_out, K);
  }
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // namespace

namespace {

// The router, and with `counter` (an int that is zero between launches) the plan as well: in the
// same kernel when a block takes one token, by the plan's own kernel after the tiled one.
int router_launch(const void* x, int x_dtype, const void* w, int w_dtype, int n, int hidden, int experts, int top_k, int mode,
                  float* logits_out, int* ids, float* scores, int* offsets, int* sorted_entry, int* slot_of_entry,
                  int* active, int* counter, cudaStream_t stream) {
  if (!x || !w || !ids || !scores || n < 0 || hidden <= 0 || experts <= 0 || top_k <= 0 || top_k > experts || mode < 0 ||
      mode > 3)
    return HB_ERR_BAD_ARG;
  if (experts > 4096) return HB_ERR_UNSUPPORTED;
  if (n == 0) return HB_OK;
  if (x_dtype == HB_DTYPE_F32 && n >= 96 && hidden % 8 == 0 && (w_dtype == HB_DTYPE_F32 || w_dtype == HB_DTYPE_BF16)) {
    // many tokens (measured: faster than one block per token from about 100): register tiles of
    // 4 tokens x 16 experts; with more than 16 experts the
    // selection needs the stored logits of all block columns
    dim3 grid((n + ROUTER_TOK - 1) / ROUTER_TOK, (experts + ROUTER_EXP - 1) / ROUTER_EXP);
    if (grid.y > 1 && !logits_out) return HB_ERR_BAD_ARG;
    if (grid.y > 65535) return HB_ERR_UNSUPPORTED;
    if (w_dtype == HB_DTYPE_F32)
      router_logits_tiled_kernel<float><<<grid, ROUTER_KPARTS * 32, 0, stream>>>(
          (const float*)x, (const float*)w, n, hidden, experts, top_k, mode, logits_out, ids, scores);
    else
      router_logits_tiled_kernel<__nv_bfloat16><<<grid, ROUTER_KPARTS * 32, 0, stream>>>(
          (const float*)x, (const __nv_bfloat16*)w, n, hidden, experts, top_k, mode, logits_out, ids, scores);
    HB_LAUNCH_CHECK();
    if (grid.y > 1) {
      router_select_kernel<<<(n + 127) / 128, 128, 0, stream>>>(logits_out, n, experts, top_k, mode, ids, scores);
      HB_LAUNCH_CHECK();
    }
    if (counter) {
      if (int rc = launch_plan(ids, n * top_k, experts, offsets, sorted_entry, slot_of_entry, active, stream)) return rc;
    }
    return HB_OK;
  }
  if (!logits_out) return HB_ERR_BAD_ARG;
  // one launch does it all while the choices of all tokens fit a block's shared memory; a longer
  // step (float32 weights with an odd width, other dtypes) selects and plans in launches of their own
  const size_t fused_smem = (2 * (size_t)experts + (size_t)n * top_k) * sizeof(int);
  int* const fused = (counter && fused_smem <= 32 * 1024) ? counter : nullptr;
  const size_t smem = fused ? fused_smem : 0;
  const int threads = ROUTER_FEW_EXP * ROUTER_KPARTS * 32;
  const int columns = (experts + ROUTER_FEW_EXP - 1) / ROUTER_FEW_EXP;
  if (columns > 65535) return HB_ERR_UNSUPPORTED;
  const dim3 grid(n, columns);
  if (x_dtype == HB_DTYPE_F32 && w_dtype == HB_DTYPE_F32)
    router_few_kernel<float, float><<<grid, threads, smem, stream>>>(
        (const float*)x, (const float*)w, n, hidden, experts, top_k, mode, logits_out, ids, scores, offsets, sorted_entry,
        slot_of_entry, active, fused);
  else if (x_dtype == HB_DTYPE_F32 && w_dtype == HB_DTYPE_BF16)
    router_few_kernel<float, __nv_bfloat16><<<grid, threads, smem, stream>>>(
        (const float*)x, (const __nv_bfloat16*)w, n, hidden, experts, top_k, mode, logits_out, ids, scores, offsets,
        sorted_entry, slot_of_entry, active, fused);
  else if (x_dtype == HB_DTYPE_BF16 && w_dtype == HB_DTYPE_BF16)
    router_few_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, threads, smem, stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, n, hidden, experts, top_k, mode, logits_out, ids, scores, offsets,
        sorted_entry, slot_of_entry, active, fused);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  if (!fused) {
    router_select_kernel<<<(n + 127) / 128, 128, 0, stream>>>(logits_out, n, experts, top_k, mode, ids, scores);
    HB_LAUNCH_CHECK();
    if (counter) {
      if (int rc = launch_plan(ids, n * top_k, experts, offsets, sorted_entry, slot_of_entry, active, stream)) return rc;
    }
  }
  return HB_OK;
}

}  // namespace

extern "C" int hb_router_topk(const void* x, int x_dtype, const void* w, int w_dtype, int n, int hidden,
                              int experts, int top_k, int mode, float* logits_out, int* ids, float* scores,
                              cudaStream_t stream) {
  return router_launch(x, x_dtype, w, w_dtype, n, hidden, experts, top_k, mode, logits_out, ids, scores, nullptr, nullptr,
                       nullptr, nullptr, nullptr, stream);
}

// Router and plan in one call; `counter` is one int that the caller zeroed once and then leaves alone.
extern "C" int hb_router_plan(const void* x, int x_dtype, const void* w, int w_dtype, int n, int hidden, int experts,
                              int top_k, int mode, float* logits_out, int* ids, float* scores, int* offsets, int* sorted_entry,
                              int* slot_of_entry, int* active, int* counter, cudaStream_t stream) {
  if (!offsets || !sorted_entry || !slot_of_entry || !active || !counter) return HB_ERR_BAD_ARG;
  if (experts <= 0 || experts > 4096) return experts <= 0 ? HB_ERR_BAD_ARG : HB_ERR_UNSUPPORTED;
  if (n == 0) {  // nothing routed: an empty plan
    return launch_plan(ids, 0, experts, offsets, sorted_entry, slot_of_entry, active, stream);
  }
  return router_launch(x, x_dtype, w, w_dtype, n, hidden, experts, top_k, mode, logits_out, ids, scores, offsets,
                       sorted_entry, slot_of_entry, active, counter, stream);
}

extern "C" int hb_moe_plan(const int* ids, int n_entries, int experts, int* offsets, int* sorted_entry,
                           int* slot_of_entry, int* active, cudaStream_t stream) {
  if (!ids || !offsets || !sorted_entry || !slot_of_entry || !active || n_entries < 0 || experts <= 0)
    return HB_ERR_BAD_ARG;
  if (experts > 4096) return HB_ERR_UNSUPPORTED;
  return launch_plan(ids, n_entries, experts, offsets, sorted_entry, slot_of_entry, active, stream);
}

// gate/up with SwiGLU: act[slot, :] (engine dtype, [n_entries, inter]).
extern "C" int hb_moe_gate_up(const void* x, int dtype, const int* sorted_entry, int top_k, const void* w_gate,
                              const void* w_up, const int* offsets, const int* active, int experts,
                              const float* scores, void* act, int n_entries, int inter, int hidden, int few_rows,
                              cudaStream_t stream) {
  if (!x || !sorted_entry || !w_gate || !w_up || !offsets || !active || !scores || !act || n_entries < 0 || inter <= 0 ||
      hidden <= 0 || experts <= 0 || top_k <= 0)
    return HB_ERR_BAD_ARG;
  if (n_entries == 0) return HB_OK;
  if (dtype == HB_DTYPE_F32)
    return launch_grouped<float>(true, x, hidden, sorted_entry, top_k, w_gate, w_up, offsets, active, experts, scores, act,
                                 n_entries, inter, hidden, few_rows, stream);
  if (dtype == HB_DTYPE_BF16)
    return launch_grouped<__nv_bfloat16>(true, x, hidden, sorted_entry, top_k, w_gate, w_up, offsets, active, experts, scores,
                                         act, n_entries, inter, hidden, few_rows, stream);
  return HB_ERR_BAD_ARG;
}

// down projection: y[slot, :] float32 [n_entries, hidden].
extern "C" int hb_moe_down(const void* act, int dtype, const void* w_down, const int* offsets, const int* active,
                           int experts, float* y, int n_entries, int hidden, int inter, int few_rows,
                           cudaStream_t stream) {
  if (!act || !w_down || !offsets || !active || !y || n_entries < 0 || inter <= 0 || hidden <= 0 || experts <= 0)
    return HB_ERR_BAD_ARG;
  if (n_entries == 0) return HB_OK;
  if (dtype == HB_DTYPE_F32)
    return launch_grouped<float>(false, act, inter, nullptr, 1, w_down, nullptr, offsets, active, experts, nullptr, y,
                                 n_entries, hidden, inter, few_rows, stream);
  if (dtype == HB_DTYPE_BF16)
    return launch_grouped<__nv_bfloat16>(false, act, inter, nullptr, 1, w_down, nullptr, offsets, active, experts, nullptr, y,
                                         n_entries, hidden, inter, few_rows, stream);
  return HB_ERR_BAD_ARG;
}
