// Grouped expert products on the 5th-generation tensor cores (tcgen05), bfloat16 in, float32
// accumulation in tensor memory:
//     C[r, n] = sum_k A[r, k] * W[e(r), n, k]      for the expert-sorted rows r
// A is [rows, K] with rows already in expert order (the caller gathers the activations), W is
// [experts, n_out, K]; both K-major. Persistent blocks (one per SM) walk 128 x BN tiles:
//   warp 0      one lane issues the TMA loads (A tile 128x64, W tile BNx64, 128-byte swizzle)
//               into a ring of stages, signalled by mbarrier transaction counts;
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (M 128, N BN, K 16, four
//               per stage) and tcgen05.commit, which frees the stage / publishes the accumulator;
//   warps 2..5  read the accumulator back with tcgen05.ld (each warp its 32 lanes = 32 rows)
//               and write the epilogue, while the next tile already accumulates into the second
//               buffer of tensor memory:
//     DUAL   two weight stacks (gate, up), two accumulators: act = silu(s*g) * (s*u), bfloat16,
//            where s is the row's router score (crates/hi-mlx/src/models.rs:6086-6100: the score
//            scales the expert input, which is the same by linearity);
//     else   the float32 product (down projection).
// Rows of a tile past the expert's last row belong to the next expert (or are zero fill): they
// are computed and not stored. Every wait on an mbarrier is bounded; on a time-out the kernel
// records where it gave up in `status` and leaves through the common exit (tensor memory is
// freed there).
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include <cstdlib>
#include "api.h"
#include "common.cuh"
#include "tc.cuh"

namespace {

constexpr int BM = 128;          // rows of a tile (UMMA M)
constexpr int BK = 64;           // k elements per stage: 128 bytes, one swizzle span
constexpr int UK = 16;           // k of one tcgen05.mma
constexpr int THREADS = 192;

struct Params {
  const int* offsets;        // [experts + 1] first sorted row of every expert
  const int* sorted_entry;   // [rows] entry of each sorted row (DUAL: to find the score)
  const float* scores;       // [entries]
  void* out;                 // DUAL: bfloat16 [rows, n_out]; else float [rows, n_out]
  int* status;               // 0, or a code of the wait that timed out
  int experts, n_out, K, rows;
};

// Tile t of the launch, in the order (expert, column tile, row tile of the expert): tiles that
// share a weight tile are neighbours, so they run at the same time and the weight tile comes from
// HBM once. Returns false past the last tile. `n_tiles` = column tiles.
struct Tile { int expert, row0, rows, n0; };
template <int BN>
__device__ __forceinline__ bool find_tile(const int* offsets, int experts, int t, int n_tiles, Tile& out) {
  for (int e = 0; e < experts; ++e) {
    const int begin = offsets[e], cnt = offsets[e + 1] - begin;
    const int m_tiles = (cnt + BM - 1) / BM;
    const int here = m_tiles * n_tiles;
    if (t < here) {
      const int nt = t / m_tiles, mt = t - nt * m_tiles;
      out.expert = e;
      out.row0 = begin + mt * BM;
      out.rows = min(BM, cnt - mt * BM);
      out.n0 = nt * BN;
      return true;
    }
    t -= here;
  }
  return false;
}

// Persistent: each block walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... The shared-memory
// ring runs on across tiles; tensor memory holds TWO accumulator buffers, so the epilogue of one
// tile overlaps the loads and MMAs of the next.
template <int BN, bool DUAL, int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w0,
                       const __grid_constant__ CUtensorMap map_w1, const Params p) {
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + (DUAL ? 2 : 1) * B_BYTES;
  constexpr int ACC_COLS = DUAL ? 2 * BN : BN;       // columns of one accumulator buffer
  constexpr int TMEM_COLS = 2 * ACC_COLS;
  static_assert(TMEM_COLS == 64 || TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;               // [2]
  uint64_t* acc_empty = acc_full + 2;                // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  int* s_offsets = reinterpret_cast<int*>(tmem_slot + 2);   // [experts + 1]: the tile search never waits on global memory

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e <= p.experts; e += THREADS) s_offsets[e] = p.offsets[e];
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { tc::mbar_init(&acc_full[b], 1); tc::mbar_init(&acc_empty[b], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {                              // tensor memory for the two accumulator buffers
    tc::alloc(tmem_slot, TMEM_COLS);
  }
  tc::fence_before();
  __syncthreads();
  tc::fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n_tiles = (p.n_out + BN - 1) / BN;
  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    if (lane == 0) {                            // ---- TMA producer
      uint32_t it = 0;                          // stages filled so far, over all tiles
      bool ok = true;
      Tile tile;
      for (int t = blockIdx.x; ok && find_tile<BN>(s_offsets, p.experts, t, n_tiles, tile); t += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !tc::mbar_wait(&empty[s], ((it / STAGES) - 1) & 1)) { atomicExch(p.status, 1); ok = false; break; }
          uint8_t* st = smem + s * STAGE_BYTES;
          tc::mbar_expect_tx(&full[s], STAGE_BYTES);
          tc::tma_load_2d(st, &map_a, kb * BK, tile.row0, &full[s]);
          tc::tma_load_2d(st + A_BYTES, &map_w0, kb * BK, tile.expert * p.n_out + tile.n0, &full[s]);
          if (DUAL) tc::tma_load_2d(st + A_BYTES + B_BYTES, &map_w1, kb * BK, tile.expert * p.n_out + tile.n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                            // ---- MMA issuer
      constexpr uint32_t idesc = tc::idesc_bf16(BM, BN, false);
      uint32_t it = 0, local = 0;
      bool ok = true;
      Tile tile;
      for (int t = blockIdx.x; ok && find_tile<BN>(s_offsets, p.experts, t, n_tiles, tile); t += gridDim.x, ++local) {
        const int b = local & 1;
        const uint32_t use = local >> 1;
        if (use > 0 && !tc::mbar_wait(&acc_empty[b], (use - 1) & 1)) { atomicExch(p.status, 4); ok = false; break; }
        tc::fence_after();
        const uint32_t acc = tmem + b * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!tc::mbar_wait(&full[s], (it / STAGES) & 1)) { atomicExch(p.status, 2); ok = false; break; }
          tc::fence_after();
          const uint32_t a_addr = tc::smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t ad = tc::desc_kmajor(a_addr + k * UK * 2);
            tc::mma(acc, ad, tc::desc_kmajor(b_addr + k * UK * 2), idesc, (kb | k) != 0);
            if (DUAL) tc::mma(acc + BN, ad, tc::desc_kmajor(b_addr + B_BYTES + k * UK * 2), idesc, (kb | k) != 0);
          }
          tc::commit(&empty[s]);                 // the stage is free once these MMAs have read it
        }
        tc::commit(&acc_full[b]);                // this tile's accumulator is complete (also on the error path)
      }
    }
  } else {                                      // ---- epilogue: warps 2..5, lanes 32*(warp % 4) ..
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;          // row of the tile = lane of tensor memory
    uint32_t local = 0;
    bool ok = true;
    Tile tile;
    for (int t = blockIdx.x; ok && find_tile<BN>(s_offsets, p.experts, t, n_tiles, tile); t += gridDim.x, ++local) {
      const int b = local & 1;
      const bool waited = __all_sync(0xffffffffu, tc::mbar_wait(&acc_full[b], (local >> 1) & 1));
      if (!waited) {
        if (lane == 0) atomicExch(p.status, 3);
        ok = false;
        break;
      }
      tc::fence_after();
      const bool row_ok = r < tile.rows;
      const size_t grow = (size_t)(tile.row0 + r);
      float score = 1.f;
      if (DUAL && row_ok) score = p.scores[p.sorted_entry[tile.row0 + r]];
      const uint32_t lane_base = tmem + b * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      const int n0 = tile.n0;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        float g[32];
        tc::ld32(lane_base + c, g);
        if (DUAL) {
          float u[32];
          tc::ld32(lane_base + BN + c, u);
          if (row_ok) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + grow * p.n_out + n0 + c;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (n0 + c + i < p.n_out) {       // n_out is a multiple of 8: the 8 columns are in or out together
                uint4 pack;
                uint32_t* w = reinterpret_cast<uint32_t*>(&pack);
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                  const float g0 = score * g[i + j], g1 = score * g[i + j + 1];
                  const float a0 = g0 / (1.f + expf(-g0)) * (score * u[i + j]);
                  const float a1 = g1 / (1.f + expf(-g1)) * (score * u[i + j + 1]);
                  __nv_bfloat162 h = __floats2bfloat162_rn(a0, a1);
                  w[j >> 1] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(dst + i) = pack;
              }
            }
          }
        } else if (row_ok) {
          float* dst = reinterpret_cast<float*>(p.out) + grow * p.n_out + n0 + c;
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            if (n0 + c + i < p.n_out)           // n_out is a multiple of 8
              *reinterpret_cast<float4*>(dst + i) = make_float4(g[i], g[i + 1], g[i + 2], g[i + 3]);
        }
      }
      // this warp is done reading the buffer: the MMA issuer may overwrite it two tiles on
      tc::fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&acc_empty[b]);
    }
  }
  tc::fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after();
    tc::dealloc(tmem, TMEM_COLS);
  }
}

// rows of x in expert-sorted order: xs[r, :] = x[sorted_entry[r] / top_k, :]
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted_entry, int top_k,
                                   __nv_bfloat16* __restrict__ xs, int hidden) {
  const size_t r = blockIdx.x;
  const size_t src = (size_t)(sorted_entry[r] / top_k);
  const uint4* s = reinterpret_cast<const uint4*>(x + src * hidden);
  uint4* d = reinterpret_cast<uint4*>(xs + r * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) d[i] = s[i];
}

template <int BN, bool DUAL, int STAGES>
int launch(const void* a, const void* w0, const void* w1, const Params& p, int max_tiles, cudaStream_t stream) {
  CUtensorMap ma, mw0, mw1;
  if (!tc::make_map_bf16(&ma, a, (uint64_t)p.rows, (uint64_t)p.K, BM) ||
      !tc::make_map_bf16(&mw0, w0, (uint64_t)p.experts * p.n_out, (uint64_t)p.K, BN) ||
      !tc::make_map_bf16(&mw1, DUAL ? w1 : w0, (uint64_t)p.experts * p.n_out, (uint64_t)p.K, BN))
    return HB_ERR_UNSUPPORTED;
  constexpr int STAGE_BYTES = BM * BK * 2 + (DUAL ? 2 : 1) * BN * BK * 2;
  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024 + 256 + 4 * ((size_t)p.experts + 1);
  if (smem > 227 * 1024) return HB_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_tc_kernel<BN, DUAL, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return (int)e;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return HB_ERR_BAD_ARG;
  const long long upper = (long long)max_tiles * ((p.n_out + BN - 1) / BN);    // tiles there can be at most
  int grid = (int)(upper < sms ? upper : sms);                            // one persistent block per SM
  if (const char* lim = getenv("HB_TC_GRID")) { int g = atoi(lim); if (g > 0 && g < grid) grid = g; }
  grouped_gemm_tc_kernel<BN, DUAL, STAGES><<<grid, THREADS, smem, stream>>>(ma, mw0, mw1, p);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // namespace

extern "C" int hb_gather_rows(const void* x, const int* sorted_entry, int top_k, void* xs, int rows, int hidden,
                              cudaStream_t stream) {
  if (!x || !sorted_entry || !xs || rows < 0 || hidden <= 0 || hidden % 8 != 0 || top_k <= 0) return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  gather_rows_kernel<<<rows, 128, 0, stream>>>((const __nv_bfloat16*)x, sorted_entry, top_k, (__nv_bfloat16*)xs, hidden);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

// gate/up with SwiGLU on tensor cores: xs [rows, hidden] sorted rows -> act [rows, inter].
// `status` is one int on the device, zero before the call; nonzero afterwards = a wait timed out.
extern "C" int hb_moe_gate_up_tc(const void* xs, const int* sorted_entry, const void* w_gate, const void* w_up,
                                 const int* offsets, int experts, const float* scores, void* act, int rows, int inter,
                                 int hidden, int* status, cudaStream_t stream) {
  if (!xs || !sorted_entry || !w_gate || !w_up || !offsets || !scores || !act || !status || rows < 0 || experts <= 0)
    return HB_ERR_BAD_ARG;
  if (hidden % 8 != 0 || inter % 8 != 0 || hidden <= 0 || inter <= 0) return HB_ERR_UNSUPPORTED;
  if (rows == 0) return HB_OK;
  const int max_tiles = (rows + BM - 1) / BM + (experts < rows ? experts : rows);
  if (max_tiles > 65535) return HB_ERR_UNSUPPORTED;
  Params p{offsets, sorted_entry, scores, act, status, experts, inter, hidden, rows};
  return launch<128, true, 4>(xs, w_gate, w_up, p, max_tiles, stream);
}

// down projection on tensor cores: act [rows, inter] -> y float32 [rows, hidden].
extern "C" int hb_moe_down_tc(const void* act, const void* w_down, const int* offsets, int experts, float* y, int rows,
                              int hidden, int inter, int* status, cudaStream_t stream) {
  if (!act || !w_down || !offsets || !y || !status || rows < 0 || experts <= 0) return HB_ERR_BAD_ARG;
  if (hidden % 8 != 0 || inter % 8 != 0 || hidden <= 0 || inter <= 0) return HB_ERR_UNSUPPORTED;
  if (rows == 0) return HB_OK;
  const int max_tiles = (rows + BM - 1) / BM + (experts < rows ? experts : rows);
  if (max_tiles > 65535) return HB_ERR_UNSUPPORTED;
  Params p{offsets, nullptr, nullptr, y, status, experts, hidden, inter, rows};
  return launch<256, false, 4>(act, w_down, nullptr, p, max_tiles, stream);
}
