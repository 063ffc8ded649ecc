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

#include "api.h"
#include "common.cuh"

namespace {

constexpr int BM = 128;          // rows of a tile (UMMA M)
constexpr int BK = 64;           // k elements per stage: 128 bytes, one swizzle span
constexpr int UK = 16;           // k of one tcgen05.mma
constexpr int THREADS = 192;
constexpr uint32_t SPIN_LIMIT = 1u << 24;

// ---- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false after SPIN_LIMIT polls (about a second), never an endless spin.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
    if (mbar_test(bar, parity)) return true;
    if (i > 64) __nanosleep(40);
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled tile whose rows are 128 bytes:
// start address, stride between 8-row groups = 1024 bytes, version 1, layout SWIZZLE_128B.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);          // bits 0-13: address / 16
  d |= (uint64_t)1 << 16;                           // bits 16-29: leading byte offset / 16 (unused for this layout)
  d |= (uint64_t)(1024 >> 4) << 32;                 // bits 32-45: stride byte offset / 16
  d |= (uint64_t)1 << 46;                           // bits 46-47: descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                           // bits 61-63: SWIZZLE_128B
  return d;
}
// Instruction descriptor, kind::f16: D float32, A and B bfloat16, both K-major, N and M.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct Params {
  const int* offsets;        // [experts + 1] first sorted row of every expert
  const int* sorted_entry;   // [rows] entry of each sorted row (DUAL: to find the score)
  const float* scores;       // [entries]
  void* out;                 // DUAL: bfloat16 [rows, n_out]; else float [rows, n_out]
  int* status;               // 0, or a code of the wait that timed out
  int experts, n_out, K, rows;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

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
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {                              // tensor memory for the two accumulator buffers
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
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
          if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1)) { atomicExch(p.status, 1); ok = false; break; }
          uint8_t* st = smem + s * STAGE_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          tma_load_2d(st, &map_a, kb * BK, tile.row0, &full[s]);
          tma_load_2d(st + A_BYTES, &map_w0, kb * BK, tile.expert * p.n_out + tile.n0, &full[s]);
          if (DUAL) tma_load_2d(st + A_BYTES + B_BYTES, &map_w1, kb * BK, tile.expert * p.n_out + tile.n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                            // ---- MMA issuer
      constexpr uint32_t idesc = instr_desc(BM, BN);
      uint32_t it = 0, local = 0;
      bool ok = true;
      Tile tile;
      for (int t = blockIdx.x; ok && find_tile<BN>(s_offsets, p.experts, t, n_tiles, tile); t += gridDim.x, ++local) {
        const int b = local & 1;
        const uint32_t use = local >> 1;
        if (use > 0 && !mbar_wait(&acc_empty[b], (use - 1) & 1)) { atomicExch(p.status, 4); ok = false; break; }
        tc_fence_after();
        const uint32_t acc = tmem + b * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&full[s], (it / STAGES) & 1)) { atomicExch(p.status, 2); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t ad = smem_desc(a_addr + k * UK * 2);
            tc_mma(acc, ad, smem_desc(b_addr + k * UK * 2), idesc, (kb | k) != 0);
            if (DUAL) tc_mma(acc + BN, ad, smem_desc(b_addr + B_BYTES + k * UK * 2), idesc, (kb | k) != 0);
          }
          tc_commit(&empty[s]);                 // the stage is free once these MMAs have read it
        }
        tc_commit(&acc_full[b]);                // this tile's accumulator is complete (also on the error path)
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
      const bool waited = __all_sync(0xffffffffu, mbar_wait(&acc_full[b], (local >> 1) & 1));
      if (!waited) {
        if (lane == 0) atomicExch(p.status, 3);
        ok = false;
        break;
      }
      tc_fence_after();
      const bool row_ok = r < tile.rows;
      const size_t grow = (size_t)(tile.row0 + r);
      float score = 1.f;
      if (DUAL && row_ok) score = p.scores[p.sorted_entry[tile.row0 + r]];
      const uint32_t lane_base = tmem + b * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      const int n0 = tile.n0;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        float g[32];
        tc_ld32(lane_base + c, g);
        if (DUAL) {
          float u[32];
          tc_ld32(lane_base + BN + c, u);
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
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

// ---- tensor maps (the driver's encoder, looked up through the runtime: no link against libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}
// [rows, K] bfloat16 row-major, box [box_rows, 64], 128-byte swizzle, zero fill outside.
int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return HB_ERR_UNSUPPORTED;
  const cuuint64_t dims[2] = {K, rows};
  const cuuint64_t strides[1] = {K * 2};
  const cuuint32_t box[2] = {BK, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? HB_OK : HB_ERR_BAD_ARG;
}

template <int BN, bool DUAL, int STAGES>
int launch(const void* a, const void* w0, const void* w1, const Params& p, int max_tiles, cudaStream_t stream) {
  CUtensorMap ma, mw0, mw1;
  int rc = make_map(&ma, a, (uint64_t)p.rows, (uint64_t)p.K, BM);
  if (rc != HB_OK) return rc;
  rc = make_map(&mw0, w0, (uint64_t)p.experts * p.n_out, (uint64_t)p.K, BN);
  if (rc != HB_OK) return rc;
  rc = make_map(&mw1, DUAL ? w1 : w0, (uint64_t)p.experts * p.n_out, (uint64_t)p.K, BN);
  if (rc != HB_OK) return rc;
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
  const int grid = (int)(upper < sms ? upper : sms);                            // one persistent block per SM
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
