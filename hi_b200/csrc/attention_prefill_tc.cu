// Prefill attention on the 5th-generation tensor cores (tcgen05), bfloat16: portions of prompts of
// at least a tile of new tokens against the paged cache. One block = 128 consecutive new tokens
// of one request and one query head:
//   warp 0      one lane issues TMA loads: the Q tile once, then K and V tiles of 64 key positions
//               (one box per page, 128-byte swizzle): K into a ring of three and a tile ahead of V,
//               V into a ring of two (a load takes about as long as a tile's work, so with two
//               stages and K and V in turn the products waited for their K: measured 5.76 -> 5.16 ms
//               for 4,096 new tokens behind 61,440);
//   warp 1      allocates tensor memory; one lane issues S = Q K^T (tcgen05.mma, M 128, N 64) into
//               one of two S buffers and, a tile behind, O += P V (P read from tensor memory, where
//               it lies over its own S; V from shared memory as the MN-major operand), so the next
//               S is computed while the softmax works on this one;
//   warps 2..5  softmax: thread r owns row r (tensor-memory lane r): it reads its S row with
//               tcgen05.ld, masks by absolute position (causal, chunk, sliding window), keeps the
//               running max and sum in float32, rescales its O row in tensor memory when the max
//               moved, and writes P as bfloat16 back into tensor memory (tcgen05.st): the products
//               are bound by what the SM can read from shared memory, and P from there would add a
//               fifth to it.
// Every mbarrier wait is bounded; on a time-out a code goes to `status` and the block leaves
// through the common exit, where tensor memory is freed.
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "api.h"
#include "common.cuh"
#include "tc.cuh"

namespace {

constexpr int BQ = 128;          // query rows per block (UMMA M)
constexpr int KST = 3;           // K tiles in flight
constexpr int BKEYS = 64;        // key positions per tile (two blocks per SM then fit: one does MMAs while the other's softmax runs)
constexpr int THREADS = 192;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Args {
  const int* block_table;
  const int* cu_seqlens;
  const int* positions;
  __nv_bfloat16* out;
  int* status;
  int table_stride, nh, nkv, page_size, chunk, window, skip_single, box_rows;
  float scale_log2;          // softmax scale * log2(e)
  // With key_splits > 1 every (query tile, head) is `key_splits` blocks, each over its share of the
  // key tiles; a block leaves its rows unnormalised in part_acc [row][split][head_dim] with (max,
  // sum) in part_ml [row][split][2] (max in natural-log units), and hb_attention_merge combines them.
  int key_splits;
  float* part_acc;
  float* part_ml;
};

template <int HD>
__global__ void __launch_bounds__(THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const Args a) {
  constexpr int DBLK = HD / 64;                 // 64-dim blocks of a row
  constexpr int QBYTES = BQ * HD * 2, KBYTES = BKEYS * HD * 2;
  constexpr int QBLOCK = BQ * 128;              // bytes of one [128 rows x 64 elements] swizzled block of Q
  constexpr int KVBLOCK = BKEYS * 128;          // the same for a K or V tile (rows = key positions)
  constexpr int S_COLS = BKEYS;                 // columns of one S buffer
  constexpr int TMEM_COLS = 256;                // S0, S1 (64 columns each), O (HD columns)
  // No slack for aligning by hand: two blocks per SM only fit without it. The swizzled tiles need
  // a 1024-byte aligned base, which dynamic shared memory has when the kernel has no static
  // shared memory; if it ever has not, the block reports it and leaves.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((tc::smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(a.status, 19);
    return;
  }
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + QBYTES;                  // [KST stages] K tiles
  uint8_t* v_s = k_s + KST * KBYTES;            // [2 stages] V tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + 2 * KBYTES);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 3   K and V have rings of their own: a K buffer is free as soon
  uint64_t* k_empty = bars + 4;       // 3   as its S is computed, long before its V is used, and K is
  uint64_t* v_full = bars + 7;        // 2   loaded a tile ahead of V
  uint64_t* v_empty = bars + 9;       // 2
  uint64_t* s_full = bars + 11;       // 2
  uint64_t* s_free = bars + 13;       // 2
  uint64_t* p_ready = bars + 15;      // 1
  uint64_t* pv_done = bars + 16;      // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  constexpr int kst = KST;

  // Blocks start in the order x, y, z: the heads are x and the query tiles y, latest first, so
  // the tiles that read the most keys start first for every head and the short ones fill the end.
  const int seq = blockIdx.z, h = blockIdx.x % a.nh, piece = blockIdx.x / a.nh;
  const int qt = gridDim.y - 1 - blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq_begin = a.cu_seqlens[seq], seq_end = a.cu_seqlens[seq + 1];
  const int tok0 = seq_begin + qt * BQ;
  const int n_valid = min(BQ, seq_end - tok0);
  if (n_valid <= 0) return;
  // a row that this block leaves out weighs nothing in the merge
  auto no_part = [&](int row) {
    float* ml = a.part_ml + (((size_t)(tok0 + row) * a.nh + h) * a.key_splits + piece) * 2;
    ml[0] = -INFINITY;
    ml[1] = 0.f;
  };
  if (a.skip_single && seq_end - seq_begin == 1) {
    if (a.key_splits > 1 && threadIdx.x == 0) no_part(0);
    return;
  }
  const int kvh = h / (a.nh / a.nkv);
  const int p_first = a.positions[tok0];
  const int p_last = p_first + n_valid - 1;
  auto first_visible = [&](int pos) {
    int lo = 0;
    if (a.chunk > 0) lo = (pos / a.chunk) * a.chunk;
    if (a.window > 0 && pos - a.window + 1 > lo) lo = pos - a.window + 1;
    return lo;
  };
  int tile_begin = first_visible(p_first) / BKEYS;
  int nt = p_last / BKEYS - tile_begin + 1;
  if (a.key_splits > 1) {                       // this block's share of the key tiles
    const int share = (nt + a.key_splits - 1) / a.key_splits;
    tile_begin += piece * share;
    nt = min(share, nt - piece * share);
    if (nt <= 0) {
      if ((int)threadIdx.x < n_valid) no_part(threadIdx.x);
      return;
    }
  }

  if (threadIdx.x == 0) {
    tc::mbar_init(q_full, 1);
    for (int i = 0; i < KST; ++i) { tc::mbar_init(&k_full[i], 1); tc::mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&v_full[i], 1); tc::mbar_init(&v_empty[i], 1);
      tc::mbar_init(&s_full[i], 1); tc::mbar_init(&s_free[i], 4);
    }
    tc::mbar_init(p_ready, 4);
    tc::mbar_init(pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tc::alloc(tmem_slot, TMEM_COLS);
  }
  tc::fence_before();
  __syncthreads();
  tc::fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_o = tmem + 2 * S_COLS;

  if (warp == 0) {
    if (lane == 0) {                            // ---- TMA producer
      const int* table = a.block_table + (size_t)seq * a.table_stride;
      tc::mbar_expect_tx(q_full, QBYTES);
      for (int c = 0; c < DBLK; ++c) tc::tma_load_2d(q_s + c * QBLOCK, &map_q, h * HD + c * 64, tok0, q_full);
      const int boxes = BKEYS / a.box_rows;
      bool ok = true;
      // one tile of K or V: a box per page
      auto load = [&](int j, uint8_t* dst, const CUtensorMap* map, uint64_t* full) {
        tc::mbar_expect_tx(full, KBYTES);
        for (int b = 0; b < boxes; ++b) {
          const int key0 = (tile_begin + j) * BKEYS + b * a.box_rows;
          const int page = key0 <= p_last ? table[key0 / a.page_size] : -1;
          // keys past the portion's last position (or without a page) are masked: any row will do
          const int row = page >= 0 ? (page * a.nkv + kvh) * a.page_size + key0 % a.page_size : 0;
          for (int c = 0; c < DBLK; ++c) tc::tma_load_2d(dst + c * KVBLOCK + b * a.box_rows * 128, map, c * 64, row, full);
        }
      };
      auto load_k = [&](int j) {
        const int s = j % kst, use = j / kst;
        if (use >= 1 && !tc::mbar_wait(&k_empty[s], (use - 1) & 1)) { atomicExch(a.status, 11); ok = false; return; }
        load(j, k_s + s * KBYTES, &map_k, &k_full[s]);
      };
      auto load_v = [&](int j) {
        const int s = j & 1;
        if (j >= 2 && !tc::mbar_wait(&v_empty[s], ((j >> 1) - 1) & 1)) { atomicExch(a.status, 20); ok = false; return; }
        load(j, v_s + s * KBYTES, &map_v, &v_full[s]);
      };
      load_k(0);
      for (int j = 0; j < nt && ok; ++j) {          // K runs a tile ahead of V
        if (j + 1 < nt) load_k(j + 1);
        if (ok) load_v(j);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                            // ---- MMA issuer: S_j = Q K_j^T, then O += P_{j-1} V_{j-1}
      constexpr uint32_t idesc_qk = tc::idesc_bf16(BQ, BKEYS, false);
      constexpr uint32_t idesc_pv = tc::idesc_bf16(BQ, HD, true);
      bool ok = tc::mbar_wait(q_full, 0);
      if (!ok) atomicExch(a.status, 12);
      tc::fence_after();
      const uint32_t q_addr = tc::smem_u32(q_s);
      for (int j = 0; j <= nt && ok; ++j) {
        if (j < nt) {
          const int s = j & 1;
          const int ks = j % kst;
          if (!tc::mbar_wait(&k_full[ks], (j / kst) & 1)) { atomicExch(a.status, 13); ok = false; break; }
          if (j >= 2 && !tc::mbar_wait(&s_free[s], ((j >> 1) - 1) & 1)) { atomicExch(a.status, 14); ok = false; break; }
          // S_j goes where P_{j-2} lies: the product that reads that P must be through (it is the last one
          // committed to this barrier so far, so the parity is its own)
          if (j >= 2 && !tc::mbar_wait(pv_done, (j - 2) & 1)) { atomicExch(a.status, 24); ok = false; break; }
          tc::fence_after();
          const uint32_t k_addr = tc::smem_u32(k_s + ks * KBYTES);
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) {
            tc::mma(tmem + s * S_COLS, tc::desc_kmajor(q_addr + (k / 4) * QBLOCK + (k % 4) * 32),
                   tc::desc_kmajor(k_addr + (k / 4) * KVBLOCK + (k % 4) * 32), idesc_qk, k != 0);
          }
          tc::commit(&s_full[s]);
          tc::commit(&k_empty[ks]);             // the K buffer is free once these MMAs have read it
        }
        if (j >= 1) {
          const int i = j - 1, s = i & 1;
          if (!tc::mbar_wait(&v_full[s], (i >> 1) & 1)) { atomicExch(a.status, 21); ok = false; break; }
          if (!tc::mbar_wait(p_ready, i & 1)) { atomicExch(a.status, 15); ok = false; break; }
          tc::fence_after();
          const uint32_t v_addr = tc::smem_u32(v_s + s * KBYTES);
          const uint32_t p_tmem = tmem + s * S_COLS;     // P_i lies over the first half of S_i's columns
#pragma unroll
          for (int k = 0; k < BKEYS / 16; ++k) {
            tc::mma_a_tmem(tmem_o, p_tmem + k * 8, tc::desc_mnmajor(v_addr + k * 2048, KVBLOCK), idesc_pv, (i | k) != 0);
          }
          tc::commit(&v_empty[s]);
          tc::commit(pv_done);
        }
      }
    }
  } else {                                      // ---- softmax: thread = row = tensor-memory lane
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const bool row_ok = r < n_valid;
    const int pos = p_first + r;
    const int lo = first_visible(pos);
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nt && ok; ++j) {
      const int sb = j & 1;
      if (!__all_sync(0xffffffffu, tc::mbar_wait(&s_full[sb], (j >> 1) & 1))) {
        if (lane == 0) atomicExch(a.status, 16);
        ok = false;
        break;
      }
      tc::fence_after();
      const int key_base = (tile_begin + j) * BKEYS;
      // a tile every row of this warp sees whole needs no masks (most tiles of a long prompt)
      const int warp_first_pos = p_first + quarter * 32;
      const bool interior = (quarter * 32 + 31 < n_valid) && (key_base + BKEYS - 1 <= warp_first_pos) &&
                            (key_base >= first_visible(warp_first_pos + 31));
      float sv[BKEYS];
      float mx = m;
      {
        // the whole S row: both loads in flight, one wait
        uint32_t raw0[32], raw1[32];
        tc::ld32_nowait(tmem + lane_addr + sb * S_COLS, raw0);
        tc::ld32_nowait(tmem + lane_addr + sb * S_COLS + 32, raw1);
        tc::wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          sv[i] = __uint_as_float(raw0[i]);
          sv[32 + i] = __uint_as_float(raw1[i]);
        }
      }
      if (interior) {
        float top = -INFINITY;
#pragma unroll
        for (int i = 0; i < BKEYS; ++i) top = fmaxf(top, sv[i]);
        mx = fmaxf(mx, top * a.scale_log2);     // the scale is positive
      } else {
#pragma unroll
        for (int i = 0; i < BKEYS; ++i) {
          const int key = key_base + i;
          // masked scores become -inf BEFORE scaling, so the same exponential code serves both paths
          const float s = (row_ok && key <= pos && key >= lo) ? sv[i] : -INFINITY;
          sv[i] = s;
          mx = fmaxf(mx, s * a.scale_log2);
        }
      }
      // the S buffer may be overwritten by the MMA two tiles on
      tc::fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&s_free[sb]);
      // The exponentials are taken against `m`, which follows the true running max lazily: it
      // moves (and O and l are rescaled) only when some row of the warp has grown by more than
      // 2^8, so P stays below 256 and most tiles skip the pass over O. The result is the same
      // sum, scaled by a common factor that the final division removes.
      const bool move = __any_sync(0xffffffffu, mx > m + 8.f || m == -INFINITY);
      float corr = 1.f;
      if (move) {
        corr = (m == -INFINITY) ? 0.f : fast_exp2(m - mx);
        m = mx;
      }
      // p = 2^(raw * scale - m): one fused multiply-add and one ex2 per score; a masked score is
      // -inf and gives 0 (m is finite here unless the whole row is still masked)
      float sum = 0.f;
      if (m == -INFINITY) {
#pragma unroll
        for (int i = 0; i < BKEYS; ++i) sv[i] = 0.f;
      } else {
        // two scores an instruction where the hardware has it (fma and add on pairs of floats);
        // the sum runs in four chains
        const float2 scale2 = make_float2(a.scale_log2, a.scale_log2), neg_m2 = make_float2(-m, -m);
        float2 part[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int i = 0; i < BKEYS; i += 4) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const float2 x = __ffma2_rn(make_float2(sv[i + 2 * c], sv[i + 2 * c + 1]), scale2, neg_m2);
            const float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
            sv[i + 2 * c] = p.x;
            sv[i + 2 * c + 1] = p.y;
            part[c] = __fadd2_rn(part[c], p);
          }
        }
        const float2 both = __fadd2_rn(part[0], part[1]);
        sum = both.x + both.y;
      }
      l = l * corr + sum;
      if (j > 0) {
        // The previous P V product must have finished: O is stable. The wait also keeps the warps
        // and the MMA issuer within a tile of one another: that product started only after every
        // warp had handed over its P of the tile before and the issuer had seen it, so the one
        // barrier that counts the hand-overs tile after tile never runs a phase ahead of anyone.
        if (!__all_sync(0xffffffffu, tc::mbar_wait(pv_done, (j - 1) & 1))) {
          if (lane == 0) atomicExch(a.status, 17);
          ok = false;
          break;
        }
        tc::fence_after();
        if (move) {
#pragma unroll 1
          for (int c = 0; c < HD; c += 32) {
            float o[32];
            tc::ld32(tmem_o + lane_addr + c, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= corr;
            tc::st32(tmem_o + lane_addr + c, o);
          }
        }
      }
      // P row r as bfloat16 goes back into tensor memory, over the first 32 columns of the S row it
      // was made from (two keys a column): the P V product takes it from there as its A operand,
      // so P costs no shared-memory traffic. The product that read the P two tiles ago from these
      // columns ran before the Q K^T that refilled them (one thread issues them, in that order).
      {
        uint32_t packed[BKEYS / 2];
#pragma unroll
        for (int i = 0; i < BKEYS / 2; ++i) {
          __nv_bfloat162 hh = __floats2bfloat162_rn(sv[2 * i], sv[2 * i + 1]);
          packed[i] = *reinterpret_cast<uint32_t*>(&hh);
        }
        tc::st32_nowait(tmem + lane_addr + sb * S_COLS, packed);
        tc::wait_st();
      }
      if (tile_begin + j == p_last / BKEYS && (p_last + 1) % BKEYS != 0) {
        // Value rows of positions past the portion's end hold whatever the page held before
        // (another request's numbers, possibly not finite): P is zero there, but 0 x NaN is NaN.
        // Once the V tile has landed, the threads of those rows zero them.
        if (!__all_sync(0xffffffffu, tc::mbar_wait(&v_full[sb], (j >> 1) & 1))) {
          if (lane == 0) atomicExch(a.status, 22);
          ok = false;
          break;
        }
        if (r < BKEYS && key_base + r > p_last) {
          uint8_t* vrow = v_s + sb * KBYTES + (r / 8) * 1024 + (r % 8) * 128;
#pragma unroll
          for (int blk = 0; blk < DBLK; ++blk)
#pragma unroll
            for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(vrow + blk * KVBLOCK + q * 16) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA
      }
      tc::fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(p_ready);
    }
    if (ok) {
      if (!__all_sync(0xffffffffu, tc::mbar_wait(pv_done, (nt - 1) & 1))) {
        if (lane == 0) atomicExch(a.status, 18);
      } else {
        tc::fence_after();
        if (a.key_splits > 1) {
          // this share of the keys only: the row as it is, with its max and sum, for the merge
          const size_t at = ((size_t)(tok0 + r) * a.nh + h) * a.key_splits + piece;
          if (row_ok) {
            a.part_ml[at * 2] = m == -INFINITY ? -INFINITY : m * 0.6931471805599453f;
            a.part_ml[at * 2 + 1] = l;
          }
#pragma unroll 1
          for (int c = 0; c < HD; c += 32) {
            float o[32];
            tc::ld32(tmem_o + lane_addr + c, o);
            if (row_ok) {
              float4* dst4 = reinterpret_cast<float4*>(a.part_acc + at * HD + c);
#pragma unroll
              for (int i = 0; i < 8; ++i) dst4[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
            }
          }
        } else {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = a.out + ((size_t)(tok0 + r) * a.nh + h) * HD;
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          float o[32];
          tc::ld32(tmem_o + lane_addr + c, o);
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 pack;
              uint32_t* w = reinterpret_cast<uint32_t*>(&pack);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 hh = __floats2bfloat162_rn(o[i + 2 * e] * inv, o[i + 2 * e + 1] * inv);
                w[e] = *reinterpret_cast<uint32_t*>(&hh);
              }
              *reinterpret_cast<uint4*>(dst + c + i) = pack;
            }
          }
        }
        }
      }
    }
  }
  tc::fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after();
    tc::dealloc(tmem, TMEM_COLS);
  }
}

template <int HD>
int launch(const void* q, const void* k_pages, const void* v_pages, const Args& a, int n_tokens, long long pool_rows,
           int n_seqs, int max_new, cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  if (!tc::make_map_bf16(&mq, q, (uint64_t)n_tokens, (uint64_t)a.nh * HD, BQ) ||
      !tc::make_map_bf16(&mk, k_pages, (uint64_t)pool_rows, HD, a.box_rows) ||
      !tc::make_map_bf16(&mv, v_pages, (uint64_t)pool_rows, HD, a.box_rows))
    return HB_ERR_UNSUPPORTED;
  const size_t smem = (size_t)BQ * HD * 2 + (KST + 2) * (size_t)BKEYS * HD * 2 + 256;
  cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int q_tiles = (max_new + BQ - 1) / BQ;
  if (q_tiles > 65535 || n_seqs > 65535) return HB_ERR_UNSUPPORTED;
  if ((long long)a.nh * a.key_splits > 0x7fffffffLL) return HB_ERR_UNSUPPORTED;
  dim3 grid(a.nh * a.key_splits, q_tiles, n_seqs);
  attn_prefill_tc_kernel<HD><<<grid, THREADS, smem, stream>>>(mq, mk, mv, a);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // namespace

// bfloat16, head_dim 64 or 128, page_size a multiple of 16 that divides 64 or is a multiple of it.
// Arguments as hb_attention_prefill, plus the number of rows of `q`, the number of pages of the
// pools, `key_splits` (1, or how many blocks share the key tiles of a query tile and head: the rows
// then go unnormalised to `part_acc` [n_tokens * nh][key_splits][hd] and `part_ml`
// [n_tokens * nh][key_splits][2] for hb_attention_merge, and `out` is not written), and `status` (one int on the device, zero before the call; nonzero afterwards = a wait
// timed out). HB_ERR_UNSUPPORTED for other shapes: the caller uses hb_attention_prefill.
extern "C" int hb_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                       int table_stride, const int* cu_seqlens, const int* positions, void* out,
                                       int n_tokens, int n_pages, int n_seqs, int max_new, int nh, int nkv, int hd,
                                       int page_size, int chunk, int window, float scale, int skip_single,
                                       int key_splits, float* part_acc, float* part_ml, int* status,
                                       cudaStream_t stream) {
  if (!q || !k_pages || !v_pages || !block_table || !cu_seqlens || !positions || !out || !status) return HB_ERR_BAD_ARG;
  if (n_tokens < 0 || n_pages <= 0 || n_seqs < 0 || max_new < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 ||
      page_size <= 0 || table_stride <= 0 || chunk < 0 || window < 0 || key_splits < 1 || key_splits > 64 ||
      (key_splits > 1 && (!part_acc || !part_ml)))
    return HB_ERR_BAD_ARG;
  if (page_size % 16 != 0 || !(BKEYS % page_size == 0 || page_size % BKEYS == 0)) return HB_ERR_UNSUPPORTED;
  if (n_seqs > 65535 || nh > 65535) return HB_ERR_UNSUPPORTED;
  if (!(scale > 0.f)) return HB_ERR_UNSUPPORTED;       // the largest raw score is taken for the largest scaled one
  if (n_seqs == 0 || max_new == 0 || n_tokens == 0) return HB_OK;
  Args a{block_table, cu_seqlens, positions, (__nv_bfloat16*)out, status, table_stride, nh, nkv, page_size, chunk,
         window, skip_single, page_size < BKEYS ? page_size : BKEYS, scale * 1.4426950408889634f, key_splits, part_acc, part_ml};
  const long long pool_rows = (long long)n_pages * nkv * page_size;
  if (hd == 128) return launch<128>(q, k_pages, v_pages, a, n_tokens, pool_rows, n_seqs, max_new, stream);
  if (hd == 64) return launch<64>(q, k_pages, v_pages, a, n_tokens, pool_rows, n_seqs, max_new, stream);
  return HB_ERR_UNSUPPORTED;
}
