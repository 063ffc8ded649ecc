// Grouped expert products on the 5th-generation tensor cores (tcgen05), bfloat16 in, float32
// accumulation in tensor memory:
//     C[r, f] = sum_k X[r, k] * W[e(r), f, k]      for the expert-sorted rows r
// X is [rows, K] with rows already in expert order (the caller gathers the activations), W is
// [experts, n_out, K]; both K-major. The product is taken TRANSPOSED: the 128 weight rows of a
// tile are the MMA's M, the expert's tokens its N. N follows the number of tokens the expert
// really has (rounded up to 16, at most 192 per tile), so an expert with 5 or 140 tokens costs
// 16 or 144 columns of tensor-core time, and a weight tile is brought into the SM once for up
// to 192 tokens. What bounds these products is how many weight bytes a block has in flight: a
// stage is 32 KB of weights (DUAL) beside at most 24 KB of tokens, four stages deep; in
// decode-sized steps a tile holds at most 64 tokens (8 KB) and the ring is five / eight stages
// deep (measured at 64 tokens over 16 experts: 427 -> 415 us and 235 -> 222 us).
// Persistent blocks (one per SM) walk the tiles (expert, 128 features, up to 192 tokens):
//   warp 0      one lane issues the TMA loads (W tile 128x64, twice when DUAL; X tile of 32, 64,
//               128 or 192 rows x 64; 128-byte swizzle) into a ring of stages, signalled by
//               mbarrier transaction counts;
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (M 128, N tokens, K 16, four
//               per stage and weight stack) and tcgen05.commit, which frees the stage / publishes
//               the accumulator;
//   warps 2..9  read the accumulator back with tcgen05.ld (each warp 32 lanes = 32 features, the
//               columns are tokens; two warps share a lane quarter and take alternate runs of 32
//               tokens) and write the epilogue:
//     DUAL   two weight stacks (gate, up), two accumulators: act = silu(s*g) * (s*u), bfloat16,
//            where s is the token's router score (crates/hi-mlx/src/models.rs:6086-6100: the score
//            scales the expert input, which is the same by linearity);
//     else   the float32 product (down projection).
// Tensor memory is two slots of 256 columns. A tile takes one slot, and the next tile
// accumulates into the other while this one is written out; only a DUAL tile of more than 128
// tokens needs both (gate in one, up in the other), and its epilogue gives them back as soon as
// the results are in registers, before it stores them.
// A down projection whose tiles do not fill the last round over the SMs cuts the tiles of that
// round along K into up to four pieces, one block each: a piece leaves its float32 partial tile in
// scratch memory and counts itself in; the piece that arrives last adds the pieces in their fixed
// order and stores the sum (the result does not depend on which one that was), and puts the
// counter back to zero for the next launch.
// Token rows of an X tile past the expert's last token belong to the next expert (or are zero
// fill), weight rows past n_out to the next expert: they are computed and not stored. Every
// wait on an mbarrier is bounded; on a time-out the kernel records where it gave up in `status`
// and leaves through the common exit (tensor memory is freed there).
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "api.h"
#include "common.cuh"
#include "tc.cuh"

namespace {

constexpr int BF = 128;          // features (weight rows) of a tile: UMMA M
constexpr int BT_LONG = 192;     // most tokens of a tile (UMMA N; the X tile of a stage is BT x 64) in steps of many
constexpr int SHORT_STEP_ROWS = 256;   // steps of up to this many routed rows use BT_SHORT
constexpr int BT_SHORT = 64;     // tokens, and in decode-sized steps: less room for tokens, more stages of weights
constexpr int SLOT_COLS = 256;   // tensor memory is two slots of 256 columns
constexpr int TMEM_COLS = 2 * SLOT_COLS;
constexpr int DUAL_SLOT_T = 128; // a DUAL tile of up to this many tokens has both accumulators in one slot
constexpr int BK = 64;           // k elements per stage: 128 bytes, one swizzle span
constexpr int UK = 16;           // k of one tcgen05.mma
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + EPI_WARPS * 32;

struct Params {
  const int* offsets;        // [experts + 1] first sorted row of every expert
  const int* sorted_entry;   // [rows] entry of each sorted row (DUAL: to find the score)
  const float* scores;       // [entries]
  void* out;                 // DUAL: bfloat16 [rows, n_out]; else float [rows, n_out]
  int* status;               // 0, or a code of the wait that timed out
  int experts, n_out, K, rows;
  float* scratch;            // not DUAL: [blocks of the launch][BT][BF] partial tiles of the last round's pieces, or null
  int* counters;             // [blocks of the launch] pieces of each cut tile that have arrived; zero between launches
};
constexpr int MAX_PIECES = 4;    // a tile of the last round is cut into at most this many pieces
constexpr int MIN_PIECE_KB = 8;  // of at least this many k blocks (512 k elements)

__host__ __device__ constexpr int x_box_rows(int box, int bt) {
  const int rows = box == 0 ? 32 : (box == 1 ? 64 : (box == 2 ? 128 : bt));
  return rows < bt ? rows : bt;
}

struct Maps {                // X boxes of 32, 64, 128 and 192 rows; the weight stacks
  CUtensorMap x[4];
  CUtensorMap w0, w1;
};

// Tile t of the launch, in the order (expert, feature tile, token tile of the expert): tiles that
// share a weight tile are neighbours, so they run at the same time and the weight tile comes from
// HBM once. Returns false past the last tile. `f_tiles` = feature tiles.
struct Tile { int expert, row0, tokens, f0; };
template <int BT>
__device__ __forceinline__ bool find_tile(const int* offsets, int experts, int t, int f_tiles, Tile& out) {
  for (int e = 0; e < experts; ++e) {
    const int begin = offsets[e], cnt = offsets[e + 1] - begin;
    const int t_tiles = (cnt + BT - 1) / BT;
    const int here = t_tiles * f_tiles;
    if (t < here) {
      const int ft = t / t_tiles, tt = t - ft * t_tiles;
      const int per = (cnt + t_tiles - 1) / t_tiles;      // the expert's tokens in equal shares
      out.expert = e;
      out.row0 = begin + tt * per;
      out.tokens = min(per, cnt - tt * per);
      out.f0 = ft * BF;
      return true;
    }
    t -= here;
  }
  return false;
}

// The work of a block, in order: its tiles of the full rounds (blockIdx.x, blockIdx.x + gridDim.x,
// ...), then its share of the last, partly filled round: a whole tile, or piece `piece` of `pieces`
// of cut tile number `cut` (k blocks kb0 .. kb1). Every role of the block walks the same list.
struct Work { Tile tile; int kb0, kb1, cut, piece, pieces; };
template <int BT>
struct WorkList {
  const int* offsets;
  int experts, f_tiles, num_kb, rounds, rest, pieces, per;
  __device__ WorkList(const int* offsets_, int experts_, int f_tiles_, int num_kb_, bool may_cut)
      : offsets(offsets_), experts(experts_), f_tiles(f_tiles_), num_kb(num_kb_) {
    int tiles = 0;
    for (int e = 0; e < experts; ++e) tiles += (offsets[e + 1] - offsets[e] + BT - 1) / BT * f_tiles;
    rounds = tiles / (int)gridDim.x;
    rest = tiles - rounds * (int)gridDim.x;
    pieces = 1;
    per = num_kb;
    if (may_cut && rest > 0) {
      int want = min(min(MAX_PIECES, (int)gridDim.x / rest), num_kb / MIN_PIECE_KB);
      if (want > 1) {
        per = (num_kb + want - 1) / want;
        pieces = (num_kb + per - 1) / per;          // no piece is empty
      }
    }
  }
  __device__ __forceinline__ bool get(int i, Work& w) const {
    w.kb0 = 0; w.kb1 = num_kb; w.cut = -1; w.piece = 0; w.pieces = 1;
    if (i < rounds) return find_tile<BT>(offsets, experts, (int)blockIdx.x + i * (int)gridDim.x, f_tiles, w.tile);
    if (i > rounds) return false;
    const int b = (int)blockIdx.x;
    if (pieces == 1) return b < rest && find_tile<BT>(offsets, experts, rounds * (int)gridDim.x + b, f_tiles, w.tile);
    if (b >= rest * pieces) return false;
    w.cut = b / pieces;                              // the pieces of one tile are neighbours: they share its tokens
    w.piece = b - w.cut * pieces;
    w.pieces = pieces;
    w.kb0 = w.piece * per;
    w.kb1 = min(num_kb, w.kb0 + per);
    return find_tile<BT>(offsets, experts, rounds * (int)gridDim.x + w.cut, f_tiles, w.tile);
  }
};

// The walk over a block's tiles that the MMA issuer and the epilogue warps share: which slot(s)
// of tensor memory a tile takes, and how often each slot has been used before.
struct SlotWalk {
  uint32_t use[2] = {0, 0};
  int next = 0;
  // returns the first slot of the tile; `both` = the tile takes the two of them
  __device__ __forceinline__ int take(bool dual, int tokens, bool& both) {
    both = dual && tokens > DUAL_SLOT_T;
    if (both) return 0;
    const int b = next;
    next ^= 1;
    return b;
  }
};

// Persistent: each block walks its work list. The shared-memory ring runs on across tiles.
template <bool DUAL, int STAGES, int BT>
__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm_tc_kernel(const __grid_constant__ Maps maps, const Params p) {
  constexpr int W_BYTES = BF * BK * 2, X_BYTES = BT * BK * 2;
  constexpr int NW = DUAL ? 2 : 1;
  constexpr int STAGE_BYTES = NW * W_BYTES + X_BYTES;
  static_assert(BT <= SLOT_COLS && 2 * DUAL_SLOT_T <= SLOT_COLS, "a slot holds one accumulator of any tile");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;               // [2]
  uint64_t* acc_empty = acc_full + 2;                // [2]
  uint64_t* cut_bar = acc_empty + 2;                 // [2]: a piece's partial tile is written; whether it came last is known
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(cut_bar + 2);
  int* s_last = reinterpret_cast<int*>(tmem_slot + 2);      // whether this block's piece arrived last
  int* s_offsets = s_last + 1;                              // [experts + 1]: the tile search never waits on global memory

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e <= p.experts; e += THREADS) s_offsets[e] = p.offsets[e];
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { tc::mbar_init(&acc_full[b], 1); tc::mbar_init(&acc_empty[b], EPI_WARPS); }
    tc::mbar_init(&cut_bar[0], EPI_WARPS);
    tc::mbar_init(&cut_bar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {                              // tensor memory for the two slots
    tc::alloc(tmem_slot, TMEM_COLS);
  }
  tc::fence_before();
  __syncthreads();
  tc::fence_after();
  const uint32_t tmem = *tmem_slot;
  const int f_tiles = (p.n_out + BF - 1) / BF;
  const int num_kb = (p.K + BK - 1) / BK;
  const WorkList<BT> list(s_offsets, p.experts, f_tiles, num_kb, !DUAL && p.scratch != nullptr);

  if (warp == 0) {
    if (lane == 0) {                            // ---- TMA producer
      uint32_t it = 0;                          // stages filled so far, over all tiles
      bool ok = true;
      Work work;
      for (int i = 0; ok && list.get(i, work); ++i) {
        const Tile& tile = work.tile;
        const int box = tile.tokens <= 32 ? 0 : (tile.tokens <= 64 ? 1 : (tile.tokens <= 128 ? 2 : 3));
        const uint32_t bytes = NW * W_BYTES + (uint32_t)x_box_rows(box, BT) * BK * 2;
        const int w_row = tile.expert * p.n_out + tile.f0;
        for (int kb = work.kb0; kb < work.kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !tc::mbar_wait(&empty[s], ((it / STAGES) - 1) & 1)) { atomicExch(p.status, 1); ok = false; break; }
          uint8_t* st = smem + s * STAGE_BYTES;
          tc::mbar_expect_tx(&full[s], bytes);
          tc::tma_load_2d(st, &maps.w0, kb * BK, w_row, &full[s]);
          if (DUAL) tc::tma_load_2d(st + W_BYTES, &maps.w1, kb * BK, w_row, &full[s]);
          tc::tma_load_2d(st + NW * W_BYTES, &maps.x[box], kb * BK, tile.row0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                            // ---- MMA issuer
      uint32_t it = 0;
      SlotWalk walk;
      bool ok = true;
      Work work;
      for (int i = 0; ok && list.get(i, work); ++i) {
        const Tile& tile = work.tile;
        bool both;
        const int b = walk.take(DUAL, tile.tokens, both);
        for (int q = b; ok && q <= (both ? 1 : b); ++q)      // the slot(s) must have been written out
          if (walk.use[q] > 0 && !tc::mbar_wait(&acc_empty[q], (walk.use[q] - 1) & 1)) { atomicExch(p.status, 4); ok = false; }
        if (!ok) break;
        tc::fence_after();
        const uint32_t idesc = tc::idesc_bf16(BF, (tile.tokens + 15) & ~15, false);
        const uint32_t acc = tmem + b * SLOT_COLS;
        const uint32_t up_off = both ? SLOT_COLS : DUAL_SLOT_T;  // where the second accumulator starts
        const int kb0 = work.kb0;
        for (int kb = kb0; kb < work.kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!tc::mbar_wait(&full[s], (it / STAGES) & 1)) { atomicExch(p.status, 2); ok = false; break; }
          tc::fence_after();
          const uint32_t w_addr = tc::smem_u32(smem + s * STAGE_BYTES);
          const uint32_t x_addr = w_addr + NW * W_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t xd = tc::desc_kmajor(x_addr + k * UK * 2);
            tc::mma(acc, tc::desc_kmajor(w_addr + k * UK * 2), xd, idesc, (kb - kb0) | k);
            if (DUAL) tc::mma(acc + up_off, tc::desc_kmajor(w_addr + W_BYTES + k * UK * 2), xd, idesc, (kb - kb0) | k);
          }
          tc::commit(&empty[s]);                 // the stage is free once these MMAs have read it
        }
        // this tile's accumulator is complete (also on the error path)
        tc::commit(&acc_full[b]);
        ++walk.use[b];
        if (both) { tc::commit(&acc_full[1]); ++walk.use[1]; }
      }
    }
  } else {                                      // ---- epilogue: warps 2..9
    const int quarter = warp & 3;               // the lanes of tensor memory this warp may read
    const int half = (warp - 2) >> 2;           // which runs of 32 tokens it takes
    SlotWalk walk;
    bool ok = true;
    Work work;
    for (int i = 0; ok && list.get(i, work); ++i) {
      const Tile& tile = work.tile;
      bool both;
      const int b = walk.take(DUAL, tile.tokens, both);
      const int f = tile.f0 + quarter * 32 + lane;        // this thread's feature = its lane of tensor memory
      const bool f_ok = f < p.n_out;
      // lane j fetches the scores of tokens c + j for this warp's runs c (at most BT / 64 of
      // them) while the tile still accumulates; the loops below take them by shuffle
      constexpr int RUNS = (BT + 63) / 64;
      float my_score[RUNS];
#pragma unroll
      for (int q = 0; q < RUNS; ++q) {
        const int tk = half * 32 + q * 64 + lane;
        my_score[q] = (DUAL && tk < tile.tokens) ? p.scores[p.sorted_entry[tile.row0 + tk]] : 1.f;
      }
      bool waited = tc::mbar_wait(&acc_full[b], walk.use[b] & 1);
      if (both) waited = tc::mbar_wait(&acc_full[1], walk.use[1] & 1) && waited;
      if (!__all_sync(0xffffffffu, waited)) {
        if (lane == 0) atomicExch(p.status, 3);
        ok = false;
        break;
      }
      tc::fence_after();
      const uint32_t lane_base = tmem + b * SLOT_COLS + ((uint32_t)(quarter * 32) << 16);
      const uint32_t up_off = both ? SLOT_COLS : DUAL_SLOT_T;
      const int live = tile.tokens;
      if (DUAL) {
        // results of this warp's runs, two bfloat16 per register
        uint32_t packed[RUNS][16];
#pragma unroll
        for (int q = 0; q < RUNS; ++q) {
          const int c = half * 32 + q * 64;
          if (c < live) {
            uint32_t g[32], u[32];
            tc::ld32_nowait(lane_base + c, g);
            tc::ld32_nowait(lane_base + up_off + c, u);
            tc::wait_ld();
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float a[2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const float s = __shfl_sync(0xffffffffu, my_score[q], j + h);
                const float gs = s * __uint_as_float(g[j + h]);
                // silu by the fast exponential and division: their error is far below the
                // bfloat16 rounding of the result
                a[h] = __fdividef(gs, 1.f + __expf(-gs)) * (s * __uint_as_float(u[j + h]));
              }
              __nv_bfloat162 pr = __floats2bfloat162_rn(a[0], a[1]);
              packed[q][j >> 1] = *reinterpret_cast<uint32_t*>(&pr);
            }
          }
        }
        // this warp is done reading the slot(s): the MMA issuer may overwrite them
        tc::fence_before();
        __syncwarp();
        if (lane == 0) {
          tc::mbar_arrive(&acc_empty[b]);
          if (both) tc::mbar_arrive(&acc_empty[1]);
        }
#pragma unroll
        for (int q = 0; q < RUNS; ++q) {
          const int c = half * 32 + q * 64;
          if (c < live && f_ok) {
            uint16_t* dst = reinterpret_cast<uint16_t*>(p.out) + (size_t)(tile.row0 + c) * p.n_out + f;
#pragma unroll
            for (int j = 0; j < 32; ++j)               // 32 lanes: 64 bytes in a row
              if (c + j < tile.tokens) dst[(size_t)j * p.n_out] = (uint16_t)(packed[q][j >> 1] >> ((j & 1) * 16));
          }
        }
      } else {
        // a whole tile goes to `out`; a piece to its place in the scratch memory, [token][feature of the tile]
        const bool cut = work.cut >= 0;
        float* part = p.scratch + ((size_t)(work.cut * work.pieces + work.piece) * BT) * BF + quarter * 32 + lane;
#pragma unroll
        for (int q = 0; q < RUNS; ++q) {
          const int c = half * 32 + q * 64;
          if (c < live) {
            float g[32];
            tc::ld32(lane_base + c, g);
            float* dst = reinterpret_cast<float*>(p.out) + (size_t)(tile.row0 + c) * p.n_out + f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {             // 32 lanes: 128 bytes in a row
              if (c + j < tile.tokens) {
                if (cut) part[(size_t)(c + j) * BF] = g[j];
                else if (f_ok) dst[(size_t)j * p.n_out] = g[j];
              }
            }
          }
        }
        tc::fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&acc_empty[b]);
        if (cut) {
          // Count this piece in once all eight epilogue warps have written theirs; the last piece of the
          // tile to arrive adds them all, in the order of the pieces. A block has at most one piece (its
          // last work), so each of the two barriers is used once; their waits are bounded like the others.
          __threadfence();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&cut_bar[0]);
          if (warp == 2 && lane == 0) {
            if (tc::mbar_wait(&cut_bar[0], 0)) {
              __threadfence();
              const int before = atomicAdd(p.counters + work.cut, 1);
              __threadfence();
              *s_last = before == work.pieces - 1;
              if (*s_last) p.counters[work.cut] = 0;     // every piece has arrived: ready for the next launch
            } else {
              atomicExch(p.status, 5);
              *s_last = 0;
            }
            tc::mbar_arrive(&cut_bar[1]);
          }
          if (!__all_sync(0xffffffffu, tc::mbar_wait(&cut_bar[1], 0))) {
            if (lane == 0) atomicExch(p.status, 5);
            ok = false;
            break;
          }
          if (*s_last) {
            const float* first = p.scratch + ((size_t)(work.cut * work.pieces) * BT) * BF + quarter * 32 + lane;
#pragma unroll
            for (int q = 0; q < RUNS; ++q) {
              const int c = half * 32 + q * 64;
              if (c >= live || !f_ok) continue;
              float* dst = reinterpret_cast<float*>(p.out) + (size_t)(tile.row0 + c) * p.n_out + f;
              for (int j0 = 0; j0 < 32; j0 += 8) {
                float sum[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) sum[j] = 0.f;
                for (int piece = 0; piece < work.pieces; ++piece) {
                  const float* src = first + ((size_t)piece * BT + c + j0) * BF;
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    if (c + j0 + j < tile.tokens) sum[j] += __ldcg(src + (size_t)j * BF);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (c + j0 + j < tile.tokens) dst[(size_t)(j0 + j) * p.n_out] = sum[j];
              }
            }
          }
        }
      }
      ++walk.use[b];
      if (both) ++walk.use[1];
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

template <bool DUAL, int STAGES, int BT>
int launch(const void* x, const void* w0, const void* w1, const Params& p, int max_tiles, cudaStream_t stream) {
  Maps maps;
  for (int b = 0; b < 4; ++b)
    if (!tc::make_map_bf16(&maps.x[b], x, (uint64_t)p.rows, (uint64_t)p.K, (uint32_t)x_box_rows(b, BT))) return HB_ERR_UNSUPPORTED;
  if (!tc::make_map_bf16(&maps.w0, w0, (uint64_t)p.experts * p.n_out, (uint64_t)p.K, BF) ||
      !tc::make_map_bf16(&maps.w1, DUAL ? w1 : w0, (uint64_t)p.experts * p.n_out, (uint64_t)p.K, BF))
    return HB_ERR_UNSUPPORTED;
  constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * BF * BK * 2 + BT * BK * 2;
  static_assert((2 * STAGES + 6) * 8 + 12 <= 256, "the barriers and the tensor-memory slot fit their 256 bytes");
  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024 + 256 + 4 * ((size_t)p.experts + 2);
  if (smem > 227 * 1024) return HB_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_tc_kernel<DUAL, STAGES, BT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return (int)e;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return HB_ERR_BAD_ARG;
  // one persistent block per SM; with fewer tiles than SMs, as many blocks as tiles and their pieces can use
  const long long upper = (long long)max_tiles * ((p.n_out + BF - 1) / BF) * (p.scratch ? MAX_PIECES : 1);
  const int grid = (int)(upper < sms ? upper : sms);
  grouped_gemm_tc_kernel<DUAL, STAGES, BT><<<grid, THREADS, smem, stream>>>(maps, p);
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
  const bool few = rows <= SHORT_STEP_ROWS;
  const int bt = few ? BT_SHORT : BT_LONG;
  const int max_tiles = (rows + bt - 1) / bt + (experts < rows ? experts : rows);
  if (max_tiles > 65535) return HB_ERR_UNSUPPORTED;
  Params p{offsets, sorted_entry, scores, act, status, experts, inter, hidden, rows, nullptr, nullptr};
  return few ? launch<true, 5, BT_SHORT>(xs, w_gate, w_up, p, max_tiles, stream)
             : launch<true, 4, BT_LONG>(xs, w_gate, w_up, p, max_tiles, stream);
}

// down projection on tensor cores: act [rows, inter] -> y float32 [rows, hidden].
// `scratch` (`scratch_floats` floats) and `counters` (`n_counters` ints, zero before the first call and
// left at zero) let the last, partly filled round of tiles be cut along K; they belong to one launch at
// a time. With room for fewer than one partial tile per block (or null) the tiles stay whole.
extern "C" int hb_moe_down_tc(const void* act, const void* w_down, const int* offsets, int experts, float* y, int rows,
                              int hidden, int inter, float* scratch, long long scratch_floats, int* counters,
                              int n_counters, int* status, cudaStream_t stream) {
  if (!act || !w_down || !offsets || !y || !status || rows < 0 || experts <= 0) return HB_ERR_BAD_ARG;
  if (hidden % 8 != 0 || inter % 8 != 0 || hidden <= 0 || inter <= 0) return HB_ERR_UNSUPPORTED;
  if (rows == 0) return HB_OK;
  const bool few = rows <= SHORT_STEP_ROWS;
  const int bt = few ? BT_SHORT : BT_LONG;
  const int max_tiles = (rows + bt - 1) / bt + (experts < rows ? experts : rows);
  if (max_tiles > 65535) return HB_ERR_UNSUPPORTED;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return HB_ERR_BAD_ARG;
  const bool room = scratch && counters && n_counters >= sms && scratch_floats >= (long long)sms * bt * BF;
  Params p{offsets, nullptr, nullptr, y, status, experts, hidden, inter, rows, room ? scratch : nullptr, counters};
  return few ? launch<false, 8, BT_SHORT>(act, w_down, nullptr, p, max_tiles, stream)
             : launch<false, 5, BT_LONG>(act, w_down, nullptr, p, max_tiles, stream);
}

extern "C" long long hb_moe_down_tc_scratch_floats(int sms) { return (long long)sms * BT_LONG * BF; }
