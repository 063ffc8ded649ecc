// Decode attention over the paged cache, bfloat16, with the K and V tiles brought in by TMA:
// the same flash-decoding as attention_decode.cu (grid (split, kv head, token); the query heads
// of a kv head are the rows of one 16-row tile; mma.sync m16n8k16 with float32 accumulation and
// softmax; four warps of 16 keys each per 64-key tile; partials merged by attention_merge), but
// one thread issues a tile's loads as a few tensor-map copies (a page's 64 rows x 64 dims per
// copy, 128-byte swizzle) that an mbarrier counts, instead of every thread issuing sixteen
// 16-byte cp.async with their address arithmetic. ldmatrix reads the swizzled tiles (16-byte
// chunk c of row r sits at chunk c ^ (r % 8)).
//
// Takes what the tile loads need: pages of 16, 32 or a multiple of 64 positions, and ranges that
// start on a multiple of 64 (no sliding window; a chunk size that is a multiple of 64). Rows of a
// tile past the token's last key lie in the same page (or in a page the request does not hold,
// which is then not loaded): K rows there are masked by position, V rows are zeroed in shared
// memory, so whatever the pool holds there cannot reach the sum. Every mbarrier wait is bounded;
// on a time-out the kernel records it in `status` and stops.
//
// The fused form (hb_attention_decode_fused) takes the q/k/v projection's output as it is and
// does in the same launch what hb_qkv_post and hb_attention_merge do around the plain form: every
// block encodes the query rows of its kv group itself (rotation or temperature, weightless norm:
// the arithmetic of qkv_post.cu, so a key is the same number whichever kernel wrote it); the block
// whose key range ends at the token's own position also encodes the token's key and value, writes
// them to their page for later steps, and puts them into its shared-memory tile in place of what
// the tile load brought from that row; and the block of a (token, kv head) that finishes last
// (a counter that is zero between launches) combines the splits, in split order.
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "api.h"
#include "common.cuh"
#include "mma.cuh"
#include "tc.cuh"

namespace {

constexpr int TILE = 64;     // keys per shared-memory tile
constexpr int NWARPS = 4;
constexpr int ROWS = 16;     // query rows of the tile (heads of one kv group, padded)
constexpr int STAGES = 2;     // measured: three stages (two blocks per SM instead of three) are no faster
constexpr int HALF_BYTES = TILE * 128;   // a tile's 64 rows x 64 dims (128 bytes a row)

struct Args {
  const __nv_bfloat16* q;
  const int* block_table;
  const int* seq_of_token;
  const int* positions;
  __nv_bfloat16* out;
  float* part_acc;
  float* part_ml;
  int* status;
  int table_stride, nh, nkv, page_size, chunk, split_size, max_splits, box_rows;
  float scale;
};

// What the fused form needs beside Args.
struct Fuse {
  const __nv_bfloat16* qkv;      // [n_tokens, (nh + 2 nkv) * head_dim]: q heads, k heads, v heads
  const float* inv_freq;         // [rot_pairs], or null: no rotation
  int rot_pairs;                 // the first 2 * rot_pairs dims of a head rotate (a multiple of 8 pairs)
  __nv_bfloat16* k_pages;
  __nv_bfloat16* v_pages;
  int* counters;                 // [n_tokens * nkv], zero between launches
  int interleaved, qk_norm, temp_on;
  float qk_eps, floor_scale, attn_scale;
};

// One head of the q/k/v row as qkv_post.cu encodes it: head_dim / 16 neighbouring lanes, each with
// 8 rotation pairs (a[i], b[i]): dims (j0 + i, rot_pairs + j0 + i), or (2 (j0 + i), 2 (j0 + i) + 1)
// when interleaved; lanes past the rotated dims own 16 consecutive elements that pass through. kind 0 = query (rotation, norm, temperature), 1 = key (rotation, norm),
// 2 = value (as it is). Every lane of the warp must call it (the norm's sum goes over lanes).
// Returns the head's 16 values of this lane as two 16-byte chunks and the dims they start at.
template <int HD>
__device__ __forceinline__ void encode_head(const __nv_bfloat16* src, int kind, bool active, int sub, const Fuse& f,
                                            const float* cs_s, const float* sn_s, int pos, uint4& c0, uint4& c1,
                                            int& d0, int& d1) {
  constexpr int LPH = HD / 16;
  const int HALF = f.rot_pairs;
  const int j0 = sub * 8;
  const bool rotates = j0 < f.rot_pairs;
  const bool consecutive = f.interleaved || !rotates;
  float a[8], b[8];
  float ss = 0.f;
  if (active) {
    if (consecutive) {
      float lo[8], hi[8];
      hb::load8(src + 2 * j0, lo);
      hb::load8(src + 2 * j0 + 8, hi);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = lo[2 * i]; b[i] = lo[2 * i + 1];
        a[4 + i] = hi[2 * i]; b[4 + i] = hi[2 * i + 1];
      }
    } else {
      hb::load8(src + j0, a);
      hb::load8(src + HALF + j0, b);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (kind != 2 && f.inv_freq != nullptr && rotates) {
        const float sn = sn_s[j0 + i], cs = cs_s[j0 + i];
        const float ra = a[i] * cs - b[i] * sn;
        const float rb = b[i] * cs + a[i] * sn;
        a[i] = ra; b[i] = rb;
      }
      ss += a[i] * a[i] + b[i] * b[i];
    }
  }
  for (int o = LPH >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  float mul = 1.f;
  if (kind != 2 && f.qk_norm) mul = rsqrtf(ss / (float)HD + f.qk_eps);
  if (kind == 0 && f.temp_on) mul *= logf(floorf(((float)pos + 1.f) / f.floor_scale) + 1.f) * f.attn_scale + 1.f;
  float lo[8], hi[8];
  if (consecutive) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo[2 * i] = a[i] * mul; lo[2 * i + 1] = b[i] * mul;
      hi[2 * i] = a[4 + i] * mul; hi[2 * i + 1] = b[4 + i] * mul;
    }
    d0 = 2 * j0; d1 = 2 * j0 + 8;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) { lo[i] = a[i] * mul; hi[i] = b[i] * mul; }
    d0 = j0; d1 = HALF + j0;
  }
  uint32_t* w0 = reinterpret_cast<uint32_t*>(&c0);
  uint32_t* w1 = reinterpret_cast<uint32_t*>(&c1);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    w0[i] = hb::pack_bf16(lo[2 * i], lo[2 * i + 1]);
    w1[i] = hb::pack_bf16(hi[2 * i], hi[2 * i + 1]);
  }
}

// byte offset of the 16-byte chunk that holds dims d .. d+7 of key row r in a swizzled tile
template <int HD>
__device__ __forceinline__ uint32_t tile_offset(int r, int d) {
  return (uint32_t)((d >> 6) * HALF_BYTES + r * 128 + ((((d & 63) >> 3) ^ (r & 7)) << 4));
}

template <int HD, bool FUSED>
__global__ void __launch_bounds__(NWARPS * 32)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const Args a,
                       const Fuse f) {
  constexpr int STRIDE = HD + 8;                 // padded query rows: ldmatrix without bank conflicts
  constexpr int CHUNKS = HD / 8;
  constexpr int HALVES = HD / 64;
  constexpr int KV_BYTES = HALVES * HALF_BYTES;  // one K (or V) tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* k_s = smem;                                          // [STAGES][KV_BYTES]
  uint8_t* v_s = smem + STAGES * KV_BYTES;                      // [STAGES][KV_BYTES]
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(v_s + STAGES * KV_BYTES);   // [ROWS][STRIDE]
  float* ml_s = reinterpret_cast<float*>(q_s + ROWS * STRIDE);  // [NWARPS][ROWS][2]
  uint64_t* full = reinterpret_cast<uint64_t*>(ml_s + NWARPS * ROWS * 2);           // [STAGES]
  float* cs_s = reinterpret_cast<float*>(full + STAGES);        // [HD / 2] cosines, [HD / 2] sines (fused form)
  float* sn_s = cs_s + HD / 2;
  float* o_s = reinterpret_cast<float*>(k_s);    // [ROWS][HD], reuses the K tiles once the key loop is over
  __shared__ int last_block;

  const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = a.nh / a.nkv;
  const int pos = a.positions[t];
  const int* table = a.block_table + (size_t)a.seq_of_token[t] * a.table_stride;
  const int lo = a.chunk > 0 ? (pos / a.chunk) * a.chunk : 0;
  const int first = lo + split * a.split_size;
  const size_t th0 = (size_t)t * a.nh + (size_t)kvh * G;      // (token, first head of the group)
  // with the merge inside (fused form with counters): this token's own splits; else all of them, and
  // the merge kernel is told which ones are empty
  const bool merge_inside = FUSED && f.counters != nullptr;
  const int n_splits = merge_inside ? (pos - lo) / a.split_size + 1 : a.max_splits;
  if (first > pos) {                                          // this token has fewer splits
    if (!merge_inside && a.max_splits > 1 && tid < G) {
      float* ml = a.part_ml + ((th0 + tid) * a.max_splits + split) * 2;
      ml[0] = -INFINITY; ml[1] = 0.f;
    }
    return;
  }
  const int last = min(pos, first + a.split_size - 1);
  const int n_tiles = (last - first + TILE) / TILE;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) tc::mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // One thread issues a tile: for every page under the tile (one, or 64 / page_size of them) that
  // holds a key of the range, the page's rows of K and of V, 64 dims per copy.
  auto issue = [&](int tile, int stage) {
    const int base = first + tile * TILE;
    const int rows_per_box = a.box_rows;           // min(page_size, 64)
    uint32_t bytes = 0;
    for (int r0 = 0; r0 < TILE; r0 += rows_per_box)
      if (base + r0 <= last && table[(base + r0) / a.page_size] >= 0) bytes += 2u * HALVES * rows_per_box * 128;
    tc::mbar_expect_tx(&full[stage], bytes);
    for (int r0 = 0; r0 < TILE; r0 += rows_per_box) {
      const int key = base + r0;
      if (key > last) break;
      const int page = table[key / a.page_size];
      if (page < 0) continue;
      const int row = (page * a.nkv + kvh) * a.page_size + key % a.page_size;
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        tc::tma_load_2d(k_s + stage * KV_BYTES + h * HALF_BYTES + r0 * 128, &map_k, h * 64, row, &full[stage]);
        tc::tma_load_2d(v_s + stage * KV_BYTES + h * HALF_BYTES + r0 * 128, &map_v, h * 64, row, &full[stage]);
      }
    }
  };
  // the first tiles are on their way while the query rows are made ready (the thread that
  // initialised the barriers issues them, so it needs no one else to have seen the barriers yet)
  if (tid == 0)
    for (int i = 0; i < STAGES - 1 && i < n_tiles; ++i) issue(i, i);

  // the query rows of this kv group
  uint4 own_c0 = make_uint4(0u, 0u, 0u, 0u), own_c1 = own_c0;   // fused: this lane's part of the token's own key or value
  int own_d0 = 0, own_d1 = 0;
  bool own_kv = false;
  if constexpr (FUSED) {
    constexpr int LPH = HD / 16, HPW = 32 / LPH;
    if (f.inv_freq != nullptr)
      for (int j = tid; j < f.rot_pairs; j += NWARPS * 32) sincosf((float)pos * f.inv_freq[j], &sn_s[j], &cs_s[j]);
    for (int c = tid; c < (ROWS - G) * CHUNKS; c += NWARPS * 32)      // the tile's rows past the group are zeros
      *reinterpret_cast<uint4*>(q_s + (G + c / CHUNKS) * STRIDE + (c % CHUNKS) * 8) = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();                               // sines and cosines; the barriers are initialised
    const __nv_bfloat16* row = f.qkv + (size_t)t * (a.nh + 2 * a.nkv) * HD;
    const int sub = lane % LPH, slot = warp * HPW + lane / LPH;     // NWARPS * HPW = 16 head slots
    {
      const bool active = slot < G;
      uint4 c0, c1;
      int d0, d1;
      encode_head<HD>(row + (size_t)(kvh * G + (active ? slot : 0)) * HD, 0, active, sub, f, cs_s, sn_s, pos, c0, c1, d0, d1);
      if (active) {
        *reinterpret_cast<uint4*>(q_s + slot * STRIDE + d0) = c0;
        *reinterpret_cast<uint4*>(q_s + slot * STRIDE + d1) = c1;
      }
    }
    if (last == pos && warp == 0) {                // this block's range ends at the token itself: its key and value
      const bool active = slot < 2;
      const int kind = 1 + (slot & 1);
      const __nv_bfloat16* src = row + (size_t)(a.nh + (kind == 2 ? a.nkv : 0) + kvh) * HD;
      encode_head<HD>(src, kind, active, sub, f, cs_s, sn_s, pos, own_c0, own_c1, own_d0, own_d1);
      own_kv = active;
      const int page = table[pos / a.page_size];
      if (active && page >= 0) {                   // the host reserved the page before the step
        __nv_bfloat16* dst = (kind == 1 ? f.k_pages : f.v_pages) +
                             (((size_t)page * a.nkv + kvh) * a.page_size + pos % a.page_size) * HD;
        *reinterpret_cast<uint4*>(dst + own_d0) = own_c0;
        *reinterpret_cast<uint4*>(dst + own_d1) = own_c1;
      }
    }
  } else {
    for (int c = tid; c < ROWS * CHUNKS; c += NWARPS * 32) {
      const int r = c / CHUNKS, ch = c % CHUNKS;
      const bool ok = r < G;
      hb::cp_async16(q_s + r * STRIDE + ch * 8, a.q + (th0 + (ok ? r : 0)) * HD + ch * 8, ok);
    }
    hb::cp_async_commit();
    __syncthreads();                               // the barriers are initialised
  }

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o_acc[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[j][e] = 0.f;
  unsigned q_frag[HD / 16][4];
  bool ok = true;

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile % STAGES;
    if (tid == 0 && tile + STAGES - 1 < n_tiles)                              // its stage was freed by the last sync
      issue(tile + STAGES - 1, (tile + STAGES - 1) % STAGES);
    if (!FUSED && tile == 0) hb::cp_async_wait<0>();                           // the query rows
    if (!tc::mbar_wait(&full[buf], (tile / STAGES) & 1)) {
      if (tid == 0) atomicExch(a.status, 31);
      ok = false;
    }
    const int base = first + tile * TILE;
    uint8_t* kt = k_s + buf * KV_BYTES;
    uint8_t* vt = v_s + buf * KV_BYTES;
    if (FUSED && own_kv && tile == n_tiles - 1) {
      // the token's own key and value take the place of what the load brought from their row of the page
      uint8_t* own = (lane / (HD / 16)) == 0 ? kt : vt;
      *reinterpret_cast<uint4*>(own + tile_offset<HD>(pos - base, own_d0)) = own_c0;
      *reinterpret_cast<uint4*>(own + tile_offset<HD>(pos - base, own_d1)) = own_c1;
    }
    if (base + TILE - 1 > last) {                  // the last tile: V rows past the range must not reach the sum
      for (int c = tid; c < TILE * HALVES * 8; c += NWARPS * 32) {
        const int r = c / (HALVES * 8), rest = c % (HALVES * 8);
        if (base + r > last)
          *reinterpret_cast<uint4*>(vt + (rest / 8) * HALF_BYTES + r * 128 + (rest % 8) * 16) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    // q rows and zeroed rows are visible to every warp; and the block agrees on whether the tile
    // arrived (a wait that ran out in some threads only must not split the block at a barrier)
    ok = __syncthreads_and(ok);
    if (!ok) break;
    if (tile == 0) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        hb::ldmatrix_x4(q_frag[ks], q_s + (lane % 16) * STRIDE + ks * 16 + (lane / 16) * 8);
    }
    // S = Q K^T for this warp's 16 keys: two 8-key column tiles
    float s_acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const int k_row = warp * 16 + (lane % 8) + (lane / 16) * 8;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      unsigned b[4];
      hb::ldmatrix_x4(b, kt + tile_offset<HD>(k_row, ks * 16 + ((lane / 8) % 2) * 8));
      hb::mma_bf16(s_acc[0], q_frag[ks], b[0], b[1]);
      hb::mma_bf16(s_acc[1], q_frag[ks], b[2], b[3]);
    }
    // scale, mask keys past the split's end, online softmax per row (rows lane/4 and lane/4 + 8)
    const int key0 = base + warp * 16 + (lane % 4) * 2;
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + nt * 8 + (e & 1);
        const float v = key <= last ? s_acc[nt][e] * a.scale : -INFINITY;
        s_acc[nt][e] = v;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = tile_max[r];
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[r], mx);
      corr[r] = (m_run[r] == -INFINITY) ? 0.f : __expf(m_run[r] - m_new);
      m_run[r] = m_new;
    }
    float row_sum[2] = {0.f, 0.f};
    unsigned p_frag[4];
    {
      float p[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const float v = (s_acc[nt][e] == -INFINITY) ? 0.f : __expf(s_acc[nt][e] - m_run[r]);
          p[nt][e] = v;
          row_sum[r] += v;
        }
      p_frag[0] = hb::pack_bf16(p[0][0], p[0][1]);
      p_frag[1] = hb::pack_bf16(p[0][2], p[0][3]);
      p_frag[2] = hb::pack_bf16(p[1][0], p[1][1]);
      p_frag[3] = hb::pack_bf16(p[1][2], p[1][3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float sum = row_sum[r];
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[r] = l_run[r] * corr[r] + sum;
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {   // the running max rarely moves
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) {
        o_acc[j][0] *= corr[0]; o_acc[j][1] *= corr[0];
        o_acc[j][2] *= corr[1]; o_acc[j][3] *= corr[1];
      }
    }
    // O += P V : V rows are keys (k), columns dims (n): transposed 8x8 loads give the B fragments
    const int v_row = warp * 16 + (lane % 8) + ((lane / 8) % 2) * 8;
#pragma unroll
    for (int j = 0; j < HD / 8; j += 2) {
      unsigned b[4];
      hb::ldmatrix_x4_trans(b, vt + tile_offset<HD>(v_row, j * 8 + (lane / 16) * 8));
      hb::mma_bf16(o_acc[j], p_frag, b[0], b[1]);
      hb::mma_bf16(o_acc[j + 1], p_frag, b[2], b[3]);
    }
    __syncthreads();      // everyone is done with this buffer before it is refilled
  }
  // fused form: the blocks of a (token, kv head) count themselves in; the last one combines the splits
  const bool counted = merge_inside && n_splits > 1;
  auto arrive = [&]() {
    __syncthreads();                                 // this block's partial results are written; one thread
    if (tid == 0) {                                  // publishes them (the fence is cumulative over the barrier)
      __threadfence();
      last_block = atomicAdd(&f.counters[t * a.nkv + kvh], 1) == n_splits - 1;
      __threadfence();
    }
    __syncthreads();
    return last_block != 0;
  };
  if (!ok) {               // a load never arrived (recorded in status): nothing sensible to write
    if (counted && arrive() && tid == 0) f.counters[t * a.nkv + kvh] = 0;
    return;
  }

  // merge the four warps (each saw a quarter of the keys), in warp order
  const int r0 = lane / 4;
  if ((lane % 4) == 0) {
    ml_s[(warp * ROWS + r0) * 2] = m_run[0];     ml_s[(warp * ROWS + r0) * 2 + 1] = l_run[0];
    ml_s[(warp * ROWS + r0 + 8) * 2] = m_run[1]; ml_s[(warp * ROWS + r0 + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  float fr[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r0 + 8 * r;
    float mx = -INFINITY;
    for (int w = 0; w < NWARPS; ++w) mx = fmaxf(mx, ml_s[(w * ROWS + row) * 2]);
    fr[r] = (m_run[r] == -INFINITY) ? 0.f : expf(m_run[r] - mx);
  }
  for (int w = 0; w < NWARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) {
        const int d = j * 8 + (lane % 4) * 2;
        float* x = o_s + r0 * HD + d;
        float* y = o_s + (r0 + 8) * HD + d;
        if (w == 0) {
          x[0] = o_acc[j][0] * fr[0]; x[1] = o_acc[j][1] * fr[0];
          y[0] = o_acc[j][2] * fr[1]; y[1] = o_acc[j][3] * fr[1];
        } else {
          x[0] += o_acc[j][0] * fr[0]; x[1] += o_acc[j][1] * fr[0];
          y[0] += o_acc[j][2] * fr[1]; y[1] += o_acc[j][3] * fr[1];
        }
      }
    }
    __syncthreads();
  }
  // rows < G are real heads; thread `tid` finishes (row, dims) pairs
  for (int i = tid; i < G * HD; i += NWARPS * 32) {
    const int row = i / HD, d = i % HD;
    float mx = -INFINITY;
    for (int w = 0; w < NWARPS; ++w) mx = fmaxf(mx, ml_s[(w * ROWS + row) * 2]);
    float l = 0.f;
    for (int w = 0; w < NWARPS; ++w) {
      const float mw = ml_s[(w * ROWS + row) * 2];
      if (mw != -INFINITY) l += ml_s[(w * ROWS + row) * 2 + 1] * expf(mw - mx);
    }
    const float o = o_s[row * HD + d];
    if (n_splits > 1) {
      a.part_acc[((th0 + row) * a.max_splits + split) * HD + d] = o;
      if (d == 0) {
        float* ml = a.part_ml + ((th0 + row) * a.max_splits + split) * 2;
        ml[0] = mx; ml[1] = l;
      }
    } else {
      a.out[(th0 + row) * HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
  }
  if (!counted || !arrive()) return;
  // The last block of this (token, kv head): o = sum_s acc_s e^{m_s - m} / sum_s l_s e^{m_s - m} over
  // the token's splits, in split order. The partial results come from other SMs: read past L1.
  float* w_s = reinterpret_cast<float*>(v_s);        // [G][n_splits] weights, then [G] 1 / l; the V tiles are done with
  float* inv_s = w_s + G * n_splits;
  // weights: thread (row, split) pairs; the maxima and sums of a row go through shared memory
  float* m_s = o_s;                                  // [G][n_splits] maxima, then the same for the sums (o_s is done with
  float* l_s = m_s + G * n_splits;                   // where G * splits fit; the launcher checks the room)
  for (int i = tid; i < G * n_splits; i += NWARPS * 32) {
    const int row = i / n_splits, sp = i % n_splits;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(a.part_ml + ((th0 + row) * a.max_splits + sp) * 2));
    m_s[i] = ml.x;
    l_s[i] = ml.y;
  }
  __syncthreads();
  for (int row = warp; row < G; row += NWARPS) {
    float mx = -INFINITY;
    for (int sp = lane; sp < n_splits; sp += 32) mx = fmaxf(mx, m_s[row * n_splits + sp]);
    mx = hb::warp_max(mx);
    float l = 0.f;
    for (int sp = lane; sp < n_splits; sp += 32) {
      const float e = expf(m_s[row * n_splits + sp] - mx);
      w_s[row * n_splits + sp] = e;
      l += l_s[row * n_splits + sp] * e;
    }
    l = hb::warp_sum(l);
    if (lane == 0) inv_s[row] = l > 0.f ? 1.f / l : 0.f;
  }
  __syncthreads();
  // outputs: a thread takes four dims of a row; up to 16 splits' loads are in flight at a time, and the
  // sum runs over the splits in their order
  constexpr int AHEAD = 16;
  for (int i = tid; i < G * (HD / 4); i += NWARPS * 32) {
    const int row = i / (HD / 4), d = (i % (HD / 4)) * 4;
    const float* acc = a.part_acc + (th0 + row) * a.max_splits * HD + d;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < n_splits; s0 += AHEAD) {
      float4 v[AHEAD];
#pragma unroll
      for (int q = 0; q < AHEAD; ++q)
        if (s0 + q < n_splits) v[q] = __ldcg(reinterpret_cast<const float4*>(acc + (size_t)(s0 + q) * HD));
#pragma unroll
      for (int q = 0; q < AHEAD; ++q)
        if (s0 + q < n_splits) {
          const float ws = w_s[row * n_splits + s0 + q];
          o.x += v[q].x * ws; o.y += v[q].y * ws; o.z += v[q].z * ws; o.w += v[q].w * ws;
        }
    }
    const float inv = inv_s[row];
    __nv_bfloat162 lo = __floats2bfloat162_rn(o.x * inv, o.y * inv), hi = __floats2bfloat162_rn(o.z * inv, o.w * inv);
    uint2 pack;
    pack.x = *reinterpret_cast<uint32_t*>(&lo);
    pack.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(a.out + (th0 + row) * HD + d) = pack;
  }
  if (tid == 0) f.counters[t * a.nkv + kvh] = 0;     // zero again for the next launch
}

template <int HD, bool FUSED>
int launch(const void* k_pages, const void* v_pages, int n_pages, int n_tokens, const Args& a, const Fuse& f,
           cudaStream_t stream) {
  const uint64_t pool_rows = (uint64_t)n_pages * a.nkv * a.page_size;
  CUtensorMap mk, mv;
  if (!tc::make_map_bf16(&mk, k_pages, pool_rows, HD, a.box_rows) || !tc::make_map_bf16(&mv, v_pages, pool_rows, HD, a.box_rows))
    return HB_ERR_UNSUPPORTED;
  constexpr int STRIDE = HD + 8;
  constexpr int KV_BYTES = (HD / 64) * HALF_BYTES;
  const size_t smem = 1024 + 2 * (size_t)STAGES * KV_BYTES + (size_t)ROWS * STRIDE * 2 +
                      (size_t)NWARPS * ROWS * 2 * sizeof(float) + STAGES * sizeof(uint64_t) + HD * sizeof(float);
  static_assert((size_t)STAGES * KV_BYTES >= (size_t)ROWS * HD * sizeof(float), "o_s aliases the K tiles");
  // the fused merge keeps [G][splits] weights and [G] sums where the V tiles were
  if (FUSED && (size_t)(a.nh / a.nkv) * (2 * a.max_splits + 1) * sizeof(float) > (size_t)STAGES * KV_BYTES) return HB_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<HD, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(a.max_splits, a.nkv, n_tokens);
  attn_decode_tma_kernel<HD, FUSED><<<grid, NWARPS * 32, smem, stream>>>(mk, mv, a, f);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // namespace

// As hb_attention_decode (bfloat16; head_dim 64 or 128; at most 16 query heads per kv head; every
// token one decode row; partials merged by hb_attention_merge), with TMA tile loads. Returns
// HB_ERR_UNSUPPORTED for what those cannot take (a sliding window, a chunk size or page size
// that breaks the 64-key tiles): the caller then uses hb_attention_decode. `status` is one int
// on the device, zero before the call; nonzero afterwards = a wait on a load timed out.
extern "C" int hb_attention_decode_tma(const void* q, const void* k_pages, const void* v_pages, int n_pages,
                                       const int* block_table, int table_stride, const int* seq_of_token,
                                       const int* positions, void* out, int n_tokens, int nh, int nkv, int hd,
                                       int page_size, int chunk, int window, float scale, int split_size,
                                       int max_splits, float* part_acc, float* part_ml, int* status,
                                       cudaStream_t stream) {
  if (!q || !k_pages || !v_pages || !block_table || !seq_of_token || !positions || !out || !status) return HB_ERR_BAD_ARG;
  if (n_tokens < 0 || n_pages <= 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || table_stride <= 0 ||
      chunk < 0 || window < 0 || max_splits < 1 || split_size <= 0 || split_size % TILE != 0)
    return HB_ERR_BAD_ARG;
  if (max_splits > 1 && (!part_acc || !part_ml)) return HB_ERR_BAD_ARG;
  if (nh / nkv > ROWS || n_tokens > 65535 || nkv > 65535) return HB_ERR_UNSUPPORTED;
  if (window > 0 || chunk % TILE != 0) return HB_ERR_UNSUPPORTED;
  if (!(page_size == 16 || page_size == 32 || page_size % TILE == 0)) return HB_ERR_UNSUPPORTED;
  if ((long long)n_pages * nkv * page_size > 0x7fffffffLL) return HB_ERR_UNSUPPORTED;   // row coordinates are 32-bit
  if (n_tokens == 0) return HB_OK;
  Args a{(const __nv_bfloat16*)q, block_table, seq_of_token, positions, (__nv_bfloat16*)out, part_acc, part_ml, status,
         table_stride, nh, nkv, page_size, chunk, split_size, max_splits, page_size < TILE ? page_size : TILE, scale};
  const Fuse none{};
  if (hd == 128) return launch<128, false>(k_pages, v_pages, n_pages, n_tokens, a, none, stream);
  if (hd == 64) return launch<64, false>(k_pages, v_pages, n_pages, n_tokens, a, none, stream);
  return HB_ERR_UNSUPPORTED;
}

// The fused form: `qkv` [n_tokens, (nh + 2 nkv) * hd] is the q/k/v projection's output; the kernel
// encodes q, k and v as hb_qkv_post does (inv_freq [rot_pairs] or null; pairs (j, j + rot_pairs) or
// (2j, 2j + 1); weightless norm; temperature on q), appends the token's key and value to its page,
// attends, and combines its own splits: `counters` holds n_tokens * nkv ints that are zero before
// the call and zero after it. With `counters` null the splits are left in part_acc / part_ml for
// hb_attention_merge, as hb_attention_decode_tma leaves them. Same shapes and refusals as hb_attention_decode_tma; every token is
// one decode row whose page the host has reserved.
extern "C" int hb_attention_decode_fused(const void* qkv, const float* inv_freq, int rot_pairs, int interleaved, int qk_norm,
                                         float qk_eps, int temp_on, float floor_scale, float attn_scale, void* k_pages,
                                         void* v_pages, int n_pages, const int* block_table, int table_stride,
                                         const int* seq_of_token, const int* positions, void* out, int n_tokens,
                                         int nh, int nkv, int hd, int page_size, int chunk, int window, float scale,
                                         int split_size, int max_splits, float* part_acc, float* part_ml,
                                         int* counters, int* status, cudaStream_t stream) {
  if (!qkv || !k_pages || !v_pages || !block_table || !seq_of_token || !positions || !out || !status) return HB_ERR_BAD_ARG;
  if (n_tokens < 0 || n_pages <= 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || table_stride <= 0 ||
      chunk < 0 || window < 0 || max_splits < 1 || split_size <= 0 || split_size % TILE != 0)
    return HB_ERR_BAD_ARG;
  if (temp_on && !(floor_scale > 0.f)) return HB_ERR_BAD_ARG;
  if (max_splits > 1 && (!part_acc || !part_ml)) return HB_ERR_BAD_ARG;
  if (!inv_freq) rot_pairs = 0;
  if (rot_pairs < 0 || 2 * rot_pairs > hd || rot_pairs % 8 != 0) return HB_ERR_UNSUPPORTED;
  if (nh / nkv > ROWS || n_tokens > 65535 || nkv > 65535) return HB_ERR_UNSUPPORTED;
  if (window > 0 || chunk % TILE != 0) return HB_ERR_UNSUPPORTED;
  if (!(page_size == 16 || page_size == 32 || page_size % TILE == 0)) return HB_ERR_UNSUPPORTED;
  if ((long long)n_pages * nkv * page_size > 0x7fffffffLL) return HB_ERR_UNSUPPORTED;
  if (n_tokens == 0) return HB_OK;
  Args a{nullptr, block_table, seq_of_token, positions, (__nv_bfloat16*)out, part_acc, part_ml, status,
         table_stride, nh, nkv, page_size, chunk, split_size, max_splits, page_size < TILE ? page_size : TILE, scale};
  Fuse f{(const __nv_bfloat16*)qkv, inv_freq, rot_pairs, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, counters,
         interleaved, qk_norm, temp_on, qk_eps, floor_scale, attn_scale};
  if (hd == 128) return launch<128, true>(k_pages, v_pages, n_pages, n_tokens, a, f, stream);
  if (hd == 64) return launch<64, true>(k_pages, v_pages, n_pages, n_tokens, a, f, stream);
  return HB_ERR_UNSUPPORTED;
}
