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

// byte offset of the 16-byte chunk that holds dims d .. d+7 of key row r in a swizzled tile
template <int HD>
__device__ __forceinline__ uint32_t tile_offset(int r, int d) {
  return (uint32_t)((d >> 6) * HALF_BYTES + r * 128 + ((((d & 63) >> 3) ^ (r & 7)) << 4));
}

template <int HD>
__global__ void __launch_bounds__(NWARPS * 32)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const Args a) {
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
  float* o_s = reinterpret_cast<float*>(k_s);    // [ROWS][HD], reuses the K tiles once the key loop is over

  const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = a.nh / a.nkv;
  const int pos = a.positions[t];
  const int* table = a.block_table + (size_t)a.seq_of_token[t] * a.table_stride;
  const int lo = a.chunk > 0 ? (pos / a.chunk) * a.chunk : 0;
  const int first = lo + split * a.split_size;
  const size_t th0 = (size_t)t * a.nh + (size_t)kvh * G;      // (token, first head of the group)
  if (first > pos) {                                          // this token has fewer splits
    if (a.max_splits > 1 && tid < G) {
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
  // the query rows of this kv group
  for (int c = tid; c < ROWS * CHUNKS; c += NWARPS * 32) {
    const int r = c / CHUNKS, ch = c % CHUNKS;
    const bool ok = r < G;
    hb::cp_async16(q_s + r * STRIDE + ch * 8, a.q + (th0 + (ok ? r : 0)) * HD + ch * 8, ok);
  }
  hb::cp_async_commit();
  __syncthreads();                                 // the barriers are initialised

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
  if (tid == 0)
    for (int i = 0; i < STAGES - 1 && i < n_tiles; ++i) issue(i, i);

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
    if (tile == 0) hb::cp_async_wait<0>();                                     // the query rows
    if (!tc::mbar_wait(&full[buf], (tile / STAGES) & 1)) {
      if (tid == 0) atomicExch(a.status, 31);
      ok = false;
    }
    const int base = first + tile * TILE;
    uint8_t* kt = k_s + buf * KV_BYTES;
    uint8_t* vt = v_s + buf * KV_BYTES;
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
  if (!ok) return;        // a load never arrived (recorded in status): nothing sensible to write

  // merge the four warps (each saw a quarter of the keys), in warp order
  const int r0 = lane / 4;
  if ((lane % 4) == 0) {
    ml_s[(warp * ROWS + r0) * 2] = m_run[0];     ml_s[(warp * ROWS + r0) * 2 + 1] = l_run[0];
    ml_s[(warp * ROWS + r0 + 8) * 2] = m_run[1]; ml_s[(warp * ROWS + r0 + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  float f[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r0 + 8 * r;
    float mx = -INFINITY;
    for (int w = 0; w < NWARPS; ++w) mx = fmaxf(mx, ml_s[(w * ROWS + row) * 2]);
    f[r] = (m_run[r] == -INFINITY) ? 0.f : expf(m_run[r] - mx);
  }
  for (int w = 0; w < NWARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) {
        const int d = j * 8 + (lane % 4) * 2;
        float* x = o_s + r0 * HD + d;
        float* y = o_s + (r0 + 8) * HD + d;
        if (w == 0) {
          x[0] = o_acc[j][0] * f[0]; x[1] = o_acc[j][1] * f[0];
          y[0] = o_acc[j][2] * f[1]; y[1] = o_acc[j][3] * f[1];
        } else {
          x[0] += o_acc[j][0] * f[0]; x[1] += o_acc[j][1] * f[0];
          y[0] += o_acc[j][2] * f[1]; y[1] += o_acc[j][3] * f[1];
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
    if (a.max_splits > 1) {
      a.part_acc[((th0 + row) * a.max_splits + split) * HD + d] = o;
      if (d == 0) {
        float* ml = a.part_ml + ((th0 + row) * a.max_splits + split) * 2;
        ml[0] = mx; ml[1] = l;
      }
    } else {
      a.out[(th0 + row) * HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
  }
}

template <int HD>
int launch(const void* k_pages, const void* v_pages, int n_pages, int n_tokens, const Args& a, cudaStream_t stream) {
  const uint64_t pool_rows = (uint64_t)n_pages * a.nkv * a.page_size;
  CUtensorMap mk, mv;
  if (!tc::make_map_bf16(&mk, k_pages, pool_rows, HD, a.box_rows) || !tc::make_map_bf16(&mv, v_pages, pool_rows, HD, a.box_rows))
    return HB_ERR_UNSUPPORTED;
  constexpr int STRIDE = HD + 8;
  constexpr int KV_BYTES = (HD / 64) * HALF_BYTES;
  const size_t smem = 1024 + 2 * (size_t)STAGES * KV_BYTES + (size_t)ROWS * STRIDE * 2 +
                      (size_t)NWARPS * ROWS * 2 * sizeof(float) + STAGES * sizeof(uint64_t);
  static_assert((size_t)STAGES * KV_BYTES >= (size_t)ROWS * HD * sizeof(float), "o_s aliases the K tiles");
  cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(a.max_splits, a.nkv, n_tokens);
  attn_decode_tma_kernel<HD><<<grid, NWARPS * 32, smem, stream>>>(mk, mv, a);
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
  if (hd == 128) return launch<128>(k_pages, v_pages, n_pages, n_tokens, a, stream);
  if (hd == 64) return launch<64>(k_pages, v_pages, n_pages, n_tokens, a, stream);
  return HB_ERR_UNSUPPORTED;
}
