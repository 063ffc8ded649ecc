// Prefill attention over the paged cache, bfloat16: portions of prompts (runs of new tokens of a
// request at consecutive positions) against every key they may read, the portion's own included.
// Flash attention on the tensor cores (mma.sync m16n8k16, float32 softmax and accumulation;
// the reference's counterpart is the wmma kernel of crates/hi-cuda/src/kernels.cu:12384-12700):
//   grid (query tile, query head, request); a block takes 64 consecutive new tokens of one
//   request and one head, 4 warps x 16 rows; key tiles of 64 positions, aligned to 64, come
//   through shared memory with cp.async (double-buffered) from the pages the block table names.
// Masks are by absolute position: key <= query, key >= the query's chunk start / window start.
// A token's result depends on its own row and keys only (tiles are walked in position order).
#include "api.h"
#include "common.cuh"
#include "mma.cuh"

namespace {

constexpr int BQ = 64;       // query rows per block
constexpr int TILE = 64;     // keys per tile
constexpr int NWARPS = 4;

template <int HD>
__global__ void __launch_bounds__(NWARPS * 32)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                    const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table,
                    int table_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ positions,
                    __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size, int chunk, int window,
                    float scale, int skip_single) {
  constexpr int STRIDE = HD + 8;
  constexpr int CHUNKS = HD / 8;
  constexpr int ROWS_PER_PASS = NWARPS * 32 / CHUNKS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [BQ][STRIDE]
  __nv_bfloat16* k_s = q_s + BQ * STRIDE;                            // [2][TILE][STRIDE]
  __nv_bfloat16* v_s = k_s + 2 * TILE * STRIDE;                      // [2][TILE][STRIDE]

  const int seq = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tok0 = cu_seqlens[seq] + qt * BQ;
  const int n_valid = min(BQ, cu_seqlens[seq + 1] - tok0);
  if (n_valid <= 0) return;
  // requests that bring one token are left to the decode kernel when the caller says so
  if (skip_single && cu_seqlens[seq + 1] - cu_seqlens[seq] == 1) return;
  const int kvh = h / (nh / nkv);
  const int p_first = positions[tok0];           // the rows of a tile are consecutive positions
  const int p_last = p_first + n_valid - 1;
  const int* table = block_table + (size_t)seq * table_stride;
  auto first_visible = [&](int pos) {
    int lo = 0;
    if (chunk > 0) lo = (pos / chunk) * chunk;
    if (window > 0 && pos - window + 1 > lo) lo = pos - window + 1;
    return lo;
  };
  const int tile_begin = first_visible(p_first) / TILE;    // lo grows with the position
  const int tile_end = p_last / TILE;                      // inclusive
  const bool tile_in_page = (page_size % TILE) == 0;

  const int ld_ch = tid % CHUNKS, ld_r0 = tid / CHUNKS;
  for (int r = ld_r0; r < BQ; r += ROWS_PER_PASS) {
    const bool ok = r < n_valid;
    hb::cp_async16(q_s + r * STRIDE + ld_ch * 8, q + ((size_t)(tok0 + (ok ? r : 0)) * nh + h) * HD + ld_ch * 8, ok);
  }
  auto load_tile = [&](int kt, int buf) {
    const int base = kt * TILE;
    __nv_bfloat16* kd = k_s + (buf * TILE + ld_r0) * STRIDE + ld_ch * 8;
    __nv_bfloat16* vd = v_s + (buf * TILE + ld_r0) * STRIDE + ld_ch * 8;
    if (tile_in_page) {
      const int page = table[base / page_size];
      const size_t off0 =
          (((size_t)(page >= 0 ? page : 0) * nkv + kvh) * page_size + (base % page_size) + ld_r0) * HD + ld_ch * 8;
#pragma unroll
      for (int i = 0; i < TILE / ROWS_PER_PASS; ++i) {
        const bool ok = page >= 0 && base + ld_r0 + i * ROWS_PER_PASS <= p_last;
        hb::cp_async16(kd + i * ROWS_PER_PASS * STRIDE, k_pages + off0 + (size_t)i * ROWS_PER_PASS * HD, ok);
        hb::cp_async16(vd + i * ROWS_PER_PASS * STRIDE, v_pages + off0 + (size_t)i * ROWS_PER_PASS * HD, ok);
      }
    } else {
#pragma unroll
      for (int i = 0; i < TILE / ROWS_PER_PASS; ++i) {
        const int key = base + ld_r0 + i * ROWS_PER_PASS;
        bool ok = key <= p_last;
        size_t off = 0;
        if (ok) {
          const int page = table[key / page_size];
          ok = page >= 0;
          off = (((size_t)(ok ? page : 0) * nkv + kvh) * page_size + (key % page_size)) * HD + ld_ch * 8;
        }
        hb::cp_async16(kd + i * ROWS_PER_PASS * STRIDE, k_pages + off, ok);
        hb::cp_async16(vd + i * ROWS_PER_PASS * STRIDE, v_pages + off, ok);
      }
    }
  };
  load_tile(tile_begin, 0);
  hb::cp_async_commit();

  // this thread's two rows of the warp's 16 (mma C layout): g and g + 8
  const int ra = warp * 16 + lane / 4, rb = ra + 8;
  const int pos_a = p_first + ra, pos_b = p_first + rb;
  const int lo_a = first_visible(pos_a), lo_b = first_visible(pos_b);
  const bool ok_a = ra < n_valid, ok_b = rb < n_valid;

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o_acc[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[j][e] = 0.f;
  unsigned q_frag[HD / 16][4];

  for (int kt = tile_begin; kt <= tile_end; ++kt) {
    const int buf = (kt - tile_begin) & 1;
    if (kt < tile_end) {
      load_tile(kt + 1, buf ^ 1);
      hb::cp_async_commit();
      hb::cp_async_wait<1>();
    } else {
      hb::cp_async_wait<0>();
    }
    __syncthreads();
    if (kt == tile_begin) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        hb::ldmatrix_x4(q_frag[ks], q_s + (warp * 16 + (lane % 16)) * STRIDE + ks * 16 + (lane / 16) * 8);
    }
    // a warp whose rows all end before this tile has nothing to add (rows of later warps still do)
    const int warp_last_pos = p_first + min(warp * 16 + 15, n_valid - 1);
    if (kt * TILE <= warp_last_pos && warp * 16 < n_valid) {
      const __nv_bfloat16* kt_s = k_s + buf * TILE * STRIDE;
      const __nv_bfloat16* vt_s = v_s + buf * TILE * STRIDE;
      float s_acc[TILE / 8][4];
#pragma unroll
      for (int nt = 0; nt < TILE / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s_acc[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < TILE / 16; ++np) {
          unsigned b[4];
          hb::ldmatrix_x4(b, kt_s + (np * 16 + (lane % 8) + (lane / 16) * 8) * STRIDE + ks * 16 + ((lane / 8) % 2) * 8);
          hb::mma_bf16(s_acc[2 * np], q_frag[ks], b[0], b[1]);
          hb::mma_bf16(s_acc[2 * np + 1], q_frag[ks], b[2], b[3]);
        }
      }
      const int key0 = kt * TILE + (lane % 4) * 2;
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < TILE / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + nt * 8 + (e & 1);
          const bool second = e >> 1;
          const bool vis = second ? (ok_b && key <= pos_b && key >= lo_b) : (ok_a && key <= pos_a && key >= lo_a);
          const float v = vis ? s_acc[nt][e] * scale : -INFINITY;
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
#pragma unroll
      for (int nt = 0; nt < TILE / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const float v = (s_acc[nt][e] == -INFINITY) ? 0.f : __expf(s_acc[nt][e] - m_run[r]);
          s_acc[nt][e] = v;
          row_sum[r] += v;
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float sum = row_sum[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l_run[r] = l_run[r] * corr[r] + sum;
      }
      if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) {
          o_acc[j][0] *= corr[0]; o_acc[j][1] *= corr[0];
          o_acc[j][2] *= corr[1]; o_acc[j][3] *= corr[1];
        }
      }
#pragma unroll
      for (int kk = 0; kk < TILE / 16; ++kk) {
        unsigned p_frag[4];
        p_frag[0] = hb::pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
        p_frag[1] = hb::pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
        p_frag[2] = hb::pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
        p_frag[3] = hb::pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
        for (int j = 0; j < HD / 8; j += 2) {
          unsigned b[4];
          hb::ldmatrix_x4_trans(b, vt_s + (kk * 16 + (lane % 8) + ((lane / 8) % 2) * 8) * STRIDE + j * 8 + (lane / 16) * 8);
          hb::mma_bf16(o_acc[j], p_frag, b[0], b[1]);
          hb::mma_bf16(o_acc[j + 1], p_frag, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  const float inv_a = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
  const float inv_b = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) {
    const int d = j * 8 + (lane % 4) * 2;
    if (ok_a)
      *reinterpret_cast<unsigned*>(out + ((size_t)(tok0 + ra) * nh + h) * HD + d) =
          hb::pack_bf16(o_acc[j][0] * inv_a, o_acc[j][1] * inv_a);
    if (ok_b)
      *reinterpret_cast<unsigned*>(out + ((size_t)(tok0 + rb) * nh + h) * HD + d) =
          hb::pack_bf16(o_acc[j][2] * inv_b, o_acc[j][3] * inv_b);
  }
}

template <int HD>
int launch_prefill(const void* q, const void* k_pages, const void* v_pages, const int* block_table, int table_stride,
                   const int* cu_seqlens, const int* positions, void* out, int n_seqs, int max_new, int nh, int nkv,
                   int page_size, int chunk, int window, float scale, int skip_single, cudaStream_t stream) {
  constexpr int STRIDE = HD + 8;
  const size_t smem = (size_t)(BQ * STRIDE + 4 * TILE * STRIDE) * sizeof(__nv_bfloat16);
  cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((max_new + BQ - 1) / BQ, nh, n_seqs);
  attn_prefill_kernel<HD><<<grid, NWARPS * 32, smem, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, table_stride,
      cu_seqlens, positions, (__nv_bfloat16*)out, nh, nkv, page_size, chunk, window, scale, skip_single);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // namespace

// bfloat16, head_dim 64 or 128. `cu_seqlens` [n_seqs + 1] are the first flat rows of the requests'
// new tokens, whose positions are consecutive; `max_new` is the longest run. Other shapes:
// HB_ERR_UNSUPPORTED (the caller uses the general kernel).
extern "C" int hb_attention_prefill(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                    int table_stride, const int* cu_seqlens, const int* positions, void* out,
                                    int n_seqs, int max_new, int nh, int nkv, int hd, int page_size, int chunk,
                                    int window, float scale, int skip_single, cudaStream_t stream) {
  if (!q || !k_pages || !v_pages || !block_table || !cu_seqlens || !positions || !out) return HB_ERR_BAD_ARG;
  if (n_seqs < 0 || max_new < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || table_stride <= 0 ||
      chunk < 0 || window < 0)
    return HB_ERR_BAD_ARG;
  if (n_seqs > 65535 || nh > 65535) return HB_ERR_UNSUPPORTED;
  if (n_seqs == 0 || max_new == 0) return HB_OK;
  if (hd == 128)
    return launch_prefill<128>(q, k_pages, v_pages, block_table, table_stride, cu_seqlens, positions, out, n_seqs,
                               max_new, nh, nkv, page_size, chunk, window, scale, skip_single, stream);
  if (hd == 64)
    return launch_prefill<64>(q, k_pages, v_pages, block_table, table_stride, cu_seqlens, positions, out, n_seqs,
                              max_new, nh, nkv, page_size, chunk, window, scale, skip_single, stream);
  return HB_ERR_UNSUPPORTED;
}
