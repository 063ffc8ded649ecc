// Decode attention over the paged cache, bfloat16: one new token per request against a long
// range of keys. Flash-decoding with the query heads of a kv head packed into one tile:
//   grid (split, kv head, token); the G = nh / nkv query heads are the rows of a 16-row tile,
//   so each key and value row is read once for all of them
//   (crates/hi-cuda/src/kernels.cu:6804-7006 does this with float32 FMAs; here the products
//   run on the tensor cores, mma.sync m16n8k16, with float32 accumulation and softmax).
// A split is a fixed run of `split_size` keys counted from the token's first visible key, so
// the cut depends on the token's own range only. K and V tiles of 64 keys are staged in shared
// memory with cp.async (double-buffered); each of the 4 warps takes 16 keys of a tile and keeps
// its own running max / sum / output, merged in warp order at the end. Partials (m, l, acc) go
// to scratch and are merged across splits by attention_merge (attention.cu).
#include <cuda_bf16.h>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int TILE = 64;     // keys per shared-memory tile
constexpr int NWARPS = 4;
constexpr int ROWS = 16;     // query rows of the tile (heads of one kv group, padded)

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = pred ? 16 : 0;   // src-size 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(NWARPS * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                   const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table,
                   int table_stride, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                   __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size, int chunk, int window,
                   float scale, int split_size, int max_splits, float* __restrict__ part_acc,
                   float* __restrict__ part_ml) {
  constexpr int STRIDE = HD + 8;                 // padded row: ldmatrix without bank conflicts
  constexpr int CHUNKS = HD / 8;                 // 16-byte chunks per row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);             // [ROWS][STRIDE]
  __nv_bfloat16* k_s = q_s + ROWS * STRIDE;                                     // [2][TILE][STRIDE]
  __nv_bfloat16* v_s = k_s + 2 * TILE * STRIDE;                                 // [2][TILE][STRIDE]
  float* ml_s = reinterpret_cast<float*>(v_s + 2 * TILE * STRIDE);              // [NWARPS][ROWS][2]
  float* o_s = reinterpret_cast<float*>(k_s);   // [ROWS][HD], reuses the K tiles once the key loop is over

  const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = nh / nkv;
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * table_stride;
  int lo = 0;
  if (chunk > 0) lo = (pos / chunk) * chunk;
  if (window > 0 && pos - window + 1 > lo) lo = pos - window + 1;
  const int first = lo + split * split_size;
  const size_t th0 = (size_t)t * nh + (size_t)kvh * G;      // (token, first head of the group)
  if (first > pos) {                                          // this token has fewer splits
    if (max_splits > 1 && tid < G) {
      float* ml = part_ml + ((th0 + tid) * max_splits + split) * 2;
      ml[0] = -INFINITY; ml[1] = 0.f;
    }
    return;
  }
  const int last = min(pos, first + split_size - 1);
  const int n_tiles = (last - first + TILE) / TILE;

  // the query rows of this kv group
  for (int c = tid; c < ROWS * CHUNKS; c += NWARPS * 32) {
    const int r = c / CHUNKS, ch = c % CHUNKS;
    const bool ok = r < G;
    cp_async16(q_s + r * STRIDE + ch * 8, q + (th0 + (ok ? r : 0)) * HD + ch * 8, ok);
  }
  // thread -> one 16-byte chunk column and every (128 / CHUNKS)-th row of a tile. When a tile
  // never straddles a page (page_size a multiple of TILE and the range starts on a TILE
  // boundary) one table lookup serves the whole tile.
  constexpr int ROWS_PER_PASS = NWARPS * 32 / CHUNKS;
  const int ld_ch = tid % CHUNKS, ld_r0 = tid / CHUNKS;
  const bool tile_in_page = (page_size % TILE == 0) && (first % TILE == 0);
  auto load_tile = [&](int tile, int buf) {
    const int base = first + tile * TILE;
    __nv_bfloat16* kd = k_s + (buf * TILE + ld_r0) * STRIDE + ld_ch * 8;
    __nv_bfloat16* vd = v_s + (buf * TILE + ld_r0) * STRIDE + ld_ch * 8;
    if (tile_in_page) {
      const int page = table[base / page_size];
      const size_t off0 = (((size_t)(page >= 0 ? page : 0) * nkv + kvh) * page_size + (base % page_size) + ld_r0) * HD + ld_ch * 8;
      const __nv_bfloat16* ks = k_pages + off0;
      const __nv_bfloat16* vs = v_pages + off0;
#pragma unroll
      for (int i = 0; i < TILE / ROWS_PER_PASS; ++i) {
        const bool ok = page >= 0 && base + ld_r0 + i * ROWS_PER_PASS <= last;
        cp_async16(kd + i * ROWS_PER_PASS * STRIDE, ks + (size_t)i * ROWS_PER_PASS * HD, ok);
        cp_async16(vd + i * ROWS_PER_PASS * STRIDE, vs + (size_t)i * ROWS_PER_PASS * HD, ok);
      }
    } else {
#pragma unroll
      for (int i = 0; i < TILE / ROWS_PER_PASS; ++i) {
        const int key = base + ld_r0 + i * ROWS_PER_PASS;
        bool ok = key <= last;
        size_t off = 0;
        if (ok) {
          const int page = table[key / page_size];
          ok = page >= 0;
          off = (((size_t)(ok ? page : 0) * nkv + kvh) * page_size + (key % page_size)) * HD + ld_ch * 8;
        }
        cp_async16(kd + i * ROWS_PER_PASS * STRIDE, k_pages + off, ok);
        cp_async16(vd + i * ROWS_PER_PASS * STRIDE, v_pages + off, ok);
      }
    }
  };
  load_tile(0, 0);
  cp_async_commit();

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o_acc[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[j][e] = 0.f;
  unsigned q_frag[HD / 16][4];

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) {
      load_tile(tile + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (tile == 0) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(q_frag[ks], q_s + (lane % 16) * STRIDE + ks * 16 + (lane / 16) * 8);
    }
    const __nv_bfloat16* kt = k_s + (buf * TILE + warp * 16) * STRIDE;
    const __nv_bfloat16* vt = v_s + (buf * TILE + warp * 16) * STRIDE;
    // S = Q K^T for this warp's 16 keys: two 8-key column tiles
    float s_acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      unsigned b[4];
      ldmatrix_x4(b, kt + ((lane % 8) + (lane / 16) * 8) * STRIDE + ks * 16 + ((lane / 8) % 2) * 8);
      mma_bf16(s_acc[0], q_frag[ks], b[0], b[1]);
      mma_bf16(s_acc[1], q_frag[ks], b[2], b[3]);
    }
    // scale, mask keys past the split's end, online softmax per row (rows lane/4 and lane/4 + 8)
    const int key0 = first + tile * TILE + warp * 16 + (lane % 4) * 2;
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + nt * 8 + (e & 1);
        const float v = key <= last ? s_acc[nt][e] * scale : -INFINITY;
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
      p_frag[0] = pack_bf16(p[0][0], p[0][1]);
      p_frag[1] = pack_bf16(p[0][2], p[0][3]);
      p_frag[2] = pack_bf16(p[1][0], p[1][1]);
      p_frag[3] = pack_bf16(p[1][2], p[1][3]);
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
#pragma unroll
    for (int j = 0; j < HD / 8; j += 2) {
      unsigned b[4];
      ldmatrix_x4_trans(b, vt + ((lane % 8) + ((lane / 8) % 2) * 8) * STRIDE + j * 8 + (lane / 16) * 8);
      mma_bf16(o_acc[j], p_frag, b[0], b[1]);
      mma_bf16(o_acc[j + 1], p_frag, b[2], b[3]);
    }
    __syncthreads();      // everyone is done with this buffer before it is refilled
  }

  // merge the four warps (each saw a quarter of the keys), in warp order
  const int r0 = lane / 4;
  if ((lane % 4) == 0) {
    ml_s[(warp * ROWS + r0) * 2] = m_run[0];     ml_s[(warp * ROWS + r0) * 2 + 1] = l_run[0];
    ml_s[(warp * ROWS + r0 + 8) * 2] = m_run[1]; ml_s[(warp * ROWS + r0 + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  float m_all[2], f[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r0 + 8 * r;
    float mx = -INFINITY;
    for (int w = 0; w < NWARPS; ++w) mx = fmaxf(mx, ml_s[(w * ROWS + row) * 2]);
    m_all[r] = mx;
    f[r] = (m_run[r] == -INFINITY) ? 0.f : expf(m_run[r] - mx);
  }
  for (int w = 0; w < NWARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) {
        const int d = j * 8 + (lane % 4) * 2;
        float* a = o_s + r0 * HD + d;
        float* b = o_s + (r0 + 8) * HD + d;
        if (w == 0) {
          a[0] = o_acc[j][0] * f[0]; a[1] = o_acc[j][1] * f[0];
          b[0] = o_acc[j][2] * f[1]; b[1] = o_acc[j][3] * f[1];
        } else {
          a[0] += o_acc[j][0] * f[0]; a[1] += o_acc[j][1] * f[0];
          b[0] += o_acc[j][2] * f[1]; b[1] += o_acc[j][3] * f[1];
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
    if (max_splits > 1) {
      part_acc[((th0 + row) * max_splits + split) * HD + d] = o;
      if (d == 0) {
        float* ml = part_ml + ((th0 + row) * max_splits + split) * 2;
        ml[0] = mx; ml[1] = l;
      }
    } else {
      out[(th0 + row) * HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
  }
  (void)m_all;
}

template <int HD>
int launch_decode(const void* q, const void* k_pages, const void* v_pages, const int* block_table, int table_stride,
                  const int* seq_of_token, const int* positions, void* out, int n_tokens, int nh, int nkv,
                  int page_size, int chunk, int window, float scale, int split_size, int max_splits, float* part_acc,
                  float* part_ml, cudaStream_t stream) {
  constexpr int STRIDE = HD + 8;
  const size_t smem = (size_t)(ROWS * STRIDE + 4 * TILE * STRIDE) * sizeof(__nv_bfloat16) +
                      (size_t)(NWARPS * ROWS * 2) * sizeof(float);
  static_assert(2 * TILE * STRIDE * sizeof(__nv_bfloat16) >= ROWS * HD * sizeof(float), "o_s aliases the K tiles");
  cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(max_splits, nkv, n_tokens);
  attn_decode_kernel<HD><<<grid, NWARPS * 32, smem, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, table_stride,
      seq_of_token, positions, (__nv_bfloat16*)out, nh, nkv, page_size, chunk, window, scale, split_size, max_splits,
      part_acc, part_ml);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // namespace

// bfloat16 only; head_dim 64 or 128; at most 16 query heads per kv head; every token is taken
// as one decode row. Returns HB_ERR_UNSUPPORTED for other shapes (the caller then uses the
// general kernel). The merge over splits is hb_attention_merge.
extern "C" int hb_attention_decode(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                   int table_stride, const int* seq_of_token, const int* positions, void* out,
                                   int n_tokens, int nh, int nkv, int hd, int page_size, int chunk, int window,
                                   float scale, int split_size, int max_splits, float* part_acc, float* part_ml,
                                   cudaStream_t stream) {
  if (!q || !k_pages || !v_pages || !block_table || !seq_of_token || !positions || !out) return HB_ERR_BAD_ARG;
  if (n_tokens < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || table_stride <= 0 || chunk < 0 ||
      window < 0 || max_splits < 1 || split_size <= 0 || split_size % TILE != 0)
    return HB_ERR_BAD_ARG;
  if (max_splits > 1 && (!part_acc || !part_ml)) return HB_ERR_BAD_ARG;
  if (nh / nkv > ROWS || n_tokens > 65535 || nkv > 65535) return HB_ERR_UNSUPPORTED;
  if (n_tokens == 0) return HB_OK;
  if (hd == 128)
    return launch_decode<128>(q, k_pages, v_pages, block_table, table_stride, seq_of_token, positions, out, n_tokens,
                              nh, nkv, page_size, chunk, window, scale, split_size, max_splits, part_acc, part_ml, stream);
  if (hd == 64)
    return launch_decode<64>(q, k_pages, v_pages, block_table, table_stride, seq_of_token, positions, out, n_tokens,
                             nh, nkv, page_size, chunk, window, scale, split_size, max_splits, part_acc, part_ml, stream);
  return HB_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------
// The entry point that allocates nothing (see attention_decode_static.h): the same kernel, its
// split partials kept in a file-scope device array instead of caller-provided scratch.
#include <stdio.h>

#include "attention_decode_static.h"

namespace {

// [acc: HB_STATIC_SCRATCH_ACC_FLOATS][ml: HB_STATIC_SCRATCH_ML_FLOATS]
static __device__ __align__(256) float g_static_scratch[HB_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_static_scratch_ptr[kMaxDevices] = {};   // device address of the array, per device

// In host code `g_static_scratch` is only a handle; the address the kernels need comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch(float** acc, float** ml) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return HB_ERR_UNSUPPORTED;
  if (!g_static_scratch_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    if (!p) return HB_ERR_BAD_ARG;
    g_static_scratch_ptr[dev] = p;
  }
  *acc = g_static_scratch_ptr[dev];
  *ml = g_static_scratch_ptr[dev] + HB_STATIC_SCRATCH_ACC_FLOATS;
  return HB_OK;
}

}  // namespace

extern "C" long long hb_attention_decode_static_need(int n_tokens, int nh, int hd, int max_splits) {
  if (max_splits <= 1) return 0;
  return (long long)n_tokens * nh * max_splits * ((long long)hd + 2);
}

extern "C" int hb_attention_decode_static_fits(int n_tokens, int nh, int hd, int max_splits) {
  if (n_tokens < 0 || nh <= 0 || hd <= 0 || max_splits < 1) return 0;
  if (max_splits == 1) return 1;
  const long long rows = (long long)n_tokens * nh * max_splits;
  return rows * hd <= HB_STATIC_SCRATCH_ACC_FLOATS && rows * 2 <= HB_STATIC_SCRATCH_ML_FLOATS ? 1 : 0;
}

extern "C" int hb_attention_decode_static(const void* q, const void* k_pages, const void* v_pages,
                                          const int* block_table, int table_stride, const int* seq_of_token,
                                          const int* positions, void* out, int n_tokens, int nh, int nkv, int hd,
                                          int page_size, int chunk, int window, float scale, int split_size,
                                          int max_splits, cudaStream_t stream) {
  if (n_tokens < 0 || nh <= 0 || hd <= 0 || max_splits < 1) return HB_ERR_BAD_ARG;
  float *acc = nullptr, *ml = nullptr;
  if (max_splits > 1) {
    const long long acc_need = (long long)n_tokens * nh * max_splits * hd;
    const long long ml_need = (long long)n_tokens * nh * max_splits * 2;
    if (!hb_attention_decode_static_fits(n_tokens, nh, hd, max_splits)) {
      fprintf(stderr,
              "hb_attention_decode_static: %d tokens x %d heads x %d splits x head_dim %d need %lld + %lld floats of "
              "scratch; the built-in array holds %d + %d. Use fewer splits or hb_attention_decode.\n",
              n_tokens, nh, max_splits, hd, acc_need, ml_need, HB_STATIC_SCRATCH_ACC_FLOATS,
              HB_STATIC_SCRATCH_ML_FLOATS);
      return HB_ERR_SCRATCH_CAPACITY;
    }
    const int rc = static_scratch(&acc, &ml);
    if (rc != HB_OK) return rc;
  }
  int rc = hb_attention_decode(q, k_pages, v_pages, block_table, table_stride, seq_of_token, positions, out, n_tokens,
                               nh, nkv, hd, page_size, chunk, window, scale, split_size, max_splits, acc, ml, stream);
  if (rc != HB_OK || max_splits == 1 || n_tokens == 0) return rc;
  return hb_attention_merge(acc, ml, out, HB_DTYPE_BF16, n_tokens * nh, hd, max_splits, stream);
}
