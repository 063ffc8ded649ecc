// A whole-sequence float32 forward of a decoder on the CPU: plain loops, no cache, no GPU. It is
// the engine's reference execution (the counterpart of the reference's `--execution cpu-reference`,
// crates/hi-cuda/src/lib.rs:205-226, crates/hi-cuda/src/qwen_cpu.rs:84-261) and a second statement
// of the formulas beside the test-suite's plain model: the two are written apart and must agree.
//
// Formulas, in the order computed (crates/hi-mlx/src/models.rs):
//   block            h = x + attn(norm(x)); y = h + ffn(norm(h))                      6143-6149
//   rmsnorm          y = x * rsqrt(mean(x^2) + eps) * w                               1977-1979
//   projections      x W^T (+ bias where the checkpoint has one)                      1839-1847
//   rotation         pairs (j, j + hd/2) or (2j, 2j + 1), angle = pos * inv_freq[j]    5997-6016
//   q/k norm         weightless, after the rotation, its own eps                      6017-6021
//   temperature      q *= 1 + attn_scale * ln(1 + floor((pos + 1) / floor_scale))     (not in the reference)
//   attention        softmax(q k^T * scale + mask) v; q head h reads kv head h / (nh / nkv);
//                    mask: key <= query, and on windowed layers the key in the query's chunk
//                    or among its last `sliding` keys                                  5963, 6024-6050
//   experts          logits = x Wr^T; the k largest (ties to the lower id); s = sigmoid(logit);
//                    y = sum_e swiglu_e(s x) + swiglu_shared(x)                       6055-6103
//   swiglu           (silu(x Wg^T) * x Wu^T) Wd^T                                      2307-2312
//   head             logits = norm(y) W^T                                             6204-6217
#include <math.h>
#include <stdint.h>

#include <algorithm>
#include <vector>

#include "runtime.h"

namespace {

void rmsnorm(const float* x, const float* w, float eps, int n, float* y) {
  float ss = 0.f;
  for (int i = 0; i < n; ++i) ss += x[i] * x[i];
  const float inv = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = 0; i < n; ++i) y[i] = x[i] * inv * (w ? w[i] : 1.f);
}

// y[o] = sum_i x[i] * w[o * n_in + i] (+ b[o])
void linear(const float* x, const float* w, const float* b, int n_in, int n_out, float* y) {
  for (int o = 0; o < n_out; ++o) {
    const float* row = w + (size_t)o * n_in;
    float s = 0.f;
    for (int i = 0; i < n_in; ++i) s += x[i] * row[i];
    y[o] = b ? s + b[o] : s;
  }
}

void swiglu(const float* x, const float* wg, const float* wu, const float* wd, int hidden, int inter, float scale,
            std::vector<float>& act, float* y_add) {
  act.resize(inter);
  for (int j = 0; j < inter; ++j) {
    const float* g = wg + (size_t)j * hidden;
    const float* u = wu + (size_t)j * hidden;
    float sg = 0.f, su = 0.f;
    for (int i = 0; i < hidden; ++i) {
      sg += x[i] * g[i];
      su += x[i] * u[i];
    }
    sg *= scale;          // the router's score scales the expert's input: by linearity, its two products
    su *= scale;
    act[j] = sg / (1.f + expf(-sg)) * su;
  }
  for (int o = 0; o < hidden; ++o) {
    const float* d = wd + (size_t)o * inter;
    float s = 0.f;
    for (int j = 0; j < inter; ++j) s += act[j] * d[j];
    y_add[o] += s;
  }
}

void rotate(float* v, int half, int pos, const float* inv_freq, int interleaved) {   // the first 2 * half dims
  for (int j = 0; j < half; ++j) {
    const float ang = (float)pos * inv_freq[j];
    const float c = cosf(ang), s = sinf(ang);
    const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
    const float a = v[ia], b = v[ib];
    v[ia] = a * c - b * s;
    v[ib] = b * c + a * s;
  }
}

}  // namespace

extern "C" int hbh_cpu_forward(const hbh_cpu_model* m, const hbh_cpu_layer* layers, const int* schedule, int n_schedule,
                               const int* tokens, int n_tokens, const int* want, int n_want, float* logits,
                               int* router_ids) {
  if (!m || !layers || !schedule || !tokens || !m->embedding || !m->head || n_tokens <= 0 || n_want < 0 ||
      (n_want > 0 && (!want || !logits)))
    return HBH_ERR_ARG;
  const int H = m->hidden, T = n_tokens;
  std::vector<float> x((size_t)T * H), z(H), tmp(H), act;
  for (int t = 0; t < T; ++t) {
    if (tokens[t] < 0 || tokens[t] >= m->vocab) return HBH_ERR_ARG;
    std::copy(m->embedding + (size_t)tokens[t] * H, m->embedding + (size_t)(tokens[t] + 1) * H, x.begin() + (size_t)t * H);
  }
  int routed_seen = 0;
  for (int si = 0; si < n_schedule; ++si) {
    const hbh_cpu_layer& L = layers[schedule[si]];
    // ---- the mixer
    if (L.mixer != HBH_CPU_ATTENTION) return HBH_ERR_ARG;
    const int nh = L.heads, nkv = L.kv_heads, hd = L.head_dim, group = nh / nkv;
    std::vector<float> q((size_t)T * nh * hd), k((size_t)T * nkv * hd), v((size_t)T * nkv * hd), o((size_t)nh * hd);
    for (int t = 0; t < T; ++t) {
      rmsnorm(&x[(size_t)t * H], L.norm_mixer, L.norm_eps, H, z.data());
      float* qt = &q[(size_t)t * nh * hd];
      float* kt = &k[(size_t)t * nkv * hd];
      linear(z.data(), L.wq, L.bq, H, nh * hd, qt);
      linear(z.data(), L.wk, L.bk, H, nkv * hd, kt);
      linear(z.data(), L.wv, L.bv, H, nkv * hd, &v[(size_t)t * nkv * hd]);
      for (int h = 0; h < nh + nkv; ++h) {
        float* head = h < nh ? qt + (size_t)h * hd : kt + (size_t)(h - nh) * hd;
        if (L.inv_freq) rotate(head, L.rot_pairs, t, L.inv_freq, L.interleaved);
        float mul = 1.f;
        if (L.qk_norm) {
          float ss = 0.f;
          for (int d = 0; d < hd; ++d) ss += head[d] * head[d];
          mul = 1.f / sqrtf(ss / (float)hd + L.qk_eps);
        }
        if (h < nh && L.temperature)
          mul *= logf(floorf(((float)t + 1.f) / L.floor_scale) + 1.f) * L.attn_scale + 1.f;
        for (int d = 0; d < hd; ++d) head[d] *= mul;
      }
    }
    std::vector<float> p(T);
    for (int t = 0; t < T; ++t) {
      int lo = 0;
      if (L.chunk > 0) lo = (t / L.chunk) * L.chunk;
      if (L.sliding > 0) lo = std::max(lo, t - L.sliding + 1);
      for (int h = 0; h < nh; ++h) {
        const float* qh = &q[((size_t)t * nh + h) * hd];
        const int kvh = h / group;
        float mx = -INFINITY;
        for (int s = lo; s <= t; ++s) {
          const float* kh = &k[((size_t)s * nkv + kvh) * hd];
          float dot = 0.f;
          for (int d = 0; d < hd; ++d) dot += qh[d] * kh[d];
          p[s] = dot * L.scale;
          mx = std::max(mx, p[s]);
        }
        float sum = 0.f;
        for (int s = lo; s <= t; ++s) {
          p[s] = expf(p[s] - mx);
          sum += p[s];
        }
        float* oh = &o[(size_t)h * hd];
        std::fill(oh, oh + hd, 0.f);
        for (int s = lo; s <= t; ++s) {
          const float w = p[s] / sum;
          const float* vh = &v[((size_t)s * nkv + kvh) * hd];
          for (int d = 0; d < hd; ++d) oh[d] += w * vh[d];
        }
      }
      linear(o.data(), L.wo, L.bo, nh * hd, H, tmp.data());
      for (int i = 0; i < H; ++i) x[(size_t)t * H + i] += tmp[i];
    }
    // ---- the feed-forward
    for (int t = 0; t < T; ++t) {
      float* xt = &x[(size_t)t * H];
      rmsnorm(xt, L.norm_feed_forward, L.norm_eps, H, z.data());
      std::fill(tmp.begin(), tmp.end(), 0.f);
      if (L.feed_forward == HBH_CPU_DENSE) {
        swiglu(z.data(), L.w_gate, L.w_up, L.w_down, H, L.inter, 1.f, act, tmp.data());
      } else if (L.feed_forward == HBH_CPU_EXPERTS) {
        const int E = L.experts, K = L.top_k;
        std::vector<float> lg(E);
        linear(z.data(), L.router, nullptr, H, E, lg.data());
        std::vector<int> chosen;
        const int* forced = L.forced_ids ? L.forced_ids + (size_t)t * K : nullptr;
        for (int r = 0; r < K; ++r) {
          int best = -1;
          if (forced) {
            best = forced[r];
            if (best < 0 || best >= E) return HBH_ERR_ARG;
          } else {
            for (int e = 0; e < E; ++e) {
              if (std::find(chosen.begin(), chosen.end(), e) != chosen.end()) continue;
              if (best < 0 || lg[e] > lg[best]) best = e;      // strict '>': the lower id on ties
            }
          }
          chosen.push_back(best);
          if (router_ids) router_ids[((size_t)routed_seen * T + t) * K + r] = best;
          const float score = 1.f / (1.f + expf(-lg[best]));
          const size_t gu = (size_t)best * L.inter * H;
          swiglu(z.data(), L.w_gate + gu, L.w_up + gu, L.w_down + (size_t)best * H * L.inter, H, L.inter, score, act,
                 tmp.data());
        }
        if (L.shared_gate)
          swiglu(z.data(), L.shared_gate, L.shared_up, L.shared_down, H, L.shared_inter, 1.f, act, tmp.data());
      } else {
        return HBH_ERR_ARG;
      }
      for (int i = 0; i < H; ++i) xt[i] += tmp[i];
    }
    if (L.feed_forward == HBH_CPU_EXPERTS) ++routed_seen;
  }
  for (int r = 0; r < n_want; ++r) {
    if (want[r] < 0 || want[r] >= T) return HBH_ERR_ARG;
    rmsnorm(&x[(size_t)want[r] * H], m->final_norm, m->final_eps, H, z.data());
    linear(z.data(), m->head, nullptr, H, m->vocab, logits + (size_t)r * m->vocab);
  }
  return HBH_OK;
}
