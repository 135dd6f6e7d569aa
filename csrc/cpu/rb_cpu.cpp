// C++ f32 reference backend.  Straightforward loops, blocked where it matters, std::thread row parallelism.
#include "rb_cpu.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

namespace {
int g_threads = 0;

int num_threads() {
  if (g_threads > 0) return g_threads;
  const unsigned hc = std::thread::hardware_concurrency();
  return hc ? (int)hc : 4;
}

// Runs f(lo, hi) over [0, n) split into contiguous ranges; small problems stay on the calling thread.
void parallel_for(int64_t n, int64_t grain, const std::function<void(int64_t, int64_t)>& f) {
  const int nt = (int)std::min<int64_t>(num_threads(), std::max<int64_t>(1, n / std::max<int64_t>(grain, 1)));
  if (nt <= 1) { f(0, n); return; }
  std::vector<std::thread> ts;
  const int64_t per = (n + nt - 1) / nt;
  for (int t = 0; t < nt; ++t) {
    const int64_t lo = t * per, hi = std::min<int64_t>(n, lo + per);
    if (lo >= hi) break;
    ts.emplace_back([=, &f] { f(lo, hi); });
  }
  for (auto& t : ts) t.join();
}

inline float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + std::tanh(k0 * (x + k1 * x * x * x)));
}
inline float act_apply(int act, float v) {
  switch (act) {
    case 1: return gelu_tanh(v);
    case 2: return v > 0.f ? v : 0.f;
    case 3: return v / (1.f + std::exp(-v));
    default: return v;
  }
}
}  // namespace

extern "C" {

void rb_cpu_set_threads(int n) { g_threads = n; }

void rb_cpu_matmul(const float* a, const float* b, float* c, int m, int k, int n) {
  parallel_for(m, 8, [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) {
      float* ci = c + i * n;
      std::memset(ci, 0, sizeof(float) * n);
      for (int p = 0; p < k; ++p) {
        const float av = a[i * k + p];
        const float* bp = b + (int64_t)p * n;
        for (int j = 0; j < n; ++j) ci[j] += av * bp[j];
      }
    }
  });
}

void rb_cpu_linear(const float* x, const float* w, const float* bias, float* y, int batch, int in, int out, int act) {
  parallel_for(batch, 4, [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) {
      const float* xi = x + i * in;
      for (int o = 0; o < out; ++o) {
        const float* wo = w + (int64_t)o * in;
        float acc = 0.f;
        for (int p = 0; p < in; ++p) acc += xi[p] * wo[p];
        if (bias) acc += bias[o];
        y[i * out + o] = act_apply(act, acc);
      }
    }
  });
}

void rb_cpu_softmax_rows(const float* x, float* y, int rows, int n, int log_mode) {
  parallel_for(rows, 16, [&](int64_t lo, int64_t hi) {
    for (int64_t r = lo; r < hi; ++r) {
      const float* xr = x + r * n;
      float* yr = y + r * n;
      float mx = xr[0];
      for (int j = 1; j < n; ++j) mx = std::max(mx, xr[j]);
      double s = 0.0;
      for (int j = 0; j < n; ++j) s += std::exp((double)xr[j] - mx);
      const float lse = mx + (float)std::log(s);
      for (int j = 0; j < n; ++j) yr[j] = log_mode ? xr[j] - lse : std::exp(xr[j] - lse);
    }
  });
}

void rb_cpu_layer_norm(const float* x, const float* gamma, const float* beta, float* y, float* mean, float* rstd,
                       int rows, int n, float eps, int rms) {
  parallel_for(rows, 16, [&](int64_t lo, int64_t hi) {
    for (int64_t r = lo; r < hi; ++r) {
      const float* xr = x + r * n;
      double mu = 0.0;
      if (!rms) { for (int j = 0; j < n; ++j) mu += xr[j]; mu /= n; }
      double var = 0.0;
      for (int j = 0; j < n; ++j) { const double d = xr[j] - mu; var += d * d; }
      var /= n;
      const float rs = 1.f / std::sqrt((float)var + eps);
      if (mean) mean[r] = (float)mu;
      if (rstd) rstd[r] = rs;
      for (int j = 0; j < n; ++j) {
        float v = ((float)(xr[j] - mu)) * rs;
        if (gamma) v *= gamma[j];
        if (beta && !rms) v += beta[j];
        y[r * n + j] = v;
      }
    }
  });
}

void rb_cpu_layer_norm_bwd(const float* dy, const float* x, const float* gamma, const float* mean, const float* rstd,
                           float* dx, float* dgamma, float* dbeta, int rows, int n, int rms) {
  if (dgamma) std::memset(dgamma, 0, sizeof(float) * n);
  if (dbeta) std::memset(dbeta, 0, sizeof(float) * n);
  for (int64_t r = 0; r < rows; ++r) {
    const float mu = rms ? 0.f : mean[r], rs = rstd[r];
    double s1 = 0.0, s2 = 0.0;
    for (int j = 0; j < n; ++j) {
      const float xh = (x[r * n + j] - mu) * rs;
      const float d = dy[r * n + j];
      if (dgamma) dgamma[j] += d * xh;
      if (dbeta && !rms) dbeta[j] += d;
      const float gd = d * (gamma ? gamma[j] : 1.f);
      s1 += gd;
      s2 += gd * xh;
    }
    s1 = rms ? 0.0 : s1 / n;
    s2 /= n;
    for (int j = 0; j < n; ++j) {
      const float xh = (x[r * n + j] - mu) * rs;
      const float gd = dy[r * n + j] * (gamma ? gamma[j] : 1.f);
      dx[r * n + j] = rs * (gd - (float)s1 - xh * (float)s2);
    }
  }
}

void rb_cpu_unary(int op, const float* x, float* y, int64_t n) {
  parallel_for(n, 1 << 14, [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) {
      const float a = x[i];
      float r;
      switch (op) {
        case 0: r = a > 0.f ? a : 0.f; break;
        case 1: r = 1.f / (1.f + std::exp(-a)); break;
        case 2: r = std::tanh(a); break;
        case 3: r = std::exp(a); break;
        case 4: r = std::log(a); break;
        case 5: r = std::sqrt(a); break;
        case 6: r = -a; break;
        case 7: r = gelu_tanh(a); break;
        case 8: r = a / (1.f + std::exp(-a)); break;
        default: r = a;
      }
      y[i] = r;
    }
  });
}

void rb_cpu_cross_entropy(const float* logits, const int64_t* targets, float* loss, float* dlogits, int rows, int n,
                          float scale, int64_t ignore_index) {
  parallel_for(rows, 8, [&](int64_t lo, int64_t hi) {
    for (int64_t r = lo; r < hi; ++r) {
      const float* xr = logits + r * n;
      float mx = xr[0];
      for (int j = 1; j < n; ++j) mx = std::max(mx, xr[j]);
      double s = 0.0;
      for (int j = 0; j < n; ++j) s += std::exp((double)xr[j] - mx);
      const float lse = mx + (float)std::log(s);
      const int64_t t = targets[r];
      const bool ignored = (t == ignore_index) || t < 0 || t >= n;
      loss[r] = ignored ? 0.f : lse - xr[t];
      if (dlogits) {
        const float gs = ignored ? 0.f : scale;
        for (int j = 0; j < n; ++j) dlogits[r * n + j] = (std::exp(xr[j] - lse) - (j == t ? 1.f : 0.f)) * gs;
      }
    }
  });
}

void rb_cpu_adam(float* p, float* m, float* v, const float* g, int64_t n, float lr, float b1, float b2, float eps,
                 float wd, int step, int decoupled) {
  const float bc1 = 1.f - std::pow(b1, (float)step), bc2 = 1.f - std::pow(b2, (float)step);
  parallel_for(n, 1 << 15, [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) {
      float gi = g[i];
      if (!decoupled) gi += wd * p[i];
      m[i] = b1 * m[i] + (1.f - b1) * gi;
      v[i] = b2 * v[i] + (1.f - b2) * gi * gi;
      float upd = (m[i] / bc1) / (std::sqrt(v[i] / bc2) + eps);
      if (decoupled) upd += wd * p[i];
      p[i] -= lr * upd;
    }
  });
}

void rb_cpu_attention(const float* q, const float* k, const float* v, float* o, int B, int Sq, int Sk, int H, int Hkv,
                      int D, int causal, float scale) {
  const int group = H / Hkv, shift = Sk - Sq;
  parallel_for((int64_t)B * H * Sq, 16, [&](int64_t lo, int64_t hi) {
    std::vector<float> sc(Sk);
    for (int64_t idx = lo; idx < hi; ++idx) {
      const int s = (int)(idx % Sq);
      const int h = (int)((idx / Sq) % H);
      const int b = (int)(idx / ((int64_t)Sq * H));
      const int hk = h / group;
      const float* qp = q + (((int64_t)b * Sq + s) * H + h) * D;
      const int lim = causal ? std::min(Sk, s + shift + 1) : Sk;
      float mx = -INFINITY;
      for (int j = 0; j < lim; ++j) {
        const float* kp = k + (((int64_t)b * Sk + j) * Hkv + hk) * D;
        float acc = 0.f;
        for (int d = 0; d < D; ++d) acc += qp[d] * kp[d];
        sc[j] = acc * scale;
        mx = std::max(mx, sc[j]);
      }
      double den = 0.0;
      for (int j = 0; j < lim; ++j) { sc[j] = std::exp(sc[j] - mx); den += sc[j]; }
      float* op = o + (((int64_t)b * Sq + s) * H + h) * D;
      for (int d = 0; d < D; ++d) op[d] = 0.f;
      for (int j = 0; j < lim; ++j) {
        const float w = (float)(sc[j] / den);
        const float* vp = v + (((int64_t)b * Sk + j) * Hkv + hk) * D;
        for (int d = 0; d < D; ++d) op[d] += w * vp[d];
      }
    }
  });
}

void rb_cpu_moe_route(const float* logits, int T, int E, int k, int renorm, int32_t* idx_out, float* w_out, float* aux_out) {
  std::vector<double> frac(E, 0.0), meanp(E, 0.0);
  std::vector<float> p(E);
  std::vector<int> order(E);
  for (int t = 0; t < T; ++t) {
    const float* x = logits + (int64_t)t * E;
    float mx = x[0];
    for (int e = 1; e < E; ++e) mx = std::max(mx, x[e]);
    double s = 0.0;
    for (int e = 0; e < E; ++e) { p[e] = std::exp(x[e] - mx); s += p[e]; }
    for (int e = 0; e < E; ++e) { p[e] = (float)(p[e] / s); meanp[e] += p[e]; order[e] = e; }
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return p[a] > p[b]; });
    float tot = 0.f;
    for (int j = 0; j < k; ++j) tot += p[order[j]];
    for (int j = 0; j < k; ++j) {
      idx_out[(int64_t)t * k + j] = order[j];
      w_out[(int64_t)t * k + j] = renorm ? p[order[j]] / tot : p[order[j]];
      frac[order[j]] += 1.0;
    }
  }
  double aux = 0.0;
  for (int e = 0; e < E; ++e) aux += (frac[e] / ((double)T * k)) * (meanp[e] / T);
  if (aux_out) *aux_out = (float)(aux * E);
}

void rb_cpu_gather_rows(const float* table, const int64_t* ids, float* out, int64_t n_ids, int cols, int64_t rows) {
  for (int64_t i = 0; i < n_ids; ++i) {
    const int64_t r = ids[i];
    if (r < 0 || r >= rows) { std::memset(out + i * cols, 0, sizeof(float) * cols); continue; }
    std::memcpy(out + i * cols, table + r * cols, sizeof(float) * cols);
  }
}

void rb_cpu_scatter_add_rows(const float* src, const int64_t* ids, float* table, int64_t n_ids, int cols, int64_t rows) {
  for (int64_t i = 0; i < n_ids; ++i) {
    const int64_t r = ids[i];
    if (r < 0 || r >= rows) continue;
    for (int c = 0; c < cols; ++c) table[r * cols + c] += src[i * cols + c];
  }
}

}  // extern "C"
