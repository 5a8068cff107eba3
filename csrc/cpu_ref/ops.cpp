// CPU restatements of the reference's scalar hot loops, used as oracles and as the timed CPU baseline:
//   flash attention  - exact softmax attention, one query at a time, streaming over the keys with a running maximum and
//                      sum (rust-nn src/tensor.rs:633-662; the same arithmetic as its WGSL shader, src/gpu.rs:95-133)
//   linear attention - causal per-token rank-1 state recurrence and the non-causal two-product form
//                      (src/linear_attention.rs:139-266)
//   selective scan   - h = exp(delta A) h + delta B u ; y = C . h   (src/tensor.rs:859-878)
//   layer norm       - last axis, biased variance, eps inside the square root (src/tensor.rs:1027-1046)
//   Adam             - m, v, p update with the bias correction folded into lr_t, 8 lanes at a time (src/optim.rs:121-168)
//   fused linear     - y = act(x W^T + b), one output per iteration (the FUSED_LINEAR shader, src/gpu.rs:69-91)
//   MLP step         - forward, softmax cross-entropy, backward and Adam of a ReLU MLP on the packed sgemm above: the
//                      reference's `Trainer::train_epoch` inner loop (src/train.rs:126-144) without its graph overheads
#include <immintrin.h>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" int b200_cpu_sgemm(int, int, int, int, int, float, const float*, int, const float*, int, float, float*, int, int);

extern "C" {

// q, k, v, out: [batch, seq, d] contiguous
int b200_cpu_flash_attention(const float* q, const float* k, const float* v, float* out, int batch, int seq, int d, float scale,
                             int causal) {
  std::vector<float> acc(d);
  for (int b = 0; b < batch; ++b) {
    const float* qb = q + (size_t)b * seq * d; const float* kb = k + (size_t)b * seq * d; const float* vb = v + (size_t)b * seq * d;
    for (int i = 0; i < seq; ++i) {
      float m = -INFINITY, l = 0.f;
      std::fill(acc.begin(), acc.end(), 0.f);
      const int last = causal ? i : seq - 1;
      for (int j = 0; j <= last; ++j) {
        float s = 0.f;
        for (int c = 0; c < d; ++c) s += qb[(size_t)i * d + c] * kb[(size_t)j * d + c];
        s *= scale;
        const float mn = std::max(m, s), corr = std::exp(m - mn), p = std::exp(s - mn);
        l = l * corr + p;
        for (int c = 0; c < d; ++c) acc[c] = acc[c] * corr + p * vb[(size_t)j * d + c];
        m = mn;
      }
      for (int c = 0; c < d; ++c) out[((size_t)b * seq + i) * d + c] = acc[c] / l;
    }
  }
  return 0;
}

static inline float phi(float x, int kind) { return kind == 0 ? (x > 0.f ? x + 1.f : std::exp(x)) : (x > 0.f ? x * x : 0.f); }

// q, k, v, out: [batch, seq, d]; kind 0 = ELU + 1, 1 = ReLU^2
int b200_cpu_linear_attention(const float* q, const float* k, const float* v, float* out, int batch, int seq, int d, float scale,
                              float eps, int causal, int kind) {
  std::vector<float> S((size_t)d * d), z(d), pq(d), pk(d);
  for (int b = 0; b < batch; ++b) {
    const size_t base = (size_t)b * seq * d;
    std::fill(S.begin(), S.end(), 0.f); std::fill(z.begin(), z.end(), 0.f);
    if (!causal) {
      for (int t = 0; t < seq; ++t) {
        for (int c = 0; c < d; ++c) pk[c] = phi(k[base + (size_t)t * d + c] * scale, kind);
        for (int a = 0; a < d; ++a) { z[a] += pk[a]; for (int c = 0; c < d; ++c) S[(size_t)a * d + c] += pk[a] * v[base + (size_t)t * d + c]; }
      }
    }
    for (int t = 0; t < seq; ++t) {
      if (causal) {
        for (int c = 0; c < d; ++c) pk[c] = phi(k[base + (size_t)t * d + c] * scale, kind);
        for (int a = 0; a < d; ++a) { z[a] += pk[a]; for (int c = 0; c < d; ++c) S[(size_t)a * d + c] += pk[a] * v[base + (size_t)t * d + c]; }
      }
      float den = eps;
      for (int a = 0; a < d; ++a) { pq[a] = phi(q[base + (size_t)t * d + a] * scale, kind); den += pq[a] * z[a]; }
      for (int c = 0; c < d; ++c) {
        float num = 0.f;
        for (int a = 0; a < d; ++a) num += pq[a] * S[(size_t)a * d + c];
        out[base + (size_t)t * d + c] = num / den;
      }
    }
  }
  return 0;
}

// u, delta, y: [B, S, D]; Bm, Cm: [B, S, N]; A: [D, N]
int b200_cpu_selective_scan(const float* u, const float* delta, const float* A, const float* Bm, const float* Cm, float* y,
                            int B, int S, int D, int N) {
  std::vector<float> h((size_t)D * N);
  for (int b = 0; b < B; ++b) {
    std::fill(h.begin(), h.end(), 0.f);
    for (int t = 0; t < S; ++t) {
      const size_t row = (size_t)b * S + t;
      for (int c = 0; c < D; ++c) {
        const float dt = delta[row * D + c], x = u[row * D + c];
        float acc = 0.f;
        for (int n = 0; n < N; ++n) {
          float& hv = h[(size_t)c * N + n];
          hv = std::exp(dt * A[(size_t)c * N + n]) * hv + dt * Bm[row * N + n] * x;
          acc += hv * Cm[row * N + n];
        }
        y[row * D + c] = acc;
      }
    }
  }
  return 0;
}

int b200_cpu_layernorm(const float* x, const float* gamma, const float* beta, float* y, long long rows, int d, float eps) {
  for (long long r = 0; r < rows; ++r) {
    const float* xr = x + r * d;
    float mean = 0.f, var = 0.f;
    for (int c = 0; c < d; ++c) mean += xr[c];
    mean /= d;
    for (int c = 0; c < d; ++c) var += (xr[c] - mean) * (xr[c] - mean);
    const float rstd = 1.f / std::sqrt(var / d + eps);
    for (int c = 0; c < d; ++c) y[r * d + c] = (xr[c] - mean) * rstd * gamma[c] + beta[c];
  }
  return 0;
}

// reference form: lr_t carries the bias correction; p -= lr_t * m / (sqrt(v) + eps)
int b200_cpu_adam(float* p, const float* g, float* m, float* v, long long n, float b1, float b2, float eps, float lr_t) {
  const __m256 vb1 = _mm256_set1_ps(b1), vb2 = _mm256_set1_ps(b2), o1 = _mm256_set1_ps(1.f - b1), o2 = _mm256_set1_ps(1.f - b2);
  const __m256 ve = _mm256_set1_ps(eps), vl = _mm256_set1_ps(lr_t);
  long long i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m256 gg = _mm256_loadu_ps(g + i);
    const __m256 mm = _mm256_fmadd_ps(vb1, _mm256_loadu_ps(m + i), _mm256_mul_ps(o1, gg));
    const __m256 vv = _mm256_fmadd_ps(vb2, _mm256_loadu_ps(v + i), _mm256_mul_ps(o2, _mm256_mul_ps(gg, gg)));
    _mm256_storeu_ps(m + i, mm); _mm256_storeu_ps(v + i, vv);
    const __m256 upd = _mm256_div_ps(_mm256_mul_ps(vl, mm), _mm256_add_ps(_mm256_sqrt_ps(vv), ve));
    _mm256_storeu_ps(p + i, _mm256_sub_ps(_mm256_loadu_ps(p + i), upd));
  }
  for (; i < n; ++i) {
    m[i] = b1 * m[i] + (1.f - b1) * g[i];
    v[i] = b2 * v[i] + (1.f - b2) * g[i] * g[i];
    p[i] -= lr_t * m[i] / (std::sqrt(v[i]) + eps);
  }
  return 0;
}

// y[batch, out] = act(x[batch, in] W[out, in]^T + b); act 0 none, 1 ReLU
int b200_cpu_fused_linear(const float* x, const float* W, const float* b, float* y, int batch, int in, int out, int act) {
  for (int r = 0; r < batch; ++r)
    for (int o = 0; o < out; ++o) {
      float s = b ? b[o] : 0.f;
      for (int c = 0; c < in; ++c) s += x[(size_t)r * in + c] * W[(size_t)o * in + c];
      y[(size_t)r * out + o] = act == 1 ? std::max(s, 0.f) : s;
    }
  return 0;
}

// One training step of a ReLU MLP with softmax cross-entropy (integer labels) or mean squared error (targets), Adam.
// dims[0..L]; W[l]: [dims[l+1], dims[l]], b[l]: [dims[l+1]]; m*, v*: Adam state of the same shapes; `step` = steps taken so far.
// loss_kind 0: cross-entropy with `labels`; 1: mean squared error against `targets` [batch, dims[L]].
// Returns the loss through *loss_out.
int b200_cpu_mlp_step(int L, const int* dims, float** W, float** b, float** mW, float** vW, float** mb, float** vb,
                      const float* x, const int* labels, const float* targets, int batch, int loss_kind, float lr, int step,
                      int threads, float* loss_out) {
  std::vector<std::vector<float>> act(L + 1), grad(L + 1);
  act[0].assign(x, x + (size_t)batch * dims[0]);
  for (int l = 0; l < L; ++l) {
    const int in = dims[l], out = dims[l + 1];
    act[l + 1].resize((size_t)batch * out);
    for (int r = 0; r < batch; ++r) std::memcpy(&act[l + 1][(size_t)r * out], b[l], sizeof(float) * out);
    b200_cpu_sgemm(0, 1, batch, out, in, 1.f, act[l].data(), in, W[l], in, 1.f, act[l + 1].data(), out, threads);
    if (l + 1 < L) for (auto& t : act[l + 1]) t = std::max(t, 0.f);
  }
  const int C = dims[L];
  std::vector<float>& logits = act[L];
  grad[L].resize((size_t)batch * C);
  double loss = 0.0;
  if (loss_kind == 0) {
    for (int r = 0; r < batch; ++r) {
      float* z = &logits[(size_t)r * C];
      float mx = z[0];
      for (int c = 1; c < C; ++c) mx = std::max(mx, z[c]);
      float sum = 0.f;
      for (int c = 0; c < C; ++c) sum += std::exp(z[c] - mx);
      loss += -(z[labels[r]] - mx - std::log(sum));
      for (int c = 0; c < C; ++c) grad[L][(size_t)r * C + c] = (std::exp(z[c] - mx) / sum - (c == labels[r] ? 1.f : 0.f)) / batch;
    }
    loss /= batch;
  } else {
    const size_t n = (size_t)batch * C;
    for (size_t i = 0; i < n; ++i) { const float e = logits[i] - targets[i]; loss += (double)e * e; grad[L][i] = 2.f * e / n; }
    loss /= n;
  }
  const float t = (float)(step + 1), b1 = 0.9f, b2 = 0.999f;
  const float lr_t = lr * std::sqrt(1.f - std::pow(b2, t)) / (1.f - std::pow(b1, t));
  for (int l = L - 1; l >= 0; --l) {
    const int in = dims[l], out = dims[l + 1];
    std::vector<float> dW((size_t)out * in), db(out, 0.f);
    b200_cpu_sgemm(1, 0, out, in, batch, 1.f, grad[l + 1].data(), out, act[l].data(), in, 0.f, dW.data(), in, threads);   // dY^T X
    for (int r = 0; r < batch; ++r) for (int o = 0; o < out; ++o) db[o] += grad[l + 1][(size_t)r * out + o];
    if (l > 0) {
      grad[l].resize((size_t)batch * in);
      b200_cpu_sgemm(0, 0, batch, in, out, 1.f, grad[l + 1].data(), out, W[l], in, 0.f, grad[l].data(), in, threads);     // dY W
      for (size_t i = 0; i < grad[l].size(); ++i) if (act[l][i] <= 0.f) grad[l][i] = 0.f;
    }
    b200_cpu_adam(W[l], dW.data(), mW[l], vW[l], (long long)out * in, b1, b2, 1e-8f, lr_t);
    b200_cpu_adam(b[l], db.data(), mb[l], vb[l], out, b1, b2, 1e-8f, lr_t);
  }
  *loss_out = (float)loss;
  return 0;
}

}  // extern "C"
