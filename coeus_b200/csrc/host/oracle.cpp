// CPU oracle: the reference's forward pass restated loop for loop in fp32 (same summation order,
// Welford layer norm, tanh GELU, powf positional table, sin init;
// plugins/model-transformer/src/lib.rs:44-129, :167-300, :328-378, :398-414, :604-611, :791-919).
// It is the correctness oracle for the GPU path and the timed CPU baseline.  `ref_compat` selects
// the reference's layer norm over the whole [S*H] buffer; without it the norm is per token.
#include "oracle.hpp"

#include <cmath>
#include <cstring>
#include <stdexcept>

namespace coeus {

static std::vector<float> matmul(const float* a, const float* b, size_t m, size_t n, size_t k) {
  std::vector<float> c(m * n, 0.0f);
  const size_t BS = 64;
  for (size_t ii = 0; ii < m; ii += BS)
    for (size_t jj = 0; jj < n; jj += BS)
      for (size_t kk = 0; kk < k; kk += BS) {
        const size_t ie = std::min(ii + BS, m), je = std::min(jj + BS, n), ke = std::min(kk + BS, k);
        for (size_t i = ii; i < ie; ++i)
          for (size_t j = jj; j < je; ++j) {
            float sum = c[i * n + j];
            for (size_t l = kk; l < ke; ++l) sum += a[i * k + l] * b[l * n + j];
            c[i * n + j] = sum;
          }
      }
  return c;
}

static void layer_norm_span(const float* in, float* out, size_t n, const float* scale,
                            const float* bias, size_t h, float eps, size_t phase) {
  float mean = 0.0f, m2 = 0.0f;
  for (size_t i = 0; i < n; ++i) {
    const float x = in[i];
    const float delta = x - mean;
    mean += delta / static_cast<float>(i + 1);
    m2 += delta * (x - mean);
  }
  const float sd = std::sqrt(m2 / static_cast<float>(n) + eps);
  for (size_t i = 0; i < n; ++i)
    out[i] = scale[(i + phase) % h] * (in[i] - mean) / sd + bias[(i + phase) % h];
}

static std::vector<float> layer_norm(const std::vector<float>& x, const float* scale,
                                     const float* bias, size_t S, size_t H, float eps,
                                     bool ref_compat) {
  std::vector<float> out(x.size());
  if (ref_compat) {
    layer_norm_span(x.data(), out.data(), S * H, scale, bias, H, eps, 0);
  } else {
    for (size_t t = 0; t < S; ++t)
      layer_norm_span(x.data() + t * H, out.data() + t * H, H, scale, bias, H, eps, 0);
  }
  return out;
}

static inline float gelu(float x) {
  return 0.5f * x * (1.0f + std::tanh(0.7978845608028654f * x * (1.0f + 0.044715f * x * x)));
}

size_t oracle_param_count(const OracleConfig& c) {
  const size_t H = c.hidden, I = c.intermediate, V = c.vocab;
  size_t per = 2 * H + 4 * H * H + 2 * H + 2 * H * I;
  if (c.use_bias) per += 4 * H + I + H;
  return V * H + per * c.layers + 2 * H + H * V;
}

void oracle_sin_init(float* p, size_t n, size_t hidden) {
  const float scale = std::sqrt(2.0f / static_cast<float>(hidden));
  for (size_t i = 0; i < n; ++i) {
    float v = std::sin(static_cast<float>(i) * 0.1234567f) * scale;
    p[i] = v < -0.1f ? -0.1f : (v > 0.1f ? 0.1f : v);
  }
}

std::vector<float> oracle_forward(const float* params, size_t n_params, const OracleConfig& c,
                                  const int64_t* ids, size_t S, bool ref_compat, bool all_positions) {
  const size_t H = c.hidden, I = c.intermediate, V = c.vocab, nh = c.heads, dh = H / nh;
  if (S == 0 || S > c.max_seq) throw std::invalid_argument("Sequence length out of range");
  if (n_params < oracle_param_count(c)) throw std::invalid_argument("parameter buffer too short");
  size_t off = 0;
  const float* embed = params;
  off += V * H;
  std::vector<float> x(S * H);
  for (size_t t = 0; t < S; ++t) {
    if (ids[t] < 0 || static_cast<size_t>(ids[t]) >= V) throw std::invalid_argument("Token ID out of range");
    std::memcpy(&x[t * H], embed + static_cast<size_t>(ids[t]) * H, H * sizeof(float));
  }
  for (size_t pos = 0; pos < S; ++pos)
    for (size_t i = 0; i < H / 2; ++i) {
      const float angle = static_cast<float>(pos) /
                          std::pow(10000.0f, 2.0f * static_cast<float>(i) / static_cast<float>(H));
      x[pos * H + 2 * i] += std::sin(angle);
      x[pos * H + 2 * i + 1] += std::cos(angle);
    }
  const float scale = 1.0f / std::sqrt(static_cast<float>(dh));
  for (size_t l = 0; l < c.layers; ++l) {
    const float* ln1s = params + off; off += H;
    const float* ln1b = params + off; off += H;
    const float* wq = params + off; const float* wk = wq + H * H; const float* wv = wk + H * H;
    const float* wo = wv + H * H; off += 4 * H * H;
    const float *bq = nullptr, *bk = nullptr, *bv = nullptr, *bo = nullptr;
    if (c.use_bias) { bq = params + off; bk = bq + H; bv = bk + H; bo = bv + H; off += 4 * H; }
    const float* ln2s = params + off; off += H;
    const float* ln2b = params + off; off += H;
    const float* wup = params + off; const float* wdown = wup + H * I; off += 2 * H * I;
    const float *bup = nullptr, *bdown = nullptr;
    if (c.use_bias) { bup = params + off; bdown = bup + I; off += I + H; }

    std::vector<float> n1 = layer_norm(x, ln1s, ln1b, S, H, c.eps, ref_compat);
    std::vector<float> q = matmul(n1.data(), wq, S, H, H), k = matmul(n1.data(), wk, S, H, H),
                       v = matmul(n1.data(), wv, S, H, H);
    if (c.use_bias)
      for (size_t i = 0; i < S * H; ++i) { q[i] += bq[i % H]; k[i] += bk[i % H]; v[i] += bv[i % H]; }
    std::vector<float> attn(S * H, 0.0f), scores(S * S), probs(S);
    for (size_t h = 0; h < nh; ++h) {
      for (size_t i = 0; i < S; ++i)
        for (size_t j = 0; j < S; ++j) {
          float s = 0.0f;
          for (size_t d = 0; d < dh; ++d) s += q[i * H + h * dh + d] * k[j * H + h * dh + d];
          scores[i * S + j] = j <= i ? s * scale : -INFINITY;
        }
      for (size_t i = 0; i < S; ++i) {
        float mx = -INFINITY;
        for (size_t j = 0; j < S; ++j) mx = std::max(mx, scores[i * S + j]);
        float sum = 0.0f;
        for (size_t j = 0; j < S; ++j) sum += std::exp(scores[i * S + j] - mx);
        for (size_t j = 0; j < S; ++j) probs[j] = std::exp(scores[i * S + j] - mx) / sum;
        for (size_t d = 0; d < dh; ++d) {
          float s = 0.0f;
          for (size_t j = 0; j < S; ++j) s += probs[j] * v[j * H + h * dh + d];
          attn[i * H + h * dh + d] = s;
        }
      }
    }
    std::vector<float> o = matmul(attn.data(), wo, S, H, H);
    for (size_t i = 0; i < S * H; ++i) x[i] += o[i] + (c.use_bias ? bo[i % H] : 0.0f);
    std::vector<float> n2 = layer_norm(x, ln2s, ln2b, S, H, c.eps, ref_compat);
    std::vector<float> u = matmul(n2.data(), wup, S, I, H);
    for (size_t i = 0; i < S * I; ++i) u[i] = gelu(u[i] + (c.use_bias ? bup[i % I] : 0.0f));
    std::vector<float> f = matmul(u.data(), wdown, S, H, I);
    for (size_t i = 0; i < S * H; ++i) x[i] += f[i] + (c.use_bias ? bdown[i % H] : 0.0f);
  }
  const float* lnfs = params + off; off += H;
  const float* lnfb = params + off; off += H;
  const float* wout = params + off;
  std::vector<float> y = layer_norm(x, lnfs, lnfb, S, H, c.eps, ref_compat);
  if (all_positions) return matmul(y.data(), wout, S, V, H);
  return matmul(y.data() + (S - 1) * H, wout, 1, V, H);
}

}  // namespace coeus
