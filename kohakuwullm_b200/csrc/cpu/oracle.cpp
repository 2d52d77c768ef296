// CPU oracles (plain C++17, fp32 storage, fp64 accumulation where a sum is long) for the device kernels.
//
// Every function restates one kernel family's arithmetic without tiling, vector types or intrinsics, so
// that a CUDA kernel and its PyTorch reference can both be checked against a third, independent
// statement of the same rule. Built as `_kwu_cpu.so` (g++), bound with ctypes
// (kohakuwullm_b200/ops/cpu_oracle.py). Rules and their reference sources:
//   rmsnorm / swiglu      src/kohakuwullm/kernels/elementwise/rmsnorm.py:20-128, swiglu.py:49-119
//   rope (rotate-half)    src/kohakuwullm/kernels/attention/rope.py:27-89
//   varlen attention      src/kohakuwullm/kernels/attention/flash_attn_fwd.py:35-154
//   mxfp8 quantise        src/kohakuwullm/kernels/mxfp8/quantize.py:39-56
//   linear CE + lse       src/kohakuwullm/kernels/loss/chunked_ce.py:94-293
//   router top-k          src/kohakuwullm/kernels/moe/router.py:76-194
//   routed experts        src/kohakuwullm/models/components/moe.py:490-518 (dense_fallback)
//   adamw / adamw16 / SR  src/kohakuwullm/kernels/optim/adamw16.py:16-106, stochastic_round.py:44-134
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#define KWO_API extern "C" __attribute__((visibility("default")))

namespace {

inline float bf16_round(float x) {  // round-to-nearest-even to bfloat16 precision, returned as float
  uint32_t u;
  std::memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;
  const uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  u &= 0xffff0000u;
  float y;
  std::memcpy(&y, &u, 4);
  return y;
}

// float -> e4m3 (fn variant: no inf, max 448, NaN = 0x7f), round-to-nearest-even, saturating.
inline uint8_t e4m3_from_float(float x) {
  if (std::isnan(x)) return 0x7f;
  const uint8_t sign = std::signbit(x) ? 0x80 : 0;
  float a = std::fabs(x);
  if (a >= 448.f) return sign | 0x7e;
  if (a < std::ldexp(1.f, -10)) return sign;  // below half of the smallest subnormal (2^-9): rounds to 0
  int e;
  std::frexp(a, &e);  // a = f * 2^e, f in [0.5, 1)
  int exp = e - 1;    // a = 1.xxx * 2^exp
  if (exp < -6) exp = -6;  // subnormal range shares the exponent of 2^-6
  const float step = std::ldexp(1.f, exp - 3);  // 3 mantissa bits
  float qf = a / step;
  float r = std::nearbyint(qf);  // default rounding mode: to nearest, ties to even
  float v = r * step;
  if (v >= 448.f) return sign | 0x7e;
  // re-derive the fields from the rounded value
  if (v < std::ldexp(1.f, -6)) {
    const int m = static_cast<int>(std::lround(v / std::ldexp(1.f, -9)));
    return sign | static_cast<uint8_t>(m);
  }
  std::frexp(v, &e);
  exp = e - 1;
  const int m = static_cast<int>(std::lround((v / std::ldexp(1.f, exp) - 1.f) * 8.f));
  return sign | static_cast<uint8_t>(((exp + 7) << 3) | m);
}

inline float e4m3_to_float(uint8_t b) {
  const int sign = b >> 7, e = (b >> 3) & 0xf, m = b & 7;
  if (e == 0xf && m == 7) return std::numeric_limits<float>::quiet_NaN();
  const float v = (e == 0) ? std::ldexp(static_cast<float>(m), -9) : std::ldexp(1.f + m / 8.f, e - 7);
  return sign ? -v : v;
}

// Philox4x32-10 (counter = (offset, 0, 0, 0), key = (seed_lo, seed_hi)).
inline void philox4x32(uint64_t seed, uint64_t offset, uint32_t out[4]) {
  uint32_t c[4] = {static_cast<uint32_t>(offset), static_cast<uint32_t>(offset >> 32), 0u, 0u};
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  for (int round = 0; round < 10; ++round) {
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c[0];
    const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c[2];
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k0;
    const uint32_t n1 = static_cast<uint32_t>(p1);
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k1;
    const uint32_t n3 = static_cast<uint32_t>(p0);
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  for (int i = 0; i < 4; ++i) out[i] = c[i];
}

inline float score_fn(float logit, int kind) {
  if (kind == 0) return 1.f / (1.f + std::exp(-logit));
  return std::sqrt(logit > 20.f ? logit : std::log1p(std::exp(logit)));  // kind 2: sqrt-softplus
}

}  // namespace

// ---------------------------------------------------------------------------------- norm / activation
KWO_API void kwo_rmsnorm_fwd(const float* x, const float* w, float* out, float* rstd, int rows, int cols, float eps,
                             int one_plus) {
  for (int r = 0; r < rows; ++r) {
    double ss = 0;
    for (int c = 0; c < cols; ++c) ss += static_cast<double>(x[r * (size_t)cols + c]) * x[r * (size_t)cols + c];
    const float rs = 1.f / std::sqrt(static_cast<float>(ss / cols) + eps);
    if (rstd) rstd[r] = rs;
    for (int c = 0; c < cols; ++c) {
      const float g = w ? (one_plus ? 1.f + w[c] : w[c]) : 1.f;
      out[r * (size_t)cols + c] = x[r * (size_t)cols + c] * rs * g;
    }
  }
}

KWO_API void kwo_rmsnorm_bwd(const float* x, const float* w, const float* dy, float* dx, float* dw, int rows, int cols,
                             float eps, int one_plus) {
  std::vector<double> dwacc(cols, 0.0);
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + r * (size_t)cols;
    const float* gr = dy + r * (size_t)cols;
    double ss = 0, dot = 0;
    for (int c = 0; c < cols; ++c) ss += static_cast<double>(xr[c]) * xr[c];
    const double rs = 1.0 / std::sqrt(ss / cols + eps);
    for (int c = 0; c < cols; ++c) {
      const double g = w ? (one_plus ? 1.0 + w[c] : w[c]) : 1.0;
      dot += gr[c] * g * xr[c];
      dwacc[c] += gr[c] * xr[c] * rs;
    }
    for (int c = 0; c < cols; ++c) {
      const double g = w ? (one_plus ? 1.0 + w[c] : w[c]) : 1.0;
      dx[r * (size_t)cols + c] = static_cast<float>(rs * (gr[c] * g - xr[c] * rs * rs * dot / cols));
    }
  }
  if (dw)
    for (int c = 0; c < cols; ++c) dw[c] = static_cast<float>(dwacc[c]);
}

// h (rows, 2H) = [gate | value] -> out (rows, H) = silu(gate) * value
KWO_API void kwo_swiglu_fwd(const float* h, float* out, int rows, int H) {
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < H; ++c) {
      const float g = h[r * (size_t)(2 * H) + c], v = h[r * (size_t)(2 * H) + H + c];
      out[r * (size_t)H + c] = g / (1.f + std::exp(-g)) * v;
    }
}

KWO_API void kwo_swiglu_bwd(const float* h, const float* dout, float* dh, int rows, int H) {
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < H; ++c) {
      const float g = h[r * (size_t)(2 * H) + c], v = h[r * (size_t)(2 * H) + H + c];
      const float s = 1.f / (1.f + std::exp(-g));
      const float d = dout[r * (size_t)H + c];
      dh[r * (size_t)(2 * H) + c] = d * v * s * (1.f + g * (1.f - s));
      dh[r * (size_t)(2 * H) + H + c] = d * g * s;
    }
}

// x (T, H, D); cos/sin (T, rot_half): rotate-half on the first 2*rot_half channels. sign = -1: inverse.
KWO_API void kwo_rope(const float* x, const float* cos_t, const float* sin_t, float* out, int T, int H, int D,
                      int rot_half, float sign) {
  for (int t = 0; t < T; ++t)
    for (int h = 0; h < H; ++h) {
      const float* xi = x + (t * (size_t)H + h) * D;
      float* oi = out + (t * (size_t)H + h) * D;
      for (int d = 0; d < D; ++d) oi[d] = xi[d];
      for (int j = 0; j < rot_half; ++j) {
        const float c = cos_t[t * (size_t)rot_half + j], s = sign * sin_t[t * (size_t)rot_half + j];
        const float a = xi[j], b = xi[j + rot_half];
        oi[j] = a * c - b * s;
        oi[j + rot_half] = b * c + a * s;
      }
    }
}

// ---------------------------------------------------------------------------------- attention
// q (T,Hq,D), k/v (T,Hkv,D) packed documents cu[0..n_docs]; causal, optional inclusive window, optional
// per-head sink log-sum-exp joining the denominator. out (T,Hq,D), lse (Hq,T) natural log incl. sink.
KWO_API void kwo_attention_varlen(const float* q, const float* k, const float* v, const int* cu, int n_docs, int T,
                                  int Hq, int Hkv, int D, int window, const float* sink_lse, float scale, float* out,
                                  float* lse) {
  const int group = Hq / Hkv;
  std::vector<double> s;
  for (int doc = 0; doc < n_docs; ++doc) {
    const int a = cu[doc], b = cu[doc + 1];
    for (int i = a; i < b; ++i)
      for (int h = 0; h < Hq; ++h) {
        const int hk = h / group;
        const int lo = (window > 0) ? std::max(a, i - window + 1) : a;
        s.assign(i - lo + 1, 0.0);
        double m = -std::numeric_limits<double>::infinity();
        for (int j = lo; j <= i; ++j) {
          double dot = 0;
          for (int d = 0; d < D; ++d) dot += static_cast<double>(q[(i * (size_t)Hq + h) * D + d]) * k[(j * (size_t)Hkv + hk) * D + d];
          s[j - lo] = dot * scale;
          m = std::max(m, s[j - lo]);
        }
        if (sink_lse) m = std::max(m, static_cast<double>(sink_lse[h]));
        double l = 0;
        for (int j = lo; j <= i; ++j) l += std::exp(s[j - lo] - m);
        if (sink_lse) l += std::exp(sink_lse[h] - m);
        for (int d = 0; d < D; ++d) {
          double acc = 0;
          for (int j = lo; j <= i; ++j) acc += std::exp(s[j - lo] - m) * v[(j * (size_t)Hkv + hk) * D + d];
          out[(i * (size_t)Hq + h) * D + d] = static_cast<float>(acc / l);
        }
        if (lse) lse[h * (size_t)T + i] = static_cast<float>(m + std::log(l));
      }
  }
}

// ---------------------------------------------------------------------------------- MXFP8
// x (M,K) -> q bytes (M,K) e4m3, exp bytes (M,K/32) UE8M0 (natural layout), optional dequantised copy.
KWO_API void kwo_mxfp8_quantize(const float* x, uint8_t* q, uint8_t* e8, float* deq, int M, int K) {
  for (int r = 0; r < M; ++r)
    for (int kb = 0; kb < K / 32; ++kb) {
      const float* blk = x + r * (size_t)K + kb * 32;
      float amax = 0.f;
      for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(blk[i]));
      amax = std::max(amax, 1e-30f);
      int e = static_cast<int>(std::ceil(std::log2(static_cast<double>(amax) / 448.0)));
      // exact ceil(log2): correct a possible off-by-one of log2 near powers of two
      while (std::ldexp(1.0, e) < static_cast<double>(amax) / 448.0) ++e;
      while (e > -127 && std::ldexp(1.0, e - 1) >= static_cast<double>(amax) / 448.0) --e;
      e = std::max(e, -127);
      e = std::min(e, 127);
      e8[r * (size_t)(K / 32) + kb] = static_cast<uint8_t>(e + 127);
      const float inv = std::ldexp(1.f, -e);
      for (int i = 0; i < 32; ++i) {
        const uint8_t b = e4m3_from_float(blk[i] * inv);
        q[r * (size_t)K + kb * 32 + i] = b;
        if (deq) deq[r * (size_t)K + kb * 32 + i] = e4m3_to_float(b) * std::ldexp(1.f, e);
      }
    }
}

// ---------------------------------------------------------------------------------- loss head
// x (T,D), W (V,D), labels (T) with ignore -100. ce[t] = lse - logit[label] (0 when ignored), lse[t].
KWO_API void kwo_linear_ce(const float* x, const float* W, const long long* labels, float* ce, float* lse, int T, int D,
                           int V) {
  std::vector<double> logit(V);
  for (int t = 0; t < T; ++t) {
    double m = -std::numeric_limits<double>::infinity();
    for (int c = 0; c < V; ++c) {
      double dot = 0;
      for (int d = 0; d < D; ++d) dot += static_cast<double>(x[t * (size_t)D + d]) * W[c * (size_t)D + d];
      logit[c] = dot;
      m = std::max(m, dot);
    }
    double l = 0;
    for (int c = 0; c < V; ++c) l += std::exp(logit[c] - m);
    const double z = m + std::log(l);
    lse[t] = static_cast<float>(z);
    ce[t] = (labels[t] >= 0 && labels[t] < V) ? static_cast<float>(z - logit[labels[t]]) : 0.f;
  }
}

// ---------------------------------------------------------------------------------- MoE
// x (T,D), Wg (E,D), bias (E) or null. Selection over score + bias, weight from the unbiased score,
// ties to the lower expert index. idx (T,k) int32, weight (T,k), counts (E).
KWO_API void kwo_router_topk(const float* x, const float* Wg, const float* bias, int* idx, float* weight, int* counts,
                             int T, int D, int E, int k, int score_kind, int norm_topk, float scaling) {
  std::vector<float> sc(E), sel(E);
  for (int e = 0; e < E; ++e) counts[e] = 0;
  for (int t = 0; t < T; ++t) {
    std::vector<double> lg(E);
    double mx = -std::numeric_limits<double>::infinity();
    for (int e = 0; e < E; ++e) {
      double dot = 0;
      for (int d = 0; d < D; ++d) dot += static_cast<double>(x[t * (size_t)D + d]) * Wg[e * (size_t)D + d];
      lg[e] = dot;
      mx = std::max(mx, dot);
    }
    if (score_kind == 1) {
      double sum = 0;
      for (int e = 0; e < E; ++e) sum += std::exp(lg[e] - mx);
      for (int e = 0; e < E; ++e) sc[e] = static_cast<float>(std::exp(lg[e] - mx) / sum);
    } else {
      for (int e = 0; e < E; ++e) sc[e] = score_fn(static_cast<float>(lg[e]), score_kind);
    }
    for (int e = 0; e < E; ++e) sel[e] = sc[e] + (bias ? bias[e] : 0.f);
    float wsum = 0.f;
    for (int j = 0; j < k; ++j) {
      int best = 0;
      for (int e = 1; e < E; ++e)
        if (sel[e] > sel[best]) best = e;
      idx[t * (size_t)k + j] = best;
      weight[t * (size_t)k + j] = sc[best];
      wsum += sc[best];
      sel[best] = -std::numeric_limits<float>::infinity();
      counts[best] += 1;
    }
    for (int j = 0; j < k; ++j) {
      float w = weight[t * (size_t)k + j];
      if (norm_topk) w = w / (wsum + 1e-20f);
      weight[t * (size_t)k + j] = w * scaling;
    }
  }
}

// y[t] = sum_j weight[t,j] * w_out[e] silu_glu(w_in[e] x[t]), e = idx[t,j]. w_in (E,2H,D), w_out (E,D,H).
KWO_API void kwo_routed_experts(const float* x, const int* idx, const float* weight, const float* w_in,
                                const float* w_out, float* y, int T, int D, int H, int E, int k) {
  std::vector<double> h(2 * H), a(H);
  for (int t = 0; t < T; ++t) {
    for (int d = 0; d < D; ++d) y[t * (size_t)D + d] = 0.f;
    for (int j = 0; j < k; ++j) {
      const int e = idx[t * (size_t)k + j];
      if (e < 0 || e >= E) continue;
      const float* wi = w_in + e * (size_t)(2 * H) * D;
      const float* wo = w_out + e * (size_t)D * H;
      for (int r = 0; r < 2 * H; ++r) {
        double dot = 0;
        for (int d = 0; d < D; ++d) dot += static_cast<double>(wi[r * (size_t)D + d]) * x[t * (size_t)D + d];
        h[r] = dot;
      }
      for (int c = 0; c < H; ++c) a[c] = h[c] / (1.0 + std::exp(-h[c])) * h[H + c];
      for (int d = 0; d < D; ++d) {
        double dot = 0;
        for (int c = 0; c < H; ++c) dot += static_cast<double>(wo[d * (size_t)H + c]) * a[c];
        y[t * (size_t)D + d] += static_cast<float>(weight[t * (size_t)k + j] * dot);
      }
    }
  }
}

// ---------------------------------------------------------------------------------- optimizers
// Decoupled-decay AdamW on fp32 buffers; g is multiplied by grad_scale first.
KWO_API void kwo_adamw(float* p, float* m, float* v, const float* g, long long n, float grad_scale, float lr,
                       float beta1, float beta2, float eps, float wd, int step) {
  const double bc1 = 1.0 - std::pow(static_cast<double>(beta1), step);
  const double bc2 = 1.0 - std::pow(static_cast<double>(beta2), step);
  for (long long i = 0; i < n; ++i) {
    const float ge = g[i] * grad_scale;
    m[i] = beta1 * m[i] + (1.f - beta1) * ge;
    v[i] = beta2 * v[i] + (1.f - beta2) * ge * ge;
    const double denom = std::sqrt(static_cast<double>(v[i]) / bc2) + eps;
    p[i] = static_cast<float>(p[i] * (1.0 - static_cast<double>(lr) * wd) - lr * (m[i] / bc1) / denom);
  }
}

// Stochastic rounding fp32 -> bf16 with 16 caller-supplied random bits per element: add the bits below the
// kept mantissa, truncate. Returns the rounded values as floats.
KWO_API void kwo_sr_round(const float* x, const uint32_t* bits16, float* out, long long n) {
  for (long long i = 0; i < n; ++i) {
    uint32_t u;
    std::memcpy(&u, &x[i], 4);
    if ((u & 0x7f800000u) != 0x7f800000u) u += (bits16[i] & 0xffffu);
    u &= 0xffff0000u;
    std::memcpy(&out[i], &u, 4);
  }
}

KWO_API void kwo_philox4x32(unsigned long long seed, unsigned long long offset, uint32_t* out4) {
  philox4x32(seed, offset, out4);
}

KWO_API float kwo_bf16_round(float x) { return bf16_round(x); }
KWO_API unsigned char kwo_e4m3_from_float(float x) { return e4m3_from_float(x); }
KWO_API float kwo_e4m3_to_float(unsigned char b) { return e4m3_to_float(b); }

// The 16 random bits the device kernels draw for flat element index i: Philox block i / 8, 32-bit word
// (i / 2) % 4, low half for even i and high half for odd i.
KWO_API unsigned int kwo_draw16(unsigned long long seed, unsigned long long i) {
  uint32_t r[4];
  philox4x32(seed, i >> 3, r);
  const uint32_t w = r[(i >> 1) & 3];
  return (i & 1) ? (w >> 16) : (w & 0xffffu);
}
