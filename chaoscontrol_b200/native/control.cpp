#include "control.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <limits>
#include <string>
#include <thread>

// The policy forward / backward are short dense loops over runtime sizes; compile them for AVX2+FMA and for
// AVX-512 as well as for the baseline ISA and let the loader pick by CPU (GNU function multi-versioning).
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__) && !defined(CCB_NO_CLONES)
#define CCB_HOT_CLONES __attribute__((target_clones("arch=x86-64-v4", "arch=x86-64-v3", "default")))
#else
#define CCB_HOT_CLONES
#endif

namespace ccb::ctrl {

// ---------------------------------------------------------------- credit ----
float recency_decay(float reward, uint64_t outcome_step, uint64_t action_step, float gamma) {
  if (outcome_step < action_step) return reward;
  const double lag = static_cast<double>(outcome_step - action_step);
  return static_cast<float>(static_cast<double>(reward) * std::pow(static_cast<double>(gamma), lag));
}

float gerber_weight(float then, float now, float threshold) {
  const float h = std::max(threshold, 0.f);
  const float tol = 1e-6f * std::max({1.f, std::fabs(then), std::fabs(now)});
  if (std::isfinite(then) && std::isfinite(now) && std::fabs(then - now) <= tol) return 1.f;
  if (std::fabs(then) <= h || std::fabs(now) <= h) return 0.f;
  return ((then > 0.f) == (now > 0.f)) ? 1.f : 0.f;
}

RollingStddev::RollingStddev(float decay) : decay_(decay) {
  if (!(decay >= 0.f && decay < 1.f)) decay_ = 0.99;
}
void RollingStddev::update(float x) {
  const double a = 1.0 - decay_;
  ema_ = decay_ * ema_ + a * x;
  ema_sq_ = decay_ * ema_sq_ + a * static_cast<double>(x) * x;
  ++count_;
}
float RollingStddev::mean() const {
  if (count_ == 0) return 0.f;
  const double corr = 1.0 - std::pow(decay_, static_cast<double>(count_));
  return corr > 0.0 ? static_cast<float>(ema_ / corr) : 0.f;
}
float RollingStddev::stddev() const {
  if (count_ < 2) return 0.f;
  const double corr = 1.0 - std::pow(decay_, static_cast<double>(count_));
  if (corr <= 0.0) return 0.f;
  const double m = ema_ / corr, m2 = ema_sq_ / corr;
  return static_cast<float>(std::sqrt(std::max(m2 - m * m, 0.0)));
}

FastSlowEma::FastSlowEma(float alpha, uint64_t interval)
    : alpha_(std::min(std::max(alpha, 0.f), 1.f)), interval_(interval == 0 ? 1 : interval) {}
void FastSlowEma::blend(float* slow, const float* fast, std::size_t n) const {
  const float keep = 1.f - alpha_;
  for (std::size_t i = 0; i < n; ++i) slow[i] = keep * slow[i] + alpha_ * fast[i];
}
void FastSlowEma::set_alpha(float a) { alpha_ = std::min(std::max(a, 0.f), 1.f); }

// -------------------------------------------------------- simplex policy ----
namespace {
// single precision throughout: the double erf / exp of the first version were two thirds of a policy forward
constexpr float kInvSqrt2 = 0.70710678118654752440f;
constexpr float kInvSqrt2Pi = 0.39894228040143267794f;
inline float gelu(float x) { return 0.5f * x * (1.f + std::erf(x * kInvSqrt2)); }
inline float gelu_grad(float x) {
  const float cdf = 0.5f * (1.f + std::erf(x * kInvSqrt2));
  const float pdf = kInvSqrt2Pi * std::exp(-0.5f * x * x);
  return cdf + x * pdf;
}
// Dot product with eight independent partial sums: a single running sum is one dependent FMA chain
// (4 cycles per element), which made the 16 x 16 x 32 attention scores the slowest part of a forward.
inline float dotf(const float* a, const float* b, std::size_t n) {
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  std::size_t i = 0;
  for (; i + 8 <= n; i += 8)
    for (int l = 0; l < 8; ++l) acc[l] += a[i + l] * b[i + l];
  float tail = 0.f;
  for (; i < n; ++i) tail += a[i] * b[i];
  return tail + ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7]));
}
void softmax_row(float* row, std::size_t n) {
  float mx = -std::numeric_limits<float>::infinity();
  for (std::size_t i = 0; i < n; ++i) mx = std::max(mx, row[i]);
  float sum = 0.f;
  for (std::size_t i = 0; i < n; ++i) { row[i] = std::exp(row[i] - mx); sum += row[i]; }
  const float inv = 1.f / sum;
  for (std::size_t i = 0; i < n; ++i) row[i] *= inv;
}
}  // namespace

void SimplexWeights::resize() {
  W_vp.assign(static_cast<std::size_t>(K_v) * H, 0.f);
  b_vp.assign(H, 0.f);
  W_lh.assign(H, 0.f);
  W_sb.assign(K_s, 0.f);
  const std::size_t hh = static_cast<std::size_t>(n_heads) * H * H;
  W_q.assign(hh, 0.f); W_k.assign(hh, 0.f); W_v.assign(hh, 0.f);
  W_o.assign(static_cast<std::size_t>(n_heads) * H, 0.f);
  W_e.assign(static_cast<std::size_t>(n_heads) * K_e, 0.f);
  bucket_embed.assign(static_cast<std::size_t>(n_buckets) * embed_dim, 0.f);
}
namespace {
inline void put(float*& o, const std::vector<float>& v) { std::memcpy(o, v.data(), v.size() * 4); o += v.size(); }
inline void get(const float*& i, std::vector<float>& v) { std::memcpy(v.data(), i, v.size() * 4); i += v.size(); }
}  // namespace
void SimplexWeights::to_flat(float* out) const {
  float* o = out;
  put(o, W_vp); put(o, b_vp); put(o, W_lh);
  *o++ = b_lh;
  put(o, W_sb);
  *o++ = alpha;
  if (n_heads) {
    *o++ = lambda_hxh;
    put(o, W_q); put(o, W_k); put(o, W_v); put(o, W_o); put(o, W_e);
  }
  put(o, bucket_embed);
}
void SimplexWeights::from_flat(const float* in) {
  const float* i = in;
  get(i, W_vp); get(i, b_vp); get(i, W_lh);
  b_lh = *i++;
  get(i, W_sb);
  alpha = *i++;
  if (n_heads) {
    lambda_hxh = *i++;
    get(i, W_q); get(i, W_k); get(i, W_v); get(i, W_o); get(i, W_e);
  }
  get(i, bucket_embed);
}
std::string SimplexWeights::validate() const {
  if (N == 0 || K_v == 0 || K_s == 0 || H == 0 || K_e == 0) return "simplex dims must be positive";
  if (!(temperature > 0.f)) return "temperature must be positive";
  if (W_vp.size() != static_cast<std::size_t>(K_v) * H) return "W_vp must have K_v*H elements";
  if (b_vp.size() != H) return "b_vp must have H elements";
  if (W_lh.size() != H) return "W_lh must have H elements";
  if (W_sb.size() != K_s) return "W_sb must have K_s elements";
  const std::size_t hh = static_cast<std::size_t>(n_heads) * H * H;
  if (n_heads == 0 && lambda_hxh != 0.f) return "n_heads must be positive when lambda_hxh != 0";
  if (W_q.size() != hh || W_k.size() != hh || W_v.size() != hh) return "W_q / W_k / W_v must have n_heads*H*H elements";
  if (W_o.size() != static_cast<std::size_t>(n_heads) * H) return "W_o must have n_heads*H elements";
  if (W_e.size() != static_cast<std::size_t>(n_heads) * K_e) return "W_e must have n_heads*K_e elements";
  if (bucket_embed.size() != static_cast<std::size_t>(n_buckets) * embed_dim)
    return "bucket_embed must have n_buckets*embed_dim elements";
  return "";
}

CCB_HOT_CLONES
SimplexForward simplex_forward(const SimplexWeights& w, const float* V, const float* E,
                               const float* feats) {
  const std::size_t N = w.N, H = w.H, Kv = w.K_v, Ke = w.K_e;
  SimplexForward f;
  f.pre.assign(N * H, 0.f);
  f.vertex_h.resize(N * H);
  f.attn.resize(N * N);
  f.mixed_h.resize(N * H);
  f.logits.resize(N);
  f.p.resize(N);
  for (std::size_t i = 0; i < N; ++i) {
    float* row = f.pre.data() + i * H;
    for (std::size_t h = 0; h < H; ++h) row[h] = w.b_vp[h];
    for (std::size_t k = 0; k < Kv; ++k) {
      const float v = V[i * Kv + k];
      const float* wr = w.W_vp.data() + k * H;
      for (std::size_t h = 0; h < H; ++h) row[h] += v * wr[h];
    }
    for (std::size_t h = 0; h < H; ++h) f.vertex_h[i * H + h] = gelu(row[h]);
  }
  const float scale = 1.f / std::sqrt(static_cast<float>(H));
  for (std::size_t i = 0; i < N; ++i) {
    float* arow = f.attn.data() + i * N;
    for (std::size_t j = 0; j < N; ++j) {
      const float dot = dotf(f.vertex_h.data() + i * H, f.vertex_h.data() + j * H, H);
      arow[j] = dot * scale + w.alpha * E[(i * N + j) * Ke];
    }
    softmax_row(arow, N);
  }
  for (std::size_t i = 0; i < N; ++i) {
    float* mrow = f.mixed_h.data() + i * H;
    for (std::size_t h = 0; h < H; ++h) mrow[h] = f.vertex_h[i * H + h];
    for (std::size_t j = 0; j < N; ++j) {
      const float a = f.attn[i * N + j];
      for (std::size_t h = 0; h < H; ++h) mrow[h] += a * f.vertex_h[j * H + h];
    }
    f.logits[i] = w.b_lh + dotf(mrow, w.W_lh.data(), H);
  }
  // residual branch: per head, attention over the vertices with learned projections
  const std::size_t nh = w.n_heads;
  f.logits_hxh.assign(N, 0.f);
  if (nh) {
    f.hq.assign(nh * N * H, 0.f); f.hk.assign(nh * N * H, 0.f); f.hv.assign(nh * N * H, 0.f);
    f.hmixed.assign(nh * N * H, 0.f);
    f.hattn.assign(nh * N * N, 0.f);
    const float inv_heads = 1.f / static_cast<float>(nh);
    for (std::size_t hd = 0; hd < nh; ++hd) {
      const float *Wq = w.W_q.data() + hd * H * H, *Wk = w.W_k.data() + hd * H * H, *Wv = w.W_v.data() + hd * H * H;
      float *q = f.hq.data() + hd * N * H, *k = f.hk.data() + hd * N * H, *v = f.hv.data() + hd * N * H;
      for (std::size_t i = 0; i < N; ++i)
        for (std::size_t a = 0; a < H; ++a) {
          const float x = f.vertex_h[i * H + a];
          const float *rq = Wq + a * H, *rk = Wk + a * H, *rv = Wv + a * H;
          for (std::size_t o = 0; o < H; ++o) {
            q[i * H + o] += x * rq[o];
            k[i * H + o] += x * rk[o];
            v[i * H + o] += x * rv[o];
          }
        }
      float* at = f.hattn.data() + hd * N * N;
      const float* We = w.W_e.data() + hd * Ke;
      for (std::size_t i = 0; i < N; ++i) {
        for (std::size_t j = 0; j < N; ++j) {
          float eb = 0.f;
          const float dot = dotf(q + i * H, k + j * H, H);
          for (std::size_t e = 0; e < Ke; ++e) eb += We[e] * E[(i * N + j) * Ke + e];
          at[i * N + j] = dot * scale + eb;
        }
        softmax_row(at + i * N, N);
      }
      float* mx = f.hmixed.data() + hd * N * H;
      const float* Wo = w.W_o.data() + hd * H;
      for (std::size_t i = 0; i < N; ++i) {
        for (std::size_t j = 0; j < N; ++j) {
          const float a = at[i * N + j];
          for (std::size_t o = 0; o < H; ++o) mx[i * H + o] += a * v[j * H + o];
        }
        f.logits_hxh[i] += dotf(mx + i * H, Wo, H) * inv_heads;
      }
    }
    for (std::size_t i = 0; i < N; ++i) f.logits[i] += w.lambda_hxh * f.logits_hxh[i];
  }
  float bias = 0.f;
  for (std::size_t k = 0; k < w.K_s; ++k) bias += w.W_sb[k] * feats[k];
  f.simplex_bias = bias;
  for (std::size_t i = 0; i < N; ++i) f.p[i] = (f.logits[i] + bias) / w.temperature;
  softmax_row(f.p.data(), N);
  return f;
}

void forward_pretrain_model(const PretrainModel& m, const float* x, std::size_t B, float* logits_out,
                            float* value_out) {
  const std::size_t F = m.F, Dg = m.Dg, L = m.L, Ds = m.Ds;
  std::vector<float> h(Dg), t(Dg);
  for (std::size_t b = 0; b < B; ++b) {
    const float* xr = x + b * F;
    for (std::size_t o = 0; o < Dg; ++o) {
      float acc = m.in_b[o];
      const float* wr = m.in_w + o * F;
      for (std::size_t k = 0; k < F; ++k) acc += xr[k] * wr[k];
      h[o] = acc;
    }
    for (std::size_t l = 0; l < L; ++l) {
      const float *dec = m.decay + l * Dg, *wi = m.w_in + l * Dg * Dg, *wo = m.w_out + l * Dg * Dg,
                  *bs = m.bias + l * Dg;
      for (std::size_t o = 0; o < Dg; ++o) t[o] = h[o] * dec[o] + bs[o];
      for (std::size_t k = 0; k < Dg; ++k) {                     // + h @ w_in (w_in is [in, out])
        const float hk = h[k];
        const float* wr = wi + k * Dg;
        for (std::size_t o = 0; o < Dg; ++o) t[o] += hk * wr[o];
      }
      for (std::size_t o = 0; o < Dg; ++o) t[o] = gelu(t[o]);
      std::fill(h.begin(), h.end(), 0.f);
      for (std::size_t k = 0; k < Dg; ++k) {                     // @ w_out
        const float tk = t[k];
        const float* wr = wo + k * Dg;
        for (std::size_t o = 0; o < Dg; ++o) h[o] += tk * wr[o];
      }
    }
    for (std::size_t s = 0; s < Ds; ++s) {
      float acc = m.pol_b[s];
      const float* wr = m.pol_w + s * Dg;
      for (std::size_t k = 0; k < Dg; ++k) acc += h[k] * wr[k];
      logits_out[b * Ds + s] = acc;
    }
    float v = m.val_b[0];
    for (std::size_t k = 0; k < Dg; ++k) v += h[k] * m.val_w[k];
    value_out[b] = v;
  }
}

CCB_HOT_CLONES
void simplex_backward(const SimplexWeights& w, const SimplexForward& f, const float* V, const float* E,
                      const float* feats, uint32_t chosen, float advantage, float entropy_beta,
                      float* grad) {
  const std::size_t N = w.N, H = w.H, Kv = w.K_v, Ks = w.K_s, Ke = w.K_e, nh = w.n_heads;
  float* gW_vp = grad;
  float* gb_vp = gW_vp + Kv * H;
  float* gW_lh = gb_vp + H;
  float* gb_lh = gW_lh + H;
  float* gW_sb = gb_lh + 1;
  float* galpha = gW_sb + Ks;
  // residual-branch block of the flat layout (present when n_heads > 0); the bucket embedding that
  // follows it takes no gradient (the forward does not read it)
  float* glambda = galpha + 1;
  float* gW_q = glambda + 1;
  float* gW_k = gW_q + nh * H * H;
  float* gW_v = gW_k + nh * H * H;
  float* gW_o = gW_v + nh * H * H;
  float* gW_e = gW_o + nh * H;

  // loss = -adv * log p[c] - beta * H(p);  z = (logits + bias) / T
  double ent = 0.0;
  for (std::size_t i = 0; i < N; ++i) if (f.p[i] > 0.f) ent -= f.p[i] * std::log(f.p[i]);
  std::vector<float> dlogit(N);
  float dbias = 0.f;
  for (std::size_t i = 0; i < N; ++i) {
    const float pi = f.p[i];
    float dz = -advantage * ((i == chosen ? 1.f : 0.f) - pi);
    if (entropy_beta != 0.f && pi > 0.f)
      dz += entropy_beta * pi * (std::log(pi) + static_cast<float>(ent));
    dlogit[i] = dz / w.temperature;
    dbias += dlogit[i];
  }
  for (std::size_t k = 0; k < Ks; ++k) gW_sb[k] += dbias * feats[k];
  std::vector<float> dmixed(N * H), dvh(N * H, 0.f);
  for (std::size_t i = 0; i < N; ++i) {
    *gb_lh += dlogit[i];
    for (std::size_t h = 0; h < H; ++h) {
      gW_lh[h] += dlogit[i] * f.mixed_h[i * H + h];
      dmixed[i * H + h] = dlogit[i] * w.W_lh[h];
      dvh[i * H + h] += dmixed[i * H + h];                      // residual path
    }
  }
  const float scale = 1.f / std::sqrt(static_cast<float>(H));
  std::vector<float> dA(N), ds(N);
  for (std::size_t i = 0; i < N; ++i) {
    float dotA = 0.f;
    for (std::size_t j = 0; j < N; ++j) {
      const float d = dotf(dmixed.data() + i * H, f.vertex_h.data() + j * H, H);
      dA[j] = d;
      dotA += f.attn[i * N + j] * d;
      const float a = f.attn[i * N + j];
      for (std::size_t h = 0; h < H; ++h) dvh[j * H + h] += a * dmixed[i * H + h];
    }
    for (std::size_t j = 0; j < N; ++j) {
      ds[j] = f.attn[i * N + j] * (dA[j] - dotA);
      *galpha += ds[j] * E[(i * N + j) * Ke];
      const float g = ds[j] * scale;
      float *di = dvh.data() + i * H, *dj = dvh.data() + j * H;      // two loops: rows i and j may be the same row
      const float *vi = f.vertex_h.data() + i * H, *vj = f.vertex_h.data() + j * H;
      for (std::size_t h = 0; h < H; ++h) di[h] += g * vj[h];
      for (std::size_t h = 0; h < H; ++h) dj[h] += g * vi[h];
    }
  }
  if (nh) {
    // d logits[i] / d logits_hxh[i] = lambda; every head contributes out_i / n_heads
    const float inv_heads = 1.f / static_cast<float>(nh);
    for (std::size_t i = 0; i < N; ++i) *glambda += dlogit[i] * f.logits_hxh[i];
    std::vector<float> dmx(N * H), dq(N * H), dk(N * H), dv(N * H), dat(N);
    for (std::size_t hd = 0; hd < nh; ++hd) {
      const float *Wq = w.W_q.data() + hd * H * H, *Wk = w.W_k.data() + hd * H * H, *Wv = w.W_v.data() + hd * H * H;
      const float *Wo = w.W_o.data() + hd * H;
      const float *q = f.hq.data() + hd * N * H, *k = f.hk.data() + hd * N * H, *v = f.hv.data() + hd * N * H;
      const float *mx = f.hmixed.data() + hd * N * H, *at = f.hattn.data() + hd * N * N;
      std::fill(dq.begin(), dq.end(), 0.f);
      std::fill(dk.begin(), dk.end(), 0.f);
      std::fill(dv.begin(), dv.end(), 0.f);
      for (std::size_t i = 0; i < N; ++i) {
        const float g = dlogit[i] * w.lambda_hxh * inv_heads;
        for (std::size_t o = 0; o < H; ++o) {
          gW_o[hd * H + o] += g * mx[i * H + o];
          dmx[i * H + o] = g * Wo[o];
        }
      }
      for (std::size_t i = 0; i < N; ++i) {
        float dot = 0.f;
        for (std::size_t j = 0; j < N; ++j) {
          const float d = dotf(dmx.data() + i * H, v + j * H, H);
          dat[j] = d;
          dot += at[i * N + j] * d;
          const float a = at[i * N + j];
          for (std::size_t o = 0; o < H; ++o) dv[j * H + o] += a * dmx[i * H + o];
        }
        for (std::size_t j = 0; j < N; ++j) {
          const float dsc = at[i * N + j] * (dat[j] - dot);        // d score[i, j]
          for (std::size_t e = 0; e < Ke; ++e) gW_e[hd * Ke + e] += dsc * E[(i * N + j) * Ke + e];
          const float gs = dsc * scale;
          for (std::size_t o = 0; o < H; ++o) {
            dq[i * H + o] += gs * k[j * H + o];
            dk[j * H + o] += gs * q[i * H + o];
          }
        }
      }
      // q = vh @ W_q (and k, v alike): weight gradients, and the branch's gradient into vertex_h
      for (std::size_t i = 0; i < N; ++i)
        for (std::size_t a = 0; a < H; ++a) {
          const float x = f.vertex_h[i * H + a];
          for (std::size_t o = 0; o < H; ++o) {
            gW_q[hd * H * H + a * H + o] += x * dq[i * H + o];
            gW_k[hd * H * H + a * H + o] += x * dk[i * H + o];
            gW_v[hd * H * H + a * H + o] += x * dv[i * H + o];
          }
          dvh[i * H + a] += dotf(dq.data() + i * H, Wq + a * H, H) + dotf(dk.data() + i * H, Wk + a * H, H) +
                            dotf(dv.data() + i * H, Wv + a * H, H);
        }
    }
  }
  std::vector<float> dpre(H);
  for (std::size_t i = 0; i < N; ++i) {
    for (std::size_t h = 0; h < H; ++h) {
      dpre[h] = dvh[i * H + h] * gelu_grad(f.pre[i * H + h]);
      gb_vp[h] += dpre[h];
    }
    for (std::size_t k = 0; k < Kv; ++k) {                          // unit stride over h: vectorises
      const float v = V[i * Kv + k];
      float* gr = gW_vp + k * H;
      for (std::size_t h = 0; h < H; ++h) gr[h] += v * dpre[h];
    }
  }
}

// -------------------------------------------------------- online learner ----
SimplexOnlineLearner::SimplexOnlineLearner(uint32_t num_slots, uint32_t max_entries, float gamma,
                                           float lr, uint32_t sgd_interval, float ema_alpha,
                                           uint64_t ema_interval, float gerber_c, float entropy_beta)
    : num_slots_(num_slots), max_entries_(max_entries), gamma_(gamma), gerber_c_(gerber_c),
      entropy_beta_(entropy_beta), sgd_interval_(sgd_interval == 0 ? 1 : sgd_interval), sgd_{lr},
      ema_(ema_alpha, ema_interval) {}

void SimplexOnlineLearner::initialize(const SimplexWeights& w) {
  fast_ = w;
  slow_ = w;
  grad_.assign(w.flat_size(), 0.f);
  init_ = true;
}

SimplexOnlineLearner::~SimplexOnlineLearner() { set_trace_path(""); }

void SimplexOnlineLearner::set_trace_path(const std::string& path) {
  if (trace_fp_) { std::fclose(trace_fp_); trace_fp_ = nullptr; }
  trace_path_ = path;
  if (!path.empty()) {
    trace_fp_ = std::fopen(path.c_str(), "a");
    if (trace_fp_) std::setvbuf(trace_fp_, nullptr, _IOLBF, 0);
  }
}

static double entropy_of(const std::vector<float>& p) {
  double ent = 0.0;
  for (float x : p) if (x > 0.f) ent -= x * std::log(x);
  return ent;
}

void SimplexOnlineLearner::trace_skip(const wire::ReplayOutcome& ev, const char* reason) {
  if (!trace_fp_) return;
  std::fprintf(trace_fp_, "{\"row_type\":\"skip\",\"status\":\"skipped\",\"status_reason\":\"%s\","
                          "\"gpu_step\":%llu,\"slot_id\":%u,\"outcome_status\":%u}\n",
               reason, static_cast<unsigned long long>(ev.gpu_step), ev.slot_id,
               static_cast<unsigned>(ev.outcome_status));
}

void SimplexOnlineLearner::record_decision(uint64_t slot_id, ActionRecord rec) {
  if (slot_id >= num_slots_) { ++tel_.invalid_slot_skips; return; }
  if (trace_fp_ && init_ && rec.V.size() == static_cast<std::size_t>(fast_.N) * fast_.K_v &&
      rec.E.size() == static_cast<std::size_t>(fast_.N) * fast_.N && rec.feats.size() == fast_.K_s) {
    SimplexForward f = simplex_forward(fast_, rec.V.data(), rec.E.data(), rec.feats.data());
    rec.entropy = static_cast<float>(entropy_of(f.p));
    std::fprintf(trace_fp_, "{\"row_type\":\"decision\",\"status\":\"ok\",\"gpu_step\":%llu,"
                            "\"slot_id\":%llu,\"chosen_idx\":%u,\"p_chosen\":%g,\"entropy\":%g,"
                            "\"temperature\":%g,\"entropy_beta\":%g,\"sgd_steps\":%llu}\n",
                 static_cast<unsigned long long>(rec.gpu_step),
                 static_cast<unsigned long long>(slot_id), rec.chosen, rec.p_chosen, entropy_of(f.p),
                 fast_.temperature, entropy_beta_, static_cast<unsigned long long>(tel_.sgd_steps));
  }
  auto& q = history_[static_cast<uint32_t>(slot_id)];
  q.push_back(std::move(rec));
  while (q.size() > max_entries_) q.pop_front();
  ++tel_.history_appends;
}

std::size_t SimplexOnlineLearner::history_size(uint32_t slot) const {
  auto it = history_.find(slot);
  return it == history_.end() ? 0 : it->second.size();
}

void SimplexOnlineLearner::on_replay_outcome(const wire::ReplayOutcome& ev) {
  ++tel_.replay_outcomes;
  if (ev.outcome_status != 0 || !std::isfinite(ev.reward_shaped)) { trace_skip(ev, "outcome_status"); return; }
  if (ev.slot_id >= num_slots_) { ++tel_.invalid_slot_skips; trace_skip(ev, "invalid_slot"); return; }
  auto it = history_.find(ev.slot_id);
  if (!init_) { ++tel_.skipped_missing_state; trace_skip(ev, "missing_weights"); return; }
  if (it == history_.end() || it->second.empty()) {
    ++tel_.skipped_missing_state; trace_skip(ev, "missing_decision"); return;
  }
  const float reward = ev.reward_shaped;
  const float mean = reward_stats_.mean();
  const float sd = reward_stats_.stddev();
  reward_stats_.update(reward);
  const float adv_raw = reward - mean;
  const float adv_std = sd > 1e-6f ? adv_raw / sd : adv_raw;
  tel_.last_advantage_raw = adv_raw;
  tel_.last_advantage_standardized = adv_std;
  for (const ActionRecord& rec : it->second) {
    if (rec.V.size() != static_cast<std::size_t>(fast_.N) * fast_.K_v ||
        rec.E.size() != static_cast<std::size_t>(fast_.N) * fast_.N || rec.feats.size() != fast_.K_s ||
        rec.chosen >= fast_.N) { ++tel_.skipped_missing_state; continue; }
    SimplexForward f = simplex_forward(fast_, rec.V.data(), rec.E.data(), rec.feats.data());
    const float n = static_cast<float>(fast_.N);
    const float then = std::log(std::max(rec.p_chosen, 1e-12f) * n);    // log-prob margin vs uniform
    const float now = std::log(std::max(f.p[rec.chosen], 1e-12f) * n);
    const float gw = gerber_weight(then, now, gerber_c_ * margin_stats_.stddev());
    margin_stats_.update(now);
    tel_.last_gerber_weight = gw;
    if (gw == 0.f) { ++tel_.gerber_rejected; continue; }
    ++tel_.gerber_accepted;
    const float adv = recency_decay(adv_std, ev.gpu_step, rec.gpu_step, gamma_);
    // trace-only diagnostics of this one credit: the W_lh block of the gradient accumulator before
    // the backward pass (its change is this credit's own W_lh gradient)
    const std::size_t lh_off = static_cast<std::size_t>(fast_.K_v) * fast_.H + fast_.H, lh_n = fast_.H;
    std::vector<float> lh_before;
    if (trace_fp_) lh_before.assign(grad_.begin() + lh_off, grad_.begin() + lh_off + lh_n);
    simplex_backward(fast_, f, rec.V.data(), rec.E.data(), rec.feats.data(), rec.chosen, adv,
                     entropy_beta_, grad_.data());
    const double ent = entropy_of(f.p);
    tel_.last_entropy = static_cast<float>(ent);
    ++tel_.credited_actions;
    if (trace_fp_) {
      double g_lh = 0.0, g_acc = 0.0, w_lh = 0.0, g_logit = 0.0;
      for (std::size_t h = 0; h < lh_n; ++h) {
        const double d = grad_[lh_off + h] - lh_before[h];
        g_lh += d * d;
        g_acc += static_cast<double>(grad_[lh_off + h]) * grad_[lh_off + h];
        w_lh += static_cast<double>(fast_.W_lh[h]) * fast_.W_lh[h];
      }
      for (std::size_t i = 0; i < f.p.size(); ++i) {             // d loss / d logits, as the backward forms it
        const float pi = f.p[i];
        float dz = -adv * ((i == rec.chosen ? 1.f : 0.f) - pi);
        if (entropy_beta_ != 0.f && pi > 0.f) dz += entropy_beta_ * pi * (std::log(pi) + static_cast<float>(ent));
        dz /= fast_.temperature;
        g_logit += static_cast<double>(dz) * dz;
      }
      std::fprintf(trace_fp_, "{\"row_type\":\"credit\",\"status\":\"ok\",\"gpu_step\":%llu,"
                              "\"slot_id\":%u,\"selection_step\":%llu,\"chosen_idx\":%u,\"p_chosen\":%g,"
                              "\"p_current_chosen\":%g,\"current_entropy\":%g,\"reward_shaped\":%g,"
                              "\"advantage_raw\":%g,\"advantage_standardized\":%g,\"gerber_weight\":%g,"
                              "\"advantage_final\":%g,\"behavior_logprob_margin\":%g,"
                              "\"current_logprob_margin\":%g,\"entropy\":%s,\"grad_logits_l2\":%g,"
                              "\"grad_w_lh_l2\":%g,\"grad_w_lh_accum_l2\":%g,\"w_lh_l2\":%g,"
                              "\"sgd_steps\":%llu,\"ema_blends\":%llu}\n",
                   static_cast<unsigned long long>(ev.gpu_step), ev.slot_id,
                   static_cast<unsigned long long>(rec.gpu_step), rec.chosen, rec.p_chosen,
                   f.p[rec.chosen], ent, reward, adv_raw, adv_std, gw, adv, then, now,
                   rec.entropy >= 0.f ? std::to_string(rec.entropy).c_str() : "null",
                   std::sqrt(g_logit), std::sqrt(g_lh), std::sqrt(g_acc), std::sqrt(w_lh),
                   static_cast<unsigned long long>(tel_.sgd_steps),
                   static_cast<unsigned long long>(tel_.ema_blends));
    }
    ++since_sgd_;
    ema_.tick();
    maybe_sgd();
  }
  if (trace_fp_)
    std::fprintf(trace_fp_, "{\"row_type\":\"replay_outcome\",\"gpu_step\":%llu,\"slot_id\":%u,"
                            "\"reward\":%g,\"advantage\":%g,\"sgd_steps\":%llu}\n",
                 static_cast<unsigned long long>(ev.gpu_step), ev.slot_id, reward, adv_std,
                 static_cast<unsigned long long>(tel_.sgd_steps));
}

void SimplexOnlineLearner::maybe_sgd() {
  if (since_sgd_ >= sgd_interval_) {
    std::vector<float> flat(fast_.flat_size());
    fast_.to_flat(flat.data());
    const float inv = 1.f / static_cast<float>(since_sgd_);
    double l2 = 0.0;
    for (float& g : grad_) { g *= inv; l2 += static_cast<double>(g) * g; }
    tel_.last_grad_l2 = static_cast<float>(std::sqrt(l2));
    sgd_.apply(flat.data(), grad_.data(), flat.size());
    fast_.from_flat(flat.data());
    std::fill(grad_.begin(), grad_.end(), 0.f);
    since_sgd_ = 0;
    ++tel_.sgd_steps;
  }
  if (ema_.should_blend()) {
    std::vector<float> f(fast_.flat_size()), s(slow_.flat_size());
    fast_.to_flat(f.data());
    slow_.to_flat(s.data());
    ema_.blend(s.data(), f.data(), s.size());
    slow_.from_flat(s.data());
    ++tel_.ema_blends;
  }
}

// ------------------------------------------------------------------ CSWG ----
float half_to_float(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {
      exp = 127 - 15 + 1;
      while ((man & 0x400u) == 0) { man <<= 1; --exp; }
      bits = sign | (exp << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
  else bits = sign | ((exp + 112) << 23) | (man << 13);
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}
uint16_t float_to_half(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t exp = static_cast<int32_t>((x >> 23) & 0xFF) - 127 + 15;
  uint32_t man = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFF) == 0xFF) return static_cast<uint16_t>(sign | 0x7C00u | (man ? 0x200u : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t hm = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (hm & 1))) ++hm;
    return static_cast<uint16_t>(sign | hm);
  }
  uint32_t hm = man >> 13;
  const uint32_t rem = man & 0x1FFFu;
  uint32_t out = sign | (static_cast<uint32_t>(exp) << 10) | hm;
  if (rem > 0x1000u || (rem == 0x1000u && (hm & 1))) ++out;
  return static_cast<uint16_t>(out);
}

std::string load_cswg(const std::string& path, CswgFile* out) {
  std::ifstream in(path, std::ios::binary);
  if (!in) return "CSWG: cannot open " + path;
  unsigned char hdr[28];
  in.read(reinterpret_cast<char*>(hdr), sizeof(hdr));
  if (in.gcount() != static_cast<std::streamsize>(sizeof(hdr))) return "CSWG: short header";
  if (std::memcmp(hdr, "CSWG", 4) != 0) return "CSWG bad magic";
  auto le32 = [&](int o) {
    return static_cast<uint32_t>(hdr[o]) | (static_cast<uint32_t>(hdr[o + 1]) << 8) |
           (static_cast<uint32_t>(hdr[o + 2]) << 16) | (static_cast<uint32_t>(hdr[o + 3]) << 24);
  };
  out->version = le32(4); out->n_layers = le32(8); out->d_global = le32(12);
  out->d_slot = le32(16); out->feature_dim = le32(20); out->dtype = le32(24);
  if (out->version != 1) return "CSWG: unsupported version";
  if (out->dtype != 1) return "CSWG: unsupported dtype (only fp16 = 1)";
  std::vector<char> rest((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
  if (rest.size() % 2) return "CSWG: payload is not a whole number of fp16 values";
  out->payload.resize(rest.size() / 2);
  for (std::size_t i = 0; i < out->payload.size(); ++i) {
    const uint16_t h = static_cast<uint8_t>(rest[2 * i]) | (static_cast<uint16_t>(static_cast<uint8_t>(rest[2 * i + 1])) << 8);
    out->payload[i] = half_to_float(h);
  }
  return "";
}

// -------------------------------------------------------- controller loop ----
uint64_t controller_main(const std::vector<std::string>& write_rings, const std::string& query_ring,
                         const std::string& replay_ring, const std::string& exit_flag_shm,
                         const std::string& stats_shm, SimplexOnlineLearner* learner,
                         ControllerCounts* counts, std::string* error) {
  auto fail = [&](const std::string& m) { if (error) *error = m; return uint64_t(0); };
  std::vector<ShmRegion> regions(write_rings.size() + 2);
  std::vector<RingView> wr(write_rings.size());
  RingView qr, rr;
  for (std::size_t i = 0; i < write_rings.size(); ++i) {
    std::string e = regions[i].open(write_rings[i], 0, false);
    if (!e.empty()) return fail(e);
    if (regions[i].size() < RingView::region_bytes(sizeof(wire::WriteEvent), wire::kWriteRingCapacity))
      return fail("write ring segment too small: " + write_rings[i]);
    wr[i].bind(regions[i].ptr(), sizeof(wire::WriteEvent), wire::kWriteRingCapacity, false);
  }
  ShmRegion& qreg = regions[write_rings.size()];
  ShmRegion& rreg = regions[write_rings.size() + 1];
  std::string e = qreg.open(query_ring, 0, false);
  if (!e.empty()) return fail(e);
  e = rreg.open(replay_ring, 0, false);
  if (!e.empty()) return fail(e);
  if (qreg.size() < RingView::region_bytes(sizeof(wire::QueryEvent), wire::kQueryRingCapacity) ||
      rreg.size() < RingView::region_bytes(sizeof(wire::ReplayOutcome), wire::kReplayRingCapacity))
    return fail("query / replay ring segment too small");
  qr.bind(qreg.ptr(), sizeof(wire::QueryEvent), wire::kQueryRingCapacity, false);
  rr.bind(rreg.ptr(), sizeof(wire::ReplayOutcome), wire::kReplayRingCapacity, false);
  ShmRegion exit_reg, stats_reg;
  e = exit_reg.open(exit_flag_shm, 0, false);
  if (!e.empty()) return fail(e);
  if (!stats_shm.empty()) {
    e = stats_reg.open(stats_shm, 0, false);
    if (!e.empty()) return fail(e);
    if (stats_reg.size() < 3 * sizeof(uint64_t)) return fail("stats shm must be at least 24 bytes");
  }
  ControllerCounts c;
  auto publish = [&]() {
    if (stats_reg.ok()) {
      const uint64_t v[3] = {c.writes, c.queries, c.replays};
      std::memcpy(stats_reg.ptr(), v, sizeof(v));
    }
  };
  publish();
  const volatile uint8_t* exit_byte = static_cast<const volatile uint8_t*>(exit_reg.ptr());
  wire::WriteEvent we;
  wire::QueryEvent qe;
  wire::ReplayOutcome ro;
  while (*exit_byte == 0) {
    bool busy = false;
    for (RingView& r : wr)
      if (r.pop(&we)) { ++c.writes; busy = true; }
    if (qr.pop(&qe)) { ++c.queries; busy = true; }
    if (rr.pop(&ro)) {
      ++c.replays;
      busy = true;
      if (learner) learner->on_replay_outcome(ro);
    }
    if (busy) publish();
    else std::this_thread::yield();
  }
  if (counts) *counts = c;
  return c.writes + c.queries + c.replays;
}

}  // namespace ccb::ctrl
