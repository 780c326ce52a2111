// CPU control plane of the episodic-memory path: credit assignment, the small
// optimizers it uses, the 16-vertex simplex policy (forward + REINFORCE
// backward), the online learner that ties them to replay outcomes, the CSWG
// weight-file reader and the controller event loop that drains the shared-
// memory rings.  Plain C++17, no torch / ATen dependency.
//
// Behavioural counterparts in the reference:
//   credit          kernels/_cpu_ssm_controller/src/credit.cpp (recency_decay,
//                   gerber_weight, RollingStddev)
//   optimizers      .../optimizer.cpp (SgdStep, FastSlowEma)
//   simplex policy  .../simplex_policy.{h,cpp}
//   online learner  .../simplex_learner.{h,cpp}
//   action history  .../action_history.cpp
//   CSWG            .../cpu_ssm_controller.cpp:41-75, 210-307
//   controller loop .../controller_main.cpp:41-99
#pragma once
#include <cstdint>
#include <deque>
#include <cstdio>
#include <string>
#include <unordered_map>
#include <vector>

#include "ring.h"
#include "wire_format.h"

namespace ccb::ctrl {

// ---------------------------------------------------------------- credit ----
// reward * gamma^(T - P) for an action taken at step P judged at step T (no
// decay when the outcome predates the action).
float recency_decay(float reward, uint64_t outcome_step, uint64_t action_step, float gamma);
// Gerber-style co-movement gate: 1 when the logit at decision time and the
// current logit agree (same sign and both beyond the threshold, or equal up to
// rounding), else 0.
float gerber_weight(float logit_then, float logit_now, float threshold);

class RollingStddev {          // bias-corrected EMA mean / stddev
 public:
  explicit RollingStddev(float decay = 0.99f);
  void update(float x);
  float mean() const;
  float stddev() const;
  uint64_t count() const { return count_; }
 private:
  double decay_, ema_ = 0.0, ema_sq_ = 0.0;
  uint64_t count_ = 0;
};

// ------------------------------------------------------------ optimizers ----
struct SgdStep {
  float lr;
  void apply(float* w, const float* g, std::size_t n) const {
    for (std::size_t i = 0; i < n; ++i) w[i] -= lr * g[i];
  }
};
class FastSlowEma {            // slow <- (1-a) slow + a fast every `interval` events
 public:
  FastSlowEma(float alpha, uint64_t interval);
  void tick() { ++events_; }
  bool should_blend() const { return events_ > 0 && events_ % interval_ == 0; }
  void blend(float* slow, const float* fast, std::size_t n) const;
  void set_alpha(float a);
  float alpha() const { return alpha_; }
  uint64_t events() const { return events_; }
 private:
  float alpha_;
  uint64_t interval_, events_ = 0;
};

// -------------------------------------------------------- simplex policy ----
struct SimplexWeights {
  uint32_t K_v = 0, K_e = 1, K_s = 0, H = 0, N = 0;
  std::vector<float> W_vp;   // [K_v, H]
  std::vector<float> b_vp;   // [H]
  std::vector<float> W_lh;   // [H]
  float b_lh = 0.f;
  std::vector<float> W_sb;   // [K_s]
  float alpha = 0.f;         // edge-vs-content mixing
  float temperature = 1.f;
  // Optional residual branch: n_heads attention heads over the N vertices with learned H x H
  // query / key / value projections and a per-head edge-feature bias; each head emits one logit
  // per vertex (W_o), the heads are averaged and lambda_hxh scales the sum into the base logits
  // (simplex_policy.h:27-53 of the reference).  n_heads == 0 leaves the base policy untouched.
  uint32_t n_heads = 0;
  float lambda_hxh = 0.f;
  std::vector<float> W_q, W_k, W_v;   // [n_heads, H, H] each, row-major (out = in @ W)
  std::vector<float> W_o;             // [n_heads, H]
  std::vector<float> W_e;             // [n_heads, K_e]
  // Write-bucket embedding table: carried by the weight file and the learner state, not read by
  // the forward pass (as in the reference's current policy).
  uint32_t n_buckets = 0, embed_dim = 0;
  std::vector<float> bucket_embed;    // [n_buckets, embed_dim]
  // flat layout: W_vp | b_vp | W_lh | b_lh | W_sb | alpha | [lambda | W_q | W_k | W_v | W_o | W_e] | bucket_embed
  std::size_t flat_size() const {
    return W_vp.size() + b_vp.size() + W_lh.size() + 1 + W_sb.size() + 1 +
           (n_heads ? 1 + W_q.size() + W_k.size() + W_v.size() + W_o.size() + W_e.size() : 0) +
           bucket_embed.size();
  }
  void resize();                    // allocate every vector from the dims
  void to_flat(float* out) const;
  void from_flat(const float* in);
  std::string validate() const;     // empty when consistent
};
struct SimplexForward {
  std::vector<float> pre;      // [N, H] pre-activation of the vertex projection
  std::vector<float> vertex_h; // [N, H] gelu(pre)
  std::vector<float> attn;     // [N, N] row softmax
  std::vector<float> mixed_h;  // [N, H] attn @ vertex_h + vertex_h
  std::vector<float> logits;   // [N] (residual branch included)
  std::vector<float> p;        // [N] softmax((logits + bias) / T)
  float simplex_bias = 0.f;
  // residual branch, saved for backward
  std::vector<float> hq, hk, hv, hmixed;   // [n_heads, N, H]
  std::vector<float> hattn;                // [n_heads, N, N]
  std::vector<float> logits_hxh;           // [N] before lambda
};
// V: [N, K_v]; E: [N, N, K_e] edge features (the base mixing reads feature 0); feats: [K_s].
SimplexForward simplex_forward(const SimplexWeights& w, const float* V, const float* E, const float* feats);
// Accumulates d(-advantage * log p[chosen] - entropy_beta * H(p)) / d weights into `grad`
// (same flat layout as SimplexWeights::to_flat).
void simplex_backward(const SimplexWeights& w, const SimplexForward& f, const float* V, const float* E,
                      const float* feats, uint32_t chosen, float advantage, float entropy_beta,
                      float* grad);

// ---------------------------------------------------- pretrain model ----
// Forward of the controller's offline-pretrained trunk (cpu_ssm_controller.cpp:309-355 of the
// reference): h = x W_in^T + b; per layer h = gelu(h * decay_l + h @ w_in_l + bias_l) @ w_out_l;
// logits = h W_p^T + b_p, value = h w_v + b_v.  x: [B, F]; logits_out: [B, D_slot]; value_out: [B].
struct PretrainModel {
  uint32_t F = 0, Dg = 0, L = 0, Ds = 0;
  const float *in_w = nullptr, *in_b = nullptr;          // [Dg, F], [Dg]
  const float *decay = nullptr, *w_in = nullptr, *w_out = nullptr, *bias = nullptr;   // [L,Dg] [L,Dg,Dg] [L,Dg,Dg] [L,Dg]
  const float *pol_w = nullptr, *pol_b = nullptr, *val_w = nullptr, *val_b = nullptr; // [Ds,Dg] [Ds] [Dg] [1]
};
void forward_pretrain_model(const PretrainModel& m, const float* x, std::size_t B, float* logits_out,
                            float* value_out);

// -------------------------------------------------------- online learner ----
struct ActionRecord {
  uint64_t gpu_step = 0;
  uint32_t policy_version = 0, chosen = 0;
  float p_chosen = 0.f;
  int32_t bucket = 0;
  float entropy = -1.f;   // policy entropy at decision time; filled only while a trace is open
  std::vector<float> V, E, feats;
};
struct LearnerTelemetry {
  uint64_t replay_outcomes = 0, history_appends = 0, credited_actions = 0, gerber_accepted = 0,
           gerber_rejected = 0, skipped_missing_state = 0, invalid_slot_skips = 0, sgd_steps = 0,
           ema_blends = 0;
  float last_advantage_raw = 0.f, last_advantage_standardized = 0.f, last_gerber_weight = 0.f,
        last_entropy = 0.f, last_grad_l2 = 0.f;
};
class SimplexOnlineLearner {
 public:
  SimplexOnlineLearner(uint32_t num_slots = 4096, uint32_t max_entries_per_slot = 64,
                       float gamma = 0.995f, float lr = 1e-3f, uint32_t sgd_interval = 256,
                       float ema_alpha = 0.25f, uint64_t ema_interval = 64, float gerber_c = 0.5f,
                       float entropy_beta = 0.f);
  void initialize(const SimplexWeights& w);
  bool initialized() const { return init_; }
  void record_decision(uint64_t slot_id, ActionRecord rec);
  void on_replay_outcome(const wire::ReplayOutcome& ev);
  const SimplexWeights& fast() const { return fast_; }
  const SimplexWeights& slow() const { return slow_; }
  const LearnerTelemetry& telemetry() const { return tel_; }
  std::size_t history_size(uint32_t slot) const;
  // NDJSON trace, one row per event: "decision" when an action is recorded, "credit" for every
  // action a replay outcome reaches, "skip" (with status_reason) when an outcome reaches none,
  // "replay_outcome" once per outcome.  An empty path closes the file.
  void set_trace_path(const std::string& path);
  ~SimplexOnlineLearner();
  SimplexOnlineLearner(const SimplexOnlineLearner&) = delete;
  SimplexOnlineLearner& operator=(const SimplexOnlineLearner&) = delete;
 private:
  void maybe_sgd();
  void trace_skip(const wire::ReplayOutcome& ev, const char* reason);
  uint32_t num_slots_, max_entries_;
  float gamma_, gerber_c_, entropy_beta_;
  uint32_t sgd_interval_, since_sgd_ = 0;
  SgdStep sgd_;
  FastSlowEma ema_;
  RollingStddev reward_stats_{0.99f};
  RollingStddev margin_stats_{0.99f};
  bool init_ = false;
  SimplexWeights fast_, slow_;
  std::vector<float> grad_;
  std::unordered_map<uint32_t, std::deque<ActionRecord>> history_;
  LearnerTelemetry tel_;
  std::string trace_path_;
  std::FILE* trace_fp_ = nullptr;
};

// ------------------------------------------------------------------ CSWG ----
// Weight file: "CSWG" magic, then six little-endian u32 (version, n_layers,
// d_global, d_slot, feature_dim, dtype) = 28-byte header, then fp16 payload.
struct CswgFile {
  uint32_t version = 0, n_layers = 0, d_global = 0, d_slot = 0, feature_dim = 0, dtype = 0;
  std::vector<float> payload;   // decoded to fp32
};
std::string load_cswg(const std::string& path, CswgFile* out);   // "" on success
float half_to_float(uint16_t h);
uint16_t float_to_half(float f);

// -------------------------------------------------------- controller loop ----
struct ControllerCounts { uint64_t writes = 0, queries = 0, replays = 0; };
// Drains the named rings until the byte in `exit_flag_shm` becomes non-zero.
// Replay outcomes are fed to `learner` when given.  Returns total events.
uint64_t controller_main(const std::vector<std::string>& write_rings, const std::string& query_ring,
                         const std::string& replay_ring, const std::string& exit_flag_shm,
                         const std::string& stats_shm, SimplexOnlineLearner* learner,
                         ControllerCounts* counts, std::string* error);

}  // namespace ccb::ctrl
