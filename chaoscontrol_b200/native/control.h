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
  std::size_t flat_size() const { return W_vp.size() + b_vp.size() + W_lh.size() + 1 + W_sb.size() + 1; }
  void to_flat(float* out) const;
  void from_flat(const float* in);
  std::string validate() const;     // empty when consistent
};
struct SimplexForward {
  std::vector<float> pre;      // [N, H] pre-activation of the vertex projection
  std::vector<float> vertex_h; // [N, H] gelu(pre)
  std::vector<float> attn;     // [N, N] row softmax
  std::vector<float> mixed_h;  // [N, H] attn @ vertex_h + vertex_h
  std::vector<float> logits;   // [N]
  std::vector<float> p;        // [N] softmax((logits + bias) / T)
  float simplex_bias = 0.f;
};
// V: [N, K_v]; E: [N, N] edge features; feats: [K_s].
SimplexForward simplex_forward(const SimplexWeights& w, const float* V, const float* E, const float* feats);
// Accumulates d(-advantage * log p[chosen] - entropy_beta * H(p)) / d weights into `grad`
// (same flat layout as SimplexWeights::to_flat).
void simplex_backward(const SimplexWeights& w, const SimplexForward& f, const float* V, const float* E,
                      const float* feats, uint32_t chosen, float advantage, float entropy_beta,
                      float* grad);

// -------------------------------------------------------- online learner ----
struct ActionRecord {
  uint64_t gpu_step = 0;
  uint32_t policy_version = 0, chosen = 0;
  float p_chosen = 0.f;
  int32_t bucket = 0;
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
