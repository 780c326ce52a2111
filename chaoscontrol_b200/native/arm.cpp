// Native pieces of the memory-maintenance plane that run on host cores:
//
//   ArmScheduler        which (probe frame, chunk of slots) the scoring rank works on next: frames
//                       in arrival order with a TTL and a bounded queue, slots of a frame handed out
//                       round-robin in chunks of <= 16 as ArmMaintenanceJob wire records, in-flight
//                       reservations, completion through ArmMaintenanceResult records
//                       (cf. kernels/_cpu_ssm_controller/src/cpu_ssm_controller.cpp:1376-1617)
//   rms_lmhead_nll      fused RMSNorm -> LM head -> per-token NLL on the CPU: bf16 operands, the
//                       vocabulary streamed in tiles through the bf16 matmul (AMX tiles when the
//                       CPU has them) with an online log-sum-exp, logits never materialised for the
//                       whole vocabulary (cf. .../amx_matmul.cpp:384-624)
//   EvidenceEngine      per-lane bookkeeping of cue frames plus the NLL of each 32-token cue under
//                       the installed LM head, with running means (cf. cpu_ssm_controller.cpp:1618-1888)
//   SlotSsmLearner      the per-slot diagonal-SSM controller: forward step, per-slot action history
//                       with eviction marks and garbage collection, credit assignment from replay
//                       outcomes (recency decay x Gerber gate x standardised reward), exact
//                       gradient of the one-step logit w.r.t. every weight, SGD every k credited
//                       actions and a slow EMA copy (cf. .../online_learning.{h,cpp},
//                       action_history.cpp, event_handlers.cpp)
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <deque>
#include <limits>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "control.h"
#include "wire_format.h"

namespace ccb::ctrl {
void matvec(const float*, const float*, float*, int, int);
void diag_step(const float*, const float*, float*, int);
int bf16_matmul(const uint16_t*, const uint16_t*, float*, int, int, int);
void pack_vnni_wt(const uint16_t* W, int V, int D, std::vector<uint16_t>* out);
int lse_over_vnni(const uint16_t* xn, int T, int Tpad, int Dpad, const uint16_t* packed, int V,
                  const int64_t* targets, float* run_m, float* run_s, float* tgt);
}  // namespace ccb::ctrl

using namespace ccb;
using namespace ccb::ctrl;

namespace {

constexpr uint64_t kNoSlot = std::numeric_limits<uint64_t>::max();
constexpr int kArmSlots = 16;

inline float bf16_to_f32(uint16_t v) {
  uint32_t b = (uint32_t)v << 16;
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {
  uint32_t b;
  std::memcpy(&b, &f, 4);
  b += 0x7FFFu + ((b >> 16) & 1u);   // round to nearest even
  return (uint16_t)(b >> 16);
}

// ------------------------------------------------------------------ scheduler
struct FrameState {
  uint64_t frame_id = 0, step = 0, cutoff = kNoSlot;
  uint8_t stream = 0;
  std::unordered_set<uint64_t> processed, reserved;
};

class ArmScheduler {
 public:
  ArmScheduler(uint32_t streams, uint32_t chunk, uint32_t ttl, uint32_t max_frames)
      : streams_(std::max<uint32_t>(1, streams)),
        chunk_(std::min<uint32_t>(std::max<uint32_t>(1, chunk), kArmSlots)),
        ttl_(ttl), max_frames_(std::max<uint32_t>(1, max_frames)) {}

  bool ingest(uint64_t frame_id, uint64_t step, uint32_t stream, uint64_t cutoff) {
    for (const auto& f : frames_)
      if (f.frame_id == frame_id) { ++c_[kDuplicate]; return false; }
    if (frames_.size() >= max_frames_) { frames_.pop_front(); ++c_[kDroppedOverflow]; }
    FrameState f;
    f.frame_id = frame_id; f.step = step; f.cutoff = cutoff; f.stream = (uint8_t)(stream % streams_);
    frames_.push_back(std::move(f));
    ++c_[kIngested];
    c_[kDepthMax] = std::max<uint64_t>(c_[kDepthMax], frames_.size());
    return true;
  }

  // 1 = job written, 0 = nothing to do
  int next_job(uint64_t step, const uint64_t* visible, int n_visible, wire::ArmMaintenanceJob* out) {
    if (ttl_)
      while (!frames_.empty() && step > frames_.front().step && step - frames_.front().step > ttl_) {
        frames_.pop_front();
        ++c_[kDroppedStale];
      }
    if (n_visible <= 0) { ++c_[kSkipNoSlots]; return 0; }
    while (!frames_.empty()) {
      FrameState& f = frames_.front();
      std::vector<uint64_t> open;
      size_t unprocessed = 0;
      for (int i = 0; i < n_visible; ++i) {
        if (f.processed.count(visible[i])) continue;
        ++unprocessed;
        if (!f.reserved.count(visible[i])) open.push_back(visible[i]);
      }
      if (unprocessed == 0) { frames_.pop_front(); ++c_[kCompleted]; continue; }
      if (open.empty()) { ++c_[kSkipInflight]; return 0; }
      const size_t start = cursor_ % open.size();
      const size_t count = std::min<size_t>(chunk_, open.size());
      std::memset(out, 0, sizeof(*out));
      out->event_type = 4; out->job_type = 1; out->stream_id = f.stream;
      out->slot_count = (uint32_t)count;
      out->job_id = next_job_++;
      out->frame_id = f.frame_id; out->step = f.step; out->cache_read_cutoff = f.cutoff;
      for (int i = 0; i < kArmSlots; ++i) out->slot_ids[i] = kNoSlot;
      auto& fl = inflight_[out->job_id];
      fl.first = f.frame_id;
      for (size_t i = 0; i < count; ++i) {
        const uint64_t s = open[(start + i) % open.size()];
        out->slot_ids[i] = s;
        f.reserved.insert(s);
        fl.second.push_back(s);
      }
      cursor_ += count;
      ++c_[kJobs];
      c_[kSlotsScheduled] += count;
      return 1;
    }
    ++c_[kSkipNoFrame];
    return 0;
  }

  void record(const wire::ArmMaintenanceResult& r) {
    auto it = inflight_.find(r.job_id);
    if (it != inflight_.end()) {
      for (auto& f : frames_) {
        if (f.frame_id != it->second.first) continue;
        for (uint64_t s : it->second.second) {
          f.reserved.erase(s);
          if (r.status == 0) f.processed.insert(s);
        }
        break;
      }
      inflight_.erase(it);
    }
    ++c_[kResults];
    c_[kSlotsScored] += r.slots_scored;
    c_[kConfirmed] += r.actions_confirmed;
    c_[kRejected] += r.actions_rejected;
    if (r.status != 0) ++c_[kResultErrors];
    secs_[0] += r.probe_seconds; secs_[1] += r.oracle_seconds; secs_[2] += r.cpu_seconds;
    secs_[3] = std::max<double>(secs_[3], r.frame_age_seconds);
  }

  enum { kIngested, kCompleted, kDroppedStale, kDroppedOverflow, kDuplicate, kJobs, kResults, kSlotsScheduled,
         kSlotsScored, kConfirmed, kRejected, kResultErrors, kSkipNoFrame, kSkipNoSlots, kSkipInflight, kDepthMax,
         kNumCounters };
  void diagnostics(uint64_t* counters17, double* seconds4) const {
    for (int i = 0; i < kNumCounters; ++i) counters17[i] = c_[i];
    counters17[kNumCounters] = frames_.size();
    for (int i = 0; i < 4; ++i) seconds4[i] = secs_[i];
  }

 private:
  uint32_t streams_, chunk_, ttl_, max_frames_;
  uint64_t next_job_ = 1;
  size_t cursor_ = 0;
  std::deque<FrameState> frames_;
  std::unordered_map<uint64_t, std::pair<uint64_t, std::vector<uint64_t>>> inflight_;
  uint64_t c_[kNumCounters] = {};
  double secs_[4] = {};
};

// --------------------------------------------------- fused CPU RMSNorm -> LM head -> NLL
constexpr int kVocabTile = 256;

struct LmHead {
  int D = 0, V = 0;
  std::vector<float> norm_w;
  std::vector<uint16_t> wt_tiles;   // per vocabulary tile: [D, kVocabTile] bf16 (W^T, zero padded)
  std::vector<uint16_t> vnni;       // the same weight in 16 x 16 x 32 VNNI tiles, packed once (AMX path)
  int tiles() const { return (V + kVocabTile - 1) / kVocabTile; }
};

void pack_lm_head(const float* norm_w, const uint16_t* W, int V, int D, LmHead* out) {
  out->D = D; out->V = V;
  out->norm_w.assign(norm_w, norm_w + D);
  out->wt_tiles.assign((size_t)out->tiles() * D * kVocabTile, 0);
  for (int v = 0; v < V; ++v) {
    uint16_t* tile = out->wt_tiles.data() + (size_t)(v / kVocabTile) * D * kVocabTile;
    for (int d = 0; d < D; ++d) tile[(size_t)d * kVocabTile + v % kVocabTile] = W[(size_t)v * D + d];
  }
  pack_vnni_wt(W, V, D, &out->vnni);
}

// hidden: [T, D] bf16; targets: [T]; nll: [T].  Returns 1 when the AMX path ran.
// mode: 0 = the VNNI-packed fused AMX path when the CPU has AMX, else the generic path;
// 1 = generic matmul path (packs per call when it uses AMX); used to pin the two against each other.
int rms_lmhead_nll_mode(const LmHead& h, const uint16_t* hidden, const int64_t* targets, int T, float eps, float* nll,
                        int mode) {
  const int D = h.D;
  const int Tpad = (T + 15) / 16 * 16, Dpad = (D + 31) / 32 * 32;
  std::vector<uint16_t> xn((size_t)Tpad * Dpad, 0);
  for (int t = 0; t < T; ++t) {
    double ss = 0.0;
    for (int d = 0; d < D; ++d) { const float v = bf16_to_f32(hidden[(size_t)t * D + d]); ss += (double)v * v; }
    const float inv = 1.0f / std::sqrt((float)(ss / D) + eps);
    for (int d = 0; d < D; ++d)
      xn[(size_t)t * Dpad + d] = f32_to_bf16(bf16_to_f32(hidden[(size_t)t * D + d]) * inv * h.norm_w[d]);
  }
  std::vector<float> run_m(T, -INFINITY), run_s(T, 0.f), tgt(T, 0.f);
  if (mode == 0 && !h.vnni.empty() &&
      lse_over_vnni(xn.data(), T, Tpad, Dpad, h.vnni.data(), h.V, targets, run_m.data(), run_s.data(), tgt.data())) {
    for (int t = 0; t < T; ++t) nll[t] = run_m[t] + std::log(run_s[t]) - tgt[t];
    return 1;
  }
  if (Dpad != D) {                       // the generic path wants densely packed rows
    for (int t = 1; t < T; ++t) std::memmove(&xn[(size_t)t * D], &xn[(size_t)t * Dpad], (size_t)D * 2);
  }
  std::vector<float> logits((size_t)T * kVocabTile);
  int used_amx = 0;
  for (int tile = 0; tile < h.tiles(); ++tile) {
    used_amx |= bf16_matmul(xn.data(), h.wt_tiles.data() + (size_t)tile * D * kVocabTile, logits.data(), T,
                            kVocabTile, D);
    const int v0 = tile * kVocabTile, nv = std::min(kVocabTile, h.V - v0);
    for (int t = 0; t < T; ++t) {
      const float* row = logits.data() + (size_t)t * kVocabTile;
      float m = run_m[t];
      for (int j = 0; j < nv; ++j) m = std::max(m, row[j]);
      float s = run_s[t] * std::exp(run_m[t] - m);
      for (int j = 0; j < nv; ++j) s += std::exp(row[j] - m);
      run_m[t] = m; run_s[t] = s;
      const int64_t y = targets[t];
      if (y >= v0 && y < v0 + nv) tgt[t] = row[y - v0];
    }
  }
  for (int t = 0; t < T; ++t) nll[t] = run_m[t] + std::log(run_s[t]) - tgt[t];
  return used_amx;
}
int rms_lmhead_nll(const LmHead& h, const uint16_t* hidden, const int64_t* targets, int T, float eps, float* nll) {
  return rms_lmhead_nll_mode(h, hidden, targets, T, eps, nll, 0);
}

// ------------------------------------------------------------------ evidence engine
constexpr int kCueTokens = 32, kCueTile = 64;

class EvidenceEngine {
 public:
  EvidenceEngine(uint32_t lanes, uint32_t d_model)
      : lanes_(std::max<uint32_t>(1, lanes)), d_model_(std::max<uint32_t>(1, d_model)), adv_(lanes_, 0),
        work_(lanes_, 0), lane_secs_(lanes_, 0.0) {}
  void set_lm_head(const float* norm_w, const uint16_t* W, int V) {
    pack_lm_head(norm_w, W, V, (int)d_model_, &head_);
    head_set_ = true;
    ++head_sets_;
  }
  // cue_hidden: [32, d_model] bf16; cue_targets: [32] int32
  int ingest(const uint16_t* cue_hidden, const int32_t* cue_targets, uint64_t frame_id, uint64_t step,
             uint32_t stream) {
    if (shutdown_) return -1;
    const uint32_t lane = stream % lanes_;
    ++frames_; last_frame_ = frame_id; last_step_ = step; last_stream_ = stream;
    ++adv_[lane];
    work_[lane] += kCueTile;
    if (head_set_) {
      const auto t0 = std::chrono::steady_clock::now();
      int64_t y[kCueTokens];
      for (int i = 0; i < kCueTokens; ++i) y[i] = cue_targets[i];
      float nll[kCueTokens];
      used_amx_ = rms_lmhead_nll(head_, cue_hidden, y, kCueTokens, 1e-6f, nll);
      double sum = 0.0, mx = -INFINITY;
      int fin = 0;
      for (float v : nll)
        if (std::isfinite(v)) { sum += v; mx = std::max<double>(mx, v); ++fin; }
      last_mean_ = fin ? sum / fin : 0.0;
      last_max_ = fin ? mx : 0.0;
      last_finite_ = (double)fin / kCueTokens;
      mean_ema_ = calls_ ? 0.95 * mean_ema_ + 0.05 * last_mean_ : last_mean_;
      finite_ema_ = calls_ ? 0.95 * finite_ema_ + 0.05 * last_finite_ : last_finite_;
      ++calls_;
      const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
      lane_secs_[lane] += dt; secs_total_ += dt; last_secs_ = dt;
    }
    return 0;
  }
  void shutdown() { shutdown_ = true; }
  // out_u64[8]: frames, last_frame, last_step, last_stream, head_sets, nll_calls, used_amx, shutdown
  // out_f64[7]: secs_total, last_secs, mean_ema, finite_ema, last_mean, last_max, last_finite
  void diagnostics(uint64_t* u, double* f, uint64_t* lane_adv, uint64_t* lane_work, double* lane_secs) const {
    u[0] = frames_; u[1] = last_frame_; u[2] = last_step_; u[3] = last_stream_; u[4] = head_sets_; u[5] = calls_;
    u[6] = (uint64_t)used_amx_; u[7] = shutdown_;
    f[0] = secs_total_; f[1] = last_secs_; f[2] = mean_ema_; f[3] = finite_ema_; f[4] = last_mean_; f[5] = last_max_;
    f[6] = last_finite_;
    for (uint32_t i = 0; i < lanes_; ++i) { lane_adv[i] = adv_[i]; lane_work[i] = work_[i]; lane_secs[i] = lane_secs_[i]; }
  }
  uint32_t lanes() const { return lanes_; }

 private:
  uint32_t lanes_, d_model_;
  bool shutdown_ = false, head_set_ = false;
  LmHead head_;
  uint64_t frames_ = 0, last_frame_ = 0, last_step_ = 0, head_sets_ = 0, calls_ = 0;
  uint32_t last_stream_ = 0;
  int used_amx_ = 0;
  std::vector<uint64_t> adv_, work_;
  std::vector<double> lane_secs_;
  double secs_total_ = 0, last_secs_ = 0, mean_ema_ = 0, finite_ema_ = 0, last_mean_ = 0, last_max_ = 0,
         last_finite_ = 0;
};

// ------------------------------------------------------------------ per-slot SSM learner
struct SsmWeights {
  int F = 0, G = 0, S = 0;
  std::vector<float> w;   // [Wg (G*F) | Ws (S*F) | dg (G) | ds (S) | og (G) | os (S) | bias]
  size_t size() const { return (size_t)G * F + (size_t)S * F + 2 * (size_t)G + 2 * (size_t)S + 1; }
  float* Wg() { return w.data(); }
  float* Ws() { return Wg() + (size_t)G * F; }
  float* dg() { return Ws() + (size_t)S * F; }
  float* ds() { return dg() + G; }
  float* og() { return ds() + S; }
  float* os() { return og() + G; }
  float* bias() { return os() + S; }
};

// new_g = dg*g + Wg f ; new_s = ds*s + Ws f ; logit = <new_g, og> + <new_s, os> + bias
float ssm_forward(SsmWeights& w, const float* f, const float* g, const float* s, float* new_g, float* new_s) {
  matvec(w.Wg(), f, new_g, w.G, w.F);
  matvec(w.Ws(), f, new_s, w.S, w.F);
  std::vector<float> hg(g, g + w.G), hs(s, s + w.S);
  diag_step(w.dg(), new_g, hg.data(), w.G);
  diag_step(w.ds(), new_s, hs.data(), w.S);
  float logit = *w.bias();
  for (int i = 0; i < w.G; ++i) { new_g[i] = hg[i]; logit += hg[i] * w.og()[i]; }
  for (int i = 0; i < w.S; ++i) { new_s[i] = hs[i]; logit += hs[i] * w.os()[i]; }
  return logit;
}

struct HistoryEntry {
  uint64_t gpu_step = 0;
  uint32_t policy_version = 0;
  float logit = 0.f;
  uint8_t rank = 0;
  std::vector<float> f, g, s;
};

class SlotSsmLearner {
 public:
  SlotSsmLearner(uint32_t slots, uint32_t max_entries, float gamma, float gerber_c, float lr, uint32_t sgd_interval,
                 float ema_alpha, uint64_t ema_interval)
      : slots_(slots), max_entries_(std::max<uint32_t>(1, max_entries)), gamma_(gamma), gerber_c_(gerber_c), lr_(lr),
        sgd_interval_(std::max<uint32_t>(1, sgd_interval)), ema_(ema_alpha, std::max<uint64_t>(1, ema_interval)),
        hist_(slots), evicted_(slots, 0), evicted_at_(slots, 0) {}

  int init(int F, int G, int S, const float* flat) {
    fast_.F = F; fast_.G = G; fast_.S = S;
    fast_.w.assign(flat, flat + fast_.size());
    slow_ = fast_;
    grad_.assign(fast_.size(), 0.f);
    init_ = true;
    return 0;
  }
  bool initialized() const { return init_; }
  SsmWeights& fast() { return fast_; }
  SsmWeights& slow() { return slow_; }

  int record(uint32_t slot, HistoryEntry e) {
    if (slot >= slots_) { ++tel_[kInvalidSlot]; return -1; }
    auto& h = hist_[slot];
    if (h.size() >= max_entries_) h.pop_front();
    h.push_back(std::move(e));
    evicted_[slot] = 0;
    ++tel_[kAppends];
    return 0;
  }
  size_t history_size(uint32_t slot) const { return slot < slots_ ? hist_[slot].size() : 0; }
  void mark_evicted(uint32_t slot, uint64_t at) { if (slot < slots_) { evicted_[slot] = 1; evicted_at_[slot] = at; } }
  bool is_evicted(uint32_t slot) const { return slot < slots_ && evicted_[slot]; }
  // histories of slots evicted more than `lookahead` events ago are dropped
  void gc(uint64_t now, uint64_t lookahead) {
    for (uint32_t s = 0; s < slots_; ++s)
      if (evicted_[s] && now >= evicted_at_[s] + lookahead) hist_[s].clear();
  }

  void on_replay_outcome(const wire::ReplayOutcome& ev) {
    ++tel_[kOutcomes];
    if (ev.slot_id >= slots_) { ++tel_[kInvalidSlot]; return; }
    if (!init_) { ++tel_[kSkipNoWeights]; return; }
    reward_stats_.update(ev.reward_shaped);
    const float sd = reward_stats_.stddev();
    const float adv = sd > 1e-6f ? ev.reward_shaped / sd : ev.reward_shaped;
    last_credit_ = 0.f;
    for (const HistoryEntry& e : hist_[ev.slot_id]) {
      if ((int)e.f.size() != fast_.F || (int)e.g.size() != fast_.G || (int)e.s.size() != fast_.S) {
        ++tel_[kSkipBadShape];
        continue;
      }
      std::vector<float> ng(fast_.G), ns(fast_.S);
      const float now = ssm_forward(fast_, e.f.data(), e.g.data(), e.s.data(), ng.data(), ns.data());
      const float credit = recency_decay(adv, ev.gpu_step, e.gpu_step, gamma_) * gerber_weight(e.logit, now, gerber_c_);
      ++tel_[kCredited];
      if (credit == 0.f) continue;
      ++tel_[kNonzero];
      last_credit_ += credit;
      accumulate(e, ng, ns, credit);
      if (++since_sgd_ >= sgd_interval_) {
        for (size_t i = 0; i < grad_.size(); ++i) { fast_.w[i] -= lr_ * grad_[i]; grad_[i] = 0.f; }
        since_sgd_ = 0;
        ++tel_[kSgd];
      }
    }
    ema_.tick();
    if (ema_.should_blend()) { ema_.blend(slow_.w.data(), fast_.w.data(), fast_.w.size()); ++tel_[kBlends]; }
  }

  enum { kOutcomes, kAppends, kCredited, kNonzero, kSkipNoWeights, kSkipBadShape, kInvalidSlot, kSgd, kBlends, kNumTel };
  void telemetry(uint64_t* out9, float* last_credit) const {
    for (int i = 0; i < kNumTel; ++i) out9[i] = tel_[i];
    *last_credit = last_credit_;
  }

 private:
  // loss = -credit * logit  (raise the logit of actions that paid off)
  void accumulate(const HistoryEntry& e, const std::vector<float>& ng, const std::vector<float>& ns, float credit) {
    SsmWeights& w = fast_;
    float* g = grad_.data();
    float* gWg = g; float* gWs = gWg + (size_t)w.G * w.F; float* gdg = gWs + (size_t)w.S * w.F;
    float* gds = gdg + w.G; float* gog = gds + w.S; float* gos = gog + w.G; float* gb = gos + w.S;
    const float c = -credit;
    for (int i = 0; i < w.G; ++i) {
      const float up = c * w.og()[i];
      for (int k = 0; k < w.F; ++k) gWg[(size_t)i * w.F + k] += up * e.f[k];
      gdg[i] += up * e.g[i];
      gog[i] += c * ng[i];
    }
    for (int i = 0; i < w.S; ++i) {
      const float up = c * w.os()[i];
      for (int k = 0; k < w.F; ++k) gWs[(size_t)i * w.F + k] += up * e.f[k];
      gds[i] += up * e.s[i];
      gos[i] += c * ns[i];
    }
    *gb += c;
  }

  uint32_t slots_, max_entries_;
  float gamma_, gerber_c_, lr_;
  uint32_t sgd_interval_, since_sgd_ = 0;
  FastSlowEma ema_;
  RollingStddev reward_stats_{0.99f};
  bool init_ = false;
  SsmWeights fast_, slow_;
  std::vector<float> grad_;
  std::vector<std::deque<HistoryEntry>> hist_;
  std::vector<uint8_t> evicted_;
  std::vector<uint64_t> evicted_at_;
  uint64_t tel_[kNumTel] = {};
  float last_credit_ = 0.f;
};

}  // namespace

extern "C" {

// ---- scheduler ----------------------------------------------------------------------
void* ccbc_arm_sched_new(uint32_t streams, uint32_t chunk, uint32_t ttl, uint32_t max_frames) {
  return new ArmScheduler(streams, chunk, ttl, max_frames);
}
void ccbc_arm_sched_free(void* s) { delete static_cast<ArmScheduler*>(s); }
int ccbc_arm_sched_ingest(void* s, uint64_t frame_id, uint64_t step, uint32_t stream, uint64_t cutoff) {
  return static_cast<ArmScheduler*>(s)->ingest(frame_id, step, stream, cutoff) ? 1 : 0;
}
int ccbc_arm_sched_next_job(void* s, uint64_t step, const uint64_t* visible, int n_visible, void* job168) {
  return static_cast<ArmScheduler*>(s)->next_job(step, visible, n_visible, static_cast<wire::ArmMaintenanceJob*>(job168));
}
void ccbc_arm_sched_record(void* s, const void* result192) {
  static_cast<ArmScheduler*>(s)->record(*static_cast<const wire::ArmMaintenanceResult*>(result192));
}
// counters17: 16 counters in the order of the enum + current queue depth; seconds4: probe, oracle, cpu, max frame age
void ccbc_arm_sched_diag(void* s, uint64_t* counters17, double* seconds4) {
  static_cast<ArmScheduler*>(s)->diagnostics(counters17, seconds4);
}

// ---- fused CPU RMSNorm -> LM head -> NLL ----------------------------------------------
void* ccbc_lmhead_pack(const float* norm_w, const uint16_t* W_bf16, int V, int D) {
  auto* h = new LmHead();
  pack_lm_head(norm_w, W_bf16, V, D, h);
  return h;
}
void ccbc_lmhead_free(void* h) { delete static_cast<LmHead*>(h); }
int ccbc_rms_lmhead_nll_mode(void* h, const uint16_t* hidden_bf16, const int64_t* targets, int T, float eps,
                             float* nll, int mode) {
  return rms_lmhead_nll_mode(*static_cast<LmHead*>(h), hidden_bf16, targets, T, eps, nll, mode);
}
int ccbc_rms_lmhead_nll(void* h, const uint16_t* hidden_bf16, const int64_t* targets, int T, float eps, float* nll) {
  return rms_lmhead_nll(*static_cast<LmHead*>(h), hidden_bf16, targets, T, eps, nll);
}

// ---- evidence engine ------------------------------------------------------------------
void* ccbc_evidence_new(uint32_t lanes, uint32_t d_model) { return new EvidenceEngine(lanes, d_model); }
void ccbc_evidence_free(void* e) { delete static_cast<EvidenceEngine*>(e); }
void ccbc_evidence_set_lm_head(void* e, const float* norm_w, const uint16_t* W_bf16, int V) {
  static_cast<EvidenceEngine*>(e)->set_lm_head(norm_w, W_bf16, V);
}
int ccbc_evidence_ingest(void* e, const uint16_t* cue_hidden, const int32_t* cue_targets, uint64_t frame_id,
                         uint64_t step, uint32_t stream) {
  return static_cast<EvidenceEngine*>(e)->ingest(cue_hidden, cue_targets, frame_id, step, stream);
}
void ccbc_evidence_shutdown(void* e) { static_cast<EvidenceEngine*>(e)->shutdown(); }
void ccbc_evidence_diag(void* e, uint64_t* u8, double* f7, uint64_t* lane_adv, uint64_t* lane_work, double* lane_secs) {
  static_cast<EvidenceEngine*>(e)->diagnostics(u8, f7, lane_adv, lane_work, lane_secs);
}

// ---- per-slot SSM controller ----------------------------------------------------------
int64_t ccbc_ssm_flat_size(int F, int G, int S) { SsmWeights w; w.F = F; w.G = G; w.S = S; return (int64_t)w.size(); }
// one controller step with explicit weights (flat layout of SsmWeights); returns the logit
float ccbc_ssm_forward_step(int F, int G, int S, const float* flat, const float* f, const float* g, const float* s,
                            float* new_g, float* new_s) {
  SsmWeights w; w.F = F; w.G = G; w.S = S;
  w.w.assign(flat, flat + w.size());
  return ssm_forward(w, f, g, s, new_g, new_s);
}
void* ccbc_ssm_learner_new(uint32_t slots, uint32_t max_entries, float gamma, float gerber_c, float lr,
                           uint32_t sgd_interval, float ema_alpha, uint64_t ema_interval) {
  return new SlotSsmLearner(slots, max_entries, gamma, gerber_c, lr, sgd_interval, ema_alpha, ema_interval);
}
void ccbc_ssm_learner_free(void* l) { delete static_cast<SlotSsmLearner*>(l); }
int ccbc_ssm_learner_init(void* l, int F, int G, int S, const float* flat) {
  return static_cast<SlotSsmLearner*>(l)->init(F, G, S, flat);
}
int ccbc_ssm_learner_record(void* l, uint32_t slot, uint64_t gpu_step, uint32_t policy_version, float logit,
                            uint8_t rank, const float* f, int nf, const float* g, int ng, const float* s, int ns) {
  HistoryEntry e;
  e.gpu_step = gpu_step; e.policy_version = policy_version; e.logit = logit; e.rank = rank;
  e.f.assign(f, f + nf); e.g.assign(g, g + ng); e.s.assign(s, s + ns);
  return static_cast<SlotSsmLearner*>(l)->record(slot, std::move(e));
}
void ccbc_ssm_learner_outcome(void* l, const void* replay_outcome_96b) {
  static_cast<SlotSsmLearner*>(l)->on_replay_outcome(*static_cast<const wire::ReplayOutcome*>(replay_outcome_96b));
}
int ccbc_ssm_learner_weights(void* l, int slow, float* flat_out) {
  auto* L = static_cast<SlotSsmLearner*>(l);
  if (!L->initialized()) return -1;
  const auto& w = slow ? L->slow() : L->fast();
  std::memcpy(flat_out, w.w.data(), w.w.size() * sizeof(float));
  return 0;
}
void ccbc_ssm_learner_telemetry(void* l, uint64_t* out9, float* last_credit) {
  static_cast<SlotSsmLearner*>(l)->telemetry(out9, last_credit);
}
int64_t ccbc_ssm_learner_history_size(void* l, uint32_t slot) { return (int64_t)static_cast<SlotSsmLearner*>(l)->history_size(slot); }
void ccbc_ssm_learner_mark_evicted(void* l, uint32_t slot, uint64_t at) { static_cast<SlotSsmLearner*>(l)->mark_evicted(slot, at); }
int ccbc_ssm_learner_is_evicted(void* l, uint32_t slot) { return static_cast<SlotSsmLearner*>(l)->is_evicted(slot) ? 1 : 0; }
void ccbc_ssm_learner_gc(void* l, uint64_t now, uint64_t lookahead) { static_cast<SlotSsmLearner*>(l)->gc(now, lookahead); }

}  // extern "C"
