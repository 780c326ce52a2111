// C ABI of libccb200_ctrl.so (bound from Python with ctypes).
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "control.h"
#include "ring.h"
#include "wire_format.h"

using namespace ccb;
using namespace ccb::ctrl;

namespace ccb::ctrl {
struct CpuFeatures { bool avx2, avx512f, amx_tile, amx_bf16, amx_enabled; };
const CpuFeatures& cpu_features();
void matvec(const float*, const float*, float*, int, int);
void matvec_scalar(const float*, const float*, float*, int, int);
void diag_step(const float*, const float*, float*, int);
void diag_step_scalar(const float*, const float*, float*, int);
int bf16_matmul(const uint16_t*, const uint16_t*, float*, int, int, int);
void bf16_matmul_scalar(const uint16_t*, const uint16_t*, float*, int, int, int);
}  // namespace ccb::ctrl

static thread_local std::string g_err;
static int fail(const std::string& m) { g_err = m; return -1; }

struct RingHandle {
  RingView view;
  ShmRegion shm;        // empty for process-local rings
  void* local = nullptr;
};

extern "C" {

const char* ccbc_last_error() { return g_err.c_str(); }

// kind: 0 TensorSlice, 1 WriteEvent, 2 QueryEvent, 3 ReplayOutcome, 4 ArmMaintenanceJob,
// 5 ArmMaintenanceResult, 6 TeacherRequest, 7 TeacherResult, 8 WeightSnapshotHeader
int64_t ccbc_wire_sizeof(int kind) {
  switch (kind) {
    case 0: return sizeof(wire::TensorSlice);
    case 1: return sizeof(wire::WriteEvent);
    case 2: return sizeof(wire::QueryEvent);
    case 3: return sizeof(wire::ReplayOutcome);
    case 4: return sizeof(wire::ArmMaintenanceJob);
    case 5: return sizeof(wire::ArmMaintenanceResult);
    case 6: return sizeof(wire::TeacherRequest);
    case 7: return sizeof(wire::TeacherResult);
    case 8: return sizeof(wire::WeightSnapshotHeader);
    default: return -1;
  }
}
int64_t ccbc_ring_capacity(int kind) {
  switch (kind) {
    case 1: return wire::kWriteRingCapacity;
    case 2: return wire::kQueryRingCapacity;
    case 3: return wire::kReplayRingCapacity;
    default: return -1;
  }
}

// ---- rings -------------------------------------------------------------------
void* ccbc_ring_create_local(int64_t elem_bytes, int64_t capacity) {
  if (!RingView::valid_capacity((size_t)capacity) || elem_bytes <= 0) {
    fail("ring capacity must be a power of two and element size positive");
    return nullptr;
  }
  auto* h = new RingHandle();
  const size_t bytes = RingView::region_bytes((size_t)elem_bytes, (size_t)capacity);
  if (posix_memalign(&h->local, kCacheLine, bytes) != 0) { delete h; fail("out of memory"); return nullptr; }
  std::memset(h->local, 0, bytes);
  h->view.bind(h->local, (size_t)elem_bytes, (size_t)capacity, true);
  return h;
}
void* ccbc_ring_open_shm(const char* name, int64_t elem_bytes, int64_t capacity, int create) {
  if (!RingView::valid_capacity((size_t)capacity) || elem_bytes <= 0) {
    fail("ring capacity must be a power of two and element size positive");
    return nullptr;
  }
  auto* h = new RingHandle();
  const size_t bytes = RingView::region_bytes((size_t)elem_bytes, (size_t)capacity);
  std::string e = h->shm.open(name, create ? bytes : 0, create != 0);
  if (!e.empty()) { delete h; fail(e); return nullptr; }
  if (h->shm.size() < bytes) { delete h; fail("shm segment smaller than the ring it should hold"); return nullptr; }
  h->view.bind(h->shm.ptr(), (size_t)elem_bytes, (size_t)capacity, create != 0);
  return h;
}
int ccbc_ring_push(void* hv, const void* item) { return static_cast<RingHandle*>(hv)->view.push(item) ? 1 : 0; }
int ccbc_ring_pop(void* hv, void* out) { return static_cast<RingHandle*>(hv)->view.pop(out) ? 1 : 0; }
int64_t ccbc_ring_size(void* hv) { return (int64_t)static_cast<RingHandle*>(hv)->view.size(); }
void ccbc_ring_close(void* hv) {
  auto* h = static_cast<RingHandle*>(hv);
  if (h->local) free(h->local);
  delete h;
}
int ccbc_shm_unlink(const char* name) { return ShmRegion::unlink(name) ? 0 : -1; }

// plain shm byte region (exit flags, stats)
void* ccbc_shm_open(const char* name, int64_t size, int create) {
  auto* r = new ShmRegion();
  std::string e = r->open(name, (size_t)size, create != 0);
  if (!e.empty()) { delete r; fail(e); return nullptr; }
  if (create) std::memset(r->ptr(), 0, r->size());
  return r;
}
void* ccbc_shm_ptr(void* r) { return static_cast<ShmRegion*>(r)->ptr(); }
int64_t ccbc_shm_size(void* r) { return (int64_t)static_cast<ShmRegion*>(r)->size(); }
void ccbc_shm_close(void* r) { delete static_cast<ShmRegion*>(r); }

// ---- credit / stats ------------------------------------------------------------
float ccbc_recency_decay(float reward, uint64_t t, uint64_t p, float gamma) { return recency_decay(reward, t, p, gamma); }
float ccbc_gerber_weight(float a, float b, float h) { return gerber_weight(a, b, h); }
void* ccbc_rolling_new(float decay) { return new RollingStddev(decay); }
void ccbc_rolling_update(void* r, float x) { static_cast<RollingStddev*>(r)->update(x); }
float ccbc_rolling_mean(void* r) { return static_cast<RollingStddev*>(r)->mean(); }
float ccbc_rolling_std(void* r) { return static_cast<RollingStddev*>(r)->stddev(); }
void ccbc_rolling_free(void* r) { delete static_cast<RollingStddev*>(r); }
void ccbc_sgd_apply(float* w, const float* g, int64_t n, float lr) { SgdStep{lr}.apply(w, g, (size_t)n); }
void ccbc_ema_blend(float* slow, const float* fast, int64_t n, float alpha) { FastSlowEma(alpha, 1).blend(slow, fast, (size_t)n); }

// ---- simplex policy ------------------------------------------------------------
static SimplexWeights make_weights(int N, int Kv, int Ks, int H, float temperature, const float* flat) {
  SimplexWeights w;
  w.N = N; w.K_v = Kv; w.K_s = Ks; w.H = H; w.temperature = temperature;
  w.W_vp.resize((size_t)Kv * H); w.b_vp.resize(H); w.W_lh.resize(H); w.W_sb.resize(Ks);
  if (flat) w.from_flat(flat);
  return w;
}
int64_t ccbc_simplex_flat_size(int Kv, int Ks, int H) { return (int64_t)Kv * H + H + H + 1 + Ks + 1; }
int ccbc_simplex_forward(int N, int Kv, int Ks, int H, float temperature, const float* flat,
                         const float* V, const float* E, const float* feats, float* p_out,
                         float* logits_out) {
  SimplexWeights w = make_weights(N, Kv, Ks, H, temperature, flat);
  std::string e = w.validate();
  if (!e.empty()) return fail(e);
  SimplexForward f = simplex_forward(w, V, E, feats);
  std::memcpy(p_out, f.p.data(), sizeof(float) * N);
  if (logits_out) std::memcpy(logits_out, f.logits.data(), sizeof(float) * N);
  return 0;
}
int ccbc_simplex_grad(int N, int Kv, int Ks, int H, float temperature, const float* flat,
                      const float* V, const float* E, const float* feats, int chosen, float advantage,
                      float entropy_beta, float* grad_out) {
  SimplexWeights w = make_weights(N, Kv, Ks, H, temperature, flat);
  std::string e = w.validate();
  if (!e.empty()) return fail(e);
  SimplexForward f = simplex_forward(w, V, E, feats);
  std::memset(grad_out, 0, sizeof(float) * w.flat_size());
  simplex_backward(w, f, V, E, feats, (uint32_t)chosen, advantage, entropy_beta, grad_out);
  return 0;
}

// Extended policy: K_e edge features per pair, n_heads residual attention heads, a stored bucket
// embedding.  With n_heads == n_buckets == 0 and K_e == 1 the flat layout equals the base one.
static SimplexWeights make_weights_ex(int N, int Kv, int Ke, int Ks, int H, int n_heads, int n_buckets,
                                      int embed_dim, float temperature, const float* flat) {
  SimplexWeights w;
  w.N = N; w.K_v = Kv; w.K_e = Ke; w.K_s = Ks; w.H = H; w.temperature = temperature;
  w.n_heads = n_heads; w.n_buckets = n_buckets; w.embed_dim = embed_dim;
  w.resize();
  if (flat) w.from_flat(flat);
  return w;
}
int64_t ccbc_simplex_flat_size_ex(int Kv, int Ke, int Ks, int H, int n_heads, int n_buckets, int embed_dim) {
  return (int64_t)make_weights_ex(1, Kv, Ke, Ks, H, n_heads, n_buckets, embed_dim, 1.f, nullptr).flat_size();
}
int ccbc_simplex_forward_ex(int N, int Kv, int Ke, int Ks, int H, int n_heads, int n_buckets, int embed_dim,
                            float temperature, const float* flat, const float* V, const float* E,
                            const float* feats, float* p_out, float* logits_out, float* logits_hxh_out) {
  SimplexWeights w = make_weights_ex(N, Kv, Ke, Ks, H, n_heads, n_buckets, embed_dim, temperature, flat);
  std::string e = w.validate();
  if (!e.empty()) return fail(e);
  SimplexForward f = simplex_forward(w, V, E, feats);
  std::memcpy(p_out, f.p.data(), sizeof(float) * N);
  if (logits_out) std::memcpy(logits_out, f.logits.data(), sizeof(float) * N);
  if (logits_hxh_out) std::memcpy(logits_hxh_out, f.logits_hxh.data(), sizeof(float) * N);
  return 0;
}
int ccbc_simplex_grad_ex(int N, int Kv, int Ke, int Ks, int H, int n_heads, int n_buckets, int embed_dim,
                         float temperature, const float* flat, const float* V, const float* E,
                         const float* feats, int chosen, float advantage, float entropy_beta, float* grad_out) {
  SimplexWeights w = make_weights_ex(N, Kv, Ke, Ks, H, n_heads, n_buckets, embed_dim, temperature, flat);
  std::string e = w.validate();
  if (!e.empty()) return fail(e);
  SimplexForward f = simplex_forward(w, V, E, feats);
  std::memset(grad_out, 0, sizeof(float) * w.flat_size());
  simplex_backward(w, f, V, E, feats, (uint32_t)chosen, advantage, entropy_beta, grad_out);
  return 0;
}
// Offline-pretrained controller trunk: logits [B, Ds] and value [B] from features [B, F].
int ccbc_forward_pretrain_model(int B, int F, int Dg, int L, int Ds, const float* x, const float* in_w,
                                const float* in_b, const float* decay, const float* w_in, const float* w_out,
                                const float* bias, const float* pol_w, const float* pol_b, const float* val_w,
                                const float* val_b, float* logits_out, float* value_out) {
  if (B <= 0 || F <= 0 || Dg <= 0 || L < 0 || Ds <= 0) return fail("forward_pretrain_model: bad dims");
  PretrainModel m;
  m.F = F; m.Dg = Dg; m.L = L; m.Ds = Ds;
  m.in_w = in_w; m.in_b = in_b; m.decay = decay; m.w_in = w_in; m.w_out = w_out; m.bias = bias;
  m.pol_w = pol_w; m.pol_b = pol_b; m.val_w = val_w; m.val_b = val_b;
  forward_pretrain_model(m, x, (size_t)B, logits_out, value_out);
  return 0;
}
int ccbc_learner_init_ex(void* l, int N, int Kv, int Ke, int Ks, int H, int n_heads, int n_buckets, int embed_dim,
                         float temperature, const float* flat) {
  SimplexWeights w = make_weights_ex(N, Kv, Ke, Ks, H, n_heads, n_buckets, embed_dim, temperature, flat);
  std::string e = w.validate();
  if (!e.empty()) return fail(e);
  static_cast<SimplexOnlineLearner*>(l)->initialize(w);
  return 0;
}

// ---- online learner ------------------------------------------------------------
void* ccbc_learner_new(int num_slots, int max_entries, float gamma, float lr, int sgd_interval,
                       float ema_alpha, int64_t ema_interval, float gerber_c, float entropy_beta) {
  return new SimplexOnlineLearner(num_slots, max_entries, gamma, lr, sgd_interval, ema_alpha,
                                  (uint64_t)ema_interval, gerber_c, entropy_beta);
}
void ccbc_learner_free(void* l) { delete static_cast<SimplexOnlineLearner*>(l); }
int ccbc_learner_init(void* l, int N, int Kv, int Ks, int H, float temperature, const float* flat) {
  SimplexWeights w = make_weights(N, Kv, Ks, H, temperature, flat);
  std::string e = w.validate();
  if (!e.empty()) return fail(e);
  static_cast<SimplexOnlineLearner*>(l)->initialize(w);
  return 0;
}
int ccbc_learner_record(void* l, uint64_t slot, uint64_t gpu_step, int chosen, float p_chosen,
                        const float* V, const float* E, const float* feats) {
  auto* L = static_cast<SimplexOnlineLearner*>(l);
  if (!L->initialized()) return fail("learner weights not initialised");
  const SimplexWeights& w = L->fast();
  ActionRecord r;
  r.gpu_step = gpu_step; r.chosen = (uint32_t)chosen; r.p_chosen = p_chosen;
  r.V.assign(V, V + (size_t)w.N * w.K_v);
  r.E.assign(E, E + (size_t)w.N * w.N);
  r.feats.assign(feats, feats + w.K_s);
  L->record_decision(slot, std::move(r));
  return 0;
}
int ccbc_learner_outcome(void* l, const void* replay_outcome_96b) {
  wire::ReplayOutcome ev;
  std::memcpy(&ev, replay_outcome_96b, sizeof(ev));
  static_cast<SimplexOnlineLearner*>(l)->on_replay_outcome(ev);
  return 0;
}
int ccbc_learner_weights(void* l, int slow, float* flat_out) {
  auto* L = static_cast<SimplexOnlineLearner*>(l);
  if (!L->initialized()) return fail("learner weights not initialised");
  (slow ? L->slow() : L->fast()).to_flat(flat_out);
  return 0;
}
// out: replay_outcomes, history_appends, credited, gerber_accepted, gerber_rejected,
//      skipped_missing_state, invalid_slot_skips, sgd_steps, ema_blends
void ccbc_learner_telemetry(void* l, uint64_t* out9, float* out5) {
  const LearnerTelemetry& t = static_cast<SimplexOnlineLearner*>(l)->telemetry();
  const uint64_t v[9] = {t.replay_outcomes, t.history_appends, t.credited_actions, t.gerber_accepted,
                         t.gerber_rejected, t.skipped_missing_state, t.invalid_slot_skips, t.sgd_steps,
                         t.ema_blends};
  std::memcpy(out9, v, sizeof(v));
  const float f[5] = {t.last_advantage_raw, t.last_advantage_standardized, t.last_gerber_weight,
                      t.last_entropy, t.last_grad_l2};
  std::memcpy(out5, f, sizeof(f));
}
int64_t ccbc_learner_history_size(void* l, int slot) { return (int64_t)static_cast<SimplexOnlineLearner*>(l)->history_size((uint32_t)slot); }
void ccbc_learner_set_trace(void* l, const char* path) { static_cast<SimplexOnlineLearner*>(l)->set_trace_path(path ? path : ""); }

// ---- CSWG ----------------------------------------------------------------------
// header_out: version, n_layers, d_global, d_slot, feature_dim, dtype.  Returns the
// payload length; call again with a buffer of that many floats to receive it.
int64_t ccbc_cswg_load(const char* path, uint32_t* header_out, float* payload_out, int64_t capacity) {
  CswgFile f;
  std::string e = load_cswg(path, &f);
  if (!e.empty()) return fail(e);
  const uint32_t h[6] = {f.version, f.n_layers, f.d_global, f.d_slot, f.feature_dim, f.dtype};
  std::memcpy(header_out, h, sizeof(h));
  if (payload_out && capacity >= (int64_t)f.payload.size())
    std::memcpy(payload_out, f.payload.data(), f.payload.size() * sizeof(float));
  return (int64_t)f.payload.size();
}
float ccbc_half_to_float(uint16_t h) { return half_to_float(h); }
uint16_t ccbc_float_to_half(float f) { return float_to_half(f); }

// ---- controller loop -----------------------------------------------------------
// write_rings: '\n'-separated names.  Blocks until the exit flag byte is set.
int64_t ccbc_controller_main(const char* write_rings, const char* query_ring, const char* replay_ring,
                             const char* exit_flag, const char* stats_shm, void* learner,
                             uint64_t* counts3) {
  std::vector<std::string> names;
  std::string cur;
  for (const char* p = write_rings; p && *p; ++p) {
    if (*p == '\n') { if (!cur.empty()) names.push_back(cur); cur.clear(); }
    else cur.push_back(*p);
  }
  if (!cur.empty()) names.push_back(cur);
  ControllerCounts c;
  std::string err;
  const uint64_t total = controller_main(names, query_ring, replay_ring, exit_flag,
                                         stats_shm ? stats_shm : "",
                                         static_cast<SimplexOnlineLearner*>(learner), &c, &err);
  if (!err.empty()) return fail(err);
  if (counts3) { counts3[0] = c.writes; counts3[1] = c.queries; counts3[2] = c.replays; }
  return (int64_t)total;
}

// ---- CPU math --------------------------------------------------------------------
// out5: avx2, avx512f, amx_tile, amx_bf16, amx_enabled
void ccbc_cpu_features(int* out5) {
  const auto& f = cpu_features();
  out5[0] = f.avx2; out5[1] = f.avx512f; out5[2] = f.amx_tile; out5[3] = f.amx_bf16; out5[4] = f.amx_enabled;
}
void ccbc_matvec(const float* W, const float* x, float* y, int rows, int cols, int force_scalar) {
  if (force_scalar) matvec_scalar(W, x, y, rows, cols); else matvec(W, x, y, rows, cols);
}
void ccbc_diag_step(const float* decay, const float* x, float* h, int n, int force_scalar) {
  if (force_scalar) diag_step_scalar(decay, x, h, n); else diag_step(decay, x, h, n);
}
int ccbc_bf16_matmul(const uint16_t* A, const uint16_t* B, float* C, int M, int N, int K, int force_scalar) {
  if (force_scalar) { bf16_matmul_scalar(A, B, C, M, N, K); return 0; }
  return bf16_matmul(A, B, C, M, N, K);
}

}  // extern "C"
