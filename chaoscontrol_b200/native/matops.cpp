// Vectorised CPU math for the controller: AVX-512 matvec / diagonal recurrence
// and an AMX-BF16 tiled matmul, each selected at run time and each with a
// portable scalar twin that defines the expected result.  (Reference:
// kernels/_cpu_ssm_controller/src/avx512_matops.cpp, avx512_recurrence.cpp,
// amx_matmul.cpp:231-381, cpu_features.cpp.)
#include <cpuid.h>
#include <immintrin.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <vector>

namespace ccb::ctrl {

struct CpuFeatures { bool avx2, avx512f, amx_tile, amx_bf16, amx_enabled; };

static bool request_amx_permission() {
#if defined(__linux__)
  constexpr int ARCH_REQ_XCOMP_PERM = 0x1023, XFEATURE_XTILEDATA = 18;
  return syscall(SYS_arch_prctl, ARCH_REQ_XCOMP_PERM, XFEATURE_XTILEDATA) == 0;
#else
  return false;
#endif
}

const CpuFeatures& cpu_features() {
  static const CpuFeatures f = [] {
    CpuFeatures r{};
    unsigned a, b, c, d;
    if (__get_cpuid_count(7, 0, &a, &b, &c, &d)) {
      r.avx2 = (b >> 5) & 1;
      r.avx512f = (b >> 16) & 1;
      r.amx_bf16 = (d >> 22) & 1;
      r.amx_tile = (d >> 24) & 1;
    }
    r.amx_enabled = r.amx_tile && r.amx_bf16 && request_amx_permission();
    return r;
  }();
  return f;
}

// ---- matvec: y[r] = sum_c W[r, c] * x[c] ------------------------------------
void matvec_scalar(const float* W, const float* x, float* y, int rows, int cols) {
  for (int r = 0; r < rows; ++r) {
    float acc = 0.f;
    for (int c = 0; c < cols; ++c) acc += W[(size_t)r * cols + c] * x[c];
    y[r] = acc;
  }
}
__attribute__((target("avx512f"))) static void matvec_avx512(const float* W, const float* x, float* y,
                                                             int rows, int cols) {
  for (int r = 0; r < rows; ++r) {
    const float* w = W + (size_t)r * cols;
    __m512 acc = _mm512_setzero_ps();
    int c = 0;
    for (; c + 16 <= cols; c += 16)
      acc = _mm512_fmadd_ps(_mm512_loadu_ps(w + c), _mm512_loadu_ps(x + c), acc);
    float s = _mm512_reduce_add_ps(acc);
    for (; c < cols; ++c) s += w[c] * x[c];
    y[r] = s;
  }
}
void matvec(const float* W, const float* x, float* y, int rows, int cols) {
  if (cpu_features().avx512f) matvec_avx512(W, x, y, rows, cols);
  else matvec_scalar(W, x, y, rows, cols);
}

// ---- diagonal recurrence step: h = decay * h + x ----------------------------
void diag_step_scalar(const float* decay, const float* x, float* h, int n) {
  for (int i = 0; i < n; ++i) h[i] = decay[i] * h[i] + x[i];
}
__attribute__((target("avx512f"))) static void diag_step_avx512(const float* decay, const float* x,
                                                                float* h, int n) {
  int i = 0;
  for (; i + 16 <= n; i += 16)
    _mm512_storeu_ps(h + i, _mm512_fmadd_ps(_mm512_loadu_ps(decay + i), _mm512_loadu_ps(h + i),
                                            _mm512_loadu_ps(x + i)));
  for (; i < n; ++i) h[i] = decay[i] * h[i] + x[i];
}
void diag_step(const float* decay, const float* x, float* h, int n) {
  if (cpu_features().avx512f) diag_step_avx512(decay, x, h, n);
  else diag_step_scalar(decay, x, h, n);
}

// ---- bf16 matmul: C[M,N] (fp32) = A[M,K] (bf16) * B[K,N] (bf16) -------------
static inline float bf16_to_f32(uint16_t v) {
  uint32_t b = (uint32_t)v << 16;
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}
void bf16_matmul_scalar(const uint16_t* A, const uint16_t* B, float* C, int M, int N, int K) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float acc = 0.f;
      for (int k = 0; k < K; ++k) acc += bf16_to_f32(A[(size_t)m * K + k]) * bf16_to_f32(B[(size_t)k * N + n]);
      C[(size_t)m * N + n] = acc;
    }
}

struct alignas(64) TileConfig {
  uint8_t palette = 1, start_row = 0, reserved[14] = {};
  uint16_t colsb[16] = {};
  uint8_t rows[16] = {};
};

// 16x16 output tiles, K consumed 32 bf16 at a time; B repacked to the VNNI
// layout (pairs of K rows interleaved) that tdpbf16ps expects.
__attribute__((target("amx-tile,amx-bf16,avx512f"))) static void bf16_matmul_amx(
    const uint16_t* A, const uint16_t* B, float* C, int M, int N, int K) {
  TileConfig cfg;
  cfg.rows[0] = 16; cfg.colsb[0] = 64;   // C tile: 16 x 16 fp32
  cfg.rows[1] = 16; cfg.colsb[1] = 64;   // A tile: 16 x 32 bf16
  cfg.rows[2] = 16; cfg.colsb[2] = 64;   // B tile (VNNI): 16 x (16 pairs)
  _tile_loadconfig(&cfg);
  alignas(64) uint16_t a_tile[16 * 32];
  alignas(64) uint16_t b_tile[16 * 32];
  alignas(64) float c_tile[16 * 16];
  for (int m0 = 0; m0 < M; m0 += 16) {
    for (int n0 = 0; n0 < N; n0 += 16) {
      _tile_zero(0);
      for (int k0 = 0; k0 < K; k0 += 32) {
        std::memset(a_tile, 0, sizeof(a_tile));
        std::memset(b_tile, 0, sizeof(b_tile));
        for (int i = 0; i < 16 && m0 + i < M; ++i)
          for (int k = 0; k < 32 && k0 + k < K; ++k) a_tile[i * 32 + k] = A[(size_t)(m0 + i) * K + k0 + k];
        for (int kp = 0; kp < 16; ++kp)
          for (int j = 0; j < 16 && n0 + j < N; ++j)
            for (int t = 0; t < 2; ++t) {
              const int k = k0 + 2 * kp + t;
              if (k < K) b_tile[kp * 32 + 2 * j + t] = B[(size_t)k * N + n0 + j];
            }
        _tile_loadd(1, a_tile, 64);
        _tile_loadd(2, b_tile, 64);
        _tile_dpbf16ps(0, 1, 2);
      }
      _tile_stored(0, c_tile, 64);
      for (int i = 0; i < 16 && m0 + i < M; ++i)
        for (int j = 0; j < 16 && n0 + j < N; ++j) C[(size_t)(m0 + i) * N + n0 + j] = c_tile[i * 16 + j];
    }
  }
  _tile_release();
}

// ---- VNNI-packed weight cache + fused logits / online log-sum-exp on AMX -------------------------
// (Reference: amx_matmul.cpp:231-251 packs the LM-head weight once, :384-624 fuses RMSNorm -> head ->
// NLL over it.)  The head weight W [V, D] is the B operand W^T of logits = xn @ W^T.  tdpbf16ps wants
// B tiles of 16 K-pairs x 16 columns with the two K values of a pair interleaved; packing it per call
// costs more than the tile multiply, so it is done ONCE per weight:
//   packed[((nt * kblocks + kb) * 16 + kp) * 32 + 2 * j + t] = W[(16 nt + j) * D + 32 kb + 2 kp + t]
// (zero past V or D).  A tiles are loaded straight from the normalised activations with their row
// stride, so the hot loop is two tile loads and one tdpbf16ps per 16 x 16 x 32 block; each finished
// 16-token x 16-vocabulary tile updates the tokens' running (max, sum) and picks up target logits.
void pack_vnni_wt(const uint16_t* W, int V, int D, std::vector<uint16_t>* out) {
  const int ntiles = (V + 15) / 16, kblocks = (D + 31) / 32;
  out->assign((size_t)ntiles * kblocks * 512, 0);
  for (int nt = 0; nt < ntiles; ++nt)
    for (int kb = 0; kb < kblocks; ++kb) {
      uint16_t* tile = out->data() + ((size_t)nt * kblocks + kb) * 512;
      for (int kp = 0; kp < 16; ++kp)
        for (int j = 0; j < 16; ++j)
          for (int t = 0; t < 2; ++t) {
            const int v = nt * 16 + j, k = kb * 32 + 2 * kp + t;
            if (v < V && k < D) tile[kp * 32 + 2 * j + t] = W[(size_t)v * D + k];
          }
    }
}

// xn: [Tpad, Dpad] bf16, Tpad a multiple of 16 and Dpad of 32 (zero padded).  run_m / run_s / tgt: [T].
__attribute__((target("amx-tile,amx-bf16,avx512f"))) static void lse_over_vnni_amx(
    const uint16_t* xn, int T, int Tpad, int Dpad, const uint16_t* packed, int V, const int64_t* targets,
    float* run_m, float* run_s, float* tgt) {
  TileConfig cfg;
  cfg.rows[0] = 16; cfg.colsb[0] = 64;
  cfg.rows[1] = 16; cfg.colsb[1] = 64;
  cfg.rows[2] = 16; cfg.colsb[2] = 64;
  _tile_loadconfig(&cfg);
  const int ntiles = (V + 15) / 16, kblocks = Dpad / 32;
  alignas(64) float c_tile[16 * 16];
  for (int m0 = 0; m0 < Tpad; m0 += 16) {
    for (int nt = 0; nt < ntiles; ++nt) {
      _tile_zero(0);
      const uint16_t* bt = packed + (size_t)nt * kblocks * 512;
      for (int kb = 0; kb < kblocks; ++kb) {
        _tile_loadd(1, xn + (size_t)m0 * Dpad + kb * 32, Dpad * 2);
        _tile_loadd(2, bt + (size_t)kb * 512, 64);
        _tile_dpbf16ps(0, 1, 2);
      }
      _tile_stored(0, c_tile, 64);
      const int v0 = nt * 16, nv = V - v0 < 16 ? V - v0 : 16;
      for (int i = 0; i < 16 && m0 + i < T; ++i) {
        const int t = m0 + i;
        const float* row = c_tile + i * 16;
        float m = run_m[t];
        for (int j = 0; j < nv; ++j) m = row[j] > m ? row[j] : m;
        float sum = run_s[t] * __builtin_expf(run_m[t] - m);
        for (int j = 0; j < nv; ++j) sum += __builtin_expf(row[j] - m);
        run_m[t] = m;
        run_s[t] = sum;
        const int64_t y = targets[t];
        if (y >= v0 && y < v0 + nv) tgt[t] = row[y - v0];
      }
    }
  }
  _tile_release();
}

// returns 1 when the AMX path ran (and filled the outputs), 0 when the CPU has no usable AMX
int lse_over_vnni(const uint16_t* xn, int T, int Tpad, int Dpad, const uint16_t* packed, int V,
                  const int64_t* targets, float* run_m, float* run_s, float* tgt) {
  if (!cpu_features().amx_enabled) return 0;
  lse_over_vnni_amx(xn, T, Tpad, Dpad, packed, V, targets, run_m, run_s, tgt);
  return 1;
}

// returns 1 when the AMX path ran, 0 for the scalar path
int bf16_matmul(const uint16_t* A, const uint16_t* B, float* C, int M, int N, int K) {
  if (cpu_features().amx_enabled) {
    bf16_matmul_amx(A, B, C, M, N, K);
    return 1;
  }
  bf16_matmul_scalar(A, B, C, M, N, K);
  return 0;
}

}  // namespace ccb::ctrl
