// Fused diagonal-SSM scan, forward and backward.
//
// Input is the packed projection P[r, 4D] = (select | candidate | gate | delta)
// raw GEMM outputs (bf16), r = b*T + t.  The kernel applies the gate
// nonlinearities, builds decay = exp(-max(softplus(delta), 1e-4) * sigmoid(log_a))
// and update = sigmoid(select) * tanh(candidate), runs the recurrence
//   h[t] = decay[t] * h[t-1] + update[t],   h[-1] = h0 (zero when absent)
// in fp32 registers and emits y = sigmoid(gate) * h.  decay / update / gate are
// never written to memory.  One thread owns two adjacent channels of one batch
// row, so every warp-wide access is a full 128-byte line.
//
// Reference semantics: src/chaoscontrol/core.py:492-507 (_diag_terms),
// core.py:26-32 (recurrence), kernels/_ssm_scan/src/ssm_scan_fwd.cu:103-126 and
// ssm_scan_bwd.cu:104-141 (the unfused serial scan these kernels replace).
// Unlike the reference kernels these take an initial state and return the
// final state, so carried-state evaluation never drops to a per-token loop.
#include "ptx.cuh"
#include <cuda_fp16.h>
#include "ccb_api.h"
#include "runtime.h"

namespace ccb {

constexpr int SCAN_THREADS = 128;

struct Gates {
  float decay, sel, cand, gate, sp_sig, delta;  // sp_sig = d softplus / d raw (0 when clamped)
};

// POLY: the two exponentials run on the FMA pipe (exp_nonpos_fma) instead of the special-function
// unit, which the three tanh and the logarithm of every channel step already keep busy.
template <bool POLY>
__device__ __forceinline__ Gates eval_gates(float s_raw, float c_raw, float g_raw, float d_raw,
                                            float a) {
  Gates g;
  g.sel = sigmoidf_fast(s_raw);
  g.cand = tanhf_fast(c_raw);
  g.gate = sigmoidf_fast(g_raw);
  const float e = POLY ? exp_nonpos_fma(-fabsf(d_raw)) : __expf(-fabsf(d_raw));
  float sp = fmaxf(d_raw, 0.f) + __logf(1.f + e);
  // d softplus / dx = sigmoid(x)
  const float inv1pe = rcpf_fast(1.f + e);
  const float sig = d_raw >= 0.f ? inv1pe : e * inv1pe;
  g.sp_sig = sp > 1e-4f ? sig : 0.f;
  g.delta = fmaxf(sp, 1e-4f);
  g.decay = POLY ? exp_nonpos_fma(-g.delta * a) : __expf(-g.delta * a);
  return g;
}

// ---- packed fp32x2 evaluation ------------------------------------------------------------------
// One thread owns two adjacent channels that go through the same arithmetic, and both kernels are
// bound by instruction issue, not by bytes: sm_100's two-wide fp32 instructions (fma / mul / add on a
// register pair) do each step for both channels at once.  Special-function ops stay one per channel.
__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }
__device__ __forceinline__ float2 f2s(float a) { return make_float2(a, a); }
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2f(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float2 sigmoid2(float2 x) {
  const float2 h = __fmul2_rn(x, f2s(0.5f));
  return __ffma2_rn(f2(tanhf_fast(h.x), tanhf_fast(h.y)), f2s(0.5f), f2s(0.5f));
}

struct Gates2 {
  float2 decay, sel, cand, gate, sp_sig, delta;
};

// nal2e = -sigmoid(log_a) * log2(e), per channel: decay = 2^(delta * nal2e)
template <bool WANT_SIG>
__device__ __forceinline__ Gates2 eval_gates2(float2 s_raw, float2 c_raw, float2 g_raw, float2 d_raw,
                                              float2 nal2e) {
  constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
  Gates2 g;
  g.sel = sigmoid2(s_raw);
  g.cand = f2(tanhf_fast(c_raw.x), tanhf_fast(c_raw.y));
  g.gate = sigmoid2(g_raw);
  const float2 t = __fmul2_rn(f2(-fabsf(d_raw.x), -fabsf(d_raw.y)), f2s(LOG2E));
  const float2 e = f2(ex2f(t.x), ex2f(t.y));
  const float2 ope = __fadd2_rn(e, f2s(1.f));
  const float2 sp = __ffma2_rn(f2(lg2f(ope.x), lg2f(ope.y)), f2s(LN2), f2(fmaxf(d_raw.x, 0.f), fmaxf(d_raw.y, 0.f)));
  if (WANT_SIG) {
    const float2 inv = f2(rcpf_fast(ope.x), rcpf_fast(ope.y));
    const float2 einv = __fmul2_rn(e, inv);
    g.sp_sig = f2(sp.x > 1e-4f ? (d_raw.x >= 0.f ? inv.x : einv.x) : 0.f,
                  sp.y > 1e-4f ? (d_raw.y >= 0.f ? inv.y : einv.y) : 0.f);
  }
  g.delta = f2(fmaxf(sp.x, 1e-4f), fmaxf(sp.y, 1e-4f));
  const float2 u = __fmul2_rn(g.delta, nal2e);
  g.decay = f2(ex2f(u.x), ex2f(u.y));
  return g;
}

// grid: (ceil(D/256), B); block: 128 threads, 2 channels per thread.
// MODE 0: scalar arithmetic; 1: scalar with FMA-pipe exponentials; 2: packed fp32x2 arithmetic.
// U time steps are loaded ahead of their arithmetic; MINB resident blocks per SM bound the registers.
template <int MODE, int U = 8, int MINB = 4>
__global__ void __launch_bounds__(SCAN_THREADS, MINB)
scan_fwd_kernel(const __nv_bfloat16* __restrict__ P, long long ldp, const float* __restrict__ log_a,
                const float* __restrict__ h0, __nv_bfloat16* __restrict__ y,
                __nv_bfloat16* __restrict__ hout, float* __restrict__ hT, int T, int D,
                long long la_bstride) {
  constexpr int SCAN_UNROLL = U;
  const int b = blockIdx.y;
  const int d = (blockIdx.x * SCAN_THREADS + threadIdx.x) * 2;
  if (d >= D) return;
  // la_bstride != 0: every batch row has its own decay vector (per-document test-time training)
  const float a0 = sigmoidf_fast(log_a[b * la_bstride + d]);
  const float a1 = sigmoidf_fast(log_a[b * la_bstride + d + 1]);
  const float2 nal2e = f2(-a0 * 1.4426950408889634f, -a1 * 1.4426950408889634f);
  float s0 = 0.f, s1 = 0.f;
  if (h0 != nullptr) {
    s0 = h0[(long long)b * D + d];
    s1 = h0[(long long)b * D + d + 1];
  }
  const uint32_t* Pw = reinterpret_cast<const uint32_t*>(P + (long long)b * T * ldp + d);
  const long long rowstride = ldp / 2;   // in uint32 units
  const int dq = D / 2;
  uint32_t* yw = reinterpret_cast<uint32_t*>(y + ((long long)b * T) * D + d);
  uint32_t* hw = hout ? reinterpret_cast<uint32_t*>(hout + ((long long)b * T) * D + d) : nullptr;

  for (int t0 = 0; t0 < T; t0 += SCAN_UNROLL) {
    uint32_t raw[SCAN_UNROLL][4];
#pragma unroll
    for (int u = 0; u < SCAN_UNROLL; ++u) {
      if (t0 + u < T) {
        const uint32_t* row = Pw + (long long)(t0 + u) * rowstride;
        raw[u][0] = __ldg(row);
        raw[u][1] = __ldg(row + dq);
        raw[u][2] = __ldg(row + 2 * dq);
        raw[u][3] = __ldg(row + 3 * dq);
      }
    }
#pragma unroll
    for (int u = 0; u < SCAN_UNROLL; ++u) {
      if (t0 + u < T) {
        const float2 sr = unpack_bf16x2(raw[u][0]);
        const float2 cr = unpack_bf16x2(raw[u][1]);
        const float2 gr = unpack_bf16x2(raw[u][2]);
        const float2 dr = unpack_bf16x2(raw[u][3]);
        const long long o = (long long)(t0 + u) * dq;
        if (MODE == 2) {
          const Gates2 g = eval_gates2<false>(sr, cr, gr, dr, nal2e);
          const float2 st = __ffma2_rn(g.decay, f2(s0, s1), __fmul2_rn(g.sel, g.cand));
          s0 = st.x;
          s1 = st.y;
          const float2 yv = __fmul2_rn(g.gate, st);
          yw[o] = pack_bf16x2(yv.x, yv.y);
        } else {
          const Gates g0 = eval_gates<MODE == 1>(sr.x, cr.x, gr.x, dr.x, a0);
          const Gates g1 = eval_gates<MODE == 1>(sr.y, cr.y, gr.y, dr.y, a1);
          s0 = g0.decay * s0 + g0.sel * g0.cand;
          s1 = g1.decay * s1 + g1.sel * g1.cand;
          yw[o] = pack_bf16x2(g0.gate * s0, g1.gate * s1);
        }
        if (hw) hw[o] = pack_bf16x2(s0, s1);
      }
    }
  }
  if (hT != nullptr) {
    hT[(long long)b * D + d] = s0;
    hT[(long long)b * D + d + 1] = s1;
  }
}

// Backward.  Walks t from T-1 down to 0 with the carry dh[t] * decay[t].
// Needs the forward states h (bf16) and the raw projections; recomputes the
// gates.  Emits dP (optionally pre-multiplied by the consumer's RMSNorm row
// scale rs[r] = rsqrt(rowss[r] * inv_dim + eps)), per-batch-row partials of
// d log_a, and optionally d h0.
template <int MODE, int U = 8, int MINB = 4>
__global__ void __launch_bounds__(SCAN_THREADS, MINB)
scan_bwd_kernel(const __nv_bfloat16* __restrict__ P, long long ldp, const float* __restrict__ log_a,
                const float* __restrict__ h0, const __nv_bfloat16* __restrict__ hstates,
                const __nv_bfloat16* __restrict__ dy, const float* __restrict__ dhT,
                const float* __restrict__ rowss, float inv_dim, float eps,
                __nv_bfloat16* __restrict__ dP, long long lddp, float* __restrict__ dloga_part,
                float* __restrict__ dh0, int T, int D, long long la_bstride) {
  constexpr int SCAN_UNROLL = U;
  const int b = blockIdx.y;
  const int d = (blockIdx.x * SCAN_THREADS + threadIdx.x) * 2;
  if (d >= D) return;
  const float a0 = sigmoidf_fast(log_a[b * la_bstride + d]);
  const float a1 = sigmoidf_fast(log_a[b * la_bstride + d + 1]);
  const float2 nal2e = f2(-a0 * 1.4426950408889634f, -a1 * 1.4426950408889634f);
  const long long rowbase = (long long)b * T;
  const int dq = D / 2;
  const uint32_t* Pw = reinterpret_cast<const uint32_t*>(P + rowbase * ldp + d);
  const long long prs = ldp / 2;
  uint32_t* dPw = reinterpret_cast<uint32_t*>(dP + rowbase * lddp + d);
  const long long dprs = lddp / 2;
  const uint32_t* hw = reinterpret_cast<const uint32_t*>(hstates + rowbase * D + d);
  const uint32_t* dyw = reinterpret_cast<const uint32_t*>(dy + rowbase * D + d);

  float c0 = 0.f, c1 = 0.f;      // carry: dL/dh[t] contribution from t+1
  if (dhT != nullptr) {
    c0 = dhT[(long long)b * D + d];
    c1 = dhT[(long long)b * D + d + 1];
  }
  float da0 = 0.f, da1 = 0.f;
  float2 hcur = unpack_bf16x2(__ldg(hw + (long long)(T - 1) * dq));

  for (int t1 = T - 1; t1 >= 0; t1 -= SCAN_UNROLL) {
    uint32_t raw[SCAN_UNROLL][4];
    uint32_t hp[SCAN_UNROLL];
    uint32_t dyr[SCAN_UNROLL];
    float rsr[SCAN_UNROLL];
#pragma unroll
    for (int u = 0; u < SCAN_UNROLL; ++u) {
      const int t = t1 - u;
      if (t >= 0) {
        const uint32_t* row = Pw + (long long)t * prs;
        raw[u][0] = __ldg(row);
        raw[u][1] = __ldg(row + dq);
        raw[u][2] = __ldg(row + 2 * dq);
        raw[u][3] = __ldg(row + 3 * dq);
        dyr[u] = __ldg(dyw + (long long)t * dq);
        hp[u] = t > 0 ? __ldg(hw + (long long)(t - 1) * dq) : 0u;
        rsr[u] = rowss ? rsqrtf(__ldg(rowss + rowbase + t) * inv_dim + eps) : 1.f;
      }
    }
#pragma unroll
    for (int u = 0; u < SCAN_UNROLL; ++u) {
      const int t = t1 - u;
      if (t >= 0) {
        const float2 sr = unpack_bf16x2(raw[u][0]);
        const float2 cr = unpack_bf16x2(raw[u][1]);
        const float2 gr = unpack_bf16x2(raw[u][2]);
        const float2 dr = unpack_bf16x2(raw[u][3]);
        const float2 dyv = unpack_bf16x2(dyr[u]);
        float2 hprev;
        if (t > 0) {
          hprev = unpack_bf16x2(hp[u]);
        } else if (h0 != nullptr) {
          hprev = make_float2(h0[(long long)b * D + d], h0[(long long)b * D + d + 1]);
        } else {
          hprev = make_float2(0.f, 0.f);
        }
        const float rs = rsr[u];
        uint32_t* orow = dPw + (long long)t * dprs;
        if (MODE == 2) {
          const Gates2 g = eval_gates2<true>(sr, cr, gr, dr, nal2e);
          const float2 one = f2s(1.f), neg1 = f2s(-1.f), rs2 = f2s(rs);
          // y = gate * h;  h = decay * hprev + sel * cand
          const float2 dgate = __fmul2_rn(dyv, hcur);
          const float2 dh = __ffma2_rn(dyv, g.gate, f2(c0, c1));
          const float2 ddec = __fmul2_rn(dh, hprev);
          const float2 cn = __fmul2_rn(dh, g.decay);
          c0 = cn.x;
          c1 = cn.y;
          const float2 ds = __fmul2_rn(__fmul2_rn(dh, g.cand), __fmul2_rn(g.sel, __ffma2_rn(g.sel, neg1, one)));
          const float2 dc = __fmul2_rn(__fmul2_rn(dh, g.sel), __ffma2_rn(__fmul2_rn(g.cand, neg1), g.cand, one));
          const float2 dg = __fmul2_rn(dgate, __fmul2_rn(g.gate, __ffma2_rn(g.gate, neg1, one)));
          // decay = exp(-delta * a): d/d delta = -a * decay ; d/d a = -delta * decay
          const float2 dd = __fmul2_rn(__fmul2_rn(ddec, __fmul2_rn(f2(-a0, -a1), g.decay)), g.sp_sig);
          const float2 dan = __ffma2_rn(__fmul2_rn(ddec, g.delta), __fmul2_rn(g.decay, neg1), f2(da0, da1));
          da0 = dan.x;
          da1 = dan.y;
          const float2 o0 = __fmul2_rn(ds, rs2), o1 = __fmul2_rn(dc, rs2), o2 = __fmul2_rn(dg, rs2),
                       o3 = __fmul2_rn(dd, rs2);
          orow[0] = pack_bf16x2(o0.x, o0.y);
          orow[dq] = pack_bf16x2(o1.x, o1.y);
          orow[2 * dq] = pack_bf16x2(o2.x, o2.y);
          orow[3 * dq] = pack_bf16x2(o3.x, o3.y);
        } else {
          const Gates g0 = eval_gates<MODE == 1>(sr.x, cr.x, gr.x, dr.x, a0);
          const Gates g1 = eval_gates<MODE == 1>(sr.y, cr.y, gr.y, dr.y, a1);
          // y = gate * h
          const float dgate0 = dyv.x * hcur.x, dgate1 = dyv.y * hcur.y;
          const float dh0_ = dyv.x * g0.gate + c0, dh1_ = dyv.y * g1.gate + c1;
          // h = decay * hprev + sel * cand
          const float ddec0 = dh0_ * hprev.x, ddec1 = dh1_ * hprev.y;
          c0 = dh0_ * g0.decay;
          c1 = dh1_ * g1.decay;
          const float ds0 = dh0_ * g0.cand * g0.sel * (1.f - g0.sel);
          const float ds1 = dh1_ * g1.cand * g1.sel * (1.f - g1.sel);
          const float dc0 = dh0_ * g0.sel * (1.f - g0.cand * g0.cand);
          const float dc1 = dh1_ * g1.sel * (1.f - g1.cand * g1.cand);
          const float dg0 = dgate0 * g0.gate * (1.f - g0.gate);
          const float dg1 = dgate1 * g1.gate * (1.f - g1.gate);
          // decay = exp(-delta * a): d/d delta = -a * decay ; d/d a = -delta * decay
          const float dd0 = ddec0 * (-a0 * g0.decay) * g0.sp_sig;
          const float dd1 = ddec1 * (-a1 * g1.decay) * g1.sp_sig;
          da0 += ddec0 * (-g0.delta * g0.decay);
          da1 += ddec1 * (-g1.delta * g1.decay);
          orow[0] = pack_bf16x2(ds0 * rs, ds1 * rs);
          orow[dq] = pack_bf16x2(dc0 * rs, dc1 * rs);
          orow[2 * dq] = pack_bf16x2(dg0 * rs, dg1 * rs);
          orow[3 * dq] = pack_bf16x2(dd0 * rs, dd1 * rs);
        }
        hcur = hprev;
      }
    }
  }
  if (dloga_part != nullptr) {
    // d a / d log_a = a (1 - a)
    dloga_part[(long long)b * D + d] = da0 * a0 * (1.f - a0);
    dloga_part[(long long)b * D + d + 1] = da1 * a1 * (1.f - a1);
  }
  if (dh0 != nullptr) {
    dh0[(long long)b * D + d] = c0;
    dh0[(long long)b * D + d + 1] = c1;
  }
}

// Plain (unfused) diagonal scan kept for API parity with the reference's
// ssm_scan(decay, update): fp32 decay, bf16 or fp32 update, fp32 states out.
// Plain recurrence state[t] = decay[t] * state[t-1] + update[t] for the public ssm_scan op, in
// the operand dtypes the reference op accepts without a cast
// (kernels/_ssm_scan/__init__.py:104-113): decay / update = bf16/bf16, bf16/fp16, fp16/fp16,
// fp32/fp32, fp32/bf16, fp32/fp16.  fp32 accumulator; the states are kept in fp32 for backward.
template <typename T> __device__ __forceinline__ float scan_ld(const T* p, long long i);
template <> __device__ __forceinline__ float scan_ld<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float scan_ld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <> __device__ __forceinline__ float scan_ld<__half>(const __half* p, long long i) { return __half2float(p[i]); }
template <typename T> __device__ __forceinline__ void scan_st(T* p, long long i, float v);
template <> __device__ __forceinline__ void scan_st<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void scan_st<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) {
  p[i] = __float2bfloat16(v);
}
template <> __device__ __forceinline__ void scan_st<__half>(__half* p, long long i, float v) { p[i] = __float2half(v); }

template <typename DT, typename UT>
__global__ void __launch_bounds__(SCAN_THREADS)
plain_scan_fwd_kernel(const DT* __restrict__ decay, const UT* __restrict__ update,
                      const float* __restrict__ h0, float* __restrict__ states, int T, int D) {
  const int b = blockIdx.y;
  const int d = blockIdx.x * SCAN_THREADS + threadIdx.x;
  if (d >= D) return;
  float s = h0 ? h0[(long long)b * D + d] : 0.f;
  const long long base = (long long)b * T * D + d;
  for (int t = 0; t < T; ++t) {
    const long long o = base + (long long)t * D;
    s = scan_ld(decay, o) * s + scan_ld(update, o);
    states[o] = s;
  }
}

// gstates / gupdate in the update dtype, gdecay in the decay dtype.
template <typename DT, typename UT>
__global__ void __launch_bounds__(SCAN_THREADS)
plain_scan_bwd_kernel(const DT* __restrict__ decay, const float* __restrict__ states,
                      const float* __restrict__ h0, const UT* __restrict__ gstates,
                      DT* __restrict__ gdecay, UT* __restrict__ gupdate,
                      float* __restrict__ gh0, int T, int D) {
  const int b = blockIdx.y;
  const int d = blockIdx.x * SCAN_THREADS + threadIdx.x;
  if (d >= D) return;
  const long long base = (long long)b * T * D + d;
  float carry = 0.f;
  for (int t = T - 1; t >= 0; --t) {
    const long long o = base + (long long)t * D;
    const float g = scan_ld(gstates, o) + carry;
    const float prev = t > 0 ? states[o - D] : (h0 ? h0[(long long)b * D + d] : 0.f);
    scan_st(gupdate, o, g);
    scan_st(gdecay, o, g * prev);
    carry = g * scan_ld(decay, o);
  }
  if (gh0) gh0[(long long)b * D + d] = carry;
}

}  // namespace ccb

using namespace ccb;

// Arithmetic of the fused scan kernels: 0 scalar fp32; 1 scalar with the gate exponentials as an FMA-pipe
// polynomial (measured slower: the kernels are bound by instruction issue, not by the special-function
// unit); 2 packed fp32x2.  Returns the old value.
static int g_scan_poly_exp = 2;
extern "C" int ccb_scan_poly_exp(int mode) {
  const int old = g_scan_poly_exp;
  if (mode >= 0 && mode <= 2) g_scan_poly_exp = mode;
  return old;
}

extern "C" int ccb_scan_fwd(const void* P, int64_t ldp, const float* log_a, const float* h0,
                            void* y, void* hout, float* hT, int64_t B, int64_t T, int64_t D,
                            int64_t la_bstride, void* stream) {
  if (B <= 0 || T <= 0) return 0;
  if (D % 8 != 0 || ldp % 2 != 0) return set_error("ccb_scan_fwd: D must be a multiple of 8");
  dim3 grid((unsigned)((D / 2 + SCAN_THREADS - 1) / SCAN_THREADS), (unsigned)B);
  // forward: six steps loaded ahead and six resident blocks per SM (72 registers) measured best: 0.286 ms at
  // 524 288 rows against 0.311 ms with eight steps ahead and four blocks
  auto kern = g_scan_poly_exp == 2 ? scan_fwd_kernel<2, 6, 6> : (g_scan_poly_exp == 1 ? scan_fwd_kernel<1> : scan_fwd_kernel<0>);
  kern<<<grid, SCAN_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)P, ldp, log_a, h0, (__nv_bfloat16*)y, (__nv_bfloat16*)hout, hT, (int)T,
      (int)D, (long long)la_bstride);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("scan_fwd launch: %s", cudaGetErrorString(e));
}

extern "C" int ccb_scan_bwd(const void* P, int64_t ldp, const float* log_a, const float* h0,
                            const void* hstates, const void* dy, const float* dhT,
                            const float* rowss, float inv_dim, float eps, void* dP, int64_t lddp,
                            float* dloga_part, float* dh0, int64_t B, int64_t T, int64_t D,
                            int64_t la_bstride, void* stream) {
  if (B <= 0 || T <= 0) return 0;
  if (D % 8 != 0) return set_error("ccb_scan_bwd: D must be a multiple of 8");
  dim3 grid((unsigned)((D / 2 + SCAN_THREADS - 1) / SCAN_THREADS), (unsigned)B);
  // backward: eight steps ahead, four blocks per SM (116 registers): 0.538 ms; six blocks with six / four steps
  // ahead measured 0.632 / 0.706 ms (fewer loads in flight cost more than the extra warps bring)
  auto kern = g_scan_poly_exp == 2 ? scan_bwd_kernel<2> : (g_scan_poly_exp == 1 ? scan_bwd_kernel<1> : scan_bwd_kernel<0>);
  kern<<<grid, SCAN_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)P, ldp, log_a, h0, (const __nv_bfloat16*)hstates,
      (const __nv_bfloat16*)dy, dhT, rowss, inv_dim, eps, (__nv_bfloat16*)dP, lddp, dloga_part, dh0,
      (int)T, (int)D, (long long)la_bstride);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("scan_bwd launch: %s", cudaGetErrorString(e));
}

// dtype codes: 0 = fp32, 1 = bf16, 2 = fp16.  Accepted (decay, update) pairs: (1,1) (1,2) (2,2) (0,0) (0,1) (0,2).
static inline bool plain_scan_combo_ok(int64_t dd, int64_t ud) {
  return (dd == 1 && ud == 1) || (dd == 1 && ud == 2) || (dd == 2 && ud == 2) || (dd == 0 && ud >= 0 && ud <= 2);
}
#define CCB_SCAN_DISPATCH(dd, ud, CALL)                                                     \
  do {                                                                                      \
    if (dd == 0 && ud == 0) { using DT = float; using UT = float; CALL; }                   \
    else if (dd == 0 && ud == 1) { using DT = float; using UT = __nv_bfloat16; CALL; }      \
    else if (dd == 0 && ud == 2) { using DT = float; using UT = __half; CALL; }             \
    else if (dd == 1 && ud == 1) { using DT = __nv_bfloat16; using UT = __nv_bfloat16; CALL; } \
    else if (dd == 1 && ud == 2) { using DT = __nv_bfloat16; using UT = __half; CALL; }     \
    else { using DT = __half; using UT = __half; CALL; }                                    \
  } while (0)

extern "C" int ccb_plain_scan_fwd(const void* decay, int64_t decay_dtype, const void* update,
                                  int64_t update_dtype, const float* h0, float* states, int64_t B,
                                  int64_t T, int64_t D, void* stream) {
  if (B <= 0 || T <= 0 || D <= 0) return 0;
  if (!plain_scan_combo_ok(decay_dtype, update_dtype))
    return set_error("ccb_plain_scan_fwd: (decay, update) dtype pair (%lld, %lld) is not supported",
                     (long long)decay_dtype, (long long)update_dtype);
  dim3 grid((unsigned)((D + SCAN_THREADS - 1) / SCAN_THREADS), (unsigned)B);
  CCB_SCAN_DISPATCH(decay_dtype, update_dtype,
                    (plain_scan_fwd_kernel<DT, UT><<<grid, SCAN_THREADS, 0, (cudaStream_t)stream>>>(
                        (const DT*)decay, (const UT*)update, h0, states, (int)T, (int)D)));
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("plain_scan_fwd launch: %s", cudaGetErrorString(e));
}

extern "C" int ccb_plain_scan_bwd(const void* decay, int64_t decay_dtype, const float* states,
                                  const float* h0, const void* gstates, int64_t update_dtype,
                                  void* gdecay, void* gupdate, float* gh0, int64_t B, int64_t T,
                                  int64_t D, void* stream) {
  if (B <= 0 || T <= 0 || D <= 0) return 0;
  if (!plain_scan_combo_ok(decay_dtype, update_dtype))
    return set_error("ccb_plain_scan_bwd: (decay, update) dtype pair (%lld, %lld) is not supported",
                     (long long)decay_dtype, (long long)update_dtype);
  dim3 grid((unsigned)((D + SCAN_THREADS - 1) / SCAN_THREADS), (unsigned)B);
  CCB_SCAN_DISPATCH(decay_dtype, update_dtype,
                    (plain_scan_bwd_kernel<DT, UT><<<grid, SCAN_THREADS, 0, (cudaStream_t)stream>>>(
                        (const DT*)decay, states, h0, (const UT*)gstates, (DT*)gdecay, (UT*)gupdate, gh0,
                        (int)T, (int)D)));
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("plain_scan_bwd launch: %s", cudaGetErrorString(e));
}
