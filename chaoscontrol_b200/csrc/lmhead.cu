// Fused LM head for sm_100a: logits GEMM + log-softmax + cross-entropy, with
// the logits recomputed in backward and never written to memory.
//
//   logits[r, v] = rs[r] * sum_d X[r, d] * W'[v, d]
//     X   final hidden state (bf16, [R, 256]), rs = rsqrt(rowss/D + eps): the
//         final RMSNorm, whose weight is folded into W' = W_lm * w_norm.
//
// Three launch modes share one pipeline (TMA ring -> tcgen05.mma -> TMEM ->
// tcgen05.ld epilogue -> bf16 tile in shared memory -> second tcgen05.mma):
//   MODE_LSE    one sweep over the vocabulary: online max/sum -> lse[r] and the
//               per-row CE (scoring / evaluation; forward only).
//   MODE_TRAIN  CTA owns a 128-row tile, X stays in shared memory.  Sweep 1
//               gives lse.  Sweep 2 recomputes each 128x128 logits tile, forms
//               g = (softmax - onehot) * gscale * rs in registers, stores it as
//               a bf16 tile in shared memory and accumulates dX += g . W' in a
//               TMEM accumulator that lives across the sweep; the final
//               epilogue applies the RMSNorm backward and writes dX.
//   MODE_TRAIN1 MODE_TRAIN in ONE sweep (no separate lse pass): the unit's first
//               32 logits fix a per-row reference m (log2 domain, plus a margin
//               of 60 so later, larger logits cannot overflow); every tile adds
//               p~ = 2^(z - m) to the row sum S and stores p~ (bf16) as the g
//               tile, so the TMEM accumulator holds sum_v p~ W'.  The final
//               epilogue forms q = (acc / S - W'[target]) * gscale * rs, then the
//               RMSNorm backward as before; lse = m + log2 S.  Saves one of the
//               five logits-sized GEMMs of a training step.
//   MODE_DW     CTA owns a 128-row tile of W' (kept in shared memory) and a
//               chunk of rows; recomputes logits tiles against streamed X
//               tiles, forms the same g tile and accumulates dW' += g^T . X in
//               TMEM; the result is one fp32 partial tile per row chunk.
//
// The g tile is stored once, as rows of 128 bytes in 1 KiB swizzle atoms, and
// is read by the second MMA either K-major (MODE_TRAIN: A = g) or MN-major
// (MODE_DW: A = g^T); the streamed / resident operand tiles are likewise read
// K-major by the logits MMA and MN-major by the second MMA, so nothing is
// transposed or loaded twice.
//
// Replaces the reference's vocab-tiled linear+CE backends, whose GEMMs are
// library calls with separate row-reduction kernels between them
// (kernels/_lm_head_loss/src/rms_norm_binding.cpp:139-551, linear_ce.cu:24-304).
//
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, then 4 * PARTS epilogue
// warps (warp w: TMEM lanes 32*(w%4).., column part (w-2)/4).  PARTS = 2 gives each epilogue warp
// two 32-column groups of every 128-column logits tile, PARTS = 4 one group (four warps per
// scheduler instead of two).
#include "ptx.cuh"
#include "ccb_api.h"
#include "runtime.h"

namespace ccb {

constexpr int LH_D = 256;            // model dim handled by this kernel
constexpr int LH_ROWS = 128;         // rows per tile
constexpr int LH_VT = 128;           // vocabulary entries per tile
constexpr int LH_CHUNK = 16384;      // one [128 rows][64 bf16] operand chunk
constexpr int LH_TILE = 4 * LH_CHUNK;   // 128 x 256 bf16
constexpr int lh_threads(int parts) { return 64 + 128 * parts; }
constexpr int LH_OFF_RES = 0;
constexpr int LH_OFF_STG = LH_TILE;
constexpr int LH_OFF_G = 3 * LH_TILE;
constexpr int LH_OFF_X = LH_OFF_G + 2 * LH_CHUNK;      // per-row exchange between parts: up to 4 x 128 floats
constexpr int LH_OFF_BAR = LH_OFF_X + 2048;
constexpr int LH_SMEM = LH_OFF_BAR + 256;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

enum { MODE_LSE = 0, MODE_TRAIN = 1, MODE_DW = 2, MODE_TRAIN1 = 3 };
constexpr float LH_REF_MARGIN = 60.f;   // log2 units between the first-logits max and the reference

struct LmHeadArgs {
  int R, V;
  int n_mtiles, n_vtiles;
  int row_chunks, mtiles_per_chunk;   // MODE_DW work decomposition
  const float* rowss;       // [R] sum of squares of X rows; null = no RMSNorm (rs = 1)
  float inv_dim, eps;
  const long long* targets; // [R]
  const float* rowweight;   // [R] or null
  float gscale;             // d loss / d (per-row CE), e.g. 1/R
  float* lse;               // [R] natural-log lse (out in LSE/TRAIN, in for DW)
  float* loss;              // [R] per-row CE (out, LSE/TRAIN)
  float* entropy;           // [R] softmax entropy in nats (out, LSE; optional)
  int skip_lse;             // TRAIN: lse[] is an input, run only the gradient sweep
  const __nv_bfloat16* X;   // [R, 256] for the final epilogue of TRAIN
  __nv_bfloat16* dX;        // [R, 256] out (TRAIN)
  const __nv_bfloat16* W;   // [V, 256] folded head weight (TRAIN1: target rows are gathered)
  float* dWpart;            // [row_chunks, V, 256] out (DW)
  int* status;
  // stage-isolation switches for bottleneck analysis (results are then wrong by design):
  // 1 = the gradient-sweep epilogue skips exp2 / pack / the shared-memory store of the g tile,
  // 2 = the second MMA (dX or dW accumulation) is not issued, 4 = the logits MMA is not issued
  int dbg;
};

struct LhBars {
  uint64_t res_full, res_empty;
  uint64_t stg_full[3], stg_empty[3];
  uint64_t d1_full[2], d1_empty[2];
  uint64_t g_full[2], g_empty[2];
  uint64_t d2_full, d2_empty;
  uint64_t xbar;            // epilogue-group rendezvous (8 warps)
  uint64_t xt_full, xt_empty;   // X row tile resident in tensor memory (A operand of the logits MMA)
  uint32_t tmem_slot;
  int abort_flag;
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// DEEP = 1 (one-sweep training only): the unit's X tile is the logits MMA's A operand from tensor
// memory instead of shared memory, the 64 KiB it occupied become a THIRD W' stage, and one logits
// buffer (handed back as soon as the epilogue holds it in registers) makes room for X in tensor
// memory.  With two stages a W' tile is pinned from its logits MMA until the dX MMA of the same tile
// retires, about one and a half tile periods, which leaves the next load half a period to cross the
// L2 -> SM fabric: measured with the MMAs and the epilogue switched off, the bare load-and-handshake
// skeleton of the two training kernels takes 3.9 of their 8.1 ms, and the stages add up instead
// of overlapping.
template <int MODE, int PARTS, int DEEP>
__global__ void __launch_bounds__(lh_threads(PARTS), 1)
lmhead_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
              const LmHeadArgs p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  LhBars* bars = reinterpret_cast<LhBars*>(smem + LH_OFF_BAR);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if ((smem_u32(smem) & 1023u) != 0u) {   // the swizzled tiles need a 1 KiB aligned base
    if (threadIdx.x == 0) atomicCAS(p.status, CCB_OK, CCB_ERR_BAD_SHAPE);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(&bars->res_full, 1);
    mbar_init(&bars->res_empty, 1);
    mbar_init(&bars->stg_full[2], 1);
    mbar_init(&bars->stg_empty[2], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->stg_full[i], 1);
      mbar_init(&bars->stg_empty[i], 1);
      mbar_init(&bars->d1_full[i], 1);
      mbar_init(&bars->d1_empty[i], 4 * PARTS);
      mbar_init(&bars->g_full[i], (MODE == MODE_DW && DEEP == 0) ? 2 * PARTS : 8);
      mbar_init(&bars->g_empty[i], 1);
    }
    mbar_init(&bars->d2_full, 1);
    mbar_init(&bars->d2_empty, 4);
    mbar_init(&bars->xbar, 4 * PARTS);
    mbar_init(&bars->xt_full, 4);
    mbar_init(&bars->xt_empty, 1);
    bars->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_slot;

  // ---- work decomposition (identical in every role) -------------------------
  // LSE / TRAIN: unit = m-tile; inner = v-tiles (x sweeps).
  // DW: unit = (v-tile, row chunk); inner = m-tiles of the chunk.
  const int n_units = (MODE == MODE_DW) ? p.n_vtiles * p.row_chunks : p.n_mtiles;
  constexpr bool IS_TRAIN = (MODE == MODE_TRAIN) || (MODE == MODE_TRAIN1);
  constexpr bool FUSED1 = (MODE == MODE_TRAIN1);
  // Scoring keeps the unit's X tile in tensor memory and feeds it to the logits MMA from there:
  // an M=128, N=128 instruction with both operands in shared memory needs 8 KiB of it per ~65
  // cycles, with A in tensor memory 4 KiB (2.02 -> 1.88 ms on 262 144 rows).  Tensor-memory
  // columns: [0,256) two logits buffers, [256,384) X.
  // The same was tried for one-sweep training (X in [128,256), ONE logits buffer released as soon
  // as the epilogue holds it in registers, dX in [256,512)): 7.95 -> 8.10 ms, i.e. no gain once
  // the second MMA shares the pipe, so training keeps A in shared memory and two logits buffers.
  static_assert(DEEP == 0 || MODE == MODE_TRAIN1 || MODE == MODE_DW,
                "the deep-ring variant exists for one-sweep training and for the dW kernel");
  // DEEP dW kernel: the logits tile is computed TRANSPOSED (lanes = vocabulary rows of the unit's W'
  // tile, which is the A operand and therefore can live in tensor memory; columns = token rows of the
  // streamed X tile), so that the dW kernel gets the same three-stage ring as the dX kernel.
  constexpr bool DWT = (MODE == MODE_DW) && (DEEP != 0);
  constexpr bool G_COLMAJ = (MODE == MODE_DW) && (DEEP == 0);   // g tile consumed MN-major (A = g^T)
  constexpr bool TA = (MODE == MODE_LSE) || (DEEP != 0);
  constexpr bool ONEBUF = (DEEP != 0);
  constexpr uint32_t X_COL = (DEEP != 0) ? 128u : 256u;   // DEEP: [0,128) logits, [128,256) A rows, [256,512) acc 2
  constexpr int NSTG = TA ? 3 : 2;     // with A in tensor memory the resident tile's 64 KiB are a third stage
  // stage s of the streamed-tile ring; the third stage lives where the resident tile would
  auto stage_ptr = [&](int st) -> uint8_t* {
    return smem + (st < 2 ? LH_OFF_STG + st * LH_TILE : LH_OFF_RES);
  };
  const int n_sweeps = (MODE == MODE_TRAIN && !p.skip_lse) ? 2 : 1;

  if (warp == 0) {
    // =========================== TMA producer ================================
    if (lane == 0) {
      uint32_t res_phase = 0;
      uint32_t n_stg = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
        int res_row, inner0, inner1;
        if (MODE == MODE_DW) {
          const int vt = unit % p.n_vtiles, ch = unit / p.n_vtiles;
          res_row = vt * LH_VT;
          inner0 = ch * p.mtiles_per_chunk;
          inner1 = min(p.n_mtiles, inner0 + p.mtiles_per_chunk);
        } else {
          res_row = unit * LH_ROWS;
          inner0 = 0;
          inner1 = p.n_vtiles;
        }
        const CUtensorMap* tmRes = (MODE == MODE_DW) ? &tmW : &tmX;
        const CUtensorMap* tmStg = (MODE == MODE_DW) ? &tmX : &tmW;
        if (!TA) {
          if (!mbar_wait(&bars->res_empty, res_phase ^ 1u, abort_flag, p.status)) { ok = false; break; }
          mbar_arrive_expect_tx(&bars->res_full, LH_TILE);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            tma_load_3d(smem + LH_OFF_RES + c * LH_CHUNK, tmRes, &bars->res_full, c * 64, res_row, 0);
          res_phase ^= 1u;
        }
        for (int sw = 0; sw < n_sweeps && ok; ++sw) {
          for (int it = inner0; it < inner1; ++it, ++n_stg) {
            const int s = (int)(n_stg % NSTG);
            const uint32_t ph = (n_stg / NSTG) & 1u;
            if (!mbar_wait(&bars->stg_empty[s], ph ^ 1u, abort_flag, p.status)) { ok = false; break; }
            mbar_arrive_expect_tx(&bars->stg_full[s], LH_TILE);
#pragma unroll
            for (int c = 0; c < 4; ++c)
              tma_load_3d(stage_ptr(s) + c * LH_CHUNK, tmStg, &bars->stg_full[s], c * 64, it * 128, 0);
          }
        }
      }
      if (!ok) {
        uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ==================================
    if (lane == 0) {
      constexpr uint32_t idesc1 = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc2 = G_COLMAJ ? make_idesc_bf16(128, 256, 1, 1)
                                           : make_idesc_bf16(128, 256, 0, 1);
      const uint32_t res_base = smem_u32(smem + LH_OFF_RES);
      const uint32_t g_base = smem_u32(smem + LH_OFF_G);
      const uint32_t d2_tmem = tmem_base + 256;
      uint32_t res_phase = 0, n_stg = 0, n_d1 = 0, n_g = 0, n_d2 = 0;
      bool ok = true;

      // second MMA for the tile that used stage `s`; `first` = first of its unit
      auto issue_mma2 = [&](int s, bool first) -> bool {
        const uint32_t stg_base = smem_u32(stage_ptr(s));
        if (first) {
          if (!mbar_wait(&bars->d2_empty, (n_d2 & 1u) ^ 1u, abort_flag, p.status)) return false;
          tc_fence_after_sync();
        }
        const uint32_t gph = n_g & 1u;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait(&bars->g_full[h], gph, abort_flag, p.status)) return false;
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint64_t adesc, bdesc;
            if (G_COLMAJ) {
              const int kk = h * 4 + k;   // 16 rows of r per step
              adesc = make_smem_desc(g_base + kk * 2048, LH_CHUNK, 1024);
              bdesc = make_smem_desc(stg_base + kk * 2048, LH_CHUNK, 1024);
            } else {
              adesc = make_smem_desc(g_base + h * LH_CHUNK + k * 32, 16, 1024);
              bdesc = make_smem_desc(stg_base + h * 8192 + k * 2048, LH_CHUNK, 1024);
            }
            if (!(p.dbg & 2)) umma_bf16(d2_tmem, adesc, bdesc, idesc2, (first && h == 0 && k == 0) ? 0u : 1u);
          }
          umma_commit(&bars->g_empty[h]);
        }
        umma_commit(&bars->stg_empty[s]);
        ++n_g;
        return true;
      };

      for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
        int inner0 = 0, inner1 = p.n_vtiles;
        if (MODE == MODE_DW) {
          const int ch = unit / p.n_vtiles;
          inner0 = ch * p.mtiles_per_chunk;
          inner1 = min(p.n_mtiles, inner0 + p.mtiles_per_chunk);
        }
        if (!TA) {
          if (!mbar_wait(&bars->res_full, res_phase, abort_flag, p.status)) { ok = false; break; }
        }
        if (TA) {
          if (!mbar_wait(&bars->xt_full, res_phase, abort_flag, p.status)) { ok = false; break; }
        }
        res_phase ^= 1u;
        tc_fence_after_sync();
        for (int sw = 0; sw < n_sweeps && ok; ++sw) {
          const bool second = (MODE == MODE_DW) || (IS_TRAIN && sw == n_sweeps - 1);
          int prev_stage = -1;
          bool prev_first = true;
          for (int it = inner0; it < inner1; ++it) {
            const int s = (int)(n_stg % NSTG);
            const uint32_t sph = (n_stg / NSTG) & 1u;
            ++n_stg;
            const int b = ONEBUF ? 0 : (n_d1 & 1);
            const uint32_t dph = ONEBUF ? (n_d1 & 1u) : ((n_d1 >> 1) & 1u);
            ++n_d1;
            if (!mbar_wait(&bars->stg_full[s], sph, abort_flag, p.status)) { ok = false; break; }
            if (!mbar_wait(&bars->d1_empty[b], dph ^ 1u, abort_flag, p.status)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t stg_base = smem_u32(stage_ptr(s));
            const uint32_t xa = (MODE == MODE_DW) ? stg_base : res_base;   // A operand when it is in shared memory
            const uint32_t wb = G_COLMAJ ? res_base : stg_base;            // B operand: W' tile, or X for transposed dW
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint64_t bdesc = make_smem_desc(wb + c * LH_CHUNK + k * 32, 16, 1024);
                if (p.dbg & 4) continue;
                if (TA) {
                  // K step (c, k) = bf16 columns [64c + 16k, +16) of X = 8 packed 32-bit columns
                  umma_bf16_ta(tmem_base + b * 128, tmem_base + X_COL + (uint32_t)(c * 4 + k) * 8u, bdesc,
                               idesc1, (c > 0 || k > 0) ? 1u : 0u);
                } else {
                  const uint64_t adesc = make_smem_desc(xa + c * LH_CHUNK + k * 32, 16, 1024);
                  umma_bf16(tmem_base + b * 128, adesc, bdesc, idesc1, (c > 0 || k > 0) ? 1u : 0u);
                }
              }
            }
            umma_commit(&bars->d1_full[b]);
            if (!second) {
              umma_commit(&bars->stg_empty[s]);
            } else {
              if (prev_stage >= 0) {
                if (!issue_mma2(prev_stage, prev_first)) { ok = false; break; }
                prev_first = false;
              }
              prev_stage = s;
            }
          }
          if (ok && second && prev_stage >= 0) {
            if (!issue_mma2(prev_stage, prev_first)) { ok = false; break; }
            umma_commit(&bars->d2_full);
            ++n_d2;
          }
        }
        if (ok) {
          if (!TA) umma_commit(&bars->res_empty);
          if (TA) umma_commit(&bars->xt_empty);   // every MMA that read the X columns has completed
        }
      }
    }
  } else {
    // =========================== epilogue ====================================
    constexpr int NG = 4 / PARTS;           // 32-column groups of each 128-column tile per warp
    const int q = warp & 3;                 // TMEM lane quadrant
    const int part = (warp - 2) >> 2;       // this warp's groups: g * PARTS + part, g < NG
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    float* xchg = reinterpret_cast<float*>(smem + LH_OFF_X);     // [PARTS][128]
    uint32_t n_d1 = 0, n_g = 0, n_d2 = 0, n_x = 0, n_xt = 0;
    bool ok = true;
    // Every wait below is made warp-uniform, so the warp-collective TMEM loads
    // that follow never run with part of the warp on the abort path.
    auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool {
      const bool w = mbar_wait(bar, parity, abort_flag, p.status);
      return __all_sync(0xffffffffu, w);
    };
    // Bounded rendezvous of all epilogue warps (orders the xchg traffic).
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->xbar);
      const bool w = wait_all(&bars->xbar, n_x & 1u);
      ++n_x;
      return w;
    };
    // A row's per-part values combined in part order: every part ends with the same bits.
    auto parts_sum = [&](float v, float& out) -> bool {
      if (!epi_sync()) return false;
      xchg[part * 128 + row_in_tile] = v;
      if (!epi_sync()) return false;
      float t = xchg[row_in_tile];
#pragma unroll
      for (int k = 1; k < PARTS; ++k) t += xchg[k * 128 + row_in_tile];
      out = t;
      return true;
    };
    auto parts_max = [&](float v, float& out) -> bool {
      if (!epi_sync()) return false;
      xchg[part * 128 + row_in_tile] = v;
      if (!epi_sync()) return false;
      float t = xchg[row_in_tile];
#pragma unroll
      for (int k = 1; k < PARTS; ++k) t = fmaxf(t, xchg[k * 128 + row_in_tile]);
      out = t;
      return true;
    };

    for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
      int inner0 = 0, inner1 = p.n_vtiles, v_unit0 = 0, ch = 0;
      if (MODE == MODE_DW) {
        const int vt = unit % p.n_vtiles;
        ch = unit / p.n_vtiles;
        v_unit0 = vt * LH_VT;
        inner0 = ch * p.mtiles_per_chunk;
        inner1 = min(p.n_mtiles, inner0 + p.mtiles_per_chunk);
      }
      // per-row constants (LSE / TRAIN: fixed for the unit; DW: reloaded per m-tile)
      int r = 0;
      bool row_ok = false;
      float c1 = 0.f, c2 = 0.f, gs = 0.f, rs = 0.f;
      int tgt = -1;
      auto load_row = [&](int mtile, bool need_lse) {
        r = mtile * LH_ROWS + row_in_tile;
        row_ok = r < p.R;
        rs = row_ok ? (p.rowss ? rsqrtf(p.rowss[r] * p.inv_dim + p.eps) : 1.f) : 0.f;
        c1 = rs * LOG2E;
        tgt = row_ok ? (int)p.targets[r] : -1;
        const float w = (row_ok && p.rowweight) ? p.rowweight[r] : 1.f;
        gs = row_ok ? p.gscale * w * rs : 0.f;
        if (need_lse) c2 = row_ok ? p.lse[r] * LOG2E : 0.f;
      };
      if (MODE != MODE_DW) load_row(unit, MODE == MODE_TRAIN && p.skip_lse);
      float inv_s = 0.f;                   // TRAIN1: 1 / row sum, known after the sweep
      if (TA) {
        // this unit's X rows -> tensor memory (one row per lane, 256 bf16 = 128 packed columns);
        // the previous unit's MMAs must have finished reading those columns
        if (part == 0) {
          if (!wait_all(&bars->xt_empty, (n_xt & 1u) ^ 1u)) { ok = false; break; }
          tc_fence_after_sync();
          // the A rows of the unit: X rows, or the unit's W' rows for the transposed dW kernel
          const bool a_ok = DWT ? (v_unit0 + row_in_tile < p.V) : row_ok;
          const uint4* xrow4 = DWT
              ? reinterpret_cast<const uint4*>(p.W + (long long)(a_ok ? v_unit0 + row_in_tile : 0) * LH_D)
              : reinterpret_cast<const uint4*>(p.X + (long long)(row_ok ? r : 0) * LH_D);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t xv[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint4 v4 = a_ok ? __ldg(xrow4 + c * 8 + j) : make_uint4(0u, 0u, 0u, 0u);
              xv[j * 4] = v4.x; xv[j * 4 + 1] = v4.y; xv[j * 4 + 2] = v4.z; xv[j * 4 + 3] = v4.w;
            }
            __syncwarp();
            tmem_st32(tmem_base + X_COL + (uint32_t)(c * 32) + lane_addr, xv);
          }
          tmem_st_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->xt_full);
        }
        ++n_xt;
      }

      if (DWT) {
        // ---- transposed dW sweep: lane = vocabulary row v_unit0 + row_in_tile, columns = the 128
        // token rows of m-tile `it`.  g^T[v, r] = sign * 2^(acc * |c1[r]| - c2[r]) with
        // c1 = +-rs * log2e (the sign is that of the row's gradient scale) and
        // c2 = lse * log2e - log2 |gs|, so the scale rides in the exponent and a column needs two
        // constants.  They sit in shared memory, double-buffered by tile parity: the warps of the
        // last part write tile it's pair before the rendezvous at the top of iteration `it`, and a
        // buffer is next written two rendezvous later, after every reader has left it.
        // The one-hot term: lane l also holds the target and the scale of column col0 + l; when the
        // target's vocabulary row lies in this warp's quadrant it subtracts gs from that element of
        // the tile it has just written (a read-modify-write of one bf16 in shared memory).
        float2* cst = reinterpret_cast<float2*>(smem + LH_OFF_X);       // [2][128]
        const bool writer = (part == PARTS - 1);
        // Raw per-row inputs are REQUESTED one tile ahead and only turned into constants at the top
        // of the next iteration, so no global-load latency sits on the path between the two MMAs.
        struct RawRow { float ss, lse, w; int tg; };
        auto fetch_raw = [&](int rr) -> RawRow {
          RawRow x;
          if (rr < p.R) {
            x.ss = p.rowss ? __ldg(p.rowss + rr) : 0.f;
            x.lse = __ldg(p.lse + rr);
            x.w = p.rowweight ? __ldg(p.rowweight + rr) : 1.f;
            x.tg = (int)__ldg(p.targets + rr);
          } else {
            x.ss = 0.f; x.lse = INFINITY; x.w = 0.f; x.tg = -1;      // row past the end: g == 0
          }
          return x;
        };
        auto scale_of = [&](const RawRow& x, float& rsv) -> float {
          rsv = p.rowss ? rsqrtf(x.ss * p.inv_dim + p.eps) : 1.f;
          return p.gscale * x.w * rsv;
        };
        RawRow wraw = {0.f, INFINITY, 0.f, -1}, graw[NG];
        if (writer) wraw = fetch_raw(inner0 * LH_ROWS + row_in_tile);
#pragma unroll
        for (int g = 0; g < NG; ++g) graw[g] = fetch_raw(inner0 * LH_ROWS + (g * PARTS + part) * 32 + lane);
        float col_gs[NG];
        int col_tg[NG];
        for (int it = inner0; it < inner1 && ok; ++it) {
          ++n_d1;
          const uint32_t dph = (n_d1 - 1) & 1u;            // one logits buffer
          const uint32_t gph = n_g & 1u;
          ++n_g;
          const int buf = (it - inner0) & 1;
          if (writer) {
            float rsv;
            const float gsv = scale_of(wraw, rsv);
            // gs == 0 (or a row past the end): c2 = +inf, so the exponential is exactly 0
            cst[buf * 128 + row_in_tile] =
                make_float2(copysignf(rsv * LOG2E, gsv), wraw.lse * LOG2E - __log2f(fabsf(gsv)));
          }
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            float rsv;
            col_gs[g] = scale_of(graw[g], rsv);
            col_tg[g] = graw[g].tg;
          }
          if (!epi_sync()) { ok = false; break; }
          if (it + 1 < inner1) {
            if (writer) wraw = fetch_raw((it + 1) * LH_ROWS + row_in_tile);
#pragma unroll
            for (int g = 0; g < NG; ++g)
              graw[g] = fetch_raw((it + 1) * LH_ROWS + (g * PARTS + part) * 32 + lane);
          }
          if (!wait_all(&bars->d1_full[0], dph)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t t_addr = tmem_base + lane_addr;
          uint32_t ah[NG][32];
          __syncwarp();
#pragma unroll
          for (int g = 0; g < NG; ++g) tmem_ld32(t_addr + (g * PARTS + part) * 32, ah[g]);
          tmem_ld_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->d1_empty[0]);
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            const int grp = g * PARTS + part;      // 32-column group: token rows 32 grp .. 32 grp + 31
            const int h = grp >> 1;
            const uint32_t (&a)[32] = ah[g];
            uint32_t packed[16];
            if (!(p.dbg & 1)) {
              const float4* c4 = reinterpret_cast<const float4*>(cst + buf * 128 + grp * 32);
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float4 k = c4[i >> 1];       // (c1, c2) of columns i and i + 1: one broadcast load
                const float p0 = ex2f(fmaf(__uint_as_float(a[i]), fabsf(k.x), -k.y));
                const float p1 = ex2f(fmaf(__uint_as_float(a[i + 1]), fabsf(k.z), -k.w));
                packed[i >> 1] = pack_bf16x2(copysignf(p0, k.x), copysignf(p1, k.z));
              }
            }
            if (!wait_all(&bars->g_empty[h], gph ^ 1u)) { ok = false; break; }
            uint8_t* grow = smem + LH_OFF_G + h * LH_CHUNK + row_in_tile * 128;
            if (!(p.dbg & 1)) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int slot = ((grp & 1) * 4 + j) ^ (row_in_tile & 7);
                *reinterpret_cast<uint4*>(grow + slot * 16) =
                    make_uint4(packed[j * 4], packed[j * 4 + 1], packed[j * 4 + 2], packed[j * 4 + 3]);
              }
              __syncwarp();
              // one-hot: column grp * 32 + lane, vocabulary row col_tg - v_unit0 (if it is one of mine)
              const int tv = col_tg[g] - v_unit0;
              if (tv >= q * 32 && tv < q * 32 + 32) {
                const int colc = (grp & 1) * 32 + lane;                 // column inside the 64-wide chunk
                uint8_t* cell = smem + LH_OFF_G + h * LH_CHUNK + tv * 128 + (((colc >> 3) ^ (tv & 7)) * 16) +
                                (colc & 7) * 2;
                __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(cell);
                *e = __float2bfloat16(__bfloat162float(*e) - col_gs[g]);
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->g_full[h]);
          }
        }
      } else
      for (int sw = 0; sw < n_sweeps && ok; ++sw) {
        const bool second = (MODE == MODE_DW) || (IS_TRAIN && sw == n_sweeps - 1);
        float run_m = -INFINITY, run_s = 0.f, run_e = 0.f, tacc = 0.f, zt = 0.f;
        for (int it = inner0; it < inner1 && ok; ++it) {
          const int b = ONEBUF ? 0 : (n_d1 & 1);
          const uint32_t dph = ONEBUF ? (n_d1 & 1u) : ((n_d1 >> 1) & 1u);
          ++n_d1;
          int v0;
          if (MODE == MODE_DW) {
            load_row(it, true);
            v0 = v_unit0;
          } else {
            v0 = it * LH_VT;
          }
          if (!wait_all(&bars->d1_full[b], dph)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t t_addr = tmem_base + b * 128 + lane_addr;
          if (!second) {
            // ---- sweep 1: online max / sum (log2 domain) ----------------------
#pragma unroll
            for (int g = 0; g < NG; ++g) {
              const int col0 = (g * PARTS + part) * 32;
              uint32_t a[32];
              __syncwarp();
              tmem_ld32(t_addr + col0, a);
              tmem_ld_wait();
              float mx = __uint_as_float(a[0]);
#pragma unroll
              for (int i = 1; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(a[i]));
              const float new_m = fmaxf(run_m, mx * c1);
              float acc = 0.f, eacc = 0.f;
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float e = ex2f(fmaf(__uint_as_float(a[i]), c1, -new_m));
                acc += e;
                if (MODE == MODE_LSE) eacc = fmaf(e, __uint_as_float(a[i]), eacc);   // sum p~ * raw
              }
              const float resc = ex2f(run_m - new_m);
              run_s = run_s * resc + acc;
              if (MODE == MODE_LSE) run_e = run_e * resc + eacc;
              run_m = new_m;
              if (MODE == MODE_LSE) {
                // a lane meets its target column once per sweep: looked up outside the hot loop
                const int tl = tgt - (v0 + col0);
                if ((unsigned)tl < 32u) {
#pragma unroll
                  for (int i = 0; i < 32; ++i)
                    if (i == tl) tacc = __uint_as_float(a[i]);
                }
              }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->d1_empty[b]);
          } else {
            // ---- sweep 2 / DW: g tile -> shared memory ------------------------
            const uint32_t gph = n_g & 1u;
            ++n_g;
            if (FUSED1 && it == inner0) {
              // per-row reference: max of the unit's first 32 logits (every warp reads the same
              // 32 columns, so all parts of a row agree without an exchange)
              uint32_t a0[32];
              __syncwarp();
              tmem_ld32(t_addr, a0);
              tmem_ld_wait();
              float mx = __uint_as_float(a0[0]);
#pragma unroll
              for (int i = 1; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(a0[i]));
              c2 = fmaf(mx, c1, LH_REF_MARGIN);
            }
            // all of this warp's groups are requested before any is used: one TMEM round trip
            // per tile on the path between the two MMAs
            uint32_t ah[NG][32];
            __syncwarp();
#pragma unroll
            for (int g = 0; g < NG; ++g) tmem_ld32(t_addr + (g * PARTS + part) * 32, ah[g]);
            tmem_ld_wait();
            // the logits now live in registers: hand the TMEM buffer back at once, so the MMA
            // warp can start the tile after next while this one is still being turned into g
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->d1_empty[b]);
            if (MODE == MODE_DW) {
              if (!wait_all(&bars->g_empty[q >> 1], gph ^ 1u)) { ok = false; break; }
            }
#pragma unroll
            for (int g = 0; g < NG; ++g) {
              const int grp = g * PARTS + part;      // 32-column group of the tile
              const int h = grp >> 1;                // 64-column chunk of the g tile
              const int col0 = grp * 32;
              const uint32_t (&a)[32] = ah[g];
              const int tl = tgt - (v0 + col0);
              uint32_t packed[16];
              if (p.dbg & 1) {
                if (MODE != MODE_DW) {
                  if (!wait_all(&bars->g_empty[h], gph ^ 1u)) { ok = false; break; }
                  __syncwarp();
                  if (lane == 0) mbar_arrive(&bars->g_full[h]);
                }
                continue;
              }
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                float z0 = fmaf(__uint_as_float(a[i]), c1, -c2);
                float z1 = fmaf(__uint_as_float(a[i + 1]), c1, -c2);
                if (FUSED1) { z0 = fminf(z0, 126.f); z1 = fminf(z1, 126.f); }
                float p0 = ex2f(z0), p1 = ex2f(z1);
                if (FUSED1) {
                  run_s += p0 + p1;
                  packed[i >> 1] = pack_bf16x2(p0, p1);
                } else {
                  packed[i >> 1] = pack_bf16x2(p0 * gs, p1 * gs);
                }
              }
              if ((unsigned)tl < 32u) {
                // the target column: handled outside the hot loop, a lane meets it once per sweep
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (i == tl) {
                    const float z = fmaf(__uint_as_float(a[i]), c1, -c2);
                    if (FUSED1) {
                      zt = fminf(z, 126.f);
                    } else {
                      zt = z;
                      // redo the target's pair with the one-hot subtracted
                      const int i0 = i & ~1;
                      float pa = ex2f(fmaf(__uint_as_float(a[i0]), c1, -c2));
                      float pb = ex2f(fmaf(__uint_as_float(a[i0 + 1]), c1, -c2));
                      if (i & 1) pb -= 1.f; else pa -= 1.f;
                      packed[i >> 1] = pack_bf16x2(pa * gs, pb * gs);
                    }
                  }
              }
              if (MODE != MODE_DW) {
                if (!wait_all(&bars->g_empty[h], gph ^ 1u)) { ok = false; break; }
              }
              // row `row_in_tile` of chunk h, 16-byte slots (grp & 1) * 4 .. + 3, 128B swizzle
              uint8_t* grow = smem + LH_OFF_G + h * LH_CHUNK + row_in_tile * 128;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int slot = ((grp & 1) * 4 + j) ^ (row_in_tile & 7);
                *reinterpret_cast<uint4*>(grow + slot * 16) =
                    make_uint4(packed[j * 4], packed[j * 4 + 1], packed[j * 4 + 2], packed[j * 4 + 3]);
              }
              if (MODE != MODE_DW) {
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->g_full[h]);
              }
            }
            if (!ok) break;
            if (MODE == MODE_DW) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) mbar_arrive(&bars->g_full[q >> 1]);
            }
          }
        }
        if (!ok) break;

        if (!second) {
          // combine the column parts of each row -> lse
          float m = 0.f, s = 0.f;
          if (!parts_max(run_m, m)) { ok = false; break; }
          const float my_resc = ex2f(run_m - m);
          if (!parts_sum(run_s * my_resc, s)) { ok = false; break; }
          const float lse2 = m + __log2f(s);
          c2 = lse2;
          if (row_ok && part == 0) p.lse[r] = lse2 * LN2;
          if (MODE == MODE_LSE) {
            // the target column lived in exactly one part
            float t_all = 0.f;
            if (!parts_sum(tacc, t_all)) { ok = false; break; }
            if (row_ok && part == 0) p.loss[r] = lse2 * LN2 - t_all * rs;
            if (p.entropy != nullptr) {
              // H = lse - E[logit],  E[logit] = rs * sum(p~ * raw) / sum(p~)
              float e_tot = 0.f;
              if (!parts_sum(run_e * my_resc, e_tot)) { ok = false; break; }
              if (row_ok && part == 0) p.entropy[r] = lse2 * LN2 - rs * e_tot / s;
            }
          }
        } else if (FUSED1) {
          // combine the parts: S = sum p~, target logit relative to the reference
          float S = 0.f, z_all = 0.f;
          if (!parts_sum(run_s, S)) { ok = false; break; }
          if (!parts_sum(zt, z_all)) { ok = false; break; }
          const float lg = __log2f(S);
          inv_s = 1.f / S;
          if (row_ok && part == 0) {
            p.lse[r] = (c2 + lg) * LN2;
            p.loss[r] = (lg - z_all) * LN2;
          }
        } else if (MODE == MODE_TRAIN) {
          // per-row CE = -log p_target = -zt * ln2 (zt captured by exactly one warp of the row)
          float z_all = 0.f;
          if (!parts_sum(zt, z_all)) { ok = false; break; }
          if (row_ok && part == 0) p.loss[r] = -z_all * LN2;
        }
      }
      if (!ok) break;

      // ---- unit epilogue: drain the second accumulator ------------------------
      if (MODE != MODE_LSE) {
        if (part == 0) {
          if (!wait_all(&bars->d2_full, n_d2 & 1u)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t t2 = tmem_base + 256 + lane_addr;
          if (IS_TRAIN) {
            // dx = q - x * (rs^2 / D) * sum_d q * x   (RMSNorm backward, weight folded)
            const __nv_bfloat16* xrow = p.X + (long long)r * LH_D;
            // TRAIN1: the accumulator holds sum_v p~ W'; q = (acc / S - W'[target]) * gs
            const __nv_bfloat16* wrow = p.W + (long long)(row_ok ? tgt : 0) * LH_D;
            auto finish_q = [&](uint32_t (&a)[32], int c) {
              if (FUSED1) {
                const uint4* w4 = reinterpret_cast<const uint4*>(wrow + c * 32);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint4 wv = __ldg(w4 + j);
                  const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = unpack_bf16x2(ww[e]);
                    a[j * 8 + 2 * e] = __float_as_uint((__uint_as_float(a[j * 8 + 2 * e]) * inv_s - f.x) * gs);
                    a[j * 8 + 2 * e + 1] =
                        __float_as_uint((__uint_as_float(a[j * 8 + 2 * e + 1]) * inv_s - f.y) * gs);
                  }
                }
              }
            };
            float dot = 0.f;
            for (int c = 0; c < 8; ++c) {
              uint32_t a[32];
              __syncwarp();
              tmem_ld32(t2 + c * 32, a);
              tmem_ld_wait();
              if (row_ok) {
                finish_q(a, c);
                const uint4* x4 = reinterpret_cast<const uint4*>(xrow + c * 32);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint4 qv = __ldg(x4 + j);
                  float2 f;
                  f = unpack_bf16x2(qv.x); dot += __uint_as_float(a[j * 8 + 0]) * f.x + __uint_as_float(a[j * 8 + 1]) * f.y;
                  f = unpack_bf16x2(qv.y); dot += __uint_as_float(a[j * 8 + 2]) * f.x + __uint_as_float(a[j * 8 + 3]) * f.y;
                  f = unpack_bf16x2(qv.z); dot += __uint_as_float(a[j * 8 + 4]) * f.x + __uint_as_float(a[j * 8 + 5]) * f.y;
                  f = unpack_bf16x2(qv.w); dot += __uint_as_float(a[j * 8 + 6]) * f.x + __uint_as_float(a[j * 8 + 7]) * f.y;
                }
              }
            }
            const float coef = p.rowss ? dot * rs * rs * p.inv_dim : 0.f;   // no norm: plain dX
            for (int c = 0; c < 8; ++c) {
              uint32_t a[32];
              __syncwarp();
              tmem_ld32(t2 + c * 32, a);
              tmem_ld_wait();
              if (row_ok) {
                finish_q(a, c);
                const uint4* x4 = reinterpret_cast<const uint4*>(xrow + c * 32);
                uint4* o4 = reinterpret_cast<uint4*>(p.dX + (long long)r * LH_D + c * 32);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint4 qv = __ldg(x4 + j);
                  const float2 f0 = unpack_bf16x2(qv.x), f1 = unpack_bf16x2(qv.y),
                               f2 = unpack_bf16x2(qv.z), f3 = unpack_bf16x2(qv.w);
                  uint4 o;
                  o.x = pack_bf16x2(__uint_as_float(a[j * 8 + 0]) - f0.x * coef, __uint_as_float(a[j * 8 + 1]) - f0.y * coef);
                  o.y = pack_bf16x2(__uint_as_float(a[j * 8 + 2]) - f1.x * coef, __uint_as_float(a[j * 8 + 3]) - f1.y * coef);
                  o.z = pack_bf16x2(__uint_as_float(a[j * 8 + 4]) - f2.x * coef, __uint_as_float(a[j * 8 + 5]) - f2.y * coef);
                  o.w = pack_bf16x2(__uint_as_float(a[j * 8 + 6]) - f3.x * coef, __uint_as_float(a[j * 8 + 7]) - f3.y * coef);
                  o4[j] = o;
                }
              }
            }
          } else {
            // MODE_DW: fp32 partial tile [v rows][256]
            const int v = v_unit0 + row_in_tile;
            float* orow = p.dWpart + ((long long)ch * p.V + v) * LH_D;
            for (int c = 0; c < 8; ++c) {
              uint32_t a[32];
              __syncwarp();
              tmem_ld32(t2 + c * 32, a);
              tmem_ld_wait();
              if (v < p.V) {
                float4* o4 = reinterpret_cast<float4*>(orow + c * 32);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  o4[j] = make_float4(__uint_as_float(a[j * 4]), __uint_as_float(a[j * 4 + 1]),
                                      __uint_as_float(a[j * 4 + 2]), __uint_as_float(a[j * 4 + 3]));
              }
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->d2_empty);
        }
        ++n_d2;
      }
    }
  }

  // =========================== teardown ========================================
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// Epilogue column parts: 2 = eight epilogue warps, 4 = sixteen; 0 = per mode, as measured on a B200
// at 262 144 rows: the scoring sweep gains from sixteen warps (1.81 -> 1.77 ms), the training kernels
// lose (7.76 -> 8.11 ms for the one-sweep kernel plus the dW kernel).
static int g_lh_parts = 0;
static int g_lh_dbg = 0;
// 1: one-sweep training and the dW kernel run their three-stage variants (7.94 -> 6.66 ms for the pair
// at 262 144 rows on a B200); 0: two stages with the resident tile in shared memory
static int g_lh_deep = 1;

template <int MODE, int PARTS, int DEEP = 0>
static int launch_lmhead_p(const void* X, const void* W, LmHeadArgs& a, cudaStream_t stream) {
  static bool attr_set[16] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = lmhead_kernel<MODE, PARTS, DEEP>;
  if (!attr_set[dev & 15]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LH_SMEM);
    if (e != cudaSuccess) return set_error("cudaFuncSetAttribute(lmhead): %s", cudaGetErrorString(e));
    attr_set[dev & 15] = true;
  }
  CUtensorMap tmX, tmW;
  if (make_tmap_bf16_3d(&tmX, X, LH_D, (uint64_t)a.R, 1, LH_D, 0, 64, 128)) return -1;
  if (make_tmap_bf16_3d(&tmW, W, LH_D, (uint64_t)a.V, 1, LH_D, 0, 64, 128)) return -1;
  a.status = ccb_status_ptr();
  a.dbg = g_lh_dbg;
  const int units = (MODE == MODE_DW) ? a.n_vtiles * a.row_chunks : a.n_mtiles;
  const int grid = units < ccb_num_sms() ? units : ccb_num_sms();
  kern<<<grid, lh_threads(PARTS), LH_SMEM, stream>>>(tmX, tmW, a);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("lmhead launch: %s", cudaGetErrorString(e));
}

template <int MODE>
static int launch_lmhead(const void* X, const void* W, LmHeadArgs& a, cudaStream_t stream) {
  const int parts = g_lh_parts ? g_lh_parts : (MODE == MODE_LSE ? 4 : 2);
  if ((MODE == MODE_TRAIN1 || MODE == MODE_DW) && g_lh_deep) {
    // the variant is instantiated for these two modes only
    constexpr int MD = (MODE == MODE_DW) ? MODE_DW : MODE_TRAIN1;
    return parts == 2 ? launch_lmhead_p<MD, 2, 1>(X, W, a, stream) : launch_lmhead_p<MD, 4, 1>(X, W, a, stream);
  }
  return parts == 2 ? launch_lmhead_p<MODE, 2>(X, W, a, stream)
                    : launch_lmhead_p<MODE, 4>(X, W, a, stream);
}

}  // namespace ccb

using namespace ccb;

// Epilogue width of the fused LM-head kernels: 2 (eight epilogue warps), 4 (sixteen) or 0 (the
// per-mode default).  Returns the previous value; other arguments leave it unchanged.
extern "C" int ccb_lmhead_epilogue_parts(int parts) {
  const int old = g_lh_parts;
  if (parts == 0 || parts == 2 || parts == 4) g_lh_parts = parts;
  return old;
}

// 1: the one-sweep training kernel uses three W' stages with X held in tensor memory; 0: two stages
// with X in shared memory.  Returns the previous value.
extern "C" int ccb_lmhead_deep_ring(int on) {
  const int old = g_lh_deep;
  if (on == 0 || on == 1) g_lh_deep = on;
  return old;
}

// Stage-isolation switches of LmHeadArgs::dbg (0 = normal operation).  For timing experiments only.
extern "C" int ccb_lmhead_debug(int bits) {
  const int old = g_lh_dbg;
  g_lh_dbg = bits;
  return old;
}

static int lmhead_common(LmHeadArgs& a, int64_t R, int64_t V, int64_t D, const float* rowss,
                         float eps, const int64_t* targets) {
  if (D != LH_D) return set_error("fused LM head: model dim must be %d (got %lld)", LH_D, (long long)D);
  if (V % LH_VT != 0) return set_error("fused LM head: vocab must be a multiple of %d", LH_VT);
  if (R <= 0) return 1;
  a.R = (int)R;
  a.V = (int)V;
  a.n_mtiles = (int)((R + LH_ROWS - 1) / LH_ROWS);
  a.n_vtiles = (int)(V / LH_VT);
  a.row_chunks = 1;
  a.mtiles_per_chunk = a.n_mtiles;
  a.rowss = rowss;
  a.inv_dim = 1.f / (float)D;
  a.eps = eps;
  a.targets = (const long long*)targets;
  return 0;
}

// lse[r], loss[r] = CE of row r.  Forward only.
extern "C" int ccb_lmhead_lse(const void* X, const void* W, const float* rowss, float eps,
                              const int64_t* targets, float* lse, float* loss, float* entropy,
                              int64_t R, int64_t V, int64_t D, void* stream) {
  LmHeadArgs a = {};
  int rc = lmhead_common(a, R, V, D, rowss, eps, targets);
  if (rc) return rc < 0 ? rc : 0;
  a.lse = lse;
  a.loss = loss;
  a.entropy = entropy;
  a.X = (const __nv_bfloat16*)X;      // rows are copied into tensor memory for the logits MMA
  return launch_lmhead<MODE_LSE>(X, W, a, (cudaStream_t)stream);
}

// lse, per-row loss and dX (gradient w.r.t. the un-normalised hidden state).
// lse_is_input: 0 = two sweeps (lse, then gradient); 1 = lse[] is read, gradient sweep only;
// 2 = one sweep with a fixed per-row reference (MODE_TRAIN1), lse[] is written.
extern "C" int ccb_lmhead_train(const void* X, const void* W, const float* rowss, float eps,
                                const int64_t* targets, const float* rowweight, float gscale,
                                float* lse, int64_t lse_is_input, float* loss, void* dX, int64_t R,
                                int64_t V, int64_t D, void* stream) {
  LmHeadArgs a = {};
  int rc = lmhead_common(a, R, V, D, rowss, eps, targets);
  if (rc) return rc < 0 ? rc : 0;
  a.rowweight = rowweight;
  a.gscale = gscale;
  a.lse = lse;
  a.skip_lse = lse_is_input == 1 ? 1 : 0;
  a.loss = loss;
  a.X = (const __nv_bfloat16*)X;
  a.dX = (__nv_bfloat16*)dX;
  a.W = (const __nv_bfloat16*)W;
  if (lse_is_input == 2) return launch_lmhead<MODE_TRAIN1>(X, W, a, (cudaStream_t)stream);
  return launch_lmhead<MODE_TRAIN>(X, W, a, (cudaStream_t)stream);
}

// dWpart[row_chunks, V, D] fp32: partial gradients of W' = W_lm * w_norm.
extern "C" int ccb_lmhead_dw(const void* X, const void* W, const float* rowss, float eps,
                             const int64_t* targets, const float* rowweight, float gscale,
                             const float* lse, float* dWpart, int64_t row_chunks, int64_t R,
                             int64_t V, int64_t D, void* stream) {
  LmHeadArgs a = {};
  int rc = lmhead_common(a, R, V, D, rowss, eps, targets);
  if (rc) return rc < 0 ? rc : 0;
  if (row_chunks < 1) row_chunks = 1;
  if (row_chunks > a.n_mtiles) row_chunks = a.n_mtiles;
  a.mtiles_per_chunk = (int)((a.n_mtiles + row_chunks - 1) / row_chunks);
  a.row_chunks = (a.n_mtiles + a.mtiles_per_chunk - 1) / a.mtiles_per_chunk;
  if (a.row_chunks != (int)row_chunks)
    return set_error("ccb_lmhead_dw: row_chunks=%lld leaves an empty chunk (use %d)",
                     (long long)row_chunks, a.row_chunks);
  a.rowweight = rowweight;
  a.gscale = gscale;
  a.lse = const_cast<float*>(lse);
  a.dWpart = dWpart;
  a.X = (const __nv_bfloat16*)X;
  a.W = (const __nv_bfloat16*)W;      // the transposed variant copies its W' rows into tensor memory
  return launch_lmhead<MODE_DW>(X, W, a, (cudaStream_t)stream);
}
