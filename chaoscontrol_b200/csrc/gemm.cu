// Generic bf16 GEMM for sm_100a: TMA-fed shared-memory ring -> tcgen05.mma
// (single-thread issue, fp32 accumulators in TMEM, two accumulators so the
// epilogue of tile i overlaps the MMAs of tile i+1) -> tcgen05.ld epilogue
// with the trunk's elementwise work fused in (RMSNorm row scale, SiLU and its
// derivative, residual add with row sum-of-squares, RMSNorm backward).
//
// One persistent CTA per SM walks tiles round-robin.  Warp roles:
//   warp 0      TMA producer (one lane)
//   warp 1      TMEM owner + MMA issuer (one lane)
//   warps 2..9  epilogue; warp w reads TMEM lanes [32*(w%4), 32*(w%4)+32), the
//               two warps of a lane quadrant take alternate 64-column groups
//
// CG = 2 runs the same pipeline on a CTA pair (2-CTA cluster, tcgen05 cta_group::2): the pair owns a
// 256-row x BN tile, each CTA stages its own 128 rows of A and HALF of the B tile, the leader CTA's
// MMA thread issues 256-row instructions that read both CTAs' shared memory, each CTA drains its own
// 128 accumulator rows.  The trunk GEMMs are bound by the weight tile every CTA re-reads from L2 for
// each row tile (about 8 TB/s of L2 -> SM traffic measured at N = 1024, K = 256), and the pair halves
// exactly that stream.  Nothing is multicast: each CTA issues its own plain TMA loads.
//
// Replaces the library GEMM call sites of the reference trunk
// (src/chaoscontrol/core.py:453-474, 503, 545, 327-335) and the batched
// Newton-Schulz matmuls (src/chaoscontrol/optim/muon.py:42-45).
#include "ptx.cuh"
#include "ccb_api.h"
#include "runtime.h"
#include <string.h>

namespace ccb {

constexpr int BM = 128;
constexpr int BK = 64;                       // 64 bf16 = one 128-byte swizzle row
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KiB
constexpr int EPI_PARTS = 2;                  // epilogue warps per TMEM lane quadrant
constexpr int EPI_WARPS = 4 * EPI_PARTS;
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;

struct GemmKArgs {
  int M, N, K;
  int batch, splits, tiles_m, tiles_n, kblocks, kper;
  int epi, out_fp32, ss_atomic, tma_store;
  long long ldc, c_batch, c_split, ldcin, cin_batch, ldr;
  void* C;
  void* C2;
  const void* Cin;
  const void* R1;
  const void* R2;
  const float* rowss;
  float* ss_out;
  float alpha, beta, inv_dim, eps;
  int* status;
  int f8, bk;                 // 8-bit operands: kind::f8f6f4, 128 elements per 128-byte row
  uint32_t idesc_f8;
  const float* dscale_a;
  const float* dscale_b;
  const void* bias;
  // pair: one CTA computes both 256-column halves of a row block into the two
  // accumulators and the epilogue treats them as one 512-column tile
  int pair;
  const long long* targets;
  const float* lse;
  const float* rowweight;
  float2* part_out;
  float* zt_out;
  // stage-isolation switches for bottleneck analysis (results are then wrong by design):
  // 1 = epilogue skips its TMA / global stores, 2 = epilogue skips math and staging too,
  // 4 = epilogue skips the TMEM loads as well, 8 = the MMA issuer issues no MMAs
  int dbg;
  int l2pf;     // L2 prefetch: 1 = A tiles two tiles ahead (producer), 2 = next tile's epilogue operands
};

// bf16 outputs leave through shared-memory staging tiles and TMA stores: each
// epilogue warp owns two 32-row x 64-column (4 KiB, 128B-swizzled) buffers.
constexpr int STG_BUF_BYTES = 32 * 128;
constexpr int STG_BUFS_PER_WARP = 2;
constexpr int STG_BYTES = EPI_WARPS * STG_BUFS_PER_WARP * STG_BUF_BYTES;   // 64 KiB

// BRES ("B resident"): every tile a CTA walks has the same N coordinate whenever the grid is a
// multiple of the N-tile count, so for K <= 256 the whole [BN x K] weight tile (128 KiB) is loaded ONCE
// and stays in shared memory; only A streams, through a four-stage ring of 16 KiB.  Measured on the
// packed-projection GEMM (N = 1024, K = 256) with MMAs and epilogue switched off, the bare load ring
// of the streaming layout (192 KiB per tile, 144 KiB in flight, 1.4 us per stage round trip) takes as
// long as the whole HBM roofline of the kernel, and MMA and epilogue time then ADD to it because no
// further tile fits in flight; with B resident a tile needs 64 KiB and a full tile of A is in flight.
// The staging area shrinks to one buffer per epilogue warp to make room.
constexpr int BRES_KBLOCKS = 4;
// On a CTA pair each CTA keeps only its half of the weight tile (BN / 2 rows), so the resident layout has
// room to spare: BRES = 1 holds K <= 256 (64 KiB) and gives the A ring eight stages (two tiles of A in
// flight per CTA); BRES = 2 holds K <= 512 (128 KiB) with a four-stage ring, which takes the weight
// re-reads (256 KiB from L2 per 128-row tile on a single CTA) out of the K = 512 input-gradient GEMMs.
// Measured at 524 288 rows against the single-CTA kernels (bit-identical outputs): packed projection
// 0.437 vs 0.331 ms, out_proj + residual 0.197 vs 0.177, dSiLU 0.367 vs 0.320, RMSNorm backward (K = 512)
// 0.386 vs 0.361, whole step 33.9 vs 33.3 ms.  A pair couples two SMs' load streams to one MMA issuer, so
// either CTA's late stage stalls both; on these memory-bound shapes that costs more than the saved weight
// traffic.  Kept behind ccb_gemm_pair_resident (default off), like the plain pair mode.

template <int BN, int CG = 1, int BRES = 0>
struct GemmCfg {
  static_assert(BRES == 0 || BRES == 1 || (BRES == 2 && CG == 2), "BRES 2 (K <= 512 resident) needs a CTA pair");
  static constexpr int B_ROWS = BN / CG;                  // rows of the B tile this CTA stages
  static constexpr int B_STAGE_BYTES = B_ROWS * BK * 2;
  static constexpr int RES_KBLOCKS = BRES == 2 ? 8 : BRES_KBLOCKS;   // k-blocks of the resident tile
  static constexpr int STAGES = BRES ? ((CG == 2 && BRES == 1) ? 8 : 4) : ((BN == 256 && CG == 1) ? 3 : 4);
  static constexpr int TMEM_COLS = 2 * BN;   // 512 or 256: powers of two
  static constexpr int STG_BUFS = BRES ? 1 : STG_BUFS_PER_WARP;
  static constexpr int A_OFF = BRES ? RES_KBLOCKS * B_STAGE_BYTES : 0;
  static constexpr int STG_OFF = BRES ? A_OFF + STAGES * A_STAGE_BYTES : STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
  static constexpr int BAR_OFF = STG_OFF + EPI_WARPS * STG_BUFS * STG_BUF_BYTES;
  static constexpr int XCH_OFF = BAR_OFF + 256;     // per-row partials exchanged between warps
  // the resident layout has no room for alignment slack: its kernel checks that the dynamic
  // shared-memory window starts on a 1 KiB boundary (it does when the kernel has no static shared memory)
  static constexpr int SMEM_BYTES = (BRES ? 0 : 1024) + XCH_OFF + 2 * EPI_PARTS * BM * 4;
  static_assert(2 * STAGES * 8 + 56 <= 256, "barrier block overflows its 256 bytes");
  static_assert(SMEM_BYTES <= 227 * 1024, "tile configuration exceeds the per-CTA shared memory limit");
};

__device__ __forceinline__ void load_bf16x32(const __nv_bfloat16* src, float (&v)[32], int nvalid) {
  if (nvalid >= 32) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 q = __ldg(s4 + i);
      float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z),
             f3 = unpack_bf16x2(q.w);
      v[i * 8 + 0] = f0.x; v[i * 8 + 1] = f0.y; v[i * 8 + 2] = f1.x; v[i * 8 + 3] = f1.y;
      v[i * 8 + 4] = f2.x; v[i * 8 + 5] = f2.y; v[i * 8 + 6] = f3.x; v[i * 8 + 7] = f3.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = (i < nvalid) ? __bfloat162float(src[i]) : 0.f;
  }
}

__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float (&v)[32], int nvalid) {
  if (nvalid >= 32) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 q;
      q.x = pack_bf16x2(v[i * 8 + 0], v[i * 8 + 1]);
      q.y = pack_bf16x2(v[i * 8 + 2], v[i * 8 + 3]);
      q.z = pack_bf16x2(v[i * 8 + 4], v[i * 8 + 5]);
      q.w = pack_bf16x2(v[i * 8 + 6], v[i * 8 + 7]);
      d4[i] = q;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < nvalid) dst[i] = __float2bfloat16(v[i]);
  }
}

__device__ __forceinline__ void store_f32x32(float* dst, const float (&v)[32], int nvalid) {
  if (nvalid >= 32) {
    float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
    for (int i = 0; i < 8; ++i) d4[i] = make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < nvalid) dst[i] = v[i];
  }
}

struct TileCoord {
  int b, sp, m0, n0, kb0, kb1;
};

__device__ __forceinline__ TileCoord decode_tile(const GemmKArgs& p, int tile, int BN, int bm = BM) {
  TileCoord t;
  int tn = tile % p.tiles_n;
  int r = tile / p.tiles_n;
  int tm = r % p.tiles_m;
  r /= p.tiles_m;
  t.sp = r % p.splits;
  t.b = r / p.splits;
  t.m0 = tm * bm;
  t.n0 = tn * BN;
  t.kb0 = t.sp * p.kper;
  t.kb1 = min(p.kblocks, t.kb0 + p.kper);
  return t;
}

constexpr float GEMM_LOG2E = 1.4426950408889634f;
constexpr float GEMM_LN2 = 0.6931471805599453f;

__device__ __forceinline__ float gemm_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// LM = 1 compiles the LM-head epilogues (LSE_PART, CE_GRAD) instead of the trunk set.
// EPI_T >= 0 fixes the epilogue at compile time (the hot trunk epilogues: no dispatch, less
// code, fewer live registers in the chunk loop); EPI_T = -1 reads it from the arguments.
template <int BN, int A_MN, int B_MN, int LM, int EPI_T, int CG, int BRES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmC2,
            const GemmKArgs p) {
  using Cfg = GemmCfg<BN, CG, BRES>;
  static_assert(CG == 1 || (A_MN == 0 && LM == 0), "CTA pairs: K-major A, trunk epilogues");
  static_assert(BRES == 0 || (A_MN == 0 && LM == 0), "resident B: K-major A, trunk epilogues");
  static_assert(BRES == 0 || EPI_T != CCB_EPI_ROWSCALE_SILU, "resident B has one staging buffer per warp: one output");
  constexpr int STG_BUFS = Cfg::STG_BUFS;
  // pair geometry: `cta_rank` 0 is the leader (issues the MMAs, owns the barriers the loads and the
  // epilogues of both CTAs report to); the pair walks tiles of BM * CG rows together
  const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
  const int walker = (int)blockIdx.x / CG, n_walkers = (int)gridDim.x / CG;
  constexpr int BM_TILE = BM * CG;
  const int epi_k = (EPI_T >= 0) ? EPI_T : p.epi;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int B_STAGE_BYTES = Cfg::B_STAGE_BYTES;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = BRES ? smem_raw
                       : reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                    ~static_cast<uintptr_t>(1023));
  if (BRES && (smem_u32(smem) & 1023u) != 0u) {   // the swizzled tiles need a 1 KiB aligned base
    if (threadIdx.x == 0) atomicCAS(p.status, CCB_OK, CCB_ERR_BAD_SHAPE);
    return;
  }
  uint8_t* sA = smem + Cfg::A_OFF;
  uint8_t* sB = BRES ? smem : smem + STAGES * A_STAGE_BYTES;     // resident: k-block kb at sB + kb * B_STAGE_BYTES
  uint8_t* sStage = smem + Cfg::STG_OFF;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* xbar = tempty_bar + 2;
  uint64_t* bres_bar = xbar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bres_bar + 1);
  float* xch = reinterpret_cast<float*>(smem + Cfg::XCH_OFF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.batch * p.splits * p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], EPI_WARPS * CG);      // the leader's collects both CTAs' epilogue warps
    }
    mbar_init(xbar, EPI_WARPS);
    mbar_init(bres_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    if (CG == 2) {
      tmem_alloc_cg2(tmem_slot, Cfg::TMEM_COLS);      // one warp of EACH CTA of the pair
      tmem_relinquish_cg2();
    } else {
      tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (CG == 2) cluster_sync_all();     // both CTAs' barriers exist before either touches the peer's
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Barriers, tensor memory and descriptors are set up: everything above overlaps the tail of the
  // previous kernel when this one was launched as a programmatic dependent.  Nothing below runs before
  // that kernel has finished; our own successor may be scheduled onto SMs as our CTAs leave them.
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (BRES && walker < total_tiles) {
        // the weight tile of this CTA's N coordinate, all k-blocks, once
        const TileCoord t0 = decode_tile(p, walker, BN, BM_TILE);
        if (CG == 2) {
          // each CTA loads its half of the tile into its own shared memory; both report to the leader's
          // barrier, which expects the bytes of the pair
          if (cta_rank == 0) mbar_arrive_expect_tx(bres_bar, (uint32_t)(2 * p.kblocks * B_STAGE_BYTES));
          const uint32_t rb = mapa_shared(smem_u32(bres_bar), 0);
          for (int kb = 0; kb < p.kblocks; ++kb) {
            uint8_t* b_dst = sB + kb * B_STAGE_BYTES;
            if (B_MN == 0) {
              tma_load_3d_cg2(b_dst, &tmB, rb, kb * p.bk, t0.n0 + Cfg::B_ROWS * (int)cta_rank, 0);
            } else {
#pragma unroll
              for (int j = 0; j < Cfg::B_ROWS / 64; ++j)
                tma_load_3d_cg2(b_dst + j * 8192, &tmB, rb, t0.n0 + Cfg::B_ROWS * (int)cta_rank + 64 * j,
                                kb * BK, 0);
            }
          }
        } else {
        mbar_arrive_expect_tx(bres_bar, (uint32_t)(p.kblocks * B_STAGE_BYTES));
        for (int kb = 0; kb < p.kblocks; ++kb) {
          uint8_t* b_dst = sB + kb * B_STAGE_BYTES;
          if (B_MN == 0) {
            tma_load_3d(b_dst, &tmB, bres_bar, kb * p.bk, t0.n0, 0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(b_dst + j * 8192, &tmB, bres_bar, t0.n0 + 64 * j, kb * BK, 0);
          }
        }
        }
      }
      for (int tile = walker; tile < total_tiles && ok; tile += n_walkers) {
        TileCoord t = decode_tile(p, tile, BN, BM_TILE);
        for (int hn = 0; hn <= p.pair && ok; ++hn, t.n0 += BN)
        for (int kb = t.kb0; kb < t.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status)) { ok = false; break; }
          uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
          uint8_t* b_dst = sB + stage * B_STAGE_BYTES;
          if (A_MN == 0 && CG == 1 && !p.pair && (p.l2pf & 1)) {
            // the same k-block of the tile after next: into L2 now, so that its load is an L2 hit
            const int t2 = tile + 2 * n_walkers;
            if (t2 < total_tiles) {
              const TileCoord tn = decode_tile(p, t2, BN, BM_TILE);
              tma_prefetch_3d(&tmA, (tn.kb0 + (kb - t.kb0)) * p.bk, tn.m0, tn.b);
            }
          }
          if (BRES) {
            if (CG == 2) {
              if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * A_STAGE_BYTES);
              tma_load_3d_cg2(a_dst, &tmA, mapa_shared(smem_u32(&full_bar[stage]), 0), kb * p.bk,
                              t.m0 + BM * (int)cta_rank, t.b);
            } else {
              mbar_arrive_expect_tx(&full_bar[stage], A_STAGE_BYTES);
              tma_load_3d(a_dst, &tmA, &full_bar[stage], kb * p.bk, t.m0, t.b);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            continue;
          }
          if (CG == 2) {
            // the stage is complete when BOTH CTAs' halves have landed: all four loads report to the
            // leader's barrier, which expects the bytes of the pair
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * (A_STAGE_BYTES + B_STAGE_BYTES));
            const uint32_t fb = mapa_shared(smem_u32(&full_bar[stage]), 0);
            tma_load_3d_cg2(a_dst, &tmA, fb, kb * p.bk, t.m0 + BM * (int)cta_rank, t.b);
            if (B_MN == 0) {
              tma_load_3d_cg2(b_dst, &tmB, fb, kb * p.bk, t.n0 + Cfg::B_ROWS * (int)cta_rank, t.b);
            } else {
#pragma unroll
              for (int j = 0; j < Cfg::B_ROWS / 64; ++j)
                tma_load_3d_cg2(b_dst + j * 8192, &tmB, fb, t.n0 + Cfg::B_ROWS * (int)cta_rank + 64 * j,
                                kb * BK, t.b);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            continue;
          }
          mbar_arrive_expect_tx(&full_bar[stage], A_STAGE_BYTES + B_STAGE_BYTES);
          if (A_MN == 0) {
            tma_load_3d(a_dst, &tmA, &full_bar[stage], kb * p.bk, t.m0, t.b);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(a_dst + j * 8192, &tmA, &full_bar[stage], t.m0 + 64 * j, kb * BK, t.b);
          }
          if (B_MN == 0) {
            tma_load_3d(b_dst, &tmB, &full_bar[stage], kb * p.bk, t.n0, t.b);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(b_dst + j * 8192, &tmB, &full_bar[stage], t.n0 + 64 * j, kb * BK, t.b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Aborting: give loads already in flight a bounded chance to land
        // before the CTA's shared memory is released.
        uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM_TILE, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      if (BRES && walker < total_tiles) {
        ok = mbar_wait(bres_bar, 0u, abort_flag, p.status);
        tc_fence_after_sync();
      }
      for (int tile = walker; tile < total_tiles && ok; tile += n_walkers, ++it) {
        TileCoord t = decode_tile(p, tile, BN, BM_TILE);
        const int acc = p.pair ? 0 : (it & 1);
        const uint32_t acc_phase = (uint32_t)(p.pair ? it : (it >> 1)) & 1u;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after_sync();
        for (int hn = 0; hn <= p.pair && ok; ++hn) {
        const uint32_t d_tmem = tmem_base + (uint32_t)((p.pair ? hn : acc) * BN);
        for (int kb = t.kb0; kb < t.kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(sA + stage * A_STAGE_BYTES);
          const uint32_t b_base = smem_u32(sB + (BRES ? (kb - t.kb0) : stage) * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc(a_base + k * 2048, 8192, 1024)
                                        : make_smem_desc(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_base + k * 2048, 8192, 1024)
                                        : make_smem_desc(b_base + k * 32, 16, 1024);
            const uint32_t accum = (kb > t.kb0 || k > 0) ? 1u : 0u;
            if (p.dbg & 8) continue;
            if (CG == 2) umma_bf16_cg2(d_tmem, adesc, bdesc, idesc, accum);   // 256 rows over the pair
            else if (p.f8) umma_f8(d_tmem, adesc, bdesc, p.idesc_f8, accum);   // 32 one-byte k per MMA
            else umma_bf16(d_tmem, adesc, bdesc, idesc, accum);           // 16 two-byte k per MMA
          }
          // stage reusable once these MMAs retire (in both CTAs of a pair)
          if (CG == 2) umma_commit_cg2(&empty_bar[stage]); else umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        }
        if (ok) { if (CG == 2) umma_commit_cg2(&tfull_bar[acc]); else umma_commit(&tfull_bar[acc]); }
      }
    }
  } else {
    // ------------------------------ epilogue -----------------------------------
    // Two warps share each TMEM lane quadrant; they take alternate 64-column
    // groups of the tile, so two warps per scheduler hide each other's
    // TMEM-load, global-load and store-drain latency.
    const int q = warp & 3;                 // TMEM lane quadrant of this warp
    const int part = (warp - 2) >> 2;       // which 64-column groups this warp takes
    const int row_in_tile = q * 32 + lane;
    int it = 0;
    int stg_n = 0;          // TMA stores issued by this warp (selects the staging buffer)
    uint32_t xphase = 0;
    bool ok = true;
    // all eight epilogue warps meet here (bounded); false = abort
    auto rendezvous = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(xbar);
      const bool w = mbar_wait(xbar, xphase, abort_flag, p.status);
      xphase ^= 1u;
      return __all_sync(0xffffffffu, w);
    };
    for (int tile = walker; tile < total_tiles && ok; tile += n_walkers, ++it) {
      TileCoord t = decode_tile(p, tile, BN, BM_TILE);
      t.m0 += BM * (int)cta_rank;             // this CTA's 128 rows of the pair's tile
      const int acc = p.pair ? 0 : (it & 1);
      const uint32_t acc_phase = (uint32_t)(p.pair ? it : (it >> 1)) & 1u;
      const uint32_t t_addr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(q * 32) << 16);
      const int m = t.m0 + row_in_tile;
      const bool row_ok = m < p.M;
      const long long out_off = (long long)t.b * p.c_batch + (long long)t.sp * p.c_split +
                                (long long)m * p.ldc;
      float rs = 1.f;
      if (p.rowss != nullptr && row_ok) rs = rsqrtf(p.rowss[m] * p.inv_dim + p.eps);
      float alpha = p.alpha;
      if (p.dscale_a != nullptr) alpha *= __ldg(p.dscale_a);
      if (p.dscale_b != nullptr) alpha *= __ldg(p.dscale_b);
      const int ncols = min(p.pair ? 2 * BN : BN, p.N - t.n0);   // valid columns in this tile
      const int nchunks = (ncols + 31) >> 5;
      // k-th 32-column chunk of this warp: groups part, part+2, ... two chunks each
      auto chunk_of = [&](int k) { return (((k >> 1) * EPI_PARTS + part) << 1) + (k & 1); };
      int nmine = 0;
      while (chunk_of(nmine) < nchunks) ++nmine;
      float* xch_acc = xch + acc * (EPI_PARTS * BM);

      // TMA-store path: 64-column groups staged in this warp's swizzled buffers
      uint8_t* my_stage = sStage + (warp - 2) * (STG_BUFS * STG_BUF_BYTES);
      const bool two_out = (epi_k == CCB_EPI_ROWSCALE_SILU);
      auto stage_write = [&](uint8_t* buf, int half, const float (&vals)[32]) {
        uint8_t* row = buf + lane * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int slot = (half * 4 + j) ^ (lane & 7);
          *reinterpret_cast<uint4*>(row + slot * 16) =
              make_uint4(pack_bf16x2(vals[j * 8 + 0], vals[j * 8 + 1]),
                         pack_bf16x2(vals[j * 8 + 2], vals[j * 8 + 3]),
                         pack_bf16x2(vals[j * 8 + 4], vals[j * 8 + 5]),
                         pack_bf16x2(vals[j * 8 + 6], vals[j * 8 + 7]));
        }
      };

      // Epilogue operands (residual / pre-activation / x / dres) do not depend on
      // the accumulator, so their loads are issued one chunk ahead -- the first
      // before this tile's MMAs have even finished -- and the other warp of the
      // scheduler covers what latency is left.
      const __nv_bfloat16* aux1_row = nullptr;
      if (epi_k == CCB_EPI_STORE) {
        if (p.Cin != nullptr)
          aux1_row = reinterpret_cast<const __nv_bfloat16*>(p.Cin) + (long long)t.b * p.cin_batch +
                     (long long)m * p.ldcin;
      } else if (p.R1 != nullptr) {
        aux1_row = reinterpret_cast<const __nv_bfloat16*>(p.R1) + (long long)m * p.ldr;
      }
      const __nv_bfloat16* aux2_row =
          (epi_k == CCB_EPI_RMSBWD && p.R2 != nullptr)
              ? reinterpret_cast<const __nv_bfloat16*>(p.R2) + (long long)m * p.ldr : nullptr;
      const int aux1_total = aux1_row ? nmine * (epi_k == CCB_EPI_RMSBWD ? 2 : 1) : 0;
      const int aux2_total = aux2_row ? nmine : 0;
      auto aux_issue = [&](const __nv_bfloat16* rowp, int s_idx, int total, uint4 (&qv)[4]) {
        if (rowp == nullptr || !row_ok || s_idx >= total) return;
        const int c = chunk_of(s_idx % nmine);
        const int n = t.n0 + c * 32;
        if (n + 32 <= p.N) {
          const uint4* src = reinterpret_cast<const uint4*>(rowp + n);
#pragma unroll
          for (int i = 0; i < 4; ++i) qv[i] = __ldg(src + i);
        }
      };
      auto aux_get = [&](const __nv_bfloat16* rowp, int c, const uint4 (&qv)[4], float (&vals)[32]) {
        const int n = t.n0 + c * 32;
        if (rowp == nullptr || !row_ok) {
#pragma unroll
          for (int i = 0; i < 32; ++i) vals[i] = 0.f;
        } else if (n + 32 <= p.N) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f0 = unpack_bf16x2(qv[i].x), f1 = unpack_bf16x2(qv[i].y),
                         f2 = unpack_bf16x2(qv[i].z), f3 = unpack_bf16x2(qv[i].w);
            vals[i * 8 + 0] = f0.x; vals[i * 8 + 1] = f0.y; vals[i * 8 + 2] = f1.x; vals[i * 8 + 3] = f1.y;
            vals[i * 8 + 4] = f2.x; vals[i * 8 + 5] = f2.y; vals[i * 8 + 6] = f3.x; vals[i * 8 + 7] = f3.y;
          }
        } else {
          load_bf16x32(rowp + n, vals, p.N - n);
        }
      };
      if ((p.l2pf & 2) && (aux1_row != nullptr || aux2_row != nullptr)) {
        // the operands the NEXT tile's epilogue will read row by row: into L2 now (one 128-byte line
        // per 64-column group of this warp), so those loads do not pay the DRAM latency in the loop
        const int t1 = tile + n_walkers;
        if (t1 < total_tiles) {
          TileCoord tn = decode_tile(p, t1, BN, BM_TILE);
          const int mn = tn.m0 + BM * (int)cta_rank + row_in_tile;
          if (mn < p.M) {
            for (int k = 0; k < nmine; k += 2) {
              const int n = tn.n0 + chunk_of(k) * 32;
              if (n < p.N) {
                if (aux1_row != nullptr)
                  prefetch_l2(aux1_row + (long long)(mn - m) * (epi_k == CCB_EPI_STORE ? p.ldcin : p.ldr) + n +
                              (long long)(epi_k == CCB_EPI_STORE ? (tn.b - t.b) * p.cin_batch : 0));
                if (aux2_row != nullptr) prefetch_l2(aux2_row + (long long)(mn - m) * p.ldr + n);
              }
            }
          }
        }
      }
      uint4 a1_cur[4], a2_cur[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a1_cur[i] = a2_cur[i] = make_uint4(0, 0, 0, 0);
      aux_issue(aux1_row, 0, aux1_total, a1_cur);
      aux_issue(aux2_row, 0, aux2_total, a2_cur);
      int a1_s = 0, a2_s = 0;      // stream positions of a1_cur / a2_cur
      // called after aux_get has unpacked the current chunk: refill for the next
      auto a1_advance = [&]() {
        ++a1_s;
        aux_issue(aux1_row, a1_s, aux1_total, a1_cur);
      };
      auto a2_advance = [&]() {
        ++a2_s;
        aux_issue(aux2_row, a2_s, aux2_total, a2_cur);
      };

      {
        // warp-uniform result: the TMEM loads below are warp-collective
        const bool w = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status);
        if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
      }
      tc_fence_after_sync();

      // LM-head epilogues: log2-domain constants and running (max, sum)
      float lm_c1 = 0.f, lm_c2 = 0.f, lm_gs = 0.f, run_m = -INFINITY, run_s = 0.f, lm_zt = 0.f;
      int lm_tgt = -1;
      bool lm_hit = false;
      if (LM && row_ok) {
        lm_c1 = rs * GEMM_LOG2E;
        lm_tgt = (int)p.targets[m];
        if (epi_k == CCB_EPI_CE_GRAD) {
          lm_c2 = p.lse[m] * GEMM_LOG2E;
          lm_gs = alpha * rs * (p.rowweight ? p.rowweight[m] : 1.f);
        }
      }

      float row_acc = 0.f;   // RESID_SS: sum of squares; RMSBWD: dot(acc, x)
      if (!LM && epi_k == CCB_EPI_RMSBWD) {
        for (int k = 0; k < nmine; ++k) {
          const int c = chunk_of(k);
          uint32_t r[32];
          __syncwarp();
          tmem_ld32(t_addr + c * 32, r);
          tmem_ld_wait();
          {
            float x[32];
            aux_get(aux1_row, c, a1_cur, x);
            a1_advance();
#pragma unroll
            for (int i = 0; i < 32; ++i) row_acc += __uint_as_float(r[i]) * x[i];
          }
        }
        // the row's dot product spans both warps of the quadrant
        xch_acc[part * BM + row_in_tile] = row_acc;
        if (!rendezvous()) { ok = false; break; }
        row_acc += xch_acc[(part ^ 1) * BM + row_in_tile];
        row_acc *= rs * rs * p.inv_dim;
      }

      // the staging buffers a 64-column group will use must have been read out by their last store
      auto store_gate = [&](int c) {
        if (p.tma_store && (c & 1) == 0) {
          __syncwarp();
          if (lane == 0) {
            // two outputs, or one staging buffer per warp: every earlier store must have left it
            if (two_out || STG_BUFS == 1) tma_store_wait_read<0>(); else tma_store_wait_read<1>();
          }
          __syncwarp();
        }
      };
      // one 32-column chunk whose accumulator values are already in `r`
      auto chunk_body = [&](int c, const uint32_t (&r)[32]) {
        if (p.dbg & 2) return;
        if (!row_ok && !p.tma_store) return;
        const int n = t.n0 + c * 32;
        const int nvalid = p.N - n;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);

        if (LM) {
          const int tl = lm_tgt - n;
          if (epi_k == CCB_EPI_LSE_PART) {
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < nvalid) mx = fmaxf(mx, v[i]);
            const float new_m = fmaxf(run_m, mx * lm_c1);
            float sacc = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (i < nvalid) sacc += gemm_ex2(fmaf(v[i], lm_c1, -new_m));
              if (i == tl) { lm_zt = v[i] * rs; lm_hit = true; }
            }
            run_s = run_s * gemm_ex2(run_m - new_m) + sacc;
            run_m = new_m;
            return;   // nothing is stored per column
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float z = fmaf(v[i], lm_c1, -lm_c2);
            float pr = gemm_ex2(z);
            if (i == tl) { pr -= 1.f; lm_zt = -z * GEMM_LN2; lm_hit = true; }
            v[i] = pr * lm_gs;
          }
        } else
        switch (epi_k) {
          case CCB_EPI_STORE: {
            if (p.Cin != nullptr) {
              float cin[32];
              aux_get(aux1_row, c, a1_cur, cin);
              a1_advance();
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = alpha * v[i] + p.beta * cin[i];
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] *= alpha;
            }
            if (p.bias != nullptr) {
              float bv[32];
              load_bf16x32(reinterpret_cast<const __nv_bfloat16*>(p.bias) + n, bv, nvalid);
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] += bv[i];
            }
          } break;
          case CCB_EPI_ROWSCALE: {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= rs;
          } break;
          case CCB_EPI_ROWSCALE_SILU: {
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              v[i] *= rs;
              // silu of the bf16-rounded pre-activation, as the unfused path would see it
              float u = __bfloat162float(__float2bfloat16(v[i]));
              f[i] = u * sigmoidf_fast(u);
            }
            if (p.tma_store) {
              stage_write(my_stage + STG_BUF_BYTES, c & 1, f);
            } else {
              store_bf16x32(reinterpret_cast<__nv_bfloat16*>(p.C2) + out_off + n, f, nvalid);
            }
          } break;
          case CCB_EPI_RESID_SS: {
            float res[32];
            aux_get(aux1_row, c, a1_cur, res);
            a1_advance();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              v[i] = __bfloat162float(__float2bfloat16(v[i] + res[i]));
              if (i < nvalid) row_acc += v[i] * v[i];
            }
          } break;
          case CCB_EPI_DSILU: {
            float u[32];
            aux_get(aux1_row, c, a1_cur, u);
            a1_advance();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float s = sigmoidf_fast(u[i]);
              v[i] = v[i] * (s * (1.f + u[i] * (1.f - s))) * rs;
            }
          } break;
          case CCB_EPI_RMSBWD: {
            float x[32], dres[32];
            aux_get(aux1_row, c, a1_cur, x);
            a1_advance();
            aux_get(aux2_row, c, a2_cur, dres);
            a2_advance();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = dres[i] + v[i] - x[i] * row_acc;
          } break;
          default: break;
        }
        if (p.tma_store) {
          uint8_t* buf = my_stage + ((two_out || STG_BUFS == 1) ? 0 : (stg_n & 1) * STG_BUF_BYTES);
          stage_write(buf, c & 1, v);
          if ((c & 1) == 1 || c == nchunks - 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && !(p.dbg & 1)) {
              const int col = t.n0 + (c >> 1) * 64;
              const int row = t.m0 + q * 32;
              tma_store_3d(&tmC, buf, col, row, t.b);
              tma_store_commit();
              if (two_out) {
                tma_store_3d(&tmC2, my_stage + STG_BUF_BYTES, col, row, t.b);
                tma_store_commit();
              }
            }
            ++stg_n;
          }
        } else if (p.out_fp32) {
          store_f32x32(reinterpret_cast<float*>(p.C) + out_off + n, v, nvalid);
        } else {
          store_bf16x32(reinterpret_cast<__nv_bfloat16*>(p.C) + out_off + n, v, nvalid);
        }
      };
      // (Keeping the next chunk's TMEM load in flight behind a second register buffer was measured
      // slower here: 0.187 -> 0.199 ms on the row-scale GEMM; two warps per scheduler already
      // cover each other's TMEM latency.)
      for (int k = 0; k < nmine; ++k) {
        const int c = chunk_of(k);
        uint32_t r[32];
        store_gate(c);
        __syncwarp();
        if (!(p.dbg & 4)) {
          tmem_ld32(t_addr + c * 32, r);
          tmem_ld_wait();
        }
        chunk_body(c, r);
      }
      if (LM) {
        if (row_ok) {
          if (epi_k == CCB_EPI_LSE_PART)
            p.part_out[(long long)((t.n0 / BN) * EPI_PARTS + part) * p.M + m] = make_float2(run_m, run_s);
          if (lm_hit && p.zt_out != nullptr) p.zt_out[m] = lm_zt;
        }
      } else if (epi_k == CCB_EPI_RESID_SS && p.ss_out != nullptr) {
        // one value per row and tile: the second warp of the quadrant hands its
        // half over, so a row split over two N tiles gets exactly two (commutative,
        // hence order-independent) atomic adds
        if (part != 0) xch_acc[part * BM + row_in_tile] = row_acc;
        if (!rendezvous()) { ok = false; break; }
        if (part == 0 && row_ok) {
          const float tot = row_acc + xch_acc[BM + row_in_tile];
          if (p.ss_atomic) atomicAdd(p.ss_out + m, tot); else p.ss_out[m] = tot;
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (CG == 2) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[acc]), 0));
        else mbar_arrive(&tempty_bar[acc]);
      }
    }
    // all of this warp's stores must have left shared memory and landed
    if (p.tma_store && lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  // a pair leaves together: the leader's barriers take remote arrivals and its MMAs read the
  // follower's shared memory until the last tile
  if (CG == 2) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    if (CG == 2) tmem_dealloc_cg2(tmem_base, Cfg::TMEM_COLS); else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
static int g_gemm_dbg = 0;
// -1: per epilogue, as measured at 262 144 rows on a B200 -- prefetching the next tile's epilogue
// operands helps the residual and dSiLU GEMMs (0.107 -> 0.099 ms, 0.193 -> 0.177 ms) and hurts the
// RMSNorm-backward GEMM, whose K = 512 operand stream already fills the L2 path (0.191 -> 0.202 ms);
// prefetching A helps only the streaming layout (0.206 -> 0.183 ms), which the resident layout beats.
static int g_gemm_l2pf = -1;
static int g_gemm_pdl = 0;

template <int BN, int A_MN, int B_MN, int LM = 0, int EPI_T = -1, int CG = 1, int BRES = 0>
static int launch_gemm(const CcbGemmArgs* a, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, CG, BRES>;
  static bool attr_set[16] = {false};
  static int max_pairs[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_kernel<BN, A_MN, B_MN, LM, EPI_T, CG, BRES>;
  if (!attr_set[dev & 15]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return set_error("cudaFuncSetAttribute(gemm): %s", cudaGetErrorString(e));
    if (CG == 2) {
      // how many 2-CTA clusters of this kernel the device runs at once (one CTA per SM by shared memory)
      cudaLaunchConfig_t qc = {};
      qc.gridDim = dim3((unsigned)(ccb_num_sms() / 2 * 2));
      qc.blockDim = dim3(GEMM_THREADS);
      qc.dynamicSmemBytes = Cfg::SMEM_BYTES;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      qc.attrs = qa; qc.numAttrs = 1;
      int n = 0;
      e = cudaOccupancyMaxActiveClusters(&n, kern, &qc);
      if (e != cudaSuccess || n < 1)
        return set_error("cudaOccupancyMaxActiveClusters(gemm pair): %s", cudaGetErrorString(e));
      max_pairs[dev & 15] = n;
    }
    attr_set[dev & 15] = true;
  }
  if (CG == 2 && (a->a_fp8 != 0 || A_MN != 0))
    return set_error("ccb_gemm: CTA pairs take K-major bf16 A operands");
  CUtensorMap tmA, tmB;
  const bool f8 = a->a_fp8 != 0;
  if (f8) {
    // one-byte operands: a 128-byte swizzle row holds 128 k-elements
    if (A_MN != 0 || B_MN != 0) return set_error("ccb_gemm: 8-bit operands must be K-major");
    if (make_tmap_u8_3d(&tmA, a->A, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->batch,
                        (uint64_t)a->lda, (uint64_t)a->a_batch, 128, BM)) return -1;
    if (make_tmap_u8_3d(&tmB, a->B, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->batch,
                        (uint64_t)a->ldb, (uint64_t)a->b_batch, 128, BN)) return -1;
  } else {
  if (A_MN == 0) {
    if (make_tmap_bf16_3d(&tmA, a->A, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->batch,
                          (uint64_t)a->lda, (uint64_t)a->a_batch, BK, BM)) return -1;
  } else {
    if (make_tmap_bf16_3d(&tmA, a->A, (uint64_t)a->M, (uint64_t)a->K, (uint64_t)a->batch,
                          (uint64_t)a->lda, (uint64_t)a->a_batch, 64, BK)) return -1;
  }
  if (B_MN == 0) {
    if (make_tmap_bf16_3d(&tmB, a->B, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->batch,
                          (uint64_t)a->ldb, (uint64_t)a->b_batch, BK, BN / CG)) return -1;
  } else {
    if (make_tmap_bf16_3d(&tmB, a->B, (uint64_t)a->N, (uint64_t)a->K, (uint64_t)a->batch,
                          (uint64_t)a->ldb, (uint64_t)a->b_batch, 64, BK)) return -1;
  }
  }
  GemmKArgs p;
  p.f8 = f8 ? 1 : 0;
  p.bk = f8 ? 128 : BK;
  p.idesc_f8 = make_idesc_f8(BM, BN, (int)a->a_fp8 - 1, (int)a->b_fp8 - 1);
  p.dscale_a = a->dscale_a; p.dscale_b = a->dscale_b; p.bias = a->bias;
  // bf16 outputs that keep rows 16-byte aligned go out through TMA stores
  CUtensorMap tmC, tmC2;
  const bool tma_ok = a->epi != CCB_EPI_LSE_PART &&
                      !a->out_fp32 && (a->ldc % 8 == 0) && (a->c_batch % 8 == 0) &&
                      ((reinterpret_cast<uintptr_t>(a->C) & 15) == 0) &&
                      (a->epi != CCB_EPI_ROWSCALE_SILU ||
                       (a->C2 != nullptr && (reinterpret_cast<uintptr_t>(a->C2) & 15) == 0));
  memset(&tmC, 0, sizeof(tmC));
  memset(&tmC2, 0, sizeof(tmC2));
  if (tma_ok) {
    if (make_tmap_bf16_3d(&tmC, a->C, (uint64_t)a->N, (uint64_t)a->M, (uint64_t)a->batch,
                          (uint64_t)a->ldc, (uint64_t)a->c_batch, 64, 32)) return -1;
    if (a->epi == CCB_EPI_ROWSCALE_SILU &&
        make_tmap_bf16_3d(&tmC2, a->C2, (uint64_t)a->N, (uint64_t)a->M, (uint64_t)a->batch,
                          (uint64_t)a->ldc, (uint64_t)a->c_batch, 64, 32)) return -1;
  }
  p.tma_store = tma_ok ? 1 : 0;
  p.M = (int)a->M; p.N = (int)a->N; p.K = (int)a->K;
  p.batch = (int)a->batch;
  p.tiles_m = (p.M + BM * CG - 1) / (BM * CG);
  p.tiles_n = (p.N + BN - 1) / BN;
  p.kblocks = (p.K + p.bk - 1) / p.bk;
  int splits = (int)(a->splits < 1 ? 1 : a->splits);
  if (splits > p.kblocks) splits = p.kblocks;
  p.kper = (p.kblocks + splits - 1) / splits;
  p.splits = (p.kblocks + p.kper - 1) / p.kper;
  if (p.splits != (int)(a->splits < 1 ? 1 : a->splits))
    return set_error("ccb_gemm: splits=%lld does not divide %d k-blocks evenly enough (got %d)",
                     (long long)a->splits, p.kblocks, p.splits);
  p.epi = (int)a->epi; p.out_fp32 = (int)a->out_fp32; p.ss_atomic = (int)a->ss_atomic;
  p.ldc = a->ldc; p.c_batch = a->c_batch; p.c_split = a->c_split;
  p.ldcin = a->ldcin; p.cin_batch = a->cin_batch; p.ldr = a->ldr;
  p.C = a->C; p.C2 = a->C2; p.Cin = a->Cin; p.R1 = a->R1; p.R2 = a->R2;
  p.rowss = a->rowss; p.ss_out = a->ss_out;
  p.alpha = a->alpha; p.beta = a->beta; p.inv_dim = a->inv_dim; p.eps = a->eps;
  p.status = ccb_status_ptr();
  p.dbg = g_gemm_dbg;
  p.l2pf = g_gemm_l2pf >= 0 ? g_gemm_l2pf
                            : ((a->epi == CCB_EPI_RESID_SS || a->epi == CCB_EPI_DSILU) ? 2 : 0);
  p.pair = 0;
  if (p.epi == CCB_EPI_RMSBWD && p.tiles_n != 1) {
    // the row reduction needs the whole row in tensor memory: both accumulators as one tile
    if (p.tiles_n != 2 || BN != 256)
      return set_error("ccb_gemm: RMSBWD epilogue needs N <= %d (got %d)", 2 * BN, p.N);
    p.pair = 1;
    p.tiles_n = 1;
  }
  p.targets = (const long long*)a->targets; p.lse = a->lse; p.rowweight = a->rowweight;
  p.part_out = (float2*)a->part_out; p.zt_out = a->zt_out;
  if (LM) {
    if (p.targets == nullptr || p.splits != 1 || p.batch != 1)
      return set_error("ccb_gemm: LM-head epilogues need targets, one split and one batch");
    if (p.epi == CCB_EPI_LSE_PART && p.part_out == nullptr)
      return set_error("ccb_gemm: LSE_PART needs part_out");
    if (p.epi == CCB_EPI_CE_GRAD && (p.lse == nullptr || !tma_ok))
      return set_error("ccb_gemm: CE_GRAD needs lse and a 16-byte aligned bf16 output");
  }
  long long total = (long long)p.batch * p.splits * p.tiles_m * p.tiles_n;
  if (total <= 0) return 0;
  if (CG == 2) {
    if (p.pair) return set_error("ccb_gemm: the 512-column RMSNorm-backward tile is not available on CTA pairs");
    int pairs = (int)(total < max_pairs[dev & 15] ? total : max_pairs[dev & 15]);
    if (BRES) {
      // every pair keeps one N coordinate: the number of walkers is a multiple of the N-tile count
      pairs -= pairs % p.tiles_n;
      if (pairs < p.tiles_n || p.kblocks > Cfg::RES_KBLOCKS || p.splits != 1 || p.batch != 1 ||
          p.epi == CCB_EPI_ROWSCALE_SILU || p.f8)
        return set_error("ccb_gemm: shape not eligible for the resident-B pair layout (dispatch error)");
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, tmC2, p);
    count_launch();
    if (e != cudaSuccess) return set_error("gemm pair launch: %s", cudaGetErrorString(e));
    return 0;
  }
  int grid = (int)(total < ccb_num_sms() ? total : ccb_num_sms());
  if (BRES) {
    // the resident tile is loaded for the CTA's first N coordinate: every tile it walks must share it
    if (p.kblocks > BRES_KBLOCKS || p.splits != 1 || p.batch != 1 || p.pair || (grid % p.tiles_n) != 0 ||
        p.epi == CCB_EPI_ROWSCALE_SILU || p.f8)
      return set_error("ccb_gemm: shape not eligible for the resident-B layout (dispatch error)");
  }
  if (g_gemm_pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, tmC2, p);
    count_launch();
    if (e != cudaSuccess) return set_error("gemm launch (programmatic dependent): %s", cudaGetErrorString(e));
    return 0;
  }
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, tmC, tmC2, p);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("gemm launch: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace ccb

static inline int64_t b_fp8_of(const CcbGemmArgs* a) { return a->b_fp8; }

// 1: every GEMM runs one CTA per tile; 2: the K-major-A bf16 GEMMs with at least one full 256-row
// pair tile run on CTA pairs (cta_group::2).
// Stage-isolation switches of GemmKArgs::dbg (0 = normal operation).  For timing experiments only.
extern "C" int ccb_gemm_debug(int bits) {
  const int old = ccb::g_gemm_dbg;
  ccb::g_gemm_dbg = bits;
  return old;
}
// L2 prefetch switches (bit 1: A tiles two tiles ahead, bit 2: the next tile's epilogue operands;
// -1: the per-epilogue default).
extern "C" int ccb_gemm_l2_prefetch(int bits) {
  const int old = ccb::g_gemm_l2pf;
  if (bits >= -1 && bits <= 3) ccb::g_gemm_l2pf = bits;
  return old;
}
// 1: single-CTA GEMMs are launched as programmatic dependents (their set-up overlaps the tail of the
// previous kernel in the stream); 0: ordinary stream order.  Returns the old value.
extern "C" int ccb_gemm_pdl(int on) {
  const int old = ccb::g_gemm_pdl;
  if (on == 0 || on == 1) ccb::g_gemm_pdl = on;
  return old;
}
// 1: K <= 256 single-output GEMMs keep their weight tile resident in shared memory (see GemmCfg).
static int g_gemm_bres = 1;
extern "C" int ccb_gemm_resident_b(int on) {
  const int old = g_gemm_bres;
  if (on == 0 || on == 1) g_gemm_bres = on;
  return old;
}
// CTA pairs with the weight tile resident, half in each CTA (bit 1: K <= 256 with an eight-stage A ring,
// bit 2: K in (256, 512] with a four-stage ring); 0: off.  Returns the old value.
static int g_gemm_pair_resident = 0;
extern "C" int ccb_gemm_pair_resident(int bits) {
  const int old = g_gemm_pair_resident;
  if (bits >= 0 && bits <= 3) g_gemm_pair_resident = bits;
  return old;
}
static int g_gemm_cta_group = 1;
extern "C" int ccb_gemm_cta_group(int cg) {
  const int old = g_gemm_cta_group;
  if (cg == 1 || cg == 2) g_gemm_cta_group = cg;
  return old;
}

extern "C" int ccb_gemm(const CcbGemmArgs* a, void* stream_) {
  using namespace ccb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (a->M <= 0 || a->N <= 0 || a->K <= 0 || a->batch <= 0) return 0;
  if ((a->a_fp8 != 0) != (b_fp8_of(a) != 0) || a->a_fp8 < 0 || a->a_fp8 > 2 || a->b_fp8 > 2)
    return set_error("ccb_gemm: a_fp8/b_fp8 must both be 0 (bf16) or both in {1: e4m3, 2: e5m2}");
  const int row_align = a->a_fp8 ? 16 : 8;
  if ((a->lda % row_align) || (a->ldb % row_align) || (a->ldc % 4))
    return set_error("ccb_gemm: row strides must keep rows 16-byte aligned");
  const int key = (int)(a->a_mn * 2 + a->b_mn);
  if (a->epi == CCB_EPI_LSE_PART || a->epi == CCB_EPI_CE_GRAD) {
    if (key != 0 || a->a_fp8) return set_error("ccb_gemm: LM-head epilogues take K-major bf16 operands");
    return launch_gemm<256, 0, 0, 1>(a, stream);
  }
  if (a->epi < 0 || a->epi > CCB_EPI_RMSBWD) return set_error("ccb_gemm: unknown epilogue %lld", (long long)a->epi);
  // 128-wide tiles only where the problem has a single narrow N tile to fill.
  const bool narrow = a->N <= 128 && a->epi == CCB_EPI_STORE;
  if (narrow) {
    switch (key) {
      case 0: return launch_gemm<128, 0, 0>(a, stream);
      case 1: return launch_gemm<128, 0, 1>(a, stream);
      case 3: return launch_gemm<128, 1, 1>(a, stream);
      default: break;
    }
  } else {
    // CTA pairs: bf16, K-major A, a whole number of 8-row-aligned rows per 256-row tile is not
    // needed (TMA clips), but tiny problems gain nothing; the 512-column RMSNorm-backward tile and
    // split-K stay on single CTAs
    {
      // pair + resident weight tile: K <= 256 with the deep A ring (BRES 1), K <= 512 (BRES 2)
      const long long tiles_n = (a->N + 255) / 256, tiles_m2 = (a->M + 255) / 256;
      const int pr = g_gemm_pair_resident;
      const bool pres_ok = pr != 0 && !a->a_fp8 && a->a_mn == 0 && a->batch == 1 && a->splits <= 1 &&
                           a->epi != CCB_EPI_ROWSCALE_SILU && !(a->epi == CCB_EPI_RMSBWD && a->N > 256) &&
                           a->K % 64 == 0 && tiles_m2 * tiles_n >= ccb_num_sms() && tiles_n <= 8;
      if (pres_ok && a->K <= 256 && (pr & 1)) {
        if (key == 0) switch ((int)a->epi) {
          case CCB_EPI_ROWSCALE: return launch_gemm<256, 0, 0, 0, CCB_EPI_ROWSCALE, 2, 1>(a, stream);
          case CCB_EPI_RESID_SS: return launch_gemm<256, 0, 0, 0, CCB_EPI_RESID_SS, 2, 1>(a, stream);
          default: return launch_gemm<256, 0, 0, 0, -1, 2, 1>(a, stream);
        }
        if (key == 1) switch ((int)a->epi) {
          case CCB_EPI_DSILU: return launch_gemm<256, 0, 1, 0, CCB_EPI_DSILU, 2, 1>(a, stream);
          case CCB_EPI_RMSBWD: return launch_gemm<256, 0, 1, 0, CCB_EPI_RMSBWD, 2, 1>(a, stream);
          default: return launch_gemm<256, 0, 1, 0, -1, 2, 1>(a, stream);
        }
      }
      if (pres_ok && a->K > 256 && a->K <= 512 && (pr & 2)) {
        if (key == 1) switch ((int)a->epi) {
          case CCB_EPI_DSILU: return launch_gemm<256, 0, 1, 0, CCB_EPI_DSILU, 2, 2>(a, stream);
          case CCB_EPI_RMSBWD: return launch_gemm<256, 0, 1, 0, CCB_EPI_RMSBWD, 2, 2>(a, stream);
          default: return launch_gemm<256, 0, 1, 0, -1, 2, 2>(a, stream);
        }
        if (key == 0) switch ((int)a->epi) {
          case CCB_EPI_RESID_SS: return launch_gemm<256, 0, 0, 0, CCB_EPI_RESID_SS, 2, 2>(a, stream);
          default: break;
        }
      }
    }
    const bool pair_ok = g_gemm_cta_group == 2 && !a->a_fp8 && a->a_mn == 0 && a->M >= 512 &&
                         a->batch == 1 && a->splits <= 1 && !(a->epi == CCB_EPI_RMSBWD && a->N > 256);
    if (pair_ok && key == 0) {
      switch ((int)a->epi) {
        case CCB_EPI_ROWSCALE: return launch_gemm<256, 0, 0, 0, CCB_EPI_ROWSCALE, 2>(a, stream);
        case CCB_EPI_ROWSCALE_SILU: return launch_gemm<256, 0, 0, 0, CCB_EPI_ROWSCALE_SILU, 2>(a, stream);
        case CCB_EPI_RESID_SS: return launch_gemm<256, 0, 0, 0, CCB_EPI_RESID_SS, 2>(a, stream);
        default: return launch_gemm<256, 0, 0, 0, -1, 2>(a, stream);
      }
    }
    if (pair_ok && key == 1) {
      switch ((int)a->epi) {
        case CCB_EPI_DSILU: return launch_gemm<256, 0, 1, 0, CCB_EPI_DSILU, 2>(a, stream);
        case CCB_EPI_RMSBWD: return launch_gemm<256, 0, 1, 0, CCB_EPI_RMSBWD, 2>(a, stream);
        default: return launch_gemm<256, 0, 1, 0, -1, 2>(a, stream);
      }
    }
    {
      const int sms = ccb_num_sms();
      const long long tiles_n = (a->N + 255) / 256, tiles_m = (a->M + 127) / 128;
      const long long grid = tiles_m * tiles_n < sms ? tiles_m * tiles_n : sms;
      const bool bres_ok = g_gemm_bres && !a->a_fp8 && a->a_mn == 0 && a->K <= 64 * BRES_KBLOCKS &&
                           a->batch == 1 && a->splits <= 1 && a->epi != CCB_EPI_ROWSCALE_SILU &&
                           !(a->epi == CCB_EPI_RMSBWD && a->N > 256) && tiles_m >= 2 * sms / tiles_n &&
                           grid % tiles_n == 0;
      if (bres_ok && key == 0) {
        switch ((int)a->epi) {
          case CCB_EPI_ROWSCALE: return launch_gemm<256, 0, 0, 0, CCB_EPI_ROWSCALE, 1, 1>(a, stream);
          case CCB_EPI_RESID_SS: return launch_gemm<256, 0, 0, 0, CCB_EPI_RESID_SS, 1, 1>(a, stream);
          default: return launch_gemm<256, 0, 0, 0, -1, 1, 1>(a, stream);
        }
      }
      if (bres_ok && key == 1) {
        switch ((int)a->epi) {
          case CCB_EPI_DSILU: return launch_gemm<256, 0, 1, 0, CCB_EPI_DSILU, 1, 1>(a, stream);
          case CCB_EPI_RMSBWD: return launch_gemm<256, 0, 1, 0, CCB_EPI_RMSBWD, 1, 1>(a, stream);
          default: return launch_gemm<256, 0, 1, 0, -1, 1, 1>(a, stream);
        }
      }
    }
    if (key == 0) {
      // K-major x K-major carries the trunk's fused epilogues: one instantiation each
      switch ((int)a->epi) {
        case CCB_EPI_ROWSCALE: return launch_gemm<256, 0, 0, 0, CCB_EPI_ROWSCALE>(a, stream);
        case CCB_EPI_ROWSCALE_SILU: return launch_gemm<256, 0, 0, 0, CCB_EPI_ROWSCALE_SILU>(a, stream);
        case CCB_EPI_RESID_SS: return launch_gemm<256, 0, 0, 0, CCB_EPI_RESID_SS>(a, stream);
        default: break;
      }
    } else if (key == 1) {
      switch ((int)a->epi) {
        case CCB_EPI_DSILU: return launch_gemm<256, 0, 1, 0, CCB_EPI_DSILU>(a, stream);
        case CCB_EPI_RMSBWD: return launch_gemm<256, 0, 1, 0, CCB_EPI_RMSBWD>(a, stream);
        default: break;
      }
    }
    switch (key) {
      case 0: return launch_gemm<256, 0, 0>(a, stream);
      case 1: return launch_gemm<256, 0, 1>(a, stream);
      case 3: return launch_gemm<256, 1, 1>(a, stream);
      default: break;
    }
  }
  return set_error("ccb_gemm: operand layout a_mn=%lld b_mn=%lld is not instantiated",
                   (long long)a->a_mn, (long long)a->b_mn);
}
