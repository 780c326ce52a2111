// Block-scaled e4m3 linear layer for sm_100a.
//
//   C[m, n] = sum_kb  sa[kb, m] * sb[n / 128, kb] * ( A8[m, kb-block] . B8[n, kb-block] )
//
// A8 [M, K] carries one fp32 scale per row and 128-wide K block ("1 x 128",
// activations / output gradients), B8 [N, K] one per 128 x 128 block (weights).
// Each K block is a separate tcgen05.mma chain (kind::f8f6f4, 4 issues of K=32)
// into its own 128-column TMEM accumulator; the epilogue warps multiply that
// partial product by the two block scales while adding it into fp32 registers,
// so the scales never touch the tensor-core path and a 4-deep ring of TMEM
// accumulators lets the MMAs of block kb+1..kb+3 run under the scaling of kb.
//
// The quantisers produce exactly the operand layouts the GEMM consumes:
//   rows:   bf16 [R, K] -> e4m3 [R, K] + scales [K/128, R]  (optionally the
//           RMSNorm of the row: the cast is fused into the norm that produces
//           the linear's input, the row never round-trips through bf16)
//   blocks: bf16 [N, K] -> e4m3 [N, K] and its transpose [K, N] + scales [N/128, K/128]
//
// The reference's fp8 path is per-tensor scaling around cuBLASLt
// (src/chaoscontrol/kernels/fp8_linear.py:171-265,
//  kernels/_cublaslt/src/cublaslt_fp8_matmul.cpp:281-291); this is the
// finer-grained replacement.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ccb_api.h"
#include "ptx.cuh"
#include "runtime.h"

namespace ccb {

constexpr float E4M3_MAX = 448.f;

__device__ __forceinline__ uint16_t e4m3x2(float a, float b) {
  return (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}

// ---------------------------------------------------------------------------
// Row quantiser (1 x 128 scales), optionally fused with RMSNorm.
// One warp per row; a lane owns 8 contiguous elements of each 256-column
// segment, so a 128-column block is 16 lanes and its amax is 4 shuffles.
// ---------------------------------------------------------------------------
constexpr int QR_MAXSEG = 8;   // K <= 2048

__global__ void __launch_bounds__(256)
fp8_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                      const __nv_bfloat16* __restrict__ norm_w, float eps,
                      uint8_t* __restrict__ q, float* __restrict__ s_t, float* __restrict__ inv_rms_out,
                      __nv_bfloat16* __restrict__ y_out, int R, int K) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= R) return;
  const int nseg = (K + 255) >> 8;
  float v[QR_MAXSEG][8];
  float ss = 0.f;
#pragma unroll
  for (int sgm = 0; sgm < QR_MAXSEG; ++sgm) {
    const int c = sgm * 256 + lane * 8;
    if (sgm < nseg && c < K) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(x + (long long)row * ldx + c));
      const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
      v[sgm][0] = f0.x; v[sgm][1] = f0.y; v[sgm][2] = f1.x; v[sgm][3] = f1.y;
      v[sgm][4] = f2.x; v[sgm][5] = f2.y; v[sgm][6] = f3.x; v[sgm][7] = f3.y;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[sgm][i] * v[sgm][i];
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[sgm][i] = 0.f;
    }
  }
  if (norm_w != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / (float)K + eps);
    if (lane == 0 && inv_rms_out != nullptr) inv_rms_out[row] = inv;
#pragma unroll
    for (int sgm = 0; sgm < QR_MAXSEG; ++sgm) {
      const int c = sgm * 256 + lane * 8;
      if (sgm < nseg && c < K) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(norm_w + c));
        const float2 w0 = unpack_bf16x2(u.x), w1 = unpack_bf16x2(u.y), w2 = unpack_bf16x2(u.z), w3 = unpack_bf16x2(u.w);
        const float wv[8] = {w0.x, w0.y, w1.x, w1.y, w2.x, w2.y, w3.x, w3.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) v[sgm][i] = v[sgm][i] * inv * wv[i];
      }
    }
  }
#pragma unroll
  for (int sgm = 0; sgm < QR_MAXSEG; ++sgm) {
    const int c = sgm * 256 + lane * 8;
    if (sgm >= nseg) break;
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[sgm][i]));
    // 16 lanes = one 128-column block
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (c < K) {
      const float scale = fmaxf(amax, 1e-12f) * (1.f / E4M3_MAX);
      const float inv = 1.f / scale;
      uint2 o;
      o.x = (uint32_t)e4m3x2(v[sgm][0] * inv, v[sgm][1] * inv) | ((uint32_t)e4m3x2(v[sgm][2] * inv, v[sgm][3] * inv) << 16);
      o.y = (uint32_t)e4m3x2(v[sgm][4] * inv, v[sgm][5] * inv) | ((uint32_t)e4m3x2(v[sgm][6] * inv, v[sgm][7] * inv) << 16);
      *reinterpret_cast<uint2*>(q + (long long)row * K + c) = o;
      if ((lane & 15) == 0) s_t[(long long)(c >> 7) * R + row] = scale;
      if (y_out != nullptr) {
        uint4 yo;
        yo.x = pack_bf16x2(v[sgm][0], v[sgm][1]); yo.y = pack_bf16x2(v[sgm][2], v[sgm][3]);
        yo.z = pack_bf16x2(v[sgm][4], v[sgm][5]); yo.w = pack_bf16x2(v[sgm][6], v[sgm][7]);
        *reinterpret_cast<uint4*>(y_out + (long long)row * K + c) = yo;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Weight quantiser (128 x 128 scales): one CTA per block, writes W8 and W8^T.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
fp8_quant_blocks_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                        uint8_t* __restrict__ qt, float* __restrict__ s, int N, int K) {
  __shared__ __nv_bfloat16 tile[128][130];   // 65-word row stride: transposed reads are conflict-free
  __shared__ float wmax[8];
  const int n0 = blockIdx.y * 128, k0 = blockIdx.x * 128;
  const int tx = threadIdx.x & 127, ty = threadIdx.x >> 7;   // 128 x 2
  float amax = 0.f;
  for (int i = ty; i < 128; i += 2) {
    const int n = n0 + i, k = k0 + tx;
    __nv_bfloat16 raw = __float2bfloat16(0.f);
    if (n < N && k < K) raw = w[(long long)n * K + k];
    tile[i][tx] = raw;
    amax = fmaxf(amax, fabsf(__bfloat162float(raw)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = wmax[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, wmax[i]);
  const float scale = fmaxf(amax, 1e-12f) * (1.f / E4M3_MAX);
  const float inv = 1.f / scale;
  if (threadIdx.x == 0) s[(long long)blockIdx.y * gridDim.x + blockIdx.x] = scale;
  for (int i = ty; i < 128; i += 2) {
    const int n = n0 + i, k = k0 + tx;
    if (n < N && k < K)
      q[(long long)n * K + k] = (uint8_t)__nv_cvt_float_to_fp8(__bfloat162float(tile[i][tx]) * inv, __NV_SATFINITE, __NV_E4M3);
  }
  if (qt != nullptr) {
    for (int i = ty; i < 128; i += 2) {
      const int k = k0 + i, n = n0 + tx;   // transposed: row k, column n
      if (n < N && k < K)
        qt[(long long)k * N + n] = (uint8_t)__nv_cvt_float_to_fp8(__bfloat162float(tile[tx][i]) * inv, __NV_SATFINITE, __NV_E4M3);
    }
  }
}

// ---------------------------------------------------------------------------
// Block-scaled GEMM
// ---------------------------------------------------------------------------
constexpr int FB_BM = 128, FB_BN = 128, FB_BK = 128;        // one-byte elements: 128 per swizzle row
constexpr int FB_STAGE = FB_BM * FB_BK;                      // 16 KiB per operand tile
constexpr int FB_STAGES = 5;
constexpr int FB_SLOTS = 4;                                  // TMEM accumulator ring (4 x 128 columns)
constexpr int FB_EPI_WARPS = 8;
constexpr int FB_THREADS = 64 + 32 * FB_EPI_WARPS;
constexpr int FB_BAR_OFF = 2 * FB_STAGES * FB_STAGE;
constexpr int FB_SMEM = 1024 + FB_BAR_OFF + 512;

struct FbArgs {
  int M, N, K, kblocks, tiles_m, tiles_n;
  const float* sa_t;        // [K/128, M]
  const float* sb;          // scale of (output column block j, k block kb) at sb[j * sb_so + kb * sb_sk]
  long long sb_so, sb_sk;
  void* C;
  long long ldc;
  int out_fp32;
  const __nv_bfloat16* bias;
  int* status;
};

__global__ void __launch_bounds__(FB_THREADS, 1)
fp8_block_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const FbArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + FB_STAGES * FB_STAGE;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + FB_BAR_OFF);
  uint64_t* empty_bar = full_bar + FB_STAGES;
  uint64_t* tfull_bar = empty_bar + FB_STAGES;
  uint64_t* tempty_bar = tfull_bar + FB_SLOTS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + FB_SLOTS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int i = 0; i < FB_STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < FB_SLOTS; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], FB_EPI_WARPS); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / p.tiles_n) * FB_BM, n0 = (tile % p.tiles_n) * FB_BN;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status)) { ok = false; break; }
          mbar_arrive_expect_tx(&full_bar[stage], 2 * FB_STAGE);
          tma_load_3d(sA + stage * FB_STAGE, &tmA, &full_bar[stage], kb * FB_BK, m0, 0);
          tma_load_3d(sB + stage * FB_STAGE, &tmB, &full_bar[stage], kb * FB_BK, n0, 0);
          if (++stage == FB_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // aborting: bounded grace period for loads still in flight
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f8(FB_BM, FB_BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0, n_slot = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < p.kblocks; ++kb, ++n_slot) {
          const int slot = n_slot % FB_SLOTS;
          const uint32_t sph = (n_slot / FB_SLOTS) & 1u;
          if (!mbar_wait(&tempty_bar[slot], sph ^ 1u, abort_flag, p.status)) { ok = false; break; }
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(sA + stage * FB_STAGE);
          const uint32_t b_base = smem_u32(sB + stage * FB_STAGE);
#pragma unroll
          for (int k = 0; k < FB_BK / 32; ++k) {
            const uint64_t adesc = make_smem_desc(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = make_smem_desc(b_base + k * 32, 16, 1024);
            umma_f8(tmem_base + (uint32_t)(slot * FB_BN), adesc, bdesc, idesc, k > 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          umma_commit(&tfull_bar[slot]);
          if (++stage == FB_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    const int q = warp & 3;                    // TMEM lane quadrant
    const int part = (warp - 2) >> 2;          // columns [64 * part, 64 * part + 64) of the tile
    const int row_in_tile = q * 32 + lane;
    uint32_t n_slot = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile / p.tiles_n) * FB_BM, n0 = (tile % p.tiles_n) * FB_BN;
      const int m = m0 + row_in_tile;
      const bool row_ok = m < p.M;
      float out[2][32];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 32; ++i) out[h][i] = 0.f;
      for (int kb = 0; kb < p.kblocks; ++kb, ++n_slot) {
        const int slot = n_slot % FB_SLOTS;
        const uint32_t sph = (n_slot / FB_SLOTS) & 1u;
        // the two block scales do not depend on the accumulator: fetch before waiting
        const float sc = (row_ok ? __ldg(p.sa_t + (long long)kb * p.M + m) : 0.f) *
                         __ldg(p.sb + (long long)(n0 / FB_BN) * p.sb_so + (long long)kb * p.sb_sk);
        {
          const bool w = mbar_wait(&tfull_bar[slot], sph, abort_flag, p.status);
          if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
        }
        tc_fence_after_sync();
        const uint32_t t_addr = tmem_base + (uint32_t)(slot * FB_BN + part * 64) + ((uint32_t)(q * 32) << 16);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          __syncwarp();
          tmem_ld32(t_addr + h * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) out[h][i] = fmaf(__uint_as_float(r[i]), sc, out[h][i]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[slot]);
      }
      if (!ok) break;
      if (row_ok) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int n = n0 + part * 64 + h * 32;
          const int nvalid = p.N - n;
          if (nvalid <= 0) continue;
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < nvalid) out[h][i] += __bfloat162float(p.bias[n + i]);
          }
          if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(p.C) + (long long)m * p.ldc + n;
            if (nvalid >= 32) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(dst)[i] = make_float4(out[h][4 * i], out[h][4 * i + 1], out[h][4 * i + 2], out[h][4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nvalid) dst[i] = out[h][i];
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)m * p.ldc + n;
            if (nvalid >= 32) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 o;
                o.x = pack_bf16x2(out[h][8 * i + 0], out[h][8 * i + 1]);
                o.y = pack_bf16x2(out[h][8 * i + 2], out[h][8 * i + 3]);
                o.z = pack_bf16x2(out[h][8 * i + 4], out[h][8 * i + 5]);
                o.w = pack_bf16x2(out[h][8 * i + 6], out[h][8 * i + 7]);
                reinterpret_cast<uint4*>(dst)[i] = o;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nvalid) dst[i] = __float2bfloat16(out[h][i]);
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace ccb

using namespace ccb;

extern "C" int ccb_fp8_quant_rows(const void* x, int64_t ldx, const void* norm_w, float eps, void* q,
                                  float* s_t, float* inv_rms_out, void* y_out, int64_t R, int64_t K,
                                  void* stream) {
  if (R <= 0) return 0;
  if (K % 128 != 0 || K > 256 * QR_MAXSEG || ldx % 8 != 0)
    return set_error("ccb_fp8_quant_rows: K must be a multiple of 128 and <= %d, rows 16-byte aligned", 256 * QR_MAXSEG);
  const int rows_per_block = 8;
  fp8_quant_rows_kernel<<<(unsigned)((R + rows_per_block - 1) / rows_per_block), 32 * rows_per_block, 0,
                          (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)norm_w, eps,
                                                  (uint8_t*)q, s_t, inv_rms_out, (__nv_bfloat16*)y_out, (int)R, (int)K);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("fp8_quant_rows launch: %s", cudaGetErrorString(e));
}

extern "C" int ccb_fp8_quant_blocks(const void* w, void* q, void* qt, float* s, int64_t N, int64_t K,
                                    void* stream) {
  if (N <= 0 || K <= 0) return 0;
  dim3 grid((unsigned)((K + 127) / 128), (unsigned)((N + 127) / 128));
  fp8_quant_blocks_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)w, (uint8_t*)q,
                                                                  (uint8_t*)qt, s, (int)N, (int)K);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("fp8_quant_blocks launch: %s", cudaGetErrorString(e));
}

extern "C" int ccb_fp8_block_gemm(const void* A8, const float* sa_t, const void* B8, const float* sb,
                                  int64_t sb_so, int64_t sb_sk, void* C, int64_t ldc, int64_t out_fp32,
                                  const void* bias, int64_t M, int64_t N, int64_t K, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 128 != 0) return set_error("ccb_fp8_block_gemm: K must be a multiple of 128 (got %lld)", (long long)K);
  if ((out_fp32 ? ldc % 4 : ldc % 8) != 0) return set_error("ccb_fp8_block_gemm: output rows must be 16-byte aligned");
  static bool attr_set[16] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 15]) {
    cudaError_t e = cudaFuncSetAttribute(fp8_block_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FB_SMEM);
    if (e != cudaSuccess) return set_error("cudaFuncSetAttribute(fp8_block_gemm): %s", cudaGetErrorString(e));
    attr_set[dev & 15] = true;
  }
  CUtensorMap tmA, tmB;
  if (make_tmap_u8_3d(&tmA, A8, (uint64_t)K, (uint64_t)M, 1, (uint64_t)K, 0, 128, FB_BM)) return -1;
  if (make_tmap_u8_3d(&tmB, B8, (uint64_t)K, (uint64_t)N, 1, (uint64_t)K, 0, 128, FB_BN)) return -1;
  FbArgs p;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.kblocks = (int)(K / 128);
  p.tiles_m = (int)((M + FB_BM - 1) / FB_BM);
  p.tiles_n = (int)((N + FB_BN - 1) / FB_BN);
  p.sa_t = sa_t; p.sb = sb; p.sb_so = sb_so; p.sb_sk = sb_sk;
  p.C = C; p.ldc = ldc; p.out_fp32 = (int)out_fp32;
  p.bias = (const __nv_bfloat16*)bias;
  p.status = ccb_status_ptr();
  const long long total = (long long)p.tiles_m * p.tiles_n;
  const int grid = (int)(total < ccb_num_sms() ? total : ccb_num_sms());
  fp8_block_gemm_kernel<<<grid, FB_THREADS, FB_SMEM, (cudaStream_t)stream>>>(tmA, tmB, p);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("fp8_block_gemm launch: %s", cudaGetErrorString(e));
}
