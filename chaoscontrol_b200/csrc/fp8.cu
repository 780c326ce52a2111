// 8-bit float support kernels for the fp8 linear layer: scaled casts with a
// running absolute maximum, the transposing cast that feeds the K-major
// operands of the backward GEMMs (with the bias-gradient column sum folded in),
// and the once-per-step amax-history flush.  The GEMMs themselves are the
// tcgen05 kind::f8f6f4 path of gemm.cu.
//
// Counterparts in the reference: fused_amax_cast_1d_kernel,
// fused_amax_cast_transpose_kernel, fused_flush_amax_kernel and its
// diagnostic variant (src/chaoscontrol/kernels/_cublaslt/src/fused_amax_cast.cu:96-291).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ccb_api.h"
#include "ptx.cuh"
#include "runtime.h"

namespace ccb {

// fmt: 1 = e4m3, 2 = e5m2 (same numbering as CcbGemmArgs::a_fp8)
__device__ __forceinline__ uint16_t cvt2(float a, float b, int fmt) {
  return (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, fmt == 1 ? __NV_E4M3 : __NV_E5M2);
}
__device__ __forceinline__ uint8_t cvt1(float a, int fmt) {
  return (uint8_t)__nv_cvt_float_to_fp8(a, __NV_SATFINITE, fmt == 1 ? __NV_E4M3 : __NV_E5M2);
}

// Non-negative floats order like their bit patterns, so the running maximum is
// one integer atomicMax per block.
__device__ __forceinline__ void block_amax_commit(float local, float* pending) {
  __shared__ float wmax[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, o));
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) wmax[w] = local;
  __syncthreads();
  if (w == 0) {
    float v = (l < (int)(blockDim.x >> 5)) ? wmax[l] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (l == 0 && pending != nullptr) atomicMax(reinterpret_cast<int*>(pending), __float_as_int(v));
  }
}

// out[i] = fp8(x[i] / scale); pending = max(pending, max|x|).  8 elements per thread.
__global__ void __launch_bounds__(256)
fp8_cast_amax_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ out,
                     const float* __restrict__ scale, float* __restrict__ pending, long long n, int fmt) {
  const float inv = 1.f / __ldg(scale);
  float amax = 0.f;
  const long long nvec = n >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(x) + i);
    const float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
    amax = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y))),
                             fmaxf(fmaxf(fabsf(f2.x), fabsf(f2.y)), fmaxf(fabsf(f3.x), fabsf(f3.y)))));
    uint2 o;
    o.x = (uint32_t)cvt2(f0.x * inv, f0.y * inv, fmt) | ((uint32_t)cvt2(f1.x * inv, f1.y * inv, fmt) << 16);
    o.y = (uint32_t)cvt2(f2.x * inv, f2.y * inv, fmt) | ((uint32_t)cvt2(f3.x * inv, f3.y * inv, fmt) << 16);
    reinterpret_cast<uint2*>(out)[i] = o;
  }
  // ragged tail (n not a multiple of 8): first block only
  if (blockIdx.x == 0) {
    for (long long i = (nvec << 3) + threadIdx.x; i < n; i += blockDim.x) {
      const float v = __bfloat162float(x[i]);
      amax = fmaxf(amax, fabsf(v));
      out[i] = cvt1(v * inv, fmt);
    }
  }
  block_amax_commit(amax, pending);
}

// out[c][r] = fp8(x[r][c] / scale) for x [R, C]; out rows are `ldo` bytes apart
// (>= R, so the caller can pad rows to the 16-byte TMA stride rule).  Optional
// colsum[c] += sum_r x[r][c] (bias gradient).  64 x 64 tiles through shared memory.
__global__ void __launch_bounds__(256)
fp8_cast_transpose_amax_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ out,
                               const float* __restrict__ scale, float* __restrict__ pending,
                               float* __restrict__ colsum, int R, int C, long long ldx, long long ldo, int fmt) {
  __shared__ float tile[64][65];
  const float inv = 1.f / __ldg(scale);
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;   // 64 x 4
  float amax = 0.f, csum = 0.f;
#pragma unroll 4
  for (int i = ty; i < 64; i += 4) {
    const int r = r0 + i, c = c0 + tx;
    float v = 0.f;
    if (r < R && c < C) v = __bfloat162float(x[(long long)r * ldx + c]);
    amax = fmaxf(amax, fabsf(v));
    csum += v;
    tile[i][tx] = v * inv;
  }
  if (colsum != nullptr) {
    // the 4 row-groups of a column live in 4 different warps pairs: reduce through smem
    __shared__ float cs[4][64];
    cs[ty][tx] = csum;
    __syncthreads();
    if (ty == 0 && c0 + tx < C) atomicAdd(colsum + c0 + tx, cs[0][tx] + cs[1][tx] + cs[2][tx] + cs[3][tx]);
  } else {
    __syncthreads();
  }
  // write transposed: thread handles out row (c0 + i), 4 consecutive r per thread
  const int rx = (threadIdx.x & 15) * 4, cy = threadIdx.x >> 4;   // 16 x 16
#pragma unroll
  for (int i = cy; i < 64; i += 16) {
    const int c = c0 + i;
    if (c >= C) continue;
    const int r = r0 + rx;
    uint8_t* dst = out + (long long)c * ldo + r;
    if (r + 3 < R && ((reinterpret_cast<uintptr_t>(dst) & 3) == 0)) {
      const uint32_t pk = (uint32_t)cvt2(tile[rx][i], tile[rx + 1][i], fmt) |
                          ((uint32_t)cvt2(tile[rx + 2][i], tile[rx + 3][i], fmt) << 16);
      *reinterpret_cast<uint32_t*>(dst) = pk;
    } else {
      for (int j = 0; j < 4; ++j)
        if (r + j < R) dst[j] = cvt1(tile[rx + j][i], fmt);
    }
  }
  block_amax_commit(amax, pending);
}

// history <- roll(history, -1); history[-1] = pending; scale = max(history) / max_rep
// (1 when the history is all zero); pending = 0.  scale == nullptr: bookkeeping only.
__global__ void fp8_flush_amax_kernel(float* history, int len, float* pending, float* scale, float max_rep) {
  extern __shared__ float h[];
  const int t = threadIdx.x;
  for (int i = t; i < len; i += blockDim.x) h[i] = (i + 1 < len) ? history[i + 1] : pending[0];
  __syncthreads();
  for (int i = t; i < len; i += blockDim.x) history[i] = h[i];
  if (t == 0) {
    if (scale != nullptr) {
      float m = 0.f;
      for (int i = 0; i < len; ++i) m = fmaxf(m, h[i]);
      scale[0] = m > 0.f ? m / max_rep : 1.f;
    }
    pending[0] = 0.f;
  }
}

}  // namespace ccb

using namespace ccb;

extern "C" int ccb_fp8_cast_amax(const void* x, void* out, const float* scale, float* pending, int64_t n,
                                 int64_t fmt, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (n <= 0) return 0;
  if (fmt != 1 && fmt != 2) return set_error("ccb_fp8_cast_amax: fmt must be 1 (e4m3) or 2 (e5m2)");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 7))
    return set_error("ccb_fp8_cast_amax: x must be 16-byte and out 8-byte aligned");
  long long blocks = ((n >> 3) + 255) / 256;
  const long long cap = (long long)ccb_num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  fp8_cast_amax_kernel<<<(int)blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                       reinterpret_cast<uint8_t*>(out), scale, pending, n, (int)fmt);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("fp8_cast_amax launch: %s", cudaGetErrorString(e));
}

extern "C" int ccb_fp8_cast_transpose_amax(const void* x, void* out, const float* scale, float* pending,
                                           float* colsum, int64_t R, int64_t C, int64_t ldx, int64_t ldo,
                                           int64_t fmt, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (R <= 0 || C <= 0) return 0;
  if (fmt != 1 && fmt != 2) return set_error("ccb_fp8_cast_transpose_amax: fmt must be 1 (e4m3) or 2 (e5m2)");
  if (ldo < R) return set_error("ccb_fp8_cast_transpose_amax: output row stride %lld < %lld rows",
                                (long long)ldo, (long long)R);
  dim3 grid((unsigned)((C + 63) / 64), (unsigned)((R + 63) / 64));
  if (grid.y > 65535u) return set_error("ccb_fp8_cast_transpose_amax: too many rows (%lld)", (long long)R);
  fp8_cast_transpose_amax_kernel<<<grid, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(out), scale, pending, colsum,
      (int)R, (int)C, ldx, ldo, (int)fmt);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("fp8_cast_transpose_amax launch: %s", cudaGetErrorString(e));
}

extern "C" int ccb_fp8_flush_amax(float* history, int64_t len, float* pending, float* scale, float max_rep,
                                  void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (len <= 0 || len > 4096) return set_error("ccb_fp8_flush_amax: history length %lld out of range", (long long)len);
  fp8_flush_amax_kernel<<<1, 32, (size_t)len * sizeof(float), stream>>>(history, (int)len, pending, scale, max_rep);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("fp8_flush_amax launch: %s", cudaGetErrorString(e));
}
