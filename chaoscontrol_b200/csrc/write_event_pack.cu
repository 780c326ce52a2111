// Packs selected (batch, position) write candidates straight into 568-byte
// WriteEvent wire records on the device, so the publisher thread copies one
// contiguous buffer to pinned host memory and pushes records into the ring
// without any per-event Python work.
//
// One WARP per event (8 events per block): every lane converts 8 key-vector
// channels to fp16 bits and stores them as two 8-byte words; the rolling
// fingerprint  h = sum_i (tok_i + 1) * base^(W-1-i)  mod (2^61 - 1)  is evaluated
// in parallel -- lane i owns token i, raises the base to its power with 64x64
// -> 128-bit multiplies reduced by the Mersenne identity, and the terms are
// summed by a shuffle tree of modular adds.  Invalid candidates (too close to a
// sequence edge for a full fingerprint window or value span) produce an all-zero
// record (event_type 0), which the host side skips.
//
// Counterpart of pack_write_events_kernel
// (src/chaoscontrol/kernels/_cpu_ssm_controller/src/write_event_pack.cu:82-153),
// and bit-compatible with the host-side fingerprint
// (src/chaoscontrol/optim/episodic_writer.py:156-173).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ccb_api.h"
#include "runtime.h"

namespace ccb {

constexpr uint64_t kMersenne61 = (uint64_t{1} << 61) - 1;
constexpr uint64_t kFpBase = 1000003ull;
constexpr int kRecordBytes = 568;
constexpr int kKeyRepWire = 256;     // fp16 channels on the wire
constexpr int kSpanWire = 4;         // uint16 value tokens on the wire

__device__ __forceinline__ uint64_t mod61(uint64_t lo, uint64_t hi) {
  // value = hi * 2^64 + lo;  2^61 == 1 (mod p)  =>  fold 61-bit limbs
  uint64_t s = (lo & kMersenne61) + ((lo >> 61) | (hi << 3));   // hi < 2^58 for operands < 2^61
  s = (s & kMersenne61) + (s >> 61);
  return s >= kMersenne61 ? s - kMersenne61 : s;
}
__device__ __forceinline__ uint64_t mulmod61(uint64_t a, uint64_t b) {
  return mod61(a * b, __umul64hi(a, b));
}
__device__ __forceinline__ uint64_t addmod61(uint64_t a, uint64_t b) {
  const uint64_t s = a + b;
  return s >= kMersenne61 ? s - kMersenne61 : s;
}
__device__ __forceinline__ uint64_t powmod61(uint64_t base, int e) {
  uint64_t r = 1, x = base;
  while (e > 0) {
    if (e & 1) r = mulmod61(r, x);
    x = mulmod61(x, x);
    e >>= 1;
  }
  return r;
}

template <typename T> __device__ __forceinline__ float rep_to_float(T v);
template <> __device__ __forceinline__ float rep_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float rep_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float rep_to_float<__half>(__half v) { return __half2float(v); }

template <typename rep_t>
__global__ void __launch_bounds__(256)
pack_write_events_kernel(uint8_t* __restrict__ out, const int64_t* __restrict__ input_ids,
                         const int64_t* __restrict__ target_ids, const rep_t* __restrict__ key_rep,
                         const float* __restrict__ pressure, const float* __restrict__ per_token_ce,
                         const int64_t* __restrict__ positions, const int64_t* __restrict__ candidate_base,
                         int M, int B, int T, int D, uint64_t gpu_step, int source_rank, int write_bucket,
                         int W, int span, int rep_dim) {
  const int lane = threadIdx.x & 31;
  const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (m >= M) return;
  uint64_t* rec = reinterpret_cast<uint64_t*>(out + (size_t)m * kRecordBytes);   // 568 = 8 * 71
  const long long b = positions[2 * m], t = positions[2 * m + 1];
  const bool valid = b >= 0 && b < B && t >= W && t + span <= T && W >= 0 && rep_dim > 0 &&
                     rep_dim <= kKeyRepWire && span > 0 && span <= kSpanWire && D >= rep_dim;
  if (!valid) {
    for (int i = lane; i < kRecordBytes / 8; i += 32) rec[i] = 0ull;
    return;
  }
  const long long row = b * (long long)T;
  // ---- fingerprint: ceil(W / 32) rounds of 32 parallel terms --------------------------------
  uint64_t h = 0;
  for (int base_i = 0; base_i < W; base_i += 32) {
    const int i = base_i + lane;
    uint64_t term = 0;
    if (i < W) {
      const uint64_t tok = (uint64_t)input_ids[row + t - W + i];
      term = mulmod61((tok + 1ull) % kMersenne61, powmod61(kFpBase, W - 1 - i));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) term = addmod61(term, __shfl_xor_sync(0xffffffffu, term, o));
    h = addmod61(h, term);
  }
  // ---- key vector: 256 fp16 slots, 8 per lane, channels >= rep_dim are zero -----------------
  const rep_t* src = key_rep + (row + t) * (long long)D;
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = lane * 8 + 2 * j;
    const float a = c < rep_dim ? rep_to_float<rep_t>(src[c]) : 0.f;
    const float d = c + 1 < rep_dim ? rep_to_float<rep_t>(src[c + 1]) : 0.f;
    w[j] = (uint32_t)__half_as_ushort(__float2half_rn(a)) | ((uint32_t)__half_as_ushort(__float2half_rn(d)) << 16);
  }
  rec[4 + lane * 2] = (uint64_t)w[0] | ((uint64_t)w[1] << 32);
  rec[4 + lane * 2 + 1] = (uint64_t)w[2] | ((uint64_t)w[3] << 32);
  if (lane == 0) {
    const uint64_t low = (uint64_t)(*candidate_base) + (uint64_t)m;
    rec[0] = 1ull | ((uint64_t)(uint8_t)source_rank << 8) | ((uint64_t)(uint8_t)write_bucket << 16);
    rec[1] = ((uint64_t)(uint8_t)source_rank << 56) | (low & ((uint64_t{1} << 56) - 1));
    rec[2] = gpu_step;
    rec[3] = h;
    uint64_t toks = 0;
    for (int j = 0; j < span; ++j) toks |= (uint64_t)(uint16_t)target_ids[row + t + j] << (16 * j);
    rec[68] = toks;                                                           // value_tok_ids @ 544
    const float pr = pressure == nullptr ? 1.0f : pressure[row + t];
    rec[69] = (uint64_t)(uint32_t)target_ids[row + t] | ((uint64_t)__float_as_uint(pr) << 32);   // anchor, pressure
    rec[70] = (uint64_t)__float_as_uint(per_token_ce[row + t]);               // pre_write_ce, pad
  }
}

}  // namespace ccb

using namespace ccb;

// rep_dtype: 0 = fp32, 1 = bf16, 2 = fp16.  positions is [M, 2] int64 (batch, position);
// candidate_base a device int64 scalar; out [M, 568] bytes.
extern "C" int ccb_pack_write_events(void* out, const int64_t* input_ids, const int64_t* target_ids,
                                     const void* key_rep, int64_t rep_dtype, const float* pressure,
                                     const float* per_token_ce, const int64_t* positions,
                                     const int64_t* candidate_base, int64_t M, int64_t B, int64_t T, int64_t D,
                                     int64_t gpu_step, int64_t source_rank, int64_t write_bucket,
                                     int64_t fingerprint_window, int64_t span_length, int64_t key_rep_dim,
                                     void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0) return 0;
  if (source_rank < 0 || source_rank > 255 || write_bucket < 0 || write_bucket > 255)
    return set_error("ccb_pack_write_events: source_rank / write_bucket must fit in a byte");
  if (reinterpret_cast<uintptr_t>(out) & 7) return set_error("ccb_pack_write_events: out must be 8-byte aligned");
  const int grid = (int)((M + 7) / 8);
#define CCB_PACK_LAUNCH(T_)                                                                              \
  pack_write_events_kernel<T_><<<grid, 256, 0, stream>>>(                                                \
      reinterpret_cast<uint8_t*>(out), input_ids, target_ids, reinterpret_cast<const T_*>(key_rep),     \
      pressure, per_token_ce, positions, candidate_base, (int)M, (int)B, (int)T, (int)D,                \
      (uint64_t)gpu_step, (int)source_rank, (int)write_bucket, (int)fingerprint_window, (int)span_length, \
      (int)key_rep_dim)
  switch (rep_dtype) {
    case 0: CCB_PACK_LAUNCH(float); break;
    case 1: CCB_PACK_LAUNCH(__nv_bfloat16); break;
    case 2: CCB_PACK_LAUNCH(__half); break;
    default: return set_error("ccb_pack_write_events: rep_dtype %lld not in {0: fp32, 1: bf16, 2: fp16}",
                              (long long)rep_dtype);
  }
#undef CCB_PACK_LAUNCH
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("pack_write_events launch: %s", cudaGetErrorString(e));
}
