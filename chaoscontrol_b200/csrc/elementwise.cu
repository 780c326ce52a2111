// Bandwidth-bound helpers around the GEMMs: embedding gather with fused row
// sum-of-squares, sorted scatter-add embedding backward, split-K reduction with
// the RMSNorm-weight fold, standalone RMSNorm (fwd/bwd) for callers outside
// the fused trunk, optimizer updates (Muon momentum / apply, AdamW, LAMB
// moments), global grad-norm clip, casts and the SGD step used by test-time
// training.  Everything is vectorised to 16-byte accesses where shapes allow.
//
// Reference counterparts: kernels/_lm_head_loss/src/rms_norm.cu:23-112 (RMSNorm),
// optim/muon.py:390-448 and 540-658 (Muon / AdamW updates),
// distributed.py:175-216 (fused grad clip).
#include "ptx.cuh"
#include "ccb_api.h"
#include "runtime.h"

namespace ccb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* sm) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) sm[w] = v;
  __syncthreads();
  float r = (threadIdx.x < nw) ? sm[threadIdx.x] : 0.f;
  if (w == 0) r = warp_sum(r);
  if (threadIdx.x == 0) sm[0] = r;
  __syncthreads();
  return sm[0];
}

// ---------------------------------------------------------------------------
// Embedding forward: x[r, :] = E[tok[r], :], ss[r] = sum x^2.  One warp per row.
// ---------------------------------------------------------------------------
template <typename TokT>
__global__ void embed_fwd_kernel(const TokT* __restrict__ tok, const __nv_bfloat16* __restrict__ E,
                                 __nv_bfloat16* __restrict__ x, float* __restrict__ ss, long long R,
                                 int D, int V) {
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= R) return;
  const int lane = threadIdx.x & 31;
  long long t = (long long)tok[r];
  t = t < 0 ? 0 : (t >= V ? V - 1 : t);
  const uint4* src = reinterpret_cast<const uint4*>(E + t * D);
  uint4* dst = reinterpret_cast<uint4*>(x + r * D);
  float acc = 0.f;
  for (int c = lane; c < D / 8; c += 32) {
    uint4 q = __ldg(src + c);
    dst[c] = q;
    float2 f;
    f = unpack_bf16x2(q.x); acc += f.x * f.x + f.y * f.y;
    f = unpack_bf16x2(q.y); acc += f.x * f.x + f.y * f.y;
    f = unpack_bf16x2(q.z); acc += f.x * f.x + f.y * f.y;
    f = unpack_bf16x2(q.w); acc += f.x * f.x + f.y * f.y;
  }
  acc = warp_sum(acc);
  if (lane == 0 && ss) ss[r] = acc;
}

// ---------------------------------------------------------------------------
// Embedding backward over token-sorted rows, bit-reproducible (no atomics).
//
// Stage 1: each warp owns CH = 32 consecutive sorted positions and sums the
// rows of each run of equal tokens in position order.  A run that lies wholly
// inside the chunk has one owner and is stored straight to dE.  A run that
// continues from the previous chunk or into the next one is written to the
// chunk's boundary slot instead: slot 0 for a run that starts at the chunk's
// first position, slot 1 for a run that starts later and runs off its end.
// Stage 1 also records, per token, the first and the last sorted position it occupies.
// Stage 2: one block per token whose rows span several chunks adds the
// boundary slots of those chunks in chunk order and stores the row of dE.
// The summation order is a function of the sorted token array alone, so two
// runs over the same batch give the same bits (the sort must be stable for
// `perm` itself to be reproducible).  dE must be zeroed by the caller: rows of
// tokens that do not occur are never written.
// ---------------------------------------------------------------------------
constexpr int EMB_CH = 32;

template <int VPL>   // uint4 vectors per lane: D = 256 * VPL
__global__ void embed_bwd_runs_kernel(const long long* __restrict__ sorted_tok,
                                      const long long* __restrict__ perm,
                                      const __nv_bfloat16* __restrict__ dx,
                                      float* __restrict__ dE, float* __restrict__ slots,
                                      long long* __restrict__ first_pos,
                                      long long* __restrict__ last_pos, long long R, int D, int V) {
  const long long chunk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long p0 = chunk * EMB_CH;
  if (p0 >= R) return;
  const long long p1 = (p0 + EMB_CH < R) ? p0 + EMB_CH : R;
  const int lane = threadIdx.x & 31;
  const int n = (int)(p1 - p0);
  // one coalesced load of the chunk's tokens and row indices, handed round by shuffles
  const long long my_tok = (lane < n) ? sorted_tok[p0 + lane] : -1;
  const long long my_row = (lane < n) ? perm[p0 + lane] : 0;
  const long long tok_before = (p0 > 0) ? sorted_tok[p0 - 1] : -1;
  const long long tok_after = (p1 < R) ? sorted_tok[p1] : -1;
  {
    // token boundaries: where a token's rows begin and end in the sorted order
    long long prev = __shfl_up_sync(0xffffffffu, my_tok, 1);
    long long next = __shfl_down_sync(0xffffffffu, my_tok, 1);
    if (lane == 0) prev = tok_before;
    if (lane == n - 1) next = tok_after;
    if (lane < n && my_tok >= 0 && my_tok < V) {
      if (prev != my_tok) first_pos[my_tok] = p0 + lane;
      if (next != my_tok) last_pos[my_tok] = p0 + lane;
    }
  }
  float acc[VPL][8];
#pragma unroll
  for (int v = 0; v < VPL; ++v)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[v][i] = 0.f;
  long long cur = __shfl_sync(0xffffffffu, my_tok, 0);
  int run_start = 0;
  auto flush = [&](long long tk, int a, int b) {
    // run of token tk over chunk positions [a, b)
    if (tk < 0 || tk >= V) return;
    const bool open_left = (a == 0) && (tok_before == tk);
    const bool open_right = (b == n) && (tok_after == tk);
    float* o;
    if (!open_left && !open_right) o = dE + tk * D;
    else o = slots + (chunk * 2 + (a == 0 ? 0 : 1)) * (long long)D;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      float4* o4 = reinterpret_cast<float4*>(o + (v * 32 + lane) * 8);
      o4[0] = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
      o4[1] = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
    }
  };
  for (int j0 = 0; j0 < n; j0 += 4) {
    // four rows are requested before any is added: the adds stay in position order
    uint4 q[4][VPL];
    long long tk[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u;
      tk[u] = __shfl_sync(0xffffffffu, my_tok, j & 31);
      const long long row = __shfl_sync(0xffffffffu, my_row, j & 31);
      if (j < n) {
        const uint4* src = reinterpret_cast<const uint4*>(dx + row * D);
#pragma unroll
        for (int v = 0; v < VPL; ++v) q[u][v] = __ldg(src + v * 32 + lane);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u;
      if (j >= n) break;
      if (tk[u] != cur) {
        flush(cur, run_start, j);
#pragma unroll
        for (int v = 0; v < VPL; ++v)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[v][i] = 0.f;
        cur = tk[u];
        run_start = j;
      }
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        float2 f;
        f = unpack_bf16x2(q[u][v].x); acc[v][0] += f.x; acc[v][1] += f.y;
        f = unpack_bf16x2(q[u][v].y); acc[v][2] += f.x; acc[v][3] += f.y;
        f = unpack_bf16x2(q[u][v].z); acc[v][4] += f.x; acc[v][5] += f.y;
        f = unpack_bf16x2(q[u][v].w); acc[v][6] += f.x; acc[v][7] += f.y;
      }
    }
  }
  flush(cur, run_start, n);
}

// grid: V blocks of 16 warps.  Warp w adds the boundary slots k = w, w + 16, ... of the token's
// chunk run in order (lane l owns columns [l * D/32, (l+1) * D/32)), then warp 0 adds the sixteen
// warp sums in warp order: a fixed tree, wide enough that the most frequent token of a Zipf batch
// (thousands of chunks) does not serialise behind one warp.
// first_pos / last_pos come from stage 1; last_pos is -1 for tokens that do not occur.
constexpr int EMB_JOIN_WARPS = 16;
template <int FPL>   // floats per lane: D = 32 * FPL
__global__ void __launch_bounds__(EMB_JOIN_WARPS * 32)
embed_bwd_join_kernel(const long long* __restrict__ first_pos, const long long* __restrict__ last_pos,
                      const float* __restrict__ slots, float* __restrict__ dE, int D) {
  const long long tk = blockIdx.x;
  const long long e = last_pos[tk] + 1;
  if (e <= 0) return;
  const long long s = first_pos[tk];
  const long long cs = s / EMB_CH, ce = (e - 1) / EMB_CH;
  if (cs == ce) return;                       // one owner: stored by stage 1
  extern __shared__ float sm_join[];          // [EMB_JOIN_WARPS][D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = lane * FPL;
  const long long n = ce - cs + 1;            // slots to add: chunk cs (first or second slot), then first slots
  const int first_slot = ((s % EMB_CH) == 0) ? 0 : 1;
  float acc[FPL];
#pragma unroll
  for (int i = 0; i < FPL; ++i) acc[i] = 0.f;
  auto slot_ptr = [&](long long k) {
    return slots + ((cs + k) * 2 + (k == 0 ? first_slot : 0)) * (long long)D + c0;
  };
  long long k = warp;
  for (; k + 3 * EMB_JOIN_WARPS < n; k += 4 * EMB_JOIN_WARPS) {
    float4 t[4][FPL / 4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float4* p = reinterpret_cast<const float4*>(slot_ptr(k + u * EMB_JOIN_WARPS));
#pragma unroll
      for (int i = 0; i < FPL / 4; ++i) t[u][i] = p[i];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int i = 0; i < FPL / 4; ++i) {
        acc[4 * i] += t[u][i].x; acc[4 * i + 1] += t[u][i].y;
        acc[4 * i + 2] += t[u][i].z; acc[4 * i + 3] += t[u][i].w;
      }
  }
  for (; k < n; k += EMB_JOIN_WARPS) {
    const float4* p = reinterpret_cast<const float4*>(slot_ptr(k));
#pragma unroll
    for (int i = 0; i < FPL / 4; ++i) {
      const float4 v = p[i];
      acc[4 * i] += v.x; acc[4 * i + 1] += v.y; acc[4 * i + 2] += v.z; acc[4 * i + 3] += v.w;
    }
  }
#pragma unroll
  for (int i = 0; i < FPL; ++i) sm_join[warp * D + c0 + i] = acc[i];
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float t = sm_join[c];
#pragma unroll
    for (int w = 1; w < EMB_JOIN_WARPS; ++w) t += sm_join[w * D + c];
    dE[tk * D + c] = t;
  }
}

// ---------------------------------------------------------------------------
// Split-K reduction.  out[n,k] (+)= colscale[k] * sum_s part[s,n,k]; when W is
// given also emits per-row-block partial column sums of sum[n,k] * W[n,k]
// (the gradient of an RMSNorm weight folded into W), reduced by a second tiny
// kernel so the result is deterministic.
// grid: ceil(N / 8); block: 256 threads striding over k.
// ---------------------------------------------------------------------------
__global__ void splitk_reduce_kernel(const float* __restrict__ part, int S, long long split_stride,
                                     int N, int K, const __nv_bfloat16* __restrict__ colscale,
                                     const __nv_bfloat16* __restrict__ W, float* __restrict__ out,
                                     int accumulate, float* __restrict__ colpart) {
  const int n0 = blockIdx.x * 8;
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const float cs = colscale ? __bfloat162float(colscale[k]) : 1.f;
    float cacc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int n = n0 + i;
      if (n < N) {
        float s = 0.f;
        const float* pp = part + (long long)n * K + k;
        int sp = 0;
        // four independent loads in flight, added in index order (the sum keeps its fixed order)
        for (; sp + 4 <= S; sp += 4) {
          const float v0 = pp[(long long)sp * split_stride], v1 = pp[(long long)(sp + 1) * split_stride];
          const float v2 = pp[(long long)(sp + 2) * split_stride], v3 = pp[(long long)(sp + 3) * split_stride];
          s += v0; s += v1; s += v2; s += v3;
        }
        for (; sp < S; ++sp) s += pp[(long long)sp * split_stride];
        const long long o = (long long)n * K + k;
        if (W) cacc += s * __bfloat162float(W[o]);
        const float val = s * cs;
        out[o] = accumulate ? out[o] + val : val;
      }
    }
    if (colpart) colpart[(long long)blockIdx.x * K + k] = cacc;
  }
}

// out[k] (+)= sum_b part[b, k].  Block: 32 columns x 32 row groups; group g adds rows g, g+32, ...
// in order, then the group sums are added in group order: a fixed tree, so the result
// does not depend on scheduling.
constexpr int COLSUM_COLS = 32, COLSUM_GROUPS = 32;
__global__ void colsum_kernel(const float* __restrict__ part, int NB, int K, float* __restrict__ out,
                              int accumulate) {
  __shared__ float sm[COLSUM_GROUPS][COLSUM_COLS];
  const int col = threadIdx.x & (COLSUM_COLS - 1), grp = threadIdx.x / COLSUM_COLS;
  const int k = blockIdx.x * COLSUM_COLS + col;
  float s = 0.f;
  if (k < K) {
    int b = grp;
    for (; b + 3 * COLSUM_GROUPS < NB; b += 4 * COLSUM_GROUPS) {
      const float v0 = part[(long long)b * K + k];
      const float v1 = part[(long long)(b + COLSUM_GROUPS) * K + k];
      const float v2 = part[(long long)(b + 2 * COLSUM_GROUPS) * K + k];
      const float v3 = part[(long long)(b + 3 * COLSUM_GROUPS) * K + k];
      s += v0; s += v1; s += v2; s += v3;
    }
    for (; b < NB; b += COLSUM_GROUPS) s += part[(long long)b * K + k];
  }
  sm[grp][col] = s;
  __syncthreads();
  if (grp == 0 && k < K) {
    float t = sm[0][col];
#pragma unroll
    for (int g = 1; g < COLSUM_GROUPS; ++g) t += sm[g][col];
    out[k] = accumulate ? out[k] + t : t;
  }
}

// W'[n,k] = W[n,k] * wn[k]  (bf16), the RMSNorm weight folded into a linear.
__global__ void fold_colscale_kernel(const __nv_bfloat16* __restrict__ W,
                                     const __nv_bfloat16* __restrict__ wn,
                                     __nv_bfloat16* __restrict__ out, long long N, int K) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * K) return;
  const int k = (int)(i % K);
  out[i] = __float2bfloat16(__bfloat162float(W[i]) * __bfloat162float(wn[k]));
}

// ---------------------------------------------------------------------------
// Standalone RMSNorm (one warp per row), fp32 statistics.
// y = x * rsqrt(mean(x^2) + eps) * w ; optional residual add x = x + res first.
// ---------------------------------------------------------------------------
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ res,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ xsum, float* __restrict__ inv_rms,
                                   long long R, int D, float eps) {
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= R) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* xr = x + r * D;
  float acc = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(xr + c));
    if (res) {
      float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(res + r * D + c));
      f.x = __bfloat162float(__float2bfloat16(f.x + g.x));
      f.y = __bfloat162float(__float2bfloat16(f.y + g.y));
      if (xsum) *reinterpret_cast<uint32_t*>(xsum + r * D + c) = pack_bf16x2(f.x, f.y);
    }
    acc += f.x * f.x + f.y * f.y;
  }
  acc = warp_sum(acc);
  const float inv = rsqrtf(acc / (float)D + eps);
  if (lane == 0 && inv_rms) inv_rms[r] = inv;
  for (int c = lane * 2; c < D; c += 64) {
    float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(xr + c));
    if (res) {
      float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(res + r * D + c));
      f.x = __bfloat162float(__float2bfloat16(f.x + g.x));
      f.y = __bfloat162float(__float2bfloat16(f.y + g.y));
    }
    float2 ww = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + c));
    *reinterpret_cast<uint32_t*>(y + r * D + c) = pack_bf16x2(f.x * inv * ww.x, f.y * inv * ww.y);
  }
}

// Backward: gx = inv * (go*w - xhat * mean(go*w*xhat)); weight grad as per-block partials
// [gridDim.x, D].  Inside a block every warp adds its rows, in row order, into its own [D] strip of
// shared memory (a lane owns its columns, so no atomics), the strips are added in warp order, and a
// second-stage column sum adds the blocks in order: the weight gradient is bit-reproducible.
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ go,
                                   const float* __restrict__ inv_rms, __nv_bfloat16* __restrict__ gx,
                                   float* __restrict__ gw_part, long long R, int D,
                                   int rows_per_block) {
  extern __shared__ float sm_gw[];   // [warps][D]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float* mine = sm_gw + warp * D;
  for (int c = lane; c < D; c += 32) mine[c] = 0.f;
  __syncwarp();
  const long long r0 = (long long)blockIdx.x * rows_per_block;
  for (long long r = r0 + warp; r < r0 + rows_per_block && r < R; r += nw) {
    const float inv = inv_rms[r];
    float dot = 0.f;
    for (int c = lane * 2; c < D; c += 64) {
      float2 xv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + r * D + c));
      float2 gv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(go + r * D + c));
      float2 wv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + c));
      dot += gv.x * wv.x * xv.x * inv + gv.y * wv.y * xv.y * inv;
    }
    dot = warp_sum(dot) / (float)D;
    for (int c = lane * 2; c < D; c += 64) {
      float2 xv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + r * D + c));
      float2 gv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(go + r * D + c));
      float2 wv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + c));
      const float xh0 = xv.x * inv, xh1 = xv.y * inv;
      *reinterpret_cast<uint32_t*>(gx + r * D + c) =
          pack_bf16x2(inv * (gv.x * wv.x - xh0 * dot), inv * (gv.y * wv.y - xh1 * dot));
      mine[c] += gv.x * xh0;
      mine[c + 1] += gv.y * xh1;
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float t = sm_gw[c];
    for (int k = 1; k < nw; ++k) t += sm_gw[k * D + c];
    gw_part[(long long)blockIdx.x * D + c] = t;
  }
}

// ---------------------------------------------------------------------------
// Optimizer kernels
// ---------------------------------------------------------------------------
// Muon momentum: buf = mu*buf + g ; dir = nesterov ? g + mu*buf : buf.  Writes dir in bf16 and the
// sum of squares of the bf16-rounded direction of each block's slice to a per-device scratch slot
// (grid: (blocks_per_mat, G); slot = matrix * blocks_per_mat + block).  No atomics: the normalise
// kernel adds a matrix's slots in index order, so the Frobenius norm is reproducible.
constexpr int MUON_PART_SLOTS = 16384;
__device__ float g_muon_part[MUON_PART_SLOTS];

__global__ void muon_momentum_kernel(const float* __restrict__ g, float* __restrict__ buf,
                                     __nv_bfloat16* __restrict__ dir, long long numel_per_mat, float mu,
                                     int nesterov) {
  __shared__ float sm[32];
  const long long base = (long long)blockIdx.y * numel_per_mat;
  float acc = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel_per_mat;
       i += (long long)gridDim.x * blockDim.x) {
    const float gv = g[base + i];
    const float b = mu * buf[base + i] + gv;
    buf[base + i] = b;
    const float dv = nesterov ? gv + mu * b : b;
    const __nv_bfloat16 q = __float2bfloat16(dv);
    dir[base + i] = q;
    const float qf = __bfloat162float(q);
    acc += qf * qf;
  }
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) g_muon_part[blockIdx.y * gridDim.x + blockIdx.x] = acc;
}

// X = dir / (||dir||_F + eps) in bf16, in place; sumsq[matrix] receives the squared norm.
// `nparts` is the momentum kernel's blocks_per_mat.
__global__ void muon_normalize_kernel(__nv_bfloat16* __restrict__ dir, float* __restrict__ sumsq,
                                      int nparts, long long numel_per_mat, float eps) {
  __shared__ float sm[32];
  float tot = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) tot += g_muon_part[blockIdx.y * nparts + i];
  tot = block_sum(tot, sm);                    // same fixed tree in every block of the matrix
  if (threadIdx.x == 0 && blockIdx.x == 0) sumsq[blockIdx.y] = tot;
  const long long base = (long long)blockIdx.y * numel_per_mat;
  const float inv = 1.f / (sqrtf(tot) + eps);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel_per_mat;
       i += (long long)gridDim.x * blockDim.x)
    dir[base + i] = __float2bfloat16(__bfloat162float(dir[base + i]) * inv);
}

// p = p * (1 - lr*wd) - lr*scale * O   (bf16 params, bf16 orthogonalised update)
__global__ void muon_apply_kernel(__nv_bfloat16* __restrict__ p, const __nv_bfloat16* __restrict__ O,
                                  long long n, float lr_scale, float decay_mul) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(p[i]) * decay_mul - lr_scale * __bfloat162float(O[i]);
    p[i] = __float2bfloat16(v);
  }
}

// Decoupled AdamW over a flat range; fp32 moments, bf16 or fp32 params.
template <typename PT>
__global__ void adamw_kernel(PT* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, long long n, float lr, float b1, float b2,
                             float eps, float wd, float bias1, float bias2_sqrt,
                             const float* __restrict__ gscale) {
  const float gs = gscale ? *gscale : 1.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gv = g[i] * gs;
    const float mi = b1 * m[i] + (1.f - b1) * gv;
    const float vi = b2 * v[i] + (1.f - b2) * gv * gv;
    m[i] = mi;
    v[i] = vi;
    float pv = (float)p[i];
    pv *= (1.f - lr * wd);
    pv -= (lr / bias1) * mi / (sqrtf(vi) / bias2_sqrt + eps);
    p[i] = (PT)pv;
  }
}

// Global L2 norm in two stages with a fixed summation order (no atomics): every block writes
// the sum of squares of its grid-stride slice to its own slot of a per-device scratch array, and
// the single-block second stage adds the slots in index order.  Two replicas that hold the same
// gradient bits therefore compute the same clip coefficient.
constexpr int SUMSQ_MAX_BLOCKS = 148 * 8;
__device__ float g_sumsq_part[SUMSQ_MAX_BLOCKS];

__global__ void sumsq_kernel(const float* __restrict__ g, long long n) {
  __shared__ float sm[32];
  float acc = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    acc += g[i] * g[i];
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) g_sumsq_part[blockIdx.x] = acc;
}

// stat = {sumsq, coef, norm}; coef = min(1, max_norm / (norm + 1e-6)).  One block of 256 threads.
__global__ void clip_coef_kernel(float* __restrict__ stat, int nparts, float max_norm) {
  __shared__ float sm[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) acc += g_sumsq_part[i];
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) {
    const float norm = sqrtf(acc);
    stat[0] = acc;
    stat[1] = fminf(1.f, max_norm / (norm + 1e-6f));
    stat[2] = norm;
  }
}
__global__ void scale_by_ptr_kernel(float* __restrict__ g, long long n, const float* __restrict__ coef) {
  const float c = *coef;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    g[i] *= c;
}

// p -= lr * g  (test-time-training SGD), bf16 params, fp32 grads.
__global__ void sgd_kernel(__nv_bfloat16* __restrict__ p, const float* __restrict__ g, long long n,
                           float lr) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    p[i] = __float2bfloat16(__bfloat162float(p[i]) - lr * g[i]);
}

// lse[m] from per-(tile, half) partials (max, sum 2^(z - max)) in the log2 domain;
// partials are laid out [nparts][M] so consecutive threads read consecutive rows.
__global__ void lse_combine_kernel(const float2* __restrict__ part, int nparts, long long M,
                                   const float* __restrict__ zt, float* __restrict__ lse,
                                   float* __restrict__ loss) {
  const long long m = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  float mx = -INFINITY;
  for (int i = 0; i < nparts; ++i) mx = fmaxf(mx, __ldg(&part[(long long)i * M + m]).x);
  float s = 0.f;
  for (int i = 0; i < nparts; ++i) {
    const float2 v = __ldg(&part[(long long)i * M + m]);
    if (v.y > 0.f) s += v.y * exp2f(v.x - mx);
  }
  const float l = (mx + log2f(s)) * 0.6931471805599453f;
  lse[m] = l;
  if (loss != nullptr && zt != nullptr) loss[m] = l - zt[m];
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ d,
                                        long long n, float scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    d[i] = __float2bfloat16(s[i] * scale);
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ s, float* __restrict__ d,
                                        long long n, float scale, int accumulate) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(s[i]) * scale;
    d[i] = accumulate ? d[i] + v : v;
  }
}

static inline int grid_for(long long n, int threads, int cap = 148 * 8) {
  long long b = (n + threads - 1) / threads;
  if (b < 1) b = 1;
  return (int)(b > cap ? cap : b);
}

}  // namespace ccb

using namespace ccb;
#define CCB_CHECK_LAUNCH(name)                                                   \
  do {                                                                           \
    count_launch();                                                              \
    cudaError_t e__ = cudaGetLastError();                                        \
    if (e__ != cudaSuccess) return set_error(name ": %s", cudaGetErrorString(e__)); \
  } while (0)

extern "C" int ccb_embed_fwd(const void* tok, int64_t tok_is_i64, const void* E, void* x, float* ss,
                             int64_t R, int64_t D, int64_t V, void* stream) {
  if (R <= 0) return 0;
  if (D % 8) return set_error("ccb_embed_fwd: D must be a multiple of 8");
  const int wpb = 8;
  const unsigned grid = (unsigned)((R + wpb - 1) / wpb);
  if (tok_is_i64)
    embed_fwd_kernel<long long><<<grid, wpb * 32, 0, (cudaStream_t)stream>>>(
        (const long long*)tok, (const __nv_bfloat16*)E, (__nv_bfloat16*)x, ss, R, (int)D, (int)V);
  else
    embed_fwd_kernel<int><<<grid, wpb * 32, 0, (cudaStream_t)stream>>>(
        (const int*)tok, (const __nv_bfloat16*)E, (__nv_bfloat16*)x, ss, R, (int)D, (int)V);
  CCB_CHECK_LAUNCH("embed_fwd");
  return 0;
}

// slots: workspace of ccb_embed_bwd_slots(R, D, V) floats, 16-byte aligned: the boundary sums of
// stage 1 followed by the per-token first / last positions (need not be initialised).
extern "C" int64_t ccb_embed_bwd_slots(int64_t R, int64_t D, int64_t V) {
  return ((R + EMB_CH - 1) / EMB_CH) * 2 * D + 4 * V;
}
extern "C" int ccb_embed_bwd_sorted(const int64_t* sorted_tok, const int64_t* perm, const void* dx,
                                    float* dE, float* slots, int64_t R, int64_t D, int64_t V,
                                    void* stream) {
  if (R <= 0) return 0;
  if (slots == nullptr) return set_error("ccb_embed_bwd_sorted: the boundary-slot workspace is required");
  const int wpb = 4;
  const long long chunks = (R + EMB_CH - 1) / EMB_CH;
  const unsigned grid = (unsigned)((chunks + wpb - 1) / wpb);
  cudaStream_t s = (cudaStream_t)stream;
  const long long* st = (const long long*)sorted_tok;
  const long long* pm = (const long long*)perm;
  const __nv_bfloat16* g = (const __nv_bfloat16*)dx;
  long long* fp = reinterpret_cast<long long*>(slots + chunks * 2 * D);
  long long* lp = fp + V;
  cudaMemsetAsync(lp, 0xFF, sizeof(long long) * (size_t)V, s);      // -1: token does not occur
  if (D == 256) {
    embed_bwd_runs_kernel<1><<<grid, wpb * 32, 0, s>>>(st, pm, g, dE, slots, fp, lp, R, (int)D, (int)V);
    CCB_CHECK_LAUNCH("embed_bwd_runs");
    embed_bwd_join_kernel<8><<<(unsigned)V, EMB_JOIN_WARPS * 32, EMB_JOIN_WARPS * D * sizeof(float), s>>>(
        fp, lp, slots, dE, (int)D);
  } else if (D == 512) {
    embed_bwd_runs_kernel<2><<<grid, wpb * 32, 0, s>>>(st, pm, g, dE, slots, fp, lp, R, (int)D, (int)V);
    CCB_CHECK_LAUNCH("embed_bwd_runs");
    embed_bwd_join_kernel<16><<<(unsigned)V, EMB_JOIN_WARPS * 32, EMB_JOIN_WARPS * D * sizeof(float), s>>>(
        fp, lp, slots, dE, (int)D);
  } else if (D == 1024) {
    embed_bwd_runs_kernel<4><<<grid, wpb * 32, 0, s>>>(st, pm, g, dE, slots, fp, lp, R, (int)D, (int)V);
    CCB_CHECK_LAUNCH("embed_bwd_runs");
    // sixteen [1024] strips are 64 KiB of shared memory: above the default limit, opt in
    cudaFuncSetAttribute(embed_bwd_join_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)(EMB_JOIN_WARPS * 1024 * sizeof(float)));
    embed_bwd_join_kernel<32><<<(unsigned)V, EMB_JOIN_WARPS * 32, EMB_JOIN_WARPS * D * sizeof(float), s>>>(
        fp, lp, slots, dE, (int)D);
  } else {
    return set_error("ccb_embed_bwd_sorted: D=%lld unsupported (256, 512, 1024)", (long long)D);
  }
  CCB_CHECK_LAUNCH("embed_bwd_join");
  return 0;
}

extern "C" int ccb_splitk_reduce(const float* part, int64_t S, int64_t split_stride, int64_t N,
                                 int64_t K, const void* colscale, const void* W, float* out,
                                 int64_t accumulate, float* colpart, float* colsum_out,
                                 int64_t colsum_accumulate, void* stream) {
  if (N <= 0 || K <= 0) return 0;
  const unsigned nb = (unsigned)((N + 7) / 8);
  cudaStream_t s = (cudaStream_t)stream;
  splitk_reduce_kernel<<<nb, 256, 0, s>>>(part, (int)S, split_stride, (int)N, (int)K,
                                          (const __nv_bfloat16*)colscale, (const __nv_bfloat16*)W,
                                          out, (int)accumulate, W ? colpart : nullptr);
  CCB_CHECK_LAUNCH("splitk_reduce");
  if (W && colpart && colsum_out) {
    colsum_kernel<<<(unsigned)((K + COLSUM_COLS - 1) / COLSUM_COLS), COLSUM_COLS * COLSUM_GROUPS, 0, s>>>(
        colpart, (int)nb, (int)K, colsum_out, (int)colsum_accumulate);
    CCB_CHECK_LAUNCH("colsum");
  }
  return 0;
}

extern "C" int ccb_colsum(const float* part, int64_t NB, int64_t K, float* out, int64_t accumulate,
                          void* stream) {
  if (K <= 0) return 0;
  colsum_kernel<<<(unsigned)((K + COLSUM_COLS - 1) / COLSUM_COLS), COLSUM_COLS * COLSUM_GROUPS, 0,
                  (cudaStream_t)stream>>>(part, (int)NB, (int)K, out, (int)accumulate);
  CCB_CHECK_LAUNCH("colsum");
  return 0;
}

extern "C" int ccb_fold_colscale(const void* W, const void* wn, void* out, int64_t N, int64_t K,
                                 void* stream) {
  if (N * K <= 0) return 0;
  fold_colscale_kernel<<<(unsigned)((N * K + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)W, (const __nv_bfloat16*)wn, (__nv_bfloat16*)out, N, (int)K);
  CCB_CHECK_LAUNCH("fold_colscale");
  return 0;
}

extern "C" int ccb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* xsum,
                               float* inv_rms, int64_t R, int64_t D, float eps, void* stream) {
  if (R <= 0) return 0;
  if (D % 2) return set_error("ccb_rmsnorm_fwd: D must be even");
  const int wpb = 8;
  rmsnorm_fwd_kernel<<<(unsigned)((R + wpb - 1) / wpb), wpb * 32, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
      (__nv_bfloat16*)xsum, inv_rms, R, (int)D, eps);
  CCB_CHECK_LAUNCH("rmsnorm_fwd");
  return 0;
}

// gw_part must hold ccb_rmsnorm_bwd_blocks(R) * D floats.  Eight per-warp [D] strips of shared
// memory bound the channel count (48 KiB without an opt-in).
constexpr int RMSNORM_BWD_MAX_DIM = 1536;
extern "C" int64_t ccb_rmsnorm_bwd_blocks(int64_t R) {
  const int64_t rpb = 256;
  return (R + rpb - 1) / rpb;
}
extern "C" int ccb_rmsnorm_bwd(const void* x, const void* w, const void* go, const float* inv_rms,
                               void* gx, float* gw_part, float* gw_out, int64_t R, int64_t D,
                               void* stream) {
  if (R <= 0) return 0;
  const int rpb = 256;
  const unsigned nb = (unsigned)ccb_rmsnorm_bwd_blocks(R);
  if (D > RMSNORM_BWD_MAX_DIM) return set_error("ccb_rmsnorm_bwd: D=%lld exceeds %d", (long long)D, RMSNORM_BWD_MAX_DIM);
  rmsnorm_bwd_kernel<<<nb, 256, (size_t)8 * D * sizeof(float), (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)go, inv_rms,
      (__nv_bfloat16*)gx, gw_part, R, (int)D, rpb);
  CCB_CHECK_LAUNCH("rmsnorm_bwd");
  if (gw_out) {
    colsum_kernel<<<(unsigned)((D + COLSUM_COLS - 1) / COLSUM_COLS), COLSUM_COLS * COLSUM_GROUPS, 0,
                    (cudaStream_t)stream>>>(gw_part, (int)nb, (int)D, gw_out, 0);
    CCB_CHECK_LAUNCH("colsum");
  }
  return 0;
}

static inline int muon_blocks_per_mat(int64_t G, int64_t numel_per_mat) {
  int cap = (int)(G >= 16 ? 74 : 1184 / G);
  if ((int64_t)cap * G > MUON_PART_SLOTS) cap = (int)(MUON_PART_SLOTS / G);
  return grid_for(numel_per_mat, 256, cap < 1 ? 1 : cap);
}
// The two calls form one unit: normalize reads the per-block sums the momentum launch left in the
// per-device scratch, so they must run back to back on one stream with the same (G, numel_per_mat).
extern "C" int ccb_muon_momentum(const float* g, float* buf, void* dir, float* sumsq, int64_t G,
                                 int64_t numel_per_mat, float mu, int64_t nesterov, void* stream) {
  if (G <= 0 || numel_per_mat <= 0) return 0;
  if (G > MUON_PART_SLOTS) return set_error("ccb_muon_momentum: at most %d matrices per call", MUON_PART_SLOTS);
  (void)sumsq;
  dim3 grid((unsigned)muon_blocks_per_mat(G, numel_per_mat), (unsigned)G);
  muon_momentum_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(g, buf, (__nv_bfloat16*)dir,
                                                               numel_per_mat, mu, (int)nesterov);
  CCB_CHECK_LAUNCH("muon_momentum");
  return 0;
}
extern "C" int ccb_muon_normalize(void* dir, float* sumsq, int64_t G, int64_t numel_per_mat,
                                  float eps, void* stream) {
  if (G <= 0 || numel_per_mat <= 0) return 0;
  if (G > MUON_PART_SLOTS) return set_error("ccb_muon_normalize: at most %d matrices per call", MUON_PART_SLOTS);
  const int nparts = muon_blocks_per_mat(G, numel_per_mat);
  dim3 grid((unsigned)nparts, (unsigned)G);
  muon_normalize_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)dir, sumsq, nparts,
                                                                numel_per_mat, eps);
  CCB_CHECK_LAUNCH("muon_normalize");
  return 0;
}
extern "C" int ccb_muon_apply(void* p, const void* O, int64_t n, float lr_scale, float decay_mul,
                              void* stream) {
  if (n <= 0) return 0;
  muon_apply_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)p, (const __nv_bfloat16*)O, n, lr_scale, decay_mul);
  CCB_CHECK_LAUNCH("muon_apply");
  return 0;
}
extern "C" int ccb_adamw(void* p, int64_t p_is_bf16, const float* g, float* m, float* v, int64_t n,
                         float lr, float b1, float b2, float eps, float wd, float bias1,
                         float bias2_sqrt, const float* gscale, void* stream) {
  if (n <= 0) return 0;
  if (p_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
        (__nv_bfloat16*)p, g, m, v, n, lr, b1, b2, eps, wd, bias1, bias2_sqrt, gscale);
  else
    adamw_kernel<float><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
        (float*)p, g, m, v, n, lr, b1, b2, eps, wd, bias1, bias2_sqrt, gscale);
  CCB_CHECK_LAUNCH("adamw");
  return 0;
}
// stat: 3 floats {sumsq, coef, norm}.  Computes the global L2 norm of g[0:n]
// and multiplies g by min(1, max_norm / (norm + 1e-6)) without a host sync.
extern "C" int ccb_clip_grad_norm(float* g, int64_t n, float max_norm, float* stat, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int nb = grid_for(n, 256, SUMSQ_MAX_BLOCKS);
  sumsq_kernel<<<nb, 256, 0, s>>>(g, n);
  CCB_CHECK_LAUNCH("sumsq");
  clip_coef_kernel<<<1, 256, 0, s>>>(stat, nb, max_norm);
  CCB_CHECK_LAUNCH("clip_coef");
  scale_by_ptr_kernel<<<grid_for(n, 256), 256, 0, s>>>(g, n, stat + 1);
  CCB_CHECK_LAUNCH("scale_by_ptr");
  return 0;
}
extern "C" int ccb_sgd(void* p, const float* g, int64_t n, float lr, void* stream) {
  if (n <= 0) return 0;
  sgd_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)p, g, n, lr);
  CCB_CHECK_LAUNCH("sgd");
  return 0;
}
extern "C" int ccb_lse_combine(const float* part, int64_t nparts, int64_t M, const float* zt, float* lse,
                               float* loss, void* stream) {
  if (M <= 0) return 0;
  lse_combine_kernel<<<(unsigned)((M + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const float2*)part, (int)nparts, (long long)M, zt, lse, loss);
  CCB_CHECK_LAUNCH("lse_combine");
  return 0;
}
extern "C" int ccb_cast_f32_to_bf16(const float* s, void* d, int64_t n, float scale, void* stream) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(s, (__nv_bfloat16*)d, n,
                                                                              scale);
  CCB_CHECK_LAUNCH("cast_f32_to_bf16");
  return 0;
}
extern "C" int ccb_cast_bf16_to_f32(const void* s, float* d, int64_t n, float scale,
                                    int64_t accumulate, void* stream) {
  if (n <= 0) return 0;
  cast_bf16_to_f32_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)s, d, n, scale, (int)accumulate);
  CCB_CHECK_LAUNCH("cast_bf16_to_f32");
  return 0;
}

// ---------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declared in ccb_noalloc.h).
// The per-block partial weight gradients live in an array that is part of the
// library image instead of a buffer handed in by the caller.
// ---------------------------------------------------------------------------
#include "ccb_noalloc.h"

namespace {
constexpr int64_t kNoallocRowsPerBlock = 256;
constexpr int64_t kNoallocMaxBlocks = CCB_NOALLOC_RMSNORM_MAX_ROWS / kNoallocRowsPerBlock;
// 256 blocks x 1024 channels x 4 B = 1 MiB, resident on every device that loads the library.
static __device__ __align__(256) float g_noalloc_rmsnorm_part[kNoallocMaxBlocks *
                                                               CCB_NOALLOC_RMSNORM_MAX_DIM];
// In host code the array's name is only a handle; the kernels need the device
// address, looked up once per device with that device current.
static float* g_noalloc_part_ptr[16] = {nullptr};
}  // namespace

extern "C" int ccb_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* go,
                                       const float* inv_rms, void* gx, float* gw_out, int64_t R,
                                       int64_t D, void* stream) {
  if (R <= 0) return 0;
  if (R > CCB_NOALLOC_RMSNORM_MAX_ROWS)
    return set_error("ccb_rmsnorm_bwd_noalloc: R=%lld exceeds the built-in workspace (max %d rows)",
                     (long long)R, CCB_NOALLOC_RMSNORM_MAX_ROWS);
  if (D <= 0 || D > CCB_NOALLOC_RMSNORM_MAX_DIM || (D % 2) != 0)
    return set_error("ccb_rmsnorm_bwd_noalloc: D=%lld unsupported (even, max %d)", (long long)D,
                     CCB_NOALLOC_RMSNORM_MAX_DIM);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error("cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 16) return set_error("ccb_rmsnorm_bwd_noalloc: device index %d unsupported", dev);
  if (g_noalloc_part_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_rmsnorm_part);
    if (e != cudaSuccess || p == nullptr)
      return set_error("cudaGetSymbolAddress(workspace): %s", cudaGetErrorString(e));
    g_noalloc_part_ptr[dev] = p;
  }
  float* part = g_noalloc_part_ptr[dev];
  const unsigned nb = (unsigned)((R + kNoallocRowsPerBlock - 1) / kNoallocRowsPerBlock);
  cudaStream_t s = (cudaStream_t)stream;
  rmsnorm_bwd_kernel<<<nb, 256, (size_t)8 * D * sizeof(float), s>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)go, inv_rms,
      (__nv_bfloat16*)gx, part, R, (int)D, (int)kNoallocRowsPerBlock);
  CCB_CHECK_LAUNCH("rmsnorm_bwd(noalloc)");
  colsum_kernel<<<(unsigned)((D + COLSUM_COLS - 1) / COLSUM_COLS), COLSUM_COLS * COLSUM_GROUPS, 0, s>>>(
      part, (int)nb, (int)D, gw_out, 0);
  CCB_CHECK_LAUNCH("colsum(noalloc)");
  return 0;
}
