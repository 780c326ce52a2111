// C ABI of libccb200: every kernel launcher is a plain `extern "C"` function
// taking raw device pointers, sizes and a CUDA stream, so the Python layer
// binds it with ctypes and no libtorch headers are compiled into the library.
// All launchers return 0 on success or a negative host-side error code; device
// side failures (a bounded wait that ran out) land in the status word returned
// by ccb_status_ptr() and are read back by ccb_read_status().
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- runtime --------------------------------------------------------------
int ccb_init(void);                      // per-process, per-current-device set-up
int* ccb_status_ptr(void);               // device int, 0 == OK
int ccb_read_status(int reset);          // synchronises; returns the status word
int ccb_num_sms(void);
int ccb_launch_count(void);              // kernels launched by this library so far
const char* ccb_last_error(void);

// ---- generic tcgen05 GEMM ---------------------------------------------------
// C[b][s] (M x N) = epilogue( sum_k opA(A)[m,k] * opB(B)[n,k] )
//   a_mn == 0: A is stored [M rows][K contiguous] (K-major)
//   a_mn == 1: A is stored [K rows][M contiguous] (MN-major, i.e. A^T in memory)
//   b_mn likewise for B with N.
// bf16 (or 8-bit float) operands, fp32 accumulation in TMEM.  `splits` > 1 partitions K; split s
// writes its own partial tile at C + s * c_split (the caller reduces).
enum CcbEpilogue {
  CCB_EPI_STORE = 0,          // out = alpha * acc + beta * Cin
  CCB_EPI_ROWSCALE = 1,       // out = rs(m) * acc,  rs = rsqrt(rowss[m] * inv_dim + eps)
  CCB_EPI_ROWSCALE_SILU = 2,  // u = rs(m) * acc -> C ; silu(u) -> C2
  CCB_EPI_RESID_SS = 3,       // out = R1 + acc ; ss_out[m] (+)= sum_n out^2
  CCB_EPI_DSILU = 4,          // out = acc * silu'(R1) * rs(m)
  CCB_EPI_RMSBWD = 5,         // out = R2 + acc - R1 * (rs^2 * inv_dim * sum_n acc * R1)   (N <= 512)
  // LM head for model dims the single-kernel fused head does not take (logits = rs(m) * acc):
  CCB_EPI_LSE_PART = 6,       // no C; part_out[(tile_n*2 + half) * M + m] = (max, sum 2^(z - max)) of
                              // z = logits * log2(e) over the half tile; zt_out[m] = logits[m, targets[m]]
  CCB_EPI_CE_GRAD = 7,        // out = (exp(logits - lse[m]) - [n == targets[m]]) * alpha * rowweight[m] * rs(m);
                              // zt_out[m] = lse[m] - logits[m, targets[m]]  (the row's cross-entropy)
};

typedef struct CcbGemmArgs {
  const void* A;
  const void* B;
  void* C;
  void* C2;
  const void* Cin;
  const void* R1;
  const void* R2;
  const float* rowss;
  float* ss_out;
  int64_t M, N, K;
  int64_t batch, splits;
  int64_t lda, ldb, ldc, ldcin, ldr;         // element strides between rows
  int64_t a_batch, b_batch, c_batch, cin_batch, c_split;  // element strides
  int64_t a_mn, b_mn;
  int64_t epi;
  int64_t out_fp32;                          // 1: C is float, 0: C is bf16
  int64_t ss_atomic;                         // RESID_SS: atomicAdd instead of store
  float alpha, beta, inv_dim, eps;
  // 8-bit float operands (tcgen05 kind::f8f6f4): 0 = bf16, 1 = e4m3, 2 = e5m2.
  // Both operands must then be K-major and K a multiple of 16.
  int64_t a_fp8, b_fp8;
  const float* dscale_a;                     // optional device scalars: alpha *= *dscale_a * *dscale_b
  const float* dscale_b;
  const void* bias;                          // optional bf16 [N], added in the STORE epilogue
  // LM-head epilogues
  const int64_t* targets;                    // [M]
  const float* lse;                          // [M] natural-log lse (CE_GRAD input)
  const float* rowweight;                    // [M] or null
  float* part_out;                           // [tiles_n * 2, M] float2 (LSE_PART)
  float* zt_out;                             // [M] or null
} CcbGemmArgs;

int ccb_gemm(const CcbGemmArgs* args, void* stream);

// lse[m] = ln sum_v exp(logits[m, v]) from the LSE_PART partials ([nparts, M] float2);
// loss[m] = lse[m] - zt[m] when both pointers are given.
int ccb_lse_combine(const float* part, int64_t nparts, int64_t M, const float* zt, float* lse, float* loss,
                    void* stream);

// ---- 8-bit float helpers (fmt: 1 = e4m3, 2 = e5m2) --------------------------
// out = fp8(x / *scale), *pending = max(*pending, max|x|)
int ccb_fp8_cast_amax(const void* x_bf16, void* out_u8, const float* scale, float* pending, int64_t n,
                      int64_t fmt, void* stream);
// out[c][r] = fp8(x[r][c] / *scale); optional colsum[c] += sum_r x[r][c]
int ccb_fp8_cast_transpose_amax(const void* x_bf16, void* out_u8, const float* scale, float* pending,
                                float* colsum, int64_t R, int64_t C, int64_t ldx, int64_t ldo, int64_t fmt,
                                void* stream);
// roll the amax history, append *pending, recompute *scale (nullptr: skip), zero *pending
int ccb_fp8_flush_amax(float* history, int64_t len, float* pending, float* scale, float max_rep, void* stream);

// ---- block-scaled e4m3 linear (1 x 128 activation scales, 128 x 128 weight scales) --------
// q[R,K] = e4m3(v / s), s_t[K/128, R]; v = x, or RMSNorm(x) * norm_w when norm_w is given
// (then inv_rms_out[R] and the bf16 normalised row y_out[R,K] are optional extra outputs).
int ccb_fp8_quant_rows(const void* x_bf16, int64_t ldx, const void* norm_w, float eps, void* q, float* s_t,
                       float* inv_rms_out, void* y_out, int64_t R, int64_t K, void* stream);
// q[N,K] = e4m3(w / s[n/128, k/128]); qt (optional) is the same matrix stored [K, N]
int ccb_fp8_quant_blocks(const void* w_bf16, void* q, void* qt, float* s, int64_t N, int64_t K, void* stream);
// C[M,N] = sum_kb sa_t[kb, m] * sb[(n/128) * sb_so + kb * sb_sk] * (A8[m, kb] . B8[n, kb]) (+ bias[n])
int ccb_fp8_block_gemm(const void* A8, const float* sa_t, const void* B8, const float* sb, int64_t sb_so,
                       int64_t sb_sk, void* C, int64_t ldc, int64_t out_fp32, const void* bias, int64_t M,
                       int64_t N, int64_t K, void* stream);

// ---- episodic write events ---------------------------------------------------
// Packs M selected (batch, position) candidates into 568-byte WriteEvent records
// (all-zero record = candidate dropped at a sequence edge).  rep_dtype: 0 fp32, 1 bf16, 2 fp16.
int ccb_pack_write_events(void* out, const int64_t* input_ids, const int64_t* target_ids, const void* key_rep,
                          int64_t rep_dtype, const float* pressure, const float* per_token_ce,
                          const int64_t* positions, const int64_t* candidate_base, int64_t M, int64_t B,
                          int64_t T, int64_t D, int64_t gpu_step, int64_t source_rank, int64_t write_bucket,
                          int64_t fingerprint_window, int64_t span_length, int64_t key_rep_dim, void* stream);

#ifdef __cplusplus
}
#endif
