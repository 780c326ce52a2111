// In-kernel gradient all-reduce over NVLink peer memory (one process per GPU,
// buffers shared with CUDA IPC, every peer mapped into every rank's address
// space).  Replaces flatten -> NCCL all_reduce -> unflatten + copy of the
// reference (src/chaoscontrol/distributed.py:86-97) with kernels that read the
// peers' buffers directly:
//
//   pack      grad (fp32) * scale -> bf16 into this rank's symmetric buffer;
//             the last block to finish publishes epoch flags to every peer.
//   one-shot  wait for all peers' flags, every rank reads the whole vector from
//             all peers (fixed rank order => bitwise identical sums on all
//             ranks), writes the fp32 gradient in place.  (ws-1) x S bytes in
//             per GPU: best for small S (the 10.7 M-parameter model: 21 MB).
//   two-shot  reduce-scatter (rank r sums slice r from all peers into an fp32
//             staging slice, publishes a second flag) then all-gather (every
//             rank reads every reduced slice).  2 (ws-1)/ws x S bytes per GPU.
//
// Flags are monotonically increasing 32-bit epochs written with
// st.release.sys into the *peer's* pad and polled locally with
// ld.acquire.sys.  Every poll is bounded: on expiry the kernel records
// CCB_ERR_PEER_TIMEOUT in the status word and returns without reducing, so a
// dead or late peer can never hang the GPU.  All remote data moves with plain
// per-thread loads; no TMA and nothing cluster-scoped touches peer memory.
#include "ptx.cuh"
#include "ccb_api.h"
#include "runtime.h"
#include <string.h>

namespace ccb {

constexpr int COMM_MAX_RANKS = 8;
constexpr int COMM_EPOCH_SLOT = 15;   // counters[15]: epoch of the last completed operation
constexpr int COMM_THREADS = 512;

struct PeerPtrs {
  __nv_bfloat16* buf[COMM_MAX_RANKS];   // symmetric bf16 data buffers
  float* buf2[COMM_MAX_RANKS];          // fp32 reduced-slice staging (two-shot)
  uint32_t* pad[COMM_MAX_RANKS];        // signal pads: [4][COMM_MAX_RANKS] uint32 each
};
struct CommRange {
  long long off8, len8;
  int owner, pad;
};
// pad rows: 0 = "packed epoch e", 1 = "done reading the packed data of epoch e",
// 2 = "slice reduced / owned parameters published, epoch e", 3 = "epoch e finished: my buffer may be reused",
// 4 / 5 = stop-flag words of even / odd sequence numbers (comm_flag_max_kernel).  A pad is 8 rows.

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// The epoch of a collective, either a host value or "device counter + add": with the counter in
// device memory nothing in a launch depends on host state, so a whole training step -- exchange
// included -- can be captured once in a CUDA graph and replayed.  The first kernel of an operation
// uses add = 1 (a new epoch), its later kernels too (the counter has not moved yet), and the last
// one stores the new epoch back (`bump` of last_block_signal); a follow-up operation that belongs
// to the same epoch (parameter publish / gather after a sharded reduce) uses add = 0.
struct EpochArg {
  const uint32_t* dev;
  uint32_t add;
  __device__ __forceinline__ uint32_t get() const { return dev ? (*dev + add) : add; }
};

// Bounded wait until *flag >= epoch.  Returns false on timeout.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t limit_ns,
                                          int* status) {
  if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if (globaltimer_ns() - t0 > limit_ns) {
      atomicCAS(status, CCB_OK, CCB_ERR_PEER_TIMEOUT);
      return false;
    }
    __nanosleep(64);
  }
}

// Block-wide: threads 0..ws-1 each wait on one peer's flag in row `row` of my pad.
__device__ __forceinline__ bool wait_all_peers(const uint32_t* my_pad, int row, int ws, uint32_t epoch,
                                               uint64_t limit_ns, int* status, int* sm_ok) {
  if (threadIdx.x == 0) *sm_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < ws) {
    if (!wait_flag(my_pad + row * COMM_MAX_RANKS + threadIdx.x, epoch, limit_ns, status))
      atomicExch(sm_ok, 0);
  }
  __syncthreads();
  return *sm_ok != 0;
}

// Last block to arrive publishes `epoch` into row `row`, column `rank` of every peer's pad.
// Every block arrives, also one whose flag wait ran out (`ok` false): the arrival counter then
// still returns to zero for the next launch, and nothing is published for an epoch whose data
// this rank did not produce.
__device__ __forceinline__ void last_block_signal(unsigned* counter, const PeerPtrs& pp, int row,
                                                  int rank, int ws, uint32_t epoch, int row2 = -1,
                                                  bool ok = true, uint32_t* bump = nullptr) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned old = atomicAdd(counter, 1u);
    if (old == gridDim.x - 1) {
      *counter = 0;
      if (bump != nullptr) *bump = epoch;      // the operation's last kernel moves the device epoch
      __threadfence_system();
      if (ok) {
        for (int p = 0; p < ws; ++p) {
          st_release_sys(pp.pad[p] + row * COMM_MAX_RANKS + rank, epoch);
          if (row2 >= 0) st_release_sys(pp.pad[p] + row2 * COMM_MAX_RANKS + rank, epoch);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(COMM_THREADS)
comm_pack_kernel(const float* __restrict__ grad, long long n, float scale, PeerPtrs pp, int rank,
                 int ws, EpochArg ea, uint32_t* bump, unsigned* counter, uint64_t limit_ns, int* status) {
  const uint32_t epoch = ea.get();
  __shared__ int sm_ok;
  // peers must have finished with everything I staged in the previous epoch
  if (!wait_all_peers(pp.pad[rank], 3, ws, epoch - 1, limit_ns, status, &sm_ok)) {
    last_block_signal(counter, pp, 0, rank, ws, epoch, -1, false, bump);   // count the arrival, publish nothing
    return;
  }
  __nv_bfloat16* out = pp.buf[rank];
  const long long n8 = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(grad)[2 * i];
    const float4 b = reinterpret_cast<const float4*>(grad)[2 * i + 1];
    uint4 q;
    q.x = pack_bf16x2(a.x * scale, a.y * scale);
    q.y = pack_bf16x2(a.z * scale, a.w * scale);
    q.z = pack_bf16x2(b.x * scale, b.y * scale);
    q.w = pack_bf16x2(b.z * scale, b.w * scale);
    reinterpret_cast<uint4*>(out)[i] = q;
  }
  last_block_signal(counter, pp, 0, rank, ws, epoch, -1, true, bump);
}

__device__ __forceinline__ void acc_bf16x8(float (&acc)[8], const uint4& q) {
  float2 f;
  f = unpack_bf16x2(q.x); acc[0] += f.x; acc[1] += f.y;
  f = unpack_bf16x2(q.y); acc[2] += f.x; acc[3] += f.y;
  f = unpack_bf16x2(q.z); acc[4] += f.x; acc[5] += f.y;
  f = unpack_bf16x2(q.w); acc[6] += f.x; acc[7] += f.y;
}

__global__ void __launch_bounds__(COMM_THREADS)
comm_oneshot_kernel(float* __restrict__ grad, long long n, PeerPtrs pp, int rank, int ws,
                    EpochArg ea, uint32_t* bump, unsigned* counter, uint64_t limit_ns, int* status) {
  const uint32_t epoch = ea.get();
  __shared__ int sm_ok;
  if (!wait_all_peers(pp.pad[rank], 0, ws, epoch, limit_ns, status, &sm_ok)) {
    last_block_signal(counter, pp, 1, rank, ws, epoch, 3, false, bump);   // count the arrival, publish nothing
    return;
  }
  const long long n8 = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 q[COMM_MAX_RANKS];
#pragma unroll
    for (int p = 0; p < COMM_MAX_RANKS; ++p)
      if (p < ws) q[p] = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(pp.buf[p]) + i);
#pragma unroll
    for (int p = 0; p < COMM_MAX_RANKS; ++p)
      if (p < ws) acc_bf16x8(acc, q[p]);
    reinterpret_cast<float4*>(grad)[2 * i] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    reinterpret_cast<float4*>(grad)[2 * i + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  last_block_signal(counter, pp, 1, rank, ws, epoch, 3, true, bump);
}

// two-shot, stage 1: this rank reduces slice `rank` into its fp32 staging buffer
__global__ void __launch_bounds__(COMM_THREADS)
comm_reduce_scatter_kernel(long long n, PeerPtrs pp, int rank, int ws, EpochArg ea, uint32_t* bump,
                           unsigned* counter, uint64_t limit_ns, int* status) {
  const uint32_t epoch = ea.get();
  __shared__ int sm_ok;
  if (!wait_all_peers(pp.pad[rank], 0, ws, epoch, limit_ns, status, &sm_ok)) {
    last_block_signal(counter, pp, 2, rank, ws, epoch, -1, false, bump);   // count the arrival, publish nothing
    return;
  }
  const long long slice8 = (n / 8) / ws;           // host guarantees divisibility
  const long long base = (long long)rank * slice8;
  float* out = pp.buf2[rank];
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < slice8;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 q[COMM_MAX_RANKS];
#pragma unroll
    for (int p = 0; p < COMM_MAX_RANKS; ++p)
      if (p < ws) q[p] = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(pp.buf[p]) + base + i);
#pragma unroll
    for (int p = 0; p < COMM_MAX_RANKS; ++p)
      if (p < ws) acc_bf16x8(acc, q[p]);
    reinterpret_cast<float4*>(out)[2 * i] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    reinterpret_cast<float4*>(out)[2 * i + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  last_block_signal(counter, pp, 2, rank, ws, epoch, -1, true, bump);
}

// two-shot, stage 2: gather every rank's reduced slice
__global__ void __launch_bounds__(COMM_THREADS)
comm_all_gather_kernel(float* __restrict__ grad, long long n, PeerPtrs pp, int rank, int ws,
                       EpochArg ea, uint32_t* bump, unsigned* counter, uint64_t limit_ns, int* status) {
  const uint32_t epoch = ea.get();
  __shared__ int sm_ok;
  if (!wait_all_peers(pp.pad[rank], 2, ws, epoch, limit_ns, status, &sm_ok)) {
    last_block_signal(counter, pp, 1, rank, ws, epoch, 3, false, bump);   // count the arrival, publish nothing
    return;
  }
  const long long slice4 = (n / 4) / ws;
  const long long total4 = slice4 * ws;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4;
       i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i / slice4);
    const long long j = i - (long long)p * slice4;
    const uint4 v = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(pp.buf2[p]) + j);
    reinterpret_cast<uint4*>(grad)[i] = v;
  }
  last_block_signal(counter, pp, 1, rank, ws, epoch, 3, true, bump);
}

// ---------------------------------------------------------------------------
// Sharded-optimizer path (distributed Muon): ownership is a list of ranges of
// the flat buffers, in units of 8 elements.  owner >= 0: that rank reduces the
// range, updates it, and publishes the new parameters; owner < 0: replicated --
// every rank reduces and updates it itself.
//
//   pack (above)       all gradients -> bf16 staging, flag row 0
//   reduce_ranges      sum of all peers' staged values over my + replicated ranges
//                      -> local fp32 gradient (written, not accumulated), row 1
//   ... local optimizer on owned matrices and replicated tensors ...
//   publish_params     my owned bf16 parameters -> my staging buffer (after every
//                      peer has finished reading my staged gradients), row 2
//   gather_params      every other owner's ranges, from its staging buffer, into
//                      my flat parameters, rows 1 + 3
// ---------------------------------------------------------------------------

__global__ void __launch_bounds__(COMM_THREADS)
comm_reduce_ranges_kernel(float* __restrict__ grad, const CommRange* __restrict__ ranges, int nranges,
                          PeerPtrs pp, int rank, int ws, EpochArg ea, uint32_t* bump, unsigned* counter,
                          uint64_t limit_ns, int* status) {
  const uint32_t epoch = ea.get();
  __shared__ int sm_ok;
  if (!wait_all_peers(pp.pad[rank], 0, ws, epoch, limit_ns, status, &sm_ok)) {
    last_block_signal(counter, pp, 1, rank, ws, epoch, -1, false, bump);   // count the arrival, publish nothing
    return;
  }
  for (int r = 0; r < nranges; ++r) {
    const CommRange rg = ranges[r];
    if (rg.owner >= 0 && rg.owner != rank) continue;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rg.len8;
         i += (long long)gridDim.x * blockDim.x) {
      const long long e = rg.off8 + i;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      uint4 q[COMM_MAX_RANKS];
#pragma unroll
      for (int p = 0; p < COMM_MAX_RANKS; ++p)
        if (p < ws) q[p] = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(pp.buf[p]) + e);
#pragma unroll
      for (int p = 0; p < COMM_MAX_RANKS; ++p)
        if (p < ws) acc_bf16x8(acc, q[p]);
      reinterpret_cast<float4*>(grad)[2 * e] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      reinterpret_cast<float4*>(grad)[2 * e + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
  last_block_signal(counter, pp, 1, rank, ws, epoch, -1, true, bump);
}

__global__ void __launch_bounds__(COMM_THREADS)
comm_publish_params_kernel(const __nv_bfloat16* __restrict__ param, const CommRange* __restrict__ ranges,
                           int nranges, PeerPtrs pp, int rank, int ws, EpochArg ea, uint32_t* bump, unsigned* counter,
                           uint64_t limit_ns, int* status) {
  const uint32_t epoch = ea.get();
  __shared__ int sm_ok;
  // my staging buffer still holds gradients until every peer has read them
  if (!wait_all_peers(pp.pad[rank], 1, ws, epoch, limit_ns, status, &sm_ok)) {
    last_block_signal(counter, pp, 2, rank, ws, epoch, -1, false, bump);   // count the arrival, publish nothing
    return;
  }
  uint4* out = reinterpret_cast<uint4*>(pp.buf[rank]);
  for (int r = 0; r < nranges; ++r) {
    const CommRange rg = ranges[r];
    if (rg.owner != rank) continue;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rg.len8;
         i += (long long)gridDim.x * blockDim.x)
      out[rg.off8 + i] = reinterpret_cast<const uint4*>(param)[rg.off8 + i];
  }
  last_block_signal(counter, pp, 2, rank, ws, epoch, -1, true, bump);
}

__global__ void __launch_bounds__(COMM_THREADS)
comm_gather_params_kernel(__nv_bfloat16* __restrict__ param, const CommRange* __restrict__ ranges,
                          int nranges, PeerPtrs pp, int rank, int ws, EpochArg ea, uint32_t* bump, unsigned* counter,
                          uint64_t limit_ns, int* status) {
  const uint32_t epoch = ea.get();
  __shared__ int sm_ok;
  if (!wait_all_peers(pp.pad[rank], 2, ws, epoch, limit_ns, status, &sm_ok)) {
    last_block_signal(counter, pp, 3, rank, ws, epoch, -1, false, bump);   // count the arrival, publish nothing
    return;
  }
  for (int r = 0; r < nranges; ++r) {
    const CommRange rg = ranges[r];
    if (rg.owner < 0 || rg.owner == rank || rg.owner >= ws) continue;
    const uint4* src = reinterpret_cast<const uint4*>(pp.buf[rg.owner]);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rg.len8;
         i += (long long)gridDim.x * blockDim.x)
      reinterpret_cast<uint4*>(param)[rg.off8 + i] = ld_relaxed_sys_v4(src + rg.off8 + i);
  }
  last_block_signal(counter, pp, 3, rank, ws, epoch, -1, true, bump);
}

// ---------------------------------------------------------------------------
// Bucketed exchange, overlapped with backward.  A bucket is a slice [r0, r1) of a
// device range table (units of 8 elements, disjoint ranges of the flat gradient).
// Each bucket is a complete one-shot all-reduce with its own epoch, launched on a
// side stream as soon as the backward pass has produced the bucket's gradients,
// with a small grid of small blocks so that it shares the GPU with the GEMMs of
// the layers still to come instead of displacing them.
// ---------------------------------------------------------------------------
constexpr int COMM_BUCKET_THREADS = 128;   // 128 x 64 registers: fits beside a resident GEMM / LM-head CTA

__global__ void __launch_bounds__(COMM_BUCKET_THREADS)
comm_pack_ranges_kernel(const float* __restrict__ grad, const CommRange* __restrict__ ranges, int r0,
                        int r1, float scale, PeerPtrs pp, int rank, int ws, EpochArg ea, uint32_t* bump,
                        unsigned* counter, uint64_t limit_ns, int* status) {
  const uint32_t epoch = ea.get();
  __shared__ int sm_ok;
  if (!wait_all_peers(pp.pad[rank], 3, ws, epoch - 1, limit_ns, status, &sm_ok)) {
    last_block_signal(counter, pp, 0, rank, ws, epoch, -1, false, bump);
    return;
  }
  uint4* out = reinterpret_cast<uint4*>(pp.buf[rank]);
  for (int r = r0; r < r1; ++r) {
    const CommRange rg = ranges[r];
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rg.len8;
         i += (long long)gridDim.x * blockDim.x) {
      const long long e = rg.off8 + i;
      const float4 a = reinterpret_cast<const float4*>(grad)[2 * e];
      const float4 b = reinterpret_cast<const float4*>(grad)[2 * e + 1];
      uint4 q;
      q.x = pack_bf16x2(a.x * scale, a.y * scale);
      q.y = pack_bf16x2(a.z * scale, a.w * scale);
      q.z = pack_bf16x2(b.x * scale, b.y * scale);
      q.w = pack_bf16x2(b.z * scale, b.w * scale);
      out[e] = q;
    }
  }
  last_block_signal(counter, pp, 0, rank, ws, epoch, -1, true, bump);
}

__global__ void __launch_bounds__(COMM_BUCKET_THREADS)
comm_oneshot_ranges_kernel(float* __restrict__ grad, const CommRange* __restrict__ ranges, int r0, int r1,
                           PeerPtrs pp, int rank, int ws, EpochArg ea, uint32_t* bump, unsigned* counter,
                           uint64_t limit_ns, int* status) {
  const uint32_t epoch = ea.get();
  __shared__ int sm_ok;
  if (!wait_all_peers(pp.pad[rank], 0, ws, epoch, limit_ns, status, &sm_ok)) {
    last_block_signal(counter, pp, 1, rank, ws, epoch, 3, false, bump);
    return;
  }
  for (int r = r0; r < r1; ++r) {
    const CommRange rg = ranges[r];
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rg.len8;
         i += (long long)gridDim.x * blockDim.x) {
      const long long e = rg.off8 + i;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      uint4 q[COMM_MAX_RANKS];
#pragma unroll
      for (int p = 0; p < COMM_MAX_RANKS; ++p)
        if (p < ws) q[p] = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(pp.buf[p]) + e);
#pragma unroll
      for (int p = 0; p < COMM_MAX_RANKS; ++p)
        if (p < ws) acc_bf16x8(acc, q[p]);
      reinterpret_cast<float4*>(grad)[2 * e] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      reinterpret_cast<float4*>(grad)[2 * e + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
  last_block_signal(counter, pp, 1, rank, ws, epoch, 3, true, bump);
}

// ---------------------------------------------------------------------------
// Broadcast through the symmetric buffers (parameter broadcast at start-up, coalesced
// parameter refresh): the root stages `n16` 16-byte words and raises flag row 0; every
// other rank waits for the ROOT's flag only, copies the words out of the root's buffer
// and, like the root, reports rows 1 and 3 ("done with the staged data of this epoch").
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(COMM_THREADS)
comm_bcast_put_kernel(const uint4* __restrict__ src, long long n16, PeerPtrs pp, int rank, int ws,
                      EpochArg ea, uint32_t* bump, unsigned* counter, uint64_t limit_ns, int* status) {
  const uint32_t epoch = ea.get();
  __shared__ int sm_ok;
  if (!wait_all_peers(pp.pad[rank], 3, ws, epoch - 1, limit_ns, status, &sm_ok)) {
    last_block_signal(counter, pp, 0, rank, ws, epoch, -1, false, bump);
    return;
  }
  uint4* out = reinterpret_cast<uint4*>(pp.buf[rank]);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = src[i];
  last_block_signal(counter, pp, 0, rank, ws, epoch, -1, true, bump);
}

__global__ void __launch_bounds__(COMM_THREADS)
comm_bcast_get_kernel(uint4* __restrict__ dst, long long n16, int root, PeerPtrs pp, int rank, int ws,
                      EpochArg ea, uint32_t* bump, unsigned* counter, uint64_t limit_ns, int* status) {
  const uint32_t epoch = ea.get();
  __shared__ int sm_ok;
  if (threadIdx.x == 0)
    sm_ok = wait_flag(pp.pad[rank] + 0 * COMM_MAX_RANKS + root, epoch, limit_ns, status) ? 1 : 0;
  __syncthreads();
  if (!sm_ok) {
    last_block_signal(counter, pp, 1, rank, ws, epoch, 3, false, bump);
    return;
  }
  if (rank != root) {
    const uint4* src = reinterpret_cast<const uint4*>(pp.buf[root]);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16;
         i += (long long)gridDim.x * blockDim.x)
      dst[i] = ld_relaxed_sys_v4(src + i);
  }
  last_block_signal(counter, pp, 1, rank, ws, epoch, 3, true, bump);
}

// ---------------------------------------------------------------------------
// Stop-flag consensus (maximum of one small integer per rank) through the signal pads:
// no collective library call and no buffer traffic.  Rows 4 and 5 alternate by the
// sequence number's parity, word = (seq << 8) | value: a rank can run at most one
// sequence ahead of the slowest peer, so the word a late reader wants is never overwritten.
// One warp; lane p talks to rank p.  out[0] = max over ranks, or -1 after a timeout.
// ---------------------------------------------------------------------------
__global__ void comm_flag_max_kernel(int value, PeerPtrs pp, int rank, int ws, uint32_t seq, int* out,
                                     uint64_t limit_ns, int* status) {
  const int p = threadIdx.x;
  const int row = 4 + (int)(seq & 1u);
  const uint32_t word = (seq << 8) | (uint32_t)(value & 0xFF);
  int got = 0;
  bool ok = true;
  if (p < ws) {
    st_release_sys(pp.pad[p] + row * COMM_MAX_RANKS + rank, word);
    const uint32_t* mine = pp.pad[rank] + row * COMM_MAX_RANKS + p;
    const uint64_t t0 = globaltimer_ns();
    while (true) {
      const uint32_t w = ld_acquire_sys(mine);
      if ((((w >> 8) - seq) & 0xFFFFFFu) < 0x800000u) { got = (int)(w & 0xFFu); break; }
      if (globaltimer_ns() - t0 > limit_ns) {
        atomicCAS(status, CCB_OK, CCB_ERR_PEER_TIMEOUT);
        ok = false;
        break;
      }
      __nanosleep(64);
    }
  }
  const bool all_ok = __all_sync(0xffffffffu, ok);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) got = max(got, __shfl_xor_sync(0xffffffffu, got, o));
  if (p == 0) out[0] = all_ok ? got : -1;
}

}  // namespace ccb

using namespace ccb;

extern "C" void* ccb_comm_malloc(int64_t bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) {
    set_error("ccb_comm_malloc(%lld): %s", (long long)bytes, cudaGetErrorString(cudaGetLastError()));
    return nullptr;
  }
  cudaMemset(p, 0, (size_t)bytes);
  cudaDeviceSynchronize();
  return p;
}
extern "C" int ccb_comm_free(void* p) {
  return cudaFree(p) == cudaSuccess ? 0 : set_error("cudaFree failed");
}
// Zero `bytes` of a communicator allocation and wait for it (pad reset during a resynchronisation).
extern "C" int ccb_comm_clear(void* p, int64_t bytes) {
  if (cudaMemset(p, 0, (size_t)bytes) != cudaSuccess) return set_error("ccb_comm_clear: cudaMemset failed");
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : set_error("ccb_comm_clear: synchronize failed");
}
extern "C" int ccb_ipc_get(void* ptr, void* out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return set_error("cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  memcpy(out64, &h, sizeof(h));
  return 0;
}
extern "C" void* ccb_ipc_open(const void* handle64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    set_error("cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    return nullptr;
  }
  return p;
}
extern "C" int ccb_ipc_close(void* p) {
  return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : set_error("cudaIpcCloseMemHandle failed");
}

// bufs / bufs2 / pads: host arrays of `ws` device pointers (peer-mapped; index
// `rank` is this rank's own allocation).  counters: 16 device uint32, zeroed: one arrival
// counter per kernel of this file, and in slot 15 the communicator's epoch (see EpochArg).
// mode 0 = one-shot, 1 = two-shot.  n must be a multiple of 8 * ws.
extern "C" int ccb_allreduce(float* grad, int64_t n, float scale, void* const* bufs,
                             void* const* bufs2, void* const* pads, int64_t rank, int64_t ws,
                             void* counters, int64_t mode, int64_t timeout_ms, void* stream) {
  if (ws < 1 || ws > COMM_MAX_RANKS) return set_error("ccb_allreduce: world size %lld unsupported", (long long)ws);
  if (n % (8 * ws) != 0) return set_error("ccb_allreduce: n=%lld must be a multiple of %lld", (long long)n, (long long)(8 * ws));
  PeerPtrs pp;
  for (int i = 0; i < COMM_MAX_RANKS; ++i) {
    pp.buf[i] = i < ws ? (__nv_bfloat16*)bufs[i] : nullptr;
    pp.buf2[i] = i < ws ? (float*)bufs2[i] : nullptr;
    pp.pad[i] = i < ws ? (uint32_t*)pads[i] : nullptr;
  }
  cudaStream_t s = (cudaStream_t)stream;
  unsigned* ctr = (unsigned*)counters;
  uint32_t* edev = ctr + COMM_EPOCH_SLOT;          // the communicator's epoch lives in device memory
  int* status = ccb_status_ptr();
  const uint64_t limit = (uint64_t)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
  const int sms = ccb_num_sms();
  long long want = (n / 8 + COMM_THREADS - 1) / COMM_THREADS;
  const int grid = (int)(want < sms ? (want < 1 ? 1 : want) : sms);
  comm_pack_kernel<<<grid, COMM_THREADS, 0, s>>>(grad, n, scale, pp, (int)rank, (int)ws,
                                                  EpochArg{edev, 1u}, nullptr, ctr + 0, limit, status);
  count_launch();
  if (mode == 0) {
    comm_oneshot_kernel<<<grid, COMM_THREADS, 0, s>>>(grad, n, pp, (int)rank, (int)ws,
                                                       EpochArg{edev, 1u}, edev, ctr + 1, limit, status);
    count_launch();
  } else {
    comm_reduce_scatter_kernel<<<grid, COMM_THREADS, 0, s>>>(n, pp, (int)rank, (int)ws,
                                                              EpochArg{edev, 1u}, nullptr, ctr + 2, limit, status);
    count_launch();
    comm_all_gather_kernel<<<grid, COMM_THREADS, 0, s>>>(grad, n, pp, (int)rank, (int)ws,
                                                          EpochArg{edev, 1u}, edev, ctr + 3, limit, status);
    count_launch();
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("allreduce launch: %s", cudaGetErrorString(e));
}

static void fill_peers(ccb::PeerPtrs& pp, void* const* bufs, void* const* bufs2, void* const* pads, int64_t ws) {
  for (int i = 0; i < ccb::COMM_MAX_RANKS; ++i) {
    pp.buf[i] = i < ws ? (__nv_bfloat16*)bufs[i] : nullptr;
    pp.buf2[i] = i < ws ? (float*)bufs2[i] : nullptr;
    pp.pad[i] = i < ws ? (uint32_t*)pads[i] : nullptr;
  }
}

// Sharded-optimizer collectives.  `ranges` is a DEVICE array of `nranges` records
// {int64 off8, int64 len8, int32 owner, int32 pad}.  phase 0: pack all gradients and
// reduce the owned + replicated ranges into `grad`; phase 1: publish the owned
// parameter ranges and gather everyone else's into `param` (bf16 flat buffer).
extern "C" int ccb_sharded_sync(int64_t phase, float* grad, void* param, int64_t n, float scale,
                                const void* ranges, int64_t nranges, void* const* bufs, void* const* bufs2,
                                void* const* pads, int64_t rank, int64_t ws, void* counters,
                                int64_t timeout_ms, void* stream) {
  if (ws < 1 || ws > COMM_MAX_RANKS) return set_error("ccb_sharded_sync: world size %lld unsupported", (long long)ws);
  if (n % 8 != 0) return set_error("ccb_sharded_sync: n=%lld must be a multiple of 8", (long long)n);
  PeerPtrs pp;
  fill_peers(pp, bufs, bufs2, pads, ws);
  cudaStream_t s = (cudaStream_t)stream;
  unsigned* ctr = (unsigned*)counters;
  uint32_t* edev = ctr + COMM_EPOCH_SLOT;          // the communicator's epoch lives in device memory
  int* status = ccb_status_ptr();
  const uint64_t limit = (uint64_t)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
  const int sms = ccb_num_sms();
  long long want = (n / 8 + COMM_THREADS - 1) / COMM_THREADS;
  const int grid = (int)(want < sms ? (want < 1 ? 1 : want) : sms);
  const CommRange* rg = reinterpret_cast<const CommRange*>(ranges);
  if (phase == 0) {
    comm_pack_kernel<<<grid, COMM_THREADS, 0, s>>>(grad, n, scale, pp, (int)rank, (int)ws, EpochArg{edev, 1u}, nullptr,
                                                    ctr + 0, limit, status);
    count_launch();
    comm_reduce_ranges_kernel<<<grid, COMM_THREADS, 0, s>>>(grad, rg, (int)nranges, pp, (int)rank, (int)ws,
                                                             EpochArg{edev, 1u}, edev, ctr + 4, limit, status);
    count_launch();
  } else {
    comm_publish_params_kernel<<<grid, COMM_THREADS, 0, s>>>((const __nv_bfloat16*)param, rg, (int)nranges, pp,
                                                              (int)rank, (int)ws, EpochArg{edev, 0u}, nullptr, ctr + 5, limit,
                                                              status);
    count_launch();
    comm_gather_params_kernel<<<grid, COMM_THREADS, 0, s>>>((__nv_bfloat16*)param, rg, (int)nranges, pp, (int)rank,
                                                             (int)ws, EpochArg{edev, 0u}, nullptr, ctr + 6, limit, status);
    count_launch();
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("sharded sync launch: %s", cudaGetErrorString(e));
}

// One bucket of the overlapped exchange: pack + one-shot reduce of ranges [r0, r1) of the device
// table (records {int64 off8, int64 len8, int32 owner, int32 pad}; owner is ignored here) on
// `stream`, with `blocks` blocks of 128 threads per kernel (0: one block per SM).
extern "C" int ccb_allreduce_ranges(float* grad, const void* ranges, int64_t r0, int64_t r1, float scale,
                                    void* const* bufs, void* const* bufs2, void* const* pads, int64_t rank,
                                    int64_t ws, void* counters, int64_t blocks,
                                    int64_t timeout_ms, void* stream) {
  if (ws < 1 || ws > COMM_MAX_RANKS) return set_error("ccb_allreduce_ranges: world size %lld unsupported", (long long)ws);
  if (r1 <= r0) return 0;
  PeerPtrs pp;
  fill_peers(pp, bufs, bufs2, pads, ws);
  cudaStream_t s = (cudaStream_t)stream;
  unsigned* ctr = (unsigned*)counters;
  uint32_t* edev = ctr + COMM_EPOCH_SLOT;          // the communicator's epoch lives in device memory
  int* status = ccb_status_ptr();
  const uint64_t limit = (uint64_t)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
  const int grid = (int)(blocks > 0 ? blocks : ccb_num_sms());
  const CommRange* rg = reinterpret_cast<const CommRange*>(ranges);
  comm_pack_ranges_kernel<<<grid, COMM_BUCKET_THREADS, 0, s>>>(grad, rg, (int)r0, (int)r1, scale, pp, (int)rank,
                                                               (int)ws, EpochArg{edev, 1u}, nullptr, ctr + 8, limit, status);
  count_launch();
  comm_oneshot_ranges_kernel<<<grid, COMM_BUCKET_THREADS, 0, s>>>(grad, rg, (int)r0, (int)r1, pp, (int)rank,
                                                                  (int)ws, EpochArg{edev, 1u}, edev, ctr + 9, limit, status);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("allreduce_ranges launch: %s", cudaGetErrorString(e));
}

// Broadcast `nbytes` (a multiple of 16, at most the symmetric buffer) from rank `root`'s `data` into every
// other rank's `data`.
extern "C" int ccb_comm_bcast(void* data, int64_t nbytes, int64_t root, void* const* bufs, void* const* bufs2,
                              void* const* pads, int64_t rank, int64_t ws, void* counters,
                              int64_t timeout_ms, void* stream) {
  if (ws < 1 || ws > COMM_MAX_RANKS) return set_error("ccb_comm_bcast: world size %lld unsupported", (long long)ws);
  if (nbytes % 16) return set_error("ccb_comm_bcast: nbytes=%lld must be a multiple of 16", (long long)nbytes);
  if (root < 0 || root >= ws) return set_error("ccb_comm_bcast: root %lld out of range", (long long)root);
  PeerPtrs pp;
  fill_peers(pp, bufs, bufs2, pads, ws);
  cudaStream_t s = (cudaStream_t)stream;
  unsigned* ctr = (unsigned*)counters;
  uint32_t* edev = ctr + COMM_EPOCH_SLOT;          // the communicator's epoch lives in device memory
  int* status = ccb_status_ptr();
  const uint64_t limit = (uint64_t)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
  const long long n16 = nbytes / 16;
  const int sms = ccb_num_sms();
  long long want = (n16 + COMM_THREADS - 1) / COMM_THREADS;
  const int grid = (int)(want < sms ? (want < 1 ? 1 : want) : sms);
  if (rank == root) {
    comm_bcast_put_kernel<<<grid, COMM_THREADS, 0, s>>>((const uint4*)data, n16, pp, (int)rank, (int)ws,
                                                        EpochArg{edev, 1u}, nullptr, ctr + 10, limit, status);
    count_launch();
  }
  comm_bcast_get_kernel<<<grid, COMM_THREADS, 0, s>>>((uint4*)data, n16, (int)root, pp, (int)rank, (int)ws,
                                                      EpochArg{edev, 1u}, edev, ctr + 11, limit, status);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("bcast launch: %s", cudaGetErrorString(e));
}

// out[0] (device int) = max over ranks of `value` (0..255), or -1 when a peer did not answer in time.
extern "C" int ccb_comm_flag_max(int64_t value, void* const* pads, int64_t rank, int64_t ws, int64_t seq,
                                 int* out, int64_t timeout_ms, void* stream) {
  if (ws < 1 || ws > COMM_MAX_RANKS) return set_error("ccb_comm_flag_max: world size %lld unsupported", (long long)ws);
  PeerPtrs pp;
  for (int i = 0; i < COMM_MAX_RANKS; ++i) {
    pp.buf[i] = nullptr;
    pp.buf2[i] = nullptr;
    pp.pad[i] = i < ws ? (uint32_t*)pads[i] : nullptr;
  }
  const uint64_t limit = (uint64_t)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
  comm_flag_max_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((int)value, pp, (int)rank, (int)ws,
                                                           (uint32_t)seq & 0xFFFFFFu, out, limit, ccb_status_ptr());
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("flag_max launch: %s", cudaGetErrorString(e));
}

// Single-GPU self-test hook: waits on a flag that nothing sets, with a short
// limit, and reports through the status word (used to test the timeout path).
namespace ccb {
__global__ void comm_wait_probe_kernel(const uint32_t* flag, uint32_t epoch, uint64_t limit_ns,
                                       int* status, int* result) {
  const bool ok = wait_flag(flag, epoch, limit_ns, status);
  *result = ok ? 1 : 0;
}
}  // namespace ccb
extern "C" int ccb_comm_wait_probe(const void* flag, int64_t epoch, int64_t timeout_ms, int* result,
                                   void* stream) {
  comm_wait_probe_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((const uint32_t*)flag, (uint32_t)epoch,
                                                            (uint64_t)timeout_ms * 1000000ull,
                                                            ccb_status_ptr(), result);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : set_error("wait probe launch: %s", cudaGetErrorString(e));
}
