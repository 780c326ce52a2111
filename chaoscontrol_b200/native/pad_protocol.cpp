// CPU statement of the epoch-flag protocol the peer-memory collectives run on
// the GPU (csrc/comm.cu): every rank owns a signal pad of 4 rows x 16 columns of
// 32-bit epochs; "rank r finished phase `row` of epoch e" is a release store of
// e into column r of that row on EVERY peer's pad, and "wait for phase `row`" is
// a bounded acquire spin until all columns of the own pad have reached e
// (wrap-safe signed comparison).  The same state machine compiled for the host
// lets failure handling be tested with threads that stall, skip a signal or
// reuse an old epoch, without involving a GPU:
//
//   status 0  every awaited flag arrived
//   status 3  a flag did not arrive within the limit          (CCB_ERR_PEER_TIMEOUT)
//   status 4  a flag is AHEAD of the awaited epoch by more than one: this rank
//             is running a stale epoch (e.g. it restarted and lost its counter)
//
// A one-shot all-reduce over host float buffers built on these waits is the
// end-to-end check that the four phases order the data accesses correctly.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <thread>

namespace {

constexpr int kMaxRanks = 16;
constexpr int kRows = 4;

inline std::atomic<uint32_t>* cell(uint32_t* pad, int row, int col) {
  return reinterpret_cast<std::atomic<uint32_t>*>(pad + row * kMaxRanks + col);
}

int wait_row(uint32_t* my_pad, int row, int ws, uint32_t epoch, int64_t timeout_us) {
  const auto t0 = std::chrono::steady_clock::now();
  for (int r = 0; r < ws; ++r) {
    for (;;) {
      const int32_t d = (int32_t)(cell(my_pad, row, r)->load(std::memory_order_acquire) - epoch);
      if (d > 1) return 4;
      if (d >= 0) break;
      const auto dt = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0);
      if (dt.count() > timeout_us) return 3;
      std::this_thread::yield();
    }
  }
  return 0;
}

}  // namespace

extern "C" {

int64_t ccbc_pad_words() { return kRows * kMaxRanks; }

// release-store `epoch` into (row, rank) of every peer's pad
void ccbc_pad_signal(uint32_t* const* pads, int ws, int row, int rank, uint32_t epoch) {
  for (int p = 0; p < ws; ++p) cell(pads[p], row, rank)->store(epoch, std::memory_order_release);
}

int ccbc_pad_wait(uint32_t* my_pad, int row, int ws, uint32_t epoch, int64_t timeout_us) {
  if (row < 0 || row >= kRows || ws < 1 || ws > kMaxRanks) return 2;
  return wait_row(my_pad, row, ws, epoch, timeout_us);
}

// One rank's side of a one-shot all-reduce (sum, optionally averaged):
//   wait row 3 of epoch-1 (peers are done with my staging buffer) -> copy grad into my staging buffer
//   -> signal row 0 -> wait row 0 -> read every peer's staging buffer, reduce into grad
//   -> signal rows 1 and 3.
// `skip_signal_row` >= 0 withholds that signal (fault injection); returns the first non-zero status.
int ccbc_pad_allreduce(float* grad, int64_t n, float* const* staging, uint32_t* const* pads, int rank, int ws,
                       uint32_t epoch, float scale, int64_t timeout_us, int skip_signal_row) {
  if (ws < 1 || ws > kMaxRanks || rank < 0 || rank >= ws) return 2;
  int st = wait_row(pads[rank], 3, ws, epoch - 1, timeout_us);
  if (st) return st;
  for (int64_t i = 0; i < n; ++i) staging[rank][i] = grad[i] * scale;
  if (skip_signal_row != 0) ccbc_pad_signal(pads, ws, 0, rank, epoch);
  st = wait_row(pads[rank], 0, ws, epoch, timeout_us);
  if (st) return st;
  for (int64_t i = 0; i < n; ++i) {
    float acc = 0.f;
    for (int p = 0; p < ws; ++p) acc += staging[p][i];   // fixed rank order: bit-identical on every rank
    grad[i] = acc;
  }
  if (skip_signal_row != 1) ccbc_pad_signal(pads, ws, 1, rank, epoch);
  if (skip_signal_row != 3) ccbc_pad_signal(pads, ws, 3, rank, epoch);
  return 0;
}

}  // extern "C"
