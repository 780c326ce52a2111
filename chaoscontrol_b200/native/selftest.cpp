// Stand-alone stress driver for the host-side lock-free code: the SPSC ring (in-process and over a
// POSIX shared-memory segment) and the signal-pad epoch protocol.  It is built with
// -fsanitize=thread or -fsanitize=address by `python -m chaoscontrol_b200._build --sanitize ...`
// and run as a plain executable, so the sanitizer sees every access of the producer / consumer /
// rank threads without a Python interpreter in the process.  Exit code 0 = every check held; the
// sanitizer's own exit code (66) = it found a race or a bad access.
//
// The memory-ordering argument these runs exercise is the one in ring.h: a slot is published by a
// release store of the write index and observed by an acquire load (and symmetrically for the read
// index); the reference states the same contract in kernels/_cpu_ssm_controller/src/spsc_ring.h:7-21.
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <thread>
#include <vector>

#include "ring.h"

extern "C" {
int64_t ccbc_pad_words();
int ccbc_pad_allreduce(float* grad, int64_t n, float* const* staging, uint32_t* const* pads, int rank, int ws,
                       uint32_t epoch, float scale, int64_t timeout_us, int skip_signal_row);
}

namespace {

struct Rec {
  uint64_t seq;
  uint64_t payload[8];
};

int fail(const char* what) {
  std::fprintf(stderr, "selftest: %s\n", what);
  return 1;
}

// one producer thread, one consumer thread, `n` records through a ring bound to `mem_p` / `mem_c`
// (the same memory, possibly through two different mappings)
int ring_stress(void* mem_p, void* mem_c, std::size_t cap, uint64_t n) {
  ccb::RingView prod, cons;
  if (!prod.bind(mem_p, sizeof(Rec), cap, true) || !cons.bind(mem_c, sizeof(Rec), cap, false)) return fail("ring bind");
  std::atomic<int> bad{0};
  std::thread tp([&] {
    for (uint64_t i = 0; i < n; ++i) {
      Rec r;
      r.seq = i;
      for (int k = 0; k < 8; ++k) r.payload[k] = i * 31 + k;
      while (!prod.push(&r)) std::this_thread::yield();
    }
  });
  std::thread tc([&] {
    for (uint64_t i = 0; i < n; ++i) {
      Rec r;
      while (!cons.pop(&r)) std::this_thread::yield();
      if (r.seq != i) bad.fetch_add(1);
      for (int k = 0; k < 8; ++k)
        if (r.payload[k] != i * 31 + k) bad.fetch_add(1);
    }
  });
  tp.join();
  tc.join();
  if (bad.load()) return fail("ring delivered a torn or reordered record");
  if (cons.size() != 0) return fail("ring not empty after the run");
  return 0;
}

int pad_stress(int ws, int epochs, int64_t n) {
  const int64_t words = ccbc_pad_words();
  std::vector<std::vector<uint32_t>> pads(ws, std::vector<uint32_t>(words, 0));
  std::vector<std::vector<float>> staging(ws, std::vector<float>(n, 0.f)), grad(ws, std::vector<float>(n));
  std::vector<uint32_t*> pad_ptrs(ws);
  std::vector<float*> stg_ptrs(ws);
  for (int r = 0; r < ws; ++r) { pad_ptrs[r] = pads[r].data(); stg_ptrs[r] = staging[r].data(); }
  std::atomic<int> bad{0};
  std::vector<std::thread> th;
  for (int r = 0; r < ws; ++r)
    th.emplace_back([&, r] {
      for (int e = 1; e <= epochs; ++e) {
        for (int64_t i = 0; i < n; ++i) grad[r][i] = (float)(r + 1) * (float)(e % 7 + 1) + (float)(i % 5);
        const int st = ccbc_pad_allreduce(grad[r].data(), n, stg_ptrs.data(), pad_ptrs.data(), r, ws, (uint32_t)e,
                                          1.0f, 5'000'000, -1);
        if (st != 0) { bad.fetch_add(1); return; }
        float want0 = 0.f;
        for (int q = 0; q < ws; ++q) want0 += (float)(q + 1) * (float)(e % 7 + 1);
        for (int64_t i = 0; i < n; ++i)
          if (grad[r][i] != want0 + (float)ws * (float)(i % 5)) { bad.fetch_add(1); return; }
      }
    });
  for (auto& t : th) t.join();
  if (bad.load()) return fail("pad all-reduce gave a wrong sum or a non-zero status");
  // a rank that never calls: the others must give up with status 3 (peer timeout), not hang
  std::vector<int> status(ws, -1);
  th.clear();
  for (int r = 0; r + 1 < ws; ++r)
    th.emplace_back([&, r] {
      status[r] = ccbc_pad_allreduce(grad[r].data(), n, stg_ptrs.data(), pad_ptrs.data(), r, ws,
                                     (uint32_t)(epochs + 1), 1.0f, 50'000, -1);
    });
  for (auto& t : th) t.join();
  for (int r = 0; r + 1 < ws; ++r)
    if (status[r] != 3) return fail("a missing rank did not produce the peer-timeout status");
  return 0;
}

}  // namespace

int main() {
  // in-process ring
  {
    const std::size_t cap = 64;
    std::vector<uint8_t> mem(ccb::RingView::region_bytes(sizeof(Rec), cap) + 64);
    void* base = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(mem.data()) + 63) & ~uintptr_t(63));
    if (ring_stress(base, base, cap, 200000)) return 1;
  }
  // the same ring through two mappings of one POSIX shared-memory segment
  {
    const std::size_t cap = 128;
    const std::string name = "/ccb_selftest_" + std::to_string((long)getpid());
    ccb::ShmRegion owner, peer;
    std::string e = owner.open(name, ccb::RingView::region_bytes(sizeof(Rec), cap), true);
    if (!e.empty()) return fail(("shm create: " + e).c_str());
    e = peer.open(name, 0, false);
    if (!e.empty()) { ccb::ShmRegion::unlink(name); return fail(("shm attach: " + e).c_str()); }
    const int rc = ring_stress(owner.ptr(), peer.ptr(), cap, 100000);
    ccb::ShmRegion::unlink(name);
    if (rc) return 1;
  }
  if (pad_stress(4, 200, 257)) return 1;
  std::puts("selftest: ok");
  return 0;
}
