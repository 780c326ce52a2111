// Lock-free single-producer / single-consumer ring over a raw memory region,
// usable in-process or across processes through POSIX shared memory.
//
// Region layout (shared with any other implementation that maps the same
// segment, cf. kernels/_cpu_ssm_controller/src/spsc_ring.h:51-118 and
// shm_ring.h:54-147 of the reference): the producer's 64-bit write index at
// byte 0, the consumer's 64-bit read index at byte 64, slots from byte 128,
// every part on its own cache line.  Element size and capacity (a power of
// two) are run-time values, so one compiled routine serves every record type.
//
// Memory ordering: the producer publishes a slot with a release store of the
// write index and the consumer observes it with an acquire load (and
// symmetrically for the read index), so a slot's bytes are always fully
// written before the consumer can see them and fully read before the producer
// can reuse them.
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <string>

namespace ccb {

constexpr std::size_t kCacheLine = 64;
constexpr std::size_t kRingHeaderBytes = 2 * kCacheLine;

struct RingView {
  std::atomic<uint64_t>* write_idx = nullptr;
  std::atomic<uint64_t>* read_idx = nullptr;
  uint8_t* slots = nullptr;
  std::size_t elem_bytes = 0;
  std::size_t capacity = 0;   // power of two

  static std::size_t region_bytes(std::size_t elem_bytes, std::size_t capacity) {
    return kRingHeaderBytes + elem_bytes * capacity;
  }
  static bool valid_capacity(std::size_t c) { return c > 0 && (c & (c - 1)) == 0; }

  // Bind to `mem` (>= region_bytes).  `init` zeroes the indices (creator only).
  bool bind(void* mem, std::size_t elem, std::size_t cap, bool init) {
    if (!mem || elem == 0 || !valid_capacity(cap)) return false;
    auto* base = static_cast<uint8_t*>(mem);
    write_idx = reinterpret_cast<std::atomic<uint64_t>*>(base);
    read_idx = reinterpret_cast<std::atomic<uint64_t>*>(base + kCacheLine);
    slots = base + kRingHeaderBytes;
    elem_bytes = elem;
    capacity = cap;
    if (init) {
      new (write_idx) std::atomic<uint64_t>(0);
      new (read_idx) std::atomic<uint64_t>(0);
    }
    return true;
  }
  bool push(const void* item) {
    const uint64_t w = write_idx->load(std::memory_order_relaxed);
    const uint64_t r = read_idx->load(std::memory_order_acquire);
    if (w - r >= capacity) return false;                       // full
    std::memcpy(slots + (w & (capacity - 1)) * elem_bytes, item, elem_bytes);
    write_idx->store(w + 1, std::memory_order_release);
    return true;
  }
  bool pop(void* out) {
    const uint64_t r = read_idx->load(std::memory_order_relaxed);
    const uint64_t w = write_idx->load(std::memory_order_acquire);
    if (r == w) return false;                                  // empty
    std::memcpy(out, slots + (r & (capacity - 1)) * elem_bytes, elem_bytes);
    read_idx->store(r + 1, std::memory_order_release);
    return true;
  }
  std::size_t size() const {
    const uint64_t r = read_idx->load(std::memory_order_acquire);
    const uint64_t w = write_idx->load(std::memory_order_acquire);
    return static_cast<std::size_t>(w - r);
  }
};

// RAII POSIX shared-memory mapping.  The creator sizes the segment; attachers
// recover the size with fstat.  Destruction unmaps and closes but never
// unlinks (the owner calls unlink() explicitly), so an attacher going away
// cannot pull the segment from under its peer.
class ShmRegion {
 public:
  ShmRegion() = default;
  ~ShmRegion() { reset(); }
  ShmRegion(const ShmRegion&) = delete;
  ShmRegion& operator=(const ShmRegion&) = delete;
  ShmRegion(ShmRegion&& o) noexcept { *this = std::move(o); }
  ShmRegion& operator=(ShmRegion&& o) noexcept;

  // Returns empty string on success, else a message.
  std::string open(const std::string& name, std::size_t size, bool create);
  void reset();
  static bool unlink(const std::string& name);

  void* ptr() const { return ptr_; }
  std::size_t size() const { return size_; }
  const std::string& name() const { return name_; }
  bool ok() const { return ptr_ != nullptr; }

 private:
  std::string name_;
  std::size_t size_ = 0;
  int fd_ = -1;
  void* ptr_ = nullptr;
};

}  // namespace ccb
