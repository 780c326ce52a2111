#include "ring.h"

#include <cerrno>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace ccb {

ShmRegion& ShmRegion::operator=(ShmRegion&& o) noexcept {
  if (this != &o) {
    reset();
    name_ = std::move(o.name_);
    size_ = o.size_;
    fd_ = o.fd_;
    ptr_ = o.ptr_;
    o.fd_ = -1;
    o.ptr_ = nullptr;
    o.size_ = 0;
  }
  return *this;
}

std::string ShmRegion::open(const std::string& name, std::size_t size, bool create) {
  reset();
  if (name.empty() || name[0] != '/') return "shm name must start with '/': '" + name + "'";
  if (create && size == 0) return "cannot create a zero-sized shm segment";
  const int flags = create ? (O_CREAT | O_RDWR) : O_RDWR;
  int fd = ::shm_open(name.c_str(), flags, create ? 0600 : 0);
  if (fd == -1) return "shm_open('" + name + "') failed: " + std::strerror(errno);
  if (create) {
    if (::ftruncate(fd, static_cast<off_t>(size)) == -1) {
      std::string msg = std::string("ftruncate failed: ") + std::strerror(errno);
      ::close(fd);
      return msg;
    }
  } else {
    struct stat st;
    if (::fstat(fd, &st) == -1) {
      std::string msg = std::string("fstat failed: ") + std::strerror(errno);
      ::close(fd);
      return msg;
    }
    size = static_cast<std::size_t>(st.st_size);
  }
  void* p = ::mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) {
    std::string msg = std::string("mmap failed: ") + std::strerror(errno);
    ::close(fd);
    return msg;
  }
  name_ = name;
  size_ = size;
  fd_ = fd;
  ptr_ = p;
  return "";
}

void ShmRegion::reset() {
  if (ptr_) ::munmap(ptr_, size_);
  if (fd_ != -1) ::close(fd_);
  ptr_ = nullptr;
  fd_ = -1;
  size_ = 0;
}

bool ShmRegion::unlink(const std::string& name) { return ::shm_unlink(name.c_str()) == 0; }

}  // namespace ccb
