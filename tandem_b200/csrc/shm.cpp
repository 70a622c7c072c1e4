#include "shm.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <system_error>
#include <utility>

namespace tb {
namespace {

[[noreturn]] void fail(const char* call, const std::string& name, int err) {
  throw std::system_error(err, std::generic_category(), std::string(call) + " " + name);
}

// Maps `bytes` of `fd` shared and read-write.  The descriptor is not needed once
// the mapping exists, so it is closed on every path out of here.
void* map_and_close(int fd, std::size_t bytes, int* err) {
  void* p = ::mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  *err = (p == MAP_FAILED) ? errno : 0;
  ::close(fd);
  return p == MAP_FAILED ? nullptr : p;
}

}  // namespace

SharedMemory SharedMemory::create(const std::string& name, std::size_t bytes) {
  int fd = ::shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) fail("shm_open", name, errno);
  const bool bad_size = bytes == 0 || static_cast<off_t>(bytes) < 0;
  if (bad_size || ::ftruncate(fd, static_cast<off_t>(bytes)) != 0) {
    int err = bad_size ? EINVAL : errno;
    ::close(fd);
    ::shm_unlink(name.c_str());
    fail("ftruncate", name, err ? err : EINVAL);
  }
  int err = 0;
  void* p = map_and_close(fd, bytes, &err);
  if (p == nullptr) {
    ::shm_unlink(name.c_str());
    fail("mmap", name, err);
  }
  SharedMemory s;
  s.name_ = name;
  s.base_ = p;
  s.bytes_ = bytes;
  s.owner_ = true;
  return s;
}

SharedMemory SharedMemory::open(const std::string& name) {
  int fd = ::shm_open(name.c_str(), O_RDWR, 0600);
  if (fd < 0) fail("shm_open", name, errno);
  struct stat st {};
  if (::fstat(fd, &st) != 0) {
    int err = errno;
    ::close(fd);
    fail("fstat", name, err);
  }
  if (st.st_size <= 0) {
    ::close(fd);
    fail("fstat", name, EINVAL);  // created but not sized yet
  }
  int err = 0;
  void* p = map_and_close(fd, static_cast<std::size_t>(st.st_size), &err);
  if (p == nullptr) fail("mmap", name, err);
  SharedMemory s;
  s.name_ = name;
  s.base_ = p;
  s.bytes_ = static_cast<std::size_t>(st.st_size);
  s.owner_ = false;
  return s;
}

void SharedMemory::steal(SharedMemory& o) noexcept {
  name_ = std::move(o.name_);
  base_ = std::exchange(o.base_, nullptr);
  bytes_ = std::exchange(o.bytes_, 0);
  owner_ = std::exchange(o.owner_, false);
  o.name_.clear();
}

void SharedMemory::drop() noexcept {
  if (base_ != nullptr) ::munmap(base_, bytes_);
  if (owner_) ::shm_unlink(name_.c_str());
  base_ = nullptr;
  bytes_ = 0;
  owner_ = false;
  name_.clear();
}

}  // namespace tb
