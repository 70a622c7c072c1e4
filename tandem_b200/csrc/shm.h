// A named POSIX shared-memory mapping with exactly one owner object.
//
// Capability parity with the reference's tandem/csrc/shm.h:14-48: the creating
// process makes a zero-filled region and removes its name when the object
// dies; other processes map it by name; the type is move-only.  Every failure
// is a std::system_error whose text starts with the libc call that failed, and
// a failed create() leaves no name, descriptor or mapping behind.
#pragma once

#include <cstddef>
#include <string>

namespace tb {

class SharedMemory {
 public:
  SharedMemory() noexcept = default;
  static SharedMemory create(const std::string& name, std::size_t bytes);
  static SharedMemory open(const std::string& name);

  SharedMemory(const SharedMemory&) = delete;
  SharedMemory& operator=(const SharedMemory&) = delete;
  SharedMemory(SharedMemory&& o) noexcept { steal(o); }
  SharedMemory& operator=(SharedMemory&& o) noexcept {
    if (this != &o) {
      drop();
      steal(o);
    }
    return *this;
  }
  ~SharedMemory() { drop(); }

  void* data() const noexcept { return base_; }
  std::size_t size() const noexcept { return bytes_; }
  const std::string& name() const noexcept { return name_; }
  bool owner() const noexcept { return owner_; }
  // Unmaps now; the creator also unlinks the name.  Idempotent.
  void drop() noexcept;

 private:
  void steal(SharedMemory& o) noexcept;

  std::string name_;
  void* base_ = nullptr;
  std::size_t bytes_ = 0;
  bool owner_ = false;
};

}  // namespace tb
