// A one-way message ring between two processes, in shared memory.
//
// One sender, one receiver.  `slots` fixed-size entries; message k sits in
// entry k % slots.  Two 64-bit counters that only grow say how many messages
// have been written and read; each lives on its own cache line with the bell
// (wait.h) its waiters sleep on.  A payload is published by a release store of
// `written` and claimed by an acquire load, and the same pairing runs the
// other way for `read`.  Capability parity: tandem/csrc/channel.h:41-79.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <utility>

#include "shm.h"
#include "wait.h"

namespace tb {

class Channel {
 public:
  Channel() = default;
  static Channel create(const std::string& name, std::size_t slots, std::size_t slot_bytes);
  static Channel open(const std::string& name);

  // Job-wide abort word checked while waiting (optional).
  void watch(const std::atomic<std::uint32_t>* abort_word) noexcept { abort_ = abort_word; }

  void send(const void* data, std::size_t n, double timeout_s);
  std::size_t recv(void* out, std::size_t capacity, double timeout_s);
  // Zero-copy receive: the payload stays in its entry until release().
  std::pair<const void*, std::size_t> peek(double timeout_s);
  void release();
  void wait_writable(double timeout_s);
  void wake_all();  // rings both bells so sleepers re-check the abort word

  std::size_t slots() const noexcept;
  std::size_t slot_bytes() const noexcept;
  bool valid() const noexcept { return shm_.data() != nullptr; }

 private:
  explicit Channel(SharedMemory shm) noexcept : shm_(std::move(shm)) {}
  SharedMemory shm_;
  const std::atomic<std::uint32_t>* abort_ = nullptr;
};

}  // namespace tb
