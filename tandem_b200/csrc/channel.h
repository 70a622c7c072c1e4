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

// What the receiver sees of the message at the head of the ring.
struct MessageView {
  const void* data;
  std::size_t size;
};

class Channel {
 public:
  Channel() = default;

  // ---- making and finding a channel
  // create(): a new region called `name` with `slot_count` entries of `slot_capacity` payload bytes (both >= 1,
  // else std::invalid_argument).  open(): a region someone else created (std::runtime_error unless it starts
  // with the channel's magic number).
  static Channel create(const std::string& name, std::size_t slot_count, std::size_t slot_capacity);
  static Channel open(const std::string& name);
  bool valid() const noexcept { return shm_.data() != nullptr; }
  std::size_t slot_count() const noexcept;
  std::size_t slot_capacity() const noexcept;

  // Every wait below gives up with Timeout after `timeout_s`, and with Aborted as soon as the watched word
  // (the job-wide abort flag, optional) becomes non-zero; wake_all() rings both bells so that sleepers look.
  void watch(const std::atomic<std::uint32_t>* abort_word) noexcept { abort_ = abort_word; }
  void wake_all();

  // ---- sender
  void wait_writable(double timeout_s);                          // returns once an entry is free
  void send(const void* bytes, std::size_t size, double timeout_s);  // size > slot_capacity(): std::invalid_argument

  // ---- receiver
  // front() waits for the next message and shows it in place; it stays there until pop().  recv() copies it out
  // and pops it; a message larger than `capacity` raises std::length_error and stays in the ring.
  MessageView front(double timeout_s);
  void pop();
  std::size_t recv(void* out, std::size_t capacity, double timeout_s);

 private:
  explicit Channel(SharedMemory region) noexcept : shm_(std::move(region)) {}
  SharedMemory shm_;
  const std::atomic<std::uint32_t>* abort_ = nullptr;
};

}  // namespace tb
