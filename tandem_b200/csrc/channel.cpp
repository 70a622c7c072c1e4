#include "channel.h"

#include <cstring>
#include <new>
#include <stdexcept>

namespace tb {
namespace {

constexpr std::uint64_t kMagic = 0x316e616863326274ull;  // "tb2chan1"

struct alignas(64) Cursor {
  std::atomic<std::uint64_t> count;
  Bell bell;
};

struct Header {
  std::uint64_t magic;
  std::uint64_t slots;
  std::uint64_t slot_bytes;
  std::uint64_t stride;  // bytes from one entry to the next
  Cursor written;        // advanced by the sender only
  Cursor read;           // advanced by the receiver only
};

struct Entry {
  std::uint64_t length;
  unsigned char bytes[1];
};

Header* header(const SharedMemory& s) { return static_cast<Header*>(s.data()); }

Entry* entry(const SharedMemory& s, std::uint64_t k) {
  Header* h = header(s);
  auto* base = static_cast<unsigned char*>(s.data()) + sizeof(Header);
  return reinterpret_cast<Entry*>(base + (k % h->slots) * h->stride);
}

std::size_t round_up(std::size_t v, std::size_t to) { return (v + to - 1) / to * to; }

}  // namespace

Channel Channel::create(const std::string& name, std::size_t slots, std::size_t slot_bytes) {
  if (slots == 0 || slot_bytes == 0) throw std::invalid_argument("a channel needs at least one slot of at least one byte");
  std::size_t stride = round_up(sizeof(std::uint64_t) + slot_bytes, 64);
  SharedMemory shm = SharedMemory::create(name, sizeof(Header) + slots * stride);
  Header* h = new (shm.data()) Header;
  h->slots = slots;
  h->slot_bytes = slot_bytes;
  h->stride = stride;
  h->written.count.store(0, std::memory_order_relaxed);
  h->written.bell.store(0, std::memory_order_relaxed);
  h->read.count.store(0, std::memory_order_relaxed);
  h->read.bell.store(0, std::memory_order_relaxed);
  std::atomic_thread_fence(std::memory_order_release);
  h->magic = kMagic;  // last: a region without it is not (yet) a channel
  return Channel(std::move(shm));
}

Channel Channel::open(const std::string& name) {
  SharedMemory shm = SharedMemory::open(name);
  if (shm.size() < sizeof(Header) || header(shm)->magic != kMagic)
    throw std::runtime_error("region " + name + " is not a channel (bad magic number)");
  Header* h = header(shm);
  if (shm.size() < sizeof(Header) + h->slots * h->stride) throw std::runtime_error("channel " + name + " is truncated");
  return Channel(std::move(shm));
}

std::size_t Channel::slot_count() const noexcept { return valid() ? header(shm_)->slots : 0; }
std::size_t Channel::slot_capacity() const noexcept { return valid() ? header(shm_)->slot_bytes : 0; }

void Channel::wait_writable(double timeout_s) {
  Header* h = header(shm_);
  std::uint64_t w = h->written.count.load(std::memory_order_relaxed);
  wait_for([&] { return w - h->read.count.load(std::memory_order_acquire) < h->slots; }, h->read.bell, timeout_s, abort_,
           "a free slot in the channel");
}

void Channel::send(const void* data, std::size_t n, double timeout_s) {
  Header* h = header(shm_);
  if (n > h->slot_bytes) throw std::invalid_argument("message of " + std::to_string(n) + " bytes exceeds the slot size");
  wait_writable(timeout_s);
  std::uint64_t w = h->written.count.load(std::memory_order_relaxed);
  Entry* e = entry(shm_, w);
  e->length = n;
  if (n) std::memcpy(e->bytes, data, n);
  h->written.count.store(w + 1, std::memory_order_release);
  ring(h->written.bell);
}

MessageView Channel::front(double timeout_s) {
  Header* h = header(shm_);
  std::uint64_t r = h->read.count.load(std::memory_order_relaxed);
  wait_for([&] { return h->written.count.load(std::memory_order_acquire) > r; }, h->written.bell, timeout_s, abort_,
           "a message in the channel");
  Entry* e = entry(shm_, r);
  return MessageView{e->bytes, static_cast<std::size_t>(e->length)};
}

void Channel::pop() {
  Header* h = header(shm_);
  std::uint64_t r = h->read.count.load(std::memory_order_relaxed);
  h->read.count.store(r + 1, std::memory_order_release);
  ring(h->read.bell);
}

void Channel::wake_all() {
  if (!valid()) return;
  ring(header(shm_)->written.bell);
  ring(header(shm_)->read.bell);
}

std::size_t Channel::recv(void* out, std::size_t capacity, double timeout_s) {
  const MessageView head = front(timeout_s);
  if (head.size > capacity)
    throw std::length_error("message of " + std::to_string(head.size) + " bytes does not fit " + std::to_string(capacity));
  if (head.size) std::memcpy(out, head.data, head.size);
  pop();
  return head.size;
}

}  // namespace tb
