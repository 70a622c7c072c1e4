// Waiting on words in shared memory: a short spin, then futex sleeps.
//
// Every counter that another process may be waiting on has a 32-bit "bell"
// next to it.  A publisher stores the counter (release), bumps the bell and
// wakes sleepers; a waiter re-checks its predicate whenever the bell moves.
// Sleeps are capped so a waiter also notices the deadline and the job-wide
// abort word without being woken.  (The reference polls with sleeps instead:
// tandem/csrc/channel.cpp:46-62.)
#pragma once

#include <linux/futex.h>
#include <sys/syscall.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace tb {

struct Timeout : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// Raised in every waiting rank once some rank has marked the job as failed.
struct Aborted : std::runtime_error {
  using std::runtime_error::runtime_error;
};

using Bell = std::atomic<std::uint32_t>;
static_assert(std::atomic<std::uint32_t>::is_always_lock_free, "bells live in shared memory");
static_assert(std::atomic<std::uint64_t>::is_always_lock_free, "counters live in shared memory");

inline double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

inline void ring(Bell& bell) {
  bell.fetch_add(1, std::memory_order_release);
  ::syscall(SYS_futex, reinterpret_cast<std::uint32_t*>(&bell), FUTEX_WAKE, INT32_MAX, nullptr, nullptr, 0);
}

// Blocks until pred() is true.  `bell` is rung by whoever can make it true.
// `abort_word` (may be null) holds 0 while the job is healthy, else 1 + the
// rank that failed.
template <class Pred>
void wait_for(Pred pred, Bell& bell, double timeout_s, const std::atomic<std::uint32_t>* abort_word,
              const char* what) {
  // A peer that is running answers within microseconds: poll for about that long before paying for a futex
  // sleep and its wake-up (tens of microseconds).
  for (int i = 0; i < 512; ++i) {
    if (pred()) return;
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  }
  const double deadline = now_s() + timeout_s;
  for (;;) {
    std::uint32_t seen = bell.load(std::memory_order_acquire);
    if (pred()) return;
    if (abort_word != nullptr) {
      std::uint32_t a = abort_word->load(std::memory_order_acquire);
      if (a != 0) throw Aborted(std::string("rank ") + std::to_string(a - 1) + " failed while this rank waited for " + what);
    }
    double left = deadline - now_s();
    if (left <= 0) throw Timeout(std::string("timed out waiting for ") + what);
    double nap = left < 0.05 ? left : 0.05;
    timespec ts;
    ts.tv_sec = static_cast<time_t>(nap);
    ts.tv_nsec = static_cast<long>((nap - static_cast<double>(ts.tv_sec)) * 1e9);
    ::syscall(SYS_futex, reinterpret_cast<std::uint32_t*>(&bell), FUTEX_WAIT, seen, &ts, nullptr, 0);
  }
}

}  // namespace tb
