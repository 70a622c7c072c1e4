// One rank's host runtime: a progress thread that runs collectives in
// submission order, the Work handles it completes, and collectives between
// CPU ranks over shared memory.
//
// Design.  Every rank owns one shared "window": `slots` staging slots plus three
// counters (rounds posted / reduced / consumed).  All ranks map all windows, so
// a collective is direct reads of the peers' windows, the same shape as the GPU
// kernels that read peers' symmetric buffers over NVLink: all-reduce is
// two-shot (each rank reduces the chunk it owns straight out of everyone's
// slot, then everyone copies the reduced chunks), with no neighbour-to-neighbour
// ring and no per-piece handshake.  The chunk a rank owns and the order in which
// it folds the operands (ranks c+1, c+2, ..., c for chunk c) are those a ring
// reduce-scatter produces, so results equal the reference engines bit for bit
// (tandem/comm.py:301-305, tandem/csrc/collectives.cpp:299-304).
// Point-to-point transfers go through one Channel per ordered pair.
//
// Capability parity: tandem/csrc/collectives.h:43-126 (Work, Engine).
#pragma once

#include <condition_variable>
#include <cstdint>
#include <deque>
#include <exception>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "channel.h"
#include "reduce_cpu.h"
#include "shm.h"

namespace tb {

struct NotImplemented : std::logic_error {
  using std::logic_error::logic_error;
};

class Work {
 public:
  void wait();                 // blocks until the job has run; rethrows its error
  bool done() const;
  double started() const;      // steady clock seconds (time.perf_counter's clock)
  double finished() const;

 private:
  friend class Engine;
  void finish(std::exception_ptr error, double t0, double t1);
  mutable std::mutex mu_;
  std::condition_variable cv_;
  bool done_ = false;
  std::exception_ptr error_;
  double t0_ = 0, t1_ = 0;
};

class Engine {
 public:
  Engine(const std::string& job, int rank, int size, std::size_t slots, std::size_t slot_bytes, double timeout_s);
  ~Engine();
  Engine(const Engine&) = delete;
  Engine& operator=(const Engine&) = delete;

  void connect();  // maps every peer's window and channels, waiting for them to appear
  void close();    // runs what is queued, then stops the thread
  void abort();    // marks the job failed: every rank's waits throw Aborted promptly

  using Sizes = std::vector<std::int64_t>;
  std::shared_ptr<Work> all_reduce(void* p, std::int64_t numel, DType d, bool average);
  std::shared_ptr<Work> reduce_scatter(void* p, std::int64_t numel, DType d, Sizes sizes, bool average);
  std::shared_ptr<Work> all_gather(void* p, std::int64_t numel, DType d, Sizes sizes);
  std::shared_ptr<Work> broadcast(void* p, std::int64_t numel, DType d, int root);
  std::shared_ptr<Work> send(const void* p, std::int64_t nbytes, int dst);
  std::shared_ptr<Work> recv(void* p, std::int64_t nbytes, int src);
  std::shared_ptr<Work> sendrecv(const void* sp, std::int64_t sbytes, int dst, void* rp, std::int64_t rbytes, int src);
  std::shared_ptr<Work> barrier();
  // Runs an arbitrary job on the progress thread, in order with the collectives.
  std::shared_ptr<Work> submit(std::function<void()> job);

  int rank() const { return rank_; }
  int size() const { return size_; }
  std::uint64_t rounds() const { return round_; }

 private:
  struct Window;
  void loop();
  Sizes chunk_sizes(std::int64_t numel, const Sizes& sizes) const;
  Window* win(int r) const;
  unsigned char* slot(int r, std::uint64_t round) const;
  void wait_count(int r, int which, std::uint64_t value, const char* what);
  void publish(int which, std::uint64_t value);
  void claim_slot(std::uint64_t round);
  void do_all_reduce(unsigned char* p, std::int64_t numel, DType d, bool average, const Sizes& sizes, bool gather);
  void do_all_gather(unsigned char* p, std::int64_t numel, DType d, const Sizes& sizes);
  void do_broadcast(unsigned char* p, std::int64_t numel, DType d, int root);
  void do_exchange(const unsigned char* sp, std::int64_t sbytes, int dst, unsigned char* rp, std::int64_t rbytes, int src);
  void do_barrier();
  void check_peer(int r, const char* what) const;
  std::string region(const char* kind, int a, int b = -1) const;

  std::string job_;
  int rank_, size_;
  std::size_t slots_, slot_bytes_, stride_;
  double timeout_s_;
  std::vector<SharedMemory> windows_;
  std::vector<Channel> out_, in_;
  std::uint64_t round_ = 0;  // touched by the progress thread only
  bool connected_ = false;

  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::pair<std::function<void()>, std::shared_ptr<Work>>> jobs_;
  bool stopping_ = false;
  std::thread thread_;
};

}  // namespace tb
