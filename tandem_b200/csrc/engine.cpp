#include "engine.h"

#include <algorithm>
#include <chrono>
#include <cstring>
#include <new>
#include <numeric>
#include <system_error>

namespace tb {
namespace {

constexpr std::uint64_t kWindowMagic = 0x316e697732627474ull;
enum { POSTED = 0, REDUCED = 1, CONSUMED = 2 };

struct alignas(64) Counter {
  std::atomic<std::uint64_t> v;
};

std::size_t round_up(std::size_t v, std::size_t to) { return (v + to - 1) / to * to; }

std::int64_t ceil_div(std::int64_t a, std::int64_t b) { return (a + b - 1) / b; }

}  // namespace

struct Engine::Window {
  std::uint64_t magic;
  std::uint32_t ranks;
  std::uint32_t slots;
  std::uint64_t stride;
  Counter count[3];
  alignas(64) Bell bell;
  alignas(64) std::atomic<std::uint32_t> abort_word;  // meaningful in rank 0's window only
};

// ------------------------------------------------------------------ Work
void Work::wait() {
  std::unique_lock<std::mutex> lk(mu_);
  cv_.wait(lk, [&] { return done_; });
  if (error_) std::rethrow_exception(error_);
}

bool Work::done() const {
  std::lock_guard<std::mutex> lk(mu_);
  return done_;
}

double Work::started() const {
  std::lock_guard<std::mutex> lk(mu_);
  return t0_;
}

double Work::finished() const {
  std::lock_guard<std::mutex> lk(mu_);
  return t1_;
}

void Work::finish(std::exception_ptr error, double t0, double t1) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    error_ = error;
    t0_ = t0;
    t1_ = t1;
    done_ = true;
  }
  cv_.notify_all();
}

// ------------------------------------------------------------------ set-up
std::string Engine::region(const char* kind, int a, int b) const {
  std::string s = "/tb2-" + job_ + "-" + kind + std::to_string(a);
  if (b >= 0) s += "-" + std::to_string(b);
  return s;
}

Engine::Engine(const std::string& job, int rank, int size, std::size_t slots, std::size_t slot_bytes, double timeout_s)
    : job_(job), rank_(rank), size_(size), slots_(slots), slot_bytes_(slot_bytes), timeout_s_(timeout_s) {
  if (size < 1 || rank < 0 || rank >= size) throw std::invalid_argument("rank must lie in [0, size)");
  if (slots == 0 || slot_bytes == 0) throw std::invalid_argument("slots and slot_bytes must be positive");
  // A slot carries one piece of every rank's chunk, so it holds at least one
  // 8-byte element per rank however small slot_bytes is.
  stride_ = round_up(std::max<std::size_t>(slot_bytes, 8u * static_cast<std::size_t>(size)), 64);
  windows_.resize(size);
  out_.resize(size);
  in_.resize(size);
  windows_[rank] = SharedMemory::create(region("w", rank), sizeof(Window) + slots * stride_);
  Window* w = new (windows_[rank].data()) Window;
  w->ranks = static_cast<std::uint32_t>(size);
  w->slots = static_cast<std::uint32_t>(slots);
  w->stride = stride_;
  for (auto& c : w->count) c.v.store(0, std::memory_order_relaxed);
  w->bell.store(0, std::memory_order_relaxed);
  w->abort_word.store(0, std::memory_order_relaxed);
  std::atomic_thread_fence(std::memory_order_release);
  w->magic = kWindowMagic;
  for (int dst = 0; dst < size; ++dst)
    if (dst != rank) out_[dst] = Channel::create(region("c", rank, dst), slots, slot_bytes);
  thread_ = std::thread([this] { loop(); });
}

void Engine::connect() {
  if (connected_) return;
  const double deadline = now_s() + timeout_s_;
  auto retry = [&](auto&& attempt, const std::string& what) {
    for (;;) {
      try {
        if (attempt()) return;
      } catch (const std::system_error&) {
        // not there yet
      } catch (const std::runtime_error&) {
        // there, but its creator has not finished initialising it
      }
      if (now_s() > deadline) throw Timeout("timed out waiting for " + what + " to appear");
      std::this_thread::sleep_for(std::chrono::microseconds(500));
    }
  };
  for (int r = 0; r < size_; ++r) {
    if (r == rank_) continue;
    retry(
        [&] {
          SharedMemory s = SharedMemory::open(region("w", r));
          if (s.size() < sizeof(Window)) return false;
          auto* w = static_cast<Window*>(s.data());
          if (reinterpret_cast<std::atomic<std::uint64_t>*>(&w->magic)->load(std::memory_order_acquire) != kWindowMagic) return false;
          if (w->ranks != static_cast<std::uint32_t>(size_) || w->slots != slots_ || w->stride != stride_)
            throw std::invalid_argument("rank " + std::to_string(r) + " was started with a different group shape");
          windows_[r] = std::move(s);
          return true;
        },
        "rank " + std::to_string(r) + "'s window");
    retry(
        [&] {
          in_[r] = Channel::open(region("c", r, rank_));
          return true;
        },
        "the channel from rank " + std::to_string(r));
  }
  const std::atomic<std::uint32_t>* abort_word = &win(0)->abort_word;
  for (int r = 0; r < size_; ++r) {
    if (r == rank_) continue;
    out_[r].watch(abort_word);
    in_[r].watch(abort_word);
  }
  connected_ = true;
}

Engine::Window* Engine::win(int r) const { return static_cast<Window*>(windows_[r].data()); }

unsigned char* Engine::slot(int r, std::uint64_t round) const {
  return static_cast<unsigned char*>(windows_[r].data()) + sizeof(Window) + (round % slots_) * stride_;
}

void Engine::abort() {
  if (!connected_) return;
  std::uint32_t expected = 0;
  win(0)->abort_word.compare_exchange_strong(expected, static_cast<std::uint32_t>(rank_) + 1, std::memory_order_acq_rel);
  for (int r = 0; r < size_; ++r) {
    ring(win(r)->bell);
    out_[r].wake_all();
    in_[r].wake_all();
  }
}

void Engine::close() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (stopping_) return;
    stopping_ = true;
  }
  cv_.notify_all();
  if (thread_.joinable()) thread_.join();
  for (auto& c : out_) c = Channel();
  for (auto& c : in_) c = Channel();
  for (auto& w : windows_) w.drop();
}

Engine::~Engine() { close(); }

// ------------------------------------------------------------------ progress thread
std::shared_ptr<Work> Engine::submit(std::function<void()> job) {
  auto work = std::make_shared<Work>();
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (stopping_) throw std::runtime_error("the engine is closed");
    jobs_.emplace_back(std::move(job), work);
  }
  cv_.notify_one();
  return work;
}

void Engine::loop() {
  for (;;) {
    std::pair<std::function<void()>, std::shared_ptr<Work>> item;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait(lk, [&] { return stopping_ || !jobs_.empty(); });
      if (jobs_.empty()) return;  // stopping, and everything queued has run
      item = std::move(jobs_.front());
      jobs_.pop_front();
    }
    double t0 = now_s();
    std::exception_ptr err;
    try {
      item.first();
    } catch (...) {
      err = std::current_exception();
    }
    item.first = nullptr;  // drop captured state before the waiter wakes
    item.second->finish(err, t0, now_s());
  }
}

// ------------------------------------------------------------------ counters
void Engine::wait_count(int r, int which, std::uint64_t value, const char* what) {
  Window* w = win(r);
  auto reached = [&] { return w->count[which].v.load(std::memory_order_acquire) >= value; };
  if (reached()) return;  // the usual case for all but the first wait of a round: no label to build
  std::string label = std::string(what) + " (rank " + std::to_string(r) + ")";
  wait_for(reached, w->bell, timeout_s_, &win(0)->abort_word, label.c_str());
}

void Engine::publish(int which, std::uint64_t value) {
  Window* w = win(rank_);
  w->count[which].v.store(value, std::memory_order_release);
  ring(w->bell);
}

// Slot `round % slots` was last used in round `round - slots`; it may be
// overwritten once every peer has finished reading that round.
void Engine::claim_slot(std::uint64_t round) {
  if (round < slots_) return;
  for (int r = 0; r < size_; ++r)
    if (r != rank_) wait_count(r, CONSUMED, round - slots_ + 1, "a rank to finish reading a slot");
}

Engine::Sizes Engine::chunk_sizes(std::int64_t numel, const Sizes& sizes) const {
  if (sizes.empty()) {  // torch.tensor_split: the first numel % size chunks are one longer
    Sizes out(size_, numel / size_);
    for (std::int64_t c = 0; c < numel % size_; ++c) ++out[c];
    return out;
  }
  if (static_cast<int>(sizes.size()) != size_ || std::accumulate(sizes.begin(), sizes.end(), std::int64_t{0}) != numel ||
      std::any_of(sizes.begin(), sizes.end(), [](std::int64_t s) { return s < 0; }))
    throw std::invalid_argument("chunk sizes do not partition " + std::to_string(numel) + " elements");
  return sizes;
}

// ------------------------------------------------------------------ collectives
// Reduce-scatter (gather == false) or all-reduce (gather == true), in place.
void Engine::do_all_reduce(unsigned char* p, std::int64_t numel, DType d, bool average, const Sizes& sizes_in,
                           bool gather) {
  if (average && !dtype_is_float(d)) throw std::invalid_argument("avg needs a floating-point tensor");
  const Sizes sizes = chunk_sizes(numel, sizes_in);
  const std::int64_t esz = static_cast<std::int64_t>(dtype_size(d));
  const int n = size_, me = rank_;
  if (n == 1) {
    return;  // dividing by one changes nothing
  }
  Sizes off(n, 0);
  for (int c = 1; c < n; ++c) off[c] = off[c - 1] + sizes[c - 1];
  const std::int64_t per = std::max<std::int64_t>(1, static_cast<std::int64_t>(stride_) / esz / n);  // elements of each chunk per round
  const std::int64_t longest = *std::max_element(sizes.begin(), sizes.end());
  const std::int64_t rounds = ceil_div(longest, per);
  const int divisor = average ? n : 0;
  for (std::int64_t k = 0; k < rounds; ++k) {
    const std::uint64_t R = round_++;
    auto piece = [&](int c, std::int64_t* lo, std::int64_t* len) {
      *lo = std::min(sizes[c], k * per);
      *len = std::min(sizes[c], (k + 1) * per) - *lo;
    };
    claim_slot(R);
    unsigned char* mine = slot(me, R);
    for (int c = 0; c < n; ++c) {
      if (c == me) continue;  // nobody reads this rank's own chunk from its slot: it is folded in from `p` below
      std::int64_t lo, len;
      piece(c, &lo, &len);
      copy_in(mine + c * per * esz, p + (off[c] + lo) * esz, static_cast<std::size_t>(len), d, divisor);
    }
    publish(POSTED, R + 1);
    std::int64_t lo, len;
    piece(me, &lo, &len);
    for (int r = 0; r < n; ++r)
      if (r != me) wait_count(r, POSTED, R + 1, "a rank to post its operands");
    if (len > 0) {
      // Fold ranks me+1, me+2, ..., me: the association a ring reduce-scatter yields for chunk `me`.  The partial
      // sum of the peers' operands is built in this rank's own slot area for the chunk (free, see above); the last
      // addition takes this rank's operand straight from `p` (divided on the way when averaging) and writes the
      // result to `p` and, for an all-reduce, to the slot where the peers will fetch it -- one pass, no copies.
      unsigned char* acc = p + (off[me] + lo) * esz;
      const std::int64_t at = me * per * esz;
      const std::size_t count = static_cast<std::size_t>(len);
      const unsigned char* sum = slot((me + 1) % n, R) + at;
      if (n > 2) {
        add2(mine + at, sum, slot((me + 2) % n, R) + at, count, d);
        for (int j = 3; j < n; ++j) add_into(mine + at, slot((me + j) % n, R) + at, count, d);
        sum = mine + at;
      }
      add_own(acc, gather ? mine + at : nullptr, sum, count, d, divisor);
    }
    publish(REDUCED, R + 1);
    if (gather) {
      for (int j = 1; j < n; ++j) {
        int r = (me + j) % n;
        wait_count(r, REDUCED, R + 1, "a rank to reduce its chunk");
        piece(r, &lo, &len);
        if (len > 0) std::memcpy(p + (off[r] + lo) * esz, slot(r, R) + r * per * esz, static_cast<std::size_t>(len * esz));
      }
    }
    publish(CONSUMED, R + 1);
  }
}

void Engine::do_all_gather(unsigned char* p, std::int64_t numel, DType d, const Sizes& sizes_in) {
  const Sizes sizes = chunk_sizes(numel, sizes_in);
  const std::int64_t esz = static_cast<std::int64_t>(dtype_size(d));
  const int n = size_, me = rank_;
  if (n == 1) return;
  Sizes off(n, 0);
  for (int c = 1; c < n; ++c) off[c] = off[c - 1] + sizes[c - 1];
  const std::int64_t per = std::max<std::int64_t>(1, static_cast<std::int64_t>(stride_) / esz);
  const std::int64_t rounds = ceil_div(*std::max_element(sizes.begin(), sizes.end()), per);
  for (std::int64_t k = 0; k < rounds; ++k) {
    const std::uint64_t R = round_++;
    auto piece = [&](int c, std::int64_t* lo, std::int64_t* len) {
      *lo = std::min(sizes[c], k * per);
      *len = std::min(sizes[c], (k + 1) * per) - *lo;
    };
    std::int64_t lo, len;
    claim_slot(R);
    piece(me, &lo, &len);
    if (len > 0) std::memcpy(slot(me, R), p + (off[me] + lo) * esz, static_cast<std::size_t>(len * esz));
    publish(POSTED, R + 1);
    publish(REDUCED, R + 1);
    for (int j = 1; j < n; ++j) {
      int r = (me + j) % n;
      piece(r, &lo, &len);
      wait_count(r, POSTED, R + 1, "a rank to post its chunk");
      if (len > 0) std::memcpy(p + (off[r] + lo) * esz, slot(r, R), static_cast<std::size_t>(len * esz));
    }
    publish(CONSUMED, R + 1);
  }
}

void Engine::do_broadcast(unsigned char* p, std::int64_t numel, DType d, int root) {
  check_peer(root, "broadcast root");
  const int n = size_, me = rank_;
  if (n == 1) return;
  const std::int64_t total = numel * static_cast<std::int64_t>(dtype_size(d));
  const std::int64_t per = static_cast<std::int64_t>(stride_);
  for (std::int64_t lo = 0; lo < total; lo += per) {
    const std::uint64_t R = round_++;
    const std::size_t len = static_cast<std::size_t>(std::min(per, total - lo));
    if (me == root) {
      claim_slot(R);
      std::memcpy(slot(me, R), p + lo, len);
    }
    publish(POSTED, R + 1);
    publish(REDUCED, R + 1);
    if (me != root) {
      wait_count(root, POSTED, R + 1, "the root to post a piece");
      std::memcpy(p + lo, slot(root, R), len);
    }
    publish(CONSUMED, R + 1);
  }
}

void Engine::do_barrier() {
  if (size_ == 1) return;
  const std::uint64_t R = round_++;
  publish(POSTED, R + 1);
  publish(REDUCED, R + 1);
  for (int r = 0; r < size_; ++r)
    if (r != rank_) wait_count(r, POSTED, R + 1, "a rank to reach the barrier");
  publish(CONSUMED, R + 1);
}

// Sends and receives piece by piece in lockstep, so two ranks that exchange
// with each other never fill both rings and stall.
void Engine::do_exchange(const unsigned char* sp, std::int64_t sbytes, int dst, unsigned char* rp, std::int64_t rbytes,
                         int src) {
  const std::int64_t per = static_cast<std::int64_t>(slot_bytes_);
  std::int64_t so = 0, ro = 0;
  while (so < sbytes || ro < rbytes) {
    if (so < sbytes) {
      std::int64_t len = std::min(per, sbytes - so);
      out_[dst].send(sp + so, static_cast<std::size_t>(len), timeout_s_);
      so += len;
    }
    if (ro < rbytes) {
      std::int64_t want = std::min(per, rbytes - ro);
      const MessageView piece = in_[src].front(timeout_s_);
      if (static_cast<std::int64_t>(piece.size) != want) {
        throw std::runtime_error("out of step with rank " + std::to_string(src) + ": expected a piece of " +
                                 std::to_string(want) + " bytes, got " + std::to_string(piece.size));
      }
      std::memcpy(rp + ro, piece.data, piece.size);
      in_[src].pop();
      ro += want;
    }
  }
}

void Engine::check_peer(int r, const char* what) const {
  if (r < 0 || r >= size_) throw std::invalid_argument(std::string(what) + " " + std::to_string(r) + " is not a rank of this group");
}

// ------------------------------------------------------------------ public entry points
std::shared_ptr<Work> Engine::all_reduce(void* p, std::int64_t numel, DType d, bool average) {
  return submit([=] { do_all_reduce(static_cast<unsigned char*>(p), numel, d, average, {}, true); });
}

std::shared_ptr<Work> Engine::reduce_scatter(void* p, std::int64_t numel, DType d, Sizes sizes, bool average) {
  chunk_sizes(numel, sizes);  // reject a bad partition on the calling thread
  return submit([=] { do_all_reduce(static_cast<unsigned char*>(p), numel, d, average, sizes, false); });
}

std::shared_ptr<Work> Engine::all_gather(void* p, std::int64_t numel, DType d, Sizes sizes) {
  chunk_sizes(numel, sizes);
  return submit([=] { do_all_gather(static_cast<unsigned char*>(p), numel, d, sizes); });
}

std::shared_ptr<Work> Engine::broadcast(void* p, std::int64_t numel, DType d, int root) {
  check_peer(root, "broadcast root");
  return submit([=] { do_broadcast(static_cast<unsigned char*>(p), numel, d, root); });
}

std::shared_ptr<Work> Engine::send(const void* p, std::int64_t nbytes, int dst) {
  check_peer(dst, "destination");
  if (dst == rank_) throw std::invalid_argument("a rank cannot send to itself");
  return submit([=] { do_exchange(static_cast<const unsigned char*>(p), nbytes, dst, nullptr, 0, -1); });
}

std::shared_ptr<Work> Engine::recv(void* p, std::int64_t nbytes, int src) {
  check_peer(src, "source");
  if (src == rank_) throw std::invalid_argument("a rank cannot receive from itself");
  return submit([=] { do_exchange(nullptr, 0, -1, static_cast<unsigned char*>(p), nbytes, src); });
}

std::shared_ptr<Work> Engine::sendrecv(const void* sp, std::int64_t sbytes, int dst, void* rp, std::int64_t rbytes, int src) {
  check_peer(dst, "destination");
  check_peer(src, "source");
  if (dst == rank_ || src == rank_) throw std::invalid_argument("a rank cannot exchange with itself");
  return submit([=] {
    do_exchange(static_cast<const unsigned char*>(sp), sbytes, dst, static_cast<unsigned char*>(rp), rbytes, src);
  });
}

std::shared_ptr<Work> Engine::barrier() {
  return submit([=] { do_barrier(); });
}

}  // namespace tb
