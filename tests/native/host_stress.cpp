// Stress program for the native host runtime, meant to be built with -fsanitize=thread or -fsanitize=address:
// every rank of a job runs as a THREAD of this one process (each with its own Engine, progress thread and mappings
// of the shared windows), so the sanitizers see the caller / progress-thread hand-offs, the Work objects and the
// channel rings.  Exits 0 when every result is right.
//
//   host_stress [ranks=4] [rounds=40]
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <unistd.h>
#include <vector>

#include "channel.h"
#include "engine.h"

using namespace tb;

static std::atomic<int> failures{0};

#define CHECK(cond, ...)                   \
  do {                                     \
    if (!(cond)) {                         \
      std::fprintf(stderr, __VA_ARGS__);   \
      std::fprintf(stderr, "\n");          \
      failures.fetch_add(1);               \
    }                                      \
  } while (0)

static void rank_main(const std::string& job, int rank, int n, int rounds) {
  Engine e(job, rank, n, 4, 1 << 16, 30.0);
  e.connect();
  for (int it = 0; it < rounds; ++it) {
    const std::int64_t numel = 1000 + 977 * it;  // crosses the slot size, uneven chunks
    std::vector<float> x(numel);
    for (std::int64_t i = 0; i < numel; ++i) x[i] = float((i % 13) + rank);
    auto w = e.all_reduce(x.data(), numel, DType::F32, false);
    // a second collective queued behind the first, waited for out of order
    std::vector<double> y(257, double(rank + 1));
    auto w2 = e.all_reduce(y.data(), (std::int64_t)y.size(), DType::F64, true);
    w2->wait();
    w->wait();
    const float add = float(n * (n - 1) / 2);
    for (std::int64_t i = 0; i < numel; i += 97) CHECK(x[i] == float(n * (i % 13)) + add, "all_reduce rank %d it %d i %lld", rank, it, (long long)i);
    CHECK(std::fabs(y[0] - (n + 1) / 2.0) < 1e-12, "avg rank %d it %d got %f", rank, it, y[0]);

    // all_gather with uneven sizes: rank r owns r + 1 + it elements
    Engine::Sizes sizes;
    std::int64_t total = 0;
    for (int r = 0; r < n; ++r) {
      sizes.push_back(r + 1 + it);
      total += r + 1 + it;
    }
    std::vector<std::int32_t> g(total, -1);
    std::int64_t off = 0;
    for (int r = 0; r < rank; ++r) off += sizes[r];
    for (std::int64_t i = 0; i < sizes[rank]; ++i) g[off + i] = rank * 1000 + (int)i;
    e.all_gather(g.data(), total, DType::I32, sizes)->wait();
    off = 0;
    for (int r = 0; r < n; ++r) {
      for (std::int64_t i = 0; i < sizes[r]; ++i) CHECK(g[off + i] == r * 1000 + (int)i, "all_gather rank %d it %d", rank, it);
      off += sizes[r];
    }

    // reduce_scatter: this rank's chunk holds the sum
    std::vector<float> rs(total);
    for (std::int64_t i = 0; i < total; ++i) rs[i] = float(i % 7) * float(rank + 1);
    e.reduce_scatter(rs.data(), total, DType::F32, sizes, false)->wait();
    off = 0;
    for (int r = 0; r < rank; ++r) off += sizes[r];
    const float tri = float(n * (n + 1) / 2);
    for (std::int64_t i = 0; i < sizes[rank]; ++i) CHECK(rs[off + i] == float((off + i) % 7) * tri, "reduce_scatter rank %d it %d", rank, it);

    // broadcast from a rotating root, ring sendrecv, barrier, and a user job on the progress thread
    std::vector<std::int64_t> b(300, rank);
    e.broadcast(b.data(), (std::int64_t)b.size(), DType::I64, it % n)->wait();
    CHECK(b[0] == it % n && b[299] == it % n, "broadcast rank %d it %d", rank, it);
    std::vector<char> out(5000 + it, char('a' + rank)), in(5000 + it, 0);
    e.sendrecv(out.data(), (std::int64_t)out.size(), (rank + 1) % n, in.data(), (std::int64_t)in.size(), (rank + n - 1) % n)->wait();
    CHECK(in[0] == char('a' + (rank + n - 1) % n) && in.back() == in[0], "sendrecv rank %d it %d", rank, it);
    int touched = 0;
    auto job_w = e.submit([&touched] { touched = 1; });
    e.barrier()->wait();
    job_w->wait();
    CHECK(touched == 1, "submit rank %d it %d", rank, it);
  }
  e.close();
}

static void channel_stress(const std::string& name, int messages) {
  Channel tx = Channel::create(name, 8, 256);
  Channel rx = Channel::open(name);
  std::thread producer([&] {
    std::vector<unsigned char> buf(256);
    for (int i = 0; i < messages; ++i) {
      const std::size_t len = 1 + (i * 7) % 255;
      std::memset(buf.data(), i & 0xff, len);
      tx.send(buf.data(), len, 30.0);
    }
  });
  std::vector<unsigned char> got(256);
  for (int i = 0; i < messages; ++i) {
    const std::size_t len = rx.recv(got.data(), got.size(), 30.0);
    CHECK(len == std::size_t(1 + (i * 7) % 255) && got[0] == (unsigned char)(i & 0xff) && got[len - 1] == got[0], "channel message %d", i);
  }
  producer.join();
}

int main(int argc, char** argv) {
  const int n = argc > 1 ? std::atoi(argv[1]) : 4;
  const int rounds = argc > 2 ? std::atoi(argv[2]) : 40;
  const std::string job = "stress" + std::to_string((long)getpid());
  channel_stress("/tb2-" + job + "-chan", 20000);
  std::vector<std::thread> ranks;
  for (int r = 0; r < n; ++r) ranks.emplace_back(rank_main, job, r, n, rounds);
  for (auto& t : ranks) t.join();
  if (failures.load() != 0) {
    std::fprintf(stderr, "%d checks failed\n", failures.load());
    return 1;
  }
  std::printf("host runtime stress: %d ranks x %d rounds ok\n", n, rounds);
  return 0;
}
