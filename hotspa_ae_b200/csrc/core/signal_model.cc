#include "signal_model.h"

#include <atomic>
#include <chrono>
#include <memory>
#include <random>
#include <thread>
#include <vector>

namespace hsb {
namespace {

using Word = std::atomic<uint32_t>;
using Clock = std::chrono::steady_clock;

inline bool epoch_reached(uint32_t seen, uint32_t want) { return static_cast<int32_t>(seen - want) >= 0; }

struct Shared {
  std::atomic<long> checks{0}, violations{0}, timeouts{0};
  std::atomic<bool> abort{false};
  void check(bool ok) {
    checks.fetch_add(1, std::memory_order_relaxed);
    if (!ok) violations.fetch_add(1, std::memory_order_relaxed);
  }
  ModelResult result() const {
    ModelResult r;
    r.checks = checks.load(); r.violations = violations.load(); r.timeouts = timeouts.load();
    return r;
  }
};

// acquire-poll until *w reaches `want`; gives up after two seconds or when another rank gave up
bool wait_word(const Word& w, uint32_t want, Shared& sh, uint32_t* seen_out = nullptr) {
  const auto t0 = Clock::now();
  uint32_t it = 0;
  for (;;) {
    const uint32_t seen = w.load(std::memory_order_acquire);
    if (epoch_reached(seen, want)) { if (seen_out) *seen_out = seen; return true; }
    if (((++it) & 0xff) == 0) {
      if (sh.abort.load(std::memory_order_relaxed)) return false;
      if (Clock::now() - t0 > std::chrono::seconds(2)) {
        sh.timeouts.fetch_add(1);
        sh.abort.store(true);
        return false;
      }
      std::this_thread::yield();
    }
  }
}

struct Jitter {
  std::mt19937_64 rng;
  explicit Jitter(uint64_t seed) : rng(seed) {}
  void operator()() {
    const uint64_t r = rng() & 63;
    if (r < 8) std::this_thread::yield();
    else if (r < 12) std::this_thread::sleep_for(std::chrono::microseconds(20 + (rng() & 127)));
    else for (volatile uint64_t i = 0; i < (r << 2); ++i) {}
  }
};

std::unique_ptr<Word[]> words(size_t n) {
  std::unique_ptr<Word[]> w(new Word[n]);
  for (size_t i = 0; i < n; ++i) w[i].store(0, std::memory_order_relaxed);
  return w;
}

template <class F>
void run_ranks(int n, F&& body) {
  std::vector<std::thread> ts;
  for (int r = 0; r < n; ++r) ts.emplace_back(body, r);
  for (auto& t : ts) t.join();
}

inline uint32_t tag(uint32_t call, int src, int a, int b) {
  return (call + 1u) * 2654435761u ^ (static_cast<uint32_t>(src) << 24) ^ (static_cast<uint32_t>(a) << 12) ^
         static_cast<uint32_t>(b);
}

}  // namespace

ModelResult run_barrier_model(int n, int calls, uint32_t first_epoch, uint64_t seed) {
  Shared sh;
  auto pads = words(static_cast<size_t>(n) * n);           // pads[owner][writer]
  auto entered = words(n);                                 // barriers entered so far, per rank
  // the wrap-aware comparison is valid while a flag is within 2^31 of the awaited epoch: true from the first
  // barrier on when epochs start at 1 over zeroed pads; a later starting point is modelled as "the previous
  // barrier has happened"
  for (int i = 0; i < n * n; ++i) pads[i].store(first_epoch - 1u, std::memory_order_relaxed);
  run_ranks(n, [&](int r) {
    Jitter jit(seed * 1315423911ull + r);
    for (int k = 0; k < calls && !sh.abort.load(); ++k) {
      const uint32_t epoch = first_epoch + static_cast<uint32_t>(k);
      jit();
      entered[r].store(static_cast<uint32_t>(k + 1), std::memory_order_relaxed);
      for (int t = 0; t < n; ++t) { pads[static_cast<size_t>(t) * n + r].store(epoch, std::memory_order_release); jit(); }
      for (int t = 0; t < n; ++t) {
        if (!wait_word(pads[static_cast<size_t>(r) * n + t], epoch, sh)) return;
        sh.check(entered[t].load(std::memory_order_relaxed) >= static_cast<uint32_t>(k + 1));
      }
    }
  });
  return sh.result();
}

ModelResult run_reduce_scatter_model(int n, int calls, int counter_sets, int recv_buffers, int row_blocks,
                                     int parts, uint64_t seed) {
  Shared sh;
  const size_t per_set = static_cast<size_t>(n) * row_blocks;
  auto counters = words(static_cast<size_t>(n) * counter_sets * per_set);              // [owner][set][src][rb]
  const size_t per_buf = static_cast<size_t>(n) * row_blocks * parts;
  auto data = words(static_cast<size_t>(n) * recv_buffers * per_buf);                  // [owner][buf][src][rb][part]
  auto cnt = [&](int owner, int set, int src, int rb) -> Word& {
    return counters[(static_cast<size_t>(owner) * counter_sets + set) * per_set + static_cast<size_t>(src) * row_blocks + rb];
  };
  auto dat = [&](int owner, int buf, int src, int rb, int part) -> Word& {
    return data[(static_cast<size_t>(owner) * recv_buffers + buf) * per_buf +
                (static_cast<size_t>(src) * row_blocks + rb) * parts + part];
  };
  run_ranks(n, [&](int r) {
    Jitter jit(seed * 2246822519ull + r);
    for (int e = 0; e < calls && !sh.abort.load(); ++e) {
      const int set = e % counter_sets, zs = (e + 2) % counter_sets, buf = e % recv_buffers;
      // the set of the call after next starts at zero
      for (int s = 0; s < n; ++s)
        for (int rb = 0; rb < row_blocks; ++rb) cnt(r, zs, s, rb).store(0, std::memory_order_relaxed);
      jit();
      // deliver every tile part to its owner (the local ones are counted the same way), owners rotated
      for (int step = 1; step <= n; ++step) {
        const int owner = (r + step) % n;
        for (int rb = 0; rb < row_blocks; ++rb) {
          for (int p = 0; p < parts; ++p) {
            dat(owner, buf, r, rb, p).store(tag(e, r, rb, p), std::memory_order_relaxed);
            cnt(owner, set, r, rb).fetch_add(1, std::memory_order_release);
          }
          jit();
        }
      }
      // trailing reduce of the own shard
      for (int rb = 0; rb < row_blocks; ++rb) {
        for (int s = 0; s < n; ++s) {
          uint32_t seen = 0;
          if (!wait_word(cnt(r, set, s, rb), static_cast<uint32_t>(parts), sh, &seen)) return;
          sh.check(seen == static_cast<uint32_t>(parts));           // more than `parts`: counts of another call leaked in
          for (int p = 0; p < parts; ++p)
            sh.check(dat(r, buf, s, rb, p).load(std::memory_order_relaxed) == tag(e, s, rb, p));
        }
        jit();
      }
    }
  });
  return sh.result();
}

ModelResult run_all_gather_model(int n, int calls, int stage_buffers, int chunks, uint64_t seed) {
  Shared sh;
  auto stage = words(static_cast<size_t>(n) * stage_buffers * chunks);     // [rank][buf][chunk]
  auto ready = words(static_cast<size_t>(n) * n);                          // ready[consumer][producer]
  auto stg = [&](int rank, int buf, int c) -> Word& {
    return stage[(static_cast<size_t>(rank) * stage_buffers + buf) * chunks + c];
  };
  run_ranks(n, [&](int r) {
    Jitter jit(seed * 3266489917ull + r);
    for (int e = 0; e < calls && !sh.abort.load(); ++e) {
      const int buf = e % stage_buffers;
      const uint32_t epoch = static_cast<uint32_t>(e + 1);
      for (int c = 0; c < chunks; ++c) stg(r, buf, c).store(tag(e, r, c, 0), std::memory_order_relaxed);
      jit();
      for (int p = 0; p < n; ++p) ready[static_cast<size_t>(p) * n + r].store(epoch, std::memory_order_release);
      for (int step = 1; step < n; ++step) {
        const int p = (r + step) % n;
        if (!wait_word(ready[static_cast<size_t>(r) * n + p], epoch, sh)) return;
        for (int c = 0; c < chunks; ++c) {
          jit();
          sh.check(stg(p, buf, c).load(std::memory_order_relaxed) == tag(e, p, c, 0));
        }
      }
    }
  });
  return sh.result();
}

}  // namespace hsb
