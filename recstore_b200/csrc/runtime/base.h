// Small host-side building blocks of the runtime: spin locks (with an optional deadlock
// detector), a per-row bit-lock table, a sense-reversing thread barrier, a bounded SPSC queue,
// a ring of free indices with lock-free range pops, a bitmap, a thread pool, a bounded Zipf generator that also
// supports exponents >= 1, and a coarse clock refreshed by a background thread.
//
// They cover the roles of src/base/{lock.h:14-209, queue.h:19-189, lf_list.h, bitmap.h, zipf.h:78-175,
// async_time.h, bind_core.cc:14-70} of the reference without folly/glog.
#pragma once
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace rs {

inline void cpu_relax() {
#if defined(__x86_64__)
  __builtin_ia32_pause();
#else
  std::this_thread::yield();
#endif
}

// Test-and-test-and-set spin lock.  With detect_ms > 0, a waiter that spins longer than that
// reports a suspected deadlock through `on_stall` (once per wait) instead of hanging silently.
class SpinLock {
 public:
  void lock() {
    uint64_t spins = 0;
    auto t0 = std::chrono::steady_clock::time_point();
    while (true) {
      if (!flag_.exchange(true, std::memory_order_acquire)) return;
      while (flag_.load(std::memory_order_relaxed)) {
        cpu_relax();
        if (detect_ms_ > 0 && (++spins & 0xFFFF) == 0) {
          auto now = std::chrono::steady_clock::now();
          if (t0 == std::chrono::steady_clock::time_point()) t0 = now;
          else if (std::chrono::duration_cast<std::chrono::milliseconds>(now - t0).count() > detect_ms_) {
            stalls_.fetch_add(1, std::memory_order_relaxed);
            t0 = now;
          }
        }
      }
    }
  }
  bool try_lock() { return !flag_.exchange(true, std::memory_order_acquire); }
  void unlock() { flag_.store(false, std::memory_order_release); }
  bool is_locked() const { return flag_.load(std::memory_order_relaxed); }
  void set_deadlock_detect_ms(int ms) { detect_ms_ = ms; }
  uint64_t stalls() const { return stalls_.load(); }

 private:
  std::atomic<bool> flag_{false};
  int detect_ms_ = 0;
  std::atomic<uint64_t> stalls_{0};
};

struct PlaceboLock {
  void lock() {}
  void unlock() {}
};

// One lock bit per row: guards in-place row updates of a host table shared by several threads.
class BitLockTable {
 public:
  explicit BitLockTable(size_t n = 0) { resize(n); }
  void resize(size_t n) {
    n_ = n;
    words_ = std::unique_ptr<std::atomic<uint64_t>[]>(new std::atomic<uint64_t>[(n + 63) / 64]);
    for (size_t i = 0; i < (n + 63) / 64; ++i) words_[i].store(0);
  }
  void lock(size_t i) {
    std::atomic<uint64_t>& w = words_[i >> 6];
    const uint64_t m = 1ull << (i & 63);
    while (w.fetch_or(m, std::memory_order_acquire) & m) {
      while (w.load(std::memory_order_relaxed) & m) cpu_relax();
    }
  }
  void unlock(size_t i) { words_[i >> 6].fetch_and(~(1ull << (i & 63)), std::memory_order_release); }
  size_t size() const { return n_; }

 private:
  size_t n_ = 0;
  std::unique_ptr<std::atomic<uint64_t>[]> words_;
};

// Reusable barrier for the threads of one process (ranks impersonated by threads in tests).
class ThreadBarrier {
 public:
  explicit ThreadBarrier(int n) : n_(n) {}
  // Returns false on timeout (timeout_ms < 0 waits forever).
  bool wait(int timeout_ms = -1) {
    std::unique_lock<std::mutex> lk(mu_);
    const uint64_t gen = gen_;
    if (++count_ == n_) {
      count_ = 0;
      ++gen_;
      cv_.notify_all();
      return true;
    }
    if (timeout_ms < 0) {
      cv_.wait(lk, [&] { return gen_ != gen; });
      return true;
    }
    const bool ok = cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return gen_ != gen; });
    if (!ok) --count_;
    return ok;
  }

 private:
  int n_, count_ = 0;
  uint64_t gen_ = 0;
  std::mutex mu_;
  std::condition_variable cv_;
};

// Bounded single-producer single-consumer ring.
template <class T>
class SpscQueue {
 public:
  explicit SpscQueue(size_t capacity) : cap_(capacity + 1), buf_(capacity + 1) {}
  bool push(const T& v) {
    const size_t h = head_.load(std::memory_order_relaxed);
    const size_t n = (h + 1) % cap_;
    if (n == tail_.load(std::memory_order_acquire)) return false;
    buf_[h] = v;
    head_.store(n, std::memory_order_release);
    return true;
  }
  bool pop(T* out) {
    const size_t t = tail_.load(std::memory_order_relaxed);
    if (t == head_.load(std::memory_order_acquire)) return false;
    *out = buf_[t];
    tail_.store((t + 1) % cap_, std::memory_order_release);
    return true;
  }
  size_t size() const {
    const size_t h = head_.load(std::memory_order_acquire), t = tail_.load(std::memory_order_acquire);
    return (h + cap_ - t) % cap_;
  }
  bool empty() const { return size() == 0; }

 private:
  size_t cap_;
  std::vector<T> buf_;
  alignas(64) std::atomic<size_t> head_{0};
  alignas(64) std::atomic<size_t> tail_{0};
};

// Ring of free indices (slots, row numbers): producers append batches, any number of consumers claim runs of
// consecutive entries with one compare-and-swap.  Role of LFList (src/base/lf_list.h), with 64-bit positions that only
// grow (no ABA when the ring wraps), entries copied out before the claim is made (a successful claim proves that the
// producer has not touched them) and a refusal instead of an abort when a batch does not fit.
class IndexRing {
 public:
  explicit IndexRing(uint32_t capacity) : cap_(capacity ? capacity : 1), slots_(new std::atomic<int32_t>[cap_]) {}
  uint32_t Capacity() const { return cap_; }
  uint32_t Size() const {
    const uint64_t h = head_.load(std::memory_order_acquire);
    const uint64_t t = tail_.load(std::memory_order_acquire);
    return static_cast<uint32_t>(t > h ? t - h : 0);
  }
  // Appends n entries; false (nothing appended) when they do not fit.
  bool Push(const int32_t* v, uint32_t n) {
    std::lock_guard<SpinLock> lk(push_mu_);
    const uint64_t t = tail_.load(std::memory_order_relaxed);
    if (t - head_.load(std::memory_order_acquire) + n > cap_) return false;
    for (uint32_t i = 0; i < n; ++i) slots_[(t + i) % cap_].store(v[i], std::memory_order_relaxed);
    tail_.store(t + n, std::memory_order_release);
    return true;
  }
  // Takes up to `want` entries in ring order; returns how many were written to out (0: the ring is empty).
  uint32_t TryPop(int32_t* out, uint32_t want) {
    uint64_t h = head_.load(std::memory_order_acquire);
    while (true) {
      const uint64_t t = tail_.load(std::memory_order_acquire);
      const uint32_t n = static_cast<uint32_t>(std::min<uint64_t>(want, t > h ? t - h : 0));
      if (n == 0) return 0;
      for (uint32_t i = 0; i < n; ++i) out[i] = slots_[(h + i) % cap_].load(std::memory_order_relaxed);
      if (head_.compare_exchange_weak(h, h + n, std::memory_order_acq_rel, std::memory_order_acquire)) return n;
    }
  }
  void Clear() {
    std::lock_guard<SpinLock> lk(push_mu_);
    head_.store(tail_.load(std::memory_order_acquire), std::memory_order_release);
  }

 private:
  const uint32_t cap_;
  std::unique_ptr<std::atomic<int32_t>[]> slots_;
  SpinLock push_mu_;
  alignas(64) std::atomic<uint64_t> head_{0};
  alignas(64) std::atomic<uint64_t> tail_{0};
};

// A clock for hot paths that stamp many items and do not need better than a few milliseconds: one relaxed load of a
// value that a background thread refreshes every `interval_ms` (role of AsyncTimeHelper, src/base/async_time.h).  The
// process-wide instance starts on first use and is stopped when the library is unloaded.
class CoarseClock {
 public:
  explicit CoarseClock(int interval_ms);
  ~CoarseClock();
  uint64_t NowNs() const { return now_.load(std::memory_order_relaxed); }
  int interval_ms() const { return interval_ms_; }
  static CoarseClock& Global();       // 10 ms
  static uint64_t SteadyNs();         // the exact clock it samples

 private:
  void run();
  const int interval_ms_;
  std::atomic<uint64_t> now_;
  std::mutex mu_;
  std::condition_variable cv_;
  bool stop_ = false;
  std::thread thread_;
};

class Bitmap {
 public:
  explicit Bitmap(size_t n = 0) : n_(n), w_((n + 63) / 64, 0) {}
  void set(size_t i) { w_[i >> 6] |= 1ull << (i & 63); }
  void clear(size_t i) { w_[i >> 6] &= ~(1ull << (i & 63)); }
  bool test(size_t i) const { return (w_[i >> 6] >> (i & 63)) & 1; }
  size_t size() const { return n_; }
  size_t count() const {
    size_t c = 0;
    for (uint64_t x : w_) c += __builtin_popcountll(x);
    return c;
  }
  // first clear bit at or after `from`, or size() when none
  size_t find_clear(size_t from = 0) const {
    for (size_t i = from; i < n_; ++i)
      if (!test(i)) return i;
    return n_;
  }

 private:
  size_t n_;
  std::vector<uint64_t> w_;
};

// Fixed-size pool running `fn(begin, end)` over a partition of [0, n).
class ThreadPool {
 public:
  explicit ThreadPool(int n_threads);
  ~ThreadPool();
  void parallel_for(size_t n, const std::function<void(size_t, size_t, int)>& fn);
  int size() const { return static_cast<int>(workers_.size()) + 1; }
  static ThreadPool& global();

 private:
  void worker(int id);
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable cv_, done_cv_;
  const std::function<void(size_t, size_t, int)>* fn_ = nullptr;
  size_t n_ = 0;
  uint64_t gen_ = 0;
  int pending_ = 0;
  bool stop_ = false;
};

// Bounded Zipf-like generator on [0, n): inverse CDF of the continuous density x^-alpha on
// [1, n+1).  Valid for every alpha >= 0 (alpha == 1 handled separately).  Matches
// recstore_b200.utils.data.zipf_from_uniform bit for bit given the same uniforms.
class ZipfGenerator {
 public:
  ZipfGenerator(uint64_t n, double alpha, uint64_t seed) : n_(n), alpha_(alpha), s_(seed ? seed : 0x9E3779B97F4A7C15ull) {
    n1_ = static_cast<double>(n) + 1.0;
    if (std::fabs(alpha - 1.0) >= 1e-9) {
      e_ = 1.0 - alpha;
      c_ = std::pow(n1_, e_) - 1.0;
    }
  }
  uint64_t from_uniform(double u) const {
    double x;
    if (std::fabs(alpha_ - 1.0) < 1e-9) x = std::exp(u * std::log(n1_));
    else x = std::pow(u * c_ + 1.0, 1.0 / e_);
    long long k = static_cast<long long>(std::floor(x)) - 1;
    if (k < 0) k = 0;
    if (k >= static_cast<long long>(n_)) k = static_cast<long long>(n_) - 1;
    return static_cast<uint64_t>(k);
  }
  double next_uniform() {  // xorshift64*
    s_ ^= s_ >> 12; s_ ^= s_ << 25; s_ ^= s_ >> 27;
    const uint64_t r = s_ * 0x2545F4914F6CDD1Dull;
    return static_cast<double>(r >> 11) * (1.0 / 9007199254740992.0);
  }
  uint64_t next() { return from_uniform(next_uniform()); }

 private:
  uint64_t n_;
  double alpha_, n1_, e_ = 0, c_ = 0;
  uint64_t s_;
};

inline uint64_t hash64(uint64_t k) {
  k ^= k >> 33; k *= 0xff51afd7ed558ccdull; k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ull; k ^= k >> 33;
  return k;
}

// Pins the calling thread to `core` (no-op where unsupported).  Returns 0 on success.
int bind_core(int core);
// Cores of NUMA node `node` as reported by sysfs (empty when unknown).
std::vector<int> numa_node_cores(int node);

}  // namespace rs
