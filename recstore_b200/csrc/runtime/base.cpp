#include "runtime/base.h"

#include <fstream>
#include <sstream>
#include <sched.h>
#include <pthread.h>

#include "common/rs_common.h"

namespace rs {

ThreadPool::ThreadPool(int n_threads) {
  for (int i = 1; i < n_threads; ++i) workers_.emplace_back([this, i] { worker(i); });
}
ThreadPool::~ThreadPool() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    stop_ = true;
    ++gen_;
  }
  cv_.notify_all();
  for (auto& t : workers_) t.join();
}
void ThreadPool::worker(int id) {
  uint64_t seen = 0;
  while (true) {
    const std::function<void(size_t, size_t, int)>* fn;
    size_t n;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait(lk, [&] { return gen_ != seen; });
      seen = gen_;
      if (stop_) return;
      fn = fn_;
      n = n_;
    }
    const int parts = size();
    const size_t per = (n + parts - 1) / parts;
    const size_t b = std::min(n, per * id), e = std::min(n, b + per);
    if (b < e) (*fn)(b, e, id);
    {
      std::lock_guard<std::mutex> lk(mu_);
      if (--pending_ == 0) done_cv_.notify_all();
    }
  }
}
void ThreadPool::parallel_for(size_t n, const std::function<void(size_t, size_t, int)>& fn) {
  const int parts = size();
  if (parts == 1 || n < 2) {
    if (n) fn(0, n, 0);
    return;
  }
  {
    std::lock_guard<std::mutex> lk(mu_);
    fn_ = &fn;
    n_ = n;
    pending_ = parts - 1;
    ++gen_;
  }
  cv_.notify_all();
  const size_t per = (n + parts - 1) / parts;
  if (per) fn(0, std::min(n, per), 0);
  std::unique_lock<std::mutex> lk(mu_);
  done_cv_.wait(lk, [&] { return pending_ == 0; });
}
ThreadPool& ThreadPool::global() {
  static ThreadPool pool([] {
    unsigned n = std::thread::hardware_concurrency();
    if (n == 0) n = 4;
    if (n > 32) n = 32;
    return static_cast<int>(n);
  }());
  return pool;
}

int bind_core(int core) {
  cpu_set_t set;
  CPU_ZERO(&set);
  CPU_SET(core, &set);
  return pthread_setaffinity_np(pthread_self(), sizeof(set), &set);
}

std::vector<int> numa_node_cores(int node) {
  std::vector<int> out;
  std::ifstream f("/sys/devices/system/node/node" + std::to_string(node) + "/cpulist");
  std::string s;
  if (!f || !std::getline(f, s)) return out;
  std::stringstream ss(s);
  std::string tok;
  while (std::getline(ss, tok, ',')) {
    const size_t dash = tok.find('-');
    if (dash == std::string::npos) out.push_back(std::stoi(tok));
    else
      for (int c = std::stoi(tok.substr(0, dash)); c <= std::stoi(tok.substr(dash + 1)); ++c) out.push_back(c);
  }
  return out;
}

uint64_t CoarseClock::SteadyNs() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
CoarseClock::CoarseClock(int interval_ms) : interval_ms_(interval_ms < 1 ? 1 : interval_ms), now_(SteadyNs()) {
  thread_ = std::thread([this] { run(); });
}
CoarseClock::~CoarseClock() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (thread_.joinable()) thread_.join();
}
void CoarseClock::run() {
  std::unique_lock<std::mutex> lk(mu_);
  while (!stop_) {
    now_.store(SteadyNs(), std::memory_order_relaxed);
    cv_.wait_for(lk, std::chrono::milliseconds(interval_ms_), [this] { return stop_; });
  }
}
CoarseClock& CoarseClock::Global() {
  static CoarseClock clock(10);
  return clock;
}

}  // namespace rs

// ---------------------------------------------------------------- C ABI
RS_API unsigned long long rs_coarse_now_ns() { return rs::CoarseClock::Global().NowNs(); }
RS_API unsigned long long rs_steady_now_ns() { return rs::CoarseClock::SteadyNs(); }

RS_API int rs_ring_new(unsigned capacity, void** out) {
  RS_REQUIRE(out && capacity > 0, "rs_ring_new: bad argument");
  RS_NOEXCEPT_BODY(*out = new rs::IndexRing(capacity); return RS_OK;)
}
RS_API int rs_ring_delete(void* h) {
  delete static_cast<rs::IndexRing*>(h);
  return RS_OK;
}
// 1: appended, 0: the batch does not fit (nothing appended).
RS_API int rs_ring_push(void* h, const int* v, unsigned n) { return static_cast<rs::IndexRing*>(h)->Push(v, n) ? 1 : 0; }
RS_API unsigned rs_ring_pop(void* h, int* out, unsigned want) { return static_cast<rs::IndexRing*>(h)->TryPop(out, want); }
RS_API unsigned rs_ring_size(void* h) { return static_cast<rs::IndexRing*>(h)->Size(); }
RS_API void rs_ring_clear(void* h) { static_cast<rs::IndexRing*>(h)->Clear(); }

RS_API int rs_bind_core(int core) { return rs::bind_core(core) == 0 ? RS_OK : rs::set_error(RS_ERR_INVALID, "cannot bind to core %d", core); }

RS_API int rs_numa_node_cores(int node, int* out, int cap) {
  auto v = rs::numa_node_cores(node);
  int n = 0;
  for (int c : v)
    if (n < cap) out[n++] = c;
  return static_cast<int>(v.size());
}

// Fills out[0..n) with ids in [0, n_rows) (or [1, n_rows] when one_based), Zipf exponent alpha.
RS_API int rs_zipf_fill(long long* out, long long n, unsigned long long n_rows, double alpha, unsigned long long seed,
                        int one_based) {
  RS_REQUIRE(out && n >= 0 && n_rows > 0 && alpha >= 0, "rs_zipf_fill: bad argument");
  rs::ZipfGenerator g(n_rows, alpha, seed);
  for (long long i = 0; i < n; ++i) out[i] = static_cast<long long>(g.next()) + (one_based ? 1 : 0);
  return RS_OK;
}
// Same mapping applied to caller-provided uniforms (bit-for-bit comparable with the Python generator).
RS_API int rs_zipf_from_uniform(const double* u, long long* out, long long n, unsigned long long n_rows, double alpha) {
  RS_REQUIRE(u && out && n_rows > 0, "rs_zipf_from_uniform: bad argument");
  rs::ZipfGenerator g(n_rows, alpha, 1);
  for (long long i = 0; i < n; ++i) out[i] = static_cast<long long>(g.from_uniform(u[i]));
  return RS_OK;
}

RS_API void rs_mfence() { std::atomic_thread_fence(std::memory_order_seq_cst); }
RS_API void rs_lfence() { std::atomic_thread_fence(std::memory_order_acquire); }
RS_API void rs_sfence() { std::atomic_thread_fence(std::memory_order_release); }
