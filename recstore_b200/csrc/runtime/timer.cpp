// Named timers and counters with mean / P50 / P99 over a sliding sample window, an ASCII report
// and an optional background report thread.  Same role as xmh::Timer / PerfCounter / Reporter of
// the reference (src/base/timer.h:292-629) and its pybind module (src/base/pybind_timer.cc:9-22).
//
// Design: one registry keyed by name; each entry keeps a fixed ring of the most recent samples
// (sharded by thread to keep recording contention-free) plus cumulative count / sum.  Recording
// is wait-free on the hot path (atomic index increment into the thread's shard).
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "common/rs_common.h"

namespace {

constexpr int kShards = 16;
constexpr int kRing = 1024;

struct Series {
  std::string name;
  bool is_time;  // nanoseconds (timers) or plain values (counters)
  struct Shard {
    std::atomic<uint64_t> n{0};
    std::atomic<double> ring[kRing];   // written by recorders (threads may share a shard), read by the reporter: relaxed atomics
  };
  Shard shards[kShards];
  std::atomic<uint64_t> count{0};
  std::atomic<double> sum{0.0};
  std::atomic<double> last{0.0};

  void record(double v) {
    static thread_local int shard = static_cast<int>(std::hash<std::thread::id>()(std::this_thread::get_id()) % kShards);
    Shard& s = shards[shard];
    const uint64_t i = s.n.fetch_add(1, std::memory_order_relaxed);
    s.ring[i % kRing].store(v, std::memory_order_relaxed);
    count.fetch_add(1, std::memory_order_relaxed);
    double old = sum.load(std::memory_order_relaxed);
    while (!sum.compare_exchange_weak(old, old + v, std::memory_order_relaxed)) {}
    last.store(v, std::memory_order_relaxed);
  }
  void snapshot(std::vector<double>* out) const {
    out->clear();
    for (const Shard& s : shards) {
      const uint64_t n = std::min<uint64_t>(s.n.load(), kRing);
      for (uint64_t i = 0; i < n; ++i) out->push_back(s.ring[i].load(std::memory_order_relaxed));
    }
  }
};

struct Registry {
  std::mutex mu;
  std::map<std::string, std::unique_ptr<Series>> series;
  std::thread reporter;
  std::mutex rmu;
  std::condition_variable rcv;
  bool stop = false;
  bool running = false;

  Series* get(const char* name, bool is_time) {
    std::lock_guard<std::mutex> lk(mu);
    auto it = series.find(name);
    if (it == series.end()) {
      auto s = std::make_unique<Series>();
      s->name = name;
      s->is_time = is_time;
      it = series.emplace(name, std::move(s)).first;
    }
    return it->second.get();
  }

  std::string report() {
    std::vector<Series*> all;
    {
      std::lock_guard<std::mutex> lk(mu);
      for (auto& kv : series) all.push_back(kv.second.get());
    }
    std::string out;
    char line[256];
    snprintf(line, sizeof(line), "+%s+\n", std::string(94, '-').c_str());
    out += line;
    snprintf(line, sizeof(line), "| %-34s | %10s | %10s | %10s | %10s | %5s |\n", "name", "count", "mean", "P50", "P99", "unit");
    out += line;
    std::vector<double> v;
    for (Series* s : all) {
      s->snapshot(&v);
      double p50 = 0, p99 = 0;
      if (!v.empty()) {
        std::sort(v.begin(), v.end());
        p50 = v[v.size() / 2];
        p99 = v[std::min(v.size() - 1, static_cast<size_t>(v.size() * 0.99))];
      }
      const uint64_t c = s->count.load();
      double mean = c ? s->sum.load() / c : 0.0;
      const char* unit = "";
      if (s->is_time) {
        unit = "us";
        mean /= 1e3; p50 /= 1e3; p99 /= 1e3;
      }
      snprintf(line, sizeof(line), "| %-34.34s | %10llu | %10.3f | %10.3f | %10.3f | %5s |\n", s->name.c_str(),
               static_cast<unsigned long long>(c), mean, p50, p99, unit);
      out += line;
    }
    snprintf(line, sizeof(line), "+%s+\n", std::string(94, '-').c_str());
    out += line;
    return out;
  }
};

Registry& reg() {
  static Registry* r = new Registry();  // leaked on purpose: threads may record during exit
  return *r;
}

uint64_t now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

}  // namespace

RS_API unsigned long long rs_now_ns() { return now_ns(); }
RS_API void* rs_timer_get(const char* name) { return reg().get(name, true); }
RS_API void* rs_counter_get(const char* name) { return reg().get(name, false); }
RS_API void rs_series_record(void* series, double v) {
  if (series) static_cast<Series*>(series)->record(v);
}
RS_API void rs_timer_record_ns(const char* name, double ns) { reg().get(name, true)->record(ns); }
RS_API void rs_counter_record(const char* name, double v) { reg().get(name, false)->record(v); }

// mean, p50, p99, last, count of one series (times in nanoseconds); returns RS_ERR_NOTFOUND if unknown.
RS_API int rs_series_stats(const char* name, double* out5) {
  Registry& r = reg();
  Series* s = nullptr;
  {
    std::lock_guard<std::mutex> lk(r.mu);
    auto it = r.series.find(name);
    if (it != r.series.end()) s = it->second.get();
  }
  if (!s) return rs::set_error(RS_ERR_NOTFOUND, "no timer or counter named %s", name);
  std::vector<double> v;
  s->snapshot(&v);
  std::sort(v.begin(), v.end());
  const uint64_t c = s->count.load();
  out5[0] = c ? s->sum.load() / c : 0.0;
  out5[1] = v.empty() ? 0.0 : v[v.size() / 2];
  out5[2] = v.empty() ? 0.0 : v[std::min(v.size() - 1, static_cast<size_t>(v.size() * 0.99))];
  out5[3] = s->last.load();
  out5[4] = static_cast<double>(c);
  return RS_OK;
}

// Writes the report table into buf (truncated to cap-1 bytes); returns the full length.
RS_API int rs_report(char* buf, int cap) {
  const std::string s = reg().report();
  if (buf && cap > 0) {
    const int n = std::min<int>(cap - 1, static_cast<int>(s.size()));
    memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return static_cast<int>(s.size());
}

RS_API int rs_report_thread_start(int period_ms) {
  Registry& r = reg();
  std::lock_guard<std::mutex> lk(r.rmu);
  if (r.running) return RS_OK;
  r.stop = false;
  r.running = true;
  r.reporter = std::thread([&r, period_ms] {
    std::unique_lock<std::mutex> lk(r.rmu);
    while (!r.stop) {
      if (r.rcv.wait_for(lk, std::chrono::milliseconds(period_ms), [&] { return r.stop; })) break;
      lk.unlock();
      const std::string s = r.report();
      fputs(s.c_str(), stderr);
      lk.lock();
    }
  });
  return RS_OK;
}
RS_API int rs_report_thread_stop() {
  Registry& r = reg();
  {
    std::lock_guard<std::mutex> lk(r.rmu);
    if (!r.running) return RS_OK;
    r.stop = true;
  }
  r.rcv.notify_all();
  r.reporter.join();
  std::lock_guard<std::mutex> lk(r.rmu);
  r.running = false;
  return RS_OK;
}
// Resets every series to empty (handles returned by rs_timer_get stay valid).
RS_API void rs_timers_clear() {
  Registry& r = reg();
  std::lock_guard<std::mutex> lk(r.mu);
  for (auto& kv : r.series) {
    Series* s = kv.second.get();
    for (auto& sh : s->shards) sh.n.store(0);
    s->count.store(0);
    s->sum.store(0.0);
    s->last.store(0.0);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Histogram over the whole life of a measurement (the rings above only keep the latest samples).  Same role as the
// Histogram of the reference (src/base/timer.h:102-204: Add / Merge / Median / Percentile / ToString with bars), with
// computed bucket bounds instead of a table: bucket 0 is [0, 1), above that every power of two is cut into 8 equal
// parts, so a percentile is off by at most 1/16 of its value; 64 octaves cover 1 ... 1.8e19.
namespace {

class Histogram {
 public:
  static constexpr int kSub = 8, kOctaves = 64, kBuckets = 1 + kSub * kOctaves;
  void Clear() { *this = Histogram(); }
  void Add(double v) {
    if (!(v >= 0)) v = 0;                       // negative values and NaN count as zero
    ++buckets_[index_of(v)];
    min_ = std::min(min_, v);
    max_ = std::max(max_, v);
    ++num_;
    sum_ += v;
    sum_sq_ += v * v;
  }
  void Merge(const Histogram& o) {
    min_ = std::min(min_, o.min_);
    max_ = std::max(max_, o.max_);
    num_ += o.num_;
    sum_ += o.sum_;
    sum_sq_ += o.sum_sq_;
    for (int b = 0; b < kBuckets; ++b) buckets_[b] += o.buckets_[b];
  }
  uint64_t Count() const { return num_; }
  double Min() const { return num_ ? min_ : 0.0; }
  double Max() const { return max_; }
  double Average() const { return num_ ? sum_ / num_ : 0.0; }
  double StdDev() const {
    if (!num_) return 0.0;
    const double n = static_cast<double>(num_), var = (sum_sq_ * n - sum_ * sum_) / (n * n);
    return var > 0 ? std::sqrt(var) : 0.0;
  }
  // Linear interpolation inside the bucket that holds the p-th percentile, clamped to the observed range.
  double Percentile(double p) const {
    if (!num_) return 0.0;
    const double want = static_cast<double>(num_) * std::min(100.0, std::max(0.0, p)) / 100.0;
    double seen = 0;
    for (int b = 0; b < kBuckets; ++b) {
      if (!buckets_[b]) continue;
      const double next = seen + static_cast<double>(buckets_[b]);
      if (next >= want) {
        const double lo = lower(b), hi = upper(b);
        const double r = lo + (hi - lo) * (want - seen) / static_cast<double>(buckets_[b]);
        return std::min(max_, std::max(min_, r));
      }
      seen = next;
    }
    return max_;
  }
  std::string ToString() const {
    char buf[256];
    std::string r;
    snprintf(buf, sizeof buf, "Count: %llu  Average: %.4f  StdDev: %.2f\nMin: %.4f  Median: %.4f  P99: %.4f  Max: %.4f\n",
             static_cast<unsigned long long>(num_), Average(), StdDev(), Min(), Percentile(50), Percentile(99), Max());
    r += buf;
    if (!num_) return r;
    double cum = 0;
    for (int b = 0; b < kBuckets; ++b) {
      if (!buckets_[b]) continue;
      cum += static_cast<double>(buckets_[b]);
      snprintf(buf, sizeof buf, "[ %12.6g, %12.6g ) %10llu %7.3f%% %7.3f%% ", lower(b), upper(b),
               static_cast<unsigned long long>(buckets_[b]), 100.0 * buckets_[b] / num_, 100.0 * cum / num_);
      r += buf;
      r.append(static_cast<size_t>(20.0 * buckets_[b] / num_ + 0.5), '#');
      r += '\n';
    }
    return r;
  }

 private:
  static int index_of(double v) {
    if (v < 1.0) return 0;
    int e;
    const double m = std::frexp(v, &e);          // v = m * 2^e, m in [0.5, 1)
    const int oct = e - 1;                       // v in [2^oct, 2^(oct+1))
    if (oct >= kOctaves) return kBuckets - 1;
    return 1 + oct * kSub + std::min(kSub - 1, static_cast<int>((m * 2.0 - 1.0) * kSub));
  }
  static double lower(int b) {
    if (b == 0) return 0.0;
    const int oct = (b - 1) / kSub, sub = (b - 1) % kSub;
    return std::ldexp(1.0 + static_cast<double>(sub) / kSub, oct);
  }
  static double upper(int b) {
    if (b == 0) return 1.0;
    const int oct = (b - 1) / kSub, sub = (b - 1) % kSub;
    return std::ldexp(1.0 + static_cast<double>(sub + 1) / kSub, oct);
  }
  uint64_t buckets_[kBuckets] = {};
  uint64_t num_ = 0;
  double min_ = 1e300, max_ = 0, sum_ = 0, sum_sq_ = 0;
};

}  // namespace

RS_API void* rs_hist_new() { return new (std::nothrow) Histogram(); }
RS_API void rs_hist_delete(void* h) { delete static_cast<Histogram*>(h); }
RS_API void rs_hist_clear(void* h) { static_cast<Histogram*>(h)->Clear(); }
RS_API void rs_hist_add(void* h, double v) { static_cast<Histogram*>(h)->Add(v); }
RS_API void rs_hist_add_many(void* h, const double* v, long long n) {
  auto* hist = static_cast<Histogram*>(h);
  for (long long i = 0; i < n; ++i) hist->Add(v[i]);
}
RS_API void rs_hist_merge(void* h, const void* other) { static_cast<Histogram*>(h)->Merge(*static_cast<const Histogram*>(other)); }
RS_API double rs_hist_percentile(void* h, double p) { return static_cast<Histogram*>(h)->Percentile(p); }
// count, min, max, average, standard deviation
RS_API void rs_hist_summary(void* h, double* out5) {
  auto* hist = static_cast<Histogram*>(h);
  out5[0] = static_cast<double>(hist->Count());
  out5[1] = hist->Min();
  out5[2] = hist->Max();
  out5[3] = hist->Average();
  out5[4] = hist->StdDev();
}
RS_API int rs_hist_to_string(void* h, char* buf, int cap) {
  const std::string s = static_cast<Histogram*>(h)->ToString();
  if (buf && cap > 0) {
    const int n = std::min<int>(cap - 1, static_cast<int>(s.size()));
    memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return static_cast<int>(s.size());
}
