// Closed-loop benchmark of a host KV engine: N threads issue batches of gets / puts on Zipf keys
// for a fixed wall time and report millions of key-values per second.
//
// Counterpart of the reference's engine benchmark (src/storage/kv_engine/benchmark_kv_engine.cc:
// 50-186: thread count, batch size, zipf theta, read ratio, Mkv/s) and of its generator check
// (benchmark_zipf.cc); here it is a library entry point so that the same loop drives every
// engine from Python and from the tests.
#include <atomic>
#include <chrono>
#include <thread>
#include <vector>

#include "common/rs_common.h"
#include "runtime/base.h"
#include "runtime/kv_engine.h"

namespace {
struct ThreadResult {
  uint64_t gets = 0, puts = 0, hits = 0, batches = 0;
  double max_batch_us = 0.0, sum_batch_us = 0.0;
};
}  // namespace

// out[0..7] = {get Mkv/s, put Mkv/s, hit ratio, batches/s, mean batch us, max batch us, seconds, threads}
RS_API int rs_kv_benchmark(void* handle, int threads, double seconds, int batch, double zipf_alpha, double read_ratio,
                           unsigned long long key_space, unsigned long long seed, double* out) {
  RS_REQUIRE(handle && out, "rs_kv_benchmark: null argument");
  RS_REQUIRE(threads > 0 && threads <= 256 && batch > 0 && seconds > 0 && key_space > 0, "rs_kv_benchmark: bad sizes");
  RS_REQUIRE(read_ratio >= 0.0 && read_ratio <= 1.0 && zipf_alpha >= 0.0, "rs_kv_benchmark: bad ratio / alpha");
  auto* kv = static_cast<rs::BaseKV*>(handle);
  const size_t vbytes = kv->value_size();
  std::vector<ThreadResult> res(threads);
  std::atomic<bool> go{false}, stop{false};
  std::atomic<int> ready{0};
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t) {
    pool.emplace_back([&, t] {
      rs::ZipfGenerator zipf(key_space, zipf_alpha, seed * 1315423911ull + static_cast<uint64_t>(t) * 2654435761ull + 1);
      std::vector<uint64_t> keys(batch);
      std::vector<uint8_t> found(batch);
      std::vector<char> vals(static_cast<size_t>(batch) * vbytes);
      float* vf = reinterpret_cast<float*>(vals.data());
      for (size_t i = 0; i < vals.size() / sizeof(float); ++i) vf[i] = static_cast<float>(t) + 0.5f;
      ThreadResult r;
      ready.fetch_add(1);
      while (!go.load(std::memory_order_acquire)) std::this_thread::yield();
      while (!stop.load(std::memory_order_relaxed)) {
        for (int i = 0; i < batch; ++i) keys[i] = zipf.next();
        const bool is_read = zipf.next_uniform() < read_ratio;
        const auto t0 = std::chrono::steady_clock::now();
        if (is_read) {
          kv->BatchGet(keys.data(), batch, vals.data(), found.data());
          for (int i = 0; i < batch; ++i) r.hits += found[i];
          r.gets += batch;
        } else {
          r.puts += kv->BatchPut(keys.data(), batch, vals.data());
        }
        const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
        r.sum_batch_us += us;
        if (us > r.max_batch_us) r.max_batch_us = us;
        ++r.batches;
      }
      res[t] = r;
    });
  }
  while (ready.load() < threads) std::this_thread::yield();
  const auto t0 = std::chrono::steady_clock::now();
  go.store(true, std::memory_order_release);
  std::this_thread::sleep_for(std::chrono::duration<double>(seconds));
  stop.store(true);
  for (auto& th : pool) th.join();
  const double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  ThreadResult tot;
  for (const auto& r : res) {
    tot.gets += r.gets; tot.puts += r.puts; tot.hits += r.hits; tot.batches += r.batches;
    tot.sum_batch_us += r.sum_batch_us;
    if (r.max_batch_us > tot.max_batch_us) tot.max_batch_us = r.max_batch_us;
  }
  out[0] = tot.gets / el / 1e6;
  out[1] = tot.puts / el / 1e6;
  out[2] = tot.gets ? static_cast<double>(tot.hits) / tot.gets : 0.0;
  out[3] = tot.batches / el;
  out[4] = tot.batches ? tot.sum_batch_us / tot.batches : 0.0;
  out[5] = tot.max_batch_us;
  out[6] = el;
  out[7] = threads;
  return RS_OK;
}

// Empirical mass of the `top` hottest ids in `n` draws: lets a caller check the generator against the analytic CDF.
RS_API int rs_zipf_check(unsigned long long key_space, double alpha, unsigned long long seed, long long n, long long top,
                         double* mass_out, double* draws_per_sec) {
  RS_REQUIRE(mass_out && n > 0 && top > 0 && key_space > 0, "rs_zipf_check: bad argument");
  rs::ZipfGenerator z(key_space, alpha, seed);
  long long hit = 0;
  const auto t0 = std::chrono::steady_clock::now();
  for (long long i = 0; i < n; ++i) hit += z.next() < static_cast<uint64_t>(top);
  const double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  *mass_out = static_cast<double>(hit) / static_cast<double>(n);
  if (draws_per_sec) *draws_per_sec = n / (el > 0 ? el : 1e-9);
  return RS_OK;
}
