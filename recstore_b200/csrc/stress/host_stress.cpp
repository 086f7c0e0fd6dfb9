// Multi-threaded stress driver of the host runtime, meant to be built with -fsanitize=thread (or address) and run
// without Python: every component that owns threads or is called from several threads is driven through its C entry
// points, with the same invariants the Python tests check.
//
//   1. KV engines: N threads of mixed batch gets / puts on Zipf keys (rs_kv_benchmark), then the engine's own
//      consistency check.
//   2. Parameter server: a loopback server and several client threads putting, getting and updating overlapping keys.
//   3. Allocators (pool / binning / fixed length on pageable host memory), the timer registry with its report thread,
//      and the shared-memory barrier, each hit from several threads.
//   3b. The ring of free indices (producers against consumers that claim runs) and the coarse clock.
//   4. Lookahead controller: "ranks" as threads sharing one controller (the layout of the reference's
//      VirtualEnvironment test, src/framework_test), background flush threads on, the read-your-updates contract
//      checked at every step against a synchronous oracle.
//
// Exit code 0 and a final "host_stress: ok" line mean that no invariant broke; a sanitizer report makes the process
// exit non-zero by itself (TSAN_OPTIONS=halt_on_error=1 exitcode=66 is set by the test that runs it).
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <unistd.h>

extern "C" {
int rs_kv_create(const char* engine, const char* json_config, void** out);
int rs_kv_destroy(void* h);
int rs_kv_check_consistency(void* h, int* ok);
int rs_kv_put(void* h, unsigned long long key, const void* value);
int rs_kv_get(void* h, unsigned long long key, void* out, int* found);
int rs_kv_erase(void* h, unsigned long long key, int* erased);
unsigned long long rs_kv_size(void* h);
int rs_kv_benchmark(void* handle, int threads, double seconds, int batch, double zipf_alpha, double read_ratio,
                    unsigned long long key_space, unsigned long long seed, double* out);
int rs_ps_create(const char* engine, const char* json, void** out);
int rs_ps_destroy(void* ps);
int rs_ps_server_start(void* ps, int port, void** server_out, int* port_out);
int rs_ps_server_stop(void* server);
int rs_ps_server_monitor_start(void* server, int period_ms, int print);
unsigned long long rs_ps_server_monitor_last(void* server, double* out3);
int rs_ps_client_connect(const char* host, int port, void** out);
int rs_ps_client_close(void* c);
int rs_ps_client_get(void* c, const unsigned long long* keys, long long n, int dim, float* out, unsigned char* found, int max_per_req);
int rs_ps_client_put(void* c, const unsigned long long* keys, long long n, int dim, const float* values, int max_per_req);
int rs_ctrl_create(const char* json, void** out);
int rs_ctrl_destroy(void* c);
int rs_ctrl_register_table(void* c, float* table, long long rows);
int rs_ctrl_register_cache(void* c, int rank, float* cache);
int rs_ctrl_start(void* c);
int rs_ctrl_stop(void* c);
int rs_ctrl_drain(void* c);
int rs_ctrl_publish_reads(void* c, int rank, long long step, const long long* ids, long long n);
int rs_ctrl_set_step_input(void* c, int rank, const long long* keys, long long n, const float* grads);
int rs_ctrl_process_one_step(void* c, long long step);
int rs_ctrl_block_to_step(void* c, long long step, int timeout_ms);
long long rs_ctrl_pending(void* c);
int rs_devpool_create(int kind, int backing, size_t initial_bytes, size_t max_bytes, size_t param, void** out);
int rs_devpool_destroy(void* h);
int rs_devpool_alloc(void* h, size_t bytes, void** out);
int rs_devpool_free(void* h, void* p);
int rs_devpool_stats(void* h, unsigned long long* out6);
void rs_timer_record_ns(const char* name, double ns);
void rs_counter_record(const char* name, double v);
int rs_series_stats(const char* name, double* out5);
int rs_report_thread_start(int period_ms);
int rs_report_thread_stop();
void rs_timers_clear();
int rs_ring_new(unsigned capacity, void** out);
int rs_ring_delete(void* h);
int rs_ring_push(void* h, const int* v, unsigned n);
unsigned rs_ring_pop(void* h, int* out, unsigned want);
unsigned rs_ring_size(void* h);
unsigned long long rs_coarse_now_ns();
unsigned long long rs_steady_now_ns();
int rs_shm_set_namespace(const char* ns);
int rs_barrier_create(const char* name, int parties, void** out_handle);
int rs_barrier_wait(void* handle, int timeout_ms);
int rs_barrier_close(void* handle);
int rs_barrier_unlink(const char* name);
const char* rs_last_error();
}

namespace {

int g_failures = 0;
std::mutex g_fail_mu;

void fail(const char* what, const std::string& detail = "") {
  std::lock_guard<std::mutex> l(g_fail_mu);
  ++g_failures;
  std::fprintf(stderr, "host_stress: FAIL %s %s (%s)\n", what, detail.c_str(), rs_last_error());
}
#define EXPECT_OK(call) do { if ((call) != 0) fail(#call); } while (0)

// Reusable barrier for the rank threads (std::barrier is C++20).
class Barrier {
 public:
  explicit Barrier(int n) : n_(n) {}
  void wait() {
    std::unique_lock<std::mutex> l(mu_);
    const long gen = gen_;
    if (++count_ == n_) { count_ = 0; ++gen_; cv_.notify_all(); return; }
    cv_.wait(l, [&] { return gen_ != gen; });
  }
 private:
  std::mutex mu_;
  std::condition_variable cv_;
  int n_, count_ = 0;
  long gen_ = 0;
};

struct Lcg {
  unsigned long long s;
  explicit Lcg(unsigned long long seed) : s(seed * 6364136223846793005ull + 1442695040888963407ull) {}
  unsigned long long next() { s = s * 6364136223846793005ull + 1442695040888963407ull; return s >> 17; }
};

void stress_kv(const char* engine, const char* json) {
  void* kv = nullptr;
  if (rs_kv_create(engine, json, &kv) != 0) { fail("rs_kv_create", engine); return; }
  double out[8];
  EXPECT_OK(rs_kv_benchmark(kv, 6, 0.3, 64, 0.99, 0.5, 20000, 7, out));
  // put / get / erase cycles: every thread owns the keys congruent to its index, so each read-back is exact while the
  // threads still collide in the engine's buckets, segments and locks
  {
    constexpr int kThreads = 6, kRounds = 3000;
    std::atomic<int> bad{0};
    std::vector<std::thread> ts;
    for (int t = 0; t < kThreads; ++t) {
      ts.emplace_back([&, t] {
        Lcg rng(900 + t);
        float val[8], got[8];
        for (int r = 0; r < kRounds; ++r) {
          const unsigned long long key = 5000000ull + (rng.next() % 4096) * kThreads + t;
          for (int d = 0; d < 8; ++d) val[d] = static_cast<float>(key % 1000 + d + r);
          int found = 0, erased = 0;
          if (rs_kv_put(kv, key, val) != 0) { bad.fetch_add(1); continue; }
          if (rs_kv_get(kv, key, got, &found) != 0 || !found || std::memcmp(got, val, sizeof(val)) != 0) bad.fetch_add(1);
          if ((r & 3) == 0) {
            if (rs_kv_erase(kv, key, &erased) != 0 || !erased) bad.fetch_add(1);
            if (rs_kv_get(kv, key, got, &found) != 0 || found) bad.fetch_add(1);
          }
        }
      });
    }
    for (auto& t : ts) t.join();
    if (bad.load() != 0) fail("kv put/get/erase cycles", std::string(engine) + ": " + std::to_string(bad.load()) + " wrong answers");
  }
  int ok = 1;
  if (rs_kv_check_consistency(kv, &ok) == 0 && !ok) fail("kv consistency", engine);   // non-zero: the engine has no checker
  std::printf("host_stress: kv %-12s get %.2f Mkv/s put %.2f Mkv/s size %llu\n", engine, out[0], out[1], rs_kv_size(kv));
  EXPECT_OK(rs_kv_destroy(kv));
}

// Writers replace the values of a small key set out of place as fast as they can while readers copy them: in a tight
// pool every superseded record is recycled within microseconds, so a reader that were handed a record too early would
// copy a mix of two versions (and ThreadSanitizer would see the two memcpy collide).
void stress_shared_keys(const char* engine, const char* json, int kDim) {
  constexpr int kKeys = 64, kWriters = 2, kReaders = 3;
  void* kv = nullptr;
  if (rs_kv_create(engine, json, &kv) != 0) { fail("rs_kv_create", engine); return; }
  const std::vector<float> zero(kDim, 0.f);
  for (int k = 0; k < kKeys; ++k) EXPECT_OK(rs_kv_put(kv, 1000 + k, zero.data()));
  std::atomic<bool> stop{false};
  std::atomic<int> torn{0}, missing{0}, refused{0};
  std::atomic<unsigned long long> reads{0}, writes{0};
  std::vector<std::thread> ts;
  for (int w = 0; w < kWriters; ++w)
    ts.emplace_back([&, w] {
      Lcg rng(50 + w);
      std::vector<float> val(kDim);
      unsigned version = 1;
      while (!stop.load(std::memory_order_relaxed)) {
        for (int d = 0; d < kDim; ++d) val[d] = static_cast<float>(w * 1000000 + version);
        ++version;
        if (rs_kv_put(kv, 1000 + rng.next() % kKeys, val.data()) != 0) refused.fetch_add(1);
        writes.fetch_add(1, std::memory_order_relaxed);
      }
    });
  for (int r = 0; r < kReaders; ++r)
    ts.emplace_back([&, r] {
      Lcg rng(70 + r);
      std::vector<float> got(kDim);
      while (!stop.load(std::memory_order_relaxed)) {
        int found = 0;
        if (rs_kv_get(kv, 1000 + rng.next() % kKeys, got.data(), &found) != 0 || !found) { missing.fetch_add(1); continue; }
        for (int d = 1; d < kDim; ++d)
          if (got[d] != got[0]) { torn.fetch_add(1); break; }
        reads.fetch_add(1, std::memory_order_relaxed);
      }
    });
  std::this_thread::sleep_for(std::chrono::milliseconds(400));
  stop.store(true);
  for (auto& t : ts) t.join();
  if (torn.load()) fail("a reader copied a mix of two versions", std::string(engine) + ": " + std::to_string(torn.load()));
  if (missing.load()) fail("a key that is only ever replaced was reported absent", engine);
  if (refused.load()) fail("a replacement was refused although the key set never grows", engine);
  std::printf("host_stress: kv %-12s shared keys: %llu reads, %llu writes\n", engine, reads.load(), writes.load());
  EXPECT_OK(rs_kv_destroy(kv));
}

void stress_ps() {
  constexpr int kDim = 8, kClients = 4, kRounds = 60, kKeys = 48;
  void* ps = nullptr;
  void* server = nullptr;
  int port = 0;
  if (rs_ps_create("KVEngineMap", "{\"capacity\": 65536, \"dim\": 8}", &ps) != 0) { fail("rs_ps_create"); return; }
  if (rs_ps_server_start(ps, 0, &server, &port) != 0) { fail("rs_ps_server_start"); rs_ps_destroy(ps); return; }
  EXPECT_OK(rs_ps_server_monitor_start(server, 5, 0));        // the monitor reads the counters the connection threads bump
  std::vector<std::thread> ts;
  for (int c = 0; c < kClients; ++c) {
    ts.emplace_back([&, c] {
      void* cl = nullptr;
      if (rs_ps_client_connect("127.0.0.1", port, &cl) != 0) { fail("rs_ps_client_connect"); return; }
      Lcg rng(100 + c);
      std::vector<unsigned long long> keys(kKeys);
      std::vector<float> vals(kKeys * kDim), got(kKeys * kDim);
      std::vector<unsigned char> found(kKeys);
      for (int r = 0; r < kRounds; ++r) {
        // own keys (exact read-back) interleaved with keys every client writes (same value from everybody)
        for (int i = 0; i < kKeys; ++i) {
          const bool shared = (i & 1) != 0;
          keys[i] = shared ? 1000000ull + rng.next() % 64 : static_cast<unsigned long long>(c) * 10000 + rng.next() % 512;
          for (int d = 0; d < kDim; ++d) vals[i * kDim + d] = shared ? static_cast<float>(keys[i] % 97) : static_cast<float>(keys[i] + d);
        }
        EXPECT_OK(rs_ps_client_put(cl, keys.data(), kKeys, kDim, vals.data(), 16));
        EXPECT_OK(rs_ps_client_get(cl, keys.data(), kKeys, kDim, got.data(), found.data(), 16));
        for (int i = 0; i < kKeys; ++i) {
          if (!found[i] || std::memcmp(&got[i * kDim], &vals[i * kDim], kDim * sizeof(float)) != 0) {
            fail("ps read-back", "client " + std::to_string(c) + " round " + std::to_string(r));
            break;
          }
        }
      }
      EXPECT_OK(rs_ps_client_close(cl));
    });
  }
  for (auto& t : ts) t.join();
  double mon[3];
  if (rs_ps_server_monitor_last(server, mon) == 0) fail("the throughput monitor never measured a period");
  EXPECT_OK(rs_ps_server_stop(server));                        // stops the monitor too
  EXPECT_OK(rs_ps_destroy(ps));
  std::printf("host_stress: ps %d clients x %d rounds\n", kClients, kRounds);
}

// Every thread allocates blocks of random sizes, fills each with its own tag, checks the tags before freeing: an
// allocator that hands one byte to two owners, or corrupts its free lists under contention, shows up as a wrong tag.
void stress_allocator(int kind, const char* name) {
  constexpr int kThreads = 6, kRounds = 400, kLive = 24;
  void* pool = nullptr;
  if (rs_devpool_create(kind, 2, size_t{1} << 20, size_t{256} << 20, kind == 2 ? 4096 : (size_t{1} << 16), &pool) != 0) {
    fail("rs_devpool_create", name);
    return;
  }
  std::atomic<int> bad{0};
  std::vector<std::thread> ts;
  for (int t = 0; t < kThreads; ++t) {
    ts.emplace_back([&, t] {
      Lcg rng(500 + t);
      struct Block { unsigned char* p; size_t n; unsigned char tag; };
      std::vector<Block> live;
      for (int r = 0; r < kRounds; ++r) {
        if (live.size() < static_cast<size_t>(kLive) && (rng.next() & 3) != 0) {
          const size_t n = kind == 2 ? 4096 : 16 + rng.next() % 30000;
          void* p = nullptr;
          if (rs_devpool_alloc(pool, n, &p) != 0 || p == nullptr) { bad.fetch_add(1); continue; }
          const unsigned char tag = static_cast<unsigned char>(1 + (t * 37 + r) % 250);
          std::memset(p, tag, n);
          live.push_back({static_cast<unsigned char*>(p), n, tag});
        } else if (!live.empty()) {
          const size_t i = rng.next() % live.size();
          const Block b = live[i];
          if (b.p[0] != b.tag || b.p[b.n / 2] != b.tag || b.p[b.n - 1] != b.tag) bad.fetch_add(1);
          if (rs_devpool_free(pool, b.p) != 0) bad.fetch_add(1);
          live[i] = live.back();
          live.pop_back();
        }
      }
      for (const Block& b : live) {
        if (b.p[0] != b.tag || b.p[b.n - 1] != b.tag) bad.fetch_add(1);
        if (rs_devpool_free(pool, b.p) != 0) bad.fetch_add(1);
      }
    });
  }
  for (auto& t : ts) t.join();
  unsigned long long st[6] = {0, 0, 0, 0, 0, 0};
  EXPECT_OK(rs_devpool_stats(pool, st));
  if (bad.load() != 0) fail("allocator blocks", std::string(name) + ": " + std::to_string(bad.load()) + " bad blocks");
  EXPECT_OK(rs_devpool_destroy(pool));
  std::printf("host_stress: allocator %s, %d threads x %d rounds\n", name, kThreads, kRounds);
}

void stress_timers_and_barrier() {
  constexpr int kThreads = 4, kRounds = 200;
  rs_timers_clear();
  EXPECT_OK(rs_report_thread_start(5));
  char ns[64];
  std::snprintf(ns, sizeof(ns), "rs_stress_%d", static_cast<int>(getpid()));       // several drivers may run at once
  EXPECT_OK(rs_shm_set_namespace(ns));
  std::vector<void*> handles(kThreads, nullptr);
  for (int t = 0; t < kThreads; ++t) EXPECT_OK(rs_barrier_create("stress_barrier", kThreads, &handles[t]));
  std::atomic<int> arrived{0}, out_of_step{0};
  std::vector<std::thread> ts;
  for (int t = 0; t < kThreads; ++t) {
    ts.emplace_back([&, t] {
      for (int r = 0; r < kRounds; ++r) {
        rs_timer_record_ns("stress.timer", 100.0 + r);
        rs_counter_record(t & 1 ? "stress.odd" : "stress.even", 1.0);
        arrived.fetch_add(1);
        if (rs_barrier_wait(handles[t], 20000) != 0) { fail("rs_barrier_wait"); return; }
        if (arrived.load() < (r + 1) * kThreads) out_of_step.fetch_add(1);     // nobody leaves before everybody arrived
      }
    });
  }
  for (auto& t : ts) t.join();
  EXPECT_OK(rs_report_thread_stop());
  double st[5] = {0, 0, 0, 0, 0};
  EXPECT_OK(rs_series_stats("stress.timer", st));
  if (out_of_step.load() != 0) fail("barrier released early");
  for (int t = 0; t < kThreads; ++t) EXPECT_OK(rs_barrier_close(handles[t]));
  EXPECT_OK(rs_barrier_unlink("stress_barrier"));
  std::printf("host_stress: timers + barrier, %d threads x %d rounds\n", kThreads, kRounds);
}

// Two producers append batches of distinct numbers to a small ring while four consumers claim runs of them: every
// number must come out exactly once, whatever the interleaving and however often the ring wraps.
void stress_index_ring() {
  constexpr int kProducers = 2, kConsumers = 4, kPerProducer = 60000, kCap = 257;
  void* ring = nullptr;
  EXPECT_OK(rs_ring_new(kCap, &ring));
  std::vector<std::atomic<unsigned char>> seen(kProducers * kPerProducer);
  for (auto& s : seen) s.store(0);
  std::atomic<int> taken{0}, producers_left{kProducers}, dup{0};
  std::vector<std::thread> ts;
  for (int p = 0; p < kProducers; ++p)
    ts.emplace_back([&, p] {
      int next = p * kPerProducer;
      const int end = next + kPerProducer;
      int batch[7];
      while (next < end) {
        const int n = std::min(1 + next % 7, end - next);
        for (int i = 0; i < n; ++i) batch[i] = next + i;
        if (rs_ring_push(ring, batch, static_cast<unsigned>(n))) next += n;
        else std::this_thread::yield();
      }
      producers_left.fetch_sub(1);
    });
  for (int c = 0; c < kConsumers; ++c)
    ts.emplace_back([&, c] {
      int got[16];
      while (true) {
        const unsigned n = rs_ring_pop(ring, got, 1 + (c * 5) % 16);
        for (unsigned i = 0; i < n; ++i)
          if (seen[got[i]].fetch_add(1) != 0) dup.fetch_add(1);
        taken.fetch_add(static_cast<int>(n));
        if (n == 0) {
          if (producers_left.load() == 0 && rs_ring_size(ring) == 0) break;
          std::this_thread::yield();
        }
      }
    });
  for (auto& t : ts) t.join();
  if (taken.load() != kProducers * kPerProducer) fail("index ring lost or invented entries");
  if (dup.load() != 0) fail("index ring handed an entry out twice");
  EXPECT_OK(rs_ring_delete(ring));
  // the coarse clock trails the exact one by about its refresh interval, never leads it, never runs backwards
  unsigned long long prev = rs_coarse_now_ns();
  for (int i = 0; i < 50; ++i) {
    std::this_thread::sleep_for(std::chrono::milliseconds(2));
    const unsigned long long c = rs_coarse_now_ns(), exact = rs_steady_now_ns();
    if (c < prev) fail("coarse clock ran backwards");
    if (c > exact) fail("coarse clock leads the exact clock");
    if (exact - c > 20000000000ull) fail("coarse clock is stale by more than twenty seconds");   // generous: sanitizer builds on busy boxes
    prev = c;
  }
  std::printf("host_stress: index ring, %d producers / %d consumers, %d entries; coarse clock\n", kProducers, kConsumers,
              kProducers * kPerProducer);
}

void stress_controller(const char* mode) {
  constexpr int kRanks = 4, kRows = 2000, kDim = 8, kL = 5, kSteps = 30, kPer = 64;
  const float clr = 0.5f;
  const int cache_rows = kRows / 20;
  char json[512];
  std::snprintf(json, sizeof(json),
                "{\"num_gpus\": %d, \"L\": %d, \"clr\": %f, \"dim\": %d, \"backwardMode\": \"%s\", \"nr_background_threads\": 2, "
                "\"full_emb_capacity\": %d, \"cache_ratio\": 0.05}", kRanks, kL, clr, kDim, mode, kRows);
  void* ctrl = nullptr;
  if (rs_ctrl_create(json, &ctrl) != 0) { fail("rs_ctrl_create", mode); return; }
  std::vector<float> table(static_cast<size_t>(kRows) * kDim, 0.f), oracle(table);
  std::vector<std::vector<float>> caches(kRanks, std::vector<float>(static_cast<size_t>(cache_rows) * kDim, 0.f));
  EXPECT_OK(rs_ctrl_register_table(ctrl, table.data(), kRows));
  for (int r = 0; r < kRanks; ++r) EXPECT_OK(rs_ctrl_register_cache(ctrl, r, caches[r].data()));
  EXPECT_OK(rs_ctrl_start(ctrl));
  const bool async = std::strncmp(mode, "CppAsync", 8) == 0;
  // batches[r][s]: ids rank r reads at step s, drawn up front; reads are published kL steps ahead
  std::vector<std::vector<std::vector<long long>>> batches(kRanks);
  for (int r = 0; r < kRanks; ++r) {
    Lcg rng(3000 + r);
    batches[r].resize(kSteps + kL);
    for (auto& b : batches[r]) { b.resize(kPer); for (auto& id : b) id = static_cast<long long>(rng.next() % kRows); }
    if (async) for (int s = 0; s < kL; ++s) EXPECT_OK(rs_ctrl_publish_reads(ctrl, r, s, batches[r][s].data(), kPer));
  }
  Barrier bar(kRanks);
  std::vector<std::vector<float>> grads(kRanks, std::vector<float>(static_cast<size_t>(kPer) * kDim));
  std::atomic<int> mismatches{0};
  std::vector<std::thread> ts;
  for (int r = 0; r < kRanks; ++r) {
    ts.emplace_back([&, r] {
      for (int step = 0; step < kSteps; ++step) {
        if (async) EXPECT_OK(rs_ctrl_publish_reads(ctrl, r, step + kL, batches[r][step + kL].data(), kPer));
        const auto& ids = batches[r][step];
        for (int i = 0; i < kPer; ++i) {                      // read through the cache placement: first rows live in the caches
          const long long id = ids[i];
          const float* row = id < static_cast<long long>(cache_rows) * kRanks
                                 ? &caches[id / cache_rows][static_cast<size_t>(id % cache_rows) * kDim]
                                 : &table[static_cast<size_t>(id) * kDim];
          for (int d = 0; d < kDim; ++d)
            if (std::fabs(row[d] - oracle[static_cast<size_t>(id) * kDim + d]) > 1e-4f) { mismatches.fetch_add(1); break; }
        }
        const float g = static_cast<float>(r + 1) * static_cast<float>(1 + step % 3);
        std::fill(grads[r].begin(), grads[r].end(), g);
        EXPECT_OK(rs_ctrl_set_step_input(ctrl, r, ids.data(), kPer, grads[r].data()));
        bar.wait();
        if (r == 0) {
          EXPECT_OK(rs_ctrl_process_one_step(ctrl, step));
          for (int rr = 0; rr < kRanks; ++rr)                 // synchronous oracle
            for (int i = 0; i < kPer; ++i)
              for (int d = 0; d < kDim; ++d)
                oracle[static_cast<size_t>(batches[rr][step][i]) * kDim + d] -= clr * grads[rr][static_cast<size_t>(i) * kDim + d];
          EXPECT_OK(rs_ctrl_block_to_step(ctrl, step + 1, 60000));
        }
        bar.wait();
      }
    });
  }
  for (auto& t : ts) t.join();
  EXPECT_OK(rs_ctrl_drain(ctrl));
  EXPECT_OK(rs_ctrl_stop(ctrl));
  if (rs_ctrl_pending(ctrl) != 0) fail("controller pending after drain", mode);
  if (mismatches.load() != 0) fail("controller read-your-updates", std::string(mode) + ": " + std::to_string(mismatches.load()) + " stale reads");
  for (int id = 0; id < kRows; ++id) {
    const float* row = id < cache_rows * kRanks ? &caches[id / cache_rows][static_cast<size_t>(id % cache_rows) * kDim]
                                                : &table[static_cast<size_t>(id) * kDim];
    if (std::fabs(row[0] - oracle[static_cast<size_t>(id) * kDim]) > 1e-3f) { fail("controller final table", mode); break; }
  }
  EXPECT_OK(rs_ctrl_destroy(ctrl));
  std::printf("host_stress: controller %s, %d ranks x %d steps\n", mode, kRanks, kSteps);
}

}  // namespace

int main(int argc, char** argv) {
  const std::string only = argc > 1 ? argv[1] : "all";
  if (only == "all" || only == "kv") {
    stress_kv("KVEngineMap", "{\"capacity\": 65536, \"value_size\": 32}");
    stress_kv("KVEngineExtendibleHash", "{\"capacity\": 65536, \"value_size\": 32}");
    stress_kv("KVEngineChunkHash", "{\"capacity\": 65536, \"value_size\": 32}");
    stress_kv("KVEnginePoolMap", "{\"capacity\": 65536, \"value_size\": 32}");
    for (const char* e : {"KVEngineMap", "KVEngineExtendibleHash", "KVEngineChunkHash", "KVEnginePoolMap"})
      stress_shared_keys(e, "{\"capacity\": 256, \"value_size\": 32}", 8);
    // 4 KB values: the pool map's pool holds a few hundred records, so writers run it dry every few milliseconds and
    // reclamation (epoch bump, scan of the readers, collection) runs all the time beside the readers
    stress_shared_keys("KVEnginePoolMap", "{\"capacity\": 128, \"value_size\": 4096}", 1024);
  }
  if (only == "all" || only == "ps") stress_ps();
  if (only == "all" || only == "alloc") {
    stress_allocator(0, "pool");
    stress_allocator(1, "binning");
    stress_allocator(2, "fixed");
  }
  if (only == "all" || only == "misc") stress_timers_and_barrier();
  if (only == "all" || only == "ring") stress_index_ring();
  if (only == "all" || only == "controller") {
    stress_controller("CppSync");
    stress_controller("CppAsyncV2");
  }
  if (g_failures) {
    std::fprintf(stderr, "host_stress: %d failure(s)\n", g_failures);
    return 1;
  }
  std::printf("host_stress: ok\n");
  return 0;
}
