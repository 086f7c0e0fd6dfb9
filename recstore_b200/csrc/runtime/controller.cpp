// Lookahead cache controller: deferred ("lazy") application of sparse updates to the big host table,
// ordered by the next step in which each id will be read.
//
// Contract kept from the reference's KGCacheController (src/framework/pytorch/kg_controller.h:36-116,
// grad_base.h:146-507, grad_async_v1.h:181-593, grad_async_v2.h:11-322): a key read at step s
// observes every update produced by steps < s (BlockToStepN), while updates of ids that nobody
// will read soon may lag behind in a priority queue.  The samplers publish the ids of the next L
// batches (lookahead); an id with pending writes has priority = its earliest future read step,
// +infinity when no read is registered.
//
// The queue is a bucket array over steps (O(1) insert / move, like ParallelPq, parallel_pq.h:164-446)
// sharded by id; background flusher threads drain the lowest bucket first and BlockToStepN helps
// draining instead of spinning.  Rows cached in HBM are updated by the owning GPU's kernel; here
// "cache" rows are the caller-registered per-rank cache tensors (used on the CPU path and by the tests).
//
// Two asynchronous strategies, chosen by "backwardMode":
//   CppAsync   (grad_async_v1.h): the samplers' read announcements go through per-rank mailboxes that a
//              "detect" thread turns into queue priorities (use_detect_thread = 0 applies them in the
//              caller instead); pending updates are flushed ONE ID AT A TIME, lowest priority first.
//              The step's (keys, grads) are upserted in one of three ways ("update_pq_use_omp",
//              grad_async_v1.h:496-541): 0 = serially on the calling thread, 1 = one task per rank,
//              2 = one task per group of queue shards, each task scanning every rank's keys and taking
//              only the ids of its own shards (no two tasks ever contend for a shard lock).
//   CppAsyncV2 (grad_async_v2.h:86-163, parallel_pq_v2.h:256-290): flushers take a WHOLE BUCKET: the id
//              list of the lowest step is swapped out under the shard lock, the pending updates of its
//              live entries are detached, and the rows are written back after the lock is released.
//
// Also here: the binary-heap priority queue with an index map and an invariant checker
// (src/base/pq.h:11-224) used as the oracle in tests.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <climits>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <shared_mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "common/rs_common.h"
#include "runtime/base.h"
#include "runtime/json_lite.h"

namespace rs {

// ============================================================== heap PQ with index map
class IndexedHeap {
 public:
  // push or change the priority of `id`
  void upsert(int64_t id, int64_t prio) {
    auto it = pos_.find(id);
    if (it == pos_.end()) {
      heap_.push_back({prio, id});
      pos_[id] = heap_.size() - 1;
      up(heap_.size() - 1);
    } else {
      const size_t i = it->second;
      const int64_t old = heap_[i].prio;
      heap_[i].prio = prio;
      if (prio < old) up(i); else down(i);
    }
  }
  bool erase(int64_t id) {
    auto it = pos_.find(id);
    if (it == pos_.end()) return false;
    const size_t i = it->second;
    swap_nodes(i, heap_.size() - 1);
    pos_.erase(heap_.back().id);
    heap_.pop_back();
    if (i < heap_.size()) { up(i); down(i); }
    return true;
  }
  bool top(int64_t* id, int64_t* prio) const {
    if (heap_.empty()) return false;
    *id = heap_[0].id; *prio = heap_[0].prio;
    return true;
  }
  bool pop(int64_t* id, int64_t* prio) {
    if (!top(id, prio)) return false;
    erase(*id);
    return true;
  }
  size_t size() const { return heap_.size(); }
  bool check() const {
    if (pos_.size() != heap_.size()) return false;
    for (size_t i = 0; i < heap_.size(); ++i) {
      if (i && heap_[(i - 1) / 2].prio > heap_[i].prio) return false;
      auto it = pos_.find(heap_[i].id);
      if (it == pos_.end() || it->second != i) return false;
    }
    return true;
  }

 private:
  struct Node { int64_t prio, id; };
  void swap_nodes(size_t a, size_t b) {
    if (a == b) return;
    std::swap(heap_[a], heap_[b]);
    pos_[heap_[a].id] = a;
    pos_[heap_[b].id] = b;
  }
  void up(size_t i) {
    while (i && heap_[(i - 1) / 2].prio > heap_[i].prio) { swap_nodes(i, (i - 1) / 2); i = (i - 1) / 2; }
  }
  void down(size_t i) {
    for (;;) {
      size_t l = 2 * i + 1, r = l + 1, m = i;
      if (l < heap_.size() && heap_[l].prio < heap_[m].prio) m = l;
      if (r < heap_.size() && heap_[r].prio < heap_[m].prio) m = r;
      if (m == i) return;
      swap_nodes(i, m);
      i = m;
    }
  }
  std::vector<Node> heap_;
  std::unordered_map<int64_t, size_t> pos_;
};

// ============================================================== controller
constexpr int64_t kInf = INT64_MAX;
constexpr int kHorizon = 1024;  // steps of lookahead the bucket array can hold (reference: kMaxPriority = 1000)

struct Elem {
  std::vector<int64_t> reads;    // future read steps, ascending, may hold duplicates (several ranks)
  std::vector<float> pending;    // accumulated -clr * sum of grads not yet applied (empty = none)
  int64_t prio = kInf;           // bucket it currently sits in (kInf = infinity bucket / not queued)
  bool queued = false;
};

class Controller {
 public:
  explicit Controller(const std::string& json) {
    JsonLite j(json);
    ranks_ = static_cast<int>(j.i64("num_gpus", 1));
    L_ = std::min<int>(static_cast<int>(j.i64("L", 10)), kHorizon - 2);
    clr_ = static_cast<float>(j.num("clr", 0.01));
    dim_ = static_cast<int>(j.i64("dim", j.i64("emb_dim", 32)));
    capacity_ = j.i64("full_emb_capacity", 0);
    const double ratio = j.num("cache_ratio", 0.0);
    cache_size_ = static_cast<int64_t>(capacity_ * ratio);
    const std::string mode = j.str("backwardMode", "CppAsyncV2");
    async_ = mode != "CppSync" && mode != "PySync";
    v2_ = mode == "CppAsyncV2";
    upsert_mode_ = static_cast<int>(j.i64("update_pq_use_omp", 1));
    detect_ = async_ && j.i64("use_detect_thread", v2_ ? 0 : 1) != 0;

    nthreads_ = static_cast<int>(j.i64("nr_background_threads", 2));
    nshards_ = std::max(1, static_cast<int>(j.i64("kUpdatePqWorkerNum", 16)));
    shards_ = std::vector<Shard>(nshards_);
    for (auto& s : shards_) s.buckets.resize(kHorizon);
    mail_ = std::vector<Mailbox>(ranks_);
    caches_.assign(ranks_, nullptr);
    inputs_.assign(ranks_, Input{});
  }
  ~Controller() { StopThreads(); }

  void RegisterTable(float* table, int64_t rows) {
    table_ = table;
    rows_ = rows;
    if (capacity_ == 0) capacity_ = rows;
    row_locks_.resize(static_cast<size_t>(rows));
  }
  void RegisterCache(int rank, float* cache) { caches_[rank] = cache; }
  int ranks() const { return ranks_; }
  void Start() {
    if (!async_ || running_) return;
    running_ = true;
    for (int t = 0; t < nthreads_; ++t) flushers_.emplace_back([this] { FlushLoop(); });
    if (detect_) flushers_.emplace_back([this] { DetectLoop(); });
  }
  void StopThreads() {
    if (!running_.exchange(false)) return;
    for (auto& t : flushers_) t.join();
    flushers_.clear();
    DrainMail();                       // announcements that were still in the mailboxes are not lost
  }
  // Flush everything that is still pending (end of training / before a checkpoint).
  void Drain() {
    DrainMail();
    for (int s = 0; s < nshards_; ++s)
      while (Flush(s, kInf, true)) {}
  }

  // The sampler tells that `rank` will read `ids` at `step` (step > current step).  With the detect thread the
  // announcement is only dropped into the rank's mailbox here.
  void PublishReads(int rank, int64_t step, const int64_t* ids, int64_t n) {
    if (!async_) return;
    if (detect_ && running_) {
      Mailbox& m = mail_[rank];
      mail_items_.fetch_add(1);
      std::lock_guard<SpinLock> lk(m.mu);
      m.q.push_back(Mail{step, std::vector<int64_t>(ids, ids + n)});
      return;
    }
    ApplyReads(step, ids, n);
  }
  void ApplyReads(int64_t step, const int64_t* ids, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
      const int64_t id = ids[i];
      if (id < 0 || id >= rows_) continue;
      Shard& sh = shard_of(id);
      std::lock_guard<SpinLock> lk(sh.mu);
      Elem& e = sh.elems[id];
      e.reads.insert(std::upper_bound(e.reads.begin(), e.reads.end(), step), step);
      Requeue(sh, id, e);
    }
    max_published_.store(std::max<int64_t>(max_published_.load(), step));
  }
  void SetStepInput(int rank, const int64_t* keys, int64_t n, const float* grads) { inputs_[rank] = Input{keys, n, grads}; }

  // Consumes the registered (keys, grads) of every rank for `step`: cached rows are updated in the
  // owning rank's cache, the rest goes to the host table now (sync) or to the queue (async).
  void ProcessOneStep(int64_t step) {
    // group = -1: every id of ranks [rb, re); group >= 0: only the ids whose queue shard belongs to that group
    const int ngroups = std::max(1, std::min(nshards_, ThreadPool::global().size() > 0 ? ThreadPool::global().size() : 1));
    auto body_ranks = [&](size_t rb, size_t re, int group) {
      for (size_t r = rb; r < re; ++r) {
        const Input& in = inputs_[r];
        for (int64_t i = 0; i < in.n; ++i) {
          const int64_t id = in.keys[i];
          if (id < 0 || id >= rows_) continue;
          if (group >= 0 && static_cast<int>(hash64(static_cast<uint64_t>(id)) % nshards_) % ngroups != group) continue;
          const float* g = in.grads + i * dim_;
          const int owner = CacheOwner(id);
          if (owner >= 0 && caches_[owner]) {
            // A registered (host-visible) cache replica is updated here; an HBM replica is updated by the
            // owning GPU's kernel.  The host table receives every update as well (grad_base.h:440-461, 509-565),
            // so it stays a complete copy that any rank may read.
            float* row = caches_[owner] + (id - owner * cache_size_) * dim_;
            BitRow cr = row_lock(id);
            std::lock_guard<BitRow> clk(cr);
            for (int d = 0; d < dim_; ++d) row[d] -= clr_ * g[d];
          }
          if (!async_) {
            BitRow br = row_lock(id);
            std::lock_guard<BitRow> lk(br);
            float* row = table_ + id * dim_;
            for (int d = 0; d < dim_; ++d) row[d] -= clr_ * g[d];
            continue;
          }
          Shard& sh = shard_of(id);
          std::lock_guard<SpinLock> lk(sh.mu);
          Elem& e = sh.elems[id];
          // this step's read of the id is over
          auto it = std::lower_bound(e.reads.begin(), e.reads.end(), step);
          if (it != e.reads.end() && *it == step) e.reads.erase(it);
          if (e.pending.empty()) e.pending.assign(dim_, 0.f);
          for (int d = 0; d < dim_; ++d) e.pending[d] -= clr_ * g[d];
          Requeue(sh, id, e);
        }
      }
    };
    // announcements of reads up to this step must be in the queue before this step's updates are ranked
    if (detect_) DrainMail();
    if (async_ && upsert_mode_ == 2 && ngroups > 1) {
      upsert_calls_[2].fetch_add(1);
      ThreadPool::global().parallel_for(ngroups, [&](size_t gb, size_t ge, int) {
        for (size_t g = gb; g < ge; ++g) body_ranks(0, ranks_, static_cast<int>(g));
      });
    } else if (ranks_ > 1 && (!async_ || upsert_mode_ != 0)) {
      upsert_calls_[1].fetch_add(1);
      ThreadPool::global().parallel_for(ranks_, [&](size_t rb, size_t re, int) { body_ranks(rb, re, -1); });
    } else {
      upsert_calls_[0].fetch_add(1);
      body_ranks(0, ranks_, -1);
    }
    // reads registered for this step by ranks that produced no gradient for the id are dropped lazily in Requeue
    cur_step_.store(step);
  }

  // Returns once no id that is read at a step <= `step` has an unapplied update (helps flushing).
  // false = timed out.
  bool BlockToStepN(int64_t step, int timeout_ms) {
    if (!async_) return true;
    const auto t0 = std::chrono::steady_clock::now();
    long long next_warn_ms = 1000;
    for (;;) {
      bool busy = false;
      if (detect_ && DrainMail()) busy = true;     // a read that is still in a mailbox has no priority yet
      for (int s = 0; s < nshards_; ++s) {
        while (Flush(s, step, false)) busy = true;
      }
      if (!busy && inflight_.load() == 0 && mail_items_.load() == 0) {
        // Every flusher holds flight_mu_ (shared) from the moment it detaches an update until the row is written.
        // Taking it exclusively means: nobody is between "detached" and "written" right now, and nobody can detach
        // anything while the queue is inspected.
        std::unique_lock<std::shared_mutex> quiet(flight_mu_);
        if (MinPriority() > step && inflight_.load() == 0 && mail_items_.load() == 0) {
          return true;
        }
      }
      const long long waited_ms =
          std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
      if (timeout_ms >= 0 && waited_ms > timeout_ms) return false;
      // A wait that drags on is reported once a second with what it is waiting for (the reference logs the same from
      // its BlockToStepN and dispatch loops, grad_async_v1.h:450-452, 553-559), so a stuck trainer is not silent.
      if (waited_ms >= next_warn_ms) {
        next_warn_ms = waited_ms + 1000;
        stall_warnings_.fetch_add(1, std::memory_order_relaxed);
        fprintf(stderr, "[recstore controller] BlockToStepN(%lld) has waited %lld ms: min priority %lld, %d updates in flight, %d announcements in mailboxes\n",
                static_cast<long long>(step), waited_ms, static_cast<long long>(MinPriority()), static_cast<int>(inflight_.load()),
                static_cast<int>(mail_items_.load()));
      }
    }
  }
  uint64_t stall_warnings() const { return stall_warnings_.load(); }
  // out: has_pending, prio, number of registered reads, earliest read (-1 = none), queued
  void DebugElem(int64_t id, long long* out) {
    Shard& sh = shard_of(id);
    std::lock_guard<SpinLock> lk(sh.mu);
    auto it = sh.elems.find(id);
    out[0] = out[2] = out[4] = 0; out[1] = out[3] = -1;
    if (it == sh.elems.end()) return;
    const Elem& e = it->second;
    out[0] = e.pending.empty() ? 0 : 1;
    out[1] = e.prio == kInf ? -2 : e.prio;
    out[2] = static_cast<long long>(e.reads.size());
    out[3] = e.reads.empty() ? -1 : e.reads.front();
    out[4] = e.queued ? 1 : 0;
  }
  int64_t MinPriority() {
    int64_t m = kInf;
    for (auto& sh : shards_) {
      std::lock_guard<SpinLock> lk(sh.mu);
      for (int64_t p = sh.min_hint; p < sh.min_hint + kHorizon; ++p) {
        if (!sh.buckets[p % kHorizon].empty()) { m = std::min(m, p); break; }
        if (p >= sh.max_prio) break;
      }
    }
    return m;
  }
  int64_t PendingCount() {
    int64_t n = 0;
    for (auto& sh : shards_) {
      std::lock_guard<SpinLock> lk(sh.mu);
      for (auto& kv : sh.elems) n += kv.second.pending.empty() ? 0 : 1;
    }
    return n;
  }
  std::string PrintPq() {
    std::string s = "pq: min=" + (MinPriority() == kInf ? std::string("inf") : std::to_string(MinPriority())) +
                    " pending=" + std::to_string(PendingCount()) + " flushed=" + std::to_string(flushed_.load()) +
                    " bucket_swaps=" + std::to_string(bucket_swaps_.load()) + " mail=" + std::to_string(mail_seen_.load());
    return s;
  }
  // out[0] rows written back, [1] whole-bucket swaps (V2), [2] announcements that went through a mailbox,
  // [3..5] ProcessOneStep calls that upserted serially / per rank / per shard group
  void Stats(long long* out) const {
    out[0] = flushed_.load(); out[1] = bucket_swaps_.load(); out[2] = mail_seen_.load();
    for (int m = 0; m < 3; ++m) out[3 + m] = upsert_calls_[m].load();
  }
  int dim() const { return dim_; }
  bool async() const { return async_; }

 private:
  struct Input { const int64_t* keys = nullptr; int64_t n = 0; const float* grads = nullptr; };
  struct Mail { int64_t step; std::vector<int64_t> ids; };
  struct Mailbox {
    SpinLock mu;
    std::vector<Mail> q;
  };
  // Moves every announcement that sits in a mailbox into the queue; true when there was any.
  bool DrainMail() {
    bool any = false;
    for (auto& m : mail_) {
      std::vector<Mail> got;
      {
        std::lock_guard<SpinLock> lk(m.mu);
        got.swap(m.q);
      }
      for (auto& x : got) {
        ApplyReads(x.step, x.ids.data(), static_cast<int64_t>(x.ids.size()));
        mail_seen_.fetch_add(1);
        mail_items_.fetch_sub(1);
        any = true;
      }
    }
    return any;
  }
  void DetectLoop() {
    while (running_) {
      if (!DrainMail()) std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
  }
  bool Flush(int s, int64_t limit, bool any) { return v2_ ? FlushBucket(s, limit, any) : FlushOne(s, limit, any); }
  struct Shard {
    SpinLock mu;
    std::unordered_map<int64_t, Elem> elems;
    std::vector<std::vector<int64_t>> buckets;  // ids per step bucket (lazy deletion: entry valid iff elem.prio matches)
    std::vector<int64_t> inf_bucket;
    int64_t min_hint = 0, max_prio = 0;
  };
  struct BitRow {
    BitLockTable* t; size_t i;
    void lock() { t->lock(i); }
    void unlock() { t->unlock(i); }
  };
  BitRow row_lock(int64_t id) { return BitRow{&row_locks_, static_cast<size_t>(id)}; }
  Shard& shard_of(int64_t id) { return shards_[hash64(static_cast<uint64_t>(id)) % nshards_]; }
  bool InCache(int64_t id) const { return cache_size_ > 0 && id < cache_size_ * ranks_; }
  int CacheOwner(int64_t id) const { return InCache(id) ? static_cast<int>(id / cache_size_) : -1; }

  // sh.mu held.  Recomputes the priority of `id` and moves it to the right bucket.
  void Requeue(Shard& sh, int64_t id, Elem& e) {
    const int64_t cur = cur_step_.load();
    while (!e.reads.empty() && e.reads.front() <= cur) e.reads.erase(e.reads.begin());  // stale reads
    int64_t prio = kInf;
    if (!e.pending.empty()) prio = e.reads.empty() ? kInf : e.reads.front();
    if (e.pending.empty()) {
      e.queued = false;
      e.prio = kInf;
      if (e.reads.empty()) sh.elems.erase(id);
      return;
    }
    if (e.queued && e.prio == prio) return;
    e.prio = prio;
    e.queued = true;
    if (prio == kInf) {
      sh.inf_bucket.push_back(id);
    } else {
      sh.buckets[prio % kHorizon].push_back(id);
      sh.min_hint = std::min(sh.min_hint, prio);
      sh.max_prio = std::max(sh.max_prio, prio);
    }
  }
  // Applies the pending update of one id of shard s whose priority is <= limit (or anything, when
  // `any`, including the infinity bucket).  Returns false when nothing qualified.
  bool FlushOne(int s, int64_t limit, bool any) {
    std::shared_lock<std::shared_mutex> in_flight(flight_mu_);
    Shard& sh = shards_[s];
    int64_t id = -1;
    std::vector<float> upd;
    {
      std::lock_guard<SpinLock> lk(sh.mu);
      const int64_t hi = std::min<int64_t>(any ? sh.max_prio : limit, sh.max_prio);
      for (int64_t p = sh.min_hint; p <= hi && id < 0; ++p) {
        auto& b = sh.buckets[p % kHorizon];
        while (!b.empty()) {
          const int64_t cand = b.back();
          b.pop_back();
          auto it = sh.elems.find(cand);
          if (it == sh.elems.end() || !it->second.queued || it->second.prio != p) continue;  // moved meanwhile
          id = cand;
          break;
        }
        if (id < 0 && b.empty() && p == sh.min_hint && sh.min_hint < sh.max_prio) ++sh.min_hint;
      }
      if (id < 0 && any) {
        while (!sh.inf_bucket.empty()) {
          const int64_t cand = sh.inf_bucket.back();
          sh.inf_bucket.pop_back();
          auto it = sh.elems.find(cand);
          if (it == sh.elems.end() || !it->second.queued || it->second.prio != kInf) continue;
          id = cand;
          break;
        }
      }
      if (id < 0) return false;
      Elem& e = sh.elems[id];
      upd.swap(e.pending);
      e.queued = false;
      e.prio = kInf;
      if (e.reads.empty()) sh.elems.erase(id);
      inflight_.fetch_add(1);
    }
    {
      BitRow br = row_lock(id);
      std::lock_guard<BitRow> lk(br);
      float* row = table_ + id * dim_;
      for (int d = 0; d < dim_; ++d) row[d] += upd[d];
    }
    flushed_.fetch_add(1, std::memory_order_relaxed);
    inflight_.fetch_sub(1);
    return true;
  }
  // V2: detaches a WHOLE bucket of shard s (the lowest one with priority <= limit; with `any` also the infinity
  // bucket) under the shard lock and writes its rows back after the lock is released.
  bool FlushBucket(int s, int64_t limit, bool any) {
    std::shared_lock<std::shared_mutex> in_flight(flight_mu_);
    Shard& sh = shards_[s];
    std::vector<std::pair<int64_t, std::vector<float>>> batch;
    {
      std::lock_guard<SpinLock> lk(sh.mu);
      std::vector<int64_t> ids;
      int64_t p_found = kInf;
      const int64_t hi = std::min<int64_t>(any ? sh.max_prio : limit, sh.max_prio);
      for (int64_t p = sh.min_hint; p <= hi; ++p) {
        auto& b = sh.buckets[p % kHorizon];
        if (!b.empty()) { ids.swap(b); p_found = p; break; }
        if (p == sh.min_hint && sh.min_hint < sh.max_prio) ++sh.min_hint;
      }
      if (ids.empty() && any && !sh.inf_bucket.empty()) ids.swap(sh.inf_bucket);
      if (ids.empty()) return false;
      bucket_swaps_.fetch_add(1, std::memory_order_relaxed);
      for (const int64_t cand : ids) {
        auto it = sh.elems.find(cand);
        if (it == sh.elems.end() || !it->second.queued || it->second.prio != p_found || it->second.pending.empty()) continue;  // moved meanwhile
        Elem& e = it->second;
        batch.emplace_back(cand, std::vector<float>());
        batch.back().second.swap(e.pending);
        e.queued = false;
        e.prio = kInf;
        if (e.reads.empty()) sh.elems.erase(it);
      }
      inflight_.fetch_add(static_cast<int>(batch.size()));
    }
    for (auto& kv : batch) {
      BitRow br = row_lock(kv.first);
      std::lock_guard<BitRow> lk(br);
      float* row = table_ + kv.first * dim_;
      for (int d = 0; d < dim_; ++d) row[d] += kv.second[d];
      inflight_.fetch_sub(1);
    }
    flushed_.fetch_add(static_cast<int64_t>(batch.size()), std::memory_order_relaxed);
    return true;
  }
  void FlushLoop() {
    int s = 0;
    while (running_) {
      bool any = false;
      for (int k = 0; k < nshards_ && running_; ++k) {
        s = (s + 1) % nshards_;
        // background threads stay within the lookahead window first, then take idle (infinity) work
        if (Flush(s, cur_step_.load() + L_ + 1, false)) any = true;
      }
      if (!any) {
        for (int k = 0; k < nshards_ && running_; ++k)
          if (Flush(k, kInf, true)) { any = true; break; }
      }
      if (!any) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }

  int ranks_ = 1, L_ = 10, dim_ = 32, nthreads_ = 2, nshards_ = 16;
  float clr_ = 0.01f;
  int64_t capacity_ = 0, cache_size_ = 0, rows_ = 0;
  bool async_ = true, v2_ = true, detect_ = false;
  int upsert_mode_ = 1;
  std::vector<Mailbox> mail_;
  std::atomic<int64_t> mail_items_{0}, mail_seen_{0}, bucket_swaps_{0};
  std::atomic<int64_t> upsert_calls_[3] = {{0}, {0}, {0}};
  float* table_ = nullptr;
  std::vector<float*> caches_;
  std::vector<Input> inputs_;
  std::vector<Shard> shards_;
  BitLockTable row_locks_;
  std::atomic<int64_t> cur_step_{-1}, max_published_{-1}, flushed_{0};
  std::atomic<int> inflight_{0};
  std::atomic<uint64_t> stall_warnings_{0};
  std::shared_mutex flight_mu_;
  std::atomic<bool> running_{false};
  std::vector<std::thread> flushers_;
};

}  // namespace rs

// ================================================================ C ABI
using rs::Controller;
using rs::IndexedHeap;

RS_API void* rs_heap_create() { return new IndexedHeap(); }
RS_API void rs_heap_destroy(void* h) { delete static_cast<IndexedHeap*>(h); }
RS_API void rs_heap_upsert(void* h, long long id, long long prio) { static_cast<IndexedHeap*>(h)->upsert(id, prio); }
RS_API int rs_heap_erase(void* h, long long id) { return static_cast<IndexedHeap*>(h)->erase(id) ? 1 : 0; }
RS_API int rs_heap_pop(void* h, long long* id, long long* prio) {
  int64_t i, p;
  if (!static_cast<IndexedHeap*>(h)->pop(&i, &p)) return 0;
  *id = i; *prio = p;
  return 1;
}
RS_API int rs_heap_top(void* h, long long* id, long long* prio) {
  int64_t i, p;
  if (!static_cast<IndexedHeap*>(h)->top(&i, &p)) return 0;
  *id = i; *prio = p;
  return 1;
}
RS_API long long rs_heap_size(void* h) { return static_cast<long long>(static_cast<IndexedHeap*>(h)->size()); }
RS_API int rs_heap_check(void* h) { return static_cast<IndexedHeap*>(h)->check() ? 1 : 0; }

RS_API int rs_ctrl_create(const char* json, void** out) {
  RS_REQUIRE(json && out, "rs_ctrl_create: null argument");
  // sizes from the config size vectors and start threads: check them before anything is built from them
  {
    rs::JsonLite j(json);
    const long long ranks = j.i64("num_gpus", 1), L = j.i64("L", 10), dim = j.i64("dim", j.i64("emb_dim", 32));
    const long long cap = j.i64("full_emb_capacity", 0), threads = j.i64("nr_background_threads", 2);
    const long long workers = j.i64("kUpdatePqWorkerNum", 16);
    const double ratio = j.num("cache_ratio", 0.0);
    RS_REQUIRE(ranks >= 1 && ranks <= 1024, "rs_ctrl_create: num_gpus = %lld outside [1, 1024]", ranks);
    RS_REQUIRE(L >= 0, "rs_ctrl_create: L = %lld is negative", L);
    RS_REQUIRE(dim >= 1 && dim <= (1 << 20), "rs_ctrl_create: dim = %lld outside [1, 2^20]", dim);
    RS_REQUIRE(cap >= 0 && cap <= (1ll << 40), "rs_ctrl_create: full_emb_capacity = %lld outside [0, 2^40]", cap);
    RS_REQUIRE(threads >= 0 && threads <= 256, "rs_ctrl_create: nr_background_threads = %lld outside [0, 256]", threads);
    RS_REQUIRE(workers <= 4096, "rs_ctrl_create: kUpdatePqWorkerNum = %lld above 4096", workers);
    RS_REQUIRE(ratio >= 0.0 && ratio <= 1.0, "rs_ctrl_create: cache_ratio = %g outside [0, 1]", ratio);
    const long long um = j.i64("update_pq_use_omp", 1);
    RS_REQUIRE(um >= 0 && um <= 2, "rs_ctrl_create: update_pq_use_omp = %lld is not 0 (serial), 1 (per rank) or 2 (per shard group)", um);
    const std::string mode = j.str("backwardMode", "CppAsyncV2");
    RS_REQUIRE(mode == "PySync" || mode == "CppSync" || mode == "CppAsync" || mode == "CppAsyncV2",
               "rs_ctrl_create: backwardMode %s is not one of PySync, CppSync, CppAsync, CppAsyncV2", mode.c_str());
  }
  RS_NOEXCEPT_BODY(
    *out = new Controller(json);
    return RS_OK;
  )
}
RS_API int rs_ctrl_destroy(void* c) { delete static_cast<Controller*>(c); return RS_OK; }
RS_API int rs_ctrl_register_table(void* c, float* table, long long rows) {
  RS_REQUIRE(c && table && rows > 0, "rs_ctrl_register_table: bad argument");
  static_cast<Controller*>(c)->RegisterTable(table, rows);
  return RS_OK;
}
RS_API int rs_ctrl_register_cache(void* c, int rank, float* cache) {
  RS_REQUIRE(c && rank >= 0 && rank < static_cast<Controller*>(c)->ranks(), "rs_ctrl_register_cache: rank %d out of range", rank);
  static_cast<Controller*>(c)->RegisterCache(rank, cache);
  return RS_OK;
}
RS_API int rs_ctrl_start(void* c) { static_cast<Controller*>(c)->Start(); return RS_OK; }
RS_API int rs_ctrl_stop(void* c) { static_cast<Controller*>(c)->StopThreads(); return RS_OK; }
RS_API int rs_ctrl_drain(void* c) { static_cast<Controller*>(c)->Drain(); return RS_OK; }
RS_API int rs_ctrl_publish_reads(void* c, int rank, long long step, const long long* ids, long long n) {
  RS_REQUIRE(c && rank >= 0 && rank < static_cast<Controller*>(c)->ranks() && n >= 0 && (ids || n == 0) && step >= 0,
             "rs_ctrl_publish_reads: bad argument (rank %d, step %lld, n %lld)", rank, step, n);
  static_cast<Controller*>(c)->PublishReads(rank, step, reinterpret_cast<const int64_t*>(ids), n);
  return RS_OK;
}
RS_API int rs_ctrl_set_step_input(void* c, int rank, const long long* keys, long long n, const float* grads) {
  RS_REQUIRE(c && rank >= 0 && rank < static_cast<Controller*>(c)->ranks() && n >= 0 && ((keys && grads) || n == 0),
             "rs_ctrl_set_step_input: bad argument (rank %d, n %lld)", rank, n);
  static_cast<Controller*>(c)->SetStepInput(rank, reinterpret_cast<const int64_t*>(keys), n, grads);
  return RS_OK;
}
RS_API int rs_ctrl_process_one_step(void* c, long long step) { static_cast<Controller*>(c)->ProcessOneStep(step); return RS_OK; }
RS_API int rs_ctrl_block_to_step(void* c, long long step, int timeout_ms) {
  return static_cast<Controller*>(c)->BlockToStepN(step, timeout_ms)
             ? RS_OK
             : rs::set_error(RS_ERR_TIMEOUT, "BlockToStepN(%lld) timed out after %d ms", step, timeout_ms);
}
RS_API int rs_ctrl_debug_elem(void* c, long long id, long long* out5) {
  RS_REQUIRE(c && out5, "rs_ctrl_debug_elem: null argument");
  static_cast<Controller*>(c)->DebugElem(id, out5);
  return RS_OK;
}
RS_API int rs_ctrl_stats(void* c, long long* out6) {
  RS_REQUIRE(c && out6, "rs_ctrl_stats: null argument");
  static_cast<Controller*>(c)->Stats(out6);
  return RS_OK;
}
RS_API long long rs_ctrl_pending(void* c) { return static_cast<Controller*>(c)->PendingCount(); }
RS_API long long rs_ctrl_min_priority(void* c) { return static_cast<Controller*>(c)->MinPriority(); }
RS_API int rs_ctrl_print_pq(void* c, char* buf, int cap) {
  const std::string s = static_cast<Controller*>(c)->PrintPq();
  if (buf && cap > 0) {
    const int n = std::min<int>(cap - 1, static_cast<int>(s.size()));
    memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return static_cast<int>(s.size());
}
