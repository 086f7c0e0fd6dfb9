// "KVEnginePoolMap": a host KV engine whose values live in a PersistSlabPool and are replaced out of place.
//
// Every value is a sealed record {key, version, seal, bytes} in its own slab.  Put writes a NEW record, swings the
// index entry over under the shard lock and retires the old record through the EpochManager; Get copies the value
// outside the shard lock, inside a protected region, so readers never block writers for the length of a copy and never
// see a torn value.  The index (64 sharded hash maps key -> slab offset) is volatile: on reopen it is rebuilt from
// the allocated slabs of the pool, keeping the highest sealed version of each key and freeing unsealed (torn) or
// superseded records.  The reference keeps values in its PersistMemoryPool and defers frees through its epoch manager
// the same way in the persistent hash engines (src/memory/persist_malloc.h:126-420, src/memory/epoch_manager.h).
#include <atomic>
#include <chrono>
#include <cstring>
#include <shared_mutex>
#include <thread>
#include <unordered_map>

#include <sys/stat.h>

#include "common/rs_common.h"
#include "runtime/kv_engine.h"
#include "runtime/persist_pool.h"

namespace rs {

namespace {

struct Record {
  uint64_t key;
  uint64_t version;
  std::atomic<uint64_t> seal;     // key ^ version ^ kSeal once the bytes are complete, 0 when unlinked
  char bytes[1];
};
constexpr uint64_t kSeal = 0x9E3779B97F4A7C15ull;
constexpr size_t kRecordHeader = 24;

class KVEnginePoolMap final : public BaseKV {
 public:
  explicit KVEnginePoolMap(const KVConfig& c) : BaseKV(c), shards_(64) {
    rec_bytes_ = kRecordHeader + c.value_size;
    const uint64_t cs = PersistSlabPool::ClassSize(rec_bytes_);
    uint64_t chunk = 2ull << 20;
    while (chunk < cs * 4 + 4096) chunk <<= 1;
    // room for every key plus the records that wait for their epoch, rounded up to whole chunks
    const uint64_t per_chunk = (chunk - 4096) / cs;
    const uint64_t chunks = (c.capacity + c.capacity / 4 + 64 + per_chunk - 1) / per_chunk + 1;
    const std::string file = c.path.empty() ? std::string() : c.path + "/poolmap.slabs";
    if (!c.path.empty()) mkdir(c.path.c_str(), 0755);
    bool rec = false;
    pool_ = PersistSlabPool::Open(file, chunks * chunk, chunk, &rec);
    if (!pool_) return;
    recovered_ = rec;
    if (rec) Rebuild();
  }
  bool ok() const { return pool_ != nullptr; }
  bool recovered() const { return recovered_; }
  uint64_t dropped_on_recovery() const { return dropped_; }

  bool Get(uint64_t key, void* out) override {
    Shard& s = shard(key);
    epoch_.Protect();
    uint64_t off = 0;
    {
      std::shared_lock<std::shared_mutex> lk(s.mu);
      auto it = s.map.find(key);
      if (it != s.map.end()) off = it->second;
    }
    if (off) memcpy(out, rec(off)->bytes, cfg_.value_size);   // the record cannot be reused while we are protected
    epoch_.Unprotect();
    return off != 0;
  }
  bool Put(uint64_t key, const void* value) override {
    uint64_t off = AllocRecord();
    // An empty pool usually means that superseded records are waiting for a reader that was descheduled inside its
    // protected region, not that the engine is full: advance the epoch, collect, and give such readers a moment (bounded)
    // before refusing the write.
    for (int attempt = 0; !off && attempt < 4000; ++attempt) {     // up to ~2 s
      epoch_.Bump();
      epoch_.Collect();
      off = AllocRecord();
      if (!off) {
        if (epoch_.Pending() == 0) break;              // nothing left to wait for: the pool really is exhausted
        std::this_thread::sleep_for(std::chrono::microseconds(attempt < 20 ? 50 : 500));
      }
    }
    if (!off) return false;
    Record* r = rec(off);
    r->key = key;
    r->version = version_.fetch_add(1, std::memory_order_relaxed);
    memcpy(r->bytes, value, cfg_.value_size);
    r->seal.store(key ^ r->version ^ kSeal, std::memory_order_release);
    Shard& s = shard(key);
    uint64_t old = 0;
    {
      std::unique_lock<std::shared_mutex> lk(s.mu);
      auto it = s.map.find(key);
      if (it == s.map.end()) {
        if (size_.load(std::memory_order_relaxed) >= cfg_.capacity) {
          lk.unlock();
          r->seal.store(0, std::memory_order_release);
          pool_->Free(off);
          return false;
        }
        s.map.emplace(key, off);
        size_.fetch_add(1, std::memory_order_relaxed);
      } else {
        old = it->second;
        it->second = off;
      }
    }
    if (old) Unlink(old);
    return true;
  }
  bool Erase(uint64_t key) override {
    Shard& s = shard(key);
    uint64_t old = 0;
    {
      std::unique_lock<std::shared_mutex> lk(s.mu);
      auto it = s.map.find(key);
      if (it == s.map.end()) return false;
      old = it->second;
      s.map.erase(it);
      size_.fetch_sub(1, std::memory_order_relaxed);
    }
    Unlink(old);
    return true;
  }
  void Clear() override {
    for (Shard& s : shards_) s.mu.lock();
    for (Shard& s : shards_) s.map.clear();
    epoch_.DrainAll();
    for (Stock& st : stocks_) {
      std::lock_guard<SpinLock> lk(st.mu);
      st.n = 0;
    }
    pool_->Reset();
    size_.store(0);
    for (Shard& s : shards_) s.mu.unlock();
  }
  uint64_t Size() const override { return size_.load(); }
  std::string DebugInfo() const override {
    const auto st = pool_->GetStats();
    return "KVEnginePoolMap size=" + std::to_string(Size()) + " capacity=" + std::to_string(cfg_.capacity) +
           " slabs=" + std::to_string(st.slabs_in_use) + " chunks=" + std::to_string(st.chunks_in_use) + "/" +
           std::to_string(st.chunks_total) + " pending_frees=" + std::to_string(epoch_.Pending()) +
           " epoch=" + std::to_string(epoch_.Current());
  }
  bool Persistent() const override { return !cfg_.path.empty(); }
  void Flush() override {
    epoch_.Bump();
    epoch_.Collect();
    for (Stock& st : stocks_) {                      // unused stock goes back, so a clean reopen drops nothing
      std::lock_guard<SpinLock> lk(st.mu);
      while (st.n > 0) pool_->Free(st.off[--st.n]);
    }
    pool_->Sync();
  }
  size_t Keys(uint64_t* out, size_t cap) const override {
    size_t n = 0;
    for (const Shard& s : shards_) {
      std::shared_lock<std::shared_mutex> lk(s.mu);
      for (auto& kv : s.map) {
        if (n >= cap) return n;
        out[n++] = kv.first;
      }
    }
    return n;
  }

 private:
  struct Shard {
    mutable std::shared_mutex mu;
    std::unordered_map<uint64_t, uint64_t> map;
  };
  // Small stocks of free slabs, one per stripe of threads, refilled 32 at a time: concurrent writers do not meet on the
  // pool's class lock.  Slabs sitting in a stock are allocated but unsealed, so a reopen after a crash frees them.
  static constexpr int kStockSlabs = 64;
  struct alignas(64) Stock {
    SpinLock mu;
    uint64_t off[kStockSlabs];
    int n = 0;
  };
  Stock& my_stock() {
    static std::atomic<unsigned> next_stripe{0};
    thread_local unsigned stripe = next_stripe.fetch_add(1, std::memory_order_relaxed);
    return stocks_[stripe % kStocks];
  }
  uint64_t AllocRecord() {
    Stock& st = my_stock();
    std::lock_guard<SpinLock> lk(st.mu);
    if (st.n == 0) st.n = static_cast<int>(pool_->MallocBatch(rec_bytes_, st.off, kStockSlabs / 2));
    return st.n > 0 ? st.off[--st.n] : 0;
  }
  static constexpr int kStocks = 16;
  Stock stocks_[kStocks];
  Shard& shard(uint64_t key) { return shards_[hash64(key) & 63]; }
  Record* rec(uint64_t off) const { return static_cast<Record*>(pool_->At(off)); }
  // The record is out of the index: it must not come back after a crash, and its slab returns to the pool once no
  // reader can still be copying from it.
  void Unlink(uint64_t off) {
    rec(off)->seal.store(0, std::memory_order_release);
    epoch_.Retire([this, off] { Recycle(off); });
  }
  // A reclaimed record goes straight into the reclaiming thread's stock when there is room (all records have one size),
  // so in steady state writers neither free to nor allocate from the pool.
  void Recycle(uint64_t off) {
    Stock& st = my_stock();
    {
      std::lock_guard<SpinLock> lk(st.mu);
      if (st.n < kStockSlabs) {
        st.off[st.n++] = off;
        return;
      }
    }
    pool_->Free(off);
  }
  void Rebuild() {
    const uint64_t want = PersistSlabPool::ClassSize(rec_bytes_);
    std::vector<uint64_t> drop;
    uint64_t max_version = 0;
    pool_->ForEachAllocated([&](uint64_t off, uint64_t cs) {
      Record* r = rec(off);
      if (cs != want || r->seal.load(std::memory_order_acquire) != (r->key ^ r->version ^ kSeal)) {
        drop.push_back(off);
        return;
      }
      max_version = std::max(max_version, r->version);
      auto& m = shard(r->key).map;
      auto it = m.find(r->key);
      if (it == m.end()) {
        m.emplace(r->key, off);
      } else if (rec(it->second)->version < r->version) {
        drop.push_back(it->second);
        it->second = off;
      } else {
        drop.push_back(off);
      }
    });
    for (uint64_t off : drop) pool_->Free(off);
    dropped_ = drop.size();
    uint64_t n = 0;
    for (Shard& s : shards_) n += s.map.size();
    size_.store(n);
    version_.store(max_version + 1);
  }

  std::vector<Shard> shards_;
  std::unique_ptr<PersistSlabPool> pool_;
  EpochManager epoch_;
  std::atomic<uint64_t> size_{0}, version_{1};
  uint64_t rec_bytes_ = 0, dropped_ = 0;
  bool recovered_ = false;
};

}  // namespace

std::unique_ptr<BaseKV> CreatePoolMapKV(const KVConfig& cfg) {
  auto p = std::make_unique<KVEnginePoolMap>(cfg);
  if (!p->ok()) return nullptr;
  return p;
}

bool PoolMapRecoveryState(BaseKV* kv, bool* recovered, uint64_t* dropped) {
  auto* e = dynamic_cast<KVEnginePoolMap*>(kv);
  if (!e) return false;
  *recovered = e->recovered();
  *dropped = e->dropped_on_recovery();
  return true;
}

}  // namespace rs
