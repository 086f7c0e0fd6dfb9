#include "runtime/kv_engine.h"

#include <algorithm>
#include <atomic>
#include <cstring>
#include <mutex>
#include <shared_mutex>
#include <thread>
#include <unordered_map>

#include <emmintrin.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "common/rs_common.h"
#include "runtime/base.h"
#include "runtime/json_lite.h"

namespace rs {

// ============================================================== value store
// Fixed-size value slots in one mapping.  File-backed (MAP_SHARED) when a path is given, so the
// values survive the process; the header keeps the high-water mark, the free list is volatile and
// rebuilt by the owning engine on reload (mark_live / rebuild_free_list).
class SlabValueStore {
 public:
  struct Header {
    uint64_t magic;
    uint64_t value_size;
    uint64_t capacity;
    std::atomic<uint64_t> bump;
  };
  static constexpr uint64_t kMagic = 0x52534232534C4142ull;

  ~SlabValueStore() { close_map(); }

  bool open(const std::string& file, uint64_t capacity, uint32_t value_size, bool* existed) {
    close_map();
    vs_ = value_size;
    cap_ = capacity;
    bytes_ = 4096 + capacity * static_cast<uint64_t>(value_size);
    *existed = false;
    if (file.empty()) {
      base_ = mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
      if (base_ == MAP_FAILED) { base_ = nullptr; return false; }
    } else {
      int fd = ::open(file.c_str(), O_RDWR | O_CREAT, 0644);
      if (fd < 0) return false;
      struct stat st;
      fstat(fd, &st);
      *existed = static_cast<uint64_t>(st.st_size) >= bytes_;
      if (!*existed && ftruncate(fd, static_cast<off_t>(bytes_)) != 0) { ::close(fd); return false; }
      base_ = mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
      ::close(fd);
      if (base_ == MAP_FAILED) { base_ = nullptr; return false; }
    }
    Header* h = hdr();
    if (*existed && (h->magic != kMagic || h->value_size != value_size || h->capacity != capacity)) *existed = false;
    if (!*existed) {
      h->magic = kMagic;
      h->value_size = value_size;
      h->capacity = capacity;
      h->bump.store(0);
    }
    free_.clear();
    return true;
  }
  // Returns a slot index or UINT32_MAX when full.
  uint32_t alloc() {
    {
      std::lock_guard<SpinLock> lk(mu_);
      if (!free_.empty()) {
        const uint32_t i = free_.back();
        free_.pop_back();
        return i;
      }
    }
    const uint64_t i = hdr()->bump.fetch_add(1, std::memory_order_relaxed);
    if (i >= cap_) {
      hdr()->bump.fetch_sub(1, std::memory_order_relaxed);
      return UINT32_MAX;
    }
    return static_cast<uint32_t>(i);
  }
  void release(uint32_t i) {
    std::lock_guard<SpinLock> lk(mu_);
    free_.push_back(i);
  }
  char* at(uint32_t i) const { return static_cast<char*>(base_) + 4096 + static_cast<uint64_t>(i) * vs_; }
  void reset() {
    hdr()->bump.store(0);
    std::lock_guard<SpinLock> lk(mu_);
    free_.clear();
  }
  // After a reload: every slot below the high-water mark that is not live becomes free.
  void rebuild_free_list(const std::vector<bool>& live) {
    std::lock_guard<SpinLock> lk(mu_);
    free_.clear();
    const uint64_t hw = std::min<uint64_t>(hdr()->bump.load(), cap_);
    for (uint64_t i = 0; i < hw; ++i)
      if (i >= live.size() || !live[i]) free_.push_back(static_cast<uint32_t>(i));
  }
  uint64_t high_water() const { return std::min<uint64_t>(hdr()->bump.load(), cap_); }
  uint64_t capacity() const { return cap_; }
  void sync() {
    if (base_) msync(base_, bytes_, MS_SYNC);
  }

 private:
  Header* hdr() const { return static_cast<Header*>(base_); }
  void close_map() {
    if (base_) munmap(base_, bytes_);
    base_ = nullptr;
  }
  void* base_ = nullptr;
  uint64_t bytes_ = 0, cap_ = 0;
  uint32_t vs_ = 0;
  SpinLock mu_;
  std::vector<uint32_t> free_;
};

// ============================================================== BaseKV defaults
void BaseKV::BatchGet(const uint64_t* keys, size_t n, void* out, uint8_t* found) {
  const uint32_t vs = cfg_.value_size;
  auto body = [&](size_t b, size_t e, int) {
    for (size_t i = b; i < e; ++i) {
      char* o = static_cast<char*>(out) + i * vs;
      const bool ok = Get(keys[i], o);
      if (!ok) memset(o, 0, vs);
      if (found) found[i] = ok ? 1 : 0;
    }
  };
  if (n >= 4096) ThreadPool::global().parallel_for(n, body);
  else body(0, n, 0);
}
size_t BaseKV::BatchPut(const uint64_t* keys, size_t n, const void* values) {
  const uint32_t vs = cfg_.value_size;
  std::atomic<size_t> stored{0};
  auto body = [&](size_t b, size_t e, int) {
    size_t s = 0;
    for (size_t i = b; i < e; ++i) s += Put(keys[i], static_cast<const char*>(values) + i * vs) ? 1 : 0;
    stored += s;
  };
  if (n >= 4096) ThreadPool::global().parallel_for(n, body);
  else body(0, n, 0);
  return stored.load();
}
void BaseKV::BulkLoad(uint64_t n) {
  const uint32_t vs = cfg_.value_size;
  const size_t nf = vs / sizeof(float);
  auto body = [&](size_t b, size_t e, int) {
    std::vector<float> v(nf ? nf : 1);
    for (size_t k = b; k < e; ++k) {
      std::fill(v.begin(), v.end(), static_cast<float>(k));
      Put(k, v.data());
    }
  };
  ThreadPool::global().parallel_for(n, body);
}

// ============================================================== KVEngineMap
class KVEngineMap final : public BaseKV {
 public:
  explicit KVEngineMap(const KVConfig& c) : BaseKV(c), shards_(64) {
    bool existed;
    ok_ = slab_.open("", c.capacity, c.value_size, &existed);
  }
  bool ok() const { return ok_; }
  bool Get(uint64_t key, void* out) override {
    Shard& s = shard(key);
    std::shared_lock<std::shared_mutex> lk(s.mu);
    auto it = s.map.find(key);
    if (it == s.map.end()) return false;
    memcpy(out, slab_.at(it->second), cfg_.value_size);
    return true;
  }
  bool Put(uint64_t key, const void* value) override {
    Shard& s = shard(key);
    std::unique_lock<std::shared_mutex> lk(s.mu);
    auto it = s.map.find(key);
    uint32_t idx;
    if (it == s.map.end()) {
      idx = slab_.alloc();
      if (idx == UINT32_MAX) return false;
      s.map.emplace(key, idx);
      size_.fetch_add(1, std::memory_order_relaxed);
    } else {
      idx = it->second;
    }
    memcpy(slab_.at(idx), value, cfg_.value_size);
    return true;
  }
  bool Erase(uint64_t key) override {
    Shard& s = shard(key);
    std::unique_lock<std::shared_mutex> lk(s.mu);
    auto it = s.map.find(key);
    if (it == s.map.end()) return false;
    slab_.release(it->second);
    s.map.erase(it);
    size_.fetch_sub(1, std::memory_order_relaxed);
    return true;
  }
  void Clear() override {
    for (Shard& s : shards_) {
      std::unique_lock<std::shared_mutex> lk(s.mu);
      s.map.clear();
    }
    slab_.reset();
    size_.store(0);
  }
  uint64_t Size() const override { return size_.load(); }
  std::string DebugInfo() const override {
    return "KVEngineMap size=" + std::to_string(Size()) + " capacity=" + std::to_string(cfg_.capacity);
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
    std::unordered_map<uint64_t, uint32_t> map;
  };
  Shard& shard(uint64_t key) { return shards_[hash64(key) & 63]; }
  std::vector<Shard> shards_;
  SlabValueStore slab_;
  std::atomic<uint64_t> size_{0};
  bool ok_ = false;
};

// ============================================================== KVEngineExtendibleHash
// Reader-writer lock for a structure that is read by every operation and written rarely (the directory): a reader
// takes only the stripe its thread hashes to, so readers on different cores do not share a cache line; the writer
// takes every stripe.
class StripedSharedMutex {
  static constexpr int kStripes = 64;
  struct alignas(64) Stripe { std::shared_mutex mu; };

 public:
  void lock_shared() { s_[slot()].mu.lock_shared(); }
  void unlock_shared() { s_[slot()].mu.unlock_shared(); }
  void lock() { for (auto& st : s_) st.mu.lock(); }
  void unlock() { for (int i = kStripes - 1; i >= 0; --i) s_[i].mu.unlock(); }

 private:
  static int slot() {
    static thread_local const int v = static_cast<int>(std::hash<std::thread::id>()(std::this_thread::get_id()) % kStripes);
    return v;
  }
  Stripe s_[kStripes];
};

class KVEngineExtendibleHash final : public BaseKV {
  static constexpr int kSegCap = 128;
  struct Segment {
    SpinLock mu;
    int local_depth = 0;
    int count = 0;
    alignas(16) uint8_t tags[kSegCap];   // one hash byte per slot: a lookup compares 16 tags at a time and reads a key only on a tag match
    uint64_t keys[kSegCap];
    uint32_t idx[kSegCap];
  };
  static uint8_t tag_of(uint64_t h) { return static_cast<uint8_t>(h >> 56); }   // the directory uses the low bits
  // slot of `key` in the segment, or -1
  static int find(const Segment* s, uint64_t key, uint8_t tag) {
    const __m128i want = _mm_set1_epi8(static_cast<char>(tag));
    for (int base = 0; base < s->count; base += 16) {
      unsigned m = static_cast<unsigned>(_mm_movemask_epi8(_mm_cmpeq_epi8(_mm_load_si128(reinterpret_cast<const __m128i*>(s->tags + base)), want)));
      while (m) {
        const int i = base + __builtin_ctz(m);
        if (i < s->count && s->keys[i] == key) return i;
        m &= m - 1;
      }
    }
    return -1;
  }

 public:
  explicit KVEngineExtendibleHash(const KVConfig& c) : BaseKV(c) {
    bool existed;
    ok_ = slab_.open("", c.capacity, c.value_size, &existed);
    reset_dir();
  }
  ~KVEngineExtendibleHash() override { free_segments(); }
  bool ok() const { return ok_; }

  bool Get(uint64_t key, void* out) override {
    const uint64_t h = hash64(key);
    std::shared_lock<StripedSharedMutex> dl(dir_mu_);
    Segment* s = dir_[h & (dir_.size() - 1)];
    std::lock_guard<SpinLock> lk(s->mu);
    const int i = find(s, key, tag_of(h));
    if (i < 0) return false;
    memcpy(out, slab_.at(s->idx[i]), cfg_.value_size);
    return true;
  }
  bool Put(uint64_t key, const void* value) override {
    const uint64_t h = hash64(key);
    for (int attempt = 0; attempt < 64; ++attempt) {
      {
        std::shared_lock<StripedSharedMutex> dl(dir_mu_);
        Segment* s = dir_[h & (dir_.size() - 1)];
        std::lock_guard<SpinLock> lk(s->mu);
        const int at = find(s, key, tag_of(h));
        if (at >= 0) {
          memcpy(slab_.at(s->idx[at]), value, cfg_.value_size);
          return true;
        }
        if (s->count < kSegCap) {
          const uint32_t v = slab_.alloc();
          if (v == UINT32_MAX) return false;
          memcpy(slab_.at(v), value, cfg_.value_size);
          s->keys[s->count] = key;
          s->tags[s->count] = tag_of(h);
          s->idx[s->count] = v;
          ++s->count;
          size_.fetch_add(1, std::memory_order_relaxed);
          return true;
        }
      }
      split(h);
    }
    return false;
  }
  bool Erase(uint64_t key) override {
    const uint64_t h = hash64(key);
    std::shared_lock<StripedSharedMutex> dl(dir_mu_);
    Segment* s = dir_[h & (dir_.size() - 1)];
    std::lock_guard<SpinLock> lk(s->mu);
    const int i = find(s, key, tag_of(h));
    if (i < 0) return false;
    slab_.release(s->idx[i]);
    s->keys[i] = s->keys[s->count - 1];
    s->tags[i] = s->tags[s->count - 1];
    s->idx[i] = s->idx[s->count - 1];
    --s->count;
    size_.fetch_sub(1, std::memory_order_relaxed);
    return true;
  }
  void Clear() override {
    std::unique_lock<StripedSharedMutex> dl(dir_mu_);
    free_segments();
    reset_dir();
    slab_.reset();
    size_.store(0);
  }
  uint64_t Size() const override { return size_.load(); }
  std::string DebugInfo() const override {
    std::shared_lock<StripedSharedMutex> dl(dir_mu_);
    return "KVEngineExtendibleHash size=" + std::to_string(Size()) + " global_depth=" + std::to_string(global_depth_) +
           " segments=" + std::to_string(segments_.size());
  }
  size_t Keys(uint64_t* out, size_t cap) const override {
    std::shared_lock<StripedSharedMutex> dl(dir_mu_);
    size_t n = 0;
    for (Segment* s : segments_) {
      std::lock_guard<SpinLock> lk(s->mu);
      for (int i = 0; i < s->count && n < cap; ++i) out[n++] = s->keys[i];
    }
    return n;
  }
  // Invariant checker used by the tests: every key sits in the segment its hash selects, local
  // depths are consistent with the directory, the counts add up.
  bool CheckConsistency() const {
    std::shared_lock<StripedSharedMutex> dl(dir_mu_);
    uint64_t total = 0;
    for (size_t d = 0; d < dir_.size(); ++d) {
      Segment* s = dir_[d];
      if (s->local_depth > global_depth_) return false;
      const uint64_t lmask = (1ull << s->local_depth) - 1;
      for (int i = 0; i < s->count; ++i) {
        const uint64_t h = hash64(s->keys[i]);
        if ((h & lmask) != (d & lmask)) return false;
        if (s->tags[i] != tag_of(h)) return false;
      }
    }
    for (Segment* s : segments_) total += s->count;
    return total == size_.load();
  }

 private:
  void reset_dir() {
    global_depth_ = 4;
    dir_.assign(1u << global_depth_, nullptr);
    for (size_t i = 0; i < dir_.size(); ++i) {
      Segment* s = new Segment();
      s->local_depth = global_depth_;
      segments_.push_back(s);
      dir_[i] = s;
    }
  }
  void free_segments() {
    for (Segment* s : segments_) delete s;
    segments_.clear();
    dir_.clear();
  }
  void split(uint64_t h) {
    std::unique_lock<StripedSharedMutex> dl(dir_mu_);
    Segment* s = dir_[h & (dir_.size() - 1)];
    if (s->count < kSegCap) return;  // somebody else split it meanwhile
    if (s->local_depth == global_depth_) {
      const size_t old = dir_.size();
      dir_.resize(old * 2);
      for (size_t i = 0; i < old; ++i) dir_[old + i] = dir_[i];
      ++global_depth_;
    }
    Segment* n = new Segment();
    segments_.push_back(n);
    const int ld = s->local_depth;
    const uint64_t bit = 1ull << ld;
    s->local_depth = n->local_depth = ld + 1;
    int keep = 0;
    for (int i = 0; i < s->count; ++i) {
      if (hash64(s->keys[i]) & bit) {
        n->keys[n->count] = s->keys[i];
        n->tags[n->count] = s->tags[i];
        n->idx[n->count] = s->idx[i];
        ++n->count;
      } else {
        s->keys[keep] = s->keys[i];
        s->tags[keep] = s->tags[i];
        s->idx[keep] = s->idx[i];
        ++keep;
      }
    }
    s->count = keep;
    const uint64_t low = h & (bit - 1);
    for (size_t d = low; d < dir_.size(); d += bit)
      if (d & bit) dir_[d] = n;
  }

  mutable StripedSharedMutex dir_mu_;
  std::vector<Segment*> dir_;
  std::vector<Segment*> segments_;
  int global_depth_ = 0;
  SlabValueStore slab_;
  std::atomic<uint64_t> size_{0};
  bool ok_ = false;
};

// ============================================================== KVEngineChunkHash
class KVEngineChunkHash final : public BaseKV {
  static constexpr int kSlots = 14;
  struct alignas(8) Chunk {
    uint8_t tags[kSlots];     // 0 = empty, else 0x80 | top hash bits
    uint8_t overflow;         // keys whose home is this chunk but live further down (saturates at 255)
    uint8_t used;
    uint32_t idx[kSlots];
    uint64_t keys[kSlots];
  };
  struct Shard {
    mutable std::shared_mutex mu;
    Chunk* chunks = nullptr;
    uint64_t nchunks = 0;
    size_t map_bytes = 0;
    uint64_t max_probe = 0;   // largest distance from its home chunk at which any key was ever placed
  };
  struct Meta {          // first 4 KiB of every dict file
    uint64_t magic;
    uint64_t nchunks;
    uint32_t clean;      // 1 after a clean Flush(), 0 while the engine is open
  };
  static constexpr uint64_t kMagic = 0x5253423243484E4Bull;

 public:
  explicit KVEngineChunkHash(const KVConfig& c) : BaseKV(c) {
    nshards_ = std::max(1, c.num_shards);
    shards_ = std::vector<Shard>(nshards_);
    const uint64_t per_shard_keys = (c.capacity + nshards_ - 1) / nshards_;
    const uint64_t nchunks = std::max<uint64_t>(8, (per_shard_keys * 10 / 7 + kSlots - 1) / kSlots);  // load <= 0.7
    bool slab_existed = false;
    const std::string dir = c.path;
    if (!dir.empty()) mkdir(dir.c_str(), 0755);
    ok_ = slab_.open(dir.empty() ? "" : dir + "/values.slab", c.capacity, c.value_size, &slab_existed);
    bool all_existed = slab_existed;
    for (int s = 0; s < nshards_ && ok_; ++s) {
      bool ex = false;
      ok_ = map_shard(shards_[s], dir.empty() ? "" : dir + "/shard_" + std::to_string(s) + ".dict", nchunks, &ex);
      all_existed = all_existed && ex;
    }
    if (!ok_) return;
    if (!dir.empty() && all_existed) {
      recovered_ = true;
      Reload();
    } else {
      ClearLocked();
    }
    set_clean(0);
  }
  ~KVEngineChunkHash() override {
    Flush();
    for (Shard& s : shards_)
      if (s.chunks) munmap(reinterpret_cast<char*>(s.chunks) - 4096, s.map_bytes);
  }
  bool ok() const { return ok_; }
  bool Persistent() const override { return !cfg_.path.empty(); }
  bool recovered() const { return recovered_; }
  bool was_clean() const { return was_clean_; }

  bool Get(uint64_t key, void* out) override {
    const uint64_t h = hash64(key);
    Shard& s = shards_[h % nshards_];
    std::shared_lock<std::shared_mutex> lk(s.mu);
    uint64_t c;
    int slot;
    if (!find(s, key, h, &c, &slot)) return false;
    memcpy(out, slab_.at(s.chunks[c].idx[slot]), cfg_.value_size);
    return true;
  }
  bool Put(uint64_t key, const void* value) override {
    const uint64_t h = hash64(key);
    Shard& s = shards_[h % nshards_];
    std::unique_lock<std::shared_mutex> lk(s.mu);
    uint64_t c;
    int slot;
    if (find(s, key, h, &c, &slot)) {
      memcpy(slab_.at(s.chunks[c].idx[slot]), value, cfg_.value_size);
      return true;
    }
    const uint64_t home = (h >> 8) % s.nchunks;
    for (uint64_t p = 0; p < s.nchunks; ++p) {
      const uint64_t ci = (home + p) % s.nchunks;
      Chunk& ch = s.chunks[ci];
      if (ch.used < kSlots) {
        const uint32_t v = slab_.alloc();
        if (v == UINT32_MAX) return false;
        memcpy(slab_.at(v), value, cfg_.value_size);
        for (int i = 0; i < kSlots; ++i)
          if (ch.tags[i] == 0) {
            ch.keys[i] = key;
            ch.idx[i] = v;
            ch.tags[i] = tag_of(h);
            ++ch.used;
            break;
          }
        if (p != 0 && s.chunks[home].overflow < 255) ++s.chunks[home].overflow;
        if (p > s.max_probe) s.max_probe = p;
        size_.fetch_add(1, std::memory_order_relaxed);
        return true;
      }
    }
    return false;
  }
  bool Erase(uint64_t key) override {
    const uint64_t h = hash64(key);
    Shard& s = shards_[h % nshards_];
    std::unique_lock<std::shared_mutex> lk(s.mu);
    uint64_t c;
    int slot;
    if (!find(s, key, h, &c, &slot)) return false;
    Chunk& ch = s.chunks[c];
    slab_.release(ch.idx[slot]);
    ch.tags[slot] = 0;
    --ch.used;
    const uint64_t home = (h >> 8) % s.nchunks;
    if (c != home && s.chunks[home].overflow != 255 && s.chunks[home].overflow > 0) --s.chunks[home].overflow;
    size_.fetch_sub(1, std::memory_order_relaxed);
    return true;
  }
  void Clear() override {
    for (Shard& s : shards_) s.mu.lock();
    ClearLocked();
    for (Shard& s : shards_) s.mu.unlock();
  }
  uint64_t Size() const override { return size_.load(); }
  std::string DebugInfo() const override {
    uint64_t ov = 0, chunks = 0;
    for (const Shard& s : shards_) {
      std::shared_lock<std::shared_mutex> lk(s.mu);
      chunks += s.nchunks;
      for (uint64_t i = 0; i < s.nchunks; ++i) ov += s.chunks[i].overflow;
    }
    return "KVEngineChunkHash size=" + std::to_string(Size()) + " chunks=" + std::to_string(chunks) +
           " overflowed_keys=" + std::to_string(ov) + (recovered_ ? (was_clean_ ? " recovered(clean)" : " recovered(crash)") : "");
  }
  size_t Keys(uint64_t* out, size_t cap) const override {
    size_t n = 0;
    for (const Shard& s : shards_) {
      std::shared_lock<std::shared_mutex> lk(s.mu);
      for (uint64_t c = 0; c < s.nchunks; ++c)
        for (int i = 0; i < kSlots; ++i)
          if (s.chunks[c].tags[i] && n < cap) out[n++] = s.chunks[c].keys[i];
    }
    return n;
  }
  void Flush() override {
    if (cfg_.path.empty() || !ok_) return;
    slab_.sync();
    for (Shard& s : shards_) msync(reinterpret_cast<char*>(s.chunks) - 4096, s.map_bytes, MS_SYNC);
    set_clean(1);
  }

  // Moves each given key into its home chunk when that chunk has room (hot keys then cost one probe).
  size_t MigrateHot(const uint64_t* keys, size_t n) {
    size_t moved = 0;
    for (size_t k = 0; k < n; ++k) {
      const uint64_t h = hash64(keys[k]);
      Shard& s = shards_[h % nshards_];
      std::unique_lock<std::shared_mutex> lk(s.mu);
      uint64_t c;
      int slot;
      if (!find(s, keys[k], h, &c, &slot)) continue;
      const uint64_t home = (h >> 8) % s.nchunks;
      if (c == home) continue;
      Chunk& hc = s.chunks[home];
      if (hc.used >= kSlots) continue;
      Chunk& oc = s.chunks[c];
      for (int i = 0; i < kSlots; ++i)
        if (hc.tags[i] == 0) {
          hc.keys[i] = oc.keys[slot];
          hc.idx[i] = oc.idx[slot];
          hc.tags[i] = oc.tags[slot];
          ++hc.used;
          break;
        }
      oc.tags[slot] = 0;
      --oc.used;
      if (hc.overflow != 255 && hc.overflow > 0) --hc.overflow;
      ++moved;
    }
    return moved;
  }

  // Rebuilds everything that is derived (tags, used counts, overflow counters, size, slab free list)
  // from the keys and value indices found in the chunk files.  Slots whose value index is out of range
  // (torn write) are dropped.
  void Reload() {
    was_clean_ = true;
    for (Shard& s : shards_) was_clean_ = was_clean_ && meta(s)->clean == 1;
    std::vector<bool> live(slab_.high_water(), false);
    uint64_t total = 0;
    for (Shard& s : shards_) {
      s.max_probe = 0;
      for (uint64_t c = 0; c < s.nchunks; ++c) s.chunks[c].overflow = 0;
      for (uint64_t c = 0; c < s.nchunks; ++c) {
        Chunk& ch = s.chunks[c];
        int used = 0;
        for (int i = 0; i < kSlots; ++i) {
          if (ch.tags[i] == 0) continue;
          const uint64_t h = hash64(ch.keys[i]);
          if (ch.idx[i] >= live.size() || live[ch.idx[i]] || (h % nshards_) != static_cast<uint64_t>(&s - &shards_[0])) {
            ch.tags[i] = 0;
            continue;
          }
          live[ch.idx[i]] = true;
          ch.tags[i] = tag_of(h);
          ++used;
          const uint64_t home = (h >> 8) % s.nchunks;
          if (home != c && s.chunks[home].overflow < 255) ++s.chunks[home].overflow;
          s.max_probe = std::max<uint64_t>(s.max_probe, (c + s.nchunks - home) % s.nchunks);
        }
        ch.used = static_cast<uint8_t>(used);
        total += used;
      }
    }
    slab_.rebuild_free_list(live);
    size_.store(total);
  }

 private:
  static uint8_t tag_of(uint64_t h) { return static_cast<uint8_t>(0x80 | (h >> 57)); }
  Meta* meta(Shard& s) const { return reinterpret_cast<Meta*>(reinterpret_cast<char*>(s.chunks) - 4096); }
  void set_clean(uint32_t v) {
    if (cfg_.path.empty()) return;
    for (Shard& s : shards_) meta(s)->clean = v;
  }
  bool map_shard(Shard& s, const std::string& file, uint64_t nchunks, bool* existed) {
    s.nchunks = nchunks;
    s.map_bytes = 4096 + nchunks * sizeof(Chunk);
    void* base;
    *existed = false;
    if (file.empty()) {
      base = mmap(nullptr, s.map_bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
    } else {
      int fd = ::open(file.c_str(), O_RDWR | O_CREAT, 0644);
      if (fd < 0) return false;
      struct stat st;
      fstat(fd, &st);
      *existed = static_cast<size_t>(st.st_size) >= s.map_bytes;
      if (!*existed && ftruncate(fd, static_cast<off_t>(s.map_bytes)) != 0) { ::close(fd); return false; }
      base = mmap(nullptr, s.map_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
      ::close(fd);
    }
    if (base == MAP_FAILED) return false;
    Meta* m = static_cast<Meta*>(base);
    if (*existed && (m->magic != kMagic || m->nchunks != nchunks)) *existed = false;
    if (!*existed) {
      m->magic = kMagic;
      m->nchunks = nchunks;
      m->clean = 0;
    }
    s.chunks = reinterpret_cast<Chunk*>(static_cast<char*>(base) + 4096);
    return true;
  }
  void ClearLocked() {
    for (Shard& s : shards_) {
      memset(s.chunks, 0, s.nchunks * sizeof(Chunk));
      s.max_probe = 0;
    }
    slab_.reset();
    size_.store(0);
  }
  bool find(const Shard& s, uint64_t key, uint64_t h, uint64_t* chunk, int* slot) const {
    const uint64_t home = (h >> 8) % s.nchunks;
    const __m128i needle = _mm_set1_epi8(static_cast<char>(tag_of(h)));
    for (uint64_t p = 0; p < s.nchunks; ++p) {
      const uint64_t ci = (home + p) % s.nchunks;
      const Chunk& ch = s.chunks[ci];
      const __m128i tags = _mm_loadu_si128(reinterpret_cast<const __m128i*>(ch.tags));
      unsigned m = static_cast<unsigned>(_mm_movemask_epi8(_mm_cmpeq_epi8(tags, needle))) & ((1u << kSlots) - 1);
      while (m) {
        const int i = __builtin_ctz(m);
        if (ch.keys[i] == key) { *chunk = ci; *slot = i; return true; }
        m &= m - 1;
      }
      // Nothing of this home chunk lives further down unless its overflow counter says so, and
      // never further than the longest displacement any insert has used.
      if (p == 0 && ch.overflow == 0) return false;
      if (p >= s.max_probe) return false;
    }
    return false;
  }

  int nshards_ = 16;
  std::vector<Shard> shards_;
  SlabValueStore slab_;
  std::atomic<uint64_t> size_{0};
  bool ok_ = false, recovered_ = false, was_clean_ = false;
};

// ============================================================== factory
KVConfig ParseKVConfig(const std::string& json) {
  KVConfig c;
  JsonLite j(json);
  c.raw_json = json;
  c.path = j.str("path", "");
  // out-of-range numbers become 0 here and are refused by CreateKV, instead of wrapping around in the casts
  const long long cap = j.i64("capacity", 1 << 20), vs = j.i64("value_size", 128);
  c.capacity = (cap > 0 && cap <= (1ll << 40)) ? static_cast<uint64_t>(cap) : 0;
  c.value_size = (vs > 0 && vs <= (1ll << 24)) ? static_cast<uint32_t>(vs) : 0;
  c.num_threads = static_cast<int>(j.i64("num_threads", 8));
  c.num_shards = static_cast<int>(j.i64("num_shards", 64));   // ChunkHash: 8 writer threads, Zipf 0.99, 50 % puts: 4.9 / 10.3 / 14.2 M puts/s at 16 / 64 / 256 shards
  c.prefetch = j.i64("prefetch", 0) != 0;
  return c;
}

std::unique_ptr<BaseKV> CreatePoolMapKV(const KVConfig& cfg);                       // kv_engine_pool.cpp
bool PoolMapRecoveryState(BaseKV* kv, bool* recovered, uint64_t* dropped);

std::vector<std::string> ListKVEngines() {
  return {"KVEngineMap", "KVEngineExtendibleHash", "KVEngineChunkHash", "KVEnginePoolMap"};
}

std::unique_ptr<BaseKV> CreateKV(const std::string& engine, const KVConfig& cfg) {
  if (cfg.value_size == 0 || cfg.capacity == 0) {
    set_error(RS_ERR_INVALID, "KV engine needs 0 < capacity <= 2^40 and 0 < value_size <= 2^24");
    return nullptr;
  }
  if (engine == "KVEngineMap") {
    auto p = std::make_unique<KVEngineMap>(cfg);
    if (p->ok()) return p;
  } else if (engine == "KVEngineExtendibleHash") {
    auto p = std::make_unique<KVEngineExtendibleHash>(cfg);
    if (p->ok()) return p;
  } else if (engine == "KVEngineChunkHash" || engine == "KVEnginePetKV") {
    auto p = std::make_unique<KVEngineChunkHash>(cfg);
    if (p->ok()) return p;
  } else if (engine == "KVEnginePoolMap") {
    auto p = CreatePoolMapKV(cfg);
    if (p) return p;
  } else {
    set_error(RS_ERR_NOTFOUND, "unknown KV engine %s", engine.c_str());
    return nullptr;
  }
  set_error(RS_ERR_CAPACITY, "cannot allocate KV engine %s (capacity %llu x %u bytes)", engine.c_str(),
            static_cast<unsigned long long>(cfg.capacity), cfg.value_size);
  return nullptr;
}

}  // namespace rs

// ============================================================== C ABI
using rs::BaseKV;

RS_API int rs_kv_create(const char* engine, const char* json_config, void** out) {
  RS_REQUIRE(engine && out, "rs_kv_create: null argument");
  RS_NOEXCEPT_BODY(
    auto kv = rs::CreateKV(engine, rs::ParseKVConfig(json_config ? json_config : "{}"));
    if (!kv) return RS_ERR_INVALID;
    *out = kv.release();
    return RS_OK;
  )
}
RS_API int rs_kv_destroy(void* h) {
  delete static_cast<BaseKV*>(h);
  return RS_OK;
}
RS_API int rs_kv_value_size(void* h) { return static_cast<int>(static_cast<BaseKV*>(h)->value_size()); }
RS_API int rs_kv_put(void* h, unsigned long long key, const void* value) {
  return static_cast<BaseKV*>(h)->Put(key, value) ? RS_OK : rs::set_error(RS_ERR_CAPACITY, "KV engine is full");
}
// *found = 1/0
RS_API int rs_kv_get(void* h, unsigned long long key, void* out, int* found) {
  const bool ok = static_cast<BaseKV*>(h)->Get(key, out);
  if (found) *found = ok ? 1 : 0;
  return RS_OK;
}
RS_API int rs_kv_erase(void* h, unsigned long long key, int* erased) {
  const bool ok = static_cast<BaseKV*>(h)->Erase(key);
  if (erased) *erased = ok ? 1 : 0;
  return RS_OK;
}
RS_API int rs_kv_batch_get(void* h, const unsigned long long* keys, long long n, void* out, unsigned char* found) {
  static_cast<BaseKV*>(h)->BatchGet(reinterpret_cast<const uint64_t*>(keys), static_cast<size_t>(n), out, found);
  return RS_OK;
}
RS_API int rs_kv_batch_put(void* h, const unsigned long long* keys, long long n, const void* values, long long* stored) {
  const size_t s = static_cast<BaseKV*>(h)->BatchPut(reinterpret_cast<const uint64_t*>(keys), static_cast<size_t>(n), values);
  if (stored) *stored = static_cast<long long>(s);
  return s == static_cast<size_t>(n) ? RS_OK : rs::set_error(RS_ERR_CAPACITY, "KV engine is full: stored %zu of %lld", s, n);
}
RS_API int rs_kv_bulk_load(void* h, unsigned long long n) {
  RS_NOEXCEPT_BODY(static_cast<BaseKV*>(h)->BulkLoad(n); return RS_OK;)
}
RS_API int rs_kv_clear(void* h) {
  static_cast<BaseKV*>(h)->Clear();
  return RS_OK;
}
RS_API unsigned long long rs_kv_size(void* h) { return static_cast<BaseKV*>(h)->Size(); }
RS_API int rs_kv_flush(void* h) {
  static_cast<BaseKV*>(h)->Flush();
  return RS_OK;
}
RS_API long long rs_kv_keys(void* h, unsigned long long* out, long long cap) {
  return static_cast<long long>(static_cast<BaseKV*>(h)->Keys(reinterpret_cast<uint64_t*>(out), static_cast<size_t>(cap)));
}
RS_API int rs_kv_debug_info(void* h, char* buf, int cap) {
  const std::string s = static_cast<BaseKV*>(h)->DebugInfo();
  if (buf && cap > 0) {
    const int n = std::min<int>(cap - 1, static_cast<int>(s.size()));
    memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return static_cast<int>(s.size());
}
// Engine-specific extras; return RS_ERR_STATE when the engine does not support them.
RS_API int rs_kv_check_consistency(void* h, int* ok) {
  if (auto* e = dynamic_cast<rs::KVEngineExtendibleHash*>(static_cast<BaseKV*>(h))) {
    *ok = e->CheckConsistency() ? 1 : 0;
    return RS_OK;
  }
  return rs::set_error(RS_ERR_STATE, "engine has no consistency checker");
}
RS_API int rs_kv_migrate_hot(void* h, const unsigned long long* keys, long long n, long long* moved) {
  if (auto* e = dynamic_cast<rs::KVEngineChunkHash*>(static_cast<BaseKV*>(h))) {
    *moved = static_cast<long long>(e->MigrateHot(reinterpret_cast<const uint64_t*>(keys), static_cast<size_t>(n)));
    return RS_OK;
  }
  return rs::set_error(RS_ERR_STATE, "engine has no hot-key migration");
}
// recovered: opened existing files; clean: they were closed by Flush (else a crash was recovered).
RS_API int rs_kv_recovery_state(void* h, int* recovered, int* clean) {
  if (auto* e = dynamic_cast<rs::KVEngineChunkHash*>(static_cast<BaseKV*>(h))) {
    *recovered = e->recovered() ? 1 : 0;
    *clean = e->was_clean() ? 1 : 0;
    return RS_OK;
  }
  bool rec = false;
  uint64_t dropped = 0;
  if (rs::PoolMapRecoveryState(static_cast<BaseKV*>(h), &rec, &dropped)) {   // clean: nothing had to be dropped
    *recovered = rec ? 1 : 0;
    *clean = (rec && dropped == 0) ? 1 : 0;
    return RS_OK;
  }
  *recovered = 0;
  *clean = 0;
  return RS_OK;
}
// Warm-up of one PS shard and its check (role of LoadDBHelper, src/storage/kv_engine/load_db.h:13-165): of the keys
// 1 ... warm_capacity, those whose partition hash(key) % num_servers equals server_id get the value float(key) repeated,
// written by `threads` threads over contiguous key ranges (or, with shuffle, by one thread in a scattered order, which
// is what an engine sees when keys arrive unsorted).  *inserted = keys stored; a full engine is an error.
RS_API int rs_kv_preload(void* h, int server_id, int num_servers, unsigned long long warm_capacity, int threads, int shuffle,
                         unsigned long long* inserted) {
  RS_REQUIRE(h && num_servers > 0 && server_id >= 0 && server_id < num_servers && threads > 0, "rs_kv_preload: bad argument");
  RS_NOEXCEPT_BODY(
    auto* kv = static_cast<BaseKV*>(h);
    const size_t nfloat = kv->value_size() / sizeof(float);
    std::atomic<uint64_t> stored{0}, refused{0};
    auto put_range = [&](uint64_t lo, uint64_t hi, uint64_t stride, uint64_t first) {
      std::vector<char> value(kv->value_size(), 0);
      float* emb = reinterpret_cast<float*>(value.data());
      uint64_t ok = 0, bad = 0;
      for (uint64_t j = lo + first; j < hi; j += stride) {
        if (rs::hash64(j) % static_cast<uint64_t>(num_servers) != static_cast<uint64_t>(server_id)) continue;
        for (size_t k = 0; k < nfloat; ++k) emb[k] = static_cast<float>(j);
        (kv->Put(j, value.data()) ? ok : bad)++;
      }
      stored += ok;
      refused += bad;
    };
    const uint64_t start = 1, end = warm_capacity + 1;
    if (shuffle) {
      // a fixed odd stride walks the range in kStride interleaved passes: deterministic, and far from sorted
      constexpr uint64_t kStride = 9973;
      for (uint64_t first = 0; first < kStride && first < warm_capacity; ++first) put_range(start, end, kStride, first);
    } else {
      const uint64_t per = (warm_capacity + threads - 1) / threads;
      std::vector<std::thread> th;
      for (int i = 0; i < threads; ++i)
        th.emplace_back(put_range, start + i * per, std::min(end, start + (i + 1) * per), uint64_t{1}, uint64_t{0});
      for (auto& t : th) t.join();
    }
    if (inserted) *inserted = stored.load();
    if (refused.load())
      return rs::set_error(RS_ERR_CAPACITY, "preload: the engine refused %llu of %llu keys",
                           static_cast<unsigned long long>(refused.load()),
                           static_cast<unsigned long long>(refused.load() + stored.load()));
    return RS_OK;
  )
}
// *right = keys of this shard whose every float equals the key; *expected = keys of this shard in 1 ... warm_capacity.
RS_API int rs_kv_check_preload(void* h, int server_id, int num_servers, unsigned long long warm_capacity, int threads,
                               unsigned long long* right, unsigned long long* expected) {
  RS_REQUIRE(h && num_servers > 0 && server_id >= 0 && server_id < num_servers && threads > 0, "rs_kv_check_preload: bad argument");
  RS_NOEXCEPT_BODY(
    auto* kv = static_cast<BaseKV*>(h);
    const size_t nfloat = kv->value_size() / sizeof(float);
    std::atomic<uint64_t> good{0}, mine{0};
    const uint64_t start = 1, end = warm_capacity + 1, per = (warm_capacity + threads - 1) / threads;
    std::vector<std::thread> th;
    for (int i = 0; i < threads; ++i)
      th.emplace_back([&, i] {
        std::vector<char> value(kv->value_size());
        const float* emb = reinterpret_cast<const float*>(value.data());
        uint64_t ok = 0, n = 0;
        for (uint64_t j = start + i * per; j < std::min(end, start + (i + 1) * per); ++j) {
          if (rs::hash64(j) % static_cast<uint64_t>(num_servers) != static_cast<uint64_t>(server_id)) continue;
          ++n;
          if (!kv->Get(j, value.data())) continue;
          bool same = true;
          for (size_t k = 0; k < nfloat; ++k) same &= emb[k] == static_cast<float>(j);
          ok += same;
        }
        good += ok;
        mine += n;
      });
    for (auto& t : th) t.join();
    if (right) *right = good.load();
    if (expected) *expected = mine.load();
    return RS_OK;
  )
}
RS_API int rs_kv_list_engines(char* buf, int cap) {
  std::string s;
  for (auto& e : rs::ListKVEngines()) s += e + "\n";
  if (buf && cap > 0) {
    const int n = std::min<int>(cap - 1, static_cast<int>(s.size()));
    memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return static_cast<int>(s.size());
}
