// Sub-allocators over large slabs of device (or pinned / pageable host) memory, so that hot paths never call
// cudaMalloc: a coalescing best-fit pool, a binning front end with power-of-two size classes, and a fixed-length
// block allocator.  Role of the reference's RMM-based pool / binning / fixed-length resources
// (src/gpu_memory/memory_pool.h:23-81); written against the CUDA runtime only.
//
// All three are thread-safe (one mutex each; allocation is off the kernel-launch critical path by design) and
// return 256-byte aligned addresses.  Slabs are allocated lazily, doubled up to `max_bytes`, and only released
// when the allocator is destroyed.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <map>
#include <set>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common/rs_common.h"

namespace {

constexpr size_t kAlign = 256;
inline size_t round_up(size_t n, size_t a) { return (n + a - 1) / a * a; }

enum Backing { kDevice = 0, kPinnedHost = 1, kPageableHost = 2 };

struct Slabs {
  int backing;
  std::vector<std::pair<char*, size_t>> slabs;
  size_t total = 0;
  explicit Slabs(int b) : backing(b) {}
  ~Slabs() {
    for (auto& s : slabs) {
      if (backing == kDevice) cudaFree(s.first);
      else if (backing == kPinnedHost) cudaFreeHost(s.first);
      else free(s.first);
    }
  }
  char* grow(size_t bytes) {
    void* p = nullptr;
    if (backing == kDevice) { if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; } }
    else if (backing == kPinnedHost) { if (cudaMallocHost(&p, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; } }
    else { if (posix_memalign(&p, kAlign, bytes) != 0) return nullptr; }
    slabs.emplace_back(static_cast<char*>(p), bytes);
    total += bytes;
    return static_cast<char*>(p);
  }
};

class Allocator {
 public:
  virtual ~Allocator() = default;
  virtual void* alloc(size_t bytes) = 0;
  virtual bool release(void* p) = 0;
  virtual void stats(unsigned long long* out) = 0;   // reserved, in use, live blocks, slabs, peak in use, failures
};

// Address-ordered free map with coalescing, best fit by size.
class PoolAllocator : public Allocator {
 public:
  PoolAllocator(int backing, size_t initial, size_t max_bytes) : slabs_(backing), next_grow_(round_up(std::max(initial, kAlign), kAlign)), max_(max_bytes) {}
  void* alloc(size_t bytes) override {
    if (bytes == 0) bytes = 1;
    bytes = round_up(bytes, kAlign);
    std::lock_guard<std::mutex> lk(mu_);
    auto it = by_size_.lower_bound({bytes, nullptr});
    if (it == by_size_.end()) {
      size_t want = std::max(bytes, next_grow_);
      if (slabs_.total + want > max_) want = bytes;
      if (slabs_.total + want > max_) { ++failures_; return nullptr; }
      char* s = slabs_.grow(want);
      if (!s) { ++failures_; return nullptr; }
      next_grow_ = std::min(next_grow_ * 2, std::max(max_ / 4, kAlign));
      insert_free(s, want);
      it = by_size_.lower_bound({bytes, nullptr});
    }
    char* p = it->second;
    const size_t have = it->first;
    erase_free(p, have);
    if (have > bytes) insert_free(p + bytes, have - bytes);
    live_[p] = bytes;
    in_use_ += bytes;
    peak_ = std::max(peak_, in_use_);
    return p;
  }
  bool release(void* ptr) override {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = live_.find(static_cast<char*>(ptr));
    if (it == live_.end()) return false;
    char* p = it->first;
    size_t n = it->second;
    live_.erase(it);
    in_use_ -= n;
    // merge with the free neighbours (never across slabs: a slab boundary is never adjacent in by_addr_ keys unless
    // the driver returned contiguous slabs, in which case merging is still sound for sub-allocation)
    auto nx = by_addr_.lower_bound(p);
    if (nx != by_addr_.end() && p + n == nx->first && same_slab(p, nx->first)) {
      n += nx->second;
      erase_free(nx->first, nx->second);
    }
    auto pv = by_addr_.lower_bound(p);
    if (pv != by_addr_.begin()) {
      --pv;
      if (pv->first + pv->second == p && same_slab(pv->first, p)) {
        p = pv->first;
        n += pv->second;
        erase_free(pv->first, pv->second);
      }
    }
    insert_free(p, n);
    return true;
  }
  void stats(unsigned long long* o) override {
    std::lock_guard<std::mutex> lk(mu_);
    o[0] = slabs_.total; o[1] = in_use_; o[2] = live_.size(); o[3] = slabs_.slabs.size(); o[4] = peak_; o[5] = failures_;
  }

 private:
  bool same_slab(char* a, char* b) const {
    for (auto& s : slabs_.slabs)
      if (a >= s.first && a < s.first + s.second) return b >= s.first && b < s.first + s.second;
    return false;
  }
  void insert_free(char* p, size_t n) { by_addr_[p] = n; by_size_.insert({n, p}); }
  void erase_free(char* p, size_t n) { by_addr_.erase(p); by_size_.erase({n, p}); }
  Slabs slabs_;
  std::mutex mu_;
  std::map<char*, size_t> by_addr_;
  std::set<std::pair<size_t, char*>> by_size_;
  std::unordered_map<char*, size_t> live_;
  size_t next_grow_, max_, in_use_ = 0, peak_ = 0, failures_ = 0;
};

// Blocks of one size: a stack of free blocks carved from slabs of `blocks_per_slab` blocks.
class FixedAllocator : public Allocator {
 public:
  FixedAllocator(int backing, size_t block, size_t initial, size_t max_bytes)
      : slabs_(backing), block_(round_up(std::max(block, size_t{1}), kAlign)), max_(max_bytes),
        per_slab_(std::max<size_t>(1, std::max(initial, block_) / block_)) {}
  void* alloc(size_t bytes) override {
    std::lock_guard<std::mutex> lk(mu_);
    if (bytes > block_) { ++failures_; return nullptr; }
    if (free_.empty()) {
      const size_t want = per_slab_ * block_;
      if (slabs_.total + want > max_) { ++failures_; return nullptr; }
      char* s = slabs_.grow(want);
      if (!s) { ++failures_; return nullptr; }
      for (size_t i = per_slab_; i-- > 0;) free_.push_back(s + i * block_);
    }
    char* p = free_.back();
    free_.pop_back();
    ++live_;
    peak_ = std::max(peak_, live_ * block_);
    return p;
  }
  bool release(void* p) override {
    std::lock_guard<std::mutex> lk(mu_);
    bool ours = false;
    for (auto& s : slabs_.slabs)
      if (static_cast<char*>(p) >= s.first && static_cast<char*>(p) < s.first + s.second && (static_cast<char*>(p) - s.first) % block_ == 0) ours = true;
    if (!ours || live_ == 0) return false;
    free_.push_back(static_cast<char*>(p));
    --live_;
    return true;
  }
  void stats(unsigned long long* o) override {
    std::lock_guard<std::mutex> lk(mu_);
    o[0] = slabs_.total; o[1] = live_ * block_; o[2] = live_; o[3] = slabs_.slabs.size(); o[4] = peak_; o[5] = failures_;
  }
  size_t block() const { return block_; }

 private:
  Slabs slabs_;
  std::mutex mu_;
  std::vector<char*> free_;
  size_t block_, max_, per_slab_, live_ = 0, peak_ = 0, failures_ = 0;
};

// Power-of-two size classes from 256 B to `max_bin`, each a FixedAllocator; anything larger goes to a pool.
class BinningAllocator : public Allocator {
 public:
  BinningAllocator(int backing, size_t initial, size_t max_bytes, size_t max_bin) : big_(backing, initial, max_bytes) {
    for (size_t b = kAlign; b <= std::max(max_bin, kAlign); b *= 2)
      bins_.emplace_back(new FixedAllocator(backing, b, std::max<size_t>(b * 64, 1 << 20), max_bytes));
  }
  void* alloc(size_t bytes) override {
    for (size_t i = 0; i < bins_.size(); ++i) {
      if (bytes <= bins_[i]->block()) {
        void* p = bins_[i]->alloc(bytes);
        if (p) { std::lock_guard<std::mutex> lk(mu_); owner_[p] = static_cast<int>(i); }
        return p;
      }
    }
    void* p = big_.alloc(bytes);
    if (p) { std::lock_guard<std::mutex> lk(mu_); owner_[p] = -1; }
    return p;
  }
  bool release(void* p) override {
    int o;
    {
      std::lock_guard<std::mutex> lk(mu_);
      auto it = owner_.find(p);
      if (it == owner_.end()) return false;
      o = it->second;
      owner_.erase(it);
    }
    return o < 0 ? big_.release(p) : bins_[o]->release(p);
  }
  void stats(unsigned long long* o) override {
    unsigned long long t[6];
    big_.stats(o);
    for (auto& b : bins_) {
      b->stats(t);
      for (int i = 0; i < 6; ++i) o[i] += t[i];
    }
  }

 private:
  PoolAllocator big_;
  std::vector<std::unique_ptr<FixedAllocator>> bins_;
  std::mutex mu_;
  std::unordered_map<void*, int> owner_;
};

}  // namespace

// kind: 0 = pool, 1 = binning (param = largest bin in bytes), 2 = fixed length (param = block bytes).
// backing: 0 = device memory of the current device, 1 = pinned host, 2 = pageable host.
RS_API int rs_devpool_create(int kind, int backing, size_t initial_bytes, size_t max_bytes, size_t param, void** out) {
  RS_REQUIRE(out && kind >= 0 && kind <= 2 && backing >= 0 && backing <= 2, "rs_devpool_create: bad kind / backing");
  RS_REQUIRE(max_bytes >= kAlign && initial_bytes <= max_bytes, "rs_devpool_create: initial size exceeds the maximum");
  if (kind == 0) *out = new PoolAllocator(backing, initial_bytes, max_bytes);
  else if (kind == 1) *out = new BinningAllocator(backing, initial_bytes, max_bytes, param ? param : (size_t{4} << 20));
  else { RS_REQUIRE(param > 0, "rs_devpool_create: fixed-length allocator needs a block size"); *out = new FixedAllocator(backing, param, initial_bytes, max_bytes); }
  return RS_OK;
}
RS_API int rs_devpool_destroy(void* h) {
  delete static_cast<Allocator*>(h);
  return RS_OK;
}
RS_API int rs_devpool_alloc(void* h, size_t bytes, void** out) {
  RS_REQUIRE(h && out, "rs_devpool_alloc: null argument");
  *out = nullptr;
  if (bytes > (size_t{1} << 48))      // rounding such a size up to the block granularity would wrap around
    return rs::set_error(RS_ERR_CAPACITY, "rs_devpool_alloc: %zu bytes do not fit (limit reached or block too large)", bytes);
  *out = static_cast<Allocator*>(h)->alloc(bytes);
  if (*out == nullptr) return rs::set_error(RS_ERR_CAPACITY, "rs_devpool_alloc: %zu bytes do not fit (limit reached or block too large)", bytes);
  return RS_OK;
}
RS_API int rs_devpool_free(void* h, void* p) {
  RS_REQUIRE(h, "rs_devpool_free: null allocator");
  if (p == nullptr) return RS_OK;
  if (!static_cast<Allocator*>(h)->release(p)) return rs::set_error(RS_ERR_INVALID, "rs_devpool_free: pointer was not allocated here (or freed twice)");
  return RS_OK;
}
RS_API int rs_devpool_stats(void* h, unsigned long long* out6) {
  RS_REQUIRE(h && out6, "rs_devpool_stats: null argument");
  static_cast<Allocator*>(h)->stats(out6);
  return RS_OK;
}
