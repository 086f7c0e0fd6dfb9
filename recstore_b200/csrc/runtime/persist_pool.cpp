#include "runtime/persist_pool.h"

#include <algorithm>
#include <chrono>
#include <cstring>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "common/rs_common.h"

namespace rs {

namespace {
inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }
inline int floor_log2(uint64_t v) { return 63 - __builtin_clzll(v); }
}  // namespace

// ============================================================== PersistSlabPool
uint64_t PersistSlabPool::ClassSize(uint64_t size) {
  if (size <= 16) return 16;
  if (size <= 256) return align_up(size, 16);
  const int e = floor_log2(size - 1);            // size in (2^e, 2^(e+1)]
  const uint64_t step = 1ull << (e - 2);
  return align_up(size, step);
}

int PersistSlabPool::class_index(uint64_t c) {
  if (c <= 256) return static_cast<int>(c / 16) - 1;
  const int e = floor_log2(c - 1);
  const uint64_t step = 1ull << (e - 2);
  const int q = static_cast<int>((c - (1ull << e)) / step) - 1;
  return 16 + (e - 8) * 4 + q;
}

std::unique_ptr<PersistSlabPool> PersistSlabPool::Open(const std::string& path, uint64_t bytes, uint64_t chunk_bytes,
                                                       bool* recovered) {
  if (recovered) *recovered = false;
  if (chunk_bytes < 4096 || (chunk_bytes & (chunk_bytes - 1)) != 0 || bytes < chunk_bytes) {
    set_error(RS_ERR_INVALID, "slab pool: chunk_bytes must be a power of two >= 4096 and <= bytes");
    return nullptr;
  }
  std::unique_ptr<PersistSlabPool> p(new PersistSlabPool());
  p->chunk_bytes_ = chunk_bytes;
  p->n_chunks_ = bytes / chunk_bytes;
  p->map_bytes_ = kSuper + p->n_chunks_ * chunk_bytes;
  bool existed = false;
  void* m;
  if (path.empty()) {
    m = mmap(nullptr, p->map_bytes_, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  } else {
    const int fd = ::open(path.c_str(), O_RDWR | O_CREAT, 0644);
    if (fd < 0) {
      set_error(RS_ERR_IO, "slab pool: cannot open %s", path.c_str());
      return nullptr;
    }
    struct stat st;
    fstat(fd, &st);
    existed = static_cast<uint64_t>(st.st_size) >= p->map_bytes_;
    if (!existed && ftruncate(fd, static_cast<off_t>(p->map_bytes_)) != 0) {
      ::close(fd);
      set_error(RS_ERR_IO, "slab pool: cannot size %s to %llu bytes", path.c_str(), static_cast<unsigned long long>(p->map_bytes_));
      return nullptr;
    }
    m = mmap(nullptr, p->map_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    p->file_backed_ = true;
  }
  if (m == MAP_FAILED) {
    set_error(RS_ERR_CAPACITY, "slab pool: cannot map %llu bytes", static_cast<unsigned long long>(p->map_bytes_));
    return nullptr;
  }
  p->base_ = static_cast<char*>(m);
  auto* sb = reinterpret_cast<SuperBlock*>(p->base_);
  if (existed && (sb->magic != kMagic || sb->chunk_bytes != chunk_bytes || sb->n_chunks != p->n_chunks_)) existed = false;
  p->classes_.resize(200);
  for (auto& c : p->classes_) c = std::make_unique<ClassState>();
  p->used_in_chunk_ = std::vector<std::atomic<uint32_t>>(p->n_chunks_);
  p->scan_hint_.assign(p->n_chunks_, 0);
  if (!existed) {
    for (uint64_t c = 0; c < p->n_chunks_; ++c) {
      ChunkHeader* h = p->chunk(c);
      h->slab_size.store(0, std::memory_order_relaxed);
      h->magic = kChunkMagic;
    }
    sb->bytes = p->map_bytes_;
    sb->chunk_bytes = chunk_bytes;
    sb->n_chunks = p->n_chunks_;
    std::atomic_thread_fence(std::memory_order_release);
    sb->magic = kMagic;
  }
  p->rebuild_volatile();
  if (recovered) *recovered = existed;
  return p;
}

PersistSlabPool::~PersistSlabPool() {
  if (base_) {
    if (file_backed_) msync(base_, map_bytes_, MS_SYNC);
    munmap(base_, map_bytes_);
  }
}

void PersistSlabPool::rebuild_volatile() {
  std::lock_guard<SpinLock> fl(free_mu_);
  free_chunks_.clear();
  for (auto& c : classes_) c->partial.clear();
  uint64_t slabs = 0, bytes = 0;
  for (uint64_t c = n_chunks_; c-- > 0;) {                 // descending, so chunk 0 is handed out first
    ChunkHeader* h = chunk(c);
    const uint64_t cs = h->slab_size.load(std::memory_order_acquire);
    uint32_t used = 0;
    const bool sane = h->magic == kChunkMagic && cs != 0 && cs == ClassSize(cs) && h->n_slabs > 0 &&
                      h->first_slab + h->n_slabs * cs <= chunk_bytes_;
    if (sane) {
      const uint64_t words = (h->n_slabs + 63) / 64;
      for (uint64_t w = 0; w < words; ++w) used += static_cast<uint32_t>(__builtin_popcountll(bitmap(h)[w].load(std::memory_order_relaxed)));
    }
    used_in_chunk_[c].store(used, std::memory_order_relaxed);
    if (!sane || used == 0) {
      h->magic = kChunkMagic;
      h->slab_size.store(0, std::memory_order_relaxed);
      free_chunks_.push_back(static_cast<uint32_t>(c));
    } else {
      slabs += used;
      bytes += used * cs;
      if (used < h->n_slabs) classes_[class_index(cs)]->partial.push_back(static_cast<uint32_t>(c));
    }
  }
  slabs_in_use_.store(slabs);
  bytes_in_use_.store(bytes);
}

bool PersistSlabPool::format_chunk(uint64_t c, uint64_t cs) {
  ChunkHeader* h = chunk(c);
  uint64_t n = (chunk_bytes_ - sizeof(ChunkHeader)) / cs;
  uint64_t first = 0;
  while (n > 0) {
    first = align_up(sizeof(ChunkHeader) + (n + 63) / 64 * 8, 64);
    if (first + n * cs <= chunk_bytes_) break;
    --n;
  }
  if (n == 0) return false;
  const uint64_t words = (n + 63) / 64;
  for (uint64_t w = 0; w < words; ++w) bitmap(h)[w].store(0, std::memory_order_relaxed);
  h->n_slabs = n;
  h->first_slab = first;
  h->magic = kChunkMagic;
  h->slab_size.store(cs, std::memory_order_release);        // the chunk counts as formatted from here on
  used_in_chunk_[c].store(0, std::memory_order_relaxed);
  scan_hint_[c] = 0;
  return true;
}

// Caller holds the class lock.
uint64_t PersistSlabPool::alloc_in_chunk(uint64_t c) {
  ChunkHeader* h = chunk(c);
  const uint64_t n = h->n_slabs, words = (n + 63) / 64;
  std::atomic<uint64_t>* bm = bitmap(h);
  const uint64_t start = scan_hint_[c] < words ? scan_hint_[c] : 0;
  for (uint64_t k = 0; k < words; ++k) {
    const uint64_t w = start + k < words ? start + k : start + k - words;
    const uint64_t v = bm[w].load(std::memory_order_relaxed);
    if (~v == 0) continue;
    const int bit = __builtin_ctzll(~v);
    const uint64_t idx = w * 64 + bit;
    if (idx >= n) continue;                                  // padding bits of the last word
    bm[w].fetch_or(1ull << bit, std::memory_order_acq_rel);
    used_in_chunk_[c].fetch_add(1, std::memory_order_relaxed);
    scan_hint_[c] = static_cast<uint32_t>(w);
    return kSuper + c * chunk_bytes_ + h->first_slab + idx * h->slab_size.load(std::memory_order_relaxed);
  }
  return 0;
}

uint64_t PersistSlabPool::Malloc(uint64_t size) {
  uint64_t off = 0;
  return MallocBatch(size, &off, 1) == 1 ? off : 0;
}

size_t PersistSlabPool::MallocBatch(uint64_t size, uint64_t* out, size_t n) {
  if (size == 0) size = 1;
  const uint64_t cs = ClassSize(size);
  if (cs + 128 > chunk_bytes_) return 0;
  ClassState& st = *classes_[class_index(cs)];
  std::lock_guard<SpinLock> lk(st.mu);
  size_t got = 0;
  while (got < n) {
    while (got < n && !st.partial.empty()) {
      const uint64_t off = alloc_in_chunk(st.partial.back());
      if (off) out[got++] = off;
      else st.partial.pop_back();                            // full: a Free puts it back
    }
    if (got == n) break;
    uint32_t c;
    {
      std::lock_guard<SpinLock> fl(free_mu_);
      if (free_chunks_.empty()) break;
      c = free_chunks_.back();
      free_chunks_.pop_back();
    }
    if (!format_chunk(c, cs)) {
      std::lock_guard<SpinLock> fl(free_mu_);
      free_chunks_.push_back(c);
      break;
    }
    st.partial.push_back(c);
  }
  slabs_in_use_.fetch_add(got, std::memory_order_relaxed);
  bytes_in_use_.fetch_add(got * cs, std::memory_order_relaxed);
  return got;
}

uint64_t PersistSlabPool::SlabSize(uint64_t off) const {
  if (off < kSuper || off >= map_bytes_) return 0;
  const uint64_t c = (off - kSuper) / chunk_bytes_;
  ChunkHeader* h = chunk(c);
  const uint64_t cs = h->slab_size.load(std::memory_order_acquire);
  const uint64_t in = off - kSuper - c * chunk_bytes_;
  if (cs == 0 || in < h->first_slab || (in - h->first_slab) % cs != 0) return 0;
  const uint64_t idx = (in - h->first_slab) / cs;
  if (idx >= h->n_slabs) return 0;
  return (bitmap(h)[idx / 64].load(std::memory_order_acquire) >> (idx % 64)) & 1 ? cs : 0;
}

void PersistSlabPool::Free(uint64_t off) {
  if (off < kSuper || off >= map_bytes_) return;
  const uint64_t c = (off - kSuper) / chunk_bytes_;
  ChunkHeader* h = chunk(c);
  const uint64_t cs = h->slab_size.load(std::memory_order_acquire);
  const uint64_t in = off - kSuper - c * chunk_bytes_;
  if (cs == 0 || in < h->first_slab || (in - h->first_slab) % cs != 0) return;
  const uint64_t idx = (in - h->first_slab) / cs;
  if (idx >= h->n_slabs) return;
  const uint64_t bit = 1ull << (idx % 64);
  const uint64_t prev = bitmap(h)[idx / 64].fetch_and(~bit, std::memory_order_acq_rel);
  if (!(prev & bit)) return;                                 // was not allocated (double free): nothing to do
  slabs_in_use_.fetch_sub(1, std::memory_order_relaxed);
  bytes_in_use_.fetch_sub(cs, std::memory_order_relaxed);
  const uint32_t before = used_in_chunk_[c].fetch_sub(1, std::memory_order_acq_rel);
  if (before != h->n_slabs && before != 1) return;
  // The chunk was full (it may have left its class queue) or has become empty (it goes back to the free chunks).
  ClassState& st = *classes_[class_index(cs)];
  std::lock_guard<SpinLock> lk(st.mu);
  if (h->slab_size.load(std::memory_order_relaxed) != cs) return;   // re-formatted meanwhile
  auto it = std::find(st.partial.begin(), st.partial.end(), static_cast<uint32_t>(c));
  if (used_in_chunk_[c].load(std::memory_order_acquire) == 0) {
    if (it != st.partial.end()) st.partial.erase(it);
    h->slab_size.store(0, std::memory_order_release);
    std::lock_guard<SpinLock> fl(free_mu_);
    free_chunks_.push_back(static_cast<uint32_t>(c));
  } else if (it == st.partial.end()) {
    st.partial.push_back(static_cast<uint32_t>(c));
  }
}

void PersistSlabPool::ForEachAllocated(const std::function<void(uint64_t, uint64_t)>& fn) const {
  for (uint64_t c = 0; c < n_chunks_; ++c) {
    ChunkHeader* h = chunk(c);
    const uint64_t cs = h->slab_size.load(std::memory_order_acquire);
    if (cs == 0) continue;
    const uint64_t n = h->n_slabs, words = (n + 63) / 64;
    for (uint64_t w = 0; w < words; ++w) {
      uint64_t v = bitmap(h)[w].load(std::memory_order_acquire);
      while (v) {
        const int bit = __builtin_ctzll(v);
        v &= v - 1;
        const uint64_t idx = w * 64 + bit;
        if (idx < n) fn(kSuper + c * chunk_bytes_ + h->first_slab + idx * cs, cs);
      }
    }
  }
}

PersistSlabPool::Stats PersistSlabPool::GetStats() const {
  Stats s{};
  s.chunk_bytes = chunk_bytes_;
  s.chunks_total = n_chunks_;
  {
    std::lock_guard<SpinLock> fl(free_mu_);
    s.chunks_in_use = n_chunks_ - free_chunks_.size();
  }
  s.slabs_in_use = slabs_in_use_.load();
  s.bytes_in_use = bytes_in_use_.load();
  s.bytes_reserved = s.chunks_in_use * chunk_bytes_;
  return s;
}

void PersistSlabPool::Sync() {
  if (base_ && file_backed_) msync(base_, map_bytes_, MS_SYNC);
}

void PersistSlabPool::Reset() {
  for (auto& c : classes_) c->mu.lock();
  for (uint64_t c = 0; c < n_chunks_; ++c) chunk(c)->slab_size.store(0, std::memory_order_release);
  rebuild_volatile();
  for (auto& c : classes_) c->mu.unlock();
}

// ============================================================== EpochManager
namespace {
std::atomic<uint64_t> g_thread_tokens{0};
std::atomic<uint64_t> g_manager_ids{0};
struct ThreadSlots {
  struct Held {
    uint64_t manager;
    std::shared_ptr<void> keep;            // keeps the slot array alive past the manager
    std::shared_ptr<std::atomic<bool>> alive;   // cleared by the manager's destructor
    std::atomic<uint64_t>* owner;
    void* slot;
  };
  uint64_t token = g_thread_tokens.fetch_add(1) + 1;
  std::vector<Held> held;
  ~ThreadSlots() {
    for (auto& h : held) h.owner->store(0, std::memory_order_release);
  }
};
thread_local ThreadSlots t_slots;
}  // namespace

EpochManager::EpochManager()
    : slots_(new Slot[kSlots]), stripes_(new Stripe[kStripes]), alive_(std::make_shared<std::atomic<bool>>(true)),
      id_(g_manager_ids.fetch_add(1) + 1) {}

EpochManager::~EpochManager() { alive_->store(false, std::memory_order_release); }

EpochManager::Slot* EpochManager::my_slot() {
  for (auto& h : t_slots.held)
    if (h.manager == id_) return static_cast<Slot*>(h.slot);
  // First use by this thread: entries of managers that have gone are dropped (with their share of the slot arrays),
  // then a free slot is claimed.
  auto& held = t_slots.held;
  held.erase(std::remove_if(held.begin(), held.end(), [](const ThreadSlots::Held& h) { return !h.alive->load(std::memory_order_acquire); }),
             held.end());
  for (int round = 0; round < 1 << 20; ++round) {
    for (int i = 0; i < kSlots; ++i) {
      uint64_t expect = 0;
      if (slots_[i].owner.compare_exchange_strong(expect, t_slots.token, std::memory_order_acq_rel)) {
        slots_[i].depth = 0;
        t_slots.held.push_back({id_, std::shared_ptr<void>(slots_, slots_.get()), alive_, &slots_[i].owner, &slots_[i]});
        return &slots_[i];
      }
    }
    cpu_relax();                           // more threads than slots: wait for one to exit
  }
  return nullptr;
}

void EpochManager::Protect() {
  Slot* s = my_slot();
  if (!s || s->depth++ > 0) return;
  while (true) {
    const uint64_t e = global_.load(std::memory_order_acquire);
    s->epoch.store(e, std::memory_order_seq_cst);
    if (global_.load(std::memory_order_seq_cst) == e) return;   // nobody bumped between the read and the publication
  }
}

void EpochManager::Unprotect() {
  Slot* s = my_slot();
  if (!s || --s->depth > 0) return;
  s->epoch.store(0, std::memory_order_release);
}

uint64_t EpochManager::MinProtected() const {
  uint64_t m = UINT64_MAX;
  std::atomic_thread_fence(std::memory_order_seq_cst);
  for (int i = 0; i < kSlots; ++i) {
    const uint64_t e = slots_[i].epoch.load(std::memory_order_acquire);
    if (e != 0 && e < m) m = e;
  }
  return m;
}

void EpochManager::Retire(std::function<void()> reclaim) {
  const uint64_t e = global_.load(std::memory_order_acquire);
  Slot* s = my_slot();
  Stripe& st = stripes_[s ? static_cast<size_t>(s - slots_.get()) % kStripes : 0];
  bool collect;
  {
    std::lock_guard<std::mutex> lk(st.mu);
    st.garbage.push_back({e, std::move(reclaim)});
    collect = (++st.retired & 63) == 0;
  }
  if (collect) {
    const uint64_t g = Bump();
    CollectStripe(st, std::min(MinProtected(), g));
  }
}

size_t EpochManager::CollectStripe(Stripe& st, uint64_t safe_below) {
  std::vector<Item> run;
  {
    std::lock_guard<std::mutex> lk(st.mu);
    size_t keep = 0;
    for (size_t i = 0; i < st.garbage.size(); ++i) {
      if (st.garbage[i].epoch < safe_below) run.push_back(std::move(st.garbage[i]));
      else {
        if (keep != i) st.garbage[keep] = std::move(st.garbage[i]);
        ++keep;
      }
    }
    st.garbage.resize(keep);
  }
  for (auto& it : run) it.fn();
  return run.size();
}

// The scan of the readers' slots says nothing about an object that is retired AFTER the scan: a reader may publish its
// epoch, find the object and start copying it between the scan and the retirement.  Objects retired after the bump
// below carry an epoch >= g, so the bound min(oldest reader, g) leaves them for a later pass; everything retired
// before the bump is judged by a scan that came after its retirement.
size_t EpochManager::Collect() {
  const uint64_t g = Bump();
  const uint64_t safe_below = std::min(MinProtected(), g);
  size_t n = 0;
  for (int i = 0; i < kStripes; ++i) n += CollectStripe(stripes_[i], safe_below);
  return n;
}

size_t EpochManager::DrainAll() {
  size_t n = 0;
  for (int i = 0; i < kStripes; ++i) {
    std::vector<Item> run;
    {
      std::lock_guard<std::mutex> lk(stripes_[i].mu);
      run.swap(stripes_[i].garbage);
    }
    for (auto& it : run) it.fn();
    n += run.size();
  }
  return n;
}

size_t EpochManager::Pending() const {
  size_t n = 0;
  for (int i = 0; i < kStripes; ++i) {
    std::lock_guard<std::mutex> lk(stripes_[i].mu);
    n += stripes_[i].garbage.size();
  }
  return n;
}

// ---------------------------------------------------------------------------------------------------------------------
namespace {
uint64_t steady_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
}  // namespace

SlabRecycler::SlabRecycler(PersistSlabPool* pool, Policy policy, uint64_t delay_ns, EpochManager* epochs, uint32_t bump_every)
    : pool_(pool), policy_(policy), delay_ns_(delay_ns), epochs_(epochs), bump_every_(bump_every ? bump_every : 1) {}

size_t SlabRecycler::drain_locked(uint64_t now_ns) {
  size_t n = 0;
  const uint64_t delay = delay_ns_.load(std::memory_order_relaxed);
  while (head_ < q_.size()) {
    const auto& e = q_[head_];
    const bool due = policy_ == kDelayed ? now_ns - e.first >= delay : epochs_->SafeToReclaim(e.first);
    if (!due) break;
    pool_->Free(e.second);
    ++head_;
    ++n;
  }
  if (head_ == q_.size()) {
    q_.clear();
    head_ = 0;
  } else if (head_ > 4096 && head_ * 2 > q_.size()) {       // drop the consumed front now and then
    q_.erase(q_.begin(), q_.begin() + static_cast<std::ptrdiff_t>(head_));
    head_ = 0;
  }
  return n;
}

size_t SlabRecycler::Recycle(uint64_t off) {
  if (policy_ == kDirect) {
    if (off) pool_->Free(off);
    return off ? 1 : 0;
  }
  std::lock_guard<SpinLock> lk(mu_);
  const uint64_t now = policy_ == kDelayed ? steady_ns() : 0;
  if (off) q_.emplace_back(policy_ == kDelayed ? now : epochs_->Current(), off);
  if (policy_ == kEpoch && ++calls_ % bump_every_ == 0) epochs_->Bump();
  return drain_locked(now);
}

size_t SlabRecycler::Clear() {
  std::lock_guard<SpinLock> lk(mu_);
  size_t n = 0;
  for (; head_ < q_.size(); ++head_, ++n) pool_->Free(q_[head_].second);
  q_.clear();
  head_ = 0;
  return n;
}

size_t SlabRecycler::Pending() const {
  std::lock_guard<SpinLock> lk(mu_);
  return q_.size() - head_;
}

}  // namespace rs

// ============================================================== C ABI
using rs::EpochManager;
using rs::PersistSlabPool;
using rs::SlabRecycler;

RS_API int rs_ppool_open(const char* path, unsigned long long bytes, unsigned long long chunk_bytes, void** out, int* recovered) {
  RS_REQUIRE(out, "rs_ppool_open: null argument");
  RS_NOEXCEPT_BODY(
    bool rec = false;
    auto p = PersistSlabPool::Open(path ? path : "", bytes, chunk_bytes, &rec);
    if (!p) return RS_ERR_INVALID;
    if (recovered) *recovered = rec ? 1 : 0;
    *out = p.release();
    return RS_OK;
  )
}
RS_API int rs_ppool_close(void* h) {
  delete static_cast<PersistSlabPool*>(h);
  return RS_OK;
}
RS_API unsigned long long rs_ppool_malloc(void* h, unsigned long long size) { return static_cast<PersistSlabPool*>(h)->Malloc(size); }
RS_API int rs_ppool_free(void* h, unsigned long long off) {
  static_cast<PersistSlabPool*>(h)->Free(off);
  return RS_OK;
}
RS_API unsigned long long rs_ppool_slab_size(void* h, unsigned long long off) { return static_cast<PersistSlabPool*>(h)->SlabSize(off); }
RS_API unsigned long long rs_ppool_class_size(unsigned long long size) { return PersistSlabPool::ClassSize(size); }
RS_API int rs_ppool_write(void* h, unsigned long long off, const void* src, unsigned long long n) {
  auto* p = static_cast<PersistSlabPool*>(h);
  if (n > p->SlabSize(off)) return rs::set_error(RS_ERR_INVALID, "rs_ppool_write: %llu bytes do not fit the slab at %llu", n, off);
  memcpy(p->At(off), src, n);
  return RS_OK;
}
RS_API int rs_ppool_read(void* h, unsigned long long off, void* dst, unsigned long long n) {
  auto* p = static_cast<PersistSlabPool*>(h);
  if (n > p->SlabSize(off)) return rs::set_error(RS_ERR_INVALID, "rs_ppool_read: %llu bytes exceed the slab at %llu", n, off);
  memcpy(dst, p->At(off), n);
  return RS_OK;
}
// out[6] = chunk_bytes, chunks_total, chunks_in_use, slabs_in_use, bytes_in_use, bytes_reserved
RS_API int rs_ppool_stats(void* h, unsigned long long* out) {
  const auto s = static_cast<PersistSlabPool*>(h)->GetStats();
  out[0] = s.chunk_bytes; out[1] = s.chunks_total; out[2] = s.chunks_in_use;
  out[3] = s.slabs_in_use; out[4] = s.bytes_in_use; out[5] = s.bytes_reserved;
  return RS_OK;
}
// Writes up to cap offsets of allocated slabs; returns how many slabs are allocated in total.
RS_API long long rs_ppool_allocated(void* h, unsigned long long* offs, long long cap) {
  long long n = 0;
  static_cast<PersistSlabPool*>(h)->ForEachAllocated([&](uint64_t off, uint64_t) {
    if (offs && n < cap) offs[n] = off;
    ++n;
  });
  return n;
}
RS_API int rs_ppool_sync(void* h) {
  static_cast<PersistSlabPool*>(h)->Sync();
  return RS_OK;
}

RS_API int rs_epoch_new(void** out) {
  RS_NOEXCEPT_BODY(*out = new EpochManager(); return RS_OK;)
}
RS_API int rs_epoch_delete(void* h) {
  delete static_cast<EpochManager*>(h);
  return RS_OK;
}
RS_API int rs_epoch_protect(void* h) { static_cast<EpochManager*>(h)->Protect(); return RS_OK; }
RS_API int rs_epoch_unprotect(void* h) { static_cast<EpochManager*>(h)->Unprotect(); return RS_OK; }
RS_API unsigned long long rs_epoch_current(void* h) { return static_cast<EpochManager*>(h)->Current(); }
RS_API unsigned long long rs_epoch_bump(void* h) { return static_cast<EpochManager*>(h)->Bump(); }
RS_API int rs_epoch_safe(void* h, unsigned long long epoch) { return static_cast<EpochManager*>(h)->SafeToReclaim(epoch) ? 1 : 0; }
// Retires the slab at off of a pool: it is freed once no protected region can still see it.
RS_API int rs_epoch_retire_slab(void* h, void* pool, unsigned long long off) {
  RS_NOEXCEPT_BODY(
    auto* p = static_cast<PersistSlabPool*>(pool);
    static_cast<EpochManager*>(h)->Retire([p, off] { p->Free(off); });
    return RS_OK;
  )
}
// Runs every pending callback whatever its epoch (the owner of the retired objects is about to go away and no reader
// is left); returns how many ran.
RS_API long long rs_epoch_drain(void* h) { return static_cast<long long>(static_cast<EpochManager*>(h)->DrainAll()); }
RS_API long long rs_epoch_collect(void* h) { return static_cast<long long>(static_cast<EpochManager*>(h)->Collect()); }
RS_API long long rs_epoch_pending(void* h) { return static_cast<long long>(static_cast<EpochManager*>(h)->Pending()); }

// policy: 0 direct, 1 delayed (delay_ns), 2 epoch (epochs must be an EpochManager that outlives the recycler).
RS_API int rs_recycler_new(void* pool, int policy, unsigned long long delay_ns, void* epochs, unsigned bump_every, void** out) {
  RS_REQUIRE(pool && out && policy >= 0 && policy <= 2, "rs_recycler_new: bad argument");
  RS_REQUIRE(policy != 2 || epochs, "rs_recycler_new: the epoch policy needs an epoch manager");
  RS_NOEXCEPT_BODY(
    *out = new SlabRecycler(static_cast<PersistSlabPool*>(pool), static_cast<SlabRecycler::Policy>(policy), delay_ns,
                            static_cast<EpochManager*>(epochs), bump_every);
    return RS_OK;
  )
}
RS_API int rs_recycler_delete(void* h) {
  delete static_cast<SlabRecycler*>(h);
  return RS_OK;
}
RS_API long long rs_recycler_recycle(void* h, unsigned long long off) {
  return static_cast<long long>(static_cast<SlabRecycler*>(h)->Recycle(off));
}
RS_API long long rs_recycler_clear(void* h) { return static_cast<long long>(static_cast<SlabRecycler*>(h)->Clear()); }
RS_API long long rs_recycler_pending(void* h) { return static_cast<long long>(static_cast<SlabRecycler*>(h)->Pending()); }
RS_API int rs_recycler_set_delay_ns(void* h, unsigned long long ns) {
  static_cast<SlabRecycler*>(h)->SetDelayNs(ns);
  return RS_OK;
}
