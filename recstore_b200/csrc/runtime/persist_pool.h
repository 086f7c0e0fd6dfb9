// A crash-recoverable slab allocator over one file mapping, and epoch-based reclamation for the slabs it hands out.
//
// PersistSlabPool plays the role of the reference's PersistMemoryPool (src/memory/persist_malloc.h:126-420: 2 MiB
// chunks, a header with the slab size and an allocation bitmap at the head of every chunk, Recovery() that recounts
// the bitmaps) with a different organisation:
//   * a persistent pointer is an OFFSET from the start of the mapping, so the file may be mapped anywhere;
//   * the only persistent allocator state is the chunk header (slab size, slab count) and the bitmap, both updated
//     with single atomic word operations; free lists, per-class chunk queues and counters are volatile and rebuilt
//     from the bitmaps when the file is opened again;
//   * size classes are 16-byte steps up to 256 bytes and quarter-octave steps above, the largest slab is one chunk.
//
// EpochManager plays the role of src/memory/epoch_manager.h (Protect / Unprotect / BumpCurrentEpoch /
// IsSafeToReclaim over a table of per-thread epochs, plus a garbage list with callbacks): a reader publishes the
// global epoch in its own cache line while it may hold a slab pointer, a writer that unlinks a slab retires it with
// the epoch at that moment, and the slab goes back to the pool once every published epoch is newer.
#pragma once
#include <atomic>
#include <cstdint>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "runtime/base.h"

namespace rs {

class PersistSlabPool {
 public:
  struct Stats {
    uint64_t chunk_bytes, chunks_total, chunks_in_use, slabs_in_use, bytes_in_use, bytes_reserved;
  };
  // path empty: anonymous (volatile) mapping.  chunk_bytes: power of two >= 4096.  *recovered is set when an
  // existing, matching file was mapped (its allocations are live again).
  static std::unique_ptr<PersistSlabPool> Open(const std::string& path, uint64_t bytes, uint64_t chunk_bytes, bool* recovered);
  ~PersistSlabPool();

  // Returns the offset of a slab of at least `size` bytes, 0 when the pool is exhausted or size exceeds a chunk.
  uint64_t Malloc(uint64_t size);
  // Up to n slabs of one size under a single acquisition of the class lock (callers keep small per-thread or per-stripe
  // stocks so that concurrent allocators do not meet on that lock); returns how many offsets were written.
  size_t MallocBatch(uint64_t size, uint64_t* out, size_t n);
  void Free(uint64_t off);
  void* At(uint64_t off) const { return base_ + off; }
  uint64_t OffsetOf(const void* p) const { return static_cast<uint64_t>(static_cast<const char*>(p) - base_); }
  // The usable size of the slab at off (its class size); 0 when off is not the start of an allocated slab.
  uint64_t SlabSize(uint64_t off) const;
  // Calls fn(offset, slab_size) for every allocated slab (after a reopen the owner rebuilds its index from this).
  void ForEachAllocated(const std::function<void(uint64_t, uint64_t)>& fn) const;
  Stats GetStats() const;
  void Sync();
  // Frees everything.
  void Reset();
  static uint64_t ClassSize(uint64_t size);

 private:
  struct ChunkHeader {
    uint64_t magic;
    std::atomic<uint64_t> slab_size;   // 0: the chunk is free
    uint64_t n_slabs;
    uint64_t first_slab;               // byte offset of slab 0 inside the chunk
    // followed by ceil(n_slabs / 64) bitmap words
  };
  struct SuperBlock {
    uint64_t magic, bytes, chunk_bytes, n_chunks;
  };
  struct ClassState {
    SpinLock mu;
    std::vector<uint32_t> partial;     // chunks of this class that may have a free slab
  };
  PersistSlabPool() = default;
  ChunkHeader* chunk(uint64_t c) const { return reinterpret_cast<ChunkHeader*>(base_ + kSuper + c * chunk_bytes_); }
  static std::atomic<uint64_t>* bitmap(ChunkHeader* h) { return reinterpret_cast<std::atomic<uint64_t>*>(h + 1); }
  static int class_index(uint64_t class_size);
  bool format_chunk(uint64_t c, uint64_t class_size);
  uint64_t alloc_in_chunk(uint64_t c);
  void rebuild_volatile();

  static constexpr uint64_t kSuper = 4096;
  static constexpr uint64_t kMagic = 0x5253504F4F4C3031ull, kChunkMagic = 0x525343484B303031ull;
  char* base_ = nullptr;
  uint64_t map_bytes_ = 0, chunk_bytes_ = 0, n_chunks_ = 0;
  bool file_backed_ = false;
  std::vector<std::unique_ptr<ClassState>> classes_;
  mutable SpinLock free_mu_;
  std::vector<uint32_t> free_chunks_;
  std::vector<std::atomic<uint32_t>> used_in_chunk_;   // volatile per-chunk counts
  std::vector<uint32_t> scan_hint_;                    // bitmap word where the last allocation of a chunk succeeded (class lock)
  std::atomic<uint64_t> slabs_in_use_{0}, bytes_in_use_{0};
};

class EpochManager {
 public:
  static constexpr int kSlots = 256;
  EpochManager();
  ~EpochManager();
  // Publishes the current epoch for the calling thread; nests (only the outermost pair publishes / clears).
  void Protect();
  void Unprotect();
  uint64_t Current() const { return global_.load(std::memory_order_acquire); }
  uint64_t Bump() { return global_.fetch_add(1, std::memory_order_acq_rel) + 1; }
  // True when no thread can still hold a pointer that was unlinked while the global epoch was `epoch`.
  bool SafeToReclaim(uint64_t epoch) const { return MinProtected() > epoch; }
  uint64_t MinProtected() const;
  // Hands over an unlinked object; `reclaim` runs (on some later caller's thread) once it is safe.
  void Retire(std::function<void()> reclaim);
  // Advances the epoch, then runs the callbacks of everything retired before that whose readers have all left; returns
  // how many ran.  Retire does the same for its own stripe every few dozen items.
  size_t Collect();
  // Runs everything regardless of epochs (shutdown, no readers left).
  size_t DrainAll();
  size_t Pending() const;

 private:
  struct alignas(64) Slot {
    std::atomic<uint64_t> epoch{0};    // 0: not inside a protected region
    std::atomic<uint64_t> owner{0};    // thread token, 0: unowned
    int depth = 0;
  };
  struct Item {
    uint64_t epoch;
    std::function<void()> fn;
  };
  Slot* my_slot();
  std::atomic<uint64_t> global_{1};
  std::shared_ptr<Slot[]> slots_;    // shared with the threads that hold a slot, which release it when they exit
  static constexpr int kStripes = 16;   // garbage lists, chosen by the retiring thread's slot: retirers rarely share one
  struct alignas(64) Stripe {
    mutable std::mutex mu;
    std::vector<Item> garbage;
    uint64_t retired = 0;
  };
  size_t CollectStripe(Stripe& st, uint64_t safe_below);
  std::unique_ptr<Stripe[]> stripes_;
  std::shared_ptr<std::atomic<bool>> alive_;   // threads drop their slot bookkeeping for a manager that is gone
  const uint64_t id_;
};

// When a freed slab goes back to its pool.  The reference has one class per policy behind ShmBaseRecycle
// (src/memory/malloc.h:34-152: DirectRecycle, DelayedRecycle / StdDelayedRecycle by age, ShmEpochRecycle by epoch);
// here one class with the policy as a value, offsets instead of pointers, and a lock, so several writers may share it.
//   kDirect   the slab is freed at once (no concurrent readers);
//   kDelayed  it is freed once it has waited delay_ns (readers are known to finish within that time);
//   kEpoch    it is freed once every protected region that began before the call has ended; the recycler bumps the
//             epoch every `bump_every` calls.
// Every call also frees what has become due; Recycle(0) only does that.
class SlabRecycler {
 public:
  enum Policy { kDirect = 0, kDelayed = 1, kEpoch = 2 };
  SlabRecycler(PersistSlabPool* pool, Policy policy, uint64_t delay_ns = 1000000000ull, EpochManager* epochs = nullptr,
               uint32_t bump_every = 1000);
  ~SlabRecycler() { Clear(); }
  // Returns how many slabs went back to the pool during the call.
  size_t Recycle(uint64_t off);
  // Frees everything that waits, due or not (no reader is left); returns how many.
  size_t Clear();
  size_t Pending() const;
  void SetDelayNs(uint64_t ns) { delay_ns_ = ns; }
  Policy policy() const { return policy_; }

 private:
  size_t drain_locked(uint64_t now_ns);
  PersistSlabPool* pool_;
  Policy policy_;
  std::atomic<uint64_t> delay_ns_;
  EpochManager* epochs_;
  uint32_t bump_every_;
  mutable SpinLock mu_;
  std::vector<std::pair<uint64_t, uint64_t>> q_;   // (stamp: ns or epoch, offset), oldest first from head_
  size_t head_ = 0;
  uint64_t calls_ = 0;
};

}  // namespace rs
