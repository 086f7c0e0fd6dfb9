// Kernels and host API of the HBM hash-table shard (see hash_table.cuh for the layout), plus a
// hash-based unique() used to deduplicate key batches before they travel between GPUs.
//
// API parity: insert/lookup of the reference's StaticHashTable (src/storage/gpu_cache/
// static_hash_table.cu:117-144, 223-268), extended with erase, dump (checkpoint enumeration) and an
// invariant checker for the tests (count of live slots == size, every key finds itself).
#include <mutex>
#include "common/rs_common.h"
#include "kv/hash_table.cuh"
#include "kv/unique_noalloc.h"

namespace {
using namespace rs;

__global__ void ht_fill_kernel(unsigned long long* keys, int* rows, unsigned long long cap) {
  const unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < cap) {
    keys[i] = kHtEmpty;
    rows[i] = kHtRowPending;
  }
}

__global__ void ht_insert_kernel(HashTableView t, const long long* keys, long long n, long long* rows_out,
                                 unsigned long long* status) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned long long k = static_cast<unsigned long long>(keys[i]);
  if (k >= kHtTomb) {  // reserved sentinels
    if (status) atomicOr(status, (unsigned long long)RS_DEV_BAD_ARG);
    if (rows_out) rows_out[i] = -1;
    return;
  }
  bool inserted, full = false;
  const int r = ht_insert(t, k, &inserted, &full);
  if (full && status) atomicOr(status, (unsigned long long)RS_DEV_TABLE_FULL);
  if (rows_out) rows_out[i] = r;
}

__global__ void ht_lookup_kernel(HashTableView t, const long long* keys, long long n, long long* rows_out) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  rows_out[i] = ht_find(t, static_cast<unsigned long long>(keys[i]));
}

__global__ void ht_erase_kernel(HashTableView t, const long long* keys, long long n, long long* rows_out,
                                unsigned long long* status) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned long long k = static_cast<unsigned long long>(keys[i]);
  if (k >= kHtTomb) {  // reserved sentinels would match an empty / erased slot: nothing is erased, nothing is freed
    if (status) atomicOr(status, (unsigned long long)RS_DEV_BAD_ARG);
    if (rows_out) rows_out[i] = -1;
    return;
  }
  const int r = ht_erase(t, k);
  if (rows_out) rows_out[i] = r;
}

__global__ void ht_dump_kernel(HashTableView t, long long* keys_out, long long* rows_out, unsigned long long* count,
                               unsigned long long cap_out) {
  const unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i > t.mask) return;
  const unsigned long long k = t.keys[i];
  if (k >= kHtTomb) return;
  const unsigned long long pos = atomicAdd(count, 1ull);
  if (pos < cap_out) {
    keys_out[pos] = static_cast<long long>(k);
    rows_out[pos] = t.rows[i];
  }
}

// counts[0] = live slots, counts[1] = keys that do not find themselves / whose row is invalid.
__global__ void ht_check_kernel(HashTableView t, unsigned long long* counts) {
  const unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i > t.mask) return;
  const unsigned long long k = t.keys[i];
  if (k >= kHtTomb) return;
  atomicAdd(&counts[0], 1ull);
  const int r = ht_find(t, k);
  if (r != t.rows[i] || r < 0 || r >= t.max_rows) atomicAdd(&counts[1], 1ull);
}

// ---------------------------------------------------------------- unique
// slots_key / slots_idx: scratch of `nslots` (power of two >= 2 n) entries, cleared by this launch's
// predecessor (unique_clear_kernel).  Every key claims a slot; the first claimer takes the next
// output position.  inverse[i] = position of keys[i] in unique_out.
__global__ void unique_clear_kernel(unsigned long long* slots_key, int* slots_idx, unsigned long long nslots, int* count) {
  const unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < nslots) {
    slots_key[i] = kHtEmpty;
    slots_idx[i] = -1;
  }
  if (i == 0) *count = 0;
}
__global__ void unique_kernel(const long long* keys, long long n, unsigned long long* slots_key, int* slots_idx,
                              unsigned long long mask, long long* unique_out, int* inverse, int* count,
                              unsigned long long* status) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned long long k = static_cast<unsigned long long>(keys[i]);
  if (k >= kHtTomb) {
    // The two reserved keys (-1 = empty marker, -2 = tombstone) cannot be told from a free slot: they take no
    // slot and no output position, their inverse is -1 and the status word says so.
    if (status) atomicOr(status, (unsigned long long)RS_DEV_BAD_ARG);
    if (inverse) inverse[i] = -1;
    return;
  }
  unsigned long long s = ht_hash(k) & mask;
  for (int p = 0; p < kHtMaxProbe; ++p) {
    unsigned long long cur = __ldcv(&slots_key[s]);
    if (cur == kHtEmpty) {
      const unsigned long long prev = atomicCAS(&slots_key[s], kHtEmpty, k);
      if (prev == kHtEmpty) {
        const int u = atomicAdd(count, 1);
        unique_out[u] = static_cast<long long>(k);
        atomicExch(&slots_idx[s], u);
        if (inverse) inverse[i] = u;
        return;
      }
      cur = prev;
    }
    if (cur == k) {
      int u = __ldcv(&slots_idx[s]);
      for (int spin = 0; u < 0 && spin < (1 << 18); ++spin) {
        __nanosleep(spin < 64 ? 20 : 200);
        u = __ldcv(&slots_idx[s]);
      }
      if (u < 0 && status) atomicOr(status, (unsigned long long)RS_DEV_WAIT_TIMEOUT);
      if (inverse) inverse[i] = u;
      return;
    }
    s = (s + 1) & mask;
  }
  if (status) atomicOr(status, (unsigned long long)RS_DEV_TABLE_FULL);
  if (inverse) inverse[i] = -1;
}

struct HtOwned {
  HashTableView v;
  unsigned long long capacity;
  int* counters;  // next_row, free_top, size
};

inline unsigned grid_for(unsigned long long n) { return static_cast<unsigned>((n + 255) / 256); }
}  // namespace

// capacity: number of slots (rounded up to a power of two); max_rows: size of the row store it indexes.
RS_API int rs_ht_create(unsigned long long capacity, int max_rows, void** handle, rs::HashTableView* view_out) {
  RS_REQUIRE(handle && view_out && capacity >= 2 && max_rows > 0, "rs_ht_create: bad argument");
  unsigned long long cap = 2;
  while (cap < capacity) cap <<= 1;
  HtOwned* h = new HtOwned();
  h->capacity = cap;
  RS_CUDA(cudaMalloc(&h->v.keys, cap * sizeof(unsigned long long)));
  RS_CUDA(cudaMalloc(&h->v.rows, cap * sizeof(int)));
  RS_CUDA(cudaMalloc(&h->v.free_rows, static_cast<size_t>(max_rows) * sizeof(int)));
  RS_CUDA(cudaMalloc(&h->counters, 4 * sizeof(int)));
  RS_CUDA(cudaMemset(h->counters, 0, 4 * sizeof(int)));
  h->v.mask = cap - 1;
  h->v.next_row = h->counters;
  h->v.free_top = h->counters + 1;
  h->v.size = h->counters + 2;
  h->v.max_rows = max_rows;
  ht_fill_kernel<<<grid_for(cap), 256>>>(h->v.keys, h->v.rows, cap);
  RS_LAUNCH_CHECK();
  RS_CUDA(cudaDeviceSynchronize());
  *handle = h;
  *view_out = h->v;
  return RS_OK;
}
RS_API int rs_ht_destroy(void* handle) {
  if (!handle) return RS_OK;
  HtOwned* h = static_cast<HtOwned*>(handle);
  cudaFree(h->v.keys);
  cudaFree(h->v.rows);
  cudaFree(h->v.free_rows);
  cudaFree(h->counters);
  delete h;
  return RS_OK;
}
RS_API int rs_ht_clear(void* handle, cudaStream_t stream) {
  RS_REQUIRE(handle, "rs_ht_clear: null handle");
  HtOwned* h = static_cast<HtOwned*>(handle);
  ht_fill_kernel<<<grid_for(h->capacity), 256, 0, stream>>>(h->v.keys, h->v.rows, h->capacity);
  RS_LAUNCH_CHECK();
  RS_CUDA(cudaMemsetAsync(h->counters, 0, 4 * sizeof(int), stream));
  return RS_OK;
}
// rows_out may be null for insert / erase.  Inserts and erases must not overlap on the device.
RS_API int rs_ht_insert(const rs::HashTableView* v, const long long* keys, long long n, long long* rows_out,
                        unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(v && keys, "rs_ht_insert: null argument");
  if (n == 0) return RS_OK;
  ht_insert_kernel<<<grid_for(n), 256, 0, stream>>>(*v, keys, n, rows_out, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
RS_API int rs_ht_lookup(const rs::HashTableView* v, const long long* keys, long long n, long long* rows_out,
                        cudaStream_t stream) {
  RS_REQUIRE(v && keys && rows_out, "rs_ht_lookup: null argument");
  if (n == 0) return RS_OK;
  ht_lookup_kernel<<<grid_for(n), 256, 0, stream>>>(*v, keys, n, rows_out);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
RS_API int rs_ht_erase(const rs::HashTableView* v, const long long* keys, long long n, long long* rows_out,
                       cudaStream_t stream) {
  RS_REQUIRE(v && keys, "rs_ht_erase: null argument");
  if (n == 0) return RS_OK;
  ht_erase_kernel<<<grid_for(n), 256, 0, stream>>>(*v, keys, n, rows_out, nullptr);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
// Same with a status word: the reserved keys -1 / -2 are refused with RS_DEV_BAD_ARG (and row -1).
RS_API int rs_ht_erase_checked(const rs::HashTableView* v, const long long* keys, long long n, long long* rows_out,
                               unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(v && keys, "rs_ht_erase_checked: null argument");
  if (n == 0) return RS_OK;
  ht_erase_kernel<<<grid_for(n), 256, 0, stream>>>(*v, keys, n, rows_out, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
// count: device counter (zeroed by this call); at most cap_out pairs are written.
RS_API int rs_ht_dump(const rs::HashTableView* v, long long* keys_out, long long* rows_out, unsigned long long* count,
                      unsigned long long cap_out, cudaStream_t stream) {
  RS_REQUIRE(v && keys_out && rows_out && count, "rs_ht_dump: null argument");
  RS_CUDA(cudaMemsetAsync(count, 0, sizeof(unsigned long long), stream));
  ht_dump_kernel<<<grid_for(v->mask + 1), 256, 0, stream>>>(*v, keys_out, rows_out, count, cap_out);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
// Synchronous: returns live keys, size counter and the number of inconsistent slots.
RS_API int rs_ht_check(const rs::HashTableView* v, unsigned long long* live, long long* size, unsigned long long* bad) {
  RS_REQUIRE(v && live && size && bad, "rs_ht_check: null argument");
  unsigned long long* d;
  RS_CUDA(cudaMalloc(&d, 2 * sizeof(unsigned long long)));
  RS_CUDA(cudaMemset(d, 0, 2 * sizeof(unsigned long long)));
  ht_check_kernel<<<grid_for(v->mask + 1), 256>>>(*v, d);
  RS_LAUNCH_CHECK();
  unsigned long long h[2];
  RS_CUDA(cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost));
  int sz = 0;
  RS_CUDA(cudaMemcpy(&sz, v->size, sizeof(int), cudaMemcpyDeviceToHost));
  cudaFree(d);
  *live = h[0];
  *bad = h[1];
  *size = sz;
  return RS_OK;
}

// Deduplicates keys[0..n).  Keys are 64-bit patterns; the two reserved ones (-1 and -2 as signed values) are not
// deduplicated: their inverse is -1, they do not appear in unique_out and RS_DEV_BAD_ARG is set in the status word.
// Scratch (caller-provided): slots_key [nslots] u64, slots_idx [nslots] i32 with
// nslots a power of two >= 2 n.  Outputs: unique_out [<= n], inverse [n] (optional), count (device int).
RS_API int rs_unique_keys(const long long* keys, long long n, void* slots_key, void* slots_idx,
                          unsigned long long nslots, long long* unique_out, int* inverse, int* count,
                          unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(keys && slots_key && slots_idx && unique_out && count, "rs_unique_keys: null argument");
  RS_REQUIRE(nslots >= 2 && (nslots & (nslots - 1)) == 0 && nslots >= 2ull * static_cast<unsigned long long>(n),
             "rs_unique_keys: nslots must be a power of two >= 2 n");
  unique_clear_kernel<<<grid_for(nslots), 256, 0, stream>>>(static_cast<unsigned long long*>(slots_key),
                                                            static_cast<int*>(slots_idx), nslots, count);
  RS_LAUNCH_CHECK();
  if (n == 0) return RS_OK;
  unique_kernel<<<grid_for(n), 256, 0, stream>>>(keys, n, static_cast<unsigned long long*>(slots_key),
                                                 static_cast<int*>(slots_idx), nslots - 1, unique_out, inverse, count, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// ------------------------------------------------------------------ allocation-free unique
// Scratch of rs_unique_keys_noalloc (see kv/unique_noalloc.h): 2 * MAX_KEYS slots, 8-byte keys first,
// then 4-byte indices.  In host code the NAME of this array is only a handle for the runtime, not a
// device address; the address every kernel gets comes from cudaGetSymbolAddress below.
namespace {
constexpr unsigned long long kNoAllocSlots = 2ull * RS_UNIQUE_NOALLOC_MAX_KEYS;
static __device__ __align__(256) unsigned char g_unique_noalloc_scratch[kNoAllocSlots * (sizeof(unsigned long long) + sizeof(int))];

constexpr int kMaxDevices = 64;
void* g_noalloc_addr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mu;
}  // namespace

RS_API int rs_unique_keys_noalloc(const long long* keys, long long n, long long* unique_out, int* inverse, int* count,
                                  unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(unique_out && count && (keys || n == 0), "rs_unique_keys_noalloc: null argument");
  RS_REQUIRE(n >= 0, "rs_unique_keys_noalloc: negative key count");
  if (n > RS_UNIQUE_NOALLOC_MAX_KEYS)
    return rs::set_error(RS_ERR_CAPACITY,
                         "rs_unique_keys_noalloc: %lld keys exceed the built-in scratch (at most %d keys per call); "
                         "split the batch or use rs_unique_keys with caller-provided scratch",
                         n, RS_UNIQUE_NOALLOC_MAX_KEYS);
  int dev = 0;
  RS_CUDA(cudaGetDevice(&dev));
  RS_REQUIRE(dev >= 0 && dev < kMaxDevices, "rs_unique_keys_noalloc: device index %d not supported", dev);
  void* base = nullptr;
  {
    // One-time set-up per device, with that device current: resolve the device address of the array.
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (g_noalloc_addr[dev] == nullptr) {
      void* p = nullptr;
      RS_CUDA(cudaGetSymbolAddress(&p, g_unique_noalloc_scratch));
      g_noalloc_addr[dev] = p;
    }
    base = g_noalloc_addr[dev];
  }
  unsigned long long nslots = 2;
  while (nslots < 2ull * static_cast<unsigned long long>(n)) nslots <<= 1;   // <= kNoAllocSlots by the check above
  unsigned long long* slots_key = static_cast<unsigned long long*>(base);
  int* slots_idx = reinterpret_cast<int*>(static_cast<unsigned char*>(base) + kNoAllocSlots * sizeof(unsigned long long));
  // The array still holds the previous call's keys: clear the slots this call will use (and the counter).
  unique_clear_kernel<<<grid_for(nslots), 256, 0, stream>>>(slots_key, slots_idx, nslots, count);
  RS_LAUNCH_CHECK();
  if (n == 0) return RS_OK;
  unique_kernel<<<grid_for(n), 256, 0, stream>>>(keys, n, slots_key, slots_idx, nslots - 1, unique_out, inverse, count, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
