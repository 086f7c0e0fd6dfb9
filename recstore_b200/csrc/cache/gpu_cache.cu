// Set-associative LRU embedding cache in HBM with the Query / Replace / Update / Dump contract of the
// cache the reference vendors from HugeCTR (src/storage/gpu_cache/nv_gpu_cache.cu:392-531 get_kernel,
// 700-852 insert_replace_kernel, 970-1074 update_kernel, 1155-1226 dump_kernel; API
// gpu_cache_api.hpp:27-50; torch wrapper src/framework/pytorch/recstore_gpu_cache.h:31-106).
//
// Layout: `nsets` sets of 32 slots; a warp probes a set with one 256-byte coalesced load (one key per
// lane) and a ballot.  Differences from the reference kernel shape (1 key per warp, 2 keys per
// 64-thread block, a per-set mutex even on reads):
//   * each warp walks a strided list of keys and keeps the next key's set line in flight while it
//     copies the current row, so many keys are in flight per SM;
//   * the hit path takes no lock: it reads keys / values and stamps the slot's counter with a relaxed store (a
//     stale stamp only makes LRU slightly approximate).  Every slot carries a sequence number that a writer makes
//     odd before it touches the slot's key or values and even again afterwards; Query reads it before and after
//     the row copy and reports the key as a MISS when it was odd or changed, so a Query that overlaps a Replace /
//     Update of the same slot on another stream never returns a torn or wrong-key row as a hit;
//   * Replace / Update take a per-set lock with a BOUNDED spin; on give-up the key is skipped and
//     RS_DEV_WAIT_TIMEOUT is recorded.
// Semantics kept: Query writes hit rows in place, leaves miss rows untouched, appends (position,
// key) of every miss in arbitrary order with a device-side count, bumps the global clock; Replace
// inserts into an empty slot or evicts the smallest stamp and refreshes the stamp when the key is
// already cached; Update overwrites values of cached keys only; Dump enumerates the keys of a set range.
#include "common/rs_common.h"
#include "kv/hash_table.cuh"

namespace {
using rs::ht_hash;

constexpr unsigned long long kEmptyKey = 0xFFFFFFFFFFFFFFFFull;
constexpr int kWays = 32;

struct CacheView {
  unsigned long long* keys;   // [nsets * 32]
  unsigned* stamps;           // [nsets * 32]
  unsigned* vers;             // [nsets * 32] slot sequence numbers (odd while a writer is inside)
  unsigned char* dirty;       // [nsets * 32] 1 = the row was changed in the cache and the backing store is behind
  float* values;              // [nsets * 32, dim]
  int* locks;                 // [nsets]
  unsigned* clock;            // global LRU clock
  unsigned long long nsets;
  int dim;
};

__device__ __forceinline__ void copy_row(float* __restrict__ dst, const float* __restrict__ src, int dim, int lane) {
  for (int v = lane; v < (dim >> 2); v += 32) reinterpret_cast<float4*>(dst)[v] = reinterpret_cast<const float4*>(src)[v];
}

// Same copy with the source read from L2 (never from a possibly stale L1 line): used by the lock-free hit path, whose
// sequence-number check only vouches for what L2 holds.
__device__ __forceinline__ void copy_row_cg(float* __restrict__ dst, const float* src, int dim, int lane) {
  for (int v = lane; v < (dim >> 2); v += 32) reinterpret_cast<float4*>(dst)[v] = __ldcg(reinterpret_cast<const float4*>(src) + v);
}

__global__ void cache_init_kernel(CacheView c) {
  const unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < c.nsets * kWays) {
    c.keys[i] = kEmptyKey;
    c.stamps[i] = 0;
    c.vers[i] = 0;
    c.dirty[i] = 0;
  }
  if (i < c.nsets) c.locks[i] = 0;
  if (i == 0) *c.clock = 0;
}

__global__ void cache_tick_kernel(unsigned* clock, int* miss_count) {
  atomicAdd(clock, 1u);
  if (miss_count) *miss_count = 0;
}

// One warp per key: the 32 lanes compare the 32 tags of the key's set (one 256-B line).  A warp takes its keys four at a
// time so that four tag lines are in flight before the first is compared, and it collects its misses in registers
// (lane r keeps the r-th miss) and appends them with ONE atomicAdd per 32 misses: a counter bumped once per missing key
// serialises the whole grid on one L2 address when the hit rate is low.
__global__ void __launch_bounds__(256) cache_query_kernel(CacheView c, const long long* __restrict__ keys, long long n,
                                                          float* __restrict__ out, long long* __restrict__ miss_index,
                                                          long long* __restrict__ miss_keys, int* __restrict__ miss_count) {
  constexpr int kAhead = 4;
  const int lane = threadIdx.x & 31;
  const long long warp = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const unsigned now = *c.clock;
  int n_miss = 0;
  long long my_miss_index = 0;
  unsigned long long my_miss_key = 0;
  auto flush_misses = [&]() {
    int base = 0;
    if (lane == 0) base = atomicAdd(miss_count, n_miss);
    base = __shfl_sync(0xffffffffu, base, 0);
    if (lane < n_miss) {
      miss_index[base + lane] = my_miss_index;
      miss_keys[base + lane] = static_cast<long long>(my_miss_key);
    }
    n_miss = 0;
  };
  for (long long i0 = warp; i0 < n; i0 += nwarps * kAhead) {
    unsigned long long key[kAhead], set[kAhead], line[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const long long i = i0 + u * nwarps;
      key[u] = i < n ? static_cast<unsigned long long>(keys[i]) : kEmptyKey;
      set[u] = ht_hash(key[u]) % c.nsets;
      line[u] = key[u] != kEmptyKey ? c.keys[set[u] * kWays + lane] : kEmptyKey;
    }
    // Hits are validated like a seqlock reader (version, key, row, version again), in three phases over the four keys so
    // that the warp pays three dependent round trips and two fences per FOUR keys, not per key.
    unsigned long long slot[kAhead], k0[kAhead];
    unsigned v0[kAhead];
    bool hit[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const unsigned m = __ballot_sync(0xffffffffu, key[u] != kEmptyKey && line[u] == key[u]);
      hit[u] = m != 0;
      slot[u] = set[u] * kWays + (hit[u] ? __ffs(m) - 1 : 0);
      v0[u] = hit[u] ? *reinterpret_cast<volatile unsigned*>(&c.vers[slot[u]]) : 1u;
    }
    __threadfence();
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      if (!hit[u]) continue;
      k0[u] = *reinterpret_cast<volatile unsigned long long*>(&c.keys[slot[u]]);
      if (out != nullptr) copy_row_cg(out + (i0 + u * nwarps) * c.dim, c.values + slot[u] * c.dim, c.dim, lane);
    }
    __threadfence();
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      if (key[u] == kEmptyKey) continue;                     // padding (or past the end): neither a hit nor a miss
      bool valid = false;
      if (hit[u]) {
        const unsigned v1 = *reinterpret_cast<volatile unsigned*>(&c.vers[slot[u]]);
        valid = __all_sync(0xffffffffu, (v0[u] & 1u) == 0u && v1 == v0[u] && k0[u] == key[u]);
        if (valid && lane == 0 && c.stamps[slot[u]] != now) c.stamps[slot[u]] = now;
      }
      if (!valid) {
        if (lane == n_miss) {
          my_miss_index = i0 + u * nwarps;
          my_miss_key = key[u];
        }
        if (++n_miss == 32) flush_misses();
      }
    }
  }
  if (n_miss > 0) flush_misses();
}

__device__ __forceinline__ bool lock_set(int* lock, int lane) {
  int ok = 0;
  if (lane == 0) {
    for (int spin = 0; spin < (1 << 20); ++spin) {
      if (atomicCAS(lock, 0, 1) == 0) { ok = 1; break; }
      __nanosleep(32);
    }
    __threadfence();
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void unlock_set(int* lock, int lane) {
  __syncwarp();
  if (lane == 0) {
    __threadfence();
    atomicExch(lock, 0);
  }
}

// mode 0: Replace (insert or evict LRU, refresh stamp when present); mode 1: Update (present keys only).
__global__ void __launch_bounds__(256) cache_write_kernel(CacheView c, const long long* __restrict__ keys, long long n,
                                                          const float* __restrict__ values, int mode,
                                                          unsigned long long* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const unsigned now = *c.clock;
  for (long long i = warp; i < n; i += nwarps) {
    const unsigned long long key = static_cast<unsigned long long>(keys[i]);
    if (key == kEmptyKey) continue;
    const unsigned long long set = ht_hash(key) % c.nsets;
    if (!lock_set(&c.locks[set], lane)) {
      if (lane == 0 && status) atomicOr(status, (unsigned long long)RS_DEV_WAIT_TIMEOUT);
      continue;
    }
    const unsigned long long line = *reinterpret_cast<volatile unsigned long long*>(&c.keys[set * kWays + lane]);
    const unsigned hit = __ballot_sync(0xffffffffu, line == key);
    int way = -1;
    bool write_value = false;
    if (hit) {
      way = __ffs(hit) - 1;
      write_value = (mode == 1);          // Replace of a cached key only refreshes its stamp
    } else if (mode == 0) {
      const unsigned empty = __ballot_sync(0xffffffffu, line == kEmptyKey);
      if (empty) {
        way = __ffs(empty) - 1;
      } else {                             // evict the least recently stamped slot
        unsigned st = *reinterpret_cast<volatile unsigned*>(&c.stamps[set * kWays + lane]);
        unsigned long long best = (static_cast<unsigned long long>(st) << 5) | lane;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
          best = other < best ? other : best;
        }
        way = static_cast<int>(best & 31);
      }
      write_value = true;
    }
    if (way >= 0) {
      const unsigned long long slot = set * kWays + way;
      if (write_value) {
        // sequence number odd -> key and values change -> even again (readers discard what they copied meanwhile)
        if (lane == 0) {
          atomicAdd(&c.vers[slot], 1u);
          __threadfence();
        }
        __syncwarp();
        copy_row(c.values + slot * c.dim, values + i * c.dim, c.dim, lane);
        if (lane == 0 && !hit) *reinterpret_cast<volatile unsigned long long*>(&c.keys[slot]) = key;
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(&c.vers[slot], 1u);
      }
      if (lane == 0 && mode == 0) c.stamps[slot] = now;
    }
    unlock_set(&c.locks[set], lane);
  }
}

// Replace that hands the evicted rows back (write-back caches) and never evicts a row stamped at or after
// `protect_from` (rows of the step in flight and of the batches already announced).  Dirty evicted rows go to
// evict_keys / evict_values (cursor evict_count); a key that finds its set full of protected rows is not inserted and is
// reported in refused_keys (cursor refused_count): the caller serves it from the backing store.
__global__ void __launch_bounds__(256) cache_replace_evict_kernel(CacheView c, const long long* __restrict__ keys, const int* n_dev,
                                                                  long long n_cap, const float* __restrict__ values, unsigned protect_from,
                                                                  long long* __restrict__ evict_keys, float* __restrict__ evict_values,
                                                                  int* evict_count, long long* __restrict__ refused_keys,
                                                                  int* refused_count, unsigned long long* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const unsigned now = *c.clock;
  const long long n = n_dev ? min(static_cast<long long>(*n_dev), n_cap) : n_cap;
  for (long long i = warp; i < n; i += nwarps) {
    const unsigned long long key = static_cast<unsigned long long>(keys[i]);
    if (key == kEmptyKey) continue;
    const unsigned long long set = ht_hash(key) % c.nsets;
    if (!lock_set(&c.locks[set], lane)) {
      if (lane == 0 && status) atomicOr(status, (unsigned long long)RS_DEV_WAIT_TIMEOUT);
      if (lane == 0 && refused_keys) refused_keys[atomicAdd(refused_count, 1)] = static_cast<long long>(key);
      continue;
    }
    const unsigned long long line = *reinterpret_cast<volatile unsigned long long*>(&c.keys[set * kWays + lane]);
    const unsigned hit = __ballot_sync(0xffffffffu, line == key);
    if (hit) {                                   // already cached (brought in by a step in between): only refresh the stamp
      if (lane == 0) c.stamps[set * kWays + (__ffs(hit) - 1)] = now;
      unlock_set(&c.locks[set], lane);
      continue;
    }
    int way = -1;
    bool evicting = false;
    const unsigned empty = __ballot_sync(0xffffffffu, line == kEmptyKey);
    if (empty) {
      way = __ffs(empty) - 1;
    } else {
      const unsigned st = *reinterpret_cast<volatile unsigned*>(&c.stamps[set * kWays + lane]);
      unsigned long long best = (static_cast<unsigned long long>(st) << 5) | lane;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other < best ? other : best;
      }
      if (static_cast<unsigned>(best >> 5) < protect_from) { way = static_cast<int>(best & 31); evicting = true; }
    }
    if (way < 0) {                               // every way holds a protected row
      if (lane == 0 && refused_keys) refused_keys[atomicAdd(refused_count, 1)] = static_cast<long long>(key);
      unlock_set(&c.locks[set], lane);
      continue;
    }
    const unsigned long long slot = set * kWays + way;
    if (evicting && c.dirty[slot] && evict_keys) {
      int pos = 0;
      if (lane == 0) pos = atomicAdd(evict_count, 1);
      pos = __shfl_sync(0xffffffffu, pos, 0);
      copy_row(evict_values + static_cast<long long>(pos) * c.dim, c.values + slot * c.dim, c.dim, lane);
      const unsigned long long old = __shfl_sync(0xffffffffu, line, way);
      if (lane == 0) evict_keys[pos] = static_cast<long long>(old);
    }
    if (lane == 0) {
      atomicAdd(&c.vers[slot], 1u);
      __threadfence();
    }
    __syncwarp();
    copy_row(c.values + slot * c.dim, values + i * c.dim, c.dim, lane);
    if (lane == 0) {
      *reinterpret_cast<volatile unsigned long long*>(&c.keys[slot]) = key;
      c.stamps[slot] = now;
      c.dirty[slot] = 0;
    }
    __threadfence();
    __syncwarp();
    if (lane == 0) atomicAdd(&c.vers[slot], 1u);
    unlock_set(&c.locks[set], lane);
  }
}

// Optimizer step on cached rows, in place.  A cached row is [D weights | state | padding] (dim = D + 4).  keys are distinct;
// grad [n, D] and norm [n] (sum of squares over the key's occurrences).  optimizer 0: w -= lr * g; 1 (row-wise Adagrad):
// state += norm / D, w -= lr * g / (sqrt(state) + eps).  A key that is not cached is appended to missing (cursor
// missing_count) with its index, for the caller to apply on the backing store.
__global__ void __launch_bounds__(256) cache_apply_kernel(CacheView c, const long long* __restrict__ keys, const int* n_dev, long long n_cap,
                                                          const float* __restrict__ grad, const float* __restrict__ norm, int D, float lr,
                                                          float eps, int optimizer, long long* __restrict__ missing_index,
                                                          int* missing_count) {
  const int lane = threadIdx.x & 31;
  const long long warp = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long n = n_dev ? min(static_cast<long long>(*n_dev), n_cap) : n_cap;
  for (long long i = warp; i < n; i += nwarps) {
    const unsigned long long key = static_cast<unsigned long long>(keys[i]);
    if (key == kEmptyKey) continue;
    const unsigned long long set = ht_hash(key) % c.nsets;
    const unsigned long long line = c.keys[set * kWays + lane];
    const unsigned hit = __ballot_sync(0xffffffffu, line == key);
    if (!hit) {
      if (lane == 0 && missing_index) missing_index[atomicAdd(missing_count, 1)] = i;
      continue;
    }
    const unsigned long long slot = set * kWays + (__ffs(hit) - 1);
    float* row = c.values + slot * c.dim;
    if (lane == 0) {
      atomicAdd(&c.vers[slot], 1u);
      __threadfence();
    }
    __syncwarp();
    float scale = -lr;
    if (optimizer == 1) {
      const float stt = row[D] + (norm ? norm[i] : 0.f) / static_cast<float>(D);
      scale = -lr / (sqrtf(stt) + eps);
      __syncwarp();
      if (lane == 0) row[D] = stt;
    }
    for (int v = lane; v < (D >> 2); v += 32) {
      float4 w = reinterpret_cast<float4*>(row)[v];
      const float4 g = __ldg(reinterpret_cast<const float4*>(grad + i * D) + v);
      w.x += scale * g.x; w.y += scale * g.y; w.z += scale * g.z; w.w += scale * g.w;
      reinterpret_cast<float4*>(row)[v] = w;
    }
    if (lane == 0) c.dirty[slot] = 1;
    __threadfence();
    __syncwarp();
    if (lane == 0) atomicAdd(&c.vers[slot], 1u);
  }
}

__global__ void cache_set_clock_kernel(unsigned* clock, unsigned v) { *clock = v; }

// Every dirty row of the set range -> (keys, values), dirty bits cleared: a flush for checkpoints.
__global__ void __launch_bounds__(256) cache_flush_dirty_kernel(CacheView c, long long* __restrict__ keys_out, float* __restrict__ values_out,
                                                                int* count) {
  const int lane = threadIdx.x & 31;
  const unsigned long long warp = static_cast<unsigned long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const unsigned long long nwarps = static_cast<unsigned long long>(gridDim.x) * (blockDim.x >> 5);
  for (unsigned long long slot = warp; slot < c.nsets * kWays; slot += nwarps) {
    if (c.keys[slot] == kEmptyKey || !c.dirty[slot]) continue;
    int pos = 0;
    if (lane == 0) pos = atomicAdd(count, 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (lane == 0) { keys_out[pos] = static_cast<long long>(c.keys[slot]); c.dirty[slot] = 0; }
    copy_row(values_out + static_cast<long long>(pos) * c.dim, c.values + slot * c.dim, c.dim, lane);
  }
}

__global__ void cache_dump_kernel(CacheView c, unsigned long long set_begin, unsigned long long set_end,
                                  long long* __restrict__ keys_out, unsigned long long* count) {
  const unsigned long long i = set_begin * kWays + static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= set_end * kWays) return;
  const unsigned long long k = c.keys[i];
  if (k == kEmptyKey) return;
  keys_out[atomicAdd(count, 1ull)] = static_cast<long long>(k);
}

struct CacheOwned {
  CacheView v;
};
}  // namespace

// num_items is rounded up to a multiple of 32; dim must be a multiple of 4.
RS_API int rs_cache_create(unsigned long long num_items, int dim, void** handle) {
  RS_REQUIRE(handle && num_items > 0 && dim > 0 && dim % 4 == 0, "rs_cache_create: bad argument (dim %% 4 == 0)");
  CacheOwned* h = new CacheOwned();
  CacheView& v = h->v;
  v.nsets = (num_items + kWays - 1) / kWays;
  v.dim = dim;
  const unsigned long long slots = v.nsets * kWays;
  RS_CUDA(cudaMalloc(&v.keys, slots * sizeof(unsigned long long)));
  RS_CUDA(cudaMalloc(&v.stamps, slots * sizeof(unsigned)));
  RS_CUDA(cudaMalloc(&v.vers, slots * sizeof(unsigned)));
  RS_CUDA(cudaMalloc(&v.dirty, slots));
  RS_CUDA(cudaMalloc(&v.values, slots * static_cast<size_t>(dim) * sizeof(float)));
  RS_CUDA(cudaMalloc(&v.locks, v.nsets * sizeof(int)));
  RS_CUDA(cudaMalloc(&v.clock, sizeof(unsigned)));
  cache_init_kernel<<<static_cast<unsigned>((slots + 255) / 256), 256>>>(v);
  RS_LAUNCH_CHECK();
  RS_CUDA(cudaDeviceSynchronize());
  *handle = h;
  return RS_OK;
}
RS_API int rs_cache_destroy(void* handle) {
  if (!handle) return RS_OK;
  CacheOwned* h = static_cast<CacheOwned*>(handle);
  cudaFree(h->v.keys); cudaFree(h->v.stamps); cudaFree(h->v.vers); cudaFree(h->v.dirty); cudaFree(h->v.values); cudaFree(h->v.locks); cudaFree(h->v.clock);
  delete h;
  return RS_OK;
}
RS_API unsigned long long rs_cache_capacity(void* handle) { return static_cast<CacheOwned*>(handle)->v.nsets * kWays; }
RS_API unsigned long long rs_cache_num_sets(void* handle) { return static_cast<CacheOwned*>(handle)->v.nsets; }

// out: [n, dim] (hit rows written, miss rows untouched); miss_index / miss_keys: [n]; miss_count: device int.
RS_API int rs_cache_query(void* handle, const long long* keys, long long n, float* out, long long* miss_index,
                          long long* miss_keys, int* miss_count, cudaStream_t stream) {
  RS_REQUIRE(handle && keys && miss_index && miss_keys && miss_count, "rs_cache_query: null argument");   // out == null: probe only
  CacheView& v = static_cast<CacheOwned*>(handle)->v;
  cache_tick_kernel<<<1, 1, 0, stream>>>(v.clock, miss_count);
  RS_LAUNCH_CHECK();
  if (n == 0) return RS_OK;
  long long warps = (n + 3) / 4;  // >= 4 keys per warp when there are enough keys
  if (warps > 148 * 24) warps = 148 * 24;    // three resident blocks of eight warps per SM (80 registers per thread)
  cache_query_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(v, keys, n, out, miss_index, miss_keys, miss_count);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
RS_API int rs_cache_replace(void* handle, const long long* keys, long long n, const float* values,
                            unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(handle && keys && values, "rs_cache_replace: null argument");
  if (n == 0) return RS_OK;
  CacheView& v = static_cast<CacheOwned*>(handle)->v;
  long long warps = n < 148 * 32 ? n : 148 * 32;
  cache_write_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(v, keys, n, values, 0, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
RS_API int rs_cache_update(void* handle, const long long* keys, long long n, const float* values,
                           unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(handle && keys && values, "rs_cache_update: null argument");
  if (n == 0) return RS_OK;
  CacheView& v = static_cast<CacheOwned*>(handle)->v;
  long long warps = n < 148 * 32 ? n : 148 * 32;
  cache_write_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(v, keys, n, values, 1, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
// keys_out must hold (set_end - set_begin) * 32 entries; count: device counter, zeroed here.
RS_API int rs_cache_dump(void* handle, unsigned long long set_begin, unsigned long long set_end, long long* keys_out,
                         unsigned long long* count, cudaStream_t stream) {
  RS_REQUIRE(handle && keys_out && count, "rs_cache_dump: null argument");
  CacheView& v = static_cast<CacheOwned*>(handle)->v;
  RS_REQUIRE(set_begin <= set_end && set_end <= v.nsets, "rs_cache_dump: set range [%llu, %llu) outside [0, %llu)",
             set_begin, set_end, v.nsets);
  RS_CUDA(cudaMemsetAsync(count, 0, sizeof(unsigned long long), stream));
  const unsigned long long slots = (set_end - set_begin) * kWays;
  if (slots == 0) return RS_OK;
  cache_dump_kernel<<<static_cast<unsigned>((slots + 255) / 256), 256, 0, stream>>>(v, set_begin, set_end, keys_out, count);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// ---- write-back cache verbs (the HBM tier of a table whose backing store is host memory)
// keys may be bounded by a device count n_dev (<= n_cap).  evict_* / refused_* outputs hold up to n_cap entries; their
// counters are NOT cleared here (one pair of counters can collect over several calls).
RS_API int rs_cache_replace_evict(void* handle, const long long* keys, const int* n_dev, long long n_cap, const float* values,
                                  unsigned protect_from, long long* evict_keys, float* evict_values, int* evict_count,
                                  long long* refused_keys, int* refused_count, unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(handle && keys && values, "rs_cache_replace_evict: null argument");
  RS_REQUIRE(!evict_keys || (evict_values && evict_count), "rs_cache_replace_evict: eviction output needs values and a counter");
  RS_REQUIRE(!refused_keys || refused_count, "rs_cache_replace_evict: refusal output needs a counter");
  if (n_cap == 0) return RS_OK;
  CacheView& v = static_cast<CacheOwned*>(handle)->v;
  long long warps = n_cap < 148 * 32 ? n_cap : 148 * 32;
  cache_replace_evict_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(v, keys, n_dev, n_cap, values, protect_from,
                                                                                        evict_keys, evict_values, evict_count,
                                                                                        refused_keys, refused_count, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
// D: weights per row; the cache was created with dim >= D + 1 (state at column D).
RS_API int rs_cache_apply(void* handle, const long long* keys, const int* n_dev, long long n_cap, const float* grad, const float* norm,
                          int D, float lr, float eps, int optimizer, long long* missing_index, int* missing_count, cudaStream_t stream) {
  RS_REQUIRE(handle && keys && grad, "rs_cache_apply: null argument");
  CacheView& v = static_cast<CacheOwned*>(handle)->v;
  RS_REQUIRE(D % 4 == 0 && D > 0 && D + 1 <= v.dim, "rs_cache_apply: rows of %d weights need a cache of at least %d columns (has %d)", D, D + 1, v.dim);
  RS_REQUIRE(!missing_index || missing_count, "rs_cache_apply: the missing list needs a counter");
  if (n_cap == 0) return RS_OK;
  long long warps = n_cap < 148 * 32 ? n_cap : 148 * 32;
  cache_apply_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(v, keys, n_dev, n_cap, grad, norm, D, lr, eps, optimizer,
                                                                                missing_index, missing_count);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
RS_API int rs_cache_set_clock(void* handle, unsigned value, cudaStream_t stream) {
  RS_REQUIRE(handle, "rs_cache_set_clock: null handle");
  cache_set_clock_kernel<<<1, 1, 0, stream>>>(static_cast<CacheOwned*>(handle)->v.clock, value);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
// keys_out / values_out: room for the whole capacity; count: device int, cleared here.
RS_API int rs_cache_flush_dirty(void* handle, long long* keys_out, float* values_out, int* count, cudaStream_t stream) {
  RS_REQUIRE(handle && keys_out && values_out && count, "rs_cache_flush_dirty: null argument");
  CacheView& v = static_cast<CacheOwned*>(handle)->v;
  RS_CUDA(cudaMemsetAsync(count, 0, sizeof(int), stream));
  cache_flush_dirty_kernel<<<148 * 4, 256, 0, stream>>>(v, keys_out, values_out, count);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
// Query variant that does not advance the clock (the caller sets it with rs_cache_set_clock) and may skip the row copy
// (out == null: probe: stamps the hits, lists the misses).
RS_API int rs_cache_query_noclock(void* handle, const long long* keys, long long n, float* out, long long* miss_index,
                                  long long* miss_keys, int* miss_count, cudaStream_t stream) {
  RS_REQUIRE(handle && keys && miss_index && miss_keys && miss_count, "rs_cache_query_noclock: null argument");
  CacheView& v = static_cast<CacheOwned*>(handle)->v;
  RS_CUDA(cudaMemsetAsync(miss_count, 0, sizeof(int), stream));
  if (n == 0) return RS_OK;
  long long warps = (n + 3) / 4;
  if (warps > 148 * 32) warps = 148 * 32;
  cache_query_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(v, keys, n, out, miss_index, miss_keys, miss_count);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// out[missing_index[i]] = retrieved[i]  (the reference's merge_op, src/framework/pytorch/merge.cu:6-18)
namespace {
__global__ void merge_rows_kernel(float* __restrict__ out, const float* __restrict__ retrieved,
                                  const long long* __restrict__ missing_index, long long n, int dim) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  const int lane = threadIdx.x & 31;
  const long long d = missing_index[i];
  if ((dim & 3) == 0) {
    for (int v = lane; v < (dim >> 2); v += 32)
      reinterpret_cast<float4*>(out + d * dim)[v] = reinterpret_cast<const float4*>(retrieved + i * dim)[v];
  } else {
    for (int v = lane; v < dim; v += 32) out[d * dim + v] = retrieved[i * dim + v];
  }
}
// dst[i] = key in [start, end) ? hbm[key - start] : host_table[key]   (uva_cache_query_op,
// src/framework/pytorch/recstore_pytorch.cu:12-37); host_table is device-accessible host memory.
__global__ void range_cache_query_kernel(float* __restrict__ dst, const long long* __restrict__ ids, long long n, int dim,
                                         const float* __restrict__ hbm, const float* __restrict__ host_table, long long start,
                                         long long end, long long host_rows, unsigned long long* status) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  const int lane = threadIdx.x & 31;
  const long long k = ids[i];
  const float* src;
  bool host = false;
  if (k >= start && k < end) src = hbm + (k - start) * dim;
  else if (k >= 0 && k < host_rows) { src = host_table + k * dim; host = true; }
  else {
    if (lane == 0 && status) atomicOr(status, (unsigned long long)RS_DEV_OOB_ROW);
    return;
  }
  // Host rows are written by the CPU between kernels: they are read around the GPU's caches, every time.
  if ((dim & 3) == 0) {
    for (int v = lane; v < (dim >> 2); v += 32)
      reinterpret_cast<float4*>(dst + i * dim)[v] = host ? __ldcv(reinterpret_cast<const float4*>(src) + v) : reinterpret_cast<const float4*>(src)[v];
  } else {
    for (int v = lane; v < dim; v += 32) dst[i * dim + v] = host ? __ldcv(src + v) : src[v];
  }
}
}  // namespace

RS_API int rs_merge_rows(float* out, const float* retrieved, const long long* missing_index, long long n, int dim,
                         cudaStream_t stream) {
  RS_REQUIRE(out && retrieved && missing_index, "rs_merge_rows: null argument");
  if (n == 0) return RS_OK;
  merge_rows_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(out, retrieved, missing_index, n, dim);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
RS_API int rs_range_cache_query(float* dst, const long long* ids, long long n, int dim, const float* hbm,
                                const float* host_table, long long start, long long end, long long host_rows,
                                unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(dst && ids && hbm && host_table, "rs_range_cache_query: null argument");
  if (n == 0) return RS_OK;
  range_cache_query_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(dst, ids, n, dim, hbm, host_table, start,
                                                                                   end, host_rows, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
