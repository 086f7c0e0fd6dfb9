// HBM-resident open-addressing hash table: 64-bit key -> 32-bit row index of a dense row store.
//
// This is the device half of a KV shard.  It takes the place of the reference's GPU
// StaticHashTable (src/storage/gpu_cache/static_hash_table.cu:44-191) and of the CPU KV
// engines behind BaseKV (src/storage/kv_engine/base_kv.h:19-56) for rows that live in HBM,
// with erase (tombstones) and enumeration added so that shards can be checkpointed.
//
// Layout: capacity is a power of two; keys[] and rows[] are parallel arrays.  Linear probing
// from fmix64(key) & mask.  A slot is claimed with one 64-bit CAS on the key; the row index is
// published afterwards, readers that see the key but not yet the row spin a bounded number of
// times (insert and lookup of the same key inside one kernel launch is supported).
//
// Reserved keys: 0xFFFF...FF (-1, empty slot) and 0xFFFF...FE (-2, tombstone).  Insert, erase and unique refuse
// them (row / inverse -1, RS_DEV_BAD_ARG in the status word); lookup of either returns -1.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace rs {

constexpr unsigned long long kHtEmpty = 0xFFFFFFFFFFFFFFFFull;
constexpr unsigned long long kHtTomb = 0xFFFFFFFFFFFFFFFEull;
constexpr int kHtRowPending = -2;
constexpr int kHtMaxProbe = 1 << 14;

struct HashTableView {
  unsigned long long* keys;  // [capacity]
  int* rows;                 // [capacity] row index, kHtRowPending while being published
  unsigned long long mask;   // capacity - 1
  int* next_row;             // bump allocator for new rows
  int* free_rows;            // stack of erased rows available for reuse
  int* free_top;             // number of entries on the free stack
  int* size;                 // live keys
  int max_rows;              // capacity of the row store
};

__host__ __device__ __forceinline__ unsigned long long ht_hash(unsigned long long k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdull;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ull;
  k ^= k >> 33;
  return k;
}

// Waits (bounded, with back-off so that a publisher in the same warp can make progress) until the
// row of a claimed slot has been published.
__device__ __forceinline__ int ht_wait_row(const int* p) {
  int r = __ldcv(p);
  for (int spin = 0; r == kHtRowPending && spin < (1 << 18); ++spin) {
    __nanosleep(spin < 64 ? 20 : 200);
    r = __ldcv(p);
  }
  return r == kHtRowPending ? -1 : r;
}

// Returns the row of `key`, or -1 when absent.
__device__ __forceinline__ int ht_find(const HashTableView& t, unsigned long long key) {
  if (key >= kHtTomb) return -1;
  unsigned long long s = ht_hash(key) & t.mask;
  for (int p = 0; p < kHtMaxProbe; ++p) {
    const unsigned long long k = __ldcv(&t.keys[s]);
    if (k == key) {
      return ht_wait_row(&t.rows[s]);
    }
    if (k == kHtEmpty) return -1;
    s = (s + 1) & t.mask;
  }
  return -1;
}

// Find-or-insert.  Returns the row, or -1 when the table or the row store is full
// (and sets *full).  `inserted` tells whether this call created the key.
// Only EMPTY slots are claimed (tombstones are skipped and reclaimed by a rebuild), so all
// concurrent inserters of one key contend for the same slot and no duplicate can appear.
// rows[] holds kHtRowPending for every slot that has no published row (set at clear time).
// Inserts and erases must not run concurrently.
__device__ __forceinline__ int ht_insert(const HashTableView& t, unsigned long long key, bool* inserted,
                                         bool* full) {
  *inserted = false;
  unsigned long long s = ht_hash(key) & t.mask;
  for (int p = 0; p < kHtMaxProbe; ++p) {
    unsigned long long k = __ldcv(&t.keys[s]);
    if (k == kHtEmpty) {
      const unsigned long long prev = atomicCAS(&t.keys[s], kHtEmpty, key);
      if (prev == kHtEmpty) {
        int row = -1;
        const int top = atomicSub(t.free_top, 1);
        if (top > 0) {
          row = t.free_rows[top - 1];
        } else {
          atomicAdd(t.free_top, 1);
          row = atomicAdd(t.next_row, 1);
          if (row >= t.max_rows) {
            atomicSub(t.next_row, 1);
            row = -1;
          }
        }
        if (row < 0) {
          atomicExch(&t.keys[s], kHtTomb);  // row store exhausted: give the slot up
          *full = true;
          return -1;
        }
        atomicExch(&t.rows[s], row);
        atomicAdd(t.size, 1);
        *inserted = true;
        return row;
      }
      k = prev;  // somebody claimed it first: fall through and compare
    }
    if (k == key) {
      return ht_wait_row(&t.rows[s]);
    }
    s = (s + 1) & t.mask;
  }
  *full = true;
  return -1;
}

// Removes `key`; returns its former row or -1.
__device__ __forceinline__ int ht_erase(const HashTableView& t, unsigned long long key) {
  unsigned long long s = ht_hash(key) & t.mask;
  for (int p = 0; p < kHtMaxProbe; ++p) {
    const unsigned long long k = __ldcv(&t.keys[s]);
    if (k == key) {
      const int r = __ldcv(&t.rows[s]);
      if (atomicCAS(&t.keys[s], key, kHtTomb) == key) {
        atomicExch(&t.rows[s], kHtRowPending);
        const int top = atomicAdd(t.free_top, 1);
        t.free_rows[top] = r;
        atomicSub(t.size, 1);
        return r;
      }
      return -1;
    }
    if (k == kHtEmpty) return -1;
    s = (s + 1) & t.mask;
  }
  return -1;
}

}  // namespace rs
