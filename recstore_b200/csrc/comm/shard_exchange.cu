// Key / row / gradient exchange for ROW-SHARDED embedding tables over peer windows (NVLink stores).
//
// A table of N rows is spread cyclically over `world` GPUs: owner(id) = id % world, local row =
// id / world (or a hash-table probe on the owner).  One lookup on rank `me`:
//   1. bucket_push_keys:  histogram the ids per owner, then every id is written STRAIGHT INTO THE
//      OWNER'S key window at region [me] (slot p inside the region from an atomic cursor); slot[i]
//      remembers (owner, p).  A tiny kernel then delivers the per-owner counts.
//   2. gather_push_rows (on every owner, after the key flags): for each source rank s and each
//      received key, read the row of the local shard and store it STRAIGHT INTO RANK s's row window
//      at region [me], same slot; also note the local row for the backward pass.
//   3. unbucket_rows (requester, after the row flags): out[i] = row_window[slot[i]].
// Backward: push_grads writes grad[i] into the owner's gradient window at slot[i]; the owner then
// runs the fused segment-reduce + optimizer kernel (rs_emb_backward) over the noted local rows.
//
// This is the reference's KnownShardedCachedEmbedding exchange (bucket keys by owner -> exchange
// keys -> local gather -> exchange rows; backward exchanges (keys, grads);
// src/python/pytorch/recstore/cache/sharded_cache.py:181-345) and its pinned-CPU staged
// all2all_data_transfer (recstore/utils.py:227-310) done by three kernels and peer stores, with no
// host staging, no pack / unpack and no collective call.
#include <cuda_bf16.h>
#include <cstdlib>

#include "comm/flags.cuh"
#include "common/rs_common.h"
#include "kv/hash_table.cuh"

namespace {

constexpr int kMaxWorld = 32;

__global__ void bucket_count_kernel(const long long* __restrict__ keys, long long n, int world, int* __restrict__ counts) {
  __shared__ int h[kMaxWorld];
  if (threadIdx.x < kMaxWorld) h[threadIdx.x] = 0;
  __syncthreads();
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long k = keys[i];
    if (k >= 0) atomicAdd(&h[static_cast<int>(k % world)], 1);
  }
  __syncthreads();
  if (threadIdx.x < world && h[threadIdx.x]) atomicAdd(&counts[threadIdx.x], h[threadIdx.x]);
}

// cursor[d] must be zero on entry.  slot[i] = d * cap + p, or -1 for a negative key / full region.
__global__ void bucket_push_keys_kernel(const long long* __restrict__ keys, long long n, int world, int me, long long cap,
                                        int* __restrict__ cursor, long long* const* __restrict__ key_win,
                                        long long* __restrict__ slot, unsigned long long* status) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long k = keys[i];
  if (k < 0) { slot[i] = -1; return; }
  const int d = static_cast<int>(k % world);
  const int p = atomicAdd(&cursor[d], 1);
  if (p >= cap) {
    if (status) atomicOr(status, (unsigned long long)RS_DEV_OOB_PEER);
    slot[i] = -1;
    return;
  }
  key_win[d][static_cast<long long>(me) * cap + p] = k;
  slot[i] = static_cast<long long>(d) * cap + p;
}

// Delivers counts[d] (clamped to cap) to rank d's count window at [me] and clears the cursors for the next call.
__global__ void push_counts_kernel(int* counts, int* cursor, int world, int me, long long cap, int* const* count_win) {
  const int d = threadIdx.x;
  if (d < world) {
    const int c = counts[d] < cap ? counts[d] : static_cast<int>(cap);
    count_win[d][me] = c;
    counts[d] = 0;
    cursor[d] = 0;
  }
}

struct GatherArgs {
  const float* weight;              // local shard [local_rows, D] (or its first hot_rows rows)
  const float* cold_weight;         // rows [hot_rows, local_rows) in device-visible host memory, or null
  long long hot_rows;
  long long local_rows;
  const long long* key_win;         // my key window   [world, cap]
  const int* count_win;             // my count window [world]
  float* const* row_win;            // peers' row windows, each [world, cap, D]
  long long* rowidx;                // [world, cap] local row of every received key (-1 = none)
  int world, me, D;
  long long cap;
  int use_hash;
  rs::HashTableView ht;
  unsigned long long* status;
};

// one warp per (source rank, slot)
__global__ void __launch_bounds__(256) gather_push_rows_kernel(const GatherArgs a) {
  const long long w = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(a.world) * a.cap) return;
  const int s = static_cast<int>(w / a.cap);
  const long long p = w % a.cap;
  if (p >= a.count_win[s]) {
    if (lane == 0) a.rowidx[w] = -1;
    return;
  }
  const long long k = a.key_win[w];
  long long r;
  if (a.use_hash) r = rs::ht_find(a.ht, static_cast<unsigned long long>(k));
  else r = k / a.world;
  if (r < 0 || r >= a.local_rows) {
    if (!a.use_hash && lane == 0 && a.status) atomicOr(a.status, (unsigned long long)RS_DEV_OOB_ROW);
    r = -1;
  }
  if (lane == 0) a.rowidx[w] = r;
  float* dst = a.row_win[s] + (static_cast<long long>(a.me) * a.cap + p) * a.D;
  for (int v = lane; v < (a.D >> 2); v += 32) {
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r >= 0) {
      if (r < a.hot_rows) x = __ldg(reinterpret_cast<const float4*>(a.weight + r * a.D) + v);
      else x = __ldcv(reinterpret_cast<const float4*>(a.cold_weight + (r - a.hot_rows) * a.D) + v);   // host tier, read in place
    }
    reinterpret_cast<float4*>(dst)[v] = x;
  }
}

// out[i] = row_win[slot[i]] (zeros for slot < 0); out may be fp32 or bf16.
__global__ void __launch_bounds__(256) unbucket_rows_kernel(const float* __restrict__ row_win, const long long* __restrict__ slot,
                                                            long long n, int D, void* __restrict__ out, int out_bf16) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  const int lane = threadIdx.x & 31;
  const long long s = slot[i];
  for (int v = lane; v < (D >> 2); v += 32) {
    const float4 x = s >= 0 ? reinterpret_cast<const float4*>(row_win + s * D)[v] : make_float4(0.f, 0.f, 0.f, 0.f);
    if (out_bf16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + i * D)[v] = o;
    } else {
      reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + i * D)[v] = x;
    }
  }
}

// grad_win[owner][me * cap + p] = grad[i]
__global__ void __launch_bounds__(256) push_grads_kernel(const float* __restrict__ grad, const long long* __restrict__ slot,
                                                         long long n, int D, int me, long long cap,
                                                         float* const* __restrict__ grad_win, const float* __restrict__ norm,
                                                         float* const* __restrict__ norm_win) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  const int lane = threadIdx.x & 31;
  const long long s = slot[i];
  if (s < 0) return;
  const int d = static_cast<int>(s / cap);
  const long long p = s % cap;
  float* dst = grad_win[d] + (static_cast<long long>(me) * cap + p) * D;
  for (int v = lane; v < (D >> 2); v += 32) reinterpret_cast<float4*>(dst)[v] = __ldg(reinterpret_cast<const float4*>(grad + i * D) + v);
  if (norm && lane == 0) norm_win[d][static_cast<long long>(me) * cap + p] = norm[i];
}

// ugrad[inverse[i]] += grad[i], unorm[inverse[i]] += |grad[i]|^2   (segment-sum of duplicate keys before the
// exchange; both outputs zeroed by the caller).  The separate sum of squares keeps row-wise Adagrad exact:
// its state needs the sum over occurrences of mean(g^2), not the square of the summed gradient.
// occ_norm (optional): the squared norm to account for occurrence i instead of |grad[i]|^2 (a caller whose rows are
// slices of a wider object, e.g. the rows of a relation matrix, passes the norm of the whole object).
__global__ void __launch_bounds__(256) segment_sum_kernel(const float* __restrict__ grad, const int* __restrict__ inverse,
                                                          long long n, int D, float* __restrict__ ugrad, float* __restrict__ unorm,
                                                          const float* __restrict__ occ_norm) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  const int lane = threadIdx.x & 31;
  const int u = inverse[i];
  if (u < 0) return;
  float sq = 0.f;
  for (int v = lane; v < (D >> 2); v += 32) {
    const float4 g = __ldg(reinterpret_cast<const float4*>(grad + i * D) + v);
    sq += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
    atomicAdd(reinterpret_cast<float4*>(ugrad + static_cast<long long>(u) * D) + v, g);
  }
  if (unorm) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if (lane == 0) atomicAdd(&unorm[u], occ_norm ? occ_norm[i] : sq);
  }
}

// The same sum with duplicates combined inside the CTA first.  With skewed keys the plain kernel sends tens of
// thousands of atomics to the hottest row (47,000 of 262,144 occurrences at Zipf 1.1: they serialise in L2 and set the
// kernel's time).  Here a CTA takes 512 occurrences, counts its distinct keys in a shared-memory hash table, gives every
// key that occurs more than once a row in shared memory, adds those occurrences there (shared-memory atomics) and sends
// ONE global atomic per such key; keys that occur once in the chunk, or that found no free row, go to global memory
// directly, so a batch without duplicates pays only the counting pass.
constexpr int kSegChunk = 512, kSegSlots = 1024, kSegMaxRows = 64;
__device__ __forceinline__ unsigned seg_hash(int u) { return (static_cast<unsigned>(u) * 2654435761u) >> 22; }   // 10 bits

__global__ void __launch_bounds__(256) segment_sum_combine_kernel(const float* __restrict__ grad, const int* __restrict__ inverse,
                                                                  long long n, int D, int R, float* __restrict__ ugrad,
                                                                  float* __restrict__ unorm, const float* __restrict__ occ_norm) {
  extern __shared__ __align__(16) unsigned char seg_smem[];
  int* hkey = reinterpret_cast<int*>(seg_smem);            // [kSegSlots] unique index or -1
  int* hcnt = hkey + kSegSlots;                            // [kSegSlots] occurrences in this chunk
  int* hrow = hcnt + kSegSlots;                            // [kSegSlots] shared row of the key or -1
  int* rkey = hrow + kSegSlots;                            // [kSegMaxRows] unique index of a shared row
  float* rnorm = reinterpret_cast<float*>(rkey + kSegMaxRows);   // [kSegMaxRows]
  float* rows = rnorm + kSegMaxRows;                       // [R, D]
  __shared__ int nrow;
  const long long c0 = static_cast<long long>(blockIdx.x) * kSegChunk;
  const int cn = static_cast<int>(min(static_cast<long long>(kSegChunk), n - c0));
  for (int s = threadIdx.x; s < kSegSlots; s += blockDim.x) { hkey[s] = -1; hcnt[s] = 0; }
  for (int v = threadIdx.x; v < R * D; v += blockDim.x) rows[v] = 0.f;
  for (int r = threadIdx.x; r < kSegMaxRows; r += blockDim.x) rnorm[r] = 0.f;
  if (threadIdx.x == 0) nrow = 0;
  __syncthreads();
  // 1: count the distinct keys of the chunk
  for (int j = threadIdx.x; j < cn; j += blockDim.x) {
    const int u = inverse[c0 + j];
    if (u < 0) continue;
    unsigned s = seg_hash(u);
    for (int probe = 0; probe < kSegSlots; ++probe, s = (s + 1) & (kSegSlots - 1)) {
      const int prev = atomicCAS(&hkey[s], -1, u);
      if (prev == -1 || prev == u) { atomicAdd(&hcnt[s], 1); break; }
    }
  }
  __syncthreads();
  // 2: a shared row for every key that occurs more than once (while rows last)
  for (int s = threadIdx.x; s < kSegSlots; s += blockDim.x) {
    int r = -1;
    if (hcnt[s] > 1) {
      r = atomicAdd(&nrow, 1);
      if (r < R) rkey[r] = hkey[s];
      else r = -1;
    }
    hrow[s] = r;
  }
  __syncthreads();
  // 3: add every occurrence to its shared row, or straight to global memory (four occurrences in flight per warp)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int nvec = D >> 2;                                  // D <= 128: one float4 per lane
  for (int j0 = warp * 4; j0 < cn; j0 += nwarp * 4) {
    int u[4], r[4];
    float4 g[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int j = j0 + q;
      u[q] = j < cn ? inverse[c0 + j] : -1;
      g[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (u[q] >= 0 && lane < nvec) g[q] = __ldg(reinterpret_cast<const float4*>(grad + (c0 + j) * D) + lane);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (u[q] < 0) continue;
      unsigned s = seg_hash(u[q]);
      while (hkey[s] != u[q]) s = (s + 1) & (kSegSlots - 1);
      r[q] = hrow[s];
      float sq = g[q].x * g[q].x + g[q].y * g[q].y + g[q].z * g[q].z + g[q].w * g[q].w;
      if (lane < nvec) {
        if (r[q] >= 0) {
          float* d = rows + r[q] * D + lane * 4;
          atomicAdd(d, g[q].x); atomicAdd(d + 1, g[q].y); atomicAdd(d + 2, g[q].z); atomicAdd(d + 3, g[q].w);
        } else {
          atomicAdd(reinterpret_cast<float4*>(ugrad + static_cast<long long>(u[q]) * D) + lane, g[q]);
        }
      }
      if (unorm) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) {
          if (occ_norm) sq = occ_norm[c0 + j0 + q];
          if (r[q] >= 0) atomicAdd(&rnorm[r[q]], sq);
          else atomicAdd(&unorm[u[q]], sq);
        }
      }
    }
  }
  __syncthreads();
  // 4: one global atomic per combined key
  const int used = min(nrow, R);
  for (int r = warp; r < used; r += nwarp) {
    const int u = rkey[r];
    for (int v = lane; v < (D >> 2); v += 32)
      atomicAdd(reinterpret_cast<float4*>(ugrad + static_cast<long long>(u) * D) + v, *reinterpret_cast<const float4*>(rows + r * D + v * 4));
    if (unorm && lane == 0) atomicAdd(&unorm[u], rnorm[r]);
  }
}

// out[i] = src[inverse[i]]
__global__ void __launch_bounds__(256) expand_rows_kernel(const float* __restrict__ src, const int* __restrict__ inverse, long long n,
                                                          int D, float* __restrict__ out) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  const int lane = threadIdx.x & 31;
  const int u = inverse[i];
  for (int v = lane; v < (D >> 2); v += 32)
    reinterpret_cast<float4*>(out + i * D)[v] = u >= 0 ? reinterpret_cast<const float4*>(src + static_cast<long long>(u) * D)[v]
                                                       : make_float4(0.f, 0.f, 0.f, 0.f);
}

inline unsigned warps_grid(long long n) { return static_cast<unsigned>((n + 7) / 8); }
}  // namespace

// counts / cursor: device int[world] scratch, zero before the first call (kept zero by the call itself).
RS_API int rs_shard_push_keys(const long long* keys, long long n, int world, int me, long long cap, int* counts, int* cursor,
                              void* const* key_win, void* const* count_win, long long* slot, unsigned long long* status,
                              cudaStream_t stream) {
  RS_REQUIRE(keys && counts && cursor && key_win && count_win && slot, "rs_shard_push_keys: null argument");
  RS_REQUIRE(world >= 1 && world <= kMaxWorld && n <= cap * world, "rs_shard_push_keys: bad sizes");
  if (n > 0) {
    int grid = static_cast<int>((n + 255) / 256);
    bucket_count_kernel<<<grid > 592 ? 592 : grid, 256, 0, stream>>>(keys, n, world, counts);
    RS_LAUNCH_CHECK();
    bucket_push_keys_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
        keys, n, world, me, cap, cursor, reinterpret_cast<long long* const*>(key_win), slot, status);
    RS_LAUNCH_CHECK();
  }
  push_counts_kernel<<<1, 32, 0, stream>>>(counts, cursor, world, me, cap, reinterpret_cast<int* const*>(count_win));
  RS_LAUNCH_CHECK();
  return RS_OK;
}

namespace {
int launch_gather(const float* weight, const float* cold_weight, long long hot_rows, long long local_rows, const long long* key_win,
                  const int* count_win, void* const* row_win, long long* rowidx, int world, int me, int D, long long cap,
                  const rs::HashTableView* ht, unsigned long long* status, cudaStream_t stream);
}  // namespace

RS_API int rs_shard_gather_push_rows(const float* weight, long long local_rows, const long long* key_win, const int* count_win,
                                     void* const* row_win, long long* rowidx, int world, int me, int D, long long cap,
                                     const rs::HashTableView* ht, unsigned long long* status, cudaStream_t stream) {
  return launch_gather(weight, nullptr, local_rows, local_rows, key_win, count_win, row_win, rowidx, world, me, D, cap, ht, status, stream);
}

// Same with a two-tier shard: rows [0, hot_rows) at `weight` (HBM), rows [hot_rows, local_rows) at `cold_weight`
// (pinned host memory, device-visible).
RS_API int rs_shard_gather_push_rows_tiered(const float* weight, const float* cold_weight, long long hot_rows, long long local_rows,
                                            const long long* key_win, const int* count_win, void* const* row_win, long long* rowidx,
                                            int world, int me, int D, long long cap, unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(hot_rows >= 0 && hot_rows <= local_rows && (hot_rows == local_rows || cold_weight), "rs_shard_gather_push_rows_tiered: bad tiers");
  return launch_gather(weight, cold_weight, hot_rows, local_rows, key_win, count_win, row_win, rowidx, world, me, D, cap, nullptr, status, stream);
}

namespace {
int launch_gather(const float* weight, const float* cold_weight, long long hot_rows, long long local_rows, const long long* key_win,
                  const int* count_win, void* const* row_win, long long* rowidx, int world, int me, int D, long long cap,
                  const rs::HashTableView* ht, unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE((weight || hot_rows == 0) && key_win && count_win && row_win && rowidx && D % 4 == 0, "rs_shard_gather_push_rows: bad argument");
  GatherArgs a;
  a.weight = weight; a.cold_weight = cold_weight; a.hot_rows = hot_rows; a.local_rows = local_rows; a.key_win = key_win; a.count_win = count_win;
  a.row_win = reinterpret_cast<float* const*>(row_win); a.rowidx = rowidx; a.world = world; a.me = me; a.D = D; a.cap = cap;
  a.use_hash = ht != nullptr;
  if (ht) a.ht = *ht; else memset(&a.ht, 0, sizeof(a.ht));
  a.status = status;
  gather_push_rows_kernel<<<warps_grid(static_cast<long long>(world) * cap), 256, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
}  // namespace

RS_API int rs_shard_unbucket_rows(const float* row_win, const long long* slot, long long n, int D, void* out, int out_bf16,
                                  cudaStream_t stream) {
  RS_REQUIRE(row_win && slot && out && D % 4 == 0, "rs_shard_unbucket_rows: bad argument");
  if (n == 0) return RS_OK;
  unbucket_rows_kernel<<<warps_grid(n), 256, 0, stream>>>(row_win, slot, n, D, out, out_bf16);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// norm / norm_win (optional): per-row sum of squares delivered next to the gradients ([world, cap] fp32 windows).
RS_API int rs_shard_push_grads(const float* grad, const long long* slot, long long n, int D, int me, long long cap,
                               void* const* grad_win, const float* norm, void* const* norm_win, cudaStream_t stream) {
  RS_REQUIRE(grad && slot && grad_win && D % 4 == 0, "rs_shard_push_grads: bad argument");
  if (n == 0) return RS_OK;
  push_grads_kernel<<<warps_grid(n), 256, 0, stream>>>(grad, slot, n, D, me, cap, reinterpret_cast<float* const*>(grad_win), norm,
                                                       reinterpret_cast<float* const*>(norm_win));
  RS_LAUNCH_CHECK();
  return RS_OK;
}

namespace {
int segment_sum_impl(const float* grad, const int* inverse, long long n, int D, float* ugrad, float* unorm, const float* occ_norm,
                     cudaStream_t stream) {
  RS_REQUIRE(grad && inverse && ugrad && D % 4 == 0, "rs_segment_sum: bad argument");
  RS_REQUIRE(!occ_norm || unorm, "rs_segment_sum: per-occurrence norms need the norm output");
  if (n == 0) return RS_OK;
  // RECSTORE_SEGMENT_SUM=direct keeps the one-atomic-per-occurrence kernel (A/B); rows wider than 128 floats use it too.
  static const bool combine = [] { const char* e = getenv("RECSTORE_SEGMENT_SUM"); return !(e && e[0] == 'd'); }();
  if (combine && D <= 128 && n >= 131072) {   // measured: below ~100 k occurrences the four passes inside a CTA cost more than the hot atomics
    int R = (32 * 1024) / (D * 4);
    if (R > kSegMaxRows) R = kSegMaxRows;
    const size_t smem = static_cast<size_t>(kSegSlots) * 12 + kSegMaxRows * 8 + static_cast<size_t>(R) * D * 4;
    static bool attr_done = false;
    if (!attr_done) {
      RS_CUDA(cudaFuncSetAttribute(segment_sum_combine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      attr_done = true;
    }
    const unsigned grid = static_cast<unsigned>((n + kSegChunk - 1) / kSegChunk);
    segment_sum_combine_kernel<<<grid, 256, smem, stream>>>(grad, inverse, n, D, R, ugrad, unorm, occ_norm);
  } else {
    segment_sum_kernel<<<warps_grid(n), 256, 0, stream>>>(grad, inverse, n, D, ugrad, unorm, occ_norm);
  }
  RS_LAUNCH_CHECK();
  return RS_OK;
}
}  // namespace

RS_API int rs_segment_sum(const float* grad, const int* inverse, long long n, int D, float* ugrad, float* unorm,
                          cudaStream_t stream) {
  return segment_sum_impl(grad, inverse, n, D, ugrad, unorm, nullptr, stream);
}
// occ_norm [n]: squared norm accounted for every occurrence instead of |grad[i]|^2.
RS_API int rs_segment_sum_ex(const float* grad, const int* inverse, long long n, int D, float* ugrad, float* unorm,
                             const float* occ_norm, cudaStream_t stream) {
  return segment_sum_impl(grad, inverse, n, D, ugrad, unorm, occ_norm, stream);
}

RS_API int rs_expand_rows(const float* src, const int* inverse, long long n, int D, float* out, cudaStream_t stream) {
  RS_REQUIRE(src && inverse && out && D % 4 == 0, "rs_expand_rows: bad argument");
  if (n == 0) return RS_OK;
  expand_rows_kernel<<<warps_grid(n), 256, 0, stream>>>(src, inverse, n, D, out);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// ------------------------------------------------------------------------------------------------------------------
// Fused forms: three launches per lookup and two per gradient exchange, flags published and awaited inside the kernels
// (comm/flags.cuh), no count / signal / wait launches in between.
//   rs_shard_keys_fused     bucket + push keys (block-aggregated slot assignment), last block delivers the per-owner counts
//                           and publishes CH_KEYS
//   rs_shard_gather_fused   owner side: waits for each source's keys, resolves them (cyclic index, or find-or-insert in the
//                           shard's hash table with a key-derived initial row), pushes the rows back, records a COMPACT
//                           (row, slot) occurrence list for the optimizer, publishes CH_ROWS
//   rs_shard_unbucket_fused waits for the rows, writes out[i] = row_window[slot[inverse[i]]] (unbucket + expand in one pass)
//                           and clears the per-key gradient accumulators for the update that follows
//   rs_shard_grads_fused    pushes per-key gradient sums and squared norms to the owners, publishes CH_GRADS
namespace {
using rs::FlagSignal;
using rs::FlagWait;

struct KeysFusedArgs {
  const long long* keys;     // [n]; negative = padding
  const int* n_dev;          // optional live count (<= n)
  long long n;
  int world, me;
  long long cap;
  int* cursor;               // [world], zero on entry, zero again on exit
  long long* const* key_win;
  int* const* count_win;
  long long* slot;           // [n]
  unsigned long long* status;
  long long range_c;         // 0: owner = key % world; > 0: owner = key / range_c for key < world * range_c, else nobody
  FlagSignal sig;            //    (such a key gets slot -2: its row lives in the host table)
};

__global__ void __launch_bounds__(256) shard_keys_fused_kernel(const KeysFusedArgs a) {
  __shared__ int s_cnt[kMaxWorld];    // keys of this block per owner
  __shared__ int s_base[kMaxWorld];   // first slot of this block in each owner's region
  __shared__ uint32_t s_epoch;
  const int tid = threadIdx.x, lane = tid & 31;
  if (tid < kMaxWorld) s_cnt[tid] = 0;
  __syncthreads();
  const long long n = a.n_dev ? min(static_cast<long long>(*a.n_dev), a.n) : a.n;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + tid;
  long long k = -1;
  if (i < n) k = a.keys[i];
  int d = -1;
  bool host_row = false;
  if (k >= 0) {
    if (a.range_c <= 0) d = static_cast<int>(k % a.world);
    else if (k < a.range_c * a.world) d = static_cast<int>(k / a.range_c);
    else host_row = true;
  }
  // rank of this key among the block's keys for the same owner: warp ballot + one shared atomic per (warp, owner)
  int pos = 0;
  for (int dd = 0; dd < a.world; ++dd) {
    const unsigned m = __ballot_sync(0xffffffffu, d == dd);
    if (m == 0u) continue;
    int wbase = 0;
    if (lane == __ffs(m) - 1) wbase = atomicAdd(&s_cnt[dd], __popc(m));
    wbase = __shfl_sync(0xffffffffu, wbase, __ffs(m) - 1);
    if (d == dd) pos = wbase + __popc(m & ((1u << lane) - 1u));
  }
  __syncthreads();
  if (tid < a.world) s_base[tid] = s_cnt[tid] ? atomicAdd(&a.cursor[tid], s_cnt[tid]) : 0;
  __syncthreads();
  if (i < a.n) {
    long long sl = host_row ? -2 : -1;
    if (d >= 0) {
      const long long p = static_cast<long long>(s_base[d]) + pos;
      if (p < a.cap) {
        a.key_win[d][static_cast<long long>(a.me) * a.cap + p] = k;
        sl = static_cast<long long>(d) * a.cap + p;
      } else if (a.status) {
        atomicOr(a.status, (unsigned long long)RS_DEV_OOB_PEER);
      }
    }
    a.slot[i] = sl;
  }
  // last block: counts to the owners, cursors back to zero, then the flag
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(a.sig.done, 1u);
    uint32_t e = 0;
    if (prev == gridDim.x - 1) {
      *a.sig.done = 0;
      e = ++a.sig.sig_counters[a.sig.channel];
      if (e == 0) e = ++a.sig.sig_counters[a.sig.channel];
    }
    s_epoch = e;
  }
  __syncthreads();
  if (s_epoch != 0 && tid < a.world) {
    __threadfence_system();
    const int c = *reinterpret_cast<volatile int*>(&a.cursor[tid]);
    a.count_win[tid][a.me] = c < a.cap ? c : static_cast<int>(a.cap);
    a.cursor[tid] = 0;
    __threadfence_system();
    if (a.sig.flags_of) rs::ptx::st_release_sys(a.sig.flags_of[tid] + a.sig.channel * a.sig.world + a.sig.me, s_epoch);
  }
}

// Initial value of a row that the hash-table shard sees for the first time: uniform in [-scale, scale), a function of the key
// and the column only, so a table does not depend on the order in which its keys arrive.
__device__ __forceinline__ float key_init_value(unsigned long long key, int col, float scale) {
  const unsigned long long h = rs::ht_hash(key * 0x9E3779B97F4A7C15ull + static_cast<unsigned long long>(col) + 1ull);
  return (static_cast<float>(h >> 40) * (1.0f / 16777216.0f) * 2.f - 1.f) * scale;
}

struct GatherFusedArgs {
  float* weight;                    // local shard rows (HBM tier)
  const float* cold_weight;         // rows [hot_rows, local_rows) in device-visible host memory, or null
  long long hot_rows, local_rows;
  const long long* key_win;         // my key window [world, cap]
  const int* count_win;             // my count window [world]
  float* const* row_win;            // peers' row windows [world, cap, D]
  long long* rowidx;                // [world, cap] local row per received key (-1 = none), or null
  long long* occ_row;               // compact occurrence list: local row ...
  int* occ_slot;                    // ... and its slot (index into the [world, cap] windows)
  int* occ_cursor;                  // zero on entry
  int world, me, D;
  long long cap;
  int use_hash;
  rs::HashTableView ht;
  long long range_c;                // > 0: this rank holds keys [me * range_c, (me + 1) * range_c), local row = key - me * range_c
  int push_rows;                    // 0: only resolve rows and record occurrences (a gradient exchange without a lookup)
  int find_only;                    // hash mode: 1 = never insert; an absent key answers with a NaN in column 0 (then zeros)
  float init_scale;
  unsigned char* row_init;          // hash mode: 1 once a row holds its initial value (readers that come earlier compute it)
  unsigned long long* status;
  FlagWait wait;
  FlagSignal sig;
};

// Persistent warps: source rank s = 0..world-1 in turn (waiting for its flag first), slots p = warp, warp + nwarps, ...
__global__ void __launch_bounds__(128) shard_gather_fused_kernel(const GatherFusedArgs a) {
  const int lane = threadIdx.x & 31;
  const long long warp = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const int nvec = a.D >> 2;
  for (int si = 0; si < a.world; ++si) {
    const int s = (a.me + si) % a.world;                 // start with my own keys (already here)
    rs::flag_wait_one_warp(a.wait, s);
    const int cnt = __ldcv(a.count_win + s);
    if (a.rowidx)   // the [world, cap] view (two-tier update): slots past this step's count hold nothing
      for (long long p = cnt + warp * 32 + lane; p < a.cap; p += nwarps * 32) a.rowidx[static_cast<long long>(s) * a.cap + p] = -1;
    for (long long p = warp; p < cnt; p += nwarps) {
      const long long w = static_cast<long long>(s) * a.cap + p;
      const long long k = __ldcv(a.key_win + w);
      long long r = -1;
      bool fresh = false;
      if (a.use_hash) {
        if (lane == 0) {
          if (a.find_only) {
            r = rs::ht_find(a.ht, static_cast<unsigned long long>(k));
          } else {
            bool ins = false, full = false;
            r = rs::ht_insert(a.ht, static_cast<unsigned long long>(k), &ins, &full);
            if (full && a.status) atomicOr(a.status, (unsigned long long)RS_DEV_TABLE_FULL);
            fresh = ins;
          }
        }
        r = __shfl_sync(0xffffffffu, r, 0);
        fresh = __shfl_sync(0xffffffffu, static_cast<int>(fresh), 0) != 0;
      } else {
        r = a.range_c > 0 ? k - static_cast<long long>(a.me) * a.range_c : k / a.world;
      }
      if (r < 0 || r >= a.local_rows) {
        if (!a.use_hash && lane == 0 && a.status) atomicOr(a.status, (unsigned long long)RS_DEV_OOB_ROW);
        r = -1;
      }
      const bool absent = a.find_only && r < 0;
      if (lane == 0) {
        if (a.rowidx) a.rowidx[w] = r;
        if (a.occ_cursor && r >= 0) {
          const int q = atomicAdd(a.occ_cursor, 1);
          a.occ_row[q] = r;
          a.occ_slot[q] = static_cast<int>(w);
        }
      }
      if (!a.push_rows && !fresh) continue;      // (a key seen for the first time gets its initial row even when nothing is sent back)
      // A key that another warp inserted a moment ago may not hold its initial value yet: such a reader computes the same
      // value from the key instead of reading the row.
      bool by_formula = fresh;
      if (a.use_hash && r >= 0 && !fresh) by_formula = *reinterpret_cast<volatile unsigned char*>(a.row_init + r) == 0;
      float* dst = a.row_win[s] + (static_cast<long long>(a.me) * a.cap + p) * a.D;
      for (int v = lane; v < nvec; v += 32) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r >= 0) {
          if (by_formula) {
            x = make_float4(key_init_value(k, v * 4, a.init_scale), key_init_value(k, v * 4 + 1, a.init_scale),
                            key_init_value(k, v * 4 + 2, a.init_scale), key_init_value(k, v * 4 + 3, a.init_scale));
            if (fresh) reinterpret_cast<float4*>(a.weight + r * a.D)[v] = x;   // first touch: the row keeps it
          } else if (r < a.hot_rows) {
            x = __ldcg(reinterpret_cast<const float4*>(a.weight + r * a.D) + v);
          } else {
            x = __ldcv(reinterpret_cast<const float4*>(a.cold_weight + (r - a.hot_rows) * a.D) + v);   // host tier, read in place
          }
        }
        if (absent && v == 0) x.x = __int_as_float(0x7fc00000);   // "no such key"
        if (a.push_rows) reinterpret_cast<float4*>(dst)[v] = x;
      }
      if (fresh) {
        __syncwarp();
        if (lane == 0) {
          __threadfence();
          *reinterpret_cast<volatile unsigned char*>(a.row_init + r) = 1;
        }
      }
    }
  }
  rs::flag_publish_when_grid_done(a.sig);
}

struct UnbucketFusedArgs {
  const float* row_win;        // my row window [world, cap, D]
  const long long* slot;       // [n_unique]
  const int* inverse;          // [n] or null (then out[i] = row_win[slot[i]])
  long long n;
  int D;
  void* out;
  int out_bf16;
  float* ugrad;                // optional: cleared for u < *ucount (per-key gradient accumulators of the coming update)
  float* unorm;
  const int* ucount;
  const long long* keys;       // the (unique) keys: a slot of -2 means "row keys[u] of the host table"
  const float* host_table;     // device-visible host memory, read in place, or null
  long long host_rows;
  unsigned long long* status;
  FlagWait wait;
};

__global__ void __launch_bounds__(128) shard_unbucket_fused_kernel(const UnbucketFusedArgs a) {
  rs::flag_wait_all(a.wait);
  const int lane = threadIdx.x & 31;
  const long long nwarps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const int nvec = a.D >> 2;
  const long long nu = a.ucount ? *a.ucount : 0;
  for (long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); i < a.n; i += nwarps) {
    const long long u = a.inverse ? a.inverse[i] : i;
    const long long s = u >= 0 ? a.slot[u] : -1;
    const float* host_src = nullptr;
    if (s == -2 && a.host_table != nullptr) {
      const long long k = a.keys[u];
      if (k >= 0 && k < a.host_rows) host_src = a.host_table + k * a.D;
      else if (lane == 0 && a.status) atomicOr(a.status, (unsigned long long)RS_DEV_OOB_ROW);
    }
    for (int v = lane; v < nvec; v += 32) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (s >= 0) x = __ldcv(reinterpret_cast<const float4*>(a.row_win + s * a.D) + v);
      else if (host_src) x = __ldcv(reinterpret_cast<const float4*>(host_src) + v);
      if (a.out_bf16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.out) + i * a.D)[v] = o;
      } else {
        reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + i * a.D)[v] = x;
      }
    }
    if (a.ugrad && i < nu) {
      for (int v = lane; v < nvec; v += 32) reinterpret_cast<float4*>(a.ugrad + i * a.D)[v] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (lane == 0 && a.unorm) a.unorm[i] = 0.f;
    }
  }
}

struct GradsFusedArgs {
  const float* grad;           // [n, D] per-key gradient sums (or per-occurrence gradients without dedup)
  const long long* slot;       // [n]
  const int* n_dev;            // optional live count
  long long n;
  int D, me;
  long long cap;
  float* const* grad_win;
  const float* norm;           // optional [n]
  float* const* norm_win;
  FlagSignal sig;
};

__global__ void __launch_bounds__(128) shard_grads_fused_kernel(const GradsFusedArgs a) {
  const int lane = threadIdx.x & 31;
  const long long nwarps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long n = a.n_dev ? min(static_cast<long long>(*a.n_dev), a.n) : a.n;
  const int nvec = a.D >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n; i += nwarps) {
    const long long s = a.slot[i];
    if (s < 0) continue;
    const int d = static_cast<int>(s / a.cap);
    const long long p = s % a.cap;
    float* dst = a.grad_win[d] + (static_cast<long long>(a.me) * a.cap + p) * a.D;
    for (int v = lane; v < nvec; v += 32) reinterpret_cast<float4*>(dst)[v] = __ldg(reinterpret_cast<const float4*>(a.grad + i * a.D) + v);
    if (a.norm && lane == 0) a.norm_win[d][static_cast<long long>(a.me) * a.cap + p] = a.norm[i];
  }
  rs::flag_publish_when_grid_done(a.sig);
}

// Owner side of a PUT: after the value push has landed (CH wait inside), every recorded occurrence overwrites its row with
// the value that arrived in its slot; the row counts as initialised from then on.
struct ScatterArgs {
  float* weight;
  const long long* occ_row;
  const int* occ_slot;
  const int* occ_cursor;
  const float* win;            // my value window [world, cap, D]
  float* state;                // optional per-row optimizer state, reset for the rows that are put
  unsigned char* row_init;     // optional (hash mode)
  int D;
  FlagWait wait;
};
__global__ void __launch_bounds__(128) shard_scatter_rows_kernel(const ScatterArgs a) {
  rs::flag_wait_all(a.wait);
  const int lane = threadIdx.x & 31;
  const long long nwarps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long n = *reinterpret_cast<const volatile int*>(a.occ_cursor);
  for (long long q = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); q < n; q += nwarps) {
    const long long r = a.occ_row[q];
    const long long s = a.occ_slot[q];
    for (int v = lane; v < (a.D >> 2); v += 32)
      reinterpret_cast<float4*>(a.weight + r * a.D)[v] = __ldcv(reinterpret_cast<const float4*>(a.win + s * a.D) + v);
    if (lane == 0) {
      if (a.state) a.state[r] = 0.f;
      if (a.row_init) a.row_init[r] = 1;
    }
  }
}

int persistent_grid(long long items, int warps_per_block) {
  long long g = (items + warps_per_block - 1) / warps_per_block;
  // CTAs per SM of the persistent exchange kernels (RECSTORE_SHARD_CTAS_PER_SM, default 8; 16 and 32 measured within 2 %).
  static const int per_sm = [] { const char* e = getenv("RECSTORE_SHARD_CTAS_PER_SM"); const int v = e ? atoi(e) : 0; return v > 0 ? v : 8; }();
  const long long capg = 148ll * per_sm;
  if (g > capg) g = capg;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}
FlagSignal make_sig(void* const* flags_of, unsigned* counters, unsigned* done, int channel, int world, int me) {
  FlagSignal s;
  s.flags_of = reinterpret_cast<uint32_t* const*>(flags_of); s.sig_counters = counters; s.done = done;
  s.channel = channel; s.world = world; s.me = me;
  return s;
}
FlagWait make_wait(const void* my_flags, const unsigned* counters, unsigned long long timeout_ns, int channel, int world,
                   unsigned long long* status) {
  FlagWait w;
  w.my_flags = reinterpret_cast<const uint32_t*>(my_flags); w.sig_counters = counters; w.timeout_ns = timeout_ns;
  w.status = status; w.world = world; w.channel = channel;
  return w;
}
}  // namespace

// n_dev (optional): device count of live keys (the output count of rs_unique_keys); n is then the capacity that sizes the grid.
// range_c: 0 = cyclic ownership (key % world); > 0 = rank r owns keys [r * range_c, (r + 1) * range_c) and larger keys belong to
// the host table (slot -2).
RS_API int rs_shard_keys_fused(const long long* keys, const int* n_dev, long long n, int world, int me, long long cap, int* cursor,
                               void* const* key_win, void* const* count_win, long long* slot, unsigned long long* status,
                               long long range_c, void* const* flags_of, unsigned* counters, unsigned* done, int channel,
                               cudaStream_t stream) {
  RS_REQUIRE(keys && cursor && key_win && count_win && slot && flags_of && counters && done, "rs_shard_keys_fused: null argument");
  RS_REQUIRE(world >= 1 && world <= kMaxWorld && n >= 0 && me >= 0 && me < world, "rs_shard_keys_fused: bad sizes");
  KeysFusedArgs a;
  a.keys = keys; a.n_dev = n_dev; a.n = n; a.world = world; a.me = me; a.cap = cap; a.cursor = cursor;
  a.key_win = reinterpret_cast<long long* const*>(key_win); a.count_win = reinterpret_cast<int* const*>(count_win);
  a.slot = slot; a.status = status; a.range_c = range_c; a.sig = make_sig(flags_of, counters, done, channel, world, me);
  const long long grid = n > 0 ? (n + 255) / 256 : 1;
  RS_REQUIRE(grid < (1ll << 31), "rs_shard_keys_fused: too many keys");
  shard_keys_fused_kernel<<<static_cast<unsigned>(grid), 256, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// ht (optional): find-or-insert in the shard's hash table instead of the cyclic index; a key seen for the first time gets a row
// initialised to uniform(-init_scale, init_scale) values derived from the key.  occ_* (optional): compact occurrence list.
RS_API int rs_shard_gather_fused(float* weight, const float* cold_weight, long long hot_rows, long long local_rows,
                                 const long long* key_win, const int* count_win, void* const* row_win, long long* rowidx,
                                 long long* occ_row, int* occ_slot, int* occ_cursor, int world, int me, int D, long long cap,
                                 const rs::HashTableView* ht, float init_scale, unsigned char* row_init, long long range_c,
                                 int push_rows, int find_only, unsigned long long* status, const void* my_flags,
                                 void* const* flags_of, unsigned* counters, unsigned* done, unsigned long long timeout_ns,
                                 int wait_channel, int sig_channel, cudaStream_t stream) {
  RS_REQUIRE((weight || hot_rows == 0) && key_win && count_win && row_win && D % 4 == 0, "rs_shard_gather_fused: bad argument");
  RS_REQUIRE(hot_rows >= 0 && hot_rows <= local_rows && (hot_rows == local_rows || cold_weight), "rs_shard_gather_fused: bad tiers");
  RS_REQUIRE(!occ_cursor || (occ_row && occ_slot), "rs_shard_gather_fused: the occurrence list needs both arrays");
  RS_REQUIRE(my_flags && flags_of && counters && done, "rs_shard_gather_fused: null flag argument");
  GatherFusedArgs a;
  a.weight = weight; a.cold_weight = cold_weight; a.hot_rows = hot_rows; a.local_rows = local_rows; a.key_win = key_win;
  a.count_win = count_win; a.row_win = reinterpret_cast<float* const*>(row_win); a.rowidx = rowidx; a.occ_row = occ_row;
  a.occ_slot = occ_slot; a.occ_cursor = occ_cursor; a.world = world; a.me = me; a.D = D; a.cap = cap;
  a.use_hash = ht != nullptr;
  if (ht) a.ht = *ht; else memset(&a.ht, 0, sizeof(a.ht));
  RS_REQUIRE(!ht || row_init, "rs_shard_gather_fused: the hash-table shard needs its row_init bytes");
  a.init_scale = init_scale; a.row_init = row_init; a.status = status; a.range_c = range_c; a.push_rows = push_rows; a.find_only = find_only;
  a.wait = make_wait(my_flags, counters, timeout_ns, wait_channel, world, status);
  a.sig = make_sig(flags_of, counters, done, sig_channel, world, me);
  shard_gather_fused_kernel<<<persistent_grid(cap, 4), 128, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// keys / host_table / host_rows (optional): rows of slot -2 are read from the host table (device-visible host memory).
RS_API int rs_shard_unbucket_fused(const float* row_win, const long long* slot, const int* inverse, long long n, int D, void* out,
                                   int out_bf16, float* ugrad, float* unorm, const int* ucount, const long long* keys,
                                   const float* host_table, long long host_rows, const void* my_flags,
                                   const unsigned* counters, unsigned long long timeout_ns, int wait_channel, int world,
                                   unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(row_win && slot && out && D % 4 == 0 && my_flags && counters, "rs_shard_unbucket_fused: bad argument");
  UnbucketFusedArgs a;
  a.row_win = row_win; a.slot = slot; a.inverse = inverse; a.n = n; a.D = D; a.out = out; a.out_bf16 = out_bf16;
  a.ugrad = ugrad; a.unorm = unorm; a.ucount = ucount; a.keys = keys; a.host_table = host_table; a.host_rows = host_rows;
  a.status = status;
  RS_REQUIRE(!host_table || keys, "rs_shard_unbucket_fused: host rows need the keys");
  a.wait = make_wait(my_flags, counters, timeout_ns, wait_channel, world, status);
  shard_unbucket_fused_kernel<<<persistent_grid(n, 4), 128, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_shard_grads_fused(const float* grad, const long long* slot, const int* n_dev, long long n, int D, int me, long long cap,
                                void* const* grad_win, const float* norm, void* const* norm_win, void* const* flags_of,
                                unsigned* counters, unsigned* done, int channel, int world, cudaStream_t stream) {
  RS_REQUIRE(grad && slot && grad_win && D % 4 == 0 && flags_of && counters && done, "rs_shard_grads_fused: bad argument");
  GradsFusedArgs a;
  a.grad = grad; a.slot = slot; a.n_dev = n_dev; a.n = n; a.D = D; a.me = me; a.cap = cap;
  a.grad_win = reinterpret_cast<float* const*>(grad_win); a.norm = norm; a.norm_win = reinterpret_cast<float* const*>(norm_win);
  a.sig = make_sig(flags_of, counters, done, channel, world, me);
  shard_grads_fused_kernel<<<persistent_grid(n, 4), 128, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_shard_scatter_rows(float* weight, const long long* occ_row, const int* occ_slot, const int* occ_cursor, const float* win,
                                 float* state, unsigned char* row_init, int D, long long cap_items, const void* my_flags,
                                 const unsigned* counters, unsigned long long timeout_ns, int wait_channel, int world,
                                 unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(weight && occ_row && occ_slot && occ_cursor && win && D % 4 == 0 && my_flags && counters, "rs_shard_scatter_rows: bad argument");
  ScatterArgs a;
  a.weight = weight; a.occ_row = occ_row; a.occ_slot = occ_slot; a.occ_cursor = occ_cursor; a.win = win; a.state = state;
  a.row_init = row_init; a.D = D;
  a.wait = make_wait(my_flags, counters, timeout_ns, wait_channel, world, status);
  shard_scatter_rows_kernel<<<persistent_grid(cap_items, 4), 128, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
