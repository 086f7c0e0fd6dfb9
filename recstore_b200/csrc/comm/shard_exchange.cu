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
__global__ void __launch_bounds__(256) segment_sum_kernel(const float* __restrict__ grad, const int* __restrict__ inverse,
                                                          long long n, int D, float* __restrict__ ugrad, float* __restrict__ unorm) {
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
    if (lane == 0) atomicAdd(&unorm[u], sq);
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

RS_API int rs_segment_sum(const float* grad, const int* inverse, long long n, int D, float* ugrad, float* unorm,
                          cudaStream_t stream) {
  RS_REQUIRE(grad && inverse && ugrad && D % 4 == 0, "rs_segment_sum: bad argument");
  if (n == 0) return RS_OK;
  segment_sum_kernel<<<warps_grid(n), 256, 0, stream>>>(grad, inverse, n, D, ugrad, unorm);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_expand_rows(const float* src, const int* inverse, long long n, int D, float* out, cudaStream_t stream) {
  RS_REQUIRE(src && inverse && out && D % 4 == 0, "rs_expand_rows: bad argument");
  if (n == 0) return RS_OK;
  expand_rows_kernel<<<warps_grid(n), 256, 0, stream>>>(src, inverse, n, D, out);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
