// Two-tier embedding storage of one GPU: the first `hot_rows` rows of a table live in HBM, the rest in pinned
// host memory that the kernels read and write in place through unified addressing (no staging copies).
//
// This is the storage shape of the reference's "known local cache" (hot id range in an HBM tensor, everything
// else in a host-DRAM table read through UVA: recstore_pytorch.cu:12-64, gpu_cache_nohash.cu:2-22, the host
// tier of uvm_table.cu) with the sparse optimizer applied on both tiers by one kernel.  Ids are expected in
// popularity order (hot ids first), which is what the renumbering step provides.
//
//   tiered_gather : out[i] = row(rows[i]); counts how many valid rows were served from HBM
//   tiered_apply  : row-wise Adagrad or SGD on UNIQUE rows (the caller folds duplicates first with
//                   unique_keys + segment_sum), plain read-modify-write: nothing is atomic, so host
//                   rows need no PCIe atomics
#include <cuda_runtime.h>

#include "common/rs_common.h"
#include "kv/hash_table.cuh"

namespace {

struct TieredArgs {
  float* hot_w; float* hot_s;        // [hot_rows, D], [hot_rows]
  float* cold_w; float* cold_s;      // [total_rows - hot_rows, D], [...]: device-visible host pointers
  long long hot_rows, total_rows;
  const long long* rows;             // [n], < 0 = skip
  long long n;
  int D;
};

__global__ void __launch_bounds__(256) tiered_gather_kernel(const TieredArgs a, float* __restrict__ out,
                                                            unsigned long long* __restrict__ counters,
                                                            unsigned long long* __restrict__ status) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= a.n) return;
  const int lane = threadIdx.x & 31;
  const long long r = a.rows[i];
  const int nvec = a.D >> 2;
  float4* o = reinterpret_cast<float4*>(out + i * a.D);
  if (r < 0 || r >= a.total_rows) {
    if (r >= a.total_rows && lane == 0 && status) atomicOr(status, (unsigned long long)RS_DEV_OOB_ROW);
    for (int v = lane; v < nvec; v += 32) o[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    return;
  }
  const bool hot = r < a.hot_rows;
  const float4* src = reinterpret_cast<const float4*>(hot ? a.hot_w + r * a.D : a.cold_w + (r - a.hot_rows) * a.D);
  for (int v = lane; v < nvec; v += 32) o[v] = hot ? __ldg(src + v) : __ldcv(src + v);   // host rows: never cached stale
  if (lane == 0 && counters) atomicAdd(&counters[hot ? 0 : 1], 1ull);
}

__global__ void __launch_bounds__(256) tiered_apply_kernel(const TieredArgs a, const float* __restrict__ grad,
                                                           const float* __restrict__ sqnorm, float lr, float eps,
                                                           int optimizer) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= a.n) return;
  const int lane = threadIdx.x & 31;
  const long long r = a.rows[i];
  if (r < 0 || r >= a.total_rows) return;
  const bool hot = r < a.hot_rows;
  float* w = hot ? a.hot_w + r * a.D : a.cold_w + (r - a.hot_rows) * a.D;
  float scale = -lr;
  if (optimizer == 1) {
    float* s = hot ? a.hot_s + r : a.cold_s + (r - a.hot_rows);
    float st = 0.f;
    if (lane == 0) {
      st = *s + sqnorm[i] / static_cast<float>(a.D);
      *s = st;
    }
    st = __shfl_sync(0xffffffffu, st, 0);
    scale = -lr / (sqrtf(st) + eps);
  }
  const float4* g = reinterpret_cast<const float4*>(grad + i * a.D);
  float4* wv = reinterpret_cast<float4*>(w);
  for (int v = lane; v < (a.D >> 2); v += 32) {
    float4 x = wv[v];
    const float4 d = __ldg(g + v);
    x.x += scale * d.x; x.y += scale * d.y; x.z += scale * d.z; x.w += scale * d.w;
    wv[v] = x;
  }
}

// Lookahead refresh: `rows` are the distinct rows that were gathered AHEAD of time for the next step into `staged`;
// those among them that the step in between has just updated (members of its duplicate-folding hash) are read again.
__global__ void __launch_bounds__(256) tiered_refresh_kernel(const TieredArgs a, float* __restrict__ staged,
                                                             const unsigned long long* __restrict__ updated_keys,
                                                             unsigned long long mask, unsigned long long* __restrict__ counters) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= a.n) return;
  const int lane = threadIdx.x & 31;
  const long long r = a.rows[i];
  if (r < 0 || r >= a.total_rows) return;
  bool hit = false;
  unsigned long long s = rs::ht_hash(static_cast<unsigned long long>(r)) & mask;
  for (int p = 0; p < rs::kHtMaxProbe; ++p) {          // warp-uniform probe of the open-addressing set
    const unsigned long long k = __ldg(&updated_keys[s]);
    if (k == rs::kHtEmpty) break;
    if (k == static_cast<unsigned long long>(r)) { hit = true; break; }
    s = (s + 1) & mask;
  }
  if (!hit) return;
  const bool hot = r < a.hot_rows;
  const float4* src = reinterpret_cast<const float4*>(hot ? a.hot_w + r * a.D : a.cold_w + (r - a.hot_rows) * a.D);
  float4* o = reinterpret_cast<float4*>(staged + i * a.D);
  for (int v = lane; v < (a.D >> 2); v += 32) o[v] = __ldcv(src + v);
  if (lane == 0 && counters) atomicAdd(&counters[2], 1ull);
}

int fill(TieredArgs& a, float* hot_w, float* hot_s, float* cold_w, float* cold_s, long long hot_rows, long long total_rows,
         const long long* rows, long long n, int D) {
  RS_REQUIRE(rows && D > 0 && D % 4 == 0 && hot_rows >= 0 && hot_rows <= total_rows, "tiered table: bad sizes");
  RS_REQUIRE(hot_rows == 0 || hot_w, "tiered table: hot tier pointer missing");
  RS_REQUIRE(hot_rows == total_rows || cold_w, "tiered table: cold tier pointer missing");
  a.hot_w = hot_w; a.hot_s = hot_s; a.cold_w = cold_w; a.cold_s = cold_s; a.hot_rows = hot_rows; a.total_rows = total_rows;
  a.rows = rows; a.n = n; a.D = D;
  return RS_OK;
}

}  // namespace

// counters (optional, device): [0] += rows served from HBM, [1] += rows served from the host tier.
RS_API int rs_tiered_gather(const float* hot_w, const float* cold_w, long long hot_rows, long long total_rows,
                            const long long* rows, long long n, int D, float* out, unsigned long long* counters,
                            unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(out, "rs_tiered_gather: null output");
  TieredArgs a;
  int rc = fill(a, const_cast<float*>(hot_w), nullptr, const_cast<float*>(cold_w), nullptr, hot_rows, total_rows, rows, n, D);
  if (rc != RS_OK) return rc;
  if (n == 0) return RS_OK;
  tiered_gather_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(a, out, counters, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// rows must be unique (or < 0); grad [n, D] = summed gradient of each row, sqnorm [n] = sum over the row's
// occurrences of |g|^2 (row-wise Adagrad: state += sqnorm / D).  optimizer: 0 = SGD, 1 = row-wise Adagrad.
RS_API int rs_tiered_apply(float* hot_w, float* hot_s, float* cold_w, float* cold_s, long long hot_rows, long long total_rows,
                           const long long* rows, long long n, int D, const float* grad, const float* sqnorm, float lr,
                           float eps, int optimizer, cudaStream_t stream) {
  RS_REQUIRE(grad && (optimizer == 0 || optimizer == 1), "rs_tiered_apply: bad argument");
  RS_REQUIRE(optimizer == 0 || (sqnorm && (hot_rows == 0 || hot_s) && (hot_rows == total_rows || cold_s)),
             "rs_tiered_apply: row-wise Adagrad needs the state tiers and the squared norms");
  TieredArgs a;
  int rc = fill(a, hot_w, hot_s, cold_w, cold_s, hot_rows, total_rows, rows, n, D);
  if (rc != RS_OK) return rc;
  if (n == 0) return RS_OK;
  tiered_apply_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(a, grad, sqnorm, lr, eps, optimizer);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// staged [n, D]: rows gathered ahead for `rows` (distinct); updated_keys: the key slots of the hash that folded the
// duplicates of the step that ran in between (nslots a power of two).  counters[2] += rows read again.
RS_API int rs_tiered_refresh(const float* hot_w, const float* cold_w, long long hot_rows, long long total_rows,
                             const long long* rows, long long n, int D, float* staged, const void* updated_keys,
                             unsigned long long nslots, unsigned long long* counters, cudaStream_t stream) {
  RS_REQUIRE(staged && updated_keys && nslots >= 2 && (nslots & (nslots - 1)) == 0, "rs_tiered_refresh: bad argument");
  TieredArgs a;
  int rc = fill(a, const_cast<float*>(hot_w), nullptr, const_cast<float*>(cold_w), nullptr, hot_rows, total_rows, rows, n, D);
  if (rc != RS_OK) return rc;
  if (n == 0) return RS_OK;
  tiered_refresh_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(
      a, staged, static_cast<const unsigned long long*>(updated_keys), nslots - 1, counters);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
