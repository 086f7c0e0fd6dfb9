// Host half of the cold tier: the rows that are not resident in the HBM cache live in one pinned host array
// [rows, ld] (weights, then per-row optimizer state, then padding).  These helpers move batches of rows between that
// array and pinned staging buffers with every core (the copies that feed cudaMemcpyAsync on the side stream), and apply
// the optimizer to rows that could not be cached.  They replace the host-side gather / scatter of the reference's
// UvmTable (src/storage/gpu_cache/uvm_table.cu:421-497: host gather into a staging block, H2D copy, scatter on the
// copy stream; evicted rows travel the other way).
#include <cmath>
#include <cstring>

#include "common/rs_common.h"
#include "runtime/base.h"

// out[i, :ld] = table[keys[i], :ld]; a key outside [0, rows) gives a zero row and counts as an error.
RS_API int rs_host_gather_rows(const float* table, long long rows, long long ld, const long long* keys, long long n, float* out) {
  RS_REQUIRE(table && keys && out && ld > 0 && rows >= 0 && n >= 0, "rs_host_gather_rows: bad argument");
  std::atomic<long long> bad{0};
  rs::ThreadPool::global().parallel_for(static_cast<size_t>(n), [&](size_t b, size_t e, int) {
    for (size_t i = b; i < e; ++i) {
      const long long k = keys[i];
      if (k < 0 || k >= rows) {
        memset(out + i * ld, 0, sizeof(float) * ld);
        bad.fetch_add(1, std::memory_order_relaxed);
        continue;
      }
      memcpy(out + i * ld, table + k * ld, sizeof(float) * ld);
    }
  });
  if (bad.load()) return rs::set_error(RS_ERR_INVALID, "rs_host_gather_rows: %lld keys outside [0, %lld)", bad.load(), rows);
  return RS_OK;
}

// table[keys[i], :ld] = in[i, :ld] (write-back of evicted rows; keys are distinct).
RS_API int rs_host_scatter_rows(float* table, long long rows, long long ld, const long long* keys, long long n, const float* in) {
  RS_REQUIRE(table && keys && in && ld > 0 && rows >= 0 && n >= 0, "rs_host_scatter_rows: bad argument");
  std::atomic<long long> bad{0};
  rs::ThreadPool::global().parallel_for(static_cast<size_t>(n), [&](size_t b, size_t e, int) {
    for (size_t i = b; i < e; ++i) {
      const long long k = keys[i];
      if (k < 0 || k >= rows) { bad.fetch_add(1, std::memory_order_relaxed); continue; }
      memcpy(table + k * ld, in + i * ld, sizeof(float) * ld);
    }
  });
  if (bad.load()) return rs::set_error(RS_ERR_INVALID, "rs_host_scatter_rows: %lld keys outside [0, %lld)", bad.load(), rows);
  return RS_OK;
}

// Optimizer step on host rows (rows whose cache set was full of protected rows): keys distinct, grad [n, D], norm [n].
// Row layout: D weights, state at column D.  optimizer 0 = SGD, 1 = row-wise Adagrad.
RS_API int rs_host_apply_rows(float* table, long long rows, long long ld, int D, const long long* keys, long long n, const float* grad,
                              const float* norm, float lr, float eps, int optimizer) {
  RS_REQUIRE(table && keys && grad && D > 0 && D + 1 <= ld && n >= 0, "rs_host_apply_rows: bad argument");
  for (long long i = 0; i < n; ++i) {
    const long long k = keys[i];
    if (k < 0 || k >= rows) continue;
    float* row = table + k * ld;
    float scale = -lr;
    if (optimizer == 1) {
      row[D] += (norm ? norm[i] : 0.f) / static_cast<float>(D);
      scale = -lr / (std::sqrt(row[D]) + eps);
    }
    for (int d = 0; d < D; ++d) row[d] += scale * grad[i * D + d];
  }
  return RS_OK;
}
