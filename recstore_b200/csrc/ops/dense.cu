// Small dense-side kernels around the tcgen05 GEMMs of the MLP stacks:
//   * rs_head_bce:      the final N=1 linear layer as a fused GEMV + sigmoid + binary cross entropy
//                       + all gradients that leave it (dX with the ReLU mask of X, dw, db).  Replaces
//                       nn.Linear(…,1) + Sigmoid + BCELoss of src/executable/dlrm/dlrm_model.py:
//                       232-245 and the BCEWithLogitsLoss of model_zoo/dlrm.py:886.
//   * rs_colsum_bf16:   bias gradient db[n] = sum_m dY[m,n].
//   * rs_dense_sgd:     fp32 master update W -= lr * g, refreshes the bf16 copies W and W^T that the
//                       forward / dgrad GEMMs read, and zeroes g for the next step's atomic wgrad.
//   * rs_pad_cast_bf16: fp32 [M, K] -> bf16 [M, ld] with zero padding (dense features 13 -> 64).
//   * rs_mse_fwd_bwd:   mean squared error + gradient (perf_rec_model.py uses MSE vs random labels).
#include <cuda_bf16.h>
#include "common/rs_common.h"

namespace {

constexpr int kHeadMaxK = 1024;

// One warp per row.  K <= 1024, K % 8 == 0.
__global__ void __launch_bounds__(256) head_bce_kernel(const __nv_bfloat16* __restrict__ X, int ldx, int M, int K,
                                                       const float* __restrict__ w, const float* __restrict__ bias,
                                                       const float* __restrict__ labels, float inv_batch,
                                                       float* __restrict__ prob, float* __restrict__ loss_sum,
                                                       __nv_bfloat16* __restrict__ dX, int lddx,
                                                       float* __restrict__ dw, float* __restrict__ db,
                                                       int rows_per_block, int with_logits_only) {
  __shared__ float s_dw[kHeadMaxK];
  __shared__ float s_loss, s_db;
  for (int i = threadIdx.x; i < K; i += blockDim.x) s_dw[i] = 0.f;
  if (threadIdx.x == 0) { s_loss = 0.f; s_db = 0.f; }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int row0 = blockIdx.x * rows_per_block;
  const int row1 = min(M, row0 + rows_per_block);
  const int nvec = K >> 3;
  const int per_lane = (nvec + 31) / 32;  // <= 4
  float wreg[4][8];
  float dwreg[4][8];
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int v = lane + c * 32;
      wreg[c][e] = (c < per_lane && v < nvec) ? w[v * 8 + e] : 0.f;
      dwreg[c][e] = 0.f;
    }
  const float b0 = bias ? bias[0] : 0.f;
  float loss_acc = 0.f, db_acc = 0.f;
  for (int r = row0 + warp; r < row1; r += nwarps) {
    float xv[4][8];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int v = lane + c * 32;
      if (c < per_lane && v < nvec) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(X + static_cast<size_t>(r) * ldx) + v);
        const __nv_bfloat16* xe = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xv[c][e] = __bfloat162float(xe[e]);
          dot += xv[c][e] * wreg[c][e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) xv[c][e] = 0.f;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float z = dot + b0;
    const float p = 1.f / (1.f + __expf(-z));
    if (prob && lane == 0) prob[r] = p;
    if (with_logits_only) continue;
    const float y = labels[r];
    // numerically stable BCE with logits: max(z,0) - z*y + log(1 + exp(-|z|))
    const float l = fmaxf(z, 0.f) - z * y + log1pf(__expf(-fabsf(z)));
    const float dz = (p - y) * inv_batch;
    if (lane == 0) { loss_acc += l; db_acc += dz; }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int v = lane + c * 32;
      if (c < per_lane && v < nvec) {
        uint4 o;
        __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          dwreg[c][e] += dz * xv[c][e];
          oe[e] = __float2bfloat16(xv[c][e] > 0.f ? dz * wreg[c][e] : 0.f);
        }
        if (dX) *(reinterpret_cast<uint4*>(dX + static_cast<size_t>(r) * lddx) + v) = o;
      }
    }
  }
  if (with_logits_only) return;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int v = lane + c * 32;
    if (c < per_lane && v < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) atomicAdd(&s_dw[v * 8 + e], dwreg[c][e]);
    }
  }
  if (lane == 0) { atomicAdd(&s_loss, loss_acc); atomicAdd(&s_db, db_acc); }
  __syncthreads();
  for (int i = threadIdx.x; i < K; i += blockDim.x) atomicAdd(&dw[i], s_dw[i]);
  if (threadIdx.x == 0) {
    atomicAdd(loss_sum, s_loss * inv_batch);
    if (db) atomicAdd(db, s_db);
  }
}

// db[n] += sum over rows of dY[m, n]; block handles 128 rows x 256 columns.
__global__ void __launch_bounds__(256) colsum_kernel(const __nv_bfloat16* __restrict__ dY, int ld, int M, int N,
                                                     float* __restrict__ db) {
  const int n = blockIdx.x * 256 + threadIdx.x;
  const int m0 = blockIdx.y * 128;
  if (n >= N) return;
  float s = 0.f;
  const int m1 = min(M, m0 + 128);
  for (int m = m0; m < m1; ++m) s += __bfloat162float(dY[static_cast<size_t>(m) * ld + n]);
  atomicAdd(&db[n], s);
}

// W[N,K] fp32 master, g fp32, writes bf16 Wb[N, ldw] and (optional) transposed Wt[K, ldt].
__global__ void __launch_bounds__(256) dense_sgd_kernel(float* __restrict__ W, float* __restrict__ g, int N, int K,
                                                        float lr, __nv_bfloat16* __restrict__ Wb, int ldw,
                                                        __nv_bfloat16* __restrict__ Wt, int ldt, int zero_grad) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int j = ty; j < 32; j += 8) {
    const int n = n0 + j, k = k0 + tx;
    float v = 0.f;
    if (n < N && k < K) {
      const size_t idx = static_cast<size_t>(n) * K + k;
      v = W[idx] - lr * g[idx];
      W[idx] = v;
      if (zero_grad) g[idx] = 0.f;
      if (Wb) Wb[static_cast<size_t>(n) * ldw + k] = __float2bfloat16(v);
    }
    tile[j][tx] = v;
  }
  __syncthreads();
  if (Wt) {
    for (int j = ty; j < 32; j += 8) {
      const int k = k0 + j, n = n0 + tx;
      if (n < N && k < K) Wt[static_cast<size_t>(k) * ldt + n] = __float2bfloat16(tile[tx][j]);
    }
  }
}

__global__ void vec_sgd_kernel(float* __restrict__ w, float* __restrict__ g, int n, float lr, int zero_grad) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    w[i] -= lr * g[i];
    if (zero_grad) g[i] = 0.f;
  }
}

__global__ void pad_cast_kernel(const float* __restrict__ in, int M, int K, int ldi, __nv_bfloat16* __restrict__ out,
                                int ldo) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(M) * ldo) return;
  const int m = static_cast<int>(i / ldo), k = static_cast<int>(i % ldo);
  out[i] = __float2bfloat16(k < K ? in[static_cast<size_t>(m) * ldi + k] : 0.f);
}

__global__ void mse_kernel(const __nv_bfloat16* __restrict__ pred, const float* __restrict__ target, int n,
                           float inv_n, float* __restrict__ loss_sum, __nv_bfloat16* __restrict__ dpred) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  float l = 0.f;
  if (i < n) {
    const float d = __bfloat162float(pred[i]) - target[i];
    l = d * d * inv_n;
    if (dpred) dpred[i] = __float2bfloat16(2.f * d * inv_n);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  if ((threadIdx.x & 31) == 0 && l != 0.f) atomicAdd(loss_sum, l);
}

}  // namespace

// labels == nullptr: inference, only `prob` is written.
RS_API int rs_head_bce(const void* X, int ldx, int M, int K, const float* w, const float* bias, const float* labels,
                       float inv_batch, float* prob, float* loss_sum, void* dX, int lddx, float* dw, float* db,
                       cudaStream_t stream) {
  RS_REQUIRE(X && w, "rs_head_bce: null argument");
  RS_REQUIRE(K % 8 == 0 && K <= kHeadMaxK && ldx % 8 == 0, "rs_head_bce: K=%d must be a multiple of 8, <= %d", K, kHeadMaxK);
  RS_REQUIRE(labels == nullptr || (loss_sum && dw), "rs_head_bce: training needs loss_sum and dw");
  if (M == 0) return RS_OK;
  const int rows_per_block = 64;
  head_bce_kernel<<<(M + rows_per_block - 1) / rows_per_block, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(X), ldx, M, K, w, bias, labels, inv_batch, prob, loss_sum,
      reinterpret_cast<__nv_bfloat16*>(dX), lddx, dw, db, rows_per_block, labels == nullptr ? 1 : 0);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_colsum_bf16(const void* dY, int ld, int M, int N, float* db, cudaStream_t stream) {
  RS_REQUIRE(dY && db, "rs_colsum_bf16: null argument");
  if (M == 0 || N == 0) return RS_OK;
  dim3 grid((N + 255) / 256, (M + 127) / 128);
  colsum_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dY), ld, M, N, db);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_dense_sgd(float* W, float* g, int N, int K, float lr, void* Wb, int ldw, void* Wt, int ldt,
                        int zero_grad, cudaStream_t stream) {
  RS_REQUIRE(W && g, "rs_dense_sgd: null argument");
  if (N == 0 || K == 0) return RS_OK;
  dim3 grid((K + 31) / 32, (N + 31) / 32);
  dense_sgd_kernel<<<grid, 256, 0, stream>>>(W, g, N, K, lr, reinterpret_cast<__nv_bfloat16*>(Wb), ldw,
                                             reinterpret_cast<__nv_bfloat16*>(Wt), ldt, zero_grad);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_vec_sgd(float* w, float* g, int n, float lr, int zero_grad, cudaStream_t stream) {
  RS_REQUIRE(w && g, "rs_vec_sgd: null argument");
  if (n == 0) return RS_OK;
  vec_sgd_kernel<<<(n + 255) / 256, 256, 0, stream>>>(w, g, n, lr, zero_grad);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_pad_cast_bf16(const float* in, int M, int K, int ldi, void* out, int ldo, cudaStream_t stream) {
  RS_REQUIRE(in && out && ldo >= K, "rs_pad_cast_bf16: bad argument");
  if (M == 0) return RS_OK;
  const long long n = static_cast<long long>(M) * ldo;
  pad_cast_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(in, M, K, ldi,
                                                                               reinterpret_cast<__nv_bfloat16*>(out), ldo);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_mse_fwd_bwd(const void* pred, const float* target, int n, float inv_n, float* loss_sum, void* dpred,
                          cudaStream_t stream) {
  RS_REQUIRE(pred && target && loss_sum, "rs_mse_fwd_bwd: null argument");
  if (n == 0) return RS_OK;
  mse_kernel<<<(n + 255) / 256, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(pred), target, n, inv_n,
                                                  loss_sum, reinterpret_cast<__nv_bfloat16*>(dpred));
  RS_LAUNCH_CHECK();
  return RS_OK;
}
