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

// db[n] += sum over rows of dY[m, n].  A block covers 256 columns (32 lanes x 8 columns, 16-byte loads) and
// kColsumRows rows (8 row-lanes, 4 loads in flight each); partial sums meet in shared memory, one atomic per column.
constexpr int kColsumRows = 128;
__global__ void __launch_bounds__(256) colsum_kernel(const __nv_bfloat16* __restrict__ dY, int ld, int M, int N,
                                                     float* __restrict__ db) {
  __shared__ float s_part[8][256];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int n0 = blockIdx.x * 256 + tx * 8;
  const int m0 = blockIdx.y * kColsumRows;
  const int m1 = min(M, m0 + kColsumRows);
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  if (n0 < N) {
    for (int m = m0 + ty; m < m1; m += 32) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int mm = m + u * 8;
        v[u] = mm < m1 ? __ldg(reinterpret_cast<const uint4*>(dY + static_cast<size_t>(mm) * ld + n0)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(p[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) s_part[ty][tx * 8 + e] = acc[e];
  __syncthreads();
  const int c = threadIdx.x;
  const int n = blockIdx.x * 256 + c;
  if (n < N) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) s += s_part[r][c];
    atomicAdd(&db[n], s);
  }
}

// Same sums for shapes the 16-byte loads cannot take (odd widths, unaligned views): one column per thread.
__global__ void __launch_bounds__(256) colsum_scalar_kernel(const __nv_bfloat16* __restrict__ dY, int ld, int M, int N,
                                                            float* __restrict__ db) {
  const int n = blockIdx.x * 256 + threadIdx.x;
  if (n >= N) return;
  const int m0 = blockIdx.y * kColsumRows;
  const int m1 = min(M, m0 + kColsumRows);
  float s = 0.f;
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

// All layers of a model in one launch.  desc holds 8 int64 per layer: W, g, Wb, Wt (addresses), N, K, ldw, ldt;
// tile_prefix[l] = first 32x32 tile of layer l; blocks past the last tile update the flat tail (biases, head).
// `zero_shift` (elements, may be 0 with zero_base == nullptr): when the gradients that are read are a reduced copy, the
// rank's own accumulation buffer holds the same layout at zero_base + (g - g_base); it is cleared here as well so
// that no separate memset launch is needed.
__global__ void __launch_bounds__(256) dense_sgd_multi_kernel(const long long* __restrict__ desc, const int* __restrict__ tile_prefix,
                                                              int n_layers, float* __restrict__ tail_w, float* __restrict__ tail_g,
                                                              int tail_n, float lr, int zero_grad, long long zero_delta,
                                                              int zero_other) {
  __shared__ float tile[32][33];
  const int total = tile_prefix[n_layers];
  int b = blockIdx.x;
  if (b >= total) {
    const int i = (b - total) * 256 + threadIdx.x;
    if (i < tail_n) {
      tail_w[i] -= lr * tail_g[i];
      if (zero_grad) tail_g[i] = 0.f;
      if (zero_other) *(tail_g + i + zero_delta) = 0.f;
    }
    return;
  }
  int l = 0;
  while (l + 1 < n_layers && tile_prefix[l + 1] <= b) ++l;
  b -= tile_prefix[l];
  const long long* d = desc + l * 8;
  float* W = reinterpret_cast<float*>(d[0]);
  float* g = reinterpret_cast<float*>(d[1]);
  __nv_bfloat16* Wb = reinterpret_cast<__nv_bfloat16*>(d[2]);
  __nv_bfloat16* Wt = reinterpret_cast<__nv_bfloat16*>(d[3]);
  const int N = static_cast<int>(d[4]), K = static_cast<int>(d[5]), ldw = static_cast<int>(d[6]), ldt = static_cast<int>(d[7]);
  const int tiles_k = (K + 31) / 32;
  const int k0 = (b % tiles_k) * 32, n0 = (b / tiles_k) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8) {
    const int n = n0 + j, k = k0 + tx;
    float v = 0.f;
    if (n < N && k < K) {
      const size_t idx = static_cast<size_t>(n) * K + k;
      v = W[idx] - lr * g[idx];
      W[idx] = v;
      if (zero_grad) g[idx] = 0.f;
      if (zero_other) *(g + idx + zero_delta) = 0.f;
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

// ---------------------------------------------------------------- DCNv2 low-rank cross layer, element-wise parts
// x_next = x0 * u + x_l                      (u = W_l (V_l x_l) + b_l comes from the GEMMs)
__global__ void __launch_bounds__(256) cross_fwd_kernel(const __nv_bfloat16* __restrict__ x0, const __nv_bfloat16* __restrict__ u,
                                                        const __nv_bfloat16* __restrict__ xl, __nv_bfloat16* __restrict__ out,
                                                        long long n8) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(x0) + i), b = __ldg(reinterpret_cast<const uint4*>(u) + i),
              c = __ldg(reinterpret_cast<const uint4*>(xl) + i);
  const __nv_bfloat16* pa = reinterpret_cast<const __nv_bfloat16*>(&a);
  const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(&b);
  const __nv_bfloat16* pc = reinterpret_cast<const __nv_bfloat16*>(&c);
  uint4 o;
  __nv_bfloat16* po = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
  for (int e = 0; e < 8; ++e) po[e] = __float2bfloat16(__bfloat162float(pa[e]) * __bfloat162float(pb[e]) + __bfloat162float(pc[e]));
  reinterpret_cast<uint4*>(out)[i] = o;
}
// dU = dX * x0 ; dx0_acc (+)= dX * u
__global__ void __launch_bounds__(256) cross_bwd_kernel(const __nv_bfloat16* __restrict__ dx, const __nv_bfloat16* __restrict__ x0,
                                                        const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ du,
                                                        float* __restrict__ dx0_acc, long long n8, int accumulate) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(dx) + i), b = __ldg(reinterpret_cast<const uint4*>(x0) + i),
              c = __ldg(reinterpret_cast<const uint4*>(u) + i);
  const __nv_bfloat16* pa = reinterpret_cast<const __nv_bfloat16*>(&a);
  const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(&b);
  const __nv_bfloat16* pc = reinterpret_cast<const __nv_bfloat16*>(&c);
  uint4 o;
  __nv_bfloat16* po = reinterpret_cast<__nv_bfloat16*>(&o);
  float acc[8];
  if (accumulate) {
    const float4 p0 = reinterpret_cast<const float4*>(dx0_acc)[2 * i], p1 = reinterpret_cast<const float4*>(dx0_acc)[2 * i + 1];
    acc[0] = p0.x; acc[1] = p0.y; acc[2] = p0.z; acc[3] = p0.w; acc[4] = p1.x; acc[5] = p1.y; acc[6] = p1.z; acc[7] = p1.w;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float d = __bfloat162float(pa[e]);
    po[e] = __float2bfloat16(d * __bfloat162float(pb[e]));
    acc[e] += d * __bfloat162float(pc[e]);
  }
  reinterpret_cast<uint4*>(du)[i] = o;
  reinterpret_cast<float4*>(dx0_acc)[2 * i] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  reinterpret_cast<float4*>(dx0_acc)[2 * i + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// Gradient of the concatenated feature matrix T[B, F, D] (acc fp32 optional + dxb bf16): feature 0 goes to the
// bottom-MLP gradient (with the ReLU mask of T[:,0]), features 1.. go STRAIGHT INTO THE OWNING RANK'S gradient
// window through peer pointers, with their squared norms (same contract as the dot-interaction backward).
struct PushArgs {
  const float* acc; const __nv_bfloat16* dxb; const __nv_bfloat16* T;
  int B, F, D;
  __nv_bfloat16* dx; int dx_ld;
  void* const* gdst; const int* owner; const int* gcol; long long grow_stride, sample_base;
  int relu_mask_dx;
  float* const* ndst; int nstride;
  const __nv_bfloat16* extra; int extra_ld;   // optional [B, >= D]: added to feature 0 only (a direct path of the dense feature)
  int world;                                  // a feature whose owner is < 0 (row-sharded table) goes to ranks 0..world-1
};
__global__ void __launch_bounds__(256) push_feature_grads_kernel(const PushArgs a) {
  const long long w = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(a.B) * a.F) return;
  const int b = static_cast<int>(w / a.F), f = static_cast<int>(w % a.F);
  const long long base = w * a.D;
  float sq = 0.f;
  for (int d = lane * 4; d < a.D; d += 128) {
    float v[4];
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(a.dxb + base + d));
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
    if (a.acc) {
      const float4 p = __ldg(reinterpret_cast<const float4*>(a.acc + base + d));
      v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
    }
    __nv_bfloat16* dst;
    if (f == 0) {
      if (a.extra) {
        const uint2 er = __ldg(reinterpret_cast<const uint2*>(a.extra + static_cast<long long>(b) * a.extra_ld + d));
        const float2 e0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&er.x));
        const float2 e1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&er.y));
        v[0] += e0.x; v[1] += e0.y; v[2] += e1.x; v[3] += e1.y;
      }
      if (a.relu_mask_dx) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (!(__bfloat162float(a.T[base + d + e]) > 0.f)) v[e] = 0.f;
      }
      dst = a.dx + static_cast<long long>(b) * a.dx_ld + d;
    } else {
      const int own = a.owner[f - 1];
      dst = reinterpret_cast<__nv_bfloat16*>(a.gdst[own < 0 ? 0 : own]) + (a.sample_base + b) * a.grow_stride + a.gcol[f - 1] + d;
    }
    __nv_bfloat162 o0 = __floats2bfloat162_rn(v[0], v[1]), o1 = __floats2bfloat162_rn(v[2], v[3]);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&o0);
    o.y = *reinterpret_cast<uint32_t*>(&o1);
    *reinterpret_cast<uint2*>(dst) = o;
    if (f > 0 && a.owner[f - 1] < 0) {          // row-sharded table: every rank holds rows of it
      for (int r = 1; r < a.world; ++r)
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.gdst[r]) + (a.sample_base + b) * a.grow_stride + a.gcol[f - 1] + d) = o;
    }
    const float2 r0 = __bfloat1622float2(o0), r1 = __bfloat1622float2(o1);
    sq += r0.x * r0.x + r0.y * r0.y + r1.x * r1.x + r1.y * r1.y;
  }
  if (a.ndst && f > 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if (lane == 0) {
      const int own = a.owner[f - 1];
      const int r0 = own < 0 ? 0 : own, r1 = own < 0 ? a.world : own + 1;
      for (int r = r0; r < r1; ++r) a.ndst[r][(a.sample_base + b) * a.nstride + a.gcol[f - 1] / a.D] = sq;
    }
  }
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
  dim3 grid((N + 255) / 256, (M + kColsumRows - 1) / kColsumRows);
  if (N % 8 != 0 || ld % 8 != 0 || (reinterpret_cast<uintptr_t>(dY) & 15) != 0) {
    colsum_scalar_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dY), ld, M, N, db);
    RS_LAUNCH_CHECK();
    return RS_OK;
  }
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

// SGD step of every dense layer plus the flat tail in one launch (see dense_sgd_multi_kernel for the descriptor).
// zero_other != 0: a second buffer with the layout of the gradient buffer that is read (e.g. the rank's own accumulation
// buffer when the step reads an all-reduced copy) lies `zero_delta` elements away from it and is cleared as well.
RS_API int rs_dense_sgd_multi(const long long* desc, const int* tile_prefix, int n_layers, int total_tiles, float* tail_w,
                              float* tail_g, int tail_n, float lr, int zero_grad, long long zero_delta, int zero_other,
                              cudaStream_t stream) {
  RS_REQUIRE(desc && tile_prefix && n_layers > 0 && total_tiles >= 0, "rs_dense_sgd_multi: bad argument");
  RS_REQUIRE(tail_n == 0 || (tail_w && tail_g), "rs_dense_sgd_multi: tail pointers missing");
  const int blocks = total_tiles + (tail_n + 255) / 256;
  if (blocks == 0) return RS_OK;
  dense_sgd_multi_kernel<<<blocks, 256, 0, stream>>>(desc, tile_prefix, n_layers, tail_w, tail_g, tail_n, lr, zero_grad, zero_delta,
                                                     zero_other);
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

RS_API int rs_cross_fwd(const void* x0, const void* u, const void* xl, void* out, long long n, cudaStream_t stream) {
  RS_REQUIRE(x0 && u && xl && out && n % 8 == 0, "rs_cross_fwd: bad argument (n must be a multiple of 8)");
  if (n == 0) return RS_OK;
  cross_fwd_kernel<<<static_cast<unsigned>((n / 8 + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x0), reinterpret_cast<const __nv_bfloat16*>(u),
      reinterpret_cast<const __nv_bfloat16*>(xl), reinterpret_cast<__nv_bfloat16*>(out), n / 8);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
RS_API int rs_cross_bwd(const void* dx, const void* x0, const void* u, void* du, float* dx0_acc, long long n, int accumulate,
                        cudaStream_t stream) {
  RS_REQUIRE(dx && x0 && u && du && dx0_acc && n % 8 == 0, "rs_cross_bwd: bad argument (n must be a multiple of 8)");
  if (n == 0) return RS_OK;
  cross_bwd_kernel<<<static_cast<unsigned>((n / 8 + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(dx), reinterpret_cast<const __nv_bfloat16*>(x0),
      reinterpret_cast<const __nv_bfloat16*>(u), reinterpret_cast<__nv_bfloat16*>(du), dx0_acc, n / 8, accumulate);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
RS_API int rs_push_feature_grads(const float* acc, const void* dxb, const void* T, int B, int F, int D, void* dx, int dx_ld,
                                 void* const* gdst, const int* owner, const int* gcol, long long grow_stride,
                                 long long sample_base, int relu_mask_dx, void* const* ndst, int nstride, const void* extra,
                                 int extra_ld, int world, cudaStream_t stream) {
  RS_REQUIRE(dxb && T && dx && gdst && owner && gcol && D % 4 == 0, "rs_push_feature_grads: bad argument");
  RS_REQUIRE(!extra || (extra_ld % 4 == 0 && extra_ld >= D), "rs_push_feature_grads: bad extra gradient");
  if (B == 0) return RS_OK;
  PushArgs a;
  a.acc = acc; a.dxb = reinterpret_cast<const __nv_bfloat16*>(dxb); a.T = reinterpret_cast<const __nv_bfloat16*>(T);
  a.B = B; a.F = F; a.D = D; a.dx = reinterpret_cast<__nv_bfloat16*>(dx); a.dx_ld = dx_ld; a.gdst = gdst; a.owner = owner;
  a.gcol = gcol; a.grow_stride = grow_stride; a.sample_base = sample_base; a.relu_mask_dx = relu_mask_dx;
  a.ndst = reinterpret_cast<float* const*>(ndst); a.nstride = nstride;
  a.extra = reinterpret_cast<const __nv_bfloat16*>(extra); a.extra_ld = extra_ld;
  a.world = world < 1 ? 1 : world;
  const long long warps = static_cast<long long>(B) * F;
  push_feature_grads_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
