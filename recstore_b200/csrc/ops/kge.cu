// Knowledge-graph embedding scoring: TransE (L2) and DistMult with chunked shared negatives and the
// log-sigmoid loss, forward and backward.
//
// Math of the reference (src/kg/kg/dgl-ke/python/dglke/models/pytorch/score_fun.py:26-108, 222-286,
// loss.py:69-99, general_models.py:568-631):
//   TransE   pos = gamma - ||h + r - t||_2          neg (tail corrupt) = gamma - ||(h + r) - t'||_2
//                                                  neg (head corrupt) = gamma - ||(t - r) - h'||_2
//            with dist(a, b) = sqrt(max(|a|^2 + |b|^2 - 2 a.b, 1e-30))
//   DistMult pos = sum h*r*t                         neg = (h*r).t'   or   (t*r).h'
//   loss = ( mean(-logsigmoid(pos)) + mean(-logsigmoid(-neg)) ) / 2
// A batch of `bs` positives is cut into chunks of `cs`; every chunk shares `ns` negative entities.
//
// The cross products a.b are ONE bf16 tensor-core GEMM over the whole batch (rs_gemm_bf16, tcgen05):
// S[bs, C*ns] = A . Neg^T; only the chunk-diagonal blocks are consumed.  This file has the three
// element-wise stages around the GEMMs:
//   kge_prepare : a = h+r | t-r | h*r | t*r (bf16 copy for the GEMM), |a|^2, |b|^2, positive scores,
//                 positive loss and positive gradients
//   kge_neg_loss: S -> negative scores -> loss, and the weight matrix W (bf16, zero outside the
//                 chunk-diagonal) with its row / column sums for the backward GEMMs
//                 GA = W . Neg (mode 2), GB = W^T . A (mode 1)
//   kge_finish  : GA, GB -> gradients of h, r, t and of the negative entities
#include <cuda_bf16.h>
#include "common/rs_common.h"

namespace {

struct KgeArgs {
  const float* h; const float* r; const float* t;   // [bs, D]
  const float* neg;                                  // [C*ns, D]
  int bs, cs, ns, C, D, Dp;                          // Dp: padded row length of the bf16 operands
  int model;                                         // 0 TransE-L2, 1 DistMult
  int corrupt_head;                                  // 0: negatives replace tails, 1: heads
  float gamma;
  __nv_bfloat16* A;                                  // [bs, Dp]
  __nv_bfloat16* Bn;                                 // [C*ns, Dp]
  float* a2; float* b2;                              // [bs], [C*ns]
  float* loss;                                       // [2]: positive part, negative part (already averaged and halved)
  float* gh; float* gr; float* gt;                   // [bs, D] gradients (written by prepare, completed by finish)
  float* gneg;                                       // [C*ns, D]
  const float* S;                                    // [bs, C*ns] cross products
  __nv_bfloat16* W;                                  // [bs, C*ns]
  float* rowsum; float* colsum;                      // [bs], [C*ns]
  const float* GA; const float* GB;                  // [bs, Dp], [C*ns, Dp]
  float* pos_score; float* neg_score;                // optional outputs (evaluation / tests): [bs], [bs, ns]
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(__expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoid(float x) { return 1.f / (1.f + __expf(-x)); }

// one warp per row: rows [0, bs) are positives, rows [bs, bs + C*ns) negatives
__global__ void __launch_bounds__(256) kge_prepare_kernel(const KgeArgs k) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int D = k.D;
  if (row >= k.bs + k.C * k.ns) return;
  if (row >= k.bs) {
    const int j = row - k.bs;
    float s = 0.f;
    for (int d = lane; d < k.Dp; d += 32) {
      const float v = d < D ? k.neg[static_cast<size_t>(j) * D + d] : 0.f;
      const __nv_bfloat16 b = __float2bfloat16(v);
      k.Bn[static_cast<size_t>(j) * k.Dp + d] = b;
      const float vb = __bfloat162float(b);
      s += vb * vb;
    }
    s = warp_sum(s);
    if (lane == 0) k.b2[j] = s;
    return;
  }
  const int i = row;
  const float* h = k.h + static_cast<size_t>(i) * D;
  const float* r = k.r + static_cast<size_t>(i) * D;
  const float* t = k.t + static_cast<size_t>(i) * D;
  float a2 = 0.f, pos = 0.f;
  for (int d = lane; d < k.Dp; d += 32) {
    float a = 0.f;
    if (d < D) {
      const float hv = h[d], rv = r[d], tv = t[d];
      if (k.model == 0) {
        a = k.corrupt_head ? tv - rv : hv + rv;
        const float diff = hv + rv - tv;
        pos += diff * diff;
      } else {
        a = k.corrupt_head ? tv * rv : hv * rv;
        pos += hv * rv * tv;
      }
    }
    const __nv_bfloat16 ab = __float2bfloat16(a);
    k.A[static_cast<size_t>(i) * k.Dp + d] = ab;
    const float av = __bfloat162float(ab);
    a2 += av * av;
  }
  a2 = warp_sum(a2);
  pos = warp_sum(pos);
  float score, dist = 1.f;
  if (k.model == 0) {
    dist = sqrtf(fmaxf(pos, 1e-30f));
    score = k.gamma - dist;
  } else {
    score = pos;
  }
  // d loss / d score of a positive: -sigmoid(-score) / bs / 2
  const float q = -sigmoid(-score) / static_cast<float>(k.bs) * 0.5f;
  if (lane == 0) {
    k.a2[i] = a2;
    if (k.pos_score) k.pos_score[i] = score;
    atomicAdd(&k.loss[0], -log_sigmoid(score) / static_cast<float>(k.bs) * 0.5f);
  }
  float* gh = k.gh + static_cast<size_t>(i) * D;
  float* gr = k.gr + static_cast<size_t>(i) * D;
  float* gt = k.gt + static_cast<size_t>(i) * D;
  for (int d = lane; d < D; d += 32) {
    const float hv = h[d], rv = r[d], tv = t[d];
    if (k.model == 0) {
      const float g = -q * (hv + rv - tv) / dist;   // d score / d h = -(h + r - t) / dist
      gh[d] = g; gr[d] = g; gt[d] = -g;
    } else {
      gh[d] = q * rv * tv; gr[d] = q * hv * tv; gt[d] = q * hv * rv;
    }
  }
}

// one thread per (positive i, negative j of its chunk); W row-major [bs, C*ns], zero outside the chunk
__global__ void __launch_bounds__(256) kge_neg_loss_kernel(const KgeArgs k) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int ncols = k.C * k.ns;
  float l = 0.f;
  if (idx < static_cast<long long>(k.bs) * ncols) {
    const int i = static_cast<int>(idx / ncols);
    const int col = static_cast<int>(idx % ncols);
    const int c = i / k.cs;
    float w = 0.f;
    if (col / k.ns == c) {
      const float dot = k.S[idx];
      float score, wgt;
      const float norm = 1.f / (static_cast<float>(k.bs) * k.ns) * 0.5f;
      if (k.model == 0) {
        const float dist = sqrtf(fmaxf(k.a2[i] + k.b2[col] - 2.f * dot, 1e-30f));
        score = k.gamma - dist;
        wgt = sigmoid(score) * norm / dist;      // q / dist
      } else {
        score = dot;
        wgt = sigmoid(score) * norm;             // q
      }
      l = -log_sigmoid(-score) * norm;
      w = wgt;
      if (k.neg_score) k.neg_score[static_cast<size_t>(i) * k.ns + (col - c * k.ns)] = score;
      const __nv_bfloat16 wb = __float2bfloat16(w);
      w = __bfloat162float(wb);
      atomicAdd(&k.rowsum[i], w);
      atomicAdd(&k.colsum[col], w);
      k.W[idx] = wb;
    } else {
      k.W[idx] = __float2bfloat16(0.f);
    }
  }
  l = warp_sum(l);
  if ((threadIdx.x & 31) == 0 && l != 0.f) atomicAdd(&k.loss[1], l);
}

// one warp per row again
__global__ void __launch_bounds__(256) kge_finish_kernel(const KgeArgs k) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int D = k.D;
  if (row >= k.bs + k.C * k.ns) return;
  if (row >= k.bs) {
    const int j = row - k.bs;
    const float cs = k.colsum[j];
    for (int d = lane; d < D; d += 32) {
      float g = k.GB[static_cast<size_t>(j) * k.Dp + d];
      if (k.model == 0) g -= cs * __bfloat162float(k.Bn[static_cast<size_t>(j) * k.Dp + d]);
      k.gneg[static_cast<size_t>(j) * D + d] = g;
    }
    return;
  }
  const int i = row;
  const float rs = k.rowsum[i];
  float* gh = k.gh + static_cast<size_t>(i) * D;
  float* gr = k.gr + static_cast<size_t>(i) * D;
  float* gt = k.gt + static_cast<size_t>(i) * D;
  for (int d = lane; d < D; d += 32) {
    float ga = k.GA[static_cast<size_t>(i) * k.Dp + d];
    if (k.model == 0) {
      ga -= rs * __bfloat162float(k.A[static_cast<size_t>(i) * k.Dp + d]);
      if (k.corrupt_head) { gt[d] += ga; gr[d] -= ga; }    // a = t - r
      else { gh[d] += ga; gr[d] += ga; }                   // a = h + r
    } else {
      const float rv = k.r[static_cast<size_t>(i) * D + d];
      if (k.corrupt_head) { gt[d] += ga * rv; gr[d] += ga * k.t[static_cast<size_t>(i) * D + d]; }
      else { gh[d] += ga * rv; gr[d] += ga * k.h[static_cast<size_t>(i) * D + d]; }
    }
  }
}

}  // namespace

// stage: 0 prepare, 1 negative loss, 2 finish.  `args` is the flat pointer / size block below.
RS_API int rs_kge_stage(int stage, const float* h, const float* r, const float* t, const float* neg, int bs, int cs, int ns,
                        int D, int Dp, int model, int corrupt_head, float gamma, void* A, void* Bn, float* a2, float* b2,
                        float* loss, float* gh, float* gr, float* gt, float* gneg, const float* S, void* W, float* rowsum,
                        float* colsum, const float* GA, const float* GB, float* pos_score, float* neg_score,
                        cudaStream_t stream) {
  RS_REQUIRE(bs > 0 && cs > 0 && bs % cs == 0 && ns > 0 && D > 0 && Dp >= D, "rs_kge_stage: bad sizes");
  RS_REQUIRE(model == 0 || model == 1, "rs_kge_stage: model must be 0 (TransE_l2) or 1 (DistMult)");
  KgeArgs k;
  k.h = h; k.r = r; k.t = t; k.neg = neg; k.bs = bs; k.cs = cs; k.ns = ns; k.C = bs / cs; k.D = D; k.Dp = Dp;
  k.model = model; k.corrupt_head = corrupt_head; k.gamma = gamma;
  k.A = reinterpret_cast<__nv_bfloat16*>(A); k.Bn = reinterpret_cast<__nv_bfloat16*>(Bn); k.a2 = a2; k.b2 = b2; k.loss = loss;
  k.gh = gh; k.gr = gr; k.gt = gt; k.gneg = gneg; k.S = S; k.W = reinterpret_cast<__nv_bfloat16*>(W);
  k.rowsum = rowsum; k.colsum = colsum; k.GA = GA; k.GB = GB; k.pos_score = pos_score; k.neg_score = neg_score;
  const int rows = bs + k.C * ns;
  if (stage == 0) {
    kge_prepare_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(k);
  } else if (stage == 1) {
    const long long n = static_cast<long long>(bs) * k.C * ns;
    kge_neg_loss_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(k);
  } else if (stage == 2) {
    kge_finish_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(k);
  } else {
    return rs::set_error(RS_ERR_INVALID, "rs_kge_stage: unknown stage %d", stage);
  }
  RS_LAUNCH_CHECK();
  return RS_OK;
}
