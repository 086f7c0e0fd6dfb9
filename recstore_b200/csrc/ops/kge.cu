// Knowledge-graph embedding scoring with chunked shared negatives and the log-sigmoid loss, forward
// and backward, for six score functions: TransE (L2 and L1), DistMult, ComplEx, SimplE, RotatE.
//
// Math of the reference (src/kg/kg/dgl-ke/python/dglke/models/pytorch/score_fun.py:26-108 TransE,
// 222-286 DistMult, 288-368 ComplEx, 440-538 RotatE, 540-641 SimplE; loss.py:69-99;
// general_models.py:568-631).  A batch of `bs` positives is cut into chunks of `cs`; every chunk
// shares `ns` negative entities; loss = ( mean(-logsigmoid(pos)) + mean(-logsigmoid(-neg)) ) / 2.
// With x the entity that is kept (h when tails are corrupted, t when heads are) and y the other one,
// every model is  score = f( a(x, r), e )  with e = y for the positive and e = a negative entity:
//   TransE_l2  a = h + r | t - r                     score = gamma - ||a - e||_2
//   DistMult   a = x * r                             score = a . e
//   ComplEx    a = x (*) r | x (*) conj(r)           score = a . e      (entities are [re | im] halves)
//   SimplE     a = [x_j * r_inv | x_i * r] / 2 (tails) or [x_j * r | x_i * r_inv] / 2 (heads)
//                                                    score = clamp(a . e, -20, 20)
//   TransE_l1  a = h + r | t - r                     score = gamma - sum |a - e|
//   RotatE     a = x (*) rot(r) | x (*) conj(rot(r)) score = gamma - sum_k |a_k - e_k| (complex modulus),
//              rot(r) = exp(i r pi / emb_init), relations are dim / 2 phases
//
// GEMM family (TransE_l2 and the three bilinear models): the cross products a.e' over all negatives
// are ONE bf16 tensor-core GEMM over the whole batch (rs_gemm_bf16, tcgen05): S[bs, C*ns] = A . Neg^T,
// of which the chunk-diagonal blocks are consumed.  This file has the element-wise stages around it:
//   kge_prepare : a (bf16 copy for the GEMM), |a|^2, |e'|^2, positive scores, positive loss and the
//                 positive gradient of y
//   kge_neg_loss: S -> negative scores -> loss, and the weight matrix W (bf16, zero outside the
//                 chunk-diagonal) with its row / column sums for the backward GEMMs
//                 GA = W . Neg (mode 2), GB = W^T . A (mode 1)
//   kge_finish  : GA, GB -> gradients of x, r and of the negative entities
// Pairwise family (TransE_l1, RotatE): sum |a - e'| is not a contraction, so three fp32 kernels walk
// the (positive, negative) pairs of each chunk: kge_pair_forward (a warp per 4 x 8 pairs),
// kge_pair_grad_pos (a thread per element of 8 positives, looping over the chunk's negatives) and
// kge_pair_grad_neg (the transpose).  No atomics on the gradients: every output element has one owner.
#include <cuda_bf16.h>
#include "common/rs_common.h"

namespace {

enum : int { kTransE2 = 0, kDistMult = 1, kComplEx = 2, kSimplE = 3, kTransE1 = 4, kRotatE = 5, kRescal = 6 };
__host__ __device__ __forceinline__ bool is_pairwise(int model) { return model == kTransE1 || model == kRotatE; }
constexpr int kRescalCols = 16;   // columns of the relation matrix per lane: D <= 512
constexpr float kPi = 3.14159265358979323846f;

struct KgeArgs {
  const float* h; const float* r; const float* t;   // [bs, D] ([bs, Dr] for r)
  const float* neg;                                  // [C*ns, D]
  int bs, cs, ns, C, D, Dp, Dr;                      // Dp: padded row length of the bf16 operands; Dr: relation row length
  int model;
  int corrupt_head;                                  // 0: negatives replace tails, 1: heads
  float gamma, emb_init;
  __nv_bfloat16* A;                                  // [bs, Dp]
  __nv_bfloat16* Bn;                                 // [C*ns, Dp]
  float* a2; float* b2;                              // [bs], [C*ns]; a2 holds d loss / d pos score for the non-TransE_l2 models
  float* loss;                                       // [2]: positive part, negative part (already averaged and halved)
  float* gh; float* gr; float* gt;                   // gradients: [bs, D], [bs, Dr], [bs, D]
  float* gneg;                                       // [C*ns, D]
  const float* S;                                    // [bs, C*ns] cross products
  __nv_bfloat16* W;                                  // [bs, C*ns]
  float* rowsum; float* colsum;                      // [bs], [C*ns]
  const float* GA; const float* GB;                  // [bs, Dp], [C*ns, Dp]
  float* A32;                                        // pairwise family: a in fp32, [bs, Dp] (the GA buffer)
  float* Wf;                                         // pairwise family: d loss / d neg score, [bs, ns] (the S buffer)
  float* pos_score; float* neg_score;                // optional outputs (evaluation / tests): [bs], [bs, ns]
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(__expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoid(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float sgn(float v) { return v > 0.f ? 1.f : (v < 0.f ? -1.f : 0.f); }

// ---- bilinear models on the element pair (k, k + D/2): a = bil(x, r) and its transpose ----------------------------
__device__ __forceinline__ void bil_fwd(int model, bool ch, float x0, float x1, float r0, float r1, float& a0, float& a1) {
  if (model == kDistMult) {
    a0 = x0 * r0; a1 = x1 * r1;
  } else if (model == kComplEx) {
    const float s = ch ? -1.f : 1.f;
    a0 = x0 * r0 - s * x1 * r1; a1 = x1 * r0 + s * x0 * r1;
  } else {  // SimplE: r0 = r, r1 = r_inv; x0 = head role, x1 = tail role
    if (!ch) { a0 = 0.5f * x1 * r1; a1 = 0.5f * x0 * r0; }
    else { a0 = 0.5f * x1 * r0; a1 = 0.5f * x0 * r1; }
  }
}
__device__ __forceinline__ void bil_bwd(int model, bool ch, float g0, float g1, float x0, float x1, float r0, float r1,
                                        float& dx0, float& dx1, float& dr0, float& dr1) {
  if (model == kDistMult) {
    dx0 = g0 * r0; dx1 = g1 * r1; dr0 = g0 * x0; dr1 = g1 * x1;
  } else if (model == kComplEx) {
    const float s = ch ? -1.f : 1.f;
    dx0 = g0 * r0 + s * g1 * r1; dx1 = g1 * r0 - s * g0 * r1;
    dr0 = g0 * x0 + g1 * x1;     dr1 = s * (g1 * x0 - g0 * x1);
  } else {
    if (!ch) { dx1 = 0.5f * g0 * r1; dr1 = 0.5f * g0 * x1; dx0 = 0.5f * g1 * r0; dr0 = 0.5f * g1 * x0; }
    else { dx1 = 0.5f * g0 * r0; dr0 = 0.5f * g0 * x1; dx0 = 0.5f * g1 * r1; dr1 = 0.5f * g1 * x0; }
  }
}

// ---- pairwise models on the element pair (k, k + D/2) -------------------------------------------------------------
// distance contribution of one pair of differences and its direction (d psi / d difference)
__device__ __forceinline__ float pair_psi(int model, float d0, float d1, float& u0, float& u1) {
  if (model == kTransE1) { u0 = sgn(d0); u1 = sgn(d1); return fabsf(d0) + fabsf(d1); }
  const float m = sqrtf(d0 * d0 + d1 * d1);
  const float inv = m > 0.f ? 1.f / m : 0.f;
  u0 = d0 * inv; u1 = d1 * inv;
  return m;
}
__device__ __forceinline__ float pair_dist(int model, float d0, float d1) {
  return model == kTransE1 ? fabsf(d0) + fabsf(d1) : sqrtf(d0 * d0 + d1 * d1);
}

// one warp per row: rows [0, bs) are positives, rows [bs, bs + C*ns) negatives
__global__ void __launch_bounds__(256) kge_prepare_kernel(const KgeArgs k) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int D = k.D, H = k.D >> 1;
  if (row >= k.bs + k.C * k.ns) return;
  if (row >= k.bs) {
    if (is_pairwise(k.model)) return;                // the pairwise kernels read the fp32 rows themselves
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
  const float* r = k.r + static_cast<size_t>(i) * k.Dr;
  const float* t = k.t + static_cast<size_t>(i) * D;
  float* gh = k.gh + static_cast<size_t>(i) * D;
  float* gr = k.gr + static_cast<size_t>(i) * k.Dr;
  float* gt = k.gt + static_cast<size_t>(i) * D;
  const float inv_bs = 0.5f / static_cast<float>(k.bs);

  if (k.model == kTransE2) {
    float a2 = 0.f, pos = 0.f;
    for (int d = lane; d < k.Dp; d += 32) {
      float a = 0.f;
      if (d < D) {
        const float hv = h[d], rv = r[d], tv = t[d];
        a = k.corrupt_head ? tv - rv : hv + rv;
        const float diff = hv + rv - tv;
        pos += diff * diff;
      }
      const __nv_bfloat16 ab = __float2bfloat16(a);
      k.A[static_cast<size_t>(i) * k.Dp + d] = ab;
      const float av = __bfloat162float(ab);
      a2 += av * av;
    }
    a2 = warp_sum(a2);
    pos = warp_sum(pos);
    const float dist = sqrtf(fmaxf(pos, 1e-30f));
    const float score = k.gamma - dist;
    const float q = -sigmoid(-score) * inv_bs;      // d loss / d score of a positive
    if (lane == 0) {
      k.a2[i] = a2;
      if (k.pos_score) k.pos_score[i] = score;
      atomicAdd(&k.loss[0], -log_sigmoid(score) * inv_bs);
    }
    for (int d = lane; d < D; d += 32) {
      const float g = -q * (h[d] + r[d] - t[d]) / dist;   // d score / d h = -(h + r - t) / dist
      gh[d] = g; gr[d] = g; gt[d] = -g;
    }
    return;
  }

  const bool ch = k.corrupt_head != 0;
  const float* x = ch ? t : h;
  const float* y = ch ? h : t;
  float* gy = ch ? gh : gt;
  if (k.model == kRescal) {
    // RESCAL: score = h^T M t with one D x D matrix M per relation (row-major in r).  Tails corrupted: a = M^T h, heads
    // corrupted: a = M t; either way pos = a . y and the negatives' scores are the cross products a . e'.
    // (score_fun.py:378-449 of the reference's DGL-KE.)
    float* a32 = k.A32 + static_cast<size_t>(i) * k.Dp;   // fp32 copy of a for this kernel (the GEMM overwrites it later)
    __nv_bfloat16* A = k.A + static_cast<size_t>(i) * k.Dp;
    if (!ch) {                                        // a_j = sum_i h_i M[i][j]: every lane owns columns j = lane + 32 c
      float acc[kRescalCols];
#pragma unroll
      for (int c = 0; c < kRescalCols; ++c) acc[c] = 0.f;
      for (int row = 0; row < D; ++row) {
        const float hv = x[row];
        const float* m = r + static_cast<size_t>(row) * D;
#pragma unroll
        for (int c = 0; c < kRescalCols; ++c) {
          const int j = lane + 32 * c;
          if (j < D) acc[c] += hv * m[j];
        }
      }
#pragma unroll
      for (int c = 0; c < kRescalCols; ++c) {
        const int j = lane + 32 * c;
        if (j < D) a32[j] = acc[c];
      }
    } else {                                          // a_i = sum_j M[i][j] t_j: a row's dot product per step
      float xv[kRescalCols];
#pragma unroll
      for (int c = 0; c < kRescalCols; ++c) {
        const int j = lane + 32 * c;
        xv[c] = j < D ? x[j] : 0.f;
      }
      for (int row = 0; row < D; ++row) {
        const float* m = r + static_cast<size_t>(row) * D;
        float p = 0.f;
#pragma unroll
        for (int c = 0; c < kRescalCols; ++c) {
          const int j = lane + 32 * c;
          if (j < D) p += m[j] * xv[c];
        }
        p = warp_sum(p);
        if (lane == 0) a32[row] = p;
      }
    }
    __syncwarp();
    float pos = 0.f;
    for (int d = lane; d < k.Dp; d += 32) {
      const float a = d < D ? a32[d] : 0.f;
      A[d] = __float2bfloat16(a);
      if (d < D) pos += a * y[d];
    }
    pos = warp_sum(pos);
    const float q = -sigmoid(-pos) * inv_bs;
    if (lane == 0) {
      k.a2[i] = q;
      if (k.pos_score) k.pos_score[i] = pos;
      atomicAdd(&k.loss[0], -log_sigmoid(pos) * inv_bs);
    }
    for (int d = lane; d < D; d += 32) gy[d] = q * a32[d];
    return;
  }
  if (k.model <= kSimplE) {                           // bilinear: a = bil(x, r), pos = a . y
    float pos = 0.f;
    __nv_bfloat16* A = k.A + static_cast<size_t>(i) * k.Dp;
    for (int kk = lane; kk < H; kk += 32) {
      float a0, a1;
      bil_fwd(k.model, ch, x[kk], x[kk + H], r[kk], r[kk + H], a0, a1);
      A[kk] = __float2bfloat16(a0); A[kk + H] = __float2bfloat16(a1);
      pos += a0 * y[kk] + a1 * y[kk + H];
    }
    for (int d = D + lane; d < k.Dp; d += 32) A[d] = __float2bfloat16(0.f);
    pos = warp_sum(pos);
    float score = pos, pass = 1.f;
    if (k.model == kSimplE) { score = fminf(fmaxf(pos, -20.f), 20.f); pass = (pos >= -20.f && pos <= 20.f) ? 1.f : 0.f; }
    const float q = -sigmoid(-score) * inv_bs * pass;
    if (lane == 0) {
      k.a2[i] = q;
      if (k.pos_score) k.pos_score[i] = score;
      atomicAdd(&k.loss[0], -log_sigmoid(score) * inv_bs);
    }
    for (int kk = lane; kk < H; kk += 32) {          // d pos / d y = a (recomputed in fp32)
      float a0, a1;
      bil_fwd(k.model, ch, x[kk], x[kk + H], r[kk], r[kk + H], a0, a1);
      gy[kk] = q * a0; gy[kk + H] = q * a1;
    }
    return;
  }

  // pairwise: a in fp32 for the pair kernels, pos = gamma - sum psi(a - y)
  const float sg = ch ? -1.f : 1.f;
  const float to_phase = kPi / k.emb_init;
  float* A32 = k.A32 + static_cast<size_t>(i) * k.Dp;
  float dist = 0.f;
  for (int kk = lane; kk < H; kk += 32) {
    float a0, a1;
    if (k.model == kTransE1) {
      a0 = x[kk] + sg * r[kk]; a1 = x[kk + H] + sg * r[kk + H];
    } else {
      float sn, c;
      __sincosf(r[kk] * to_phase, &sn, &c);
      a0 = x[kk] * c - sg * x[kk + H] * sn; a1 = sg * x[kk] * sn + x[kk + H] * c;
    }
    A32[kk] = a0; A32[kk + H] = a1;
    dist += pair_dist(k.model, a0 - y[kk], a1 - y[kk + H]);
  }
  dist = warp_sum(dist);
  const float score = k.gamma - dist;
  const float q = -sigmoid(-score) * inv_bs;
  if (lane == 0) {
    k.a2[i] = q;
    if (k.pos_score) k.pos_score[i] = score;
    atomicAdd(&k.loss[0], -log_sigmoid(score) * inv_bs);
  }
  for (int kk = lane; kk < H; kk += 32) {            // d loss / d y = q * (-1) * (-u)
    float u0, u1;
    pair_psi(k.model, A32[kk] - y[kk], A32[kk + H] - y[kk + H], u0, u1);
    gy[kk] = q * u0; gy[kk + H] = q * u1;
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
      if (k.model == kTransE2) {
        const float dist = sqrtf(fmaxf(k.a2[i] + k.b2[col] - 2.f * dot, 1e-30f));
        score = k.gamma - dist;
        wgt = sigmoid(score) * norm / dist;      // q / dist
      } else if (k.model == kSimplE) {
        score = fminf(fmaxf(dot, -20.f), 20.f);
        wgt = (dot >= -20.f && dot <= 20.f) ? sigmoid(score) * norm : 0.f;
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
  const int D = k.D, H = k.D >> 1;
  if (row >= k.bs + k.C * k.ns) return;
  if (row >= k.bs) {
    const int j = row - k.bs;
    const float cs = k.colsum[j];
    for (int d = lane; d < D; d += 32) {
      float g = k.GB[static_cast<size_t>(j) * k.Dp + d];
      if (k.model == kTransE2) g -= cs * __bfloat162float(k.Bn[static_cast<size_t>(j) * k.Dp + d]);
      k.gneg[static_cast<size_t>(j) * D + d] = g;
    }
    return;
  }
  const int i = row;
  float* gh = k.gh + static_cast<size_t>(i) * D;
  float* gr = k.gr + static_cast<size_t>(i) * k.Dr;
  float* gt = k.gt + static_cast<size_t>(i) * D;
  const float* GA = k.GA + static_cast<size_t>(i) * k.Dp;
  if (k.model == kTransE2) {
    const float rs = k.rowsum[i];
    for (int d = lane; d < D; d += 32) {
      const float ga = GA[d] - rs * __bfloat162float(k.A[static_cast<size_t>(i) * k.Dp + d]);
      if (k.corrupt_head) { gt[d] += ga; gr[d] -= ga; }    // a = t - r
      else { gh[d] += ga; gr[d] += ga; }                   // a = h + r
    }
    return;
  }
  if (k.model == kRescal) {
    // g = d loss / d a = q * y + GA.  Tails corrupted (a = M^T h): dh = M g, dM[i][j] = h_i g_j.  Heads corrupted
    // (a = M t): dt = M^T g, dM[i][j] = g_i t_j.  rowsum[i] receives |dM|^2 = |g|^2 |x|^2, the squared norm of this
    // occurrence's whole matrix gradient: the row-blocked relation table turns it into ONE Adagrad state per relation.
    const bool chr = k.corrupt_head != 0;
    const float* x = (chr ? k.t : k.h) + static_cast<size_t>(i) * D;
    const float* y = (chr ? k.h : k.t) + static_cast<size_t>(i) * D;
    const float* M = k.r + static_cast<size_t>(i) * k.Dr;
    float* gx = chr ? gt : gh;
    float* g = const_cast<float*>(GA);               // this kernel is the last reader of GA: g is formed in place
    const float q = k.a2[i];
    float g2 = 0.f, x2 = 0.f;
    for (int d = lane; d < D; d += 32) {
      const float gv = q * y[d] + GA[d];
      g[d] = gv;
      g2 += gv * gv;
      x2 += x[d] * x[d];
    }
    g2 = warp_sum(g2);
    x2 = warp_sum(x2);
    if (lane == 0) k.rowsum[i] = g2 * x2;
    __syncwarp();
    float gv[kRescalCols], xv[kRescalCols], acc[kRescalCols];
#pragma unroll
    for (int c = 0; c < kRescalCols; ++c) {
      const int j = lane + 32 * c;
      gv[c] = j < D ? g[j] : 0.f;
      xv[c] = j < D ? x[j] : 0.f;
      acc[c] = 0.f;
    }
    for (int row = 0; row < D; ++row) {
      const float* m = M + static_cast<size_t>(row) * D;
      float* dm = gr + static_cast<size_t>(row) * D;
      if (!chr) {                                     // dh_row = M[row,:] . g ; dM[row][j] = h_row g_j
        const float hv = x[row];
        float p = 0.f;
#pragma unroll
        for (int c = 0; c < kRescalCols; ++c) {
          const int j = lane + 32 * c;
          if (j < D) { p += m[j] * gv[c]; dm[j] = hv * gv[c]; }
        }
        p = warp_sum(p);
        if (lane == 0) gx[row] = p;
      } else {                                        // dt_j += g_row M[row][j] ; dM[row][j] = g_row t_j
        const float gr_ = g[row];
#pragma unroll
        for (int c = 0; c < kRescalCols; ++c) {
          const int j = lane + 32 * c;
          if (j < D) { acc[c] += gr_ * m[j]; dm[j] = gr_ * xv[c]; }
        }
      }
    }
    if (chr) {
#pragma unroll
      for (int c = 0; c < kRescalCols; ++c) {
        const int j = lane + 32 * c;
        if (j < D) gx[j] = acc[c];
      }
    }
    return;
  }
  // bilinear: d loss / d a = q * y (positive) + GA (negatives); chain through a = bil(x, r)
  const bool ch = k.corrupt_head != 0;
  const float* x = (ch ? k.t : k.h) + static_cast<size_t>(i) * D;
  const float* y = (ch ? k.h : k.t) + static_cast<size_t>(i) * D;
  const float* r = k.r + static_cast<size_t>(i) * k.Dr;
  float* gx = ch ? gt : gh;
  const float q = k.a2[i];
  for (int kk = lane; kk < H; kk += 32) {
    const float g0 = q * y[kk] + GA[kk], g1 = q * y[kk + H] + GA[kk + H];
    float dx0, dx1, dr0, dr1;
    bil_bwd(k.model, ch, g0, g1, x[kk], x[kk + H], r[kk], r[kk + H], dx0, dx1, dr0, dr1);
    gx[kk] = dx0; gx[kk + H] = dx1; gr[kk] = dr0; gr[kk + H] = dr1;
  }
}

// ---- pairwise family ---------------------------------------------------------------------------------------------
// A warp scores 4 positives against 8 negatives of their chunk: every lane strides over the element pairs and keeps
// 32 partial distances, which a transposing butterfly reduces so that lane l ends with pair (l / 8, l % 8).
__global__ void __launch_bounds__(256) kge_pair_forward_kernel(const KgeArgs k) {
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int jt = k.ns >> 3;                        // tiles of 8 negatives per chunk
  const int n_warps = (k.bs >> 2) * jt;
  float l = 0.f;
  if (warp < n_warps) {
    const int i0 = (warp / jt) << 2, j0 = (warp % jt) << 3;
    const int c = i0 / k.cs;
    const int H = k.D >> 1;
    const float* a = k.A32 + static_cast<size_t>(i0) * k.Dp;
    const float* n = k.neg + (static_cast<size_t>(c) * k.ns + j0) * k.D;
    float v[32];
#pragma unroll
    for (int p = 0; p < 32; ++p) v[p] = 0.f;
    for (int kk = lane; kk < H; kk += 32) {
      float a0[4], a1[4], n0[8], n1[8];
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) { a0[ii] = a[ii * k.Dp + kk]; a1[ii] = a[ii * k.Dp + kk + H]; }
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) { n0[jj] = n[jj * k.D + kk]; n1[jj] = n[jj * k.D + kk + H]; }
#pragma unroll
      for (int ii = 0; ii < 4; ++ii)
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) v[ii * 8 + jj] += pair_dist(k.model, a0[ii] - n0[jj], a1[ii] - n1[jj]);
    }
#pragma unroll
    for (int o = 16, cnt = 32; o > 0; o >>= 1, cnt >>= 1) {
      const bool upper = (lane & o) != 0;
#pragma unroll
      for (int p = 0; p < cnt / 2; ++p) {
        const float send = upper ? v[p] : v[p + cnt / 2];
        const float keep = upper ? v[p + cnt / 2] : v[p];
        v[p] = keep + __shfl_xor_sync(0xffffffffu, send, o);
      }
    }
    const int i = i0 + (lane >> 3), j = j0 + (lane & 7);
    const float score = k.gamma - v[0];
    const float norm = 1.f / (static_cast<float>(k.bs) * k.ns) * 0.5f;
    k.Wf[static_cast<size_t>(i) * k.ns + j] = sigmoid(score) * norm;     // d loss / d score
    if (k.neg_score) k.neg_score[static_cast<size_t>(i) * k.ns + j] = score;
    l = -log_sigmoid(-score) * norm;
  }
  l = warp_sum(l);
  if (lane == 0 && l != 0.f) atomicAdd(&k.loss[1], l);
}

constexpr int kPairRows = 8;      // rows that share one pass over the other side
constexpr int kPairTile = 256;    // weights staged per pass
constexpr int kPairThreads = 128;

// Block = 8 positives of one chunk x a slab of 128 element pairs; a thread owns one pair index of all 8 rows, walks
// the chunk's negatives and then chains d loss / d a (negatives and the positive) to x and r.
__global__ void __launch_bounds__(kPairThreads) kge_pair_grad_pos_kernel(const KgeArgs k) {
  __shared__ float w[kPairRows][kPairTile];
  const int i0 = blockIdx.x * kPairRows;
  const int c = i0 / k.cs;
  const int H = k.D >> 1;
  const int kk = blockIdx.y * kPairThreads + threadIdx.x;
  const bool live = kk < H;
  float a0[kPairRows], a1[kPairRows], g0[kPairRows], g1[kPairRows];
#pragma unroll
  for (int rr = 0; rr < kPairRows; ++rr) {
    a0[rr] = live ? k.A32[static_cast<size_t>(i0 + rr) * k.Dp + kk] : 0.f;
    a1[rr] = live ? k.A32[static_cast<size_t>(i0 + rr) * k.Dp + kk + H] : 0.f;
    g0[rr] = 0.f; g1[rr] = 0.f;
  }
  for (int jb = 0; jb < k.ns; jb += kPairTile) {
    const int nj = min(kPairTile, k.ns - jb);
    __syncthreads();
    for (int e = threadIdx.x; e < kPairRows * nj; e += kPairThreads) {
      const int rr = e / nj, j = e - rr * nj;
      w[rr][j] = k.Wf[static_cast<size_t>(i0 + rr) * k.ns + jb + j];
    }
    __syncthreads();
    if (live) {
      const float* n = k.neg + (static_cast<size_t>(c) * k.ns + jb) * k.D + kk;
      for (int j = 0; j < nj; ++j) {
        const float n0 = n[static_cast<size_t>(j) * k.D], n1 = n[static_cast<size_t>(j) * k.D + H];
#pragma unroll
        for (int rr = 0; rr < kPairRows; ++rr) {
          float u0, u1;
          pair_psi(k.model, a0[rr] - n0, a1[rr] - n1, u0, u1);
          g0[rr] -= w[rr][j] * u0; g1[rr] -= w[rr][j] * u1;
        }
      }
    }
  }
  if (!live) return;
  const bool ch = k.corrupt_head != 0;
  const float sg = ch ? -1.f : 1.f;
  const float to_phase = kPi / k.emb_init;
#pragma unroll
  for (int rr = 0; rr < kPairRows; ++rr) {
    const int i = i0 + rr;
    const float* x = (ch ? k.t : k.h) + static_cast<size_t>(i) * k.D;
    const float* y = (ch ? k.h : k.t) + static_cast<size_t>(i) * k.D;
    float* gx = (ch ? k.gt : k.gh) + static_cast<size_t>(i) * k.D;
    float* gr = k.gr + static_cast<size_t>(i) * k.Dr;
    float u0, u1;
    pair_psi(k.model, a0[rr] - y[kk], a1[rr] - y[kk + H], u0, u1);
    const float q = k.a2[i];
    const float ga0 = g0[rr] - q * u0, ga1 = g1[rr] - q * u1;
    if (k.model == kTransE1) {
      gx[kk] = ga0; gx[kk + H] = ga1; gr[kk] = sg * ga0; gr[kk + H] = sg * ga1;
    } else {
      float sn, cs_;
      __sincosf(k.r[static_cast<size_t>(i) * k.Dr + kk] * to_phase, &sn, &cs_);
      const float x0 = x[kk], x1 = x[kk + H];
      gx[kk] = ga0 * cs_ + sg * ga1 * sn;
      gx[kk + H] = ga1 * cs_ - sg * ga0 * sn;
      const float dc = ga0 * x0 + ga1 * x1, ds = sg * (ga1 * x0 - ga0 * x1);
      gr[kk] = (ds * cs_ - dc * sn) * to_phase;
    }
  }
}

// Block = 8 negatives of one chunk x a slab of 128 element pairs; a thread walks the chunk's positives.
__global__ void __launch_bounds__(kPairThreads) kge_pair_grad_neg_kernel(const KgeArgs k) {
  __shared__ float w[kPairTile][kPairRows];
  const int col0 = blockIdx.x * kPairRows;          // index into [C*ns]
  const int c = col0 / k.ns, j0 = col0 - c * k.ns;
  const int H = k.D >> 1;
  const int kk = blockIdx.y * kPairThreads + threadIdx.x;
  const bool live = kk < H;
  float n0[kPairRows], n1[kPairRows], g0[kPairRows], g1[kPairRows];
#pragma unroll
  for (int jj = 0; jj < kPairRows; ++jj) {
    n0[jj] = live ? k.neg[static_cast<size_t>(col0 + jj) * k.D + kk] : 0.f;
    n1[jj] = live ? k.neg[static_cast<size_t>(col0 + jj) * k.D + kk + H] : 0.f;
    g0[jj] = 0.f; g1[jj] = 0.f;
  }
  for (int ib = 0; ib < k.cs; ib += kPairTile) {
    const int ni = min(kPairTile, k.cs - ib);
    __syncthreads();
    for (int e = threadIdx.x; e < ni * kPairRows; e += kPairThreads) {
      const int ii = e / kPairRows, jj = e - ii * kPairRows;
      w[ii][jj] = k.Wf[static_cast<size_t>(c * k.cs + ib + ii) * k.ns + j0 + jj];
    }
    __syncthreads();
    if (live) {
      const float* a = k.A32 + static_cast<size_t>(c * k.cs + ib) * k.Dp + kk;
      for (int ii = 0; ii < ni; ++ii) {
        const float a0 = a[static_cast<size_t>(ii) * k.Dp], a1 = a[static_cast<size_t>(ii) * k.Dp + H];
#pragma unroll
        for (int jj = 0; jj < kPairRows; ++jj) {
          float u0, u1;
          pair_psi(k.model, a0 - n0[jj], a1 - n1[jj], u0, u1);
          g0[jj] += w[ii][jj] * u0; g1[jj] += w[ii][jj] * u1;     // d loss / d dist = -w, d dist / d e' = -u
        }
      }
    }
  }
  if (!live) return;
#pragma unroll
  for (int jj = 0; jj < kPairRows; ++jj) {
    k.gneg[static_cast<size_t>(col0 + jj) * k.D + kk] = g0[jj];
    k.gneg[static_cast<size_t>(col0 + jj) * k.D + kk + H] = g1[jj];
  }
}

}  // namespace

// stage: 0 prepare, 1 negative loss, 2 finish.  model: 0 TransE_l2, 1 DistMult, 2 ComplEx, 3 SimplE (these four
// have the GEMMs S = A.Bn^T between stages 0 and 1 and GA = W.Bn, GB = W^T.A between 1 and 2), 4 TransE_l1,
// 5 RotatE (no GEMM: stage 1 and 2 walk the pairs; GA doubles as the fp32 copy of a, S as the pair weights), 6 RESCAL
// (GEMM family; r holds a row-major D x D matrix per positive, gr receives its gradient, rowsum the squared norm of it).
RS_API int rs_kge_stage(int stage, const float* h, const float* r, const float* t, const float* neg, int bs, int cs, int ns,
                        int D, int Dp, int Dr, int model, int corrupt_head, float gamma, float emb_init, void* A, void* Bn,
                        float* a2, float* b2, float* loss, float* gh, float* gr, float* gt, float* gneg, float* S, void* W,
                        float* rowsum, float* colsum, float* GA, const float* GB, float* pos_score, float* neg_score,
                        cudaStream_t stream) {
  RS_REQUIRE(bs > 0 && cs > 0 && bs % cs == 0 && ns > 0 && D > 0 && Dp >= D, "rs_kge_stage: bad sizes");
  RS_REQUIRE(model >= kTransE2 && model <= kRescal, "rs_kge_stage: model must be 0..6");
  RS_REQUIRE(model == kTransE2 || D % 2 == 0, "rs_kge_stage: this model splits the embedding into two halves");
  RS_REQUIRE(Dr == (model == kRotatE ? D / 2 : model == kRescal ? D * D : D), "rs_kge_stage: relation row length");
  RS_REQUIRE(model != kRescal || D <= 32 * kRescalCols, "rs_kge_stage: RESCAL needs dim <= 512");
  const bool pairwise = is_pairwise(model);
  RS_REQUIRE(!pairwise || (cs % kPairRows == 0 && ns % kPairRows == 0 && emb_init > 0.f),
             "rs_kge_stage: TransE_l1 / RotatE need chunk and negative counts that are multiples of 8");
  KgeArgs k;
  k.h = h; k.r = r; k.t = t; k.neg = neg; k.bs = bs; k.cs = cs; k.ns = ns; k.C = bs / cs; k.D = D; k.Dp = Dp; k.Dr = Dr;
  k.model = model; k.corrupt_head = corrupt_head; k.gamma = gamma; k.emb_init = emb_init;
  k.A = reinterpret_cast<__nv_bfloat16*>(A); k.Bn = reinterpret_cast<__nv_bfloat16*>(Bn); k.a2 = a2; k.b2 = b2; k.loss = loss;
  k.gh = gh; k.gr = gr; k.gt = gt; k.gneg = gneg; k.S = S; k.W = reinterpret_cast<__nv_bfloat16*>(W);
  k.rowsum = rowsum; k.colsum = colsum; k.GA = GA; k.GB = GB; k.A32 = GA; k.Wf = S;
  k.pos_score = pos_score; k.neg_score = neg_score;
  const int rows = bs + k.C * ns;
  const int H = D / 2;
  if (stage == 0) {
    kge_prepare_kernel<<<((pairwise ? bs : rows) + 7) / 8, 256, 0, stream>>>(k);
  } else if (stage == 1) {
    if (pairwise) {
      const int warps = (bs / 4) * (ns / 8);
      kge_pair_forward_kernel<<<(warps + 7) / 8, 256, 0, stream>>>(k);
    } else {
      const long long n = static_cast<long long>(bs) * k.C * ns;
      kge_neg_loss_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(k);
    }
  } else if (stage == 2) {
    if (pairwise) {
      const dim3 gp(bs / kPairRows, (H + kPairThreads - 1) / kPairThreads);
      kge_pair_grad_pos_kernel<<<gp, kPairThreads, 0, stream>>>(k);
      RS_LAUNCH_CHECK();
      const dim3 gn(k.C * ns / kPairRows, (H + kPairThreads - 1) / kPairThreads);
      kge_pair_grad_neg_kernel<<<gn, kPairThreads, 0, stream>>>(k);
    } else {
      kge_finish_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(k);
    }
  } else {
    return rs::set_error(RS_ERR_INVALID, "rs_kge_stage: unknown stage %d", stage);
  }
  RS_LAUNCH_CHECK();
  return RS_OK;
}
