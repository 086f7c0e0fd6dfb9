// Projection interaction of DLRM_Projection: the pairwise products of two learned projections of the
// feature matrix replace the all-pairs dot interaction.
//
// Reference: InteractionProjectionArch (model_zoo/dlrm.py:289-404).  With the flattened features
// X [B, F*D], two branches b1 = relu(X P1^T + c1) [B, I1*D] and b2 = relu(X P2^T + c2) [B, I2*D] are
// produced (tcgen05 GEMMs with the ReLU in their epilogue, ops/gemm_tcgen05.cu); this file has what
// lies between them and the over-arch:
//   forward : z[b] = [ x_dense[b] | b1[b] (I1 x D) . b2[b] (I2 x D)^T flattened | 0 pad ]
//   backward: db1[b, i, :] = [b1 > 0] * sum_j dz[b, D + i*I2 + j] * b2[b, j, :]   (and the mirror for db2)
// One warp per sample; a lane owns 4 contiguous elements of every row, so all loads are 8-byte and the
// I1*I2 dot products are reduced with shuffles.  The ReLU masks of the branches are applied here, so the
// dgrad / wgrad GEMMs that follow take db1, db2 as they are.
#include <cuda_bf16.h>
#include <cstdint>

#include "common/rs_common.h"

namespace {

constexpr int kMaxBranch = 8;       // rows per branch (kernels are instantiated for up to 4 and up to 8)

__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 o0 = __floats2bfloat162_rn(v[0], v[1]), o1 = __floats2bfloat162_rn(v[2], v[3]);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t*>(&o0);
  o.y = *reinterpret_cast<uint32_t*>(&o1);
  *reinterpret_cast<uint2*>(p) = o;
}

struct ProjArgs {
  const __nv_bfloat16* T; int ldT;          // features [B, >= D]: the dense part is columns [0, D)
  const __nv_bfloat16* b1; const __nv_bfloat16* b2;   // [B, I1*D], [B, I2*D]
  int B, I1, I2, D;
  __nv_bfloat16* z; int ldz, Kz;            // forward output / backward input [B, Kz]
  __nv_bfloat16* db1; __nv_bfloat16* db2;   // backward outputs
};

template <int MI>
__global__ void __launch_bounds__(256) proj_inter_fwd_kernel(const ProjArgs a) {
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= a.B) return;
  float acc[MI][MI];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < MI; ++j) acc[i][j] = 0.f;
  const __nv_bfloat16* r1 = a.b1 + static_cast<size_t>(b) * a.I1 * a.D;
  const __nv_bfloat16* r2 = a.b2 + static_cast<size_t>(b) * a.I2 * a.D;
  __nv_bfloat16* z = a.z + static_cast<size_t>(b) * a.ldz;
  for (int d = lane * 4; d < a.D; d += 128) {
    float p[MI][4], q[MI][4];
#pragma unroll
    for (int i = 0; i < MI; ++i)
      if (i < a.I1) load4(r1 + i * a.D + d, p[i]);
#pragma unroll
    for (int j = 0; j < MI; ++j)
      if (j < a.I2) load4(r2 + j * a.D + d, q[j]);
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int j = 0; j < MI; ++j)
        if (i < a.I1 && j < a.I2) acc[i][j] += p[i][0] * q[j][0] + p[i][1] * q[j][1] + p[i][2] * q[j][2] + p[i][3] * q[j][3];
    *reinterpret_cast<uint2*>(z + d) = __ldg(reinterpret_cast<const uint2*>(a.T + static_cast<size_t>(b) * a.ldT + d));
  }
  const int npair = a.I1 * a.I2;
  float mine[2] = {0.f, 0.f};                // pairs lane and lane + 32
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < MI; ++j) {
      if (i < a.I1 && j < a.I2) {
        float v = acc[i][j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        const int pidx = i * a.I2 + j;
        if ((pidx & 31) == lane) mine[pidx >> 5] = v;
      }
    }
  for (int c = a.D + lane; c < a.Kz; c += 32) {
    const int pidx = c - a.D;
    z[c] = __float2bfloat16(pidx < npair ? mine[pidx >> 5] : 0.f);
  }
}

template <int MI>
__global__ void __launch_bounds__(256) proj_inter_bwd_kernel(const ProjArgs a) {
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= a.B) return;
  float g[MI][MI];
  const __nv_bfloat16* dz = a.z + static_cast<size_t>(b) * a.ldz + a.D;
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < MI; ++j) g[i][j] = (i < a.I1 && j < a.I2) ? __bfloat162float(dz[i * a.I2 + j]) : 0.f;
  const size_t o1 = static_cast<size_t>(b) * a.I1 * a.D, o2 = static_cast<size_t>(b) * a.I2 * a.D;
  for (int d = lane * 4; d < a.D; d += 128) {
    float p[MI][4], q[MI][4];
#pragma unroll
    for (int i = 0; i < MI; ++i)
      if (i < a.I1) load4(a.b1 + o1 + i * a.D + d, p[i]);
#pragma unroll
    for (int j = 0; j < MI; ++j)
      if (j < a.I2) load4(a.b2 + o2 + j * a.D + d, q[j]);
#pragma unroll
    for (int i = 0; i < MI; ++i) {
      if (i < a.I1) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < MI; ++j)
          if (j < a.I2) {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] += g[i][j] * q[j][e];
          }
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (!(p[i][e] > 0.f)) v[e] = 0.f;
        store4(a.db1 + o1 + i * a.D + d, v);
      }
    }
#pragma unroll
    for (int j = 0; j < MI; ++j) {
      if (j < a.I2) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < MI; ++i)
          if (i < a.I1) {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] += g[i][j] * p[i][e];
          }
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (!(q[j][e] > 0.f)) v[e] = 0.f;
        store4(a.db2 + o2 + j * a.D + d, v);
      }
    }
  }
}

int check(const ProjArgs& a, const char* who) {
  RS_REQUIRE(a.b1 && a.b2 && a.z && a.B >= 0, "%s: null argument", who);
  RS_REQUIRE(a.I1 >= 1 && a.I1 <= kMaxBranch && a.I2 >= 1 && a.I2 <= kMaxBranch, "%s: branch sizes must be 1..%d", who, kMaxBranch);
  RS_REQUIRE(a.D > 0 && a.D % 4 == 0 && a.ldz % 4 == 0 && a.Kz >= a.D + a.I1 * a.I2 && a.ldz >= a.Kz, "%s: bad sizes", who);
  return RS_OK;
}

}  // namespace

RS_API int rs_proj_inter_fwd(const void* T, int ldT, const void* b1, const void* b2, int B, int I1, int I2, int D, void* z,
                             int ldz, int Kz, cudaStream_t stream) {
  ProjArgs a{};
  a.T = reinterpret_cast<const __nv_bfloat16*>(T); a.ldT = ldT;
  a.b1 = reinterpret_cast<const __nv_bfloat16*>(b1); a.b2 = reinterpret_cast<const __nv_bfloat16*>(b2);
  a.B = B; a.I1 = I1; a.I2 = I2; a.D = D; a.z = reinterpret_cast<__nv_bfloat16*>(z); a.ldz = ldz; a.Kz = Kz;
  if (int rc = check(a, "rs_proj_inter_fwd")) return rc;
  RS_REQUIRE(T && ldT % 4 == 0 && ldT >= D, "rs_proj_inter_fwd: bad feature matrix");
  if (B == 0) return RS_OK;
  if (I1 <= 4 && I2 <= 4) proj_inter_fwd_kernel<4><<<(B + 7) / 8, 256, 0, stream>>>(a);
  else proj_inter_fwd_kernel<kMaxBranch><<<(B + 7) / 8, 256, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_proj_inter_bwd(const void* dz, int ldz, int Kz, const void* b1, const void* b2, int B, int I1, int I2, int D,
                             void* db1, void* db2, cudaStream_t stream) {
  ProjArgs a{};
  a.b1 = reinterpret_cast<const __nv_bfloat16*>(b1); a.b2 = reinterpret_cast<const __nv_bfloat16*>(b2);
  a.B = B; a.I1 = I1; a.I2 = I2; a.D = D;
  a.z = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dz)); a.ldz = ldz; a.Kz = Kz;
  a.db1 = reinterpret_cast<__nv_bfloat16*>(db1); a.db2 = reinterpret_cast<__nv_bfloat16*>(db2);
  if (int rc = check(a, "rs_proj_inter_bwd")) return rc;
  RS_REQUIRE(db1 && db2, "rs_proj_inter_bwd: null output");
  if (B == 0) return RS_OK;
  if (I1 <= 4 && I2 <= 4) proj_inter_bwd_kernel<4><<<(B + 7) / 8, 256, 0, stream>>>(a);
  else proj_inter_bwd_kernel<kMaxBranch><<<(B + 7) / 8, 256, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
