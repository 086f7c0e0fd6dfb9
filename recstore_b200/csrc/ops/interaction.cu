// DLRM pairwise-dot feature interaction, forward and backward, one warp per sample.
//
// Forward: T = [x; e_1 .. e_{F-1}] (F x D, bf16, read in place from the buffer that the embedding
// all-to-all and the bottom MLP wrote), Z = T.T^T on tensor cores, output row =
// [x (D values), Z[i][j] for i > j in row-major order (1,0),(2,0),(2,1),...], zero padded to
// `out_ld`.  This is interact_features of the reference (src/executable/dlrm/dlrm_model.py:
// 316-340: bmm + strictly-lower-triangle gather + cat) in one pass over the data.
//
// Backward: dT = (dZ + dZ^T).T with dT[0] += dOut[0:D]; row 0 goes to the bottom-MLP gradient,
// rows 1.. are stored STRAIGHT INTO THE OWNING RANK'S GRADIENT WINDOW through peer pointers
// (the backward all-to-all of extend_distributed.py:444-486 done by the producing kernel).
//
// The per-sample products are 32x32x128 / 32x128x32, far below one tcgen05 tile, and the op is
// bound by the bytes of T; warp-level mma.m16n8k16 keeps it at memory speed.
#include <cuda_bf16.h>
#include "comm/flags.cuh"
#include "common/rs_common.h"

namespace {

constexpr int kMaxF = 32;
constexpr int kMaxD = 128;
constexpr int kLd = kMaxD + 8;       // padded smem row (elements): 272 B, conflict-free ldmatrix
constexpr int kWarps = 4;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Asynchronous 16-byte global -> shared copies: no registers held, so a lane keeps all of its copies of a tile in
// flight at once (a register-staged loop with a run-time trip count issues them one after the other).
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Zero-fills rows F..31 of a padded tile (they never change afterwards).
__device__ __forceinline__ void zero_tail_rows(__nv_bfloat16* sT, int F, int D, int lane) {
  const int vec_per_row = D >> 3;
  for (int i = F * vec_per_row + lane; i < 32 * vec_per_row; i += 32)
    *reinterpret_cast<uint4*>(sT + (i / vec_per_row) * kLd + (i % vec_per_row) * 8) = make_uint4(0, 0, 0, 0);
}
// Starts the copy of the F x D tile of one sample into padded shared memory (rows 0..F-1); the caller waits.
__device__ __forceinline__ void load_tile_async(__nv_bfloat16* sT, const __nv_bfloat16* src, int F, int D, int lane) {
  const int vec_per_row = D >> 3;  // 16 bytes = 8 bf16
  const int total = F * vec_per_row;
  if (vec_per_row == 16) {         // D = 128: shifts instead of a division by a run-time value in every iteration
    for (int i = lane; i < total; i += 32) cp_async16(sT + (i >> 4) * kLd + (i & 15) * 8, src + static_cast<size_t>(i) * 8);
    return;
  }
  for (int i = lane; i < total; i += 32) {
    const int r = i / vec_per_row, v = i % vec_per_row;
    cp_async16(sT + r * kLd + v * 8, src + static_cast<size_t>(r) * D + v * 8);
  }
}

// Persistent warps: every warp walks samples b = first, first + stride, ...; the positions of this lane's
// accumulator elements inside the output row (strict lower triangle, row-major) are worked out once.
__global__ void __launch_bounds__(kWarps * 32) interaction_fwd_kernel(const __nv_bfloat16* __restrict__ T, int B, int F,
                                                                      int D, __nv_bfloat16* __restrict__ out, int out_ld,
                                                                      const rs::FlagWait wait) {
  __shared__ __align__(16) __nv_bfloat16 sT[kWarps][32 * kLd];
  __shared__ __align__(16) __nv_bfloat16 sO[kWarps][kMaxD + kMaxF * (kMaxF - 1) / 2 + 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  rs::flag_wait_all(wait);   // multi-GPU: the peers' pooled rows have landed in T (no-op without flags)
  __nv_bfloat16* t = sT[warp];
  __nv_bfloat16* o = sO[warp];
  zero_tail_rows(t, F, D, lane);
  const int g = lane >> 2, q = lane & 3;
  // offset of acc[mt][nt][e] in the staging row, or -1 outside the strict lower triangle / past F
  short off[2][4][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = mt * 16 + g + (e >> 1) * 8;
        const int j = nt * 8 + q * 2 + (e & 1);
        off[mt][nt][e] = (i < F && j < i) ? static_cast<short>(D + i * (i - 1) / 2 + j) : static_cast<short>(-1);
      }
  const int nvalid = D + F * (F - 1) / 2;
  const int nfull = (nvalid + 7) >> 3;
  const int ksteps = D >> 4;
  for (int b = blockIdx.x * kWarps + warp; b < B; b += gridDim.x * kWarps) {
    load_tile_async(t, T + static_cast<size_t>(b) * F * D, F, D, lane);
    cp_async_wait_all();
    __syncwarp();

    // acc[mt][nt]: rows mt*16.., cols nt*8..; only tiles that touch the strict lower triangle.
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[i][j][k] = 0.f;
    for (int ks = 0; ks < ksteps; ++ks) {
      const int k0 = ks * 16;
      uint32_t a0[4], a1[4], b01[4], b23[4];
      ldmatrix_x4(a0, t + ((lane & 7) + ((lane >> 3) & 1) * 8) * kLd + k0 + (lane >> 4) * 8);
      ldmatrix_x4(a1, t + (16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kLd + k0 + (lane >> 4) * 8);
      // B fragments from the same tile viewed as [n][k]: n-tiles {0,1} and {2,3}.
      ldmatrix_x4(b01, t + ((lane & 7) + (lane >> 4) * 8) * kLd + k0 + ((lane >> 3) & 1) * 8);
      ldmatrix_x4(b23, t + (16 + (lane & 7) + (lane >> 4) * 8) * kLd + k0 + ((lane >> 3) & 1) * 8);
      mma_bf16(acc[0][0], a0, b01[0], b01[1]);
      mma_bf16(acc[0][1], a0, b01[2], b01[3]);
      mma_bf16(acc[1][0], a1, b01[0], b01[1]);
      mma_bf16(acc[1][1], a1, b01[2], b01[3]);
      mma_bf16(acc[1][2], a1, b23[0], b23[1]);
      mma_bf16(acc[1][3], a1, b23[2], b23[3]);
    }

    for (int d = lane * 8; d < D; d += 256) *reinterpret_cast<uint4*>(o + d) = *reinterpret_cast<const uint4*>(t + d);  // row 0 = dense features
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        if (mt == 0 && nt >= 2) continue;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (off[mt][nt][e] >= 0) o[off[mt][nt][e]] = __float2bfloat16(acc[mt][nt][e]);
      }
    // zero the padding inside the last 16-byte group, then copy whole groups; groups past nvalid are zeros
    for (int idx = nvalid + lane; idx < ((nvalid + 7) & ~7); idx += 32) o[idx] = __float2bfloat16(0.f);
    __syncwarp();
    __nv_bfloat16* dst = out + static_cast<size_t>(b) * out_ld;
    for (int v = lane; v < (out_ld >> 3); v += 32) {
      const uint4 x = v < nfull ? *reinterpret_cast<const uint4*>(o + v * 8) : make_uint4(0, 0, 0, 0);
      *(reinterpret_cast<uint4*>(dst) + v) = x;
    }
    __syncwarp();   // the next sample's copies overwrite t and o
  }
}

struct InterBwdArgs {
  const __nv_bfloat16* T;     // [B, F, D]
  const __nv_bfloat16* dout;  // [B, dout_ld]
  int B, F, D, dout_ld;
  __nv_bfloat16* dx;          // [B, dx_ld] gradient of feature 0 (bottom MLP output)
  int dx_ld;
  void* const* gdst;          // [world] gradient windows of the owning ranks
  const int* owner;           // [F-1] owning rank of each embedding feature
  const int* gcol;            // [F-1] element offset inside the owner's gradient row
  long long grow_stride;      // elements per sample row in a gradient window
  long long sample_base;      // this rank's first global sample index (rank * B_local)
  int relu_mask_dx;           // feature 0 is a ReLU output: zero dx where it is not positive
  float* const* ndst;         // optional [world]: per-owner [B_global, nstride] sum of squares of each pushed row
  int nstride;
  int rows;                   // 0 = every row; 1 = only feature 0 (dx); 2 = only the embedding rows (pushed to their owners)
};

constexpr int kWarpsBwd = 6;  // 17 KB of shared memory per warp: two CTAs (12 warps) per SM
constexpr int kOutLd = 72;    // staging row: 64 columns + 8 pad (144 B, 16-byte aligned, conflict-free)
constexpr int kDoutMax = kMaxD + kMaxF * (kMaxF - 1) / 2 + 16;
// per-warp shared memory of the backward kernel (bytes): T tile, symmetric dZ, output staging, dOut row
constexpr int kBwdWarpBytes = 32 * kLd * 2 + 32 * 40 * 2 + 32 * kOutLd * 2 + kDoutMax * 2;

__device__ __forceinline__ void stmatrix_x4(void* p, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Persistent warps: every warp walks samples b = first, first + stride, ...  Everything that does not depend on
// the sample (pair -> (i, j) table, destination pointers of the rows a lane stores) is set up once.
__global__ void __launch_bounds__(kWarpsBwd * 32) interaction_bwd_kernel(const InterBwdArgs a) {
  extern __shared__ __align__(16) unsigned char smem_bwd[];
  __shared__ unsigned short s_ij[kMaxF * (kMaxF - 1) / 2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int F = a.F, D = a.D;
  const int npairs = F * (F - 1) / 2;
  for (int p = threadIdx.x; p < npairs; p += blockDim.x) {
    int i = static_cast<int>((1.f + sqrtf(1.f + 8.f * p)) * 0.5f);
    while (i * (i - 1) / 2 > p) --i;
    while ((i + 1) * i / 2 <= p) ++i;
    s_ij[p] = static_cast<unsigned short>((i << 8) | (p - i * (i - 1) / 2));
  }
  unsigned char* base = smem_bwd + warp * kBwdWarpBytes;
  __nv_bfloat16* t = reinterpret_cast<__nv_bfloat16*>(base);
  __nv_bfloat16* s = t + 32 * kLd;
  __nv_bfloat16* o = s + 32 * 40;
  __nv_bfloat16* sd = o + 32 * kOutLd;
  for (int i = lane; i < 32 * 40 / 8; i += 32) reinterpret_cast<uint4*>(s)[i] = make_uint4(0, 0, 0, 0);
  zero_tail_rows(t, F, D, lane);
  __syncthreads();

  const int g = lane >> 2, q = lane & 3;
  const int orow = lane >> 3, ochunk = lane & 7;  // store phase: 4 rows x 8 chunks of 16 B per instruction
  // destination of the rows this lane stores (row i = it * 4 + orow), without the per-sample offset
  __nv_bfloat16* dst_base[8];
  float* nrm_base[8];
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int i = it * 4 + orow;
    dst_base[it] = nullptr;
    nrm_base[it] = nullptr;
    if (i == 0) {
      if (a.rows != 2) dst_base[it] = a.dx + ochunk * 8;
    } else if (i < F && a.rows != 1) {
      const int f = i - 1;
      dst_base[it] = reinterpret_cast<__nv_bfloat16*>(a.gdst[a.owner[f]]) + a.sample_base * a.grow_stride + a.gcol[f] + ochunk * 8;
      if (a.ndst) nrm_base[it] = a.ndst[a.owner[f]] + a.sample_base * a.nstride + a.gcol[f] / D;
    }
  }
  const int dvec = (a.dout_ld * 2) >> 4;  // uint4 per dOut row

  for (int b = blockIdx.x * kWarpsBwd + warp; b < a.B; b += gridDim.x * kWarpsBwd) {
    load_tile_async(t, a.T + static_cast<size_t>(b) * F * D, F, D, lane);
    const __nv_bfloat16* dout = a.dout + static_cast<size_t>(b) * a.dout_ld;
    for (int v = lane; v < dvec; v += 32) cp_async16(sd + v * 8, dout + v * 8);
    cp_async_wait_all();
    __syncwarp();
    for (int p = lane; p < npairs; p += 32) {
      const int ij = s_ij[p];
      const int i = ij >> 8, j = ij & 255;
      const __nv_bfloat16 v = sd[D + p];
      s[i * 40 + j] = v;
      s[j * 40 + i] = v;
    }
    __syncwarp();

    uint32_t sa[2][2][4];  // [mt][ks]
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int ks = 0; ks < 2; ++ks)
        ldmatrix_x4(sa[mt][ks], s + (mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * 40 + ks * 16 + (lane >> 4) * 8);

    float rownorm[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) rownorm[i] = 0.f;

    for (int n0 = 0; n0 < D; n0 += 64) {
      float acc[2][8][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
          for (int k = 0; k < 4; ++k) acc[i][j][k] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          if (n0 + np * 16 >= D) continue;
          uint32_t bb[4];
          ldmatrix_x4_trans(bb, t + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kLd + n0 + np * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            mma_bf16(acc[mt][np * 2], sa[mt][ks], bb[0], bb[1]);
            mma_bf16(acc[mt][np * 2 + 1], sa[mt][ks], bb[2], bb[3]);
          }
        }
      }
      // row 0 (feature 0): + dOut[0:D], ReLU mask.  Row 0 lives in lanes with g == 0, m-tile 0, elements 0 and 1.
      if (g == 0) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const int col = n0 + nt * 8 + q * 2;
          if (col < D) {
            float v0 = acc[0][nt][0] + __bfloat162float(sd[col]);
            float v1 = acc[0][nt][1] + __bfloat162float(sd[col + 1]);
            if (a.relu_mask_dx) {
              if (!(__bfloat162float(t[col]) > 0.f)) v0 = 0.f;
              if (!(__bfloat162float(t[col + 1]) > 0.f)) v1 = 0.f;
            }
            acc[0][nt][0] = v0;
            acc[0][nt][1] = v1;
          }
        }
      }
      // fragments -> staging tile: one stmatrix.x4 per (m-tile, pair of n-tiles)
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          __nv_bfloat16* dstm = o + (mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kOutLd + (np * 2 + (lane >> 4)) * 8;
          stmatrix_x4(dstm, pack2(acc[mt][np * 2][0], acc[mt][np * 2][1]), pack2(acc[mt][np * 2][2], acc[mt][np * 2][3]),
                      pack2(acc[mt][np * 2 + 1][0], acc[mt][np * 2 + 1][1]), pack2(acc[mt][np * 2 + 1][2], acc[mt][np * 2 + 1][3]));
        }
      __syncwarp();
      // staging tile -> global, 16 bytes per lane, 4 rows per instruction
      if (n0 + ochunk * 8 < D) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          if (dst_base[it] == nullptr) continue;
          const int i = it * 4 + orow;
          const uint4 v = *reinterpret_cast<const uint4*>(o + i * kOutLd + ochunk * 8);
          const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&v);
          float sq = 0.f;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f2 = __bfloat1622float2(vp[e]);
            sq += f2.x * f2.x + f2.y * f2.y;
          }
          rownorm[it] += sq;
          const long long off = (i == 0) ? static_cast<long long>(b) * a.dx_ld : static_cast<long long>(b) * a.grow_stride;
          *reinterpret_cast<uint4*>(dst_base[it] + off + n0) = v;
        }
      }
      __syncwarp();
    }
    if (a.ndst) {
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        float sq = rownorm[it];
        sq += __shfl_xor_sync(0xffffffffu, sq, 1);
        sq += __shfl_xor_sync(0xffffffffu, sq, 2);
        sq += __shfl_xor_sync(0xffffffffu, sq, 4);
        if (ochunk == 0 && nrm_base[it] != nullptr) nrm_base[it][static_cast<long long>(b) * a.nstride] = sq;
      }
    }
  }
}

// Gradient of feature 0 only (the bottom MLP's output): dx = dOut[0:D] + sum_{j>=1} dZ[j][0] * T[j], ReLU-masked.
// One warp per sample, every row load independent: a matrix-vector product at memory speed, so that the bottom
// MLP's backward can start while the full backward (which pushes the embedding gradients) is still running.
__global__ void __launch_bounds__(256, 2) interaction_dx_kernel(const __nv_bfloat16* __restrict__ T, const __nv_bfloat16* __restrict__ dout,
                                                             int B, int F, int D, int dout_ld, __nv_bfloat16* __restrict__ dx,
                                                             int dx_ld, int relu_mask) {
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= B) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* t = T + static_cast<size_t>(b) * F * D;
  const __nv_bfloat16* go = dout + static_cast<size_t>(b) * dout_ld;
  // lane j (1 <= j < F) fetches its coefficient dZ[j][0]; they are broadcast by shuffles below
  float coef = 0.f;
  if (lane >= 1 && lane < F) coef = __bfloat162float(go[D + lane * (lane - 1) / 2]);
  for (int c0 = lane * 4; c0 < D; c0 += 128) {
    float acc[4];
    const uint2 g0 = *reinterpret_cast<const uint2*>(go + c0);
    const uint2 x0 = *reinterpret_cast<const uint2*>(t + c0);
    {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g0.x));
      const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g0.y));
      acc[0] = a.x; acc[1] = a.y; acc[2] = c.x; acc[3] = c.y;
    }
    uint2 rows[kMaxF];
#pragma unroll
    for (int j = 1; j < kMaxF; ++j)
      if (j < F) rows[j] = __ldg(reinterpret_cast<const uint2*>(t + static_cast<size_t>(j) * D + c0));
#pragma unroll
    for (int j = 1; j < kMaxF; ++j) {
      const float w = __shfl_sync(0xffffffffu, coef, j);
      if (j < F) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rows[j].x));
        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rows[j].y));
        acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * c.x; acc[3] += w * c.y;
      }
    }
    if (relu_mask) {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x0.x));
      const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x0.y));
      if (!(a.x > 0.f)) acc[0] = 0.f;
      if (!(a.y > 0.f)) acc[1] = 0.f;
      if (!(c.x > 0.f)) acc[2] = 0.f;
      if (!(c.y > 0.f)) acc[3] = 0.f;
    }
    uint2 o;
    o.x = pack2(acc[0], acc[1]);
    o.y = pack2(acc[2], acc[3]);
    *reinterpret_cast<uint2*>(dx + static_cast<size_t>(b) * dx_ld + c0) = o;
  }
}

}  // namespace

RS_API int rs_interaction_dx(const void* T, const void* dout, int B, int F, int D, int dout_ld, void* dx, int dx_ld,
                             int relu_mask_dx, cudaStream_t stream) {
  RS_REQUIRE(T && dout && dx, "rs_interaction_dx: null argument");
  RS_REQUIRE(F >= 1 && F <= kMaxF && D % 16 == 0 && D >= 16 && D <= kMaxD, "rs_interaction_dx: F=%d D=%d unsupported", F, D);
  RS_REQUIRE(dout_ld % 4 == 0 && dx_ld % 4 == 0, "rs_interaction_dx: leading dimensions must be multiples of 4");
  if (B == 0) return RS_OK;
  interaction_dx_kernel<<<(B + 7) / 8, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(T),
                                                         reinterpret_cast<const __nv_bfloat16*>(dout), B, F, D, dout_ld,
                                                         reinterpret_cast<__nv_bfloat16*>(dx), dx_ld, relu_mask_dx);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

namespace {
int interaction_forward_impl(const void* T, int B, int F, int D, void* out, int out_ld, const rs::FlagWait& wait, cudaStream_t stream);
}
RS_API int rs_interaction_forward(const void* T, int B, int F, int D, void* out, int out_ld, cudaStream_t stream) {
  rs::FlagWait w;
  memset(&w, 0, sizeof(w));
  return interaction_forward_impl(T, B, F, D, out, out_ld, w, stream);
}
// Same, but every CTA first waits (bounded) until all ranks' flags on `wait_channel` have reached this rank's own epoch:
// the forward all-to-all has delivered the peers' rows into T.
RS_API int rs_interaction_forward_ex(const void* T, int B, int F, int D, void* out, int out_ld, const void* wait_flags,
                                     const unsigned* counters, unsigned long long timeout_ns, int wait_channel, int world,
                                     unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(!wait_flags || (counters && world >= 1 && world <= 32), "rs_interaction_forward_ex: bad flag arguments");
  rs::FlagWait w;
  memset(&w, 0, sizeof(w));
  w.my_flags = reinterpret_cast<const uint32_t*>(wait_flags); w.sig_counters = counters; w.timeout_ns = timeout_ns;
  w.status = status; w.world = world; w.channel = wait_channel;
  return interaction_forward_impl(T, B, F, D, out, out_ld, w, stream);
}
namespace {
int interaction_forward_impl(const void* T, int B, int F, int D, void* out, int out_ld, const rs::FlagWait& wait, cudaStream_t stream) {
  RS_REQUIRE(T && out, "rs_interaction_forward: null argument");
  RS_REQUIRE(F >= 1 && F <= kMaxF && D % 16 == 0 && D >= 16 && D <= kMaxD, "rs_interaction_forward: F=%d D=%d unsupported", F, D);
  RS_REQUIRE(out_ld % 8 == 0 && out_ld >= D + F * (F - 1) / 2, "rs_interaction_forward: out_ld=%d too small or unaligned", out_ld);
  if (B == 0) return RS_OK;
  int grid = (B + kWarps - 1) / kWarps;
  if (grid > 148 * 5) grid = 148 * 5;   // persistent: 5 CTAs of 4 warps fit one SM's shared memory
  interaction_fwd_kernel<<<grid, kWarps * 32, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(T), B, F, D, reinterpret_cast<__nv_bfloat16*>(out), out_ld, wait);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
}  // namespace

RS_API int rs_interaction_backward(const void* T, const void* dout, int B, int F, int D, int dout_ld, void* dx,
                                   int dx_ld, void* const* gdst, const int* owner, const int* gcol,
                                   long long grow_stride, long long sample_base, int relu_mask_dx,
                                   void* const* ndst, int nstride, int rows, cudaStream_t stream) {
  RS_REQUIRE(T && dout && dx && gdst && owner && gcol, "rs_interaction_backward: null argument");
  RS_REQUIRE(rows >= 0 && rows <= 2, "rs_interaction_backward: rows must be 0 (all), 1 (feature 0) or 2 (embedding rows)");
  RS_REQUIRE(F >= 1 && F <= kMaxF && D % 16 == 0 && D >= 16 && D <= kMaxD, "rs_interaction_backward: F=%d D=%d unsupported", F, D);
  if (B == 0) return RS_OK;
  InterBwdArgs a;
  a.T = reinterpret_cast<const __nv_bfloat16*>(T);
  a.dout = reinterpret_cast<const __nv_bfloat16*>(dout);
  a.B = B; a.F = F; a.D = D; a.dout_ld = dout_ld;
  a.dx = reinterpret_cast<__nv_bfloat16*>(dx); a.dx_ld = dx_ld;
  a.gdst = gdst; a.owner = owner; a.gcol = gcol; a.grow_stride = grow_stride; a.sample_base = sample_base;
  a.relu_mask_dx = relu_mask_dx;
  a.ndst = reinterpret_cast<float* const*>(ndst); a.nstride = nstride; a.rows = rows;
  RS_REQUIRE(dout_ld % 8 == 0 && dout_ld <= kDoutMax, "rs_interaction_backward: dout_ld=%d must be a multiple of 8, <= %d", dout_ld, kDoutMax);
  const size_t smem = static_cast<size_t>(kWarpsBwd) * kBwdWarpBytes;
  static bool attr_done = false;
  if (!attr_done) {
    RS_CUDA(cudaFuncSetAttribute(interaction_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attr_done = true;
  }
  int grid = (B + kWarpsBwd - 1) / kWarpsBwd;
  if (grid > 148 * 4) grid = 148 * 4;   // persistent: warps loop over the samples
  interaction_bwd_kernel<<<grid, kWarpsBwd * 32, smem, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
