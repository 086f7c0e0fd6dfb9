// bf16 GEMM for sm_100a: tcgen05.mma with the accumulator in TMEM, operands staged in
// shared memory by TMA (per-CTA loads only), persistent warp-specialised CTAs.
//
// It replaces the cuBLAS calls behind nn.Linear forward / dgrad / wgrad of the
// reference's MLP stacks (src/executable/dlrm/dlrm_model.py:72-110,
// model_zoo/dlrm.py:132-141, 407-425) and the two skinny GEMMs of the low-rank
// DCNv2 cross layer (model_zoo/dlrm.py:261-286).
//
// Two operand layouts:
//   mode 0 ("TN"):  D[M,N] = A[M,K] . B[N,K]^T   A and B row-major, K contiguous
//                   (forward: A = activations, B = W;  dgrad: A = dY, B = W^T)
//   mode 1 ("NT"):  D[M,N] = A[K,M]^T . B[K,N]   A and B row-major, reduction over rows
//                   (wgrad: A = dY[batch,N_out], B = X[batch,K_in]); split over the
//                   reduction with fp32 atomic accumulation into D.
//   mode 2 ("NN"):  D[M,N] = A[M,K]   . B[K,N]   A K-major as in mode 0, B row-major [K,N] as in
//                   mode 1 (e.g. W[bs, negs] . Neg[negs, dim] in the KG gradient)
// Epilogues (fused into the TMEM read-back):
//   0  D = acc (+ bias[n])                       bf16 store
//   1  D = relu(acc + bias[n])                   bf16 store
//   2  D = acc * (aux[m,n] > 0)                  bf16 store (ReLU backward)
//   3  D += acc                                  fp32 atomic add (split reduction)
//   4  D = acc (+ bias[n])                       fp32 store
//   5  D = x0[m,n] * (acc + bias[n]) + aux[m,n]  bf16 store (DCNv2 cross update)
//   6  D = acc + aux[m,n]                        bf16 store (residual add)
//
// CTA = 10 warps: warp 0 issues TMA loads, warp 1 owns TMEM and issues the MMAs,
// warps 2..9 read the accumulator back: two groups of four warps (one warp per TMEM
// lane quadrant in each group) take alternate 64-column chunks of a tile, convert
// them in registers, stage them in 128-byte-swizzled shared memory and hand them to
// a TMA store, so no thread issues global stores for the bf16 epilogues.  Two
// accumulators are kept in TMEM so that the epilogue of tile i overlaps the main
// loop of tile i+1.  Every mbarrier wait is bounded; on give-up the kernel sets
// RS_DEV_WAIT_TIMEOUT in the status word, frees TMEM and returns.
#include <cuda_bf16.h>
#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include "common/ptx.cuh"
#include "common/rs_common.h"

namespace {
using namespace rs::ptx;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kEpiWarps = 8;               // two warps per TMEM lane quadrant: one scheduler alone cannot hide the epilogue's latencies
constexpr int kThreads = 64 + kEpiWarps * 32;
constexpr uint32_t kABytes = BM * BK * 2;  // 16 KiB per stage
constexpr uint32_t kTmemCols = 512;
constexpr int kEpiGroups = kEpiWarps / 4;
constexpr uint32_t kChunkBytes = BM * 128;               // staging of one 128-row x 64-column bf16 chunk (one TMA store box)
constexpr uint32_t kBiasBytes = 256 * 4;                 // bias slice of one tile
constexpr uint32_t kStageBytes = kEpiGroups * (kChunkBytes + kBiasBytes);
constexpr uint32_t kWarpStage = kStageBytes / kEpiWarps;   // ReLU-backward epilogue: 32 rows x 128 B + 64 bias values per warp
static_assert(kWarpStage >= 4096 + 256 && kWarpStage % 16 == 0, "per-warp staging slice");

struct GemmArgs {
  int M, N, K;          // logical problem (see modes above); K = reduction length
  int bn;               // tile width in N (multiple of 32, <= 256)
  int stages;
  int tiles_m, tiles_n;
  int splits;           // reduction splits (mode 1 / epilogue 3), else 1
  int units_per_cta;    // > 0: balanced decomposition of epilogue 3 (see WorkIter), else 0
  int kblocks;          // ceil(K / 64)
  int epi;
  int ldd, ldaux, ldx0;
  void* D;
  const float* bias;
  const __nv_bfloat16* aux;
  const __nv_bfloat16* x0;
  int tma_out;          // bf16 epilogue through shared memory and a TMA store (tile width multiple of 64)
  unsigned long long* status;
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Work of one CTA as a sequence of (tile, k-block range) segments; the three roles of a CTA walk identical copies.
//   units_per_cta == 0: items (tile, split) handed out round-robin (it = cta, cta + grid, ...)
//   units_per_cta  > 0: the tiles x k-blocks units are cut into equal contiguous ranges, one per CTA, so every CTA
//                       does the same number of k-blocks whatever tiles x splits would have divided the SMs into;
//                       a range that crosses a tile boundary yields two segments (fp32 atomic epilogue only).
struct WorkIter {
  int cur_tile, cur_split, splits, stride, tiles, kb_per_split, kblocks;
  long long u, uend;
  bool balanced;
  __device__ WorkIter(const GemmArgs& g, int cta, int grid) {
    tiles = g.tiles_m * g.tiles_n;
    kblocks = g.kblocks;
    balanced = g.units_per_cta > 0;
    stride = grid; splits = g.splits;
    cur_tile = cta % tiles; cur_split = cta / tiles;       // the only divisions: next() is on the MMA thread's path
    kb_per_split = (g.kblocks + g.splits - 1) / g.splits;
    u = static_cast<long long>(cta) * g.units_per_cta;
    uend = u + g.units_per_cta;
    const long long total = static_cast<long long>(tiles) * kblocks;
    if (uend > total) uend = total;
  }
  __device__ bool next(int& tile, int& kb0, int& kb1) {
    if (!balanced) {
      if (cur_split >= splits) return false;
      tile = cur_tile;
      kb0 = cur_split * kb_per_split;
      kb1 = min(kblocks, kb0 + kb_per_split);
      cur_tile += stride;                                   // item index advances by the grid size
      while (cur_tile >= tiles) { cur_tile -= tiles; ++cur_split; }
      return true;
    }
    if (u >= uend) return false;
    tile = static_cast<int>(u / kblocks);
    kb0 = static_cast<int>(u % kblocks);
    const long long room = uend - u;
    kb1 = static_cast<int>(min(static_cast<long long>(kblocks), kb0 + room));
    u += kb1 - kb0;
    return true;
  }
};

// CG = 1: one CTA per 128 x bn tile.  CG = 2: a pair of CTAs (cluster of 2) per 256 x bn tile: CTA `rank` holds
// rows [rank * 128, +128) of A and rows [rank * bn / 2, + bn / 2) of B, the leader (rank 0) issues cta_group::2 MMAs
// that read both CTAs' shared memory, and each CTA reads back its own 128 accumulator rows.  The pair halves the
// B-operand traffic per CTA (48 KB -> 32 KB per k-block), which is what bounds the single-CTA main loop.
template <int MODE, int CG>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ CUtensorMap tma_d, const GemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw;   // the kernel has no static shared memory: the dynamic window starts 1024-byte aligned (checked below)
  const int stages = g.stages;
  const uint32_t rank = CG == 2 ? cluster_ctarank() : 0u;
  const bool leader_cta = rank == 0;
  const int bn_cta = g.bn / CG;                          // rows of the B tile this CTA loads
  const uint32_t b_bytes = static_cast<uint32_t>(bn_cta) * BK * 2;
  const int cta_id = blockIdx.x / CG, n_ctas = gridDim.x / CG;   // work is handed out per CTA (CG = 1) or per pair
  uint8_t* sA = smem;
  uint8_t* sB = smem + static_cast<size_t>(stages) * kABytes;
  uint8_t* sStage = sB + static_cast<size_t>(stages) * b_bytes;   // per epilogue group: one chunk; then the bias slices
  uint64_t* full = reinterpret_cast<uint64_t*>(sStage + kStageBytes);
  uint64_t* empty = full + stages;
  uint64_t* tfull = empty + stages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if ((smem_u32(smem_raw) & 1023u) != 0u) {   // swizzled TMA tiles need 1024-byte aligned bases
    if (threadIdx.x == 0 && g.status) atomicOr(g.status, (unsigned long long)RS_DEV_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], kEpiWarps * 32 * CG);   // the leader's barrier collects both CTAs' epilogue threads
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (g.tma_out) tma_prefetch_desc(&tma_d);
  }
  if (warp == 1) {
    if (CG == 2) { tmem_alloc_pair(tmem_slot, kTmemCols); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (CG == 2) cluster_sync_all();   // the peer's barriers are initialised before anything is signalled across CTAs
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above (barriers, TMEM, descriptor prefetch) touched no tensor: with a programmatic dependent launch it
  // ran while the previous kernel on the stream was still draining.  From here on its results are needed.
  pdl_launch_dependents();
  pdl_wait();
  // Releasing an accumulator: an arrival on the leader's tempty barrier (local for CG = 1).
  auto release_acc = [&](int a) {
    if (CG == 2) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty[a]), 0));
    else mbar_arrive(&tempty[a]);
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int last_stage = -1;
      uint32_t last_phase = 0;
      WorkIter w(g, cta_id, n_ctas);
      int tile, kb0, kb1;
      while (ok && w.next(tile, kb0, kb1)) {
        const int m0 = (tile / g.tiles_n) * (BM * CG) + static_cast<int>(rank) * BM;
        const int n0 = (tile % g.tiles_n) * g.bn + static_cast<int>(rank) * bn_cta;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* a_dst = sA + static_cast<size_t>(stage) * kABytes;
          uint8_t* b_dst = sB + static_cast<size_t>(stage) * b_bytes;
          if (CG == 1) {
            mbar_expect_tx(&full[stage], kABytes + b_bytes);
            if (MODE != 1) {
              tma_load_2d(a_dst, &tma_a, &full[stage], kb * BK, m0);
            } else {
              for (int h = 0; h < BM / 64; ++h) tma_load_2d(a_dst + h * 8192, &tma_a, &full[stage], m0 + h * 64, kb * BK);
            }
            if (MODE == 0) {
              tma_load_2d(b_dst, &tma_b, &full[stage], kb * BK, n0);
            } else {
              for (int h = 0; h < bn_cta / 64; ++h) tma_load_2d(b_dst + h * 8192, &tma_b, &full[stage], n0 + h * 64, kb * BK);
            }
          } else {
            // Both CTAs' copies are counted on the leader's barrier; only the leader announces the bytes (of both).
            if (leader_cta) mbar_expect_tx(&full[stage], 2u * (kABytes + b_bytes));
            const uint32_t bar = mapa_shared(smem_u32(&full[stage]), 0);
            if (MODE != 1) {
              tma_load_2d_pair(a_dst, &tma_a, bar, kb * BK, m0);
            } else {
              for (int h = 0; h < BM / 64; ++h) tma_load_2d_pair(a_dst + h * 8192, &tma_a, bar, m0 + h * 64, kb * BK);
            }
            if (MODE == 0) {
              tma_load_2d_pair(b_dst, &tma_b, bar, kb * BK, n0);
            } else {
              for (int h = 0; h < bn_cta / 64; ++h) tma_load_2d_pair(b_dst + h * 8192, &tma_b, bar, n0 + h * 64, kb * BK);
            }
          }
          last_stage = stage;
          last_phase = phase;
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && last_stage >= 0) {
        // Leaving early: let the copies already in flight land before the CTA's shared memory goes away.  (The peer
        // of a pair cannot see the leader's barrier complete; it just gives its copies time.)
        if (CG == 1 || leader_cta) mbar_wait(&full[last_stage], last_phase, nullptr, 1u << 16);
        else for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader_cta) {
      const uint32_t idesc = make_idesc_bf16(BM * CG, static_cast<uint32_t>(g.bn), MODE == 1 ? 1u : 0u, MODE != 0 ? 1u : 0u);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      WorkIter w(g, cta_id, n_ctas);
      int tile, kb0, kb1;
      while (ok && w.next(tile, kb0, kb1)) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * g.bn);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + static_cast<size_t>(stage) * kABytes);
          const uint32_t b_addr = smem_u32(sB + static_cast<size_t>(stage) * b_bytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            uint64_t ad, bd;
            // K-major, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart; a K step of 16
            // elements moves the start address by 32 B inside the swizzled row.
            // MN-major, 128-byte swizzle: each TMA box holds 64 reduction rows x 64 columns; 8-row
            // groups are 1024 B apart (SBO), the next 64 columns start one box (8 KiB) later (LBO).
            if (MODE != 1) ad = make_smem_desc(a_addr + k * 32, 16, 1024, 2);
            else ad = make_smem_desc(a_addr + k * 2048, 8192, 1024, 2);
            if (MODE == 0) bd = make_smem_desc(b_addr + k * 32, 16, 1024, 2);
            else bd = make_smem_desc(b_addr + k * 2048, 8192, 1024, 2);
            if (CG == 2) umma_f16_pair(tmem_d, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else umma_f16(tmem_d, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          if (CG == 2) umma_commit_pair(&empty[stage], 3);   // frees the stage in both CTAs
          else umma_commit(&empty[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (CG == 2) umma_commit_pair(&tfull[acc], 3);     // each CTA's epilogue waits on its own barrier
        else umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    const int q = warp & 3;            // TMEM lane quadrant this warp may read
    const int part = (warp - 2) >> 2;  // epilogue group of this warp
    constexpr int kParts = kEpiGroups;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    if (g.tma_out && g.epi != 2) {
      uint8_t* so = sStage + part * kChunkBytes;
      float* sbias = reinterpret_cast<float*>(sStage + kEpiGroups * kChunkBytes + part * kBiasBytes);
      const int gtid = ((warp - 2) & 3) * 32 + lane;   // 0..127 inside the group
      const bool leader = gtid == 0;
      const uint32_t bar_id = 1u + static_cast<uint32_t>(part);
      const int srow = q * 32 + lane;                  // row of the tile (= TMEM lane) this thread converts
      uint8_t* srow_ptr = so + srow * 128;
      const uint32_t sw = static_cast<uint32_t>(srow & 7);
      const __nv_bfloat162 zero2 = __floats2bfloat162_rn(0.f, 0.f);
      const int nchunks = g.bn / 64;
      WorkIter w(g, cta_id, n_ctas);
      int tile, kb0, kb1;
      while (w.next(tile, kb0, kb1)) {
        const int m0 = (tile / g.tiles_n) * (BM * CG) + static_cast<int>(rank) * BM;
        const int n0 = (tile % g.tiles_n) * g.bn;
        // The tile's bias slice is requested before the accumulator is ready, so its latency hides behind the wait.
        float2 bv = make_float2(0.f, 0.f);
        if (g.bias != nullptr && n0 + gtid * 2 < g.N && gtid * 2 < g.bn) bv = __ldg(reinterpret_cast<const float2*>(g.bias + n0) + gtid);
        const bool mine = mbar_wait(&tfull[acc], acc_phase, abort_flag);
        reinterpret_cast<float2*>(sbias)[gtid] = bv;
        // One verdict for the whole group (a thread that gave up must not leave the others at a barrier); the same
        // barrier publishes the bias slice.
        ok = bar_red_and(bar_id, 128, mine);
        if (!ok) break;
        tc_fence_after_sync();
        bool released = false;
        for (int c = part; c < nchunks; c += kParts) {
          const int col0 = n0 + c * 64;
          if (col0 >= g.N) break;
          uint32_t r[64];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * g.bn + c * 64);
          tmem_ld_32x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          tmem_ld_32x32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          // Operands from global memory (ReLU mask source, residual, x0) are fetched row-contiguously, four rows
          // of 128 bytes per warp instruction, while the accumulator is on its way.  They reach the thread that
          // owns the row through this warp's 32 rows of the staging buffer, in the layout a TMA load would give.
          const bool use_aux = g.epi == 2 || g.epi >= 5;
          const int lrow = lane >> 3, lchunk = lane & 7;
          uint4 ax[8], xx[8];
          if (use_aux) {
            const bool col_in = col0 + lchunk * 8 < g.N;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int grow = m0 + q * 32 + j * 4 + lrow;
              const bool in = col_in && grow < g.M;
              const size_t r_eff = in ? static_cast<size_t>(grow) : 0;
              ax[j] = __ldg(reinterpret_cast<const uint4*>(g.aux + r_eff * g.ldaux + (in ? col0 + lchunk * 8 : 0)));
              if (g.epi == 5) xx[j] = __ldg(reinterpret_cast<const uint4*>(g.x0 + r_eff * g.ldx0 + (in ? col0 + lchunk * 8 : 0)));
            }
          }
          if (leader) tma_store_wait_read<0>();   // the previous chunk's store has finished reading the staging
          named_bar_sync(bar_id, 128);
          if (use_aux) {
            uint8_t* wbase = so + (q * 32) * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int rr = j * 4 + lrow;
              *reinterpret_cast<uint4*>(wbase + rr * 128 + ((static_cast<uint32_t>(lchunk) ^ (rr & 7)) << 4)) = ax[j];
            }
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j) ax[j] = *reinterpret_cast<const uint4*>(srow_ptr + ((static_cast<uint32_t>(j) ^ sw) << 4));
            if (g.epi == 5) {   // second operand: same route, after the first has been read back
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int rr = j * 4 + lrow;
                *reinterpret_cast<uint4*>(wbase + rr * 128 + ((static_cast<uint32_t>(lchunk) ^ (rr & 7)) << 4)) = xx[j];
              }
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 8; ++j) xx[j] = *reinterpret_cast<const uint4*>(srow_ptr + ((static_cast<uint32_t>(j) ^ sw) << 4));
            }
            __syncwarp();   // every lane has its row before anyone overwrites the staging with results
          }
          tmem_ld_wait();
          if (c + kParts >= nchunks || col0 + kParts * 64 >= g.N) {   // last chunk of this thread in the tile
            tc_fence_before_sync();
            release_acc(acc);
            released = true;
          }
          uint32_t pk[32];
          const float* sb = sbias + c * 64;
#pragma unroll
          for (int j = 0; j < 64; j += 4) {
            float v0 = __uint_as_float(r[j]), v1 = __uint_as_float(r[j + 1]);
            float v2 = __uint_as_float(r[j + 2]), v3 = __uint_as_float(r[j + 3]);
            if (g.bias != nullptr) {
              const float4 b = *reinterpret_cast<const float4*>(sb + j);   // same address in every lane: broadcast
              v0 += b.x; v1 += b.y; v2 += b.z; v3 += b.w;
            }
            if (g.epi >= 5) {
              const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ax[j >> 3]) + ((j & 4) >> 1);
              const float2 a0 = __bfloat1622float2(pa[0]), a1 = __bfloat1622float2(pa[1]);
              if (g.epi == 5) {
                const __nv_bfloat162* px = reinterpret_cast<const __nv_bfloat162*>(&xx[j >> 3]) + ((j & 4) >> 1);
                const float2 x0v = __bfloat1622float2(px[0]), x1v = __bfloat1622float2(px[1]);
                v0 = x0v.x * v0 + a0.x; v1 = x0v.y * v1 + a0.y;
                v2 = x1v.x * v2 + a1.x; v3 = x1v.y * v3 + a1.y;
              } else {
                v0 += a0.x; v1 += a0.y; v2 += a1.x; v3 += a1.y;
              }
            }
            __nv_bfloat162 p0 = __floats2bfloat162_rn(v0, v1), p1 = __floats2bfloat162_rn(v2, v3);
            if (g.epi == 1) {          // max commutes with the rounding, so ReLU runs on packed pairs
              p0 = __hmax2(p0, zero2);
              p1 = __hmax2(p1, zero2);
            } else if (g.epi == 2) {   // ReLU backward: multiply by (forward activation > 0) as 1.0 / 0.0
              const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ax[j >> 3]) + ((j & 4) >> 1);
              p0 = __hmul2(p0, __hgt2(pa[0], zero2));
              p1 = __hmul2(p1, __hgt2(pa[1], zero2));
            }
            pk[j >> 1] = *reinterpret_cast<uint32_t*>(&p0);
            pk[(j >> 1) + 1] = *reinterpret_cast<uint32_t*>(&p1);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(srow_ptr + ((static_cast<uint32_t>(j) ^ sw) << 4)) =
                make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
          fence_proxy_async_smem();
          named_bar_sync(bar_id, 128);
          if (leader) {
            tma_store_2d(&tma_d, so, col0, m0);   // rows >= M and columns >= N are clipped by the tensor map
            tma_store_commit();
          }
        }
        if (!released) {
          tc_fence_before_sync();
          release_acc(acc);
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (leader) tma_store_wait<0>();   // shared memory must outlive the stores that read it
    } else {
    WorkIter w(g, cta_id, n_ctas);
    int tile, kb0, kb1;
    while (ok && w.next(tile, kb0, kb1)) {
      const int m0 = (tile / g.tiles_n) * (BM * CG) + static_cast<int>(rank) * BM;
      const int n0 = (tile % g.tiles_n) * g.bn;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < g.M;
      if (g.epi == 2 && (g.bn & 63) == 0) {
        // bf16 output staged through shared memory: every thread owns one row of the accumulator, but
        // global memory is touched row-contiguously (4 rows x 128 B per warp instruction) for both the
        // output store and the ReLU-mask load.  16-byte chunks are XOR-swizzled by (row & 7).
        uint8_t* so = sStage + (warp - 2) * kWarpStage;   // per-warp slices of the same staging region
        float* sbias = reinterpret_cast<float*>(so + 4096);
        const int lrow = lane >> 3, lchunk = lane & 7;
        for (int c = part; c < g.bn / 64; c += kParts) {
          const int col0 = n0 + c * 64;
          if (col0 >= g.N) break;
          // Both 32-column halves of the accumulator are requested first; the global loads this group
          // needs (bias, ReLU mask) are issued while they are in flight.
          uint32_t r0[32], r1[32];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * g.bn + c * 64);
          tmem_ld_32x32(taddr, r0);
          tmem_ld_32x32(taddr + 32, r1);
          float2 bv = make_float2(0.f, 0.f);
          if (g.bias != nullptr && col0 + lane * 2 < g.N) bv = __ldg(reinterpret_cast<const float2*>(g.bias + col0) + lane);
          const bool col_ok = col0 + lchunk * 8 < g.N;
          uint4 m[8];   // ReLU mask source, row-contiguous like the store phase: rows it*4+lrow, 16-byte chunk lchunk
          if (g.epi == 2) {
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int grow = m0 + q * 32 + it * 4 + lrow;
              m[it] = make_uint4(0, 0, 0, 0);
              if (grow < g.M && col_ok)
                m[it] = __ldg(reinterpret_cast<const uint4*>(g.aux + static_cast<size_t>(grow) * g.ldaux + col0) + lchunk);
            }
          }
          reinterpret_cast<float2*>(sbias)[lane] = bv;
          __syncwarp();
          tmem_ld_wait();
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(half == 0 ? r0[j] : r1[j]);
            if (g.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const float4 b = *reinterpret_cast<const float4*>(sbias + half * 32 + j);   // same address in every lane: broadcast
                v[j] += b.x; v[j + 1] += b.y; v[j + 2] += b.z; v[j + 3] += b.w;
              }
            }
            if (g.epi == 1) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
            }
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int chunk = half * 4 + (j >> 3);
              uint4 o;
              o.x = pack_bf16(v[j], v[j + 1]);
              o.y = pack_bf16(v[j + 2], v[j + 3]);
              o.z = pack_bf16(v[j + 4], v[j + 5]);
              o.w = pack_bf16(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(so + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = o;
            }
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + lrow;
            const int grow = m0 + q * 32 + r;
            uint4 o = *reinterpret_cast<const uint4*>(so + r * 128 + ((lchunk ^ (r & 7)) << 4));
            if (g.epi == 2) {   // ReLU backward: zero where the forward activation was not positive
              __nv_bfloat162* oe = reinterpret_cast<__nv_bfloat162*>(&o);
              const __nv_bfloat162* me = reinterpret_cast<const __nv_bfloat162*>(&m[it]);
              const __nv_bfloat162 z2 = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
              for (int e = 0; e < 4; ++e) oe[e] = __hmul2(oe[e], __hgt2(me[e], z2));   // (activation > 0) as 1.0 / 0.0
            }
            if (grow < g.M && col_ok) {
              *(reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(g.D) + static_cast<size_t>(grow) * g.ldd + col0) + lchunk) = o;
            }
          }
          __syncwarp();
        }
        tc_fence_before_sync();
        release_acc(acc);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
        continue;
      }
      for (int c = part; c < g.bn / 32; c += kParts) {
        const int col0 = n0 + c * 32;
        if (col0 >= g.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * g.bn + c * 32), r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (g.epi == 3) {
          if (row_ok) {
            float* d = reinterpret_cast<float*>(g.D) + static_cast<size_t>(row) * g.ldd + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col0 + j < g.N) atomicAdd(reinterpret_cast<float4*>(d + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
            }
          }
          continue;
        }
        if (g.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (col0 + j < g.N) {
              const float4 b = __ldg(reinterpret_cast<const float4*>(g.bias + col0 + j));
              v[j] += b.x; v[j + 1] += b.y; v[j + 2] += b.z; v[j + 3] += b.w;
            }
          }
        }
        if (g.epi == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
        } else if (g.epi == 2 && row_ok) {
          const __nv_bfloat16* a = g.aux + static_cast<size_t>(row) * g.ldaux + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j < g.N) {
              const uint4 m = __ldg(reinterpret_cast<const uint4*>(a + j));
              const __nv_bfloat16* mb = reinterpret_cast<const __nv_bfloat16*>(&m);
#pragma unroll
              for (int t = 0; t < 8; ++t) v[j + t] = (__bfloat162float(mb[t]) > 0.f) ? v[j + t] : 0.f;
            }
          }
        } else if (g.epi == 6 && row_ok) {
          const __nv_bfloat16* a = g.aux + static_cast<size_t>(row) * g.ldaux + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j < g.N) {
              const uint4 ma = __ldg(reinterpret_cast<const uint4*>(a + j));
              const __nv_bfloat16* pa = reinterpret_cast<const __nv_bfloat16*>(&ma);
#pragma unroll
              for (int t = 0; t < 8; ++t) v[j + t] += __bfloat162float(pa[t]);
            }
          }
        } else if (g.epi == 5 && row_ok) {
          const __nv_bfloat16* a = g.aux + static_cast<size_t>(row) * g.ldaux + col0;
          const __nv_bfloat16* x = g.x0 + static_cast<size_t>(row) * g.ldx0 + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j < g.N) {
              const uint4 ma = __ldg(reinterpret_cast<const uint4*>(a + j));
              const uint4 mx = __ldg(reinterpret_cast<const uint4*>(x + j));
              const __nv_bfloat16* pa = reinterpret_cast<const __nv_bfloat16*>(&ma);
              const __nv_bfloat16* px = reinterpret_cast<const __nv_bfloat16*>(&mx);
#pragma unroll
              for (int t = 0; t < 8; ++t) v[j + t] = __bfloat162float(px[t]) * v[j + t] + __bfloat162float(pa[t]);
            }
          }
        }
        if (row_ok) {
          if (g.epi == 4) {
            float* d = reinterpret_cast<float*>(g.D) + static_cast<size_t>(row) * g.ldd + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              if (col0 + j < g.N) *reinterpret_cast<float4*>(d + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
            __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(g.D) + static_cast<size_t>(row) * g.ldd + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < g.N) {
                uint4 o;
                o.x = pack_bf16(v[j], v[j + 1]);
                o.y = pack_bf16(v[j + 2], v[j + 3]);
                o.z = pack_bf16(v[j + 4], v[j + 5]);
                o.w = pack_bf16(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(d + j) = o;
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      release_acc(acc);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (CG == 2) cluster_sync_all();   // the leader's MMAs read the peer's shared memory until the very end
  if (warp == 1) {
    tc_fence_after_sync();
    if (CG == 2) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && g.status) atomicOr(g.status, (unsigned long long)RS_DEV_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct MapKey {
  const void* p; uint64_t rows, cols, ld; uint32_t box_r, box_c;
  bool operator==(const MapKey& o) const {
    return p == o.p && rows == o.rows && cols == o.cols && ld == o.ld && box_r == o.box_r && box_c == o.box_c;
  }
};
struct MapHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.p);
    h = h * 1000003u ^ k.rows; h = h * 1000003u ^ k.cols; h = h * 1000003u ^ k.ld;
    h = h * 1000003u ^ k.box_r; h = h * 1000003u ^ k.box_c;
    return h;
  }
};

// 2-D bf16 row-major tensor [rows, cols] with leading dimension ld (elements); box = box_r x box_c,
// 128-byte swizzle, zero fill outside the tensor.
int make_map_bf16(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_r,
                  uint32_t box_c) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
  MapKey key{ptr, rows, cols, ld, box_r, box_c};
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return RS_OK; }
  }
  EncodeTiledFn enc = get_encode();
  if (!enc) return rs::set_error(RS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * 2) & 15))
    return rs::set_error(RS_ERR_INVALID, "TMA operand must be 16-byte aligned with a 16-byte multiple row pitch");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_c, box_r};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return rs::set_error(RS_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  std::lock_guard<std::mutex> lk(mu);
  if (cache.size() > 4096) cache.clear();
  cache[key] = *out;
  return RS_OK;
}

int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}
}  // namespace

// D = epilogue(A x B) as described at the top of the file.  All leading dimensions in elements.
// bn / splits: 0 selects automatically.  `status` is a device word that receives RsDevErr bits.
RS_API int rs_gemm_bf16(const void* A, const void* B, void* D, const float* bias, const void* aux, const void* x0,
                        int M, int N, int K, int lda, int ldb, int ldd, int ldaux, int ldx0, int mode, int epi,
                        int bn, int splits, unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(A && B && D, "rs_gemm_bf16: null operand");
  RS_REQUIRE(M > 0 && N > 0 && K > 0, "rs_gemm_bf16: empty problem %d %d %d", M, N, K);
  RS_REQUIRE(mode >= 0 && mode <= 2, "rs_gemm_bf16: mode must be 0, 1 or 2");
  RS_REQUIRE(epi >= 0 && epi <= 6, "rs_gemm_bf16: unknown epilogue %d", epi);
  RS_REQUIRE(N % 8 == 0, "rs_gemm_bf16: N (%d) must be a multiple of 8", N);
  RS_REQUIRE(mode != 1 || M % 8 == 0, "rs_gemm_bf16: mode 1 needs M to be a multiple of 8");
  RS_REQUIRE((epi != 2 && epi != 6) || aux, "rs_gemm_bf16: epilogues 2 and 6 need aux");
  RS_REQUIRE(epi != 5 || (aux && x0), "rs_gemm_bf16: epilogue 5 needs aux and x0");
  const bool f32_out = (epi == 3 || epi == 4);
  RS_REQUIRE((ldd * (f32_out ? 4 : 2)) % 16 == 0 && (reinterpret_cast<uintptr_t>(D) & 15) == 0,
             "rs_gemm_bf16: D must be 16-byte aligned with a 16-byte multiple pitch");
  static const bool pairs_allowed = [] {                 // RECSTORE_GEMM_CTA_PAIRS=0 keeps every GEMM on single CTAs
    const char* e = getenv("RECSTORE_GEMM_CTA_PAIRS");
    return !(e && e[0] == '0');
  }();
  const bool pairs_possible = pairs_allowed && M >= 2 * BM && num_sms() % 2 == 0;
  int cg = 0;
  if (bn == 0) {
    // Tile width and CTA pairing are chosen together.  A large problem takes the largest tile (best operand reuse);
    // a problem with fewer tiles than SMs takes a smaller one so that the machine is filled (M = 8192, N = 256 as
    // 256-wide pair tiles would occupy 64 of 148 SMs).  Estimated time = waves x tile width x a reuse penalty.
    double best = 0.0;
    int cand[4], nc = 0;
    for (int w = 256; w >= 64; w >>= 1)
      if (N % w == 0) cand[nc++] = w;                                  // whole tiles only
    if (mode == 0 && N % 32 == 0 && N % 64 != 0) cand[nc++] = 32;
    for (int ci = 0; ci < nc; ++ci) {
      const int w = cand[ci];
      for (int c = 2; c >= 1; --c) {
        if (c == 2 && (!pairs_possible || w % 128 != 0)) continue;
        const long long tiles = static_cast<long long>((M + BM * c - 1) / (BM * c)) * (N / w);
        const long long units = num_sms() / c;
        const double penalty = (c == 2 ? 0.9 : 1.0) * (w == 256 ? 1.0 : w == 128 ? 1.15 : w == 64 ? 1.4 : 1.8);
        // The split-reduction GEMM (weight gradients) fills the machine with splits whatever the tile: largest tile wins.
        const double est = epi == 3 ? penalty : static_cast<double>((tiles + units - 1) / units) * w * penalty;
        if (cg == 0 || est < best) { best = est; bn = w; cg = c; }
      }
    }
    if (cg == 0) { bn = 64; cg = 1; }                                    // ragged N: 64-wide tiles, the last one partial
  }
  RS_REQUIRE(bn % 32 == 0 && bn <= 256 && bn >= 32, "rs_gemm_bf16: bad tile width %d", bn);
  RS_REQUIRE(mode == 0 || bn % 64 == 0, "rs_gemm_bf16: modes 1 and 2 need a tile width multiple of 64");
  // CTA pairs (cta_group::2) need at least one 256-row tile and a B tile that splits into two 64-column-aligned halves.
  if (cg == 0) cg = (pairs_possible && bn % 128 == 0) ? 2 : 1;
  GemmArgs g;
  g.M = M; g.N = N; g.K = K; g.bn = bn;
  g.tiles_m = (M + BM * cg - 1) / (BM * cg);
  g.tiles_n = (N + bn - 1) / bn;
  g.kblocks = (K + BK - 1) / BK;
  const int sms = num_sms() / cg;   // schedulable units: CTAs or CTA pairs
  g.units_per_cta = 0;
  int grid_override = 0;
  if (epi == 3) {
    const int tiles = g.tiles_m * g.tiles_n;
    if (splits < 0) {
      // On request: cut tiles x k-blocks into one equal contiguous range per SM.  Perfectly balanced, but CTAs that
      // run together then read different reduction rows and nothing is shared through L2: measured 253 us against
      // 166 us for the 1024 x 1024 x 65536 weight gradient, so it is not the default.
      const long long total = static_cast<long long>(tiles) * g.kblocks;
      const int ctas = static_cast<int>(total < sms ? total : sms);
      g.units_per_cta = static_cast<int>((total + ctas - 1) / ctas);
      grid_override = static_cast<int>((total + g.units_per_cta - 1) / g.units_per_cta);
      splits = 1;
    } else if (splits == 0) {
      // One wave: as many splits as fit on the SMs (rounding up instead gives e.g. 160 items on 148 SMs, which take
      // the time of two waves).  Items of one split run together and share their reduction rows through L2.
      splits = tiles >= sms ? 1 : sms / tiles;
      if (splits > g.kblocks) splits = g.kblocks;
      if (splits < 1) splits = 1;
    }
  } else {
    splits = 1;
  }
  // Make every split non-empty.
  {
    const int per = (g.kblocks + splits - 1) / splits;
    splits = (g.kblocks + per - 1) / per;
  }
  g.splits = splits;
  const uint32_t stage_bytes = kABytes + static_cast<uint32_t>(bn / cg) * BK * 2;
  int stages = static_cast<int>((227u * 1024u - kStageBytes - 256u) / stage_bytes);
  if (stages > 8) stages = 8;
  if (stages < 2) stages = 2;
  g.stages = stages;
  g.epi = epi; g.ldd = ldd; g.ldaux = ldaux; g.ldx0 = ldx0;
  g.D = D; g.bias = bias;
  g.aux = reinterpret_cast<const __nv_bfloat16*>(aux);
  g.x0 = reinterpret_cast<const __nv_bfloat16*>(x0);
  g.status = status;
  g.tma_out = (!f32_out && bn % 64 == 0) ? 1 : 0;

  CUtensorMap ma, mb, md;
  int rc;
  if (mode != 1) { if ((rc = make_map_bf16(&ma, A, M, K, lda, BM, BK)) != RS_OK) return rc; }
  else { if ((rc = make_map_bf16(&ma, A, K, M, lda, BK, 64)) != RS_OK) return rc; }
  if (mode == 0) { if ((rc = make_map_bf16(&mb, B, N, K, ldb, bn / cg, BK)) != RS_OK) return rc; }
  else { if ((rc = make_map_bf16(&mb, B, K, N, ldb, BK, 64)) != RS_OK) return rc; }
  if (g.tma_out) { if ((rc = make_map_bf16(&md, D, M, N, ldd, BM, 64)) != RS_OK) return rc; }
  else md = ma;   // unused by the kernel
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + kStageBytes + 256;
  using Kern = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const GemmArgs);
  static const Kern kernels[2][3] = {{gemm_tcgen05_kernel<0, 1>, gemm_tcgen05_kernel<1, 1>, gemm_tcgen05_kernel<2, 1>},
                                     {gemm_tcgen05_kernel<0, 2>, gemm_tcgen05_kernel<1, 2>, gemm_tcgen05_kernel<2, 2>}};
  static bool attr_set[2][3] = {{false, false, false}, {false, false, false}};
  const Kern kern = kernels[cg - 1][mode];
  if (!attr_set[cg - 1][mode]) {
    RS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set[cg - 1][mode] = true;
  }
  const int items = g.tiles_m * g.tiles_n * g.splits;
  const int units = grid_override > 0 ? grid_override : (items < sms ? items : sms);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(units * cg));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // Programmatic dependent launch (RECSTORE_GEMM_PDL=0 switches it off): the prologue of this GEMM overlaps the tail
  // of the kernel before it on the stream, which matters when a step is a chain of short GEMMs.
  static const bool pdl = [] {
    const char* e = getenv("RECSTORE_GEMM_PDL");
    return !(e && e[0] == '0');
  }();
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (cg == 2) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = static_cast<unsigned>(cg);
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  RS_CUDA(cudaLaunchKernelEx(&cfg, kern, ma, mb, md, g));
  RS_LAUNCH_CHECK();
  return RS_OK;
}
