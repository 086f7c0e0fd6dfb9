// Fused embedding forward and backward for model-parallel embedding shards on sm_100a.
//
// Forward (rs_emb_forward): for every (local table, sample) bag it resolves the ids to rows of
// the shard (direct index or hash-table probe), sum-pools the rows (optional per-sample
// weights) and stores the pooled vector STRAIGHT INTO THE DESTINATION RANK'S BUFFER through a
// peer pointer: destination rank = sample / B_local, address = dst[rank] + (sample % B_local) *
// row_stride + dst_col[table].  With peer windows mapped over NVLink this is the table-wise
// all-to-all of the reference (nn.EmbeddingBag per table, src/executable/dlrm/dlrm_model.py:
// 255-314, followed by all_to_all_single, extend_distributed.py:389-426) done by the gather
// kernel itself, with no pack/unpack and no collective call.  It also replaces the plain
// gather kernels uva_cache_query / UVAQueryKernel / LookupKernel
// (src/framework/pytorch/recstore_pytorch.cu:12-37, src/storage/gpu_cache/gpu_cache_nohash.cu:
// 2-12, static_hash_table.cu:223-268).
//
// Backward (rs_emb_backward): consumes per-bag gradients (as pushed by the peers into this
// rank's gradient window), counting-sorts each 256-occurrence group by row in shared memory so
// that equal rows are adjacent, sums every run in registers and applies SGD or row-wise Adagrad in
// place with one vector atomic per run.  Semantics follow the reference optimizers
// (src/python/pytorch/recstore/DistOpt.py:511-557): state[row] += sum over occurrences of
// mean(g^2); W[row] -= lr * sum over occurrences of g / (sqrt(state[row]) + eps), with the
// state read after all occurrences of the step were accumulated (hence two passes).
//
// No kernel here traps: out-of-range ids set RS_DEV_OOB_ROW in the status word and are skipped.
#include <cuda_bf16.h>
#include <cstdlib>
#include "common/rs_common.h"
#include "comm/flags.cuh"
#include "kv/hash_table.cuh"

namespace {

struct EmbFwdArgs {
  const float* weight;
  const long long* table_base;   // [T] first row of each local table inside `weight`
  const long long* table_rows;   // [T] number of rows of each local table
  const long long* indices;      // [nnz]
  const long long* offsets;      // [T*B + 1] or null when hotness is fixed per table
  const int* hotness;            // [T] used when offsets == null
  const long long* hot_base;     // [T] start of table t's ids inside `indices` when offsets == null
  const float* psw;              // optional per-sample weights [nnz]
  int T, B, D, B_local;
  void* const* dst;              // [world] destination base pointers
  long long dst_row_stride;      // elements
  const int* dst_col;            // [T] element offset of the table's feature inside a destination row
  int out_bf16;
  long long* row_idx;            // optional [nnz]: resolved row per id (-1 if invalid)
  int* occ2bag;                  // optional [nnz]
  int use_hash;
  rs::HashTableView ht;
  unsigned long long* status;
  // Row-sharded tables (a table spread cyclically over the ranks, this rank holding ids with id % id_div == id_rem at
  // local row id / id_div): the ids of a bag arrive from the sample's rank in a fixed-capacity region of `hotness`
  // slots, of which only counts[bag] are filled.
  const int* counts;             // [T*B] or null
  int id_div, id_rem;            // 1, 0 for whole tables
  // Occurrence list for the backward pass, compacted: positions come from an atomic cursor instead of the id's index
  // (the regions above are mostly holes).  Null = write at the id's own index.
  int* occ_cursor;
  rs::FlagWait wait;             // optional: wait for the source rank's keys before reading a bag
  rs::FlagSignal sig;            // optional: publish "my pooled rows have landed" when the grid is done
};

constexpr int kMaxChunks = 4;  // D <= 512

template <int NC>
__device__ __forceinline__ void store_pooled(const EmbFwdArgs& a, int t, int b, const float4 (&acc)[NC], int lane, int nvec) {
  const int dst_rank = b / a.B_local;
  const long long off = static_cast<long long>(b - dst_rank * a.B_local) * a.dst_row_stride + a.dst_col[t];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int v = lane + c * 32;
    if (v < nvec) {
      if (a.out_bf16) {
        __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(a.dst[dst_rank]) + off;
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc[c].x, acc[c].y);
        __nv_bfloat162 hi = __floats2bfloat162_rn(acc[c].z, acc[c].w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        *(reinterpret_cast<uint2*>(d) + v) = o;
      } else {
        float* d = reinterpret_cast<float*>(a.dst[dst_rank]) + off;
        *(reinterpret_cast<float4*>(d) + v) = acc[c];
      }
    }
  }
}

// One warp per block of 32 consecutive bags of one table.  Lane i first resolves the metadata of
// bag i (id range, and for single-id bags the row itself) with coalesced loads; the rows are then
// fetched 8 bags at a time so that every warp keeps 8 independent 512-byte reads in flight.
template <int NC>
__device__ __forceinline__ void emb_fwd_body(const EmbFwdArgs& a, long long blk) {
  const int lane = threadIdx.x & 31;
  const int blocks_per_table = (a.B + 31) >> 5;
  const int t = static_cast<int>(blk / blocks_per_table);
  const int b0 = static_cast<int>(blk % blocks_per_table) << 5;
  const int nb = min(32, a.B - b0);
  const long long base = a.table_base[t];
  const long long nrows = a.table_rows[t];
  const int nvec = a.D >> 2;

  if (a.wait.my_flags != nullptr) {
    // The bags of this warp come from one source rank (two when the block of 32 straddles a boundary).
    const int s0 = b0 / a.B_local, s1 = (b0 + nb - 1) / a.B_local;
    for (int src = s0; src <= s1; ++src) rs::flag_wait_one_warp(a.wait, src);
  }
  long long beg = 0, end = 0;
  if (lane < nb) {
    const long long bag = static_cast<long long>(t) * a.B + b0 + lane;
    if (a.offsets) {
      beg = a.offsets[bag];
      end = a.offsets[bag + 1];
    } else {
      const int h = a.hotness[t];
      beg = a.hot_base[t] + static_cast<long long>(b0 + lane) * h;
      end = beg + (a.counts ? min(max(__ldcv(a.counts + bag), 0), h) : h);
    }
  }
  const bool sharded = a.id_div > 1;
  auto resolve = [&](long long id) -> long long {
    if (a.use_hash) return rs::ht_find(a.ht, static_cast<unsigned long long>(id));
    if (!sharded) {
      if (id >= 0 && id < nrows) return base + id;
    } else if (id >= 0 && id % a.id_div == a.id_rem && id / a.id_div < nrows) {
      return base + id / a.id_div;
    }
    if (a.status) atomicOr(a.status, (unsigned long long)RS_DEV_OOB_ROW);
    return -1;
  };
  const bool single = a.counts == nullptr && a.occ_cursor == nullptr && __all_sync(0xffffffffu, lane >= nb || end - beg == 1);
  if (single && a.psw == nullptr) {
    long long my_row = -1;
    if (lane < nb) {
      const long long id = a.indices[beg];
      my_row = resolve(id);
      if (a.row_idx) a.row_idx[beg] = my_row;
      if (a.occ2bag) a.occ2bag[beg] = static_cast<int>(static_cast<long long>(t) * a.B + b0 + lane);
    }
    for (int j0 = 0; j0 < nb; j0 += 8) {
      float4 x[8][NC];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const long long r = __shfl_sync(0xffffffffu, my_row, (j0 + u) & 31);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int v = lane + c * 32;
          x[u][c] = (j0 + u < nb && r >= 0 && v < nvec) ? __ldg(reinterpret_cast<const float4*>(a.weight + r * a.D) + v)
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (j0 + u < nb) store_pooled<NC>(a, t, b0 + j0 + u, x[u], lane, nvec);
    }
    return;
  }

  // General path: pooled bags (several ids, optional per-sample weights).
  for (int j = 0; j < nb; ++j) {
    const long long jb = __shfl_sync(0xffffffffu, beg, j);
    const long long je = __shfl_sync(0xffffffffu, end, j);
    const long long bag = static_cast<long long>(t) * a.B + b0 + j;
    float4 acc[NC];
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long i0 = jb; i0 < je; i0 += 32) {
      const int n = static_cast<int>(min(32ll, je - i0));
      long long my_row = -1;
      float my_w = 1.f;
      long long opos = i0;                        // where this chunk's occurrences are recorded
      if (a.occ_cursor != nullptr) {
        int p = 0;
        if (lane == 0) p = atomicAdd(a.occ_cursor, n);
        opos = __shfl_sync(0xffffffffu, p, 0);
      }
      if (lane < n) {
        const long long id = a.counts ? __ldcv(a.indices + i0 + lane) : a.indices[i0 + lane];   // pushed by a peer: not through L1
        my_row = resolve(id);
        if (a.psw) my_w = a.psw[i0 + lane];
        if (a.row_idx) a.row_idx[opos + lane] = my_row;
        if (a.occ2bag) a.occ2bag[opos + lane] = static_cast<int>(bag);
      }
      for (int k0 = 0; k0 < n; k0 += 4) {
        long long r[4];
        float w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          r[u] = __shfl_sync(0xffffffffu, my_row, (k0 + u) & 31);
          w[u] = __shfl_sync(0xffffffffu, my_w, (k0 + u) & 31);
          if (k0 + u >= n) r[u] = -1;
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int v = lane + c * 32;
          if (v < nvec) {
            float4 x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
              x[u] = r[u] >= 0 ? __ldg(reinterpret_cast<const float4*>(a.weight + r[u] * a.D) + v)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              acc[c].x += w[u] * x[u].x; acc[c].y += w[u] * x[u].y;
              acc[c].z += w[u] * x[u].z; acc[c].w += w[u] * x[u].w;
            }
          }
        }
      }
    }
    store_pooled<NC>(a, t, b0 + j, acc, lane, nvec);
  }
}

template <int NC>
__global__ void __launch_bounds__(256) emb_fwd_kernel(const EmbFwdArgs a) {
  // Warps loop over the blocks of 32 bags, so the grid can be a single resident wave (see launch_emb_fwd).
  const int warps_per_block = blockDim.x >> 5;
  const long long total = static_cast<long long>(a.T) * ((a.B + 31) >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * warps_per_block;
  for (long long blk = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); blk < total; blk += stride)
    emb_fwd_body<NC>(a, blk);
  rs::flag_publish_when_grid_done(a.sig);   // (no-op without a signal) every thread arrives here
}

// ------------------------------------------------------------------ backward
struct EmbBwdArgs {
  float* weight;
  float* state;                  // [rows] row-wise Adagrad accumulator (null for SGD)
  const long long* row_idx;      // [nnz] resolved rows (-1 = skip)
  const int* occ2bag;            // [nnz] or null (bag == occurrence)
  long long nnz;
  const void* grad;              // per-bag gradients
  const int* grad_col;           // [T] element offset of the table's slice inside a gradient row, or null
  long long grad_row_stride;     // elements between samples
  const float* gnorm;            // optional [B, gnorm_stride]: sum of squares of each bag gradient
  int gnorm_stride;
  int B, D, grad_bf16;
  const float* psw;
  float lr, eps;
  int optimizer;                 // 0 = SGD, 1 = row-wise Adagrad
  long long total_rows;
  unsigned long long* status;
  const int* nnz_dev;            // optional: the live number of occurrences (<= nnz) as counted on the device
  rs::FlagWait wait;             // optional: wait for the peers' gradient pushes first
};

__device__ __forceinline__ long long live_nnz(const EmbBwdArgs& a) {
  if (a.nnz_dev == nullptr) return a.nnz;
  const long long n = *reinterpret_cast<const volatile int*>(a.nnz_dev);
  return n < a.nnz ? n : a.nnz;
}

constexpr int kGroup = 256;
constexpr int kSlots = 512;

template <int NC>
__device__ __forceinline__ void load_grad(const EmbBwdArgs& a, long long goff, int lane, int nvec, float4 (&g)[NC]) {
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int v = lane + c * 32;
    if (v < nvec) {
      if (a.grad_bf16) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.grad) + goff) + v);
        const float2 flo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 fhi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        g[c] = make_float4(flo.x, flo.y, fhi.x, fhi.y);
      } else {
        g[c] = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.grad) + goff) + v);
      }
    } else {
      g[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

// Pass 1 of row-wise Adagrad: state[row] += w^2 * |g_bag|^2 / D for every occurrence.
// With precomputed bag norms this is one thread per occurrence; otherwise one warp per occurrence.
template <int NC>
__global__ void __launch_bounds__(256) emb_state_kernel(const EmbBwdArgs a) {
  const float inv_d = 1.f / static_cast<float>(a.D);
  const long long nnz = live_nnz(a);
  if (a.gnorm) {
    if (static_cast<long long>(blockIdx.x) * blockDim.x >= nnz) return;   // whole block past the live occurrences
    rs::flag_wait_all(a.wait);
    // One thread per occurrence; equal rows of the block are combined in a shared-memory hash first, so a hot
    // row costs one global atomic per block instead of one per occurrence.
    __shared__ long long s_key[kSlots];
    __shared__ float s_val[kSlots];
    for (int s = threadIdx.x; s < kSlots; s += blockDim.x) {
      s_key[s] = -1;
      s_val[s] = 0.f;
    }
    __syncthreads();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < nnz) {
      const long long row = a.row_idx[i];
      if (row >= 0 && row < a.total_rows) {
        const long long bag = a.occ2bag ? a.occ2bag[i] : i;
        const int t = static_cast<int>(bag / a.B);
        const long long b = bag % a.B;
        const float w = a.psw ? a.psw[i] : 1.f;
        const float v = w * w * a.gnorm[b * a.gnorm_stride + t] * inv_d;
        unsigned s = static_cast<unsigned>(rs::ht_hash(static_cast<unsigned long long>(row))) & (kSlots - 1);
        for (int p = 0; p < kSlots; ++p) {
          const long long prev = static_cast<long long>(atomicCAS(reinterpret_cast<unsigned long long*>(&s_key[s]),
                                                                   static_cast<unsigned long long>(-1ll),
                                                                   static_cast<unsigned long long>(row)));
          if (prev == -1 || prev == row) {
            atomicAdd(&s_val[s], v);
            break;
          }
          s = (s + 1) & (kSlots - 1);
        }
      }
    }
    __syncthreads();
    for (int s = threadIdx.x; s < kSlots; s += blockDim.x)
      if (s_key[s] >= 0) atomicAdd(&a.state[s_key[s]], s_val[s]);
    return;
  }
  if (static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) >= nnz) return;
  rs::flag_wait_all(a.wait);
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= nnz) return;
  const int lane = threadIdx.x & 31;
  const long long row = a.row_idx[i];
  if (row < 0 || row >= a.total_rows) return;
  const long long bag = a.occ2bag ? a.occ2bag[i] : i;
  const int t = static_cast<int>(bag / a.B);
  const long long b = bag % a.B;
  const long long goff = b * a.grad_row_stride + (a.grad_col ? a.grad_col[t] : 0);
  const float w = a.psw ? a.psw[i] : 1.f;
  float4 g[NC];
  load_grad<NC>(a, goff, lane, a.D >> 2, g);
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) sq += g[c].x * g[c].x + g[c].y * g[c].y + g[c].z * g[c].z + g[c].w * g[c].w;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if (lane == 0) atomicAdd(&a.state[row], w * w * sq * inv_d);
}

// Apply pass: one CTA per group of 256 occurrences.  The group is counting-sorted by row in shared memory (hash
// slot -> count -> exclusive scan -> position), so equal rows sit next to each other.  Every warp then owns 32
// consecutive sorted positions, whatever the skew of the ids: it streams their gradients with kApplyInFlight
// loads (and the matching Adagrad states) in flight, sums runs of equal rows in registers and issues one vector
// atomic per run.  A row that straddles warps or groups simply receives several atomics.
constexpr int kApplyInFlight = 8;

// Raw (unconverted) gradient chunk: the loads of a batch are issued back to back with no branch and no use of
// their results in between, so all of them are in flight together; conversion happens when they are consumed.
template <bool BF16> struct RawGrad;
template <> struct RawGrad<true> {
  uint2 v;
  __device__ __forceinline__ void load(const void* base, long long goff, int vec) {
    v = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + goff) + vec);
  }
  __device__ __forceinline__ float4 get() const {
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
  }
};
template <> struct RawGrad<false> {
  float4 v;
  __device__ __forceinline__ void load(const void* base, long long goff, int vec) {
    v = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + goff) + vec);
  }
  __device__ __forceinline__ float4 get() const { return v; }
};

template <int NC, bool BF16>
__global__ void __launch_bounds__(kGroup) emb_apply_kernel(const EmbBwdArgs a) {
  __shared__ long long s_key[kSlots];
  __shared__ int s_cnt[kSlots];        // occurrences per slot, then exclusive offsets
  __shared__ long long s_goff[kGroup];  // sorted: gradient offset
  __shared__ long long s_row[kGroup];   // sorted: row
  __shared__ float s_w[kGroup];         // sorted: per-sample weight
  __shared__ int s_warp_sum[kGroup / 32];
  __shared__ int s_total;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const long long g0 = static_cast<long long>(blockIdx.x) * kGroup;
  const long long nnz = live_nnz(a);
  if (g0 >= nnz) return;                       // whole group past the live occurrences
  rs::flag_wait_all(a.wait);
  for (int s = tid; s < kSlots; s += kGroup) {
    s_key[s] = -1;
    s_cnt[s] = 0;
  }
  __syncthreads();

  long long row = -1, goff = 0;
  float w = 1.f;
  int slot = -1, rank = 0;
  if (g0 + tid < nnz) {
    const long long occ = g0 + tid;
    row = a.row_idx[occ];
    if (row >= a.total_rows) {
      if (a.status) atomicOr(a.status, (unsigned long long)RS_DEV_OOB_ROW);
      row = -1;
    }
    const long long bag = a.occ2bag ? a.occ2bag[occ] : occ;
    const int t = static_cast<int>(bag / a.B);
    const long long b = bag % a.B;
    goff = b * a.grad_row_stride + (a.grad_col ? a.grad_col[t] : 0);
    if (a.psw) w = a.psw[occ];
  }
  if (row >= 0) {
    unsigned s = static_cast<unsigned>(rs::ht_hash(static_cast<unsigned long long>(row))) & (kSlots - 1);
    for (int p = 0; p < kSlots; ++p) {
      const long long prev = static_cast<long long>(atomicCAS(reinterpret_cast<unsigned long long*>(&s_key[s]),
                                                               static_cast<unsigned long long>(-1ll),
                                                               static_cast<unsigned long long>(row)));
      if (prev == -1 || prev == row) {
        slot = static_cast<int>(s);
        rank = atomicAdd(&s_cnt[s], 1);
        break;
      }
      s = (s + 1) & (kSlots - 1);
    }
  }
  __syncthreads();
  // exclusive scan of the 512 slot counts: two slots per thread, warp shuffles, then the warp totals
  {
    const int c0 = s_cnt[2 * tid], c1 = s_cnt[2 * tid + 1];
    int incl = c0 + c1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    if (lane == 31) s_warp_sum[warp] = incl;
    __syncthreads();
    int base = 0;
#pragma unroll
    for (int q = 0; q < kGroup / 32; ++q) base += q < warp ? s_warp_sum[q] : 0;
    const int excl = base + incl - (c0 + c1);
    s_cnt[2 * tid] = excl;
    s_cnt[2 * tid + 1] = excl + c0;
    if (tid == kGroup - 1) s_total = base + incl;
  }
  __syncthreads();
  if (slot >= 0) {
    const int pos = s_cnt[slot] + rank;
    s_goff[pos] = goff;
    s_row[pos] = row;
    s_w[pos] = w;
  }
  __syncthreads();

  const int total = s_total;
  const int nvec = a.D >> 2;
  const int p_end = min(total, warp * 32 + 32);
  long long cur = -1;
  float cur_state = 0.f;
  float4 acc[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);

  auto flush = [&]() {
    if (cur < 0) return;
    float scale = -a.lr;
    if (a.optimizer == 1) scale = -a.lr / (sqrtf(cur_state) + a.eps);
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int v = lane + c * 32;
      if (v < nvec) {
        float4 u = make_float4(scale * acc[c].x, scale * acc[c].y, scale * acc[c].z, scale * acc[c].w);
        atomicAdd(reinterpret_cast<float4*>(a.weight + cur * a.D) + v, u);
      }
      acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };

  constexpr int U = NC == 1 ? kApplyInFlight : (NC == 2 ? 4 : 2);
  for (int p0 = warp * 32; p0 < p_end; p0 += U) {
    RawGrad<BF16> g[U][NC];
    float st[U];
    long long r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int p = min(p0 + u, p_end - 1);   // past the end: re-read the last valid position, ignored below
      r[u] = s_row[p];
      const long long go = s_goff[p];
#pragma unroll
      for (int c = 0; c < NC; ++c) g[u][c].load(a.grad, go, min(lane + c * 32, nvec - 1));
      st[u] = a.optimizer == 1 ? __ldcv(&a.state[r[u]]) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (p0 + u >= p_end) break;
      if (r[u] != cur) {
        flush();
        cur = r[u];
        cur_state = st[u];
      }
      const float wu = s_w[p0 + u];
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const float4 x = g[u][c].get();
        acc[c].x += wu * x.x; acc[c].y += wu * x.y;
        acc[c].z += wu * x.z; acc[c].w += wu * x.w;
      }
    }
  }
  flush();
}

// Plain row gather / scatter used by the PS get / put verbs: out[i] = W[rows[i]] (zeros when rows[i] < 0).
__global__ void rows_gather_kernel(const float* __restrict__ w, const long long* __restrict__ rows, long long n, int D,
                                   float* __restrict__ out) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  const int lane = threadIdx.x & 31;
  const long long r = rows[i];
  for (int v = lane; v < (D >> 2); v += 32) {
    const float4 x = r >= 0 ? __ldg(reinterpret_cast<const float4*>(w + r * D) + v) : make_float4(0.f, 0.f, 0.f, 0.f);
    *(reinterpret_cast<float4*>(out + i * D) + v) = x;
  }
}
// Same gather with the row range checked: rows >= total_rows give zeros and set RS_DEV_OOB_ROW in the status word.
__global__ void rows_gather_checked_kernel(const float* __restrict__ w, long long total_rows, const long long* __restrict__ rows,
                                           long long n, int D, float* __restrict__ out, unsigned long long* status) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  const int lane = threadIdx.x & 31;
  long long r = rows[i];
  if (r >= total_rows) {
    if (lane == 0 && status) atomicOr(status, (unsigned long long)RS_DEV_OOB_ROW);
    r = -1;
  }
  for (int v = lane; v < (D >> 2); v += 32) {
    const float4 x = r >= 0 ? __ldg(reinterpret_cast<const float4*>(w + r * D) + v) : make_float4(0.f, 0.f, 0.f, 0.f);
    *(reinterpret_cast<float4*>(out + i * D) + v) = x;
  }
}
__global__ void rows_scatter_kernel(float* __restrict__ w, const long long* __restrict__ rows, long long n, int D,
                                    const float* __restrict__ in) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  const int lane = threadIdx.x & 31;
  const long long r = rows[i];
  if (r < 0) return;
  for (int v = lane; v < (D >> 2); v += 32)
    *(reinterpret_cast<float4*>(w + r * D) + v) = __ldg(reinterpret_cast<const float4*>(in + i * D) + v);
}

}  // namespace

namespace {
int launch_emb_fwd(const EmbFwdArgs& a, cudaStream_t stream) {
  if (a.T == 0 || a.B == 0) return RS_OK;
  const long long nblocks = static_cast<long long>(a.T) * ((a.B + 31) / 32);
  // Four warps per CTA: at 64 registers per thread such a CTA still fits on an SM beside one persistent GEMM CTA, so the
  // lookup and its NVLink pushes really run at the same time as the MLP that is launched beside them.
  static const int wpb = [] { const char* e = getenv("RECSTORE_EMB_FWD_WARPS"); return (e && e[0] == '8') ? 8 : 4; }();
  long long grid = (nblocks + wpb - 1) / wpb;
  // RECSTORE_EMB_FWD_CTAS_PER_SM=c (0 = one CTA per 4 or 8 blocks of bags, the default): at most c CTAs per SM, the
  // warps looping over the bags.  The hardware hands out the CTAs of a later kernel only once every CTA of the earlier
  // one has been placed, so a lookup with thousands of CTAs holds back the GEMMs launched beside it on another stream
  // until its last wave; a grid that is resident as a whole does not.
  static const int per_sm = [] { const char* e = getenv("RECSTORE_EMB_FWD_CTAS_PER_SM"); return e ? atoi(e) : 0; }();
  if (per_sm > 0 && grid > 148ll * per_sm) grid = 148ll * per_sm;
  RS_REQUIRE(grid < (1ll << 31), "rs_emb_forward: too many bags");
  if (a.D <= 128) emb_fwd_kernel<1><<<static_cast<unsigned>(grid), wpb * 32, 0, stream>>>(a);
  else if (a.D <= 256) emb_fwd_kernel<2><<<static_cast<unsigned>(grid), wpb * 32, 0, stream>>>(a);
  else emb_fwd_kernel<4><<<static_cast<unsigned>(grid), wpb * 32, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
}  // namespace

RS_API int rs_emb_forward(const float* weight, const long long* table_base, const long long* table_rows,
                          const long long* indices, const long long* offsets, const int* hotness,
                          const long long* hot_base, const float* psw, int T, int B, int D, int B_local,
                          void* const* dst, long long dst_row_stride, const int* dst_col, int out_bf16,
                          long long* row_idx, int* occ2bag, const rs::HashTableView* ht,
                          unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(weight && table_base && table_rows && indices && dst && dst_col, "rs_emb_forward: null argument");
  RS_REQUIRE(offsets || (hotness && hot_base), "rs_emb_forward: need offsets or fixed hotness");
  RS_REQUIRE(D % 4 == 0 && D > 0 && D <= 128 * kMaxChunks, "rs_emb_forward: D=%d must be a multiple of 4, <= 512", D);
  RS_REQUIRE(T >= 0 && B >= 0 && B_local > 0, "rs_emb_forward: bad sizes");
  EmbFwdArgs a;
  memset(&a, 0, sizeof(a));
  a.weight = weight; a.table_base = table_base; a.table_rows = table_rows; a.indices = indices;
  a.offsets = offsets; a.hotness = hotness; a.hot_base = hot_base; a.psw = psw;
  a.T = T; a.B = B; a.D = D; a.B_local = B_local; a.dst = dst; a.dst_row_stride = dst_row_stride;
  a.dst_col = dst_col; a.out_bf16 = out_bf16; a.row_idx = row_idx; a.occ2bag = occ2bag;
  a.use_hash = ht != nullptr;
  if (ht) a.ht = *ht;
  a.status = status;
  a.id_div = 1; a.id_rem = 0;
  return launch_emb_fwd(a, stream);
}

// The same lookup with the extras of the multi-GPU engine.
//   counts / id_div / id_rem / occ_cursor: bags of a row-sharded table (see EmbFwdArgs); occ_cursor must be zero on entry.
//   wait_flags ... wait_channel:  each warp first waits (bounded) for the flag of the rank its bags come from.
//   sig_flags_of ... sig_channel: when the whole grid is done its last block publishes this rank's next epoch on the
//                                  channel to every rank (data then flag, one launch).  sig_done: a zeroed device counter.
RS_API int rs_emb_forward_ex(const float* weight, const long long* table_base, const long long* table_rows,
                             const long long* indices, const int* hotness, const long long* hot_base, int T, int B, int D,
                             int B_local, void* const* dst, long long dst_row_stride, const int* dst_col, int out_bf16,
                             long long* row_idx, int* occ2bag, unsigned long long* status,
                             const int* counts, int id_div, int id_rem, int* occ_cursor,
                             const void* wait_flags, const unsigned* counters, unsigned long long timeout_ns, int wait_channel,
                             void* const* sig_flags_of, unsigned* sig_done, int sig_channel, int world, int me,
                             cudaStream_t stream) {
  RS_REQUIRE(weight && table_base && table_rows && indices && dst && dst_col && hotness && hot_base, "rs_emb_forward_ex: null argument");
  RS_REQUIRE(D % 4 == 0 && D > 0 && D <= 128 * kMaxChunks, "rs_emb_forward_ex: D=%d must be a multiple of 4, <= 512", D);
  RS_REQUIRE(T >= 0 && B >= 0 && B_local > 0 && id_div >= 1 && id_rem >= 0 && id_rem < id_div, "rs_emb_forward_ex: bad sizes");
  RS_REQUIRE(world >= 1 && world <= 32 && me >= 0 && me < world, "rs_emb_forward_ex: bad rank / world");
  RS_REQUIRE((!wait_flags && !sig_flags_of) || counters, "rs_emb_forward_ex: flags need the epoch counters");
  RS_REQUIRE(!sig_flags_of || sig_done, "rs_emb_forward_ex: a signal needs its done counter");
  EmbFwdArgs a;
  memset(&a, 0, sizeof(a));
  a.weight = weight; a.table_base = table_base; a.table_rows = table_rows; a.indices = indices;
  a.hotness = hotness; a.hot_base = hot_base;
  a.T = T; a.B = B; a.D = D; a.B_local = B_local; a.dst = dst; a.dst_row_stride = dst_row_stride;
  a.dst_col = dst_col; a.out_bf16 = out_bf16; a.row_idx = row_idx; a.occ2bag = occ2bag;
  a.status = status;
  a.counts = counts; a.id_div = id_div; a.id_rem = id_rem; a.occ_cursor = occ_cursor;
  a.wait.my_flags = reinterpret_cast<const uint32_t*>(wait_flags); a.wait.sig_counters = counters;
  a.wait.timeout_ns = timeout_ns; a.wait.status = status; a.wait.world = world; a.wait.channel = wait_channel;
  a.sig.flags_of = reinterpret_cast<uint32_t* const*>(sig_flags_of); a.sig.sig_counters = const_cast<unsigned*>(counters);
  a.sig.done = sig_done; a.sig.world = world; a.sig.me = me; a.sig.channel = sig_channel;
  if ((T == 0 || B == 0) && sig_flags_of) return rs::set_error(RS_ERR_INVALID, "rs_emb_forward_ex: an empty lookup cannot carry the signal");
  return launch_emb_fwd(a, stream);
}

// optimizer: 0 SGD (one launch), 1 row-wise Adagrad (two launches: state pass, apply pass).
// gnorm (optional): precomputed sum of squares of every bag gradient, [B, gnorm_stride] fp32 indexed
// [sample, local table]; saves the state pass a full read of the gradients.
namespace {
int emb_backward_impl(float* weight, float* state, long long total_rows, const long long* row_idx,
                      const int* occ2bag, long long nnz, const void* grad, const int* grad_col,
                      long long grad_row_stride, const float* gnorm, int gnorm_stride, int B, int D,
                      int grad_bf16, const float* psw, float lr, float eps, int optimizer,
                      unsigned long long* status, const int* nnz_dev, const rs::FlagWait& wait, cudaStream_t stream);
}  // namespace

RS_API int rs_emb_backward(float* weight, float* state, long long total_rows, const long long* row_idx,
                           const int* occ2bag, long long nnz, const void* grad, const int* grad_col,
                           long long grad_row_stride, const float* gnorm, int gnorm_stride, int B, int D,
                           int grad_bf16, const float* psw, float lr, float eps, int optimizer,
                           unsigned long long* status, cudaStream_t stream) {
  rs::FlagWait w;
  memset(&w, 0, sizeof(w));
  return emb_backward_impl(weight, state, total_rows, row_idx, occ2bag, nnz, grad, grad_col, grad_row_stride, gnorm, gnorm_stride,
                           B, D, grad_bf16, psw, lr, eps, optimizer, status, nullptr, w, stream);
}

// The same update with the extras of the multi-GPU engine: nnz_dev (optional) is the live occurrence count on the device
// (nnz is then the capacity of the lists and sizes the grids); wait_flags (optional) makes the first kernel wait, bounded,
// until every rank's flag on `wait_channel` has reached this rank's own epoch (the peers' gradient pushes have landed).
RS_API int rs_emb_backward_ex(float* weight, float* state, long long total_rows, const long long* row_idx,
                              const int* occ2bag, long long nnz, const void* grad, const int* grad_col,
                              long long grad_row_stride, const float* gnorm, int gnorm_stride, int B, int D,
                              int grad_bf16, float lr, float eps, int optimizer, unsigned long long* status,
                              const int* nnz_dev, const void* wait_flags, const unsigned* counters, unsigned long long timeout_ns,
                              int wait_channel, int world, cudaStream_t stream) {
  rs::FlagWait w;
  memset(&w, 0, sizeof(w));
  w.my_flags = reinterpret_cast<const uint32_t*>(wait_flags); w.sig_counters = counters; w.timeout_ns = timeout_ns;
  w.status = status; w.world = world; w.channel = wait_channel;
  RS_REQUIRE(!wait_flags || (counters && world >= 1 && world <= 32), "rs_emb_backward_ex: bad flag arguments");
  return emb_backward_impl(weight, state, total_rows, row_idx, occ2bag, nnz, grad, grad_col, grad_row_stride, gnorm, gnorm_stride,
                           B, D, grad_bf16, nullptr, lr, eps, optimizer, status, nnz_dev, w, stream);
}

namespace {
int emb_backward_impl(float* weight, float* state, long long total_rows, const long long* row_idx,
                      const int* occ2bag, long long nnz, const void* grad, const int* grad_col,
                      long long grad_row_stride, const float* gnorm, int gnorm_stride, int B, int D,
                      int grad_bf16, const float* psw, float lr, float eps, int optimizer,
                      unsigned long long* status, const int* nnz_dev, const rs::FlagWait& wait, cudaStream_t stream) {
  RS_REQUIRE(weight && row_idx && grad, "rs_emb_backward: null argument");
  RS_REQUIRE(optimizer == 0 || (optimizer == 1 && state), "rs_emb_backward: row-wise Adagrad needs a state tensor");
  RS_REQUIRE(D % 4 == 0 && D > 0 && D <= 128 * kMaxChunks, "rs_emb_backward: D=%d must be a multiple of 4, <= 512", D);
  RS_REQUIRE(B > 0, "rs_emb_backward: B must be positive");
  if (nnz == 0) return RS_OK;
  EmbBwdArgs a;
  a.weight = weight; a.state = state; a.row_idx = row_idx; a.occ2bag = occ2bag; a.nnz = nnz; a.grad = grad;
  a.grad_col = grad_col; a.grad_row_stride = grad_row_stride; a.gnorm = gnorm; a.gnorm_stride = gnorm_stride;
  a.B = B; a.D = D; a.grad_bf16 = grad_bf16;
  a.psw = psw; a.lr = lr; a.eps = eps; a.optimizer = optimizer; a.total_rows = total_rows; a.status = status;
  a.nnz_dev = nnz_dev; a.wait = wait;
  const long long grid = (nnz + kGroup - 1) / kGroup;
  RS_REQUIRE(grid < (1ll << 31), "rs_emb_backward: too many occurrences");
  const int nc = D <= 128 ? 1 : (D <= 256 ? 2 : 4);
  if (optimizer == 1) {
    const long long g1 = gnorm ? (nnz + 255) / 256 : (nnz + 7) / 8;
    RS_REQUIRE(g1 < (1ll << 31), "rs_emb_backward: too many occurrences");
    if (nc == 1) emb_state_kernel<1><<<static_cast<unsigned>(g1), 256, 0, stream>>>(a);
    else if (nc == 2) emb_state_kernel<2><<<static_cast<unsigned>(g1), 256, 0, stream>>>(a);
    else emb_state_kernel<4><<<static_cast<unsigned>(g1), 256, 0, stream>>>(a);
    RS_LAUNCH_CHECK();
  }
  const unsigned g = static_cast<unsigned>(grid);
  if (grad_bf16) {
    if (nc == 1) emb_apply_kernel<1, true><<<g, kGroup, 0, stream>>>(a);
    else if (nc == 2) emb_apply_kernel<2, true><<<g, kGroup, 0, stream>>>(a);
    else emb_apply_kernel<4, true><<<g, kGroup, 0, stream>>>(a);
  } else {
    if (nc == 1) emb_apply_kernel<1, false><<<g, kGroup, 0, stream>>>(a);
    else if (nc == 2) emb_apply_kernel<2, false><<<g, kGroup, 0, stream>>>(a);
    else emb_apply_kernel<4, false><<<g, kGroup, 0, stream>>>(a);
  }
  RS_LAUNCH_CHECK();
  return RS_OK;
}

}  // namespace

RS_API int rs_rows_gather(const float* weight, const long long* rows, long long n, int D, float* out,
                          cudaStream_t stream) {
  RS_REQUIRE(weight && rows && out && D % 4 == 0, "rs_rows_gather: bad argument");
  if (n == 0) return RS_OK;
  rows_gather_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(weight, rows, n, D, out);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
RS_API int rs_rows_gather_checked(const float* weight, long long total_rows, const long long* rows, long long n, int D, float* out,
                                  unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(weight && rows && out && D % 4 == 0 && total_rows >= 0, "rs_rows_gather_checked: bad argument");
  if (n == 0) return RS_OK;
  rows_gather_checked_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(weight, total_rows, rows, n, D, out, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_rows_scatter(float* weight, const long long* rows, long long n, int D, const float* in,
                           cudaStream_t stream) {
  RS_REQUIRE(weight && rows && in && D % 4 == 0, "rs_rows_scatter: bad argument");
  if (n == 0) return RS_OK;
  rows_scatter_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(weight, rows, n, D, in);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
