// Data movement of the model-parallel embedding layers between the GPUs of one box, as thin kernels that
// co-reside with the persistent tcgen05 GEMM CTAs (128 threads, few registers, no shared memory to speak of), so
// the NVLink-bound transfers overlap the MLP math instead of taking the SMs away from it.  Each kernel publishes its
// flag itself when its grid is done (comm/flags.cuh); consumers wait inside their own prologue.
//
//   rs_push_rows            backward all-to-all of table-wise placement: per-(sample, table) gradient rows staged
//                           locally by the interaction backward go to the owning rank's gradient window together with
//                           their squared norms (extend_distributed.py:444-486 of the reference does this with
//                           all_to_all_single after a pack); a table that is row-sharded over all ranks is fanned out
//                           to every rank.
//   rs_rw_push_keys         row-sharded tables, forward, step 1 (the reference buckets keys by owner and exchanges them
//                           with all_to_all: src/python/pytorch/recstore/cache/sharded_cache.py:181-232): every id of a
//                           local bag is written into its owner's key window (owner = id % world) in the bag's
//                           fixed-capacity region, the per-(bag, owner) counts go beside them.
//   rs_rw_reduce_partials   step 3: every owner has pushed the pooled partial sum of its share of each bag (step 2 is
//                           rs_emb_forward_ex on the owner); the partials are added up into the feature slot.
#include <cuda_bf16.h>
#include <cstdlib>

#include "comm/flags.cuh"
#include "common/rs_common.h"

namespace {

constexpr int kThreads = 128;

struct PushRowsArgs {
  const __nv_bfloat16* src;   // [B, src_ld]: feature f at column f * D
  long long src_ld;
  int B, T, D, world;
  void* const* gdst;          // [world] gradient windows
  const int* owner;           // [T] owning rank, or < 0: every rank (row-sharded table)
  const int* gcol;            // [T] element offset of the table's slice inside a destination row
  long long grow_stride;      // elements between samples in a window
  long long sample_base;      // first global sample of this rank
  float* const* ndst;         // [world] squared-norm windows (fp32 [B_global, nstride]) or null
  int nstride;
  rs::FlagSignal sig;
};

// One warp per (sample, table) row, two rows in flight per warp.
__global__ void __launch_bounds__(kThreads) push_rows_kernel(const PushRowsArgs a) {
  const int lane = threadIdx.x & 31;
  const long long nwarps = static_cast<long long>(gridDim.x) * (kThreads / 32);
  const long long items = static_cast<long long>(a.B) * a.T;
  const int nvec = a.D >> 2;                           // 8-byte chunks (4 bf16) per row; lane takes chunks lane, lane + 32, ...
  for (long long w = static_cast<long long>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); w < items; w += nwarps) {
    const long long b = w / a.T;
    const int f = static_cast<int>(w % a.T);
    const __nv_bfloat16* s = a.src + b * a.src_ld + static_cast<long long>(f) * a.D;
    float sq = 0.f;
    uint2 v[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (c * 32 + lane < nvec) {
        v[c] = __ldg(reinterpret_cast<const uint2*>(s) + c * 32 + lane);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v[c].x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v[c].y));
        sq += lo.x * lo.x + lo.y * lo.y + hi.x * hi.x + hi.y * hi.y;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const int own = a.owner[f];
    const int r0 = own < 0 ? 0 : own, r1 = own < 0 ? a.world : own + 1;
    const long long off = (a.sample_base + b) * a.grow_stride + a.gcol[f];
    for (int r = r0; r < r1; ++r) {
      __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(a.gdst[r]) + off;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c * 32 + lane < nvec) *(reinterpret_cast<uint2*>(d) + c * 32 + lane) = v[c];
      if (a.ndst && lane == 0) a.ndst[r][(a.sample_base + b) * a.nstride + a.gcol[f] / a.D] = sq;
    }
  }
  rs::flag_publish_when_grid_done(a.sig);
}

struct RwKeysArgs {
  const long long* ids;        // this rank's samples: table k at ids + id_base[k], [B_local, hot[k]]
  const long long* id_base;    // [K]
  const int* hot;              // [K]
  const long long* key_base;   // [K] start of table k's region inside a key window (in keys): sum_{j<k} B * hot[j]
  int K, B_local, B, world, me;
  long long* const* key_win;   // [world] key windows
  int* const* cnt_win;         // [world] count windows, int [K, B]
  int* occ_cursor;             // cleared here for the owner-side lookup that follows on this stream (may be null)
  unsigned long long* status;
  rs::FlagSignal sig;
};

// One warp per (table, local bag).  Lane d (< world) keeps the number of ids already sent to rank d.
__global__ void __launch_bounds__(kThreads) rw_push_keys_kernel(const RwKeysArgs a) {
  const int lane = threadIdx.x & 31;
  const long long nwarps = static_cast<long long>(gridDim.x) * (kThreads / 32);
  const long long items = static_cast<long long>(a.K) * a.B_local;
  if (blockIdx.x == 0 && threadIdx.x == 0 && a.occ_cursor) *a.occ_cursor = 0;
  for (long long w = static_cast<long long>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); w < items; w += nwarps) {
    const int k = static_cast<int>(w / a.B_local);
    const int b = static_cast<int>(w % a.B_local);
    const int h = a.hot[k];
    const long long gb = static_cast<long long>(a.me) * a.B_local + b;          // global sample
    const long long* src = a.ids + a.id_base[k] + static_cast<long long>(b) * h;
    const long long region = a.key_base[k] + gb * h;                            // same offset in every owner's window
    int sent = 0;                                                               // lane d: ids sent to rank d so far
    for (int i0 = 0; i0 < h; i0 += 32) {
      const bool valid = i0 + lane < h;
      long long id = valid ? src[i0 + lane] : 0;
      int d = -1;
      if (valid) {
        if (id >= 0) d = static_cast<int>(id % a.world);
        else if (a.status) atomicOr(a.status, (unsigned long long)RS_DEV_OOB_ROW);
      }
      int pos = 0, base = 0;
      for (int dd = 0; dd < a.world; ++dd) {
        const unsigned m = __ballot_sync(0xffffffffu, d == dd);
        const int before = __shfl_sync(0xffffffffu, sent, dd);
        if (d == dd) { pos = __popc(m & ((1u << lane) - 1u)); base = before; }
        if (lane == dd) sent += __popc(m);
      }
      if (d >= 0) a.key_win[d][region + base + pos] = id;
    }
    if (lane < a.world) a.cnt_win[lane][static_cast<long long>(k) * a.B + gb] = sent;
  }
  rs::flag_publish_when_grid_done(a.sig);
}

struct RwReduceArgs {
  const __nv_bfloat16* part;   // this rank's partial window: [B_local, K, world, D]
  __nv_bfloat16* out;          // feature buffer [B_local, out_ld]
  const int* dst_col;          // [K] element offset of the table's slot in a feature row
  long long out_ld;
  int B_local, K, world, D;
  rs::FlagWait wait;
};

// One warp per (local sample, table): fp32 sum of the `world` bf16 partials.
__global__ void __launch_bounds__(kThreads) rw_reduce_partials_kernel(const RwReduceArgs a) {
  rs::flag_wait_all(a.wait);
  const int lane = threadIdx.x & 31;
  const long long nwarps = static_cast<long long>(gridDim.x) * (kThreads / 32);
  const long long items = static_cast<long long>(a.B_local) * a.K;
  const int nvec = a.D >> 2;
  for (long long w = static_cast<long long>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); w < items; w += nwarps) {
    const long long b = w / a.K;
    const int k = static_cast<int>(w % a.K);
    const __nv_bfloat16* p = a.part + (w * a.world) * a.D;
    float acc[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) acc[e] = 0.f;
    for (int r = 0; r < a.world; ++r) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (c * 32 + lane < nvec) {
          const uint2 v = __ldcv(reinterpret_cast<const uint2*>(p + static_cast<long long>(r) * a.D) + c * 32 + lane);   // written by a peer
          const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
          const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
          acc[c * 4] += lo.x; acc[c * 4 + 1] += lo.y; acc[c * 4 + 2] += hi.x; acc[c * 4 + 3] += hi.y;
        }
      }
    }
    __nv_bfloat16* o = a.out + b * a.out_ld + a.dst_col[k];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (c * 32 + lane < nvec) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc[c * 4], acc[c * 4 + 1]), hi = __floats2bfloat162_rn(acc[c * 4 + 2], acc[c * 4 + 3]);
        uint2 v;
        v.x = *reinterpret_cast<uint32_t*>(&lo);
        v.y = *reinterpret_cast<uint32_t*>(&hi);
        *(reinterpret_cast<uint2*>(o) + c * 32 + lane) = v;
      }
    }
  }
}

int grid_for(long long items) {
  long long g = (items + (kThreads / 32) - 1) / (kThreads / 32);
  // A few CTAs per SM; warps loop over the items.  RECSTORE_EXCHANGE_CTAS_PER_SM lowers it to a grid that is resident as
  // a whole beside a GEMM CTA (two 128-thread CTAs fit in the registers a GEMM CTA leaves), so that the exchange does
  // not hold back the dispatch of GEMMs launched after it on other streams.
  static const int per_sm = [] { const char* e = getenv("RECSTORE_EXCHANGE_CTAS_PER_SM"); const int v = e ? atoi(e) : 0; return v > 0 ? v : 8; }();
  const long long cap = 148ll * per_sm;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

void fill_sig(rs::FlagSignal& s, void* const* flags_of, unsigned* counters, unsigned* done, int channel, int world, int me) {
  s.flags_of = reinterpret_cast<uint32_t* const*>(flags_of);
  s.sig_counters = counters; s.done = done; s.channel = channel; s.world = world; s.me = me;
}
}  // namespace

// src: bf16 [B, src_ld].  D a multiple of 4, <= 512; rows 8-byte aligned.  sig_flags_of (optional): publish on sig_channel when done.
RS_API int rs_push_rows(const void* src, long long src_ld, int B, int T, int D, int world, void* const* gdst, const int* owner,
                        const int* gcol, long long grow_stride, long long sample_base, void* const* ndst, int nstride,
                        void* const* sig_flags_of, unsigned* counters, unsigned* sig_done, int sig_channel, int me,
                        cudaStream_t stream) {
  RS_REQUIRE(src && gdst && owner && gcol, "rs_push_rows: null argument");
  RS_REQUIRE(D % 4 == 0 && D > 0 && D <= 512 && world >= 1 && world <= 32, "rs_push_rows: D=%d must be a multiple of 4, <= 512", D);
  RS_REQUIRE(!sig_flags_of || (counters && sig_done), "rs_push_rows: a signal needs its counters");
  PushRowsArgs a;
  a.src = reinterpret_cast<const __nv_bfloat16*>(src); a.src_ld = src_ld; a.B = B; a.T = T; a.D = D; a.world = world;
  a.gdst = gdst; a.owner = owner; a.gcol = gcol; a.grow_stride = grow_stride; a.sample_base = sample_base;
  a.ndst = reinterpret_cast<float* const*>(ndst); a.nstride = nstride;
  fill_sig(a.sig, sig_flags_of, counters, sig_done, sig_channel, world, me);
  push_rows_kernel<<<grid_for(static_cast<long long>(B) * T), kThreads, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_rw_push_keys(const long long* ids, const long long* id_base, const int* hot, const long long* key_base, int K,
                           int B_local, int B, int world, int me, void* const* key_win, void* const* cnt_win, int* occ_cursor,
                           unsigned long long* status, void* const* sig_flags_of, unsigned* counters, unsigned* sig_done,
                           int sig_channel, cudaStream_t stream) {
  RS_REQUIRE(ids && id_base && hot && key_base && key_win && cnt_win, "rs_rw_push_keys: null argument");
  RS_REQUIRE(K >= 1 && B_local >= 1 && B == B_local * world && world >= 1 && world <= 32 && me >= 0 && me < world, "rs_rw_push_keys: bad sizes");
  RS_REQUIRE(!sig_flags_of || (counters && sig_done), "rs_rw_push_keys: a signal needs its counters");
  RwKeysArgs a;
  a.ids = ids; a.id_base = id_base; a.hot = hot; a.key_base = key_base; a.K = K; a.B_local = B_local; a.B = B; a.world = world;
  a.me = me; a.key_win = reinterpret_cast<long long* const*>(key_win); a.cnt_win = reinterpret_cast<int* const*>(cnt_win);
  a.occ_cursor = occ_cursor; a.status = status;
  fill_sig(a.sig, sig_flags_of, counters, sig_done, sig_channel, world, me);
  rw_push_keys_kernel<<<grid_for(static_cast<long long>(K) * B_local), kThreads, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_rw_reduce_partials(const void* part, void* out, const int* dst_col, long long out_ld, int B_local, int K, int world,
                                 int D, const void* wait_flags, const unsigned* counters, unsigned long long timeout_ns,
                                 int wait_channel, unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(part && out && dst_col, "rs_rw_reduce_partials: null argument");
  RS_REQUIRE(D % 4 == 0 && D > 0 && D <= 512 && world >= 1 && world <= 32, "rs_rw_reduce_partials: D=%d must be a multiple of 4, <= 512", D);
  RS_REQUIRE(!wait_flags || counters, "rs_rw_reduce_partials: a wait needs the epoch counters");
  RwReduceArgs a;
  a.part = reinterpret_cast<const __nv_bfloat16*>(part); a.out = reinterpret_cast<__nv_bfloat16*>(out); a.dst_col = dst_col;
  a.out_ld = out_ld; a.B_local = B_local; a.K = K; a.world = world; a.D = D;
  a.wait.my_flags = reinterpret_cast<const uint32_t*>(wait_flags); a.wait.sig_counters = counters; a.wait.timeout_ns = timeout_ns;
  a.wait.status = status; a.wait.world = world; a.wait.channel = wait_channel;
  rw_reduce_partials_kernel<<<grid_for(static_cast<long long>(B_local) * K), kThreads, 0, stream>>>(a);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
