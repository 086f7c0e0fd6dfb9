// Cross-GPU flag channels used INSIDE producer / consumer kernels (no separate signal / wait launches).
//
// Layout (shared with comm/peer.cu): rank d owns flags[channel * world + src]; a producer publishes its epoch number
// there with a system-scope release store once its peer stores are complete, a consumer polls with acquire loads.
// Epochs are device-resident counters (sig_counters[channel]) that the producing kernel advances itself, so a captured
// CUDA graph can be replayed.
//
// Producer side: every thread calls flag_publish_when_grid_done() as its last action.  The last block of the grid to
// arrive advances the epoch and writes the flags of all ranks, so "data then flag" costs no extra launch.
//
// Consumer side: flag_wait_all() at the top of the consuming kernel.  The epoch to wait for is this rank's OWN signal
// count on the channel: on these channels every rank signals exactly once per round and a consumer kernel always runs
// after this rank's own producer of the round (stream order), so the two counts agree.  The poll is bounded by
// wall-clock time; when it runs out RS_DEV_WAIT_TIMEOUT (with the rank and channel) goes into the status word and the
// kernel carries on with whatever data is there, the host raises afterwards, the context stays usable.
#pragma once
#include "common/ptx.cuh"
#include "common/rs_common.h"

namespace rs {

struct FlagSignal {
  uint32_t* const* flags_of;   // [world] base of every rank's flag array (peer pointers); null = no signal
  uint32_t* sig_counters;      // this rank's per-channel signal epochs
  unsigned* done;              // one counter per launch site, zero between launches
  int world, me, channel;
};

struct FlagWait {
  const uint32_t* my_flags;    // this rank's flag array; null = no wait
  const uint32_t* sig_counters;
  unsigned long long timeout_ns;
  unsigned long long* status;
  int world, channel;
};

__device__ __forceinline__ unsigned long long flag_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// All threads of the block must call it (it contains block barriers).  Blocks may be of any size >= world threads.
__device__ __forceinline__ void flag_publish_when_grid_done(const FlagSignal& s) {
  if (s.flags_of == nullptr) return;
  __shared__ uint32_t sh_epoch;
  __threadfence_system();                 // this thread's peer stores are ordered before what follows
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    const unsigned prev = atomicAdd(s.done, 1u);
    uint32_t e = 0;
    if (prev == total - 1) {
      *s.done = 0;                        // ready for the next launch of this site
      e = ++s.sig_counters[s.channel];
      if (e == 0) e = ++s.sig_counters[s.channel];   // 0 means "not the last block" below
    }
    sh_epoch = e;
  }
  __syncthreads();
  const uint32_t epoch = sh_epoch;
  if (epoch != 0 && static_cast<int>(threadIdx.x) < s.world) {
    __threadfence_system();               // acquire side of the counter hand-over, then release of the flag
    ptx::st_release_sys(s.flags_of[threadIdx.x] + s.channel * s.world + s.me, epoch);
  }
}

// Waits until every source rank's flag on the channel has reached this rank's own epoch.  All threads of the block
// must call it.  Returns false when the wait ran out (the status word has the details).
__device__ __forceinline__ bool flag_wait_all(const FlagWait& w) {
  if (w.my_flags == nullptr) return true;
  __shared__ int sh_ok;
  if (threadIdx.x == 0) sh_ok = 1;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < w.world) {
    const int s = threadIdx.x;
    const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(&w.sig_counters[w.channel]);
    const uint32_t* f = w.my_flags + w.channel * w.world + s;
    const unsigned long long t0 = flag_now_ns();
    unsigned spins = 0;
    while (true) {
      const uint32_t v = ptx::ld_acquire_sys(f);
      if (static_cast<int32_t>(v - epoch) >= 0) break;
      if ((++spins & 63u) == 0u) {
        if (flag_now_ns() - t0 > w.timeout_ns) {
          if (w.status) atomicOr(w.status, (unsigned long long)RS_DEV_WAIT_TIMEOUT | (static_cast<unsigned long long>(s) << 32) |
                                               (static_cast<unsigned long long>(w.channel) << 48));
          sh_ok = 0;
          break;
        }
        __nanosleep(64);
      }
    }
  }
  __syncthreads();
  return sh_ok != 0;
}

// Waits for ONE source rank only (a consumer whose work items depend on a single producer, e.g. the keys of rank s).
// Called by one warp; lane 0 polls.  Same bound and status reporting as flag_wait_all.
__device__ __forceinline__ bool flag_wait_one_warp(const FlagWait& w, int src) {
  if (w.my_flags == nullptr) return true;
  int ok = 1;
  if ((threadIdx.x & 31) == 0) {
    const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(&w.sig_counters[w.channel]);
    const uint32_t* f = w.my_flags + w.channel * w.world + src;
    const unsigned long long t0 = flag_now_ns();
    unsigned spins = 0;
    while (true) {
      const uint32_t v = ptx::ld_acquire_sys(f);
      if (static_cast<int32_t>(v - epoch) >= 0) break;
      if ((++spins & 63u) == 0u) {
        if (flag_now_ns() - t0 > w.timeout_ns) {
          if (w.status) atomicOr(w.status, (unsigned long long)RS_DEV_WAIT_TIMEOUT | (static_cast<unsigned long long>(src) << 32) |
                                               (static_cast<unsigned long long>(w.channel) << 48));
          ok = 0;
          break;
        }
        __nanosleep(64);
      }
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  __syncwarp();
  return ok != 0;
}

}  // namespace rs
