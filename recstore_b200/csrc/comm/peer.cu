// In-box NVLink transport: peer windows, cross-GPU flags with bounded waits, and the fused
// data-parallel gradient all-reduce.
//
// One process drives one GPU.  A window is plain device memory (cudaMalloc) whose CUDA IPC
// handle is exchanged through the host process group; every rank maps all peers' windows and
// kernels receive a table of base pointers.  This replaces the reference's shm + cudaIpc
// "IPCTensor" data plane (src/framework/pytorch/IPCTensor.h:281-317, 504-530), its
// pinned-CPU-staged all-to-all (src/python/pytorch/recstore/utils.py:227-310) and the rank-0
// cross-GPU index_add_ (src/framework/pytorch/grad_base.h:440-461).
//
// Flags: every rank owns flags[channel][src]; a producer rank writes its epoch number into
// flags[channel][me] of every consumer with a system-scope release store once its data stores
// are complete; the consumer polls with acquire loads.  The poll is bounded by wall-clock
// (globaltimer): when it runs out the kernel records RS_DEV_WAIT_TIMEOUT and returns, the
// context stays usable, and the host raises.
//
// All-reduce (two-shot, push): rank r sums slice r of every peer's gradient buffer with peer
// loads, scales it, and stores the result into slice r of every peer's "reduced" buffer.  The
// optimizer kernels then read only local memory.
#include "common/ptx.cuh"
#include "common/rs_common.h"

namespace {
using namespace rs::ptx;

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// flags_of[d] = base of rank d's flag array.  The epoch is a per-channel device counter that the
// kernel itself advances (so a captured CUDA graph can be replayed): it writes the new value to
// flags_of[d][channel * world + me] of every rank d.
__global__ void signal_kernel(uint32_t* const* flags_of, int world, int me, int channel, uint32_t* sig_counters) {
  const int d = threadIdx.x;
  uint32_t epoch = 0;
  if (d == 0) epoch = ++sig_counters[channel];
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  if (d < world) {
    __threadfence_system();
    st_release_sys(flags_of[d] + channel * world + me, epoch);
  }
}

// Advances this rank's per-channel wait counter and waits until my_flags[channel * world + s] has
// reached it (wrap-safe) for every source rank s.
__global__ void wait_kernel(const uint32_t* my_flags, int world, int channel, uint32_t* wait_counters,
                            unsigned long long timeout_ns, unsigned long long* status) {
  const int s = threadIdx.x;
  uint32_t epoch = 0;
  if (s == 0) epoch = ++wait_counters[channel];
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  if (s >= world) return;
  const uint32_t* f = my_flags + channel * world + s;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (true) {
    const uint32_t v = ld_acquire_sys(f);
    if (static_cast<int32_t>(v - epoch) >= 0) break;
    if ((++spins & 63u) == 0u) {
      if (globaltimer_ns() - t0 > timeout_ns) {
        if (status) atomicOr(status, (unsigned long long)RS_DEV_WAIT_TIMEOUT | (static_cast<unsigned long long>(s) << 32) |
                                         (static_cast<unsigned long long>(channel) << 48));
        break;
      }
      __nanosleep(64);
    }
  }
}

// Same wait, but for this rank's OWN signal epoch on the channel (no wait counter): for channels on which every rank
// signals exactly once per round from inside a producing kernel (comm/flags.cuh) and the consumer cannot wait in its own
// prologue (a GEMM fed by TMA).
__global__ void wait_own_kernel(const uint32_t* my_flags, int world, int channel, const uint32_t* sig_counters,
                                unsigned long long timeout_ns, unsigned long long* status) {
  const int s = threadIdx.x;
  if (s >= world) return;
  const uint32_t epoch = sig_counters[channel];
  const uint32_t* f = my_flags + channel * world + s;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (true) {
    const uint32_t v = ld_acquire_sys(f);
    if (static_cast<int32_t>(v - epoch) >= 0) break;
    if ((++spins & 63u) == 0u) {
      if (globaltimer_ns() - t0 > timeout_ns) {
        if (status) atomicOr(status, (unsigned long long)RS_DEV_WAIT_TIMEOUT | (static_cast<unsigned long long>(s) << 32) |
                                         (static_cast<unsigned long long>(channel) << 48));
        break;
      }
      __nanosleep(64);
    }
  }
}

// Signal then wait on one channel in ONE launch (a barrier of the ranks): lane d publishes this rank's new epoch to
// rank d, then waits for rank d's flag to reach this rank's new wait epoch.  Same bounds as wait_kernel.
__global__ void sync_kernel(uint32_t* const* flags_of, const uint32_t* my_flags, int world, int me, int channel,
                            uint32_t* sig_counters, uint32_t* wait_counters, unsigned long long timeout_ns,
                            unsigned long long* status) {
  const int d = threadIdx.x;
  uint32_t se = 0, we = 0;
  if (d == 0) { se = ++sig_counters[channel]; we = ++wait_counters[channel]; }
  se = __shfl_sync(0xffffffffu, se, 0);
  we = __shfl_sync(0xffffffffu, we, 0);
  if (d >= world) return;
  __threadfence_system();
  st_release_sys(flags_of[d] + channel * world + me, se);
  const uint32_t* f = my_flags + channel * world + d;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (true) {
    const uint32_t v = ld_acquire_sys(f);
    if (static_cast<int32_t>(v - we) >= 0) break;
    if ((++spins & 63u) == 0u) {
      if (globaltimer_ns() - t0 > timeout_ns) {
        if (status) atomicOr(status, (unsigned long long)RS_DEV_WAIT_TIMEOUT | (static_cast<unsigned long long>(d) << 32) |
                                         (static_cast<unsigned long long>(channel) << 48));
        break;
      }
      __nanosleep(64);
    }
  }
}

// grads_of[p]: peer p's gradient buffer; reduced_of[p]: peer p's output buffer; n elements (fp32),
// slice boundaries in float4 units.
__global__ void __launch_bounds__(256) allreduce_push_kernel(const float* const* grads_of, float* const* reduced_of,
                                                             int world, int me, long long off4, long long n4, float scale) {
  const long long per = (n4 + world - 1) / world;
  const long long beg = off4 + per * me;
  const long long end = off4 + min(n4, per * (me + 1));
  for (long long i = beg + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < end;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < world; ++p) {
      const int src = (me + p) % world;  // start with the local copy, spread peer traffic
      const float4 v = *(reinterpret_cast<const float4*>(grads_of[src]) + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    for (int p = 0; p < world; ++p) {
      const int dst = (me + p) % world;
      *(reinterpret_cast<float4*>(reduced_of[dst]) + i) = acc;
    }
  }
}

}  // namespace

RS_API int rs_device_count(int* n) {
  RS_CUDA(cudaGetDeviceCount(n));
  return RS_OK;
}

// Zero-initialised device allocation that can be exported to peer processes.
RS_API int rs_peer_alloc(size_t bytes, void** out) {
  RS_REQUIRE(out && bytes > 0, "rs_peer_alloc: bad argument");
  RS_CUDA(cudaMalloc(out, bytes));
  RS_CUDA(cudaMemset(*out, 0, bytes));
  RS_CUDA(cudaDeviceSynchronize());
  return RS_OK;
}
RS_API int rs_peer_free(void* p) {
  if (p) RS_CUDA(cudaFree(p));
  return RS_OK;
}
// handle_out: 64 bytes.
RS_API int rs_ipc_get_handle(void* p, void* handle_out) {
  RS_REQUIRE(p && handle_out, "rs_ipc_get_handle: null argument");
  cudaIpcMemHandle_t h;
  RS_CUDA(cudaIpcGetMemHandle(&h, p));
  static_assert(sizeof(h) == 64, "unexpected IPC handle size");
  memcpy(handle_out, &h, sizeof(h));
  return RS_OK;
}
RS_API int rs_ipc_open(const void* handle, void** out) {
  RS_REQUIRE(handle && out, "rs_ipc_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  RS_CUDA(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return RS_OK;
}
RS_API int rs_ipc_close(void* p) {
  if (p) RS_CUDA(cudaIpcCloseMemHandle(p));
  return RS_OK;
}

RS_API int rs_peer_signal(void* const* flags_of, int world, int me, int channel, unsigned* sig_counters,
                          cudaStream_t stream) {
  RS_REQUIRE(flags_of && sig_counters && world >= 1 && world <= 32, "rs_peer_signal: bad argument");
  signal_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<uint32_t* const*>(flags_of), world, me, channel, sig_counters);
  RS_LAUNCH_CHECK();
  return RS_OK;
}
RS_API int rs_peer_wait(const void* my_flags, int world, int channel, unsigned* wait_counters,
                        unsigned long long timeout_ns, unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(my_flags && wait_counters && world >= 1 && world <= 32, "rs_peer_wait: bad argument");
  wait_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const uint32_t*>(my_flags), world, channel, wait_counters, timeout_ns, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_peer_wait_own(const void* my_flags, int world, int channel, const unsigned* sig_counters,
                            unsigned long long timeout_ns, unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(my_flags && sig_counters && world >= 1 && world <= 32, "rs_peer_wait_own: bad argument");
  wait_own_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const uint32_t*>(my_flags), world, channel, sig_counters, timeout_ns, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

RS_API int rs_peer_sync(void* const* flags_of, const void* my_flags, int world, int me, int channel, unsigned* sig_counters,
                        unsigned* wait_counters, unsigned long long timeout_ns, unsigned long long* status, cudaStream_t stream) {
  RS_REQUIRE(flags_of && my_flags && sig_counters && wait_counters && world >= 1 && world <= 32, "rs_peer_sync: bad argument");
  sync_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<uint32_t* const*>(flags_of), reinterpret_cast<const uint32_t*>(my_flags), world,
                                    me, channel, sig_counters, wait_counters, timeout_ns, status);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// n must be a multiple of 4; buffers 16-byte aligned.  The caller brackets this with signal/wait
// pairs: peers' gradients complete before, reduced buffers complete after.
// Reduces elements [off, off + n) of the flat buffers (a bucket); off and n multiples of 4.
RS_API int rs_allreduce_push(const void* const* grads_of, void* const* reduced_of, int world, int me, long long off, long long n,
                             float scale, cudaStream_t stream) {
  RS_REQUIRE(grads_of && reduced_of && n % 4 == 0 && off % 4 == 0 && off >= 0, "rs_allreduce_push: bad argument (off and n must be multiples of 4)");
  if (n == 0) return RS_OK;
  const long long n4 = n / 4;
  const long long per = (n4 + world - 1) / world;
  // 256-thread CTAs: small enough in registers to sit on an SM beside a persistent GEMM CTA
  int grid = static_cast<int>((per + 255) / 256);
  if (grid > 592) grid = 592;
  if (grid < 1) grid = 1;
  allreduce_push_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const float* const*>(grads_of),
                                                  reinterpret_cast<float* const*>(reduced_of), world, me, off / 4, n4, scale);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// One-thread kernel that stores the GPU's nanosecond timer: a time stamp that orders with the kernels around it on
// the stream (and inside a captured graph), for phase-level timelines without a profiler.
namespace {
__global__ void stamp_kernel(unsigned long long* slot) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  *slot = t;
}
}  // namespace
RS_API int rs_stamp_time(unsigned long long* slot, cudaStream_t stream) {
  RS_REQUIRE(slot != nullptr, "rs_stamp_time: null slot");
  stamp_kernel<<<1, 1, 0, stream>>>(slot);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// Generic device helpers the Python layer needs without going through torch.
RS_API int rs_memset_async(void* p, int value, size_t bytes, cudaStream_t stream) {
  RS_CUDA(cudaMemsetAsync(p, value, bytes, stream));
  return RS_OK;
}
RS_API int rs_read_status(const unsigned long long* dev_status, unsigned long long* host_out, int reset) {
  RS_CUDA(cudaMemcpy(host_out, dev_status, sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  if (reset) RS_CUDA(cudaMemset(const_cast<unsigned long long*>(dev_status), 0, sizeof(unsigned long long)));
  return RS_OK;
}
