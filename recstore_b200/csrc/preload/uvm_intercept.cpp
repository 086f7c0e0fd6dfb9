// LD_PRELOAD shim that turns device allocations into managed (unified-memory) allocations, so that an
// unmodified program can oversubscribe HBM and serve as the "UVM" baseline of an embedding workload:
//
//   LD_PRELOAD=.../librecstore_uvm_intercept.so python train.py
//
// cudaMalloc(p, n) becomes cudaMallocManaged(p, n, cudaMemAttachGlobal) for n >= RECSTORE_UVM_MIN_BYTES
// (default 0: every allocation).  It only catches programs that resolve cudaMalloc dynamically (a shared
// libcudart, as PyTorch uses); a statically linked runtime never reaches the shim.  Same idea as the
// reference's interposer (src/uvm/intercept.cpp:7-18).  The next definitions of both symbols are looked
// up with dlsym(RTLD_NEXT), so the shim has no link-time dependency on CUDA.
#include <dlfcn.h>

#include <atomic>
#include <cstddef>
#include <cstdio>
#include <cstdlib>

namespace {
using MallocFn = int (*)(void**, size_t);
using ManagedFn = int (*)(void**, size_t, unsigned);
constexpr unsigned kAttachGlobal = 1;   // cudaMemAttachGlobal
constexpr int kErrorUnknown = 999;      // cudaErrorUnknown

std::atomic<unsigned long long> g_calls{0}, g_managed{0}, g_bytes{0};

size_t min_bytes() {
  static const size_t v = [] {
    const char* e = getenv("RECSTORE_UVM_MIN_BYTES");
    return e ? static_cast<size_t>(strtoull(e, nullptr, 10)) : size_t{0};
  }();
  return v;
}
}  // namespace

extern "C" {

__attribute__((visibility("default"))) int cudaMalloc(void** ptr, size_t size) {
  static MallocFn next_malloc = reinterpret_cast<MallocFn>(dlsym(RTLD_NEXT, "cudaMalloc"));
  static ManagedFn next_managed = reinterpret_cast<ManagedFn>(dlsym(RTLD_NEXT, "cudaMallocManaged"));
  g_calls.fetch_add(1, std::memory_order_relaxed);
  if (next_managed != nullptr && size >= min_bytes()) {
    g_managed.fetch_add(1, std::memory_order_relaxed);
    g_bytes.fetch_add(size, std::memory_order_relaxed);
    if (getenv("RECSTORE_UVM_LOG")) fprintf(stderr, "[uvm_intercept] cudaMalloc(%zu) -> managed\n", size);
    return next_managed(ptr, size, kAttachGlobal);
  }
  if (next_malloc != nullptr) return next_malloc(ptr, size);
  return kErrorUnknown;
}

// calls seen, calls redirected to managed memory, bytes redirected
__attribute__((visibility("default"))) void rs_uvm_intercept_stats(unsigned long long* out3) {
  out3[0] = g_calls.load();
  out3[1] = g_managed.load();
  out3[2] = g_bytes.load();
}

}  // extern "C"
