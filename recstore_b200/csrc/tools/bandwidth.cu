// Bandwidth probes: host<->device copies (pinned or pageable), device-to-device copies, a STREAM-style
// copy kernel, GPU reads of pinned host memory through UVA, and peer-to-peer copies / peer reads.
//
// Counterparts of the reference's probe programs (src/small_tests/test_h2d_bandwidth.cu,
// test_d2d_bandwidth.cu, test_uva_h2d.cu, test_uva_multigpu.cu, perf_uva.cu); here they are library entry
// points timed with CUDA events after a warm-up, returning GB/s (1e9 bytes per second).
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

#include "common/rs_common.h"

namespace {

__global__ void copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = src[i];
}

// Reads `n` 16-byte words and keeps a checksum so that the loads cannot be dropped.
__global__ void read_kernel(const uint4* __restrict__ src, size_t n, unsigned* __restrict__ sink) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  unsigned acc = 0;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const uint4 v = src[i];
    acc ^= v.x ^ v.y ^ v.z ^ v.w;
  }
  if (acc == 0x9E3779B9u) atomicAdd(sink, 1u);
}

struct EventPair {
  cudaEvent_t a = nullptr, b = nullptr;
  ~EventPair() {
    if (a) cudaEventDestroy(a);
    if (b) cudaEventDestroy(b);
  }
};

template <typename F>
int time_gbs(F&& fn, size_t bytes, int iters, double* gbs) {
  EventPair ev;
  RS_CUDA(cudaEventCreate(&ev.a));
  RS_CUDA(cudaEventCreate(&ev.b));
  for (int i = 0; i < 3; ++i) fn();
  RS_CUDA(cudaDeviceSynchronize());
  RS_CUDA(cudaEventRecord(ev.a));
  for (int i = 0; i < iters; ++i) fn();
  RS_CUDA(cudaEventRecord(ev.b));
  RS_CUDA(cudaEventSynchronize(ev.b));
  float ms = 0.f;
  RS_CUDA(cudaEventElapsedTime(&ms, ev.a, ev.b));
  *gbs = static_cast<double>(bytes) * iters / (ms * 1e-3) / 1e9;
  return RS_OK;
}

}  // namespace

// kind: 0 = host->device, 1 = device->host, 2 = device->device (copy engine), 3 = copy kernel (read + write counted
// once each, like STREAM copy), 4 = GPU kernel reading pinned host memory through UVA.
RS_API int rs_probe_bandwidth(int kind, size_t bytes, int iters, int pinned, double* gbs) {
  RS_REQUIRE(gbs && bytes >= 4096 && bytes % 16 == 0 && iters > 0, "rs_probe_bandwidth: bytes must be a multiple of 16, >= 4096");
  RS_REQUIRE(kind >= 0 && kind <= 4, "rs_probe_bandwidth: unknown kind %d", kind);
  void *h = nullptr, *d0 = nullptr, *d1 = nullptr;
  unsigned* sink = nullptr;
  int rc = RS_OK;
  auto cleanup = [&] {
    if (h) { if (pinned || kind == 4) cudaFreeHost(h); else free(h); }
    if (d0) cudaFree(d0);
    if (d1) cudaFree(d1);
    if (sink) cudaFree(sink);
  };
  if (kind == 0 || kind == 1 || kind == 4) {
    if (pinned || kind == 4) { if (cudaMallocHost(&h, bytes) != cudaSuccess) { cleanup(); return rs::set_error(RS_ERR_CUDA, "pinned allocation of %zu bytes failed", bytes); } }
    else { h = malloc(bytes); if (!h) { cleanup(); return rs::set_error(RS_ERR_CAPACITY, "malloc failed"); } }
    memset(h, 1, bytes);
  }
  if (cudaMalloc(&d0, bytes) != cudaSuccess) { cleanup(); return rs::set_error(RS_ERR_CUDA, "device allocation of %zu bytes failed", bytes); }
  if (kind == 2 || kind == 3) { if (cudaMalloc(&d1, bytes) != cudaSuccess) { cleanup(); return rs::set_error(RS_ERR_CUDA, "device allocation failed"); } }
  if (kind == 4) { if (cudaMalloc(reinterpret_cast<void**>(&sink), 4) != cudaSuccess) { cleanup(); return rs::set_error(RS_ERR_CUDA, "device allocation failed"); } cudaMemset(sink, 0, 4); }
  cudaMemset(d0, 0, bytes);
  const size_t n16 = bytes / 16;
  size_t counted = bytes;
  switch (kind) {
    case 0: rc = time_gbs([&] { cudaMemcpyAsync(d0, h, bytes, cudaMemcpyHostToDevice, 0); }, counted, iters, gbs); break;
    case 1: rc = time_gbs([&] { cudaMemcpyAsync(h, d0, bytes, cudaMemcpyDeviceToHost, 0); }, counted, iters, gbs); break;
    case 2: rc = time_gbs([&] { cudaMemcpyAsync(d1, d0, bytes, cudaMemcpyDeviceToDevice, 0); }, counted, iters, gbs); break;
    case 3:
      counted = 2 * bytes;
      rc = time_gbs([&] { copy_kernel<<<148 * 8, 512>>>(static_cast<const uint4*>(d0), static_cast<uint4*>(d1), n16); }, counted, iters, gbs);
      break;
    case 4: rc = time_gbs([&] { read_kernel<<<148 * 4, 512>>>(static_cast<const uint4*>(h), n16, sink); }, counted, iters, gbs); break;
  }
  if (rc == RS_OK && cudaGetLastError() != cudaSuccess) rc = rs::set_error(RS_ERR_CUDA, "bandwidth probe kernel failed");
  cleanup();
  return rc;
}

// Peer-to-peer: mode 0 = cudaMemcpyPeerAsync src_dev -> dst_dev, mode 1 = kernel on dst_dev reading src_dev's memory.
RS_API int rs_probe_p2p(int src_dev, int dst_dev, size_t bytes, int iters, int mode, double* gbs, int* can_access) {
  RS_REQUIRE(gbs && bytes >= 4096 && bytes % 16 == 0 && iters > 0 && src_dev != dst_dev, "rs_probe_p2p: bad argument");
  int ndev = 0;
  RS_CUDA(cudaGetDeviceCount(&ndev));
  RS_REQUIRE(src_dev >= 0 && dst_dev >= 0 && src_dev < ndev && dst_dev < ndev, "rs_probe_p2p: device out of range (have %d)", ndev);
  int prev = 0, ok = 0;
  RS_CUDA(cudaGetDevice(&prev));
  RS_CUDA(cudaDeviceCanAccessPeer(&ok, dst_dev, src_dev));
  if (can_access) *can_access = ok;
  void *s = nullptr, *d = nullptr;
  unsigned* sink = nullptr;
  int rc = RS_OK;
  cudaSetDevice(src_dev);
  if (cudaMalloc(&s, bytes) != cudaSuccess) rc = rs::set_error(RS_ERR_CUDA, "allocation on device %d failed", src_dev);
  if (rc == RS_OK) cudaMemset(s, 1, bytes);
  cudaSetDevice(dst_dev);
  if (rc == RS_OK && cudaMalloc(&d, bytes) != cudaSuccess) rc = rs::set_error(RS_ERR_CUDA, "allocation on device %d failed", dst_dev);
  if (rc == RS_OK && cudaMalloc(reinterpret_cast<void**>(&sink), 4) != cudaSuccess) rc = rs::set_error(RS_ERR_CUDA, "allocation failed");
  if (rc == RS_OK && ok) {
    const cudaError_t e = cudaDeviceEnablePeerAccess(src_dev, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) rc = rs::set_error(RS_ERR_CUDA, "cannot enable peer access %d -> %d", dst_dev, src_dev);
    cudaGetLastError();
  }
  if (rc == RS_OK) {
    if (mode == 0) {
      rc = time_gbs([&] { cudaMemcpyPeerAsync(d, dst_dev, s, src_dev, bytes, 0); }, bytes, iters, gbs);
    } else if (ok) {
      rc = time_gbs([&] { read_kernel<<<148 * 4, 512>>>(static_cast<const uint4*>(s), bytes / 16, sink); }, bytes, iters, gbs);
    } else {
      rc = rs::set_error(RS_ERR_STATE, "device %d cannot map device %d's memory", dst_dev, src_dev);
    }
  }
  if (d) cudaFree(d);
  if (sink) cudaFree(sink);
  cudaSetDevice(src_dev);
  if (s) cudaFree(s);
  cudaSetDevice(prev);
  return rc;
}
