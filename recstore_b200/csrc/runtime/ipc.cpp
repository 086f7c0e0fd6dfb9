// Named tensors and barriers shared between the processes of one box through POSIX shared memory.
//
// Every named tensor is its own shm object "/rsb200.<uid>.<namespace>.<name>": a 4 KiB header
// (dtype, shape, owner pid, an atomic "sliced end" for variable-length views, and a 128-byte
// blob that carries e.g. a CUDA IPC handle for GPU-resident tensors) followed by the data.
// Unlike the reference's single arena mapped at a fixed virtual address
// (src/framework/pytorch/IPCTensor.h:202-240) nothing depends on address-space layout, segments
// can be created and removed independently, and stale state is removed by name
// (rs_shm_clear_all = ClearIPCMemory).  The barrier is the counterpart of MultiProcessBarrier
// (src/framework/pytorch/IPC_barrier.h:20-51) with a timeout: a rank that never arrives makes the
// others return RS_ERR_TIMEOUT instead of spinning forever.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <thread>
#include <vector>

#include <dirent.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "common/rs_common.h"
#include "runtime/base.h"

namespace {

constexpr uint64_t kMagic = 0x5253423230305348ull;  // "RSB200SH"
constexpr size_t kHeaderBytes = 4096;

struct ShmHeader {
  uint64_t magic;
  uint32_t version;
  int32_t dtype;      // caller-defined code
  int32_t ndim;
  int64_t shape[8];
  uint64_t data_bytes;
  int32_t owner_pid;
  int32_t device;     // -1 = host data follows the header; >= 0 = data lives on that GPU
  std::atomic<int64_t> sliced_end;
  std::atomic<int32_t> ready;
  unsigned char blob[128];
};
static_assert(sizeof(ShmHeader) <= kHeaderBytes, "header too large");

struct ShmHandle {
  std::string path;
  void* base;
  size_t bytes;
};

std::string g_namespace = "default";

std::string obj_name(const char* name) {
  std::string n = "/rsb200." + std::to_string(getuid()) + "." + g_namespace + "." + name;
  for (size_t i = 1; i < n.size(); ++i)
    if (n[i] == '/') n[i] = '_';
  return n;
}
std::string prefix() { return "rsb200." + std::to_string(getuid()) + "." + g_namespace + "."; }

// An attaching process can open an object between its creator's shm_open and ftruncate: the file then still has size
// zero, mapping it fails, and touching a mapping beyond its end would raise SIGBUS.  So whoever attaches first waits
// (bounded) until the file has reached the size that every object of this kind has at least.
bool wait_for_size(int fd, size_t min_bytes, struct stat* st, int timeout_ms = 5000) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  while (true) {
    if (fstat(fd, st) != 0) return false;
    if (static_cast<size_t>(st->st_size) >= min_bytes) return true;
    if (std::chrono::steady_clock::now() > deadline) return false;
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}

struct BarrierState {
  uint64_t magic;
  int32_t parties;
  std::atomic<int32_t> arrived;
  std::atomic<uint32_t> generation;
};

}  // namespace

RS_API int rs_shm_set_namespace(const char* ns) {
  RS_REQUIRE(ns && *ns, "rs_shm_set_namespace: empty namespace");
  g_namespace = ns;
  return RS_OK;
}

// Creates (or, when it exists and exclusive == 0, attaches to) a named tensor.  *created tells which.
RS_API int rs_shm_create(const char* name, int dtype, int ndim, const long long* shape, unsigned long long data_bytes,
                         int device, int exclusive, void** out_handle, int* created) {
  RS_REQUIRE(name && out_handle && ndim >= 0 && ndim <= 8, "rs_shm_create: bad argument");
  const std::string path = obj_name(name);
  const size_t bytes = kHeaderBytes + (device < 0 ? data_bytes : 0);
  int fd = shm_open(path.c_str(), O_RDWR | O_CREAT | O_EXCL, 0600);
  bool made = fd >= 0;
  if (!made) {
    if (exclusive) return rs::set_error(RS_ERR_STATE, "shared tensor %s already exists", name);
    fd = shm_open(path.c_str(), O_RDWR, 0600);
    if (fd < 0) return rs::set_error(RS_ERR_IO, "shm_open(%s) failed", path.c_str());
  } else if (ftruncate(fd, static_cast<off_t>(bytes)) != 0) {
    close(fd);
    shm_unlink(path.c_str());
    return rs::set_error(RS_ERR_CAPACITY, "cannot size shared tensor %s to %zu bytes (is /dev/shm large enough?)", name, bytes);
  }
  struct stat st;
  if (!wait_for_size(fd, kHeaderBytes, &st)) {
    close(fd);
    return rs::set_error(RS_ERR_STATE, "shared object %s never reached the size of a tensor header (creator gone, or a foreign object)", name);
  }
  void* base = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (base == MAP_FAILED) return rs::set_error(RS_ERR_IO, "mmap of %s failed", path.c_str());
  ShmHeader* h = static_cast<ShmHeader*>(base);
  if (made) {
    h->magic = kMagic;
    h->version = 1;
    h->dtype = dtype;
    h->ndim = ndim;
    for (int i = 0; i < ndim; ++i) h->shape[i] = shape[i];
    h->data_bytes = data_bytes;
    h->owner_pid = static_cast<int32_t>(getpid());
    h->device = device;
    h->sliced_end.store(ndim > 0 ? shape[0] : 0);
    h->ready.store(1, std::memory_order_release);
  } else {
    for (int spin = 0; h->ready.load(std::memory_order_acquire) == 0 && spin < 100000; ++spin) std::this_thread::yield();
    if (h->magic != kMagic) {
      munmap(base, static_cast<size_t>(st.st_size));
      return rs::set_error(RS_ERR_STATE, "shared object %s is not a recstore tensor", name);
    }
  }
  *out_handle = new ShmHandle{path, base, static_cast<size_t>(st.st_size)};
  if (created) *created = made ? 1 : 0;
  return RS_OK;
}

RS_API int rs_shm_open(const char* name, void** out_handle) {
  RS_REQUIRE(name && out_handle, "rs_shm_open: bad argument");
  const std::string path = obj_name(name);
  int fd = shm_open(path.c_str(), O_RDWR, 0600);
  if (fd < 0) return rs::set_error(RS_ERR_NOTFOUND, "no shared tensor named %s", name);
  struct stat st;
  if (!wait_for_size(fd, kHeaderBytes, &st, 1000)) {      // smaller than a header for a second: not one of ours
    close(fd);
    return rs::set_error(RS_ERR_STATE, "shared object %s is not a recstore tensor", name);
  }
  void* base = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (base == MAP_FAILED) return rs::set_error(RS_ERR_IO, "mmap of %s failed", path.c_str());
  ShmHeader* h = static_cast<ShmHeader*>(base);
  for (int spin = 0; h->ready.load(std::memory_order_acquire) == 0 && spin < 100000; ++spin) std::this_thread::yield();
  // the header is trusted by every reader afterwards: a foreign or damaged object must not describe more than is mapped
  const bool sane = h->magic == kMagic && h->ndim >= 0 && h->ndim <= 8 &&
                    (h->device >= 0 || h->data_bytes <= static_cast<unsigned long long>(st.st_size) - kHeaderBytes);
  if (!sane) {
    munmap(base, static_cast<size_t>(st.st_size));
    return rs::set_error(RS_ERR_STATE, "shared object %s is not a recstore tensor", name);
  }
  *out_handle = new ShmHandle{path, base, static_cast<size_t>(st.st_size)};
  return RS_OK;
}

RS_API void* rs_shm_data(void* handle) {
  return static_cast<char*>(static_cast<ShmHandle*>(handle)->base) + kHeaderBytes;
}
RS_API void* rs_shm_blob(void* handle) { return static_cast<ShmHeader*>(static_cast<ShmHandle*>(handle)->base)->blob; }

RS_API int rs_shm_meta(void* handle, int* dtype, int* ndim, long long* shape8, unsigned long long* data_bytes, int* device,
                       int* owner_pid) {
  RS_REQUIRE(handle, "rs_shm_meta: null handle");
  ShmHeader* h = static_cast<ShmHeader*>(static_cast<ShmHandle*>(handle)->base);
  if (dtype) *dtype = h->dtype;
  if (ndim) *ndim = h->ndim;
  if (shape8) for (int i = 0; i < 8; ++i) shape8[i] = i < h->ndim ? h->shape[i] : 0;
  if (data_bytes) *data_bytes = h->data_bytes;
  if (device) *device = h->device;
  if (owner_pid) *owner_pid = h->owner_pid;
  return RS_OK;
}
RS_API long long rs_shm_get_sliced_end(void* handle) {
  return static_cast<ShmHeader*>(static_cast<ShmHandle*>(handle)->base)->sliced_end.load(std::memory_order_acquire);
}
RS_API void rs_shm_set_sliced_end(void* handle, long long v) {
  static_cast<ShmHeader*>(static_cast<ShmHandle*>(handle)->base)->sliced_end.store(v, std::memory_order_release);
}
RS_API int rs_shm_close(void* handle) {
  if (!handle) return RS_OK;
  ShmHandle* h = static_cast<ShmHandle*>(handle);
  munmap(h->base, h->bytes);
  delete h;
  return RS_OK;
}
RS_API int rs_shm_unlink(const char* name) {
  RS_REQUIRE(name, "rs_shm_unlink: null name");
  shm_unlink(obj_name(name).c_str());
  return RS_OK;
}

// Names (without the namespace prefix) of all shared tensors and barriers, '\n'-separated.
RS_API int rs_shm_list(char* buf, int cap) {
  std::string out;
  const std::string pre = prefix();
  if (DIR* d = opendir("/dev/shm")) {
    while (dirent* e = readdir(d)) {
      const std::string n = e->d_name;
      if (n.compare(0, pre.size(), pre) == 0) {
        out += n.substr(pre.size());
        out += '\n';
      }
    }
    closedir(d);
  }
  if (buf && cap > 0) {
    const int n = std::min<int>(cap - 1, static_cast<int>(out.size()));
    memcpy(buf, out.data(), n);
    buf[n] = 0;
  }
  return static_cast<int>(out.size());
}

// Removes every shared object of the current namespace (stale state of a crashed run included).
RS_API int rs_shm_clear_all() {
  const std::string pre = prefix();
  std::vector<std::string> names;
  if (DIR* d = opendir("/dev/shm")) {
    while (dirent* e = readdir(d)) {
      const std::string n = e->d_name;
      if (n.compare(0, pre.size(), pre) == 0) names.push_back("/" + n);
    }
    closedir(d);
  }
  for (auto& n : names) shm_unlink(n.c_str());
  return static_cast<int>(names.size());
}

// ---------------------------------------------------------------- barrier
RS_API int rs_barrier_create(const char* name, int parties, void** out_handle) {
  RS_REQUIRE(name && parties > 0 && out_handle, "rs_barrier_create: bad argument");
  const std::string path = obj_name((std::string("barrier.") + name).c_str());
  int fd = shm_open(path.c_str(), O_RDWR | O_CREAT | O_EXCL, 0600);
  const bool made = fd >= 0;
  if (!made) fd = shm_open(path.c_str(), O_RDWR, 0600);
  if (fd < 0) return rs::set_error(RS_ERR_IO, "shm_open(%s) failed", path.c_str());
  if (made && ftruncate(fd, 4096) != 0) {
    close(fd);
    return rs::set_error(RS_ERR_IO, "ftruncate(%s) failed", path.c_str());
  }
  struct stat bst;
  if (!made && !wait_for_size(fd, 4096, &bst)) {
    close(fd);
    return rs::set_error(RS_ERR_STATE, "barrier %s was never sized by its creator", name);
  }
  void* base = mmap(nullptr, 4096, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (base == MAP_FAILED) return rs::set_error(RS_ERR_IO, "mmap of %s failed", path.c_str());
  BarrierState* b = static_cast<BarrierState*>(base);
  if (made) {
    b->parties = parties;
    b->arrived.store(0);
    b->generation.store(0);
    std::atomic_thread_fence(std::memory_order_release);
    b->magic = kMagic;
  } else {
    for (int spin = 0; b->magic != kMagic && spin < 1000000; ++spin) std::this_thread::yield();
    if (b->magic != kMagic || b->parties != parties) {
      munmap(base, 4096);
      return rs::set_error(RS_ERR_STATE, "barrier %s exists with a different party count", name);
    }
  }
  *out_handle = new ShmHandle{path, base, 4096};
  return RS_OK;
}

// Returns RS_OK, or RS_ERR_TIMEOUT when not all parties arrived within timeout_ms (< 0: wait forever).
// After a timeout the barrier must be recreated (its count is no longer meaningful).
RS_API int rs_barrier_wait(void* handle, int timeout_ms) {
  RS_REQUIRE(handle, "rs_barrier_wait: null handle");
  BarrierState* b = static_cast<BarrierState*>(static_cast<ShmHandle*>(handle)->base);
  const uint32_t gen = b->generation.load(std::memory_order_acquire);
  if (b->arrived.fetch_add(1, std::memory_order_acq_rel) + 1 == b->parties) {
    b->arrived.store(0, std::memory_order_relaxed);
    b->generation.fetch_add(1, std::memory_order_release);
    return RS_OK;
  }
  const auto t0 = std::chrono::steady_clock::now();
  uint64_t spins = 0;
  while (b->generation.load(std::memory_order_acquire) == gen) {
    if (++spins < 2000) rs::cpu_relax();
    else std::this_thread::sleep_for(std::chrono::microseconds(50));
    if (timeout_ms >= 0 && (spins & 255) == 0 &&
        std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() > timeout_ms)
      return rs::set_error(RS_ERR_TIMEOUT, "barrier timed out after %d ms (%d of %d parties arrived)", timeout_ms,
                           b->arrived.load(), b->parties);
  }
  return RS_OK;
}
RS_API int rs_barrier_close(void* handle) { return rs_shm_close(handle); }
RS_API int rs_barrier_unlink(const char* name) {
  RS_REQUIRE(name, "rs_barrier_unlink: null name");
  shm_unlink(obj_name((std::string("barrier.") + name).c_str()).c_str());
  return RS_OK;
}
