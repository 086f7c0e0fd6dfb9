// Shared host-side helpers for the C ABI of librecstore_b200.
//
// Every exported function returns 0 on success and a non-zero code on failure;
// the message of the last failure on the calling thread is kept for
// rs_last_error().  Nothing here throws across the ABI boundary.
#pragma once
#include <exception>
#include <new>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <cstring>
#include <string>

#define RS_API extern "C" __attribute__((visibility("default")))

enum RsStatus : int {
  RS_OK = 0,
  RS_ERR_INVALID = 1,     // bad argument (size, alignment, null pointer)
  RS_ERR_CUDA = 2,        // a CUDA runtime / driver call failed
  RS_ERR_TIMEOUT = 3,     // a bounded device- or host-side wait ran out
  RS_ERR_CAPACITY = 4,    // table / cache / window is full or a size limit was exceeded
  RS_ERR_NOTFOUND = 5,
  RS_ERR_IO = 6,
  RS_ERR_STATE = 7,       // object used in the wrong state
};

namespace rs {
char* last_error_buf();                       // thread-local, 1024 bytes
int set_error(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
}  // namespace rs

// Body of an extern "C" entry point that may allocate from sizes it was handed: an exception must not cross the C
// boundary (it would terminate the process), it becomes an error code.
#define RS_NOEXCEPT_BODY(...)                                                                          \
  try {                                                                                                \
    __VA_ARGS__                                                                                        \
  } catch (const std::bad_alloc&) {                                                                    \
    return rs::set_error(RS_ERR_CAPACITY, "%s: out of memory", __func__);                              \
  } catch (const std::exception& e) {                                                                  \
    return rs::set_error(RS_ERR_INVALID, "%s: %s", __func__, e.what());                                \
  }

#define RS_REQUIRE(cond, ...)                                   \
  do {                                                          \
    if (!(cond)) return rs::set_error(RS_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#ifdef __CUDACC__
#include <cuda_runtime.h>
#define RS_CUDA(call)                                                                  \
  do {                                                                                 \
    cudaError_t _e = (call);                                                           \
    if (_e != cudaSuccess)                                                             \
      return rs::set_error(RS_ERR_CUDA, "%s:%d %s -> %s", __FILE__, __LINE__, #call,  \
                           cudaGetErrorString(_e));                                    \
  } while (0)
#define RS_LAUNCH_CHECK() RS_CUDA(cudaGetLastError())
#endif

// Device-side status word layout (one 64-bit word per kernel family, owned by the
// caller).  Kernels never trap: a failed bounds check or an exhausted wait ORs a
// code into the word, records where, and skips the access.
enum RsDevErr : unsigned {
  RS_DEV_OK = 0,
  RS_DEV_OOB_ROW = 1u << 0,       // row index outside the table
  RS_DEV_OOB_SLOT = 1u << 1,      // hash / cache slot outside capacity
  RS_DEV_OOB_PEER = 1u << 2,      // offset outside a peer window
  RS_DEV_WAIT_TIMEOUT = 1u << 3,  // bounded spin (mbarrier / flag) ran out
  RS_DEV_TABLE_FULL = 1u << 4,    // probe sequence exhausted on insert
  RS_DEV_BAD_ARG = 1u << 5,
};
