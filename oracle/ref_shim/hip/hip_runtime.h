// Host-only stand-in for the HIP runtime header, just wide enough to compile the
// reference's host-side weight loader and buffer class on a machine without
// ROCm.  "Device" memory is ordinary host memory.  Test infrastructure only.
#pragma once
#include <cstddef>
#include <cstdlib>
#include <cstring>

typedef int hipError_t;
static const hipError_t hipSuccess = 0;
static const hipError_t hipErrorOutOfMemory = 2;
typedef void *hipStream_t;
typedef void *hipGraphNode_t;
enum hipMemcpyKind { hipMemcpyHostToHost = 0, hipMemcpyHostToDevice = 1, hipMemcpyDeviceToHost = 2, hipMemcpyDeviceToDevice = 3 };

static inline hipError_t hipMalloc(void **p, size_t n) {
  *p = std::malloc(n ? n : 1);
  return *p ? hipSuccess : hipErrorOutOfMemory;
}
static inline hipError_t hipHostMalloc(void **p, size_t n) { return hipMalloc(p, n); }
static inline hipError_t hipFree(void *p) {
  std::free(p);
  return hipSuccess;
}
static inline hipError_t hipHostFree(void *p) { return hipFree(p); }
static inline hipError_t hipMemcpy(void *d, const void *s, size_t n, hipMemcpyKind) {
  std::memcpy(d, s, n);
  return hipSuccess;
}
static inline const char *hipGetErrorString(hipError_t e) { return e == hipSuccess ? "hipSuccess" : "hipError"; }
