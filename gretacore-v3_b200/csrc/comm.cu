// Tensor-parallel exchange: a thin C ABI over NCCL (one process per GPU).
#include <nccl.h>

#include <cstring>

#include "greta_common.cuh"

using namespace greta;

static int nccl_fail(ncclResult_t r, const char *what) {
  set_error("%s: %s", what, ncclGetErrorString(r));
  return r == ncclInvalidArgument || r == ncclInvalidUsage ? GRETA_ERR_INVALID_ARGS : GRETA_ERR_KERNEL_LAUNCH;
}
#define NCCL_TRY(expr)                                   \
  do {                                                   \
    ncclResult_t _r = (expr);                            \
    if (_r != ncclSuccess) return nccl_fail(_r, #expr);  \
  } while (0)

extern "C" {

int greta_cuda_comm_unique_id(void *unique_id128) {
  GRETA_REQUIRE(unique_id128, "comm_unique_id: null buffer");
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is expected to be 128 bytes");
  ncclUniqueId id;
  NCCL_TRY(ncclGetUniqueId(&id));
  std::memcpy(unique_id128, &id, sizeof(id));
  return GRETA_OK;
}

int greta_cuda_comm_init(void **comm, const void *unique_id128, int nranks, int rank) {
  GRETA_REQUIRE(comm && unique_id128, "comm_init: null argument");
  GRETA_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "comm_init: rank %d of %d", rank, nranks);
  ncclUniqueId id;
  std::memcpy(&id, unique_id128, sizeof(id));
  ncclComm_t c = nullptr;
  NCCL_TRY(ncclCommInitRank(&c, nranks, id, rank));
  *comm = c;
  return GRETA_OK;
}

int greta_cuda_comm_destroy(void *comm) {
  if (comm) NCCL_TRY(ncclCommDestroy(static_cast<ncclComm_t>(comm)));
  return GRETA_OK;
}

int greta_cuda_comm_allreduce_f32(void *comm, float *buf, size_t count, greta_stream_t stream) {
  GRETA_REQUIRE(comm && buf, "comm_allreduce: null argument");
  NCCL_TRY(ncclAllReduce(buf, buf, count, ncclFloat, ncclSum, static_cast<ncclComm_t>(comm), static_cast<cudaStream_t>(stream)));
  count_launch(1);
  return GRETA_OK;
}

// Shares a device allocation with the other ranks' processes (slot buffers of the fused exchange).
int greta_cuda_ipc_export(void *device_ptr, void *handle64) {
  GRETA_REQUIRE(device_ptr && handle64, "ipc_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t is expected to be 64 bytes");
  cudaIpcMemHandle_t h;
  GRETA_CUDA_TRY(cudaIpcGetMemHandle(&h, device_ptr));
  std::memcpy(handle64, &h, sizeof(h));
  return GRETA_OK;
}

int greta_cuda_ipc_open(const void *handle64, void **device_ptr) {
  GRETA_REQUIRE(handle64 && device_ptr, "ipc_open: null argument");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  GRETA_CUDA_TRY(cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return GRETA_OK;
}

int greta_cuda_ipc_close(void *device_ptr) {
  if (device_ptr) GRETA_CUDA_TRY(cudaIpcCloseMemHandle(device_ptr));
  return GRETA_OK;
}

}  // extern "C"
