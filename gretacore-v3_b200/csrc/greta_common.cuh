// Shared helpers of the sm_100a kernels: error plumbing, format constants, load
// and conversion primitives.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "greta_cuda.h"

namespace greta {

void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);     // records the text, maps to a GRETA_ERR_* code
void count_launch(unsigned n = 1);
int sm_count();                                     // SMs of the current device (cached per device)

#define GRETA_CUDA_TRY(expr)                                       \
  do {                                                             \
    cudaError_t _e = (expr);                                       \
    if (_e != cudaSuccess) return ::greta::cuda_fail(_e, #expr);   \
  } while (0)

#define GRETA_REQUIRE(cond, ...)                                   \
  do {                                                             \
    if (!(cond)) {                                                 \
      ::greta::set_error(__VA_ARGS__);                             \
      return GRETA_ERR_INVALID_ARGS;                               \
    }                                                              \
  } while (0)

// Checks the launch that was just issued.
inline int launched(const char *kernel, unsigned n = 1) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    cuda_fail(e, kernel);
    return GRETA_ERR_KERNEL_LAUNCH;
  }
  count_launch(n);
  return GRETA_OK;
}

// Programmatic dependent launch: a kernel launched with the attribute may start while its predecessor
// in the stream is still draining; it must execute pdl_wait() before it touches anything the
// predecessor produces (and before it overwrites anything the predecessor reads).  Weight prefetch
// sits in front of that wait.  pdl_enabled() is read once from GRETA_PDL (default on) and can be
// switched with greta_cuda_set_pdl().
bool pdl_enabled();
void set_pdl(bool on);

// Tuning switches.  Each one takes its start value from an environment variable that is read ONCE, when the
// first of them is looked at (never on a call path), and can be changed with greta_cuda_set_tuning().
struct Tuning {
  int attn_cluster;          // GRETA_ATTN_CLUSTER: 1 = the splits of a head meet in a thread-block cluster, 0 = through scratch
  int gemm_tile_tokens;      // GRETA_GEMM_TILE=<tokens>x<row tiles>: forced tile shape of the prefill GEMM, 0 = automatic
  int gemm_tile_rows;
  long long gemv_r2_cells;   // GRETA_GEMV_R2_CELLS: below this many 4-row cells a GEMV uses 2-row cells; < 0 = automatic
  int step_stages;           // GRETA_STEP_STAGES: ring depth cap of the persistent decode-step kernel, 0 = automatic
  unsigned peer_poll_limit;  // GRETA_PEER_POLL_LIMIT: polls a consumer spends on one missing partial before it gives up
  int attn_mma;              // GRETA_ATTN_MMA: 1 = prefill and grouped-query batched decode attention on the tensor cores
  int peer_two_level_min_tp; // GRETA_PEER_TWO_LEVEL_MIN_TP: ranks from which an exchange consumer gathers in two levels (see gemv_device.cuh)
  int skinny_max_rows;       // GRETA_SKINNY_MAX_ROWS: activation rows up to which the weights-read-once batched GEMV is used
  int gemv_ring_stages;      // GRETA_GEMV_RING_STAGES: 3 or 5 = forced depth of the single-row GEMV's weight ring, 0 = automatic
  int gemm_splitk;           // GRETA_GEMM_SPLITK: 1 = prefill GEMMs with few 512-token tiles share each tile's K loop between SMs (needs the workspace; changes the fp32 summation order, so off by default)
  int gemm_pair;             // GRETA_GEMM_PAIR: 1 = prefill GEMMs with 512-token tiles run as CTA pairs (two-CTA MMA, each CTA stages half of the tokens), 2 = every GEMM, 0 = none
};
Tuning &tuning();
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same, with the CTAs grouped in thread-block clusters of `cluster_x` along x.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned cluster_x, size_t smem, cudaStream_t stream,
                                      Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Payload bytes per block of 32 weights in the qs plane; 0 for unknown formats.
__host__ __device__ constexpr int payload_bytes(int fmt) {
  return fmt == GRETA_FMT_Q4_0 ? 16 : fmt == GRETA_FMT_Q8_0 ? 32 : fmt == GRETA_FMT_F16 ? 64
       : fmt == GRETA_FMT_REF_INT4 ? 16 : fmt == GRETA_FMT_REF_INT8 ? 32 : 0;
}

// Scales per row in the fp16 d plane of a GGUF format: the K/32 block scales padded to a multiple
// of 8, so every row of the plane starts on a 16-byte boundary whatever K is.
__host__ __device__ constexpr uint32_t d_row_stride(uint32_t blocks_per_row) { return (blocks_per_row + 7u) & ~7u; }

// 128-bit streaming load of weights that are read once: bypass L1 allocation.
__device__ __forceinline__ uint4 ld_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_stream8(const void *p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Sums R per-lane values (R = 2 or 4) over the warp with a butterfly that halves the number of live values at
// each of the first log2(R) steps: R + 3 (R = 4: 6) shuffles instead of 5 R.  On return lane L holds the total of
// value index warp_sum_rows_index<R>(L); the lanes with (L & 7) == 0 cover every index once.
template <int R>
__device__ __forceinline__ int warp_sum_rows_index(int lane) {
  return R == 4 ? ((lane >> 4) & 1) * 2 + ((lane >> 3) & 1) : (R == 2 ? (lane >> 4) & 1 : 0);
}
template <int R>
__device__ __forceinline__ float warp_sum_rows(const float (&v)[R], int lane) {
  static_assert(R == 1 || R == 2 || R == 4, "warp_sum_rows: 1, 2 or 4 values");
  float k0 = v[0];
  if (R == 4) {
    const bool up = lane & 16;
    float a = up ? v[2] : v[0], b = up ? v[3] : v[1];
    a += __shfl_xor_sync(0xffffffffu, up ? v[0] : v[2], 16);
    b += __shfl_xor_sync(0xffffffffu, up ? v[1] : v[3], 16);
    const bool up2 = lane & 8;
    k0 = (up2 ? b : a) + __shfl_xor_sync(0xffffffffu, up2 ? a : b, 8);
  } else if (R == 2) {
    const bool up = lane & 16;
    k0 = (up ? v[1] : v[0]) + __shfl_xor_sync(0xffffffffu, up ? v[0] : v[1], 16);
    k0 += __shfl_xor_sync(0xffffffffu, k0, 8);
  } else {
    k0 += __shfl_xor_sync(0xffffffffu, k0, 16);
    k0 += __shfl_xor_sync(0xffffffffu, k0, 8);
  }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) k0 += __shfl_xor_sync(0xffffffffu, k0, o);
  return k0;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float2 h2_to_f2(uint32_t h2) {
  return __half22float2(*reinterpret_cast<const __half2 *>(&h2));
}

}  // namespace greta
