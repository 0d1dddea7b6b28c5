// Runtime section of the C ABI: device, memory, stream, event and graph
// primitives that the C++ L0 layer (gcore::rt on CUDA) is written against.
#include <atomic>
#include <mutex>
#include <unordered_map>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "greta_common.cuh"

namespace greta {

static thread_local char g_err[512] = "";
static std::atomic<uint64_t> g_launches{0};

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  if (e == cudaErrorMemoryAllocation) return GRETA_ERR_OUT_OF_MEM;
  if (e == cudaErrorInvalidValue || e == cudaErrorInvalidDevice) return GRETA_ERR_INVALID_ARGS;
  if (e >= cudaErrorStreamCaptureUnsupported && e <= cudaErrorStreamCaptureWrongThread)
    return GRETA_ERR_GRAPH_CAPTURE;
  return GRETA_ERR_KERNEL_LAUNCH;
}

void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Launches recorded into a graph do not run at capture time; they run once per
// replay.  The count taken between capture begin and end is moved onto the graph
// and added at every greta_cuda_graph_launch.
static std::mutex g_graph_mu;
static std::unordered_map<void *, uint64_t> g_graph_nodes;
static thread_local uint64_t g_capture_mark = 0;

static int g_pdl = -1;
bool pdl_enabled() {
  if (g_pdl < 0) {
    const char *e = getenv("GRETA_PDL");
    g_pdl = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pdl != 0;
}
void set_pdl(bool on) { g_pdl = on ? 1 : 0; }

Tuning &tuning() {
  static Tuning t = [] {
    Tuning v{};
    const char *e = getenv("GRETA_ATTN_CLUSTER");
    v.attn_cluster = (e && e[0] == '0') ? 0 : 1;
    int a = 0, b = 0;
    e = getenv("GRETA_GEMM_TILE");
    if (e && sscanf(e, "%dx%d", &a, &b) == 2) {
      v.gemm_tile_tokens = a;
      v.gemm_tile_rows = b;
    }
    e = getenv("GRETA_GEMV_R2_CELLS");
    v.gemv_r2_cells = e ? atoll(e) : -1;
    e = getenv("GRETA_STEP_STAGES");
    v.step_stages = e ? atoi(e) : 0;
    e = getenv("GRETA_PEER_POLL_LIMIT");
    v.peer_poll_limit = e ? (unsigned)strtoul(e, nullptr, 10) : (1u << 22);
    e = getenv("GRETA_ATTN_MMA");
    v.attn_mma = (e && e[0] == '0') ? 0 : 1;
    e = getenv("GRETA_PEER_TWO_LEVEL_MIN_TP");
    v.peer_two_level_min_tp = e ? atoi(e) : 4;
    e = getenv("GRETA_SKINNY_MAX_ROWS");
    v.skinny_max_rows = e ? atoi(e) : 32;
    e = getenv("GRETA_GEMV_RING_STAGES");
    v.gemv_ring_stages = e ? atoi(e) : 0;
    e = getenv("GRETA_GEMM_SPLITK");
    v.gemm_splitk = (e && (e[0] == '1' || e[0] == '2')) ? e[0] - '0' : 0;
    e = getenv("GRETA_GEMM_PAIR");
    v.gemm_pair = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 0;
    return v;
  }();
  return t;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace greta

using namespace greta;
static inline cudaStream_t S(greta_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

extern "C" {

const char *greta_cuda_last_error(void) { return g_err; }
uint64_t greta_cuda_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
int greta_cuda_set_pdl(int on) {
  set_pdl(on != 0);
  return GRETA_OK;
}
int greta_cuda_set_tuning(const char *name, long long value) {
  GRETA_REQUIRE(name, "set_tuning: null name");
  Tuning &t = tuning();
  if (!strcmp(name, "pdl")) {
    set_pdl(value != 0);
  } else if (!strcmp(name, "attn_cluster")) {
    t.attn_cluster = value != 0;
  } else if (!strcmp(name, "gemm_tile")) {  // tokens * 10 + row tiles, 0 = automatic
    t.gemm_tile_tokens = (int)(value / 10);
    t.gemm_tile_rows = (int)(value % 10);
  } else if (!strcmp(name, "gemv_r2_cells")) {
    t.gemv_r2_cells = value;
  } else if (!strcmp(name, "step_stages")) {
    t.step_stages = (int)value;
  } else if (!strcmp(name, "peer_poll_limit")) {
    GRETA_REQUIRE(value >= 1 && value <= (1ll << 30), "set_tuning: peer_poll_limit=%lld outside 1..2^30", value);
    t.peer_poll_limit = (unsigned)value;
  } else if (!strcmp(name, "attn_mma")) {
    t.attn_mma = value != 0;
  } else if (!strcmp(name, "peer_two_level_min_tp")) {
    t.peer_two_level_min_tp = (int)value;
  } else if (!strcmp(name, "skinny_max_rows")) {
    GRETA_REQUIRE(value >= 1 && value <= 32, "set_tuning: skinny_max_rows=%lld outside 1..32", value);
    t.skinny_max_rows = (int)value;
  } else if (!strcmp(name, "gemv_ring_stages")) {
    GRETA_REQUIRE(value == 0 || value == 3 || value == 5, "set_tuning: gemv_ring_stages=%lld is not 0, 3 or 5", value);
    t.gemv_ring_stages = (int)value;
  } else if (!strcmp(name, "gemm_splitk")) {
    GRETA_REQUIRE(value >= 0 && value <= 2, "set_tuning: gemm_splitk=%lld outside 0..2", value);
    t.gemm_splitk = (int)value;
  } else if (!strcmp(name, "gemm_pair")) {
    GRETA_REQUIRE(value >= 0 && value <= 2, "set_tuning: gemm_pair=%lld outside 0..2", value);
    t.gemm_pair = (int)value;
  } else {
    set_error("set_tuning: unknown switch '%s'", name);
    return GRETA_ERR_INVALID_ARGS;
  }
  return GRETA_OK;
}

int greta_cuda_device_count(int *count) {
  GRETA_REQUIRE(count, "device_count: null out pointer");
  GRETA_CUDA_TRY(cudaGetDeviceCount(count));
  return GRETA_OK;
}
int greta_cuda_set_device(int device) {
  GRETA_CUDA_TRY(cudaSetDevice(device));
  return GRETA_OK;
}
int greta_cuda_get_device(int *device) {
  GRETA_REQUIRE(device, "get_device: null out pointer");
  GRETA_CUDA_TRY(cudaGetDevice(device));
  return GRETA_OK;
}
int greta_cuda_device_info(int device, char *name, size_t name_cap, int *sms, size_t *total_mem,
                           int *cc_major, int *cc_minor) {
  cudaDeviceProp p;
  GRETA_CUDA_TRY(cudaGetDeviceProperties(&p, device));
  if (name && name_cap) {
    strncpy(name, p.name, name_cap - 1);
    name[name_cap - 1] = 0;
  }
  if (sms) *sms = p.multiProcessorCount;
  if (total_mem) *total_mem = p.totalGlobalMem;
  if (cc_major) *cc_major = p.major;
  if (cc_minor) *cc_minor = p.minor;
  return GRETA_OK;
}

int greta_cuda_malloc(void **ptr, size_t bytes) {
  GRETA_REQUIRE(ptr, "malloc: null out pointer");
  *ptr = nullptr;
  GRETA_CUDA_TRY(cudaMalloc(ptr, bytes ? bytes : 1));
  return GRETA_OK;
}
int greta_cuda_free(void *ptr) {
  if (ptr) GRETA_CUDA_TRY(cudaFree(ptr));
  return GRETA_OK;
}
int greta_cuda_malloc_host(void **ptr, size_t bytes) {
  GRETA_REQUIRE(ptr, "malloc_host: null out pointer");
  *ptr = nullptr;
  GRETA_CUDA_TRY(cudaMallocHost(ptr, bytes ? bytes : 1));
  return GRETA_OK;
}
int greta_cuda_free_host(void *ptr) {
  if (ptr) GRETA_CUDA_TRY(cudaFreeHost(ptr));
  return GRETA_OK;
}
int greta_cuda_memcpy_h2d(void *dst, const void *src, size_t bytes, greta_stream_t stream) {
  GRETA_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, S(stream)));
  return GRETA_OK;
}
int greta_cuda_memcpy_d2h(void *dst, const void *src, size_t bytes, greta_stream_t stream) {
  GRETA_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, S(stream)));
  return GRETA_OK;
}
int greta_cuda_memcpy_d2d(void *dst, const void *src, size_t bytes, greta_stream_t stream) {
  GRETA_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, S(stream)));
  return GRETA_OK;
}
int greta_cuda_memcpy_2d_d2d(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width, size_t height, greta_stream_t stream) {
  GRETA_CUDA_TRY(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width, height, cudaMemcpyDeviceToDevice, S(stream)));
  return GRETA_OK;
}
int greta_cuda_memcpy_h2d_sync(void *dst, const void *src, size_t bytes) {
  GRETA_CUDA_TRY(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
  return GRETA_OK;
}
int greta_cuda_memcpy_d2h_sync(void *dst, const void *src, size_t bytes) {
  GRETA_CUDA_TRY(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
  return GRETA_OK;
}
int greta_cuda_memset(void *dst, int value, size_t bytes, greta_stream_t stream) {
  GRETA_CUDA_TRY(cudaMemsetAsync(dst, value, bytes, S(stream)));
  return GRETA_OK;
}

int greta_cuda_stream_create(greta_stream_t *stream) {
  GRETA_REQUIRE(stream, "stream_create: null out pointer");
  cudaStream_t s;
  GRETA_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return GRETA_OK;
}
int greta_cuda_stream_destroy(greta_stream_t stream) {
  if (stream) GRETA_CUDA_TRY(cudaStreamDestroy(S(stream)));
  return GRETA_OK;
}
int greta_cuda_stream_synchronize(greta_stream_t stream) {
  GRETA_CUDA_TRY(cudaStreamSynchronize(S(stream)));
  return GRETA_OK;
}
int greta_cuda_device_synchronize(void) {
  GRETA_CUDA_TRY(cudaDeviceSynchronize());
  return GRETA_OK;
}

int greta_cuda_event_create(void **event) {
  GRETA_REQUIRE(event, "event_create: null out pointer");
  cudaEvent_t e;
  GRETA_CUDA_TRY(cudaEventCreate(&e));
  *event = e;
  return GRETA_OK;
}
int greta_cuda_event_destroy(void *event) {
  if (event) GRETA_CUDA_TRY(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
  return GRETA_OK;
}
int greta_cuda_event_record(void *event, greta_stream_t stream) {
  GRETA_CUDA_TRY(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), S(stream)));
  return GRETA_OK;
}
int greta_cuda_event_synchronize(void *event) {
  GRETA_CUDA_TRY(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(event)));
  return GRETA_OK;
}
int greta_cuda_event_elapsed_ms(void *start, void *end, float *ms) {
  GRETA_REQUIRE(ms, "event_elapsed_ms: null out pointer");
  GRETA_CUDA_TRY(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(start), reinterpret_cast<cudaEvent_t>(end)));
  return GRETA_OK;
}
int greta_cuda_stream_wait_event(greta_stream_t stream, void *event) {
  GRETA_CUDA_TRY(cudaStreamWaitEvent(S(stream), reinterpret_cast<cudaEvent_t>(event), 0));
  return GRETA_OK;
}

int greta_cuda_graph_capture_begin(greta_stream_t stream) {
  cudaError_t e = cudaStreamBeginCapture(S(stream), cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaStreamBeginCapture");
    return GRETA_ERR_GRAPH_CAPTURE;
  }
  g_capture_mark = g_launches.load();
  return GRETA_OK;
}
int greta_cuda_graph_capture_end(greta_stream_t stream, void **graph) {
  GRETA_REQUIRE(graph, "graph_capture_end: null out pointer");
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(S(stream), &g);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaStreamEndCapture");
    return GRETA_ERR_GRAPH_CAPTURE;
  }
  *graph = g;
  {
    uint64_t now = g_launches.load(), n = now - g_capture_mark;
    g_launches.fetch_sub(n);
    std::lock_guard<std::mutex> lk(g_graph_mu);
    g_graph_nodes[g] = n;
  }
  return GRETA_OK;
}
int greta_cuda_graph_instantiate(void *graph, void **exec) {
  GRETA_REQUIRE(graph && exec, "graph_instantiate: null argument");
  cudaGraphExec_t x = nullptr;
  cudaError_t e = cudaGraphInstantiate(&x, reinterpret_cast<cudaGraph_t>(graph), 0);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaGraphInstantiate");
    return GRETA_ERR_GRAPH_CAPTURE;
  }
  *exec = x;
  {
    std::lock_guard<std::mutex> lk(g_graph_mu);
    g_graph_nodes[x] = g_graph_nodes[graph];
  }
  return GRETA_OK;
}
int greta_cuda_graph_launch(void *exec, greta_stream_t stream) {
  GRETA_REQUIRE(exec, "graph_launch: null graph");
  GRETA_CUDA_TRY(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(exec), S(stream)));
  {
    std::lock_guard<std::mutex> lk(g_graph_mu);
    auto it = g_graph_nodes.find(exec);
    if (it != g_graph_nodes.end()) g_launches.fetch_add(it->second);
  }
  return GRETA_OK;
}
int greta_cuda_stream_is_capturing(greta_stream_t stream, int *capturing) {
  GRETA_REQUIRE(capturing, "stream_is_capturing: null out pointer");
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  GRETA_CUDA_TRY(cudaStreamIsCapturing(S(stream), &st));
  *capturing = st != cudaStreamCaptureStatusNone;
  return GRETA_OK;
}
int greta_cuda_graph_destroy(void *graph) {
  if (graph) GRETA_CUDA_TRY(cudaGraphDestroy(reinterpret_cast<cudaGraph_t>(graph)));
  return GRETA_OK;
}
int greta_cuda_graph_exec_destroy(void *exec) {
  if (exec) GRETA_CUDA_TRY(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(exec)));
  return GRETA_OK;
}

}  // extern "C"
