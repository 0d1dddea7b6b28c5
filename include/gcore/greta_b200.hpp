// C++ host API of the B200 build, name-for-name with the reference's three
// levels for the quantized-matmul path:
//   L0  gcore::rt          stream / event / graph / memory / context
//       (reference: src/rt/include/gcore/rt/greta_runtime.hpp:15-97,
//        src/rt/backend/hip/include/gcore/rt/hip/{greta_runtime_hip,buffer}.hpp)
//   L1  gcore::compute     GretaCompute::{gemm, attention_decode, rmsnorm}, GretaFused
//       (reference: src/compute/include/gcore/compute/greta_compute.hpp:44-73)
//       gcore::rt::cuda::kernels::launch_*   (reference: src/rt/backend/hip/include/gcore/rt/hip/kernels/*.hpp)
//   L2  gcore::inference   ModelConfig, BlockScheduler, Generator
//       (reference: src/inference/include/gcore/inference/{model_config,block_scheduler,generator}.hpp)
// Everything here is host code that reaches the GPU only through the C ABI of
// greta_cuda.h; it needs no CUDA toolkit header to compile.  `gcore::rt::hip` is an
// alias of `gcore::rt::cuda`, so code written against the reference's HIP backend
// names keeps compiling.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../greta_cuda.h"

struct CUstream_st;
typedef CUstream_st *cudaStream_t;  // same declaration as the CUDA runtime's

// The host library is compiled with hidden visibility; the classes and functions declared here are its interface.
#pragma GCC visibility push(default)

namespace gcore::rt {

constexpr int GRETA_API_VERSION_MAJOR = 0;
constexpr int GRETA_API_VERSION_MINOR = 1;

enum class GretaResult { SUCCESS = 0, ERROR_OUT_OF_MEM, ERROR_GRAPH_CAPTURE, ERROR_KERNEL_LAUNCH, ERROR_INVALID_ARGS, ERROR_NOT_IMPLEMENTED };

// Values 0..7 are the reference's; Q4_0 / Q8_0 are the GGUF block formats this
// build stores natively (planar layout, see greta_cuda.h).
enum class GretaDataType { FP32 = 0, FP16, BF16, INT8, INT4, Q4_K, FP8_E4M3, FP8_E5M2, Q4_0 = 8, Q8_0 = 9 };

// For INT8 / INT4: `scales` = fp32 per group, as in the reference.  For Q4_0 /
// Q8_0: `scales` = the fp16 d plane, group_size 32.  head_scales is honoured for
// INT4 only (the reference multiplies Q/K/V outputs by it); leave it null.
struct GretaQuantInfo {
  const void *scales = nullptr;
  const void *head_scales = nullptr;
  float zero_point = 0.0f;
  uint32_t group_size = 0;
  uint32_t num_heads = 0;
};

class GretaStream;

class GretaEvent {
public:
  virtual ~GretaEvent() = default;
  virtual void record(GretaStream *stream) = 0;
  virtual float elapsed_time_since(GretaEvent *start) = 0;  // milliseconds, blocks until this event is reached
};

class GretaMemory {
public:
  virtual ~GretaMemory() = default;
  virtual void *data() = 0;
  virtual const void *data() const = 0;
  virtual size_t size() const = 0;
  virtual GretaDataType data_type() const = 0;
  virtual GretaQuantInfo quant_info() const = 0;
  virtual bool copy_from_host(const void *src, size_t size) = 0;
  virtual bool copy_to_host(void *dst, size_t size) const = 0;
};

class GretaStream {
public:
  virtual ~GretaStream() = default;
  virtual void synchronize() = 0;
  virtual void wait_event(GretaEvent *event) = 0;
  virtual void record_event(GretaEvent *event) = 0;
};

class GretaGraph {
public:
  virtual ~GretaGraph() = default;
  virtual void capture_start(GretaStream *stream) = 0;
  virtual void capture_end(GretaStream *stream) = 0;
  virtual GretaResult instantiate() = 0;
  virtual GretaResult launch(GretaStream *stream) = 0;
};

// Process-wide context.  create_* return owning raw pointers the caller deletes,
// the reference's convention (greta_runtime_hip.cpp:161-167).
class GretaContext {
public:
  static GretaContext &instance();
  virtual ~GretaContext() = default;
  virtual GretaResult initialize() = 0;
  virtual GretaStream *create_stream() = 0;
  virtual GretaGraph *create_graph() = 0;
  virtual GretaEvent *create_event() = 0;
  virtual GretaMemory *create_memory(size_t size, GretaDataType type = GretaDataType::FP32, bool host_visible = false) = 0;
};

namespace cuda {

enum class BufferUsage { DeviceOnly, HostVisible };

// RAII device (or pinned host) buffer; the reference's gcore::rt::hip::Buffer
// (buffer.hpp:14-52, buffer.cpp:7-84).
class Buffer : public GretaMemory {
public:
  Buffer() = default;
  ~Buffer() override;
  Buffer(const Buffer &) = delete;
  Buffer &operator=(const Buffer &) = delete;

  bool allocate(size_t size, BufferUsage usage, GretaDataType type = GretaDataType::FP32, std::string *err = nullptr);
  void free();

  void *data() override { return ptr_; }
  const void *data() const override { return ptr_; }
  size_t size() const override { return size_; }
  GretaDataType data_type() const override { return type_; }
  GretaQuantInfo quant_info() const override { return qinfo_; }

  bool copy_to_device(const void *host_ptr, size_t size, std::string *err);
  bool copy_to_host(void *host_ptr, size_t size, std::string *err) const;
  bool copy_to_host_offset(void *host_ptr, size_t offset, size_t size, std::string *err) const;
  bool copy_from_host(const void *src, size_t size) override { return copy_to_device(src, size, nullptr); }
  bool copy_to_host(void *dst, size_t size) const override { return copy_to_host(dst, size, nullptr); }
  void set_quant_info(const GretaQuantInfo &info) { qinfo_ = info; }

private:
  void *ptr_ = nullptr;
  size_t size_ = 0;
  GretaDataType type_ = GretaDataType::FP32;
  GretaQuantInfo qinfo_;
  BufferUsage usage_ = BufferUsage::DeviceOnly;
};

// Bump allocator over large device chunks; the reference's gcore::rt::hip::GretaArena (arena.hpp:8-30,
// arena.cpp:14-53): allocations are rounded up to 256 bytes, a chunk that cannot take the next one is followed by
// a new chunk (of the request's size if that is larger), nothing is freed before the arena itself.
class GretaArena {
public:
  explicit GretaArena(size_t chunk_size = 256u * 1024 * 1024);
  GretaArena(const GretaArena &) = delete;
  GretaArena &operator=(const GretaArena &) = delete;
  bool allocate(size_t size, void **out_ptr, std::string *err);
  size_t total_allocated() const { return total_allocated_; }
  size_t num_chunks() const { return chunks_.size(); }

private:
  size_t chunk_size_, current_offset_ = 0, total_allocated_ = 0;
  std::vector<std::unique_ptr<Buffer>> chunks_;
  std::mutex mutex_;
};

class GretaEventCuda : public GretaEvent {
public:
  GretaEventCuda();
  ~GretaEventCuda() override;
  void record(GretaStream *stream) override;
  float elapsed_time_since(GretaEvent *start) override;
  void *handle() const { return event_; }

private:
  void *event_ = nullptr;
};

class GretaStreamCuda : public GretaStream {
public:
  GretaStreamCuda();
  explicit GretaStreamCuda(cudaStream_t existing);
  ~GretaStreamCuda() override;
  void synchronize() override;
  void wait_event(GretaEvent *event) override;
  void record_event(GretaEvent *event) override;
  cudaStream_t handle() const { return stream_; }

private:
  cudaStream_t stream_ = nullptr;
  bool own_ = true;
};

class GretaGraphCuda : public GretaGraph {
public:
  ~GretaGraphCuda() override;
  void capture_start(GretaStream *stream) override;
  void capture_end(GretaStream *stream) override;
  GretaResult instantiate() override;
  GretaResult launch(GretaStream *stream) override;

private:
  void *graph_ = nullptr, *exec_ = nullptr;
  bool capturing_ = false;
};

class GretaMemoryCuda : public Buffer {
public:
  GretaMemoryCuda(size_t size, GretaDataType type, bool host_visible);
};

class GretaContextCuda : public GretaContext {
public:
  GretaResult initialize() override;
  GretaStream *create_stream() override;
  GretaGraph *create_graph() override;
  GretaEvent *create_event() override;
  GretaMemory *create_memory(size_t size, GretaDataType type = GretaDataType::FP32, bool host_visible = false) override;
  // Scratch for split decode attention behind the reference-signature launchers (allocated by initialize()).
  void *attention_scratch(size_t *bytes) const;
  // [256 * 128] floats behind it: the rotated copy of Q for launch_flash_attention_decode_fused_rope.
  float *query_scratch() const;

private:
  bool ready_ = false;
  Buffer attn_scratch_;
};

// Kernel launchers with the reference's names.  They return void and do nothing
// on empty shapes, like the reference's; errors are read with last_launch_error()
// (the reference's callers poll hipGetLastError, block_scheduler.cpp:1600-1623).
namespace kernels {

int last_launch_error();            // GretaResult value of the most recent launcher call on this thread
const char *last_launch_error_string();

// gemm_kernels.hpp:46-58.  b/scales are the reference's INT8 / INT4 planes.  M <= 32
// (or force_gemv) takes the GEMV kernel; larger M loops it over rows of A.
void launch_gemm_mfma_int8_wt_fp32_acc32(cudaStream_t stream, const float *a, const int8_t *b, float *c, const float *scales,
                                         uint32_t M, uint32_t N, uint32_t K, uint32_t lda, uint32_t ldb, uint32_t ldc,
                                         uint32_t group_size);
void launch_gemm_mfma_int4_wt_fp32_acc32(cudaStream_t stream, const void *a, const int8_t *b, float *c, const float *scales,
                                         const float *head_scales, uint32_t M, uint32_t N, uint32_t K, uint32_t lda,
                                         uint32_t ldb, uint32_t ldc, uint32_t group_size, uint32_t head_dim, bool is_fp16_a,
                                         bool force_gemv);
// gemm_kernels.hpp:31-39: fp32 activations x fp16 weights [N x K] -> fp32.
void launch_gemm_mixed_f16f32(cudaStream_t stream, const float *a, const uint16_t *b_f16, float *c, uint32_t M, uint32_t N,
                              uint32_t K, uint32_t lda, uint32_t ldb, uint32_t ldc);
void launch_lm_head_gemv(cudaStream_t stream, const float *x, const uint16_t *w_f16, float *y, uint32_t M, uint32_t N, uint32_t K);
// New with this build: GGUF Q4_0 / Q8_0 in the planar layout; GEMV for M <= 32, tensor-core GEMM above.
void launch_gemm_q_wt_fp32_acc32(cudaStream_t stream, GretaDataType fmt, const void *a, bool is_fp16_a, const void *qs,
                                 const void *d, void *c, bool is_fp16_c, uint32_t M, uint32_t N, uint32_t K, void *workspace);

// basic_kernels.hpp
void launch_rmsnorm_naive(cudaStream_t stream, const float *x, const float *gamma, float *y, uint32_t rows, uint32_t cols, float eps);
void launch_add(cudaStream_t stream, const float *a, const float *b, float *c, size_t n);
void launch_silu(cudaStream_t stream, const float *x, float *y, size_t n);
void launch_mul(cudaStream_t stream, const float *a, const float *b, float *c, size_t n);
void launch_embedding_lookup(cudaStream_t stream, const int32_t *tokens, const float *embeddings, float *output, uint32_t seq_len,
                             uint32_t dim, uint32_t vocab_size, bool row_major);
void launch_argmax(cudaStream_t stream, const float *d_logits, uint32_t n, int32_t *h_out);  // synchronises, like the reference's

// attention_kernels.hpp
void launch_rope(cudaStream_t stream, float *x, uint32_t seq_len, uint32_t num_heads, uint32_t head_dim, float base, uint32_t pos_offset);
void launch_rope(cudaStream_t stream, float *x, uint32_t seq_len, uint32_t num_heads, uint32_t head_dim, float base, const uint32_t *d_pos);
// The KV cache of this build is fp16 [num_heads_kv][max_seq_len][head_dim] (the reference's is fp32).
void launch_kv_update(cudaStream_t stream, uint16_t *cache_k_f16, uint16_t *cache_v_f16, const float *new_k, const float *new_v,
                      uint32_t pos, uint32_t max_seq_len, uint32_t num_heads, uint32_t head_dim);
void launch_kv_update(cudaStream_t stream, uint16_t *cache_k_f16, uint16_t *cache_v_f16, const float *new_k, const float *new_v,
                      const uint32_t *d_pos, uint32_t max_seq_len, uint32_t num_heads, uint32_t head_dim);
// fp32 cache, the reference's own signatures (attention_kernels.hpp:75-89).
void launch_flash_attention_decode(cudaStream_t stream, const float *Q, const float *K, const float *V, float *O, uint32_t num_heads,
                                   uint32_t num_heads_kv, uint32_t seq_len, uint32_t max_seq_len, uint32_t head_dim, float scale,
                                   int accum_mode = 0);
void launch_flash_attention_decode(cudaStream_t stream, const float *Q, const float *K, const float *V, float *O, uint32_t num_heads,
                                   uint32_t num_heads_kv, const uint32_t *d_pos, uint32_t max_seq_len, uint32_t head_dim, float scale,
                                   int accum_mode = 0);
// fp16 cache.
void launch_flash_attention_decode_f16kv(cudaStream_t stream, const float *Q, const uint16_t *K, const uint16_t *V, float *O,
                                         uint32_t num_heads, uint32_t num_heads_kv, const uint32_t *d_pos, uint32_t seq_len,
                                         uint32_t max_seq_len, uint32_t head_dim, float scale);
// fused_attention_kernels.hpp:14-20: Q arrives un-rotated, K in the (fp32) cache is already rotated; Q is rotated at
// *d_pos into scratch of the context and attends over *d_pos + 1 keys.  One KV head per query head, as in the reference.
void launch_flash_attention_decode_fused_rope(cudaStream_t stream, const float *Q, const float *K, const float *V, float *O,
                                              uint32_t num_heads, const uint32_t *d_pos, uint32_t max_seq_len, uint32_t head_dim,
                                              float scale, float rope_base);
// attention_kernels.hpp:124-128: Q, O [seq_len][num_heads][head_dim], K, V [seq_len][num_heads_kv][head_dim], all fp32.
void launch_flash_attention_prefill(cudaStream_t stream, const float *Q, const float *K, const float *V, float *O, uint32_t seq_len,
                                    uint32_t num_heads, uint32_t num_heads_kv, uint32_t head_dim, float scale, bool causal);
void launch_flash_attention_prefill_f16kv(cudaStream_t stream, const float *Q, const uint16_t *K_cache, const uint16_t *V_cache, float *O,
                                          uint32_t seq_len, uint32_t pos0, uint32_t num_heads, uint32_t num_heads_kv, uint32_t head_dim,
                                          uint32_t max_seq_len, float scale);

}  // namespace kernels
}  // namespace cuda

namespace hip = cuda;  // the reference's backend namespace

}  // namespace gcore::rt

namespace gcore::compute {

using namespace gcore::rt;

// Kept for source compatibility; only the routing fields are filled.
struct GemmAuditInfo {
  std::string op_label, route, quant_mode;
  int type_a = 0, type_b = 0, accum_type = 0;
  uint32_t m = 0, n = 0, k = 0, lda = 0, ldb = 0, ldc = 0;
  uintptr_t a_ptr = 0, b_ptr_base = 0, c_ptr = 0, scales_ptr = 0, head_scales_ptr = 0;
  bool perhead_enabled = false;
};

class GretaCompute {
public:
  // C[M x N] = A[M x K] * W^T, W = B [N x K] in the format B->data_type() names
  // (Q4_0, Q8_0, INT4, INT8 or FP16) with B->quant_info().scales.  A is FP32 or
  // FP16, C is FP32 or FP16.  M <= 32 takes the decode GEMV, M > 32 the
  // tensor-core GEMM (the reference's threshold, greta_compute_hip.cpp:166-167).
  // Routing depends on the arguments only: no environment is read here.
  static GretaResult gemm(GretaStream *stream, GretaMemory *A, GretaMemory *B, GretaMemory *C, uint32_t M, uint32_t N, uint32_t K,
                          bool transpose_A = false, bool transpose_B = false, GretaDataType accum_type = GretaDataType::FP32);
  // K_cache / V_cache: FP16 (this build) or FP32 (the reference's) [Hkv][max_seq][Dh]; seq_len = *d_pos + 1 when d_pos is given.
  static GretaResult attention_decode(GretaStream *stream, GretaMemory *Q, GretaMemory *K_cache, GretaMemory *V_cache, GretaMemory *d_pos,
                                      GretaMemory *O, uint32_t num_heads, uint32_t num_heads_kv, uint32_t head_dim, uint32_t seq_len,
                                      uint32_t max_seq_len, float scale, float rope_base);
  // A real RMSNorm (the reference's entry is an empty placeholder); rows = input->size() / (4 * dim).
  static GretaResult rmsnorm(GretaStream *stream, GretaMemory *input, GretaMemory *weight, GretaMemory *output, uint32_t dim, float eps);
  static void set_op_label(const char *label);
  static GemmAuditInfo get_last_gemm_audit();
  // The M > 32 route converts FP32 activations to FP16 in device scratch owned by the calling thread.  This sizes it
  // for A of up to max_M x max_K ahead of time.  gemm() grows it on demand otherwise - an allocation, so not while
  // its stream is capturing a graph: gemm() then returns ERROR_GRAPH_CAPTURE and asks for this call first.
  static GretaResult reserve_gemm_workspace(uint32_t max_M, uint32_t max_K);
};

class GretaFused {
public:
  // q = Wq n, k = Wk n, v = Wv n with n = rmsnorm(x, gamma): the entry the reference declares
  // (greta_compute.hpp:68-72) and never defines.  Weights Q4_0 / Q8_0 / FP16; D = hidden size;
  // output sizes come from the weight buffers.
  static GretaResult rmsnorm_qkv(GretaStream *stream, GretaMemory *x, GretaMemory *gamma, GretaMemory *w_q, GretaMemory *w_k,
                                 GretaMemory *w_v, GretaMemory *q_out, GretaMemory *k_out, GretaMemory *v_out, uint32_t D, float eps);
  // The full decode front: norm, projections, RoPE at *d_pos, K/V written into the fp16 caches.
  static GretaResult rmsnorm_qkv_rope_kv(GretaStream *stream, GretaMemory *x, GretaMemory *gamma, GretaMemory *w_q, GretaMemory *w_k,
                                         GretaMemory *w_v, GretaMemory *q_out, GretaMemory *k_cache, GretaMemory *v_cache,
                                         GretaMemory *d_pos, uint32_t num_heads, uint32_t num_heads_kv, uint32_t head_dim,
                                         uint32_t max_seq_len, float rope_base, uint32_t D, float eps);
  // y = silu(W1 n) * (W3 n), n = rmsnorm(x, gamma).
  static GretaResult rmsnorm_ffn_front(GretaStream *stream, GretaMemory *x, GretaMemory *gamma, GretaMemory *w1, GretaMemory *w3,
                                       GretaMemory *y, uint32_t D, uint32_t F, float eps);
  // y = resid + W x  (O-projection / down-projection with the residual add).
  static GretaResult gemv_residual(GretaStream *stream, GretaMemory *x, GretaMemory *w, GretaMemory *resid, GretaMemory *y, uint32_t N,
                                   uint32_t K);
};

}  // namespace gcore::compute

namespace gcore::inference {

struct ModelConfig {
  uint32_t dim = 4096;
  uint32_t num_heads = 32;
  uint32_t num_heads_kv = 32;
  uint32_t num_layers = 32;
  uint32_t vocab_size = 32000;
  uint32_t hidden_dim = 11008;
  uint32_t head_dim = 128;
  uint32_t max_seq_len = 2048;
  float rope_base = 10000.0f;
  float rms_eps = 1e-5f;
  std::vector<std::string> vocabulary;
  // B200 build: storage format of the projection weights and of the LM head.
  gcore::rt::GretaDataType weight_type = gcore::rt::GretaDataType::Q4_0;
  gcore::rt::GretaDataType lm_head_type = gcore::rt::GretaDataType::FP16;
  // Tensor parallelism (Megatron style): this process holds shard tp_rank of tp_size.
  uint32_t tp_rank = 0, tp_size = 1;

  static ModelConfig llama2_7b() { return ModelConfig{}; }
  static ModelConfig llama2_13b() {
    ModelConfig c;
    c.dim = 5120; c.num_heads = 40; c.num_heads_kv = 40; c.num_layers = 40; c.hidden_dim = 13824; c.max_seq_len = 4096;
    return c;
  }
  static ModelConfig llama3_70b() {
    ModelConfig c;
    c.dim = 8192; c.num_heads = 64; c.num_heads_kv = 8; c.num_layers = 80; c.vocab_size = 128256; c.hidden_dim = 28672;
    c.max_seq_len = 8192; c.rope_base = 500000.0f;
    return c;
  }
  size_t param_count() const {
    size_t kv = (size_t)num_heads_kv * head_dim;
    return (size_t)2 * vocab_size * dim + (size_t)num_layers * ((size_t)2 * dim * dim + 2 * dim * kv + (size_t)3 * dim * hidden_dim);
  }
};

// Which tensor of a layer; also the order of the synthetic-weight streams.
enum class LayerTensor : int { WQ = 0, WK, WV, WO, W1_GATE, W2_DOWN, W3_UP, ATTN_NORM, FFN_NORM };
enum class GlobalTensor : int { TOK_EMBD = 0, OUT_NORM, OUT_WEIGHT };

// Shard of a projection held by rank tp_rank of tp_size (Megatron style): Q/K/V/gate/up are split by
// rows (output features), O and down by columns (input features, whole quant blocks).
struct TensorShard {
  uint32_t rows, cols;    // local shard [rows x cols]
  uint32_t grows, gcols;  // global shape
  uint32_t row0, col0;    // offset of the shard in the global matrix
};
TensorShard tensor_shard(const ModelConfig &config, LayerTensor which);

// Weight files.  The reference's interface (weight_loader.hpp:14-92); GGUF is the format read here.
struct TensorInfo {
  std::string name;
  std::vector<size_t> shape;  // outermost first
  size_t offset = 0;          // inside the file's data section
  size_t size_bytes = 0;      // 0 for storage types this path does not read
  std::string dtype;          // "F32", "F16", "Q4_0", "Q8_0", ...
};

class WeightLoader {
public:
  virtual ~WeightLoader() = default;
  virtual bool open(const std::string &path, std::string *err) = 0;
  virtual std::vector<TensorInfo> list_tensors() const = 0;
  virtual bool load_tensor(const std::string &name, gcore::rt::cuda::Buffer &buffer, std::string *err) = 0;        // F32 / F16 -> fp32
  virtual bool load_tensor_fp16(const std::string &name, gcore::rt::cuda::Buffer &buffer, std::string *err) = 0;   // any readable type -> fp16
  // The reference's host-side re-quantisers; not carried over (GGUF blocks are stored as they are): they fail with a message.
  virtual bool load_tensor_int8(const std::string &name, gcore::rt::cuda::Buffer &buffer, gcore::rt::cuda::Buffer &scales, std::string *err) = 0;
  virtual bool load_tensor_int4(const std::string &name, gcore::rt::cuda::Buffer &buffer, gcore::rt::cuda::Buffer &scales,
                                gcore::rt::cuda::Buffer &head_scales, std::string *err) = 0;
  virtual ModelConfig get_config() const = 0;
};

class GGUFLoader : public WeightLoader {
public:
  GGUFLoader();
  ~GGUFLoader() override;
  bool open(const std::string &path, std::string *err) override;
  std::vector<TensorInfo> list_tensors() const override;
  bool load_tensor(const std::string &name, gcore::rt::cuda::Buffer &buffer, std::string *err) override;
  bool load_tensor_fp16(const std::string &name, gcore::rt::cuda::Buffer &buffer, std::string *err) override;
  bool load_tensor_int8(const std::string &name, gcore::rt::cuda::Buffer &buffer, gcore::rt::cuda::Buffer &scales, std::string *err) override;
  bool load_tensor_int4(const std::string &name, gcore::rt::cuda::Buffer &buffer, gcore::rt::cuda::Buffer &scales,
                        gcore::rt::cuda::Buffer &head_scales, std::string *err) override;
  // Shape from the file's metadata; weight_type / lm_head_type from the storage types of blk.0.attn_q.weight and output.weight.
  ModelConfig get_config() const override;
  // B200 build: the tensor's bytes as they lie in the (memory-mapped) file, and a tensor decoded to fp16 on the host.
  bool tensor_data(const std::string &name, const void **data, size_t *bytes, std::string *dtype, std::string *err) const;
  bool read_as_fp16(const std::string &name, std::vector<uint16_t> *out, std::string *err) const;

private:
  struct Impl;
  std::unique_ptr<Impl> impl_;
};

std::unique_ptr<WeightLoader> create_weight_loader(const std::string &path, std::string *err);

struct BlockBuffers {
  gcore::rt::cuda::Buffer wq, wk, wv, wo, w1, w2, w3;            // qs planes (w1 gate, w2 down, w3 up)
  gcore::rt::cuda::Buffer s_wq, s_wk, s_wv, s_wo, s_w1, s_w2, s_w3;  // d planes
  gcore::rt::cuda::Buffer attn_norm, ffn_norm;                   // fp32 [dim]
};

struct ActivationBuffers {
  gcore::rt::cuda::Buffer x, q, k, v, attn_out, mlp_gate, mlp_up, mlp_out, norm_out;
  gcore::rt::cuda::Buffer kv_cache_k, kv_cache_v;   // fp16 [L][Hkv_local][max_seq][Dh]
  gcore::rt::cuda::Buffer tokens, d_pos, d_next, attn_scratch, gemm_ws, out_tokens;
};

// Hook for the exchange step of tensor parallelism: in-place sum of `count`
// floats over the ranks on `stream`.  Installed by the multi-GPU driver.
using AllReduceFn = std::function<int(float *buf, size_t count, cudaStream_t stream)>;

class BlockScheduler {
public:
  BlockScheduler();
  ~BlockScheduler();

  bool init(const ModelConfig &config, std::string *err);
  bool allocate_weights(std::string *err);
  bool allocate_activations(size_t batch_size, size_t max_seq_len, std::string *err);
  // Seeded random weights of the configured shape (GGUF blocks generated on the host, uploaded, repacked on the device).
  bool load_synthetic_weights(uint64_t seed, std::string *err);
  // From a GGUF file whose projections are stored as Q4_0 or Q8_0 (block_scheduler.hpp:83 in the reference): the blocks go
  // to the device as they lie in the file; under tensor parallelism every rank keeps its shard.
  bool load_weights(WeightLoader &loader, std::string *err);
  // One tensor from host memory: GGUF blocks for the projections, fp32 for the norms, fp16 for embedding / LM head.
  bool set_layer_tensor(size_t layer, LayerTensor which, const void *host, size_t bytes, std::string *err);
  bool set_global_tensor(GlobalTensor which, const void *host, size_t bytes, std::string *err);
  // The same for a tensor stored as K-quant super-blocks (ggml_type GRETA_GGML_Q4_K / GRETA_GGML_Q6_K): the global tensor is
  // decoded on the device with the reference loader's arithmetic and re-stored as Q8_0 blocks, so weight_type (or lm_head_type
  // for OUT_WEIGHT) must be Q8_0.  The reference re-quantises such tensors as well (to its INT4: weight_loader.cpp:920-957).
  bool set_layer_tensor_kquant(size_t layer, LayerTensor which, int ggml_type, const void *host, size_t bytes, std::string *err);
  bool set_global_tensor_kquant(GlobalTensor which, int ggml_type, const void *host, size_t bytes, std::string *err);

  bool execute_layer(size_t layer_idx, size_t seq_start, size_t seq_len, const int32_t *tokens, std::string *err);
  // Runs seq_len tokens starting at seq_start; logits of the last position are left in get_logits().
  bool forward(const int32_t *tokens, size_t seq_start, size_t seq_len, std::string *err);
  int32_t sample_greedy_gpu(size_t logits_offset_bytes, std::string *err);

  // Decode fast path: one token per call, everything on the device.  The step (embedding of the
  // previous arg-max, all layers, LM head, arg-max, position bump) is captured once into a CUDA
  // graph; decode_step() replays it.  begin_decode() seeds it with the first token and position.
  bool begin_decode(int32_t first_token, size_t pos, std::string *err);
  // B200 build: a batch of sequences decoding in step (allocate_activations(batch, ...)).  Prefill fills one sequence's
  // cache at a time: set_sequence(b), then forward() as usual.  begin_decode_batch takes every sequence's first token
  // and position; decode_step() then advances all of them; read_generated() returns [batch][n] ids;
  // decode_step_host() moves `batch` ids each way.
  bool set_sequence(size_t seq, std::string *err);
  bool begin_decode_batch(const int32_t *first_tokens, const uint32_t *positions, std::string *err);
  size_t batch_size() const { return batch_; }
  bool decode_step(std::string *err);                 // asynchronous
  bool read_generated(int32_t *out, size_t n, std::string *err);  // synchronises; ids produced since begin_decode()
  // Host-driven step: token id in from pinned host memory, sampled id out to pinned host memory, synchronised.
  bool decode_step_host(const int32_t *pinned_token_in, int32_t *pinned_token_out, std::string *err);

  gcore::rt::cuda::Buffer &get_hidden_state() { return activations_.x; }
  gcore::rt::cuda::Buffer &get_norm_out() { return activations_.norm_out; }
  const gcore::rt::cuda::Buffer &get_logits() const { return logits_; }
  const gcore::rt::cuda::Buffer &get_output_weight() const { return output_weight_; }
  const ModelConfig &config() const { return config_; }
  size_t num_layers() const { return blocks_.size(); }
  size_t max_seq_len() const { return max_seq_; }
  gcore::rt::GretaStream *stream() { return stream_; }
  void set_all_reduce(AllReduceFn fn);  // drops a captured decode step: it holds the old hook
  // Tensor-parallel decode with the exchange fused into the operators over peer memory (greta_cuda.h,
  // greta_peer_exchange): used by the captured decode step; forward() keeps the all-reduce hook.
  bool set_peer_exchange(const greta_peer_exchange &ex, std::string *err);
  uint64_t weight_bytes() const { return weight_bytes_; }
  bool decode_trace(long long *out25);

private:
  bool decode_layers(std::string *err, bool fused_exchange = false, const float **x_final = nullptr);
  bool decode_layers_batch(std::string *err);
  bool lm_head_batch(std::string *err);
  bool step_fits(std::string *err) const;
  void invalidate_graph();
  bool build_decode_plan(std::string *err);
  bool lm_head(const float *x_row, std::string *err);
  ModelConfig config_;
  std::vector<BlockBuffers> blocks_;
  ActivationBuffers activations_;
  gcore::rt::cuda::Buffer token_embd_, output_norm_, output_weight_, s_output_weight_, logits_;
  gcore::rt::cuda::Buffer decode_plan_;   // persistent decode-step kernel: descriptors + barrier state
  bool persistent_step_ = false;
  gcore::rt::GretaStream *stream_ = nullptr;
  gcore::rt::GretaGraph *graph_ = nullptr;
  bool graph_captured_ = false, initialized_ = false;
  size_t decode_steps_ = 0, decode_pos0_ = 0, max_seq_ = 0;
  uint32_t batch_ = 1, cur_seq_ = 0;      // sequences held; the one forward() / execute_layer() work on
  gcore::rt::cuda::Buffer batch_ws_;      // batched decode: activations prepared for the tensor-core matmul kernels
  gcore::rt::cuda::Buffer logits_local_;  // tensor-parallel batch: this rank's slice of the logits before placement
  AllReduceFn all_reduce_;
  greta_peer_exchange peer_{};            // tp == 0: not installed
  gcore::rt::cuda::Buffer x_alt_;         // second copy of the residual stream for the fused exchange
  uint64_t weight_bytes_ = 0;
  // local (per-rank) shapes
  uint32_t heads_l_ = 0, kv_heads_l_ = 0, hidden_l_ = 0, vocab_l_ = 0;
};

struct SamplingParams {
  float temperature = 1.0f;
  int32_t top_k = 50;
  float top_p = 1.0f;
  int32_t max_tokens = 128;
  int32_t seed = 42;
  bool greedy = false;
  // B200 build: id that ends generation (the reference asks its tokenizer, which is outside this path); -1 = none.
  int32_t eos_token_id = -1;
};

struct GenerationStats {
  size_t prompt_tokens = 0, generated_tokens = 0;
  double total_time_ms = 0.0, tokens_per_second = 0.0, time_to_first_token_ms = 0.0;
  double decode_time_ms = 0.0;  // device time of the decode steps alone
};

// Greedy generation over token ids (the tokenizer is outside this path).
class Generator {
public:
  bool init(const ModelConfig &config, BlockScheduler *scheduler, std::string *err);
  std::vector<int32_t> generate_tokens(const std::vector<int32_t> &prompt_tokens, const SamplingParams &params,
                                       GenerationStats *stats = nullptr, std::string *err = nullptr);
  // B200 build: greedy generation for every sequence of the scheduler's batch (prompts.size() == batch_size()):
  // the prompts are prefilled one sequence at a time, then all sequences decode in step on the device.
  std::vector<std::vector<int32_t>> generate_batch(const std::vector<std::vector<int32_t>> &prompts, const SamplingParams &params,
                                                   std::string *err = nullptr);
  // First maximum wins, as the reference's host sampler does (generator.cpp:735-744).
  int32_t sample(const float *logits, size_t vocab_size, const SamplingParams &params);

private:
  ModelConfig config_;
  BlockScheduler *scheduler_ = nullptr;
};

// Counter-based synthetic data (splitmix64 over seed, stream and index): the same call gives the
// same bytes on every machine, so a CPU checker and the GPU can be fed identical tensors.
namespace synth {
void quant_blocks(uint64_t seed, uint64_t stream, gcore::rt::GretaDataType fmt, uint8_t *out, size_t first_block, size_t n_blocks, float sigma = 0.02f);
void normal_f32(uint64_t seed, uint64_t stream, float sigma, float *out, size_t first, size_t n);
void normal_f16(uint64_t seed, uint64_t stream, float sigma, uint16_t *out, size_t first, size_t n);
void normal_f16_as_f32(uint64_t seed, uint64_t stream, float sigma, float *out, size_t first, size_t n);  // rounded through fp16
void tokens(uint64_t seed, uint64_t stream, uint32_t vocab, int32_t *out, size_t n);
uint64_t tensor_stream(uint32_t layer, int which);  // stream id of a model tensor
}  // namespace synth

}  // namespace gcore::inference

#pragma GCC visibility pop
