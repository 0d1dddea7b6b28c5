// L2: BlockScheduler (owns weights, activations and the KV cache; runs the layer
// sequence) and Generator (prefill + greedy decode loop), on top of the C ABI.
//
// Per decode token and layer the reference launches 15 kernels
// (src/inference/src/block_scheduler.cpp:1814-3032); here it is 5:
//   1. RMSNorm -> Q/K/V GEMV -> RoPE -> fp16 KV-cache write   (one kernel)
//   2. split decode attention over the cache
//   3. O-projection GEMV + residual
//   4. RMSNorm -> gate/up GEMV -> SwiGLU
//   5. down-projection GEMV + residual
// and the whole step (embedding of the previous arg-max, layers, final norm + LM
// head, arg-max, position bump) is captured into one CUDA graph, so a step is a
// single graph launch with no host round trip.
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "gcore/greta_b200.hpp"
#include "host_util.hpp"

namespace gcore::inference {

using gcore::host::fail;
using gcore::rt::GretaDataType;
using gcore::rt::GretaQuantInfo;
using gcore::rt::cuda::Buffer;
using gcore::rt::cuda::BufferUsage;
using gcore::rt::cuda::GretaStreamCuda;

namespace {

inline size_t block_bytes(GretaDataType t) { return t == GretaDataType::Q4_0 ? 18 : 34; }
inline int fmt_of(GretaDataType t) { return t == GretaDataType::Q4_0 ? GRETA_FMT_Q4_0 : t == GretaDataType::Q8_0 ? GRETA_FMT_Q8_0 : GRETA_FMT_F16; }

using Shape = TensorShard;

// Local shard of a projection under Megatron-style tensor parallelism: Q/K/V/gate/up are split by
// rows (output features), O and down by columns (input features, whole quant blocks).
Shape shard_of(const ModelConfig &c, LayerTensor t) { return tensor_shard(c, t); }
}  // namespace

TensorShard tensor_shard(const ModelConfig &c, LayerTensor t) {
  const uint32_t tp = c.tp_size, r = c.tp_rank;
  const uint32_t q = c.num_heads * c.head_dim, kv = c.num_heads_kv * c.head_dim;
  switch (t) {
    case LayerTensor::WQ: return {q / tp, c.dim, q, c.dim, r * (q / tp), 0};
    case LayerTensor::WK:
    case LayerTensor::WV: return {kv / tp, c.dim, kv, c.dim, r * (kv / tp), 0};
    case LayerTensor::WO: return {c.dim, q / tp, c.dim, q, 0, r * (q / tp)};
    case LayerTensor::W1_GATE:
    case LayerTensor::W3_UP: return {c.hidden_dim / tp, c.dim, c.hidden_dim, c.dim, r * (c.hidden_dim / tp), 0};
    case LayerTensor::W2_DOWN: return {c.dim, c.hidden_dim / tp, c.dim, c.hidden_dim, 0, r * (c.hidden_dim / tp)};
    default: return {c.dim, 1, c.dim, 1, 0, 0};
  }
}

namespace {
struct PlanePair {
  Buffer *qs, *d;
};

PlanePair planes(BlockBuffers &b, LayerTensor t) {
  switch (t) {
    case LayerTensor::WQ: return {&b.wq, &b.s_wq};
    case LayerTensor::WK: return {&b.wk, &b.s_wk};
    case LayerTensor::WV: return {&b.wv, &b.s_wv};
    case LayerTensor::WO: return {&b.wo, &b.s_wo};
    case LayerTensor::W1_GATE: return {&b.w1, &b.s_w1};
    case LayerTensor::W2_DOWN: return {&b.w2, &b.s_w2};
    default: return {&b.w3, &b.s_w3};
  }
}

inline cudaStream_t H(gcore::rt::GretaStream *s) { return static_cast<GretaStreamCuda *>(s)->handle(); }

#define GRETA_TRY(call, what)                                                     \
  do {                                                                            \
    if ((call) != GRETA_OK) return fail(err, gcore::host::cuda_error(what));      \
  } while (0)

}  // namespace

BlockScheduler::BlockScheduler() = default;
BlockScheduler::~BlockScheduler() {
  delete graph_;
  delete stream_;
}

bool BlockScheduler::init(const ModelConfig &config, std::string *err) {
  config_ = config;
  const ModelConfig &c = config_;
  if (c.tp_size == 0 || c.tp_rank >= c.tp_size) return fail(err, "init: bad tensor-parallel rank");
  if (c.dim % 256 || c.hidden_dim % (32 * c.tp_size) || c.num_heads % c.tp_size || c.num_heads_kv % c.tp_size ||
      c.num_heads % c.num_heads_kv || c.vocab_size % c.tp_size)
    return fail(err, "init: model shape is not divisible by the quant block / tensor-parallel degree");
  if (c.head_dim != 64 && c.head_dim != 128) return fail(err, "init: head_dim must be 64 or 128");
  if (c.weight_type != GretaDataType::Q4_0 && c.weight_type != GretaDataType::Q8_0) return fail(err, "init: weight_type must be Q4_0 or Q8_0");
  if (c.lm_head_type != GretaDataType::FP16 && c.lm_head_type != GretaDataType::Q4_0 && c.lm_head_type != GretaDataType::Q8_0)
    return fail(err, "init: lm_head_type must be FP16, Q4_0 or Q8_0");
  if (gcore::rt::GretaContext::instance().initialize() != gcore::rt::GretaResult::SUCCESS)
    return fail(err, "init: no usable CUDA device (this path has no CPU fallback)");
  heads_l_ = c.num_heads / c.tp_size;
  kv_heads_l_ = c.num_heads_kv / c.tp_size;
  hidden_l_ = c.hidden_dim / c.tp_size;
  vocab_l_ = c.vocab_size / c.tp_size;
  stream_ = gcore::rt::GretaContext::instance().create_stream();
  blocks_.clear();
  initialized_ = true;
  return true;
}

bool BlockScheduler::allocate_weights(std::string *err) {
  if (!initialized_) return fail(err, "allocate_weights: init() first");
  const ModelConfig &c = config_;
  const int fmt = fmt_of(c.weight_type);
  blocks_ = std::vector<BlockBuffers>(c.num_layers);
  weight_bytes_ = 0;
  for (auto &b : blocks_) {
    for (int t = 0; t <= (int)LayerTensor::W3_UP; ++t) {
      Shape s = shard_of(c, (LayerTensor)t);
      PlanePair p = planes(b, (LayerTensor)t);
      size_t qb = greta_cuda_qs_bytes(fmt, s.rows, s.cols), db = greta_cuda_d_bytes(fmt, s.rows, s.cols);
      if (!p.qs->allocate(qb, BufferUsage::DeviceOnly, c.weight_type, err)) return false;
      if (!p.d->allocate(db, BufferUsage::DeviceOnly, GretaDataType::FP16, err)) return false;
      GretaQuantInfo qi;
      qi.scales = p.d->data();
      qi.group_size = 32;
      p.qs->set_quant_info(qi);
      weight_bytes_ += qb + db;
    }
    if (!b.attn_norm.allocate((size_t)c.dim * 4, BufferUsage::DeviceOnly, GretaDataType::FP32, err)) return false;
    if (!b.ffn_norm.allocate((size_t)c.dim * 4, BufferUsage::DeviceOnly, GretaDataType::FP32, err)) return false;
  }
  if (!token_embd_.allocate((size_t)c.vocab_size * c.dim * 2, BufferUsage::DeviceOnly, GretaDataType::FP16, err)) return false;
  if (!output_norm_.allocate((size_t)c.dim * 4, BufferUsage::DeviceOnly, GretaDataType::FP32, err)) return false;
  if (c.lm_head_type == GretaDataType::FP16) {
    if (!output_weight_.allocate((size_t)vocab_l_ * c.dim * 2, BufferUsage::DeviceOnly, GretaDataType::FP16, err)) return false;
    weight_bytes_ += output_weight_.size();
  } else {
    const int lf = fmt_of(c.lm_head_type);
    if (!output_weight_.allocate(greta_cuda_qs_bytes(lf, vocab_l_, c.dim), BufferUsage::DeviceOnly, c.lm_head_type, err)) return false;
    if (!s_output_weight_.allocate(greta_cuda_d_bytes(lf, vocab_l_, c.dim), BufferUsage::DeviceOnly, GretaDataType::FP16, err)) return false;
    GretaQuantInfo qi;
    qi.scales = s_output_weight_.data();
    qi.group_size = 32;
    output_weight_.set_quant_info(qi);
    weight_bytes_ += output_weight_.size() + s_output_weight_.size();
  }
  return true;
}

bool BlockScheduler::allocate_activations(size_t batch_size, size_t max_seq_len, std::string *err) {
  if (!initialized_) return fail(err, "allocate_activations: init() first");
  // The reference runs one sequence (its cache has no batch dimension, block_scheduler.cpp:1490-1494).  Here up to 32
  // sequences decode in step, each with its own cache and position; prefill still runs one sequence at a time.
  if (batch_size < 1 || batch_size > 32) return fail(err, "allocate_activations: batch_size must be 1..32");
  const ModelConfig &c = config_;
  max_seq_ = max_seq_len;
  batch_ = (uint32_t)batch_size;
  cur_seq_ = 0;
  const size_t S = std::max(max_seq_len, batch_size), D = c.dim, B = batch_size;
  const size_t ql = (size_t)heads_l_ * c.head_dim, kvl = (size_t)kv_heads_l_ * c.head_dim;
  auto dev = [&](Buffer &b, size_t bytes, GretaDataType t = GretaDataType::FP32) { return b.allocate(bytes, BufferUsage::DeviceOnly, t, err); };
  ActivationBuffers &a = activations_;
  if (!dev(a.x, S * D * 4) || !dev(a.norm_out, S * D * 4) || !dev(a.q, S * ql * 4) || !dev(a.k, S * kvl * 4) || !dev(a.v, S * kvl * 4) ||
      !dev(a.attn_out, S * ql * 4) || !dev(a.mlp_gate, S * hidden_l_ * 4) || !dev(a.mlp_up, S * hidden_l_ * 4) || !dev(a.mlp_out, S * D * 4))
    return false;
  const size_t cache = (size_t)c.num_layers * B * kv_heads_l_ * max_seq_len * c.head_dim * 2;  // [L][B][Hkv][S][Dh] fp16
  if (!dev(a.kv_cache_k, cache, GretaDataType::FP16) || !dev(a.kv_cache_v, cache, GretaDataType::FP16)) return false;
  // d_pos: B positions, then B counts of ids produced; d_next: B token ids; out_tokens: [B][max_seq]
  if (!dev(a.tokens, S * 4) || !dev(a.d_pos, std::max<size_t>(16, 2 * B * 4)) || !dev(a.d_next, std::max<size_t>(16, B * 4)) ||
      !dev(a.out_tokens, B * max_seq_len * 4))
    return false;
  if (!dev(a.attn_scratch, greta_cuda_attn_decode_scratch_bytes((uint32_t)B * heads_l_, c.head_dim))) return false;
  if (!dev(a.gemm_ws, greta_cuda_gemm_workspace_bytes((uint32_t)max_seq_len, std::max(c.dim, c.hidden_dim)))) return false;
  if (!dev(logits_, B * (size_t)c.vocab_size * 4)) return false;
  if (B > 1 && c.tp_size > 1 && !dev(logits_local_, B * (size_t)vocab_l_ * 4)) return false;
  if (B > 1 && !dev(batch_ws_, greta_cuda_gemv_batch_workspace_bytes((uint32_t)B, std::max({c.dim, (uint32_t)ql, hidden_l_})))) return false;
  greta_cuda_memset(a.attn_scratch.data(), 0, a.attn_scratch.size(), nullptr);
  greta_cuda_memset(a.kv_cache_k.data(), 0, cache, nullptr);
  greta_cuda_memset(a.kv_cache_v.data(), 0, cache, nullptr);
  greta_cuda_memset(a.d_pos.data(), 0, a.d_pos.size(), nullptr);
  greta_cuda_memset(a.d_next.data(), 0, a.d_next.size(), nullptr);
  GRETA_TRY(greta_cuda_device_synchronize(), "allocate_activations");
  delete graph_;
  graph_ = nullptr;
  graph_captured_ = false;
  return true;
}

bool BlockScheduler::set_sequence(size_t seq, std::string *err) {
  if (seq >= batch_) return fail(err, "set_sequence: sequence index beyond the batch");
  cur_seq_ = (uint32_t)seq;
  return true;
}

// Uploads GGUF blocks of a [rows x cols] shard (host memory) and splits them into the planes.
static bool upload_blocks(GretaDataType type, const uint8_t *host, uint32_t rows, uint32_t cols, Buffer &qs, Buffer &d, Buffer &staging,
                          std::string *err) {
  const size_t bytes = (size_t)rows * (cols / 32) * block_bytes(type);
  if (staging.size() < bytes && !staging.allocate(bytes, BufferUsage::DeviceOnly, GretaDataType::INT8, err)) return false;
  GRETA_TRY(greta_cuda_memcpy_h2d_sync(staging.data(), host, bytes), "weight upload");
  GRETA_TRY(greta_cuda_repack_gguf(nullptr, fmt_of(type), staging.data(), qs.data(), d.data(), rows, cols), "repack_gguf");
  GRETA_TRY(greta_cuda_device_synchronize(), "repack_gguf");
  return true;
}

bool BlockScheduler::set_layer_tensor(size_t layer, LayerTensor which, const void *host, size_t bytes, std::string *err) {
  if (layer >= blocks_.size()) return fail(err, "set_layer_tensor: layer out of range (allocate_weights first)");
  BlockBuffers &b = blocks_[layer];
  if (which == LayerTensor::ATTN_NORM || which == LayerTensor::FFN_NORM) {
    Buffer &dst = which == LayerTensor::ATTN_NORM ? b.attn_norm : b.ffn_norm;
    if (bytes != dst.size()) return fail(err, "set_layer_tensor: norm size mismatch");
    return dst.copy_to_device(host, bytes, err);
  }
  // `host` holds the GLOBAL tensor as GGUF blocks; this rank keeps its shard.
  const ModelConfig &c = config_;
  Shape s = shard_of(c, which);
  const size_t bb = block_bytes(c.weight_type);
  if (bytes != (size_t)s.grows * (s.gcols / 32) * bb) return fail(err, "set_layer_tensor: byte size does not match the global tensor shape");
  PlanePair p = planes(b, which);
  Buffer staging;
  const uint8_t *src = static_cast<const uint8_t *>(host);
  if (s.rows == s.grows && s.cols == s.gcols) return upload_blocks(c.weight_type, src, s.rows, s.cols, *p.qs, *p.d, staging, err);
  std::vector<uint8_t> local((size_t)s.rows * (s.cols / 32) * bb);
  const size_t grow_b = (size_t)(s.gcols / 32) * bb, lrow_b = (size_t)(s.cols / 32) * bb;
  for (uint32_t r = 0; r < s.rows; ++r)
    std::memcpy(local.data() + r * lrow_b, src + (size_t)(s.row0 + r) * grow_b + (size_t)(s.col0 / 32) * bb, lrow_b);
  return upload_blocks(c.weight_type, local.data(), s.rows, s.cols, *p.qs, *p.d, staging, err);
}

// K-quant rows [row0, row0 + rows) of a [grows x gcols] tensor -> Q8_0 planes of the column range [col0, col0 + cols).
// Whole rows are converted on the device (a column range need not be whole super-blocks), then the range is copied out.
static bool upload_kquant(int ggml_type, const uint8_t *host, uint32_t gcols, uint32_t row0, uint32_t rows, uint32_t col0, uint32_t cols, Buffer &qs,
                          Buffer &d, std::string *err) {
  if (gcols % 256) return fail(err, "K-quant tensor: row length is not a multiple of the super-block size 256");
  const size_t row_b = greta_cuda_kquant_bytes(ggml_type, gcols);
  if (row_b == 0) return fail(err, "K-quant tensor: GGML type is not Q4_K or Q6_K");
  Buffer staging, fq, fd;
  if (!staging.allocate(rows * row_b, BufferUsage::DeviceOnly, GretaDataType::INT8, err)) return false;
  GRETA_TRY(greta_cuda_memcpy_h2d_sync(staging.data(), host + (size_t)row0 * row_b, rows * row_b), "weight upload");
  if (cols == gcols) {
    GRETA_TRY(greta_cuda_kquant_to_q8_0(nullptr, ggml_type, staging.data(), qs.data(), d.data(), rows, cols), "kquant_to_q8_0");
    GRETA_TRY(greta_cuda_device_synchronize(), "kquant_to_q8_0");
    return true;
  }
  const int f = GRETA_FMT_Q8_0;
  if (!fq.allocate(greta_cuda_qs_bytes(f, rows, gcols), BufferUsage::DeviceOnly, GretaDataType::INT8, err)) return false;
  if (!fd.allocate(greta_cuda_d_bytes(f, rows, gcols), BufferUsage::DeviceOnly, GretaDataType::FP16, err)) return false;
  GRETA_TRY(greta_cuda_kquant_to_q8_0(nullptr, ggml_type, staging.data(), fq.data(), fd.data(), rows, gcols), "kquant_to_q8_0");
  GRETA_TRY(greta_cuda_memcpy_2d_d2d(qs.data(), (size_t)cols, static_cast<const uint8_t *>(fq.data()) + col0, (size_t)gcols, (size_t)cols, rows, nullptr),
            "shard copy");
  GRETA_TRY(greta_cuda_memset(d.data(), 0, greta_cuda_d_bytes(f, rows, cols), nullptr), "shard copy");  // row padding of the scale plane
  GRETA_TRY(greta_cuda_memcpy_2d_d2d(d.data(), greta_cuda_d_bytes(f, 1, cols), static_cast<const uint8_t *>(fd.data()) + (size_t)(col0 / 32) * 2,
                                     greta_cuda_d_bytes(f, 1, gcols), (size_t)(cols / 32) * 2, rows, nullptr),
            "shard copy");
  GRETA_TRY(greta_cuda_device_synchronize(), "shard copy");
  return true;
}

bool BlockScheduler::set_layer_tensor_kquant(size_t layer, LayerTensor which, int ggml_type, const void *host, size_t bytes, std::string *err) {
  if (layer >= blocks_.size()) return fail(err, "set_layer_tensor_kquant: layer out of range (allocate_weights first)");
  if (which == LayerTensor::ATTN_NORM || which == LayerTensor::FFN_NORM) return fail(err, "set_layer_tensor_kquant: norm weights are plain floats");
  const ModelConfig &c = config_;
  if (c.weight_type != GretaDataType::Q8_0) return fail(err, "set_layer_tensor_kquant: K-quant tensors are re-stored as Q8_0; initialise the scheduler with weight_type Q8_0");
  Shape s = shard_of(c, which);
  if (bytes != (size_t)s.grows * greta_cuda_kquant_bytes(ggml_type, s.gcols) || bytes == 0)
    return fail(err, "set_layer_tensor_kquant: byte size does not match the global tensor shape");
  PlanePair p = planes(blocks_[layer], which);
  return upload_kquant(ggml_type, static_cast<const uint8_t *>(host), s.gcols, s.row0, s.rows, s.col0, s.cols, *p.qs, *p.d, err);
}

bool BlockScheduler::set_global_tensor_kquant(GlobalTensor which, int ggml_type, const void *host, size_t bytes, std::string *err) {
  const ModelConfig &c = config_;
  if (which != GlobalTensor::OUT_WEIGHT) return fail(err, "set_global_tensor_kquant: only the LM head is kept quantised");
  if (c.lm_head_type != GretaDataType::Q8_0) return fail(err, "set_global_tensor_kquant: a K-quant LM head is re-stored as Q8_0; set lm_head_type to Q8_0");
  if (bytes != (size_t)c.vocab_size * greta_cuda_kquant_bytes(ggml_type, c.dim) || bytes == 0)
    return fail(err, "set_global_tensor_kquant: LM head size mismatch");
  return upload_kquant(ggml_type, static_cast<const uint8_t *>(host), c.dim, c.tp_rank * vocab_l_, vocab_l_, 0, c.dim, output_weight_, s_output_weight_, err);
}

bool BlockScheduler::set_global_tensor(GlobalTensor which, const void *host, size_t bytes, std::string *err) {
  const ModelConfig &c = config_;
  if (which == GlobalTensor::TOK_EMBD) {
    if (bytes != token_embd_.size()) return fail(err, "set_global_tensor: embedding size mismatch");
    return token_embd_.copy_to_device(host, bytes, err);
  }
  if (which == GlobalTensor::OUT_NORM) {
    if (bytes != output_norm_.size()) return fail(err, "set_global_tensor: norm size mismatch");
    return output_norm_.copy_to_device(host, bytes, err);
  }
  const uint8_t *src = static_cast<const uint8_t *>(host);
  if (c.lm_head_type == GretaDataType::FP16) {
    if (bytes != (size_t)c.vocab_size * c.dim * 2) return fail(err, "set_global_tensor: LM head size mismatch");
    return output_weight_.copy_to_device(src + (size_t)c.tp_rank * vocab_l_ * c.dim * 2, output_weight_.size(), err);
  }
  const size_t row_b = (size_t)(c.dim / 32) * block_bytes(c.lm_head_type);
  if (bytes != (size_t)c.vocab_size * row_b) return fail(err, "set_global_tensor: LM head size mismatch");
  Buffer staging;
  return upload_blocks(c.lm_head_type, src + (size_t)c.tp_rank * vocab_l_ * row_b, vocab_l_, c.dim, output_weight_, s_output_weight_, staging, err);
}

bool BlockScheduler::load_synthetic_weights(uint64_t seed, std::string *err) {
  if (blocks_.empty()) return fail(err, "load_synthetic_weights: allocate_weights first");
  const ModelConfig &c = config_;
  const size_t bb = block_bytes(c.weight_type);
  Buffer staging;
  std::vector<uint8_t> hostbuf;
  std::vector<float> norm(c.dim);
  for (uint32_t l = 0; l < c.num_layers; ++l) {
    BlockBuffers &b = blocks_[l];
    for (int t = 0; t <= (int)LayerTensor::W3_UP; ++t) {
      Shape s = shard_of(c, (LayerTensor)t);
      const size_t nb_l = s.cols / 32, nb_g = s.gcols / 32;
      hostbuf.resize((size_t)s.rows * nb_l * bb);
      const uint64_t stream = synth::tensor_stream(l, t);
      if (s.cols == s.gcols) {
        synth::quant_blocks(seed, stream, c.weight_type, hostbuf.data(), (size_t)s.row0 * nb_g, (size_t)s.rows * nb_g);
      } else {
        for (uint32_t r = 0; r < s.rows; ++r)
          synth::quant_blocks(seed, stream, c.weight_type, hostbuf.data() + (size_t)r * nb_l * bb, (size_t)r * nb_g + s.col0 / 32, nb_l);
      }
      PlanePair p = planes(b, (LayerTensor)t);
      if (!upload_blocks(c.weight_type, hostbuf.data(), s.rows, s.cols, *p.qs, *p.d, staging, err)) return false;
    }
    synth::normal_f16_as_f32(seed, synth::tensor_stream(l, (int)LayerTensor::ATTN_NORM), 0.02f, norm.data(), 0, c.dim);
    if (!b.attn_norm.copy_to_device(norm.data(), (size_t)c.dim * 4, err)) return false;
    synth::normal_f16_as_f32(seed, synth::tensor_stream(l, (int)LayerTensor::FFN_NORM), 0.02f, norm.data(), 0, c.dim);
    if (!b.ffn_norm.copy_to_device(norm.data(), (size_t)c.dim * 4, err)) return false;
  }
  const uint32_t G = c.num_layers;  // global tensors use the layer index one past the last layer
  {
    std::vector<uint16_t> emb((size_t)c.vocab_size * c.dim);
    synth::normal_f16(seed, synth::tensor_stream(G, (int)GlobalTensor::TOK_EMBD), 0.02f, emb.data(), 0, emb.size());
    if (!token_embd_.copy_to_device(emb.data(), emb.size() * 2, err)) return false;
  }
  synth::normal_f16_as_f32(seed, synth::tensor_stream(G, (int)GlobalTensor::OUT_NORM), 0.02f, norm.data(), 0, c.dim);
  if (!output_norm_.copy_to_device(norm.data(), (size_t)c.dim * 4, err)) return false;
  const uint64_t so = synth::tensor_stream(G, (int)GlobalTensor::OUT_WEIGHT);
  if (c.lm_head_type == GretaDataType::FP16) {
    std::vector<uint16_t> w((size_t)vocab_l_ * c.dim);
    synth::normal_f16(seed, so, 0.02f, w.data(), (size_t)c.tp_rank * vocab_l_ * c.dim, w.size());
    if (!output_weight_.copy_to_device(w.data(), w.size() * 2, err)) return false;
  } else {
    const size_t nb = c.dim / 32, lb = block_bytes(c.lm_head_type);
    hostbuf.resize((size_t)vocab_l_ * nb * lb);
    synth::quant_blocks(seed, so, c.lm_head_type, hostbuf.data(), (size_t)c.tp_rank * vocab_l_ * nb, (size_t)vocab_l_ * nb);
    if (!upload_blocks(c.lm_head_type, hostbuf.data(), vocab_l_, c.dim, output_weight_, s_output_weight_, staging, err)) return false;
  }
  return true;
}

// ------------------------------------------------------------------ forward
// Final norm + LM head on one hidden row -> logits_ (full vocabulary on every rank).
bool BlockScheduler::lm_head(const float *x_row, std::string *err) {
  const ModelConfig &c = config_;
  cudaStream_t s = H(stream_);
  float *dst = static_cast<float *>(logits_.data()) + (size_t)c.tp_rank * vocab_l_;
  const int lf = fmt_of(c.lm_head_type);
  GRETA_TRY(greta_cuda_rmsnorm_gemv(s, lf, x_row, static_cast<const float *>(output_norm_.data()), c.rms_eps, output_weight_.data(),
                                    lf == GRETA_FMT_F16 ? nullptr : s_output_weight_.data(), dst, vocab_l_, c.dim),
            "lm head");
  if (c.tp_size > 1) {
    // every rank wrote its own slice of a zeroed buffer: a sum over ranks is the gather
    if (!all_reduce_) return fail(err, "tensor parallel run without an all-reduce hook");
    if (all_reduce_(static_cast<float *>(logits_.data()), c.vocab_size, s) != 0) return fail(err, "all-reduce of the logits failed");
  }
  return true;
}

bool BlockScheduler::set_peer_exchange(const greta_peer_exchange &ex, std::string *err) {
  const ModelConfig &c = config_;
  if (ex.tp != c.tp_size || ex.rank != c.tp_rank) return fail(err, "set_peer_exchange: group does not match the model's tensor-parallel rank");
  if (c.dim > 8192 || 2 * c.num_layers > 256) return fail(err, "set_peer_exchange: model too large for the exchange tags");
  if (!all_reduce_) return fail(err, "set_peer_exchange: install the all-reduce hook first (barriers, last layer, logits)");
  if (!x_alt_.allocate((size_t)c.dim * 4, BufferUsage::DeviceOnly, GretaDataType::FP32, err)) return false;
  const size_t least = greta_cuda_peer_slot_bytes(ex.tp, c.dim);
  if (ex.slot_bytes != 0 && ex.slot_bytes < least) return fail(err, "set_peer_exchange: slot buffers are smaller than greta_cuda_peer_slot_bytes(tp, dim)");
  peer_ = ex;
  if (peer_.slot_bytes == 0) peer_.slot_bytes = least;
  invalidate_graph();  // a captured step holds the old exchange's pointers
  return true;
}

void BlockScheduler::set_all_reduce(AllReduceFn fn) {
  all_reduce_ = std::move(fn);
  invalidate_graph();
}

void BlockScheduler::invalidate_graph() {
  if (graph_) greta_cuda_stream_synchronize(H(stream_));
  delete graph_;
  graph_ = nullptr;
  graph_captured_ = false;
}

// The five decode kernels of every layer, reading the position from d_pos.  With fused_exchange the
// row-parallel projections scatter their partial products into every rank's slots and the next operator
// sums them while it stages its input; the residual stream then alternates between two buffers and
// *x_final tells where the last layer left it.  The last down-projection keeps the all-reduce: the LM head
// that follows is not an exchange consumer.
bool BlockScheduler::decode_layers(std::string *err, bool fused_exchange, const float **x_final) {
  const ModelConfig &c = config_;
  ActivationBuffers &a = activations_;
  cudaStream_t s = H(stream_);
  const int fmt = fmt_of(c.weight_type);
  const uint32_t D = c.dim, Dh = c.head_dim, ql = heads_l_ * Dh;
  const float scale = 1.0f / std::sqrt((float)Dh);
  const size_t cache_l = (size_t)kv_heads_l_ * max_seq_ * Dh;  // elements per layer
  const uint32_t *dpos = static_cast<const uint32_t *>(a.d_pos.data());
  float *x = static_cast<float *>(a.x.data());
  const bool tp = c.tp_size > 1;
  if (fused_exchange) {
    if (!tp || peer_.tp != c.tp_size) return fail(err, "decode_layers: no peer exchange installed");
    float *cur = x, *other = static_cast<float *>(x_alt_.data());
    for (uint32_t l = 0; l < c.num_layers; ++l) {
      BlockBuffers &b = blocks_[l];
      uint16_t *kc = static_cast<uint16_t *>(a.kv_cache_k.data()) + l * cache_l;
      uint16_t *vc = static_cast<uint16_t *>(a.kv_cache_v.data()) + l * cache_l;
      if (l == 0) {
        GRETA_TRY(greta_cuda_fused_rmsnorm_qkv_rope_kv(s, fmt, cur, static_cast<const float *>(b.attn_norm.data()), c.rms_eps, b.wq.data(),
                                                       b.s_wq.data(), b.wk.data(), b.s_wk.data(), b.wv.data(), b.s_wv.data(),
                                                       static_cast<float *>(a.q.data()), nullptr, nullptr, kc, vc, dpos, heads_l_, kv_heads_l_,
                                                       Dh, (uint32_t)max_seq_, c.rope_base, D),
                  "fused qkv");
      } else {  // consumes the down-projection partials of layer l - 1
        GRETA_TRY(greta_cuda_fused_rmsnorm_qkv_rope_kv_peer(s, fmt, cur, other, &peer_, 2 * l - 1, static_cast<const float *>(b.attn_norm.data()),
                                                            c.rms_eps, b.wq.data(), b.s_wq.data(), b.wk.data(), b.s_wk.data(), b.wv.data(),
                                                            b.s_wv.data(), static_cast<float *>(a.q.data()), kc, vc, dpos, heads_l_, kv_heads_l_,
                                                            Dh, (uint32_t)max_seq_, c.rope_base, D),
                  "fused qkv (exchange)");
        std::swap(cur, other);
      }
      GRETA_TRY(greta_cuda_attn_decode(s, static_cast<const float *>(a.q.data()), kc, vc, static_cast<float *>(a.attn_out.data()), dpos, 0, heads_l_,
                                       kv_heads_l_, Dh, (uint32_t)max_seq_, scale, a.attn_scratch.data(), a.attn_scratch.size()),
                "attention decode");
      GRETA_TRY(greta_cuda_gemv_peer_scatter(s, fmt, static_cast<const float *>(a.attn_out.data()), b.wo.data(), b.s_wo.data(), &peer_, 2 * l, dpos, D,
                                             ql),
                "wo (exchange)");
      GRETA_TRY(greta_cuda_fused_ffn_front_peer(s, fmt, cur, other, &peer_, 2 * l, dpos, static_cast<const float *>(b.ffn_norm.data()), c.rms_eps,
                                                b.w1.data(), b.s_w1.data(), b.w3.data(), b.s_w3.data(), static_cast<float *>(a.mlp_gate.data()), D,
                                                hidden_l_),
                "ffn front (exchange)");
      std::swap(cur, other);
      if (l + 1 < c.num_layers) {
        GRETA_TRY(greta_cuda_gemv_peer_scatter(s, fmt, static_cast<const float *>(a.mlp_gate.data()), b.w2.data(), b.s_w2.data(), &peer_, 2 * l + 1,
                                               dpos, D, hidden_l_),
                  "w2 (exchange)");
      } else {
        if (c.tp_rank == 0)
          GRETA_TRY(greta_cuda_gemv_residual(s, fmt, static_cast<const float *>(a.mlp_gate.data()), b.w2.data(), b.s_w2.data(), cur, cur, D, hidden_l_),
                    "w2");
        else
          GRETA_TRY(greta_cuda_gemv(s, fmt, a.mlp_gate.data(), 0, b.w2.data(), b.s_w2.data(), cur, 1, D, hidden_l_), "w2");
        if (all_reduce_(cur, D, s) != 0) return fail(err, "all-reduce after the last down-projection failed");
      }
    }
    if (x_final) *x_final = cur;
    return true;
  }
  if (x_final) *x_final = x;
  for (uint32_t l = 0; l < c.num_layers; ++l) {
    BlockBuffers &b = blocks_[l];
    uint16_t *kc = static_cast<uint16_t *>(a.kv_cache_k.data()) + l * cache_l;
    uint16_t *vc = static_cast<uint16_t *>(a.kv_cache_v.data()) + l * cache_l;
    GRETA_TRY(greta_cuda_fused_rmsnorm_qkv_rope_kv(s, fmt, x, static_cast<const float *>(b.attn_norm.data()), c.rms_eps, b.wq.data(),
                                                   b.s_wq.data(), b.wk.data(), b.s_wk.data(), b.wv.data(), b.s_wv.data(),
                                                   static_cast<float *>(a.q.data()), nullptr, nullptr, kc, vc, dpos, heads_l_, kv_heads_l_, Dh,
                                                   (uint32_t)max_seq_, c.rope_base, D),
              "fused qkv");
    GRETA_TRY(greta_cuda_attn_decode(s, static_cast<const float *>(a.q.data()), kc, vc, static_cast<float *>(a.attn_out.data()), dpos, 0, heads_l_,
                                     kv_heads_l_, Dh, (uint32_t)max_seq_, scale, a.attn_scratch.data(), a.attn_scratch.size()),
              "attention decode");
    // Row-parallel projections under TP: rank 0 folds the residual in, the others overwrite their copy
    // of x with their partial product; the all-reduce then leaves x + sum of partials on every rank.
    if (!tp || c.tp_rank == 0)
      GRETA_TRY(greta_cuda_gemv_residual(s, fmt, static_cast<const float *>(a.attn_out.data()), b.wo.data(), b.s_wo.data(), x, x, D, ql), "wo");
    else
      GRETA_TRY(greta_cuda_gemv(s, fmt, a.attn_out.data(), 0, b.wo.data(), b.s_wo.data(), x, 1, D, ql), "wo");
    if (tp && all_reduce_(x, D, s) != 0) return fail(err, "all-reduce after the O-projection failed");
    GRETA_TRY(greta_cuda_fused_ffn_front(s, fmt, x, static_cast<const float *>(b.ffn_norm.data()), c.rms_eps, b.w1.data(), b.s_w1.data(),
                                         b.w3.data(), b.s_w3.data(), static_cast<float *>(a.mlp_gate.data()), D, hidden_l_),
              "ffn front");
    if (!tp || c.tp_rank == 0)
      GRETA_TRY(greta_cuda_gemv_residual(s, fmt, static_cast<const float *>(a.mlp_gate.data()), b.w2.data(), b.s_w2.data(), x, x, D, hidden_l_),
                "w2");
    else
      GRETA_TRY(greta_cuda_gemv(s, fmt, a.mlp_gate.data(), 0, b.w2.data(), b.s_w2.data(), x, 1, D, hidden_l_), "w2");
    if (tp && all_reduce_(x, D, s) != 0) return fail(err, "all-reduce after the down-projection failed");
  }
  return true;
}

// The decode step of a batch: the same five kernels per layer in their batched forms (weights streamed once for all
// sequences, every sequence at its own position).  Under tensor parallelism the partial products of the row-parallel
// projections are summed by the all-reduce hook over [batch x dim].
bool BlockScheduler::decode_layers_batch(std::string *err) {
  const ModelConfig &c = config_;
  ActivationBuffers &a = activations_;
  cudaStream_t s = H(stream_);
  const int fmt = fmt_of(c.weight_type);
  const uint32_t D = c.dim, Dh = c.head_dim, ql = heads_l_ * Dh, B = batch_;
  const float scale = 1.0f / std::sqrt((float)Dh);
  const size_t cache_l = (size_t)B * kv_heads_l_ * max_seq_ * Dh;  // elements per layer: [B][Hkv][S][Dh]
  const uint32_t *dpos = static_cast<const uint32_t *>(a.d_pos.data());
  float *x = static_cast<float *>(a.x.data()), *q = static_cast<float *>(a.q.data()), *att = static_cast<float *>(a.attn_out.data());
  float *gate = static_cast<float *>(a.mlp_gate.data());
  const bool tp = c.tp_size > 1, fold = !tp || c.tp_rank == 0;  // one rank folds the residual in, the others contribute bare partials
  void *ws = batch_ws_.data();  // prepared activations of the operator in flight (one buffer serves them all: stream order)
  // With slot buffers large enough for [batch x dim] the sums over the ranks go through peer memory (one kernel per rank);
  // the logits gather and the prefill keep the all-reduce hook, which also separates one step's exchanges from the next's.
  const bool peer_ar = tp && peer_.tp == c.tp_size && peer_.slot_bytes >= greta_cuda_peer_allreduce_slot_bytes((size_t)B * D) && 2 * c.num_layers <= 256;
  for (uint32_t l = 0; l < c.num_layers; ++l) {
    BlockBuffers &b = blocks_[l];
    uint16_t *kc = static_cast<uint16_t *>(a.kv_cache_k.data()) + l * cache_l;
    uint16_t *vc = static_cast<uint16_t *>(a.kv_cache_v.data()) + l * cache_l;
    GRETA_TRY(greta_cuda_fused_rmsnorm_qkv_rope_kv_batch(s, fmt, x, static_cast<const float *>(b.attn_norm.data()), c.rms_eps, b.wq.data(),
                                                         b.s_wq.data(), b.wk.data(), b.s_wk.data(), b.wv.data(), b.s_wv.data(), q, nullptr, nullptr,
                                                         kc, vc, dpos, B, heads_l_, kv_heads_l_, Dh, (uint32_t)max_seq_, c.rope_base, D, ws),
              "fused qkv (batch)");
    GRETA_TRY(greta_cuda_attn_decode_batch(s, q, kc, vc, att, dpos, B, heads_l_, kv_heads_l_, Dh, (uint32_t)max_seq_, scale, a.attn_scratch.data(),
                                           a.attn_scratch.size()),
              "attention decode (batch)");
    GRETA_TRY(greta_cuda_gemv_batch(s, fmt, att, nullptr, 0.f, b.wo.data(), b.s_wo.data(), fold ? x : nullptr, x, B, D, ql, 0, ws), "wo (batch)");
    if (peer_ar) {
      GRETA_TRY(greta_cuda_peer_allreduce_f32(s, x, (size_t)B * D, &peer_, 2 * l, dpos), "exchange after the O-projection");
    } else if (tp && all_reduce_(x, (size_t)B * D, s) != 0) {
      return fail(err, "all-reduce after the O-projection failed");
    }
    GRETA_TRY(greta_cuda_fused_ffn_front_batch(s, fmt, x, static_cast<const float *>(b.ffn_norm.data()), c.rms_eps, b.w1.data(), b.s_w1.data(),
                                               b.w3.data(), b.s_w3.data(), gate, B, D, hidden_l_, ws),
              "ffn front (batch)");
    GRETA_TRY(greta_cuda_gemv_batch(s, fmt, gate, nullptr, 0.f, b.w2.data(), b.s_w2.data(), fold ? x : nullptr, x, B, D, hidden_l_, 0, ws), "w2 (batch)");
    if (peer_ar) {
      GRETA_TRY(greta_cuda_peer_allreduce_f32(s, x, (size_t)B * D, &peer_, 2 * l + 1, dpos), "exchange after the down-projection");
    } else if (tp && all_reduce_(x, (size_t)B * D, s) != 0) {
      return fail(err, "all-reduce after the down-projection failed");
    }
  }
  return true;
}

// Final norm + LM head for every sequence of the batch -> logits_ [B][vocab] (full vocabulary on every rank).
bool BlockScheduler::lm_head_batch(std::string *err) {
  const ModelConfig &c = config_;
  cudaStream_t s = H(stream_);
  const int lf = fmt_of(c.lm_head_type);
  const float *x = static_cast<const float *>(activations_.x.data());
  const void *d = lf == GRETA_FMT_F16 ? nullptr : s_output_weight_.data();
  float *logits = static_cast<float *>(logits_.data());
  if (c.tp_size == 1) {
    GRETA_TRY(greta_cuda_gemv_batch(s, lf, x, static_cast<const float *>(output_norm_.data()), c.rms_eps, output_weight_.data(), d, nullptr, logits,
                                    batch_, c.vocab_size, c.dim, 0, batch_ws_.data()),
              "lm head (batch)");
    return true;
  }
  // every rank computes its slice of the vocabulary, places it in a zeroed [B][vocab] buffer; the sum over ranks is the gather
  if (!all_reduce_) return fail(err, "tensor parallel run without an all-reduce hook");
  float *local = static_cast<float *>(logits_local_.data());
  GRETA_TRY(greta_cuda_gemv_batch(s, lf, x, static_cast<const float *>(output_norm_.data()), c.rms_eps, output_weight_.data(), d, nullptr, local,
                                  batch_, vocab_l_, c.dim, 0, batch_ws_.data()),
            "lm head (batch)");
  GRETA_TRY(greta_cuda_memcpy_2d_d2d(logits + (size_t)c.tp_rank * vocab_l_, (size_t)c.vocab_size * 4, local, (size_t)vocab_l_ * 4,
                                     (size_t)vocab_l_ * 4, batch_, s),
            "logits placement");
  if (all_reduce_(logits, (size_t)batch_ * c.vocab_size, s) != 0) return fail(err, "all-reduce of the logits failed");
  return true;
}

bool BlockScheduler::execute_layer(size_t layer_idx, size_t seq_start, size_t seq_len, const int32_t *, std::string *err) {
  // Prefill form of one layer over S = seq_len rows (the reference's operator order,
  // block_scheduler.cpp:1814-3032), projections through GretaCompute-style routing: GEMV for
  // S <= 32, tensor-core GEMM above.
  const ModelConfig &c = config_;
  ActivationBuffers &a = activations_;
  if (layer_idx >= blocks_.size()) return fail(err, "execute_layer: layer out of range");
  BlockBuffers &b = blocks_[layer_idx];
  cudaStream_t s = H(stream_);
  const int fmt = fmt_of(c.weight_type);
  const uint32_t S = (uint32_t)seq_len, D = c.dim, Dh = c.head_dim, ql = heads_l_ * Dh, kvl = kv_heads_l_ * Dh;
  const float scale = 1.0f / std::sqrt((float)Dh);
  const size_t cache_s = (size_t)kv_heads_l_ * max_seq_ * Dh;  // one sequence's cache of one layer
  uint16_t *kc = static_cast<uint16_t *>(a.kv_cache_k.data()) + (layer_idx * batch_ + cur_seq_) * cache_s;
  uint16_t *vc = static_cast<uint16_t *>(a.kv_cache_v.data()) + (layer_idx * batch_ + cur_seq_) * cache_s;
  float *x = static_cast<float *>(a.x.data()), *nrm = static_cast<float *>(a.norm_out.data());
  float *q = static_cast<float *>(a.q.data()), *k = static_cast<float *>(a.k.data()), *v = static_cast<float *>(a.v.data());
  float *att = static_cast<float *>(a.attn_out.data()), *gate = static_cast<float *>(a.mlp_gate.data()), *up = static_cast<float *>(a.mlp_up.data());
  float *tmp = static_cast<float *>(a.mlp_out.data());
  const bool tp = c.tp_size > 1;
  auto proj = [&](const float *in, Buffer &w, Buffer &sw, float *out, uint32_t N, uint32_t K) -> int {
    if (S <= 32) return greta_cuda_gemv(s, fmt, in, 0, w.data(), sw.data(), out, S, N, K);
    return greta_cuda_gemm(s, fmt, in, 0, w.data(), sw.data(), out, 0, S, N, K, a.gemm_ws.data());
  };
  GRETA_TRY(greta_cuda_rmsnorm(s, x, static_cast<const float *>(b.attn_norm.data()), nrm, S, D, c.rms_eps), "rmsnorm");
  GRETA_TRY(proj(nrm, b.wq, b.s_wq, q, ql, D), "wq");
  GRETA_TRY(proj(nrm, b.wk, b.s_wk, k, kvl, D), "wk");
  GRETA_TRY(proj(nrm, b.wv, b.s_wv, v, kvl, D), "wv");
  GRETA_TRY(greta_cuda_rope(s, q, S, heads_l_, Dh, c.rope_base, (uint32_t)seq_start, nullptr), "rope q");
  GRETA_TRY(greta_cuda_rope(s, k, S, kv_heads_l_, Dh, c.rope_base, (uint32_t)seq_start, nullptr), "rope k");
  GRETA_TRY(greta_cuda_kv_update(s, kc, vc, k, v, S, (uint32_t)seq_start, nullptr, (uint32_t)max_seq_, kv_heads_l_, Dh), "kv update");
  GRETA_TRY(greta_cuda_attn_prefill(s, q, kc, vc, att, S, (uint32_t)seq_start, heads_l_, kv_heads_l_, Dh, (uint32_t)max_seq_, scale), "attention");
  GRETA_TRY(proj(att, b.wo, b.s_wo, tmp, D, ql), "wo");
  if (tp && all_reduce_(tmp, (size_t)S * D, s) != 0) return fail(err, "all-reduce failed");
  GRETA_TRY(greta_cuda_add(s, x, tmp, x, (size_t)S * D), "residual");
  GRETA_TRY(greta_cuda_rmsnorm(s, x, static_cast<const float *>(b.ffn_norm.data()), nrm, S, D, c.rms_eps), "rmsnorm");
  GRETA_TRY(proj(nrm, b.w1, b.s_w1, gate, hidden_l_, D), "w1");
  GRETA_TRY(proj(nrm, b.w3, b.s_w3, up, hidden_l_, D), "w3");
  GRETA_TRY(greta_cuda_silu_mul(s, gate, up, gate, (size_t)S * hidden_l_), "swiglu");
  GRETA_TRY(proj(gate, b.w2, b.s_w2, tmp, D, hidden_l_), "w2");
  if (tp && all_reduce_(tmp, (size_t)S * D, s) != 0) return fail(err, "all-reduce failed");
  GRETA_TRY(greta_cuda_add(s, x, tmp, x, (size_t)S * D), "residual");
  return true;
}

bool BlockScheduler::forward(const int32_t *tokens, size_t seq_start, size_t seq_len, std::string *err) {
  if (blocks_.empty() || !activations_.x.data()) return fail(err, "forward: allocate weights and activations first");
  if (seq_len == 0 || seq_start + seq_len > max_seq_) return fail(err, "forward: sequence exceeds max_seq_len");
  if (config_.tp_size > 1 && !all_reduce_) return fail(err, "forward: tensor-parallel run without an all-reduce hook");
  const ModelConfig &c = config_;
  ActivationBuffers &a = activations_;
  cudaStream_t s = H(stream_);
  GRETA_TRY(greta_cuda_memcpy_h2d(a.tokens.data(), tokens, seq_len * 4, s), "token upload");
  GRETA_TRY(greta_cuda_embedding(s, static_cast<const int32_t *>(a.tokens.data()), token_embd_.data(), 1, static_cast<float *>(a.x.data()),
                                 (uint32_t)seq_len, c.dim, c.vocab_size),
            "embedding");
  if (c.tp_size > 1) GRETA_TRY(greta_cuda_memset(logits_.data(), 0, logits_.size(), s), "logits clear");
  if (seq_len == 1 && batch_ == 1) {
    uint32_t pos = (uint32_t)seq_start;
    GRETA_TRY(greta_cuda_memcpy_h2d(a.d_pos.data(), &pos, 4, s), "position upload");
    GRETA_TRY(greta_cuda_stream_synchronize(s), "position upload");  // `pos` lives on this stack frame
    if (!decode_layers(err)) return false;
  } else {  // prefill form, on the current sequence's cache (also a single token when the scheduler holds a batch)
    for (size_t l = 0; l < blocks_.size(); ++l)
      if (!execute_layer(l, seq_start, seq_len, tokens, err)) return false;
  }
  if (!lm_head(static_cast<const float *>(a.x.data()) + (seq_len - 1) * c.dim, err)) return false;
  GRETA_TRY(greta_cuda_stream_synchronize(s), "forward");
  return true;
}

int32_t BlockScheduler::sample_greedy_gpu(size_t logits_offset_bytes, std::string *err) {
  int32_t id = -1;
  gcore::rt::cuda::kernels::launch_argmax(H(stream_), static_cast<const float *>(logits_.data()) + logits_offset_bytes / 4, config_.vocab_size, &id);
  if (gcore::rt::cuda::kernels::last_launch_error() && err) *err = gcore::rt::cuda::kernels::last_launch_error_string();
  return id;
}

// Describes the model to the persistent decode-step kernel (single GPU only).
static void fill_decode_desc(greta_decode_desc &d, const ModelConfig &c, ActivationBuffers &a, Buffer &embd, size_t max_seq) {
  d = greta_decode_desc{};
  d.weight_fmt = fmt_of(c.weight_type);
  d.dim = c.dim; d.num_heads = c.num_heads; d.num_heads_kv = c.num_heads_kv; d.head_dim = c.head_dim; d.hidden_dim = c.hidden_dim;
  d.max_seq_len = (uint32_t)max_seq; d.num_layers = c.num_layers; d.vocab_size = c.vocab_size;
  d.rope_base = c.rope_base; d.rms_eps = c.rms_eps; d.attn_scale = 1.0f / std::sqrt((float)c.head_dim);
  d.x = static_cast<float *>(a.x.data()); d.q = static_cast<float *>(a.q.data());
  d.attn_out = static_cast<float *>(a.attn_out.data()); d.mlp_gate = static_cast<float *>(a.mlp_gate.data());
  d.d_pos = static_cast<const uint32_t *>(a.d_pos.data()); d.d_token = static_cast<const int32_t *>(a.d_next.data());
  d.tok_embd_f16 = embd.data(); d.attn_scratch = a.attn_scratch.data(); d.attn_scratch_bytes = a.attn_scratch.size();
}

bool BlockScheduler::build_decode_plan(std::string *err) {
  const ModelConfig &c = config_;
  greta_decode_desc d;
  fill_decode_desc(d, c, activations_, token_embd_, max_seq_);
  std::vector<greta_decode_layer> layers(c.num_layers);
  const size_t cache_l = (size_t)kv_heads_l_ * max_seq_ * c.head_dim;
  for (uint32_t l = 0; l < c.num_layers; ++l) {
    BlockBuffers &b = blocks_[l];
    greta_decode_layer &w = layers[l];
    w.wq_qs = b.wq.data(); w.wq_d = b.s_wq.data(); w.wk_qs = b.wk.data(); w.wk_d = b.s_wk.data(); w.wv_qs = b.wv.data(); w.wv_d = b.s_wv.data();
    w.wo_qs = b.wo.data(); w.wo_d = b.s_wo.data(); w.w1_qs = b.w1.data(); w.w1_d = b.s_w1.data(); w.w2_qs = b.w2.data(); w.w2_d = b.s_w2.data();
    w.w3_qs = b.w3.data(); w.w3_d = b.s_w3.data();
    w.attn_norm = static_cast<const float *>(b.attn_norm.data()); w.ffn_norm = static_cast<const float *>(b.ffn_norm.data());
    w.k_cache = static_cast<uint16_t *>(activations_.kv_cache_k.data()) + l * cache_l;
    w.v_cache = static_cast<uint16_t *>(activations_.kv_cache_v.data()) + l * cache_l;
  }
  const size_t bytes = greta_cuda_decode_plan_bytes(c.num_layers);
  if (!decode_plan_.allocate(bytes, BufferUsage::DeviceOnly, GretaDataType::INT8, err)) return false;
  GRETA_TRY(greta_cuda_memset(decode_plan_.data(), 0, bytes, nullptr), "decode plan");
  GRETA_TRY(greta_cuda_device_synchronize(), "decode plan");
  GRETA_TRY(greta_cuda_decode_plan_build(H(stream_), &d, layers.data(), decode_plan_.data(), bytes), "decode plan");
  return true;
}

bool BlockScheduler::decode_trace(long long *out25) {
  for (int i = 0; i < 25; ++i) out25[i] = 0;
  if (!persistent_step_ || !decode_plan_.data()) return true;
  return greta_cuda_decode_trace(decode_plan_.data(), out25) == GRETA_OK;
}

// ------------------------------------------------------------------ device-side decode loop
bool BlockScheduler::begin_decode(int32_t first_token, size_t pos, std::string *err) {
  if (batch_ != 1) return fail(err, "begin_decode: this scheduler holds a batch; use begin_decode_batch");
  const uint32_t p32 = (uint32_t)pos;
  return begin_decode_batch(&first_token, &p32, err);
}

bool BlockScheduler::begin_decode_batch(const int32_t *first_tokens, const uint32_t *positions, std::string *err) {
  if (!first_tokens || !positions) return fail(err, "begin_decode_batch: null argument");
  ActivationBuffers &a = activations_;
  cudaStream_t s = H(stream_);
  const uint32_t B = batch_;
  std::vector<uint32_t> init(std::max<size_t>(4, 2 * B), 0u);  // B positions, then B counts of ids produced
  std::vector<int32_t> tok(std::max<size_t>(4, B), 0);
  size_t pos_max = 0;
  for (uint32_t b = 0; b < B; ++b) {
    if (positions[b] >= max_seq_) return fail(err, "begin_decode: position exceeds max_seq_len");
    init[b] = positions[b];
    tok[b] = first_tokens[b];
    pos_max = std::max<size_t>(pos_max, positions[b]);
  }
  GRETA_TRY(greta_cuda_memcpy_h2d_sync(a.d_pos.data(), init.data(), init.size() * 4), "begin_decode");
  GRETA_TRY(greta_cuda_memcpy_h2d_sync(a.d_next.data(), tok.data(), tok.size() * 4), "begin_decode");
  decode_steps_ = 0;
  decode_pos0_ = pos_max;  // the sequence closest to the end of its cache bounds the number of steps
  if (peer_.tp > 1) {
    GRETA_TRY(greta_cuda_peer_reset(s), "exchange status reset");
    // Exchange tags grow with the position: a session that restarts earlier must not meet the tags of the
    // last one.  Every rank clears its slots, then a collective keeps anyone from storing into a buffer
    // that is still being cleared.
    GRETA_TRY(greta_cuda_memset(peer_.slots[peer_.rank], 0, (size_t)peer_.slot_bytes, s), "exchange reset");
    if (all_reduce_(static_cast<float *>(logits_.data()), 1, s) != 0) return fail(err, "begin_decode: barrier failed");
    GRETA_TRY(greta_cuda_stream_synchronize(s), "begin_decode");
  }
  if (!graph_captured_) {
    const ModelConfig &c = config_;
    // The step is a graph of the per-layer operators chained by programmatic dependent launch.
    // GRETA_PERSISTENT_STEP=1 (one GPU only) runs all layers as one persistent kernel instead; it
    // gives identical results and is kept as an option: measured slower so far (the per-phase
    // activation staging and grid barriers cost more than the launches they replace).
    const char *env = std::getenv("GRETA_PERSISTENT_STEP");
    persistent_step_ = c.tp_size == 1 && batch_ == 1 && env && env[0] == '1';
    if (persistent_step_ && !build_decode_plan(err)) return false;
    greta_decode_desc desc;
    fill_decode_desc(desc, c, a, token_embd_, max_seq_);
    graph_ = gcore::rt::GretaContext::instance().create_graph();
    graph_->capture_start(stream_);  // void, as in the reference: a capture that failed shows at instantiate()
    bool ok;
    const float *x_last = static_cast<const float *>(a.x.data());
    if (batch_ > 1) {
      ok = greta_cuda_embedding(s, static_cast<const int32_t *>(a.d_next.data()), token_embd_.data(), 1, static_cast<float *>(a.x.data()), batch_,
                                c.dim, c.vocab_size) == GRETA_OK;
      if (ok && c.tp_size > 1) ok = greta_cuda_memset(logits_.data(), 0, logits_.size(), s) == GRETA_OK;
      ok = ok && decode_layers_batch(err) && lm_head_batch(err);
      uint32_t *dp = static_cast<uint32_t *>(a.d_pos.data());
      ok = ok && greta_cuda_argmax_advance_batch(s, static_cast<const float *>(logits_.data()), c.vocab_size, batch_,
                                                 static_cast<int32_t *>(a.d_next.data()), dp, static_cast<int32_t *>(a.out_tokens.data()), dp + batch_,
                                                 (uint32_t)max_seq_) == GRETA_OK;
    } else if (persistent_step_) {
      ok = greta_cuda_decode_layers(s, &desc, decode_plan_.data()) == GRETA_OK;
      if (!ok && err) *err = gcore::host::cuda_error("decode_layers");
    } else {
      ok = greta_cuda_embedding(s, static_cast<const int32_t *>(a.d_next.data()), token_embd_.data(), 1, static_cast<float *>(a.x.data()), 1,
                                c.dim, c.vocab_size) == GRETA_OK;
      if (ok && c.tp_size > 1) ok = greta_cuda_memset(logits_.data(), 0, logits_.size(), s) == GRETA_OK;
      ok = ok && decode_layers(err, peer_.tp > 1, &x_last);
    }
    if (batch_ == 1) ok = ok && lm_head(x_last, err);
    uint32_t *dp = static_cast<uint32_t *>(a.d_pos.data());
    if (batch_ == 1) ok = ok && greta_cuda_argmax_advance(s, static_cast<const float *>(logits_.data()), c.vocab_size, static_cast<int32_t *>(a.d_next.data()), dp,
                                         static_cast<int32_t *>(a.out_tokens.data()), dp + 1, (uint32_t)max_seq_) == GRETA_OK;
    graph_->capture_end(stream_);
    if (!ok || graph_->instantiate() != gcore::rt::GretaResult::SUCCESS) {
      delete graph_;
      graph_ = nullptr;
      return fail(err, err && !err->empty() ? *err : gcore::host::cuda_error("capturing the decode step failed"));
    }
    graph_captured_ = true;
  }
  return true;
}

// The step about to run reads and writes cache row decode_pos0_ + decode_steps_: it must exist.
bool BlockScheduler::step_fits(std::string *err) const {
  if (decode_pos0_ + decode_steps_ >= max_seq_)
    return fail(err, "decode step at position " + std::to_string(decode_pos0_ + decode_steps_) + " exceeds max_seq_len " + std::to_string(max_seq_));
  return true;
}

bool BlockScheduler::decode_step(std::string *err) {
  if (!graph_captured_) return fail(err, "decode_step: begin_decode() first");
  if (!step_fits(err)) return false;
  if (graph_->launch(stream_) != gcore::rt::GretaResult::SUCCESS) return fail(err, gcore::host::cuda_error("decode step launch failed"));
  ++decode_steps_;
  return true;
}

bool BlockScheduler::decode_step_host(const int32_t *token_in, int32_t *token_out, std::string *err) {
  if (!graph_captured_) return fail(err, "decode_step_host: begin_decode() first");
  if (!step_fits(err)) return false;
  cudaStream_t s = H(stream_);
  GRETA_TRY(greta_cuda_memcpy_h2d(activations_.d_next.data(), token_in, (size_t)batch_ * 4, s), "token upload");
  if (graph_->launch(stream_) != gcore::rt::GretaResult::SUCCESS) return fail(err, gcore::host::cuda_error("decode step launch failed"));
  GRETA_TRY(greta_cuda_memcpy_d2h(token_out, activations_.d_next.data(), (size_t)batch_ * 4, s), "token download");
  GRETA_TRY(greta_cuda_stream_synchronize(s), "decode_step_host");
  ++decode_steps_;
  return true;
}

bool BlockScheduler::read_generated(int32_t *out, size_t n, std::string *err) {
  GRETA_TRY(greta_cuda_stream_synchronize(H(stream_)), "read_generated");
  if (n > decode_steps_) return fail(err, "read_generated: fewer steps were run");
  for (uint32_t b = 0; b < batch_; ++b)  // out is [batch][n]; the device list is [batch][max_seq]
    if (!activations_.out_tokens.copy_to_host_offset(out + (size_t)b * n, (size_t)b * max_seq_ * 4, n * 4, err)) return false;
  return true;
}

// ------------------------------------------------------------------ Generator
bool Generator::init(const ModelConfig &config, BlockScheduler *scheduler, std::string *err) {
  if (!scheduler) return fail(err, "Generator::init: null scheduler");
  config_ = config;
  scheduler_ = scheduler;
  return true;
}

int32_t Generator::sample(const float *logits, size_t vocab_size, const SamplingParams &) {
  int32_t id = 0;
  float mv = logits[0];
  for (size_t i = 1; i < vocab_size; ++i)
    if (logits[i] > mv) {
      mv = logits[i];
      id = (int32_t)i;
    }
  return id;
}

std::vector<std::vector<int32_t>> Generator::generate_batch(const std::vector<std::vector<int32_t>> &prompts, const SamplingParams &params,
                                                            std::string *err) {
  std::vector<std::vector<int32_t>> out;
  if (!scheduler_ || params.max_tokens <= 0) return out;
  const size_t B = scheduler_->batch_size();
  if (prompts.size() != B) {
    if (err) *err = "generate_batch: one prompt per sequence of the batch";
    return out;
  }
  if (!params.greedy) {
    if (err) *err = "only greedy decoding is on this path";
    return out;
  }
  const size_t steps = (size_t)params.max_tokens - 1;
  std::vector<int32_t> first(B);
  std::vector<uint32_t> pos(B);
  for (size_t b = 0; b < B; ++b) {  // prefill, one sequence at a time, into that sequence's cache
    if (prompts[b].empty() || prompts[b].size() + steps > scheduler_->max_seq_len()) {
      if (err) *err = "generate_batch: empty prompt, or prompt + max_tokens exceeds max_seq_len";
      return out;
    }
    if (!scheduler_->set_sequence(b, err) || !scheduler_->forward(prompts[b].data(), 0, prompts[b].size(), err)) return out;
    first[b] = scheduler_->sample_greedy_gpu(0, err);
    pos[b] = (uint32_t)prompts[b].size();
  }
  std::vector<int32_t> rest(B * steps);
  if (steps > 0) {
    if (!scheduler_->begin_decode_batch(first.data(), pos.data(), err)) return out;
    for (size_t i = 0; i < steps; ++i)
      if (!scheduler_->decode_step(err)) return out;
    if (!scheduler_->read_generated(rest.data(), steps, err)) return out;
  }
  out.resize(B);
  for (size_t b = 0; b < B; ++b) {
    out[b].push_back(first[b]);
    out[b].insert(out[b].end(), rest.begin() + b * steps, rest.begin() + (b + 1) * steps);
  }
  return out;
}

std::vector<int32_t> Generator::generate_tokens(const std::vector<int32_t> &prompt, const SamplingParams &params, GenerationStats *stats,
                                                std::string *err) {
  std::vector<int32_t> out;
  if (!scheduler_ || prompt.empty() || params.max_tokens <= 0) return out;
  if (!params.greedy) {
    if (err) *err = "only greedy decoding is on this path";
    return out;
  }
  using clk = std::chrono::steady_clock;
  auto t0 = clk::now();
  if (!scheduler_->forward(prompt.data(), 0, prompt.size(), err)) return out;
  int32_t first = scheduler_->sample_greedy_gpu(0, err);
  auto t1 = clk::now();
  out.push_back(first);
  const size_t steps = (size_t)params.max_tokens - 1;
  double decode_ms = 0.0;
  // The reference stops when the sampled id is the tokenizer's end-of-sequence id (generator.cpp:1128-1129); the
  // tokenizer is outside this path, so the id comes in through SamplingParams (-1: never stop early).
  const bool watch_eos = params.eos_token_id >= 0;
  if (steps > 0 && !(watch_eos && first == params.eos_token_id)) {
    if (prompt.size() + steps > scheduler_->max_seq_len()) {
      if (err) *err = "generate_tokens: prompt + max_tokens exceeds max_seq_len";
      return out;
    }
    if (!scheduler_->begin_decode(first, prompt.size(), err)) return out;
    std::unique_ptr<gcore::rt::GretaEvent> e0(gcore::rt::GretaContext::instance().create_event()),
        e1(gcore::rt::GretaContext::instance().create_event());
    e0->record(scheduler_->stream());
    // The steps run on the device without a host round trip.  With an end-of-sequence id to watch for they run in
    // chunks: after each chunk the ids produced so far come back and the loop ends at the first match.
    const size_t chunk = watch_eos ? 16 : steps;
    size_t done = 0;
    bool stop = false;
    while (done < steps && !stop) {
      const size_t n = std::min(chunk, steps - done);
      for (size_t i = 0; i < n; ++i)
        if (!scheduler_->decode_step(err)) return out;
      done += n;
      if (watch_eos) {
        out.resize(1 + done);
        if (!scheduler_->read_generated(out.data() + 1, done, err)) {
          out.resize(1);
          return out;
        }
        for (size_t i = done - n; i < done && !stop; ++i)
          if (out[1 + i] == params.eos_token_id) {
            out.resize(2 + i);  // the end-of-sequence id is the last one returned
            stop = true;
          }
      }
    }
    e1->record(scheduler_->stream());
    if (!watch_eos) {
      out.resize(1 + steps);
      if (!scheduler_->read_generated(out.data() + 1, steps, err)) {
        out.resize(1);
        return out;
      }
    }
    decode_ms = e1->elapsed_time_since(e0.get());
  }
  auto t2 = clk::now();
  if (stats) {
    stats->prompt_tokens = prompt.size();
    stats->generated_tokens = out.size();
    stats->time_to_first_token_ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
    stats->total_time_ms = std::chrono::duration<double, std::milli>(t2 - t0).count();
    stats->decode_time_ms = decode_ms;
    stats->tokens_per_second = stats->total_time_ms > 0 ? 1e3 * out.size() / stats->total_time_ms : 0.0;
  }
  return out;
}

}  // namespace gcore::inference
