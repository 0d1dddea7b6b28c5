// C handles onto the C++ host layer (see greta_host.h).
#include <cstring>
#include <memory>
#include <string>

#include "gcore/greta_b200.hpp"
#include "greta_host.h"
#include "host_util.hpp"

using namespace gcore::inference;
using gcore::rt::GretaDataType;

namespace {
thread_local std::string g_err;
struct Model {
  BlockScheduler sched;
  Generator gen;
  ModelConfig cfg;
};
inline int done(bool ok, const std::string &err) {
  if (!ok) g_err = err.empty() ? "failed" : err;
  return ok ? 0 : 1;
}
inline GretaDataType dtype(int fmt) {
  return fmt == GRETA_FMT_Q4_0 ? GretaDataType::Q4_0 : fmt == GRETA_FMT_Q8_0 ? GretaDataType::Q8_0 : GretaDataType::FP16;
}
}  // namespace

#define M(m) static_cast<Model *>(m)

extern "C" {

const char *greta_host_last_error(void) { return g_err.c_str(); }

int greta_host_synth_quant_blocks(uint64_t seed, uint64_t stream, int fmt, void *out, size_t first_block, size_t n_blocks) {
  if (fmt != GRETA_FMT_Q4_0 && fmt != GRETA_FMT_Q8_0) return done(false, "synth_quant_blocks: format must be Q4_0 or Q8_0");
  synth::quant_blocks(seed, stream, dtype(fmt), static_cast<uint8_t *>(out), first_block, n_blocks);
  return 0;
}
int greta_host_synth_normal_f16(uint64_t seed, uint64_t stream, float sigma, void *out, size_t first, size_t n) {
  synth::normal_f16(seed, stream, sigma, static_cast<uint16_t *>(out), first, n);
  return 0;
}
int greta_host_synth_normal_f16_as_f32(uint64_t seed, uint64_t stream, float sigma, float *out, size_t first, size_t n) {
  synth::normal_f16_as_f32(seed, stream, sigma, out, first, n);
  return 0;
}
int greta_host_synth_normal_f32(uint64_t seed, uint64_t stream, float sigma, float *out, size_t first, size_t n) {
  synth::normal_f32(seed, stream, sigma, out, first, n);
  return 0;
}
int greta_host_synth_tokens(uint64_t seed, uint64_t stream, uint32_t vocab, int32_t *out, size_t n) {
  synth::tokens(seed, stream, vocab, out, n);
  return 0;
}
uint64_t greta_host_tensor_stream(uint32_t layer, int which) { return synth::tensor_stream(layer, which); }

int greta_host_tensor_shard(const greta_model_config *c, int which, uint32_t *out6) {
  if (!c || !out6 || which < 0 || which > (int)LayerTensor::W3_UP || c->tp_size == 0 || c->tp_rank >= c->tp_size)
    return done(false, "tensor_shard: bad argument");
  ModelConfig k;
  k.dim = c->dim; k.num_heads = c->num_heads; k.num_heads_kv = c->num_heads_kv; k.hidden_dim = c->hidden_dim; k.head_dim = c->head_dim;
  k.tp_rank = c->tp_rank; k.tp_size = c->tp_size;
  TensorShard s = tensor_shard(k, (LayerTensor)which);
  out6[0] = s.rows; out6[1] = s.cols; out6[2] = s.grows; out6[3] = s.gcols; out6[4] = s.row0; out6[5] = s.col0;
  return 0;
}

// GGUFLoader::open + get_config + list_tensors, without a device: the parsed shape (and how many tensors the file holds).
int greta_host_gguf_info(const char *path, greta_model_config *cfg, uint32_t *n_tensors) {
  std::string err;
  GGUFLoader ld;
  if (!path || !ld.open(path, &err)) return done(false, err.empty() ? "gguf_info: null path" : err);
  const ModelConfig k = ld.get_config();
  if (cfg) {
    cfg->dim = k.dim; cfg->num_heads = k.num_heads; cfg->num_heads_kv = k.num_heads_kv; cfg->num_layers = k.num_layers;
    cfg->vocab_size = k.vocab_size; cfg->hidden_dim = k.hidden_dim; cfg->head_dim = k.head_dim; cfg->max_seq_len = k.max_seq_len;
    cfg->rope_base = k.rope_base; cfg->rms_eps = k.rms_eps;
    cfg->weight_fmt = k.weight_type == GretaDataType::Q8_0 ? GRETA_FMT_Q8_0 : GRETA_FMT_Q4_0;
    cfg->lm_head_fmt = k.lm_head_type == GretaDataType::Q4_0 ? GRETA_FMT_Q4_0 : k.lm_head_type == GretaDataType::Q8_0 ? GRETA_FMT_Q8_0 : GRETA_FMT_F16;
    cfg->tp_rank = 0; cfg->tp_size = 1;
  }
  if (n_tensors) *n_tensors = (uint32_t)ld.list_tensors().size();
  return 0;
}
// GGUFLoader::read_as_fp16: a tensor of the file decoded to fp16 bits in host memory (no device).
int greta_host_gguf_read_fp16(const char *path, const char *name, void *out_f16, size_t capacity_elems, size_t *elems) {
  std::string err;
  GGUFLoader ld;
  if (!path || !name || !ld.open(path, &err)) return done(false, err.empty() ? "gguf_read_fp16: null argument" : err);
  std::vector<uint16_t> v;
  if (!ld.read_as_fp16(name, &v, &err)) return done(false, err);
  if (elems) *elems = v.size();
  if (out_f16 && v.size() <= capacity_elems) std::memcpy(out_f16, v.data(), v.size() * 2);
  return 0;
}
// BlockScheduler::load_weights(GGUFLoader): the model must have been created with the file's shape and storage types.
int greta_model_load_gguf(greta_model_t m, const char *path) {
  std::string err;
  GGUFLoader ld;
  if (!path || !ld.open(path, &err)) return done(false, err.empty() ? "load_gguf: null path" : err);
  return done(M(m)->sched.load_weights(ld, &err), err);
}

int greta_model_create(const greta_model_config *c, greta_model_t *out) { return greta_model_create_batch(c, 1, out); }

int greta_model_create_batch(const greta_model_config *c, uint32_t batch, greta_model_t *out) {
  if (!c || !out) return done(false, "model_create: null argument");
  auto m = std::make_unique<Model>();
  ModelConfig &k = m->cfg;
  k.dim = c->dim; k.num_heads = c->num_heads; k.num_heads_kv = c->num_heads_kv; k.num_layers = c->num_layers;
  k.vocab_size = c->vocab_size; k.hidden_dim = c->hidden_dim; k.head_dim = c->head_dim; k.max_seq_len = c->max_seq_len;
  k.rope_base = c->rope_base; k.rms_eps = c->rms_eps;
  k.weight_type = dtype(c->weight_fmt); k.lm_head_type = dtype(c->lm_head_fmt);
  k.tp_rank = c->tp_rank; k.tp_size = c->tp_size ? c->tp_size : 1;
  std::string err;
  bool ok = m->sched.init(k, &err) && m->sched.allocate_weights(&err) && m->sched.allocate_activations(batch, k.max_seq_len, &err) &&
            m->gen.init(k, &m->sched, &err);
  if (!ok) return done(false, err);
  *out = m.release();
  return 0;
}
int greta_model_destroy(greta_model_t m) {
  delete static_cast<Model *>(m);
  return 0;
}
int greta_model_load_synthetic(greta_model_t m, uint64_t seed) {
  std::string err;
  return done(M(m)->sched.load_synthetic_weights(seed, &err), err);
}
int greta_model_set_layer_tensor(greta_model_t m, uint32_t layer, int which, const void *host, size_t bytes) {
  std::string err;
  return done(M(m)->sched.set_layer_tensor(layer, (LayerTensor)which, host, bytes, &err), err);
}
int greta_model_set_global_tensor(greta_model_t m, int which, const void *host, size_t bytes) {
  std::string err;
  return done(M(m)->sched.set_global_tensor((GlobalTensor)which, host, bytes, &err), err);
}
int greta_model_forward(greta_model_t m, const int32_t *tokens, uint32_t seq_start, uint32_t seq_len) {
  std::string err;
  return done(M(m)->sched.forward(tokens, seq_start, seq_len, &err), err);
}
int greta_model_get_logits(greta_model_t m, float *out, uint32_t n) {
  std::string err;
  return done(M(m)->sched.get_logits().copy_to_host(out, (size_t)n * 4, &err), err);
}
int greta_model_get_hidden(greta_model_t m, float *out, uint32_t row, uint32_t n) {
  std::string err;
  return done(M(m)->sched.get_hidden_state().copy_to_host_offset(out, (size_t)row * M(m)->cfg.dim * 4, (size_t)n * 4, &err), err);
}
int greta_model_sample_greedy(greta_model_t m, int32_t *id) {
  std::string err;
  *id = M(m)->sched.sample_greedy_gpu(0, &err);
  return done(err.empty(), err);
}
int greta_model_generate(greta_model_t m, const int32_t *prompt, uint32_t n_prompt, uint32_t n_new, int32_t *out, double *stats5) {
  std::string err;
  SamplingParams sp;
  sp.greedy = true;
  sp.max_tokens = (int32_t)n_new;
  GenerationStats st;
  std::vector<int32_t> ids = M(m)->gen.generate_tokens(std::vector<int32_t>(prompt, prompt + n_prompt), sp, &st, &err);
  if (ids.size() != n_new) return done(false, err.empty() ? "generation stopped early" : err);
  std::memcpy(out, ids.data(), ids.size() * 4);
  if (stats5) {
    stats5[0] = (double)st.prompt_tokens; stats5[1] = (double)st.generated_tokens; stats5[2] = st.total_time_ms;
    stats5[3] = st.time_to_first_token_ms; stats5[4] = st.decode_time_ms;
  }
  return 0;
}
int greta_model_generate_eos(greta_model_t m, const int32_t *prompt, uint32_t n_prompt, uint32_t max_new, int32_t eos_id, int32_t *out,
                             uint32_t *n_out) {
  std::string err;
  SamplingParams sp;
  sp.greedy = true;
  sp.max_tokens = (int32_t)max_new;
  sp.eos_token_id = eos_id;
  std::vector<int32_t> ids = M(m)->gen.generate_tokens(std::vector<int32_t>(prompt, prompt + n_prompt), sp, nullptr, &err);
  if (!err.empty() || ids.empty()) return done(false, err.empty() ? "generation produced nothing" : err);
  std::memcpy(out, ids.data(), ids.size() * 4);
  *n_out = (uint32_t)ids.size();
  return 0;
}
int greta_model_set_sequence(greta_model_t m, uint32_t seq) {
  std::string err;
  return done(M(m)->sched.set_sequence(seq, &err), err);
}
int greta_model_begin_decode_batch(greta_model_t m, const int32_t *first_tokens, const uint32_t *positions) {
  std::string err;
  return done(M(m)->sched.begin_decode_batch(first_tokens, positions, &err), err);
}
int greta_model_generate_batch(greta_model_t m, const int32_t *prompts, uint32_t n_prompt, uint32_t n_new, int32_t *out) {
  std::string err;
  SamplingParams sp;
  sp.greedy = true;
  sp.max_tokens = (int32_t)n_new;
  const size_t B = M(m)->sched.batch_size();
  std::vector<std::vector<int32_t>> in(B);
  for (size_t b = 0; b < B; ++b) in[b].assign(prompts + b * n_prompt, prompts + (b + 1) * n_prompt);
  std::vector<std::vector<int32_t>> ids = M(m)->gen.generate_batch(in, sp, &err);
  if (ids.size() != B) return done(false, err.empty() ? "batched generation failed" : err);
  for (size_t b = 0; b < B; ++b) {
    if (ids[b].size() != n_new) return done(false, err.empty() ? "generation stopped early" : err);
    std::memcpy(out + b * n_new, ids[b].data(), (size_t)n_new * 4);
  }
  return 0;
}
int greta_model_begin_decode(greta_model_t m, int32_t first_token, uint32_t pos) {
  std::string err;
  return done(M(m)->sched.begin_decode(first_token, pos, &err), err);
}
int greta_model_decode_step(greta_model_t m) {
  std::string err;
  return done(M(m)->sched.decode_step(&err), err);
}
int greta_model_read_generated(greta_model_t m, int32_t *out, uint32_t n) {
  std::string err;
  return done(M(m)->sched.read_generated(out, n, &err), err);
}
int greta_model_decode_timed(greta_model_t m, uint32_t steps, float *ms) {
  std::string err;
  auto &ctx = gcore::rt::GretaContext::instance();
  std::unique_ptr<gcore::rt::GretaEvent> e0(ctx.create_event()), e1(ctx.create_event());
  e0->record(M(m)->sched.stream());
  for (uint32_t i = 0; i < steps; ++i)
    if (!M(m)->sched.decode_step(&err)) return done(false, err);
  e1->record(M(m)->sched.stream());
  *ms = e1->elapsed_time_since(e0.get());
  return 0;
}
int greta_model_decode_e2e(greta_model_t m, int32_t first_token, uint32_t pos, uint32_t steps, int32_t *out, float *ms) {
  return greta_model_decode_e2e_batch(m, &first_token, &pos, steps, out, ms);
}
int greta_model_decode_e2e_batch(greta_model_t m, const int32_t *first_tokens, const uint32_t *positions, uint32_t steps, int32_t *out, float *ms) {
  std::string err;
  const size_t B = M(m)->sched.batch_size();
  if (!M(m)->sched.begin_decode_batch(first_tokens, positions, &err)) return done(false, err);
  gcore::rt::cuda::Buffer pin;
  if (!pin.allocate(2 * B * 4 + 64, gcore::rt::cuda::BufferUsage::HostVisible, GretaDataType::FP32, &err)) return done(false, err);
  int32_t *tok = static_cast<int32_t *>(pin.data()), *got = tok + B;
  std::memcpy(tok, first_tokens, B * 4);
  auto &ctx = gcore::rt::GretaContext::instance();
  std::unique_ptr<gcore::rt::GretaEvent> e0(ctx.create_event()), e1(ctx.create_event());
  e0->record(M(m)->sched.stream());
  for (uint32_t i = 0; i < steps; ++i) {
    if (!M(m)->sched.decode_step_host(tok, got, &err)) return done(false, err);
    for (size_t b = 0; b < B; ++b) out[b * steps + i] = got[b];  // out is [batch][steps]
    std::memcpy(tok, got, B * 4);
  }
  e1->record(M(m)->sched.stream());
  *ms = e1->elapsed_time_since(e0.get());
  return 0;
}
int greta_model_decode_trace(greta_model_t m, long long *out25) { return done(M(m)->sched.decode_trace(out25), "decode_trace failed"); }
uint64_t greta_model_weight_bytes(greta_model_t m) { return M(m)->sched.weight_bytes(); }
void *greta_model_stream(greta_model_t m) { return static_cast<gcore::rt::cuda::GretaStreamCuda *>(M(m)->sched.stream())->handle(); }
int greta_model_set_peer_exchange(greta_model_t m, const greta_peer_exchange *ex) {
  if (!ex) return done(false, "model_set_peer_exchange: null descriptor");
  std::string err;
  return done(M(m)->sched.set_peer_exchange(*ex, &err), err);
}

int greta_model_set_comm(greta_model_t m, void *comm) {
  if (!comm) return done(false, "model_set_comm: null communicator");
  M(m)->sched.set_all_reduce([comm](float *buf, size_t count, cudaStream_t stream) { return greta_cuda_comm_allreduce_f32(comm, buf, count, stream); });
  return 0;
}

}  // extern "C"
