/*
 * greta_host.h - C handles onto the C++ host layer (libgreta_host.so), for
 * callers that are not C++: the Python tests and the benchmark drive the model
 * through these.  Each function forwards to the gcore::inference class method
 * named beside it (include/gcore/greta_b200.hpp), which mirrors the reference's
 * BlockScheduler / Generator (src/inference/include/gcore/inference/
 * block_scheduler.hpp:67-142, generator.hpp:55-90).  Return 0 on success,
 * non-zero on failure with the text in greta_host_last_error().
 */
#ifndef GRETA_HOST_H
#define GRETA_HOST_H

#include <stddef.h>
#include <stdint.h>

#include "greta_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

#ifndef GRETA_API
#define GRETA_API __attribute__((visibility("default")))
#endif

typedef void *greta_model_t;

/* Same fields as gcore::inference::ModelConfig. weight_fmt / lm_head_fmt take GRETA_FMT_* values. */
typedef struct greta_model_config {
  uint32_t dim, num_heads, num_heads_kv, num_layers, vocab_size, hidden_dim, head_dim, max_seq_len;
  float rope_base, rms_eps;
  int weight_fmt, lm_head_fmt;
  uint32_t tp_rank, tp_size;
} greta_model_config;

GRETA_API const char *greta_host_last_error(void);

/* gcore::inference::synth: seeded, counter-based synthetic tensors (host memory). */
GRETA_API int greta_host_synth_quant_blocks(uint64_t seed, uint64_t stream, int fmt, void *out, size_t first_block, size_t n_blocks);
GRETA_API int greta_host_synth_normal_f16(uint64_t seed, uint64_t stream, float sigma, void *out_f16, size_t first, size_t n);
GRETA_API int greta_host_synth_normal_f16_as_f32(uint64_t seed, uint64_t stream, float sigma, float *out, size_t first, size_t n);
GRETA_API int greta_host_synth_normal_f32(uint64_t seed, uint64_t stream, float sigma, float *out, size_t first, size_t n);
GRETA_API int greta_host_synth_tokens(uint64_t seed, uint64_t stream, uint32_t vocab, int32_t *out, size_t n);
GRETA_API uint64_t greta_host_tensor_stream(uint32_t layer, int which);

/* gcore::inference::tensor_shard: out6 = {rows, cols, global rows, global cols, row0, col0} of the shard of
 * projection `which` (LayerTensor 0..6) that rank cfg->tp_rank holds.  Needs no device. */
GRETA_API int greta_host_tensor_shard(const greta_model_config *cfg, int which, uint32_t *out6);

/* GGUF files (gcore::inference::GGUFLoader; the reference's parser is src/inference/src/weight_loader.cpp:210-505).
 * greta_host_gguf_info: open + get_config + list_tensors - the model shape and storage types the file declares, no device
 * needed.  greta_host_gguf_read_fp16: one tensor (F16, F32, Q4_0 or Q8_0) decoded to fp16 bits on the host; *elems receives
 * its element count (out_f16 may be NULL to ask for the size). */
GRETA_API int greta_host_gguf_info(const char *path, greta_model_config *cfg, uint32_t *n_tensors);
GRETA_API int greta_host_gguf_read_fp16(const char *path, const char *name, void *out_f16, size_t capacity_elems, size_t *elems);

/* BlockScheduler::init + allocate_weights + allocate_activations(1, max_seq_len). */
GRETA_API int greta_model_create(const greta_model_config *cfg, greta_model_t *out);
/* The same with allocate_activations(batch, max_seq_len): `batch` sequences (1..32) that decode in step, each with its own
 * KV cache and position.  New with this build: the reference's scheduler holds one sequence. */
GRETA_API int greta_model_create_batch(const greta_model_config *cfg, uint32_t batch, greta_model_t *out);
GRETA_API int greta_model_destroy(greta_model_t m);
GRETA_API int greta_model_load_synthetic(greta_model_t m, uint64_t seed);                 /* load_synthetic_weights */
/* BlockScheduler::load_weights from a GGUF file whose projections are stored as Q4_0 / Q8_0: blocks go to the device as
 * they lie in the file (the model must have been created with the shape and formats greta_host_gguf_info reports). */
GRETA_API int greta_model_load_gguf(greta_model_t m, const char *path);
/* set_layer_tensor / set_global_tensor: `which` is a LayerTensor / GlobalTensor value; host points at the GLOBAL tensor. */
GRETA_API int greta_model_set_layer_tensor(greta_model_t m, uint32_t layer, int which, const void *host, size_t bytes);
GRETA_API int greta_model_set_global_tensor(greta_model_t m, int which, const void *host, size_t bytes);
GRETA_API int greta_model_forward(greta_model_t m, const int32_t *tokens, uint32_t seq_start, uint32_t seq_len);  /* forward */
GRETA_API int greta_model_get_logits(greta_model_t m, float *out, uint32_t n);           /* get_logits() -> host */
GRETA_API int greta_model_get_hidden(greta_model_t m, float *out, uint32_t row, uint32_t n); /* get_hidden_state() row -> host */
GRETA_API int greta_model_sample_greedy(greta_model_t m, int32_t *id);                   /* sample_greedy_gpu */
/* Generator::generate_tokens (greedy). stats5 = {prompt tokens, generated tokens, total ms, time to first token ms, decode ms}. */
GRETA_API int greta_model_generate(greta_model_t m, const int32_t *prompt, uint32_t n_prompt, uint32_t n_new, int32_t *out,
                                   double *stats5);
/* The same with SamplingParams::eos_token_id = eos_id: generation ends with the first eos_id produced (it is the last id
 * returned), as the reference's loop does with its tokenizer's id (src/inference/src/generator.cpp:1128-1129).  out holds
 * max_new ids; *n_out receives how many were produced. */
GRETA_API int greta_model_generate_eos(greta_model_t m, const int32_t *prompt, uint32_t n_prompt, uint32_t max_new, int32_t eos_id,
                                       int32_t *out, uint32_t *n_out);
GRETA_API int greta_model_begin_decode(greta_model_t m, int32_t first_token, uint32_t pos); /* begin_decode */
/* Batch: set_sequence (which sequence's cache forward() fills), begin_decode_batch (first token and position of every
 * sequence), Generator::generate_batch (prompts [batch][n_prompt] of equal length -> out [batch][n_new]). */
GRETA_API int greta_model_set_sequence(greta_model_t m, uint32_t seq);
GRETA_API int greta_model_begin_decode_batch(greta_model_t m, const int32_t *first_tokens, const uint32_t *positions);
GRETA_API int greta_model_generate_batch(greta_model_t m, const int32_t *prompts, uint32_t n_prompt, uint32_t n_new, int32_t *out);
GRETA_API int greta_model_decode_step(greta_model_t m);                                   /* decode_step (asynchronous) */
GRETA_API int greta_model_read_generated(greta_model_t m, int32_t *out, uint32_t n);      /* read_generated (synchronises); out is [batch][n] */
/* `steps` decode_step() calls bracketed by events on the model's stream; *ms = device time. */
GRETA_API int greta_model_decode_timed(greta_model_t m, uint32_t steps, float *ms);
/* The reference's decode loop shape (src/inference/src/generator.cpp:1128-1156): every step uploads the
 * previous token id from pinned host memory, runs forward for one position and reads the sampled id back
 * to the host before the next step.  *ms = device time of the whole loop (events), copies included;
 * out receives the `steps` ids.  Bytes per step: 4 up, 4 down. */
GRETA_API int greta_model_decode_e2e(greta_model_t m, int32_t first_token, uint32_t pos, uint32_t steps, int32_t *out, float *ms);
/* The same for a batch: every step uploads `batch` ids and reads `batch` ids back; out is [batch][steps]. */
GRETA_API int greta_model_decode_e2e_batch(greta_model_t m, const int32_t *first_tokens, const uint32_t *positions, uint32_t steps,
                                           int32_t *out, float *ms);
/* greta_cuda_decode_trace of the model's persistent decode step (zeros when that path is off). */
GRETA_API int greta_model_decode_trace(greta_model_t m, long long *out25);
GRETA_API uint64_t greta_model_weight_bytes(greta_model_t m);
GRETA_API void *greta_model_stream(greta_model_t m);
/* Installs the tensor-parallel exchange: an NCCL communicator made with greta_cuda_comm_init. */
GRETA_API int greta_model_set_comm(greta_model_t m, void *comm);
/* Installs the fused tensor-parallel exchange for the decode step (greta_cuda.h: greta_peer_exchange); call after
 * greta_model_set_comm, whose all-reduce still serves prefill, the last layer, the logits and the session barrier. */
GRETA_API int greta_model_set_peer_exchange(greta_model_t m, const greta_peer_exchange *ex);

#ifdef __cplusplus
}
#endif
#endif /* GRETA_HOST_H */
