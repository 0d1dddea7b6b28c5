/*
 * greta_cuda.h - C ABI of the sm_100a (B200) quantized-matmul hot path for GRETA CORE.
 *
 * Every entry point is plain C: raw device pointers, sizes, a stream handle.  No
 * exceptions, no hidden synchronisation, and (runtime/memory section apart) no
 * allocation.  Return value: 0 on success, otherwise a gcore::rt::GretaResult
 * value (src/rt/include/gcore/rt/greta_runtime.hpp:15-22 in the reference):
 *   1 out of memory, 2 graph capture, 3 kernel launch, 4 invalid arguments,
 *   5 not implemented.  greta_cuda_last_error() gives the text of the last failure
 *   on the calling thread.
 *
 * Each function names the reference interface it stands in for (path:line inside
 * the reference project).
 *
 * WEIGHT LAYOUT ("planar GGUF").  A weight W[N x K] (K contiguous, y = x * W^T)
 * quantised in GGUF blocks of 32 along K is held as two planes:
 *   qs plane: N * (K/32) quant payloads, row-major, 16 bytes each for Q4_0 (byte j
 *             of a payload = element j in the low nibble, element j+16 in the
 *             high nibble, q in 0..15, value (q-8)*d) and 32 bytes for Q8_0
 *             (int8 q, value q*d) - i.e. the GGUF block with its scale removed;
 *   d  plane: N rows of fp16 scales, K/32 per row, each row padded to a multiple of 8
 *             scales (16 bytes) - no padding when K is a multiple of 256.
 * Bytes per weight are those of GGUF (18/32 and 34/32; the row padding adds at most
 * 14 bytes per row); the split makes every payload and every scale row 16-byte
 * aligned for 128-bit loads and TMA.  The pair (qs, d) plays
 * the role of the reference's (weights, GretaQuantInfo::scales) pair with
 * group_size 32 (greta_runtime.hpp:35-41).  K must be a multiple of 32 and both
 * planes 16-byte aligned.  greta_cuda_qs_bytes / greta_cuda_d_bytes give the sizes.
 */
#ifndef GRETA_CUDA_H
#define GRETA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GRETA_API __attribute__((visibility("default")))

typedef void *greta_stream_t; /* a cudaStream_t; NULL = the legacy default stream */

enum {
  GRETA_OK = 0,
  GRETA_ERR_OUT_OF_MEM = 1,
  GRETA_ERR_GRAPH_CAPTURE = 2,
  GRETA_ERR_KERNEL_LAUNCH = 3,
  GRETA_ERR_INVALID_ARGS = 4,
  GRETA_ERR_NOT_IMPLEMENTED = 5
};

/* Weight formats.  Values continue gcore::rt::GretaDataType (greta_runtime.hpp:24-33,
 * FP32=0 .. FP8_E5M2=7) so that the C++ layer can pass data_type() straight through. */
enum {
  GRETA_FMT_F16 = 1,
  GRETA_FMT_REF_INT8 = 3, /* reference storage: int8 w[N][K], fp32 scale per 32 along the flat index */
  GRETA_FMT_REF_INT4 = 4, /* reference storage: uint8 w[N][K/2], elem 2j low nibble, two's complement, fp32 scales */
  GRETA_FMT_Q4_0 = 8,
  GRETA_FMT_Q8_0 = 9
};

/* ------------------------------------------------------------------ runtime
 * Stand-ins for the hip* calls of the reference's L0 backend
 * (src/rt/backend/hip/src/greta_runtime_hip.cpp:7-179, buffer.cpp:7-84,
 * backend.cpp:11-87). */
GRETA_API const char *greta_cuda_last_error(void);
GRETA_API int greta_cuda_device_count(int *count);
GRETA_API int greta_cuda_set_device(int device);
GRETA_API int greta_cuda_get_device(int *device);
/* name_cap bytes of name; any out pointer may be NULL. */
GRETA_API int greta_cuda_device_info(int device, char *name, size_t name_cap, int *sm_count,
                                     size_t *total_mem, int *cc_major, int *cc_minor);
GRETA_API int greta_cuda_malloc(void **ptr, size_t bytes);
GRETA_API int greta_cuda_free(void *ptr);
GRETA_API int greta_cuda_malloc_host(void **ptr, size_t bytes); /* pinned host memory */
GRETA_API int greta_cuda_free_host(void *ptr);
/* Copies are asynchronous on `stream` when the host side is pinned; _sync variants block. */
GRETA_API int greta_cuda_memcpy_h2d(void *dst, const void *src, size_t bytes, greta_stream_t stream);
GRETA_API int greta_cuda_memcpy_d2h(void *dst, const void *src, size_t bytes, greta_stream_t stream);
GRETA_API int greta_cuda_memcpy_d2d(void *dst, const void *src, size_t bytes, greta_stream_t stream);
/* height rows of width bytes between pitched device arrays, asynchronous on `stream` (hipMemcpy2DAsync in the reference's runtime). */
GRETA_API int greta_cuda_memcpy_2d_d2d(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width, size_t height,
                                       greta_stream_t stream);
GRETA_API int greta_cuda_memcpy_h2d_sync(void *dst, const void *src, size_t bytes);
GRETA_API int greta_cuda_memcpy_d2h_sync(void *dst, const void *src, size_t bytes);
GRETA_API int greta_cuda_memset(void *dst, int value, size_t bytes, greta_stream_t stream);
GRETA_API int greta_cuda_stream_create(greta_stream_t *stream);
GRETA_API int greta_cuda_stream_destroy(greta_stream_t stream);
GRETA_API int greta_cuda_stream_synchronize(greta_stream_t stream);
GRETA_API int greta_cuda_device_synchronize(void);
GRETA_API int greta_cuda_event_create(void **event);
GRETA_API int greta_cuda_event_destroy(void *event);
GRETA_API int greta_cuda_event_record(void *event, greta_stream_t stream);
GRETA_API int greta_cuda_event_synchronize(void *event);
GRETA_API int greta_cuda_event_elapsed_ms(void *start, void *end, float *ms);
GRETA_API int greta_cuda_stream_wait_event(greta_stream_t stream, void *event);
/* Graphs: GretaGraphHip capture_start/capture_end/instantiate/launch
 * (greta_runtime_hip.cpp:84-141). */
GRETA_API int greta_cuda_graph_capture_begin(greta_stream_t stream);
GRETA_API int greta_cuda_graph_capture_end(greta_stream_t stream, void **graph);
GRETA_API int greta_cuda_graph_instantiate(void *graph, void **exec);
GRETA_API int greta_cuda_graph_launch(void *exec, greta_stream_t stream);
/* *capturing = 1 while `stream` is recording a graph (hipStreamIsCapturing in the reference's runtime). */
GRETA_API int greta_cuda_stream_is_capturing(greta_stream_t stream, int *capturing);
GRETA_API int greta_cuda_graph_destroy(void *graph);
GRETA_API int greta_cuda_graph_exec_destroy(void *exec);
/* Programmatic dependent launch between consecutive kernels of this library on one stream (the next
 * kernel's weight prefetch overlaps the previous kernel's tail).  On by default; GRETA_PDL=0 in the
 * environment or greta_cuda_set_pdl(0) turns it off.  Results do not depend on it. */
GRETA_API int greta_cuda_set_pdl(int on);
/* Tuning switches, for tests and measurements; results do not depend on them.  Each switch starts from an
 * environment variable that is read once, at the first use of any of them - never on a call path (the
 * reference reads its switches from the environment inside GretaCompute::gemm,
 * src/compute/src/greta_compute_hip.cpp:148-374):
 *   "pdl" (GRETA_PDL, 0/1), "attn_cluster" (GRETA_ATTN_CLUSTER, 0/1: splits of a head meet in a thread-block
 *   cluster or through scratch), "gemm_tile" (GRETA_GEMM_TILE=<tokens>x<row tiles>; value = tokens * 10 + row
 *   tiles, 0 = automatic), "gemv_r2_cells" (GRETA_GEMV_R2_CELLS, < 0 = automatic), "step_stages"
 *   (GRETA_STEP_STAGES, 0 = automatic), "peer_poll_limit" (GRETA_PEER_POLL_LIMIT: polls a tensor-parallel
 *   consumer spends on one missing partial before it gives up, default 2^22), "attn_mma" (GRETA_ATTN_MMA, 0/1: prefill and grouped-query batched decode
 *   attention on the tensor cores), "peer_two_level_min_tp"
 *   (GRETA_PEER_TWO_LEVEL_MIN_TP: ranks from which an exchange consumer gathers in two levels, default 4), "skinny_max_rows"
 *   (GRETA_SKINNY_MAX_ROWS, 1..32), "gemv_ring_stages" (GRETA_GEMV_RING_STAGES: 3 or 5 forces the depth of the single-row GEMV's weight ring,
 *   0 = automatic), "gemm_splitk" (GRETA_GEMM_SPLITK, default 0: 1 = a prefill GEMM with fewer 512-token tiles than
 *   SMs shares each tile's K loop between CTAs where that is predicted to pay, 2 = wherever it is feasible; needs the workspace; the partial sums change the
 *   fp32 summation order, deterministically), "gemm_pair" (GRETA_GEMM_PAIR: 1 = prefill GEMMs that take 512-token tiles
 *   run as pairs of CTAs sharing one two-CTA tensor-core instruction, 2 = every GEMM does, 0 = none). */
GRETA_API int greta_cuda_set_tuning(const char *name, long long value);
/* Number of kernel launches this library has issued on the calling process (all threads). */
GRETA_API uint64_t greta_cuda_launch_count(void);

/* ------------------------------------------------------------------ formats */
/* Bytes of the qs plane and of the d plane of an [N x K] weight. */
GRETA_API size_t greta_cuda_qs_bytes(int fmt, uint32_t N, uint32_t K);
GRETA_API size_t greta_cuda_d_bytes(int fmt, uint32_t N, uint32_t K);
/* K-quant super-blocks (256 weights; GGML type codes as in a GGUF file).  Decoding follows the reference loader
 * (src/inference/src/weight_loader.cpp:125-177) bit for bit, including its own reading of the two layouts. */
#define GRETA_GGML_Q4_K 12 /* 144 bytes: fp16 d, fp16 dmin, 12 bytes of 6-bit scales and mins, 128 payload bytes */
#define GRETA_GGML_Q6_K 14 /* 210 bytes: 128 low-nibble bytes, 64 high-bit bytes, 16 int8 scales, fp16 d */
/* Bytes of n_elems weights stored as that type; 0 for another type or a count that is not whole super-blocks. */
GRETA_API size_t greta_cuda_kquant_bytes(int ggml_type, size_t n_elems);
/* blocks (device, as in the file) -> n_elems fp32 or fp16 values (GGUFLoader::load_tensor, weight_loader.cpp:551-565). */
GRETA_API int greta_cuda_kquant_dequant(greta_stream_t stream, int ggml_type, const void *blocks, size_t n_elems, void *out, int out_is_f16);
/* blocks of an [N x K] weight -> the qs and d planes of GRETA_FMT_Q8_0 (sizes from greta_cuda_qs_bytes / greta_cuda_d_bytes):
 * each group of 32 decoded values becomes one Q8_0 block, d = amax / 127 rounded to fp16, q = round(x / d).  The reference
 * re-quantises K-quant tensors too, to its INT4 storage (weight_loader.cpp:920-957). */
GRETA_API int greta_cuda_kquant_to_q8_0(greta_stream_t stream, int ggml_type, const void *blocks, void *qs, void *d, uint32_t N, uint32_t K);
/* y[M x N] = x[M x K] * W^T with W [N x K] kept as K-quant super-blocks exactly as in the file (nothing re-quantised): the
 * weight-only GEMV of the reference's M <= 32 route (gemm_kernels.hip:742-760) for the block formats its models are shipped in.
 * x, y fp32; 1 <= M <= 32 (the weights are streamed once per activation row, as the reference's grid(N, M) does). */
GRETA_API int greta_cuda_gemv_kquant(greta_stream_t stream, int ggml_type, const float *x, const void *blocks, float *y, uint32_t M, uint32_t N,
                                     uint32_t K);
/* Device-side split of raw GGUF blocks (18 B Q4_0 / 34 B Q8_0, as stored in a GGUF
 * file: src/inference/src/weight_loader.cpp:60-75 sizes, :703-712 Q8_0 split) into
 * the two planes. */
GRETA_API int greta_cuda_repack_gguf(greta_stream_t stream, int fmt, const void *gguf_blocks, void *qs,
                                     void *d, uint32_t N, uint32_t K);
/* Dequantise to fp32, bit-exact (float)q * fp32(d)
 * (read_weight_value, src/inference/src/block_scheduler.cpp:639-671). */
GRETA_API int greta_cuda_dequant(greta_stream_t stream, int fmt, const void *qs, const void *d,
                                 float *out, uint32_t N, uint32_t K);
GRETA_API int greta_cuda_f32_to_f16(greta_stream_t stream, const float *in, void *out_f16, size_t n);
GRETA_API int greta_cuda_f16_to_f32(greta_stream_t stream, const void *in_f16, float *out, size_t n);

/* ------------------------------------------------------------------ decode GEMV
 * y[M x N] = x[M x K] * dequant(W)^T, fp32 accumulation, fp32 output.
 * Replaces the GEMV route (M <= 32) of launch_gemm_mfma_int4_wt_fp32_acc32 and
 * launch_gemm_mfma_int8_wt_fp32_acc32 (src/rt/backend/hip/kernels/gemm_kernels.hip:
 * 763-817, 594-634, launchers :742-760 and :910-942) and, for GRETA_FMT_F16
 * (qs = fp16 W[N x K], d = NULL), launch_gemm_mixed_f16f32 / launch_lm_head_gemv
 * (:466-507, :533-589).  x is fp32, or fp16 when x_is_f16 != 0 (the INT4 kernel's
 * T_A = __half instantiation).  For the two GRETA_FMT_REF_* formats qs/d are the
 * reference's own planes (d = fp32 scales). */
GRETA_API int greta_cuda_gemv(greta_stream_t stream, int fmt, const void *x, int x_is_f16,
                              const void *qs, const void *d, float *y, uint32_t M, uint32_t N,
                              uint32_t K);

/* y[N] = dequant(W)[N x K] * rmsnorm(x, gamma, eps)   (M = 1): the final norm fused
 * into the LM-head projection (launch_rmsnorm_naive + gemm, block_scheduler.cpp:4207,
 * 4295-4304, on the last position only).  Formats: Q4_0, Q8_0, F16. */
GRETA_API int greta_cuda_rmsnorm_gemv(greta_stream_t stream, int fmt, const float *x, const float *gamma,
                                      float eps, const void *qs, const void *d, float *y, uint32_t N,
                                      uint32_t K);

/* y[N] = resid[N] + dequant(W)[N x K] * x[K]   (M = 1; y may alias resid).
 * O-projection / down-projection followed by the residual add
 * (block_scheduler.cpp:2769-2775 + launch_add :2896; :3003-3006 + :3032). */
GRETA_API int greta_cuda_gemv_residual(greta_stream_t stream, int fmt, const float *x, const void *qs,
                                       const void *d, const float *resid, float *y, uint32_t N,
                                       uint32_t K);

/* Fused decode QKV: xn = rmsnorm(x, gamma, eps); q = Wq xn; k = Wk xn; v = Wv xn;
 * rotate-half RoPE at position *d_pos on q and k; q -> q_out fp32 [H*Dh];
 * k, v -> fp16 caches [Hkv][max_seq][Dh] at row *d_pos.  gamma may be NULL (no
 * norm).  k_out / v_out (fp32 [Hkv*Dh], post-RoPE k) are optional copies.
 * With d_pos == NULL no rotation is applied and nothing is cached: q, k, v go to
 * q_out / k_out / v_out only (all three required then).  Formats: Q4_0, Q8_0, F16.
 * Replaces launch_rmsnorm_naive + 3 x GretaCompute::gemm + 2 x launch_rope +
 * launch_kv_update (block_scheduler.cpp:1814-1977) and is the Q4_0/Q8_0 form of
 * launch_fused_rmsnorm_qkv_gemv_f16 (fused_compute_kernels.hip:22-157) and
 * launch_fused_rope_kv_update_decode (fused_attention_kernels.hip:35-108); it is
 * what GretaFused::rmsnorm_qkv (greta_compute.hpp:68-72) is declared for. */
GRETA_API int greta_cuda_fused_rmsnorm_qkv_rope_kv(
    greta_stream_t stream, int fmt, const float *x, const float *gamma, float eps, const void *wq_qs,
    const void *wq_d, const void *wk_qs, const void *wk_d, const void *wv_qs, const void *wv_d,
    float *q_out, float *k_out, float *v_out, void *k_cache_f16, void *v_cache_f16,
    const uint32_t *d_pos, uint32_t num_heads, uint32_t num_heads_kv, uint32_t head_dim,
    uint32_t max_seq_len, float rope_base, uint32_t D);

/* Fused FFN front: xn = rmsnorm(x, gamma, eps); y[F] = silu(W1 xn) * (W3 xn).
 * gamma may be NULL.  Replaces launch_rmsnorm_naive + 2 x gemm + launch_silu +
 * launch_mul (block_scheduler.cpp:2913-2995); Q4_0/Q8_0 form of
 * launch_fused_ffn_front_f16 (fused_compute_kernels.hip:167-243). */
GRETA_API int greta_cuda_fused_ffn_front(greta_stream_t stream, int fmt, const float *x,
                                         const float *gamma, float eps, const void *w1_qs,
                                         const void *w1_d, const void *w3_qs, const void *w3_d,
                                         float *y, uint32_t D, uint32_t F);

/* ------------------------------------------------------------------ batched decode (M = 1..32 sequences)
 * The same operators for a batch of M sequences that decode in step, each with its own position: the weights are
 * streamed once for all M activation rows (tensor-core block products on exact integer weights, fp32 block sums
 * and scales; the activations keep fp32 precision as a pair of fp16 values).  The reference has no batch
 * dimension: its GEMV route launches grid.y = M and re-reads the weights per row
 * (src/rt/backend/hip/kernels/gemm_kernels.hip:742-760, 910-942), and its scheduler holds one sequence
 * (src/inference/src/block_scheduler.cpp:1490-1494).  Formats: Q4_0, Q8_0, F16.  x is fp32 [M][K], row-major,
 * 16-byte aligned; outputs are [M][...] row-major.  k_slices forces the number of K slices (1, 2, 4 or 8; 0 =
 * chosen from the shape).
 * workspace: greta_cuda_gemv_batch_workspace_bytes(M, K) bytes of device memory, 16-byte aligned, or NULL.  With it the
 * activations are converted once, by a small kernel in front, into the layout the tensor-core kernel consumes; without
 * it every CTA of the matmul kernel repeats that conversion for itself (about 2.5 times slower, same results to the
 * last bit of the fp16 pairs).  One workspace can serve every call on a stream.
 *
 * y[M][N] = (resid ? resid[M][N] : 0) + rmsnorm?(x)[M][K] * dequant(W)^T; gamma == NULL: no norm. */
GRETA_API size_t greta_cuda_gemv_batch_workspace_bytes(uint32_t M, uint32_t K);
GRETA_API int greta_cuda_gemv_batch(greta_stream_t stream, int fmt, const float *x, const float *gamma, float eps,
                                    const void *qs, const void *d, const float *resid, float *y, uint32_t M, uint32_t N,
                                    uint32_t K, uint32_t k_slices, void *workspace);
/* greta_cuda_fused_rmsnorm_qkv_rope_kv for M sequences: q_out [M][H*Dh]; row m is rotated at d_pos[m] and its K / V
 * go to row d_pos[m] of sequence m's cache; caches are fp16 [M][Hkv][max_seq][Dh]. */
GRETA_API int greta_cuda_fused_rmsnorm_qkv_rope_kv_batch(
    greta_stream_t stream, int fmt, const float *x, const float *gamma, float eps, const void *wq_qs, const void *wq_d,
    const void *wk_qs, const void *wk_d, const void *wv_qs, const void *wv_d, float *q_out, float *k_out, float *v_out,
    void *k_cache_f16, void *v_cache_f16, const uint32_t *d_pos, uint32_t M, uint32_t num_heads, uint32_t num_heads_kv,
    uint32_t head_dim, uint32_t max_seq_len, float rope_base, uint32_t D, void *workspace);
/* greta_cuda_fused_ffn_front for M rows: y [M][F]. */
GRETA_API int greta_cuda_fused_ffn_front_batch(greta_stream_t stream, int fmt, const float *x, const float *gamma, float eps,
                                               const void *w1_qs, const void *w1_d, const void *w3_qs, const void *w3_d,
                                               float *y, uint32_t M, uint32_t D, uint32_t F, void *workspace);

/* ------------------------------------------------------------------ whole decode step, one launch
 * All decoder layers of one batch-1 decode step as a single persistent kernel: the five operators
 * above, per layer, as phases of one launch separated by grid-wide barriers, with the weight stream
 * kept in flight across the phases.  Stands in for the per-layer loop of BlockScheduler::forward
 * (src/inference/src/block_scheduler.cpp:4199-4202) replayed from a graph (:4186-4191).  Results are
 * identical to calling the operators one by one.  Single GPU, Q4_0 / Q8_0 weights, M = 1.
 * The caller describes the model once (greta_decode_desc + one greta_decode_layer per layer, all
 * device pointers), provides greta_cuda_decode_plan_bytes() bytes of zeroed device memory for the plan,
 * builds it, then calls greta_cuda_decode_layers once per token: it reads the token id from
 * *d_token, writes its embedding to x, runs the layers at position *d_pos and leaves the final hidden
 * state in x.  Every device-side wait is bounded; greta_cuda_decode_status returns a non-zero code if
 * one ever gave up (the plan memory must then be zeroed and rebuilt). */
typedef struct greta_decode_layer {
  const void *wq_qs, *wq_d, *wk_qs, *wk_d, *wv_qs, *wv_d, *wo_qs, *wo_d, *w1_qs, *w1_d, *w2_qs, *w2_d, *w3_qs, *w3_d;
  const float *attn_norm, *ffn_norm;
  void *k_cache, *v_cache; /* fp16 [Hkv][max_seq][Dh] of this layer */
} greta_decode_layer;
typedef struct greta_decode_desc {
  int weight_fmt;
  uint32_t dim, num_heads, num_heads_kv, head_dim, hidden_dim, max_seq_len, num_layers, vocab_size;
  float rope_base, rms_eps, attn_scale;
  float *x, *q, *attn_out, *mlp_gate;      /* activations: [dim], [H*Dh], [H*Dh], [hidden] */
  const uint32_t *d_pos;
  const int32_t *d_token;
  const void *tok_embd_f16;                /* [vocab][dim] */
  void *attn_scratch;
  size_t attn_scratch_bytes;
} greta_decode_desc;
GRETA_API size_t greta_cuda_decode_plan_bytes(uint32_t num_layers);
GRETA_API int greta_cuda_decode_plan_build(greta_stream_t stream, const greta_decode_desc *desc,
                                           const greta_decode_layer *layers_host, void *plan, size_t plan_bytes);
GRETA_API int greta_cuda_decode_layers(greta_stream_t stream, const greta_decode_desc *desc, void *plan);
GRETA_API int greta_cuda_decode_status(const void *plan, int *code);
/* Timing probe: SM clock stamps taken by CTA 0 in layer 1 of the last step, 5 phases (QKV, attention, O,
 * gate/up, down) x 5 marks (phase start, activations staged, weights consumed, epilogue done, barrier
 * passed).  Synchronises. */
GRETA_API int greta_cuda_decode_trace(const void *plan, long long *out25);

/* ------------------------------------------------------------------ prefill GEMM
 * C[M x N] = half(A[M x K]) * half(dequant(W))^T, fp32 accumulation on the
 * tensor cores (tcgen05, TMEM accumulators); A fp32 or fp16, C fp32 or fp16.
 * Replaces the M > 32 route: gemm_mfma_int4_wt_kernel / gemm_mfma_int8_wt_kernel
 * (gemm_kernels.hip:820-908, 640-740) with the row-major contraction.
 * workspace: device scratch of greta_cuda_gemm_workspace_bytes(M, K) bytes: room for the partial sums of a K loop
 * shared between CTAs (one 128 x 512 fp32 tile per SM, used when the product has fewer 512-token tiles than the GPU has
 * SMs) followed by the fp16 copy of A when A is fp32.  May be NULL when a_is_f16: the product is then computed with
 * fixed tiles only.  Its contents need not be initialised or kept; two products that may run at the same time
 * (different streams) need a workspace each. */
GRETA_API size_t greta_cuda_gemm_workspace_bytes(uint32_t M, uint32_t K);
/* Which kernel greta_cuda_gemm would take for a shape under the tuning switches as they stand (nothing is launched):
 * *kind 0 = fixed tiles of *tile_tokens tokens x 128 rows, 1 = CTA pairs, 2 = K loops shared between CTAs; *ctas = CTAs of the
 * launch, *share = K stages (of 64) each CTA runs. */
GRETA_API int greta_cuda_gemm_route(uint32_t M, uint32_t N, uint32_t K, int has_workspace, int *kind, uint32_t *ctas, uint32_t *share,
                                    uint32_t *tile_tokens);
/* Every wait inside the GEMM kernel is bounded; if one ever gives up the kernel drains, frees its tensor
 * memory and records a non-zero code (100 * role + stage) that this call returns in *code (0 = none).
 * Synchronises with the device. */
GRETA_API int greta_cuda_gemm_status(int *code);
GRETA_API int greta_cuda_gemm(greta_stream_t stream, int fmt, const void *A, int a_is_f16,
                              const void *qs, const void *d, void *C, int c_is_f16, uint32_t M,
                              uint32_t N, uint32_t K, void *workspace);

/* ------------------------------------------------------------------ attention
 * Decode attention of one query per head over the fp16 KV cache
 * [Hkv][max_seq][Dh], split over the sequence; seq_len = *d_pos + 1 when d_pos
 * is non-NULL, else `seq_len`.  scratch: greta_cuda_attn_decode_scratch_bytes()
 * bytes of device memory for the per-split partial results.
 * Replaces launch_flash_attention_decode (attention_kernels.hip:167-380) behind
 * GretaCompute::attention_decode (src/compute/src/greta_compute_hip.cpp:376-412). */
GRETA_API size_t greta_cuda_attn_decode_scratch_bytes(uint32_t num_heads, uint32_t head_dim);
GRETA_API int greta_cuda_attn_decode(greta_stream_t stream, const float *q, const void *k_cache_f16,
                                     const void *v_cache_f16, float *o, const uint32_t *d_pos,
                                     uint32_t seq_len, uint32_t num_heads, uint32_t num_heads_kv,
                                     uint32_t head_dim, uint32_t max_seq_len, float scale,
                                     void *scratch, size_t scratch_bytes);
/* Same with an fp32 cache, the reference's own cache type (block_scheduler.cpp:1490-1494). */
GRETA_API int greta_cuda_attn_decode_f32cache(greta_stream_t stream, const float *q,
                                              const float *k_cache, const float *v_cache, float *o,
                                              const uint32_t *d_pos, uint32_t seq_len,
                                              uint32_t num_heads, uint32_t num_heads_kv,
                                              uint32_t head_dim, uint32_t max_seq_len, float scale,
                                              void *scratch, size_t scratch_bytes);
/* Decode attention for a batch of M sequences that decode in step: q, o fp32 [M][H*Dh]; fp16 caches
 * [M][Hkv][max_seq][Dh]; sequence m attends to its keys 0..d_pos[m].  With 2..16 query heads per KV head (grouped-query
 * attention) one CTA serves all query heads of a KV head from one staged copy of its keys, so the cache is read once per
 * KV head; otherwise the per-head kernels run with one (sequence, head) per CTA group.  scratch: greta_cuda_attn_decode_
 * scratch_bytes(M * H, Dh) bytes (tickets zero before the first call), used by the per-head scratch-merge route only.
 * The reference has no batch dimension (one cache per layer, src/inference/src/block_scheduler.cpp:1490-1494); per
 * sequence this is launch_flash_attention_decode (attention_kernels.hip:167-380). */
GRETA_API int greta_cuda_attn_decode_batch(greta_stream_t stream, const float *q, const void *k_cache_f16,
                                           const void *v_cache_f16, float *o, const uint32_t *d_pos, uint32_t M,
                                           uint32_t num_heads, uint32_t num_heads_kv, uint32_t head_dim, uint32_t max_seq_len,
                                           float scale, void *scratch, size_t scratch_bytes);
/* Decode attention for callers that must not allocate and have no scratch to lend.  No counterpart in
 * the reference: its launchers take no scratch argument because its attention kernel needs none, and
 * the split-sequence kernel here does.  Such callers are, for example, a host application that gives
 * this library raw pointers out of a memory pool it owns in full (a fixed budget, no cudaMalloc allowed
 * after start-up), or code on a latency-critical serving path where cudaMalloc / cudaFree would
 * synchronise the whole device.  Same arguments and results as greta_cuda_attn_decode (fp16 cache), minus
 * the scratch: this entry always runs the scratch-merge kernel (never the cluster kernel, which needs no
 * scratch), and the per-split partial results and per-head tickets go to an array built into the library, about 1 MiB that every GPU
 * loading the library holds until the process exits.  Limit: num_heads <= 64 and head_dim <= 128 (larger
 * shapes are rejected with GRETA_ERR_INVALID_ARGS; use greta_cuda_attn_decode).  The call allocates
 * nothing.  Its first call on a device looks up the array's device address; make that call outside any
 * stream capture.  All calls share the one array and it keeps the last call's contents (the call clears
 * the words that must start at zero), so two calls that may overlap on the GPU - different streams without
 * an ordering between them - race; keep them on one stream or order them with events. */
GRETA_API int greta_cuda_attn_decode_static(greta_stream_t stream, const float *q, const void *k_cache_f16,
                                            const void *v_cache_f16, float *o, const uint32_t *d_pos,
                                            uint32_t seq_len, uint32_t num_heads, uint32_t num_heads_kv,
                                            uint32_t head_dim, uint32_t max_seq_len, float scale);
/* Causal prefill attention: q [S][H][Dh] fp32 against rows [pos0, pos0+S) of the
 * fp16 cache (keys 0 .. pos0+s for query s), o [S][H][Dh] fp32.
 * Replaces launch_flash_attention_prefill (attention_kernels.hip:543-618). */
GRETA_API int greta_cuda_attn_prefill(greta_stream_t stream, const float *q, const void *k_cache_f16,
                                      const void *v_cache_f16, float *o, uint32_t S, uint32_t pos0,
                                      uint32_t num_heads, uint32_t num_heads_kv, uint32_t head_dim,
                                      uint32_t max_seq_len, float scale);
/* The reference's own prefill entry, launch_flash_attention_prefill (attention_kernels.hpp:124-128, kernel
 * attention_kernels.hip:543-618): q, o fp32 [S][H][Dh]; k, v fp32 [S][Hkv][Dh] (the prompt's own keys, not a cache);
 * causal != 0: query s sees keys 0..s, else all S. */
GRETA_API int greta_cuda_attn_prefill_f32(greta_stream_t stream, const float *q, const float *k, const float *v, float *o,
                                          uint32_t S, uint32_t num_heads, uint32_t num_heads_kv, uint32_t head_dim,
                                          float scale, int causal);
/* RoPE in place on x [S][H][Dh]; position pos_offset + s, or *d_pos + s when
 * d_pos != NULL.  launch_rope, both overloads (attention_kernels.hip:28-84). */
GRETA_API int greta_cuda_rope(greta_stream_t stream, float *x, uint32_t S, uint32_t num_heads,
                              uint32_t head_dim, float base, uint32_t pos_offset,
                              const uint32_t *d_pos);
/* Write S new K/V rows (fp32 [S][Hkv][Dh]) into the fp16 caches at rows pos.. .
 * launch_kv_update, both overloads (attention_kernels.hip:103-158), without the
 * reference's one-launch-per-token loop in prefill (block_scheduler.cpp:1970-1976). */
GRETA_API int greta_cuda_kv_update(greta_stream_t stream, void *k_cache_f16, void *v_cache_f16,
                                   const float *new_k, const float *new_v, uint32_t S,
                                   uint32_t pos, const uint32_t *d_pos, uint32_t max_seq_len,
                                   uint32_t num_heads_kv, uint32_t head_dim);

/* ------------------------------------------------------------------ small operators */
/* launch_rmsnorm_naive (basic_kernels.hip:21-64); also what GretaCompute::rmsnorm
 * (greta_compute_hip.cpp:414-419, an empty placeholder in the reference) calls. */
GRETA_API int greta_cuda_rmsnorm(greta_stream_t stream, const float *x, const float *gamma, float *y,
                                 uint32_t rows, uint32_t cols, float eps);
/* launch_add (basic_kernels.hip:127-140). */
GRETA_API int greta_cuda_add(greta_stream_t stream, const float *a, const float *b, float *c, size_t n);
/* launch_silu, launch_mul (basic_kernels.hip:141-167), separately. */
GRETA_API int greta_cuda_silu(greta_stream_t stream, const float *x, float *y, size_t n);
GRETA_API int greta_cuda_mul(greta_stream_t stream, const float *a, const float *b, float *c, size_t n);
/* launch_silu then launch_mul in one pass (basic_kernels.hip:141-167): y = silu(gate) * up. */
GRETA_API int greta_cuda_silu_mul(greta_stream_t stream, const float *gate, const float *up, float *y,
                                  size_t n);
/* launch_embedding_lookup, row-major table (basic_kernels.hip:169-206); table fp16
 * (table_is_f16) or fp32; ids outside [0, vocab) give zeros. */
GRETA_API int greta_cuda_embedding(greta_stream_t stream, const int32_t *tokens, const void *table,
                                   int table_is_f16, float *out, uint32_t S, uint32_t dim,
                                   uint32_t vocab);
/* launch_argmax (basic_kernels.hip:330-373) without its per-call allocation and
 * synchronisation: writes the index of the first maximum to *d_out (device). */
GRETA_API int greta_cuda_argmax(greta_stream_t stream, const float *logits, uint32_t n, int32_t *d_out);
/* Arg-max that also closes a decode step on the device, so the next step can start
 * without a host round trip (the reference returns to the host for every token,
 * generator.cpp:1142-1156): *d_next = id; d_out_tokens[*d_count] = id when
 * *d_count < out_capacity; ++*d_count; ++*d_pos. */
GRETA_API int greta_cuda_argmax_advance(greta_stream_t stream, const float *logits, uint32_t n,
                                        int32_t *d_next, uint32_t *d_pos, int32_t *d_out_tokens,
                                        uint32_t *d_count, uint32_t out_capacity);

/* The same for `batch` sequences: logits [batch][n]; d_next, d_pos, d_count are arrays of `batch`; sequence b's ids go
 * to d_out_tokens[b * out_capacity + ...]. */
GRETA_API int greta_cuda_argmax_advance_batch(greta_stream_t stream, const float *logits, uint32_t n, uint32_t batch,
                                              int32_t *d_next, uint32_t *d_pos, int32_t *d_out_tokens, uint32_t *d_count,
                                              uint32_t out_capacity);

/* ------------------------------------------------------------------ tensor-parallel exchange
 * The reference is single-GPU (hipSetDevice(0), greta_runtime_hip.cpp:153); these are new.
 * One process per GPU; NCCL over NVLink / NVSwitch.  unique_id128 is a 128-byte buffer made on
 * rank 0 and handed to every rank by the launcher. */
GRETA_API int greta_cuda_comm_unique_id(void *unique_id128);
GRETA_API int greta_cuda_comm_init(void **comm, const void *unique_id128, int nranks, int rank);
GRETA_API int greta_cuda_comm_destroy(void *comm);
/* In-place sum over ranks of `count` floats, enqueued on `stream` (capturable into a graph). */
GRETA_API int greta_cuda_comm_allreduce_f32(void *comm, float *buf, size_t count, greta_stream_t stream);

/* ---- Tensor-parallel exchange fused into the operators, over peer memory (NVLink) ----------------
 * The reference has no counterpart (it is single-GPU); this replaces "row-parallel projection, then
 * all-reduce, then the next operator's RMSNorm" of a Megatron-sharded decoder layer
 * by two kernels and no collective launch:
 *   producer  greta_cuda_gemv_peer_scatter: y_r = x W_r^T, every element stored as {value, tag} straight into
 *             slot r of EVERY rank's slot buffer (plain 8-byte stores over NVLink; no flag, no fence: the tag
 *             travels with the value);
 *   consumer  ..._peer forms of the fused QKV and FFN-front operators: the activation staging waits (bounded)
 *             for the tp tagged partials in the local slot buffer, adds them to the residual stream x_in in
 *             rank order (bit-identical on every rank), normalises and goes on; the new stream is written
 *             to x_out (a different buffer from x_in).  From 4 ranks on the gather has two levels: the CTAs
 *             split the vector, each sums its blocks of 32 once and publishes the tagged sums in the local
 *             buffer, and every CTA then reads dim summed words instead of tp x dim partial words.
 * Tags are ((*d_pos + 1) << 8) | exch_idx: they grow with the position, so a slot buffer must be zeroed,
 * on every rank and with a barrier after it, whenever a decode session restarts at an earlier position.
 * Consecutive exchanges must alternate exch_idx parity (two halves of the slot buffer), or be separated by
 * a collective.  A wait that gives up sets a status word (greta_cuda_peer_status) and uses what it has.
 * Slot buffers are plain device allocations shared between the processes with the ipc calls below. */
typedef struct greta_peer_exchange {
  uint32_t tp, rank;   /* ranks of the group (<= 8), this rank */
  void *slots[8];      /* slot buffer of every rank, the same size on all; slots[rank] is local */
  uint64_t slot_bytes; /* size of each slot buffer: at least greta_cuda_peer_slot_bytes(tp, dim); greta_cuda_peer_allreduce_f32
                          wants greta_cuda_peer_allreduce_slot_bytes(count).  0 is read as greta_cuda_peer_slot_bytes(tp, dim). */
} greta_peer_exchange;
GRETA_API size_t greta_cuda_peer_slot_bytes(uint32_t tp, uint32_t dim);
GRETA_API int greta_cuda_peer_status(int *code);
/* Clears the status word (on `stream`): after a time-out every later wait gives up at once until this is called. */
GRETA_API int greta_cuda_peer_reset(greta_stream_t stream);
/* In-place sum of `count` floats over the ranks through the slot buffers: one kernel per rank, no collective launch
 * (scatter of slices, sum in rank order by the slice's owner, gather; every rank receives the same bits).  Meant for
 * the [batch x dim] partial products of a batch of sequences, where the exchange cannot ride in a GEMV epilogue; count must
 * divide by tp.  Tags and the alternation of exch_idx parity as above; d_pos points at the first sequence's position.
 * Waits are bounded like those of the fused exchange (greta_cuda_peer_status). */
GRETA_API size_t greta_cuda_peer_allreduce_slot_bytes(size_t max_count);
GRETA_API int greta_cuda_peer_allreduce_f32(greta_stream_t stream, float *x, size_t count, const greta_peer_exchange *ex, uint32_t exch_idx,
                                            const uint32_t *d_pos);
GRETA_API int greta_cuda_ipc_export(void *device_ptr, void *handle64);         /* 64-byte handle of a greta_cuda_malloc block */
GRETA_API int greta_cuda_ipc_open(const void *handle64, void **device_ptr);    /* maps another process's block */
GRETA_API int greta_cuda_ipc_close(void *device_ptr);
GRETA_API int greta_cuda_gemv_peer_scatter(greta_stream_t stream, int fmt, const float *x, const void *qs, const void *d,
                                           const greta_peer_exchange *ex, uint32_t exch_idx, const uint32_t *d_pos, uint32_t N, uint32_t K);
GRETA_API int greta_cuda_fused_rmsnorm_qkv_rope_kv_peer(greta_stream_t stream, int fmt, const float *x_in, float *x_out,
                                                        const greta_peer_exchange *ex, uint32_t exch_idx, const float *gamma, float eps,
                                                        const void *wq_qs, const void *wq_d, const void *wk_qs, const void *wk_d,
                                                        const void *wv_qs, const void *wv_d, float *q_out, void *k_cache, void *v_cache,
                                                        const uint32_t *d_pos, uint32_t H, uint32_t Hkv, uint32_t Dh, uint32_t max_seq,
                                                        float rope_base, uint32_t D);
GRETA_API int greta_cuda_fused_ffn_front_peer(greta_stream_t stream, int fmt, const float *x_in, float *x_out,
                                              const greta_peer_exchange *ex, uint32_t exch_idx, const uint32_t *d_pos, const float *gamma,
                                              float eps, const void *w1_qs, const void *w1_d, const void *w3_qs, const void *w3_d, float *y,
                                              uint32_t D, uint32_t F);

#ifdef __cplusplus
}
#endif
#endif /* GRETA_CUDA_H */
