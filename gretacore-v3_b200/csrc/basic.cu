// Format conversion and the small element-wise / reduction operators of the
// decode path (norm, residual add, SwiGLU, embedding gather, greedy arg-max).
#include "greta_common.cuh"

using namespace greta;
static inline cudaStream_t S(greta_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

namespace {

// One thread per GGUF block: splits {fp16 d; payload} into the two planes.
template <int FMT>
__global__ void repack_kernel(const uint8_t *__restrict__ blocks, uint8_t *__restrict__ qs,
                              uint16_t *__restrict__ d, size_t n_blocks, uint32_t nb_row) {
  constexpr int PB = payload_bytes(FMT), BB = PB + 2;
  size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_blocks) return;
  const uint8_t *src = blocks + b * BB;   // 2-byte aligned only (18 / 34 byte stride)
  const uint16_t *s16 = reinterpret_cast<const uint16_t *>(src);
  d[(b / nb_row) * d_row_stride(nb_row) + b % nb_row] = s16[0];
  uint16_t *dst = reinterpret_cast<uint16_t *>(qs + b * PB);
#pragma unroll
  for (int i = 0; i < PB / 2; ++i) dst[i] = s16[1 + i];
}

// One thread per block of 32 weights; bit-exact (float)q * fp32(d).
template <int FMT>
__global__ void dequant_kernel(const uint8_t *__restrict__ qs, const void *__restrict__ d,
                               float *__restrict__ out, size_t n_blocks, uint32_t nb_row) {
  size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_blocks) return;
  const size_t sb = (b / nb_row) * d_row_stride(nb_row) + b % nb_row;  // index in the padded fp16 d plane
  float *o = out + b * 32;
  if (FMT == GRETA_FMT_Q4_0) {
    float s = __half2float(reinterpret_cast<const __half *>(d)[sb]);
    const uint8_t *p = qs + b * 16;
    for (int j = 0; j < 16; ++j) {
      o[j] = __fmul_rn((float)((int)(p[j] & 0xF) - 8), s);
      o[j + 16] = __fmul_rn((float)((int)(p[j] >> 4) - 8), s);
    }
  } else if (FMT == GRETA_FMT_Q8_0) {
    float s = __half2float(reinterpret_cast<const __half *>(d)[sb]);
    const int8_t *p = reinterpret_cast<const int8_t *>(qs) + b * 32;
    for (int j = 0; j < 32; ++j) o[j] = __fmul_rn((float)p[j], s);
  } else if (FMT == GRETA_FMT_REF_INT4) {
    float s = reinterpret_cast<const float *>(d)[b];
    const uint8_t *p = qs + b * 16;
    for (int j = 0; j < 16; ++j) {
      int lo = p[j] & 0xF, hi = p[j] >> 4;
      o[2 * j] = __fmul_rn((float)(lo >= 8 ? lo - 16 : lo), s);
      o[2 * j + 1] = __fmul_rn((float)(hi >= 8 ? hi - 16 : hi), s);
    }
  } else {  // REF_INT8
    float s = reinterpret_cast<const float *>(d)[b];
    const int8_t *p = reinterpret_cast<const int8_t *>(qs) + b * 32;
    for (int j = 0; j < 32; ++j) o[j] = __fmul_rn((float)p[j], s);
  }
}

__global__ void f32_to_f16_kernel(const float *__restrict__ in, __half *__restrict__ out, size_t n) {
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    float4 v = *reinterpret_cast<const float4 *>(in + i);
    __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t *>(&a);
    o.y = *reinterpret_cast<uint32_t *>(&b);
    *reinterpret_cast<uint2 *>(out + i) = o;
  } else {
    for (; i < n; ++i) out[i] = __float2half_rn(in[i]);
  }
}
__global__ void f16_to_f32_kernel(const __half *__restrict__ in, float *__restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __half2float(in[i]);
}

__device__ __forceinline__ float block_sum(float v, float *sm) {
  v = warp_sum(v);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) sm[w] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? sm[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) sm[0] = t;
  }
  __syncthreads();
  t = sm[0];
  __syncthreads();
  return t;
}

// One CTA per row: y = (x * rsqrt(mean(x^2) + eps)) * gamma.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                                                      float *__restrict__ y, uint32_t cols, float eps) {
  __shared__ float sm[32];
  const float *xr = x + (size_t)blockIdx.x * cols;
  float *yr = y + (size_t)blockIdx.x * cols;
  float ss = 0.f;
  for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
  ss = block_sum(ss, sm);
  float inv = rsqrtf(ss / (float)cols + eps);
  for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) yr[c] = (xr[c] * inv) * gamma[c];
}

__global__ void add_kernel(const float *a, const float *b, float *c, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) c[i] = a[i] + b[i];
}
__global__ void silu_kernel(const float *x, float *y, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    float v = x[i];
    y[i] = v / (1.0f + expf(-v));
  }
}
__global__ void mul_kernel(const float *a, const float *b, float *c, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) c[i] = a[i] * b[i];
}
__global__ void silu_mul_kernel(const float *g, const float *u, float *y, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    float v = g[i];
    y[i] = (v / (1.0f + expf(-v))) * u[i];
  }
}

template <bool F16>
__global__ void embedding_kernel(const int32_t *__restrict__ tokens, const void *__restrict__ table,
                                 float *__restrict__ out, uint32_t S, uint32_t dim, uint32_t vocab) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)S * dim) return;
  uint32_t s = i / dim, dd = i % dim;
  int32_t t = tokens[s];
  float v = 0.f;
  if (t >= 0 && t < (int32_t)vocab) {
    size_t src = (size_t)t * dim + dd;
    v = F16 ? __half2float(reinterpret_cast<const __half *>(table)[src]) : reinterpret_cast<const float *>(table)[src];
  }
  out[i] = v;
}

// One CTA of 1024 threads per row of logits (per sequence of a batch): first maximum (lowest index among equal values).
__global__ void __launch_bounds__(1024) argmax_kernel(const float *__restrict__ logits, uint32_t n,
                                                      int32_t *__restrict__ out, uint32_t *d_pos, int32_t *out_tokens,
                                                      uint32_t *d_count, uint32_t out_capacity) {
  __shared__ float sv[32];
  __shared__ uint32_t si[32];
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t b = blockIdx.x;  // sequence: its own logits row, result, position, counter and output list
  logits += (size_t)b * n;
  out += b;
  if (d_pos) d_pos += b;
  if (d_count) d_count += b;
  if (out_tokens) out_tokens += (size_t)b * out_capacity;
  float best = -INFINITY;
  uint32_t bi = 0xffffffffu;
  for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
    float v = logits[i];
    if (v > best || bi == 0xffffffffu) {   // strided scan keeps the lowest index of this thread's maximum
      best = v;
      bi = i;
    }
  }
  auto better = [](float v, uint32_t i, float bv, uint32_t bidx) { return v > bv || (v == bv && i < bidx); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, best, bi)) {
      best = ov;
      bi = oi;
    }
  }
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) {
    sv[w] = best;
    si[w] = bi;
  }
  __syncthreads();
  if (w == 0) {
    best = sv[l];
    bi = si[l];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, best, bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (l == 0) {
      *out = (int32_t)bi;
      if (d_count) {
        uint32_t c = *d_count;
        if (out_tokens && c < out_capacity) out_tokens[c] = (int32_t)bi;
        *d_count = c + 1;
      }
      if (d_pos) *d_pos = *d_pos + 1;
    }
  }
}

inline unsigned blocks_for(size_t n, unsigned t) { return (unsigned)((n + t - 1) / t); }

}  // namespace

extern "C" {

size_t greta_cuda_qs_bytes(int fmt, uint32_t N, uint32_t K) {
  return (size_t)N * (K / 32) * payload_bytes(fmt);
}
size_t greta_cuda_d_bytes(int fmt, uint32_t N, uint32_t K) {
  if (fmt == GRETA_FMT_F16) return 0;
  if (fmt == GRETA_FMT_REF_INT4 || fmt == GRETA_FMT_REF_INT8) return (size_t)N * (K / 32) * 4;
  return (size_t)N * d_row_stride(K / 32) * 2;
}

int greta_cuda_repack_gguf(greta_stream_t stream, int fmt, const void *blocks, void *qs, void *d, uint32_t N,
                           uint32_t K) {
  GRETA_REQUIRE(fmt == GRETA_FMT_Q4_0 || fmt == GRETA_FMT_Q8_0, "repack_gguf: format %d is not a GGUF block format", fmt);
  GRETA_REQUIRE(K % 32 == 0, "repack_gguf: K=%u is not a multiple of 32", K);
  size_t nb = (size_t)N * (K / 32);
  if (nb == 0) return GRETA_OK;
  GRETA_REQUIRE(blocks && qs && d, "repack_gguf: null pointer");
  GRETA_REQUIRE(((uintptr_t)blocks & 1) == 0 && aligned16(qs) && ((uintptr_t)d & 1) == 0, "repack_gguf: misaligned pointer");
  if (d_row_stride(K / 32) != K / 32) GRETA_CUDA_TRY(cudaMemsetAsync(d, 0, greta_cuda_d_bytes(fmt, N, K), S(stream)));  // row padding
  if (fmt == GRETA_FMT_Q4_0)
    repack_kernel<GRETA_FMT_Q4_0><<<blocks_for(nb, 256), 256, 0, S(stream)>>>((const uint8_t *)blocks, (uint8_t *)qs, (uint16_t *)d, nb, K / 32);
  else
    repack_kernel<GRETA_FMT_Q8_0><<<blocks_for(nb, 256), 256, 0, S(stream)>>>((const uint8_t *)blocks, (uint8_t *)qs, (uint16_t *)d, nb, K / 32);
  return launched("repack_kernel");
}

int greta_cuda_dequant(greta_stream_t stream, int fmt, const void *qs, const void *d, float *out, uint32_t N, uint32_t K) {
  GRETA_REQUIRE(K % 32 == 0, "dequant: K=%u is not a multiple of 32", K);
  size_t nb = (size_t)N * (K / 32);
  if (nb == 0) return GRETA_OK;
  GRETA_REQUIRE(qs && d && out, "dequant: null pointer");
  unsigned g = blocks_for(nb, 128);
  switch (fmt) {
    case GRETA_FMT_Q4_0: dequant_kernel<GRETA_FMT_Q4_0><<<g, 128, 0, S(stream)>>>((const uint8_t *)qs, d, out, nb, K / 32); break;
    case GRETA_FMT_Q8_0: dequant_kernel<GRETA_FMT_Q8_0><<<g, 128, 0, S(stream)>>>((const uint8_t *)qs, d, out, nb, K / 32); break;
    case GRETA_FMT_REF_INT4: dequant_kernel<GRETA_FMT_REF_INT4><<<g, 128, 0, S(stream)>>>((const uint8_t *)qs, d, out, nb, K / 32); break;
    case GRETA_FMT_REF_INT8: dequant_kernel<GRETA_FMT_REF_INT8><<<g, 128, 0, S(stream)>>>((const uint8_t *)qs, d, out, nb, K / 32); break;
    default: GRETA_REQUIRE(false, "dequant: unsupported format %d", fmt);
  }
  return launched("dequant_kernel");
}

int greta_cuda_f32_to_f16(greta_stream_t stream, const float *in, void *out, size_t n) {
  if (n == 0) return GRETA_OK;
  GRETA_REQUIRE(in && out, "f32_to_f16: null pointer");
  GRETA_REQUIRE(aligned16(in) && ((uintptr_t)out & 7) == 0, "f32_to_f16: misaligned pointer");
  f32_to_f16_kernel<<<blocks_for((n + 3) / 4, 256), 256, 0, S(stream)>>>(in, (__half *)out, n);
  return launched("f32_to_f16_kernel");
}
int greta_cuda_f16_to_f32(greta_stream_t stream, const void *in, float *out, size_t n) {
  if (n == 0) return GRETA_OK;
  GRETA_REQUIRE(in && out, "f16_to_f32: null pointer");
  f16_to_f32_kernel<<<blocks_for(n, 256), 256, 0, S(stream)>>>((const __half *)in, out, n);
  return launched("f16_to_f32_kernel");
}

int greta_cuda_rmsnorm(greta_stream_t stream, const float *x, const float *gamma, float *y, uint32_t rows, uint32_t cols, float eps) {
  if (rows == 0 || cols == 0) return GRETA_OK;
  GRETA_REQUIRE(x && gamma && y, "rmsnorm: null pointer");
  rmsnorm_kernel<<<rows, 256, 0, S(stream)>>>(x, gamma, y, cols, eps);
  return launched("rmsnorm_kernel");
}
int greta_cuda_add(greta_stream_t stream, const float *a, const float *b, float *c, size_t n) {
  if (n == 0) return GRETA_OK;
  GRETA_REQUIRE(a && b && c, "add: null pointer");
  add_kernel<<<blocks_for(n, 256), 256, 0, S(stream)>>>(a, b, c, n);
  return launched("add_kernel");
}
int greta_cuda_silu_mul(greta_stream_t stream, const float *g, const float *u, float *y, size_t n) {
  if (n == 0) return GRETA_OK;
  GRETA_REQUIRE(g && u && y, "silu_mul: null pointer");
  silu_mul_kernel<<<blocks_for(n, 256), 256, 0, S(stream)>>>(g, u, y, n);
  return launched("silu_mul_kernel");
}
int greta_cuda_embedding(greta_stream_t stream, const int32_t *tokens, const void *table, int table_is_f16, float *out,
                         uint32_t Sq, uint32_t dim, uint32_t vocab) {
  size_t n = (size_t)Sq * dim;
  if (n == 0) return GRETA_OK;
  GRETA_REQUIRE(tokens && table && out, "embedding: null pointer");
  if (table_is_f16)
    GRETA_CUDA_TRY(launch_pdl(embedding_kernel<true>, dim3(blocks_for(n, 256)), dim3(256), 0, S(stream), tokens, table, out, Sq, dim, vocab));
  else
    GRETA_CUDA_TRY(launch_pdl(embedding_kernel<false>, dim3(blocks_for(n, 256)), dim3(256), 0, S(stream), tokens, table, out, Sq, dim, vocab));
  return launched("embedding_kernel");
}
int greta_cuda_argmax(greta_stream_t stream, const float *logits, uint32_t n, int32_t *d_out) {
  GRETA_REQUIRE(n > 0, "argmax: empty input");
  GRETA_REQUIRE(logits && d_out, "argmax: null pointer");
  GRETA_CUDA_TRY(launch_pdl(argmax_kernel, dim3(1), dim3(1024), 0, S(stream), logits, n, d_out, (uint32_t *)nullptr, (int32_t *)nullptr,
                            (uint32_t *)nullptr, 0u));
  return launched("argmax_kernel");
}
int greta_cuda_argmax_advance(greta_stream_t stream, const float *logits, uint32_t n, int32_t *d_next, uint32_t *d_pos,
                              int32_t *d_out_tokens, uint32_t *d_count, uint32_t out_capacity) {
  GRETA_REQUIRE(n > 0, "argmax_advance: empty input");
  GRETA_REQUIRE(logits && d_next, "argmax_advance: null pointer");
  GRETA_CUDA_TRY(launch_pdl(argmax_kernel, dim3(1), dim3(1024), 0, S(stream), logits, n, d_next, d_pos, d_out_tokens, d_count, out_capacity));
  return launched("argmax_kernel");
}
int greta_cuda_argmax_advance_batch(greta_stream_t stream, const float *logits, uint32_t n, uint32_t batch, int32_t *d_next, uint32_t *d_pos,
                                    int32_t *d_out_tokens, uint32_t *d_count, uint32_t out_capacity) {
  GRETA_REQUIRE(n > 0 && batch >= 1 && batch <= 65535, "argmax_advance_batch: n=%u, batch=%u", n, batch);
  GRETA_REQUIRE(logits && d_next, "argmax_advance_batch: null pointer");
  GRETA_CUDA_TRY(launch_pdl(argmax_kernel, dim3(batch), dim3(1024), 0, S(stream), logits, n, d_next, d_pos, d_out_tokens, d_count, out_capacity));
  return launched("argmax_kernel");
}
int greta_cuda_silu(greta_stream_t stream, const float *x, float *y, size_t n) {
  if (n == 0) return GRETA_OK;
  GRETA_REQUIRE(x && y, "silu: null pointer");
  silu_kernel<<<blocks_for(n, 256), 256, 0, S(stream)>>>(x, y, n);
  return launched("silu_kernel");
}
int greta_cuda_mul(greta_stream_t stream, const float *a, const float *b, float *c, size_t n) {
  if (n == 0) return GRETA_OK;
  GRETA_REQUIRE(a && b && c, "mul: null pointer");
  mul_kernel<<<blocks_for(n, 256), 256, 0, S(stream)>>>(a, b, c, n);
  return launched("mul_kernel");
}

}  // extern "C"
