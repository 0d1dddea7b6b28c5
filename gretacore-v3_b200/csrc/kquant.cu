// K-quant super-blocks (GGUF Q4_K and Q6_K, 256 weights each) on the device: decoding to fp32 / fp16 and
// re-storing as the planar Q8_0 layout the matmul kernels read.
//
// The decoding is the reference loader's (src/inference/src/weight_loader.cpp:125-156 Q4_K, :158-177 Q6_K),
// which reads both layouts in its own way: in Q4_K byte l of sub-block j carries elements 2l and 2l+1 of that
// sub-block, and scale / min entries 4..7 are (byte j >> 6) | (nibble of byte 4 + j/2 resp. 10 + j/2) << 2; in Q6_K
// element i takes nibble i of ql, bit pair i of qh and scale i / 16.  Every value is computed with the reference's
// fp32 operations in its order (no fused multiply-add), so the results are the loader's bit for bit.
//
// The reference then re-quantises such tensors to its INT4 storage (weight_loader.cpp:920-957).  Here they are
// re-stored as Q8_0 blocks instead (d = amax / 127, the quantiser published with the format), which the decode and
// prefill kernels stream like any Q8_0 weight.
#include "greta_common.cuh"

using namespace greta;

namespace {

constexpr int Q4_K_BYTES = 144, Q6_K_BYTES = 210;

// The 32 values of sub-block j (0..7) of one super-block.
template <int TYPE>
__device__ __forceinline__ void decode_sub_block(const uint8_t *blk, int j, float (&v)[32]) {
  if (TYPE == GRETA_GGML_Q4_K) {
    const uint8_t *sc = blk + 4, *qs = blk + 16 + j * 16;
    const float d = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(blk[2] | (blk[3] << 8))));
    uint32_t s6, m6;
    if (j < 4) {
      s6 = sc[j] & 0x3F;
      m6 = sc[6 + j] & 0x3F;
    } else {
      const int i = j - 4;
      const uint32_t ns = (i & 1) ? (sc[4 + i / 2] >> 4) : (sc[4 + i / 2] & 0x0F);
      const uint32_t nm = (i & 1) ? (sc[10 + i / 2] >> 4) : (sc[10 + i / 2] & 0x0F);
      s6 = ((uint32_t)sc[i] >> 6) | (ns << 2);
      m6 = ((uint32_t)sc[6 + i] >> 6) | (nm << 2);
    }
    const float scale = __fmul_rn(d, (float)s6), minv = __fmul_rn(dmin, (float)m6);
#pragma unroll
    for (int l = 0; l < 16; ++l) {
      const uint32_t q = qs[l];
      v[2 * l] = __fsub_rn(__fmul_rn(scale, (float)(q & 0x0F)), minv);
      v[2 * l + 1] = __fsub_rn(__fmul_rn(scale, (float)(q >> 4)), minv);
    }
  } else {
    const uint8_t *ql = blk + j * 16, *qh = blk + 128 + j * 8;
    const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192) + j * 2;
    const float d = __half2float(__ushort_as_half((unsigned short)(blk[208] | (blk[209] << 8))));
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int lo = (ql[i / 2] >> ((i % 2) * 4)) & 0x0F, hi = (qh[i / 4] >> ((i % 4) * 2)) & 0x03;
      const int q = (lo | (hi << 4)) - 32;
      v[i] = __fmul_rn(__fmul_rn(d, (float)q), (float)sc[i / 16]);
    }
  }
}

template <int TYPE>
__device__ __forceinline__ const uint8_t *super_block(const uint8_t *blocks, size_t sub) {
  return blocks + (sub >> 3) * (TYPE == GRETA_GGML_Q4_K ? Q4_K_BYTES : Q6_K_BYTES);
}

// One thread per sub-block of 32 values.
template <int TYPE, bool OUT_F16>
__global__ void kquant_dequant_kernel(const uint8_t *__restrict__ blocks, void *__restrict__ out, size_t n_sub) {
  const size_t sub = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (sub >= n_sub) return;
  float v[32];
  decode_sub_block<TYPE>(super_block<TYPE>(blocks, sub), (int)(sub & 7), v);
  if (OUT_F16) {
    __half *o = static_cast<__half *>(out) + sub * 32;
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = __float2half_rn(v[i]);
  } else {
    float4 *o = reinterpret_cast<float4 *>(static_cast<float *>(out) + sub * 32);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  }
}

// One thread per sub-block: decode, quantise to one Q8_0 block, store payload and scale in the two planes.
template <int TYPE>
__global__ void kquant_to_q8_0_kernel(const uint8_t *__restrict__ blocks, uint8_t *__restrict__ qs, __half *__restrict__ dpl, size_t n_sub,
                                      uint32_t nb_row) {
  const size_t sub = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (sub >= n_sub) return;
  float v[32];
  decode_sub_block<TYPE>(super_block<TYPE>(blocks, sub), (int)(sub & 7), v);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float d = __fdiv_rn(amax, 127.0f), id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    w[i] = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) w[i] |= ((uint32_t)(int)roundf(__fmul_rn(v[4 * i + k], id)) & 0xFFu) << (8 * k);
  }
  uint4 *o = reinterpret_cast<uint4 *>(qs + sub * 32);
  o[0] = make_uint4(w[0], w[1], w[2], w[3]);
  o[1] = make_uint4(w[4], w[5], w[6], w[7]);
  dpl[(sub / nb_row) * d_row_stride(nb_row) + sub % nb_row] = __float2half_rn(d);
}

inline cudaStream_t S(greta_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }
inline unsigned grid_for(size_t n, unsigned threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace

extern "C" {

size_t greta_cuda_kquant_bytes(int ggml_type, size_t n_elems) {
  if (n_elems % 256) return 0;
  if (ggml_type == GRETA_GGML_Q4_K) return n_elems / 256 * Q4_K_BYTES;
  if (ggml_type == GRETA_GGML_Q6_K) return n_elems / 256 * Q6_K_BYTES;
  return 0;
}

int greta_cuda_kquant_dequant(greta_stream_t stream, int ggml_type, const void *blocks, size_t n_elems, void *out, int out_is_f16) {
  GRETA_REQUIRE(ggml_type == GRETA_GGML_Q4_K || ggml_type == GRETA_GGML_Q6_K, "kquant_dequant: GGML type %d is not Q4_K (12) or Q6_K (14)", ggml_type);
  GRETA_REQUIRE(n_elems % 256 == 0, "kquant_dequant: %zu values are not whole super-blocks of 256", n_elems);
  if (n_elems == 0) return GRETA_OK;
  GRETA_REQUIRE(blocks && out && aligned16(out), "kquant_dequant: null or misaligned pointer");
  const size_t n_sub = n_elems / 32;
  GRETA_REQUIRE(n_sub / 128 < (1u << 31), "kquant_dequant: tensor too large for one launch");
  const uint8_t *b = static_cast<const uint8_t *>(blocks);
  const unsigned g = grid_for(n_sub, 128);
  if (ggml_type == GRETA_GGML_Q4_K) {
    if (out_is_f16) kquant_dequant_kernel<GRETA_GGML_Q4_K, true><<<g, 128, 0, S(stream)>>>(b, out, n_sub);
    else kquant_dequant_kernel<GRETA_GGML_Q4_K, false><<<g, 128, 0, S(stream)>>>(b, out, n_sub);
  } else {
    if (out_is_f16) kquant_dequant_kernel<GRETA_GGML_Q6_K, true><<<g, 128, 0, S(stream)>>>(b, out, n_sub);
    else kquant_dequant_kernel<GRETA_GGML_Q6_K, false><<<g, 128, 0, S(stream)>>>(b, out, n_sub);
  }
  return launched("kquant_dequant_kernel");
}

int greta_cuda_kquant_to_q8_0(greta_stream_t stream, int ggml_type, const void *blocks, void *qs, void *d, uint32_t N, uint32_t K) {
  GRETA_REQUIRE(ggml_type == GRETA_GGML_Q4_K || ggml_type == GRETA_GGML_Q6_K, "kquant_to_q8_0: GGML type %d is not Q4_K (12) or Q6_K (14)", ggml_type);
  GRETA_REQUIRE(K % 256 == 0, "kquant_to_q8_0: K=%u is not a multiple of the super-block size 256", K);
  const size_t n_sub = (size_t)N * (K / 32);
  if (n_sub == 0) return GRETA_OK;
  GRETA_REQUIRE(blocks && qs && d && aligned16(qs) && aligned16(d), "kquant_to_q8_0: null or misaligned pointer");
  GRETA_REQUIRE(n_sub / 128 < (1u << 31), "kquant_to_q8_0: tensor too large for one launch");
  if (d_row_stride(K / 32) != K / 32) GRETA_CUDA_TRY(cudaMemsetAsync(d, 0, greta_cuda_d_bytes(GRETA_FMT_Q8_0, N, K), S(stream)));  // row padding
  const uint8_t *b = static_cast<const uint8_t *>(blocks);
  if (ggml_type == GRETA_GGML_Q4_K)
    kquant_to_q8_0_kernel<GRETA_GGML_Q4_K><<<grid_for(n_sub, 128), 128, 0, S(stream)>>>(b, (uint8_t *)qs, (__half *)d, n_sub, K / 32);
  else
    kquant_to_q8_0_kernel<GRETA_GGML_Q6_K><<<grid_for(n_sub, 128), 128, 0, S(stream)>>>(b, (uint8_t *)qs, (__half *)d, n_sub, K / 32);
  return launched("kquant_to_q8_0_kernel");
}

}  // extern "C"
