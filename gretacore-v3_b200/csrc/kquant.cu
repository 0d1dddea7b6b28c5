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
#include <algorithm>

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

// ---- GEMV straight from the super-blocks ----------------------------------------------------------
// y[m][n] = sum_k x[m][k] * w[n][k] with w decoded as above, the weights read as they lie in the file (4.5 bits per
// weight for Q4_K, 6.56 for Q6_K): nothing is re-quantised on this route.  A warp owns a row at a time; a lane owns one
// group of weights that shares a scale (a Q4_K sub-block of 32, a Q6_K group of 16) and uses
//   sum x (a q - b) = a sum(x (q - 8)) + (8 a - b) sum(x),   a = d * sc, b = dmin * m   (Q4_K);    sum x (d q sc) = (d sc) sum(x q)   (Q6_K)
// with sum(x) per group of 32 taken once per CTA when the activations are staged.  fp32 throughout; against the
// double-accumulating oracle over the exactly decoded weights the difference is rounding (1e-6 relative).
constexpr int KQ_WARPS = 8;

__device__ __forceinline__ uint32_t kq_and_or(uint32_t a, uint32_t m, uint32_t o) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(m), "r"(o));  // (a & m) | o
  return r;
}
__device__ __forceinline__ float2 kq_h2f2(uint32_t h2) { return __half22float2(*reinterpret_cast<__half2 *>(&h2)); }
// sum x * (q - 8) over the 8 nibbles of one payload word.  The nibbles become exact fp16 integers through the 0x6400
// exponent trick, two at a time; byte l of the word holds elements 2l (low) and 2l + 1 (high), so the pairs are
// (e0, e4), (e2, e6), (e1, e5), (e3, e7) and x is staged in that order: xa = {x0, x4, x2, x6}, xb = {x1, x5, x3, x7}.
__device__ __forceinline__ float2 kq_dot_nib8(uint32_t w, float4 xa, float4 xb, float2 s) {
  const uint32_t MAGIC = 0x64006400u;
  const __half2 c1032 = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));
  const __half2 sixteenth = __halves2half2(__ushort_as_half(0x2C00), __ushort_as_half(0x2C00));
  const __half2 cm72 = __halves2half2(__ushort_as_half(0xD480), __ushort_as_half(0xD480));
  const uint32_t w8 = w >> 8;
  uint32_t lo = kq_and_or(w, 0x000F000Fu, MAGIC), hi = kq_and_or(w, 0x00F000F0u, MAGIC);
  uint32_t lo2 = kq_and_or(w8, 0x000F000Fu, MAGIC), hi2 = kq_and_or(w8, 0x00F000F0u, MAGIC);
  const float2 a = __half22float2(__hsub2(*reinterpret_cast<__half2 *>(&lo), c1032));
  const float2 a2 = __half22float2(__hsub2(*reinterpret_cast<__half2 *>(&lo2), c1032));
  const float2 b = __half22float2(__hfma2(*reinterpret_cast<__half2 *>(&hi), sixteenth, cm72));
  const float2 b2 = __half22float2(__hfma2(*reinterpret_cast<__half2 *>(&hi2), sixteenth, cm72));
  s = __ffma2_rn(make_float2(xa.x, xa.y), a, s);
  s = __ffma2_rn(make_float2(xa.z, xa.w), a2, s);
  s = __ffma2_rn(make_float2(xb.x, xb.y), b, s);
  s = __ffma2_rn(make_float2(xb.z, xb.w), b2, s);
  return s;
}

template <int TYPE>
__global__ void __launch_bounds__(KQ_WARPS * 32) kquant_gemv_kernel(const uint8_t *__restrict__ blocks, const float *__restrict__ x,
                                                                     float *__restrict__ y, uint32_t N, uint32_t K) {
  extern __shared__ __align__(16) float kq_smem[];
  // activations of row blockIdx.y, 4 floats of padding after every 32 (a lane reads its own group of 32 with 128-bit
  // loads: 36-float strides spread a quarter-warp over all banks), then their sums per group of 32
  float *xs = kq_smem;
  float *xsum = kq_smem + K + K / 8;
  auto at = [](uint32_t k) { return k + 4 * (k >> 5); };
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float *xrow = x + (size_t)blockIdx.y * K;
  if (TYPE == GRETA_GGML_Q4_K) {  // inside every group of 8 in the order e0, e4, e2, e6, e1, e5, e3, e7 (see kq_dot_nib8)
    for (uint32_t i = tid; i < K; i += KQ_WARPS * 32) {
      const uint32_t e = i & 7u;
      xs[at((i & ~7u) | ((e & 1u) << 2) | (e & 2u) | (e >> 2))] = __ldg(xrow + i);
    }
  } else {
    for (uint32_t i = tid * 4; i < K; i += KQ_WARPS * 32 * 4) *reinterpret_cast<float4 *>(xs + at(i)) = __ldg(reinterpret_cast<const float4 *>(xrow + i));
  }
  __syncthreads();
  for (uint32_t g = tid; g < K / 32; g += KQ_WARPS * 32) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) t += xs[g * 36 + i];
    xsum[g] = t;
  }
  __syncthreads();
  constexpr int SB = TYPE == GRETA_GGML_Q4_K ? Q4_K_BYTES : Q6_K_BYTES;
  const uint32_t nsuper = K / 256;
  for (uint32_t row = blockIdx.x * KQ_WARPS + warp; row < N; row += gridDim.x * KQ_WARPS) {
    const uint8_t *wrow = blocks + (size_t)row * nsuper * SB;
    float acc = 0.f;
    if (TYPE == GRETA_GGML_Q4_K) {
#pragma unroll 1
      for (uint32_t sub = lane; sub < nsuper * 8; sub += 32) {  // one sub-block of 32 weights per lane (unrolling by 4 measured slower: 64 vs 56 us at 28672 x 8192)
        const uint8_t *blk = wrow + (size_t)(sub >> 3) * SB;
        const int j = sub & 7;
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(blk);
        const uint32_t *sc32 = reinterpret_cast<const uint32_t *>(blk + 4);
        const uint32_t s0 = sc32[0], s1 = sc32[1], s2 = sc32[2];
        auto byte_of = [&](int i) -> uint32_t { return ((i < 4 ? s0 : (i < 8 ? s1 : s2)) >> (8 * (i & 3))) & 0xFFu; };
        uint32_t s6, m6;
        if (j < 4) {
          s6 = byte_of(j) & 0x3F;
          m6 = byte_of(6 + j) & 0x3F;
        } else {
          const int i = j - 4;
          const uint32_t ns = (i & 1) ? (byte_of(4 + i / 2) >> 4) : (byte_of(4 + i / 2) & 0x0F);
          const uint32_t nm = (i & 1) ? (byte_of(10 + i / 2) >> 4) : (byte_of(10 + i / 2) & 0x0F);
          s6 = (byte_of(i) >> 6) | (ns << 2);
          m6 = (byte_of(6 + i) >> 6) | (nm << 2);
        }
        const float a = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFFu))) * (float)s6;
        const float b = __half2float(__ushort_as_half((unsigned short)(dd >> 16))) * (float)m6;
        const uint4 q = ld_stream(blk + 16 + j * 16);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        const float *xb = xs + (size_t)sub * 36;
        float2 d2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          d2 = kq_dot_nib8(w[i], *reinterpret_cast<const float4 *>(xb + 8 * i), *reinterpret_cast<const float4 *>(xb + 8 * i + 4), d2);
        const float dot8 = d2.x + d2.y;  // sum x (q - 8)
        acc += a * dot8 + (8.f * a - b) * xsum[sub];
      }
    } else {
#pragma unroll 4
      for (uint32_t grp = lane; grp < nsuper * 16; grp += 32) {  // one group of 16 weights (one scale) per lane
        const uint8_t *blk = wrow + (size_t)(grp >> 4) * SB;
        const int l = grp & 15;
        const uint16_t *ql = reinterpret_cast<const uint16_t *>(blk + 8 * l);      // 8 bytes: the 16 low nibbles
        const uint16_t *qh = reinterpret_cast<const uint16_t *>(blk + 128 + 4 * l);  // 4 bytes: the 16 high bit pairs
        const uint32_t lo0 = (uint32_t)ql[0] | ((uint32_t)ql[1] << 16), lo1 = (uint32_t)ql[2] | ((uint32_t)ql[3] << 16);
        const uint32_t hi = (uint32_t)qh[0] | ((uint32_t)qh[1] << 16);
        const float sc = (float)reinterpret_cast<const int8_t *>(blk + 192)[l];
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(blk + 208)));
        const float *xb = xs + at(grp * 16);
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint32_t lo = ((i < 8 ? lo0 : lo1) >> (4 * (i & 7))) & 15u, h2 = (hi >> (2 * i)) & 3u;
          dot = fmaf((float)((int)(lo | (h2 << 4)) - 32), xb[i], dot);
        }
        acc += (d * sc) * dot;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[(size_t)blockIdx.y * N + row] = acc;
  }
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

// The M <= 32 route of the reference's weight-only GEMV (gemm_kernels.hip:742-760: one pass over the weights per
// activation row) on weights kept as K-quant super-blocks.
int greta_cuda_gemv_kquant(greta_stream_t stream, int ggml_type, const float *x, const void *blocks, float *y, uint32_t M, uint32_t N, uint32_t K) {
  GRETA_REQUIRE(ggml_type == GRETA_GGML_Q4_K || ggml_type == GRETA_GGML_Q6_K, "gemv_kquant: GGML type %d is not Q4_K (12) or Q6_K (14)", ggml_type);
  GRETA_REQUIRE(K % 256 == 0 && K > 0, "gemv_kquant: K=%u is not a positive multiple of the super-block size 256", K);
  GRETA_REQUIRE(M >= 1 && M <= 32, "gemv_kquant: M=%u outside 1..32", M);
  if (N == 0) return GRETA_OK;
  GRETA_REQUIRE(x && blocks && y && aligned16(x) && ((uintptr_t)blocks & (ggml_type == GRETA_GGML_Q4_K ? 15 : 1)) == 0, "gemv_kquant: null or misaligned pointer");
  const size_t smem = ((size_t)K + K / 8 + K / 32) * sizeof(float);
  GRETA_REQUIRE(smem <= 200 * 1024, "gemv_kquant: K=%u does not fit the activation staging (at most 44032)", K);
  static bool attr_set[64][2] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int ti = ggml_type == GRETA_GGML_Q4_K ? 0 : 1;
  if (dev >= 0 && dev < 64 && !attr_set[dev][ti]) {
    if (ti == 0) GRETA_CUDA_TRY(cudaFuncSetAttribute(kquant_gemv_kernel<GRETA_GGML_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    else GRETA_CUDA_TRY(cudaFuncSetAttribute(kquant_gemv_kernel<GRETA_GGML_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_set[dev][ti] = true;
  }
  const unsigned per_sm = smem <= 48 * 1024 ? 4u : (smem <= 100 * 1024 ? 2u : 1u);
  const unsigned ctas = std::min<unsigned>((N + KQ_WARPS - 1) / KQ_WARPS, (unsigned)sm_count() * per_sm);
  dim3 grid(ctas, M);
  const uint8_t *b = static_cast<const uint8_t *>(blocks);
  if (ti == 0) kquant_gemv_kernel<GRETA_GGML_Q4_K><<<grid, KQ_WARPS * 32, smem, S(stream)>>>(b, x, y, N, K);
  else kquant_gemv_kernel<GRETA_GGML_Q6_K><<<grid, KQ_WARPS * 32, smem, S(stream)>>>(b, x, y, N, K);
  return launched("kquant_gemv_kernel");
}

}  // extern "C"
