// CPU oracle for the quantized-matmul hot path of GRETA CORE.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, as plain loops, the arithmetic
// of the reference's GPU kernels so that the CUDA library can be checked against
// it.  It is never linked into, imported by or called from the product path; the
// only callers are the tests, the smoke check and the CPU-baseline leg of the
// benchmark.
//
// Parity status: the reference ships no golden vector for its INT4/INT8 kernels,
// its RoPE or its attention ("parity unpinned" by tests for those).  What IS
// pinned, by running the reference's own host code (oracle/_ref, built from the
// reference sources by oracle/Makefile): fp16<->fp32 conversion, the Q8_0 block
// split, the reference INT4 quantiser/packing, dense GEMM and RMSNorm (including
// the reference's own known-answer tests).  Everything else follows the kernel
// source line by line; each function cites the lines it restates (paths are
// relative to the reference project root).
//
// Conventions: weights are [N x K] with K contiguous ("row" layout, y = x * W^T),
// quantisation blocks of 32 run along K.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#define OAPI extern "C" __attribute__((visibility("default")))

namespace {

// ---------------------------------------------------------------------------
// fp16 <-> fp32.  Decoding follows src/inference/src/weight_loader.cpp:91-110
// (exact for every finite half, subnormals included).  Encoding is IEEE
// round-to-nearest-even like the device intrinsic the kernels use
// (__float2half / __float2half_rn, gemm_kernels.hip:845,887) and like
// src/rt/ref/cpu/include/gcore/rt/ref/cpu_reference.hpp:19-37 for normal
// results; for subnormal results the CPU reference truncates whereas the device
// intrinsic rounds, and this oracle rounds (it models the kernels).
// ---------------------------------------------------------------------------
inline float h2f(uint16_t h) {
  uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1Fu, mant = h & 0x3FFu;
  uint32_t out;
  if (exp == 0) {
    if (mant == 0) {
      out = sign << 31;
    } else {
      exp = 1;
      while ((mant & 0x400u) == 0) {
        mant <<= 1;
        exp--;
      }
      mant &= 0x3FFu;
      out = (sign << 31) | ((exp + 112u) << 23) | (mant << 13);
    }
  } else if (exp == 31) {
    out = (sign << 31) | 0x7F800000u | (mant << 13);
  } else {
    out = (sign << 31) | ((exp + 112u) << 23) | (mant << 13);
  }
  float f;
  std::memcpy(&f, &out, 4);
  return f;
}

inline uint16_t f2h(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t ax = x & 0x7FFFFFFFu;
  if (ax >= 0x7F800000u)  // inf / nan
    return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x200u : 0u));
  if (ax >= 0x477FF000u)  // rounds to >= 65520 -> inf
    return (uint16_t)(sign | 0x7C00u);
  if (ax < 0x33000001u)  // <= 2^-25 -> +-0 (ties-to-even at exactly 2^-25)
    return (uint16_t)sign;
  int e = (int)(ax >> 23) - 127;
  uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
  int shift = (e < -14) ? (13 + (-14 - e)) : 13;
  uint32_t q = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1u))) q++;
  uint32_t res;
  if (e < -14)
    res = q;  // subnormal (may carry into the smallest normal, which is right)
  else
    res = ((uint32_t)(e + 15) << 10) + (q - 0x400u);  // carry bumps the exponent
  return (uint16_t)(sign | res);
}

inline float round_h(float f) { return h2f(f2h(f)); }

// Reference INT4 nibble: two's complement in 4 bits
// (src/rt/backend/hip/kernels/gemm_kernels.hip:786-791).
inline int sext4(uint32_t nib) {
  int v = (int)(nib & 0xFu);
  return (v & 8) ? v - 16 : v;
}

// GGUF Q4_0: block = {fp16 d; uint8 qs[16]}; element j is the low nibble of
// qs[j], element j+16 the high nibble, value = (q - 8) * d.  GGUF Q8_0:
// block = {fp16 d; int8 qs[32]}, value = q * d
// (src/inference/src/weight_loader.cpp:703-712 for the Q8_0 split).
constexpr int QK = 32;
constexpr int Q4_BYTES = 18;
constexpr int Q8_BYTES = 34;

inline void unpack_q4_0(const uint8_t *blk, float *d, int *q /*32*/) {
  uint16_t dh;
  std::memcpy(&dh, blk, 2);
  *d = h2f(dh);
  for (int j = 0; j < 16; ++j) {
    q[j] = (int)(blk[2 + j] & 0xF) - 8;
    q[j + 16] = (int)(blk[2 + j] >> 4) - 8;
  }
}

inline void unpack_q8_0(const uint8_t *blk, float *d, int *q) {
  uint16_t dh;
  std::memcpy(&dh, blk, 2);
  *d = h2f(dh);
  for (int j = 0; j < 32; ++j) q[j] = (int)(int8_t)blk[2 + j];
}

// Tree reduction over 256 partial sums exactly as the reference kernels do in
// shared memory (gemm_kernels.hip:621-629, 800-808; basic_kernels.hip:39-50).
inline float tree256(float *s) {
  for (int st = 128; st > 0; st >>= 1)
    for (int t = 0; t < st; ++t) s[t] += s[t + st];
  return s[0];
}

enum { FMT_Q4_0 = 0, FMT_Q8_0 = 1 };
enum { ACC_F64 = 0, ACC_REF_F32 = 1, ACC_FAST_F32 = 2 };

// One output of the decode GEMV.  acc_mode:
//  ACC_F64      double accumulation of x * (float(q) * d): the parity oracle.
//  ACC_REF_F32  the kernel's own order: thread t sums k = t, t+256, ... in fp32
//               with fused multiply-add (hipcc contracts a += b*c), then the
//               256-wide tree (gemm_kernels.hip:611-632 and 783-809).
//  ACC_FAST_F32 straight fp32 loop, vectorisable: the timed CPU baseline.
template <typename XT>
float gemv_one(const XT *x, const uint8_t *wrow, int fmt, uint32_t K, int acc_mode) {
  const uint32_t nb = K / QK;
  const int bb = fmt == FMT_Q4_0 ? Q4_BYTES : Q8_BYTES;
  if (acc_mode == ACC_F64) {
    double acc = 0.0;
    for (uint32_t b = 0; b < nb; ++b) {
      float d;
      int q[32];
      if (fmt == FMT_Q4_0)
        unpack_q4_0(wrow + (size_t)b * bb, &d, q);
      else
        unpack_q8_0(wrow + (size_t)b * bb, &d, q);
      for (int j = 0; j < 32; ++j) {
        float w = (float)q[j] * d;  // the dequantised value, fp32, exact product rounding
        acc += (double)(float)x[b * 32 + j] * (double)w;
      }
    }
    return (float)acc;
  }
  if (acc_mode == ACC_REF_F32) {
    float part[256];
    for (int t = 0; t < 256; ++t) part[t] = 0.f;
    // Q8_0 kernel: element k belongs to thread k % 256.  INT4 kernel: byte k
    // (elements 2k, 2k+1) belongs to thread k % 256.
    for (uint32_t b = 0; b < nb; ++b) {
      float d;
      int q[32];
      if (fmt == FMT_Q4_0)
        unpack_q4_0(wrow + (size_t)b * bb, &d, q);
      else
        unpack_q8_0(wrow + (size_t)b * bb, &d, q);
      for (int j = 0; j < 32; ++j) {
        uint32_t k = b * 32 + j;
        uint32_t t = (fmt == FMT_Q4_0) ? ((k / 2) % 256) : (k % 256);
        part[t] = fmaf((float)x[k], (float)q[j] * d, part[t]);
      }
    }
    return tree256(part);
  }
  float acc = 0.f;
  for (uint32_t b = 0; b < nb; ++b) {
    float d;
    int q[32];
    if (fmt == FMT_Q4_0)
      unpack_q4_0(wrow + (size_t)b * bb, &d, q);
    else
      unpack_q8_0(wrow + (size_t)b * bb, &d, q);
    float s = 0.f;
    for (int j = 0; j < 32; ++j) s += (float)x[b * 32 + j] * ((float)q[j] * d);
    acc += s;
  }
  return acc;
}

struct HalfT {
  uint16_t v;
  operator float() const { return h2f(v); }
};

inline size_t row_bytes(int fmt, uint32_t K) {
  return (size_t)(K / QK) * (fmt == FMT_Q4_0 ? Q4_BYTES : Q8_BYTES);
}

// Dequantise one weight row to fp32 (bit-exact (float)q * d).
void dequant_row(const uint8_t *wrow, int fmt, uint32_t K, float *out) {
  const int bb = fmt == FMT_Q4_0 ? Q4_BYTES : Q8_BYTES;
  for (uint32_t b = 0; b < K / QK; ++b) {
    float d;
    int q[32];
    if (fmt == FMT_Q4_0)
      unpack_q4_0(wrow + (size_t)b * bb, &d, q);
    else
      unpack_q8_0(wrow + (size_t)b * bb, &d, q);
    for (int j = 0; j < 32; ++j) out[b * 32 + j] = (float)q[j] * d;
  }
}

}  // namespace

// ===========================================================================
// C entry points (called through ctypes by the tests)
// ===========================================================================

OAPI int oracle_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// Thread count of the parallel loops (a launcher may have exported OMP_NUM_THREADS=1 for its workers).
OAPI void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

OAPI float oracle_fp16_to_fp32(uint16_t h) { return h2f(h); }
OAPI uint16_t oracle_fp32_to_fp16(float f) { return f2h(f); }

OAPI void oracle_fp16_to_fp32_n(const uint16_t *h, float *f, size_t n) {
  for (size_t i = 0; i < n; ++i) f[i] = h2f(h[i]);
}
OAPI void oracle_fp32_to_fp16_n(const float *f, uint16_t *h, size_t n) {
  for (size_t i = 0; i < n; ++i) h[i] = f2h(f[i]);
}

// Dequantise n_blocks GGUF blocks to fp32.  fmt 0 = Q4_0, 1 = Q8_0.
OAPI void oracle_dequant(const uint8_t *blocks, int fmt, size_t n_blocks, float *out) {
  const int bb = fmt == FMT_Q4_0 ? Q4_BYTES : Q8_BYTES;
#pragma omp parallel for if (n_blocks > 4096)
  for (size_t b = 0; b < n_blocks; ++b) {
    float d;
    int q[32];
    if (fmt == FMT_Q4_0)
      unpack_q4_0(blocks + b * bb, &d, q);
    else
      unpack_q8_0(blocks + b * bb, &d, q);
    for (int j = 0; j < 32; ++j) out[b * 32 + j] = (float)q[j] * d;
  }
}

// K-quant super-blocks of 256 weights, decoded the way the reference decodes them
// (src/inference/src/weight_loader.cpp:125-156 for Q4_K, :158-177 for Q6_K).  The reference's reading of these
// two layouts is its own: for Q4_K byte l of sub-block j holds elements 2l (low nibble) and 2l+1 (high nibble)
// of that sub-block, and the eight 6-bit scales and mins are unpacked as written below; for Q6_K element i takes
// its low four bits from nibble i of ql, its high two bits from bit pair i of qh and its scale from entry i / 16.
// (Upstream ggml orders the nibbles and packs the scales differently; the reference's results are what counts
// here.)  fp32 arithmetic in the reference's order, no fused multiply-add.
// Q4_K block: fp16 d, fp16 dmin, 12 scale bytes, 128 payload bytes (144 bytes).
OAPI void oracle_dequant_q4_k(const uint8_t *blocks, size_t n_super, float *out) {
#pragma omp parallel for if (n_super > 1024)
  for (size_t b = 0; b < n_super; ++b) {
    const uint8_t *blk = blocks + b * 144, *sc = blk + 4, *qs = blk + 16;
    uint16_t dh, mh;
    std::memcpy(&dh, blk, 2);
    std::memcpy(&mh, blk + 2, 2);
    const float d = h2f(dh), dmin = h2f(mh);
    uint8_t s8[8], m8[8];
    for (int j = 0; j < 4; ++j) {
      s8[j] = sc[j] & 0x3F;
      m8[j] = sc[6 + j] & 0x3F;
    }
    for (int j = 0; j < 4; ++j) {  // entry 4 + j: top two bits of byte j, and a nibble of byte 4 + j / 2 shifted up by two
      const uint8_t ns = (j & 1) ? (sc[4 + j / 2] >> 4) : (sc[4 + j / 2] & 0x0F);
      const uint8_t nm = (j & 1) ? (sc[10 + j / 2] >> 4) : (sc[10 + j / 2] & 0x0F);
      s8[4 + j] = (uint8_t)((sc[j] >> 6) | (ns << 2));
      m8[4 + j] = (uint8_t)((sc[6 + j] >> 6) | (nm << 2));
    }
    for (int j = 0; j < 8; ++j) {
      const float scale = d * (float)s8[j], minv = dmin * (float)m8[j];
      for (int l = 0; l < 16; ++l) {
        const uint8_t q = qs[j * 16 + l];
        out[b * 256 + j * 32 + 2 * l] = scale * (float)(q & 0x0F) - minv;
        out[b * 256 + j * 32 + 2 * l + 1] = scale * (float)(q >> 4) - minv;
      }
    }
  }
}
// Q6_K block: ql[128], qh[64], int8 scales[16], fp16 d (210 bytes).
OAPI void oracle_dequant_q6_k(const uint8_t *blocks, size_t n_super, float *out) {
#pragma omp parallel for if (n_super > 1024)
  for (size_t b = 0; b < n_super; ++b) {
    const uint8_t *blk = blocks + b * 210, *ql = blk, *qh = blk + 128;
    const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192);
    uint16_t dh;
    std::memcpy(&dh, blk + 208, 2);
    const float d = h2f(dh);
    for (int i = 0; i < 256; ++i) {
      const int lo = (ql[i / 2] >> ((i % 2) * 4)) & 0x0F, hi = (qh[i / 4] >> ((i % 4) * 2)) & 0x03;
      const int q = (lo | (hi << 4)) - 32;
      out[b * 256 + i] = (d * (float)q) * (float)sc[i / 16];
    }
  }
}
// fp32 values -> GGUF Q8_0 blocks (fp16 d, 32 int8), the round-to-nearest quantiser published with the format
// (ggml, quantize_row_q8_0 reference form; ggml is not part of the reference checkout): d = amax / 127,
// q = roundf(x / d) with the reciprocal taken in fp32 before d is rounded to fp16 for storage.
OAPI void oracle_quantize_q8_0(const float *x, size_t n_blocks, uint8_t *blocks) {
#pragma omp parallel for if (n_blocks > 4096)
  for (size_t b = 0; b < n_blocks; ++b) {
    float amax = 0.f;
    for (int j = 0; j < 32; ++j) amax = std::max(amax, std::fabs(x[b * 32 + j]));
    const float d = amax / 127.0f, id = d != 0.f ? 1.0f / d : 0.f;
    const uint16_t dh = f2h(d);
    std::memcpy(blocks + b * 34, &dh, 2);
    for (int j = 0; j < 32; ++j) blocks[b * 34 + 2 + j] = (uint8_t)(int8_t)std::roundf(x[b * 32 + j] * id);
  }
}

// The reference's own INT4 storage: uint8 w[n/2], element 2j in the low nibble
// and 2j+1 in the high nibble, two's complement, fp32 scale per group of
// group_size along the flat index (gemm_kernels.hip:784-797;
// src/inference/src/block_scheduler.cpp:639-655 read_weight_value).
OAPI void oracle_dequant_ref_int4(const uint8_t *packed, const float *scales, uint32_t group_size,
                                  size_t n, float *out) {
  for (size_t i = 0; i < n; ++i) {
    uint8_t p = packed[i / 2];
    int v = sext4((i % 2 == 0) ? (p & 0x0F) : (p >> 4));
    float s = scales ? scales[i / group_size] : 1.0f;
    out[i] = (float)v * s;
  }
}

// The reference's INT8 storage: int8 w[n] + fp32 scale per group
// (gemm_kernels.hip:611-616; block_scheduler.cpp:656-663).
OAPI void oracle_dequant_ref_int8(const int8_t *w, const float *scales, uint32_t group_size,
                                  size_t n, float *out) {
  for (size_t i = 0; i < n; ++i) out[i] = (float)w[i] * (scales ? scales[i / group_size] : 1.0f);
}

// Lossless re-expression of GGUF Q4_0 blocks in the reference's INT4 storage
// (v = q - 8, s = fp32(d)): shows both formats hold identical fp32 values.
OAPI void oracle_q4_0_to_ref_int4(const uint8_t *blocks, size_t n_blocks, uint8_t *packed,
                                  float *scales) {
  for (size_t b = 0; b < n_blocks; ++b) {
    float d;
    int q[32];
    unpack_q4_0(blocks + b * Q4_BYTES, &d, q);
    scales[b] = d;
    for (int j = 0; j < 32; j += 2)
      packed[b * 16 + j / 2] = (uint8_t)((q[j] & 0xF) | ((q[j + 1] & 0xF) << 4));
  }
}

// Split Q8_0 blocks the way the reference loader's Q8_0 branch does
// (weight_loader.cpp:703-712): int8 plane + fp32 scale per block.  That branch
// cannot be reached by running the reference: its tensor-type naming has no
// Q8_0 case (weight_loader.cpp:178-193), so a Q8_0 tensor is re-read as F32.
// The split is therefore pinned by restatement only.
OAPI void oracle_q8_0_split(const uint8_t *blocks, size_t n_blocks, int8_t *w, float *scales) {
  for (size_t b = 0; b < n_blocks; ++b) {
    uint16_t dh;
    std::memcpy(&dh, blocks + b * Q8_BYTES, 2);
    scales[b] = h2f(dh);
    std::memcpy(w + b * 32, blocks + b * Q8_BYTES + 2, 32);
  }
}

// Re-quantise fp32 values to the reference INT4 format exactly as
// weight_loader.cpp:925-957 does (max/7 scale, round half away, clamp -8..7).
OAPI void oracle_quantize_ref_int4(const float *x, size_t n, uint8_t *packed, float *scales) {
  size_t ng = (n + 31) / 32;
  for (size_t g = 0; g < ng; ++g) {
    float mx = 0.f;
    for (size_t i = 0; i < 32 && g * 32 + i < n; ++i) mx = std::max(mx, std::fabs(x[g * 32 + i]));
    float scale = mx / 7.0f;
    scales[g] = scale;
    float inv = scale > 1e-9f ? 1.0f / scale : 0.0f;
    for (size_t i = 0; i < 32 && g * 32 + i < n; i += 2) {
      size_t i0 = g * 32 + i, i1 = i0 + 1;
      int8_t v0 = (int8_t)std::round(x[i0] * inv);
      v0 = std::max((int8_t)-8, std::min((int8_t)7, v0));
      int8_t v1 = 0;
      if (i1 < n) {
        v1 = (int8_t)std::round(x[i1] * inv);
        v1 = std::max((int8_t)-8, std::min((int8_t)7, v1));
      }
      packed[i0 / 2] = (uint8_t)((v0 & 0x0F) | ((v1 & 0x0F) << 4));
    }
  }
}

// Re-quantise fp32 values to the reference INT8 format as weight_loader.cpp:790-803
// does (max/127 scale per 32, round half away from zero).
OAPI void oracle_quantize_ref_int8(const float *x, size_t n, int8_t *w, float *scales) {
  size_t nb = (n + 31) / 32;
  for (size_t b = 0; b < nb; ++b) {
    float mx = 0.f;
    for (size_t i = 0; i < 32 && b * 32 + i < n; ++i) mx = std::max(mx, std::fabs(x[b * 32 + i]));
    float scale = mx / 127.0f;
    scales[b] = scale;
    float inv = scale > 1e-9f ? 1.0f / scale : 0.0f;
    for (size_t i = 0; i < 32 && b * 32 + i < n; ++i) w[b * 32 + i] = (int8_t)std::round(x[b * 32 + i] * inv);
  }
}

// Decode GEMV  y[m,n] = sum_k x[m,k] * dequant(W)[n,k]
// (gemv_int8_wt_kernel gemm_kernels.hip:594-634, gemv_int4_wt_kernel :763-817,
// head_scales = nullptr).  x is fp32 (x_is_f16 = 0) or fp16 bits (1), as the
// INT4 kernel is instantiated for both (:921-931).  W = GGUF blocks, row n at
// n * (K/32) * block_bytes.
OAPI void oracle_gemv(const void *x, int x_is_f16, const uint8_t *w, int fmt, float *y, uint32_t M,
                      uint32_t N, uint32_t K, int acc_mode) {
  const size_t rb = row_bytes(fmt, K);
  for (uint32_t m = 0; m < M; ++m) {
#pragma omp parallel for schedule(static)
    for (uint32_t n = 0; n < N; ++n) {
      const uint8_t *wr = w + (size_t)n * rb;
      if (x_is_f16)
        y[(size_t)m * N + n] = gemv_one((const HalfT *)x + (size_t)m * K, wr, fmt, K, acc_mode);
      else
        y[(size_t)m * N + n] = gemv_one((const float *)x + (size_t)m * K, wr, fmt, K, acc_mode);
    }
  }
}

// Prefill GEMM  C[M x N] = half(A) * half(dequant(W))^T with wide accumulation.
// Operand rounding follows gemm_mfma_int4_wt_kernel (gemm_kernels.hip:845:
// A -> __float2half; :886-887: W -> __float2half((float)v * scale)) and the INT8
// twin (:640-740).  The contraction is the row-major one (W is [N x K]); the
// MFMA kernel's transposed store (:896-897) is a known defect of the reference
// and is not reproduced.  Products of two halves are exact in fp32, so the only
// freedom left is summation order; acc_mode 0 sums in double, 2 in fp32.
// a_is_f16: A holds fp16 bits, else fp32 that is rounded to fp16 first.
// out_f16: C is written as fp16 bits (round-to-nearest-even), else fp32.
OAPI void oracle_gemm(const void *A, int a_is_f16, const uint8_t *w, int fmt, void *C, int out_f16,
                      uint32_t M, uint32_t N, uint32_t K, int acc_mode) {
  std::vector<float> Ah((size_t)M * K);
  for (size_t i = 0; i < (size_t)M * K; ++i)
    Ah[i] = a_is_f16 ? h2f(((const uint16_t *)A)[i]) : round_h(((const float *)A)[i]);
  const size_t rb = row_bytes(fmt, K);
#pragma omp parallel
  {
    std::vector<float> wr(K);
#pragma omp for schedule(static)
    for (uint32_t n = 0; n < N; ++n) {
      dequant_row(w + (size_t)n * rb, fmt, K, wr.data());
      for (uint32_t k = 0; k < K; ++k) wr[k] = round_h(wr[k]);
      for (uint32_t m = 0; m < M; ++m) {
        const float *a = Ah.data() + (size_t)m * K;
        float r;
        if (acc_mode == ACC_F64) {
          double acc = 0.0;
          for (uint32_t k = 0; k < K; ++k) acc += (double)a[k] * (double)wr[k];
          r = (float)acc;
        } else {
          float acc = 0.f;
          for (uint32_t k = 0; k < K; ++k) acc += a[k] * wr[k];
          r = acc;
        }
        if (out_f16)
          ((uint16_t *)C)[(size_t)m * N + n] = f2h(r);
        else
          ((float *)C)[(size_t)m * N + n] = r;
      }
    }
  }
}

// Dense fp16-weight GEMV/GEMM used by the LM head: y = x * W^T, W fp16 [N x K],
// x fp32 (gemv_mixed_f16f32_kernel gemm_kernels.hip:466-507,
// gemm_mixed_f16f32_kernel :293-345: weights converted with __half2float, x kept
// in fp32).
OAPI void oracle_gemm_f16w(const float *x, const uint16_t *w, float *y, uint32_t M, uint32_t N,
                           uint32_t K, int acc_mode) {
#pragma omp parallel for schedule(static)
  for (uint32_t n = 0; n < N; ++n) {
    const uint16_t *wr = w + (size_t)n * K;
    for (uint32_t m = 0; m < M; ++m) {
      const float *xr = x + (size_t)m * K;
      if (acc_mode == ACC_F64) {
        double acc = 0.0;
        for (uint32_t k = 0; k < K; ++k) acc += (double)xr[k] * (double)h2f(wr[k]);
        y[(size_t)m * N + n] = (float)acc;
      } else {
        float acc = 0.f;
        for (uint32_t k = 0; k < K; ++k) acc += xr[k] * h2f(wr[k]);
        y[(size_t)m * N + n] = acc;
      }
    }
  }
}

// RMSNorm  y = (x * rsqrt(mean(x^2) + eps)) * gamma, that association
// (rmsnorm_parallel_kernel src/rt/backend/hip/kernels/basic_kernels.hip:21-55).
// mode 0: sum of squares and the inverse root in double
// (cpu_reference.hpp:73-88), then the kernel's fp32 product order.
// mode 1: the kernel's order: thread t sums c = t, t+256, ... in fp32, tree.
OAPI void oracle_rmsnorm(const float *x, const float *gamma, float *y, uint32_t rows, uint32_t cols,
                         float eps, int mode) {
  for (uint32_t r = 0; r < rows; ++r) {
    const float *xr = x + (size_t)r * cols;
    float *yr = y + (size_t)r * cols;
    float inv;
    if (mode == 0) {
      double ms = 0.0;
      for (uint32_t c = 0; c < cols; ++c) ms += (double)xr[c] * (double)xr[c];
      inv = (float)(1.0 / std::sqrt(ms / (double)cols + (double)eps));
    } else {
      float part[256];
      for (int t = 0; t < 256; ++t) part[t] = 0.f;
      for (uint32_t c = 0; c < cols; ++c) part[c % 256] = fmaf(xr[c], xr[c], part[c % 256]);
      float ms = tree256(part);
      inv = 1.0f / std::sqrt(ms / (float)cols + eps);
    }
    for (uint32_t c = 0; c < cols; ++c) yr[c] = (xr[c] * inv) * gamma[c];
  }
}

// Rotate-half RoPE in place on x [seq_len][num_heads][head_dim]: pair
// (i, i + head_dim/2), theta = pos * base^(-2i/head_dim), fp32 powf/cosf/sinf
// (rope_logic src/rt/backend/hip/kernels/attention_kernels.hip:28-52).
OAPI void oracle_rope(float *x, uint32_t seq_len, uint32_t num_heads, uint32_t head_dim, float base,
                      uint32_t pos_offset) {
  uint32_t hd2 = head_dim / 2;
  for (uint32_t s = 0; s < seq_len; ++s)
    for (uint32_t h = 0; h < num_heads; ++h)
      for (uint32_t i = 0; i < hd2; ++i) {
        uint32_t pos = pos_offset + s;
        float theta = (float)pos * powf(base, -2.0f * (float)i / (float)head_dim);
        float c = cosf(theta), sn = sinf(theta);
        size_t bi = (size_t)s * num_heads * head_dim + (size_t)h * head_dim + i;
        float v0 = x[bi], v1 = x[bi + hd2];
        x[bi] = v0 * c - v1 * sn;
        x[bi + hd2] = v0 * sn + v1 * c;
      }
}

// Decode attention for one query per head against the cache
// [num_heads_kv][max_seq_len][head_dim].  Follows the reference's own host
// references compute_attention_ref_fp32 / _fp64
// (src/inference/src/block_scheduler.cpp:721-766 and :814-864), which are the
// two-pass form of flash_attention_decode_logic (attention_kernels.hip:167-298).
// cache_is_f16: K/V hold fp16 bits (the B200 build's cache format) and are
// widened exactly; else fp32 as in the reference.  mode 0: all sums in double
// (the _fp64 reference); mode 1: fp32 dot and exp, double sums (the _fp32 one).
OAPI void oracle_attention_decode(const float *q, const void *k_cache, const void *v_cache,
                                  int cache_is_f16, float *out, uint32_t num_heads,
                                  uint32_t num_heads_kv, uint32_t head_dim, uint32_t seq_len,
                                  uint32_t max_seq_len, float scale, int mode) {
  const uint32_t group = num_heads_kv ? num_heads / num_heads_kv : 0;
#pragma omp parallel for schedule(static)
  for (uint32_t h = 0; h < num_heads; ++h) {
    const uint32_t kvh = group ? h / group : 0;
    const float *qp = q + (size_t)h * head_dim;
    const size_t base = (size_t)kvh * max_seq_len * head_dim;
    auto kv = [&](const void *c, uint32_t t, uint32_t d) -> float {
      size_t i = base + (size_t)t * head_dim + d;
      return cache_is_f16 ? h2f(((const uint16_t *)c)[i]) : ((const float *)c)[i];
    };
    std::vector<double> sc(seq_len);
    double mx = -INFINITY;
    for (uint32_t t = 0; t < seq_len; ++t) {
      double s;
      if (mode == 0) {
        double dot = 0.0;
        for (uint32_t d = 0; d < head_dim; ++d) dot += (double)qp[d] * (double)kv(k_cache, t, d);
        s = dot * (double)scale;
      } else {
        float dot = 0.f;
        for (uint32_t d = 0; d < head_dim; ++d) dot += qp[d] * kv(k_cache, t, d);
        s = (double)(dot * scale);
      }
      sc[t] = s;
      if (s > mx) mx = s;
    }
    double sum = 0.0;
    for (uint32_t t = 0; t < seq_len; ++t) {
      sc[t] = (mode == 0) ? std::exp(sc[t] - mx) : (double)std::exp((float)sc[t] - (float)mx);
      sum += sc[t];
    }
    const double inv = sum > 0.0 ? 1.0 / sum : 0.0;
    for (uint32_t d = 0; d < head_dim; ++d) {
      double acc = 0.0;
      for (uint32_t t = 0; t < seq_len; ++t) acc += sc[t] * (double)kv(v_cache, t, d);
      out[(size_t)h * head_dim + d] = (float)(acc * inv);
    }
  }
}

// Causal prefill attention over the prompt's own K/V, q/k/v/o
// [seq_len][heads][head_dim] fp32, GQA by kv_head = head / (H/Hkv)
// (flash_attention_prefill_kernel attention_kernels.hip:543-618).  K and V can
// be passed through fp16 rounding first (kv_round_f16) to model the fp16 cache
// the B200 build reads back.  Sums in double.
OAPI void oracle_attention_prefill(const float *q, const float *k, const float *v, float *o,
                                   uint32_t seq_len, uint32_t num_heads, uint32_t num_heads_kv,
                                   uint32_t head_dim, float scale, int causal, int kv_round_f16) {
  const uint32_t group = num_heads / num_heads_kv;
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t h = 0; h < num_heads; ++h)
    for (uint32_t s = 0; s < seq_len; ++s) {
      const uint32_t kvh = h / group;
      const float *qp = q + ((size_t)s * num_heads + h) * head_dim;
      uint32_t lim = causal ? s + 1 : seq_len;
      std::vector<double> sc(lim);
      double mx = -INFINITY;
      for (uint32_t t = 0; t < lim; ++t) {
        const float *kp = k + ((size_t)t * num_heads_kv + kvh) * head_dim;
        double dot = 0.0;
        for (uint32_t d = 0; d < head_dim; ++d)
          dot += (double)qp[d] * (double)(kv_round_f16 ? round_h(kp[d]) : kp[d]);
        sc[t] = dot * (double)scale;
        mx = std::max(mx, sc[t]);
      }
      double sum = 0.0;
      for (uint32_t t = 0; t < lim; ++t) {
        sc[t] = std::exp(sc[t] - mx);
        sum += sc[t];
      }
      float *op = o + ((size_t)s * num_heads + h) * head_dim;
      for (uint32_t d = 0; d < head_dim; ++d) {
        double acc = 0.0;
        for (uint32_t t = 0; t < lim; ++t) {
          float vv = v[((size_t)t * num_heads_kv + kvh) * head_dim + d];
          acc += sc[t] * (double)(kv_round_f16 ? round_h(vv) : vv);
        }
        op[d] = (float)(acc / sum);
      }
    }
}

// add / SiLU / mul (basic_kernels.hip:127-160): c = a + b; y = v / (1 + expf(-v)); c = a * b.
OAPI void oracle_add(const float *a, const float *b, float *c, size_t n) {
  for (size_t i = 0; i < n; ++i) c[i] = a[i] + b[i];
}
OAPI void oracle_silu_mul(const float *gate, const float *up, float *y, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    float g = gate[i];
    y[i] = (g / (1.0f + expf(-g))) * up[i];
  }
}

// Greedy pick: first maximum, lowest index on ties
// (src/inference/src/generator.cpp:735-744).  *tie is set when the maximum
// occurs more than once.
OAPI int32_t oracle_argmax(const float *logits, size_t n, int *tie) {
  int32_t id = 0;
  float mv = logits[0];
  int ties = 0;
  for (size_t i = 1; i < n; ++i) {
    if (logits[i] > mv) {
      mv = logits[i];
      id = (int32_t)i;
      ties = 0;
    } else if (logits[i] == mv) {
      ties = 1;
    }
  }
  if (tie) *tie = ties;
  return id;
}

// Embedding gather from an fp16 table [vocab][dim] widened to fp32 (the
// reference up-converts its table to fp32 at load, block_scheduler.cpp:1591, and
// gathers rows, basic_kernels.hip:169-196); out-of-range ids give zeros.
OAPI void oracle_embedding(const int32_t *tokens, const uint16_t *table, float *out,
                           uint32_t seq_len, uint32_t dim, uint32_t vocab) {
  for (uint32_t s = 0; s < seq_len; ++s)
    for (uint32_t d = 0; d < dim; ++d) {
      int32_t t = tokens[s];
      out[(size_t)s * dim + d] =
          (t >= 0 && t < (int32_t)vocab) ? h2f(table[(size_t)t * dim + d]) : 0.0f;
    }
}

// ---------------------------------------------------------------------------
// Model-level oracle: Llama-style decoder with GGUF-quantised projections, the
// operator order of BlockScheduler::execute_layer / forward
// (src/inference/src/block_scheduler.cpp:1814-3032 functional lines, :4078-4316).
// Differences from the reference that the B200 build makes on purpose, mirrored
// here: the KV cache holds fp16 (K after RoPE and V are rounded when written and
// attention reads the rounded values); the LM head runs on the last position
// only.  Prefill uses the GEMM operand rounding (both operands to
// fp16) when seq_len > 32, else the GEMV form keeps x in fp32, as the reference's two routes do
// (greta_compute_hip.cpp:166-167).  All reductions accumulate in double.
// ---------------------------------------------------------------------------
struct OracleLayer {
  const uint8_t *wq, *wk, *wv, *wo, *w1, *w2, *w3;  // GGUF blocks; w1 gate, w3 up, w2 down
  const float *attn_norm, *ffn_norm;                // fp32 [dim]
};
struct OracleModel {
  uint32_t dim, num_heads, num_heads_kv, head_dim, hidden_dim, num_layers, vocab, max_seq;
  float rope_base, rms_eps;
  int fmt;  // FMT_Q4_0 / FMT_Q8_0
  const OracleLayer *layers;
  const uint16_t *tok_embd;   // fp16 [vocab][dim]
  const float *out_norm;      // fp32 [dim]
  const uint16_t *out_weight; // fp16 [vocab][dim]
  uint16_t *k_cache, *v_cache; // fp16 [layers][Hkv][max_seq][Dh]
};

namespace {
// Accumulation of the model-level functions: ACC_F64 for parity checks (the default); ACC_FAST_F32 when the
// model is timed as the CPU baseline (fp32 sums as the kernels' arithmetic has them, vectorisable loops).
int g_model_acc = ACC_F64;
void proj(const OracleModel *m, const float *x, const uint8_t *w, float *y, uint32_t S, uint32_t N,
          uint32_t K) {
  if (S <= 32)  // the reference's route threshold (greta_compute_hip.cpp:166-167)
    oracle_gemv(x, 0, w, m->fmt, y, S, N, K, g_model_acc);
  else
    oracle_gemm(x, 0, w, m->fmt, y, 0, S, N, K, g_model_acc);
}
}  // namespace
OAPI void oracle_set_model_acc(int acc) { g_model_acc = acc; }

// Runs seq_len tokens starting at position seq_start through all layers and
// writes the logits of the LAST position to logits[vocab].  x_dump (optional,
// [dim]) receives the final hidden state of the last position before the output
// norm.
OAPI int oracle_model_forward(const OracleModel *m, const int32_t *tokens, uint32_t seq_start,
                              uint32_t S, float *logits, float *x_dump) {
  const uint32_t D = m->dim, H = m->num_heads, Hkv = m->num_heads_kv, Dh = m->head_dim,
                 F = m->hidden_dim;
  if (seq_start + S > m->max_seq) return 1;
  std::vector<float> x((size_t)S * D), nrm((size_t)S * D), q((size_t)S * H * Dh),
      k((size_t)S * Hkv * Dh), v((size_t)S * Hkv * Dh), att((size_t)S * H * Dh),
      tmp((size_t)S * D), gate((size_t)S * F), up((size_t)S * F);
  oracle_embedding(tokens, m->tok_embd, x.data(), S, D, m->vocab);
  const float scale = 1.0f / std::sqrt((float)Dh);
  for (uint32_t l = 0; l < m->num_layers; ++l) {
    const OracleLayer &L = m->layers[l];
    oracle_rmsnorm(x.data(), L.attn_norm, nrm.data(), S, D, m->rms_eps, 0);
    proj(m, nrm.data(), L.wq, q.data(), S, H * Dh, D);
    proj(m, nrm.data(), L.wk, k.data(), S, Hkv * Dh, D);
    proj(m, nrm.data(), L.wv, v.data(), S, Hkv * Dh, D);
    oracle_rope(q.data(), S, H, Dh, m->rope_base, seq_start);
    oracle_rope(k.data(), S, Hkv, Dh, m->rope_base, seq_start);
    uint16_t *kc = m->k_cache + (size_t)l * Hkv * m->max_seq * Dh;
    uint16_t *vc = m->v_cache + (size_t)l * Hkv * m->max_seq * Dh;
    for (uint32_t s = 0; s < S; ++s)
      for (uint32_t h = 0; h < Hkv; ++h)
        for (uint32_t d = 0; d < Dh; ++d) {
          size_t dst = ((size_t)h * m->max_seq + seq_start + s) * Dh + d;
          kc[dst] = f2h(k[((size_t)s * Hkv + h) * Dh + d]);
          vc[dst] = f2h(v[((size_t)s * Hkv + h) * Dh + d]);
        }
    for (uint32_t s = 0; s < S; ++s)
      oracle_attention_decode(q.data() + (size_t)s * H * Dh, kc, vc, 1,
                              att.data() + (size_t)s * H * Dh, H, Hkv, Dh, seq_start + s + 1,
                              m->max_seq, scale, g_model_acc == ACC_F64 ? 0 : 1);
    proj(m, att.data(), L.wo, tmp.data(), S, D, H * Dh);
    oracle_add(x.data(), tmp.data(), x.data(), (size_t)S * D);
    oracle_rmsnorm(x.data(), L.ffn_norm, nrm.data(), S, D, m->rms_eps, 0);
    proj(m, nrm.data(), L.w1, gate.data(), S, F, D);
    proj(m, nrm.data(), L.w3, up.data(), S, F, D);
    oracle_silu_mul(gate.data(), up.data(), gate.data(), (size_t)S * F);
    proj(m, gate.data(), L.w2, tmp.data(), S, D, F);
    oracle_add(x.data(), tmp.data(), x.data(), (size_t)S * D);
  }
  const float *xl = x.data() + (size_t)(S - 1) * D;
  if (x_dump) std::memcpy(x_dump, xl, (size_t)D * 4);
  oracle_rmsnorm(xl, m->out_norm, nrm.data(), 1, D, m->rms_eps, 0);
  oracle_gemm_f16w(nrm.data(), m->out_weight, logits, 1, m->vocab, D, g_model_acc);
  return 0;
}
