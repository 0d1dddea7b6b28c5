// Device-side building blocks of the decode GEMV kernels: formats, row-group resolution, epilogues,
// activation staging (fp32, or block fixed point for the integer dot-product path), the per-block
// dot products and the cp.async helpers.  Shared by gemv.cu (one operator per launch) and
// decode_step.cu (all layers of a decode step in one persistent launch).
#pragma once
#include <math.h>

#include "greta_common.cuh"

using namespace greta;

namespace {

constexpr int WARPS = 16;
constexpr int THREADS = WARPS * 32;
constexpr int XPAD = 36;       // floats per staged block of 32 fp32 activations (4 pad -> conflict-free LDS.128)
constexpr int XQ_WORDS = 28;   // 32-bit words per staged fixed-point block: 3 planes x 8 words + 4 words of meta
constexpr int MAX_STAGES = 8;
constexpr size_t SMEM_LIMIT = 220 * 1024;

enum { EPI_PLAIN = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2, EPI_QKV = 3, EPI_PEER = 4 };
constexpr int MAX_TP = 8;

struct WPlane {
  const uint8_t *qs;
  const void *d;
};

struct GemvParams {
  const void *x;
  int x_is_f16;
  const float *gamma;
  float eps;
  WPlane w[3];
  uint32_t K, N, M;
  float *y;
  const float *resid;
  float *q_out, *k_out, *v_out;
  __half *k_cache, *v_cache;
  const uint32_t *d_pos;
  uint32_t H, Hkv, Dh, max_seq;
  float rope_base;
  uint32_t groups;  // row groups
  // simple kernel
  uint32_t kw, iters;
  // pipelined kernel
  uint32_t stages, slots;
  uint32_t gq, gr;  // row groups per CTA: CTA b owns gq (+1 when b < gr) groups
  // Tensor-parallel exchange over peer memory.  A slot buffer holds [tp][dim] words {value bits, tag}; a
  // row-parallel projection (EPI_PEER) stores its partial product, tagged, into slot `rank` of every rank's
  // buffer; the next operator's staging waits for the tp tagged partials, adds them to the residual stream
  // in rank order and (CTA 0) writes the new stream to x_out.
  uint2 *peer_out[MAX_TP];
  const uint2 *peer_in;
  float *x_out;
  uint32_t tp, rank, exch_idx;
  uint32_t poll_limit;  // polls a consumer spends on one missing partial before it gives up (tuning switch peer_poll_limit)
  // Two-level gather (tp >= tuning switch peer_two_level_min_tp): the CTAs of a consumer split the vector into blocks of 32,
  // each sums the tp partials of its blocks into the residual stream once and publishes {sum, tag} words in the local
  // sum buffer; then every CTA reads the dim summed words instead of tp x dim partial words.
  const uint2 *sum_in;
  uint2 *sum_out;
  uint32_t two_level;
  // Batched form with prepared activations (gemv_batch.cu): x already split into fp16 pairs in matrix-instruction
  // fragment order, and the factor that finishes each activation row (1 / power-of-two scale, times 1 / rms).
  const uint8_t *xprep;
  const float *rowmul;
};

// Tag of exchange number exch_idx at the current position: strictly increasing within a decode session.
__device__ __forceinline__ uint32_t peer_tag(const GemvParams &p) { return ((__ldcg(p.d_pos) + 1u) << 8) | p.exch_idx; }

// Set when a wait for a peer's partial gave up.  Once it is set every later wait gives up after a single look, so
// a step with a missing rank drains in about one poll budget instead of one budget per thread, pass and kernel;
// greta_cuda_peer_reset() clears it for the next session.
__device__ int g_peer_error = 0;
__device__ __forceinline__ bool peer_failed() { return *reinterpret_cast<volatile int *>(&g_peer_error) != 0; }

__device__ __forceinline__ void st_peer(uint2 *dst, uint2 v) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ uint4 ld_peer16(const void *src) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_peer8(const void *src) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(src) : "memory");
  return v;
}
// Adds the `nsrc` tagged vectors at `base` ([nsrc][K] words) for elements idx .. idx+3 to v, in order, waiting (bounded) for
// their tags.  The loads of four sources at a time are issued before any tag is looked at: one round trip to L2 per
// four sources when the words are already there, not one per source.
__device__ __forceinline__ void add_tagged_words(const GemvParams &p, const uint2 *base, uint32_t nsrc, uint32_t idx, uint32_t tag, float (&v)[4]) {
  constexpr int BATCH = 4;
  const uint32_t budget = peer_failed() ? 0u : p.poll_limit;
  for (uint32_t r0 = 0; r0 < nsrc; r0 += BATCH) {
    uint4 a[BATCH], b[BATCH];
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      if (r0 + i < nsrc) {
        const uint2 *src = base + (size_t)(r0 + i) * p.K + idx;
        a[i] = ld_peer16(src);
        b[i] = ld_peer16(src + 2);
      }
    }
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      if (r0 + i < nsrc) {
        uint32_t polls = 0;
        while (!(a[i].y == tag && a[i].w == tag && b[i].y == tag && b[i].w == tag)) {
          if (++polls > budget || ((polls & 255u) == 0 && peer_failed())) {
            g_peer_error = 1;
            break;
          }
          const uint2 *src = base + (size_t)(r0 + i) * p.K + idx;
          a[i] = ld_peer16(src);
          b[i] = ld_peer16(src + 2);
        }
        v[0] += __uint_as_float(a[i].x);
        v[1] += __uint_as_float(a[i].z);
        v[2] += __uint_as_float(b[i].x);
        v[3] += __uint_as_float(b[i].z);
      }
    }
  }
}

// First level of the two-level gather: this CTA's blocks of 32 elements (block b belongs to CTA b % gridDim.x, one warp per
// block, one element per lane): residual stream + the tp partials in rank order -> the local sum buffer, tagged, and x_out.
__device__ __forceinline__ void peer_sum_slice(const GemvParams &p, uint32_t tag) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t nbk = p.K / 32;
  const uint32_t budget = peer_failed() ? 0u : p.poll_limit;
  const float *xin = reinterpret_cast<const float *>(p.x);
  for (uint32_t b = blockIdx.x + gridDim.x * warp; b < nbk; b += gridDim.x * (blockDim.x >> 5)) {
    const uint32_t e = b * 32 + lane;
    float v = __ldcg(xin + e);
    uint2 w[MAX_TP];
#pragma unroll
    for (int r = 0; r < MAX_TP; ++r)
      if ((uint32_t)r < p.tp) w[r] = ld_peer8(p.peer_in + (size_t)r * p.K + e);  // all sources in flight before any tag is looked at
#pragma unroll
    for (int r = 0; r < MAX_TP; ++r) {
      if ((uint32_t)r < p.tp) {
        uint32_t polls = 0;
        while (w[r].y != tag) {
          if (++polls > budget || ((polls & 255u) == 0 && peer_failed())) {
            g_peer_error = 1;
            break;
          }
          w[r] = ld_peer8(p.peer_in + (size_t)r * p.K + e);
        }
        v += __uint_as_float(w[r].x);
      }
    }
    st_peer(p.sum_out + e, make_uint2(__float_as_uint(v), tag));
    p.x_out[e] = v;
  }
}

template <int FMT>
struct Fmt;
template <>
struct Fmt<GRETA_FMT_Q4_0> {
  static constexpr int QV = 1, SCALE_BYTES = 2;
  static constexpr bool INTEGER = true, NIBBLES = true;
};
template <>
struct Fmt<GRETA_FMT_Q8_0> {
  static constexpr int QV = 2, SCALE_BYTES = 2;
  static constexpr bool INTEGER = true, NIBBLES = false;
};
template <>
struct Fmt<GRETA_FMT_REF_INT4> {
  static constexpr int QV = 1, SCALE_BYTES = 4;
  static constexpr bool INTEGER = true, NIBBLES = true;
};
template <>
struct Fmt<GRETA_FMT_REF_INT8> {
  static constexpr int QV = 2, SCALE_BYTES = 4;
  static constexpr bool INTEGER = true, NIBBLES = false;
};
template <>
struct Fmt<GRETA_FMT_F16> {
  static constexpr int QV = 4, SCALE_BYTES = 0;
  static constexpr bool INTEGER = false, NIBBLES = false;
};

// ------------------------------------------------------------------ shared pieces
// Maps (row group, slot) to a weight plane and a row; false for a slot without a
// row (ragged tail).  A group holds R/2 "pairs": slot j and slot j + R/2 are the
// two rows an epilogue combines (gate/up of one output, the two halves of one
// rotation pair).
template <int EPI, int R>
__device__ __forceinline__ bool resolve(const GemvParams &p, uint32_t grp, int slot, int *mat, uint32_t *row) {
  constexpr int PAIRS = R / 2;
  if (EPI == EPI_PLAIN || EPI == EPI_RESIDUAL || EPI == EPI_PEER) {
    *mat = 0;
    *row = grp * R + slot;
    return *row < p.N;
  }
  if (EPI == EPI_SWIGLU) {
    *mat = slot / PAIRS;
    *row = grp * PAIRS + slot % PAIRS;
    return *row < p.N;
  }
  const uint32_t gph = (p.Dh / 2) / PAIRS, nq = p.H * gph, nk = p.Hkv * gph;
  if (grp < nq + nk) {
    uint32_t g = grp < nq ? grp : grp - nq;
    *mat = grp < nq ? 0 : 1;
    uint32_t head = g / gph, i = (g % gph) * PAIRS + slot % PAIRS;
    *row = head * p.Dh + i + (slot / PAIRS) * (p.Dh / 2);
    return true;
  }
  *mat = 2;
  *row = (grp - nq - nk) * R + slot;
  return *row < p.Hkv * p.Dh;
}

// Applies the epilogue of one row group; v[r] are the finished dot products.
template <int EPI, int R>
__device__ __forceinline__ void epilogue(const GemvParams &p, uint32_t grp, uint32_t m, uint32_t pos, const float (&v)[R]) {
  constexpr int PAIRS = R / 2;
  if (EPI == EPI_PLAIN) {
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (grp * R + r < p.N) p.y[(size_t)m * p.N + grp * R + r] = v[r];
  } else if (EPI == EPI_RESIDUAL) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint32_t row = grp * R + r;
      if (row < p.N) p.y[row] = __ldcg(p.resid + row) + v[r];
    }
  } else if (EPI == EPI_PEER) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint32_t row = grp * R + r;
      if (row < p.N)
        for (uint32_t j = 0; j < p.tp; ++j) st_peer(p.peer_out[j] + (size_t)p.rank * p.N + row, make_uint2(__float_as_uint(v[r]), pos));
    }
  } else if (EPI == EPI_SWIGLU) {
#pragma unroll
    for (int j = 0; j < PAIRS; ++j) {
      uint32_t o = grp * PAIRS + j;
      if (o < p.N) {
        float g = v[j], u = v[j + PAIRS];
        p.y[o] = (g / (1.0f + expf(-g))) * u;
      }
    }
  } else {
    const uint32_t gph = (p.Dh / 2) / PAIRS, nq = p.H * gph, nk = p.Hkv * gph;
    if (grp < nq + nk) {
      const bool is_q = grp < nq;
      uint32_t g = is_q ? grp : grp - nq;
      uint32_t head = g / gph;
#pragma unroll
      for (int j = 0; j < PAIRS; ++j) {
        uint32_t i = (g % gph) * PAIRS + j;
        float o0 = v[j], o1 = v[j + PAIRS];
        if (p.d_pos) {
          float theta = (float)pos * powf(p.rope_base, -2.0f * (float)i / (float)p.Dh);
          float c = cosf(theta), s = sinf(theta);
          o0 = v[j] * c - v[j + PAIRS] * s;
          o1 = v[j] * s + v[j + PAIRS] * c;
        }
        if (is_q) {
          p.q_out[head * p.Dh + i] = o0;
          p.q_out[head * p.Dh + i + p.Dh / 2] = o1;
        } else {
          if (p.k_out) {
            p.k_out[head * p.Dh + i] = o0;
            p.k_out[head * p.Dh + i + p.Dh / 2] = o1;
          }
          if (p.k_cache && pos < p.max_seq) {  // a position past the cache is never written
            size_t dst = ((size_t)head * p.max_seq + pos) * p.Dh + i;
            p.k_cache[dst] = __float2half_rn(o0);
            p.k_cache[dst + p.Dh / 2] = __float2half_rn(o1);
          }
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        uint32_t row = (grp - nq - nk) * R + r;
        if (row < p.Hkv * p.Dh) {
          if (p.v_out) p.v_out[row] = v[r];
          uint32_t head = row / p.Dh, dd = row % p.Dh;
          if (p.v_cache && pos < p.max_seq) p.v_cache[((size_t)head * p.max_seq + pos) * p.Dh + dd] = __float2half_rn(v[r]);
        }
      }
    }
  }
}

// Lane-parallel form of the epilogue: lane `lane` of a warp finishes its share of row group `grp`
// (one output row, one gate/up pair or one rotation pair).  rope_cs, when given, holds (cos, sin) of the
// rotation angle of every pair index for the current position.
template <int EPI, int R>
__device__ __forceinline__ void epilogue_lane(const GemvParams &p, uint32_t grp, uint32_t m, uint32_t pos, const float (&v)[R], int lane,
                                              const float2 *rope_cs) {
  constexpr int PAIRS = R / 2;
  float mine = v[0], partner = v[PAIRS];  // v[lane] and v[lane + PAIRS] without dynamic indexing
#pragma unroll
  for (int r = 1; r < R; ++r) mine = (lane == r) ? v[r] : mine;
#pragma unroll
  for (int r = 1; r < PAIRS; ++r) partner = (lane == r) ? v[r + PAIRS] : partner;
  if (EPI == EPI_PLAIN) {
    const uint32_t row = grp * R + lane;
    if (lane < R && row < p.N) p.y[(size_t)m * p.N + row] = mine;
  } else if (EPI == EPI_RESIDUAL) {
    const uint32_t row = grp * R + lane;
    if (lane < R && row < p.N) p.y[row] = __ldcg(p.resid + row) + mine;
  } else if (EPI == EPI_PEER) {  // pos carries the tag
    const uint32_t row = grp * R + lane;
    if (lane < R && row < p.N)
      for (uint32_t j = 0; j < p.tp; ++j) st_peer(p.peer_out[j] + (size_t)p.rank * p.N + row, make_uint2(__float_as_uint(mine), pos));
  } else if (EPI == EPI_SWIGLU) {
    const uint32_t o = grp * PAIRS + lane;
    if (lane < PAIRS && o < p.N) p.y[o] = (mine / (1.0f + expf(-mine))) * partner;
  } else {
    const uint32_t gph = (p.Dh / 2) / PAIRS, nq = p.H * gph, nk = p.Hkv * gph;
    if (grp < nq + nk) {
      if (lane < PAIRS) {
        const bool is_q = grp < nq;
        const uint32_t g = is_q ? grp : grp - nq;
        const uint32_t head = g / gph, i = (g % gph) * PAIRS + lane;
        float o0 = mine, o1 = partner;
        if (p.d_pos) {
          float c, s;
          if (rope_cs) {
            c = rope_cs[i].x;
            s = rope_cs[i].y;
          } else {
            const float theta = (float)pos * powf(p.rope_base, -2.0f * (float)i / (float)p.Dh);
            c = cosf(theta);
            s = sinf(theta);
          }
          o0 = mine * c - partner * s;
          o1 = mine * s + partner * c;
        }
        if (is_q) {
          p.q_out[head * p.Dh + i] = o0;
          p.q_out[head * p.Dh + i + p.Dh / 2] = o1;
        } else {
          if (p.k_out) {
            p.k_out[head * p.Dh + i] = o0;
            p.k_out[head * p.Dh + i + p.Dh / 2] = o1;
          }
          if (p.k_cache && pos < p.max_seq) {
            const size_t dst = ((size_t)head * p.max_seq + pos) * p.Dh + i;
            p.k_cache[dst] = __float2half_rn(o0);
            p.k_cache[dst + p.Dh / 2] = __float2half_rn(o1);
          }
        }
      }
    } else {
      const uint32_t row = (grp - nq - nk) * R + lane;
      if (lane < R && row < p.Hkv * p.Dh) {
        if (p.v_out) p.v_out[row] = mine;
        const uint32_t head = row / p.Dh, dd = row % p.Dh;
        if (p.v_cache && pos < p.max_seq) p.v_cache[((size_t)head * p.max_seq + pos) * p.Dh + dd] = __float2half_rn(mine);
      }
    }
  }
}

// (cos, sin) of the rotation angles of all pair indices at the current position, once per kernel.
__device__ __forceinline__ void fill_rope_table(const GemvParams &p, uint32_t pos, float2 *rope_cs) {
  for (uint32_t i = threadIdx.x; i < p.Dh / 2; i += blockDim.x) {
    const float theta = (float)pos * powf(p.rope_base, -2.0f * (float)i / (float)p.Dh);
    rope_cs[i] = make_float2(cosf(theta), sinf(theta));
  }
}

// Epilogue of a CTA's row groups [g0, g1) after the pipelined cell loop: one warp per group, lanes 0..15
// fetch the contributions of the 16 warps (a group's cells can be split over several warps), a butterfly
// sums them in a fixed order, then the lanes finish one row / pair each.
template <int EPI, int R>
__device__ __forceinline__ void cta_epilogue(const GemvParams &p, const float *part, uint32_t slots, uint32_t g0, uint32_t g1, uint32_t C,
                                             uint32_t T, uint32_t m, uint32_t pos, const float2 *rope_cs) {
  // Two groups per warp iteration, one per half-warp: lane hl of a half fetches the contribution of source warp hl.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = lane >> 4, hl = lane & 15;
  static_assert(WARPS == 16, "one source warp per lane of a half-warp");
  const uint32_t wc0 = (uint32_t)((uint64_t)hl * T / WARPS), wc1 = (uint32_t)((uint64_t)(hl + 1) * T / WARPS);
  const uint32_t wfirst = wc0 / C;  // first group (relative to g0) the source warp touched
  for (uint32_t gbase = g0 + 2 * warp; gbase < g1; gbase += 2 * WARPS) {
    const uint32_t grp = gbase + half;
    const bool valid = grp < g1;
    const uint32_t lo = (grp - g0) * C, hi = lo + C;
    float v[R];
    const bool has = valid && wc0 < hi && wc1 > lo && wc1 > wc0;
    const float *src = part + ((size_t)hl * slots + (grp - g0 - wfirst)) * R;
#pragma unroll
    for (int r = 0; r < R; ++r) v[r] = has ? src[r] : 0.f;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {  // sums within each half-warp, in a fixed order
#pragma unroll
      for (int r = 0; r < R; ++r) v[r] += __shfl_xor_sync(0xffffffffu, v[r], o);
    }
    if (valid) epilogue_lane<EPI, R>(p, grp, m, pos, v, hl, rope_cs);
  }
}

// Sum of squares of the activation row over the CTA -> 1/rms.
__device__ __forceinline__ float cta_inv_rms(const float *xf, const __half *xh, uint32_t K, float eps, float *red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float ss = 0.f;
  for (uint32_t k = threadIdx.x; k < K; k += THREADS) {
    float v = xf ? __ldcg(xf + k) : __half2float(__ldcg(xh + k));
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float t = (lane < WARPS) ? red[lane] : 0.f;
  t = warp_sum(t);
  return rsqrtf(t / (float)K + eps);
}

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

// ------------------------------------------------------------------ float math (fp16 weights, simple kernel)
__device__ __forceinline__ uint32_t lop_and_or(uint32_t a, uint32_t m, uint32_t o) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(m), "r"(o));  // (a & m) | o
  return r;
}
__device__ __forceinline__ uint32_t hsub2_u(uint32_t a, uint32_t b) {
  __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
  return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
  __half2 r = __hfma2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b),
                      *reinterpret_cast<__half2 *>(&c));
  return *reinterpret_cast<uint32_t *>(&r);
}

// Position of element j (0..31) of a block inside its staged 32-float slot (float path).
template <int FMT>
__device__ __forceinline__ int xs_slot(int j) {
  if (FMT == GRETA_FMT_Q4_0) {
    int hi = j >> 4, jj = j & 15, wi = jj >> 2, r = jj & 3;
    int pr = (r == 1) ? 2 : (r == 2) ? 1 : r;  // order e0,e2,e1,e3
    return 8 * wi + 4 * hi + pr;
  }
  if (FMT == GRETA_FMT_REF_INT4) {
    int wi = j >> 3, e = j & 7;  // staged order e0,e4,e2,e6,e1,e5,e3,e7: the 3-bit reversal of e
    return 8 * wi + ((e & 1) << 2 | (e & 2) | (e >> 2));
  }
  return j;
}

// x * (q - 8) over the 8 nibbles of one payload word (exact fp16 integers via the 0x6400 exponent trick).
__device__ __forceinline__ float2 dot_nib8(uint32_t w, float4 xa, float4 xb, float2 s) {
  const uint32_t MAGIC = 0x64006400u, C1032 = 0x64086408u, SIXTEENTH = 0x2C002C00u, CM72 = 0xD480D480u;
  uint32_t w8 = w >> 8;
  uint32_t lo = lop_and_or(w, 0x000F000Fu, MAGIC), hi = lop_and_or(w, 0x00F000F0u, MAGIC);
  uint32_t lo2 = lop_and_or(w8, 0x000F000Fu, MAGIC), hi2 = lop_and_or(w8, 0x00F000F0u, MAGIC);
  float2 a = h2_to_f2(hsub2_u(lo, C1032)), a2 = h2_to_f2(hsub2_u(lo2, C1032));
  float2 b = h2_to_f2(hfma2_u(hi, SIXTEENTH, CM72)), b2 = h2_to_f2(hfma2_u(hi2, SIXTEENTH, CM72));
  s = ffma2(make_float2(xa.x, xa.y), a, s);
  s = ffma2(make_float2(xa.z, xa.w), a2, s);
  s = ffma2(make_float2(xb.x, xb.y), b, s);
  s = ffma2(make_float2(xb.z, xb.w), b2, s);
  return s;
}
__device__ __forceinline__ float2 dot_i8x4(uint32_t w, float4 xv, float2 s) {
  const uint32_t C1152 = 0x64806480u;  // 1024 + 128
  uint32_t t = w ^ 0x80808080u;
  uint32_t h01 = __byte_perm(t, 0x64646464u, 0x5140), h23 = __byte_perm(t, 0x64646464u, 0x7362);
  s = ffma2(make_float2(xv.x, xv.y), h2_to_f2(hsub2_u(h01, C1152)), s);
  s = ffma2(make_float2(xv.z, xv.w), h2_to_f2(hsub2_u(h23, C1152)), s);
  return s;
}
template <int FMT>
__device__ __forceinline__ float block_dot_f(const uint4 *q, const float4 *xv) {
  float2 s = make_float2(0.f, 0.f);
  if (FMT == GRETA_FMT_Q4_0 || FMT == GRETA_FMT_REF_INT4) {
    const uint32_t flip = (FMT == GRETA_FMT_REF_INT4) ? 0x88888888u : 0u;  // two's complement -> offset 8
    s = dot_nib8(q[0].x ^ flip, xv[0], xv[1], s);
    s = dot_nib8(q[0].y ^ flip, xv[2], xv[3], s);
    s = dot_nib8(q[0].z ^ flip, xv[4], xv[5], s);
    s = dot_nib8(q[0].w ^ flip, xv[6], xv[7], s);
  } else if (FMT == GRETA_FMT_Q8_0 || FMT == GRETA_FMT_REF_INT8) {
    s = dot_i8x4(q[0].x, xv[0], s);
    s = dot_i8x4(q[0].y, xv[1], s);
    s = dot_i8x4(q[0].z, xv[2], s);
    s = dot_i8x4(q[0].w, xv[3], s);
    s = dot_i8x4(q[1].x, xv[4], s);
    s = dot_i8x4(q[1].y, xv[5], s);
    s = dot_i8x4(q[1].z, xv[6], s);
    s = dot_i8x4(q[1].w, xv[7], s);
  } else {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      s = ffma2(make_float2(xv[2 * v].x, xv[2 * v].y), h2_to_f2(q[v].x), s);
      s = ffma2(make_float2(xv[2 * v].z, xv[2 * v].w), h2_to_f2(q[v].y), s);
      s = ffma2(make_float2(xv[2 * v + 1].x, xv[2 * v + 1].y), h2_to_f2(q[v].z), s);
      s = ffma2(make_float2(xv[2 * v + 1].z, xv[2 * v + 1].w), h2_to_f2(q[v].w), s);
    }
  }
  return s.x + s.y;
}

template <int FMT>
__device__ __forceinline__ float load_scale(const void *d, size_t idx) {
  if (Fmt<FMT>::SCALE_BYTES == 0) return 1.0f;
  if (Fmt<FMT>::SCALE_BYTES == 2) return __half2float(__ldg(reinterpret_cast<const __half *>(d) + idx));
  return __ldg(reinterpret_cast<const float *>(d) + idx);
}


// ------------------------------------------------------------------ pipelined kernel
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void *smem_dst, const void *gsrc) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_c() {  // at most N groups still in flight
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void cp_async_wait(int pending) {  // at most `pending` groups still in flight
  switch (pending) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
  }
}

__device__ __forceinline__ int dp4a_su(uint32_t x_s8x4, uint32_t w_u8x4, int c) {
  int r;
  asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(x_s8x4), "r"(w_u8x4), "r"(c));
  return r;
}
__device__ __forceinline__ int dp4a_ss(uint32_t x_s8x4, uint32_t w_s8x4, int c) {
  int r;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(x_s8x4), "r"(w_s8x4), "r"(c));
  return r;
}

// Element of the block that sits in byte slot s (0..31) of the unpacked weight
// bytes: slots 8w..8w+3 are the masked low nibbles of payload word w, 8w+4..8w+7
// its high nibbles; int8 payloads are in natural order.
template <int FMT>
__device__ __forceinline__ int slot_element(int s) {
  if (FMT == GRETA_FMT_Q4_0) return ((s >> 2) & 1) * 16 + (s >> 3) * 4 + (s & 3);
  if (FMT == GRETA_FMT_REF_INT4) return (s >> 3) * 8 + (s & 3) * 2 + ((s >> 2) & 1);
  return s;
}

// Stages the (normalised) activations as block fixed point.  Thread t of each
// group of 8 owns byte slots 4j..4j+3 (j = t & 7) of block t >> 3.
// Layout per block, 28 words: plane p word j at [8p + j]; meta at [24..27] =
// {c0, c1, c2, scale bits}, c_p = -8 * sum of plane p's digits for the offset-8
// nibble formats (0 for int8), folded into the dp4a accumulators.
// Quantises the four values a thread owns (byte slots 4j..4j+3 of block b) together with the seven other
// threads of its block, and stores the block's digit words and meta.  All 32 lanes must call.
template <int FMT>
__device__ __forceinline__ void quantize_store(const float (&v)[4], uint32_t *xq, uint32_t b, int j, bool live) {
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    amax = fmaxf(amax, fabsf(v[k]));
    if (v[k] != v[k]) amax = INFINITY;  // NaN in -> NaN out
  }
#pragma unroll
  for (int o = 1; o <= 4; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  // amax in [2^E, 2^(E+1)): X = rint(x * 2^(21-E)) has |X| <= 2^22, so the signed byte digits
  // d0, d1 in [-128, 127] leave d2 in [-64, 64] even after their carries.
  const uint32_t ab = __float_as_uint(amax);
  const int E = (int)(ab >> 23) - 127;
  float sc, isc;
  if (amax == INFINITY) {
    sc = __uint_as_float(0x7FC00000u);  // poison the block
    isc = 0.f;
  } else if (E < -100) {
    sc = 0.f;  // all (near) zero
    isc = 0.f;
  } else {
    sc = __uint_as_float((uint32_t)(127 + E - 21) << 23);
    isc = __uint_as_float((uint32_t)(127 + 21 - E) << 23);
  }
  uint32_t w0 = 0, w1 = 0, w2 = 0;
  int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    int X = __float2int_rn(v[k] * isc);
    int d0 = (int)(int8_t)(X & 0xFF);  // X = d0 + 256 d1 + 65536 d2, signed byte digits
    int X1 = (X - d0) >> 8;
    int d1 = (int)(int8_t)(X1 & 0xFF);
    int d2 = (X1 - d1) >> 8;
    w0 |= (uint32_t)(d0 & 0xFF) << (8 * k);
    w1 |= (uint32_t)(d1 & 0xFF) << (8 * k);
    w2 |= (uint32_t)(d2 & 0xFF) << (8 * k);
    s0 += d0;
    s1 += d1;
    s2 += d2;
  }
#pragma unroll
  for (int o = 1; o <= 4; o <<= 1) {
    s0 += __shfl_xor_sync(0xffffffffu, s0, o);
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  if (live) {
    uint32_t *blk = xq + (size_t)b * XQ_WORDS;
    blk[j] = w0;
    blk[8 + j] = w1;
    blk[16 + j] = w2;
    if (j == 0) {
      const int off = Fmt<FMT>::NIBBLES ? -8 : 0;
      blk[24] = (uint32_t)(off * s0);
      blk[25] = (uint32_t)(off * s1);
      blk[26] = (uint32_t)(off * s2);
      blk[27] = __float_as_uint(sc);
    }
  }
}

// The four values of byte slots 4j..4j+3 of block b.  For Q4_0 and the int8 formats they are four
// consecutive activations: one 128-bit load.
template <int FMT>
__device__ __forceinline__ void load_slot_values(const float *xf, const __half *xh, const float *gamma, uint32_t b, int j, float (&v)[4],
                                                 float (&gm)[4]) {
  if (FMT != GRETA_FMT_REF_INT4) {
    const uint32_t idx = b * 32 + slot_element<FMT>(4 * j);
    if (xf) {
      const float4 t = __ldcg(reinterpret_cast<const float4 *>(xf + idx));  // bypass L1: another SM may have just written x
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
      const uint2 t = __ldcg(reinterpret_cast<const uint2 *>(xh + idx));
      const float2 a = h2_to_f2(t.x), c = h2_to_f2(t.y);
      v[0] = a.x; v[1] = a.y; v[2] = c.x; v[3] = c.y;
    }
    if (gamma) {
      const float4 t = __ldg(reinterpret_cast<const float4 *>(gamma + idx));
      gm[0] = t.x; gm[1] = t.y; gm[2] = t.z; gm[3] = t.w;
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t idx = b * 32 + slot_element<FMT>(4 * j + k);
      v[k] = xf ? __ldcg(xf + idx) : __half2float(__ldcg(xh + idx));
      if (gamma) gm[k] = gamma[idx];
    }
  }
}

// Stages the (normalised) activations as block fixed point.  Thread t of each group of 8 owns byte
// slots 4j..4j+3 (j = t & 7) of blocks (t >> 3) + 64 i.
//  - RMS-normalised input of up to 4096 values (the decode path of a 4096-wide model): every thread
//    loads its two passes first (one round trip to L2), the RMS comes from those registers, then the
//    blocks are quantised.
//  - otherwise: the RMS, if any, in a pass of its own, then one rolled loop over the blocks.
// The kernel's instruction count per warp is of the order of its code size, so code executed once is
// kept small: two unrolled passes, not one per possible K.
template <int FMT, bool PEER>
__device__ void stage_fixed_point(const GemvParams &p, uint32_t m, uint32_t *xq, float *red) {
  const uint32_t K = p.K, nb = K / 32;
  const float *xf = p.x_is_f16 ? nullptr : reinterpret_cast<const float *>(p.x) + (size_t)m * K;
  const __half *xh = p.x_is_f16 ? reinterpret_cast<const __half *>(p.x) + (size_t)m * K : nullptr;
  const int j = threadIdx.x & 7;
  const uint32_t b0 = threadIdx.x >> 3;
  constexpr int NPR = PEER ? 4 : 2;  // passes kept in registers (the peer form has no other path: K <= 8192)
  if ((p.gamma && nb <= 64 * NPR) || PEER) {
    if (PEER && p.two_level) peer_sum_slice(p, peer_tag(p));
    float v[NPR][4], gm[NPR][4];
#pragma unroll
    for (int i = 0; i < NPR; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[i][k] = 0.f;
        gm[i][k] = 0.f;
      }
      if (b0 + 64 * i < nb) {
        load_slot_values<FMT>(xf, xh, p.gamma, b0 + 64 * i, j, v[i], gm[i]);
        if (PEER) {
          const uint32_t idx = (b0 + 64 * i) * 32 + slot_element<FMT>(4 * j);
          if (p.two_level) {  // the summed stream, published by the CTA that owns the block
#pragma unroll
            for (int k = 0; k < 4; ++k) v[i][k] = 0.f;
            add_tagged_words(p, p.sum_in, 1, idx, peer_tag(p), v[i]);
          } else {
            add_tagged_words(p, p.peer_in, p.tp, idx, peer_tag(p), v[i]);
            if (blockIdx.x == 0) *reinterpret_cast<float4 *>(p.x_out + idx) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
          }
        }
      }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NPR; ++i)
#pragma unroll
      for (int k = 0; k < 4; ++k) ss = fmaf(v[i][k], v[i][k], ss);
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float t = (lane < WARPS) ? red[lane] : 0.f;
    t = warp_sum(t);
    const float inv = rsqrtf(t / (float)K + p.eps);
#pragma unroll
    for (int i = 0; i < NPR; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k) v[i][k] = (v[i][k] * inv) * gm[i][k];
      if ((uint32_t)(64 * i) < nb) quantize_store<FMT>(v[i], xq, b0 + 64 * i, j, b0 + 64 * i < nb);
    }
    return;
  }
  const float inv = p.gamma ? cta_inv_rms(xf, xh, K, p.eps, red) : 1.0f;
  const uint32_t bend = (nb + 63) / 64 * 64;  // uniform trip count for the shuffles
#pragma unroll 1
  for (uint32_t b = b0; b < bend; b += THREADS / 8) {
    const bool live = b < nb;
    float v[4] = {0.f, 0.f, 0.f, 0.f}, gm[4] = {1.f, 1.f, 1.f, 1.f};
    if (live) {
      load_slot_values<FMT>(xf, xh, p.gamma, b, j, v, gm);
      if (p.gamma) {
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = (v[k] * inv) * gm[k];
      }
    }
    quantize_store<FMT>(v, xq, b, j, live);
  }
}

// One block of 32 weights of one row against the fixed-point activations.
// Returns sum_i X_i * q_i (offset already applied) as fp32.
template <int FMT>
__device__ __forceinline__ float block_dot_i(const uint4 *q, const uint4 (&xp)[7]) {
  int s0 = (int)xp[6].x, s1 = (int)xp[6].y, s2 = (int)xp[6].z;
  const uint32_t *p0 = reinterpret_cast<const uint32_t *>(&xp[0]);  // plane p word j at p0[8p + j]
  if (Fmt<FMT>::NIBBLES) {
    const uint32_t flip = (FMT == GRETA_FMT_REF_INT4) ? 0x88888888u : 0u;
    const uint32_t w[4] = {q[0].x ^ flip, q[0].y ^ flip, q[0].z ^ flip, q[0].w ^ flip};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t lo = w[i] & 0x0F0F0F0Fu, hi = (w[i] >> 4) & 0x0F0F0F0Fu;
      s0 = dp4a_su(p0[2 * i], lo, s0);
      s1 = dp4a_su(p0[8 + 2 * i], lo, s1);
      s2 = dp4a_su(p0[16 + 2 * i], lo, s2);
      s0 = dp4a_su(p0[2 * i + 1], hi, s0);
      s1 = dp4a_su(p0[8 + 2 * i + 1], hi, s1);
      s2 = dp4a_su(p0[16 + 2 * i + 1], hi, s2);
    }
  } else {
    const uint32_t w[8] = {q[0].x, q[0].y, q[0].z, q[0].w, q[1].x, q[1].y, q[1].z, q[1].w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s0 = dp4a_ss(p0[i], w[i], s0);
      s1 = dp4a_ss(p0[8 + i], w[i], s1);
      s2 = dp4a_ss(p0[16 + i], w[i], s2);
    }
  }
  // X = d0 + 256 d1 + 65536 d2; |s0 + 256 s1| < 2^31, each term exact in fp32
  return fmaf(65536.f, (float)s2, (float)(s0 + (s1 << 8)));
}


}  // namespace
