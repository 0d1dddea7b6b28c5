// Batched decode matmul: y[M x N] = x[M x K] * dequant(W)^T for M = 2..32 activation rows (one per
// sequence of a decode batch), with the same RMSNorm prologue and RoPE / KV-cache / SwiGLU / residual
// epilogues as the single-row GEMV.  The weights are streamed from HBM ONCE for all M rows, so the work
// stays HBM-bound (0.5625 B per weight for Q4_0) where a per-row GEMV would read them M times.
//
//   * A CTA owns 128 or 256 weight rows (16-row tiles, one or two per warp, 8 warps) over one slice of K.
//     Weight tiles travel global -> shared with 16-byte cp.async copies into a per-warp ring of 8-block
//     cells (a row of a cell is 8 quant payloads followed by their 8 fp16 scales: 144 bytes for Q4_0, a
//     stride that keeps the 4-byte fragment reads free of bank conflicts).
//   * One weight block meets all M activation rows in the tensor cores: the nibbles (bytes, halves) are
//     unpacked to the exact small integers q - 8 as fp16 and fed to mma.sync m16n8k16 as the 16-row
//     operand, the activations are the 8-column operand, fp32 accumulation over the 32 values of the
//     block; the block's fp16 scale is applied to the 16 x 8 block sums with fp32 FMAs.  Per-block
//     scales rule out accumulating across blocks inside the tensor core (and with it TMEM): the block
//     sums have to come back to registers every 32 values, which is what mma.sync does by construction.
//     The kernel is bound by HBM and by instruction issue, not by the tensor pipe.
//   * Activations keep fp32 precision: each value is split into two fp16 numbers, hi = half(x * s) and
//     lo = half(x * s - hi), s a power of two chosen per row and per K-chunk so that the chunk's largest
//     value sits near 2^14; both parts run through the same accumulator.  Every product is exact; the
//     split loses less than 2^-22 of the chunk's largest value.
//   * The rows of x are converted once per CTA and K-chunk (1024 values) into the fragment order of the
//     matrix instruction; the raw values of the next chunk are fetched into registers while the current
//     chunk is being multiplied.  With an RMSNorm in front, the weights gamma are folded into x during
//     the conversion and 1/rms is applied to the finished sums (it is a per-row factor), so no CTA has
//     to see a whole row before it starts.
//   * K is split over the CTAs of a thread-block cluster (1, 2, 4 or 8); partial sums and the partial
//     sums of squares meet through distributed shared memory in rank order (deterministic), each CTA
//     finishing a share of the tiles: 1/rms, RoPE at each sequence's own position, the fp16 KV-cache
//     write, SwiGLU or the residual add.
//   * Rows that an epilogue combines (gate / up of one output, the two halves of a rotation pair) are
//     rows j and j + 8 of a tile: the matrix instruction leaves both in the same thread.
#include <cooperative_groups.h>
#include <math.h>

#include <algorithm>

#include "gemv_device.cuh"

namespace {

namespace cg = cooperative_groups;

constexpr int BW = 8;                  // warps per CTA
constexpr int BTHREADS = BW * 32;
constexpr int CELL = 8;                // quant blocks per cell (256 values of K)
constexpr size_t BSMEM_LIMIT = 224 * 1024;

template <int FMT>
struct BFmt;
template <>
struct BFmt<GRETA_FMT_Q4_0> {
  static constexpr int PB = 16, SCALE_PIECES = 1, TPW_MAX = 2, XBLOCKS = 64;  // XBLOCKS: quant blocks of x staged per chunk and 8 rows
};
template <>
struct BFmt<GRETA_FMT_Q8_0> {
  static constexpr int PB = 32, SCALE_PIECES = 1, TPW_MAX = 1, XBLOCKS = 32;
};
template <>
struct BFmt<GRETA_FMT_F16> {
  static constexpr int PB = 64, SCALE_PIECES = 0, TPW_MAX = 1, XBLOCKS = 32;
};

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The two k16 operand sets of one quant block of one weight row, as exact fp16 integers (or the fp16 weights
// themselves).  `row` points at the block's payload in the staged cell, t = lane & 3.
// Element order inside a matrix-instruction step follows the unpacking; the activations are staged in the
// same order (unit_order below).
template <int FMT>
__device__ __forceinline__ void weight_frags(const uint8_t *row, int t, uint32_t (&lo)[2], uint32_t (&hi)[2]) {
  if (FMT == GRETA_FMT_Q4_0) {  // word t: low nibbles = elements 4t..4t+3, high nibbles = elements 16+4t..16+4t+3
    const uint32_t w = *reinterpret_cast<const uint32_t *>(row + 4 * t), w8 = w >> 8;
    const uint32_t MAGIC = 0x64006400u, C1032 = 0x64086408u, SIXTEENTH = 0x2C002C00u, CM72 = 0xD480D480u;
    lo[0] = hsub2_u(lop_and_or(w, 0x000F000Fu, MAGIC), C1032);              // (e4t, e4t+2)
    lo[1] = hsub2_u(lop_and_or(w8, 0x000F000Fu, MAGIC), C1032);             // (e4t+1, e4t+3)
    hi[0] = hfma2_u(lop_and_or(w, 0x00F000F0u, MAGIC), SIXTEENTH, CM72);    // (e16+4t, e16+4t+2)
    hi[1] = hfma2_u(lop_and_or(w8, 0x00F000F0u, MAGIC), SIXTEENTH, CM72);   // (e16+4t+1, e16+4t+3)
  } else if (FMT == GRETA_FMT_Q8_0) {  // word t = elements 4t..4t+3, word 4+t = elements 16+4t..16+4t+3
    const uint32_t C1152 = 0x64806480u;
    const uint32_t a = *reinterpret_cast<const uint32_t *>(row + 4 * t) ^ 0x80808080u;
    const uint32_t b = *reinterpret_cast<const uint32_t *>(row + 16 + 4 * t) ^ 0x80808080u;
    lo[0] = hsub2_u(__byte_perm(a, 0x64646464u, 0x5140), C1152);
    lo[1] = hsub2_u(__byte_perm(a, 0x64646464u, 0x7362), C1152);
    hi[0] = hsub2_u(__byte_perm(b, 0x64646464u, 0x5140), C1152);
    hi[1] = hsub2_u(__byte_perm(b, 0x64646464u, 0x7362), C1152);
  } else {  // fp16 weights: word w = elements 2w, 2w+1
    const uint32_t *wp = reinterpret_cast<const uint32_t *>(row);
    lo[0] = wp[t];
    lo[1] = wp[4 + t];
    hi[0] = wp[8 + t];
    hi[1] = wp[12 + t];
  }
}

// The eight activations of a block that thread t of a quad multiplies, in the order the weight fragments
// pair them: e[0..3] belong to the first k16 step (b0 = e0,e1; b1 = e2,e3), e[4..7] to the second.
// `raw` holds what load_unit fetched.
template <int FMT>
__device__ __forceinline__ void unit_order(const float (&raw)[8], float (&e)[8]) {
  if (FMT == GRETA_FMT_Q4_0) {  // raw = x[4t..4t+3], x[16+4t..16+4t+3]
    e[0] = raw[0]; e[1] = raw[2]; e[2] = raw[1]; e[3] = raw[3];
    e[4] = raw[4]; e[5] = raw[6]; e[6] = raw[5]; e[7] = raw[7];
  } else {                      // Q8_0: same loads, natural order; F16: raw = x[2t,2t+1], x[8+2t..], x[16+2t..], x[24+2t..]
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = raw[j];
  }
}
template <int FMT>
__device__ __forceinline__ void load_unit(const float *xk, const float *gk, int t, float (&raw)[8]) {  // xk: first value of the block
  if (FMT == GRETA_FMT_F16) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 v = __ldcg(reinterpret_cast<const float2 *>(xk + 8 * j + 2 * t));
      raw[2 * j] = v.x;
      raw[2 * j + 1] = v.y;
    }
  } else {
    const float4 a = __ldcg(reinterpret_cast<const float4 *>(xk + 4 * t)), b = __ldcg(reinterpret_cast<const float4 *>(xk + 16 + 4 * t));
    raw[0] = a.x; raw[1] = a.y; raw[2] = a.z; raw[3] = a.w;
    raw[4] = b.x; raw[5] = b.y; raw[6] = b.z; raw[7] = b.w;
  }
}
template <int FMT>
__device__ __forceinline__ void load_unit_gamma(const float *gk, int t, float (&gm)[8]) {
  if (FMT == GRETA_FMT_F16) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 v = __ldg(reinterpret_cast<const float2 *>(gk + 8 * j + 2 * t));
      gm[2 * j] = v.x;
      gm[2 * j + 1] = v.y;
    }
  } else {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(gk + 4 * t)), b = __ldg(reinterpret_cast<const float4 *>(gk + 16 + 4 * t));
    gm[0] = a.x; gm[1] = a.y; gm[2] = a.z; gm[3] = a.w;
    gm[4] = b.x; gm[5] = b.y; gm[6] = b.z; gm[7] = b.w;
  }
}

__device__ __forceinline__ uint32_t pack_h2(__half a, __half b) {
  return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
}

// The epilogue of one accumulator fragment of tile `grp`: v.x / v.y are row slot g of the tile for activation rows m0 and
// m0 + 1, v.z / v.w row slot g + 8 (the partner row of an epilogue pair) for the same two activation rows.
template <int EPI>
__device__ __forceinline__ void finish_fragment(const GemvParams &p, uint32_t grp, int g, uint32_t m0, float4 v, const float2 *rope_cs) {
  const float va[2] = {v.x, v.y}, vb[2] = {v.z, v.w};
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const uint32_t m = m0 + e;
    if (m >= p.M) continue;
    const float a = va[e], b = vb[e];
    if (EPI == EPI_PLAIN || EPI == EPI_RESIDUAL) {
      const uint32_t ra = grp * 16 + g, rb = ra + 8;
      if (ra < p.N) p.y[(size_t)m * p.N + ra] = (EPI == EPI_RESIDUAL ? __ldcg(p.resid + (size_t)m * p.N + ra) : 0.f) + a;
      if (rb < p.N) p.y[(size_t)m * p.N + rb] = (EPI == EPI_RESIDUAL ? __ldcg(p.resid + (size_t)m * p.N + rb) : 0.f) + b;
    } else if (EPI == EPI_SWIGLU) {
      const uint32_t o = grp * 8 + g;
      if (o < p.N) p.y[(size_t)m * p.N + o] = (a / (1.0f + expf(-a))) * b;
    } else {  // EPI_QKV
      const uint32_t gph = (p.Dh / 2) / 8, nq = p.H * gph, nk = p.Hkv * gph;
      const uint32_t pos = p.d_pos ? __ldcg(p.d_pos + m) : 0u;
      if (grp < nq + nk) {
        const bool is_q = grp < nq;
        const uint32_t gi = is_q ? grp : grp - nq, head = gi / gph, i = (gi % gph) * 8 + g;
        float o0 = a, o1 = b;
        if (p.d_pos) {
          const float2 c = rope_cs[m * 64 + i];
          o0 = a * c.x - b * c.y;
          o1 = a * c.y + b * c.x;
        }
        if (is_q) {
          float *q = p.q_out + (size_t)m * p.H * p.Dh + head * p.Dh + i;
          q[0] = o0;
          q[p.Dh / 2] = o1;
        } else {
          if (p.k_out) {
            float *k = p.k_out + (size_t)m * p.Hkv * p.Dh + head * p.Dh + i;
            k[0] = o0;
            k[p.Dh / 2] = o1;
          }
          if (p.k_cache && pos < p.max_seq) {  // a position past the cache is never written
            __half *k = p.k_cache + (((size_t)m * p.Hkv + head) * p.max_seq + pos) * p.Dh + i;
            k[0] = __float2half_rn(o0);
            k[p.Dh / 2] = __float2half_rn(o1);
          }
        }
      } else {
        const float vv[2] = {a, b};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t row = (grp - nq - nk) * 16 + g + 8 * h;
          if (row < p.Hkv * p.Dh) {
            if (p.v_out) p.v_out[(size_t)m * p.Hkv * p.Dh + row] = vv[h];
            if (p.v_cache && pos < p.max_seq)
              p.v_cache[(((size_t)m * p.Hkv + row / p.Dh) * p.max_seq + pos) * p.Dh + row % p.Dh] = __float2half_rn(vv[h]);
          }
        }
      }
    }
  }
}

// (cos, sin) of every row's rotation angles at its own position: [rows][64] for head_dim <= 128.
__device__ __forceinline__ void fill_rope_rows(const GemvParams &p, float2 *rope_cs, int tid, int nthreads) {
  for (uint32_t idx = tid; idx < p.M * (p.Dh / 2); idx += nthreads) {
    const uint32_t m = idx / (p.Dh / 2), i = idx % (p.Dh / 2);
    const float theta = (float)__ldcg(p.d_pos + m) * powf(p.rope_base, -2.0f * (float)i / (float)p.Dh);
    rope_cs[m * 64 + i] = make_float2(cosf(theta), sinf(theta));
  }
}

struct RowSrc {
  const uint8_t *qs;  // payload of the row's first block
  const uint8_t *d;   // the row's first scale
};

// MT: 8-row groups of activations (M <= 8 MT).  TPW: 16-row weight tiles per warp.
template <int FMT, int EPI, int MT, int TPW>
__global__ void __launch_bounds__(BTHREADS, 1) gemv_batch_kernel(const GemvParams p) {
  using F = BFmt<FMT>;
  constexpr int PB = F::PB;
  constexpr int ROWB = CELL * PB + 16;                        // staged bytes per weight row and cell (payloads, then scales / padding)
  constexpr int PPR = CELL * PB / 16 + F::SCALE_PIECES;       // 16-byte copies per row and cell
  constexpr int STAGE = TPW * 16 * ROWB;                      // bytes per warp and ring stage
  constexpr int XB = F::XBLOCKS / MT;                         // quant blocks of x per chunk
  constexpr int XCELLS = XB / CELL;
  constexpr int XFRAG = XB * MT * 1024;                       // bytes: per block and row group 32 lanes x (16 B hi + 16 B lo)
  constexpr int ROWTAB = BW * TPW * 16 * (int)sizeof(RowSrc);
  constexpr int DEPTH_ROOM = (int)((BSMEM_LIMIT - XFRAG - ROWTAB) / (BW * STAGE));
  constexpr int DEPTH = DEPTH_ROOM > 6 ? 6 : DEPTH_ROOM;
  constexpr int MP = 8 * MT;                                  // activation rows, padded
  constexpr int TPT = BTHREADS / MP;                          // threads that convert one activation row
  constexpr int UPT = XB * 4 / TPT;                           // 8-value units per thread and chunk
  static_assert(XCELLS >= 1 && DEPTH >= 2 && UPT >= 1, "shared memory plan");
  static_assert(BW * TPW * MT * 512 <= XFRAG && MP * 8 + MP * 64 * 8 <= BW * DEPTH * STAGE, "the finishing data reuses the staging buffers");

  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t *xfrag = smem;
  RowSrc *rowtab = reinterpret_cast<RowSrc *>(smem + XFRAG);
  uint8_t *ring = smem + XFRAG + ROWTAB;
  __shared__ float inv_s[MP];

  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const uint32_t kw = gridDim.x, rank = blockIdx.x;           // the cluster spans x: one CTA per K slice
  const uint32_t nb = p.K / 32, ncell = (nb + CELL - 1) / CELL;
  const uint32_t cs = (uint32_t)((uint64_t)rank * ncell / kw), ce = (uint32_t)((uint64_t)(rank + 1) * ncell / kw);
  const uint32_t tile0 = (blockIdx.y * BW + warp) * TPW;      // this warp's first tile (row group of 16)
  const uint32_t M = p.M;

  // ---- where this warp's rows live
  RowSrc *mytab = rowtab + warp * TPW * 16;
  for (int r = lane; r < TPW * 16; r += 32) {
    int mat;
    uint32_t row;
    if (!resolve<EPI, 16>(p, tile0 + r / 16, r % 16, &mat, &row)) {  // ragged tail: stream row 0, never stored
      mat = 0;
      row = 0;
    }
    RowSrc s;
    s.qs = p.w[mat].qs + (size_t)row * nb * PB;
    s.d = F::SCALE_PIECES ? reinterpret_cast<const uint8_t *>(p.w[mat].d) + (size_t)row * d_row_stride(nb) * 2 : nullptr;
    mytab[r] = s;
  }
  __syncwarp();

  uint8_t *myring = ring + (size_t)warp * DEPTH * STAGE;
  uint32_t pc = cs, pstage = 0;
  auto request = [&]() {  // requests cell pc into stage pstage
    if (pc < ce) {
      uint8_t *st = myring + pstage * STAGE;
#pragma unroll 1
      for (int q = lane; q < TPW * 16 * PPR; q += 32) {
        const int r = q / PPR, part = q - r * PPR;
        const RowSrc s = mytab[r];
        if (part < CELL * PB / 16) {
          const uint32_t blk = pc * CELL + (uint32_t)(part * 16) / PB;
          if (blk < nb) cp_async16(st + r * ROWB + part * 16, s.qs + (size_t)pc * CELL * PB + part * 16);
        } else {
          cp_async16(st + r * ROWB + CELL * PB, s.d + (size_t)pc * CELL * 2);  // 8 scales; rows are padded to 8
        }
      }
      ++pc;
    }
    cp_async_commit();
    pstage = (pstage + 1 == DEPTH) ? 0 : pstage + 1;
  };
  for (int s = 0; s + 1 < DEPTH; ++s) request();
  pdl_launch_dependents();
  pdl_wait();  // everything below reads what the previous kernel wrote

  // ---- activation conversion: thread owns units (block kbl, quad lane ut) of row cm
  const int cm = tid / TPT, cj = tid % TPT;
  const bool crow = (uint32_t)cm < M;
  const float *xrow = reinterpret_cast<const float *>(p.x) + (size_t)cm * p.K;
  float xr[UPT][8];
  float ss_run = 0.f;
  auto fetch = [&](uint32_t chunk_cell) {  // raw values of the chunk that starts at cell chunk_cell
#pragma unroll
    for (int i = 0; i < UPT; ++i) {
      const int u = cj + TPT * i, kbl = u >> 2, ut = u & 3;
      const uint32_t blk = chunk_cell * CELL + kbl;
      if (crow && blk < nb && blk < ce * CELL) {
        load_unit<FMT>(xrow + (size_t)blk * 32, nullptr, ut, xr[i]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) xr[i][j] = 0.f;
      }
    }
  };
  auto convert = [&](uint32_t chunk_cell) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < UPT; ++i) {
      const int u = cj + TPT * i, kbl = u >> 2, ut = u & 3;
      const uint32_t blk = chunk_cell * CELL + kbl;
      if (p.gamma) {
        float gm[8];
        if (blk < nb) {
          load_unit_gamma<FMT>(p.gamma + (size_t)blk * 32, ut, gm);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) gm[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ss_run = fmaf(xr[i][j], xr[i][j], ss_run);
          xr[i][j] *= gm[j];
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        amax = fmaxf(amax, fabsf(xr[i][j]));
        if (xr[i][j] != xr[i][j]) amax = INFINITY;
      }
    }
#pragma unroll
    for (int o = 1; o < TPT; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // amax in [2^E, 2^(E+1)): scale by 2^(14-E), the largest value lands in [2^14, 2^15)
    float s = 1.f, is = 1.f;
    if (amax > 0.f && amax < INFINITY) {
      const int E = (int)(__float_as_uint(amax) >> 23) - 127;
      const int e = max(-100, min(100, 14 - E));
      s = __uint_as_float((uint32_t)(127 + e) << 23);
      is = __uint_as_float((uint32_t)(127 - e) << 23);
    }
    if (cj == 0) inv_s[cm] = is;
#pragma unroll
    for (int i = 0; i < UPT; ++i) {
      const int u = cj + TPT * i, kbl = u >> 2, ut = u & 3;
      float e[8];
      unit_order<FMT>(xr[i], e);
      __half h[8], l[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = e[j] * s;
        h[j] = __float2half_rn(f);
        l[j] = __float2half_rn(f - __half2float(h[j]));
      }
      uint8_t *dst = xfrag + ((size_t)(kbl * MT + (cm >> 3)) * 2) * 512 + ((cm & 7) * 4 + ut) * 16;
      *reinterpret_cast<uint4 *>(dst) = make_uint4(pack_h2(h[0], h[1]), pack_h2(h[2], h[3]), pack_h2(h[4], h[5]), pack_h2(h[6], h[7]));
      *reinterpret_cast<uint4 *>(dst + 512) = make_uint4(pack_h2(l[0], l[1]), pack_h2(l[2], l[3]), pack_h2(l[4], l[5]), pack_h2(l[6], l[7]));
    }
  };

  float acc[TPW][MT][4];
#pragma unroll
  for (int i = 0; i < TPW; ++i)
#pragma unroll
    for (int G = 0; G < MT; ++G)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][G][j] = 0.f;

  fetch(cs);
  uint32_t cstage = 0;
  for (uint32_t chunk = cs; chunk < ce; chunk += XCELLS) {
    __syncthreads();  // every warp is done with the previous chunk's activations
    convert(chunk);
    __syncthreads();
    if (chunk + XCELLS < ce) fetch(chunk + XCELLS);  // in flight while this chunk is multiplied
    float part[TPW][MT][4];
#pragma unroll
    for (int i = 0; i < TPW; ++i)
#pragma unroll
      for (int G = 0; G < MT; ++G)
#pragma unroll
        for (int j = 0; j < 4; ++j) part[i][G][j] = 0.f;
    const uint32_t cend = min(ce, chunk + XCELLS);
    for (uint32_t c = chunk; c < cend; ++c) {
      cp_async_wait_c<DEPTH - 2>();
      __syncwarp();
      request();  // refills the stage that the previous iteration consumed
      const uint8_t *st = myring + cstage * STAGE;
      cstage = (cstage + 1 == DEPTH) ? 0 : cstage + 1;
      const uint32_t nvalid = min((uint32_t)CELL, nb - c * CELL);
#pragma unroll 2
      for (uint32_t kb = 0; kb < nvalid; ++kb) {
        const uint32_t kbl = (c - chunk) * CELL + kb;
        uint4 xh[MT], xl[MT];
#pragma unroll
        for (int G = 0; G < MT; ++G) {
          const uint8_t *src = xfrag + ((size_t)(kbl * MT + G) * 2) * 512 + lane * 16;
          xh[G] = *reinterpret_cast<const uint4 *>(src);
          xl[G] = *reinterpret_cast<const uint4 *>(src + 512);
        }
#pragma unroll
        for (int i = 0; i < TPW; ++i) {
          const uint8_t *r0 = st + (i * 16 + g) * ROWB, *r1 = r0 + 8 * ROWB;
          uint32_t lo0[2], hi0[2], lo1[2], hi1[2];
          weight_frags<FMT>(r0 + kb * PB, t, lo0, hi0);
          weight_frags<FMT>(r1 + kb * PB, t, lo1, hi1);
          float d0 = 1.f, d1 = 1.f;
          if (F::SCALE_PIECES) {
            d0 = __half2float(*reinterpret_cast<const __half *>(r0 + CELL * PB + kb * 2));
            d1 = __half2float(*reinterpret_cast<const __half *>(r1 + CELL * PB + kb * 2));
          }
#pragma unroll
          for (int G = 0; G < MT; ++G) {
            float s4[4] = {0.f, 0.f, 0.f, 0.f};
            mma_f16(s4, lo0[0], lo1[0], lo0[1], lo1[1], xh[G].x, xh[G].y);
            mma_f16(s4, hi0[0], hi1[0], hi0[1], hi1[1], xh[G].z, xh[G].w);
            mma_f16(s4, lo0[0], lo1[0], lo0[1], lo1[1], xl[G].x, xl[G].y);
            mma_f16(s4, hi0[0], hi1[0], hi0[1], hi1[1], xl[G].z, xl[G].w);
            part[i][G][0] = fmaf(s4[0], d0, part[i][G][0]);
            part[i][G][1] = fmaf(s4[1], d0, part[i][G][1]);
            part[i][G][2] = fmaf(s4[2], d1, part[i][G][2]);
            part[i][G][3] = fmaf(s4[3], d1, part[i][G][3]);
          }
        }
      }
    }
    // fold the chunk in: undo the chunk's power-of-two scale of each activation row
#pragma unroll
    for (int G = 0; G < MT; ++G) {
      const float i0 = inv_s[8 * G + 2 * t], i1 = inv_s[8 * G + 2 * t + 1];
#pragma unroll
      for (int i = 0; i < TPW; ++i) {
        acc[i][G][0] = fmaf(part[i][G][0], i0, acc[i][G][0]);
        acc[i][G][1] = fmaf(part[i][G][1], i1, acc[i][G][1]);
        acc[i][G][2] = fmaf(part[i][G][2], i0, acc[i][G][2]);
        acc[i][G][3] = fmaf(part[i][G][3], i1, acc[i][G][3]);
      }
    }
  }
  cp_async_wait(0);
  __syncthreads();  // the activation buffer is free: it now carries the finishing data

  // ---- publish this CTA's share: partial sums per tile in fragment order, partial sums of squares, rotation table
  float4 *pub = reinterpret_cast<float4 *>(xfrag);            // [BW * TPW tiles][MT][32 lanes], in the activation buffer
  float *pss = reinterpret_cast<float *>(ring);                // [MP], in the (drained) weight ring
  float2 *rope_cs = reinterpret_cast<float2 *>(ring + MP * 8); // [MP][64]: (cos, sin) per row and pair index, head_dim <= 128
#pragma unroll
  for (int i = 0; i < TPW; ++i)
#pragma unroll
    for (int G = 0; G < MT; ++G) pub[((warp * TPW + i) * MT + G) * 32 + lane] = make_float4(acc[i][G][0], acc[i][G][1], acc[i][G][2], acc[i][G][3]);
  if (p.gamma) {
#pragma unroll
    for (int o = 1; o < TPT; o <<= 1) ss_run += __shfl_xor_sync(0xffffffffu, ss_run, o);
    if (cj == 0) pss[cm] = ss_run;
  }
  if (EPI == EPI_QKV && p.d_pos) fill_rope_rows(p, rope_cs, tid, BTHREADS);
  cluster.sync();

  // ---- finish: tile L of this row group is finished by the CTA of rank L % kw
  for (uint32_t L = warp; L < (uint32_t)(BW * TPW); L += BW) {
    if (L % kw != rank) continue;
    const uint32_t grp = blockIdx.y * BW * TPW + L;
    if (grp >= p.groups) continue;
#pragma unroll
    for (int G = 0; G < MT; ++G) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      float ss0 = 0.f, ss1 = 0.f;
      const uint32_t m0 = 8 * G + 2 * t, m1 = m0 + 1;
      for (uint32_t j = 0; j < kw; ++j) {  // rank order: the result does not depend on which CTA finished first
        const float4 q = cluster.map_shared_rank(pub, j)[(L * MT + G) * 32 + lane];
        v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
        if (p.gamma) {
          const float *ps = cluster.map_shared_rank(pss, j);
          ss0 += ps[m0];
          ss1 += ps[m1];
        }
      }
      if (p.gamma) {
        const float r0 = rsqrtf(ss0 / (float)p.K + p.eps), r1 = rsqrtf(ss1 / (float)p.K + p.eps);
        v.x *= r0; v.z *= r0;
        v.y *= r1; v.w *= r1;
      }
      finish_fragment<EPI>(p, grp, g, m0, v, rope_cs);
    }
  }
  cluster.sync();  // a CTA's shared memory must outlive the other ranks' reads
}

// ------------------------------------------------------------------ prepared activations
// The conversion of x into fragment-ordered fp16 pairs does not depend on the weight rows: done inside the matmul kernel,
// every CTA of every row group repeats it (a third of that kernel's instructions).  Given workspace, the batched entry
// points run it once instead, in a small kernel of its own (one CTA per activation row), and the matmul kernel copies the
// prepared fragments straight from global to shared memory.
//   workspace: [32 floats] row factors (1 / power-of-two scale of the row, times 1 / rms with an RMSNorm in front), then
//   [K / 32 blocks][MT groups][hi | lo][32 lanes][16 B]: 4 bytes per value, the layout the kernel above builds in shared memory.
constexpr int PREP_THREADS = 512;
constexpr size_t PREP_HEADER = 256;

template <int FMT, int MT>
__global__ void __launch_bounds__(PREP_THREADS) prep_rows_kernel(const float *__restrict__ x, const float *__restrict__ gamma, float eps, uint32_t M,
                                                                 uint32_t K, uint8_t *__restrict__ ws) {
  __shared__ float red_max[PREP_THREADS / 32], red_ss[PREP_THREADS / 32];
  pdl_launch_dependents();
  pdl_wait();  // x comes from the previous kernel; the previous matmul kernel has finished with the workspace
  const uint32_t m = blockIdx.x, nb = K / 32, units = nb * 4;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint8_t *frag = ws + PREP_HEADER;
  const float *xrow = x + (size_t)m * K;
  const bool live = m < M;
  float amax = 0.f, ss = 0.f;
  if (live) {
    for (uint32_t u = tid; u < units; u += PREP_THREADS) {
      float raw[8], gm[8];
      load_unit<FMT>(xrow + (size_t)(u >> 2) * 32, nullptr, u & 3, raw);
      if (gamma) load_unit_gamma<FMT>(gamma + (size_t)(u >> 2) * 32, u & 3, gm);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        ss = fmaf(raw[j], raw[j], ss);
        const float v = gamma ? raw[j] * gm[j] : raw[j];
        amax = fmaxf(amax, fabsf(v));
        if (v != v) amax = INFINITY;
      }
    }
  }
  amax = warp_max(amax);
  ss = warp_sum(ss);
  if (lane == 0) {
    red_max[warp] = amax;
    red_ss[warp] = ss;
  }
  __syncthreads();
  amax = 0.f;
  ss = 0.f;
#pragma unroll
  for (int w = 0; w < PREP_THREADS / 32; ++w) {  // fixed order
    amax = fmaxf(amax, red_max[w]);
    ss += red_ss[w];
  }
  float s = 1.f, is = 1.f;
  if (amax > 0.f && amax < INFINITY) {  // amax in [2^E, 2^(E+1)): scale by 2^(14-E)
    const int E = (int)(__float_as_uint(amax) >> 23) - 127;
    const int e = max(-100, min(100, 14 - E));
    s = __uint_as_float((uint32_t)(127 + e) << 23);
    is = __uint_as_float((uint32_t)(127 - e) << 23);
  }
  if (tid == 0) reinterpret_cast<float *>(ws)[m] = live ? is * (gamma ? rsqrtf(ss / (float)K + eps) : 1.f) : 0.f;
  const uint32_t G = m >> 3, g = m & 7;
  for (uint32_t u = tid; u < units; u += PREP_THREADS) {
    const uint32_t kbl = u >> 2, ut = u & 3;
    float raw[8], gm[8], e[8];
    if (live) {
      load_unit<FMT>(xrow + (size_t)kbl * 32, nullptr, ut, raw);
      if (gamma) {
        load_unit_gamma<FMT>(gamma + (size_t)kbl * 32, ut, gm);
#pragma unroll
        for (int j = 0; j < 8; ++j) raw[j] *= gm[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) raw[j] = 0.f;
    }
    unit_order<FMT>(raw, e);
    __half h[8], l[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = e[j] * s;
      h[j] = __float2half_rn(f);
      l[j] = __float2half_rn(f - __half2float(h[j]));
    }
    uint8_t *dst = frag + ((size_t)(kbl * MT + G) * 2) * 512 + (g * 4 + ut) * 16;
    *reinterpret_cast<uint4 *>(dst) = make_uint4(pack_h2(h[0], h[1]), pack_h2(h[2], h[3]), pack_h2(h[4], h[5]), pack_h2(h[6], h[7]));
    *reinterpret_cast<uint4 *>(dst + 512) = make_uint4(pack_h2(l[0], l[1]), pack_h2(l[2], l[3]), pack_h2(l[4], l[5]), pack_h2(l[6], l[7]));
  }
}

template <int FMT>
struct PFmt;  // warps per CTA, CTAs per SM the shared-memory plan aims at
template <>
struct PFmt<GRETA_FMT_Q4_0> {
  static constexpr int NW = 8, CTAS_PER_SM = 2;  // 3 (a two-stage weight ring) was measured: 28672 x 8192 gate/up 186 vs 210 us, but 8192 x 8192 41.5 vs 31.0 us
};
template <>
struct PFmt<GRETA_FMT_Q8_0> {
  static constexpr int NW = 8, CTAS_PER_SM = 2;
};
template <>
struct PFmt<GRETA_FMT_F16> {
  static constexpr int NW = 8, CTAS_PER_SM = 1;
};

template <int FMT, int MT>
struct PPlan {
  static constexpr int NW = PFmt<FMT>::NW, PB = BFmt<FMT>::PB;
  static constexpr int ROWB = CELL * PB + 16, STAGE = 16 * ROWB;
  static constexpr int ROWTAB = NW * 16 * (int)sizeof(RowSrc);
  static constexpr int room_in(int limit, int xcells) { return (limit - 2 * xcells * CELL * MT * 1024 - ROWTAB) / (NW * STAGE); }
  // CTAs per SM this plan fits: the most that the format aims at and that leaves a weight ring of at least two stages
  static constexpr int CTAS = (PFmt<FMT>::CTAS_PER_SM >= 3 && room_in(74 * 1024, 1) >= 2) ? 3 : ((PFmt<FMT>::CTAS_PER_SM >= 2 && room_in(112 * 1024, 1) >= 2) ? 2 : 1);
  static constexpr int LIMIT = CTAS == 3 ? 74 * 1024 : (CTAS == 2 ? 112 * 1024 : (int)BSMEM_LIMIT);
  // Two activation buffers of XCELLS cells each; a buffer is refilled XCELLS cells ahead, which the weight ring must
  // cover: XCELLS <= DEPTH - 1.  Two CTAs of 8 warps per SM (128 rows each) balance the SMs better than one of 16.
  static constexpr int room(int xcells) { return room_in(LIMIT, xcells); }
  static constexpr int XCELLS = (MT < 4 && room(2) >= 3) ? 2 : 1;
  static constexpr int DEPTH = room(XCELLS) > 4 ? 4 : room(XCELLS);
  static constexpr int XBUF = XCELLS * CELL * MT * 1024;
  static constexpr size_t SMEM = (size_t)2 * XBUF + ROWTAB + (size_t)NW * DEPTH * STAGE;
  static_assert(DEPTH >= 2 && XCELLS <= DEPTH - 1, "shared memory plan");
};

__device__ __forceinline__ void mma_f16_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// The matmul on prepared activations: NW warps, one 16-row tile per warp, K split over the cluster as above.  All warps
// walk the cells of the slice in step; the prepared activations of the next cells arrive by cp.async in the same commit
// groups as the weight cells, one CTA-wide barrier per activation buffer.
template <int FMT, int EPI, int MT>
__global__ void __launch_bounds__(PFmt<FMT>::NW * 32, PPlan<FMT, MT>::CTAS) gemv_batchp_kernel(const GemvParams p) {
  using F = BFmt<FMT>;
  using P = PPlan<FMT, MT>;
  constexpr int NW = P::NW, PB = F::PB, ROWB = P::ROWB, STAGE = P::STAGE, DEPTH = P::DEPTH, XCELLS = P::XCELLS, XBUF = P::XBUF;
  constexpr int PPR = CELL * PB / 16 + F::SCALE_PIECES;
  constexpr int NT = NW * 32;
  static_assert(NW * MT * 512 <= 2 * XBUF && 8 * MT * 64 * 8 <= NW * DEPTH * STAGE, "the finishing data reuses the staging buffers");

  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t *xbuf = smem;
  RowSrc *rowtab = reinterpret_cast<RowSrc *>(smem + 2 * XBUF);
  uint8_t *ring = smem + 2 * XBUF + P::ROWTAB;

  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const uint32_t kw = gridDim.x, rank = blockIdx.x;
  const uint32_t nb = p.K / 32, ncell = (nb + CELL - 1) / CELL;
  const uint32_t cs = (uint32_t)((uint64_t)rank * ncell / kw), ce = (uint32_t)((uint64_t)(rank + 1) * ncell / kw);
  const uint32_t tile = blockIdx.y * NW + warp;

  RowSrc *mytab = rowtab + warp * 16;
  if (lane < 16) {
    int mat;
    uint32_t row;
    if (!resolve<EPI, 16>(p, tile, lane, &mat, &row)) {  // ragged tail: stream row 0, never stored
      mat = 0;
      row = 0;
    }
    RowSrc s;
    s.qs = p.w[mat].qs + (size_t)row * nb * PB;
    s.d = F::SCALE_PIECES ? reinterpret_cast<const uint8_t *>(p.w[mat].d) + (size_t)row * d_row_stride(nb) * 2 : nullptr;
    mytab[lane] = s;
  }
  __syncwarp();

  uint8_t *myring = ring + (size_t)warp * DEPTH * STAGE;
  uint32_t pc = cs, pstage = 0;
  auto request_weights = [&]() {  // copies of cell pc into stage pstage (no commit)
    if (pc < ce) {
      uint8_t *st = myring + pstage * STAGE;
#pragma unroll 1
      for (int q = lane; q < 16 * PPR; q += 32) {
        const int r = q / PPR, part = q - r * PPR;
        const RowSrc s = mytab[r];
        if (part < CELL * PB / 16) {
          const uint32_t blk = pc * CELL + (uint32_t)(part * 16) / PB;
          if (blk < nb) cp_async16(st + r * ROWB + part * 16, s.qs + (size_t)pc * CELL * PB + part * 16);
        } else {
          cp_async16(st + r * ROWB + CELL * PB, s.d + (size_t)pc * CELL * 2);
        }
      }
      ++pc;
    }
    pstage = (pstage + 1 == DEPTH) ? 0 : pstage + 1;
  };
  const uint8_t *xsrc = p.xprep + PREP_HEADER;
  auto request_x = [&](uint32_t chunk) {  // this thread's share of activation chunk `chunk` (XCELLS cells from cell cs + chunk * XCELLS)
    const uint32_t c0 = cs + chunk * XCELLS;
    if (c0 >= ce) return;
    const uint32_t b0 = c0 * CELL, b1 = min(nb, min(ce, c0 + XCELLS) * CELL);
    const uint32_t pieces = (b1 - b0) * MT * 64;
    uint8_t *dst = xbuf + (chunk & 1) * XBUF;
    const uint8_t *src = xsrc + (size_t)b0 * MT * 1024;
    for (uint32_t q = tid; q < pieces; q += NT) cp_async16(dst + q * 16, src + (size_t)q * 16);
  };
  for (int s = 0; s + 1 < DEPTH; ++s) {  // the weights do not depend on the previous kernel
    request_weights();
    cp_async_commit();
  }
  pdl_launch_dependents();
  pdl_wait();  // the prepared activations come from the kernel in front
  request_x(0);
  cp_async_commit();

  float acc[MT][4];
#pragma unroll
  for (int G = 0; G < MT; ++G)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[G][j] = 0.f;

  uint32_t cstage = 0;
  for (uint32_t c = cs; c < ce; ++c) {
    if (c == cs)
      cp_async_wait(0);  // the first activation chunk is the newest group
    else
      cp_async_wait_c<DEPTH - 2>();
    const uint32_t rel = c - cs, chunk = rel / XCELLS;
    if (rel % XCELLS == 0) {
      __syncthreads();  // everybody's pieces of this chunk are in; everybody is done with the chunk before
      request_x(chunk + 1);
    } else {
      __syncwarp();
    }
    request_weights();
    cp_async_commit();
    const uint8_t *st = myring + cstage * STAGE;
    cstage = (cstage + 1 == DEPTH) ? 0 : cstage + 1;
    const uint8_t *xc = xbuf + (chunk & 1) * XBUF + (size_t)(rel % XCELLS) * CELL * MT * 1024 + lane * 16;
    const uint32_t nvalid = min((uint32_t)CELL, nb - c * CELL);
    const uint8_t *r0 = st + g * ROWB, *r1 = r0 + 8 * ROWB;
#pragma unroll
    for (uint32_t kb = 0; kb < (uint32_t)CELL; ++kb) {
      if (kb < nvalid) {
        uint32_t lo0[2], hi0[2], lo1[2], hi1[2];
        weight_frags<FMT>(r0 + kb * PB, t, lo0, hi0);
        weight_frags<FMT>(r1 + kb * PB, t, lo1, hi1);
        float d0 = 1.f, d1 = 1.f;
        if (F::SCALE_PIECES) {
          d0 = __half2float(*reinterpret_cast<const __half *>(r0 + CELL * PB + kb * 2));
          d1 = __half2float(*reinterpret_cast<const __half *>(r1 + CELL * PB + kb * 2));
        }
#pragma unroll
        for (int G = 0; G < MT; ++G) {
          const uint4 xh = *reinterpret_cast<const uint4 *>(xc + (size_t)(kb * MT + G) * 1024);
          const uint4 xl = *reinterpret_cast<const uint4 *>(xc + (size_t)(kb * MT + G) * 1024 + 512);
          float sh[4], sl[4];  // two short chains instead of one long one
          mma_f16_first(sh, lo0[0], lo1[0], lo0[1], lo1[1], xh.x, xh.y);
          mma_f16_first(sl, lo0[0], lo1[0], lo0[1], lo1[1], xl.x, xl.y);
          mma_f16(sh, hi0[0], hi1[0], hi0[1], hi1[1], xh.z, xh.w);
          mma_f16(sl, hi0[0], hi1[0], hi0[1], hi1[1], xl.z, xl.w);
          acc[G][0] = fmaf(sh[0] + sl[0], d0, acc[G][0]);
          acc[G][1] = fmaf(sh[1] + sl[1], d0, acc[G][1]);
          acc[G][2] = fmaf(sh[2] + sl[2], d1, acc[G][2]);
          acc[G][3] = fmaf(sh[3] + sl[3], d1, acc[G][3]);
        }
      }
    }
  }
  cp_async_wait(0);
  __syncthreads();  // the staging buffers are free: they now carry the finishing data

  float4 *pub = reinterpret_cast<float4 *>(xbuf);  // [NW tiles][MT][32 lanes]
  float2 *rope_cs = reinterpret_cast<float2 *>(ring);
#pragma unroll
  for (int G = 0; G < MT; ++G) {  // undo each activation row's scale (and apply 1 / rms)
    const float f0 = __ldcg(p.rowmul + 8 * G + 2 * t), f1 = __ldcg(p.rowmul + 8 * G + 2 * t + 1);
    pub[(warp * MT + G) * 32 + lane] = make_float4(acc[G][0] * f0, acc[G][1] * f1, acc[G][2] * f0, acc[G][3] * f1);
  }
  if (EPI == EPI_QKV && p.d_pos) fill_rope_rows(p, rope_cs, tid, NT);
  cluster.sync();
  if ((uint32_t)warp % kw == rank) {  // tile `warp` of this row group is finished by the CTA of rank warp % kw
    const uint32_t grp = blockIdx.y * NW + warp;
    if (grp < p.groups) {
#pragma unroll
      for (int G = 0; G < MT; ++G) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t j = 0; j < kw; ++j) {  // rank order: the result does not depend on which CTA finished first
          const float4 q = cluster.map_shared_rank(pub, j)[(warp * MT + G) * 32 + lane];
          v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
        }
        finish_fragment<EPI>(p, grp, g, 8 * G + 2 * t, v, rope_cs);
      }
    }
  }
  cluster.sync();  // a CTA's shared memory must outlive the other ranks' reads
}

template <int EPI>
uint32_t count_tiles(const GemvParams &p) {
  if (EPI == EPI_PLAIN || EPI == EPI_RESIDUAL) return (p.N + 15) / 16;
  if (EPI == EPI_SWIGLU) return (p.N + 7) / 8;
  return (p.H + p.Hkv) * ((p.Dh / 2) / 8) + (p.Hkv * p.Dh + 15) / 16;
}

uint32_t pick_k_slices(uint32_t row_groups, uint32_t K, uint32_t forced, uint32_t ctas_per_sm);

template <int FMT, int EPI, int MT, int TPW>
int launch_batch_cfg(cudaStream_t stream, GemvParams p) {
  using F = BFmt<FMT>;
  constexpr int ROWB = CELL * F::PB + 16, STAGE = TPW * 16 * ROWB, XB = F::XBLOCKS / MT, XFRAG = XB * MT * 1024;
  constexpr int ROWTAB = BW * TPW * 16 * (int)sizeof(RowSrc);
  constexpr int DEPTH_ROOM = (int)((BSMEM_LIMIT - XFRAG - ROWTAB) / (BW * STAGE));
  constexpr int DEPTH = DEPTH_ROOM > 6 ? 6 : DEPTH_ROOM;
  constexpr size_t SMEM = (size_t)XFRAG + ROWTAB + (size_t)BW * DEPTH * STAGE;
  auto kern = gemv_batch_kernel<FMT, EPI, MT, TPW>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    GRETA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    attr_set[dev] = true;
  }
  const uint32_t row_groups = (p.groups + BW * TPW - 1) / (BW * TPW);
  const uint32_t best_kw = pick_k_slices(row_groups, p.K, p.kw, 1);
  GRETA_REQUIRE(row_groups <= 65535, "batched gemv: %u row groups exceed the grid", row_groups);
  dim3 grid(best_kw, row_groups);
  GRETA_CUDA_TRY(launch_pdl_cluster(kern, grid, dim3(BTHREADS), best_kw, SMEM, stream, p));
  return launched("gemv_batch_kernel");
}

template <int FMT, int EPI, int MT>
int launch_batch_mt(cudaStream_t stream, GemvParams p) {
  p.groups = count_tiles<EPI>(p);
  // Two tiles per warp halve the number of CTAs that convert the same activations; one tile per warp when that
  // would leave SMs without a CTA.
  if (BFmt<FMT>::TPW_MAX >= 2 && (uint64_t)p.groups >= (uint64_t)2 * BW * sm_count())
    return launch_batch_cfg<FMT, EPI, MT, (BFmt<FMT>::TPW_MAX >= 2 ? 2 : 1)>(stream, p);
  return launch_batch_cfg<FMT, EPI, MT, 1>(stream, p);
}

uint32_t pick_k_slices(uint32_t row_groups, uint32_t K, uint32_t forced, uint32_t ctas_per_sm) {
  // K slices: the split that fills the CTA slots of the GPU best in whole waves, each slice at least 4 cells (1024 values) long.
  const uint32_t ncell = (K / 32 + CELL - 1) / CELL, sms = (uint32_t)sm_count() * ctas_per_sm;
  if (forced >= 1 && forced <= 8 && (forced & (forced - 1)) == 0 && forced <= ncell) return forced;
  uint32_t best_kw = 1;
  double best = -1.0;
  for (uint32_t kw = 1; kw <= 8; kw *= 2) {
    if (kw > 1 && ncell / kw < 4) break;
    const uint64_t ctas = (uint64_t)row_groups * kw, waves = (ctas + sms - 1) / sms;
    const double eff = (double)ctas / (double)(waves * sms) - 0.01 * kw;  // a small price for the extra reduction
    if (eff > best) {
      best = eff;
      best_kw = kw;
    }
  }
  return best_kw;
}

template <int FMT, int EPI, int MT>
int launch_batch_prepared(cudaStream_t stream, GemvParams p, void *workspace) {
  using P = PPlan<FMT, MT>;
  p.groups = count_tiles<EPI>(p);
  p.xprep = static_cast<const uint8_t *>(workspace);
  p.rowmul = static_cast<const float *>(workspace);
  auto prep = prep_rows_kernel<FMT, MT>;
  auto kern = gemv_batchp_kernel<FMT, EPI, MT>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    GRETA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P::SMEM));
    GRETA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
    GRETA_CUDA_TRY(cudaFuncSetAttribute(prep, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
    attr_set[dev] = true;
  }
  GRETA_CUDA_TRY(launch_pdl(prep, dim3(8 * MT), dim3(PREP_THREADS), 0, stream, static_cast<const float *>(p.x), p.gamma, p.eps, p.M, p.K,
                            static_cast<uint8_t *>(workspace)));
  if (int rc = launched("prep_rows_kernel")) return rc;
  const uint32_t row_groups = (p.groups + P::NW - 1) / P::NW;
  GRETA_REQUIRE(row_groups <= 65535, "batched gemv: %u row groups exceed the grid", row_groups);
  const uint32_t kw = pick_k_slices(row_groups, p.K, p.kw, P::CTAS);
  GRETA_CUDA_TRY(launch_pdl_cluster(kern, dim3(kw, row_groups), dim3(P::NW * 32), kw, P::SMEM, stream, p));
  return launched("gemv_batchp_kernel");
}

// With workspace the activations are prepared once by a kernel of their own; without it every CTA converts them itself.
template <int FMT, int EPI>
int launch_batch(cudaStream_t stream, const GemvParams &p, void *workspace = nullptr) {
  if (workspace) {
    if (p.M <= 8) return launch_batch_prepared<FMT, EPI, 1>(stream, p, workspace);
    if (p.M <= 16) return launch_batch_prepared<FMT, EPI, 2>(stream, p, workspace);
    return launch_batch_prepared<FMT, EPI, 4>(stream, p, workspace);
  }
  if (p.M <= 8) return launch_batch_mt<FMT, EPI, 1>(stream, p);
  if (p.M <= 16) return launch_batch_mt<FMT, EPI, 2>(stream, p);
  return launch_batch_mt<FMT, EPI, 4>(stream, p);
}

template <int EPI>
int dispatch_batch(cudaStream_t stream, int fmt, const GemvParams &p, void *workspace = nullptr) {
  GRETA_REQUIRE(!workspace || aligned16(workspace), "batched gemv: the workspace must be 16-byte aligned");
  switch (fmt) {
    case GRETA_FMT_Q4_0: return launch_batch<GRETA_FMT_Q4_0, EPI>(stream, p, workspace);
    case GRETA_FMT_Q8_0: return launch_batch<GRETA_FMT_Q8_0, EPI>(stream, p, workspace);
    case GRETA_FMT_F16: return launch_batch<GRETA_FMT_F16, EPI>(stream, p, workspace);
    default: break;
  }
  set_error("batched gemv: format %d is not supported (Q4_0, Q8_0 or F16)", fmt);
  return GRETA_ERR_INVALID_ARGS;
}

int check_batch_plane(const char *what, const void *qs, const void *d, int fmt) {
  GRETA_REQUIRE(qs != nullptr && aligned16(qs), "%s: weight plane is null or not 16-byte aligned", what);
  GRETA_REQUIRE(fmt == GRETA_FMT_F16 || (d != nullptr && aligned16(d)), "%s: scale plane is null or not 16-byte aligned", what);
  return GRETA_OK;
}

int check_batch_common(const char *what, uint32_t M, uint32_t K, const void *x) {
  GRETA_REQUIRE(M >= 1 && M <= 32, "%s: M=%u outside 1..32", what, M);
  GRETA_REQUIRE(K % 32 == 0 && K > 0, "%s: K=%u is not a positive multiple of the block size 32", what, K);
  GRETA_REQUIRE(x && aligned16(x), "%s: activation pointer is null or not 16-byte aligned", what);
  return GRETA_OK;
}

}  // namespace

namespace greta {
// Used by greta_cuda_gemv for 2 <= M <= 32 rows of fp32 activations (GGUF formats and fp16 weights).
int gemv_batch_plain(cudaStream_t stream, int fmt, const float *x, const void *qs, const void *d, float *y, uint32_t M, uint32_t N, uint32_t K,
                     uint32_t force_kw) {
  GemvParams p{};
  p.x = x;
  p.w[0] = {(const uint8_t *)qs, d};
  p.K = K;
  p.N = N;
  p.M = M;
  p.y = y;
  p.kw = force_kw;
  return dispatch_batch<EPI_PLAIN>(stream, fmt, p);
}
}  // namespace greta

extern "C" {

size_t greta_cuda_gemv_batch_workspace_bytes(uint32_t M, uint32_t K) {
  const size_t mt = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  return PREP_HEADER + (size_t)(K / 32) * mt * 1024;
}

int greta_cuda_gemv_batch(greta_stream_t stream, int fmt, const float *x, const float *gamma, float eps, const void *qs, const void *d,
                          const float *resid, float *y, uint32_t M, uint32_t N, uint32_t K, uint32_t k_slices, void *workspace) {
  if (N == 0) return GRETA_OK;
  if (int rc = check_batch_common("gemv_batch", M, K, x)) return rc;
  if (int rc = check_batch_plane("gemv_batch", qs, d, fmt)) return rc;
  GRETA_REQUIRE(y, "gemv_batch: null output pointer");
  GemvParams p{};
  p.x = x;
  p.gamma = gamma;
  p.eps = eps;
  p.w[0] = {(const uint8_t *)qs, d};
  p.K = K;
  p.N = N;
  p.M = M;
  p.y = y;
  p.resid = resid;
  p.kw = k_slices;
  return resid ? dispatch_batch<EPI_RESIDUAL>((cudaStream_t)stream, fmt, p, workspace) : dispatch_batch<EPI_PLAIN>((cudaStream_t)stream, fmt, p, workspace);
}

int greta_cuda_fused_rmsnorm_qkv_rope_kv_batch(greta_stream_t stream, int fmt, const float *x, const float *gamma, float eps, const void *wq_qs,
                                               const void *wq_d, const void *wk_qs, const void *wk_d, const void *wv_qs, const void *wv_d,
                                               float *q_out, float *k_out, float *v_out, void *k_cache, void *v_cache, const uint32_t *d_pos,
                                               uint32_t M, uint32_t H, uint32_t Hkv, uint32_t Dh, uint32_t max_seq, float rope_base, uint32_t D,
                                               void *workspace) {
  if (int rc = check_batch_common("fused_qkv_batch", M, D, x)) return rc;
  GRETA_REQUIRE(H && Hkv && H % Hkv == 0 && (Dh == 64 || Dh == 128), "fused_qkv_batch: heads %u / %u of dim %u (64 or 128)", H, Hkv, Dh);
  GRETA_REQUIRE(q_out, "fused_qkv_batch: null q_out");
  GRETA_REQUIRE(d_pos ? (k_cache && v_cache) : (k_out && v_out), "fused_qkv_batch: with d_pos the caches are required, without it k_out and v_out");
  if (int rc = check_batch_plane("fused_qkv_batch(wq)", wq_qs, wq_d, fmt)) return rc;
  if (int rc = check_batch_plane("fused_qkv_batch(wk)", wk_qs, wk_d, fmt)) return rc;
  if (int rc = check_batch_plane("fused_qkv_batch(wv)", wv_qs, wv_d, fmt)) return rc;
  GemvParams p{};
  p.x = x;
  p.gamma = gamma;
  p.eps = eps;
  p.w[0] = {(const uint8_t *)wq_qs, wq_d};
  p.w[1] = {(const uint8_t *)wk_qs, wk_d};
  p.w[2] = {(const uint8_t *)wv_qs, wv_d};
  p.K = D;
  p.M = M;
  p.q_out = q_out;
  p.k_out = k_out;
  p.v_out = v_out;
  p.k_cache = (__half *)k_cache;
  p.v_cache = (__half *)v_cache;
  p.d_pos = d_pos;
  p.H = H;
  p.Hkv = Hkv;
  p.Dh = Dh;
  p.max_seq = max_seq;
  p.rope_base = rope_base;
  return dispatch_batch<EPI_QKV>((cudaStream_t)stream, fmt, p, workspace);
}

int greta_cuda_fused_ffn_front_batch(greta_stream_t stream, int fmt, const float *x, const float *gamma, float eps, const void *w1_qs,
                                     const void *w1_d, const void *w3_qs, const void *w3_d, float *y, uint32_t M, uint32_t D, uint32_t F,
                                     void *workspace) {
  if (F == 0) return GRETA_OK;
  if (int rc = check_batch_common("fused_ffn_front_batch", M, D, x)) return rc;
  GRETA_REQUIRE(y, "fused_ffn_front_batch: null output pointer");
  if (int rc = check_batch_plane("fused_ffn_front_batch(w1)", w1_qs, w1_d, fmt)) return rc;
  if (int rc = check_batch_plane("fused_ffn_front_batch(w3)", w3_qs, w3_d, fmt)) return rc;
  GemvParams p{};
  p.x = x;
  p.gamma = gamma;
  p.eps = eps;
  p.w[0] = {(const uint8_t *)w1_qs, w1_d};
  p.w[1] = {(const uint8_t *)w3_qs, w3_d};
  p.K = D;
  p.N = F;
  p.M = M;
  p.y = y;
  return dispatch_batch<EPI_SWIGLU>((cudaStream_t)stream, fmt, p, workspace);
}

}  // extern "C"
