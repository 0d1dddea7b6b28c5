// Decode GEMV over block-quantised weights, with the RMSNorm prologue and the
// RoPE / KV-cache / SwiGLU / residual epilogues of the per-layer decode path.
//
// The work is HBM-bound (0.5625 B per weight for Q4_0): the kernel is shaped
// around memory traffic and around the issue budget of the SIMT pipes, not around
// tensor cores.
//
//   * Persistent CTAs, one per SM, 16 warps.  A CTA owns a contiguous range of
//     row groups; its (row group, 32-block chunk of K) cells are split evenly
//     over the warps, so the load is balanced to within one cell per warp.
//   * Weights travel global -> shared with 16-byte cp.async copies, one payload
//     per lane, into a per-warp ring several cells deep (the ring, not the
//     register file, holds the bytes in flight: ~100 KB per SM).  One warp-wide
//     copy instruction covers 512 contiguous bytes of a row.  The first cells
//     are requested before the activations are touched.
//   * The activation vector is staged once per CTA (after the optional RMSNorm).
//     For the integer formats it is turned into block fixed point: per block of
//     32 a power-of-two scale and 23-bit integers, stored as three planes of
//     signed bytes.  A block of weights then needs only masks to unpack nibbles
//     to bytes and 4-way integer dot products (dp4a) against the three planes;
//     every product is exact, the three partial sums are recombined in fp32 and
//     scaled by (block scale of x) * (fp16 block scale of W).  Rounding x to
//     22 fraction bits relative to its block maximum is the only approximation -
//     the order of an fp32 rounding of the largest term.  This costs ~1.5 issue
//     slots per weight where unpack-to-float needs ~2.5 and is conversion bound.
//   * Lanes accumulate in fp32 across the cells of a row group; a butterfly
//     shuffle reduction runs once per group and warp; partial sums of a group
//     that spans warps meet in shared memory in a fixed order (deterministic).
//   * A warp executes only a few thousand instructions per launch, about as many
//     as the kernel has: code that runs once (staging, epilogue, set-up) is kept
//     compact, and the ring depth is a template parameter (5 or 3 stages) so
//     that waits and wrap-arounds are constants.
//   * Launches are chained by programmatic dependent launch: the ring is filled
//     before the kernel waits for its predecessor, everything that reads the
//     predecessor's output comes after the wait.
//   * Tensor parallelism: the row-parallel projections (EPI_PEER) store their
//     partial products, tagged, straight into every rank's slot buffer over
//     NVLink, and the consuming kernel (PEER staging) adds the partials to the
//     residual stream while it stages its input - no collective in between.
//
// fp16 weights (the LM head) use the same pipeline with fp32 activations and
// packed fp32 FMAs.  A simpler kernel (direct loads, float math) remains for K so
// large that the staged activations leave no room for the ring.
#include <math.h>
#include <algorithm>
#include <cstdlib>

#include "gemv_device.cuh"

namespace greta {
int gemv_batch_plain(cudaStream_t stream, int fmt, const float *x, const void *qs, const void *d, float *y, uint32_t M, uint32_t N, uint32_t K,
                     uint32_t force_kw);  // gemv_batch.cu
}

namespace {

// ------------------------------------------------------------------ simple kernel (any K % 32 == 0)
// Direct register loads, two stages, float math; a warp owns one row group over
// the whole K (optionally a 1/kw part of it).
template <int FMT, int EPI, int R>
__global__ void __launch_bounds__(THREADS, 1) gemv_simple_kernel(const GemvParams p) {
  constexpr int QV = Fmt<FMT>::QV;
  constexpr int PB = QV * 16;
  extern __shared__ __align__(16) float xs[];
  __shared__ float red[32];
  __shared__ float part[WARPS][R];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t nb = p.K / 32;
  const uint32_t gw_total = gridDim.x * WARPS;
  const uint32_t gw = blockIdx.x * WARPS + warp;
  const uint32_t bps = (nb + p.kw - 1) / p.kw;
  const uint32_t m = blockIdx.y;

  const uint8_t *qrow[R];
  const void *drow[R];
  size_t dbase[R];
  uint32_t grp = 0, kp = 0, b = 0, bend = 0;
  bool active = false;
  uint4 qa[R][QV], qb[R][QV];
  float da[R], db[R];

  auto setup = [&](uint32_t it) {
    uint32_t t = it * gw_total + gw;
    grp = t / p.kw;
    kp = t % p.kw;
    active = grp < p.groups;
    if (!active) return;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      int mat;
      uint32_t row;
      if (!resolve<EPI, R>(p, grp, r, &mat, &row)) {  // ragged tail: compute on row 0, never stored
        mat = 0;
        row = 0;
      }
      qrow[r] = p.w[mat].qs + (size_t)row * nb * PB;
      drow[r] = p.w[mat].d;
      dbase[r] = (size_t)row * (Fmt<FMT>::SCALE_BYTES == 2 ? d_row_stride(nb) : nb);
    }
    b = kp * bps + lane;
    bend = min(nb, (kp + 1) * bps);
  };
  auto load = [&](uint4(&q)[R][QV], float(&dd)[R], uint32_t blk) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int v = 0; v < QV; ++v) q[r][v] = ld_stream(qrow[r] + (size_t)blk * PB + v * 16);
      dd[r] = load_scale<FMT>(drow[r], dbase[r] + blk);
    }
  };

  setup(0);
  if (active && b < bend) load(qa, da, b);

  {
    const uint32_t K = p.K;
    const float *xf = p.x_is_f16 ? nullptr : reinterpret_cast<const float *>(p.x) + (size_t)m * K;
    const __half *xh = p.x_is_f16 ? reinterpret_cast<const __half *>(p.x) + (size_t)m * K : nullptr;
    float inv = p.gamma ? cta_inv_rms(xf, xh, K, p.eps, red) : 1.0f;
    for (uint32_t k = threadIdx.x; k < K; k += THREADS) {
      float v = xf ? __ldcg(xf + k) : __half2float(__ldcg(xh + k));
      if (p.gamma) v = (v * inv) * p.gamma[k];
      xs[(k >> 5) * XPAD + xs_slot<FMT>(k & 31)] = v;
    }
  }
  __syncthreads();

  const uint32_t pos = (EPI == EPI_QKV && p.d_pos) ? *p.d_pos : 0u;

  for (uint32_t it = 0; it < p.iters; ++it) {
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    auto compute = [&](uint4(&q)[R][QV], float(&dd)[R], uint32_t blk) {
      float4 xv[8];
      const float4 *xp = reinterpret_cast<const float4 *>(xs + (size_t)blk * XPAD);
#pragma unroll
      for (int i = 0; i < 8; ++i) xv[i] = xp[i];
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = fmaf(dd[r], block_dot_f<FMT>(q[r], xv), acc[r]);
    };
    if (active && b < bend) {
      while (true) {
        bool hb = b + 32 < bend;
        if (hb) load(qb, db, b + 32);
        compute(qa, da, b);
        if (!hb) break;
        bool ha = b + 64 < bend;
        if (ha) load(qa, da, b + 64);
        compute(qb, db, b + 32);
        if (!ha) break;
        b += 64;
      }
    }
    const bool cur_active = active;
    const uint32_t cur_grp = grp, cur_kp = kp;
    if (it + 1 < p.iters) {
      setup(it + 1);
      if (active && b < bend) load(qa, da, b);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
    if (p.kw > 1) {
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) part[warp][r] = cur_active ? acc[r] : 0.f;
      }
      __syncthreads();
      if (cur_kp == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float t = 0.f;
          for (uint32_t j = 0; j < p.kw; ++j) t += part[warp + j][r];
          acc[r] = t;
        }
      }
      __syncthreads();
    }
    if (cur_active && cur_kp == 0 && lane == 0) epilogue<EPI, R>(p, cur_grp, m, pos, acc);
  }
}

// DT: ring depth fixed at compile time (waits and stage wrap-arounds fold to constants), 0 = taken from p.stages.
// PEER: the activations are the residual stream plus the tensor-parallel partials waiting in this rank's slots.
template <int FMT, int EPI, int R, int DT, bool PEER>
__global__ void __launch_bounds__(THREADS, 1) gemv_pipe_kernel(const GemvParams p) {
  using F = Fmt<FMT>;
  constexpr int QV = F::QV, PB = QV * 16;
  constexpr int SCALE_ROW = 32 * F::SCALE_BYTES;                 // bytes of scales per row per cell
  constexpr int STAGE_BYTES = R * (32 * PB + SCALE_ROW);
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float red[32];
  __shared__ float2 rope_cs[64];                                  // head_dim <= 128

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t nb = p.K / 32, C = (nb + 31) / 32;               // chunks (cells) per row group
  const uint32_t m = blockIdx.y;
  const uint32_t D = DT ? (uint32_t)DT : p.stages;
  const size_t xs_bytes = F::INTEGER ? (size_t)nb * XQ_WORDS * 4 : (size_t)nb * XPAD * 4;
  uint8_t *ring = smem + ((xs_bytes + 15) & ~(size_t)15) + (size_t)warp * D * STAGE_BYTES;
  float *part = reinterpret_cast<float *>(smem + ((xs_bytes + 15) & ~(size_t)15) + (size_t)WARPS * D * STAGE_BYTES);
  // part[warp][slot][R]

  // This CTA's row groups and this warp's cells.
  const uint32_t g0 = blockIdx.x * p.gq + min(blockIdx.x, p.gr);
  const uint32_t g1 = g0 + p.gq + (blockIdx.x < p.gr ? 1u : 0u);
  const uint32_t T = (g1 - g0) * C;
  const uint32_t c0 = (uint32_t)((uint64_t)warp * T / WARPS), c1 = (uint32_t)((uint64_t)(warp + 1) * T / WARPS);

  // ---- producer state: next cell to request.  Source pointers run along the rows (one add per cell). ----
  uint32_t pc = c0, pg = g0 + (c0 / C), pk = c0 % C, pstage = 0;
  const uint8_t *qsrc[R];       // this lane's payload of the next cell, per row
  const uint8_t *dsrc4[R];      // fp32-scale formats: this lane's scale, per row
  const uint8_t *dsrc = nullptr;  // fp16-scale formats: lanes < 4R copy 8 scales each: (row lane/4, segment lane%4)
  const uint32_t dst_q = (uint32_t)lane * PB;
  const uint32_t dst_d = R * 32 * PB + (F::SCALE_BYTES == 2 ? (uint32_t)(lane >> 2) * SCALE_ROW + (uint32_t)(lane & 3) * 16 : (uint32_t)lane * 4);
  auto producer_rows = [&]() {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      int mat;
      uint32_t row;
      if (!resolve<EPI, R>(p, pg, r, &mat, &row)) {  // ragged tail: stream row 0, result never stored
        mat = 0;
        row = 0;
      }
      qsrc[r] = p.w[mat].qs + ((size_t)row * nb + pk * 32 + lane) * PB;
      const uint8_t *dbase = reinterpret_cast<const uint8_t *>(p.w[mat].d);
      if (F::SCALE_BYTES == 2) {
        if ((lane >> 2) == r) dsrc = dbase + ((size_t)row * d_row_stride(nb) + pk * 32 + (lane & 3) * 8) * 2;
      } else if (F::SCALE_BYTES == 4) {
        dsrc4[r] = dbase + ((size_t)row * nb + pk * 32 + lane) * 4;
      }
    }
  };
  if (pc < c1) producer_rows();
  auto request = [&]() {  // requests cell pc into stage pstage, advances the producer
    if (pc < c1) {
      uint8_t *st = ring + pstage * STAGE_BYTES;
      if (pk * 32 + lane < nb) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
          for (int v = 0; v < QV; ++v) cp_async16(st + r * 32 * PB + dst_q + v * 16, qsrc[r] + v * 16);
          if (F::SCALE_BYTES == 4) cp_async4(st + dst_d + r * SCALE_ROW, dsrc4[r]);
        }
      }
      if (F::SCALE_BYTES == 2 && lane < 4 * R && pk * 32 + (lane & 3) * 8 < nb) cp_async16(st + dst_d, dsrc);
      ++pc;
      if (++pk == C) {
        pk = 0;
        ++pg;
        if (pc < c1) producer_rows();
      } else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          qsrc[r] += 32 * PB;
          if (F::SCALE_BYTES == 4) dsrc4[r] += 128;
        }
        if (F::SCALE_BYTES == 2) dsrc += 64;
      }
    }
    cp_async_commit();
    pstage = (pstage + 1 == D) ? 0 : pstage + 1;
  };

  // Request the first cells before touching the activations: weights do not
  // depend on the previous kernel's output.
  for (uint32_t s = 0; s + 1 < D; ++s) request();
  pdl_launch_dependents();  // the next kernel may begin its own weight prefetch as SMs free up
  pdl_wait();               // everything below reads what the previous kernel wrote

  // ---- stage activations ----
  if (F::INTEGER) {
    stage_fixed_point<FMT, PEER>(p, m, reinterpret_cast<uint32_t *>(smem), red);
  } else {
    float *xs = reinterpret_cast<float *>(smem);
    const uint32_t K = p.K;
    const float *xf = p.x_is_f16 ? nullptr : reinterpret_cast<const float *>(p.x) + (size_t)m * K;
    const __half *xh = p.x_is_f16 ? reinterpret_cast<const __half *>(p.x) + (size_t)m * K : nullptr;
    float inv = p.gamma ? cta_inv_rms(xf, xh, K, p.eps, red) : 1.0f;
    for (uint32_t k = threadIdx.x; k < K; k += THREADS) {
      float v = xf ? __ldcg(xf + k) : __half2float(__ldcg(xh + k));
      if (p.gamma) v = (v * inv) * p.gamma[k];
      xs[(k >> 5) * XPAD + (k & 31)] = v;
    }
  }
  if (EPI == EPI_QKV && p.d_pos) fill_rope_table(p, __ldcg(p.d_pos), rope_cs);
  __syncthreads();

  // ---- consume ----
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  const uint32_t first_grp = g0 + c0 / C;
  uint32_t cg = first_grp, ck = c0 % C, cstage = 0;
  constexpr uint32_t X_BLOCK_BYTES = F::INTEGER ? XQ_WORDS * 4 : XPAD * 4;
  const uint8_t *xrun = smem + (size_t)(ck * 32 + lane) * X_BLOCK_BYTES;  // this lane's activation block, runs along K
  for (uint32_t c = c0; c < c1; ++c) {
    if (DT)
      cp_async_wait_c<(DT ? DT : 2) - 2>();
    else
      cp_async_wait((int)D - 2);
    __syncwarp();
    const uint8_t *st = ring + cstage * STAGE_BYTES;
    cstage = (cstage + 1 == D) ? 0 : cstage + 1;
    const bool live = ck * 32 + lane < nb;
    uint4 q[R][QV];
    float dsc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int v = 0; v < QV; ++v) q[r][v] = *reinterpret_cast<const uint4 *>(st + r * 32 * PB + dst_q + v * 16);
      if (F::SCALE_BYTES == 2)
        dsc[r] = __half2float(*reinterpret_cast<const __half *>(st + R * 32 * PB + r * SCALE_ROW + lane * 2));
      else if (F::SCALE_BYTES == 4)
        dsc[r] = *reinterpret_cast<const float *>(st + R * 32 * PB + r * SCALE_ROW + lane * 4);
      else
        dsc[r] = 1.0f;
    }
    __syncwarp();  // every lane has read its stage (scales are shared between lanes)
    request();     // refill the stage consumed in the previous iteration
    if (live) {
      if (F::INTEGER) {
        uint4 xp[7];
        const uint4 *xb = reinterpret_cast<const uint4 *>(xrun);
#pragma unroll
        for (int i = 0; i < 7; ++i) xp[i] = xb[i];
        const float xsc = __uint_as_float(xp[6].w);
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = fmaf(dsc[r] * xsc, block_dot_i<FMT>(q[r], xp), acc[r]);
      } else {
        float4 xv[8];
        const float4 *xb = reinterpret_cast<const float4 *>(xrun);
#pragma unroll
        for (int i = 0; i < 8; ++i) xv[i] = xb[i];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] += block_dot_f<FMT>(q[r], xv);
      }
    }
    xrun += 32 * X_BLOCK_BYTES;
    if (++ck == C || c + 1 == c1) {  // group finished for this warp: reduce and publish
      const float total = warp_sum_rows<R>(acc, lane);  // lanes 0, 8, 16, 24 end up with rows 0..R-1 between them
      if ((lane & (R == 4 ? 7 : (R == 2 ? 15 : 31))) == 0)
        part[((size_t)warp * p.slots + (cg - first_grp)) * R + warp_sum_rows_index<R>(lane)] = total;
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = 0.f;
      if (ck == C) {
        ck = 0;
        ++cg;
        xrun = smem + (size_t)lane * X_BLOCK_BYTES;
      }
    }
  }
  cp_async_wait(0);
  __syncthreads();

  // ---- epilogue: one warp per row group ----
  const uint32_t pos = (EPI == EPI_QKV && p.d_pos) ? __ldcg(p.d_pos) : (EPI == EPI_PEER ? peer_tag(p) : 0u);
  cta_epilogue<EPI, R>(p, part, p.slots, g0, g1, C, T, m, pos, (EPI == EPI_QKV && p.d_pos) ? rope_cs : nullptr);
}

// ------------------------------------------------------------------ host side
// Opt-in to large dynamic shared memory, once per kernel and device.  `attr_set`
// must be a flag array owned by the caller's template instantiation: every
// kernel here has the same function type, so a static inside this helper would
// be shared by all of them.
template <typename Kern>
int ensure_smem_attr(Kern kern, bool (&attr_set)[64]) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    GRETA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT));
    // every kernel of the decode chain asks for the same (largest) shared-memory carve-out: an SM need not be
    // reconfigured, and so drained, between two of them
    GRETA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
    attr_set[dev] = true;
  }
  return GRETA_OK;
}

template <int FMT, int EPI, int R>
int launch_simple(cudaStream_t stream, GemvParams p) {
  const uint32_t nb = p.K / 32;
  const size_t smem = (size_t)nb * XPAD * sizeof(float);
  GRETA_REQUIRE(smem <= SMEM_LIMIT, "gemv: K=%u needs %zu bytes of shared memory (max %zu)", p.K, smem, SMEM_LIMIT);
  static bool attr_set[64] = {};
  if (int rc = ensure_smem_attr(gemv_simple_kernel<FMT, EPI, R>, attr_set)) return rc;
  const uint32_t sms = (uint32_t)sm_count();
  uint32_t kw = 1;
  while (kw < (uint32_t)WARPS && (uint64_t)p.groups * kw * 2 <= (uint64_t)sms * WARPS && nb / (kw * 2) >= 32) kw *= 2;
  p.kw = kw;
  const uint64_t tasks = (uint64_t)p.groups * kw;
  uint32_t ctas = (uint32_t)std::min<uint64_t>(sms, (tasks + WARPS - 1) / WARPS);
  if (ctas == 0) ctas = 1;
  p.iters = (uint32_t)((tasks + (uint64_t)ctas * WARPS - 1) / ((uint64_t)ctas * WARPS));
  dim3 grid(ctas, p.M ? p.M : 1);
  gemv_simple_kernel<FMT, EPI, R><<<grid, THREADS, smem, stream>>>(p);
  return launched("gemv_simple_kernel");
}

template <int FMT, int EPI, int R, bool PEER, int DFIX>
int launch_pipe_fixed(cudaStream_t stream, GemvParams p, dim3 grid, size_t xs_bytes, size_t stage_bytes, size_t part_bytes) {
  p.stages = DFIX;
  const size_t smem = xs_bytes + (size_t)WARPS * DFIX * stage_bytes + part_bytes;
  static bool attr_set[64] = {};
  if (int rc = ensure_smem_attr(gemv_pipe_kernel<FMT, EPI, R, DFIX, PEER>, attr_set)) return rc;
  GRETA_CUDA_TRY(launch_pdl(gemv_pipe_kernel<FMT, EPI, R, DFIX, PEER>, grid, dim3(THREADS), smem, stream, p));
  return launched("gemv_pipe_kernel");
}

template <int FMT, int EPI, int R, bool PEER = false>
int launch_pipe(cudaStream_t stream, GemvParams p) {
  using F = Fmt<FMT>;
  const uint32_t nb = p.K / 32, C = (nb + 31) / 32;
  const size_t stage_bytes = (size_t)R * (32 * F::QV * 16 + 32 * F::SCALE_BYTES);
  const size_t xs_bytes = ((F::INTEGER ? (size_t)nb * XQ_WORDS * 4 : (size_t)nb * XPAD * 4) + 15) & ~(size_t)15;
  const uint32_t sms = (uint32_t)sm_count();
  const uint32_t ctas = std::max(1u, std::min(sms, p.groups));
  const uint32_t gmax = (p.groups + ctas - 1) / ctas;                        // row groups per CTA (max)
  const uint32_t cells_per_warp = (uint32_t)(((uint64_t)gmax * C + WARPS - 1) / WARPS);
  p.slots = cells_per_warp / C + 2;                                          // groups one warp can touch
  const size_t part_bytes = (size_t)WARPS * p.slots * R * sizeof(float);
  if (xs_bytes + part_bytes + 2 * WARPS * stage_bytes > SMEM_LIMIT) {
    GRETA_REQUIRE(!PEER && EPI != EPI_PEER, "gemv: K=%u is too large for the tensor-parallel exchange form", p.K);
    return launch_simple<FMT, EPI == EPI_PEER ? EPI_PLAIN : EPI, R>(stream, p);
  }
  uint32_t stages = (uint32_t)((SMEM_LIMIT - xs_bytes - part_bytes) / (WARPS * stage_bytes));
  stages = std::min<uint32_t>(stages, MAX_STAGES);
  stages = std::min<uint32_t>(stages, std::max(2u, cells_per_warp + 1));     // no deeper than the work
  p.gq = p.groups / ctas;
  p.gr = p.groups % ctas;
  dim3 grid(ctas, p.M ? p.M : 1);
  // Deeper than the work is harmless: requests past the last cell are empty groups.  (Measured in the decode
  // step: 8 stages for the 2-row cells are 7 % slower than 5.)
  const size_t room = (SMEM_LIMIT - xs_bytes - part_bytes) / (WARPS * stage_bytes);
  // Ring depth, fixed at compile time: 5 stages, or 3 where the smaller footprint pays more than the deeper prefetch:
  // kernels with 4-row cells (a 5-stage ring of those fills the SM, with 3 stages the next kernel's CTA fits beside it
  // and starts its own weight prefetch early) and the residual projections (O, down; their scattering form under tensor
  // parallelism too) with 2-row cells.  Measured in the 7B-shape decode step: 632 -> 638 -> 645 tok/s (766 against 761 on
  // two GPUs); the fused QKV operator loses 5 % with 3 stages and keeps 5.
  const int want = tuning().gemv_ring_stages;  // 0 = the rule above, 3 or 5 = forced
  const bool shallow = want == 3 || (want != 5 && (R == 4 || EPI == EPI_RESIDUAL || EPI == EPI_PEER));
  if (F::INTEGER && room >= 5 && !shallow) return launch_pipe_fixed<FMT, EPI, R, PEER, F::INTEGER ? 5 : 0>(stream, p, grid, xs_bytes, stage_bytes, part_bytes);
  if (F::INTEGER && room >= 3) return launch_pipe_fixed<FMT, EPI, R, PEER, F::INTEGER ? 3 : 0>(stream, p, grid, xs_bytes, stage_bytes, part_bytes);
  p.stages = stages;
  const size_t smem = xs_bytes + (size_t)WARPS * stages * stage_bytes + part_bytes;
  static bool attr_set[64] = {};
  if (int rc = ensure_smem_attr(gemv_pipe_kernel<FMT, EPI, R, 0, PEER>, attr_set)) return rc;
  GRETA_CUDA_TRY(launch_pdl(gemv_pipe_kernel<FMT, EPI, R, 0, PEER>, grid, dim3(THREADS), smem, stream, p));
  return launched("gemv_pipe_kernel");
}

// Row groups of R rows for an operator with `rows` output rows per matrix.
template <int EPI, int R>
uint32_t count_groups(const GemvParams &p) {
  if (EPI == EPI_PLAIN || EPI == EPI_RESIDUAL || EPI == EPI_PEER) return (p.N + R - 1) / R;
  if (EPI == EPI_SWIGLU) return (p.N + R / 2 - 1) / (R / 2);
  return (p.H + p.Hkv) * ((p.Dh / 2) / (R / 2)) + (p.Hkv * p.Dh + R - 1) / R;
}

template <int FMT, int EPI, int R, bool PEER = false>
int launch_any(cudaStream_t stream, GemvParams p) {
  p.groups = count_groups<EPI, R>(p);
  return launch_pipe<FMT, EPI, R, PEER>(stream, p);  // falls back to the simple kernel when K does not fit in shared memory
}

// Groups of 2 rows give twice as many cells to balance over the warps: measured faster in the decode step up to
// about ten 4-row cells per warp; above that the 4-row cell's lower overhead wins.  The fused gate/up operator
// switches earlier, at four: at the 7B shape (22016 rows x 4096) 4-row cells take 12.6 us against 13.4 and the
// decode step gains 1.6 %; its half on two GPUs (11008 rows) gains 2 % (783 against 767 tok/s), its quarter on four
// gains nothing.  The residual projections (O, down) take them from one cell per warp: with the 3-stage ring of
// launch_pipe 654 -> 657 tok/s for the O projection (4096 x 4096) and 645 -> 654 for the down projection; the plain
// GEMV likewise (alone: 11008 x 4096 7.3 against 8.4 us, 22016 x 4096 11.5 against 12.7, 8192 x 8192 9.7 against 10.8).
// The fused QKV operator of the same model loses 7 % with them.
template <int FMT, int EPI, bool PEER = false>
int launch_quant(cudaStream_t stream, const GemvParams &p, uint64_t total_rows) {
  const uint64_t cells4 = (total_rows / 4) * ((p.K / 32 + 31) / 32);
  if (EPI == EPI_QKV && (p.Dh / 2) % 2 != 0) return launch_any<FMT, EPI, 2, PEER>(stream, p);
  const uint64_t r2_cells = tuning().gemv_r2_cells >= 0 ? (uint64_t)tuning().gemv_r2_cells : (uint64_t)sm_count() * WARPS * (EPI == EPI_SWIGLU ? 4 : ((EPI == EPI_RESIDUAL || EPI == EPI_PLAIN) ? 1 : 10));
  if (cells4 < r2_cells) return launch_any<FMT, EPI, 2, PEER>(stream, p);
  return launch_any<FMT, EPI, 4, PEER>(stream, p);
}

// The operators of the tensor-parallel exchange exist for the GGUF formats only.
template <int EPI, bool PEER>
int dispatch_peer(cudaStream_t stream, int fmt, const GemvParams &p, uint64_t total_rows) {
  if (fmt == GRETA_FMT_Q4_0) return launch_quant<GRETA_FMT_Q4_0, EPI, PEER>(stream, p, total_rows);
  if (fmt == GRETA_FMT_Q8_0) return launch_quant<GRETA_FMT_Q8_0, EPI, PEER>(stream, p, total_rows);
  set_error("tensor-parallel exchange: format %d is not supported (Q4_0 or Q8_0)", fmt);
  return GRETA_ERR_INVALID_ARGS;
}

// ---- all-reduce over peer memory (a batch of sequences) ---------------------------------------------
// In-place sum over the ranks of `count` floats, as one kernel per rank and no collective launch.  Three phases
// over {value, tag} words in the ranks' slot buffers (the tag travels with the value: no flag, no fence):
//   A  every rank stores slice j of its vector into region A of rank j's buffer (row `rank` of [tp][count / tp]);
//   B  every rank sums the tp rows of its own slice in rank order (bounded waits on the tags) and stores the sums
//      into region B ([count]) of every rank's buffer: all ranks receive the same bits;
//   C  every rank waits for the count words of its region B and writes the values back to x.
// Two sets of regions alternate with the parity of exch_idx, which is enough: a rank can be at most one all-reduce
// ahead of another, because it cannot finish one without every rank's contribution to it.  The tag is
// ((*d_pos + 1) << 8) | exch_idx, read on the device, so a captured decode step replays with fresh tags.
struct PeerArParams {
  float *x;
  uint32_t count, tp, rank, exch_idx;
  const uint32_t *d_pos;
  uint2 *slots[MAX_TP];
  unsigned poll_limit;
};

__device__ __forceinline__ uint2 wait_tagged(const uint2 *src, uint32_t tag, uint32_t budget) {
  uint2 w = ld_peer8(src);
  uint32_t polls = 0;
  while (w.y != tag) {
    if (++polls > budget || ((polls & 255u) == 0 && peer_failed())) {
      g_peer_error = 1;
      break;
    }
    w = ld_peer8(src);
  }
  return w;
}

__global__ void __launch_bounds__(256) peer_allreduce_kernel(const PeerArParams p) {
  pdl_launch_dependents();
  pdl_wait();  // x comes from the kernel in front
  const uint32_t tag = ((__ldcg(p.d_pos) + 1u) << 8) | p.exch_idx;
  const uint32_t slice = p.count / p.tp, nthreads = gridDim.x * blockDim.x, gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const size_t set = (size_t)(p.exch_idx & 1u) * 2u * p.count;  // words: region A, then region B
  const uint32_t budget = peer_failed() ? 0u : p.poll_limit;
  // A: scatter the slices
  for (uint32_t i = gtid; i < p.count; i += nthreads) {
    const uint32_t owner = i / slice, e = i - owner * slice;
    st_peer(p.slots[owner] + set + (size_t)p.rank * slice + e, make_uint2(__float_as_uint(__ldcg(p.x + i)), tag));
  }
  // B: sum this rank's slice, publish it everywhere
  const uint2 *mine = p.slots[p.rank] + set;
  for (uint32_t e = gtid; e < slice; e += nthreads) {
    uint2 w[MAX_TP];
#pragma unroll
    for (int r = 0; r < MAX_TP; ++r)
      if ((uint32_t)r < p.tp) w[r] = ld_peer8(mine + (size_t)r * slice + e);  // all rows in flight before any tag is looked at
    float v = 0.f;
#pragma unroll
    for (int r = 0; r < MAX_TP; ++r) {
      if ((uint32_t)r < p.tp) {
        if (w[r].y != tag) w[r] = wait_tagged(mine + (size_t)r * slice + e, tag, budget);
        v += __uint_as_float(w[r].x);
      }
    }
    const uint2 out = make_uint2(__float_as_uint(v), tag);
#pragma unroll
    for (int j = 0; j < MAX_TP; ++j)
      if ((uint32_t)j < p.tp) st_peer(p.slots[j] + set + p.count + (size_t)p.rank * slice + e, out);
  }
  // C: collect
  const uint2 *sums = mine + p.count;
  for (uint32_t i = gtid; i < p.count; i += nthreads) {
    uint2 w = ld_peer8(sums + i);
    if (w.y != tag) w = wait_tagged(sums + i, tag, budget);
    p.x[i] = __uint_as_float(w.x);
  }
}

int fill_exchange(GemvParams &p, const greta_peer_exchange *ex, uint32_t exch_idx, const uint32_t *d_pos, uint32_t dim, bool as_producer) {
  GRETA_REQUIRE(ex && d_pos, "tensor-parallel exchange: null exchange descriptor or position");
  GRETA_REQUIRE(ex->tp >= 1 && ex->tp <= (uint32_t)MAX_TP && ex->rank < ex->tp, "tensor-parallel exchange: rank %u of %u", ex->rank, ex->tp);
  GRETA_REQUIRE(exch_idx < 256, "tensor-parallel exchange: index %u out of range (256 per step)", exch_idx);
  GRETA_REQUIRE(dim % 32 == 0 && dim <= 8192, "tensor-parallel exchange: dim=%u must be a multiple of 32, at most 8192", dim);
  const size_t parity_words = (size_t)(ex->tp + 1) * dim;  // {value, tag} words per parity: tp partial vectors, then the sum vector
  for (uint32_t j = 0; j < ex->tp; ++j) {
    GRETA_REQUIRE(ex->slots[j] && aligned16(ex->slots[j]), "tensor-parallel exchange: slot buffer %u is null or misaligned", j);
    p.peer_out[j] = as_producer ? static_cast<uint2 *>(ex->slots[j]) + (exch_idx & 1) * parity_words : nullptr;
  }
  p.peer_in = as_producer ? nullptr : static_cast<const uint2 *>(ex->slots[ex->rank]) + (exch_idx & 1) * parity_words;
  if (!as_producer) {
    p.sum_out = static_cast<uint2 *>(ex->slots[ex->rank]) + (exch_idx & 1) * parity_words + (size_t)ex->tp * dim;
    p.sum_in = p.sum_out;
    p.two_level = ex->tp >= (uint32_t)tuning().peer_two_level_min_tp ? 1u : 0u;
  }
  p.tp = ex->tp;
  p.rank = ex->rank;
  p.exch_idx = exch_idx;
  p.d_pos = d_pos;
  p.poll_limit = tuning().peer_poll_limit;
  return GRETA_OK;
}

template <int EPI>
int dispatch_quant(cudaStream_t stream, int fmt, const GemvParams &p, uint64_t total_rows) {
  switch (fmt) {
    case GRETA_FMT_Q4_0: return launch_quant<GRETA_FMT_Q4_0, EPI>(stream, p, total_rows);
    case GRETA_FMT_Q8_0: return launch_quant<GRETA_FMT_Q8_0, EPI>(stream, p, total_rows);
    case GRETA_FMT_F16: return launch_any<GRETA_FMT_F16, EPI, 2>(stream, p);
    default: break;
  }
  set_error("gemv: format %d is not supported by this operator", fmt);
  return GRETA_ERR_INVALID_ARGS;
}

int check_plane(const char *what, const void *qs, const void *d, int fmt) {
  GRETA_REQUIRE(qs != nullptr, "%s: null weight pointer", what);
  GRETA_REQUIRE(fmt == GRETA_FMT_F16 || d != nullptr, "%s: null scale pointer", what);
  GRETA_REQUIRE(aligned16(qs), "%s: weight plane is not 16-byte aligned", what);
  if (fmt == GRETA_FMT_Q4_0 || fmt == GRETA_FMT_Q8_0)
    GRETA_REQUIRE(aligned16(d), "%s: scale plane is not 16-byte aligned", what);
  else if (fmt != GRETA_FMT_F16)
    GRETA_REQUIRE(((uintptr_t)d & 3) == 0, "%s: scale plane is not 4-byte aligned", what);
  return GRETA_OK;
}

}  // namespace

extern "C" {

int greta_cuda_gemv(greta_stream_t stream, int fmt, const void *x, int x_is_f16, const void *qs, const void *d, float *y,
                    uint32_t M, uint32_t N, uint32_t K) {
  if (M == 0 || N == 0 || K == 0) return GRETA_OK;  // the reference launchers return silently (gemm_kernels.hip:746,915)
  GRETA_REQUIRE(K % 32 == 0, "gemv: K=%u is not a multiple of the block size 32", K);
  GRETA_REQUIRE(x && y, "gemv: null activation or output pointer");
  GRETA_REQUIRE(M <= 65535, "gemv: M=%u exceeds 65535", M);
  GRETA_REQUIRE(fmt == GRETA_FMT_Q4_0 || fmt == GRETA_FMT_Q8_0 || fmt == GRETA_FMT_REF_INT4 || fmt == GRETA_FMT_REF_INT8 ||
                    fmt == GRETA_FMT_F16,
                "gemv: unknown weight format %d", fmt);
  if (int rc = check_plane("gemv", qs, d, fmt)) return rc;
  // Several rows of fp32 activations against a GGUF-format or fp16 weight: the batched kernel reads the weights
  // once for up to 32 rows (the per-row kernel below would read them M times).
  if (M > 1 && !x_is_f16 && tuning().skinny_max_rows > 1 && aligned16(x) && (fmt == GRETA_FMT_F16 || aligned16(d)) &&
      (fmt == GRETA_FMT_Q4_0 || fmt == GRETA_FMT_Q8_0 || fmt == GRETA_FMT_F16)) {
    const uint32_t step = (uint32_t)tuning().skinny_max_rows;
    for (uint32_t m0 = 0; m0 < M; m0 += step) {
      const uint32_t rows = std::min(step, M - m0);
      if (int rc = gemv_batch_plain((cudaStream_t)stream, fmt, static_cast<const float *>(x) + (size_t)m0 * K, qs, d, y + (size_t)m0 * N, rows, N, K, 0))
        return rc;
    }
    return GRETA_OK;
  }
  GemvParams p{};
  p.x = x;
  p.x_is_f16 = x_is_f16;
  p.w[0] = {(const uint8_t *)qs, d};
  p.K = K;
  p.N = N;
  p.M = M;
  p.y = y;
  cudaStream_t s = (cudaStream_t)stream;
  switch (fmt) {
    case GRETA_FMT_Q4_0: return launch_quant<GRETA_FMT_Q4_0, EPI_PLAIN>(s, p, N);
    case GRETA_FMT_Q8_0: return launch_quant<GRETA_FMT_Q8_0, EPI_PLAIN>(s, p, N);
    case GRETA_FMT_REF_INT4: return launch_any<GRETA_FMT_REF_INT4, EPI_PLAIN, 4>(s, p);
    case GRETA_FMT_REF_INT8: return launch_any<GRETA_FMT_REF_INT8, EPI_PLAIN, 4>(s, p);
    default: return launch_any<GRETA_FMT_F16, EPI_PLAIN, 2>(s, p);
  }
}

int greta_cuda_rmsnorm_gemv(greta_stream_t stream, int fmt, const float *x, const float *gamma, float eps, const void *qs,
                            const void *d, float *y, uint32_t N, uint32_t K) {
  if (N == 0 || K == 0) return GRETA_OK;
  GRETA_REQUIRE(K % 32 == 0, "rmsnorm_gemv: K=%u is not a multiple of 32", K);
  GRETA_REQUIRE(x && y && gamma, "rmsnorm_gemv: null pointer");
  if (int rc = check_plane("rmsnorm_gemv", qs, d, fmt)) return rc;
  GemvParams p{};
  p.x = x;
  p.gamma = gamma;
  p.eps = eps;
  p.w[0] = {(const uint8_t *)qs, d};
  p.K = K;
  p.N = N;
  p.M = 1;
  p.y = y;
  return dispatch_quant<EPI_PLAIN>((cudaStream_t)stream, fmt, p, N);
}

int greta_cuda_gemv_residual(greta_stream_t stream, int fmt, const float *x, const void *qs, const void *d,
                             const float *resid, float *y, uint32_t N, uint32_t K) {
  if (N == 0 || K == 0) return GRETA_OK;
  GRETA_REQUIRE(K % 32 == 0, "gemv_residual: K=%u is not a multiple of 32", K);
  GRETA_REQUIRE(x && y && resid, "gemv_residual: null pointer");
  if (int rc = check_plane("gemv_residual", qs, d, fmt)) return rc;
  GemvParams p{};
  p.x = x;
  p.w[0] = {(const uint8_t *)qs, d};
  p.K = K;
  p.N = N;
  p.M = 1;
  p.y = y;
  p.resid = resid;
  return dispatch_quant<EPI_RESIDUAL>((cudaStream_t)stream, fmt, p, N);
}

int greta_cuda_fused_rmsnorm_qkv_rope_kv(greta_stream_t stream, int fmt, const float *x, const float *gamma, float eps,
                                         const void *wq_qs, const void *wq_d, const void *wk_qs, const void *wk_d,
                                         const void *wv_qs, const void *wv_d, float *q_out, float *k_out, float *v_out,
                                         void *k_cache, void *v_cache, const uint32_t *d_pos, uint32_t H, uint32_t Hkv,
                                         uint32_t Dh, uint32_t max_seq, float rope_base, uint32_t D) {
  GRETA_REQUIRE(D && H && Hkv && Dh, "fused_qkv: zero dimension");
  GRETA_REQUIRE(D % 32 == 0, "fused_qkv: D=%u is not a multiple of 32", D);
  GRETA_REQUIRE(Dh % 2 == 0, "fused_qkv: head_dim=%u is odd", Dh);
  GRETA_REQUIRE(H % Hkv == 0, "fused_qkv: num_heads=%u is not a multiple of num_heads_kv=%u", H, Hkv);
  GRETA_REQUIRE(x && q_out, "fused_qkv: null pointer");
  GRETA_REQUIRE(d_pos ? (k_cache && v_cache) : (k_out && v_out),
                "fused_qkv: with d_pos the caches are required, without it k_out and v_out");
  if (int rc = check_plane("fused_qkv(wq)", wq_qs, wq_d, fmt)) return rc;
  if (int rc = check_plane("fused_qkv(wk)", wk_qs, wk_d, fmt)) return rc;
  if (int rc = check_plane("fused_qkv(wv)", wv_qs, wv_d, fmt)) return rc;
  GemvParams p{};
  p.x = x;
  p.gamma = gamma;
  p.eps = eps;
  p.w[0] = {(const uint8_t *)wq_qs, wq_d};
  p.w[1] = {(const uint8_t *)wk_qs, wk_d};
  p.w[2] = {(const uint8_t *)wv_qs, wv_d};
  p.K = D;
  p.M = 1;
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
  return dispatch_quant<EPI_QKV>((cudaStream_t)stream, fmt, p, (uint64_t)(H + 2 * Hkv) * Dh);
}

int greta_cuda_fused_ffn_front(greta_stream_t stream, int fmt, const float *x, const float *gamma, float eps,
                               const void *w1_qs, const void *w1_d, const void *w3_qs, const void *w3_d, float *y,
                               uint32_t D, uint32_t F) {
  if (F == 0 || D == 0) return GRETA_OK;
  GRETA_REQUIRE(D % 32 == 0, "fused_ffn_front: D=%u is not a multiple of 32", D);
  GRETA_REQUIRE(x && y, "fused_ffn_front: null pointer");
  if (int rc = check_plane("fused_ffn_front(w1)", w1_qs, w1_d, fmt)) return rc;
  if (int rc = check_plane("fused_ffn_front(w3)", w3_qs, w3_d, fmt)) return rc;
  GemvParams p{};
  p.x = x;
  p.gamma = gamma;
  p.eps = eps;
  p.w[0] = {(const uint8_t *)w1_qs, w1_d};
  p.w[1] = {(const uint8_t *)w3_qs, w3_d};
  p.K = D;
  p.N = F;
  p.M = 1;
  p.y = y;
  return dispatch_quant<EPI_SWIGLU>((cudaStream_t)stream, fmt, p, (uint64_t)2 * F);
}

// ---- tensor-parallel exchange over peer memory ---------------------------------------------------
size_t greta_cuda_peer_slot_bytes(uint32_t tp, uint32_t dim) { return (size_t)2 * (tp + 1) * dim * sizeof(uint2); }

int greta_cuda_peer_status(int *code) {
  GRETA_REQUIRE(code, "peer_status: null out pointer");
  GRETA_CUDA_TRY(cudaMemcpyFromSymbol(code, g_peer_error, sizeof(int)));
  return GRETA_OK;
}

int greta_cuda_peer_reset(greta_stream_t stream) {
  void *addr = nullptr;
  GRETA_CUDA_TRY(cudaGetSymbolAddress(&addr, g_peer_error));
  GRETA_CUDA_TRY(cudaMemsetAsync(addr, 0, sizeof(int), (cudaStream_t)stream));
  return GRETA_OK;
}

int greta_cuda_gemv_peer_scatter(greta_stream_t stream, int fmt, const float *x, const void *qs, const void *d,
                                 const greta_peer_exchange *ex, uint32_t exch_idx, const uint32_t *d_pos, uint32_t N, uint32_t K) {
  GRETA_REQUIRE(N && K && K % 32 == 0, "gemv_peer_scatter: N=%u, K=%u (K must be a positive multiple of 32)", N, K);
  GRETA_REQUIRE(x, "gemv_peer_scatter: null activation pointer");
  if (int rc = check_plane("gemv_peer_scatter", qs, d, fmt)) return rc;
  GemvParams p{};
  p.x = x;
  p.w[0] = {(const uint8_t *)qs, d};
  p.K = K;
  p.N = N;
  p.M = 1;
  if (int rc = fill_exchange(p, ex, exch_idx, d_pos, N, true)) return rc;
  return dispatch_peer<EPI_PEER, false>((cudaStream_t)stream, fmt, p, N);
}

int greta_cuda_fused_rmsnorm_qkv_rope_kv_peer(greta_stream_t stream, int fmt, const float *x_in, float *x_out,
                                              const greta_peer_exchange *ex, uint32_t exch_idx, const float *gamma, float eps,
                                              const void *wq_qs, const void *wq_d, const void *wk_qs, const void *wk_d,
                                              const void *wv_qs, const void *wv_d, float *q_out, void *k_cache, void *v_cache,
                                              const uint32_t *d_pos, uint32_t H, uint32_t Hkv, uint32_t Dh, uint32_t max_seq,
                                              float rope_base, uint32_t D) {
  GRETA_REQUIRE(D && H && Hkv && Dh && Dh % 2 == 0 && H % Hkv == 0, "fused_qkv_peer: bad dimensions");
  GRETA_REQUIRE(x_in && x_out && x_in != x_out && gamma && q_out && k_cache && v_cache, "fused_qkv_peer: null pointer, or x_out aliases x_in");
  if (int rc = check_plane("fused_qkv_peer(wq)", wq_qs, wq_d, fmt)) return rc;
  if (int rc = check_plane("fused_qkv_peer(wk)", wk_qs, wk_d, fmt)) return rc;
  if (int rc = check_plane("fused_qkv_peer(wv)", wv_qs, wv_d, fmt)) return rc;
  GemvParams p{};
  p.x = x_in;
  p.x_out = x_out;
  p.gamma = gamma;
  p.eps = eps;
  p.w[0] = {(const uint8_t *)wq_qs, wq_d};
  p.w[1] = {(const uint8_t *)wk_qs, wk_d};
  p.w[2] = {(const uint8_t *)wv_qs, wv_d};
  p.K = D;
  p.M = 1;
  p.q_out = q_out;
  p.k_cache = (__half *)k_cache;
  p.v_cache = (__half *)v_cache;
  p.H = H;
  p.Hkv = Hkv;
  p.Dh = Dh;
  p.max_seq = max_seq;
  p.rope_base = rope_base;
  if (int rc = fill_exchange(p, ex, exch_idx, d_pos, D, false)) return rc;
  return dispatch_peer<EPI_QKV, true>((cudaStream_t)stream, fmt, p, (uint64_t)(H + 2 * Hkv) * Dh);
}

int greta_cuda_fused_ffn_front_peer(greta_stream_t stream, int fmt, const float *x_in, float *x_out, const greta_peer_exchange *ex,
                                    uint32_t exch_idx, const uint32_t *d_pos, const float *gamma, float eps, const void *w1_qs,
                                    const void *w1_d, const void *w3_qs, const void *w3_d, float *y, uint32_t D, uint32_t F) {
  GRETA_REQUIRE(D && F, "fused_ffn_front_peer: zero dimension");
  GRETA_REQUIRE(x_in && x_out && x_in != x_out && gamma && y, "fused_ffn_front_peer: null pointer, or x_out aliases x_in");
  if (int rc = check_plane("fused_ffn_front_peer(w1)", w1_qs, w1_d, fmt)) return rc;
  if (int rc = check_plane("fused_ffn_front_peer(w3)", w3_qs, w3_d, fmt)) return rc;
  GemvParams p{};
  p.x = x_in;
  p.x_out = x_out;
  p.gamma = gamma;
  p.eps = eps;
  p.w[0] = {(const uint8_t *)w1_qs, w1_d};
  p.w[1] = {(const uint8_t *)w3_qs, w3_d};
  p.K = D;
  p.N = F;
  p.M = 1;
  p.y = y;
  if (int rc = fill_exchange(p, ex, exch_idx, d_pos, D, false)) return rc;
  return dispatch_peer<EPI_SWIGLU, true>((cudaStream_t)stream, fmt, p, (uint64_t)2 * F);
}

size_t greta_cuda_peer_allreduce_slot_bytes(size_t max_count) { return (size_t)4 * max_count * sizeof(uint2); }

int greta_cuda_peer_allreduce_f32(greta_stream_t stream, float *x, size_t count, const greta_peer_exchange *ex, uint32_t exch_idx,
                                  const uint32_t *d_pos) {
  GRETA_REQUIRE(ex && d_pos && x, "peer_allreduce: null pointer");
  GRETA_REQUIRE(ex->tp >= 1 && ex->tp <= (uint32_t)MAX_TP && ex->rank < ex->tp, "peer_allreduce: rank %u of %u", ex->rank, ex->tp);
  GRETA_REQUIRE(exch_idx < 256, "peer_allreduce: index %u out of range (256 per step)", exch_idx);
  GRETA_REQUIRE(count > 0 && count % ex->tp == 0 && count < (1u << 28), "peer_allreduce: %zu values do not split over %u ranks", count, ex->tp);
  GRETA_REQUIRE(ex->slot_bytes >= greta_cuda_peer_allreduce_slot_bytes(count), "peer_allreduce: slot buffers of %zu bytes are too small for %zu values",
                (size_t)ex->slot_bytes, count);
  PeerArParams p{};
  p.x = x;
  p.count = (uint32_t)count;
  p.tp = ex->tp;
  p.rank = ex->rank;
  p.exch_idx = exch_idx;
  p.d_pos = d_pos;
  for (uint32_t j = 0; j < ex->tp; ++j) {
    GRETA_REQUIRE(ex->slots[j] && aligned16(ex->slots[j]), "peer_allreduce: slot buffer %u is null or misaligned", j);
    p.slots[j] = static_cast<uint2 *>(ex->slots[j]);
  }
  p.poll_limit = tuning().peer_poll_limit;
  // enough threads to have every word of a phase in flight at once, not more CTAs than SMs
  const unsigned ctas = (unsigned)std::min<size_t>((count / ex->tp + 255) / 256, (size_t)sm_count());
  GRETA_CUDA_TRY(launch_pdl(peer_allreduce_kernel, dim3(ctas ? ctas : 1), dim3(256), 0, (cudaStream_t)stream, p));
  return launched("peer_allreduce_kernel");
}

}  // extern "C"
