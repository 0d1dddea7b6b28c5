// Attention side of the decode path: split-sequence decode attention over the
// KV cache (fp16, or the reference's fp32), the causal prefill form built on the
// same inner loop, RoPE and the KV-cache write.
//
// Decode attention streams the cache once: HBM-bound.  A CTA owns one
// (query, head, sequence split); eight lanes share a key (16 or 8 head dims
// each, 128-bit loads), four keys per warp step, so one warp load instruction
// covers four whole cache rows.  Each lane group keeps its own running maximum,
// normaliser and output slice (online softmax); groups, warps and finally splits
// are merged with the usual (max, sum, vector) rescaling.  The splits of a head
// meet in one of two ways:
//   * attn_cluster_kernel (the default): the splits form a thread-block cluster,
//     every CTA leaves its partial result in its own shared memory and CTA 0 reads
//     them through distributed shared memory after a cluster barrier - no scratch;
//   * attn_kernel (tuning switch attn_cluster = 0, the persistent decode step, and
//     always for greta_cuda_attn_decode_static): through a scratch buffer - every
//     CTA publishes its partial result, bumps a per-head ticket, and the CTA that
//     draws the last ticket does the merge; no CTA ever waits on another.
#include <cooperative_groups.h>
#include <math.h>

#include <algorithm>
#include <mutex>

#include "attention_device.cuh"

namespace greta {
int attn_mma_decode(cudaStream_t stream, const AttnParams &p, uint32_t batch, uint32_t nsplit, uint32_t ng, uint32_t Dh);  // attention_mma.cu
int attn_mma_prefill(cudaStream_t stream, const AttnParams &p, uint32_t S, uint32_t pos0, uint32_t Dh);
}  // namespace greta

namespace {

constexpr int ATT_WARPS = 4;
constexpr int ATT_THREADS = ATT_WARPS * 32;

template <typename KV, int DPL>
__global__ void __launch_bounds__(ATT_THREADS) attn_kernel(const AttnParams p) {
  pdl_launch_dependents();
  pdl_wait();  // q, the position and the newest cache row come from the previous kernel
  attn_body<KV, DPL, ATT_WARPS, false>(p, blockIdx.x, blockIdx.y, blockIdx.z);
}

// The same work with the splits of one head in one thread-block cluster: every CTA leaves its partial
// result in its own shared memory, the cluster meets at a hardware barrier and CTA 0 reads the others'
// results through distributed shared memory.  No scratch, no fences, no atomics on the critical path.
constexpr int CL_SPLITS = 8;
constexpr int CL_WARPS = 8;

template <typename KV, int DPL>
__global__ void __launch_bounds__(CL_WARPS * 32) attn_cluster_kernel(const AttnParams p) {
  namespace cg = cooperative_groups;
  constexpr int Dh = DPL * 8;
  __shared__ float res[Dh + 2];  // running maximum, normaliser, unnormalised output of this CTA's keys
  cg::cluster_group cluster = cg::this_cluster();
  pdl_launch_dependents();
  pdl_wait();  // q, the position and the newest cache row come from the previous kernel
  const uint32_t split = cluster.block_rank(), head = blockIdx.y, qi = blockIdx.z;
  const uint32_t L = min((p.d_pos ? __ldcg(p.d_pos + qi * p.pos_stride) + 1 : p.len0) + qi * p.len_step, p.max_seq);  // never past the cache
  const uint32_t chunk = (L + CL_SPLITS - 1) / CL_SPLITS;
  const uint32_t k0 = split * chunk, k1 = min(L, k0 + chunk);
  const int tid = threadIdx.x;
  float fm, fl, fo;
  if (sizeof(KV) == 2) {
    extern __shared__ __align__(16) uint8_t stage[];
    attn_partial_staged<DPL, CL_WARPS>(p, min(k0, k1), k1, head, qi, stage, fm, fl, fo);
  } else {
    attn_partial<KV, DPL, CL_WARPS, false>(p, min(k0, k1), k1, head, qi, fm, fl, fo);
  }
  if (tid < Dh) res[2 + tid] = fo;
  if (tid == 0) {
    res[0] = fm;
    res[1] = fl;
  }
  cluster.sync();
  if (split == 0 && tid < Dh) {
    float rm[CL_SPLITS], rl[CL_SPLITS], ro[CL_SPLITS], gm = -INFINITY;
#pragma unroll
    for (int r = 0; r < CL_SPLITS; ++r) {
      const float *rp = cluster.map_shared_rank(res, r);
      rm[r] = rp[0];
      rl[r] = rp[1];
      ro[r] = rp[2 + tid];
      gm = fmaxf(gm, rm[r]);
    }
    float gl = 0.f, go = 0.f;
#pragma unroll
    for (int r = 0; r < CL_SPLITS; ++r) {  // fixed order: the result does not depend on which CTA finished first
      const float c = (rm[r] == -INFINITY) ? 0.f : expf(rm[r] - gm);
      gl += rl[r] * c;
      go += ro[r] * c;
    }
    p.o[((size_t)qi * p.H + head) * Dh + tid] = go / gl;
  }
  cluster.sync();  // a CTA's shared memory must outlive the reads of CTA 0
}

__global__ void rope_kernel(float *x, uint32_t S, uint32_t H, uint32_t Dh, float base, uint32_t pos_offset,
                            const uint32_t *d_pos) {
  uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
  uint32_t hd2 = Dh / 2, total = S * H * hd2;
  if (idx >= total) return;
  uint32_t i = idx % hd2, h = (idx / hd2) % H, s = idx / (hd2 * H);
  uint32_t pos = (d_pos ? *d_pos : pos_offset) + s;
  float theta = (float)pos * powf(base, -2.0f * (float)i / (float)Dh);
  float c = cosf(theta), sn = sinf(theta);
  size_t bi = (size_t)s * H * Dh + (size_t)h * Dh + i;
  float v0 = x[bi], v1 = x[bi + hd2];
  x[bi] = v0 * c - v1 * sn;
  x[bi + hd2] = v0 * sn + v1 * c;
}

__global__ void kv_update_kernel(__half *kc, __half *vc, const float *nk, const float *nv, uint32_t S, uint32_t pos,
                                 const uint32_t *d_pos, uint32_t max_seq, uint32_t Hkv, uint32_t Dh) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t total = (size_t)S * Hkv * Dh;
  if (idx >= total) return;
  uint32_t d = idx % Dh, h = (idx / Dh) % Hkv, s = idx / ((size_t)Dh * Hkv);
  uint32_t pp = (d_pos ? *d_pos : pos) + s;
  if (pp >= max_seq) return;
  size_t dst = ((size_t)h * max_seq + pp) * Dh + d;
  kc[dst] = __float2half_rn(nk[idx]);
  vc[dst] = __float2half_rn(nv[idx]);
}

size_t counters_bytes(uint32_t H) { return ((size_t)H * 4 + 255) / 256 * 256; }

template <typename KV>
int launch_attn(cudaStream_t stream, AttnParams p, uint32_t nq, uint32_t Dh) {
  dim3 grid(p.splits, p.H, nq);
  if (Dh == 128)
    GRETA_CUDA_TRY(launch_pdl(attn_kernel<KV, 16>, grid, dim3(ATT_THREADS), 0, stream, p));
  else if (Dh == 64)
    GRETA_CUDA_TRY(launch_pdl(attn_kernel<KV, 8>, grid, dim3(ATT_THREADS), 0, stream, p));
  else {
    set_error("attention: head_dim=%u is not supported (64 or 128)", Dh);
    return GRETA_ERR_NOT_IMPLEMENTED;
  }
  return launched("attn_kernel");
}

template <typename KV>
int launch_attn_cluster(cudaStream_t stream, AttnParams p, uint32_t Dh, uint32_t nq = 1) {
  dim3 grid(CL_SPLITS, p.H, nq);
  // Same shared-memory / L1 split as the GEMV kernels on either side of it in the decode step: an SM does
  // not have to be reconfigured (and drained for it) at every kernel boundary.
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const size_t s16 = sizeof(KV) == 2 ? attn_stage_bytes<16>() : 0, s8 = sizeof(KV) == 2 ? attn_stage_bytes<8>() : 0;  // fp16 cache: staged tiles
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    GRETA_CUDA_TRY(cudaFuncSetAttribute(attn_cluster_kernel<KV, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s16));
    GRETA_CUDA_TRY(cudaFuncSetAttribute(attn_cluster_kernel<KV, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s8));
    GRETA_CUDA_TRY(cudaFuncSetAttribute(attn_cluster_kernel<KV, 16>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
    GRETA_CUDA_TRY(cudaFuncSetAttribute(attn_cluster_kernel<KV, 8>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
    cudaFuncSetAttribute(attn_cluster_kernel<KV, 16>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(attn_cluster_kernel<KV, 8>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    attr_set[dev] = true;
  }
  if (Dh == 128)
    GRETA_CUDA_TRY(launch_pdl_cluster(attn_cluster_kernel<KV, 16>, grid, dim3(CL_WARPS * 32), CL_SPLITS, s16, stream, p));
  else if (Dh == 64)
    GRETA_CUDA_TRY(launch_pdl_cluster(attn_cluster_kernel<KV, 8>, grid, dim3(CL_WARPS * 32), CL_SPLITS, s8, stream, p));
  else {
    set_error("attention: head_dim=%u is not supported (64 or 128)", Dh);
    return GRETA_ERR_NOT_IMPLEMENTED;
  }
  return launched("attn_cluster_kernel");
}

// scratch_merge_only: the splits meet through `scratch` whatever the attn_cluster switch says.
template <typename KV>
int attn_decode_impl(greta_stream_t stream, const float *q, const void *kc, const void *vc, float *o,
                     const uint32_t *d_pos, uint32_t seq_len, uint32_t H, uint32_t Hkv, uint32_t Dh, uint32_t max_seq,
                     float scale, void *scratch, size_t scratch_bytes, bool scratch_merge_only = false, uint32_t batch = 0) {
  GRETA_REQUIRE(H && Hkv && H % Hkv == 0, "attn_decode: num_heads=%u must be a positive multiple of num_heads_kv=%u", H, Hkv);
  GRETA_REQUIRE(q && kc && vc && o, "attn_decode: null pointer");
  GRETA_REQUIRE(aligned16(q) && aligned16(kc) && aligned16(vc), "attn_decode: pointers must be 16-byte aligned");
  GRETA_REQUIRE(d_pos || (seq_len >= 1 && seq_len <= max_seq), "attn_decode: seq_len=%u outside 1..max_seq_len=%u", seq_len, max_seq);
  // Splits are sized for the longest sequence this cache can hold, so that a captured launch stays valid as the position advances.
  const uint32_t Lmax = d_pos ? max_seq : seq_len;
  const uint32_t nq = batch ? batch : 1u, slots = nq * H;  // (sequence, head) pairs
  uint32_t want = (2u * (uint32_t)sm_count() + slots - 1) / slots;
  uint32_t splits = std::max(1u, std::min({want, (uint32_t)MAX_SPLITS, (Lmax + 63) / 64}));
  AttnParams p{};
  p.q = q; p.kc = kc; p.vc = vc; p.o = o; p.d_pos = d_pos; p.len0 = seq_len;
  p.H = H; p.Hkv = Hkv; p.max_seq = max_seq; p.scale = scale; p.splits = splits; p.len_step = batch ? 0 : 1;
  if (batch) {  // every query is its own sequence: own cache, own position
    p.seq_stride = (size_t)Hkv * max_seq * Dh;
    p.pos_stride = 1;
  }
  if (splits > 1) {
    GRETA_REQUIRE(scratch && scratch_bytes >= greta_cuda_attn_decode_scratch_bytes(slots, Dh),
                  "attn_decode: scratch of %zu bytes needed, %zu given", greta_cuda_attn_decode_scratch_bytes(slots, Dh), scratch_bytes);
    p.counters = reinterpret_cast<uint32_t *>(scratch);
    p.partial = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(scratch) + counters_bytes(slots));
    if (!scratch_merge_only && tuning().attn_cluster) return launch_attn_cluster<KV>((cudaStream_t)stream, p, Dh, nq);
  }
  return launch_attn<KV>((cudaStream_t)stream, p, nq, Dh);
}

// ------------------------------------------------------------------ grouped-query batched decode attention
// One CTA per (KV head, sequence, key split): the K / V rows of its keys travel global -> shared once (cp.async, tiles of
// 64 keys, three in flight) and every warp runs one of the NG query heads that share the KV head over the staged tile, so
// the cache is read from HBM once per KV head instead of once per query head.  The splits of a (KV head, sequence) pair
// form a thread-block cluster; CTA 0 merges their (max, sum, output) triples through distributed shared memory in rank
// order.  fp16 cache only.
template <int DPL, int NG>
__global__ void __launch_bounds__(NG * 32) attn_gqa_kernel(const AttnParams p) {
  namespace cg = cooperative_groups;
  constexpr int Dh = DPL * 8, ROW = Dh * 2, TK = ATT_TILE_KEYS, NT = ATT_TILES_IN_FLIGHT, TILE_BYTES = TK * ROW * 2;
  extern __shared__ __align__(16) uint8_t stage[];
  __shared__ float res[NG][Dh + 2];  // per query head: running maximum, normaliser, unnormalised output of this CTA's keys
  cg::cluster_group cluster = cg::this_cluster();
  pdl_launch_dependents();
  pdl_wait();  // q, the positions and the newest cache rows come from the previous kernel
  const uint32_t nsplit = gridDim.x, split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, sub = lane & 7, grp = lane >> 3;
  const uint32_t head = kvh * NG + warp;
  const uint32_t L = min((p.d_pos ? __ldcg(p.d_pos + seq * p.pos_stride) + 1 : p.len0), p.max_seq);
  const uint32_t chunk = (L + nsplit - 1) / nsplit;
  const uint32_t k0 = min(split * chunk, L), k1 = min(L, k0 + chunk);
  const uint8_t *kg = reinterpret_cast<const uint8_t *>(p.kc) + ((size_t)seq * p.seq_stride + (size_t)kvh * p.max_seq * Dh) * 2;
  const uint8_t *vg = reinterpret_cast<const uint8_t *>(p.vc) + ((size_t)seq * p.seq_stride + (size_t)kvh * p.max_seq * Dh) * 2;
  const uint32_t n_tiles = k1 > k0 ? (k1 - k0 + TK - 1) / TK : 0;
  auto issue = [&](uint32_t t) {
    if (t < n_tiles) {
      const uint32_t key0 = k0 + t * TK, nk = min((uint32_t)TK, k1 - key0);
      uint8_t *slot = stage + (t % NT) * TILE_BYTES;
      for (uint32_t piece = tid; piece < nk * (ROW / 8); piece += NG * 32) {  // ROW / 16 K pieces and as many V pieces of 16 bytes per key
        const uint32_t row = piece / (ROW / 8), c = piece % (ROW / 8), is_v = c / (ROW / 16), cc = c % (ROW / 16);
        const uint8_t *src = (is_v ? vg : kg) + (size_t)(key0 + row) * ROW + cc * 16;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(slot + is_v * (TK * ROW) + row * ROW + cc * 16);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int t = 0; t < NT; ++t) issue(t);

  float qv[DPL];
  {
    const float *qp = p.q + ((size_t)seq * p.H + head) * Dh + sub * DPL;
#pragma unroll
    for (int i = 0; i < DPL; i += 4) {
      float4 t4 = __ldcg(reinterpret_cast<const float4 *>(qp + i));
      qv[i] = t4.x * p.scale; qv[i + 1] = t4.y * p.scale; qv[i + 2] = t4.z * p.scale; qv[i + 3] = t4.w * p.scale;
    }
  }
  float m = -INFINITY, l = 0.f, o[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) o[i] = 0.f;

  for (uint32_t t = 0; t < n_tiles; ++t) {
    asm volatile("cp.async.wait_group %0;" ::"n"(NT - 1) : "memory");
    __syncthreads();  // every thread's pieces of tile t have landed
    const uint32_t nk = min((uint32_t)TK, k1 - (k0 + t * TK));
    const uint8_t *slot = stage + (t % NT) * TILE_BYTES;
    for (uint32_t base = 0; base < nk; base += 4) {  // this warp's head against every key of the tile, one key per lane group
      const uint32_t j = base + grp;
      const bool valid = j < nk;
      float kf[DPL], vf[DPL];
      if (valid) {
#pragma unroll
        for (int v = 0; v < DPL / 8; ++v) {
          const uint4 ku = *reinterpret_cast<const uint4 *>(slot + j * ROW + sub * (DPL * 2) + v * 16);
          const uint4 vu = *reinterpret_cast<const uint4 *>(slot + TK * ROW + j * ROW + sub * (DPL * 2) + v * 16);
          float2 a = h2_to_f2(ku.x), b = h2_to_f2(ku.y), c = h2_to_f2(ku.z), d = h2_to_f2(ku.w);
          kf[8 * v + 0] = a.x; kf[8 * v + 1] = a.y; kf[8 * v + 2] = b.x; kf[8 * v + 3] = b.y;
          kf[8 * v + 4] = c.x; kf[8 * v + 5] = c.y; kf[8 * v + 6] = d.x; kf[8 * v + 7] = d.y;
          a = h2_to_f2(vu.x); b = h2_to_f2(vu.y); c = h2_to_f2(vu.z); d = h2_to_f2(vu.w);
          vf[8 * v + 0] = a.x; vf[8 * v + 1] = a.y; vf[8 * v + 2] = b.x; vf[8 * v + 3] = b.y;
          vf[8 * v + 4] = c.x; vf[8 * v + 5] = c.y; vf[8 * v + 6] = d.x; vf[8 * v + 7] = d.y;
        }
      }
      float sc = 0.f;
      if (valid) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) sc = fmaf(qv[i], kf[i], sc);
      }
#pragma unroll
      for (int off = 4; off > 0; off >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, off);  // the 8 lanes that share a key
      if (valid) {
        float mn = fmaxf(m, sc), c = expf(m - mn), pe = expf(sc - mn);
        l = l * c + pe;
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[i] = fmaf(pe, vf[i], o[i] * c);
        m = mn;
      }
    }
    __syncthreads();  // the slot is free again
    issue(t + NT);
  }
  // merge the four lane groups of the warp (same dims, different keys): the warp's head is complete for this CTA's keys
#pragma unroll
  for (int off = 8; off <= 16; off <<= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, off), l2 = __shfl_xor_sync(0xffffffffu, l, off), o2[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) o2[i] = __shfl_xor_sync(0xffffffffu, o[i], off);
    merge<DPL>(m, l, o, m2, l2, o2);
  }
  float *out = p.o + ((size_t)seq * p.H + head) * Dh;
  if (nsplit == 1) {
    if (grp == 0) {
#pragma unroll
      for (int i = 0; i < DPL; ++i) out[sub * DPL + i] = o[i] / l;
    }
    return;
  }
  if (grp == 0) {
    if (sub == 0) {
      res[warp][0] = m;
      res[warp][1] = l;
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) res[warp][2 + sub * DPL + i] = o[i];
  }
  cluster.sync();
  if (split == 0) {
    for (int d = lane; d < Dh; d += 32) {
      float gm = -INFINITY;
      for (uint32_t r = 0; r < nsplit; ++r) gm = fmaxf(gm, cluster.map_shared_rank(&res[warp][0], r)[0]);
      float gl = 0.f, go = 0.f;
      for (uint32_t r = 0; r < nsplit; ++r) {  // rank order: the result does not depend on which CTA finished first
        const float *rp = cluster.map_shared_rank(&res[warp][0], r);
        const float c = (rp[0] == -INFINITY) ? 0.f : expf(rp[0] - gm);
        gl += rp[1] * c;
        go += rp[2 + d] * c;
      }
      out[d] = go / gl;
    }
  }
  cluster.sync();  // a CTA's shared memory must outlive the reads of CTA 0
}

template <int DPL, int NG>
int launch_attn_gqa_cfg(cudaStream_t stream, const AttnParams &p, uint32_t batch, uint32_t nsplit) {
  auto kern = attn_gqa_kernel<DPL, NG>;
  const size_t smem = attn_stage_bytes<DPL>();
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    GRETA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set[dev] = true;
  }
  dim3 grid(nsplit, p.Hkv, batch);
  GRETA_CUDA_TRY(launch_pdl_cluster(kern, grid, dim3(NG * 32), nsplit, smem, stream, p));
  return launched("attn_gqa_kernel");
}

template <int DPL>
int launch_attn_gqa(cudaStream_t stream, const AttnParams &p, uint32_t batch, uint32_t nsplit, uint32_t ng) {
  switch (ng) {
    case 2: return launch_attn_gqa_cfg<DPL, 2>(stream, p, batch, nsplit);
    case 4: return launch_attn_gqa_cfg<DPL, 4>(stream, p, batch, nsplit);
    case 8: return launch_attn_gqa_cfg<DPL, 8>(stream, p, batch, nsplit);
    case 16: return launch_attn_gqa_cfg<DPL, 16>(stream, p, batch, nsplit);
    default: break;
  }
  set_error("attention: %u query heads per KV head are not supported by the grouped kernel (2, 4, 8 or 16)", ng);
  return GRETA_ERR_NOT_IMPLEMENTED;
}

}  // namespace

extern "C" {

// Layout of the scratch: per-head tickets (zero before the first call; every call
// leaves them zero), then [H][MAX_SPLITS][Dh + 2] floats of partial results.
size_t greta_cuda_attn_decode_scratch_bytes(uint32_t H, uint32_t Dh) {
  return counters_bytes(H) + (size_t)H * MAX_SPLITS * (Dh + 2) * sizeof(float);
}

int greta_cuda_attn_decode(greta_stream_t stream, const float *q, const void *kc, const void *vc, float *o,
                           const uint32_t *d_pos, uint32_t seq_len, uint32_t H, uint32_t Hkv, uint32_t Dh,
                           uint32_t max_seq, float scale, void *scratch, size_t scratch_bytes) {
  return attn_decode_impl<__half>(stream, q, kc, vc, o, d_pos, seq_len, H, Hkv, Dh, max_seq, scale, scratch, scratch_bytes);
}

int greta_cuda_attn_decode_f32cache(greta_stream_t stream, const float *q, const float *kc, const float *vc, float *o,
                                    const uint32_t *d_pos, uint32_t seq_len, uint32_t H, uint32_t Hkv, uint32_t Dh,
                                    uint32_t max_seq, float scale, void *scratch, size_t scratch_bytes) {
  return attn_decode_impl<float>(stream, q, kc, vc, o, d_pos, seq_len, H, Hkv, Dh, max_seq, scale, scratch, scratch_bytes);
}

int greta_cuda_attn_decode_batch(greta_stream_t stream, const float *q, const void *kc, const void *vc, float *o, const uint32_t *d_pos,
                                 uint32_t M, uint32_t H, uint32_t Hkv, uint32_t Dh, uint32_t max_seq, float scale, void *scratch,
                                 size_t scratch_bytes) {
  GRETA_REQUIRE(M >= 1 && M <= 65535, "attn_decode_batch: batch=%u outside 1..65535", M);
  GRETA_REQUIRE(d_pos, "attn_decode_batch: the positions live on the device (d_pos[batch])");
  GRETA_REQUIRE(H && Hkv && H % Hkv == 0, "attn_decode_batch: num_heads=%u must be a positive multiple of num_heads_kv=%u", H, Hkv);
  const uint32_t ng = H / Hkv;
  if (ng >= 2 && ng <= 16 && (ng & (ng - 1)) == 0 && (Dh == 64 || Dh == 128) && tuning().attn_cluster) {
    GRETA_REQUIRE(q && kc && vc && o && aligned16(q) && aligned16(kc) && aligned16(vc), "attn_decode_batch: null or misaligned pointer");
    // Splits (a power of two up to 8, one cluster) so that about two CTAs per SM exist, sized for the longest sequence the
    // cache can hold: a captured launch stays valid as the positions advance.
    const uint32_t pairs = Hkv * M, want = (2u * (uint32_t)sm_count() + pairs - 1) / pairs;
    uint32_t nsplit = 1;
    while (nsplit < 8 && nsplit < want && nsplit * 2 * 64 <= max_seq) nsplit *= 2;
    AttnParams p{};
    p.q = q; p.kc = kc; p.vc = vc; p.o = o; p.d_pos = d_pos; p.H = H; p.Hkv = Hkv; p.max_seq = max_seq; p.scale = scale;
    p.seq_stride = (size_t)Hkv * max_seq * Dh;
    p.pos_stride = 1;
    if (tuning().attn_mma) return attn_mma_decode((cudaStream_t)stream, p, M, nsplit, ng, Dh);  // tensor cores: the group's heads are the rows
    return Dh == 128 ? launch_attn_gqa<16>((cudaStream_t)stream, p, M, nsplit, ng) : launch_attn_gqa<8>((cudaStream_t)stream, p, M, nsplit, ng);
  }
  return attn_decode_impl<__half>(stream, q, kc, vc, o, d_pos, 0, H, Hkv, Dh, max_seq, scale, scratch, scratch_bytes, false, M);
}

// ---- allocation-free variant --------------------------------------------------------------
// Scratch for greta_cuda_attn_decode_static: lives in the module image, so every GPU that loads
// this library carries it (about 1 MiB) until the process exits.  Sized for 64 query heads of
// head_dim 128: the ticket words first, then the per-split partial results.
constexpr uint32_t STATIC_MAX_HEADS = 64, STATIC_MAX_HEAD_DIM = 128;
constexpr size_t STATIC_SCRATCH_BYTES = 256 + (size_t)STATIC_MAX_HEADS * MAX_SPLITS * (STATIC_MAX_HEAD_DIM + 2) * sizeof(float);
static __device__ __align__(256) unsigned char g_static_attn_scratch[STATIC_SCRATCH_BYTES];

// In host code the array's name is only a handle for the runtime, not an address a kernel can
// use; the device address is looked up once per device, with that device current.
static int static_scratch_address(void **out) {
  static std::mutex mu;
  static void *addr[64] = {};
  int dev = 0;
  GRETA_CUDA_TRY(cudaGetDevice(&dev));
  GRETA_REQUIRE(dev >= 0 && dev < 64, "attn_decode_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (!addr[dev]) {
    void *p = nullptr;
    GRETA_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_attn_scratch));
    addr[dev] = p;
  }
  *out = addr[dev];
  return GRETA_OK;
}

int greta_cuda_attn_decode_static(greta_stream_t stream, const float *q, const void *kc, const void *vc, float *o,
                                  const uint32_t *d_pos, uint32_t seq_len, uint32_t H, uint32_t Hkv, uint32_t Dh,
                                  uint32_t max_seq, float scale) {
  GRETA_REQUIRE(H <= STATIC_MAX_HEADS && Dh <= STATIC_MAX_HEAD_DIM,
                "attn_decode_static: %u heads of dim %u exceed the built-in scratch (at most %u heads of dim %u); "
                "use greta_cuda_attn_decode with caller-provided scratch",
                H, Dh, STATIC_MAX_HEADS, STATIC_MAX_HEAD_DIM);
  void *scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  // The array keeps whatever the previous call left; the tickets must start at zero.
  GRETA_CUDA_TRY(cudaMemsetAsync(scratch, 0, counters_bytes(H), (cudaStream_t)stream));
  // Always the scratch-buffer merge (attn_kernel): the partial results and tickets of the splits live in the array.
  return attn_decode_impl<__half>(stream, q, kc, vc, o, d_pos, seq_len, H, Hkv, Dh, max_seq, scale, scratch, STATIC_SCRATCH_BYTES,
                                  /*scratch_merge_only=*/true);
}

int greta_cuda_attn_prefill(greta_stream_t stream, const float *q, const void *kc, const void *vc, float *o, uint32_t S,
                            uint32_t pos0, uint32_t H, uint32_t Hkv, uint32_t Dh, uint32_t max_seq, float scale) {
  if (S == 0) return GRETA_OK;
  GRETA_REQUIRE(H && Hkv && H % Hkv == 0, "attn_prefill: num_heads=%u must be a positive multiple of num_heads_kv=%u", H, Hkv);
  GRETA_REQUIRE(q && kc && vc && o, "attn_prefill: null pointer");
  GRETA_REQUIRE(pos0 + S <= max_seq, "attn_prefill: positions %u..%u exceed max_seq_len=%u", pos0, pos0 + S, max_seq);
  GRETA_REQUIRE(S <= 65535, "attn_prefill: S=%u exceeds 65535", S);
  AttnParams p{};
  p.q = q; p.kc = kc; p.vc = vc; p.o = o; p.d_pos = nullptr; p.len0 = pos0 + 1;
  p.H = H; p.Hkv = Hkv; p.max_seq = max_seq; p.scale = scale; p.splits = 1; p.len_step = 1;
  // Prompts run on the tensor cores (16 positions of a head per warp, K / V tiles staged once per 64 positions); a few
  // positions, or the switch off, take one CTA per (position, head) on the decode inner loop.
  if (tuning().attn_mma && S >= 8 && (Dh == 64 || Dh == 128) && aligned16(q) && aligned16(kc) && aligned16(vc) && aligned16(o))
    return attn_mma_prefill((cudaStream_t)stream, p, S, pos0, Dh);
  return launch_attn<__half>((cudaStream_t)stream, p, S, Dh);
}

int greta_cuda_attn_prefill_f32(greta_stream_t stream, const float *q, const float *k, const float *v, float *o, uint32_t S, uint32_t H,
                                uint32_t Hkv, uint32_t Dh, float scale, int causal) {
  if (S == 0) return GRETA_OK;
  GRETA_REQUIRE(H && Hkv && H % Hkv == 0, "attn_prefill_f32: num_heads=%u must be a positive multiple of num_heads_kv=%u", H, Hkv);
  GRETA_REQUIRE(q && k && v && o, "attn_prefill_f32: null pointer");
  GRETA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v), "attn_prefill_f32: pointers must be 16-byte aligned");
  GRETA_REQUIRE(S <= 65535, "attn_prefill_f32: S=%u exceeds 65535", S);
  AttnParams p{};
  p.q = q; p.kc = k; p.vc = v; p.o = o; p.d_pos = nullptr;
  p.len0 = causal ? 1 : S; p.len_step = causal ? 1 : 0;
  p.H = H; p.Hkv = Hkv; p.max_seq = S; p.scale = scale; p.splits = 1;
  p.head_stride = Dh; p.row_stride = Hkv * Dh;  // K/V are [S][Hkv][Dh]
  return launch_attn<float>((cudaStream_t)stream, p, S, Dh);
}

int greta_cuda_rope(greta_stream_t stream, float *x, uint32_t S, uint32_t H, uint32_t Dh, float base, uint32_t pos_offset,
                    const uint32_t *d_pos) {
  uint32_t total = S * H * (Dh / 2);
  if (total == 0) return GRETA_OK;
  GRETA_REQUIRE(x, "rope: null pointer");
  GRETA_REQUIRE(Dh % 2 == 0, "rope: head_dim=%u must be even", Dh);
  rope_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(x, S, H, Dh, base, pos_offset, d_pos);
  return launched("rope_kernel");
}

int greta_cuda_kv_update(greta_stream_t stream, void *kc, void *vc, const float *nk, const float *nv, uint32_t S,
                         uint32_t pos, const uint32_t *d_pos, uint32_t max_seq, uint32_t Hkv, uint32_t Dh) {
  size_t total = (size_t)S * Hkv * Dh;
  if (total == 0) return GRETA_OK;
  GRETA_REQUIRE(kc && vc && nk && nv, "kv_update: null pointer");
  GRETA_REQUIRE(d_pos || pos + S <= max_seq, "kv_update: rows %u..%u exceed max_seq_len=%u", pos, pos + S, max_seq);
  kv_update_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((__half *)kc, (__half *)vc, nk, nv, S, pos,
                                                                                    d_pos, max_seq, Hkv, Dh);
  return launched("kv_update_kernel");
}

}  // extern "C"
