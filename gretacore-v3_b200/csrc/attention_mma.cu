// Attention on the tensor cores (mma.sync m16n8k16, fp16 operands, fp32 accumulation) over the fp16 KV cache, for the two
// places where one KV row meets several queries:
//   * grouped-query batched decode: the 2..16 query heads that share a KV head are the 16 rows of the matrix instruction,
//     so a key / value row is read from HBM once, multiplied once, for all of them (attn_mma_decode_kernel);
//   * causal prefill: 16 consecutive prompt positions of one head are the rows; a CTA of four warps (64 positions) stages
//     each K / V tile once in shared memory (attn_mma_prefill_kernel).
// Scores S = Q K^T: Q is the row operand, split into two fp16 values per element (hi = half(q * scale), lo = half(q *
// scale - hi)) so the product keeps fp32 precision; K rows come out of shared memory with ldmatrix as the column operand.
// Softmax is the online form in fp32, per row, in the accumulator layout.  O += P V: the probabilities, again as fp16
// pairs, are already laid out as the row operand (the accumulator layout of S is the operand layout of P); V rows come
// out of shared memory with ldmatrix.trans.  K / V tiles of 64 keys travel global -> shared by cp.async, three in flight,
// rows padded by 16 bytes so that the ldmatrix row addresses fall into different banks.
#include <cooperative_groups.h>
#include <math.h>

#include <algorithm>

#include "attention_device.cuh"

namespace {

namespace cg = cooperative_groups;

constexpr int MMA_TK = 64, MMA_NT = 3, MMA_WARPS = 4;
template <int DH>
__host__ __device__ constexpr int mma_rowp() { return DH * 2 + 16; }
template <int DH>
__host__ __device__ constexpr size_t mma_stage_bytes() { return (size_t)MMA_NT * MMA_TK * mma_rowp<DH>() * 2; }

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void *p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void *p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}
// (a, b) as fp16 pairs: hi = half(x), lo = half(x - hi).
__device__ __forceinline__ void split2(float a, float b, uint32_t &hi, uint32_t &lo) {
  const __half ha = __float2half_rn(a), hb = __float2half_rn(b);
  hi = (uint32_t)__half_as_ushort(ha) | ((uint32_t)__half_as_ushort(hb) << 16);
  lo = pack2(a - __half2float(ha), b - __half2float(hb));
}

// Rows of the matrix instruction held by one warp: the query fragments (hi / lo), the running maximum and normaliser
// of rows g and g + 8, the unnormalised output.
template <int DH>
struct RowState {
  uint32_t qh[DH / 16][4], ql[DH / 16][4];
  float m[2], l[2];
  float o[DH / 8][4];
};

// Loads and splits the two query rows of this thread (either may be absent: zeros).
template <int DH>
__device__ __forceinline__ void load_queries(RowState<DH> &st, const float *q0, const float *q1, float scale, int t) {
#pragma unroll
  for (int ks = 0; ks < DH / 16; ++ks) {
    float2 a = make_float2(0.f, 0.f), b = a, c = a, d = a;
    if (q0) {
      a = __ldcg(reinterpret_cast<const float2 *>(q0 + ks * 16 + 2 * t));
      c = __ldcg(reinterpret_cast<const float2 *>(q0 + ks * 16 + 8 + 2 * t));
    }
    if (q1) {
      b = __ldcg(reinterpret_cast<const float2 *>(q1 + ks * 16 + 2 * t));
      d = __ldcg(reinterpret_cast<const float2 *>(q1 + ks * 16 + 8 + 2 * t));
    }
    split2(a.x * scale, a.y * scale, st.qh[ks][0], st.ql[ks][0]);
    split2(b.x * scale, b.y * scale, st.qh[ks][1], st.ql[ks][1]);
    split2(c.x * scale, c.y * scale, st.qh[ks][2], st.ql[ks][2]);
    split2(d.x * scale, d.y * scale, st.qh[ks][3], st.ql[ks][3]);
  }
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;
#pragma unroll
  for (int dn = 0; dn < DH / 8; ++dn)
#pragma unroll
    for (int j = 0; j < 4; ++j) st.o[dn][j] = 0.f;
}

// One group of 16 keys (rows `krow` .. krow + 15 of the staged tile, absolute indices kabs ..) against the warp's 16 rows.
// lim0 / lim1: first key index rows g / g + 8 must not see.
template <int DH>
__device__ __forceinline__ void attend16(RowState<DH> &st, const uint8_t *ktile, const uint8_t *vtile, uint32_t krow, uint32_t kabs, uint32_t lim0,
                                         uint32_t lim1, int lane) {
  constexpr int ROWP = mma_rowp<DH>();
  const int t = lane & 3, mat = lane >> 3, r8 = lane & 7;
  float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  const uint8_t *kaddr = ktile + (size_t)(krow + (mat >> 1) * 8 + r8) * ROWP + (mat & 1) * 16;
#pragma unroll
  for (int ks = 0; ks < DH / 16; ++ks) {
    uint32_t kb[4];
    ldsm_x4(kb, kaddr + ks * 32);
    mma16816(s[0], st.qh[ks], kb[0], kb[1]);
    mma16816(s[1], st.qh[ks], kb[2], kb[3]);
    mma16816(s[0], st.ql[ks], kb[0], kb[1]);
    mma16816(s[1], st.ql[ks], kb[2], kb[3]);
  }
  // mask, row maxima
  float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint32_t key = kabs + nt * 8 + 2 * t + c;
      if (key >= lim0) s[nt][c] = -INFINITY;
      if (key >= lim1) s[nt][2 + c] = -INFINITY;
      tm0 = fmaxf(tm0, s[nt][c]);
      tm1 = fmaxf(tm1, s[nt][2 + c]);
    }
  tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1));
  tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
  tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1));
  tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
  const float mn0 = fmaxf(st.m[0], tm0), mn1 = fmaxf(st.m[1], tm1);
  const float c0 = (mn0 == -INFINITY) ? 1.f : expf(st.m[0] - mn0), c1 = (mn1 == -INFINITY) ? 1.f : expf(st.m[1] - mn1);
  const float b0 = (mn0 == -INFINITY) ? 0.f : mn0, b1 = (mn1 == -INFINITY) ? 0.f : mn1;  // exp(-inf - 0) = 0 for masked scores
  float p[2][4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    p[nt][0] = expf(s[nt][0] - b0);
    p[nt][1] = expf(s[nt][1] - b0);
    p[nt][2] = expf(s[nt][2] - b1);
    p[nt][3] = expf(s[nt][3] - b1);
  }
  st.l[0] = st.l[0] * c0 + (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
  st.l[1] = st.l[1] * c1 + (p[0][2] + p[0][3] + p[1][2] + p[1][3]);
  st.m[0] = mn0;
  st.m[1] = mn1;
  uint32_t ph[4], pl[4];  // the probabilities as the row operand of P V: keys 2t, 2t+1 (a0, a1) and 8+2t, 8+2t+1 (a2, a3)
  split2(p[0][0], p[0][1], ph[0], pl[0]);
  split2(p[0][2], p[0][3], ph[1], pl[1]);
  split2(p[1][0], p[1][1], ph[2], pl[2]);
  split2(p[1][2], p[1][3], ph[3], pl[3]);
  const uint8_t *vaddr = vtile + (size_t)(krow + (mat & 1) * 8 + r8) * ROWP + (mat >> 1) * 16;
#pragma unroll
  for (int dn = 0; dn < DH / 8; dn += 2) {
    uint32_t vb[4];
    ldsm_x4_trans(vb, vaddr + dn * 16);
    st.o[dn][0] *= c0; st.o[dn][1] *= c0; st.o[dn][2] *= c1; st.o[dn][3] *= c1;
    st.o[dn + 1][0] *= c0; st.o[dn + 1][1] *= c0; st.o[dn + 1][2] *= c1; st.o[dn + 1][3] *= c1;
    mma16816(st.o[dn], ph, vb[0], vb[1]);
    mma16816(st.o[dn + 1], ph, vb[2], vb[3]);
    mma16816(st.o[dn], pl, vb[0], vb[1]);
    mma16816(st.o[dn + 1], pl, vb[2], vb[3]);
  }
}

// Requests tile `t` (keys key0 + 64 t ..) of the range [key0, k1) into its ring slot; all `nthreads` threads take part.
template <int DH>
__device__ __forceinline__ void issue_tile(uint8_t *stage, const uint8_t *kg, const uint8_t *vg, uint32_t key0, uint32_t k1, uint32_t t, uint32_t n_tiles,
                                           int tid, int nthreads) {
  constexpr int ROW = DH * 2, ROWP = mma_rowp<DH>(), PPK = ROW / 16;  // 16-byte pieces per key and per K or V row
  if (t < n_tiles) {
    const uint32_t kt0 = key0 + t * MMA_TK, nk = min((uint32_t)MMA_TK, k1 - kt0);
    uint8_t *slot = stage + (size_t)(t % MMA_NT) * (MMA_TK * ROWP * 2);
    for (uint32_t piece = tid; piece < nk * 2 * PPK; piece += nthreads) {
      const uint32_t row = piece / (2 * PPK), c = piece % (2 * PPK), is_v = c / PPK, cc = c % PPK;
      const uint8_t *src = (is_v ? vg : kg) + (size_t)(kt0 + row) * ROW + cc * 16;
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(slot + is_v * (MMA_TK * ROWP) + row * ROWP + cc * 16);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    }
    // A last group of 16 keys that is only partly there is still multiplied as a whole (its surplus scores are masked):
    // its surplus rows must hold numbers, not whatever the memory held (0 x NaN is NaN).  The stores become visible with
    // the barrier that also publishes the copies.
    const uint32_t pad_rows = ((nk + 15) & ~15u) - nk;
    for (uint32_t piece = tid; piece < pad_rows * 2 * PPK; piece += nthreads) {
      const uint32_t row = nk + piece / (2 * PPK), c = piece % (2 * PPK), is_v = c / PPK, cc = c % PPK;
      *reinterpret_cast<uint4 *>(slot + is_v * (MMA_TK * ROWP) + row * ROWP + cc * 16) = make_uint4(0, 0, 0, 0);
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// ------------------------------------------------------------------ grouped-query batched decode
// grid (splits, Hkv, sequences), cluster over the splits; 4 warps, each takes 16 of the 64 keys of every staged tile.
template <int DH>
__global__ void __launch_bounds__(MMA_WARPS * 32) attn_mma_decode_kernel(const AttnParams p, const uint32_t NG) {
  constexpr int ROWP = mma_rowp<DH>();
  extern __shared__ __align__(16) uint8_t stage[];
  __shared__ float res[16][DH + 2];  // per query head of the group: maximum, normaliser, unnormalised output over this CTA's keys
  cg::cluster_group cluster = cg::this_cluster();
  pdl_launch_dependents();
  pdl_wait();  // q, the positions and the newest cache rows come from the previous kernel
  const uint32_t nsplit = gridDim.x, split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const uint32_t L = min(__ldcg(p.d_pos + seq * p.pos_stride) + 1, p.max_seq);
  const uint32_t chunk = (L + nsplit - 1) / nsplit;
  const uint32_t k0 = min(split * chunk, L), k1 = min(L, k0 + chunk);
  const uint8_t *kg = reinterpret_cast<const uint8_t *>(p.kc) + ((size_t)seq * p.seq_stride + (size_t)kvh * p.max_seq * DH) * 2;
  const uint8_t *vg = reinterpret_cast<const uint8_t *>(p.vc) + ((size_t)seq * p.seq_stride + (size_t)kvh * p.max_seq * DH) * 2;
  const uint32_t n_tiles = k1 > k0 ? (k1 - k0 + MMA_TK - 1) / MMA_TK : 0;
#pragma unroll
  for (int i = 0; i < MMA_NT; ++i) issue_tile<DH>(stage, kg, vg, k0, k1, i, n_tiles, tid, MMA_WARPS * 32);

  RowState<DH> st;
  {
    const float *qb = p.q + ((size_t)seq * p.H + (size_t)kvh * NG) * DH;
    load_queries<DH>(st, (uint32_t)g < NG ? qb + (size_t)g * DH : nullptr, (uint32_t)(g + 8) < NG ? qb + (size_t)(g + 8) * DH : nullptr, p.scale, t);
  }
  for (uint32_t ti = 0; ti < n_tiles; ++ti) {
    asm volatile("cp.async.wait_group %0;" ::"n"(MMA_NT - 1) : "memory");
    __syncthreads();  // every thread's pieces of tile ti have landed
    const uint32_t kt0 = k0 + ti * MMA_TK, nk = min((uint32_t)MMA_TK, k1 - kt0);
    const uint8_t *slot = stage + (size_t)(ti % MMA_NT) * (MMA_TK * ROWP * 2);
    if ((uint32_t)warp * 16 < nk) attend16<DH>(st, slot, slot + MMA_TK * ROWP, warp * 16, kt0 + warp * 16, k1, k1, lane);
    __syncthreads();  // the slot is free again
    issue_tile<DH>(stage, kg, vg, k0, k1, ti + MMA_NT, n_tiles, tid, MMA_WARPS * 32);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  // ---- merge the four warps (different keys, same rows) through the (now idle) staging memory
  st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 1);
  st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 2);
  st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 1);
  st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 2);
  float *wres = reinterpret_cast<float *>(stage) + (size_t)warp * 16 * (DH + 2);  // [16 rows][DH + 2]
  if (t == 0) {
    wres[g * (DH + 2)] = st.m[0];
    wres[g * (DH + 2) + 1] = st.l[0];
    wres[(g + 8) * (DH + 2)] = st.m[1];
    wres[(g + 8) * (DH + 2) + 1] = st.l[1];
  }
#pragma unroll
  for (int dn = 0; dn < DH / 8; ++dn) {
    *reinterpret_cast<float2 *>(&wres[g * (DH + 2) + 2 + dn * 8 + 2 * t]) = make_float2(st.o[dn][0], st.o[dn][1]);
    *reinterpret_cast<float2 *>(&wres[(g + 8) * (DH + 2) + 2 + dn * 8 + 2 * t]) = make_float2(st.o[dn][2], st.o[dn][3]);
  }
  __syncthreads();
  const float *all = reinterpret_cast<const float *>(stage);
  for (uint32_t idx = tid; idx < NG * DH; idx += MMA_WARPS * 32) {
    const uint32_t r = idx / DH, d = idx % DH;
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < MMA_WARPS; ++w) gm = fmaxf(gm, all[((size_t)w * 16 + r) * (DH + 2)]);
    float gl = 0.f, go = 0.f;
#pragma unroll
    for (int w = 0; w < MMA_WARPS; ++w) {  // fixed order
      const float *rp = all + ((size_t)w * 16 + r) * (DH + 2);
      const float c = (rp[0] == -INFINITY) ? 0.f : expf(rp[0] - gm);
      gl += rp[1] * c;
      go += rp[2 + d] * c;
    }
    if (nsplit == 1) {
      p.o[((size_t)seq * p.H + (size_t)kvh * NG + r) * DH + d] = go / gl;
    } else {
      res[r][2 + d] = go;
      if (d == 0) {
        res[r][0] = gm;
        res[r][1] = gl;
      }
    }
  }
  if (nsplit == 1) return;
  cluster.sync();
  if (split == 0) {
    for (uint32_t idx = tid; idx < NG * DH; idx += MMA_WARPS * 32) {
      const uint32_t r = idx / DH, d = idx % DH;
      float gm = -INFINITY;
      for (uint32_t s = 0; s < nsplit; ++s) gm = fmaxf(gm, cluster.map_shared_rank(&res[r][0], s)[0]);
      float gl = 0.f, go = 0.f;
      for (uint32_t s = 0; s < nsplit; ++s) {  // rank order: the result does not depend on which CTA finished first
        const float *rp = cluster.map_shared_rank(&res[r][0], s);
        const float c = (rp[0] == -INFINITY) ? 0.f : expf(rp[0] - gm);
        gl += rp[1] * c;
        go += rp[2 + d] * c;
      }
      p.o[((size_t)seq * p.H + (size_t)kvh * NG + r) * DH + d] = go / gl;
    }
  }
  cluster.sync();  // a CTA's shared memory must outlive the reads of CTA 0
}

// ------------------------------------------------------------------ causal prefill
// grid (query blocks of 64, heads); warp w owns queries 64 b + 16 w .. + 15 of the chunk; query s of the chunk sits at
// position pos0 + s and sees keys 0 .. pos0 + s of the cache.
template <int DH>
__global__ void __launch_bounds__(MMA_WARPS * 32) attn_mma_prefill_kernel(const AttnParams p, const uint32_t S, const uint32_t pos0) {
  constexpr int ROWP = mma_rowp<DH>();
  extern __shared__ __align__(16) uint8_t stage[];
  const uint32_t qb = blockIdx.x, head = blockIdx.y, kvh = head / (p.H / p.Hkv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const uint8_t *kg = reinterpret_cast<const uint8_t *>(p.kc) + (size_t)kvh * p.max_seq * DH * 2;
  const uint8_t *vg = reinterpret_cast<const uint8_t *>(p.vc) + (size_t)kvh * p.max_seq * DH * 2;
  const uint32_t q_first = qb * 64, q_last = min(S, q_first + 64) - 1;  // this CTA's queries (chunk indices)
  const uint32_t k1 = pos0 + q_last + 1;                                 // keys the last query sees
  const uint32_t n_tiles = (k1 + MMA_TK - 1) / MMA_TK;
#pragma unroll
  for (int i = 0; i < MMA_NT; ++i) issue_tile<DH>(stage, kg, vg, 0, k1, i, n_tiles, tid, MMA_WARPS * 32);

  const uint32_t s0 = q_first + warp * 16 + g, s1 = s0 + 8;  // this thread's two queries
  RowState<DH> st;
  load_queries<DH>(st, s0 < S ? p.q + ((size_t)s0 * p.H + head) * DH : nullptr, s1 < S ? p.q + ((size_t)s1 * p.H + head) * DH : nullptr, p.scale, t);
  const uint32_t lim0 = s0 < S ? pos0 + s0 + 1 : 0, lim1 = s1 < S ? pos0 + s1 + 1 : 0;
  const uint32_t warp_lim = min(k1, pos0 + q_first + warp * 16 + 16);  // no query of this warp sees keys from here on
  for (uint32_t ti = 0; ti < n_tiles; ++ti) {
    asm volatile("cp.async.wait_group %0;" ::"n"(MMA_NT - 1) : "memory");
    __syncthreads();
    const uint32_t kt0 = ti * MMA_TK, nk = min((uint32_t)MMA_TK, k1 - kt0);
    const uint8_t *slot = stage + (size_t)(ti % MMA_NT) * (MMA_TK * ROWP * 2);
    for (uint32_t kk = 0; kk < nk && kt0 + kk < warp_lim; kk += 16) attend16<DH>(st, slot, slot + MMA_TK * ROWP, kk, kt0 + kk, lim0, lim1, lane);
    __syncthreads();
    issue_tile<DH>(stage, kg, vg, 0, k1, ti + MMA_NT, n_tiles, tid, MMA_WARPS * 32);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 1);
  st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 2);
  st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 1);
  st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 2);
  const float i0 = 1.f / st.l[0], i1 = 1.f / st.l[1];
#pragma unroll
  for (int dn = 0; dn < DH / 8; ++dn) {
    if (s0 < S) *reinterpret_cast<float2 *>(p.o + ((size_t)s0 * p.H + head) * DH + dn * 8 + 2 * t) = make_float2(st.o[dn][0] * i0, st.o[dn][1] * i0);
    if (s1 < S) *reinterpret_cast<float2 *>(p.o + ((size_t)s1 * p.H + head) * DH + dn * 8 + 2 * t) = make_float2(st.o[dn][2] * i1, st.o[dn][3] * i1);
  }
}

template <typename Kern>
int ensure_mma_smem(Kern kern, size_t smem, bool (&done)[64]) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !done[dev]) {
    GRETA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    GRETA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
    done[dev] = true;
  }
  return GRETA_OK;
}

}  // namespace

namespace greta {

// Grouped-query batched decode on the tensor cores; ng = query heads per KV head (2..16).
int attn_mma_decode(cudaStream_t stream, const AttnParams &p, uint32_t batch, uint32_t nsplit, uint32_t ng, uint32_t Dh) {
  dim3 grid(nsplit, p.Hkv, batch);
  if (Dh == 128) {
    static bool done[64] = {};
    if (int rc = ensure_mma_smem(attn_mma_decode_kernel<128>, mma_stage_bytes<128>(), done)) return rc;
    GRETA_CUDA_TRY(launch_pdl_cluster(attn_mma_decode_kernel<128>, grid, dim3(MMA_WARPS * 32), nsplit, mma_stage_bytes<128>(), stream, p, ng));
  } else {
    static bool done[64] = {};
    if (int rc = ensure_mma_smem(attn_mma_decode_kernel<64>, mma_stage_bytes<64>(), done)) return rc;
    GRETA_CUDA_TRY(launch_pdl_cluster(attn_mma_decode_kernel<64>, grid, dim3(MMA_WARPS * 32), nsplit, mma_stage_bytes<64>(), stream, p, ng));
  }
  return launched("attn_mma_decode_kernel");
}

// Causal prefill of S queries at positions pos0 .. against the fp16 cache.
int attn_mma_prefill(cudaStream_t stream, const AttnParams &p, uint32_t S, uint32_t pos0, uint32_t Dh) {
  dim3 grid((S + 63) / 64, p.H);
  if (Dh == 128) {
    static bool done[64] = {};
    if (int rc = ensure_mma_smem(attn_mma_prefill_kernel<128>, mma_stage_bytes<128>(), done)) return rc;
    attn_mma_prefill_kernel<128><<<grid, MMA_WARPS * 32, mma_stage_bytes<128>(), stream>>>(p, S, pos0);
  } else {
    static bool done[64] = {};
    if (int rc = ensure_mma_smem(attn_mma_prefill_kernel<64>, mma_stage_bytes<64>(), done)) return rc;
    attn_mma_prefill_kernel<64><<<grid, MMA_WARPS * 32, mma_stage_bytes<64>(), stream>>>(p, S, pos0);
  }
  return launched("attn_mma_prefill_kernel");
}

}  // namespace greta
