// Device-side body of the split decode attention (see attention.cu for the scheme), shared by the
// stand-alone kernel and by the persistent decode-step kernel.
#pragma once
#include <math.h>

#include "greta_common.cuh"

using namespace greta;

namespace {

constexpr int MAX_SPLITS = 32;

__device__ __forceinline__ uint4 ld_cg16(const void *p) {  // L2-coherent 128-bit load (no L1)
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}


template <typename KV, int DPL, bool CG>
__device__ __forceinline__ void load_row(const KV *p, float (&f)[DPL]) {
  if (sizeof(KV) == 2) {
#pragma unroll
    for (int v = 0; v < DPL / 8; ++v) {
      uint4 u = CG ? ld_cg16(reinterpret_cast<const uint8_t *>(p) + v * 16) : ld_stream(reinterpret_cast<const uint8_t *>(p) + v * 16);
      float2 a = h2_to_f2(u.x), b = h2_to_f2(u.y), c = h2_to_f2(u.z), d = h2_to_f2(u.w);
      f[8 * v + 0] = a.x; f[8 * v + 1] = a.y; f[8 * v + 2] = b.x; f[8 * v + 3] = b.y;
      f[8 * v + 4] = c.x; f[8 * v + 5] = c.y; f[8 * v + 6] = d.x; f[8 * v + 7] = d.y;
    }
  } else {
#pragma unroll
    for (int v = 0; v < DPL / 4; ++v) {
      uint4 u = CG ? ld_cg16(reinterpret_cast<const uint8_t *>(p) + v * 16) : ld_stream(reinterpret_cast<const uint8_t *>(p) + v * 16);
      f[4 * v + 0] = __uint_as_float(u.x); f[4 * v + 1] = __uint_as_float(u.y);
      f[4 * v + 2] = __uint_as_float(u.z); f[4 * v + 3] = __uint_as_float(u.w);
    }
  }
}

}  // namespace

namespace greta {
// Shared by every attention kernel of the library (one definition across the translation units).
struct AttnParams {
  const float *q;        // [nq][H][Dh]
  const void *kc, *vc;   // [Hkv][max_seq][Dh]
  float *o;              // [nq][H][Dh]
  const uint32_t *d_pos; // optional device position
  uint32_t len0;         // keys visible to query 0 when d_pos == NULL (query z sees len0 + z)
  uint32_t H, Hkv, max_seq;
  float scale;
  uint32_t splits;
  // Element strides of the K/V arrays: the cache [Hkv][max_seq][Dh] has head_stride = max_seq * Dh and row_stride = Dh;
  // the prompt-major arrays [S][Hkv][Dh] of the reference's prefill entry have head_stride = Dh, row_stride = Hkv * Dh.
  // 0 = the cache layout.  len_step: keys query z sees beyond query 0's (1 = causal, 0 = every query sees len0 keys).
  uint32_t head_stride, row_stride, len_step;
  // Batched decode: query z belongs to sequence z, whose cache starts seq_stride elements after sequence z - 1's and
  // whose position is d_pos[z * pos_stride].  Both 0 for a single sequence.
  size_t seq_stride;
  uint32_t pos_stride;
  uint32_t *counters;    // [H] zero on entry, left zero
  float *partial;        // [H][splits][Dh + 2]
};
}  // namespace greta

namespace {


// Merge (m2, l2, o2) into (m, l, o).
template <int DPL>
__device__ __forceinline__ void merge(float &m, float &l, float (&o)[DPL], float m2, float l2, const float (&o2)[DPL]) {
  float mn = fmaxf(m, m2);
  float c1 = (m == -INFINITY) ? 0.f : expf(m - mn);
  float c2 = (m2 == -INFINITY) ? 0.f : expf(m2 - mn);
  l = l * c1 + l2 * c2;
#pragma unroll
  for (int i = 0; i < DPL; ++i) o[i] = o[i] * c1 + o2[i] * c2;
  m = mn;
}

// Merges the per-lane-group running (max, sum, output slice) of all NW warps of the CTA.  On return thread
// tid < Dh holds the CTA's maximum, normaliser and unnormalised output for dim tid.
template <int DPL, int NW>
__device__ __forceinline__ void attn_merge_cta(float m, float l, float (&o)[DPL], float &fm, float &fl, float &fo) {
  constexpr int Dh = DPL * 8;
  __shared__ float sm_m[NW], sm_l[NW];
  __shared__ float sm_o[NW][Dh];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 7, grp = lane >> 3;
  // merge the four lane groups of the warp (same dims, different keys)
#pragma unroll
  for (int off = 8; off <= 16; off <<= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, off), l2 = __shfl_xor_sync(0xffffffffu, l, off), o2[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) o2[i] = __shfl_xor_sync(0xffffffffu, o[i], off);
    merge<DPL>(m, l, o, m2, l2, o2);
  }
  // merge warps through shared memory
  if (grp == 0) {
    if (sub == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < DPL; ++i) sm_o[warp][sub * DPL + i] = o[i];
  }
  __syncthreads();
  const int tid = threadIdx.x;
  fm = -INFINITY, fl = 0.f, fo = 0.f;  // thread tid < Dh owns output dim tid
  if (tid < Dh) {
#pragma unroll
    for (int w = 0; w < NW; ++w) fm = fmaxf(fm, sm_m[w]);
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      float c = (sm_m[w] == -INFINITY) ? 0.f : expf(sm_m[w] - fm);
      fl += sm_l[w] * c;
      fo += sm_o[w][tid] * c;
    }
  }
}

// Online-softmax attention of one query head over keys [k0, k1), by the NW warps of the calling CTA (all of
// them must call).  On return thread tid < Dh holds, for output dim tid, the CTA's running maximum, normaliser
// and unnormalised output.  CG: read K/V through L2 only (needed when the newest cache row was written
// earlier in the same launch).
template <typename KV, int DPL, int NW, bool CG>
__device__ __forceinline__ void attn_partial(const AttnParams &p, const uint32_t k0, const uint32_t k1, const uint32_t head, const uint32_t qi,
                                             float &fm, float &fl, float &fo) {
  constexpr int ATT_WARPS = NW;
  constexpr int Dh = DPL * 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 7, grp = lane >> 3;  // 8 lanes per key, 4 keys per warp step
  const uint32_t kvh = head / (p.H / p.Hkv);

  const size_t hs = p.head_stride ? p.head_stride : (size_t)p.max_seq * Dh, rs = p.row_stride ? p.row_stride : Dh;
  const KV *kbase = reinterpret_cast<const KV *>(p.kc) + (size_t)qi * p.seq_stride + (size_t)kvh * hs + sub * DPL;
  const KV *vbase = reinterpret_cast<const KV *>(p.vc) + (size_t)qi * p.seq_stride + (size_t)kvh * hs + sub * DPL;

  float qv[DPL];
  {
    const float *qp = p.q + ((size_t)qi * p.H + head) * Dh + sub * DPL;
#pragma unroll
    for (int i = 0; i < DPL; i += 4) {
      float4 t = __ldcg(reinterpret_cast<const float4 *>(qp + i));
      qv[i] = t.x * p.scale; qv[i + 1] = t.y * p.scale; qv[i + 2] = t.z * p.scale; qv[i + 3] = t.w * p.scale;
    }
  }

  float m = -INFINITY, l = 0.f, o[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) o[i] = 0.f;

  // warp step j covers keys tw .. tw+3 and tw+16 .. tw+19 (two steps in flight), one key per lane group
  for (uint32_t tw = k0 + 4 * warp; tw < k1; tw += 4 * ATT_WARPS * 2) {
    const uint32_t ta = tw + grp, tb = tw + 4 * ATT_WARPS + grp;
    const bool va = ta < k1, vb = tb < k1;
    float ka[DPL], kb[DPL], xa[DPL], xb[DPL];
    if (va) { load_row<KV, DPL, CG>(kbase + (size_t)ta * rs, ka); load_row<KV, DPL, CG>(vbase + (size_t)ta * rs, xa); }
    if (vb) { load_row<KV, DPL, CG>(kbase + (size_t)tb * rs, kb); load_row<KV, DPL, CG>(vbase + (size_t)tb * rs, xb); }
    float sa = 0.f, sb = 0.f;
    if (va) {
#pragma unroll
      for (int i = 0; i < DPL; ++i) sa = fmaf(qv[i], ka[i], sa);
    }
    if (vb) {
#pragma unroll
      for (int i = 0; i < DPL; ++i) sb = fmaf(qv[i], kb[i], sb);
    }
    // reduce across the 8 lanes that share a key (all lanes take part in the shuffles)
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) {
      sa += __shfl_xor_sync(0xffffffffu, sa, off);
      sb += __shfl_xor_sync(0xffffffffu, sb, off);
    }
    if (va) {
      float mn = fmaxf(m, sa), c = expf(m - mn), pe = expf(sa - mn);
      l = l * c + pe;
#pragma unroll
      for (int i = 0; i < DPL; ++i) o[i] = fmaf(pe, xa[i], o[i] * c);
      m = mn;
    }
    if (vb) {
      float mn = fmaxf(m, sb), c = expf(m - mn), pe = expf(sb - mn);
      l = l * c + pe;
#pragma unroll
      for (int i = 0; i < DPL; ++i) o[i] = fmaf(pe, xb[i], o[i] * c);
      m = mn;
    }
  }

  attn_merge_cta<DPL, NW>(m, l, o, fm, fl, fo);
}

// The same for an fp16 cache, with the K and V rows travelling global -> shared by cp.async in tiles of 64
// keys, three tiles in flight: every byte of the CTA's share (up to 192 keys) is requested before the first
// one is used, so a CTA pays one HBM latency where the register-staged loop pays one per 64 keys.
constexpr int ATT_TILE_KEYS = 64, ATT_TILES_IN_FLIGHT = 3;
template <int DPL>
constexpr size_t attn_stage_bytes() { return (size_t)ATT_TILES_IN_FLIGHT * ATT_TILE_KEYS * DPL * 8 * 2 * 2; }

template <int DPL, int NW>
__device__ __forceinline__ void attn_partial_staged(const AttnParams &p, const uint32_t k0, const uint32_t k1, const uint32_t head,
                                                    const uint32_t qi, uint8_t *stage, float &fm, float &fl, float &fo) {
  constexpr int Dh = DPL * 8, ROW = Dh * 2, TK = ATT_TILE_KEYS, NT = ATT_TILES_IN_FLIGHT, TILE_BYTES = TK * ROW * 2;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane & 7, grp = lane >> 3;
  const uint32_t kvh = head / (p.H / p.Hkv);
  const uint8_t *kg = reinterpret_cast<const uint8_t *>(p.kc) + ((size_t)qi * p.seq_stride + (size_t)kvh * p.max_seq * Dh) * 2;
  const uint8_t *vg = reinterpret_cast<const uint8_t *>(p.vc) + ((size_t)qi * p.seq_stride + (size_t)kvh * p.max_seq * Dh) * 2;
  const uint32_t n_tiles = k1 > k0 ? (k1 - k0 + TK - 1) / TK : 0;
  auto issue = [&](uint32_t t) {
    if (t < n_tiles) {
      const uint32_t key0 = k0 + t * TK, nk = min((uint32_t)TK, k1 - key0);
      uint8_t *slot = stage + (t % NT) * TILE_BYTES;
      for (uint32_t piece = tid; piece < nk * 32; piece += NW * 32) {  // 16 K pieces and 16 V pieces of 16 bytes per key
        const uint32_t row = piece >> 5, c = piece & 31, is_v = c >> 4, cc = c & 15;
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
    const float *qp = p.q + ((size_t)qi * p.H + head) * Dh + sub * DPL;
#pragma unroll
    for (int i = 0; i < DPL; i += 4) {
      float4 t = __ldcg(reinterpret_cast<const float4 *>(qp + i));
      qv[i] = t.x * p.scale; qv[i + 1] = t.y * p.scale; qv[i + 2] = t.z * p.scale; qv[i + 3] = t.w * p.scale;
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
    for (uint32_t base = 4 * warp; base < nk; base += 4 * NW) {  // one key per lane group and step
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
  attn_merge_cta<DPL, NW>(m, l, o, fm, fl, fo);
}

// One (query qi, head, split) work item: the CTA's share of the keys, then the merge of the splits through
// the scratch buffer (every CTA publishes its partial result and takes a ticket; the last one merges).
template <typename KV, int DPL, int NW, bool CG>
__device__ void attn_body(const AttnParams &p, const uint32_t split, const uint32_t head, const uint32_t qi) {
  constexpr int Dh = DPL * 8;
  __shared__ uint32_t sm_last;
  const uint32_t L = min((p.d_pos ? __ldcg(p.d_pos + qi * p.pos_stride) + 1 : p.len0) + qi * p.len_step, p.max_seq);  // never past the cache
  const uint32_t chunk = (L + p.splits - 1) / p.splits;
  const uint32_t k0 = split * chunk, k1 = min(L, k0 + chunk);
  const int tid = threadIdx.x;
  float fm, fl, fo;
  attn_partial<KV, DPL, NW, CG>(p, k0, k1, head, qi, fm, fl, fo);
  float *out = p.o + ((size_t)qi * p.H + head) * Dh;
  if (p.splits == 1) {
    if (tid < Dh) out[tid] = fo / fl;
    return;
  }
  // publish the partial result, take a ticket; the last CTA of this head merges all splits
  const uint32_t slot = qi * p.H + head;  // one ticket and one set of partials per query and head
  float *mine = p.partial + ((size_t)slot * p.splits + split) * (Dh + 2);
  if (tid < Dh) mine[2 + tid] = fo;
  if (tid == 0) { mine[0] = fm; mine[1] = fl; }
  __threadfence();
  __syncthreads();
  if (tid == 0) sm_last = (atomicAdd(&p.counters[slot], 1u) == p.splits - 1) ? 1u : 0u;
  __syncthreads();
  if (!sm_last) return;
  __threadfence();
  if (tid < Dh) {
    const float *ph = p.partial + (size_t)slot * p.splits * (Dh + 2);
    float gm = -INFINITY;
    for (uint32_t s = 0; s < p.splits; ++s) gm = fmaxf(gm, __ldcg(ph + (size_t)s * (Dh + 2)));
    float gl = 0.f, go = 0.f;
    for (uint32_t s = 0; s < p.splits; ++s) {
      const float *ps = ph + (size_t)s * (Dh + 2);
      float ms = __ldcg(ps);
      float c = (ms == -INFINITY) ? 0.f : expf(ms - gm);
      gl += __ldcg(ps + 1) * c;
      go += __ldcg(ps + 2 + tid) * c;
    }
    out[tid] = go / gl;
  }
  if (tid == 0) p.counters[slot] = 0;  // ready for the next call on this stream
}

}  // namespace
