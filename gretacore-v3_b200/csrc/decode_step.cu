// All decoder layers of one batch-1 decode step in a single persistent launch.
//
// Launching the five per-layer operators as separate kernels costs ~4 us of launch, activation
// staging and drain per kernel during which HBM sits idle - as much as the memory time of the
// kernels themselves at batch 1.  Here one CTA per SM stays resident for the whole step:
//   * the layer sequence (QKV+RoPE+KV write, attention, O-projection+residual, gate/up+SwiGLU,
//     down-projection+residual) runs as phases separated by a grid-wide barrier (an arrival
//     counter in global memory; the wait is bounded and raises an error flag instead of hanging);
//   * each warp's cp.async weight ring is never drained between phases: when a warp has requested
//     the last cell of its share of one projection it goes straight on to its share of the next
//     one, so the weight stream keeps flowing through barriers, attention and activation staging;
//   * activations move between phases through L2 (loads that bypass L1, which is not coherent
//     across SMs); the token embedding is fetched by every CTA at the start.
// The arithmetic is that of gemv.cu / attention.cu (same device functions), so results are
// bit-identical to the operator-by-operator path.
#include <algorithm>
#include <cstdlib>
#include <vector>

#include "attention_device.cuh"
#include "gemv_device.cuh"

namespace {

constexpr int R = 4;  // rows per group in every projection phase
constexpr long long BARRIER_LIMIT_CYCLES = 4000000000ll;
constexpr size_t DYN_SMEM_LIMIT = 208 * 1024;  // the attention phase keeps ~13 KB of static shared memory

struct LayerPlan {
  GemvParams qkv, wo, ffn, down;
  AttnParams attn;
};

struct StepPlan {
  const LayerPlan *layers;
  uint32_t num_layers;
  uint32_t stages;     // ring depth
  uint32_t xs_bytes;   // bytes reserved for staged activations (largest K)
  uint32_t slots;      // partial-sum slots per warp
  uint32_t head_dim;
  // embedding of the token to decode
  const __half *embed;
  const int32_t *d_token;
  float *x;
  uint32_t dim, vocab;
  // grid barrier state
  unsigned long long *bar;
  uint32_t *gen;
  int *err;
  long long *trace;  // [5 phases][5 marks] clock64 stamps of CTA 0 in layer 1 (phase start, staged, consumed, epilogue done, barrier passed)
};

struct Geom {
  uint32_t nb, C, g0, g1, T, c0, c1;
};
__device__ __forceinline__ Geom geom_of(const GemvParams &P, int warp) {
  Geom g;
  g.nb = P.K / 32;
  g.C = (g.nb + 31) / 32;
  g.g0 = (uint32_t)((uint64_t)blockIdx.x * P.groups / gridDim.x);
  g.g1 = (uint32_t)((uint64_t)(blockIdx.x + 1) * P.groups / gridDim.x);
  g.T = (g.g1 - g.g0) * g.C;
  g.c0 = (uint32_t)((uint64_t)warp * g.T / WARPS);
  g.c1 = (uint32_t)((uint64_t)(warp + 1) * g.T / WARPS);
  return g;
}

__device__ __forceinline__ const GemvParams *gemv_phase(const LayerPlan *layers, uint32_t gi) {
  const LayerPlan &L = layers[gi >> 2];
  switch (gi & 3) {
    case 0: return &L.qkv;
    case 1: return &L.wo;
    case 2: return &L.ffn;
    default: return &L.down;
  }
}
__device__ __forceinline__ bool resolve_rt(uint32_t gi, const GemvParams &P, uint32_t grp, int slot, int *mat, uint32_t *row) {
  switch (gi & 3) {
    case 0: return resolve<EPI_QKV, R>(P, grp, slot, mat, row);
    case 2: return resolve<EPI_SWIGLU, R>(P, grp, slot, mat, row);
    default: return resolve<EPI_RESIDUAL, R>(P, grp, slot, mat, row);
  }
}

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// All CTAs arrive, then wait until `target` arrivals have been counted.  Returns false when the step is
// being abandoned (a wait ran out somewhere): the caller then skips the remaining work.
__device__ __forceinline__ bool grid_barrier(const StepPlan &plan, unsigned long long target, int code) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(plan.bar, 1ull);
    const long long t0 = clock64();
    while (ld_acquire_u64(plan.bar) < target) {
      if (*reinterpret_cast<volatile int *>(plan.err)) break;
      if (clock64() - t0 > BARRIER_LIMIT_CYCLES) {
        atomicCAS(plan.err, 0, code);
        break;
      }
    }
    __threadfence();
  }
  __syncthreads();
  return *reinterpret_cast<volatile int *>(plan.err) == 0;
}

template <int FMT>
__global__ void __launch_bounds__(THREADS, 1) decode_layers_kernel(const StepPlan plan) {
  using F = Fmt<FMT>;
  constexpr int QV = F::QV, PB = QV * 16;
  constexpr int SCALE_ROW = 32 * F::SCALE_BYTES;
  constexpr int STAGE_BYTES = R * (32 * PB + SCALE_ROW);
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float red[32];
  __shared__ uint32_t s_gen;
  __shared__ float2 rope_cs[64];  // rotation (cos, sin) per pair index at this step's position: the same for every layer

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t D = plan.stages;
  uint8_t *ring = smem + plan.xs_bytes + (size_t)warp * D * STAGE_BYTES;
  float *part = reinterpret_cast<float *>(smem + plan.xs_bytes + (size_t)WARPS * D * STAGE_BYTES);
  const uint32_t n_gemv = plan.num_layers * 4;

  // ---- producer: walks this warp's cells of projection 0, 1, 2, ... without ever draining the ring ----
  uint32_t gi_p = 0;
  const GemvParams *pp = gemv_phase(plan.layers, 0);
  Geom gp = geom_of(*pp, warp);
  uint32_t pc = gp.c0, pg = gp.g0 + gp.c0 / gp.C, pk = gp.c0 % gp.C, pstage = 0;
  const uint8_t *qsrc[R];
  const uint8_t *dsrc = nullptr;
  const uint32_t dst_q = (uint32_t)lane * PB;
  const uint32_t dst_d = R * 32 * PB + (uint32_t)(lane >> 2) * SCALE_ROW + (uint32_t)(lane & 3) * 16;
  auto producer_rows = [&]() {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      int mat;
      uint32_t row;
      if (!resolve_rt(gi_p, *pp, pg, r, &mat, &row)) {
        mat = 0;
        row = 0;
      }
      qsrc[r] = pp->w[mat].qs + ((size_t)row * gp.nb + pk * 32 + lane) * PB;
      if ((lane >> 2) == r)
        dsrc = reinterpret_cast<const uint8_t *>(pp->w[mat].d) + ((size_t)row * d_row_stride(gp.nb) + pk * 32 + (lane & 3) * 8) * 2;
    }
  };
  if (pc < gp.c1) producer_rows();
  auto request = [&]() {
    while (pc >= gp.c1 && gi_p + 1 < n_gemv) {  // this warp's share of the projection is requested: on to the next one
      ++gi_p;
      pp = gemv_phase(plan.layers, gi_p);
      gp = geom_of(*pp, warp);
      pc = gp.c0;
      pg = gp.g0 + gp.c0 / gp.C;
      pk = gp.c0 % gp.C;
      if (pc < gp.c1) producer_rows();
    }
    if (pc < gp.c1) {
      uint8_t *st = ring + pstage * STAGE_BYTES;
      if (pk * 32 + lane < gp.nb) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
          for (int v = 0; v < QV; ++v) cp_async16(st + r * 32 * PB + dst_q + v * 16, qsrc[r] + v * 16);
        }
      }
      if (lane < 4 * R && pk * 32 + (lane & 3) * 8 < gp.nb) cp_async16(st + dst_d, dsrc);
      ++pc;
      if (++pk == gp.C) {
        pk = 0;
        ++pg;
        if (pc < gp.c1) producer_rows();
      } else {
#pragma unroll
        for (int r = 0; r < R; ++r) qsrc[r] += 32 * PB;
        dsrc += 64;
      }
    }
    cp_async_commit();
    pstage = (pstage + 1 == D) ? 0 : pstage + 1;
  };
  for (uint32_t s = 0; s + 1 < D; ++s) request();

  // ---- launch generation (for the barrier targets) and the token embedding ----
  if (threadIdx.x == 0) s_gen = *reinterpret_cast<volatile uint32_t *>(plan.gen);
  {
    const int32_t tok = __ldcg(plan.d_token);
    const bool valid = tok >= 0 && tok < (int32_t)plan.vocab;
    for (uint32_t d = threadIdx.x; d < plan.dim; d += THREADS)
      plan.x[d] = valid ? __half2float(plan.embed[(size_t)tok * plan.dim + d]) : 0.f;  // every CTA writes the same values
    __threadfence();
  }
  const uint32_t step_pos = __ldcg(plan.layers[0].qkv.d_pos);
  fill_rope_table(plan.layers[0].qkv, step_pos, rope_cs);
  __syncthreads();
  const unsigned long long bar_base = (unsigned long long)s_gen * (5ull * plan.num_layers) * gridDim.x;
  uint32_t n_bar = 0;
  bool ok = true;
  uint32_t cstage = 0;

  for (uint32_t layer = 0; layer < plan.num_layers && ok; ++layer) {
    const LayerPlan &L = plan.layers[layer];
    for (int sub = 0; sub < 5 && ok; ++sub) {
      const bool tr = layer == 1 && blockIdx.x == 0 && threadIdx.x == 0;
      if (tr) plan.trace[sub * 5 + 0] = clock64();
      if (sub == 1) {
        // ---------------- attention: one (head, split) item per CTA ----------------
        const AttnParams &A = L.attn;
        const uint32_t items = A.H * A.splits;
        if (blockIdx.x < items) {
          const uint32_t head = blockIdx.x / A.splits, split = blockIdx.x % A.splits;
          if (plan.head_dim == 128)
            attn_body<__half, 16, WARPS, true>(A, split, head, 0);
          else
            attn_body<__half, 8, WARPS, true>(A, split, head, 0);
        }
      } else {
        // ---------------- projection phase ----------------
        const uint32_t gi = layer * 4 + (sub == 0 ? 0 : sub - 1);
        const GemvParams &P = *gemv_phase(plan.layers, gi);
        const Geom g = geom_of(P, warp);
        stage_fixed_point<FMT, false>(P, 0, reinterpret_cast<uint32_t *>(smem), red);
        __syncthreads();
        if (tr) plan.trace[sub * 5 + 1] = clock64();
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.f;
        const uint32_t first_grp = g.g0 + g.c0 / g.C;
        uint32_t cg = first_grp, ck = g.c0 % g.C;
        const uint8_t *xrun = smem + (size_t)(ck * 32 + lane) * (XQ_WORDS * 4);
        for (uint32_t c = g.c0; c < g.c1; ++c) {
          cp_async_wait((int)D - 2);
          __syncwarp();
          const uint8_t *st = ring + cstage * STAGE_BYTES;
          cstage = (cstage + 1 == D) ? 0 : cstage + 1;
          const bool live = ck * 32 + lane < g.nb;
          request();  // refills the stage consumed in the previous iteration (every lane is past it: __syncwarp above)
          if (live) {
            uint4 xp[7];
            const uint4 *xb = reinterpret_cast<const uint4 *>(xrun);
#pragma unroll
            for (int i = 0; i < 7; ++i) xp[i] = xb[i];
            const float xsc = __uint_as_float(xp[6].w);
#pragma unroll
            for (int r = 0; r < R; ++r) {  // rows one after the other: payloads are read from the ring right before use
              uint4 q[QV];
#pragma unroll
              for (int v = 0; v < QV; ++v) q[v] = *reinterpret_cast<const uint4 *>(st + r * 32 * PB + dst_q + v * 16);
              const float dsc = __half2float(*reinterpret_cast<const __half *>(st + R * 32 * PB + r * SCALE_ROW + lane * 2));
              acc[r] = fmaf(dsc * xsc, block_dot_i<FMT>(q, xp), acc[r]);
            }
          }
          xrun += 32 * XQ_WORDS * 4;
          if (++ck == g.C || c + 1 == g.c1) {
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
            if (lane == 0) {
              float *dst = part + ((size_t)warp * plan.slots + (cg - first_grp)) * R;
#pragma unroll
              for (int r = 0; r < R; ++r) dst[r] = acc[r];
            }
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] = 0.f;
            if (ck == g.C) {
              ck = 0;
              ++cg;
              xrun = smem + (size_t)lane * (XQ_WORDS * 4);
            }
          }
        }
        __syncthreads();
        if (tr) plan.trace[sub * 5 + 2] = clock64();
        // epilogue: one warp per row group
        if (sub == 0)
          cta_epilogue<EPI_QKV, R>(P, part, plan.slots, g.g0, g.g1, g.C, g.T, 0, step_pos, rope_cs);
        else if (sub == 3)
          cta_epilogue<EPI_SWIGLU, R>(P, part, plan.slots, g.g0, g.g1, g.C, g.T, 0, 0, nullptr);
        else
          cta_epilogue<EPI_RESIDUAL, R>(P, part, plan.slots, g.g0, g.g1, g.C, g.T, 0, 0, nullptr);
      }
      if (tr) plan.trace[sub * 5 + 3] = clock64();
      ++n_bar;
      ok = grid_barrier(plan, bar_base + (unsigned long long)n_bar * gridDim.x, (int)(layer * 8 + sub + 1));
      if (tr) plan.trace[sub * 5 + 4] = clock64();
    }
  }
  cp_async_wait(0);
  if (ok && blockIdx.x == 0 && threadIdx.x == 0) *plan.gen = s_gen + 1;  // every CTA has passed the last barrier's arrival
}

struct PlanHeader {  // start of the caller-provided plan memory
  unsigned long long bar;
  uint32_t gen;
  int err;
  uint32_t pad[4];
  long long trace[32];
};

}  // namespace

extern "C" {

size_t greta_cuda_decode_plan_bytes(uint32_t num_layers) { return sizeof(PlanHeader) + (size_t)num_layers * sizeof(LayerPlan); }

int greta_cuda_decode_plan_build(greta_stream_t stream, const greta_decode_desc *d, const greta_decode_layer *layers, void *plan, size_t plan_bytes) {
  GRETA_REQUIRE(d && layers && plan, "decode_plan_build: null argument");
  GRETA_REQUIRE(plan_bytes >= greta_cuda_decode_plan_bytes(d->num_layers), "decode_plan_build: plan memory too small");
  GRETA_REQUIRE(d->weight_fmt == GRETA_FMT_Q4_0 || d->weight_fmt == GRETA_FMT_Q8_0, "decode_plan_build: weights must be Q4_0 or Q8_0");
  GRETA_REQUIRE(d->head_dim == 64 || d->head_dim == 128, "decode_plan_build: head_dim must be 64 or 128");
  GRETA_REQUIRE(d->dim % 32 == 0 && d->hidden_dim % 32 == 0 && (d->head_dim / 2) % 2 == 0 && d->num_heads % d->num_heads_kv == 0,
                "decode_plan_build: unsupported shape");
  const uint32_t D = d->dim, Dh = d->head_dim, H = d->num_heads, Hkv = d->num_heads_kv, Fh = d->hidden_dim;
  const uint32_t sms = (uint32_t)sm_count();
  GRETA_REQUIRE(greta_cuda_attn_decode_scratch_bytes(H, Dh) <= d->attn_scratch_bytes, "decode_plan_build: attention scratch too small");
  std::vector<uint8_t> host(greta_cuda_decode_plan_bytes(d->num_layers), 0);
  LayerPlan *lp = reinterpret_cast<LayerPlan *>(host.data() + sizeof(PlanHeader));
  const uint32_t splits = std::max(1u, std::min<uint32_t>(MAX_SPLITS, sms / H));
  for (uint32_t l = 0; l < d->num_layers; ++l) {
    const greta_decode_layer &w = layers[l];
    LayerPlan &L = lp[l];
    GemvParams q{};
    q.x = d->x; q.gamma = w.attn_norm; q.eps = d->rms_eps;
    q.w[0] = {(const uint8_t *)w.wq_qs, w.wq_d}; q.w[1] = {(const uint8_t *)w.wk_qs, w.wk_d}; q.w[2] = {(const uint8_t *)w.wv_qs, w.wv_d};
    q.K = D; q.M = 1; q.q_out = d->q; q.k_cache = (__half *)w.k_cache; q.v_cache = (__half *)w.v_cache; q.d_pos = d->d_pos;
    q.H = H; q.Hkv = Hkv; q.Dh = Dh; q.max_seq = d->max_seq_len; q.rope_base = d->rope_base;
    q.groups = (H + Hkv) * ((Dh / 2) / (R / 2)) + (Hkv * Dh + R - 1) / R;
    L.qkv = q;
    GemvParams o{};
    o.x = d->attn_out; o.w[0] = {(const uint8_t *)w.wo_qs, w.wo_d}; o.K = H * Dh; o.N = D; o.M = 1; o.y = d->x; o.resid = d->x;
    o.groups = (D + R - 1) / R;
    L.wo = o;
    GemvParams f{};
    f.x = d->x; f.gamma = w.ffn_norm; f.eps = d->rms_eps;
    f.w[0] = {(const uint8_t *)w.w1_qs, w.w1_d}; f.w[1] = {(const uint8_t *)w.w3_qs, w.w3_d};
    f.K = D; f.N = Fh; f.M = 1; f.y = d->mlp_gate; f.groups = (Fh + 1) / 2;
    L.ffn = f;
    GemvParams dn{};
    dn.x = d->mlp_gate; dn.w[0] = {(const uint8_t *)w.w2_qs, w.w2_d}; dn.K = Fh; dn.N = D; dn.M = 1; dn.y = d->x; dn.resid = d->x;
    dn.groups = (D + R - 1) / R;
    L.down = dn;
    AttnParams a{};
    a.q = d->q; a.kc = w.k_cache; a.vc = w.v_cache; a.o = d->attn_out; a.d_pos = d->d_pos; a.len0 = 0;
    a.H = H; a.Hkv = Hkv; a.max_seq = d->max_seq_len; a.scale = d->attn_scale; a.splits = splits;
    a.counters = reinterpret_cast<uint32_t *>(d->attn_scratch);
    a.partial = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(d->attn_scratch) + ((size_t)H * 4 + 255) / 256 * 256);
    L.attn = a;
  }
  GRETA_CUDA_TRY(cudaMemcpyAsync(plan, host.data(), host.size(), cudaMemcpyHostToDevice, (cudaStream_t)stream));
  GRETA_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));  // `host` is a local
  return GRETA_OK;
}

int greta_cuda_decode_layers(greta_stream_t stream, const greta_decode_desc *d, void *plan_mem) {
  GRETA_REQUIRE(d && plan_mem, "decode_layers: null argument");
  const uint32_t sms = (uint32_t)sm_count();
  const uint32_t Kmax = std::max(std::max(d->dim, d->hidden_dim), d->num_heads * d->head_dim);
  StepPlan plan{};
  PlanHeader *hdr = reinterpret_cast<PlanHeader *>(plan_mem);
  plan.layers = reinterpret_cast<const LayerPlan *>(hdr + 1);
  plan.num_layers = d->num_layers;
  plan.head_dim = d->head_dim;
  plan.embed = reinterpret_cast<const __half *>(d->tok_embd_f16);
  plan.d_token = d->d_token;
  plan.x = d->x;
  plan.dim = d->dim;
  plan.vocab = d->vocab_size;
  plan.bar = &hdr->bar;
  plan.gen = &hdr->gen;
  plan.err = &hdr->err;
  plan.trace = hdr->trace;
  plan.xs_bytes = (uint32_t)((((size_t)(Kmax / 32) * XQ_WORDS * 4) + 15) & ~(size_t)15);
  // the phase with the most cells per warp fixes the partial-sum slots
  const uint32_t H = d->num_heads, Hkv = d->num_heads_kv, Dh = d->head_dim;
  const uint32_t groups[4] = {(H + Hkv) * (Dh / 4) + (Hkv * Dh + 3) / 4, (d->dim + 3) / 4, (d->hidden_dim + 1) / 2, (d->dim + 3) / 4};
  const uint32_t Ks[4] = {d->dim, H * Dh, d->dim, d->hidden_dim};
  uint32_t slots = 2;
  for (int i = 0; i < 4; ++i) {
    const uint32_t C = (Ks[i] / 32 + 31) / 32, gmax = (groups[i] + sms - 1) / sms;
    slots = std::max(slots, (uint32_t)(((uint64_t)gmax * C + WARPS - 1) / WARPS) / C + 2);
  }
  plan.slots = slots;
  const bool q4 = d->weight_fmt == GRETA_FMT_Q4_0;
  const size_t stage_bytes = (size_t)R * (32 * (q4 ? 16 : 32) + 64);
  const size_t part_bytes = (size_t)WARPS * slots * R * sizeof(float);
  GRETA_REQUIRE(plan.xs_bytes + part_bytes + 2 * WARPS * stage_bytes <= DYN_SMEM_LIMIT, "decode_layers: shapes do not fit in shared memory");
  GRETA_REQUIRE(d->num_heads <= sms, "decode_layers: more heads than SMs");
  plan.stages = (uint32_t)std::min<size_t>(MAX_STAGES, (DYN_SMEM_LIMIT - plan.xs_bytes - part_bytes) / (WARPS * stage_bytes));
  if (tuning().step_stages > 0) plan.stages = std::max(2u, std::min<uint32_t>(plan.stages, (uint32_t)tuning().step_stages));
  const size_t smem = plan.xs_bytes + (size_t)WARPS * plan.stages * stage_bytes + part_bytes;
  auto kern = q4 ? decode_layers_kernel<GRETA_FMT_Q4_0> : decode_layers_kernel<GRETA_FMT_Q8_0>;
  static bool attr_set[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[q4][dev]) {
    GRETA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DYN_SMEM_LIMIT));
    attr_set[q4][dev] = true;
  }
  // One CTA per SM, all co-resident: a cooperative launch makes the driver guarantee it.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sms);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  GRETA_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, plan));
  return launched("decode_layers_kernel");
}

int greta_cuda_decode_trace(const void *plan_mem, long long *out25) {
  GRETA_REQUIRE(plan_mem && out25, "decode_trace: null argument");
  PlanHeader h;
  GRETA_CUDA_TRY(cudaMemcpy(&h, plan_mem, sizeof(h), cudaMemcpyDeviceToHost));
  for (int i = 0; i < 25; ++i) out25[i] = h.trace[i];
  return GRETA_OK;
}

int greta_cuda_decode_status(const void *plan_mem, int *code) {
  GRETA_REQUIRE(plan_mem && code, "decode_status: null argument");
  PlanHeader h;
  GRETA_CUDA_TRY(cudaMemcpy(&h, plan_mem, sizeof(h), cudaMemcpyDeviceToHost));
  *code = h.err;
  return GRETA_OK;
}

}  // extern "C"
