// Prefill GEMM over block-quantised weights on the 5th-generation tensor cores:
//   C[M x N] = half(A[M x K]) * half(dequant(W[N x K]))^T, fp32 accumulation in TMEM.
//
// The weight side is the 128-row operand of the MMA and the tokens are its N
// dimension ("swapped" roles): a CTA owns 128 weight rows and up to 256 tokens,
// so each weight tile is dequantised once and its accumulator (128 lanes x TN
// fp32 columns) lives in tensor memory for the whole K loop.
//
// Warp roles (192 threads):
//   warp 0     producer: TMA loads of the activation tile (TN x 64 fp16, 128-byte
//              swizzle) into a 4-stage ring, completion on an mbarrier;
//   warp 1     allocates TMEM, issues tcgen05.mma (one elected lane, 4 x K=16 per
//              stage), commits each stage back to the producers, deallocates;
//   warps 2-5  one thread per weight row: 128-bit loads of the quant payloads and
//              scales (software-prefetched two stages ahead), in-register dequant to
//              the exact fp16 value half((q - 8) * d), 128-bit stores into the
//              swizzled K-major smem tile the tensor core reads; afterwards the
//              epilogue: tcgen05.ld of the accumulator, conversion, stores to C.
// Every wait on an mbarrier is bounded: on a timeout the kernel raises a flag that
// all roles poll, drains, frees its tensor memory and returns; the host reads the
// flag with greta_cuda_gemm_status().
#include <cuda.h>

#include <mutex>

#include "greta_common.cuh"

using namespace greta;

namespace {

constexpr int BK = 64;          // K elements per stage (one 128-byte swizzle row of fp16)
constexpr int TILE_N = 128;     // weight rows per CTA (the MMA's M)
constexpr int STAGES = 4;
constexpr int B_STAGE_BYTES = TILE_N * BK * 2;
constexpr int NUM_THREADS = 192;
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;  // ~2 s at 2 GHz

__device__ int g_gemm_error = 0;  // 0 ok; otherwise 100 * role + stage of the wait that gave up

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the kernel is aborting (this wait timed out, or another role's did).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int code) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
      *abort_flag = code;
      atomicCAS(&g_gemm_error, 0, code);
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]^T, fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and 128-byte swizzle:
// 8-row groups 1024 bytes apart, descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp16 x fp16 -> fp32, both operands K-major, shape M x N.
__host__ __device__ constexpr uint32_t instr_desc_f16(uint32_t M, uint32_t N) {
  return (1u << 4) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// ---- dequant to exact fp16 -----------------------------------------------------------------
__device__ __forceinline__ uint32_t h2sub(uint32_t a, uint32_t b) {
  __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
  return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t h2fma(uint32_t a, uint32_t b, uint32_t c) {
  __half2 r = __hfma2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b), *reinterpret_cast<__half2 *>(&c));
  return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t h2mul(uint32_t a, uint32_t b) {
  __half2 r = __hmul2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
  return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t lop_and_or(uint32_t a, uint32_t m, uint32_t o) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(m), "r"(o));
  return r;
}
// One Q4_0 payload word -> 4 low-nibble elements (lo[0..1]) and 4 high-nibble elements (hi[0..1]) as half2,
// each half = round_to_half((q - 8) * d): the product of two halves rounded once, the same value as
// __float2half((float)(q - 8) * (float)d).
__device__ __forceinline__ void dq4_word(uint32_t w, uint32_t d2, uint32_t (&lo)[2], uint32_t (&hi)[2]) {
  const uint32_t MAGIC = 0x64006400u, C1032 = 0x64086408u, SIXTEENTH = 0x2C002C00u, CM72 = 0xD480D480u;
  uint32_t w8 = w >> 8;
  uint32_t a = h2mul(h2sub(lop_and_or(w, 0x000F000Fu, MAGIC), C1032), d2);            // e0, e2
  uint32_t b = h2mul(h2sub(lop_and_or(w8, 0x000F000Fu, MAGIC), C1032), d2);           // e1, e3
  uint32_t c = h2mul(h2fma(lop_and_or(w, 0x00F000F0u, MAGIC), SIXTEENTH, CM72), d2);  // E0, E2
  uint32_t e = h2mul(h2fma(lop_and_or(w8, 0x00F000F0u, MAGIC), SIXTEENTH, CM72), d2); // E1, E3
  lo[0] = __byte_perm(a, b, 0x5410);
  lo[1] = __byte_perm(a, b, 0x7632);
  hi[0] = __byte_perm(c, e, 0x5410);
  hi[1] = __byte_perm(c, e, 0x7632);
}
// One Q8_0 payload word (4 int8) -> 4 elements as two half2.
__device__ __forceinline__ void dq8_word(uint32_t w, uint32_t d2, uint32_t (&o)[2]) {
  const uint32_t C1152 = 0x64806480u;
  uint32_t t = w ^ 0x80808080u;
  o[0] = h2mul(h2sub(__byte_perm(t, 0x64646464u, 0x5140), C1152), d2);
  o[1] = h2mul(h2sub(__byte_perm(t, 0x64646464u, 0x7362), C1152), d2);
}

template <int FMT>
struct Raw {  // one thread's weights for one stage: 64 weights of its row
  static constexpr int QV = (FMT == GRETA_FMT_Q4_0) ? 2 : 4;
  uint4 q[QV];
  uint32_t d;  // two fp16 scales
};

// Stage kt covers blocks 2kt and 2kt+1 of the row; when K is an odd number of blocks the last stage
// has only the first one, and the missing half is made zero (the activations there are zero-filled
// by TMA, but 0 * garbage must not produce a NaN).
template <int FMT>
__device__ __forceinline__ void load_raw(Raw<FMT> &r, const uint8_t *qs_row, const __half *d_row, uint32_t kt, uint32_t nb) {
  constexpr int QV = Raw<FMT>::QV;
  const uint8_t *p = qs_row + (size_t)kt * QV * 16;
  const bool second = 2 * kt + 1 < nb;
#pragma unroll
  for (int v = 0; v < QV; ++v) r.q[v] = (v < QV / 2 || second) ? ld_stream(p + v * 16) : make_uint4(0, 0, 0, 0);
  r.d = __ldg(reinterpret_cast<const uint32_t *>(d_row + 2 * kt));  // rows of the d plane are padded: always in bounds
  if (!second) r.d &= 0xFFFFu;                                      // scale 0 for the absent block
}

// Dequantises the thread's 64 weights and writes its 128-byte row of the swizzled B tile.
template <int FMT>
__device__ __forceinline__ void dequant_store(const Raw<FMT> &r, uint8_t *row_base, int row_in_atom) {
  uint4 chunk[8];  // chunk c = elements 8c .. 8c+7
  const uint32_t d_lo = r.d & 0xFFFFu, d_hi = r.d >> 16;
  const uint32_t d2[2] = {d_lo | (d_lo << 16), d_hi | (d_hi << 16)};
  if (FMT == GRETA_FMT_Q4_0) {
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const uint32_t w[4] = {r.q[blk].x, r.q[blk].y, r.q[blk].z, r.q[blk].w};
      uint32_t lo[4][2], hi[4][2];
#pragma unroll
      for (int i = 0; i < 4; ++i) dq4_word(w[i], d2[blk], lo[i], hi[i]);
      chunk[4 * blk + 0] = make_uint4(lo[0][0], lo[0][1], lo[1][0], lo[1][1]);
      chunk[4 * blk + 1] = make_uint4(lo[2][0], lo[2][1], lo[3][0], lo[3][1]);
      chunk[4 * blk + 2] = make_uint4(hi[0][0], hi[0][1], hi[1][0], hi[1][1]);
      chunk[4 * blk + 3] = make_uint4(hi[2][0], hi[2][1], hi[3][0], hi[3][1]);
    }
  } else {
#pragma unroll
    for (int v = 0; v < 4; ++v) {  // payload v: 16 int8 = elements 16v .. 16v+15 (block v / 2)
      const uint32_t w[4] = {r.q[v].x, r.q[v].y, r.q[v].z, r.q[v].w};
      uint32_t o[4][2];
#pragma unroll
      for (int i = 0; i < 4; ++i) dq8_word(w[i], d2[v >> 1], o[i]);
      chunk[2 * v + 0] = make_uint4(o[0][0], o[0][1], o[1][0], o[1][1]);
      chunk[2 * v + 1] = make_uint4(o[2][0], o[2][1], o[3][0], o[3][1]);
    }
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4 *>(row_base + ((c ^ row_in_atom) << 4)) = chunk[c];
}

template <int FMT, int TN, bool OUT_F16>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const uint8_t *__restrict__ qs, const __half *__restrict__ dsc, void *__restrict__ Cout,
               uint32_t M, uint32_t N, uint32_t K) {
  constexpr int A_STAGE_BYTES = TN * BK * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzle atoms need 1024-byte alignment
  uint8_t *a_tiles = smem;                                  // [STAGES][TN][128 B]   tokens   (MMA operand B)
  uint8_t *b_tiles = smem + STAGES * A_STAGE_BYTES;         // [STAGES][128][128 B]  weights  (MMA operand A)
  uint64_t *bars = reinterpret_cast<uint64_t *>(b_tiles + STAGES * B_STAGE_BYTES);
  uint64_t *a_full = bars, *b_full = bars + STAGES, *empty = bars + 2 * STAGES, *acc_full = bars + 3 * STAGES;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * STAGES + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t n0 = blockIdx.x * TILE_N, m0 = blockIdx.y * TN;
  const uint32_t KT = (K + BK - 1) / BK, nb = K / 32;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&b_full[s], 4);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t issued = 0;
      for (uint32_t kt = 0; kt < KT; ++kt) {
        const uint32_t s = kt % STAGES, ph = (kt / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, 100 + s)) break;
        mbar_arrive_expect_tx(&a_full[s], A_STAGE_BYTES);
        tma_load_2d(a_tiles + s * A_STAGE_BYTES, &tmap_a, (int)(kt * BK), (int)m0, &a_full[s]);
        ++issued;
      }
      if (*abort_flag) {  // give the copies still in flight a bounded chance to land before the CTA exits
        for (uint32_t j = issued > (uint32_t)STAGES ? issued - STAGES : 0; j < issued; ++j) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&a_full[j % STAGES], (j / STAGES) & 1) && clock64() - t0 < 20000000ll) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_f16(TILE_N, TN);
      bool ok = true;
      for (uint32_t kt = 0; kt < KT && ok; ++kt) {
        const uint32_t s = kt % STAGES, ph = (kt / STAGES) & 1;
        ok = mbar_wait(&a_full[s], ph, abort_flag, 200 + s) && mbar_wait(&b_full[s], ph, abort_flag, 300 + s);
        if (!ok) break;
        tc_fence_after();
        const uint32_t wa = smem_u32(b_tiles + s * B_STAGE_BYTES), ta = smem_u32(a_tiles + s * A_STAGE_BYTES);
#pragma unroll
        for (int k16 = 0; k16 < BK / 16; ++k16)
          umma_f16(tmem_base, smem_desc_sw128(wa + k16 * 32), smem_desc_sw128(ta + k16 * 32), idesc, (kt | (uint32_t)k16) != 0);
        umma_commit(&empty[s]);  // stage s may be refilled once these MMAs have read it
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    // ---------------- dequant warps, then epilogue ----------------
    const int t = threadIdx.x - 64;  // weight row inside the tile, 0..127
    const uint32_t n = min(n0 + (uint32_t)t, N - 1);
    const uint8_t *qs_row = qs + (size_t)n * nb * (FMT == GRETA_FMT_Q4_0 ? 16 : 32);
    const __half *d_row = dsc + (size_t)n * d_row_stride(nb);
    Raw<FMT> r0, r1, r2;
    load_raw<FMT>(r0, qs_row, d_row, 0, nb);
    if (KT > 1) load_raw<FMT>(r1, qs_row, d_row, 1, nb);
    bool ok = true;
    for (uint32_t kt = 0; kt < KT; ++kt) {
      const uint32_t s = kt % STAGES, ph = (kt / STAGES) & 1;
      if (kt + 2 < KT) load_raw<FMT>(r2, qs_row, d_row, kt + 2, nb);
      ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, 400 + s);
      if (!ok) break;
      dequant_store<FMT>(r0, b_tiles + s * B_STAGE_BYTES + t * 128, t & 7);
      fence_proxy_async();  // make the generic-proxy stores visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(&b_full[s]);
      r0 = r1;
      r1 = r2;
    }
    // epilogue: accumulator rows = weight rows (TMEM lanes), columns = tokens
    if (ok) ok = mbar_wait(acc_full, 0, abort_flag, 500);
    if (ok) {
      tc_fence_after();
      const int quad = warp & 3;  // a warp may only touch TMEM lanes 32 * (warp % 4) .. +31
      const uint32_t row = n0 + quad * 32 + lane;
      for (int c = 0; c < TN; c += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + c, v);
        tmem_ld_wait();
        if (row < N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const uint32_t m = m0 + c + j;
            if (m < M) {
              if (OUT_F16)
                reinterpret_cast<__half *>(Cout)[(size_t)m * N + row] = __float2half_rn(__uint_as_float(v[j]));
              else
                reinterpret_cast<float *>(Cout)[(size_t)m * N + row] = __uint_as_float(v[j]);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TN);
  }
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

template <int FMT, int TN, bool OUT_F16>
int launch_tc(cudaStream_t stream, const CUtensorMap &map, const void *qs, const void *d, void *C, uint32_t M, uint32_t N, uint32_t K) {
  const size_t smem = (size_t)STAGES * (TN * BK * 2 + B_STAGE_BYTES) + 1024 + 256;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    GRETA_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<FMT, TN, OUT_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set[dev] = true;
  }
  dim3 grid((N + TILE_N - 1) / TILE_N, (M + TN - 1) / TN);
  gemm_tc_kernel<FMT, TN, OUT_F16><<<grid, NUM_THREADS, smem, stream>>>(map, (const uint8_t *)qs, (const __half *)d, C, M, N, K);
  return launched("gemm_tc_kernel");
}

template <int FMT>
int dispatch_tc(cudaStream_t stream, const CUtensorMap &m128, const CUtensorMap &m256, bool wide, bool out_f16, const void *qs, const void *d,
                void *C, uint32_t M, uint32_t N, uint32_t K) {
  if (wide) return out_f16 ? launch_tc<FMT, 256, true>(stream, m256, qs, d, C, M, N, K) : launch_tc<FMT, 256, false>(stream, m256, qs, d, C, M, N, K);
  return out_f16 ? launch_tc<FMT, 128, true>(stream, m128, qs, d, C, M, N, K) : launch_tc<FMT, 128, false>(stream, m128, qs, d, C, M, N, K);
}

}  // namespace

extern "C" {

size_t greta_cuda_gemm_workspace_bytes(uint32_t M, uint32_t K) { return ((size_t)M * K * 2 + 255) / 256 * 256; }

int greta_cuda_gemm_status(int *code) {
  GRETA_REQUIRE(code, "gemm_status: null out pointer");
  GRETA_CUDA_TRY(cudaMemcpyFromSymbol(code, g_gemm_error, sizeof(int)));
  return GRETA_OK;
}

int greta_cuda_gemm(greta_stream_t stream, int fmt, const void *A, int a_is_f16, const void *qs, const void *d, void *Cout, int c_is_f16,
                    uint32_t M, uint32_t N, uint32_t K, void *workspace) {
  if (M == 0 || N == 0 || K == 0) return GRETA_OK;
  GRETA_REQUIRE(fmt == GRETA_FMT_Q4_0 || fmt == GRETA_FMT_Q8_0, "gemm: format %d is not supported (Q4_0 or Q8_0)", fmt);
  GRETA_REQUIRE(K % 32 == 0, "gemm: K=%u is not a multiple of the block size 32", K);
  GRETA_REQUIRE(A && qs && d && Cout, "gemm: null pointer");
  GRETA_REQUIRE(aligned16(A) && aligned16(qs) && ((uintptr_t)d & 3) == 0 && aligned16(Cout), "gemm: misaligned pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const void *a16 = A;
  if (!a_is_f16) {
    GRETA_REQUIRE(workspace && aligned16(workspace), "gemm: fp32 activations need a workspace of greta_cuda_gemm_workspace_bytes(M, K)");
    if (int rc = greta_cuda_f32_to_f16(stream, static_cast<const float *>(A), workspace, (size_t)M * K)) return rc;
    a16 = workspace;
  }
  EncodeTiledFn enc = encode_tiled();
  if (!enc) {
    set_error("gemm: cuTensorMapEncodeTiled is not available from this driver");
    return GRETA_ERR_NOT_IMPLEMENTED;
  }
  const bool wide = M > 128;
  CUtensorMap map;
  const cuuint64_t dims[2] = {K, M};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {BK, wide ? 256u : 128u};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(a16), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("gemm: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return GRETA_ERR_INVALID_ARGS;
  }
  if (fmt == GRETA_FMT_Q4_0) return dispatch_tc<GRETA_FMT_Q4_0>(s, map, map, wide, c_is_f16 != 0, qs, d, Cout, M, N, K);
  return dispatch_tc<GRETA_FMT_Q8_0>(s, map, map, wide, c_is_f16 != 0, qs, d, Cout, M, N, K);
}

}  // extern "C"
