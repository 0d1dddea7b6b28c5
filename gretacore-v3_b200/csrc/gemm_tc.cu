// Prefill GEMM over block-quantised weights on the 5th-generation tensor cores:
//   C[M x N] = half(A[M x K]) * half(dequant(W[N x K]))^T, fp32 accumulation in TMEM.
//
// The weight side is the 128-row operand of the MMA and the tokens are its N
// dimension ("swapped" roles): a CTA owns 128 weight rows and 128, 256 or 512
// tokens, so each weight tile is dequantised once and its accumulator (128 lanes x
// TN fp32 columns, up to all 512 columns of tensor memory) stays there for the
// whole K loop.  A 512-token tile is two N=256 MMAs per K=16 step.
//
// Warp roles (320 threads):
//   warp 0     producer: TMA loads of activation units (up to 256 tokens x 64 fp16,
//              128-byte swizzle) into a ring, completion on an mbarrier per unit;
//   warp 1     allocates TMEM, issues tcgen05.mma (one elected lane, 4 x K=16 per
//              unit), commits each unit and each weight stage back to its producer,
//              deallocates;
//   warps 2-9  two threads per weight row, one 32-weight block each per stage:
//              cp.async of the quant payload and scales into a raw ring several
//              stages ahead of use, in-register dequant to the exact fp16 value
//              half((q - 8) * d), 128-bit stores into the swizzled K-major smem tile
//              the tensor core reads; afterwards the epilogue: tcgen05.ld of the
//              accumulator, conversion, stores to C.
// Every wait on an mbarrier is bounded: on a timeout the kernel raises a flag that
// all roles poll, drains, frees its tensor memory and returns; the host reads the
// flag with greta_cuda_gemm_status().
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <chrono>
#include <mutex>

#include "greta_common.cuh"

using namespace greta;

namespace {

constexpr int BK = 64;          // K elements per stage (one 128-byte swizzle row of fp16)
constexpr int TILE_N = 128;     // weight rows per MMA (its M)
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
// Arrival on a barrier of the pair's even CTA.  CTA-scope release on purpose: what the arrival publishes are this
// thread's shared-memory stores, already fenced towards the async proxy, and the tensor core of this SM is what reads
// them; a cluster-scope release would also wait for the thread's outstanding cp.async prefetches (about one DRAM
// latency per stage: measured, it doubled the kernel's time).
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
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
// The common case, a barrier that has already completed, is one try_wait; the polling loop with its
// clock reads is kept out of line so the issuing threads' instruction streams stay short.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
  const long long t0 = clock64();
  for (;;) {
    uint32_t ok;
    asm volatile(  // with a time hint the thread sleeps in hardware until the phase completes instead of spinning through issue slots
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(1000u)
        : "memory");
    if (ok) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
      *abort_flag = code;
      atomicCAS(&g_gemm_error, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(smem_u32(bar), parity, abort_flag, code);
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
// D[tmem] (+)= A[smem desc] * B[smem desc]^T, fp16 inputs, fp32 accumulate.  The descriptors are passed as
// their low words (start address and leading offset); the high word is the same for every tile.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint32_t desc_a_lo, uint32_t desc_b_lo, uint32_t desc_hi, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(tmem_d),
      "r"(desc_a_lo), "r"(desc_b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
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

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and 128-byte swizzle: start address
// and leading offset 1 in the low word; 8-row groups 1024 bytes apart, descriptor version 1 (Blackwell) and
// layout type 2 (SWIZZLE_128B) in the high word.  Shared addresses are below 256 KB, so address / 16 fits
// the 14-bit field and tiles are stepped by adding bytes / 16 to the low word.
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr) { return ((smem_addr >> 4) & 0x3FFFu) | (1u << 16); }
constexpr uint32_t SMEM_DESC_HI_SW128 = (1024u >> 4) | (1u << 14) | (2u << 29);
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

// Tile shapes.  A CTA owns RT tiles of 128 weight rows and TN tokens, RT * TN <= 512 accumulator
// columns of tensor memory.  An activation "unit" is (up to) 256 tokens x 64 K = 32 KB and feeds
// 4 * RT MMAs, so with RT = 2 one unit carries twice the tensor-core time: a slot of the activation
// ring is recycled through commit -> producer -> TMA -> issuer, about 2 us, and the ring has to hold
// that much tensor-core time for the MMAs to run back to back.
template <int FMT, int TN, int RT>
struct Cfg {
  static constexpr int ROWS = RT * TILE_N;
  static constexpr int QV = (FMT == GRETA_FMT_Q4_0) ? 1 : 2;  // 16-byte payload pieces per 32-weight block
  static constexpr int DEQ_THREADS = 2 * ROWS;                 // two threads per weight row: one block each per stage
  static constexpr int THREADS = 64 + DEQ_THREADS;
  static constexpr int RAW_SCALES = 2 * QV * ROWS * 16;        // raw stage: pieces [block][v][row], then one scale word per thread
  static constexpr int RAW_STAGE = RAW_SCALES + 2 * ROWS * 4;
  static constexpr int B_STAGE = ROWS * BK * 2;                // RT swizzled 128-row tiles back to back
  static constexpr int UNIT_ROWS = TN < 256 ? TN : 256;
  static constexpr int UPS = TN / UNIT_ROWS;  // units per stage
  static constexpr int UNIT_BYTES = UNIT_ROWS * BK * 2;
  static constexpr bool Q4 = FMT == GRETA_FMT_Q4_0;
  static constexpr int AU = RT == 2 ? (TN == 256 ? (Q4 ? 4 : 3) : 6) : (TN == 128 ? 6 : (TN == 512 && Q4 ? 5 : 4));
  static constexpr int BS = RT == 2 ? (TN == 256 || !Q4 ? 2 : 3) : ((TN == 256 && !Q4) || TN == 512 ? 3 : 4);
  static constexpr int RS = RT == 2 ? 3 : (TN == 512 ? 3 : (TN == 256 ? (Q4 ? 6 : 4) : (Q4 ? 8 : 6)));
  static constexpr int U = (RT == 1 && TN <= 256 && BS >= 3 && RS >= 4) ? 2 : 1;  // stages per pass of the dequant loop
  static constexpr int NBARS = 2 * AU + 2 * BS + 1;
  static constexpr size_t SMEM = (size_t)AU * UNIT_BYTES + (size_t)BS * B_STAGE + (size_t)RS * RAW_STAGE + 1024 + 256;
  static_assert(RT * TN <= 512, "accumulators exceed tensor memory");
  static_assert(SMEM <= 232448, "tile configuration exceeds shared memory");
};

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void *smem_dst, const void *gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Starts the copy of one thread's share of stage kt into the raw ring: block 2kt + hb of its row and the
// 4-byte word holding both scales of the stage.  When K is an odd number of blocks the last stage has
// only the first block; the thread of the absent one copies nothing and stores zeros.
template <class C>
__device__ __forceinline__ void raw_issue(uint8_t *stage, int row, int hb, const uint8_t *qs_row, const __half *d_row, uint32_t kt, uint32_t nb) {
  if (2 * kt + hb >= nb) return;
  const uint8_t *p = qs_row + ((size_t)2 * kt + hb) * C::QV * 16;
#pragma unroll
  for (int v = 0; v < C::QV; ++v) cp_async16(stage + ((hb * C::QV + v) * C::ROWS + row) * 16, p + v * 16);
  cp_async4(stage + C::RAW_SCALES + (hb * C::ROWS + row) * 4, d_row + 2 * kt);  // rows of the d plane are padded: always in bounds
}

// Dequantises the thread's block of one stage from the raw ring into four 16-byte chunks of fp16
// (chunk c = elements 8c .. 8c+7 of the block).
template <class C>
__device__ __forceinline__ void dequant_block(const uint8_t *stage, int row, int hb, bool present, uint4 (&chunk)[4]) {
  if (present) {
    const uint32_t dw = *reinterpret_cast<const uint32_t *>(stage + C::RAW_SCALES + (hb * C::ROWS + row) * 4);
    const uint32_t dh = hb ? (dw >> 16) : (dw & 0xFFFFu);
    const uint32_t d2 = dh | (dh << 16);
    if (C::Q4) {
      const uint4 q = *reinterpret_cast<const uint4 *>(stage + (hb * C::ROWS + row) * 16);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      uint32_t lo[4][2], hi[4][2];
#pragma unroll
      for (int i = 0; i < 4; ++i) dq4_word(w[i], d2, lo[i], hi[i]);
      chunk[0] = make_uint4(lo[0][0], lo[0][1], lo[1][0], lo[1][1]);
      chunk[1] = make_uint4(lo[2][0], lo[2][1], lo[3][0], lo[3][1]);
      chunk[2] = make_uint4(hi[0][0], hi[0][1], hi[1][0], hi[1][1]);
      chunk[3] = make_uint4(hi[2][0], hi[2][1], hi[3][0], hi[3][1]);
    } else {
#pragma unroll
      for (int v = 0; v < 2; ++v) {  // payload v: 16 int8 = elements 16v .. 16v+15 of the block
        const uint4 q = *reinterpret_cast<const uint4 *>(stage + ((hb * C::QV + v) * C::ROWS + row) * 16);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t o[4][2];
#pragma unroll
        for (int i = 0; i < 4; ++i) dq8_word(w[i], d2, o[i]);
        chunk[2 * v + 0] = make_uint4(o[0][0], o[0][1], o[1][0], o[1][1]);
        chunk[2 * v + 1] = make_uint4(o[2][0], o[2][1], o[3][0], o[3][1]);
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) chunk[c] = make_uint4(0, 0, 0, 0);  // the activations there are zero-filled by TMA; 0 * 0, never 0 * garbage
  }
}

// The dequant warps' share of the K loop, common to the one-CTA and the two-CTA kernel.  Stages 0 .. RS-1 of
// the raw ring have been requested, one commit group each.  A pass of the loop takes U consecutive stages: the
// dependent chain of one stage (shared-memory load -> half2 math -> wait for the slot -> stores -> proxy fence ->
// arrival) is about 950 cycles at 128 tokens, several times its issue time, and every warp works on every stage,
// so one stage per pass makes that chain the stage period whenever the token tile is short; U stages per pass
// interleave U chains and share the fence.  U <= BS and U <= RS.
// b_full_remote0 != 0: arrivals go to the barrier array at that cluster-window address (the pair's even CTA).
template <class C, int U>
__device__ __forceinline__ bool dequant_stages(uint8_t *raw, uint8_t *b_tiles, uint64_t *b_empty, uint64_t *b_full, uint32_t b_full_remote0, int row,
                                               int hb, uint32_t row_off, const uint8_t *qs_row, const __half *d_row, uint32_t KT, uint32_t nb,
                                               volatile int *abort_flag, int lane) {
  constexpr int BS = C::BS, RS = C::RS, RAW_STAGE = C::RAW_STAGE, B_STAGE = C::B_STAGE;
  static_assert(U >= 1 && U <= BS && U <= RS, "stages per pass");
  bool ok = true;
  uint32_t s = 0, sph = 1, rs_use = 0;  // a fresh barrier passes a wait on parity 1
  for (uint32_t kt = 0; kt < KT; kt += U) {
    cp_async_wait<RS - U>();  // this thread's shares of stages kt .. kt+U-1 have landed (it reads only what it copied)
    uint4 chunk[U][4];
    uint32_t slot[U], par[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      uint32_t r = rs_use + j;
      if (r >= (uint32_t)RS) r -= RS;
      slot[j] = s + j;
      par[j] = sph;
      if (slot[j] >= (uint32_t)BS) {
        slot[j] -= BS;
        par[j] ^= 1;
      }
      if (kt + j < KT) dequant_block<C>(raw + r * RAW_STAGE, row, hb, 2 * (kt + j) + hb < nb, chunk[j]);  // the math does not wait for the slot
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
      if (kt + j < KT && ok) {
        ok = mbar_wait(&b_empty[slot[j]], par[j], abort_flag, 400 + slot[j]);
        if (ok) {
          uint8_t *row_base = b_tiles + slot[j] * B_STAGE + row_off;
#pragma unroll
          for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4 *>(row_base + (((4 * hb + c) ^ (row & 7)) << 4)) = chunk[j][c];
        }
      }
    }
    if (!ok) break;
    fence_proxy_async();  // make the generic-proxy stores visible to the tensor core's reads
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < U; ++j) {
        if (kt + j < KT) {
          if (b_full_remote0)
            mbar_arrive_remote(b_full_remote0 + slot[j] * 8);
          else
            mbar_arrive(&b_full[slot[j]]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {  // refill the raw slots just read
      uint32_t r = rs_use + j;
      if (r >= (uint32_t)RS) r -= RS;
      if (kt + j + RS < KT) raw_issue<C>(raw + r * RAW_STAGE, row, hb, qs_row, d_row, kt + j + RS, nb);
      cp_async_commit();
    }
    s += U;
    if (s >= (uint32_t)BS) {
      s -= BS;
      sph ^= 1;
    }
    rs_use += U;
    if (rs_use >= (uint32_t)RS) rs_use -= RS;
  }
  cp_async_wait<0>();
  return ok;
}

template <int FMT, int TN, int RT, bool OUT_F16>
__global__ void __launch_bounds__(Cfg<FMT, TN, RT>::THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const uint8_t *__restrict__ qs, const __half *__restrict__ dsc, void *__restrict__ Cout,
               uint32_t M, uint32_t N, uint32_t K) {
  using C = Cfg<FMT, TN, RT>;
  constexpr int AU = C::AU, BS = C::BS, RS = C::RS, UPS = C::UPS, UNIT_BYTES = C::UNIT_BYTES, UNIT_ROWS = C::UNIT_ROWS;
  constexpr int RAW_STAGE = C::RAW_STAGE, B_STAGE = C::B_STAGE, ROWS = C::ROWS, COLS = RT * TN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzle atoms need 1024-byte alignment
  uint8_t *a_units = smem;                       // [AU][UNIT_ROWS][128 B]  tokens   (MMA operand B)
  uint8_t *b_tiles = a_units + AU * UNIT_BYTES;  // [BS][RT][128][128 B]    weights  (MMA operand A)
  uint8_t *raw = b_tiles + BS * B_STAGE;         // [RS] raw quantised stages
  uint64_t *bars = reinterpret_cast<uint64_t *>(raw + RS * RAW_STAGE);
  uint64_t *a_full = bars, *a_empty = bars + AU, *b_full = bars + 2 * AU, *b_empty = bars + 2 * AU + BS, *acc_full = bars + 2 * AU + 2 * BS;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + C::NBARS);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t n0 = blockIdx.x * ROWS, m0 = blockIdx.y * TN;
  const uint32_t KT = (K + BK - 1) / BK, nb = K / 32;
  const uint32_t G_PRE = min((uint32_t)AU, KT * UPS);  // activation units requested before the set-up barrier

  if (threadIdx.x == 0) {
    for (int s = 0; s < AU; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&a_empty[s], 1);
    }
    for (int s = 0; s < BS; ++s) {
      mbar_init(&b_full[s], C::DEQ_THREADS / 32);
      mbar_init(&b_empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // The thread that made the barriers is the TMA producer: the first ring-full of activation units goes out
    // now, under the TMEM allocation and the set-up barrier (a_empty needs no wait the first time round).
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
    for (uint32_t g = 0; g < G_PRE; ++g) {
      mbar_arrive_expect_tx(&a_full[g], UNIT_BYTES);
      tma_load_2d(a_units + g * UNIT_BYTES, &tmap_a, (int)((g / UPS) * BK), (int)(m0 + (g % UPS) * UNIT_ROWS), &a_full[g]);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, COLS);
    tmem_relinquish();
  }
  // Dequant threads: the first raw-weight stages are requested before the set-up barrier as well.
  const int t = (int)threadIdx.x - 64;
  const int row = t >= 0 ? t % ROWS : 0, hb = t >= 0 ? t / ROWS : 0;  // weight row inside the CTA's rows, and which block of the stage
  const uint32_t n_row = min(n0 + (uint32_t)row, N - 1);
  const uint8_t *qs_row = qs + (size_t)n_row * nb * (C::Q4 ? 16 : 32);
  const __half *d_row = dsc + (size_t)n_row * d_row_stride(nb);
  if (warp >= 2) {
#pragma unroll
    for (int j = 0; j < RS; ++j) {
      if ((uint32_t)j < KT) raw_issue<C>(raw + j * RAW_STAGE, row, hb, qs_row, d_row, j, nb);
      cp_async_commit();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t issued = G_PRE, u = G_PRE % AU, ph = G_PRE == (uint32_t)AU ? 0u : 1u;
      for (uint32_t g = G_PRE; g < KT * UPS; ++g) {
        if (!mbar_wait(&a_empty[u], ph, abort_flag, 100 + u)) break;
        mbar_arrive_expect_tx(&a_full[u], UNIT_BYTES);
        tma_load_2d(a_units + u * UNIT_BYTES, &tmap_a, (int)((g / UPS) * BK), (int)(m0 + (g % UPS) * UNIT_ROWS), &a_full[u]);
        ++issued;
        if (++u == AU) {
          u = 0;
          ph ^= 1;
        }
      }
      if (*abort_flag) {  // give the copies still in flight a bounded chance to land before the CTA exits
        for (uint32_t j = issued > (uint32_t)AU ? issued - AU : 0; j < issued; ++j) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&a_full[j % AU], (j / AU) & 1) && clock64() - t0 < 20000000ll) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_f16(TILE_N, UNIT_ROWS);
      const uint32_t w_lo0 = smem_desc_lo(smem_u32(b_tiles)), a_lo0 = smem_desc_lo(smem_u32(a_units));
      bool ok = true;
      uint32_t s = 0, sph = 0, u = 0, uph = 0, acc = 0;
      for (uint32_t kt = 0; kt < KT && ok; ++kt) {
        ok = mbar_wait(&b_full[s], sph, abort_flag, 300 + s);
        if (!ok) break;
        const uint32_t w_lo = w_lo0 + s * (B_STAGE >> 4);
#pragma unroll
        for (int h = 0; h < UPS; ++h) {
          ok = mbar_wait(&a_full[u], uph, abort_flag, 200 + u);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + u * (UNIT_BYTES >> 4);
#pragma unroll
          for (int k16 = 0; k16 < BK / 16; ++k16) {  // accumulator (r, h) sits at column (r * UPS + h) * UNIT_ROWS
#pragma unroll
            for (int r = 0; r < RT; ++r)
              umma_f16(tmem_base + (r * UPS + h) * UNIT_ROWS, w_lo + r * ((TILE_N * BK * 2) >> 4) + k16 * 2, a_lo + k16 * 2, SMEM_DESC_HI_SW128, idesc,
                       k16 == 0 ? acc : 1u);
          }
          umma_commit(&a_empty[u]);  // the unit may be refilled once these MMAs have read it
          if (++u == AU) {
            u = 0;
            uph ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&b_empty[s]);
        acc = 1;
        if (++s == BS) {
          s = 0;
          sph ^= 1;
        }
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    // ---------------- dequant warps, then epilogue ----------------
    // this thread's half (64 bytes) of its row in the swizzled tile of its 128-row group
    const uint32_t row_off = (row >> 7) * (TILE_N * BK * 2) + (row & 127) * 128;
    bool ok = dequant_stages<C, C::U>(raw, b_tiles, b_empty, b_full, 0u, row, hb, row_off, qs_row, d_row, KT, nb, abort_flag, lane);
    // epilogue: accumulator rows = weight rows (TMEM lanes), columns = tokens.  A warp may only touch TMEM
    // lanes 32 * (warp % 4) .. +31; the 2 * RT warps of a lane quadrant split row tiles and token halves.
    if (ok) ok = mbar_wait(acc_full, 0, abort_flag, 500);
    const int quad = warp & 3, share = (warp - 2) >> 2;
    const int r = share % RT, half = share / RT;
    // fp16 output of a whole row tile goes through shared memory (the rings are idle by now): the TMEM
    // layout gives a lane one row and 32 tokens, i.e. 2-byte stores 2N bytes apart; transposed in shared
    // memory the tile leaves as 16-byte stores, 256 contiguous bytes per token.
    const bool staged = OUT_F16 && n0 + ROWS <= N && N % 8 == 0;
    if (ok) {
      tc_fence_after();
      const uint32_t orow = n0 + r * TILE_N + quad * 32 + lane;
      for (int c = half * (TN / 2); c < (half + 1) * (TN / 2); c += 32) {
        if (m0 + c >= M) break;
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + r * TN + c, v);
        tmem_ld_wait();
        if (staged) {
          __half *tile = reinterpret_cast<__half *>(smem) + (size_t)c * ROWS + r * TILE_N + quad * 32 + lane;
#pragma unroll
          for (int j = 0; j < 32; ++j) tile[(size_t)j * ROWS] = __float2half_rn(__uint_as_float(v[j]));
        } else if (orow < N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const uint32_t m = m0 + c + j;
            if (m < M) {
              if (OUT_F16)
                reinterpret_cast<__half *>(Cout)[(size_t)m * N + orow] = __float2half_rn(__uint_as_float(v[j]));
              else
                reinterpret_cast<float *>(Cout)[(size_t)m * N + orow] = __uint_as_float(v[j]);
            }
          }
        }
      }
    }
    if (staged) {  // uniform over the CTA; every dequant thread arrives, whatever `ok` says
      asm volatile("bar.sync 1, %0;" ::"n"(C::DEQ_THREADS) : "memory");
      if (ok) {
        constexpr uint32_t PIECES_PER_TOKEN = ROWS / 8;  // 16-byte pieces
        const uint32_t tokens = min((uint32_t)TN, M - m0);
        for (uint32_t piece = t; piece < tokens * PIECES_PER_TOKEN; piece += C::DEQ_THREADS) {
          const uint32_t tok = piece / PIECES_PER_TOKEN, off = piece % PIECES_PER_TOKEN;
          const uint4 val = *reinterpret_cast<const uint4 *>(smem + ((size_t)tok * ROWS + off * 8) * 2);
          *reinterpret_cast<uint4 *>(reinterpret_cast<__half *>(Cout) + (size_t)(m0 + tok) * N + n0 + off * 8) = val;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, COLS);
  }
}

// ---- two-CTA form ------------------------------------------------------------------------------
// A cluster of two CTAs owns 256 weight rows (128 each) and 256 * UPS tokens.  One tcgen05.mma with
// cta_group::2 (M = 256, N = 256), issued by a thread of the even CTA, multiplies both CTAs' weight
// tiles with a 256-token unit of which each CTA has staged 128 tokens: per 64-K stage a CTA writes, and
// its tensor core reads, half the token bytes of the one-CTA form, whose pace shared-memory bandwidth
// set.  Each CTA's accumulator (its 128 rows x all tokens) stays in its own tensor memory, so the
// epilogue is the one-CTA one.  The "full" barriers that the issuing thread waits on live in the even
// CTA: the odd CTA's TMA loads complete their bytes there and its dequant warps arrive there through
// the cluster window.  The "empty" barriers and acc_full exist in both CTAs and one commit signals both.
// No load is multicast; every mbarrier wait is bounded as in the one-CTA kernel, and both CTAs always
// reach the closing cluster barrier, so neither leaves while the other may still address its memory.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// TMA load of this CTA's half of a token unit; the bytes are counted on a barrier given by its address in
// the cluster window (the even CTA's).
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint32_t desc_a_lo, uint32_t desc_b_lo, uint32_t desc_hi, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(tmem_d),
      "r"(desc_a_lo), "r"(desc_b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in both CTAs of the pair once every MMA issued so far has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "h"((uint16_t)3)
               : "memory");
}

template <int FMT, int UPS_>
struct PairCfg {
  static constexpr int ROWS = TILE_N;  // weight rows per CTA
  static constexpr int UPS = UPS_;     // 256-token units per stage
  static constexpr int TN = 256 * UPS;
  static constexpr int QV = (FMT == GRETA_FMT_Q4_0) ? 1 : 2;
  static constexpr int DEQ_THREADS = 2 * ROWS;
  static constexpr int THREADS = 64 + DEQ_THREADS;
  static constexpr int RAW_SCALES = 2 * QV * ROWS * 16;
  static constexpr int RAW_STAGE = RAW_SCALES + 2 * ROWS * 4;
  static constexpr int B_STAGE = ROWS * BK * 2;
  static constexpr int HALF_ROWS = 128;  // tokens of a unit that one CTA stages
  static constexpr int HALF_BYTES = HALF_ROWS * BK * 2;
  static constexpr bool Q4 = FMT == GRETA_FMT_Q4_0;
  static constexpr int AU = Q4 ? 8 : 5;
  static constexpr int BS = 4;
  static constexpr int RS = 6;
  static constexpr int U = 2;  // stages per pass of the dequant loop
  static constexpr int NBARS = 2 * AU + 2 * BS + 1;
  static constexpr size_t SMEM = (size_t)AU * HALF_BYTES + (size_t)BS * B_STAGE + (size_t)RS * RAW_STAGE + 1024 + 256;
  static_assert((size_t)TN * ROWS * 2 <= (size_t)AU * HALF_BYTES + (size_t)BS * B_STAGE, "the fp16 output tile is staged in the idle rings");
  static_assert(SMEM <= 232448, "tile configuration exceeds shared memory");
};

template <int FMT, int UPS, bool OUT_F16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<FMT, UPS>::THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const uint8_t *__restrict__ qs, const __half *__restrict__ dsc,
                    void *__restrict__ Cout, uint32_t M, uint32_t N, uint32_t K) {
  using C = PairCfg<FMT, UPS>;
  constexpr int AU = C::AU, BS = C::BS, RS = C::RS, HALF_BYTES = C::HALF_BYTES;
  constexpr int RAW_STAGE = C::RAW_STAGE, B_STAGE = C::B_STAGE, ROWS = C::ROWS, TN = C::TN, COLS = C::TN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *a_units = smem;                       // [AU][128 tokens][128 B]   this CTA's half of each token unit (MMA operand B)
  uint8_t *b_tiles = a_units + AU * HALF_BYTES;  // [BS][128 rows][128 B]     this CTA's weights (MMA operand A)
  uint8_t *raw = b_tiles + BS * B_STAGE;         // [RS] raw quantised stages
  uint64_t *bars = reinterpret_cast<uint64_t *>(raw + RS * RAW_STAGE);
  uint64_t *a_full = bars, *a_empty = bars + AU, *b_full = bars + 2 * AU, *b_empty = bars + 2 * AU + BS, *acc_full = bars + 2 * AU + 2 * BS;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + C::NBARS);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: the CTA whose thread issues the MMAs and whose "full" barriers are used
  const uint32_t n0 = blockIdx.x * ROWS, m0 = blockIdx.y * TN;
  const uint32_t KT = (K + BK - 1) / BK, nb = K / 32;

  if (threadIdx.x == 0) {
    for (int s = 0; s < AU; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&a_empty[s], 1);
    }
    for (int s = 0; s < BS; ++s) {
      mbar_init(&b_full[s], 2 * (C::DEQ_THREADS / 32));  // the dequant warps of both CTAs
      mbar_init(&b_empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
  }
  if (warp == 1) {  // the same warp of both CTAs
    tmem_alloc_pair(tmem_slot, COLS);
    tmem_relinquish_pair();
  }
  const int t = (int)threadIdx.x - 64;
  const int row = t >= 0 ? t % ROWS : 0, hb = t >= 0 ? t / ROWS : 0;
  const uint32_t n_row = min(n0 + (uint32_t)row, N - 1);  // a CTA past the last row tile re-reads the last row and stores nothing
  const uint8_t *qs_row = qs + (size_t)n_row * nb * (C::Q4 ? 16 : 32);
  const __half *d_row = dsc + (size_t)n_row * d_row_stride(nb);
  if (warp >= 2) {
#pragma unroll
    for (int j = 0; j < RS; ++j) {
      if ((uint32_t)j < KT) raw_issue<C>(raw + j * RAW_STAGE, row, hb, qs_row, d_row, j, nb);
      cp_async_commit();
    }
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs: tokens rank * 128 .. + 127 of every unit) ----------------
    if (lane == 0) {
      const uint32_t full0 = map_to_cta(smem_u32(a_full), 0);
      uint32_t u = 0, ph = 1;  // a fresh barrier passes a wait on parity 1: the first round needs no release
      for (uint32_t g = 0; g < KT * UPS; ++g) {
        if (!mbar_wait(&a_empty[u], ph, abort_flag, 100 + u)) break;
        if (rank == 0) mbar_arrive_expect_tx(&a_full[u], 2 * HALF_BYTES);
        tma_load_2d_pair(a_units + u * HALF_BYTES, &tmap_a, (int)((g / UPS) * BK), (int)(m0 + (g % UPS) * 256 + rank * C::HALF_ROWS), full0 + u * 8);
        if (++u == AU) {
          u = 0;
          ph ^= 1;
        }
      }
      if (*abort_flag) {  // copies may still be in flight: leave them time to land before the closing barrier
        const long long t0 = clock64();
        while (clock64() - t0 < 20000000ll) {
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = instr_desc_f16(2 * TILE_N, 256);
      const uint32_t w_lo0 = smem_desc_lo(smem_u32(b_tiles)), a_lo0 = smem_desc_lo(smem_u32(a_units));
      bool ok = true;
      uint32_t s = 0, sph = 0, u = 0, uph = 0, acc = 0;
      for (uint32_t kt = 0; kt < KT && ok; ++kt) {
        ok = mbar_wait(&b_full[s], sph, abort_flag, 300 + s);
        if (!ok) break;
        const uint32_t w_lo = w_lo0 + s * (B_STAGE >> 4);
#pragma unroll
        for (int h = 0; h < UPS; ++h) {
          ok = mbar_wait(&a_full[u], uph, abort_flag, 200 + u);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + u * (HALF_BYTES >> 4);
#pragma unroll
          for (int k16 = 0; k16 < BK / 16; ++k16)
            umma_f16_pair(tmem_base + h * 256, w_lo + k16 * 2, a_lo + k16 * 2, SMEM_DESC_HI_SW128, idesc, k16 == 0 ? acc : 1u);
          umma_commit_pair(&a_empty[u]);
          if (++u == AU) {
            u = 0;
            uph ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(&b_empty[s]);
        acc = 1;
        if (++s == BS) {
          s = 0;
          sph ^= 1;
        }
      }
      if (ok) umma_commit_pair(acc_full);
    }
  } else {
    // ---------------- dequant warps, then epilogue ----------------
    const uint32_t bfull0 = map_to_cta(smem_u32(b_full), 0);
    const uint32_t row_off = row * 128;
    bool ok = dequant_stages<C, C::U>(raw, b_tiles, b_empty, b_full, bfull0, row, hb, row_off, qs_row, d_row, KT, nb, abort_flag, lane);
    if (ok) ok = mbar_wait(acc_full, 0, abort_flag, 500);
    // epilogue: as in the one-CTA kernel; the two warps of a lane quadrant take one half of the tokens each
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const bool staged = OUT_F16 && n0 + ROWS <= N && N % 8 == 0;
    if (ok) {
      tc_fence_after();
      const uint32_t orow = n0 + quad * 32 + lane;
      for (int c = half * (TN / 2); c < (half + 1) * (TN / 2); c += 32) {
        if (m0 + c >= M) break;
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + c, v);
        tmem_ld_wait();
        if (staged) {
          __half *tile = reinterpret_cast<__half *>(smem) + (size_t)c * ROWS + quad * 32 + lane;
#pragma unroll
          for (int j = 0; j < 32; ++j) tile[(size_t)j * ROWS] = __float2half_rn(__uint_as_float(v[j]));
        } else if (orow < N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const uint32_t m = m0 + c + j;
            if (m < M) {
              if (OUT_F16)
                reinterpret_cast<__half *>(Cout)[(size_t)m * N + orow] = __float2half_rn(__uint_as_float(v[j]));
              else
                reinterpret_cast<float *>(Cout)[(size_t)m * N + orow] = __uint_as_float(v[j]);
            }
          }
        }
      }
    }
    if (staged) {
      asm volatile("bar.sync 1, %0;" ::"n"(C::DEQ_THREADS) : "memory");
      if (ok) {
        constexpr uint32_t PIECES_PER_TOKEN = ROWS / 8;
        const uint32_t tokens = min((uint32_t)TN, M - m0);
        for (uint32_t piece = t; piece < tokens * PIECES_PER_TOKEN; piece += C::DEQ_THREADS) {
          const uint32_t tok = piece / PIECES_PER_TOKEN, off = piece % PIECES_PER_TOKEN;
          const uint4 val = *reinterpret_cast<const uint4 *>(smem + ((size_t)tok * ROWS + off * 8) * 2);
          *reinterpret_cast<uint4 *>(reinterpret_cast<__half *>(Cout) + (size_t)(m0 + tok) * N + n0 + off * 8) = val;
        }
      }
    }
  }
  tc_fence_before();
  cluster_sync_all();  // both CTAs are done with each other's barriers and with their tensor memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, COLS);
  }
}

// ---- split over K ------------------------------------------------------------------------------
// Fixed tiles leave SMs idle when there are fewer tiles than SMs, or not a multiple of them (11008 rows x 512
// tokens: 86 tiles on 148 SMs).  Here the work is counted in K stages of 128-row x 512-token tiles and cut into
// one contiguous share per CTA, shares being at most one tile's K loop long, so a CTA runs at most two
// "segments": the end of one tile's K range, then the beginning of the next tile's.  A segment that does not
// start at stage 0 is a contribution: its fp32 accumulator goes to the CTA's slot of a workspace, followed by a
// flag.  The segment that starts a tile owns it: after its own stages it waits (bounded) for the flags of the
// CTAs that hold the rest of the tile's K range, adds their partial sums in ascending K order (so the result
// does not depend on timing) and stores the tile.  The owner's segment is the last thing its CTA does and
// the contributions it needs are the first thing their CTAs do, so it hardly ever waits; the grid is launched
// cooperatively (all CTAs resident), so it cannot wait for a CTA that has not started.
// Flags carry a launch number that is unique in the process: nothing has to be cleared between launches.
struct SplitPlan {
  uint32_t share;        // K stages per CTA (<= KT)
  uint32_t KT;           // K stages per tile
  uint32_t units;        // tiles * KT
  uint32_t token_tiles;  // tiles along the tokens (tile index = row tile * token_tiles + token tile)
  unsigned long long epoch;
  float *partials;               // [CTAs][512 / 32 token chunks][4 lane quadrants][8 pieces][32 lanes][4] fp32
  unsigned long long *flags;     // [CTAs]
};
constexpr size_t SPLIT_PARTIAL_FLOATS = (size_t)TILE_N * 512;

template <int FMT, bool OUT_F16>
__global__ void __launch_bounds__(Cfg<FMT, 512, 1>::THREADS, 1)
gemm_tc_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const uint8_t *__restrict__ qs, const __half *__restrict__ dsc,
                      void *__restrict__ Cout, uint32_t M, uint32_t N, uint32_t K, const SplitPlan plan) {
  using C = Cfg<FMT, 512, 1>;
  constexpr int AU = C::AU, BS = C::BS, RS = C::RS, UPS = C::UPS, UNIT_BYTES = C::UNIT_BYTES, UNIT_ROWS = C::UNIT_ROWS;
  constexpr int RAW_STAGE = C::RAW_STAGE, B_STAGE = C::B_STAGE, ROWS = C::ROWS, TN = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *a_units = smem;
  uint8_t *b_tiles = a_units + AU * UNIT_BYTES;
  uint8_t *raw = b_tiles + BS * B_STAGE;
  uint64_t *bars = reinterpret_cast<uint64_t *>(raw + RS * RAW_STAGE);
  uint64_t *a_full = bars, *a_empty = bars + AU, *b_full = bars + 2 * AU, *b_empty = bars + 2 * AU + BS;
  uint64_t *acc_full = bars + 2 * AU + 2 * BS, *acc_empty = bars + C::NBARS;  // one barrier more than the tiled kernel: the accumulator handed back
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + C::NBARS + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t KT = plan.KT, nb = K / 32;
  // this CTA's share [u0, u1) of the stage units, as at most two segments
  const uint32_t u0 = min(blockIdx.x * plan.share, plan.units), u1 = min(u0 + plan.share, plan.units);
  uint32_t seg_tile[2], seg_k0[2], seg_k1[2], nseg = 0;
  for (uint32_t u = u0; u < u1;) {
    const uint32_t tile = u / KT, k0 = u - tile * KT, k1 = min(KT, k0 + (u1 - u));
    seg_tile[nseg] = tile;
    seg_k0[nseg] = k0;
    seg_k1[nseg] = k1;
    ++nseg;
    u += k1 - k0;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < AU; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&a_empty[s], 1);
    }
    for (int s = 0; s < BS; ++s) {
      mbar_init(&b_full[s], C::DEQ_THREADS / 32);
      mbar_init(&b_empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, C::DEQ_THREADS / 32);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
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
      uint32_t u = 0, ph = 1, issued = 0;  // a fresh barrier passes a wait on parity 1
      bool ok = true;
      for (uint32_t sg = 0; sg < nseg && ok; ++sg) {
        const uint32_t m0 = (seg_tile[sg] % plan.token_tiles) * TN;
        for (uint32_t kt = seg_k0[sg]; kt < seg_k1[sg] && ok; ++kt) {
#pragma unroll
          for (int h = 0; h < UPS; ++h) {
            ok = mbar_wait(&a_empty[u], ph, abort_flag, 100 + u);
            if (!ok) break;
            mbar_arrive_expect_tx(&a_full[u], UNIT_BYTES);
            tma_load_2d(a_units + u * UNIT_BYTES, &tmap_a, (int)(kt * BK), (int)(m0 + h * UNIT_ROWS), &a_full[u]);
            ++issued;
            if (++u == AU) {
              u = 0;
              ph ^= 1;
            }
          }
        }
      }
      if (*abort_flag) {  // give the copies still in flight a bounded chance to land before the CTA exits
        for (uint32_t j = issued > (uint32_t)AU ? issued - AU : 0; j < issued; ++j) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&a_full[j % AU], (j / AU) & 1) && clock64() - t0 < 20000000ll) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_f16(TILE_N, UNIT_ROWS);
      const uint32_t w_lo0 = smem_desc_lo(smem_u32(b_tiles)), a_lo0 = smem_desc_lo(smem_u32(a_units));
      bool ok = true;
      uint32_t s = 0, sph = 0, u = 0, uph = 0;
      for (uint32_t sg = 0; sg < nseg && ok; ++sg) {
        if (sg > 0) {  // the accumulator of the segment before has been read out
          ok = mbar_wait(acc_empty, (sg - 1) & 1, abort_flag, 600);
          if (!ok) break;
          tc_fence_after();
        }
        uint32_t acc = 0;
        for (uint32_t kt = seg_k0[sg]; kt < seg_k1[sg] && ok; ++kt) {
          ok = mbar_wait(&b_full[s], sph, abort_flag, 300 + s);
          if (!ok) break;
          const uint32_t w_lo = w_lo0 + s * (B_STAGE >> 4);
#pragma unroll
          for (int h = 0; h < UPS; ++h) {
            ok = mbar_wait(&a_full[u], uph, abort_flag, 200 + u);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_lo = a_lo0 + u * (UNIT_BYTES >> 4);
#pragma unroll
            for (int k16 = 0; k16 < BK / 16; ++k16)
              umma_f16(tmem_base + h * UNIT_ROWS, w_lo + k16 * 2, a_lo + k16 * 2, SMEM_DESC_HI_SW128, idesc, k16 == 0 ? acc : 1u);
            umma_commit(&a_empty[u]);
            if (++u == AU) {
              u = 0;
              uph ^= 1;
            }
          }
          if (!ok) break;
          umma_commit(&b_empty[s]);
          acc = 1;
          if (++s == BS) {
            s = 0;
            sph ^= 1;
          }
        }
        if (ok) umma_commit(acc_full);
      }
    }
  } else {
    // ---------------- dequant warps; after each segment's stages, its epilogue ----------------
    const int t = (int)threadIdx.x - 64;
    const int row = t % ROWS, hb = t / ROWS;
    const uint32_t row_off = row * 128;
    const int quad = warp & 3, half = (warp - 2) >> 2;
    bool ok = true;
    uint32_t s = 0, sph = 1;
    auto prologue = [&](uint32_t sg) {  // requests the first RS - 1 raw stages of segment sg
      const uint32_t nr = min((seg_tile[sg] / plan.token_tiles) * ROWS + (uint32_t)row, N - 1);
      const uint8_t *qr = qs + (size_t)nr * nb * (C::Q4 ? 16 : 32);
      const __half *dr = dsc + (size_t)nr * d_row_stride(nb);
#pragma unroll
      for (int j = 0; j < RS - 1; ++j) {
        if (seg_k0[sg] + j < seg_k1[sg]) raw_issue<C>(raw + j * RAW_STAGE, row, hb, qr, dr, seg_k0[sg] + j, nb);
        cp_async_commit();
      }
    };
    for (uint32_t sg = 0; sg < nseg && ok; ++sg) {
      const uint32_t tile = seg_tile[sg], k0 = seg_k0[sg], k1 = seg_k1[sg];
      const uint32_t n0 = (tile / plan.token_tiles) * ROWS, m0 = (tile % plan.token_tiles) * TN;
      const uint32_t n_row = min(n0 + (uint32_t)row, N - 1);
      const uint8_t *qs_row = qs + (size_t)n_row * nb * (C::Q4 ? 16 : 32);
      const __half *d_row = dsc + (size_t)n_row * d_row_stride(nb);
      if (sg == 0) prologue(0);  // a later segment's first stages were requested before the epilogue of the one before
      uint32_t rs_load = RS - 1, rs_use = 0;
      for (uint32_t kt = k0; kt < k1; ++kt) {
        if (kt + RS - 1 < k1) raw_issue<C>(raw + rs_load * RAW_STAGE, row, hb, qs_row, d_row, kt + RS - 1, nb);
        cp_async_commit();
        cp_async_wait<RS - 1>();
        uint4 chunk[4];
        dequant_block<C>(raw + rs_use * RAW_STAGE, row, hb, 2 * kt + hb < nb, chunk);
        ok = mbar_wait(&b_empty[s], sph, abort_flag, 400 + s);
        if (!ok) break;
        uint8_t *row_base = b_tiles + s * B_STAGE + row_off;
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4 *>(row_base + (((4 * hb + c) ^ (row & 7)) << 4)) = chunk[c];
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&b_full[s]);
        if (++s == BS) {
          s = 0;
          sph ^= 1;
        }
        if (++rs_load == RS) rs_load = 0;
        if (++rs_use == RS) rs_use = 0;
      }
      cp_async_wait<0>();
      if (!ok) break;
      if (sg + 1 < nseg) prologue(sg + 1);  // travels while this segment's accumulator is read out
      ok = mbar_wait(acc_full, sg & 1, abort_flag, 500);
      if (!ok) break;
      tc_fence_after();
      const uint32_t orow = n0 + quad * 32 + lane;
      if (k0 > 0) {
        // ---- contribution: the fp32 accumulator goes to this CTA's slot, then the flag
        float *slot = plan.partials + (size_t)blockIdx.x * SPLIT_PARTIAL_FLOATS;
        for (int c = half * (TN / 2); c < (half + 1) * (TN / 2); c += 32) {
          if (m0 + c >= M) break;
          uint32_t v[32];
          tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + c, v);
          tmem_ld_wait();
          // piece j of lane l at 16-byte index j * 32 + l of the warp's 4 KB: every store instruction writes 512 contiguous bytes
          uint4 *dst = reinterpret_cast<uint4 *>(slot + ((size_t)(c >> 5) * ROWS + quad * 32) * 32) + lane;
#pragma unroll
          for (int j = 0; j < 8; ++j) dst[j * 32] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(C::DEQ_THREADS) : "memory");
        if (t == 0) {
          asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(plan.flags + blockIdx.x), "l"(plan.epoch) : "memory");
        }
      } else {
        // ---- this CTA stores the tile; when its stages end before the tile's K does, the rest comes from the CTAs after it
        const bool staged = OUT_F16 && n0 + ROWS <= N && N % 8 == 0;
        uint32_t first_c = 0, n_contrib = 0;  // contributors are CTAs blockIdx.x + 1 .. + n_contrib
        if (k1 < KT) {
          first_c = blockIdx.x + 1;
          n_contrib = (KT - k1 + plan.share - 1) / plan.share;
          if (t < (int)n_contrib) {  // one thread per contributor waits for its flag
            const unsigned long long *f = plan.flags + first_c + t;
            const long long t0 = clock64();
            for (;;) {
              unsigned long long got;
              asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(got) : "l"(f) : "memory");
              if (got == plan.epoch) break;
              if (*abort_flag) break;
              if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                *abort_flag = 700;
                atomicCAS(&g_gemm_error, 0, 700);
                break;
              }
              __nanosleep(200);
            }
          }
          asm volatile("bar.sync 1, %0;" ::"n"(C::DEQ_THREADS) : "memory");
          if (*abort_flag) ok = false;
        }
        if (ok) {
          for (int c = half * (TN / 2); c < (half + 1) * (TN / 2); c += 32) {
            if (m0 + c >= M) break;
            uint32_t v[32];
            tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + c, v);
            tmem_ld_wait();
            for (uint32_t ci = 0; ci < n_contrib; ++ci) {  // ascending K order
              const float4 *src = reinterpret_cast<const float4 *>(plan.partials + (size_t)(first_c + ci) * SPLIT_PARTIAL_FLOATS +
                                                                   ((size_t)(c >> 5) * ROWS + quad * 32) * 32) + lane;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 a = __ldcg(src + j * 32);
                v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + a.x);
                v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + a.y);
                v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + a.z);
                v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + a.w);
              }
            }
            if (staged) {
              __half *tile_h = reinterpret_cast<__half *>(smem) + (size_t)c * ROWS + quad * 32 + lane;
#pragma unroll
              for (int j = 0; j < 32; ++j) tile_h[(size_t)j * ROWS] = __float2half_rn(__uint_as_float(v[j]));
            } else if (orow < N) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const uint32_t m = m0 + c + j;
                if (m < M) {
                  if (OUT_F16)
                    reinterpret_cast<__half *>(Cout)[(size_t)m * N + orow] = __float2half_rn(__uint_as_float(v[j]));
                  else
                    reinterpret_cast<float *>(Cout)[(size_t)m * N + orow] = __uint_as_float(v[j]);
                }
              }
            }
          }
        }
        if (staged) {  // the segment that stores a tile is the CTA's last: the rings are idle
          asm volatile("bar.sync 1, %0;" ::"n"(C::DEQ_THREADS) : "memory");
          if (ok) {
            constexpr uint32_t PIECES_PER_TOKEN = ROWS / 8;
            const uint32_t tokens = min((uint32_t)TN, M - m0);
            for (uint32_t piece = t; piece < tokens * PIECES_PER_TOKEN; piece += C::DEQ_THREADS) {
              const uint32_t tok = piece / PIECES_PER_TOKEN, off = piece % PIECES_PER_TOKEN;
              const uint4 val = *reinterpret_cast<const uint4 *>(smem + ((size_t)tok * ROWS + off * 8) * 2);
              *reinterpret_cast<uint4 *>(reinterpret_cast<__half *>(Cout) + (size_t)(m0 + tok) * N + n0 + off * 8) = val;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
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

template <int FMT, int TN, int RT, bool OUT_F16>
int launch_tc(cudaStream_t stream, const CUtensorMap &map, const void *qs, const void *d, void *C, uint32_t M, uint32_t N, uint32_t K) {
  using Cf = Cfg<FMT, TN, RT>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    GRETA_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<FMT, TN, RT, OUT_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cf::SMEM));
    attr_set[dev] = true;
  }
  dim3 grid((N + Cf::ROWS - 1) / Cf::ROWS, (M + TN - 1) / TN);
  gemm_tc_kernel<FMT, TN, RT, OUT_F16><<<grid, Cf::THREADS, Cf::SMEM, stream>>>(map, (const uint8_t *)qs, (const __half *)d, C, M, N, K);
  return launched("gemm_tc_kernel");
}

void pick_tile(uint32_t M, uint32_t N, int *tn, int *rt);

size_t split_scratch_bytes() {
  const size_t ctas = (size_t)sm_count();
  return (ctas * SPLIT_PARTIAL_FLOATS * 4 + ctas * 8 + 255) / 256 * 256;
}
unsigned long long next_split_epoch() {
  static std::atomic<unsigned long long> counter{0};
  static const unsigned long long base = ((unsigned long long)std::chrono::steady_clock::now().time_since_epoch().count() << 16) | 1ull;
  return base + counter.fetch_add(1);
}

// Whether the split over K pays for this shape, and the plan if so: 512-token tiles, fewer tiles than SMs (or not many
// more: above that the tiled kernel's waves are full enough), shares of at least 8 stages.
bool plan_splitk(uint32_t M, uint32_t N, uint32_t K, SplitPlan *pl, uint32_t *ctas) {
  const uint32_t row_tiles = (N + TILE_N - 1) / TILE_N, token_tiles = (M + 511) / 512, tiles = row_tiles * token_tiles;
  const uint32_t KT = (K + BK - 1) / BK, sms = (uint32_t)sm_count();
  if (M <= 256 || M % 512 > 0 && M % 512 <= 256) return false;  // a token tile that is mostly padding
  if (tiles >= sms || (uint64_t)tiles * KT >= (1ull << 31)) return false;
  const uint32_t units = tiles * KT;
  uint32_t share = (units + sms - 1) / sms;
  if (share < 8) share = 8;
  if (share > KT) return false;
  // Worth it?  In units of one 512-token stage: the tiled kernel needs waves * KT stages of its tile width (a 256-token
  // stage costs about 0.8 of a 512-token one, a 128-token stage 0.66: the issuing thread, not the tensor core, sets
  // their pace), the split needs one share plus about 24 stages' worth of partial sums, flags and a second pipeline start
  // (measured: 11008 x 4096 at 512 tokens 48.7 vs 50.3 us, 4096 x 11008 55 vs 83, 12288 x 4096 52.1 vs 51.1).
  int tn = 128, rt = 1;
  pick_tile(M, N, &tn, &rt);
  const uint32_t tile_ctas = ((N + TILE_N * rt - 1) / (TILE_N * rt)) * ((M + tn - 1) / tn);
  const double per_stage = tn == 512 ? 1.0 : (tn == 256 ? 0.8 : 0.66);
  if (tuning().gemm_splitk != 2 && share + 24.0 >= (double)((tile_ctas + sms - 1) / sms) * KT * per_stage * rt) return false;  // 2: whenever feasible
  pl->share = share;
  pl->KT = KT;
  pl->units = units;
  pl->token_tiles = token_tiles;
  *ctas = (units + share - 1) / share;
  return *ctas <= sms;
}

template <int FMT, bool OUT_F16>
int launch_splitk(cudaStream_t stream, const CUtensorMap &map, const void *qs, const void *d, void *C, uint32_t M, uint32_t N, uint32_t K,
                  SplitPlan plan, uint32_t ctas, void *scratch) {
  using Cf = Cfg<FMT, 512, 1>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    GRETA_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_splitk_kernel<FMT, OUT_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cf::SMEM));
    attr_set[dev] = true;
  }
  plan.partials = static_cast<float *>(scratch);
  plan.flags = reinterpret_cast<unsigned long long *>(static_cast<uint8_t *>(scratch) + (size_t)sm_count() * SPLIT_PARTIAL_FLOATS * 4);
  plan.epoch = next_split_epoch();
  const uint8_t *qs8 = static_cast<const uint8_t *>(qs);
  const __half *d16 = static_cast<const __half *>(d);
  void *args[] = {(void *)&map, (void *)&qs8, (void *)&d16, (void *)&C, (void *)&M, (void *)&N, (void *)&K, (void *)&plan};
  // cooperative: every CTA is resident, so a tile's owner never waits for a CTA that has not started
  GRETA_CUDA_TRY(cudaLaunchCooperativeKernel((const void *)gemm_tc_splitk_kernel<FMT, OUT_F16>, dim3(ctas), dim3(Cf::THREADS), args, Cf::SMEM, stream));
  return launched("gemm_tc_splitk_kernel");
}

template <int FMT, int UPS, bool OUT_F16>
int launch_pair(cudaStream_t stream, const CUtensorMap &map, const void *qs, const void *d, void *C, uint32_t M, uint32_t N, uint32_t K) {
  using Cf = PairCfg<FMT, UPS>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    GRETA_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_pair_kernel<FMT, UPS, OUT_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cf::SMEM));
    attr_set[dev] = true;
  }
  const uint32_t row_tiles = (N + TILE_N - 1) / TILE_N;
  dim3 grid((row_tiles + 1) / 2 * 2, (M + Cf::TN - 1) / Cf::TN);  // whole pairs
  gemm_tc_pair_kernel<FMT, UPS, OUT_F16><<<grid, Cf::THREADS, Cf::SMEM, stream>>>(map, (const uint8_t *)qs, (const __half *)d, C, M, N, K);
  return launched("gemm_tc_pair_kernel");
}

template <int FMT, bool OUT_F16>
int dispatch_tile(cudaStream_t stream, const CUtensorMap &map, int tn, int rt, const void *qs, const void *d, void *C, uint32_t M, uint32_t N,
                  uint32_t K) {
  if (rt == 2) {
    if (tn == 256) return launch_tc<FMT, 256, 2, OUT_F16>(stream, map, qs, d, C, M, N, K);
    return launch_tc<FMT, 128, 2, OUT_F16>(stream, map, qs, d, C, M, N, K);
  }
  if (tn == 512) return launch_tc<FMT, 512, 1, OUT_F16>(stream, map, qs, d, C, M, N, K);
  if (tn == 256) return launch_tc<FMT, 256, 1, OUT_F16>(stream, map, qs, d, C, M, N, K);
  return launch_tc<FMT, 128, 1, OUT_F16>(stream, map, qs, d, C, M, N, K);
}

// Tile shape (tokens x 128-row tiles per CTA): the widest token tile that still leaves most SMs a CTA.
// With one MMA row tile per CTA the token operand is written to shared memory once and read once per
// stage, and together with the weight tile that traffic (about 185 KB per 64-K stage at 512 tokens), not
// the tensor core, sets the pace; the two-row-tile shapes move no less of it and have a shallower
// weight ring, so they are never picked here.  The tuning switch gemm_tile (<tokens>x<row tiles>) forces one
// (512x1, 256x1, 128x1, 256x2, 128x2).
void pick_tile(uint32_t M, uint32_t N, int *tn, int *rt) {
  *rt = 1;
  {
    const int a = tuning().gemm_tile_tokens, b = tuning().gemm_tile_rows;
    if ((a == 128 || a == 256 || a == 512) && (b == 1 || b == 2) && a * b <= 512) {
      *tn = a;
      *rt = b;
      return;
    }
  }
  const uint32_t row_tiles = (N + TILE_N - 1) / TILE_N;
  const int widths[3] = {512, 256, 128};
  for (int w : widths) {
    *tn = w;
    if (w > 128 && M <= (uint32_t)w / 2) continue;  // would be mostly padding
    if (row_tiles * ((M + w - 1) / w) >= 80) return;
  }
}

}  // namespace

extern "C" {

size_t greta_cuda_gemm_workspace_bytes(uint32_t M, uint32_t K) { return split_scratch_bytes() + ((size_t)M * K * 2 + 255) / 256 * 256; }

// Which kernel greta_cuda_gemm would launch for this shape with the tuning switches as they stand, without launching it:
// kind 0 = tiled (ctas = tiles of tile_tokens x 128 * row tiles), 1 = CTA pairs, 2 = split over K (ctas CTAs of `share` K
// stages each).  Host arithmetic only.
int greta_cuda_gemm_route(uint32_t M, uint32_t N, uint32_t K, int has_workspace, int *kind, uint32_t *ctas, uint32_t *share, uint32_t *tile_tokens) {
  GRETA_REQUIRE(kind && ctas && share && tile_tokens, "gemm_route: null out pointer");
  GRETA_REQUIRE(M && N && K && K % 32 == 0, "gemm_route: M=%u N=%u K=%u", M, N, K);
  int tn = 128, rt = 1;
  pick_tile(M, N, &tn, &rt);
  const bool pair = tuning().gemm_pair == 2 || (tuning().gemm_pair == 1 && tn == 512 && rt == 1 && tuning().gemm_tile_tokens == 0);
  SplitPlan sp{};
  uint32_t sc = 0;
  if (tuning().gemm_splitk && !pair && has_workspace && tuning().gemm_tile_tokens == 0 && plan_splitk(M, N, K, &sp, &sc)) {
    *kind = 2;
    *ctas = sc;
    *share = sp.share;
    *tile_tokens = 512;
    return GRETA_OK;
  }
  *share = (K + BK - 1) / BK;
  if (pair) {
    *kind = 1;
    *tile_tokens = 512;
    *ctas = (((N + TILE_N - 1) / TILE_N + 1) / 2 * 2) * ((M + 511) / 512);
    return GRETA_OK;
  }
  *kind = 0;
  *tile_tokens = (uint32_t)tn;
  *ctas = ((N + TILE_N * rt - 1) / (TILE_N * rt)) * ((M + tn - 1) / tn);
  return GRETA_OK;
}

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
    void *a_area = static_cast<uint8_t *>(workspace) + split_scratch_bytes();  // the front of the workspace is the split-K scratch
    if (int rc = greta_cuda_f32_to_f16(stream, static_cast<const float *>(A), a_area, (size_t)M * K)) return rc;
    a16 = a_area;
  }
  EncodeTiledFn enc = encode_tiled();
  if (!enc) {
    set_error("gemm: cuTensorMapEncodeTiled is not available from this driver");
    return GRETA_ERR_NOT_IMPLEMENTED;
  }
  int tn = 128, rt = 1;
  pick_tile(M, N, &tn, &rt);
  // 512-token tiles run as CTA pairs unless a tile shape is forced or the switch is off (2: always, whatever the shape)
  const bool pair = tuning().gemm_pair == 2 || (tuning().gemm_pair == 1 && tn == 512 && rt == 1 && tuning().gemm_tile_tokens == 0);
  SplitPlan splan;
  uint32_t split_ctas = 0;
  const bool split = tuning().gemm_splitk && !pair && workspace && aligned16(workspace) && tuning().gemm_tile_tokens == 0 &&
                     plan_splitk(M, N, K, &splan, &split_ctas);
  const cuuint64_t dims[2] = {K, M};
  CUtensorMap map;
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {BK, ((tn >= 256 && !pair) || split) ? 256u : 128u};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(a16), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("gemm: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return GRETA_ERR_INVALID_ARGS;
  }
  if (split) {
    if (fmt == GRETA_FMT_Q4_0)
      return c_is_f16 ? launch_splitk<GRETA_FMT_Q4_0, true>(s, map, qs, d, Cout, M, N, K, splan, split_ctas, workspace)
                      : launch_splitk<GRETA_FMT_Q4_0, false>(s, map, qs, d, Cout, M, N, K, splan, split_ctas, workspace);
    return c_is_f16 ? launch_splitk<GRETA_FMT_Q8_0, true>(s, map, qs, d, Cout, M, N, K, splan, split_ctas, workspace)
                    : launch_splitk<GRETA_FMT_Q8_0, false>(s, map, qs, d, Cout, M, N, K, splan, split_ctas, workspace);
  }
  if (pair) {
    if (fmt == GRETA_FMT_Q4_0)
      return c_is_f16 ? launch_pair<GRETA_FMT_Q4_0, 2, true>(s, map, qs, d, Cout, M, N, K) : launch_pair<GRETA_FMT_Q4_0, 2, false>(s, map, qs, d, Cout, M, N, K);
    return c_is_f16 ? launch_pair<GRETA_FMT_Q8_0, 2, true>(s, map, qs, d, Cout, M, N, K) : launch_pair<GRETA_FMT_Q8_0, 2, false>(s, map, qs, d, Cout, M, N, K);
  }
  if (fmt == GRETA_FMT_Q4_0)
    return c_is_f16 ? dispatch_tile<GRETA_FMT_Q4_0, true>(s, map, tn, rt, qs, d, Cout, M, N, K) : dispatch_tile<GRETA_FMT_Q4_0, false>(s, map, tn, rt, qs, d, Cout, M, N, K);
  return c_is_f16 ? dispatch_tile<GRETA_FMT_Q8_0, true>(s, map, tn, rt, qs, d, Cout, M, N, K) : dispatch_tile<GRETA_FMT_Q8_0, false>(s, map, tn, rt, qs, d, Cout, M, N, K);
}

}  // extern "C"
