// Counter-based synthetic tensors for the benchmark configurations: GGUF Q4_0 /
// Q8_0 blocks with uniform quants and |N(0, sigma)| / 8 (or / 127) scales, and
// normal fp16 / fp32 values.  Every value is a pure function of (seed, stream,
// index), so any slice of any tensor can be produced independently - by a rank
// that holds only a shard, or by a CPU checker that wants the same bytes.
#include <cmath>
#include <cstring>

#include "gcore/greta_b200.hpp"
#include "host_util.hpp"

namespace gcore::inference::synth {

namespace {
inline uint64_t mix(uint64_t seed, uint64_t stream, uint64_t idx) {
  uint64_t z = seed * 0x9E3779B97F4A7C15ull + stream * 0xD1B54A32D192ED03ull + idx * 0x94D049BB133111EBull + 0x2545F4914F6CDD1Dull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
inline double uniform01(uint64_t r) { return ((r >> 11) + 0.5) * (1.0 / 9007199254740992.0); }  // (0, 1)
// One standard normal per index (Box-Muller on two independent draws).
inline double normal(uint64_t seed, uint64_t stream, uint64_t idx) {
  double u1 = uniform01(mix(seed, stream, 2 * idx)), u2 = uniform01(mix(seed, stream, 2 * idx + 1));
  return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586476925 * u2);
}
}  // namespace

uint64_t tensor_stream(uint32_t layer, int which) { return (uint64_t)layer * 16 + (uint64_t)which; }

void quant_blocks(uint64_t seed, uint64_t stream, gcore::rt::GretaDataType fmt, uint8_t *out, size_t first_block, size_t n_blocks,
                  float sigma) {
  const bool q4 = fmt == gcore::rt::GretaDataType::Q4_0;
  const size_t bb = q4 ? 18 : 34;
  const uint64_t s_scale = stream * 2 + 0, s_q = stream * 2 + 1;
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n_blocks; ++i) {
    const uint64_t b = first_block + i;
    uint8_t *blk = out + i * bb;
    float d = (float)(std::fabs(normal(seed, s_scale, b)) * sigma / (q4 ? 8.0 : 127.0));
    uint16_t dh = host::f32_to_f16(d);
    std::memcpy(blk, &dh, 2);
    if (q4) {
      uint64_t r0 = mix(seed, s_q, 2 * b), r1 = mix(seed, s_q, 2 * b + 1);
      std::memcpy(blk + 2, &r0, 8);
      std::memcpy(blk + 10, &r1, 8);
    } else {
      for (int w = 0; w < 4; ++w) {
        uint64_t r = mix(seed, s_q, 4 * b + w);
        for (int j = 0; j < 8; ++j) {
          int q = (int)((r >> (8 * j)) & 0xFF) % 255 - 127;  // uniform in [-127, 127]
          blk[2 + 8 * w + j] = (uint8_t)(int8_t)q;
        }
      }
    }
  }
}

void normal_f32(uint64_t seed, uint64_t stream, float sigma, float *out, size_t first, size_t n) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; ++i) out[i] = (float)(normal(seed, stream, first + i) * sigma);
}
void normal_f16(uint64_t seed, uint64_t stream, float sigma, uint16_t *out, size_t first, size_t n) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; ++i) out[i] = host::f32_to_f16((float)(normal(seed, stream, first + i) * sigma));
}
void normal_f16_as_f32(uint64_t seed, uint64_t stream, float sigma, float *out, size_t first, size_t n) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; ++i) out[i] = host::f16_to_f32(host::f32_to_f16((float)(normal(seed, stream, first + i) * sigma)));
}
void tokens(uint64_t seed, uint64_t stream, uint32_t vocab, int32_t *out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = (int32_t)(mix(seed, stream, i) % vocab);
}

}  // namespace gcore::inference::synth
