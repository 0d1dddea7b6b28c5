// C entry points around the reference's OWN host code, compiled from the
// reference sources where they lie (see oracle/Makefile, target `ref`).  Used to
// pin the CPU oracle and to generate the golden vectors under tests/golden/.
// Test infrastructure only; nothing here is part of the product.
#include <gcore/inference/weight_loader.hpp>
#include <gcore/rt/ref/cpu_reference.hpp>

#include <cstdint>
#include <cstring>
#include <string>

using gcore::rt::ref::CpuReference;
#define RAPI extern "C" __attribute__((visibility("default")))

RAPI float ref_half_to_float(uint16_t h) { return CpuReference::half_to_float(h); }
RAPI uint16_t ref_float_to_half(float f) { return CpuReference::float_to_half(f); }
RAPI void ref_cpu_gemm(const float *A, const float *B, float *C, int M, int N, int K) {
  CpuReference::gemm(A, B, C, M, N, K);
}
RAPI void ref_cpu_rmsnorm(const float *x, float *y, const float *w, int rows, int cols, float eps) {
  CpuReference::rmsnorm(x, y, w, rows, cols, eps);
}
RAPI void ref_cpu_softmax(const float *x, float *y, int rows, int cols) {
  CpuReference::softmax(x, y, rows, cols);
}

// GGUFLoader::load_tensor_int8: Q8_0 tensor -> int8 plane + fp32 scales.
RAPI int ref_gguf_load_int8(const char *path, const char *name, int8_t *w, size_t w_cap, float *scales,
                            size_t s_cap) {
  std::string err;
  gcore::inference::GGUFLoader ld;
  if (!ld.open(path, &err)) return 1;
  gcore::rt::hip::Buffer wb, sb;
  if (!ld.load_tensor_int8(name, wb, sb, &err)) return 2;
  if (wb.size() > w_cap || sb.size() > s_cap * 4) return 3;
  std::memcpy(w, wb.data(), wb.size());
  std::memcpy(scales, sb.data(), sb.size());
  return 0;
}

// GGUFLoader::load_tensor_int4: F32/F16 tensor -> the reference's INT4 packing,
// group scales and per-head scales.
RAPI int ref_gguf_load_int4(const char *path, const char *name, uint8_t *packed, size_t p_cap, float *scales,
                            size_t s_cap, float *head_scales, size_t h_cap, uint32_t *n_heads_out) {
  std::string err;
  gcore::inference::GGUFLoader ld;
  if (!ld.open(path, &err)) return 1;
  gcore::rt::hip::Buffer wb, sb, hb;
  if (!ld.load_tensor_int4(name, wb, sb, hb, &err)) return 2;
  if (wb.size() > p_cap || sb.size() > s_cap * 4 || hb.size() > h_cap * 4) return 3;
  std::memcpy(packed, wb.data(), wb.size());
  std::memcpy(scales, sb.data(), sb.size());
  if (hb.size()) std::memcpy(head_scales, hb.data(), hb.size());
  if (n_heads_out) *n_heads_out = (uint32_t)(hb.size() / 4);
  return 0;
}

// GGUFLoader::load_tensor: F32 / F16 / Q4_K / Q6_K tensor -> fp32 (weight_loader.cpp:520-570).
RAPI int ref_gguf_load_fp32(const char *path, const char *name, float *out, size_t cap) {
  std::string err;
  gcore::inference::GGUFLoader ld;
  if (!ld.open(path, &err)) return 1;
  gcore::rt::hip::Buffer b;
  if (!ld.load_tensor(name, b, &err)) return 2;
  if (b.size() > cap * 4) return 3;
  std::memcpy(out, b.data(), b.size());
  return 0;
}

// GGUFLoader::get_config after open(): the model shape the reference parses.
RAPI int ref_gguf_config(const char *path, uint32_t *out10) {
  std::string err;
  gcore::inference::GGUFLoader ld;
  if (!ld.open(path, &err)) return 1;
  auto c = ld.get_config();
  out10[0] = c.dim; out10[1] = c.num_heads; out10[2] = c.num_heads_kv; out10[3] = c.num_layers;
  out10[4] = c.vocab_size; out10[5] = c.hidden_dim; out10[6] = c.head_dim; out10[7] = c.max_seq_len;
  std::memcpy(&out10[8], &c.rope_base, 4); std::memcpy(&out10[9], &c.rms_eps, 4);
  return 0;
}
