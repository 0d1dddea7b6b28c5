// C entry points around host-side checkers that the reference keeps INSIDE its block scheduler
// (src/inference/src/block_scheduler.cpp): the CPU attention references compute_attention_ref_fp32 /
// _fp64 (:721-864), the host dequantiser read_weight_value (:639-671) with its weight-cache struct
// (:584-593) and fp16 decoder (:547-567).  That file does not compile without the HIP toolkit, so the
// build recipe (oracle/Makefile, target `ref`) cuts exactly those definitions out of the reference
// source where it lies, by their signatures, into _ref/block_scheduler_extract.inc at build time;
// nothing of the reference is stored in this repository.  Test infrastructure only.
#include <gcore/rt/greta_runtime.hpp>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "_ref/block_scheduler_extract.inc"

#define RAPI extern "C" __attribute__((visibility("default")))

// mode 0: compute_attention_ref_fp64; mode 1: compute_attention_ref_fp32.  Caches are fp32 [Hkv][max_seq][Dh].
RAPI void ref_sched_attention(const float *q, const float *k_cache, const float *v_cache, uint32_t num_heads, uint32_t num_heads_kv,
                              uint32_t head_dim, uint32_t seq_len, uint32_t max_seq_len, float scale, int mode, float *out) {
  std::vector<float> o;
  if (mode == 0)
    compute_attention_ref_fp64(q, k_cache, v_cache, num_heads, num_heads_kv, head_dim, seq_len, max_seq_len, (double)scale, o);
  else
    compute_attention_ref_fp32(q, k_cache, v_cache, num_heads, num_heads_kv, head_dim, seq_len, max_seq_len, scale, o);
  std::memcpy(out, o.data(), o.size() * sizeof(float));
}

// read_weight_value over a whole tensor.  type: GretaDataType value (INT8 = 3, INT4 = 4, FP16 = 1, FP32 = 0).
RAPI void ref_sched_read_weights(int type, const uint8_t *raw, size_t raw_bytes, const float *scales, size_t n_scales, uint32_t group_size,
                                 size_t elems, float *out) {
  QkvWeightHostCache c;
  c.ready = true;
  c.type = static_cast<gcore::rt::GretaDataType>(type);
  c.bytes = raw_bytes;
  c.elems = elems;
  c.group_size = group_size;
  c.raw.assign(raw, raw + raw_bytes);
  if (scales) c.scales.assign(scales, scales + n_scales);
  for (size_t i = 0; i < elems; ++i) out[i] = read_weight_value(c, i);
}
