// GGUF file -> device layout: the reference's WeightLoader / GGUFLoader interface
// (src/inference/include/gcore/inference/weight_loader.hpp:14-92, src/inference/src/weight_loader.cpp:210-505) and
// BlockScheduler::load_weights (src/inference/src/block_scheduler.cpp:1511-1623).
//
// The reference parses the file, then RE-QUANTISES every projection to its own INT4 / INT8 planes on the host
// (weight_loader.cpp:668-1005) and cannot load Q4_0 at all (load_tensor_int4 rejects it, :857-875).  Here the GGUF
// blocks are the storage format: a Q4_0 / Q8_0 tensor's blocks go to the device as they lie in the file and are split
// there into the payload plane and the scale plane (greta_cuda_repack_gguf); norms travel as fp32, the embedding and the
// LM head as fp16.  Nothing is re-quantised, so what the kernels multiply is bit for bit what the file holds.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <map>

#include "gcore/greta_b200.hpp"
#include "host_util.hpp"

namespace gcore::inference {

using gcore::host::fail;
using gcore::rt::GretaDataType;

namespace {

enum GgmlType : uint32_t { GGML_F32 = 0, GGML_F16 = 1, GGML_Q4_0 = 2, GGML_Q8_0 = 8, GGML_Q4_K = GRETA_GGML_Q4_K, GGML_Q6_K = GRETA_GGML_Q6_K };
inline bool is_kquant(uint32_t t) { return t == GGML_Q4_K || t == GGML_Q6_K; }

const char *ggml_name(uint32_t t) {
  switch (t) {
    case GGML_F32: return "F32";
    case GGML_F16: return "F16";
    case GGML_Q4_0: return "Q4_0";
    case GGML_Q8_0: return "Q8_0";
    case 3: return "Q4_1";
    case 12: return "Q4_K";
    case 14: return "Q6_K";
    default: return "other";
  }
}
size_t ggml_bytes(uint32_t t, size_t elems) {
  switch (t) {
    case GGML_F32: return elems * 4;
    case GGML_F16: return elems * 2;
    case GGML_Q4_0: return elems / 32 * 18;
    case GGML_Q8_0: return elems / 32 * 34;
    case GGML_Q4_K:
    case GGML_Q6_K: return greta_cuda_kquant_bytes((int)t, elems);
    default: return 0;
  }
}

float half_bits_to_float(uint16_t h) {
  const uint32_t s = (h >> 15) & 1u, e = (h >> 10) & 31u, m = h & 1023u;
  uint32_t f;
  if (e == 0) {
    if (m == 0) {
      f = s << 31;
    } else {
      int sh = 0;
      uint32_t mm = m;
      while (!(mm & 1024u)) {
        mm <<= 1;
        ++sh;
      }
      f = (s << 31) | ((uint32_t)(113 - sh) << 23) | ((mm & 1023u) << 13);
    }
  } else if (e == 31) {
    f = (s << 31) | 0x7F800000u | (m << 13);
  } else {
    f = (s << 31) | ((e + 112u) << 23) | (m << 13);
  }
  float r;
  std::memcpy(&r, &f, 4);
  return r;
}
uint16_t float_to_half_bits(float v) {  // round to nearest even, subnormals included
  uint32_t x;
  std::memcpy(&x, &v, 4);
  const uint32_t s = (x >> 16) & 0x8000u, a = x & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) return (uint16_t)(s | 0x7C00u | (a > 0x7F800000u ? 0x200u : 0u));
  if (a >= 0x477FF000u) return (uint16_t)(s | 0x7C00u);  // rounds to infinity
  if (a < 0x33000001u) return (uint16_t)s;               // rounds to zero
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
  int shift = e < -14 ? 13 + (-14 - e) : 13;
  uint32_t q = m >> shift, rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1))) ++q;
  if (e < -14) return (uint16_t)(s | q);  // subnormal (q may carry into the smallest normal: the bit pattern is right)
  return (uint16_t)(s | (((uint32_t)(e + 15) << 10) + (q - 1024u)));
}

struct Cursor {
  const uint8_t *p, *end;
  bool ok = true;
  template <typename T>
  T get() {
    T v{};
    if (p + sizeof(T) > end) {
      ok = false;
      return v;
    }
    std::memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  std::string str() {
    const uint64_t n = get<uint64_t>();
    if (!ok || n > (uint64_t)(end - p)) {
      ok = false;
      return {};
    }
    std::string s(reinterpret_cast<const char *>(p), (size_t)n);
    p += n;
    return s;
  }
  void skip(uint64_t n) {
    if (n > (uint64_t)(end - p)) ok = false;
    else p += n;
  }
};
size_t scalar_size(uint32_t t) {  // GGUF metadata value types 0..12 without string (8) and array (9)
  switch (t) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    default: return 0;
  }
}

}  // namespace

struct GGUFLoader::Impl {
  struct Entry {
    TensorInfo info;
    uint32_t ggml_type = 0;
    size_t elems = 0;
  };
  int fd = -1;
  const uint8_t *map = nullptr;
  size_t map_bytes = 0, data_offset = 0;
  std::vector<Entry> tensors;
  std::map<std::string, size_t> by_name;
  ModelConfig config;
  bool rms_eps_seen = false;

  ~Impl() { close_file(); }
  void close_file() {
    if (map) munmap(const_cast<uint8_t *>(map), map_bytes);
    if (fd >= 0) ::close(fd);
    map = nullptr;
    fd = -1;
  }
  const Entry *find(const std::string &name) const {
    auto it = by_name.find(name);
    return it == by_name.end() ? nullptr : &tensors[it->second];
  }
  const uint8_t *data(const Entry &e) const { return map + data_offset + e.info.offset; }
};

GGUFLoader::GGUFLoader() : impl_(new Impl) {}
GGUFLoader::~GGUFLoader() = default;

bool GGUFLoader::open(const std::string &path, std::string *err) {
  Impl &im = *impl_;
  im.close_file();
  im.tensors.clear();
  im.by_name.clear();
  im.config = ModelConfig{};
  im.config.num_heads_kv = 0;
  im.config.vocab_size = 0;  // from the tokenizer's token list, else from the embedding's shape
  im.fd = ::open(path.c_str(), O_RDONLY);
  if (im.fd < 0) return fail(err, "GGUF: cannot open " + path);
  struct stat st;
  if (fstat(im.fd, &st) != 0 || st.st_size < 24) return fail(err, "GGUF: file too short");
  im.map_bytes = (size_t)st.st_size;
  void *m = mmap(nullptr, im.map_bytes, PROT_READ, MAP_PRIVATE, im.fd, 0);
  if (m == MAP_FAILED) return fail(err, "GGUF: mmap failed");
  im.map = static_cast<const uint8_t *>(m);
  Cursor c{im.map, im.map + im.map_bytes};
  if (std::memcmp(c.p, "GGUF", 4) != 0) return fail(err, "GGUF: bad magic");
  c.p += 4;
  const uint32_t version = c.get<uint32_t>();
  if (version < 2 || version > 3) return fail(err, "GGUF: unsupported version " + std::to_string(version));
  const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
  if (n_tensors > (1u << 20) || n_kv > (1u << 20)) return fail(err, "GGUF: implausible header counts");
  uint32_t alignment = 32;
  ModelConfig &cfg = im.config;
  bool heads_kv_seen = false;
  for (uint64_t i = 0; i < n_kv && c.ok; ++i) {
    const std::string key = c.str();
    const uint32_t vt = c.get<uint32_t>();
    auto as_u32 = [&](uint32_t &out) {
      switch (vt) {
        case 0: out = c.get<uint8_t>(); break;
        case 1: out = (uint32_t)c.get<int8_t>(); break;
        case 2: out = c.get<uint16_t>(); break;
        case 3: out = (uint32_t)c.get<int16_t>(); break;
        case 4: out = c.get<uint32_t>(); break;
        case 5: out = (uint32_t)c.get<int32_t>(); break;
        case 10: out = (uint32_t)c.get<uint64_t>(); break;
        case 11: out = (uint32_t)c.get<int64_t>(); break;
        case 6: out = (uint32_t)c.get<float>(); break;
        case 12: out = (uint32_t)c.get<double>(); break;
        default: c.ok = false;
      }
    };
    auto as_f32 = [&](float &out) {
      if (vt == 6) out = c.get<float>();
      else if (vt == 12) out = (float)c.get<double>();
      else c.ok = false;
    };
    // the keys the reference reads (weight_loader.cpp:338-423), by suffix so that other architectures' prefixes work too
    auto ends = [&](const char *suffix) { const size_t n = std::strlen(suffix); return key.size() >= n && key.compare(key.size() - n, n, suffix) == 0; };
    if (ends(".embedding_length")) as_u32(cfg.dim);
    else if (ends(".feed_forward_length")) as_u32(cfg.hidden_dim);
    else if (ends(".block_count")) as_u32(cfg.num_layers);
    else if (ends(".attention.head_count")) as_u32(cfg.num_heads);
    else if (ends(".attention.head_count_kv")) { as_u32(cfg.num_heads_kv); heads_kv_seen = true; }
    else if (ends(".context_length")) as_u32(cfg.max_seq_len);
    else if (ends(".rope.freq_base")) as_f32(cfg.rope_base);
    else if (ends(".norm_eps") || ends(".attention.layer_norm_rms_epsilon")) as_f32(cfg.rms_eps);
    else if (key == "general.alignment") as_u32(alignment);
    else if (key == "tokenizer.ggml.tokens" && vt == 9) {
      const uint32_t at = c.get<uint32_t>();
      const uint64_t n = c.get<uint64_t>();
      if (at != 8 || n > (1u << 24)) return fail(err, "GGUF: tokenizer.ggml.tokens is not a string array");
      cfg.vocabulary.clear();
      cfg.vocabulary.reserve((size_t)n);
      for (uint64_t j = 0; j < n && c.ok; ++j) cfg.vocabulary.push_back(c.str());
      cfg.vocab_size = (uint32_t)n;
    } else if (vt == 8) {
      c.str();
    } else if (vt == 9) {
      const uint32_t at = c.get<uint32_t>();
      const uint64_t n = c.get<uint64_t>();
      if (at == 8) {
        for (uint64_t j = 0; j < n && c.ok; ++j) c.str();
      } else if (scalar_size(at)) {
        c.skip(n * scalar_size(at));
      } else {
        c.ok = false;
      }
    } else if (scalar_size(vt)) {
      c.skip(scalar_size(vt));
    } else {
      c.ok = false;
    }
  }
  if (!c.ok) return fail(err, "GGUF: metadata is truncated or malformed");
  if (!heads_kv_seen || cfg.num_heads_kv == 0) cfg.num_heads_kv = cfg.num_heads;
  if (cfg.num_heads) cfg.head_dim = cfg.dim / cfg.num_heads;
  for (uint64_t i = 0; i < n_tensors && c.ok; ++i) {
    Impl::Entry e;
    e.info.name = c.str();
    const uint32_t nd = c.get<uint32_t>();
    if (nd > 4) return fail(err, "GGUF: tensor with more than 4 dimensions");
    std::vector<size_t> dims(nd);
    e.elems = 1;
    for (uint32_t d = 0; d < nd; ++d) {
      dims[d] = (size_t)c.get<uint64_t>();
      e.elems *= dims[d];
    }
    e.info.shape.assign(dims.rbegin(), dims.rend());  // the file stores the innermost dimension first
    e.ggml_type = c.get<uint32_t>();
    e.info.offset = (size_t)c.get<uint64_t>();
    e.info.dtype = ggml_name(e.ggml_type);
    e.info.size_bytes = ggml_bytes(e.ggml_type, e.elems);
    im.by_name[e.info.name] = im.tensors.size();
    im.tensors.push_back(std::move(e));
  }
  if (!c.ok) return fail(err, "GGUF: tensor table is truncated");
  if (alignment == 0) alignment = 32;
  im.data_offset = ((size_t)(c.p - im.map) + alignment - 1) / alignment * alignment;
  for (const auto &e : im.tensors)
    if (e.info.size_bytes && im.data_offset + e.info.offset + e.info.size_bytes > im.map_bytes)
      return fail(err, "GGUF: tensor " + e.info.name + " reaches past the end of the file");
  // Storage format of the projections: what the first layer's query projection is stored as.
  if (const Impl::Entry *wq = im.find("blk.0.attn_q.weight")) {
    if (wq->ggml_type == GGML_Q4_0) cfg.weight_type = GretaDataType::Q4_0;
    else if (wq->ggml_type == GGML_Q8_0 || is_kquant(wq->ggml_type)) cfg.weight_type = GretaDataType::Q8_0;  // K-quants are re-stored as Q8_0
  }
  if (const Impl::Entry *emb = im.find("token_embd.weight"))
    if (cfg.vocab_size == 0 && emb->info.shape.size() == 2) cfg.vocab_size = (uint32_t)emb->info.shape[0];
  if (cfg.vocab_size == 0) cfg.vocab_size = ModelConfig{}.vocab_size;
  const Impl::Entry *out = im.find("output.weight");
  if (!out) out = im.find("token_embd.weight");  // tied embeddings
  if (out)
    cfg.lm_head_type = out->ggml_type == GGML_Q4_0 ? GretaDataType::Q4_0
                       : (out->ggml_type == GGML_Q8_0 || is_kquant(out->ggml_type)) ? GretaDataType::Q8_0
                                                                                    : GretaDataType::FP16;
  return true;
}

std::vector<TensorInfo> GGUFLoader::list_tensors() const {
  std::vector<TensorInfo> v;
  for (const auto &e : impl_->tensors) v.push_back(e.info);
  return v;
}
ModelConfig GGUFLoader::get_config() const { return impl_->config; }

bool GGUFLoader::tensor_data(const std::string &name, const void **data, size_t *bytes, std::string *dtype, std::string *err) const {
  const Impl::Entry *e = impl_->find(name);
  if (!e) return fail(err, "GGUF: tensor not found: " + name);
  if (!e->info.size_bytes) return fail(err, "GGUF: tensor " + name + " has storage type " + e->info.dtype + ", which this path does not read");
  if (data) *data = impl_->data(*e);
  if (bytes) *bytes = e->info.size_bytes;
  if (dtype) *dtype = e->info.dtype;
  return true;
}

// F32 / F16 / Q4_K / Q6_K tensor -> fp32 on the device (norm weights; any tensor a caller wants as plain floats).
bool GGUFLoader::load_tensor(const std::string &name, gcore::rt::cuda::Buffer &buffer, std::string *err) {
  const Impl::Entry *e = impl_->find(name);
  if (!e) return fail(err, "GGUF: tensor not found: " + name);
  if (is_kquant(e->ggml_type)) {  // decoded on the device, as GGUFLoader::load_tensor of the reference decodes them on the host (weight_loader.cpp:551-565)
    gcore::rt::cuda::Buffer raw;
    if (!raw.allocate(e->info.size_bytes, gcore::rt::cuda::BufferUsage::DeviceOnly, GretaDataType::INT8, err)) return false;
    if (!raw.copy_to_device(impl_->data(*e), e->info.size_bytes, err)) return false;
    if (buffer.size() < e->elems * 4 && !buffer.allocate(e->elems * 4, gcore::rt::cuda::BufferUsage::DeviceOnly, GretaDataType::FP32, err)) return false;
    if (greta_cuda_kquant_dequant(nullptr, (int)e->ggml_type, raw.data(), e->elems, buffer.data(), 0) != GRETA_OK || greta_cuda_device_synchronize() != GRETA_OK)
      return fail(err, std::string("GGUF: decoding ") + name + ": " + greta_cuda_last_error());
    return true;
  }
  std::vector<float> tmp(e->elems);
  if (e->ggml_type == GGML_F32) {
    std::memcpy(tmp.data(), impl_->data(*e), e->elems * 4);
  } else if (e->ggml_type == GGML_F16) {
    const uint16_t *h = reinterpret_cast<const uint16_t *>(impl_->data(*e));
    for (size_t i = 0; i < e->elems; ++i) tmp[i] = half_bits_to_float(h[i]);
  } else {
    return fail(err, "GGUF: load_tensor reads F32 / F16, " + name + " is " + e->info.dtype);
  }
  if (buffer.size() < e->elems * 4 && !buffer.allocate(e->elems * 4, gcore::rt::cuda::BufferUsage::DeviceOnly, GretaDataType::FP32, err)) return false;
  return buffer.copy_to_device(tmp.data(), e->elems * 4, err);
}

// F16 / F32 / Q4_0 / Q8_0 / Q4_K / Q6_K tensor -> fp16 values in host memory (embedding table, fp16 LM head).
bool GGUFLoader::read_as_fp16(const std::string &name, std::vector<uint16_t> *out, std::string *err) const {
  const Impl::Entry *e = impl_->find(name);
  if (!e) return fail(err, "GGUF: tensor not found: " + name);
  out->resize(e->elems);
  const uint8_t *p = impl_->data(*e);
  if (e->ggml_type == GGML_F16) {
    std::memcpy(out->data(), p, e->elems * 2);
  } else if (e->ggml_type == GGML_F32) {
    const float *f = reinterpret_cast<const float *>(p);
    for (size_t i = 0; i < e->elems; ++i) (*out)[i] = float_to_half_bits(f[i]);
  } else if (e->ggml_type == GGML_Q4_0 || e->ggml_type == GGML_Q8_0) {  // value = (float)q * fp32(d), then rounded to fp16
    const bool q4 = e->ggml_type == GGML_Q4_0;
    const size_t bb = q4 ? 18 : 34;
    for (size_t b = 0; b < e->elems / 32; ++b) {
      const uint8_t *blk = p + b * bb;
      uint16_t dh;
      std::memcpy(&dh, blk, 2);
      const float d = half_bits_to_float(dh);
      for (int j = 0; j < 32; ++j) {
        const int q = q4 ? (j < 16 ? (blk[2 + j] & 15) : (blk[2 + j - 16] >> 4)) - 8 : (int)(int8_t)blk[2 + j];
        (*out)[b * 32 + j] = float_to_half_bits((float)q * d);
      }
    }
  } else if (is_kquant(e->ggml_type)) {  // decoded and rounded to fp16 on the device
    gcore::rt::cuda::Buffer raw, half;
    if (!raw.allocate(e->info.size_bytes, gcore::rt::cuda::BufferUsage::DeviceOnly, GretaDataType::INT8, err)) return false;
    if (!half.allocate(e->elems * 2, gcore::rt::cuda::BufferUsage::DeviceOnly, GretaDataType::FP16, err)) return false;
    if (!raw.copy_to_device(p, e->info.size_bytes, err)) return false;
    if (greta_cuda_kquant_dequant(nullptr, (int)e->ggml_type, raw.data(), e->elems, half.data(), 1) != GRETA_OK ||
        greta_cuda_memcpy_d2h_sync(out->data(), half.data(), e->elems * 2) != GRETA_OK)
      return fail(err, std::string("GGUF: decoding ") + name + ": " + greta_cuda_last_error());
  } else {
    return fail(err, "GGUF: " + name + " has storage type " + e->info.dtype + ", which this path does not read");
  }
  return true;
}

bool GGUFLoader::load_tensor_fp16(const std::string &name, gcore::rt::cuda::Buffer &buffer, std::string *err) {
  std::vector<uint16_t> tmp;
  if (!read_as_fp16(name, &tmp, err)) return false;
  if (buffer.size() < tmp.size() * 2 && !buffer.allocate(tmp.size() * 2, gcore::rt::cuda::BufferUsage::DeviceOnly, GretaDataType::FP16, err)) return false;
  return buffer.copy_to_device(tmp.data(), tmp.size() * 2, err);
}

// The reference's quantising loaders (F32 / F16 / K-quant tensor -> its own INT8 / INT4 planes, weight_loader.cpp:668-1005)
// are its workaround for not storing GGUF blocks; this build stores them, so there is nothing to re-quantise.
bool GGUFLoader::load_tensor_int8(const std::string &name, gcore::rt::cuda::Buffer &, gcore::rt::cuda::Buffer &, std::string *err) {
  return fail(err, "GGUF: load_tensor_int8(" + name + ") is not carried over: GGUF Q8_0 / Q4_0 blocks are loaded as they are (BlockScheduler::load_weights)");
}
bool GGUFLoader::load_tensor_int4(const std::string &name, gcore::rt::cuda::Buffer &, gcore::rt::cuda::Buffer &, gcore::rt::cuda::Buffer &,
                                  std::string *err) {
  return fail(err, "GGUF: load_tensor_int4(" + name + ") is not carried over: GGUF Q8_0 / Q4_0 blocks are loaded as they are (BlockScheduler::load_weights)");
}

std::unique_ptr<WeightLoader> create_weight_loader(const std::string &path, std::string *err) {
  if (path.size() >= 5 && path.compare(path.size() - 5, 5, ".gguf") == 0) {
    auto l = std::make_unique<GGUFLoader>();
    if (!l->open(path, err)) return nullptr;
    return l;
  }
  fail(err, "create_weight_loader: only .gguf files are read on this path");
  return nullptr;
}

// ------------------------------------------------------------------ BlockScheduler::load_weights
bool BlockScheduler::load_weights(WeightLoader &loader, std::string *err) {
  auto *gguf = dynamic_cast<GGUFLoader *>(&loader);
  if (!gguf) return fail(err, "load_weights: this path reads GGUF files (GGUFLoader)");
  if (blocks_.empty()) return fail(err, "load_weights: allocate_weights first");
  const ModelConfig &c = config_;
  const char *want = c.weight_type == GretaDataType::Q4_0 ? "Q4_0" : "Q8_0";
  static const char *kNames[7] = {"attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_down", "ffn_up"};  // LayerTensor order
  for (uint32_t l = 0; l < c.num_layers; ++l) {
    const std::string prefix = "blk." + std::to_string(l) + ".";
    for (int t = 0; t < 7; ++t) {
      const void *data;
      size_t bytes;
      std::string dtype;
      const std::string name = prefix + kNames[t] + ".weight";
      if (!gguf->tensor_data(name, &data, &bytes, &dtype, err)) return false;
      if (dtype == "Q4_K" || dtype == "Q6_K") {  // re-stored as Q8_0 on the device
        if (!set_layer_tensor_kquant(l, (LayerTensor)t, dtype == "Q4_K" ? GRETA_GGML_Q4_K : GRETA_GGML_Q6_K, data, bytes, err)) return false;
        continue;
      }
      if (dtype != want) return fail(err, "load_weights: " + name + " is stored as " + dtype + ", the scheduler was initialised for " + want);
      if (!set_layer_tensor(l, (LayerTensor)t, data, bytes, err)) return false;
    }
    if (!loader.load_tensor(prefix + "attn_norm.weight", blocks_[l].attn_norm, err)) return false;
    if (!loader.load_tensor(prefix + "ffn_norm.weight", blocks_[l].ffn_norm, err)) return false;
  }
  if (!loader.load_tensor("output_norm.weight", output_norm_, err)) return false;
  std::vector<uint16_t> emb;
  if (!gguf->read_as_fp16("token_embd.weight", &emb, err)) return false;
  if (!set_global_tensor(GlobalTensor::TOK_EMBD, emb.data(), emb.size() * 2, err)) return false;
  std::string head = "output.weight", tmp;
  if (!gguf->tensor_data(head, nullptr, nullptr, nullptr, &tmp)) head = "token_embd.weight";  // tied embeddings
  if (c.lm_head_type == GretaDataType::FP16) {
    std::vector<uint16_t> w;
    if (head == "token_embd.weight") w = emb;
    else if (!gguf->read_as_fp16(head, &w, err)) return false;
    return set_global_tensor(GlobalTensor::OUT_WEIGHT, w.data(), w.size() * 2, err);
  }
  const void *data;
  size_t bytes;
  std::string dtype;
  if (!gguf->tensor_data(head, &data, &bytes, &dtype, err)) return false;
  if (dtype == "Q4_K" || dtype == "Q6_K") return set_global_tensor_kquant(GlobalTensor::OUT_WEIGHT, dtype == "Q4_K" ? GRETA_GGML_Q4_K : GRETA_GGML_Q6_K, data, bytes, err);
  if (dtype != (c.lm_head_type == GretaDataType::Q4_0 ? "Q4_0" : "Q8_0")) return fail(err, "load_weights: " + head + " is stored as " + dtype + ", not as the configured LM-head type");
  return set_global_tensor(GlobalTensor::OUT_WEIGHT, data, bytes, err);
}

}  // namespace gcore::inference
