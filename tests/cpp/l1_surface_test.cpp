// Drives the C++ operator surface that mirrors the reference's (include/gcore/greta_b200.hpp: Buffer, GretaArena,
// GretaCompute, GretaFused, the launch_* functions) on inputs and expected outputs that the Python side of the
// test wrote to a file: the expected values come from the CPU oracle.  Prints one line per check and exits
// non-zero when any check fails.  Built by gretacore-v3_b200/csrc/Makefile (target l1_surface_test) and run by
// tests/test_cpp_surface_gpu.py.
//
// File format: repeated records { u32 name_len; name; u64 byte_count; bytes }.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "gcore/compute/greta_compute.hpp"
#include "gcore/rt/hip/kernels/attention_kernels.hpp"
#include "gcore/rt/hip/kernels/basic_kernels.hpp"
#include "gcore/rt/hip/kernels/gemm_kernels.hpp"

using namespace gcore::rt;
using gcore::compute::GretaCompute;
using gcore::compute::GretaFused;
using gcore::rt::hip::Buffer;
using gcore::rt::hip::BufferUsage;
namespace K = gcore::rt::hip::kernels;

static std::map<std::string, std::vector<uint8_t>> g_data;
static int g_failed = 0, g_checks = 0;

static bool load(const char *path) {
  FILE *f = fopen(path, "rb");
  if (!f) return false;
  for (;;) {
    uint32_t nl;
    if (fread(&nl, 4, 1, f) != 1) break;
    std::string name(nl, 0);
    uint64_t n;
    if (fread(&name[0], 1, nl, f) != nl || fread(&n, 8, 1, f) != 1) return false;
    std::vector<uint8_t> v(n);
    if (n && fread(v.data(), 1, n, f) != n) return false;
    g_data[name] = std::move(v);
  }
  fclose(f);
  return true;
}
static const std::vector<uint8_t> &raw(const std::string &name) {
  auto it = g_data.find(name);
  if (it == g_data.end()) {
    fprintf(stderr, "missing tensor %s\n", name.c_str());
    exit(3);
  }
  return it->second;
}
static const float *f32(const std::string &name) { return reinterpret_cast<const float *>(raw(name).data()); }
static size_t count_f32(const std::string &name) { return raw(name).size() / 4; }
static uint32_t u32(const std::string &name, size_t i = 0) { return reinterpret_cast<const uint32_t *>(raw(name).data())[i]; }

static void report(const std::string &what, bool ok, double err = 0.0) {
  ++g_checks;
  if (!ok) ++g_failed;
  printf("%s %s err=%.3e\n", ok ? "PASS" : "FAIL", what.c_str(), err);
}
// max |got - want| / max |want|, the acceptance metric of the parity tests.
static double max_abs_rel(const float *got, const float *want, size_t n) {
  double mx = 0, den = 0;
  for (size_t i = 0; i < n; ++i) {
    if (!std::isfinite(got[i])) return INFINITY;
    mx = std::max(mx, std::fabs((double)got[i] - (double)want[i]));
    den = std::max(den, std::fabs((double)want[i]));
  }
  return mx / (den > 0 ? den : 1.0);
}
static void upload(Buffer &b, const std::string &name, GretaDataType t) {
  std::string err;
  const auto &v = raw(name);
  if (!b.allocate(v.size() ? v.size() : 16, BufferUsage::DeviceOnly, t, &err) || !b.copy_to_device(v.data(), v.size(), &err)) {
    fprintf(stderr, "upload %s: %s\n", name.c_str(), err.c_str());
    exit(3);
  }
}
static void device_out(Buffer &b, size_t bytes, GretaDataType t = GretaDataType::FP32) {
  std::string err;
  if (!b.allocate(bytes, BufferUsage::DeviceOnly, t, &err)) exit(3);
  greta_cuda_memset(b.data(), 0xFF, bytes, nullptr);  // NaN pattern: an unwritten output is caught
  greta_cuda_device_synchronize();
}
static std::vector<float> download(Buffer &b, size_t n) {
  std::vector<float> v(n);
  std::string err;
  greta_cuda_device_synchronize();
  if (!b.copy_to_host(v.data(), n * 4, &err)) {
    fprintf(stderr, "download: %s\n", err.c_str());
    exit(3);
  }
  return v;
}
static float half_to_float(uint16_t h) {
  uint32_t s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023, f;
  if (e == 0) {
    if (!m) f = s << 31;
    else {
      e = 1;
      while (!(m & 1024)) { m <<= 1; --e; }
      f = (s << 31) | ((e + 112) << 23) | ((m & 1023) << 13);
    }
  } else if (e == 31) f = (s << 31) | 0x7F800000u | (m << 13);
  else f = (s << 31) | ((e + 112) << 23) | (m << 13);
  float r;
  memcpy(&r, &f, 4);
  return r;
}

// GretaCompute::gemm for one weight format at M = 1, 32 and 33: results against the oracle and the route at the threshold.
static void gemm_cases(GretaStream *stream, const std::string &fmt, GretaDataType wtype, bool tensor_core_above_32) {
  const uint32_t N = u32("gemm.N"), Kd = u32("gemm.K");
  Buffer w, scales;
  upload(w, "gemm." + fmt + ".w", wtype);
  if (wtype != GretaDataType::FP16) {
    upload(scales, "gemm." + fmt + ".scales", wtype == GretaDataType::Q4_0 || wtype == GretaDataType::Q8_0 ? GretaDataType::FP16 : GretaDataType::FP32);
    GretaQuantInfo qi;
    qi.scales = scales.data();
    qi.group_size = 32;
    w.set_quant_info(qi);
  }
  for (uint32_t M : {1u, 32u, 33u}) {
    const std::string tag = "gemm." + fmt + ".M" + std::to_string(M);
    Buffer a, c;
    upload(a, "gemm.A" + std::to_string(M), GretaDataType::FP32);
    device_out(c, (size_t)M * N * 4);
    GretaCompute::set_op_label(tag.c_str());
    GretaResult r = GretaCompute::gemm(stream, &a, &w, &c, M, N, Kd);
    auto got = download(c, (size_t)M * N);
    const bool tc = M > 32 && tensor_core_above_32;
    const std::string want = "gemm." + fmt + (tc ? ".want_tc" : ".want") + std::to_string(M);
    double err = max_abs_rel(got.data(), f32(want), (size_t)M * N);
    report(tag + " result", r == GretaResult::SUCCESS && err < (tc ? 1e-4 : 2e-5), err);
    auto audit = GretaCompute::get_last_gemm_audit();
    report(tag + " route " + audit.route, audit.route == (tc ? "TCGEN05" : "GEMV") && audit.op_label == tag && audit.m == M && audit.n == N && audit.k == Kd);
  }
}

int main(int argc, char **argv) {
  if (argc < 2 || !load(argv[1])) {
    fprintf(stderr, "usage: l1_surface_test <cases file>\n");
    return 2;
  }
  GretaContext &ctx = GretaContext::instance();
  if (ctx.initialize() != GretaResult::SUCCESS) {
    fprintf(stderr, "no CUDA device\n");
    return 2;
  }
  std::unique_ptr<GretaStream> stream(ctx.create_stream());
  cudaStream_t s = static_cast<gcore::rt::hip::GretaStreamCuda *>(stream.get())->handle();

  // ---- L1: GretaCompute::gemm, every weight format the reference's data types name plus the GGUF ones
  gemm_cases(stream.get(), "q4_0", GretaDataType::Q4_0, true);
  gemm_cases(stream.get(), "q8_0", GretaDataType::Q8_0, true);
  gemm_cases(stream.get(), "int4", GretaDataType::INT4, false);
  gemm_cases(stream.get(), "int8", GretaDataType::INT8, false);
  gemm_cases(stream.get(), "f16", GretaDataType::FP16, false);
  {  // weights kept as Q4_K super-blocks: the GEMV route up to 32 rows, refused above
    const uint32_t N = u32("gemm.N"), Kd = u32("gemm.K");
    Buffer w;
    upload(w, "gemm.q4_k.w", GretaDataType::Q4_K);
    for (uint32_t M : {1u, 32u}) {
      const std::string tag = "gemm.q4_k.M" + std::to_string(M);
      Buffer a, c;
      upload(a, "gemm.A" + std::to_string(M), GretaDataType::FP32);
      device_out(c, (size_t)M * N * 4);
      GretaCompute::set_op_label(tag.c_str());
      GretaResult r = GretaCompute::gemm(stream.get(), &a, &w, &c, M, N, Kd);
      auto got = download(c, (size_t)M * N);
      double err = max_abs_rel(got.data(), f32("gemm.q4_k.want" + std::to_string(M)), (size_t)M * N);
      report(tag + " result", r == GretaResult::SUCCESS && err < 2e-5, err);
      auto audit = GretaCompute::get_last_gemm_audit();
      report(tag + " route " + audit.route, audit.route == "GEMV" && audit.quant_mode == "Q4_K" && audit.op_label == tag);
    }
    Buffer a, c;
    upload(a, "gemm.A33", GretaDataType::FP32);
    device_out(c, (size_t)33 * N * 4);
    report("gemm q4_k above 32 rows refused", GretaCompute::gemm(stream.get(), &a, &w, &c, 33, N, Kd) == GretaResult::ERROR_NOT_IMPLEMENTED);
  }
  {  // FP16 output forces the tensor-core route even at M = 1; transposes and non-fp32 accumulation are refused
    Buffer w, sc, a, c;
    upload(w, "gemm.q4_0.w", GretaDataType::Q4_0);
    upload(sc, "gemm.q4_0.scales", GretaDataType::FP16);
    GretaQuantInfo qi;
    qi.scales = sc.data();
    qi.group_size = 32;
    w.set_quant_info(qi);
    upload(a, "gemm.A33", GretaDataType::FP32);
    const uint32_t N = u32("gemm.N"), Kd = u32("gemm.K");
    device_out(c, (size_t)33 * N * 2, GretaDataType::FP16);
    report("gemm reserve workspace", GretaCompute::reserve_gemm_workspace(64, Kd) == GretaResult::SUCCESS);
    GretaResult r = GretaCompute::gemm(stream.get(), &a, &w, &c, 33, N, Kd);
    std::vector<uint16_t> h((size_t)33 * N);
    greta_cuda_device_synchronize();
    c.copy_to_host(h.data(), h.size() * 2, nullptr);
    std::vector<float> got(h.size());
    for (size_t i = 0; i < h.size(); ++i) got[i] = half_to_float(h[i]);
    double err = max_abs_rel(got.data(), f32("gemm.q4_0.want_tc33"), got.size());
    report("gemm q4_0 fp16 output", r == GretaResult::SUCCESS && err < 1e-3, err);
    report("gemm transpose refused", GretaCompute::gemm(stream.get(), &a, &w, &c, 33, N, Kd, true) == GretaResult::ERROR_NOT_IMPLEMENTED);
    report("gemm null refused", GretaCompute::gemm(stream.get(), nullptr, &w, &c, 33, N, Kd) == GretaResult::ERROR_INVALID_ARGS);
  }

  // ---- L1: attention_decode (fp16 cache and the reference's fp32 cache), rmsnorm
  {
    const uint32_t H = u32("attn.shape", 0), Hkv = u32("attn.shape", 1), Dh = u32("attn.shape", 2), L = u32("attn.shape", 3), S = u32("attn.shape", 4);
    const float scale = f32("attn.scale")[0];
    Buffer q, k16, v16, k32, v32, o, dpos;
    upload(q, "attn.q", GretaDataType::FP32);
    upload(k16, "attn.k16", GretaDataType::FP16);
    upload(v16, "attn.v16", GretaDataType::FP16);
    upload(k32, "attn.k32", GretaDataType::FP32);
    upload(v32, "attn.v32", GretaDataType::FP32);
    upload(dpos, "attn.dpos", GretaDataType::FP32);
    device_out(o, (size_t)H * Dh * 4);
    GretaResult r = GretaCompute::attention_decode(stream.get(), &q, &k16, &v16, nullptr, &o, H, Hkv, Dh, L, S, scale, 10000.0f);
    auto got = download(o, (size_t)H * Dh);
    double err = max_abs_rel(got.data(), f32("attn.want"), got.size());
    report("attention_decode fp16 cache", r == GretaResult::SUCCESS && err < 1e-5, err);
    device_out(o, (size_t)H * Dh * 4);
    r = GretaCompute::attention_decode(stream.get(), &q, &k32, &v32, &dpos, &o, H, Hkv, Dh, 0, S, scale, 10000.0f);
    got = download(o, (size_t)H * Dh);
    err = max_abs_rel(got.data(), f32("attn.want"), got.size());
    report("attention_decode fp32 cache, device position", r == GretaResult::SUCCESS && err < 1e-5, err);
    // the launcher with the reference's signature
    device_out(o, (size_t)H * Dh * 4);
    K::launch_flash_attention_decode(s, static_cast<const float *>(q.data()), static_cast<const float *>(k32.data()),
                                     static_cast<const float *>(v32.data()), static_cast<float *>(o.data()), H, Hkv, L, S, Dh, scale);
    got = download(o, (size_t)H * Dh);
    err = max_abs_rel(got.data(), f32("attn.want"), got.size());
    report("launch_flash_attention_decode", K::last_launch_error() == 0 && err < 1e-5, err);
  }
  {
    const uint32_t rows = u32("rms.shape", 0), cols = u32("rms.shape", 1);
    Buffer x, g, y;
    upload(x, "rms.x", GretaDataType::FP32);
    upload(g, "rms.gamma", GretaDataType::FP32);
    device_out(y, (size_t)rows * cols * 4);
    GretaResult r = GretaCompute::rmsnorm(stream.get(), &x, &g, &y, cols, 1e-5f);
    auto got = download(y, (size_t)rows * cols);
    double err = max_abs_rel(got.data(), f32("rms.want"), got.size());
    report("rmsnorm", r == GretaResult::SUCCESS && err < 1e-6, err);
  }

  // ---- GretaFused::rmsnorm_qkv (norm + three projections, no rotation), sizes taken from the output buffers
  {
    const uint32_t D = u32("fused.shape", 0), nq = u32("fused.shape", 1), nkv = u32("fused.shape", 2);
    Buffer x, g, wq, wk, wv, sq, sk, sv, q, k, v;
    upload(x, "fused.x", GretaDataType::FP32);
    upload(g, "fused.gamma", GretaDataType::FP32);
    Buffer *ws[3] = {&wq, &wk, &wv}, *ss[3] = {&sq, &sk, &sv};
    const char *names[3] = {"wq", "wk", "wv"};
    for (int i = 0; i < 3; ++i) {
      upload(*ws[i], std::string("fused.") + names[i] + ".w", GretaDataType::Q4_0);
      upload(*ss[i], std::string("fused.") + names[i] + ".scales", GretaDataType::FP16);
      GretaQuantInfo qi;
      qi.scales = ss[i]->data();
      qi.group_size = 32;
      ws[i]->set_quant_info(qi);
    }
    device_out(q, (size_t)nq * 4);
    device_out(k, (size_t)nkv * 4);
    device_out(v, (size_t)nkv * 4);
    GretaResult r = GretaFused::rmsnorm_qkv(stream.get(), &x, &g, &wq, &wk, &wv, &q, &k, &v, D, 1e-5f);
    auto gq = download(q, nq), gk = download(k, nkv), gv = download(v, nkv);
    double e = std::max({max_abs_rel(gq.data(), f32("fused.want_q"), nq), max_abs_rel(gk.data(), f32("fused.want_k"), nkv),
                         max_abs_rel(gv.data(), f32("fused.want_v"), nkv)});
    report("GretaFused::rmsnorm_qkv", r == GretaResult::SUCCESS && e < 2e-5, e);
  }

  // ---- launch_* with the reference's signatures
  {
    const uint32_t N = u32("gemm.N"), Kd = u32("gemm.K");
    Buffer w, sc, a, c;
    upload(w, "gemm.int4.w", GretaDataType::INT4);
    upload(sc, "gemm.int4.scales", GretaDataType::FP32);
    upload(a, "gemm.A33", GretaDataType::FP32);
    device_out(c, (size_t)33 * N * 4);
    K::launch_gemm_mfma_int4_wt_fp32_acc32(s, a.data(), static_cast<const int8_t *>(w.data()), static_cast<float *>(c.data()),
                                           static_cast<const float *>(sc.data()), nullptr, 33, N, Kd, Kd, Kd, N, 32, 128, false, false);
    auto got = download(c, (size_t)33 * N);
    double err = max_abs_rel(got.data(), f32("gemm.int4.want33"), got.size());
    report("launch_gemm_mfma_int4_wt_fp32_acc32 M=33", K::last_launch_error() == 0 && err < 2e-5, err);
    K::launch_gemm_mfma_int4_wt_fp32_acc32(s, a.data(), static_cast<const int8_t *>(w.data()), static_cast<float *>(c.data()),
                                           static_cast<const float *>(sc.data()), static_cast<const float *>(sc.data()), 33, N, Kd, Kd, Kd, N, 32,
                                           128, false, false);
    report("launch_gemm_mfma_int4 refuses per-head scales", K::last_launch_error() == GRETA_ERR_INVALID_ARGS);
  }
  {
    const size_t n = count_f32("argmax.logits");
    Buffer lg;
    upload(lg, "argmax.logits", GretaDataType::FP32);
    int32_t id = -1;
    K::launch_argmax(s, static_cast<const float *>(lg.data()), (uint32_t)n, &id);
    report("launch_argmax", K::last_launch_error() == 0 && id == (int32_t)u32("argmax.want"));
  }
  {  // fused-rope decode attention: un-rotated Q, fp32 cache, one KV head per head
    const uint32_t H = u32("frope.shape", 0), Dh = u32("frope.shape", 1), S = u32("frope.shape", 2);
    Buffer q, k, v, o, dpos;
    upload(q, "frope.q", GretaDataType::FP32);
    upload(k, "frope.k", GretaDataType::FP32);
    upload(v, "frope.v", GretaDataType::FP32);
    upload(dpos, "frope.dpos", GretaDataType::FP32);
    device_out(o, (size_t)H * Dh * 4);
    K::launch_flash_attention_decode_fused_rope(s, static_cast<const float *>(q.data()), static_cast<const float *>(k.data()),
                                                static_cast<const float *>(v.data()), static_cast<float *>(o.data()), H,
                                                static_cast<const uint32_t *>(dpos.data()), S, Dh, f32("frope.scale")[0], 10000.0f);
    auto got = download(o, (size_t)H * Dh);
    double err = max_abs_rel(got.data(), f32("frope.want"), got.size());
    report("launch_flash_attention_decode_fused_rope", K::last_launch_error() == 0 && err < 1e-4, err);
  }
  for (const char *mode : {"causal", "full"}) {  // the reference's prefill entry: prompt-major fp32 K/V
    const uint32_t S = u32("prefill.shape", 0), H = u32("prefill.shape", 1), Hkv = u32("prefill.shape", 2), Dh = u32("prefill.shape", 3);
    Buffer q, k, v, o;
    upload(q, "prefill.q", GretaDataType::FP32);
    upload(k, "prefill.k", GretaDataType::FP32);
    upload(v, "prefill.v", GretaDataType::FP32);
    device_out(o, (size_t)S * H * Dh * 4);
    K::launch_flash_attention_prefill(s, static_cast<const float *>(q.data()), static_cast<const float *>(k.data()),
                                      static_cast<const float *>(v.data()), static_cast<float *>(o.data()), S, H, Hkv, Dh, f32("prefill.scale")[0],
                                      std::string(mode) == "causal");
    auto got = download(o, (size_t)S * H * Dh);
    double err = max_abs_rel(got.data(), f32(std::string("prefill.want_") + mode), got.size());
    report(std::string("launch_flash_attention_prefill ") + mode, K::last_launch_error() == 0 && err < 1e-5, err);
  }

  // ---- L0: GretaArena, Buffer bounds, graph capture of a launcher
  {
    gcore::rt::hip::GretaArena arena(1 << 20);
    void *p1 = nullptr, *p2 = nullptr, *p3 = nullptr;
    std::string err;
    bool ok = arena.allocate(1000, &p1, &err) && arena.allocate(5, &p2, &err) && arena.allocate(3 << 20, &p3, &err);
    ok = ok && (char *)p2 - (char *)p1 == 1024 && arena.num_chunks() == 2 && arena.total_allocated() == 1024 + 256 + (3 << 20) &&
         ((uintptr_t)p3 & 255) == 0;
    report("GretaArena bump allocation", ok);
    Buffer b;
    b.allocate(64, BufferUsage::DeviceOnly, GretaDataType::FP32, &err);
    char tmp[128];
    report("Buffer refuses out-of-bounds copies", !b.copy_to_host_offset(tmp, 32, 64, &err) && !b.copy_to_device(tmp, 128, &err));
  }
  {
    const size_t n = count_f32("rms.x");
    Buffer a, c;
    upload(a, "rms.x", GretaDataType::FP32);
    device_out(c, n * 4);
    std::unique_ptr<GretaGraph> graph(ctx.create_graph());
    graph->capture_start(stream.get());
    K::launch_add(s, static_cast<const float *>(a.data()), static_cast<const float *>(a.data()), static_cast<float *>(c.data()), n);
    graph->capture_end(stream.get());
    bool ok = graph->instantiate() == GretaResult::SUCCESS && graph->launch(stream.get()) == GretaResult::SUCCESS;
    stream->synchronize();
    auto got = download(c, n);
    for (size_t i = 0; i < n && ok; ++i) ok = got[i] == 2.0f * f32("rms.x")[i];
    report("GretaGraph capture / instantiate / launch of launch_add", ok);
  }
  printf("%d checks, %d failed\n", g_checks, g_failed);
  return g_failed ? 1 : 0;
}
