// Prefill GEMM over block-quantised weights on the 5th-generation tensor cores.
#include "greta_common.cuh"

using namespace greta;

extern "C" {

size_t greta_cuda_gemm_workspace_bytes(uint32_t M, uint32_t K) { return ((size_t)M * K * 2 + 255) / 256 * 256; }

int greta_cuda_gemm(greta_stream_t stream, int fmt, const void *A, int a_is_f16, const void *qs, const void *d, void *Cout,
                    int c_is_f16, uint32_t M, uint32_t N, uint32_t K, void *workspace) {
  (void)stream; (void)fmt; (void)A; (void)a_is_f16; (void)qs; (void)d; (void)Cout; (void)c_is_f16; (void)M; (void)N; (void)K; (void)workspace;
  set_error("gemm: the tensor-core prefill kernel is not built yet");
  return GRETA_ERR_NOT_IMPLEMENTED;
}

}  // extern "C"
