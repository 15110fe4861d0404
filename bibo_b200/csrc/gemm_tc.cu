// Tensor-core (tcgen05 / TMEM / TMA) kernels: placeholder until the kernels land.
#include "common.cuh"
namespace bibo {
int router_tc_supported(int, int, int) { return 0; }
int router_tc_launch(const void*, const void*, const float*, int64_t, int, int, int, int, float, float*,
                     int32_t*, float*, int32_t*, int32_t*, cudaStream_t) {
  return fail(BIBO_ERR_UNSUPPORTED, "router_tc: not built");
}
int gemm1_tc_supported(int, int, int) { return 0; }
int gemm1_tc_launch(const void*, const void*, const float*, const int32_t*, int64_t, int, int, int, int, int,
                    void*, void*, float*, cudaStream_t) {
  return fail(BIBO_ERR_UNSUPPORTED, "gemm1_tc: not built");
}
int gemm2_tc_supported(int, int, int) { return 0; }
int gemm2_tc_launch(const void*, const void*, const int32_t*, int64_t, int, int, int, int, int, void*,
                    cudaStream_t) {
  return fail(BIBO_ERR_UNSUPPORTED, "gemm2_tc: not built");
}
}  // namespace bibo
