// Shared helpers of libbibo_moe: error reporting, dtype traits, plan layout.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/bibo_moe.h"

namespace bibo {

// ---- host-side error string (per thread) ------------------------------------------------------
inline char* err_buf() {
  static thread_local char buf[512] = "no error";
  return buf;
}
inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(err_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}
inline std::atomic<long long>& launch_counter() {
  static std::atomic<long long> c{0};
  return c;
}
#define BIBO_CHECK_LAUNCH(name)                                                       \
  do {                                                                                \
    bibo::launch_counter().fetch_add(1, std::memory_order_relaxed);                   \
    cudaError_t e_ = cudaGetLastError();                                              \
    if (e_ != cudaSuccess)                                                            \
      return bibo::fail(BIBO_ERR_CUDA, "%s launch: %s", name, cudaGetErrorString(e_)); \
  } while (0)
#define BIBO_CUDA(call)                                                                   \
  do {                                                                                    \
    cudaError_t e_ = (call);                                                              \
    if (e_ != cudaSuccess)                                                                \
      return bibo::fail(BIBO_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_));           \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- one-time set-up per device ---------------------------------------------------------------------
// Function attributes (dynamic shared memory size, carve-out) and occupancy figures belong to a device,
// not to the process: a launcher keeps one DeviceOnce and runs its set-up the first time it is called
// with a given device current, under a mutex (host threads may share the library).
constexpr int BIBO_MAX_DEVICES = 64;
struct DeviceOnce {
  std::mutex mu;
  bool done[BIBO_MAX_DEVICES] = {};
  int value[BIBO_MAX_DEVICES] = {};
  template <typename F> int get(F&& init, int* value_out = nullptr) {
    int dev = 0;
    BIBO_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= BIBO_MAX_DEVICES) return fail(BIBO_ERR_UNSUPPORTED, "device index %d", dev);
    std::lock_guard<std::mutex> g(mu);
    if (!done[dev]) {
      const int rc = init(&value[dev]);
      if (rc) return rc;
      done[dev] = true;
    }
    if (value_out) *value_out = value[dev];
    return BIBO_OK;
  }
};
// SM count of the current device
inline int sm_count() {
  static DeviceOnce once;
  int n = 0;
  const int rc = once.get([](int* v) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(v, cudaDevAttrMultiProcessorCount, dev);
    if (*v <= 0) *v = 148;
    return BIBO_OK;
  }, &n);
  return rc == BIBO_OK && n > 0 ? n : 148;
}

// ---- plan layout (int32 words) ------------------------------------------------------------------
constexpr int PLAN_N_TILES = 0, PLAN_ROWS_USED = 1, PLAN_STATUS = 2, PLAN_N_PAIRS = 3, PLAN_HDR = 4;
__host__ __device__ inline int64_t router_blocks(int64_t n_tokens) {
  return (n_tokens + BIBO_ROUTER_BLOCK_TOKENS - 1) / BIBO_ROUTER_BLOCK_TOKENS;
}
__host__ __device__ inline int64_t rows_cap(int64_t n, int k, int n_glu) {
  int64_t r = n * k + (int64_t)n_glu * (BIBO_TILE_M - 1);
  return (r + BIBO_TILE_M - 1) / BIBO_TILE_M * BIBO_TILE_M;
}
__host__ __device__ inline int64_t tiles_cap(int64_t n, int k, int n_glu) {
  return rows_cap(n, k, n_glu) / BIBO_TILE_M;
}
__host__ __device__ inline int64_t plan_off_counts() { return PLAN_HDR; }
__host__ __device__ inline int64_t plan_off_expert_off(int E) { return PLAN_HDR + E; }
__host__ __device__ inline int64_t plan_off_block_base(int E, int n_glu) {
  return PLAN_HDR + E + n_glu + 1;
}
__host__ __device__ inline int64_t plan_off_tiles(int64_t n, int E, int n_glu) {
  int64_t o = plan_off_block_base(E, n_glu) + router_blocks(n) * E;
  return (o + 3) / 4 * 4;  // int4-aligned tile records
}
// tile pairs (int2 {tile a, tile b or -1}: two consecutive tiles of one expert, for the kernels that
// run a row-tile pair on a two-CTA tensor-core instruction)
__host__ __device__ inline int64_t plan_off_pairs(int64_t n, int k, int E, int n_glu) {
  return plan_off_tiles(n, E, n_glu) + tiles_cap(n, k, n_glu) * 4;
}
// scratch of the gate/up kernel: partial sums of squares and flags that two 2-CTA clusters (the two
// column blocks of one row pair) exchange through global memory; per CTA 2 x 128 floats + 2 flags
constexpr int XG_MAX_CTAS = 256;
constexpr int64_t XG_PART_WORDS = (int64_t)XG_MAX_CTAS * 2 * 128;
constexpr int64_t XG_WORDS = XG_PART_WORDS + XG_MAX_CTAS * 2;
__host__ __device__ inline int64_t plan_off_scratch(int64_t n, int k, int E, int n_glu) {
  return plan_off_pairs(n, k, E, n_glu) + tiles_cap(n, k, n_glu) * 2;
}
// ... followed by one arrival counter per tile pair for the kernels that gather their own A rows
__host__ __device__ inline int64_t plan_words(int64_t n, int k, int E, int n_glu) {
  return plan_off_scratch(n, k, E, n_glu) + XG_WORDS + tiles_cap(n, k, n_glu);
}

// What a grouped-GEMM launcher needs to know about a row plan: where the header / tile list live and
// how many rows / tiles the expert-contiguous buffers were allocated for.
struct PlanView {
  const int32_t* plan;   // header at [0..3]
  int64_t tiles_off;     // word offset of the int4 tile records
  int64_t pairs_off;     // word offset of the int2 tile-pair records
  int64_t scratch_off;   // word offset of the XG_WORDS exchange scratch
  int64_t tiles_cap;     // upper bound of tiles (grid sizing)
  int64_t rows_alloc;    // rows of the expert-contiguous buffers
  int max_ctas;          // 0 = all SMs; otherwise an upper bound for persistent grids
};
inline PlanView local_plan_view(const int32_t* plan, int64_t n_tokens, int top_k, int n_experts, int n_glu) {
  return PlanView{plan, plan_off_tiles(n_tokens, n_experts, n_glu), plan_off_pairs(n_tokens, top_k, n_experts, n_glu),
                  plan_off_scratch(n_tokens, top_k, n_experts, n_glu), tiles_cap(n_tokens, top_k, n_glu),
                  rows_cap(n_tokens, top_k, n_glu), 0};
}

// ---- dtype helpers ------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// accurate sigmoid: IEEE division and expf (no fast-math), so scores round as torch's do
__device__ __forceinline__ float sigmoid_accurate(float x) {
  return __fdiv_rn(1.0f, 1.0f + expf(-x));
}

}  // namespace bibo
