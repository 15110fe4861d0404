// bibo_moe_route_noalloc: routing (router + per-expert histogram) for callers that may not allocate
// device memory.
//
// Who needs this: a host program that was handed its input and output buffers by somebody else and
// has no allocator of its own -- for instance a serving runtime that reserves all device memory at
// start-up and forbids later cudaMalloc calls, or a latency-critical loop in which the implicit
// device synchronisation of cudaMalloc/cudaFree is not acceptable.  The regular routing calls need
// three caller-allocated intermediates (slot ranks, per-block histograms, the plan buffer); here
// those live in one file-scope device array of fixed size instead, so the call needs nothing but
// its inputs and outputs.
//
// Limits and rules
//   * at most BIBO_NOALLOC_MAX_TOKENS tokens per call (larger calls are refused with BIBO_ERR_UNSUPPORTED);
//     the array costs about 1.1 MB on every GPU that loads the library, for the life of the process;
//   * the FIRST call on each device looks up the array's device address (cudaGetSymbolAddress) and
//     sets kernel attributes; make that first call outside any stream capture;
//   * every call on a device shares the one array: the array keeps the previous call's contents (the
//     status word is cleared at the start of each call), and two calls whose kernels overlap on the
//     GPU (different streams, or different host threads) race on it -- serialise them;
//   * no cudaMalloc / cudaFree / allocating library routine is called on this path.
#include <mutex>

#include "common.cuh"

namespace bibo {

constexpr int64_t NA_TOKENS = BIBO_NOALLOC_MAX_TOKENS;
constexpr size_t align256(size_t v) { return (v + 255) / 256 * 256; }
constexpr size_t NA_RANK_BYTES = align256(NA_TOKENS * BIBO_MAX_TOP_K * sizeof(int32_t));
constexpr size_t NA_BLOCKS_BYTES =
    align256((NA_TOKENS / BIBO_ROUTER_BLOCK_TOKENS) * BIBO_MAX_EXPERTS * sizeof(int32_t));
constexpr size_t NA_PLAN_BYTES = align256(
    (PLAN_HDR + BIBO_MAX_EXPERTS + BIBO_MAX_EXPERTS + 1 + 3 + (NA_TOKENS / BIBO_ROUTER_BLOCK_TOKENS) * BIBO_MAX_EXPERTS +
     ((NA_TOKENS * BIBO_MAX_TOP_K + (int64_t)BIBO_MAX_EXPERTS * (BIBO_TILE_M - 1)) / BIBO_TILE_M + 1) * 7 + XG_WORDS) *
    sizeof(int32_t));
constexpr size_t NA_BYTES = NA_RANK_BYTES + NA_BLOCKS_BYTES + NA_PLAN_BYTES;

// The scratch itself.  In host code this name is only a stand-in for the symbol: the device address
// has to be asked for (below) before it can be given to a kernel.
static __device__ __align__(256) unsigned char g_route_scratch[NA_BYTES];

constexpr int NA_MAX_DEVICES = 64;
static std::mutex g_na_mu;
static unsigned char* g_na_ptr[NA_MAX_DEVICES] = {};

// Device address of the scratch array on the CURRENT device (looked up once per device).
static int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  BIBO_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= NA_MAX_DEVICES) return fail(BIBO_ERR_UNSUPPORTED, "route_noalloc: device index %d", dev);
  std::lock_guard<std::mutex> g(g_na_mu);
  if (g_na_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_route_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(BIBO_ERR_CUDA, "route_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                  cudaGetErrorString(e));
    g_na_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_na_ptr[dev];
  return BIBO_OK;
}

}  // namespace bibo

using namespace bibo;

extern "C" int bibo_moe_route_noalloc(const void* x, const void* w_router, const float* bias, int64_t n_tokens,
                                      int hidden, int n_experts, int top_k, int norm_mode, float scale, int dtype,
                                      int32_t* topk_idx, float* topk_w, int32_t* counts, void* stream) {
  if (n_tokens <= 0) {   // nothing to route: the histogram is all zeros (no scratch, no kernel)
    if (counts && n_experts > 0 && n_experts <= BIBO_MAX_EXPERTS)
      BIBO_CUDA(cudaMemsetAsync(counts, 0, (size_t)n_experts * sizeof(int32_t), static_cast<cudaStream_t>(stream)));
    return BIBO_OK;
  }
  if (!x || !w_router || !bias || !topk_idx || !topk_w || !counts)
    return fail(BIBO_ERR_ARG, "route_noalloc: null pointer");
  if (n_tokens > NA_TOKENS)
    return fail(BIBO_ERR_UNSUPPORTED,
                "route_noalloc: %lld tokens exceed the fixed scratch (max %lld per call); split the batch or use "
                "bibo_moe_router_fwd with caller-allocated buffers",
                (long long)n_tokens, (long long)NA_TOKENS);
  if (n_experts < 1 || n_experts > BIBO_MAX_EXPERTS || top_k < 1 || top_k > BIBO_MAX_TOP_K || top_k > n_experts)
    return fail(BIBO_ERR_UNSUPPORTED, "route_noalloc: n_experts=%d (max %d) top_k=%d (max %d)", n_experts,
                BIBO_MAX_EXPERTS, top_k, BIBO_MAX_TOP_K);
  if ((size_t)plan_words(n_tokens, top_k, n_experts, n_experts) * sizeof(int32_t) > NA_PLAN_BYTES)
    return fail(BIBO_ERR_UNSUPPORTED, "route_noalloc: plan does not fit the fixed scratch");
  unsigned char* base = nullptr;
  int rc = scratch_for_current_device(&base);
  if (rc) return rc;
  int32_t* slot_rank = reinterpret_cast<int32_t*>(base);
  int32_t* block_counts = reinterpret_cast<int32_t*>(base + NA_RANK_BYTES);
  int32_t* plan = reinterpret_cast<int32_t*>(base + NA_RANK_BYTES + NA_BLOCKS_BYTES);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the plan header (tile count, rows, sticky status word) must start at zero; everything else in
  // the scratch is fully rewritten by the two kernels before it is read
  BIBO_CUDA(cudaMemsetAsync(plan, 0, PLAN_HDR * sizeof(int32_t), st));
  rc = bibo_moe_router_fwd(x, w_router, bias, nullptr, n_tokens, hidden, n_experts, top_k, norm_mode, scale, dtype,
                           nullptr, topk_idx, topk_w, slot_rank, block_counts, plan + PLAN_STATUS, stream);
  if (rc) return rc;
  rc = bibo_moe_plan(block_counts, n_tokens, top_k, n_experts, n_experts, plan, stream);
  if (rc) return rc;
  BIBO_CUDA(cudaMemcpyAsync(counts, plan + plan_off_counts(), (size_t)n_experts * sizeof(int32_t),
                            cudaMemcpyDeviceToDevice, st));
  return BIBO_OK;
}

extern "C" int64_t bibo_moe_route_noalloc_max_tokens(void) { return NA_TOKENS; }

// The status word of the last bibo_moe_route_noalloc call on the current device lives inside the shared
// array; this copies it into a caller-owned device word (stream-ordered, no allocation, no synchronisation).
// 0 = fine; 1 = histogram total too large; 102 = a bounded wait of the router kernel gave up.
extern "C" int bibo_moe_route_noalloc_status(int32_t* status_out, void* stream) {
  if (!status_out) return fail(BIBO_ERR_ARG, "route_noalloc_status: null pointer");
  unsigned char* base = nullptr;
  int rc = scratch_for_current_device(&base);
  if (rc) return rc;
  const int32_t* plan = reinterpret_cast<const int32_t*>(base + NA_RANK_BYTES + NA_BLOCKS_BYTES);
  BIBO_CUDA(cudaMemcpyAsync(status_out, plan + PLAN_STATUS, sizeof(int32_t), cudaMemcpyDeviceToDevice,
                            static_cast<cudaStream_t>(stream)));
  return BIBO_OK;
}
