// K1 on tensor cores (bf16, 64 experts): one CTA per 128 tokens.  x tiles and the router weight
// stream through a TMA pipeline into tcgen05.mma (M=128 tokens, N=64 experts, fp32 accumulators in
// tensor memory); the logits tile is then copied to shared memory and the shared selection stage
// (router_select.cuh) produces indices, weights, ranks and the block histogram.  HBM-bound: x is
// read exactly once.
#include "router_select.cuh"
#include "tc_common.cuh"

namespace bibo {
namespace tc {

constexpr int R_BM = BIBO_ROUTER_BLOCK_TOKENS, R_BN = 64, R_BK = 64, R_STAGES = 4;
constexpr int R_A_BYTES = R_BM * R_BK * 2, R_B_BYTES = R_BN * R_BK * 2;
constexpr int R_LD = R_BN + 1;
constexpr int R_OFF_A = 0;
constexpr int R_OFF_B = R_OFF_A + R_STAGES * R_A_BYTES;
constexpr int R_OFF_SEL = R_OFF_B + R_STAGES * R_B_BYTES;          // select_and_rank scratch
constexpr int R_OFF_BAR = R_OFF_SEL + 2048;
constexpr int R_SMEM = R_OFF_BAR + 128 + 1024;
static_assert(R_BM * R_LD * 4 <= R_STAGES * R_A_BYTES, "the logits tile reuses the A stages");

__global__ void __launch_bounds__(128)
router_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                 const float* __restrict__ bias, int64_t n_tokens, int k_blocks, int top_k, int norm_mode,
                 float scale, float* __restrict__ logits_out, int32_t* __restrict__ topk_idx,
                 float* __restrict__ topk_w, int32_t* __restrict__ slot_rank, int32_t* __restrict__ block_counts,
                 int32_t* __restrict__ status, float* __restrict__ trace_blocks) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + R_OFF_BAR);
  uint64_t* empty = full + R_STAGES;
  uint64_t* done = empty + R_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* lg = reinterpret_cast<float*>(smem + R_OFF_A);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t0 = (int64_t)blockIdx.x * R_BM;
  const int rows = (int)min((int64_t)R_BM, n_tokens - t0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < R_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(done, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmX); prefetch_tmap(&tmW);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, R_BN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) break;
        mbar_expect_tx(&full[stage], R_A_BYTES + R_B_BYTES);
        tma_load_2d(smem + R_OFF_A + stage * R_A_BYTES, &tmX, &full[stage], kb * R_BK, (int)t0);
        tma_load_2d(smem + R_OFF_B + stage * R_B_BYTES, &tmW, &full[stage], kb * R_BK, 0);
        if (++stage == R_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(R_BM, R_BN);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < k_blocks; ++kb) {
        ok = mbar_wait(&full[stage], phase, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint64_t da = make_sdesc_k128(smem_u32(smem + R_OFF_A + stage * R_A_BYTES));
        const uint64_t db = make_sdesc_k128(smem_u32(smem + R_OFF_B + stage * R_B_BYTES));
#pragma unroll
        for (int k = 0; k < R_BK / 16; ++k) umma_bf16(tmem_base, da + k * 2, db + k * 2, idesc, (kb | k) != 0);
        umma_commit(&empty[stage]);
        if (++stage == R_STAGES) { stage = 0; phase ^= 1; }
      }
      if (ok) umma_commit(done);
    }
  }
  __syncwarp();
  const bool ok = mbar_wait(done, 0, abort_flag);
  tc_fence_after();
  if (ok) {
    // every load has landed and every MMA has finished reading shared memory: reuse the A stages
#pragma unroll
    for (int c = 0; c < R_BN / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) lg[(warp * 32 + lane) * R_LD + c * 32 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, R_BN); }
  if (!ok) {
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 102);
    return;
  }
  if (logits_out != nullptr) {
    for (int i = threadIdx.x; i < rows * R_BN; i += 128) {
      const int r = i / R_BN, c = i % R_BN;
      logits_out[(t0 + r) * R_BN + c] = lg[r * R_LD + c];
    }
    __syncthreads();
  }
  select_and_rank(lg, R_LD, reinterpret_cast<uint32_t*>(smem + R_OFF_SEL), bias, t0, rows, R_BN, top_k, norm_mode,
                  scale, topk_idx, topk_w, slot_rank, block_counts + (int64_t)blockIdx.x * R_BN,
                  trace_blocks ? trace_blocks + (int64_t)blockIdx.x * BIBO_TRACE_WORDS : nullptr);
}

}  // namespace tc

int router_tc_supported(int hidden, int n_experts, int dtype) {
  return dtype == BIBO_BF16 && n_experts == 64 && hidden % 64 == 0 && hidden >= 64;
}

int router_tc_launch(const void* x, const void* w_router, const float* bias, int64_t n_tokens, int hidden,
                     int n_experts, int top_k, int norm_mode, float scale, float* logits_out, int32_t* topk_idx,
                     float* topk_w, int32_t* slot_rank, int32_t* block_counts, int32_t* status, float* trace_blocks,
                     cudaStream_t st) {
  using namespace tc;
  CUtensorMap tmX, tmW;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tmX, x, (uint64_t)n_tokens, hidden, hidden, R_BM))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmW, w_router, (uint64_t)n_experts, hidden, hidden, R_BN))) return rc;
  static bool attr_done = false;
  if (!attr_done) {
    BIBO_CUDA(cudaFuncSetAttribute(router_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, R_SMEM));
    // same carve-out as the grouped GEMMs, so this kernel can share SMs with them (see ep.cu)
    cudaFuncSetAttribute(router_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         (int)cudaSharedmemCarveoutMaxShared);
    attr_done = true;
  }
  router_tc_kernel<<<(unsigned)router_blocks(n_tokens), 128, R_SMEM, st>>>(
      tmX, tmW, bias, n_tokens, hidden / R_BK, top_k, norm_mode, scale, logits_out, topk_idx, topk_w, slot_rank,
      block_counts, status, trace_blocks);
  BIBO_CHECK_LAUNCH("router_tc_kernel");
  return BIBO_OK;
}

}  // namespace bibo
