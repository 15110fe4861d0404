// K1 on tensor cores (bf16, 64 experts): one CTA per 128 tokens.  x tiles and the router weight
// stream through a TMA pipeline into tcgen05.mma (M=128 tokens, N=64 experts, fp32 accumulators in
// tensor memory); the logits tile is then copied to shared memory and the shared selection stage
// (router_select.cuh) produces indices, weights, ranks and the block histogram.  HBM-bound: x is
// read exactly once.
//
// NORM variant (the post-attention RMSNorm of BiBoDecoderLayer._ffn_forward, src/modeling/layers.py:60,
// folded into the loads): the tiles hold the raw residual stream h and the B operand is the router
// weight with the norm weight folded in (bf16(w_c W_ec), fold_norm_weight_kernel below).  Two otherwise
// idle warps read every staged tile next to the tensor core and add up h^2 per row; the accumulators
// are scaled by rstd = rsqrt(mean h^2 + eps) in the epilogue (rstd * sum_c h_c (w_c W_ec) = logits of
// the normalised row, with one bf16 rounding of an operand instead of the reference's two) and rstd is
// written out for the permute kernel, which produces the normalised rows for the experts.  The
// normalised activations never exist in HBM.
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
constexpr int R_OFF_SS = R_OFF_BAR + 128;                           // NORM: per-row sum of squares
constexpr int R_SMEM_NORM = R_OFF_SS + R_BM * 4 + 1024;
static_assert(R_BM * R_LD * 4 <= R_STAGES * R_A_BYTES, "the logits tile reuses the A stages");

template <bool NORM>
__global__ void __launch_bounds__(128)
router_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                 const float* __restrict__ bias, int64_t n_tokens, int k_blocks, int top_k, int norm_mode,
                 float scale, float* __restrict__ logits_out, int32_t* __restrict__ topk_idx,
                 float* __restrict__ topk_w, int32_t* __restrict__ slot_rank, int32_t* __restrict__ block_counts,
                 int32_t* __restrict__ status, float* __restrict__ trace_blocks,
                 float eps, float* __restrict__ rstd_out) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + R_OFF_BAR);
  uint64_t* empty = full + R_STAGES;
  uint64_t* done = empty + R_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* lg = reinterpret_cast<float*>(smem + R_OFF_A);
  float* s_ss = reinterpret_cast<float*>(smem + R_OFF_SS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t0 = (int64_t)blockIdx.x * R_BM;
  const int rows = (int)min((int64_t)R_BM, n_tokens - t0);
  if (threadIdx.x == 0) {
    // NORM: a stage is free once the tensor core and the two reading warps are done with it
    for (int s = 0; s < R_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], NORM ? 3 : 1); }
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
  } else if (NORM) {
    // warps 2 and 3: thread q owns rows q and q + 64 of every staged tile (any order of a row's eight
    // 16-byte pieces gives the same set of squares, so the 128-byte swizzle needs no undoing).  Lane l
    // starts at piece l & 7, so the eight lanes of a quarter warp touch eight different bank groups.
    const int q = threadIdx.x - 64;
    float ss[2] = {0.f, 0.f};
    int stage = 0; uint32_t phase = 0;
    for (int kb = 0; kb < k_blocks; ++kb) {
      if (!mbar_wait(&full[stage], phase, abort_flag)) break;
      const unsigned char* tile = smem + R_OFF_A + stage * R_A_BYTES;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = q + half * 64;
        float part = 0.f;                              // this k-block's 64 squares, added to the row total below
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 v = *reinterpret_cast<const uint4*>(tile + r * 128 + (((j + lane) & 7) << 4));
          const uint32_t* hv = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float a = bf16_lo(hv[i]), b = bf16_hi(hv[i]);
            part = fmaf(a, a, part);
            part = fmaf(b, b, part);
          }
        }
        ss[half] += part;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
      if (++stage == R_STAGES) { stage = 0; phase ^= 1; }
    }
    s_ss[q] = ss[0];
    s_ss[q + 64] = ss[1];
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
  if (NORM) {   // logits of the normalised row; s_ss was written before the barrier above
    const float rs = rsqrtf(s_ss[threadIdx.x] / (float)(k_blocks * R_BK) + eps);
    if ((int)threadIdx.x < rows) rstd_out[t0 + threadIdx.x] = rs;
#pragma unroll 8
    for (int c = 0; c < R_BN; ++c) lg[threadIdx.x * R_LD + c] *= rs;
    __syncthreads();
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

// w_fold[e][c] = bf16(w_router[e][c] * norm_w[c]): the B operand of the NORM variant
__global__ void fold_norm_weight_kernel(const uint4* __restrict__ w_router, const uint4* __restrict__ norm_w,
                                        int chunks_per_row, int64_t chunks, uint4* __restrict__ w_fold) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= chunks) return;
  uint4 a = __ldg(w_router + i);
  const uint4 b = __ldg(norm_w + (i % chunks_per_row));
  uint32_t* av = reinterpret_cast<uint32_t*>(&a);
  const uint32_t* bv = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
  for (int k = 0; k < 4; ++k)
    av[k] = tc::pack_bf16(tc::bf16_lo(av[k]) * tc::bf16_lo(bv[k]), tc::bf16_hi(av[k]) * tc::bf16_hi(bv[k]));
  w_fold[i] = a;
}

int fold_norm_weight_launch(const void* w_router, const void* norm_w, int n_experts, int hidden, void* w_fold,
                            cudaStream_t st) {
  const int64_t chunks = (int64_t)n_experts * hidden / 8;
  fold_norm_weight_kernel<<<(unsigned)((chunks + 255) / 256), 256, 0, st>>>(
      static_cast<const uint4*>(w_router), static_cast<const uint4*>(norm_w), hidden / 8, chunks,
      static_cast<uint4*>(w_fold));
  BIBO_CHECK_LAUNCH("fold_norm_weight_kernel");
  return BIBO_OK;
}

int router_tc_supported(int hidden, int n_experts, int dtype) {
  return dtype == BIBO_BF16 && n_experts == 64 && hidden % 64 == 0 && hidden >= 64;
}

int router_tc_launch(const void* x, const void* w_router, const float* bias, int64_t n_tokens, int hidden,
                     int n_experts, int top_k, int norm_mode, float scale, float* logits_out, int32_t* topk_idx,
                     float* topk_w, int32_t* slot_rank, int32_t* block_counts, int32_t* status, float* trace_blocks,
                     float eps, float* rstd_out, cudaStream_t st) {
  using namespace tc;
  const bool norm = rstd_out != nullptr;   // then x is the raw stream and w_router carries the norm weight
  CUtensorMap tmX, tmW;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tmX, x, (uint64_t)n_tokens, hidden, hidden, R_BM))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmW, w_router, (uint64_t)n_experts, hidden, hidden, R_BN))) return rc;
  static DeviceOnce once;
  rc = once.get([](int*) {
    BIBO_CUDA(cudaFuncSetAttribute(router_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, R_SMEM));
    BIBO_CUDA(cudaFuncSetAttribute(router_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, R_SMEM_NORM));
    // same carve-out as the grouped GEMMs, so this kernel can share SMs with them (see ep.cu)
    cudaFuncSetAttribute(router_tc_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         (int)cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(router_tc_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         (int)cudaSharedmemCarveoutMaxShared);
    return (int)BIBO_OK;
  });
  if (rc) return rc;
  if (norm)
    router_tc_kernel<true><<<(unsigned)router_blocks(n_tokens), 128, R_SMEM_NORM, st>>>(
        tmX, tmW, bias, n_tokens, hidden / R_BK, top_k, norm_mode, scale, logits_out, topk_idx, topk_w, slot_rank,
        block_counts, status, trace_blocks, eps, rstd_out);
  else
    router_tc_kernel<false><<<(unsigned)router_blocks(n_tokens), 128, R_SMEM, st>>>(
        tmX, tmW, bias, n_tokens, hidden / R_BK, top_k, norm_mode, scale, logits_out, topk_idx, topk_w, slot_rank,
        block_counts, status, trace_blocks, 0.f, nullptr);
  BIBO_CHECK_LAUNCH("router_tc_kernel");
  return BIBO_OK;
}

}  // namespace bibo
