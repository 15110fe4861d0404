// K1 (general path): router logits + sigmoid + biased top-k + normalised weights + per-block
// histogram and in-block ranks, and the plan kernel that turns the histograms into row offsets.
//
// This file holds the CUDA-core version that accepts any dtype / hidden size / expert count; the
// bf16 tensor-core version (router_tc.cu) shares select_and_rank() below through router_select.cuh.
#include "common.cuh"
#include "router_select.cuh"

namespace bibo {

constexpr int RB = BIBO_ROUTER_BLOCK_TOKENS;  // tokens per block
constexpr int RK = 32;                        // k-chunk of the logits product
constexpr int RE = 64;                        // experts per accumulation pass

// One block: RB tokens.  256 threads; thread (ty,tx) owns 8 tokens x 4 experts of the pass.
template <typename T>
__global__ void __launch_bounds__(256)
router_simt_kernel(const T* __restrict__ x, const T* __restrict__ w_router,
                   const float* __restrict__ bias, const float* __restrict__ logits_in,
                   int64_t n_tokens, int hidden, int n_experts, int top_k, int norm_mode,
                   float scale, float* __restrict__ logits_out, int32_t* __restrict__ topk_idx,
                   float* __restrict__ topk_w, int32_t* __restrict__ slot_rank,
                   int32_t* __restrict__ block_counts, float* __restrict__ trace_blocks) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int ld = n_experts | 1;  // odd leading dimension -> conflict-free column walks
  float* lg = reinterpret_cast<float*>(smem_raw);                 // [RB][ld]
  float* As = lg + RB * ld;                                        // [RK][RB+1]
  float* Bs = As + RK * (RB + 1);                                  // [RK][RE+1]
  uint32_t* mask = reinterpret_cast<uint32_t*>(Bs + RK * (RE + 1));  // select_and_rank scratch

  const int tid = threadIdx.x;
  const int64_t t0 = (int64_t)blockIdx.x * RB;
  const int rows = (int)min((int64_t)RB, n_tokens - t0);

  if (logits_in != nullptr) {
    for (int i = tid; i < RB * n_experts; i += 256) {
      int r = i / n_experts, c = i % n_experts;
      lg[r * ld + c] = r < rows ? logits_in[(t0 + r) * n_experts + c] : 0.f;
    }
  } else {
    const int ty = tid / 16, tx = tid % 16;
    for (int e0 = 0; e0 < n_experts; e0 += RE) {
      float acc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
      for (int k0 = 0; k0 < hidden; k0 += RK) {
        for (int i = tid; i < RB * RK; i += 256) {
          int r = i / RK, c = i % RK;
          float v = 0.f;
          if (r < rows && k0 + c < hidden) v = to_f32<T>(x[(t0 + r) * hidden + k0 + c]);
          As[c * (RB + 1) + r] = v;
        }
        for (int i = tid; i < RE * RK; i += 256) {
          int r = i / RK, c = i % RK;
          float v = 0.f;
          if (e0 + r < n_experts && k0 + c < hidden)
            v = to_f32<T>(w_router[(int64_t)(e0 + r) * hidden + k0 + c]);
          Bs[c * (RE + 1) + r] = v;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < RK; ++kk) {
          float a[8], b[4];
#pragma unroll
          for (int i = 0; i < 8; ++i) a[i] = As[kk * (RB + 1) + ty * 8 + i];
#pragma unroll
          for (int j = 0; j < 4; ++j) b[j] = Bs[kk * (RE + 1) + tx * 4 + j];
#pragma unroll
          for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int e = e0 + tx * 4 + j;
          if (e < n_experts) lg[(ty * 8 + i) * ld + e] = acc[i][j];
        }
    }
  }
  __syncthreads();
  if (logits_out != nullptr) {
    for (int i = tid; i < rows * n_experts; i += 256) {
      int r = i / n_experts, c = i % n_experts;
      logits_out[(t0 + r) * n_experts + c] = lg[r * ld + c];
    }
    __syncthreads();
  }
  select_and_rank(lg, ld, mask, bias, t0, rows, n_experts, top_k, norm_mode, scale, topk_idx,
                  topk_w, slot_rank, block_counts + (int64_t)blockIdx.x * n_experts,
                  trace_blocks ? trace_blocks + (int64_t)blockIdx.x * BIBO_TRACE_WORDS : nullptr);
}

// ---- ranks for routing decided elsewhere ------------------------------------------------------------
// Same histogram / rank outputs as the router kernel, for callers that bring their own top-k
// indices (the BiBoFusedExperts.forward(x, idx, w) seam, src/modeling/ffn/moe.py:47-52).
__global__ void __launch_bounds__(RB)
rank_kernel(const int32_t* __restrict__ topk_idx, int64_t n_tokens, int n_experts, int top_k,
            int32_t* __restrict__ slot_rank, int32_t* __restrict__ block_counts,
            int32_t* __restrict__ status) {
  constexpr int WORDS = RB / 32;
  extern __shared__ uint32_t rmask[];  // [n_experts][WORDS]
  const int tid = threadIdx.x;
  const int64_t t = (int64_t)blockIdx.x * RB + tid;
  for (int i = tid; i < n_experts * WORDS; i += RB) rmask[i] = 0u;
  __syncthreads();
  int sel[BIBO_MAX_TOP_K];
  if (t < n_tokens) {
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) {
      if (j < top_k) {
        int e = topk_idx[t * top_k + j];
        if (e >= n_experts) { if (status) atomicExch(status, 2); e = -1; }   // out of range: reported, then ignored
        sel[j] = e;                                                          // negative = empty slot
        if (e >= 0) {
          uint32_t old = atomicOr(&rmask[e * WORDS + (tid >> 5)], 1u << (tid & 31));
          if ((old & (1u << (tid & 31))) && status) atomicExch(status, 3);  // one expert twice in a token
        }
      }
    }
  }
  __syncthreads();
  if (t < n_tokens) {
    const int wq = tid >> 5;
    const uint32_t lt = (1u << (tid & 31)) - 1u;
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) {
      if (j < top_k) {
        int r = 0;
        if (sel[j] >= 0) {
          const uint32_t* m = rmask + sel[j] * WORDS;
          r = __popc(m[wq] & lt);
          for (int q = 0; q < wq; ++q) r += __popc(m[q]);
        }
        slot_rank[t * top_k + j] = r;
      }
    }
  }
  for (int e = tid; e < n_experts; e += RB) {
    int c = 0;
#pragma unroll
    for (int q = 0; q < WORDS; ++q) c += __popc(rmask[e * WORDS + q]);
    block_counts[(int64_t)blockIdx.x * n_experts + e] = c;
  }
}

// ---- plan -----------------------------------------------------------------------------------------
// One block of 1024 threads.  Expert e is served by SUB = 1024 / EP threads (EP = experts rounded up
// to a power of two); each sums a contiguous run of blocks, the partial sums are scanned through
// shared memory, and a second pass writes the exclusive prefix per block.  Thread (sub, e) has
// index sub * EP + e, so a warp reads consecutive experts of one block row.
constexpr int PLAN_THREADS = 1024;
__global__ void __launch_bounds__(PLAN_THREADS)
plan_kernel(const int32_t* __restrict__ block_counts, int64_t n_tokens, int top_k, int n_experts,
            int n_glu, int ep, int32_t* __restrict__ plan, const float* __restrict__ trace_blocks,
            float* __restrict__ trace_acc, float* __restrict__ trace_counts, float* __restrict__ trace_gap) {
  __shared__ int s_part[PLAN_THREADS];
  __shared__ int s_padded[BIBO_MAX_EXPERTS + 1];
  __shared__ int s_count[BIBO_MAX_EXPERTS];
  const int tid = threadIdx.x;
  const int e = tid % ep, sub = tid / ep, n_sub = PLAN_THREADS / ep;
  const int nb = (int)router_blocks(n_tokens);
  const int per = (nb + n_sub - 1) / n_sub;
  const int b0 = min(sub * per, nb), b1 = min(b0 + per, nb);
  int32_t* counts = plan + plan_off_counts();
  int32_t* expert_off = plan + plan_off_expert_off(n_experts);
  int32_t* block_base = plan + plan_off_block_base(n_experts, n_glu);
  int4* tiles = reinterpret_cast<int4*>(plan + plan_off_tiles(n_tokens, n_experts, n_glu));
  int2* pairs = reinterpret_cast<int2*>(plan + plan_off_pairs(n_tokens, top_k, n_experts, n_glu));
  __shared__ int s_pair_off[BIBO_MAX_EXPERTS + 1];

  int sum = 0;
  if (e < n_experts)
    for (int b = b0; b < b1; ++b) sum += block_counts[(int64_t)b * n_experts + e];
  s_part[tid] = sum;
  __syncthreads();
  if (tid < ep) {  // one thread per expert scans its n_sub partial sums
    int acc = 0;
    for (int q = 0; q < n_sub; ++q) {
      const int v = s_part[q * ep + tid];
      s_part[q * ep + tid] = acc;
      acc += v;
    }
    if (tid < n_experts) {
      counts[tid] = acc;
      s_count[tid] = acc;
    }
    s_padded[tid] = (tid < n_glu) ? (acc + BIBO_TILE_M - 1) / BIBO_TILE_M * BIBO_TILE_M : 0;
  }
  __syncthreads();
  if (tid == 0) {  // exclusive scan of the padded row counts (<= 256 entries) and the total check
    int acc = 0, total = 0, pacc = 0;
    for (int i = 0; i < n_experts; ++i) total += s_count[i];
    for (int i = 0; i < n_glu; ++i) {
      const int v = s_padded[i];
      s_padded[i] = acc;
      s_pair_off[i] = pacc;
      acc += v;
      pacc += (v / BIBO_TILE_M + 1) / 2;
    }
    s_padded[n_glu] = acc;
    plan[PLAN_N_TILES] = acc / BIBO_TILE_M;
    plan[PLAN_ROWS_USED] = acc;
    plan[PLAN_N_PAIRS] = pacc;
    if (total > (long long)n_tokens * top_k) atomicMax(&plan[PLAN_STATUS], 1);  // sticky (fewer = empty slots)
  }
  if (e < n_experts) {
    int run = s_part[tid];
    for (int b = b0; b < b1; ++b) {
      const int c = block_counts[(int64_t)b * n_experts + e];
      block_base[(int64_t)b * n_experts + e] = run;
      run += c;
    }
  }
  __syncthreads();
  if (tid <= n_glu) expert_off[tid] = s_padded[tid];
  // tile list: thread (sub, e) writes every n_sub-th tile of expert e
  if (e < n_glu) {
    const int row0 = s_padded[e], cnt = s_count[e];
    const int t0 = row0 / BIBO_TILE_M;
    const int nt = (cnt + BIBO_TILE_M - 1) / BIBO_TILE_M;
    for (int i = sub; i < nt; i += n_sub) {
      tiles[t0 + i] = make_int4(e, row0 + i * BIBO_TILE_M, min(BIBO_TILE_M, cnt - i * BIBO_TILE_M), 0);
      if ((i & 1) == 0) pairs[s_pair_off[e] + i / 2] = make_int2(t0 + i, i + 1 < nt ? t0 + i + 1 : -1);
    }
  }
  // router diagnostics: warp j adds up word j of the router blocks' sums (lanes stride over the blocks,
  // then a fixed shuffle tree: the same bits every run) and folds it into the caller's accumulators
  // the way RouterTrace._hook / _router_hook do (ablate/common/router_trace.py:106-130)
  if (trace_blocks != nullptr) {
    const int w = tid >> 5, lane = tid & 31;
    if (w < BIBO_TRACE_WORDS) {
      float s = 0.f;
      for (int b = lane; b < nb; b += 32) s += trace_blocks[(int64_t)b * BIBO_TRACE_WORDS + w];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) {
        if (w == 6) {                          // mean boundary gap of this forward
          s = s / (float)n_tokens;
          if (trace_gap != nullptr) *trace_gap = s;
        }
        if (w == 7) s = 1.f;                   // router forwards seen
        if (trace_acc != nullptr) trace_acc[w] += s;
      }
    }
    if (trace_counts != nullptr && tid < n_experts) trace_counts[tid] += (float)s_count[tid];
  }
}

}  // namespace bibo

using namespace bibo;

extern "C" int bibo_moe_router_fwd(const void* x, const void* w_router, const float* bias,
                                   const float* logits_in, int64_t n_tokens, int hidden,
                                   int n_experts, int top_k, int norm_mode, float scale, int dtype,
                                   float* logits_out, int32_t* topk_idx, float* topk_w,
                                   int32_t* slot_rank, int32_t* block_counts, int32_t* status,
                                   void* stream);

namespace bibo {
int router_tc_supported(int hidden, int n_experts, int dtype);
int router_tc_launch(const void* x, const void* w_router, const float* bias, int64_t n_tokens,
                     int hidden, int n_experts, int top_k, int norm_mode, float scale,
                     float* logits_out, int32_t* topk_idx, float* topk_w, int32_t* slot_rank,
                     int32_t* block_counts, int32_t* status, float* trace_blocks, float eps, float* rstd_out,
                     cudaStream_t st);
int fold_norm_weight_launch(const void* w_router, const void* norm_w, int n_experts, int hidden, void* w_fold,
                            cudaStream_t st);
}

int bibo_moe_router_fwd(const void* x, const void* w_router, const float* bias,
                        const float* logits_in, int64_t n_tokens, int hidden, int n_experts,
                        int top_k, int norm_mode, float scale, int dtype, float* logits_out,
                        int32_t* topk_idx, float* topk_w, int32_t* slot_rank,
                        int32_t* block_counts, int32_t* status, void* stream) {
  return bibo_moe_router_fwd_trace(x, w_router, bias, logits_in, n_tokens, hidden, n_experts, top_k, norm_mode, scale,
                                   dtype, logits_out, topk_idx, topk_w, slot_rank, block_counts, status, nullptr, stream);
}

extern "C" int bibo_moe_router_fwd_trace(const void* x, const void* w_router, const float* bias,
                                         const float* logits_in, int64_t n_tokens, int hidden, int n_experts,
                                         int top_k, int norm_mode, float scale, int dtype, float* logits_out,
                                         int32_t* topk_idx, float* topk_w, int32_t* slot_rank,
                                         int32_t* block_counts, int32_t* status, float* trace_blocks,
                                         void* stream) {
  if (n_tokens <= 0) return BIBO_OK;
  if (!bias || !topk_idx || !topk_w || !slot_rank || !block_counts)
    return fail(BIBO_ERR_ARG, "router_fwd: null output or bias pointer");
  if (!logits_in && (!x || !w_router)) return fail(BIBO_ERR_ARG, "router_fwd: null x / w_router");
  if (n_experts < 1 || n_experts > BIBO_MAX_EXPERTS || top_k < 1 || top_k > BIBO_MAX_TOP_K ||
      top_k > n_experts)
    return fail(BIBO_ERR_UNSUPPORTED, "router_fwd: n_experts=%d (max %d) top_k=%d (max %d)",
                n_experts, BIBO_MAX_EXPERTS, top_k, BIBO_MAX_TOP_K);
  if (norm_mode < BIBO_NORM_RAW || norm_mode > BIBO_NORM_SOFTMAX)
    return fail(BIBO_ERR_ARG, "router_fwd: norm_mode=%d", norm_mode);
  if (dtype != BIBO_F32 && dtype != BIBO_BF16) return fail(BIBO_ERR_ARG, "router_fwd: dtype=%d", dtype);
  if (!logits_in && hidden < 1) return fail(BIBO_ERR_ARG, "router_fwd: hidden=%d", hidden);
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  if (!logits_in && router_tc_supported(hidden, n_experts, dtype) && aligned16(x) && aligned16(w_router))
    return router_tc_launch(x, w_router, bias, n_tokens, hidden, n_experts, top_k, norm_mode,
                            scale, logits_out, topk_idx, topk_w, slot_rank, block_counts, status, trace_blocks, 0.f,
                            nullptr, st);

  const int ld = n_experts | 1;
  size_t smem = sizeof(float) * ((size_t)RB * ld + RK * (RB + 1) + RK * (RE + 1)) +
                select_smem_bytes(n_experts);
  dim3 grid((unsigned)router_blocks(n_tokens));
  if (dtype == BIBO_F32) {
    auto kern = router_simt_kernel<float>;
    BIBO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, 256, smem, st>>>((const float*)x, (const float*)w_router, bias, logits_in,
                                  n_tokens, hidden, n_experts, top_k, norm_mode, scale, logits_out,
                                  topk_idx, topk_w, slot_rank, block_counts, trace_blocks);
  } else {
    auto kern = router_simt_kernel<__nv_bfloat16>;
    BIBO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, 256, smem, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w_router, bias,
                                  logits_in, n_tokens, hidden, n_experts, top_k, norm_mode, scale,
                                  logits_out, topk_idx, topk_w, slot_rank, block_counts, trace_blocks);
  }
  BIBO_CHECK_LAUNCH("router_simt_kernel");
  return BIBO_OK;
}

extern "C" int bibo_moe_router_norm_supported(int hidden, int n_experts, int dtype) {
  return router_tc_supported(hidden, n_experts, dtype);
}

extern "C" int bibo_moe_fold_norm_weight(const void* w_router, const void* norm_weight, int n_experts, int hidden,
                                         void* w_fold, void* stream) {
  if (!w_router || !norm_weight || !w_fold) return fail(BIBO_ERR_ARG, "fold_norm_weight: null pointer");
  if (n_experts < 1 || hidden < 8 || hidden % 8 != 0)
    return fail(BIBO_ERR_UNSUPPORTED, "fold_norm_weight: n_experts=%d hidden=%d", n_experts, hidden);
  if (!aligned16(w_router) || !aligned16(norm_weight) || !aligned16(w_fold))
    return fail(BIBO_ERR_ALIGN, "fold_norm_weight: pointers not 16-byte aligned");
  return fold_norm_weight_launch(w_router, norm_weight, n_experts, hidden, w_fold, static_cast<cudaStream_t>(stream));
}

extern "C" int bibo_moe_router_norm_fwd(const void* h, const void* w_fold, float eps, const float* bias,
                                        int64_t n_tokens, int hidden, int n_experts, int top_k, int norm_mode,
                                        float scale, float* logits_out, int32_t* topk_idx, float* topk_w,
                                        int32_t* slot_rank, int32_t* block_counts, int32_t* status,
                                        float* block_sums, float* rstd_out, void* stream) {
  if (n_tokens <= 0) return BIBO_OK;
  if (!h || !w_fold || !bias || !topk_idx || !topk_w || !slot_rank || !block_counts || !rstd_out)
    return fail(BIBO_ERR_ARG, "router_norm_fwd: null pointer");
  if (!bibo_moe_router_norm_supported(hidden, n_experts, BIBO_BF16))
    return fail(BIBO_ERR_UNSUPPORTED, "router_norm_fwd: bf16, 64 experts and hidden %% 64 == 0 only (hidden=%d, "
                "n_experts=%d)", hidden, n_experts);
  if (top_k < 1 || top_k > BIBO_MAX_TOP_K || top_k > n_experts)
    return fail(BIBO_ERR_UNSUPPORTED, "router_norm_fwd: top_k=%d", top_k);
  if (norm_mode < BIBO_NORM_RAW || norm_mode > BIBO_NORM_SOFTMAX)
    return fail(BIBO_ERR_ARG, "router_norm_fwd: norm_mode=%d", norm_mode);
  if (!aligned16(h) || !aligned16(w_fold)) return fail(BIBO_ERR_ALIGN, "router_norm_fwd: h / w_fold not 16-byte aligned");
  return router_tc_launch(h, w_fold, bias, n_tokens, hidden, n_experts, top_k, norm_mode, scale, logits_out, topk_idx,
                          topk_w, slot_rank, block_counts, status, block_sums, eps, rstd_out,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int bibo_moe_route_from_indices(const int32_t* topk_idx, int64_t n_tokens, int n_experts,
                                           int top_k, int32_t* slot_rank, int32_t* block_counts,
                                           int32_t* status, void* stream) {
  if (n_tokens <= 0) return BIBO_OK;
  if (!topk_idx || !slot_rank || !block_counts) return fail(BIBO_ERR_ARG, "route_from_indices: null pointer");
  if (n_experts < 1 || n_experts > BIBO_MAX_EXPERTS || top_k < 1 || top_k > BIBO_MAX_TOP_K)
    return fail(BIBO_ERR_UNSUPPORTED, "route_from_indices: n_experts=%d top_k=%d", n_experts, top_k);
  rank_kernel<<<(unsigned)router_blocks(n_tokens), RB, sizeof(uint32_t) * n_experts * (RB / 32),
                static_cast<cudaStream_t>(stream)>>>(topk_idx, n_tokens, n_experts, top_k, slot_rank,
                                                     block_counts, status);
  BIBO_CHECK_LAUNCH("rank_kernel");
  return BIBO_OK;
}

extern "C" int bibo_moe_plan(const int32_t* block_counts, int64_t n_tokens, int top_k,
                             int n_experts, int n_glu, int32_t* plan, void* stream) {
  return bibo_moe_plan_trace(block_counts, n_tokens, top_k, n_experts, n_glu, plan, nullptr, stream);
}

extern "C" int bibo_moe_plan_trace(const int32_t* block_counts, int64_t n_tokens, int top_k, int n_experts,
                                   int n_glu, int32_t* plan, const bibo_moe_router_trace* trace, void* stream) {
  if (trace && !trace->block_sums) return fail(BIBO_ERR_ARG, "plan: trace without block_sums");
  if (!block_counts || !plan) return fail(BIBO_ERR_ARG, "plan: null pointer");
  if (n_experts < 1 || n_experts > BIBO_MAX_EXPERTS || n_glu < 0 || n_glu > n_experts)
    return fail(BIBO_ERR_UNSUPPORTED, "plan: n_experts=%d n_glu=%d", n_experts, n_glu);
  if (n_tokens <= 0) return fail(BIBO_ERR_ARG, "plan: n_tokens=%lld", (long long)n_tokens);
  static DeviceOnce carve;   // same carve-out as the grouped GEMMs, so this kernel can share SMs with them (see ep.cu)
  int rc0 = carve.get([](int*) {
    BIBO_CUDA(cudaFuncSetAttribute(plan_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   (int)cudaSharedmemCarveoutMaxShared));
    return (int)BIBO_OK;
  });
  if (rc0) return rc0;
  int ep = 1;
  while (ep < n_experts) ep <<= 1;
  plan_kernel<<<1, PLAN_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(block_counts, n_tokens, top_k, n_experts,
                                                                       n_glu, ep, plan,
                                                                       trace ? trace->block_sums : nullptr,
                                                                       trace ? trace->acc : nullptr,
                                                                       trace ? trace->counts : nullptr,
                                                                       trace ? trace->gap : nullptr);
  BIBO_CHECK_LAUNCH("plan_kernel");
  return BIBO_OK;
}

extern "C" int64_t bibo_moe_rows_cap(int64_t n, int k, int g) { return rows_cap(n, k, g); }
extern "C" int64_t bibo_moe_tiles_cap(int64_t n, int k, int g) { return tiles_cap(n, k, g); }
extern "C" int64_t bibo_moe_router_blocks(int64_t n) { return router_blocks(n); }
extern "C" int64_t bibo_moe_plan_words(int64_t n, int k, int E, int g) { return plan_words(n, k, E, g); }
extern "C" int64_t bibo_moe_plan_off_counts(void) { return plan_off_counts(); }
extern "C" int64_t bibo_moe_plan_off_expert_off(int E) { return plan_off_expert_off(E); }
extern "C" int64_t bibo_moe_plan_off_block_base(int E, int g) { return plan_off_block_base(E, g); }
extern "C" int64_t bibo_moe_plan_off_tiles(int64_t n, int E, int g) { return plan_off_tiles(n, E, g); }
