// Selection stage of the router, shared by the CUDA-core and the tensor-core logits kernels.
//
// Input: a shared-memory tile of fp32 logits, one row per token of the block.
// Follows BiBoMoERouter.forward (src/modeling/ffn/router.py:31-51): score = sigmoid(logit);
// selection on score + bias; weights gathered from the un-biased scores; "sum" normalisation
// divides by (sum + 1e-20).  Ties go to the lower expert index, and the k experts are written in
// ascending expert index.
//
// Optional diagnostics (trace_row != nullptr): the block's sums of the per-token quantities that the
// boundary-gap probe (src/modeling/ffn/router.py:33-36) and RouterTrace._hook
// (ablate/common/router_trace.py:113-130) compute with extra launches:
//   [0] max_j p_j   [1] -sum_j |p_j| log |p_j|   [2] 1   [3] max_j w_j   [4] sum_j w_j   [5] min_j w_j
//   [6] score of rank k minus score of rank k+1 (raw scores, no bias)   [7] unused
// with w the weights as written and p = w / max(sum |w|, 1e-9).
#pragma once
#include "common.cuh"

namespace bibo {

// Shared-memory words select_and_rank needs after the logits tile.
__host__ __device__ inline size_t select_smem_bytes(int n_experts) {
  return sizeof(uint32_t) * (size_t)n_experts * (BIBO_ROUTER_BLOCK_TOKENS / 32) +
         sizeof(float) * (size_t)n_experts;
}

// lg: [BIBO_ROUTER_BLOCK_TOKENS][ld] logits (overwritten with scores); scratch: select_smem_bytes.
// Must be called by every thread of the block (blockDim.x >= BIBO_ROUTER_BLOCK_TOKENS) after the
// tile is complete and visible (the caller synchronises before the call).
__device__ __forceinline__ void select_and_rank(
    float* lg, int ld, uint32_t* scratch, const float* __restrict__ bias, int64_t t0, int rows,
    int n_experts, int top_k, int norm_mode, float scale, int32_t* __restrict__ topk_idx,
    float* __restrict__ topk_w, int32_t* __restrict__ slot_rank,
    int32_t* __restrict__ block_counts_row, float* __restrict__ trace_row = nullptr) {
  constexpr int WORDS = BIBO_ROUTER_BLOCK_TOKENS / 32;
  __shared__ float s_trace[BIBO_ROUTER_BLOCK_TOKENS / 32][BIBO_TRACE_WORDS];
  float tr[BIBO_TRACE_WORDS];
#pragma unroll
  for (int j = 0; j < BIBO_TRACE_WORDS; ++j) tr[j] = 0.f;
  uint32_t* mask = scratch;                                            // [n_experts][WORDS]
  float* bias_s = reinterpret_cast<float*>(scratch + n_experts * WORDS);  // [n_experts]
  const int tid = threadIdx.x;
  for (int i = tid; i < n_experts * WORDS; i += blockDim.x) mask[i] = 0u;
  for (int i = tid; i < n_experts; i += blockDim.x) bias_s[i] = bias[i];
  __syncthreads();

  int sel_idx[BIBO_MAX_TOP_K];
  float sel_s[BIBO_MAX_TOP_K];
  const bool active = tid < rows;
  if (active) {
    float* row = lg + tid * ld;
    // One pass over the experts keeps the BIBO_MAX_TOP_K best (key, index) pairs in registers, ordered by
    // key descending and, among equal keys, index ascending (a later expert never displaces an equal
    // key: strict '>'), which is the order k successive arg-max passes would produce; the first top_k
    // entries are the selection.
    float best_v[BIBO_MAX_TOP_K], best_s[BIBO_MAX_TOP_K];
    int best_i[BIBO_MAX_TOP_K];
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) { best_v[j] = -INFINITY; best_s[j] = 0.f; best_i[j] = -1; }
    for (int e = 0; e < n_experts; ++e) {
      const float s = sigmoid_accurate(row[e]);
      row[e] = s;
      const float v = s + bias_s[e];
      if (v > best_v[BIBO_MAX_TOP_K - 1] || best_i[BIBO_MAX_TOP_K - 1] < 0) {
        // shift down every entry that v beats (strictly, or an empty slot), then drop v into the gap
#pragma unroll
        for (int j = BIBO_MAX_TOP_K - 1; j >= 0; --j) {
          const bool beats = v > best_v[j] || best_i[j] < 0;
          const bool beats_prev = j > 0 && (v > best_v[j - 1] || best_i[j - 1] < 0);
          if (beats) {
            if (beats_prev) { best_v[j] = best_v[j - 1]; best_s[j] = best_s[j - 1]; best_i[j] = best_i[j - 1]; }
            else { best_v[j] = v; best_s[j] = s; best_i[j] = e; }
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) {
      sel_idx[j] = best_i[j];
      sel_s[j] = best_s[j];
    }
    // ascending expert index (insertion sort, k <= 8)
#pragma unroll
    for (int a = 1; a < BIBO_MAX_TOP_K; ++a) {
      if (a < top_k) {
#pragma unroll
        for (int b = a; b > 0; --b) {
          if (sel_idx[b] < sel_idx[b - 1]) {
            int ti = sel_idx[b]; sel_idx[b] = sel_idx[b - 1]; sel_idx[b - 1] = ti;
            float tf = sel_s[b]; sel_s[b] = sel_s[b - 1]; sel_s[b - 1] = tf;
          }
        }
      }
    }
    float w[BIBO_MAX_TOP_K];
    if (top_k > 1 && norm_mode == BIBO_NORM_SUM) {
      float tot = 0.f;
#pragma unroll
      for (int j = 0; j < BIBO_MAX_TOP_K; ++j) if (j < top_k) tot += sel_s[j];
      tot += 1e-20f;
#pragma unroll
      for (int j = 0; j < BIBO_MAX_TOP_K; ++j) if (j < top_k) w[j] = __fdiv_rn(sel_s[j], tot);
    } else if (top_k > 1 && norm_mode == BIBO_NORM_SOFTMAX) {
      float m = -INFINITY, tot = 0.f;
#pragma unroll
      for (int j = 0; j < BIBO_MAX_TOP_K; ++j) if (j < top_k) m = fmaxf(m, sel_s[j]);
#pragma unroll
      for (int j = 0; j < BIBO_MAX_TOP_K; ++j) if (j < top_k) { w[j] = expf(sel_s[j] - m); tot += w[j]; }
#pragma unroll
      for (int j = 0; j < BIBO_MAX_TOP_K; ++j) if (j < top_k) w[j] = __fdiv_rn(w[j], tot);
    } else {
#pragma unroll
      for (int j = 0; j < BIBO_MAX_TOP_K; ++j) if (j < top_k) w[j] = sel_s[j];
    }
    const int64_t base = (t0 + tid) * top_k;
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) {
      if (j < top_k) {
        topk_idx[base + j] = sel_idx[j];
        w[j] = (scale == 1.0f) ? w[j] : w[j] * scale;
        topk_w[base + j] = w[j];
        atomicOr(&mask[sel_idx[j] * WORDS + (tid >> 5)], 1u << (tid & 31));
      }
    }
    if (trace_row != nullptr) {
      float w_max = -INFINITY, w_min = INFINITY, w_sum = 0.f, l1 = 0.f;
#pragma unroll
      for (int j = 0; j < BIBO_MAX_TOP_K; ++j)
        if (j < top_k) { w_max = fmaxf(w_max, w[j]); w_min = fminf(w_min, w[j]); w_sum += w[j]; l1 += fabsf(w[j]); }
      l1 = fmaxf(l1, 1e-9f);
      float ent = 0.f;
#pragma unroll
      for (int j = 0; j < BIBO_MAX_TOP_K; ++j)
        if (j < top_k) { const float a = fabsf(__fdiv_rn(w[j], l1)); ent -= a * logf(fmaxf(a, 1e-12f)); }
      tr[0] = __fdiv_rn(w_max, l1); tr[1] = ent; tr[2] = 1.f; tr[3] = w_max; tr[4] = w_sum; tr[5] = w_min;
      if (top_k < n_experts) {
        // the top_k + 1 largest raw scores (the row now holds scores), descending; values only
        float tv[BIBO_MAX_TOP_K + 1];
#pragma unroll
        for (int j = 0; j <= BIBO_MAX_TOP_K; ++j) tv[j] = -INFINITY;
        for (int e = 0; e < n_experts; ++e) {
          const float s = row[e];
          if (s > tv[BIBO_MAX_TOP_K]) {
#pragma unroll
            for (int j = BIBO_MAX_TOP_K; j >= 0; --j) {
              const bool beats = s > tv[j];
              const bool beats_prev = j > 0 && s > tv[j - 1];
              if (beats) tv[j] = beats_prev ? tv[j - 1] : s;
            }
          }
        }
        float hi = 0.f, lo = 0.f;
#pragma unroll
        for (int j = 0; j <= BIBO_MAX_TOP_K; ++j) { if (j == top_k - 1) hi = tv[j]; if (j == top_k) lo = tv[j]; }
        tr[6] = hi - lo;
      }
    }
  }
  if (trace_row != nullptr) {   // fixed-order block sum: shuffle tree per warp, then the warps in order
#pragma unroll
    for (int j = 0; j < BIBO_TRACE_WORDS; ++j) {
      float v = tr[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if ((tid & 31) == 0 && tid < BIBO_ROUTER_BLOCK_TOKENS) s_trace[tid >> 5][j] = v;
    }
  }
  __syncthreads();
  if (trace_row != nullptr && tid < BIBO_TRACE_WORDS) {
    float v = 0.f;
#pragma unroll
    for (int q = 0; q < BIBO_ROUTER_BLOCK_TOKENS / 32; ++q) v += s_trace[q][tid];
    trace_row[tid] = v;
  }
  if (active) {
    const int64_t base = (t0 + tid) * top_k;
    const int wq = tid >> 5;
    const uint32_t lt = (1u << (tid & 31)) - 1u;
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) {
      if (j < top_k) {
        const uint32_t* m = mask + sel_idx[j] * WORDS;
        int r = __popc(m[wq] & lt);
        for (int q = 0; q < wq; ++q) r += __popc(m[q]);
        slot_rank[base + j] = r;
      }
    }
  }
  for (int e = tid; e < n_experts; e += blockDim.x) {
    int c = 0;
#pragma unroll
    for (int q = 0; q < WORDS; ++q) c += __popc(mask[e * WORDS + q]);
    block_counts_row[e] = c;
  }
}

}  // namespace bibo
