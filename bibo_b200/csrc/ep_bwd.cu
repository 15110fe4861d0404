// Expert-parallel backward.  Mirror image of the forward exchange, again fused into the neighbouring
// kernels over peer memory:
//   home rank : combine-backward reads y rows from the owner ranks (peer loads) for dw = <dOut, y> and
//               writes dY = w * dOut straight into the owners' dY buffers (peer stores);
//   owner rank: the backward GEMMs and the radial backward run on the received rows (tensor cores);
//   home rank : the dx gather reads the dXp rows back from the owners (peer loads) and adds the
//               router term; the router weight gradient is formed from the local tokens.
// Expert weight gradients stay on the owner rank (each expert lives on exactly one rank); the router
// weight gradient is the LOCAL tokens' contribution (the caller all-reduces it like any replicated
// parameter).  bf16 only, tile-friendly shapes only (the tensor-core backward GEMMs).
#include <algorithm>

#include "backward_vec.cuh"
#include "ep_common.cuh"

namespace bibo {

// gemm_bwd_tc.cu
int gemm_dx_tc_supported(int k_dim, int n_out);
int gemm_dx_tc_launch(const void* A, const void* W, void* C, const PlanView& pv, int k_dim, int n_out,
                      int n_weight_experts, cudaStream_t st);
int gemm_dw_tc_supported(int m_dim, int n_dim);
int gemm_dw_tc_launch(const void* A, const void* B, void* C, const int32_t* plan, int64_t counts_off,
                      int64_t expert_off_off, int64_t rows_alloc, int n_experts, int m_dim, int n_dim,
                      cudaStream_t st);
__global__ void ep_barrier_kernel(PeerPtrs flags, int rank, int world, int epoch, int32_t* status);
__global__ void ep_zero_tile_padding_kernel(uint8_t* buf, const int32_t* plan, int64_t tiles_off, int row_bytes);

using bf16 = __nv_bfloat16;

// dY[owner,row] = w * dOut[t] (peer store), dw[t,j] = <dOut[t], y[owner,row]> (peer load); warp per token
template <int K>
__global__ void __launch_bounds__(256)
ep_combine_bwd_kernel(const bf16* __restrict__ dout, PeerPtrs y_peers, PeerPtrs dy_peers,
                      const int32_t* __restrict__ slot_row, const float* __restrict__ topk_w,
                      const int32_t* __restrict__ ep_plan, int64_t n_tokens, int hidden, int rows_cap_recv,
                      float* __restrict__ dw) {
  const int lane = threadIdx.x & 31;
  if (ep_plan[PLAN_STATUS] != 0) return;
  const int chunks = hidden / 8;
  for (int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); t < n_tokens; t += (int64_t)gridDim.x * 8) {
    const bf16* go = dout + t * hidden;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int g = slot_row[t * K + j];
      const float w = topk_w[t * K + j];
      const int o = g / rows_cap_recv, r = g % rows_cap_recv;
      const bf16* yr = static_cast<const bf16*>(y_peers.p[o]) + (int64_t)r * hidden;
      bf16* dr = static_cast<bf16*>(dy_peers.p[o]) + (int64_t)r * hidden;
      float dot = 0.f;
      for (int c = lane; c < chunks; c += 32) {
        float gv[8], yv[8], ov[8];
        V16<bf16>::load(go + c * 8, gv);
        V16<bf16>::load(yr + c * 8, yv);
#pragma unroll
        for (int i = 0; i < 8; ++i) { dot = fmaf(gv[i], yv[i], dot); ov[i] = gv[i] * w; }
        V16<bf16>::store(dr + c * 8, ov);
      }
      dot = wsum(dot);
      if (lane == 0) dw[t * K + j] = dot;
    }
  }
}

// per local expert: dtheta[le] = sum of dtheta_row over the expert's row range (padding rows hold 0)
__global__ void __launch_bounds__(256)
ep_dtheta_reduce_kernel(const float* __restrict__ dtheta_row, const int32_t* __restrict__ le_off,
                        float* __restrict__ dtheta) {
  __shared__ float sh[256];
  const int e = blockIdx.x;
  const int row0 = le_off[e], cnt = le_off[e + 1] - le_off[e];
  float s = 0.f;
  for (int i = threadIdx.x; i < cnt; i += 256) s += dtheta_row[row0 + i];
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) dtheta[e] = sh[0];
}

// dx gather with the dXp rows on the owner ranks; also dlogit[t,j] and dlogit_row[local row]
template <int K>
__global__ void __launch_bounds__(256)
ep_gather_dx_kernel(PeerPtrs dxp_peers, const bf16* __restrict__ x, const bf16* __restrict__ w_router,
                    const int32_t* __restrict__ slot_row, const int32_t* __restrict__ topk_idx,
                    const int32_t* __restrict__ slot_rank, const int32_t* __restrict__ local_plan,
                    const float* __restrict__ topk_w, const float* __restrict__ dw,
                    const int32_t* __restrict__ ep_plan, int64_t n_tokens, int hidden, int n_experts,
                    int rows_cap_recv, int norm_mode, float scale, bf16* __restrict__ dx,
                    float* __restrict__ dlogit_row) {
  const int lane = threadIdx.x & 31;
  if (ep_plan[PLAN_STATUS] != 0) return;
  const int chunks = hidden / 8;
  const int32_t* expert_off = local_plan + plan_off_expert_off(n_experts);
  const int32_t* block_base = local_plan + plan_off_block_base(n_experts, n_experts);
  for (int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); t < n_tokens; t += (int64_t)gridDim.x * 8) {
    const bf16* xr = x + t * hidden;
    int ex[K];
    float s[K], dl[K], dot[K];
    const bf16* src[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      ex[j] = topk_idx[t * K + j];
      const int g = slot_row[t * K + j];
      src[j] = static_cast<const bf16*>(dxp_peers.p[g / rows_cap_recv]) + (int64_t)(g % rows_cap_recv) * hidden;
      dot[j] = 0.f;
    }
    for (int c = lane; c < chunks; c += 32) {
      float xv[8];
      V16<bf16>::load(xr + c * 8, xv);
#pragma unroll
      for (int j = 0; j < K; ++j) {
        float wv[8];
        V16<bf16>::load(w_router + (int64_t)ex[j] * hidden + c * 8, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot[j] = fmaf(xv[i], wv[i], dot[j]);
      }
    }
    float tot = 0.f, mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      s[j] = sigmoid_accurate(V16<bf16>::round(wsum(dot[j])));
      tot += s[j];
      mx = fmaxf(mx, s[j]);
    }
    float wn[K], dsum = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) wn[j] = 0.f;
    if (K > 1 && norm_mode == BIBO_NORM_SUM) {
      tot += 1e-20f;
#pragma unroll
      for (int j = 0; j < K; ++j) wn[j] = s[j] / tot;
    } else if (K > 1 && norm_mode == BIBO_NORM_SOFTMAX) {
      float z = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) { wn[j] = expf(s[j] - mx); z += wn[j]; }
#pragma unroll
      for (int j = 0; j < K; ++j) wn[j] /= z;
    }
#pragma unroll
    for (int j = 0; j < K; ++j) dsum += dw[t * K + j] * scale * wn[j];
    const int64_t blk = t / BIBO_ROUTER_BLOCK_TOKENS;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const float dwn = dw[t * K + j] * scale;
      float ds;
      if (K > 1 && norm_mode == BIBO_NORM_SUM) ds = (dwn - dsum) / tot;
      else if (K > 1 && norm_mode == BIBO_NORM_SOFTMAX) ds = wn[j] * (dwn - dsum);
      else ds = dwn;
      dl[j] = V16<bf16>::round(ds * s[j] * (1.0f - s[j]));
      if (lane == 0)
        dlogit_row[expert_off[ex[j]] + block_base[blk * n_experts + ex[j]] + slot_rank[t * K + j]] = dl[j];
    }
    for (int c = lane; c < chunks; c += 32) {
      float acc[8], racc[8], v[K][8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = racc[i] = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) V16<bf16>::load(src[j] + c * 8, v[j]);
#pragma unroll
      for (int j = 0; j < K; ++j) {
        float wv[8];
        V16<bf16>::load(w_router + (int64_t)ex[j] * hidden + c * 8, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) { acc[i] += v[j][i]; racc[i] = fmaf(dl[j], wv[i], racc[i]); }
      }
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = acc[i] + V16<bf16>::round(racc[i]);
      V16<bf16>::store(dx + t * hidden + c * 8, o);
    }
  }
}

// dW_r[e, cols] = sum over the rows of expert e in the LOCAL expert-sorted order of
// dlogit_row[row] * x[row_token[row], cols]   (grid = (E, ceil(H/256)), 8 row lanes x 32 column groups)
__global__ void __launch_bounds__(256)
ep_router_dw_kernel(const float* __restrict__ dlogit_row, const int32_t* __restrict__ row_token,
                    const bf16* __restrict__ x, const int32_t* __restrict__ local_plan, int n_experts, int hidden,
                    bf16* __restrict__ dw_router) {
  __shared__ float sh[8][32 * 8 + 1];
  const int e = blockIdx.x;
  const int rl = threadIdx.x >> 5, cg = threadIdx.x & 31;
  const int col = (blockIdx.y * 32 + cg) * 8;
  const int row0 = local_plan[plan_off_expert_off(n_experts) + e], cnt = local_plan[plan_off_counts() + e];
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (col < hidden) {
#pragma unroll 4
    for (int r = rl; r < cnt; r += 8) {
      float v[8];
      V16<bf16>::load(x + (int64_t)row_token[row0 + r] * hidden + col, v);
      const float d = dlogit_row[row0 + r];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(d, v[i], acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) sh[rl][cg * 8 + i] = acc[i];
  __syncthreads();
  if (rl == 0 && col < hidden) {
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float s = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) s += sh[q][cg * 8 + i];
      o[i] = s;
    }
    V16<bf16>::store(dw_router + (int64_t)e * hidden + col, o);
  }
}

static PeerPtrs to_peers(void* const* tab, int world) {
  PeerPtrs pp = {};
  for (int i = 0; i < world; ++i) pp.p[i] = tab[i];
  return pp;
}

}  // namespace bibo

using namespace bibo;

extern "C" int bibo_moe_ep_barrier(void* const* flags_peers, int rank, int world, int epoch, int32_t* status,
                                   void* stream);

extern "C" int bibo_moe_ep_backward(const bibo_moe_ep_args* a, const bibo_moe_ep_bwd_args* b, void* stream) {
  if (!a || !b) return fail(BIBO_ERR_ARG, "ep_backward: null args");
  if (!a->gate_up_recv || !a->rnorm_recv || !a->row_token)
    return fail(BIBO_ERR_ARG, "ep_backward: the forward must have kept gate_up_recv, rnorm_recv and row_token");
  if (!b->dout || !b->dy_peers || !b->dh || !b->dw || !b->dlogit_row || !b->dtheta_row || !b->dx || !b->d_w_router ||
      !b->d_gate_up_proj || !b->d_down_proj || !b->d_theta)
    return fail(BIBO_ERR_ARG, "ep_backward: null pointer in the backward arguments");
  const int H = a->hidden, I = a->inter, E = a->n_experts, R = a->world, EL = E / R, k = a->top_k;
  if (!gemm_dx_tc_supported(H, I) || !gemm_dx_tc_supported(2 * I, H) || !gemm_dw_tc_supported(H, I) ||
      !gemm_dw_tc_supported(2 * I, H))
    return fail(BIBO_ERR_UNSUPPORTED, "ep_backward: hidden=%d inter=%d is outside the tensor-core backward kernels", H, I);
  if (k < 1 || k > BIBO_MAX_TOP_K) return fail(BIBO_ERR_UNSUPPORTED, "ep_backward: top_k=%d", k);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t n = a->n_tokens, cap = a->rows_cap_recv;
  int32_t* status = a->ep_plan + PLAN_STATUS;
  const PlanView pv = ep_plan_view(a->ep_plan, E, cap, a->max_ctas);
  const PeerPtrs yp = to_peers(a->y_peers, R), dyp = to_peers(b->dy_peers, R);
  void* dy_local = b->dy_peers[a->rank];
  void* dxp_local = a->y_peers[a->rank];   // y is dead after the combine backward: reused for dXp
  int64_t blocks = (n + 7) / 8;
  if (a->comm_ctas > 0) blocks = std::min<int64_t>(blocks, a->comm_ctas);
  int rc;

#define BIBO_EPK(KERNEL, ...)                                                                       \
  switch (k) {                                                                                      \
    case 1: KERNEL<1><<<(unsigned)blocks, 256, 0, st>>>(__VA_ARGS__); break;                        \
    case 2: KERNEL<2><<<(unsigned)blocks, 256, 0, st>>>(__VA_ARGS__); break;                        \
    case 3: KERNEL<3><<<(unsigned)blocks, 256, 0, st>>>(__VA_ARGS__); break;                        \
    case 4: KERNEL<4><<<(unsigned)blocks, 256, 0, st>>>(__VA_ARGS__); break;                        \
    case 5: KERNEL<5><<<(unsigned)blocks, 256, 0, st>>>(__VA_ARGS__); break;                        \
    case 6: KERNEL<6><<<(unsigned)blocks, 256, 0, st>>>(__VA_ARGS__); break;                        \
    case 7: KERNEL<7><<<(unsigned)blocks, 256, 0, st>>>(__VA_ARGS__); break;                        \
    default: KERNEL<8><<<(unsigned)blocks, 256, 0, st>>>(__VA_ARGS__); break;                       \
  }
  BIBO_EPK(ep_combine_bwd_kernel, static_cast<const bf16*>(b->dout), yp, dyp, a->slot_row, a->topk_w, a->ep_plan, n, H,
           (int)cap, b->dw);
  BIBO_CHECK_LAUNCH("ep_combine_bwd_kernel");
  if ((rc = bibo_moe_ep_barrier(a->flags_peers, a->rank, R, b->epoch_base + 1, status, stream))) return rc;

  // owner side: every dY row has landed
  ep_zero_tile_padding_kernel<<<(unsigned)pv.tiles_cap, 128, 0, st>>>(static_cast<uint8_t*>(dy_local), a->ep_plan,
                                                                     pv.tiles_off, H * 2);
  BIBO_CHECK_LAUNCH("ep_zero_tile_padding_kernel");
  if ((rc = gemm_dx_tc_launch(dy_local, a->down_proj, b->dh, pv, H, I, EL, st))) return rc;
  if ((rc = gemm_dw_tc_launch(dy_local, a->h, b->d_down_proj, a->ep_plan, ep_off_le_span(E), ep_off_le_off(E), cap, EL,
                              H, I, st)))
    return rc;
  const unsigned rgrid = (unsigned)((cap + 7) / 8);
  if (I == 512)
    radial_bwd_reg_kernel<bf16, 2><<<rgrid, 256, 0, st>>>(static_cast<const bf16*>(b->dh),
                                                          static_cast<bf16*>(a->gate_up_recv), a->rnorm_recv, a->theta,
                                                          a->ep_plan, pv.tiles_off, I, b->dtheta_row);
  else if (I == 256)
    radial_bwd_reg_kernel<bf16, 1><<<rgrid, 256, 0, st>>>(static_cast<const bf16*>(b->dh),
                                                          static_cast<bf16*>(a->gate_up_recv), a->rnorm_recv, a->theta,
                                                          a->ep_plan, pv.tiles_off, I, b->dtheta_row);
  else
    radial_bwd_vec_kernel<bf16><<<rgrid, 256, 0, st>>>(
        static_cast<const bf16*>(b->dh), static_cast<bf16*>(a->gate_up_recv), a->rnorm_recv, a->theta, a->ep_plan,
        pv.tiles_off, I, b->dtheta_row);
  BIBO_CHECK_LAUNCH("radial_bwd_vec_kernel");
  ep_dtheta_reduce_kernel<<<EL, 256, 0, st>>>(b->dtheta_row, a->ep_plan + ep_off_le_off(E), b->d_theta);
  BIBO_CHECK_LAUNCH("ep_dtheta_reduce_kernel");
  if ((rc = gemm_dx_tc_launch(a->gate_up_recv, a->gate_up_proj, dxp_local, pv, 2 * I, H, EL, st))) return rc;
  if ((rc = gemm_dw_tc_launch(a->gate_up_recv, a->xp_peers[a->rank], b->d_gate_up_proj, a->ep_plan, ep_off_le_span(E),
                              ep_off_le_off(E), cap, EL, 2 * I, H, st)))
    return rc;
  if ((rc = bibo_moe_ep_barrier(a->flags_peers, a->rank, R, b->epoch_base + 2, status, stream))) return rc;

  // home side: every dXp row is final
  BIBO_EPK(ep_gather_dx_kernel, yp, static_cast<const bf16*>(a->x), static_cast<const bf16*>(a->w_router), a->slot_row,
           a->topk_idx, a->slot_rank, a->local_plan, a->topk_w, b->dw, a->ep_plan, n, H, E, (int)cap, a->norm_mode,
           a->scale, static_cast<bf16*>(b->dx), b->dlogit_row);
  BIBO_CHECK_LAUNCH("ep_gather_dx_kernel");
#undef BIBO_EPK
  dim3 g((unsigned)E, (unsigned)((H + 255) / 256));
  ep_router_dw_kernel<<<g, 256, 0, st>>>(b->dlogit_row, a->row_token, static_cast<const bf16*>(a->x), a->local_plan, E,
                                         H, static_cast<bf16*>(b->d_w_router));
  BIBO_CHECK_LAUNCH("ep_router_dw_kernel");
  // the next forward's dispatch must not overwrite peers' buffers while they still read dXp: the
  // caller's next call starts with a barrier (histogram exchange) that every rank reaches only after
  // its own gather above has been enqueued and, in stream order, completed.
  return BIBO_OK;
}
