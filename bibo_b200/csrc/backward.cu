// Backward pass of the MoE block.  The reference has no hand-written backward: gradients come from
// autograd over src/modeling/ffn/router.py:25-51 and src/modeling/ffn/moe.py:47-101.  The kernels below
// implement the closed forms of those derivatives on the expert-contiguous layout of the forward:
//
//   combine_bwd      dY[row] = w * dOut[token]           dw[t,j] = <dOut[t], y[row]>   (moe.py:93)
//   gemm_bkn         dH  = dY  @ down_proj[e]            dXp = dGU @ gate_up_proj[e]   (moe.py:92,84)
//   gemm_dw          dW_d[e] = dY_e^T @ h_e              dW_gu[e] = dGU_e^T @ xp_e
//   radial_bwd       (dH, gate, up, r, theta) -> dGate|dUp, d theta                    (moe.py:85-92)
//   gather_dx        dx[t] = sum_j dXp[row(t,j)] + identity terms + router term; also the router's
//                    sum-norm / softmax Jacobian and sigmoid' -> dlogit[t,j]          (router.py:31-45)
//   router_dw        dW_r[e] = sum_t dlogit[t,e] * x[t]                                (router.py:26)
//
// With z = g/r, A = silu(z) r^p, h = a*u (a = A cast to the model dtype):
//   du = dh a,  dA = dh u,  dz = dA r^p silu'(z),  silu'(z) = s(z)(1 + z(1 - s(z))),
//   dr = sum_i dA_i silu(z_i) p r^(p-1) - sum_i dz_i g_i / r^2,  dg_i = dz_i / r + dr g_i / (I r),
//   dtheta_e += p(1-p) ln r sum_i dA_i A_i.
// All reductions run in a fixed order (no floating-point atomics), so gradients are deterministic.
// These are CUDA-core kernels (fp32 accumulation) for both dtypes.
#include <type_traits>

#include "backward_vec.cuh"
#include "common.cuh"

namespace bibo {

constexpr int BW = 8;  // warps per block in the row / token kernels

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- combine backward -----------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(BW * 32)
combine_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ y, const T* __restrict__ x,
                   const int32_t* __restrict__ slot_row, const int32_t* __restrict__ topk_idx,
                   const float* __restrict__ topk_w, int64_t n_tokens, int hidden, int top_k, int n_glu, int n_pos,
                   T* __restrict__ dy, float* __restrict__ dw) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * BW + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const T* go = dout + t * hidden;
  for (int j = 0; j < top_k; ++j) {
    const int row = slot_row[t * top_k + j];
    const float w = topk_w[t * top_k + j];
    float dot = 0.f;
    if (row >= 0) {
      const T* yr = y + (int64_t)row * hidden;
      T* dr = dy + (int64_t)row * hidden;
      for (int c = lane; c < hidden; c += 32) {
        const float g = to_f32<T>(go[c]);
        dot = fmaf(g, to_f32<T>(yr[c]), dot);
        dr[c] = from_f32<T>(g * w);
      }
    } else {  // +Identity / -Identity: output = +-w x
      const float sign = topk_idx[t * top_k + j] >= n_glu + n_pos ? -1.f : 1.f;
      const T* xr = x + t * hidden;
      for (int c = lane; c < hidden; c += 32) dot = fmaf(to_f32<T>(go[c]), sign * to_f32<T>(xr[c]), dot);
    }
    dot = warp_sum(dot);
    if (lane == 0) dw[t * top_k + j] = dot;
  }
}

// ---- grouped GEMM with B stored [K][N]: C[row, n] = sum_k A[row, k] B[e][k][n] -----------------------
template <typename T>
__global__ void __launch_bounds__(256)
grouped_gemm_bkn_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C,
                        const int32_t* __restrict__ plan, int64_t tiles_off, int k_dim, int n_out,
                        int64_t row_limit = INT64_MAX) {   // rows >= row_limit are neither read nor written
  if ((int)blockIdx.x >= plan[PLAN_N_TILES]) return;
  const int4 tile = reinterpret_cast<const int4*>(plan + tiles_off)[blockIdx.x];
  const int e = tile.x, row0 = tile.y, n0 = blockIdx.y * 64;
  __shared__ float As[16][BIBO_TILE_M + 1];
  __shared__ float Bs[16][64 + 1];
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const T* Ab = A + (int64_t)row0 * k_dim;
  const T* Bb = B + (int64_t)e * k_dim * n_out;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < k_dim; k0 += 16) {
    for (int i = tid; i < BIBO_TILE_M * 16; i += 256) {
      const int r = i / 16, c = i % 16;
      As[c][r] = (k0 + c < k_dim && row0 + r < row_limit) ? to_f32<T>(Ab[(int64_t)r * k_dim + k0 + c]) : 0.f;
    }
    for (int i = tid; i < 16 * 64; i += 256) {
      const int c = i / 64, n = i % 64;
      Bs[c][n] = (k0 + c < k_dim && n0 + n < n_out) ? to_f32<T>(Bb[(int64_t)(k0 + c) * n_out + n0 + n]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[8], b[4];
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = As[kk][ty * 8 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
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
      const int n = n0 + tx * 4 + j;
      if (n < n_out && row0 + ty * 8 + i < row_limit) C[(int64_t)(row0 + ty * 8 + i) * n_out + n] = from_f32<T>(acc[i][j]);
    }
}

// ---- weight gradients: C[e][m, n] = sum_{r in rows of e} A[r, m] B[r, n] ------------------------------
// grid = (ceil(m_dim/64), ceil(n_dim/64), E); the reduction runs over the expert's valid rows only.
template <typename T>
__global__ void __launch_bounds__(256)
grouped_gemm_dw_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C,
                       const int32_t* __restrict__ counts, const int32_t* __restrict__ expert_off, int m_dim,
                       int n_dim) {
  const int e = blockIdx.z, m0 = blockIdx.x * 64, n0 = blockIdx.y * 64;
  const int row0 = expert_off[e], cnt = counts[e];
  __shared__ float As[16][64 + 1];
  __shared__ float Bs[16][64 + 1];
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int r0 = 0; r0 < cnt; r0 += 16) {
    for (int i = tid; i < 16 * 64; i += 256) {
      const int r = i / 64, c = i % 64;
      const bool ok = r0 + r < cnt;
      As[r][c] = (ok && m0 + c < m_dim) ? to_f32<T>(A[(int64_t)(row0 + r0 + r) * m_dim + m0 + c]) : 0.f;
      Bs[r][c] = (ok && n0 + c < n_dim) ? to_f32<T>(B[(int64_t)(row0 + r0 + r) * n_dim + n0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  T* Cb = C + (int64_t)e * m_dim * n_dim;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < m_dim && n < n_dim) Cb[(int64_t)m * n_dim + n] = from_f32<T>(acc[i][j]);
    }
}

// ---- Radial NormSiLU backward: one warp per row, in place on gate_up -> dGate|dUp ------------------------
template <typename T>
__global__ void __launch_bounds__(BW * 32)
radial_bwd_kernel(const T* __restrict__ dh, T* __restrict__ gate_up, const float* __restrict__ rnorm,
                  const float* __restrict__ theta, const int32_t* __restrict__ plan, int64_t tiles_off, int inter,
                  float* __restrict__ dtheta_row) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * BW + (threadIdx.x >> 5);
  if (row >= plan[PLAN_ROWS_USED]) return;
  const int4 tile = reinterpret_cast<const int4*>(plan + tiles_off)[row / BIBO_TILE_M];
  if (row >= tile.y + tile.z) {  // padding row
    if (lane == 0) dtheta_row[row] = 0.f;
    return;
  }
  T* g = gate_up + row * 2 * inter;
  T* u = g + inter;
  const T* dhr = dh + row * inter;
  const float r = rnorm[row];
  const float p = sigmoid_accurate(theta[tile.x]);
  const float gain = powf(r, p);
  const float inv_r = __fdiv_rn(1.0f, r);
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;   // sum dA silu(z), sum dz g, sum dA A
  for (int i = lane; i < inter; i += 32) {
    const float gi = to_f32<T>(g[i]), ui = to_f32<T>(u[i]), d = to_f32<T>(dhr[i]);
    const float z = gi * inv_r;
    const float sg = __fdiv_rn(1.0f, 1.0f + expf(-z));
    const float sl = z * sg;
    const float dA = d * ui;
    const float dz = dA * gain * (sg * (1.0f + z * (1.0f - sg)));
    s1 = fmaf(dA, sl, s1);
    s2 = fmaf(dz, gi, s2);
    s3 = fmaf(dA, sl * gain, s3);
  }
  s1 = warp_sum(s1); s2 = warp_sum(s2); s3 = warp_sum(s3);
  const float dr = s1 * p * powf(r, p - 1.0f) - s2 * inv_r * inv_r;
  const float kg = dr * inv_r / (float)inter;
  if (lane == 0) dtheta_row[row] = p * (1.0f - p) * logf(r) * s3;
  for (int i = lane; i < inter; i += 32) {
    const float gi = to_f32<T>(g[i]), ui = to_f32<T>(u[i]), d = to_f32<T>(dhr[i]);
    const float z = gi * inv_r;
    const float sg = __fdiv_rn(1.0f, 1.0f + expf(-z));
    const float a = to_f32<T>(from_f32<T>(z * sg * gain));          // the activation as the forward cast it
    const float dz = d * ui * gain * (sg * (1.0f + z * (1.0f - sg)));
    g[i] = from_f32<T>(dz * inv_r + kg * gi);
    u[i] = from_f32<T>(d * a);
  }
}

// dtheta[e] = sum over the expert's rows, fixed order: one block per expert
__global__ void __launch_bounds__(256)
dtheta_reduce_kernel(const float* __restrict__ dtheta_row, const int32_t* __restrict__ counts,
                     const int32_t* __restrict__ expert_off, float* __restrict__ dtheta) {
  __shared__ float sh[256];
  const int e = blockIdx.x;
  const int row0 = expert_off[e], cnt = counts[e];
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

// ---- dx gather + router Jacobian --------------------------------------------------------------------------
// One warp per token.  Recomputes the k selected logits (dot products with the router rows), applies
// the normalisation Jacobian and sigmoid', writes dlogit[t,j] (and dlogit_row[row] for experts with
// rows), and accumulates dx[t] = sum_j dXp[row_j] + identity terms + sum_j dlogit_j W_r[e_j].
template <typename T>
__global__ void __launch_bounds__(BW * 32)
gather_dx_kernel(const T* __restrict__ dxp, const T* __restrict__ dout, const T* __restrict__ x,
                 const T* __restrict__ w_router, const int32_t* __restrict__ slot_row,
                 const int32_t* __restrict__ topk_idx, const float* __restrict__ topk_w, const float* __restrict__ dw,
                 int64_t n_tokens, int hidden, int top_k, int n_glu, int n_pos, int norm_mode, float scale,
                 T* __restrict__ dx, float* __restrict__ dlogit, float* __restrict__ dlogit_row) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * BW + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const T* xr = x + t * hidden;
  int ex[BIBO_MAX_TOP_K], rows[BIBO_MAX_TOP_K];
  float s[BIBO_MAX_TOP_K], dl[BIBO_MAX_TOP_K], wj[BIBO_MAX_TOP_K];
#pragma unroll
  for (int j = 0; j < BIBO_MAX_TOP_K; ++j) {
    if (j < top_k) {
      ex[j] = topk_idx[t * top_k + j];
      rows[j] = slot_row[t * top_k + j];
      wj[j] = topk_w[t * top_k + j];
      const T* wr = w_router + (int64_t)ex[j] * hidden;
      float dot = 0.f;
      for (int c = lane; c < hidden; c += 32) dot = fmaf(to_f32<T>(xr[c]), to_f32<T>(wr[c]), dot);
      dot = warp_sum(dot);
      // the reference rounds the logits to the model dtype before widening (router.py:26)
      s[j] = sigmoid_accurate(to_f32<T>(from_f32<T>(dot)));
    }
  }
  // normalisation Jacobian on the k selected scores
  float tot = 0.f, dsum = 0.f, mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < BIBO_MAX_TOP_K; ++j) if (j < top_k) { tot += s[j]; mx = fmaxf(mx, s[j]); }
  float wn[BIBO_MAX_TOP_K];
#pragma unroll
  for (int j = 0; j < BIBO_MAX_TOP_K; ++j) wn[j] = 0.f;
  if (top_k > 1 && norm_mode == BIBO_NORM_SUM) {
    tot += 1e-20f;
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) if (j < top_k) wn[j] = s[j] / tot;
  } else if (top_k > 1 && norm_mode == BIBO_NORM_SOFTMAX) {
    float z = 0.f;
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) if (j < top_k) { wn[j] = expf(s[j] - mx); z += wn[j]; }
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) if (j < top_k) wn[j] /= z;
  }
#pragma unroll
  for (int j = 0; j < BIBO_MAX_TOP_K; ++j) if (j < top_k) dsum += dw[t * top_k + j] * scale * wn[j];
#pragma unroll
  for (int j = 0; j < BIBO_MAX_TOP_K; ++j) {
    if (j < top_k) {
      const float dwn = dw[t * top_k + j] * scale;
      float ds;
      if (top_k > 1 && norm_mode == BIBO_NORM_SUM) ds = (dwn - dsum) / tot;
      else if (top_k > 1 && norm_mode == BIBO_NORM_SOFTMAX) ds = wn[j] * (dwn - dsum);
      else ds = dwn;
      // the gradient passes through the cast of the logits to the model dtype
      dl[j] = to_f32<T>(from_f32<T>(ds * s[j] * (1.0f - s[j])));
      if (lane == 0) {
        dlogit[t * top_k + j] = dl[j];
        if (rows[j] >= 0) dlogit_row[rows[j]] = dl[j];
      }
    }
  }
  const T* go = dout + t * hidden;
  for (int c = lane; c < hidden; c += 32) {
    float acc = 0.f, racc = 0.f;
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) {
      if (j < top_k) {
        if (rows[j] >= 0) acc += to_f32<T>(dxp[(int64_t)rows[j] * hidden + c]);
        else acc += (ex[j] >= n_glu + n_pos ? -wj[j] : wj[j]) * to_f32<T>(go[c]);
        racc = fmaf(dl[j], to_f32<T>(w_router[(int64_t)ex[j] * hidden + c]), racc);
      }
    }
    // expert path and router path are separate autograd branches, each cast to the model dtype
    dx[t * hidden + c] = from_f32<T>(acc + to_f32<T>(from_f32<T>(racc)));
  }
}

// ---- router weight gradient --------------------------------------------------------------------------------
// Experts with rows: dW_r[e, h] = sum over the expert's rows of dlogit_row[row] * xp[row, h]
// (grid = (E_glu, ceil(H/256)), thread per column, rows in ascending order).
template <typename T>
__global__ void __launch_bounds__(256)
router_dw_rows_kernel(const float* __restrict__ dlogit_row, const T* __restrict__ xp,
                      const int32_t* __restrict__ counts, const int32_t* __restrict__ expert_off, int hidden,
                      T* __restrict__ dw_router) {
  const int e = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
  if (c >= hidden) return;
  const int row0 = expert_off[e], cnt = counts[e];
  float acc = 0.f;
  for (int i = 0; i < cnt; ++i) acc = fmaf(dlogit_row[row0 + i], to_f32<T>(xp[(int64_t)(row0 + i) * hidden + c]), acc);
  dw_router[(int64_t)e * hidden + c] = from_f32<T>(acc);
}
// Experts without rows (+-Identity): scan all tokens (grid = (n_special, ceil(H/256))).
template <typename T>
__global__ void __launch_bounds__(256)
router_dw_scan_kernel(const float* __restrict__ dlogit, const int32_t* __restrict__ topk_idx, const T* __restrict__ x,
                      int64_t n_tokens, int hidden, int top_k, int n_glu, T* __restrict__ dw_router) {
  const int e = n_glu + blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
  if (c >= hidden) return;
  float acc = 0.f;
  for (int64_t t = 0; t < n_tokens; ++t)
    for (int j = 0; j < top_k; ++j)
      if (topk_idx[t * top_k + j] == e) acc = fmaf(dlogit[t * top_k + j], to_f32<T>(x[t * hidden + c]), acc);
  dw_router[(int64_t)e * hidden + c] = from_f32<T>(acc);
}

// Zero the padding rows of an expert-contiguous buffer (one warp per possible padding row): the
// weight-gradient GEMMs on the tensor cores reduce over whole 64-row blocks, padding included.
__global__ void __launch_bounds__(BW * 32)
zero_padding_rows_kernel(uint8_t* __restrict__ buf, const int32_t* __restrict__ counts,
                         const int32_t* __restrict__ expert_off, int n_glu, int row_bytes) {
  const int lane = threadIdx.x & 31;
  const int64_t p = (int64_t)blockIdx.x * BW + (threadIdx.x >> 5);
  const int e = (int)(p / (BIBO_TILE_M - 1));
  if (e >= n_glu) return;
  const int row = expert_off[e] + counts[e] + (int)(p % (BIBO_TILE_M - 1));
  if (row >= expert_off[e + 1]) return;
  uint4* dst = reinterpret_cast<uint4*>(buf + (int64_t)row * row_bytes);
  for (int c = lane; c < row_bytes / 16; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
}

// gemm_bwd_tc.cu
int gemm_dx_tc_supported(int k_dim, int n_out);
int gemm_dx_tc_launch(const void* A, const void* W, void* C, const PlanView& pv, int k_dim, int n_out,
                      int n_weight_experts, cudaStream_t st);
int gemm_dw_tc_supported(int m_dim, int n_dim);
int gemm_dw_tc_launch(const void* A, const void* B, void* C, const int32_t* plan, int64_t counts_off,
                      int64_t expert_off_off, int64_t rows_alloc, int n_experts, int m_dim, int n_dim,
                      cudaStream_t st);

template <typename T>
static int backward_t(const bibo_moe_shape* s, const T* x, const T* w_router, const T* gate_up_proj, const T* down_proj,
                      const float* theta, const bibo_moe_workspace* ws, const T* dout, const bibo_moe_bwd_workspace* b,
                      T* dx, T* d_w_router, T* d_gate_up_proj, T* d_down_proj, float* d_theta, cudaStream_t st) {
  const int64_t n = s->n_tokens;
  const int H = s->hidden, I = s->inter, E = s->n_experts, G = s->n_glu, k = s->top_k;
  const PlanView pv = local_plan_view(ws->plan, n, k, E, G);
  const int32_t* counts = ws->plan + plan_off_counts();
  const int32_t* expert_off = ws->plan + plan_off_expert_off(E);
  T* dy = static_cast<T*>(b->dy);
  T* dh = static_cast<T*>(b->dh);
  T* gu = static_cast<T*>(ws->gate_up);   // becomes dGate|dUp in place
  T* dxp = static_cast<T*>(ws->y);        // y is dead after combine_bwd: reused for dXp
  // tensor-core path: bf16, tile-friendly shapes, and a forward that zeroed the padding rows
  const bool use_tc = std::is_same<T, __nv_bfloat16>::value && (s->zero_padding & 1) && G > 0 && (H * 2) % 16 == 0 &&
                      gemm_dx_tc_supported(H, I) && gemm_dx_tc_supported(2 * I, H) && gemm_dw_tc_supported(H, I) &&
                      gemm_dw_tc_supported(2 * I, H) && aligned16(dy) && aligned16(dh) && aligned16(gu) &&
                      aligned16(dxp) && aligned16(ws->h) && aligned16(ws->xp) && aligned16(d_down_proj) &&
                      aligned16(d_gate_up_proj) && aligned16(down_proj) && aligned16(gate_up_proj);
  int rc;
  dim3 tok_grid((unsigned)((n + BW - 1) / BW));
  if (use_tc) {
    const int64_t pad_warps = (int64_t)G * (BIBO_TILE_M - 1);
    zero_padding_rows_kernel<<<(unsigned)((pad_warps + BW - 1) / BW), BW * 32, 0, st>>>(
        reinterpret_cast<uint8_t*>(dy), counts, expert_off, G, H * 2);
    BIBO_CHECK_LAUNCH("zero_padding_rows_kernel");
  }
  // 16-byte vectorised row kernels when every row size is a multiple of 16 bytes
  const bool vec = (H * sizeof(T)) % 16 == 0 && (I * sizeof(T)) % 16 == 0 && aligned16(dout) && aligned16(x) &&
                   aligned16(dx) && aligned16(ws->y) && aligned16(dy) && aligned16(dh) && aligned16(gu) &&
                   aligned16(w_router) && aligned16(d_w_router) && aligned16(ws->xp);
  if (vec)
    combine_bwd_vec_kernel<T><<<tok_grid, 256, 0, st>>>(dout, static_cast<const T*>(ws->y), x, ws->slot_row,
                                                        ws->topk_idx, ws->topk_w, n, H, k, G, s->n_pos, dy, b->dw);
  else
    combine_bwd_kernel<T><<<tok_grid, BW * 32, 0, st>>>(dout, static_cast<const T*>(ws->y), x, ws->slot_row,
                                                        ws->topk_idx, ws->topk_w, n, H, k, G, s->n_pos, dy, b->dw);
  BIBO_CHECK_LAUNCH("combine_bwd_kernel");
  if (G > 0) {
    if (use_tc) {
      if ((rc = gemm_dx_tc_launch(dy, down_proj, dh, pv, H, I, G, st))) return rc;
      if ((rc = gemm_dw_tc_launch(dy, ws->h, d_down_proj, ws->plan, plan_off_counts(), plan_off_expert_off(E),
                                  pv.rows_alloc, G, H, I, st)))
        return rc;
    } else {
      dim3 g1((unsigned)pv.tiles_cap, (unsigned)((I + 63) / 64));
      grouped_gemm_bkn_kernel<T><<<g1, 256, 0, st>>>(dy, down_proj, dh, pv.plan, pv.tiles_off, H, I);
      BIBO_CHECK_LAUNCH("grouped_gemm_bkn_kernel");
      dim3 g2((unsigned)((H + 63) / 64), (unsigned)((I + 63) / 64), (unsigned)G);
      grouped_gemm_dw_kernel<T><<<g2, 256, 0, st>>>(dy, static_cast<const T*>(ws->h), d_down_proj, counts, expert_off,
                                                    H, I);
      BIBO_CHECK_LAUNCH("grouped_gemm_dw_kernel");
    }
    dim3 rgrid((unsigned)((pv.rows_alloc + BW - 1) / BW));
    if (vec && I == 32 * V16<T>::N)
      radial_bwd_reg_kernel<T, 1><<<rgrid, 256, 0, st>>>(dh, gu, ws->rnorm, theta, pv.plan, pv.tiles_off, I, b->dtheta_row);
    else if (vec && I == 64 * V16<T>::N)
      radial_bwd_reg_kernel<T, 2><<<rgrid, 256, 0, st>>>(dh, gu, ws->rnorm, theta, pv.plan, pv.tiles_off, I, b->dtheta_row);
    else if (vec)
      radial_bwd_vec_kernel<T><<<rgrid, 256, 0, st>>>(dh, gu, ws->rnorm, theta, pv.plan, pv.tiles_off, I, b->dtheta_row);
    else
      radial_bwd_kernel<T><<<rgrid, BW * 32, 0, st>>>(dh, gu, ws->rnorm, theta, pv.plan, pv.tiles_off, I, b->dtheta_row);
    BIBO_CHECK_LAUNCH("radial_bwd_kernel");
    dtheta_reduce_kernel<<<G, 256, 0, st>>>(b->dtheta_row, counts, expert_off, d_theta);
    BIBO_CHECK_LAUNCH("dtheta_reduce_kernel");
    if (use_tc) {
      if ((rc = gemm_dx_tc_launch(gu, gate_up_proj, dxp, pv, 2 * I, H, G, st))) return rc;
      if ((rc = gemm_dw_tc_launch(gu, ws->xp, d_gate_up_proj, ws->plan, plan_off_counts(), plan_off_expert_off(E),
                                  pv.rows_alloc, G, 2 * I, H, st)))
        return rc;
    } else {
      dim3 g3((unsigned)pv.tiles_cap, (unsigned)((H + 63) / 64));
      grouped_gemm_bkn_kernel<T><<<g3, 256, 0, st>>>(gu, gate_up_proj, dxp, pv.plan, pv.tiles_off, 2 * I, H);
      BIBO_CHECK_LAUNCH("grouped_gemm_bkn_kernel");
      dim3 g4((unsigned)((2 * I + 63) / 64), (unsigned)((H + 63) / 64), (unsigned)G);
      grouped_gemm_dw_kernel<T><<<g4, 256, 0, st>>>(gu, static_cast<const T*>(ws->xp), d_gate_up_proj, counts,
                                                    expert_off, 2 * I, H);
      BIBO_CHECK_LAUNCH("grouped_gemm_dw_kernel");
    }
  }
  if (vec) {
#define BIBO_GDX(KK)                                                                                                \
  case KK:                                                                                                          \
    gather_dx_vec_kernel<T, KK><<<tok_grid, 256, 0, st>>>(dxp, dout, x, w_router, ws->slot_row, ws->topk_idx,       \
                                                          ws->topk_w, b->dw, n, H, G, s->n_pos, s->norm_mode,       \
                                                          s->scale, dx, b->dlogit, b->dlogit_row, ws->logits, E);    \
    break;
    switch (k) {
      BIBO_GDX(1) BIBO_GDX(2) BIBO_GDX(3) BIBO_GDX(4) BIBO_GDX(5) BIBO_GDX(6) BIBO_GDX(7) BIBO_GDX(8)
      default: return fail(BIBO_ERR_UNSUPPORTED, "backward: top_k=%d", k);
    }
#undef BIBO_GDX
  } else {
    gather_dx_kernel<T><<<tok_grid, BW * 32, 0, st>>>(dxp, dout, x, w_router, ws->slot_row, ws->topk_idx, ws->topk_w,
                                                      b->dw, n, H, k, G, s->n_pos, s->norm_mode, s->scale, dx,
                                                      b->dlogit, b->dlogit_row);
  }
  BIBO_CHECK_LAUNCH("gather_dx_kernel");
  if (G > 0) {
    if (vec) {
      constexpr int cols = 32 * V16<T>::N;
      dim3 g5v((unsigned)G, (unsigned)((H + cols - 1) / cols));
      router_dw_rows_vec_kernel<T><<<g5v, 256, 0, st>>>(b->dlogit_row, static_cast<const T*>(ws->xp), counts,
                                                        expert_off, H, d_w_router);
    } else {
      dim3 g5((unsigned)G, (unsigned)((H + 255) / 256));
      router_dw_rows_kernel<T><<<g5, 256, 0, st>>>(b->dlogit_row, static_cast<const T*>(ws->xp), counts, expert_off, H,
                                                   d_w_router);
    }
    BIBO_CHECK_LAUNCH("router_dw_rows_kernel");
  }
  if (E > G) {
    dim3 g6((unsigned)(E - G), (unsigned)((H + 255) / 256));
    router_dw_scan_kernel<T><<<g6, 256, 0, st>>>(b->dlogit, ws->topk_idx, x, n, H, k, G, d_w_router);
    BIBO_CHECK_LAUNCH("router_dw_scan_kernel");
  }
  return BIBO_OK;
}

// ---- CUDA-core pieces of the dense MLP backward (float32 and shapes outside the tensor-core kernels) -----
// [gate | up] rows -> [dGate | dUp] in place: a = T(silu(g)), dUp = dh * a, dGate = dh * up * silu'(g)
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_bwd_rows_kernel(const T* __restrict__ dh, T* __restrict__ gate_up, int64_t n_rows, int inter) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n_rows * inter) return;
  const int64_t r = i / inter;
  const int c = (int)(i % inter);
  T* g = gate_up + r * 2 * inter + c;
  T* u = g + inter;
  const float gg = to_f32<T>(*g), uu = to_f32<T>(*u), dd = to_f32<T>(dh[i]);
  const float sg = __fdiv_rn(1.0f, 1.0f + expf(-gg));
  const float a = to_f32<T>(from_f32<T>(gg * sg));
  *u = from_f32<T>(dd * a);
  *g = from_f32<T>(dd * uu * (sg * (1.0f + gg * (1.0f - sg))));
}

int mlp_backward_simt(const void* x, const void* w_gu, const void* down_proj, void* gate_up, const void* h,
                      const void* dout, int64_t n, int hidden, int inter, int dtype, const PlanView& pv,
                      const int32_t* counts, const int32_t* expert_off, void* dh, void* dx, void* d_w_gu, void* d_down,
                      cudaStream_t st) {
  auto run = [&](auto tag) {
    using T = decltype(tag);
    const T* X = static_cast<const T*>(x);
    const T* DO = static_cast<const T*>(dout);
    T* GU = static_cast<T*>(gate_up);
    dim3 g1((unsigned)pv.tiles_cap, (unsigned)((inter + 63) / 64));
    grouped_gemm_bkn_kernel<T><<<g1, 256, 0, st>>>(DO, static_cast<const T*>(down_proj), static_cast<T*>(dh), pv.plan,
                                                   pv.tiles_off, hidden, inter, n);
    dim3 g2((unsigned)((hidden + 63) / 64), (unsigned)((inter + 63) / 64), 1);
    grouped_gemm_dw_kernel<T><<<g2, 256, 0, st>>>(DO, static_cast<const T*>(h), static_cast<T*>(d_down), counts,
                                                  expert_off, hidden, inter);
    swiglu_bwd_rows_kernel<T><<<(unsigned)((n * inter + 255) / 256), 256, 0, st>>>(static_cast<const T*>(dh), GU, n, inter);
    dim3 g3((unsigned)pv.tiles_cap, (unsigned)((hidden + 63) / 64));
    grouped_gemm_bkn_kernel<T><<<g3, 256, 0, st>>>(GU, static_cast<const T*>(w_gu), static_cast<T*>(dx), pv.plan,
                                                   pv.tiles_off, 2 * inter, hidden, n);
    dim3 g4((unsigned)((2 * inter + 63) / 64), (unsigned)((hidden + 63) / 64), 1);
    grouped_gemm_dw_kernel<T><<<g4, 256, 0, st>>>(GU, X, static_cast<T*>(d_w_gu), counts, expert_off, 2 * inter, hidden);
  };
  if (dtype == BIBO_F32) run(float{});
  else run(__nv_bfloat16{});
  BIBO_CHECK_LAUNCH("mlp_backward_simt");
  return BIBO_OK;
}

}  // namespace bibo

using namespace bibo;

extern "C" int bibo_moe_backward(const bibo_moe_shape* s, const void* x, const void* w_router, const void* gate_up_proj,
                                 const void* down_proj, const float* theta, const bibo_moe_workspace* ws,
                                 const void* dout, const bibo_moe_bwd_workspace* bws, void* dx, void* d_w_router,
                                 void* d_gate_up_proj, void* d_down_proj, float* d_theta, void* stream) {
  if (!s || !ws || !bws) return fail(BIBO_ERR_ARG, "backward: null shape / workspace");
  if (s->n_tokens <= 0) return BIBO_OK;
  if (!x || !w_router || !theta || !dout || !dx || !d_w_router || !d_theta)
    return fail(BIBO_ERR_ARG, "backward: null tensor pointer");
  if (s->n_glu > 0 && (!gate_up_proj || !down_proj || !d_gate_up_proj || !d_down_proj))
    return fail(BIBO_ERR_ARG, "backward: null expert weight / gradient pointer");
  if (!ws->plan || !ws->slot_row || !ws->topk_idx || !ws->topk_w || !ws->xp || !ws->h || !ws->y || !ws->gate_up ||
      !ws->rnorm)
    return fail(BIBO_ERR_ARG, "backward: the forward workspace must keep xp, h, y, gate_up and rnorm");
  if (!bws->dy || !bws->dh || !bws->dw || !bws->dlogit || !bws->dlogit_row || !bws->dtheta_row)
    return fail(BIBO_ERR_ARG, "backward: incomplete backward workspace");
  if (s->top_k < 1 || s->top_k > BIBO_MAX_TOP_K || s->n_experts > BIBO_MAX_EXPERTS)
    return fail(BIBO_ERR_UNSUPPORTED, "backward: top_k=%d n_experts=%d", s->top_k, s->n_experts);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (s->dtype == BIBO_F32)
    return backward_t<float>(s, (const float*)x, (const float*)w_router, (const float*)gate_up_proj,
                             (const float*)down_proj, theta, ws, (const float*)dout, bws, (float*)dx,
                             (float*)d_w_router, (float*)d_gate_up_proj, (float*)d_down_proj, d_theta, st);
  if (s->dtype == BIBO_BF16)
    return backward_t<__nv_bfloat16>(s, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_router,
                                     (const __nv_bfloat16*)gate_up_proj, (const __nv_bfloat16*)down_proj, theta, ws,
                                     (const __nv_bfloat16*)dout, bws, (__nv_bfloat16*)dx, (__nv_bfloat16*)d_w_router,
                                     (__nv_bfloat16*)d_gate_up_proj, (__nv_bfloat16*)d_down_proj, d_theta, st);
  return fail(BIBO_ERR_ARG, "backward: dtype=%d", s->dtype);
}
