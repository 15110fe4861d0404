// 16-byte vectorised versions of the memory-bound backward kernels (same arithmetic as the scalar
// kernels in backward.cu; used when the row sizes are multiples of 16 bytes).
#pragma once
#include "common.cuh"

namespace bibo {

template <typename T> struct V16;
template <> struct V16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
  static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct V16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(u[i] << 16);
      f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* f) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = v;
  }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

// acc[0..N) += w * (16 bytes of T)
template <typename T> __device__ __forceinline__ void fma16(const uint4& v, float w, float* acc);
template <> __device__ __forceinline__ void fma16<float>(const uint4& v, float w, float* acc) {
  acc[0] = fmaf(__uint_as_float(v.x), w, acc[0]);
  acc[1] = fmaf(__uint_as_float(v.y), w, acc[1]);
  acc[2] = fmaf(__uint_as_float(v.z), w, acc[2]);
  acc[3] = fmaf(__uint_as_float(v.w), w, acc[3]);
}
template <> __device__ __forceinline__ void fma16<__nv_bfloat16>(const uint4& v, float w, float* acc) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] = fmaf(__uint_as_float(u[i] << 16), w, acc[2 * i]);
    acc[2 * i + 1] = fmaf(__uint_as_float(u[i] & 0xffff0000u), w, acc[2 * i + 1]);
  }
}

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// dY[row] = w * dOut[token], dw[t,j] = <dOut[t], y[row]>   (one warp per token)
template <typename T>
__global__ void __launch_bounds__(256)
combine_bwd_vec_kernel(const T* __restrict__ dout, const T* __restrict__ y, const T* __restrict__ x,
                       const int32_t* __restrict__ slot_row, const int32_t* __restrict__ topk_idx,
                       const float* __restrict__ topk_w, int64_t n_tokens, int hidden, int top_k, int n_glu, int n_pos,
                       T* __restrict__ dy, float* __restrict__ dw) {
  constexpr int VN = V16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const T* go = dout + t * hidden;
  const int chunks = hidden / VN;
  for (int j = 0; j < top_k; ++j) {
    const int row = slot_row[t * top_k + j];
    const float w = topk_w[t * top_k + j];
    float dot = 0.f;
    if (row >= 0) {
      const T* yr = y + (int64_t)row * hidden;
      T* dr = dy + (int64_t)row * hidden;
      for (int c = lane; c < chunks; c += 32) {
        float g[VN], yv[VN], o[VN];
        V16<T>::load(go + c * VN, g);
        V16<T>::load(yr + c * VN, yv);
#pragma unroll
        for (int i = 0; i < VN; ++i) { dot = fmaf(g[i], yv[i], dot); o[i] = g[i] * w; }
        V16<T>::store(dr + c * VN, o);
      }
    } else {
      const float sign = topk_idx[t * top_k + j] >= n_glu + n_pos ? -1.f : 1.f;
      const T* xr = x + t * hidden;
      for (int c = lane; c < chunks; c += 32) {
        float g[VN], xv[VN];
        V16<T>::load(go + c * VN, g);
        V16<T>::load(xr + c * VN, xv);
#pragma unroll
        for (int i = 0; i < VN; ++i) dot = fmaf(g[i], sign * xv[i], dot);
      }
    }
    dot = wsum(dot);
    if (lane == 0) dw[t * top_k + j] = dot;
  }
}

// Radial NormSiLU backward, one warp per row, in place on gate_up (see backward.cu for the formulas)
template <typename T>
__global__ void __launch_bounds__(256)
radial_bwd_vec_kernel(const T* __restrict__ dh, T* __restrict__ gate_up, const float* __restrict__ rnorm,
                      const float* __restrict__ theta, const int32_t* __restrict__ plan, int64_t tiles_off, int inter,
                      float* __restrict__ dtheta_row) {
  constexpr int VN = V16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= plan[PLAN_ROWS_USED]) return;
  const int4 tile = reinterpret_cast<const int4*>(plan + tiles_off)[row / BIBO_TILE_M];
  if (row >= tile.y + tile.z) {
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
  const int chunks = inter / VN;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int c = lane; c < chunks; c += 32) {
    float gv[VN], uv[VN], dv[VN];
    V16<T>::load(g + c * VN, gv); V16<T>::load(u + c * VN, uv); V16<T>::load(dhr + c * VN, dv);
#pragma unroll
    for (int i = 0; i < VN; ++i) {
      const float z = gv[i] * inv_r;
      const float sg = __fdiv_rn(1.0f, 1.0f + expf(-z));
      const float sl = z * sg;
      const float dA = dv[i] * uv[i];
      const float dz = dA * gain * (sg * (1.0f + z * (1.0f - sg)));
      s1 = fmaf(dA, sl, s1);
      s2 = fmaf(dz, gv[i], s2);
      s3 = fmaf(dA, sl * gain, s3);
    }
  }
  s1 = wsum(s1); s2 = wsum(s2); s3 = wsum(s3);
  const float dr = s1 * p * powf(r, p - 1.0f) - s2 * inv_r * inv_r;
  const float kg = dr * inv_r / (float)inter;
  if (lane == 0) dtheta_row[row] = p * (1.0f - p) * logf(r) * s3;
  for (int c = lane; c < chunks; c += 32) {
    float gv[VN], uv[VN], dv[VN], og[VN], ou[VN];
    V16<T>::load(g + c * VN, gv); V16<T>::load(u + c * VN, uv); V16<T>::load(dhr + c * VN, dv);
#pragma unroll
    for (int i = 0; i < VN; ++i) {
      const float z = gv[i] * inv_r;
      const float sg = __fdiv_rn(1.0f, 1.0f + expf(-z));
      const float a = V16<T>::round(z * sg * gain);
      const float dz = dv[i] * uv[i] * gain * (sg * (1.0f + z * (1.0f - sg)));
      og[i] = dz * inv_r + kg * gv[i];
      ou[i] = dv[i] * a;
    }
    V16<T>::store(g + c * VN, og);
    V16<T>::store(u + c * VN, ou);
  }
}

// sigmoid for the backward of the activation: exact form for fp32 tensors, one tanh.approx for bf16
// tensors (absolute error about 5e-4, below the bf16 resolution of the results)
template <typename T> __device__ __forceinline__ float bwd_sigmoid(float z) { return __fdiv_rn(1.0f, 1.0f + expf(-z)); }
template <> __device__ __forceinline__ float bwd_sigmoid<__nv_bfloat16>(float z) {
  float th;
  asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * z));
  return fmaf(0.5f, th, 0.5f);
}

// Same backward with the row held in registers (CPL 16-byte chunks per lane, inter == CPL * 32 * VN): every
// input is read once and the sigmoid evaluated once per element.
template <typename T, int CPL>
__global__ void __launch_bounds__(256)
radial_bwd_reg_kernel(const T* __restrict__ dh, T* __restrict__ gate_up, const float* __restrict__ rnorm,
                      const float* __restrict__ theta, const int32_t* __restrict__ plan, int64_t tiles_off, int inter,
                      float* __restrict__ dtheta_row) {
  constexpr int VN = V16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= plan[PLAN_ROWS_USED]) return;
  const int4 tile = reinterpret_cast<const int4*>(plan + tiles_off)[row / BIBO_TILE_M];
  if (row >= tile.y + tile.z) {
    if (lane == 0) dtheta_row[row] = 0.f;
    return;
  }
  T* g = gate_up + row * 2 * inter;
  T* u = g + inter;
  const T* dhr = dh + row * inter;
  float gv[CPL][VN], uv[CPL][VN], dv[CPL][VN];
#pragma unroll
  for (int q = 0; q < CPL; ++q) {
    const int c = q * 32 + lane;
    V16<T>::load(g + c * VN, gv[q]); V16<T>::load(u + c * VN, uv[q]); V16<T>::load(dhr + c * VN, dv[q]);
  }
  const float r = rnorm[row];
  const float p = sigmoid_accurate(theta[tile.x]);
  const float gain = powf(r, p);
  const float inv_r = __fdiv_rn(1.0f, r);
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
  for (int q = 0; q < CPL; ++q)
#pragma unroll
    for (int i = 0; i < VN; ++i) {
      const float z = gv[q][i] * inv_r;
      const float sg = bwd_sigmoid<T>(z);
      const float sl = z * sg;
      const float dA = dv[q][i] * uv[q][i];
      const float dz = dA * gain * (sg * (1.0f + z * (1.0f - sg)));
      s1 = fmaf(dA, sl, s1);
      s2 = fmaf(dz, gv[q][i], s2);
      s3 = fmaf(dA, sl * gain, s3);
      uv[q][i] = dv[q][i] * V16<T>::round(sl * gain);   // dUp
      dv[q][i] = dz * inv_r;                             // dGate without the norm term
    }
  s1 = wsum(s1); s2 = wsum(s2); s3 = wsum(s3);
  const float dr = s1 * p * powf(r, p - 1.0f) - s2 * inv_r * inv_r;
  const float kg = dr * inv_r / (float)inter;
  if (lane == 0) dtheta_row[row] = p * (1.0f - p) * logf(r) * s3;
#pragma unroll
  for (int q = 0; q < CPL; ++q) {
    const int c = q * 32 + lane;
#pragma unroll
    for (int i = 0; i < VN; ++i) dv[q][i] = fmaf(kg, gv[q][i], dv[q][i]);
    V16<T>::store(g + c * VN, dv[q]);
    V16<T>::store(u + c * VN, uv[q]);
  }
}

// dW_r[e, cols] = sum over the expert's rows of dlogit_row[row] * xp[row, cols].
// grid = (E_glu, ceil(H / (32*VN))), 256 threads = 8 row lanes x 32 column groups of VN columns.
template <typename T>
__global__ void __launch_bounds__(256)
router_dw_rows_vec_kernel(const float* __restrict__ dlogit_row, const T* __restrict__ xp,
                          const int32_t* __restrict__ counts, const int32_t* __restrict__ expert_off, int hidden,
                          T* __restrict__ dw_router) {
  constexpr int VN = V16<T>::N;
  __shared__ float sh[8][32 * VN + 1];
  const int e = blockIdx.x;
  const int rl = threadIdx.x >> 5, cg = threadIdx.x & 31;
  const int col = (blockIdx.y * 32 + cg) * VN;
  const int row0 = expert_off[e], cnt = counts[e];
  float acc[VN];
#pragma unroll
  for (int i = 0; i < VN; ++i) acc[i] = 0.f;
  if (col < hidden) {
#pragma unroll 4
    for (int r = rl; r < cnt; r += 8) {
      float v[VN];
      V16<T>::load(xp + (int64_t)(row0 + r) * hidden + col, v);
      const float d = dlogit_row[row0 + r];
#pragma unroll
      for (int i = 0; i < VN; ++i) acc[i] = fmaf(d, v[i], acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < VN; ++i) sh[rl][cg * VN + i] = acc[i];
  __syncthreads();
  if (rl == 0 && col < hidden) {
    float o[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) {
      float s = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) s += sh[q][cg * VN + i];   // fixed order
      o[i] = s;
    }
    V16<T>::store(dw_router + (int64_t)e * hidden + col, o);
  }
}

// dx gather + router Jacobian, one warp per token (see gather_dx_kernel in backward.cu)
template <typename T, int K>
__global__ void __launch_bounds__(256)
gather_dx_vec_kernel(const T* __restrict__ dxp, const T* __restrict__ dout, const T* __restrict__ x,
                     const T* __restrict__ w_router, const int32_t* __restrict__ slot_row,
                     const int32_t* __restrict__ topk_idx, const float* __restrict__ topk_w,
                     const float* __restrict__ dw, int64_t n_tokens, int hidden, int n_glu, int n_pos, int norm_mode,
                     float scale, T* __restrict__ dx, float* __restrict__ dlogit, float* __restrict__ dlogit_row,
                     const float* __restrict__ logits, int n_experts) {
  constexpr int VN = V16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const T* xr = x + t * hidden;
  const int chunks = hidden / VN;
  int ex[K], rows[K];
  float s[K], dl[K], wj[K], dot[K];
#pragma unroll
  for (int j = 0; j < K; ++j) {
    ex[j] = topk_idx[t * K + j];
    rows[j] = slot_row[t * K + j];
    wj[j] = topk_w[t * K + j];
    dot[j] = 0.f;
  }
  // the K selected logits: taken from the forward's logits when it kept them, else recomputed (x read once)
  for (int c = lane; logits == nullptr && c < chunks; c += 32) {
    float xv[VN];
    V16<T>::load(xr + c * VN, xv);
#pragma unroll
    for (int j = 0; j < K; ++j) {
      float wv[VN];
      V16<T>::load(w_router + (int64_t)ex[j] * hidden + c * VN, wv);
#pragma unroll
      for (int i = 0; i < VN; ++i) dot[j] = fmaf(xv[i], wv[i], dot[j]);
    }
  }
  float tot = 0.f, mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < K; ++j) {
    s[j] = logits != nullptr ? sigmoid_accurate(logits[t * n_experts + ex[j]])
                             : sigmoid_accurate(V16<T>::round(wsum(dot[j])));
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
#pragma unroll
  for (int j = 0; j < K; ++j) {
    const float dwn = dw[t * K + j] * scale;
    float ds;
    if (K > 1 && norm_mode == BIBO_NORM_SUM) ds = (dwn - dsum) / tot;
    else if (K > 1 && norm_mode == BIBO_NORM_SOFTMAX) ds = wn[j] * (dwn - dsum);
    else ds = dwn;
    dl[j] = V16<T>::round(ds * s[j] * (1.0f - s[j]));
    if (lane == 0) {
      dlogit[t * K + j] = dl[j];
      if (rows[j] >= 0) dlogit_row[rows[j]] = dl[j];
    }
  }
  // dx[t] = sum_j f_j * row_j + round(sum_j dl_j * W_r[e_j]); all 2K 16-byte loads of a chunk are issued
  // before the first is used (raw registers, converted at accumulation) to keep HBM busy
  const T* go = dout + t * hidden;
  const uint4* src[K];
  const uint4* wsrc[K];
  float f[K];
#pragma unroll
  for (int j = 0; j < K; ++j) {
    src[j] = reinterpret_cast<const uint4*>(rows[j] >= 0 ? dxp + (int64_t)rows[j] * hidden : go);
    wsrc[j] = reinterpret_cast<const uint4*>(w_router + (int64_t)ex[j] * hidden);
    f[j] = rows[j] >= 0 ? 1.0f : (ex[j] >= n_glu + n_pos ? -wj[j] : wj[j]);
  }
  for (int c = lane; c < chunks; c += 32) {
    uint4 v[K], wv[K];
#pragma unroll
    for (int j = 0; j < K; ++j) { v[j] = __ldcs(src[j] + c); wv[j] = __ldg(wsrc[j] + c); }
    float acc[VN], racc[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) acc[i] = racc[i] = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) { fma16<T>(v[j], f[j], acc); fma16<T>(wv[j], dl[j], racc); }
    float o[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) o[i] = acc[i] + V16<T>::round(racc[i]);
    V16<T>::store(dx + t * hidden + c * VN, o);
  }
}

}  // namespace bibo
