// RMSNorm in front of the feed-forward block (BiBoRMSNorm.forward, src/modeling/norm.py:19-24, called as
// post_attention_layernorm in BiBoDecoderLayer._ffn_forward, src/modeling/layers.py:57-67):
//   v = float(h);  y = T(v * rsqrt(mean(v^2) + eps));  out = weight * y   (product rounded to T)
// One warp per row, the row held in registers between the reduction and the output (one read, one write;
// HBM-bound).  Rows longer than 32 * 16-byte chunks * RN_MAX_CHUNKS take the two-pass loop.
#include "common.cuh"

namespace bibo {

constexpr int RN_MAX_CHUNKS = 8;   // 16-byte chunks a lane keeps in registers

template <typename T> struct RnVec;
template <> struct RnVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct RnVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(u[i] << 16); f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
  }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const T* __restrict__ h, const T* __restrict__ weight, float eps, int64_t n_rows, int hidden,
               T* __restrict__ out) {
  constexpr int VN = RnVec<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const uint4* src = reinterpret_cast<const uint4*>(h + row * hidden);
  const uint4* wv = reinterpret_cast<const uint4*>(weight);
  uint4* dst = reinterpret_cast<uint4*>(out + row * hidden);
  const int chunks = hidden / VN;
  const bool in_regs = chunks <= 32 * RN_MAX_CHUNKS;
  uint4 keep[RN_MAX_CHUNKS];
  float ss = 0.f;
  if (in_regs) {
#pragma unroll
    for (int q = 0; q < RN_MAX_CHUNKS; ++q) {
      const int c = q * 32 + lane;
      if (c < chunks) {
        keep[q] = __ldcs(src + c);
        float f[VN];
        RnVec<T>::unpack(keep[q], f);
#pragma unroll
        for (int i = 0; i < VN; ++i) ss = fmaf(f[i], f[i], ss);
      }
    }
  } else {
    for (int c = lane; c < chunks; c += 32) {
      float f[VN];
      RnVec<T>::unpack(src[c], f);
#pragma unroll
      for (int i = 0; i < VN; ++i) ss = fmaf(f[i], f[i], ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rs = rsqrtf(ss / (float)hidden + eps);
  auto emit = [&](int c, const uint4& raw) {
    float f[VN], w[VN];
    RnVec<T>::unpack(raw, f);
    RnVec<T>::unpack(__ldg(wv + c), w);
#pragma unroll
    for (int i = 0; i < VN; ++i) f[i] = w[i] * RnVec<T>::round(f[i] * rs);
    dst[c] = RnVec<T>::pack(f);
  };
  if (in_regs) {
#pragma unroll
    for (int q = 0; q < RN_MAX_CHUNKS; ++q) {
      const int c = q * 32 + lane;
      if (c < chunks) emit(c, keep[q]);
    }
  } else {
    for (int c = lane; c < chunks; c += 32) emit(c, src[c]);
  }
}

}  // namespace bibo

using namespace bibo;

extern "C" int bibo_moe_rmsnorm_fwd(const void* h, const void* weight, float eps, int64_t n_rows, int hidden, int dtype,
                                    void* out, void* stream) {
  if (n_rows <= 0) return BIBO_OK;
  if (!h || !weight || !out) return fail(BIBO_ERR_ARG, "rmsnorm_fwd: null pointer");
  if (dtype != BIBO_F32 && dtype != BIBO_BF16) return fail(BIBO_ERR_ARG, "rmsnorm_fwd: dtype=%d", dtype);
  const int row_bytes = hidden * (dtype == BIBO_F32 ? 4 : 2);
  if (hidden < 1 || row_bytes % 16 != 0)
    return fail(BIBO_ERR_UNSUPPORTED, "rmsnorm_fwd: row of %d bytes is not a multiple of 16", row_bytes);
  if (!aligned16(h) || !aligned16(weight) || !aligned16(out))
    return fail(BIBO_ERR_ALIGN, "rmsnorm_fwd: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((n_rows + 7) / 8);
  if (dtype == BIBO_F32)
    rmsnorm_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(h), static_cast<const float*>(weight), eps, n_rows,
                                               hidden, static_cast<float*>(out));
  else
    rmsnorm_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(h),
                                                       static_cast<const __nv_bfloat16*>(weight), eps, n_rows, hidden,
                                                       static_cast<__nv_bfloat16*>(out));
  BIBO_CHECK_LAUNCH("rmsnorm_kernel");
  return BIBO_OK;
}

// ---- backward ---------------------------------------------------------------------------------------------
// With v = float(h), rs = rsqrt(mean(v^2) + eps), xhat = v * rs, out = weight * T(xhat):
//   g      = float(T(dy * weight))                       (the reference multiplies in T)
//   dh     = T(rs * (g - xhat * mean(g * xhat)))
//   dweight[c] = sum over rows of dy[r,c] * T(xhat[r,c])
// Kernel 1: one warp per row writes dh and adds its dy * T(xhat) into the block's shared partial
// (RB rows per block, fixed order), blocks write partial[block][H] fp32.  Kernel 2 sums the partials of
// a column in block order.  No float atomics: results are deterministic.
namespace bibo {

constexpr int RB_WARPS = 8, RB_ROWS = 64;   // rows per block in the backward (8 warps x 8 rows each)

template <typename T>
__global__ void __launch_bounds__(RB_WARPS * 32)
rmsnorm_bwd_kernel(const T* __restrict__ h, const T* __restrict__ weight, const T* __restrict__ dy, float eps,
                   int64_t n_rows, int hidden, T* __restrict__ dh, float* __restrict__ partial) {
  extern __shared__ float acc_s[];                    // [RB_WARPS][hidden]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* mine = acc_s + (size_t)warp * hidden;
  for (int c = lane; c < hidden; c += 32) mine[c] = 0.f;
  const int64_t row0 = (int64_t)blockIdx.x * RB_ROWS;
  for (int i = 0; i < RB_ROWS / RB_WARPS; ++i) {
    const int64_t row = row0 + warp + (int64_t)i * RB_WARPS;
    if (row >= n_rows) break;
    const T* hr = h + row * hidden;
    const T* gr = dy + row * hidden;
    float ss = 0.f;
    for (int c = lane; c < hidden; c += 32) { const float v = to_f32<T>(hr[c]); ss = fmaf(v, v, ss); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rs = rsqrtf(ss / (float)hidden + eps);
    float dot = 0.f;
    for (int c = lane; c < hidden; c += 32) {
      const float xhat = to_f32<T>(hr[c]) * rs;
      const float g = to_f32<T>(from_f32<T>(to_f32<T>(gr[c]) * to_f32<T>(weight[c])));
      dot = fmaf(g, xhat, dot);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float m = dot / (float)hidden;
    for (int c = lane; c < hidden; c += 32) {
      const float xhat = to_f32<T>(hr[c]) * rs;
      const float gy = to_f32<T>(gr[c]);
      const float g = to_f32<T>(from_f32<T>(gy * to_f32<T>(weight[c])));
      dh[row * hidden + c] = from_f32<T>(rs * (g - xhat * m));
      mine[c] = fmaf(gy, to_f32<T>(from_f32<T>(xhat)), mine[c]);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < hidden; c += RB_WARPS * 32) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < RB_WARPS; ++w) s += acc_s[(size_t)w * hidden + c];   // fixed order
    partial[(int64_t)blockIdx.x * hidden + c] = s;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_dweight_kernel(const float* __restrict__ partial, int n_parts, int hidden, T* __restrict__ dweight) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= hidden) return;
  float s = 0.f;
  for (int p = 0; p < n_parts; ++p) s += partial[(int64_t)p * hidden + c];
  dweight[c] = from_f32<T>(s);
}

}  // namespace bibo

extern "C" int64_t bibo_moe_rmsnorm_bwd_parts(int64_t n_rows) { return (n_rows + RB_ROWS - 1) / RB_ROWS; }

extern "C" int bibo_moe_rmsnorm_bwd(const void* h, const void* weight, const void* dy, float eps, int64_t n_rows,
                                    int hidden, int dtype, void* dh, float* partial, void* dweight, void* stream) {
  if (n_rows <= 0) return BIBO_OK;
  if (!h || !weight || !dy || !dh || !partial || !dweight) return fail(BIBO_ERR_ARG, "rmsnorm_bwd: null pointer");
  if (dtype != BIBO_F32 && dtype != BIBO_BF16) return fail(BIBO_ERR_ARG, "rmsnorm_bwd: dtype=%d", dtype);
  const size_t smem = sizeof(float) * RB_WARPS * (size_t)hidden;
  if (hidden < 1 || smem > 200 * 1024) return fail(BIBO_ERR_UNSUPPORTED, "rmsnorm_bwd: hidden=%d", hidden);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n_parts = (int)bibo_moe_rmsnorm_bwd_parts(n_rows);
  if (dtype == BIBO_F32) {
    BIBO_CUDA(cudaFuncSetAttribute(rmsnorm_bwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    rmsnorm_bwd_kernel<float><<<n_parts, RB_WARPS * 32, smem, st>>>(
        static_cast<const float*>(h), static_cast<const float*>(weight), static_cast<const float*>(dy), eps, n_rows, hidden,
        static_cast<float*>(dh), partial);
    rmsnorm_dweight_kernel<float><<<(hidden + 255) / 256, 256, 0, st>>>(partial, n_parts, hidden,
                                                                        static_cast<float*>(dweight));
  } else {
    BIBO_CUDA(cudaFuncSetAttribute(rmsnorm_bwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    rmsnorm_bwd_kernel<__nv_bfloat16><<<n_parts, RB_WARPS * 32, smem, st>>>(
        static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(weight),
        static_cast<const __nv_bfloat16*>(dy), eps, n_rows, hidden, static_cast<__nv_bfloat16*>(dh), partial);
    rmsnorm_dweight_kernel<__nv_bfloat16><<<(hidden + 255) / 256, 256, 0, st>>>(partial, n_parts, hidden,
                                                                                static_cast<__nv_bfloat16*>(dweight));
  }
  BIBO_CHECK_LAUNCH("rmsnorm_bwd_kernel");
  return BIBO_OK;
}
