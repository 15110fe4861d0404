// K2 permute (token rows -> expert-contiguous rows) and K5 combine (weighted sum of a token's k
// expert rows).  Both are pure HBM-bandwidth kernels: one warp per token, 16-byte accesses.
#include "common.cuh"

namespace bibo {

constexpr int PW = 8;  // warps per block

// ---- K2 -------------------------------------------------------------------------------------------
// Warps [0, n_tokens): lane j < k computes the destination row of slot j; the rows are broadcast by
// shuffle and every lane copies its 16-byte chunks of x[t] to all k rows (x is read once).
// Warps [n_tokens, n_tokens + n_glu*(TILE_M-1)): mark (and optionally zero) one padding row each.
// With rstd / norm_w (bf16 rows only) x holds the raw residual stream and the copies are the RMSNorm
// of the row, rounded where BiBoRMSNorm.forward rounds (src/modeling/norm.py:19-24):
// bf16(w * bf16(h * rstd)).  A token with a slot on a +/-Identity expert also leaves its normalised row
// in xn[t] (the only rows of xn ever written), where the combine kernel finds it.
template <int VEC_BYTES>
__global__ void __launch_bounds__(PW * 32)
permute_kernel(const uint8_t* __restrict__ x, const int32_t* __restrict__ topk_idx,
               const int32_t* __restrict__ slot_rank, const int32_t* __restrict__ plan,
               int64_t n_tokens, int row_bytes, int n_experts, int n_glu, int top_k,
               int zero_padding, uint8_t* __restrict__ xp, int32_t* __restrict__ slot_row,
               int32_t* __restrict__ row_token, const float* __restrict__ rstd = nullptr,
               const uint8_t* __restrict__ norm_w = nullptr, uint8_t* __restrict__ xn = nullptr) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * PW + (threadIdx.x >> 5);
  const int32_t* counts = plan + plan_off_counts();
  const int32_t* expert_off = plan + plan_off_expert_off(n_experts);
  const int32_t* block_base = plan + plan_off_block_base(n_experts, n_glu);
  const int chunks = row_bytes / 16;

  if (w < n_tokens) {
    int my_row = -1;
    bool identity = false;       // a slot on a +/-Identity expert: the combine kernel reads the normalised row itself
    if (lane < top_k) {
      const int e = topk_idx[w * top_k + lane];
      identity = e >= n_glu && e < n_experts;
      if (e >= 0 && e < n_glu) {   // a negative index is an empty slot, one beyond the experts is ignored: no row
        const int64_t b = w / BIBO_ROUTER_BLOCK_TOKENS;
        my_row = expert_off[e] + block_base[b * n_experts + e] + slot_rank[w * top_k + lane];
        row_token[my_row] = (int32_t)w;
      }
      slot_row[w * top_k + lane] = my_row;
    }
    int rows[BIBO_MAX_TOP_K];
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) rows[j] = __shfl_sync(0xffffffffu, my_row, j);
    const uint4* src = reinterpret_cast<const uint4*>(x + w * row_bytes);
    const float rs = rstd != nullptr ? rstd[w] : 0.f;
    uint4* keep = (xn != nullptr && __any_sync(0xffffffffu, identity)) ? reinterpret_cast<uint4*>(xn + w * row_bytes)
                                                                      : nullptr;
    // a token without any row (all its slots empty or on +/-Identity experts) is not even read, unless its
    // normalised row has to be kept for the combine kernel
    const bool copy = __any_sync(0xffffffffu, my_row >= 0) || keep != nullptr;
    // eight 16-byte loads of the row are in flight per lane before the first of the (up to k x 8) stores
    for (int c0 = lane; c0 < (copy ? chunks : 0); c0 += 256) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (c0 + u * 32 < chunks) v[u] = __ldg(src + c0 + u * 32);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int c = c0 + u * 32;
        if (c >= chunks) continue;
        if (rstd != nullptr) {
          const uint4 wv = __ldg(reinterpret_cast<const uint4*>(norm_w) + c);
          uint32_t* hv = reinterpret_cast<uint32_t*>(&v[u]);
          const uint32_t* ww = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float a = __uint_as_float(hv[i] << 16), b = __uint_as_float(hv[i] & 0xffff0000u);
            const float na = __bfloat162float(__float2bfloat16_rn(a * rs)), nb = __bfloat162float(__float2bfloat16_rn(b * rs));
            const __nv_bfloat162 o = __floats2bfloat162_rn(na * __uint_as_float(ww[i] << 16),
                                                           nb * __uint_as_float(ww[i] & 0xffff0000u));
            hv[i] = *reinterpret_cast<const uint32_t*>(&o);
          }
          if (keep != nullptr) keep[c] = v[u];
        }
#pragma unroll
        for (int j = 0; j < BIBO_MAX_TOP_K; ++j)
          if (j < top_k && rows[j] >= 0)
            reinterpret_cast<uint4*>(xp + (int64_t)rows[j] * row_bytes)[c] = v[u];
      }
    }
  } else {
    const int64_t p = w - n_tokens;
    const int e = (int)(p / (BIBO_TILE_M - 1));
    if (e >= n_glu) return;
    const int row = expert_off[e] + counts[e] + (int)(p % (BIBO_TILE_M - 1));
    if (row >= expert_off[e + 1]) return;
    if (lane == 0) row_token[row] = -1;
    if (zero_padding) {
      uint4* dst = reinterpret_cast<uint4*>(xp + (int64_t)row * row_bytes);
      for (int c = lane; c < chunks; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
    }
  }
}

// ---- K2 without the copy ------------------------------------------------------------------------------
// The row maps alone (slot_row, row_token), for the gate/up kernel that gathers its own rows: thread per
// slot; threads beyond the slots mark one padding row each.  A slot whose expert index is negative is an
// empty slot (no row); indices >= n_glu are +/-Identity experts (no row either).
__global__ void __launch_bounds__(256)
rowmap_kernel(const int32_t* __restrict__ topk_idx, const int32_t* __restrict__ slot_rank,
              const int32_t* __restrict__ plan, int64_t n_tokens, int n_experts, int n_glu, int top_k,
              int32_t* __restrict__ slot_row, int32_t* __restrict__ row_token) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t slots = n_tokens * top_k;
  const int32_t* counts = plan + plan_off_counts();
  const int32_t* expert_off = plan + plan_off_expert_off(n_experts);
  const int32_t* block_base = plan + plan_off_block_base(n_experts, n_glu);
  if (i < slots) {
    const int64_t t = i / top_k;
    const int e = topk_idx[i];
    int row = -1;
    if (e >= 0 && e < n_glu) {
      row = expert_off[e] + block_base[(t / BIBO_ROUTER_BLOCK_TOKENS) * n_experts + e] + slot_rank[i];
      row_token[row] = (int32_t)t;
    }
    slot_row[i] = row;
  } else {
    const int64_t p = i - slots;
    const int e = (int)(p / (BIBO_TILE_M - 1));
    if (e >= n_glu) return;
    const int row = expert_off[e] + counts[e] + (int)(p % (BIBO_TILE_M - 1));
    if (row < expert_off[e + 1]) row_token[row] = -1;
  }
}

// ---- K5 -------------------------------------------------------------------------------------------
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const void* p, float* f) {
    float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(void* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const void* p, float* f) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ void store(void* p, const float* f) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = v;
  }
};

// 16 bytes of T -> fp32 multiply-accumulate
template <typename T> struct Acc16;
template <> struct Acc16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void fma(const uint4& v, float w, float* acc) {
    acc[0] = fmaf(__uint_as_float(v.x), w, acc[0]);
    acc[1] = fmaf(__uint_as_float(v.y), w, acc[1]);
    acc[2] = fmaf(__uint_as_float(v.z), w, acc[2]);
    acc[3] = fmaf(__uint_as_float(v.w), w, acc[3]);
  }
};
template <> struct Acc16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void fma(const uint4& v, float w, float* acc) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] = fmaf(__uint_as_float(u[i] << 16), w, acc[2 * i]);
      acc[2 * i + 1] = fmaf(__uint_as_float(u[i] & 0xffff0000u), w, acc[2 * i + 1]);
    }
  }
};

// acc[i] = T(acc[i]) + v[i]: the sum is rounded to T before the second term is added
template <typename T> __device__ __forceinline__ void add_rounded(float* acc, const uint4& v);
template <> __device__ __forceinline__ void add_rounded<float>(float* acc, const uint4& v) {
  acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y);
  acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void add_rounded<__nv_bfloat16>(float* acc, const uint4& v) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] = __bfloat162float(__float2bfloat16_rn(acc[2 * i])) + __uint_as_float(u[i] << 16);
    acc[2 * i + 1] = __bfloat162float(__float2bfloat16_rn(acc[2 * i + 1])) + __uint_as_float(u[i] & 0xffff0000u);
  }
}

// One warp per token; the k rows are summed in slot order (= ascending expert index), fp32.
// All k 16-byte loads of a chunk are issued before the first is used (raw registers, converted
// only at accumulation), and two chunks are in flight per lane, to keep HBM busy.
template <typename T, int K>
__global__ void __launch_bounds__(PW * 32, 4)
combine_kernel(const T* __restrict__ y, const T* __restrict__ x, const int32_t* __restrict__ slot_row,
               const int32_t* __restrict__ topk_idx, const float* __restrict__ topk_w,
               int64_t n_tokens, int hidden, int n_glu, int n_pos, T* __restrict__ out,
               const T* __restrict__ addend) {
  constexpr int VN = Acc16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * PW + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  int my_row = -1;
  float my_w = 0.f;
  if (lane < K) {
    my_row = slot_row[t * K + lane];
    my_w = topk_w[t * K + lane];
    if (my_row < 0) {  // +Identity / -Identity expert: contributes +w*x or -w*x; a negative index is an empty slot
      const int e = topk_idx[t * K + lane];
      if (e >= n_glu + n_pos) my_w = -my_w;
      if (e < 0) my_w = 0.f;
    }
  }
  const uint4* src[K];
  float ws[K];
#pragma unroll
  for (int j = 0; j < K; ++j) {
    const int r = __shfl_sync(0xffffffffu, my_row, j);
    ws[j] = __shfl_sync(0xffffffffu, my_w, j);
    src[j] = reinterpret_cast<const uint4*>(r >= 0 ? y + (int64_t)r * hidden : x + t * hidden);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + t * hidden);
  // optional second term (the shared expert's output): out = T(T(sum) + addend), the reference's two roundings
  const uint4* add = addend ? reinterpret_cast<const uint4*>(addend + t * hidden) : nullptr;
  const int chunks = hidden / VN;
  int c = lane;
  for (; c + 32 < chunks; c += 64) {
    uint4 v0[K], v1[K];
#pragma unroll
    for (int j = 0; j < K; ++j) { v0[j] = __ldcs(src[j] + c); v1[j] = __ldcs(src[j] + c + 32); }
    float a0[VN], a1[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) a0[i] = a1[i] = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) { Acc16<T>::fma(v0[j], ws[j], a0); Acc16<T>::fma(v1[j], ws[j], a1); }
    if (add != nullptr) { add_rounded<T>(a0, __ldcs(add + c)); add_rounded<T>(a1, __ldcs(add + c + 32)); }
    Vec16<T>::store(dst + c, a0);
    Vec16<T>::store(dst + c + 32, a1);
  }
  for (; c < chunks; c += 32) {
    uint4 v0[K];
#pragma unroll
    for (int j = 0; j < K; ++j) v0[j] = __ldcs(src[j] + c);
    float a0[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) a0[i] = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) Acc16<T>::fma(v0[j], ws[j], a0);
    if (add != nullptr) add_rounded<T>(a0, __ldcs(add + c));
    Vec16<T>::store(dst + c, a0);
  }
}

template <typename T>
static int combine_launch(const void* y, const void* x, const int32_t* slot_row, const int32_t* topk_idx,
                          const float* topk_w, int64_t n_tokens, int hidden, int top_k, int n_glu, int n_pos,
                          void* out, const void* addend, cudaStream_t st) {
  dim3 grid((unsigned)((n_tokens + PW - 1) / PW));
#define BIBO_COMBINE_CASE(KK)                                                                                   \
  case KK:                                                                                                       \
    combine_kernel<T, KK><<<grid, PW * 32, 0, st>>>((const T*)y, (const T*)x, slot_row, topk_idx, topk_w,        \
                                                    n_tokens, hidden, n_glu, n_pos, (T*)out, (const T*)addend);  \
    break;
  switch (top_k) {
    BIBO_COMBINE_CASE(1) BIBO_COMBINE_CASE(2) BIBO_COMBINE_CASE(3) BIBO_COMBINE_CASE(4)
    BIBO_COMBINE_CASE(5) BIBO_COMBINE_CASE(6) BIBO_COMBINE_CASE(7) BIBO_COMBINE_CASE(8)
    default: return fail(BIBO_ERR_UNSUPPORTED, "combine_fwd: top_k=%d", top_k);
  }
#undef BIBO_COMBINE_CASE
  BIBO_CHECK_LAUNCH("combine_kernel");
  return BIBO_OK;
}

}  // namespace bibo

using namespace bibo;

extern "C" int bibo_moe_permute_fwd(const void* x, const int32_t* topk_idx, const int32_t* slot_rank,
                                    const int32_t* plan, int64_t n_tokens, int hidden, int n_experts,
                                    int n_glu, int top_k, int dtype, int zero_padding, void* xp,
                                    int32_t* slot_row, int32_t* row_token, void* stream) {
  if (n_tokens <= 0) return BIBO_OK;
  if (!x || !topk_idx || !slot_rank || !plan || !xp || !slot_row || !row_token)
    return fail(BIBO_ERR_ARG, "permute_fwd: null pointer");
  if (dtype != BIBO_F32 && dtype != BIBO_BF16) return fail(BIBO_ERR_ARG, "permute_fwd: dtype=%d", dtype);
  if (top_k < 1 || top_k > BIBO_MAX_TOP_K) return fail(BIBO_ERR_UNSUPPORTED, "permute_fwd: top_k=%d", top_k);
  const int row_bytes = hidden * (dtype == BIBO_F32 ? 4 : 2);
  if (row_bytes % 16 != 0)
    return fail(BIBO_ERR_UNSUPPORTED, "permute_fwd: row of %d bytes is not a multiple of 16", row_bytes);
  if (!aligned16(x) || !aligned16(xp)) return fail(BIBO_ERR_ALIGN, "permute_fwd: x / xp not 16-byte aligned");
  const int64_t warps = n_tokens + (int64_t)n_glu * (BIBO_TILE_M - 1);
  dim3 grid((unsigned)((warps + PW - 1) / PW));
  permute_kernel<16><<<grid, PW * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)x, topk_idx, slot_rank, plan, n_tokens, row_bytes, n_experts, n_glu, top_k,
      zero_padding, (uint8_t*)xp, slot_row, row_token);
  BIBO_CHECK_LAUNCH("permute_kernel");
  return BIBO_OK;
}

extern "C" int bibo_moe_rowmap_fwd(const int32_t* topk_idx, const int32_t* slot_rank, const int32_t* plan,
                                   int64_t n_tokens, int n_experts, int n_glu, int top_k, int32_t* slot_row,
                                   int32_t* row_token, void* stream) {
  if (n_tokens <= 0) return BIBO_OK;
  if (!topk_idx || !slot_rank || !plan || !slot_row || !row_token) return fail(BIBO_ERR_ARG, "rowmap_fwd: null pointer");
  if (top_k < 1 || top_k > BIBO_MAX_TOP_K || n_experts < 1 || n_experts > BIBO_MAX_EXPERTS || n_glu < 0 ||
      n_glu > n_experts)
    return fail(BIBO_ERR_UNSUPPORTED, "rowmap_fwd: n_experts=%d n_glu=%d top_k=%d", n_experts, n_glu, top_k);
  const int64_t threads = n_tokens * top_k + (int64_t)n_glu * (BIBO_TILE_M - 1);
  rowmap_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      topk_idx, slot_rank, plan, n_tokens, n_experts, n_glu, top_k, slot_row, row_token);
  BIBO_CHECK_LAUNCH("rowmap_kernel");
  return BIBO_OK;
}

extern "C" int bibo_moe_permute_norm_fwd(const void* h, const float* rstd, const void* norm_weight,
                                         const int32_t* topk_idx, const int32_t* slot_rank, const int32_t* plan,
                                         int64_t n_tokens, int hidden, int n_experts, int n_glu, int top_k,
                                         int zero_padding, void* xp, int32_t* slot_row, int32_t* row_token,
                                         void* xn, void* stream) {
  if (n_tokens <= 0) return BIBO_OK;
  if (!h || !rstd || !norm_weight || !topk_idx || !slot_rank || !plan || !xp || !slot_row || !row_token)
    return fail(BIBO_ERR_ARG, "permute_norm_fwd: null pointer");
  if (n_glu < n_experts && (!xn || !aligned16(xn)))
    return fail(BIBO_ERR_ARG, "permute_norm_fwd: identity experts need the xn buffer (16-byte aligned)");
  if (top_k < 1 || top_k > BIBO_MAX_TOP_K) return fail(BIBO_ERR_UNSUPPORTED, "permute_norm_fwd: top_k=%d", top_k);
  const int row_bytes = hidden * 2;
  if (row_bytes % 16 != 0)
    return fail(BIBO_ERR_UNSUPPORTED, "permute_norm_fwd: row of %d bytes is not a multiple of 16", row_bytes);
  if (!aligned16(h) || !aligned16(xp) || !aligned16(norm_weight))
    return fail(BIBO_ERR_ALIGN, "permute_norm_fwd: h / xp / norm_weight not 16-byte aligned");
  const int64_t warps = n_tokens + (int64_t)n_glu * (BIBO_TILE_M - 1);
  dim3 grid((unsigned)((warps + PW - 1) / PW));
  permute_kernel<16><<<grid, PW * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)h, topk_idx, slot_rank, plan, n_tokens, row_bytes, n_experts, n_glu, top_k, zero_padding,
      (uint8_t*)xp, slot_row, row_token, rstd, (const uint8_t*)norm_weight, n_glu < n_experts ? (uint8_t*)xn : nullptr);
  BIBO_CHECK_LAUNCH("permute_kernel");
  return BIBO_OK;
}

extern "C" int bibo_moe_combine_add_fwd(const void* y, const void* x, const int32_t* slot_row,
                                        const int32_t* topk_idx, const float* topk_w, const void* addend,
                                        int64_t n_tokens, int hidden, int top_k, int n_glu, int n_pos, int dtype,
                                        void* out, void* stream) {
  if (n_tokens <= 0) return BIBO_OK;
  if (!y || !x || !slot_row || !topk_idx || !topk_w || !out)
    return fail(BIBO_ERR_ARG, "combine_fwd: null pointer");
  if (dtype != BIBO_F32 && dtype != BIBO_BF16) return fail(BIBO_ERR_ARG, "combine_fwd: dtype=%d", dtype);
  if (top_k < 1 || top_k > BIBO_MAX_TOP_K) return fail(BIBO_ERR_UNSUPPORTED, "combine_fwd: top_k=%d", top_k);
  const int row_bytes = hidden * (dtype == BIBO_F32 ? 4 : 2);
  if (row_bytes % 16 != 0)
    return fail(BIBO_ERR_UNSUPPORTED, "combine_fwd: row of %d bytes is not a multiple of 16", row_bytes);
  if (!aligned16(y) || !aligned16(x) || !aligned16(out) || !aligned16(addend))
    return fail(BIBO_ERR_ALIGN, "combine_fwd: y / x / out / addend not 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == BIBO_F32)
    return combine_launch<float>(y, x, slot_row, topk_idx, topk_w, n_tokens, hidden, top_k, n_glu, n_pos, out, addend, st);
  return combine_launch<__nv_bfloat16>(y, x, slot_row, topk_idx, topk_w, n_tokens, hidden, top_k, n_glu, n_pos, out,
                                       addend, st);
}

extern "C" int bibo_moe_combine_fwd(const void* y, const void* x, const int32_t* slot_row,
                                    const int32_t* topk_idx, const float* topk_w, int64_t n_tokens,
                                    int hidden, int top_k, int n_glu, int n_pos, int dtype, void* out,
                                    void* stream) {
  return bibo_moe_combine_add_fwd(y, x, slot_row, topk_idx, topk_w, nullptr, n_tokens, hidden, top_k, n_glu, n_pos,
                                  dtype, out, stream);
}
