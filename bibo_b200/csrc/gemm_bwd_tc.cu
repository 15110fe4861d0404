// Backward GEMMs on the tensor cores (bf16, fp32 accumulation in tensor memory).
//
//   MODE_DX  C[row, n] = sum_k A[row, k] * B[e][k][n]      dH = dY @ down_proj[e],  dXp = dGU @ gate_up_proj[e]
//            A is K-major (rows of the expert-contiguous buffer), B is the weight as stored, i.e. with
//            the OUTPUT dimension contiguous ("MN-major" operand).
//   MODE_DW  C[e][m, n] = sum_{r in rows of e} A[r, m] * B[r, n]   dW_d[e] = dY_e^T h_e,  dW_gu[e] = dGU_e^T xp_e
//            the reduction runs over the expert's rows, so BOTH operands are MN-major.
//
// An MN-major operand tile is staged as boxes of [64 k-rows x 64 elements (128 bytes)] written by TMA
// with the 128-byte swizzle: inside a box the 8-row swizzle atoms are 1024 bytes apart (stride byte
// offset), boxes along the M/N dimension are 8192 bytes apart (leading byte offset), and one
// tcgen05.mma k-step (16 rows) advances the start address by 2048 bytes.
// MODE_DW relies on zero rows in the padding of every expert block (the reduction includes them).
// Same warp roles, pipeline and bounded waits as the forward kernels (gemm_tc.cu).
#include <algorithm>

#include "tc_common.cuh"

namespace bibo {
namespace tc {

constexpr int MODE_DX = 0, MODE_DW = 1;
constexpr int XBN = 256, XSTAGES = 4;
constexpr int XB_BYTES = XBN * BK * 2;
constexpr int MN_BOX = 64 * BK * 2;   // one [64 k-rows x 128 B] box

struct XLayout {
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + XSTAGES * A_BYTES;
  static constexpr int OFF_C = OFF_B + XSTAGES * XB_BYTES;
  static constexpr int OFF_BAR = OFF_C + 2 * C_SUB;
  static constexpr int BYTES = OFF_BAR + 256 + 1024;
};

__device__ __forceinline__ uint64_t make_sdesc_mn128(uint32_t smem_addr) {
  uint64_t d = (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(MN_BOX >> 4) << 16;   // leading byte offset: next 64 elements along M/N
  d |= (uint64_t)(1024 >> 4) << 32;     // stride byte offset: next 8 k-rows
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

struct BwdWork {
  int e, row0, m0, n0, k_blocks, krow0;
  bool valid;
};

// work item w -> coordinates (identical in every warp role)
template <int MODE>
__device__ __forceinline__ BwdWork decode_work(int w, const int32_t* plan, const int4* tiles,
                                               const int32_t* counts, const int32_t* expert_off, int n_chunks,
                                               int m_tiles, int k_blocks_dx) {
  BwdWork o;
  if (MODE == MODE_DX) {
    const int4 t = tiles[w / n_chunks];
    o.e = t.x; o.row0 = t.y; o.m0 = t.y; o.n0 = (w % n_chunks) * XBN; o.k_blocks = k_blocks_dx; o.krow0 = 0;
    o.valid = true;
  } else {
    const int per = m_tiles * n_chunks;
    o.e = w / per;
    const int rem = w % per;
    o.m0 = (rem / n_chunks) * BM; o.n0 = (rem % n_chunks) * XBN;
    o.krow0 = expert_off[o.e]; o.row0 = 0;
    o.k_blocks = (expert_off[o.e + 1] - expert_off[o.e]) / BK;
    o.valid = true;          // an expert without rows has k_blocks == 0: its gradient tile is written as zeros
  }
  return o;
}

// MODE_DX: tmA = A [rows, K] (box 128 rows), tmB = weights viewed [E*K, N] (box 64 x 64), tmC = C [rows, N].
// MODE_DW: tmA = A [rows, M] (box 64 x 64), tmB = B [rows, N] (box 64 x 64), tmC = C viewed [E*M, N].
template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bwd_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmC, int32_t* __restrict__ plan, int64_t tiles_off,
                   int64_t counts_off, int64_t expert_off_off, int n_experts, int n_chunks, int m_tiles,
                   int k_dim, int m_dim) {
  using L = XLayout;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* empty = full + XSTAGES;
  uint64_t* tfull = empty + XSTAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < XSTAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 4); }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB); prefetch_tmap(&tmC);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 2 * XBN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int4* tiles = reinterpret_cast<const int4*>(plan + tiles_off);
  const int32_t* counts = plan + counts_off;
  const int32_t* expert_off = plan + expert_off_off;
  const int n_work = (MODE == MODE_DX) ? plan[PLAN_N_TILES] * n_chunks : n_experts * m_tiles * n_chunks;
  const int k_blocks_dx = k_dim / BK;

  if (warp == 0) {
    if (elect_one()) {
      PipeState ps;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const BwdWork wk = decode_work<MODE>(w, plan, tiles, counts, expert_off, n_chunks, m_tiles, k_blocks_dx);
        if (!wk.valid) continue;
        for (int kb = 0; kb < wk.k_blocks; ++kb) {
          ok = mbar_wait(&empty[ps.stage], ps.phase ^ 1, abort_flag);
          if (!ok) break;
          mbar_expect_tx(&full[ps.stage], A_BYTES + XB_BYTES);
          unsigned char* sa = smem + L::OFF_A + ps.stage * A_BYTES;
          unsigned char* sb = smem + L::OFF_B + ps.stage * XB_BYTES;
          if (MODE == MODE_DX) {
            tma_load_2d(sa, &tmA, &full[ps.stage], kb * BK, wk.row0);
#pragma unroll
            for (int b = 0; b < XBN / 64; ++b)
              tma_load_2d(sb + b * MN_BOX, &tmB, &full[ps.stage], wk.n0 + b * 64, wk.e * k_dim + kb * BK);
          } else {
            const int kr = wk.krow0 + kb * BK;
#pragma unroll
            for (int a = 0; a < BM / 64; ++a) tma_load_2d(sa + a * MN_BOX, &tmA, &full[ps.stage], wk.m0 + a * 64, kr);
#pragma unroll
            for (int b = 0; b < XBN / 64; ++b) tma_load_2d(sb + b * MN_BOX, &tmB, &full[ps.stage], wk.n0 + b * 64, kr);
          }
          ps.next<XSTAGES>();
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      // bit 15: A is MN-major, bit 16: B is MN-major
      constexpr uint32_t idesc = make_idesc_bf16(BM, XBN) | (MODE == MODE_DW ? (1u << 15) : 0u) | (1u << 16);
      PipeState ps;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const BwdWork wk = decode_work<MODE>(w, plan, tiles, counts, expert_off, n_chunks, m_tiles, k_blocks_dx);
        if (!wk.valid) continue;
        ok = mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < wk.k_blocks; ++kb) {
          ok = mbar_wait(&full[ps.stage], ps.phase, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + L::OFF_A + ps.stage * A_BYTES);
          const uint32_t sb = smem_u32(smem + L::OFF_B + ps.stage * XB_BYTES);
          const uint64_t da = (MODE == MODE_DW) ? make_sdesc_mn128(sa) : make_sdesc_k128(sa);
          const uint64_t db = make_sdesc_mn128(sb);
          constexpr int a_step = (MODE == MODE_DW) ? (2048 >> 4) : (32 >> 4);
#pragma unroll
          for (int k = 0; k < BK / UK; ++k)
            umma_bf16(tmem_base + acc * XBN, da + k * a_step, db + k * (2048 >> 4), idesc, (kb | k) != 0);
          umma_commit(&empty[ps.stage]);
          ps.next<XSTAGES>();
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool issuer = (threadIdx.x == 64);
    int acc = 0, buf = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
      const BwdWork wk = decode_work<MODE>(w, plan, tiles, counts, expert_off, n_chunks, m_tiles, k_blocks_dx);
      if (!wk.valid) continue;
      const int crow = (MODE == MODE_DX) ? wk.row0 : wk.e * m_dim + wk.m0;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
#pragma unroll 1
      for (int g = 0; g < XBN / 64; ++g) {
        uint32_t r0[32], r1[32];
        const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + acc * XBN + g * 64;
        tmem_ld32(ta, r0);
        tmem_ld32(ta + 32, r1);
        tmem_ld_wait();
        if (wk.k_blocks == 0) {   // nothing was accumulated: the buffer holds stale values
#pragma unroll
          for (int i = 0; i < 32; ++i) r0[i] = r1[i] = 0u;
        }
        if (g == XBN / 64 - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[acc]);
        }
        if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        named_bar_sync(1, EPI_THREADS);
        unsigned char* cbuf = smem + L::OFF_C + buf * C_SUB;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
          v.y = pack_bf16(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
          v.z = pack_bf16(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
          v.w = pack_bf16(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
          *reinterpret_cast<uint4*>(cbuf + swz(row, j)) = v;
          v.x = pack_bf16(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
          v.y = pack_bf16(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
          v.z = pack_bf16(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
          v.w = pack_bf16(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
          *reinterpret_cast<uint4*>(cbuf + swz(row, 4 + j)) = v;
        }
        fence_proxy_async_smem();
        named_bar_sync(1, EPI_THREADS);
        if (issuer) {
          tma_store_2d(&tmC, cbuf, wk.n0 + g * 64, crow);
          tma_store_commit();
        }
        buf ^= 1;
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (issuer) tma_store_wait_all();
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 2 * XBN); }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&plan[PLAN_STATUS], 110 + MODE);
}

template <int MODE>
static int bwd_launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const int32_t* plan,
                      int64_t tiles_off, int64_t counts_off, int64_t expert_off_off, int n_experts, int n_chunks,
                      int m_tiles, int k_dim, int m_dim, int64_t work_cap, cudaStream_t st) {
  auto kern = gemm_bwd_tc_kernel<MODE>;
  static DeviceOnce once;
  const int rc = once.get([&](int*) {
    BIBO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, XLayout::BYTES));
    return (int)BIBO_OK;
  });
  if (rc) return rc;
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(sm_count(), work_cap));
  kern<<<grid, NUM_THREADS, XLayout::BYTES, st>>>(tmA, tmB, tmC, const_cast<int32_t*>(plan), tiles_off, counts_off,
                                                  expert_off_off, n_experts, n_chunks, m_tiles, k_dim, m_dim);
  BIBO_CHECK_LAUNCH("gemm_bwd_tc_kernel");
  return BIBO_OK;
}

}  // namespace tc

using namespace tc;

// C[rows, n_out] = A[rows, k_dim] @ W[e][k_dim][n_out]   (W as stored: n_out contiguous)
int gemm_dx_tc_supported(int k_dim, int n_out) { return k_dim % BK == 0 && k_dim >= BK && n_out % XBN == 0; }
int gemm_dx_tc_launch(const void* A, const void* W, void* C, const PlanView& pv, int k_dim, int n_out,
                      int n_weight_experts, cudaStream_t st) {
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tmA, A, pv.rows_alloc, k_dim, k_dim, BM))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmB, W, (uint64_t)n_weight_experts * k_dim, n_out, n_out, 64))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmC, C, pv.rows_alloc, n_out, n_out, BM))) return rc;
  return bwd_launch<MODE_DX>(tmA, tmB, tmC, pv.plan, pv.tiles_off, 0, 0, 0, n_out / XBN, 0, k_dim, 0,
                             pv.tiles_cap * (n_out / XBN), st);
}

// C[e][m_dim, n_dim] = sum over the rows of expert e of A[r, m_dim]^T B[r, n_dim]; padding rows of A must be 0
// and those of B finite.  counts / expert_off live in `plan` at the given word offsets.
int gemm_dw_tc_supported(int m_dim, int n_dim) { return m_dim % BM == 0 && n_dim % XBN == 0; }
int gemm_dw_tc_launch(const void* A, const void* B, void* C, const int32_t* plan, int64_t counts_off,
                      int64_t expert_off_off, int64_t rows_alloc, int n_experts, int m_dim, int n_dim,
                      cudaStream_t st) {
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tmA, A, rows_alloc, m_dim, m_dim, 64))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmB, B, rows_alloc, n_dim, n_dim, 64))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmC, C, (uint64_t)n_experts * m_dim, n_dim, n_dim, BM))) return rc;
  const int m_tiles = m_dim / BM, n_chunks = n_dim / XBN;
  return bwd_launch<MODE_DW>(tmA, tmB, tmC, plan, 0, counts_off, expert_off_off, n_experts, n_chunks, m_tiles, 0,
                             m_dim, (int64_t)n_experts * m_tiles * n_chunks, st);
}

}  // namespace bibo
