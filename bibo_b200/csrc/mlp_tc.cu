// Dense SwiGLU MLP on the tensor-core kernels of the MoE block (bf16):
//   y = (silu(x Wg^T) * (x Wu^T)) Wd^T                  (src/modeling/ffn/mlp.py:33-34)
// used for the shared expert of the MoE layer and for dense feed-forward layers.
//
// The batch is one "expert" that owns every row: a small kernel writes the tile / tile-pair lists for
// ceil(N/128) row tiles, x itself is the A operand (rows beyond N read as zeros through the tensor
// map), and the down projection is the grouped down kernel with a single weight matrix.  The gate/up
// kernel is the CTA-pair kernel of the experts (256-row tcgen05.mma.cta_group::2, gate pass then up
// pass into 2 x 256 TMEM columns, bf16 gate stashed in swizzled shared memory) with three differences:
// gate and up weights are two tensors, the activation needs no row statistics (so the column blocks
// of a row pair are independent work items), and there is nothing to keep for a backward pass.
#include <algorithm>

#include "tc_common.cuh"

namespace bibo {
// gemm_simt.cu
int gemm_simt_launch(const void* A, const void* B, void* C, const PlanView& pv, int k_dim, int n_out, int dtype,
                     cudaStream_t st, int ldc, int64_t row_limit);
int swiglu_rows_launch(const void* gate_up, int64_t n_rows, int inter, int dtype, void* h, cudaStream_t st);
// gemm_tc.cu
int gemm2_tc_supported(int hidden, int inter, int dtype);
int gemm2_tc_launch(const void* h, const void* down_proj, const PlanView& pv, int hidden, int inter,
                    int n_weight_experts, void* y, cudaStream_t st);
int gemm2_tc_residual_launch(const void* h, const void* down_proj, const PlanView& pv, int hidden, int inter,
                             int n_weight_experts, void* y, const void* residual, cudaStream_t st);

namespace tc {

constexpr int M_NC = 256, M_STAGES = 5;
constexpr int M_EG = 2;                                  // epilogue groups of four warps; group e drains 64-column
constexpr int M_THREADS = 64 + EPI_THREADS * M_EG;       // sub-blocks 2e and 2e+1 of both accumulators
constexpr int M_BH_BYTES = (M_NC / 2) * BK * 2;
constexpr int M_OFF_A = 0;
constexpr int M_OFF_B = M_OFF_A + M_STAGES * A_BYTES;
constexpr int M_OFF_STASH = M_OFF_B + M_STAGES * M_BH_BYTES;
constexpr int M_OFF_BAR = M_OFF_STASH + (M_NC / 64) * C_SUB;
constexpr int M_SMEM = M_OFF_BAR + 256 + 1024;

// plan words of the dense layout: header[4], tiles int4[n_tiles], pairs int2[(n_tiles+1)/2]
__host__ __device__ inline int64_t mlp_tiles(int64_t n) { return (n + BM - 1) / BM; }
__host__ __device__ inline int64_t mlp_off_tiles() { return 4; }
__host__ __device__ inline int64_t mlp_off_pairs(int64_t n) { return 4 + 4 * mlp_tiles(n); }
__host__ __device__ inline int64_t mlp_plan_words(int64_t n) { return mlp_off_pairs(n) + 2 * ((mlp_tiles(n) + 1) / 2) + 4; }

__global__ void mlp_plan_kernel(int64_t n_tokens, int32_t* __restrict__ plan) {
  const int n_tiles = (int)mlp_tiles(n_tokens);
  int4* tiles = reinterpret_cast<int4*>(plan + mlp_off_tiles());
  int2* pairs = reinterpret_cast<int2*>(plan + mlp_off_pairs(n_tokens));
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) {
    plan[PLAN_N_TILES] = n_tiles;
    plan[PLAN_ROWS_USED] = n_tiles * BM;
    plan[PLAN_N_PAIRS] = (n_tiles + 1) / 2;
    // one-"expert" row range for the weight-gradient reductions of the backward: counts[0], expert_off[0..1]
    int32_t* range = plan + mlp_off_pairs(n_tokens) + 2 * ((n_tiles + 1) / 2);
    range[0] = (int32_t)n_tokens; range[1] = 0; range[2] = n_tiles * BM;
  }
  if (i < n_tiles) {
    tiles[i] = make_int4(0, i * BM, (int)min((int64_t)BM, n_tokens - (int64_t)i * BM), 0);
    if ((i & 1) == 0) pairs[i / 2] = make_int2(i, i + 1 < n_tiles ? i + 1 : -1);
  }
}

// Work item w = pair * n_cblocks + column block.  Cluster of two CTAs = one MMA pair.
__global__ void __launch_bounds__(M_THREADS, 1)
mlp_gemm1_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmG,
                      const __grid_constant__ CUtensorMap tmU, const __grid_constant__ CUtensorMap tmH,
                      int32_t* __restrict__ plan, int64_t tiles_off, int64_t pairs_off, int k_blocks, int n_cblocks,
                      __nv_bfloat16* __restrict__ gate_up_out, int64_t n_rows) {
  constexpr int NC = M_NC, STAGES = M_STAGES;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + M_OFF_BAR);   // used in the pair leader only
  uint64_t* empty = full + STAGES;
  uint64_t* gfull = empty + STAGES;
  uint64_t* gempty = gfull + 1;       // pair leader: 8 arrivals (4 epilogue warps of each CTA)
  uint64_t* ufull = gempty + 1;
  uint64_t* uempty = ufull + 1;       // pair leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(uempty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t pr = cluster_ctarank() & 1u;
  constexpr uint32_t leader = 0;
  constexpr uint16_t pair_mask = 3;
  const int cluster_id = blockIdx.x / 2, n_clusters = gridDim.x / 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(gfull, 1); mbar_init(ufull, 1);
    mbar_init(gempty, 8 * M_EG); mbar_init(uempty, 8 * M_EG);   // 4 warps x groups x 2 CTAs
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmG); prefetch_tmap(&tmU); prefetch_tmap(&tmH);
  }
  if (warp == 1) { tmem_alloc_cg2(tmem_slot, 2 * NC); tmem_relinquish_cg2(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int n_work = plan[PLAN_N_PAIRS] * n_cblocks;
  const int4* tiles = reinterpret_cast<const int4*>(plan + tiles_off);
  const int2* pairs = reinterpret_cast<const int2*>(plan + pairs_off);

  if (warp == 0) {
    if (elect_one()) {
      PipeState ps;
      bool ok = true;
      for (int w = cluster_id; w < n_work && ok; w += n_clusters) {
        const int2 pp = pairs[w / n_cblocks];
        const int cb = w % n_cblocks;
        const int4 t = tiles[(pr == 1 && pp.y >= 0) ? pp.y : pp.x];
        const int brow = cb * NC + (int)pr * (NC / 2);
        for (int pass = 0; pass < 2 && ok; ++pass) {
          for (int kb = 0; kb < k_blocks; ++kb) {
            ok = mbar_wait(&empty[ps.stage], ps.phase ^ 1, abort_flag);
            if (!ok) break;
            if (pr == 0) mbar_expect_tx(&full[ps.stage], 2 * (A_BYTES + M_BH_BYTES));
            const uint32_t bar0 = map_to_cta(&full[ps.stage], leader);
            tma_load_2d_cg2(smem + M_OFF_A + ps.stage * A_BYTES, &tmA, bar0, kb * BK, t.y);
            tma_load_2d_cg2(smem + M_OFF_B + ps.stage * M_BH_BYTES, pass == 0 ? &tmG : &tmU, bar0, kb * BK, brow);
            ps.next<STAGES>();
          }
        }
      }
    }
  } else if (warp == 1) {
    if (pr == 0 && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, NC);
      PipeState ps;
      uint32_t it = 0;
      bool ok = true;
      for (int w = cluster_id; w < n_work && ok; w += n_clusters, ++it) {
        for (int pass = 0; pass < 2 && ok; ++pass) {
          ok = mbar_wait<true>(pass == 0 ? gempty : uempty, (it & 1) ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          for (int kb = 0; kb < k_blocks; ++kb) {
            ok = mbar_wait<true>(&full[ps.stage], ps.phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint64_t da = make_sdesc_k128(smem_u32(smem + M_OFF_A + ps.stage * A_BYTES));
            const uint64_t db = make_sdesc_k128(smem_u32(smem + M_OFF_B + ps.stage * M_BH_BYTES));
#pragma unroll
            for (int k = 0; k < BK / UK; ++k)
              umma_bf16_cg2(tmem_base + pass * NC, da + k * 2, db + k * 2, idesc, (kb | k) != 0);
            umma_commit_cg2_mc(&empty[ps.stage], pair_mask);
            ps.next<STAGES>();
          }
          if (ok) umma_commit_cg2_mc(pass == 0 ? gfull : ufull, pair_mask);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int eg = (warp - 2) >> 2;                         // epilogue group
    constexpr int SUBS = (M_NC / 64) / M_EG;               // sub-blocks per group
    const int c_lo = eg * SUBS, c_hi = c_lo + SUBS;
    const bool issuer = (threadIdx.x == 64 + eg * EPI_THREADS);
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    unsigned char* stash = smem + M_OFF_STASH;
    uint32_t it = 0;
    for (int w = cluster_id; w < n_work; w += n_clusters, ++it) {
      const int2 pp = pairs[w / n_cblocks];
      const int cb = w % n_cblocks;
      const bool twin = (pr == 1 && pp.y < 0);     // duplicate of the leader's tile: compute, write nothing
      const int4 t = tiles[(pr == 1 && pp.y >= 0) ? pp.y : pp.x];
      if (issuer) tma_store_wait_read();           // this group's previous stores are done with its sub-blocks
      named_bar_sync(1 + eg, EPI_THREADS);
      if (!mbar_wait(gfull, it & 1, abort_flag)) break;
      tc_fence_after();
#pragma unroll 1
      for (int c = c_lo; c < c_hi; ++c) {          // gate -> bf16 -> stash
        uint32_t r0[32], r1[32];
        tmem_ld32(lane_addr + c * 64, r0);
        tmem_ld32(lane_addr + c * 64 + 32, r1);
        tmem_ld_wait();
        unsigned char* sub = stash + c * C_SUB;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const uint32_t* r = hh ? r1 : r0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
            v.y = pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            v.z = pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            v.w = pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            *reinterpret_cast<uint4*>(sub + swz(row, hh * 4 + j)) = v;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_addr(map_to_cta(gempty, leader));
      if (!mbar_wait(ufull, it & 1, abort_flag)) break;
      tc_fence_after();
      // training: the raw gate | up rows [N, 2I] are kept for the backward pass
      const int inter = n_cblocks * NC;
      __nv_bfloat16* gu_row = (gate_up_out && !twin && t.y + row < n_rows)
                                  ? gate_up_out + (int64_t)(t.y + row) * 2 * inter + cb * NC : nullptr;
#pragma unroll 1
      for (int c2 = c_lo; c2 < c_hi; ++c2) {       // h = bf16(silu(gate)) * bf16(up), in place in the stash
        uint32_t rr0[32], rr1[32];
        tmem_ld32(lane_addr + NC + c2 * 64, rr0);
        tmem_ld32(lane_addr + NC + c2 * 64 + 32, rr1);
        tmem_ld_wait();
        unsigned char* sub = stash + c2 * C_SUB;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int j = jj & 3;
          const uint32_t* r = (jj >> 2) ? rr1 : rr0;
          uint4* slot = reinterpret_cast<uint4*>(sub + swz(row, jj));
          const uint4 gv = *slot;
          const uint32_t* pg = reinterpret_cast<const uint32_t*>(&gv);
          uint4 hv, uv;
          uint32_t* ph = reinterpret_cast<uint32_t*>(&hv);
          uint32_t* pu = reinterpret_cast<uint32_t*>(&uv);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t upk = pack_bf16(__uint_as_float(r[8 * j + 2 * i]), __uint_as_float(r[8 * j + 2 * i + 1]));
            pu[i] = upk;
            float hval[2];
#pragma unroll
            for (int s = 0; s < 2; ++s) {
              const float g = s ? bf16_hi(pg[i]) : bf16_lo(pg[i]);
              const float u = s ? bf16_hi(upk) : bf16_lo(upk);
              // z * sigmoid(z) = zh + zh * tanh(zh), zh = z / 2  (one special-function op per element)
              const float zh = 0.5f * g;
              float th;
              asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(zh));
              hval[s] = round_bf16(fmaf(zh, th, zh)) * u;
            }
            ph[i] = pack_bf16(hval[0], hval[1]);
          }
          *slot = hv;
          if (gu_row != nullptr) {
            const int col = c2 * 64 + (jj >> 2) * 32 + j * 8;
            *reinterpret_cast<uint4*>(gu_row + col) = gv;
            *reinterpret_cast<uint4*>(gu_row + inter + col) = uv;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_addr(map_to_cta(uempty, leader));
      fence_proxy_async_smem();
      named_bar_sync(1 + eg, EPI_THREADS);
      if (issuer && !twin) {
        for (int s = c_lo; s < c_hi; ++s) tma_store_2d(&tmH, stash + s * C_SUB, cb * NC + s * 64, t.y);
        tma_store_commit();
      }
    }
    if (issuer) tma_store_wait_all();
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // nobody leaves while the pair peer may still signal or read this CTA
  if (warp == 1) { tc_fence_after(); tmem_dealloc_cg2(tmem_base, 2 * NC); }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&plan[PLAN_STATUS], 106);
}

}  // namespace tc
}  // namespace bibo

using namespace bibo;
using namespace bibo::tc;

extern "C" int64_t bibo_moe_mlp_plan_words(int64_t n_tokens) { return n_tokens > 0 ? mlp_plan_words(n_tokens) : 8; }

extern "C" int bibo_moe_mlp_supported(int hidden, int inter, int dtype) {
  return dtype == BIBO_BF16 && hidden % 256 == 0 && inter % M_NC == 0 && inter >= M_NC;
}

extern "C" int bibo_moe_mlp_forward(const void* x, const void* gate_proj, const void* up_proj, const void* down_proj,
                                    int64_t n_tokens, int hidden, int inter, int dtype, int32_t* plan, void* h, void* y,
                                    void* gate_up_out, void* stream) {
  return bibo_moe_mlp_forward_residual(x, gate_proj, up_proj, down_proj, n_tokens, hidden, inter, dtype, plan, h, y,
                                       gate_up_out, nullptr, stream);
}

extern "C" int bibo_moe_mlp_forward_residual(const void* x, const void* gate_proj, const void* up_proj,
                                             const void* down_proj, int64_t n_tokens, int hidden, int inter, int dtype,
                                             int32_t* plan, void* h, void* y, void* gate_up_out, const void* residual,
                                             void* stream) {
  if (n_tokens <= 0) return BIBO_OK;
  if (residual && (!bibo_moe_mlp_supported(hidden, inter, dtype) || !aligned16(residual)))
    return fail(BIBO_ERR_UNSUPPORTED, "mlp_forward_residual: the residual add lives in the tensor-core down kernel "
                "(bf16 shapes of bibo_moe_mlp_supported, 16-byte aligned residual)");
  if (!x || !gate_proj || !up_proj || !down_proj || !plan || !h || !y)
    return fail(BIBO_ERR_ARG, "mlp_forward: null pointer");
  if (dtype != BIBO_F32 && dtype != BIBO_BF16) return fail(BIBO_ERR_ARG, "mlp_forward: dtype=%d", dtype);
  if (n_tokens > 0x7fffff00LL) return fail(BIBO_ERR_UNSUPPORTED, "mlp_forward: n_tokens=%lld", (long long)n_tokens);
  if (!bibo_moe_mlp_supported(hidden, inter, dtype)) {
    // float32 (the 1e-4 parity bar rules out tensor cores) and shapes outside the tensor-core kernels:
    // CUDA-core GEMMs into the gate | up buffer, an elementwise SwiGLU, a CUDA-core down GEMM
    if (!gate_up_out)
      return fail(BIBO_ERR_ARG, "mlp_forward: this dtype/shape runs the CUDA-core path and needs the gate_up buffer");
    cudaStream_t st0 = static_cast<cudaStream_t>(stream);
    const int nt = (int)mlp_tiles(n_tokens);
    BIBO_CUDA(cudaMemsetAsync(plan, 0, 4 * sizeof(int32_t), st0));
    mlp_plan_kernel<<<(nt + 255) / 256, 256, 0, st0>>>(n_tokens, plan);
    BIBO_CHECK_LAUNCH("mlp_plan_kernel");
    PlanView pv0 = {};
    pv0.plan = plan;
    pv0.tiles_off = mlp_off_tiles();
    pv0.pairs_off = mlp_off_pairs(n_tokens);
    pv0.tiles_cap = nt;
    pv0.rows_alloc = n_tokens;
    const size_t es = dtype == BIBO_F32 ? 4 : 2;
    int rc0;
    if ((rc0 = gemm_simt_launch(x, gate_proj, gate_up_out, pv0, hidden, inter, dtype, st0, 2 * inter, n_tokens))) return rc0;
    if ((rc0 = gemm_simt_launch(x, up_proj, static_cast<char*>(gate_up_out) + (size_t)inter * es, pv0, hidden, inter, dtype,
                                st0, 2 * inter, n_tokens)))
      return rc0;
    if ((rc0 = swiglu_rows_launch(gate_up_out, n_tokens, inter, dtype, h, st0))) return rc0;
    return gemm_simt_launch(h, down_proj, y, pv0, inter, hidden, dtype, st0, hidden, n_tokens);
  }
  if (!aligned16(x) || !aligned16(gate_proj) || !aligned16(up_proj) || !aligned16(down_proj) || !aligned16(h) ||
      !aligned16(y) || !aligned16(gate_up_out))
    return fail(BIBO_ERR_ALIGN, "mlp_forward: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n_tiles = (int)mlp_tiles(n_tokens);
  BIBO_CUDA(cudaMemsetAsync(plan, 0, 4 * sizeof(int32_t), st));
  mlp_plan_kernel<<<(n_tiles + 255) / 256, 256, 0, st>>>(n_tokens, plan);
  BIBO_CHECK_LAUNCH("mlp_plan_kernel");

  PlanView pv = {};
  pv.plan = plan;
  pv.tiles_off = mlp_off_tiles();
  pv.pairs_off = mlp_off_pairs(n_tokens);
  pv.tiles_cap = n_tiles;
  pv.rows_alloc = n_tokens;      // loads beyond the last row read zeros, stores beyond it are dropped
  pv.max_ctas = 0;

  CUtensorMap tmA, tmG, tmU, tmH;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tmA, x, (uint64_t)n_tokens, hidden, hidden, BM))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmG, gate_proj, (uint64_t)inter, hidden, hidden, 128))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmU, up_proj, (uint64_t)inter, hidden, hidden, 128))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmH, h, (uint64_t)n_tokens, inter, inter, BM))) return rc;
  static DeviceOnce once;
  int max_clusters = 0;
  const int sms = sm_count();
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(M_THREADS);
  cfg.dynamicSmemBytes = M_SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  rc = once.get([&](int* v) {
    BIBO_CUDA(cudaFuncSetAttribute(mlp_gemm1_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, M_SMEM));
    cfg.gridDim = dim3((sms / 2) * 2);
    int n = 0;
    BIBO_CUDA(cudaOccupancyMaxActiveClusters(&n, mlp_gemm1_pair_kernel, &cfg));
    *v = n > 0 ? n : 1;
    return (int)BIBO_OK;
  }, &max_clusters);
  if (rc) return rc;
  const int64_t n_work = (int64_t)((n_tiles + 1) / 2) * (inter / M_NC);
  const int clusters = (int)std::max<int64_t>(1, std::min<int64_t>(std::min(max_clusters, sms / 2), n_work));
  cfg.gridDim = dim3(clusters * 2);
  BIBO_CUDA(cudaLaunchKernelEx(&cfg, mlp_gemm1_pair_kernel, tmA, tmG, tmU, tmH, plan, pv.tiles_off, pv.pairs_off,
                               hidden / BK, inter / M_NC, static_cast<__nv_bfloat16*>(gate_up_out), n_tokens));
  launch_counter().fetch_add(1, std::memory_order_relaxed);
  if (residual) return gemm2_tc_residual_launch(h, down_proj, pv, hidden, inter, 1, y, residual, st);
  return gemm2_tc_launch(h, down_proj, pv, hidden, inter, 1, y, st);
}

// ---- backward -------------------------------------------------------------------------------------------
namespace bibo {
// gemm_bwd_tc.cu
int gemm_dx_tc_supported(int k_dim, int n_out);
int gemm_dx_tc_launch(const void* A, const void* W, void* C, const PlanView& pv, int k_dim, int n_out,
                      int n_weight_experts, cudaStream_t st);
int gemm_dw_tc_supported(int m_dim, int n_dim);
int gemm_dw_tc_launch(const void* A, const void* B, void* C, const int32_t* plan, int64_t counts_off,
                      int64_t expert_off_off, int64_t rows_alloc, int n_experts, int m_dim, int n_dim, cudaStream_t st);

// backward.cu: the same backward on CUDA cores
int mlp_backward_simt(const void* x, const void* w_gu, const void* down_proj, void* gate_up, const void* h,
                      const void* dout, int64_t n, int hidden, int inter, int dtype, const PlanView& pv,
                      const int32_t* counts, const int32_t* expert_off, void* dh, void* dx, void* d_w_gu, void* d_down,
                      cudaStream_t st);

// [gate | up] rows -> [dGate | dUp] in place: a = bf16(silu(g)), dUp = dh * a, dGate = dh * up * silu'(g).
// One warp per row, 16-byte accesses; the sigmoid is one tanh.approx (error below the bf16 resolution).
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dh, __nv_bfloat16* __restrict__ gate_up, int64_t n_rows, int inter) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  uint4* g = reinterpret_cast<uint4*>(gate_up + row * 2 * inter);
  uint4* u = g + inter / 8;
  const uint4* d = reinterpret_cast<const uint4*>(dh + row * inter);
  for (int c = lane; c < inter / 8; c += 32) {
    const uint4 gv = g[c], uv = u[c], dv = __ldcs(d + c);
    const uint32_t* pg = reinterpret_cast<const uint32_t*>(&gv);
    const uint32_t* pu = reinterpret_cast<const uint32_t*>(&uv);
    const uint32_t* pd = reinterpret_cast<const uint32_t*>(&dv);
    uint4 og, ou;
    uint32_t* qg = reinterpret_cast<uint32_t*>(&og);
    uint32_t* qu = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float dg2[2], du2[2];
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const float gg = s ? tc::bf16_hi(pg[i]) : tc::bf16_lo(pg[i]);
        const float uu = s ? tc::bf16_hi(pu[i]) : tc::bf16_lo(pu[i]);
        const float dd = s ? tc::bf16_hi(pd[i]) : tc::bf16_lo(pd[i]);
        float th;
        asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * gg));
        const float sg = fmaf(0.5f, th, 0.5f);
        du2[s] = dd * tc::round_bf16(gg * sg);
        dg2[s] = dd * uu * (sg * (1.0f + gg * (1.0f - sg)));
      }
      qg[i] = tc::pack_bf16(dg2[0], dg2[1]);
      qu[i] = tc::pack_bf16(du2[0], du2[1]);
    }
    g[c] = og;
    u[c] = ou;
  }
}
}  // namespace bibo

extern "C" int bibo_moe_mlp_backward(const void* x, const void* gate_up_weight, const void* down_proj, void* gate_up,
                                     const void* h, const void* dout, int64_t n_tokens, int hidden, int inter, int dtype,
                                     int32_t* plan, void* dh, void* dx, void* d_gate_up_weight, void* d_down_proj,
                                     void* stream) {
  if (n_tokens <= 0) return BIBO_OK;
  if (!x || !gate_up_weight || !down_proj || !gate_up || !h || !dout || !plan || !dh || !dx || !d_gate_up_weight ||
      !d_down_proj)
    return fail(BIBO_ERR_ARG, "mlp_backward: null pointer");
  if (dtype != BIBO_F32 && dtype != BIBO_BF16) return fail(BIBO_ERR_ARG, "mlp_backward: dtype=%d", dtype);
  const bool tensor_cores = bibo_moe_mlp_supported(hidden, inter, dtype) && gemm_dx_tc_supported(hidden, inter) &&
                            gemm_dx_tc_supported(2 * inter, hidden) && gemm_dw_tc_supported(hidden, inter) &&
                            gemm_dw_tc_supported(2 * inter, hidden);
  if (!tensor_cores) {   // float32 and other shapes: CUDA-core kernels, same order of operations
    const int64_t ex = mlp_off_pairs(n_tokens) + 2 * ((mlp_tiles(n_tokens) + 1) / 2);
    PlanView pv0 = {};
    pv0.plan = plan;
    pv0.tiles_off = mlp_off_tiles();
    pv0.pairs_off = mlp_off_pairs(n_tokens);
    pv0.tiles_cap = (int)mlp_tiles(n_tokens);
    pv0.rows_alloc = n_tokens;
    return mlp_backward_simt(x, gate_up_weight, down_proj, gate_up, h, dout, n_tokens, hidden, inter, dtype, pv0,
                             plan + ex, plan + ex + 1, dh, dx, d_gate_up_weight, d_down_proj,
                             static_cast<cudaStream_t>(stream));
  }
  if (!aligned16(x) || !aligned16(gate_up_weight) || !aligned16(down_proj) || !aligned16(gate_up) || !aligned16(h) ||
      !aligned16(dout) || !aligned16(dh) || !aligned16(dx) || !aligned16(d_gate_up_weight) || !aligned16(d_down_proj))
    return fail(BIBO_ERR_ALIGN, "mlp_backward: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n_tiles = (int)mlp_tiles(n_tokens);
  // the forward's plan (tiles, pairs) plus a one-expert row range for the weight-gradient reductions; rows past N
  // read as zeros through the tensor maps, so the padded range needs no zero-filled buffers
  const int64_t extra = mlp_off_pairs(n_tokens) + 2 * ((mlp_tiles(n_tokens) + 1) / 2);
  // (written by the forward's plan kernel: counts[0], expert_off[0..1])
  PlanView pv = {};
  pv.plan = plan;
  pv.tiles_off = mlp_off_tiles();
  pv.pairs_off = mlp_off_pairs(n_tokens);
  pv.tiles_cap = n_tiles;
  pv.rows_alloc = n_tokens;
  int rc;
  // dH = dOut W_d ; dW_d = dOut^T h
  if ((rc = gemm_dx_tc_launch(dout, down_proj, dh, pv, hidden, inter, 1, st))) return rc;
  if ((rc = gemm_dw_tc_launch(dout, h, d_down_proj, plan, extra, extra + 1, n_tokens, 1, hidden, inter, st))) return rc;
  swiglu_bwd_kernel<<<(unsigned)((n_tokens + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dh),
                                                                   static_cast<__nv_bfloat16*>(gate_up), n_tokens, inter);
  BIBO_CHECK_LAUNCH("swiglu_bwd_kernel");
  // dX = [dGate | dUp] [W_g ; W_u] ; d[W_g ; W_u] = [dGate | dUp]^T x
  if ((rc = gemm_dx_tc_launch(gate_up, gate_up_weight, dx, pv, 2 * inter, hidden, 1, st))) return rc;
  return gemm_dw_tc_launch(gate_up, x, d_gate_up_weight, plan, extra, extra + 1, n_tokens, 1, 2 * inter, hidden, st);
}
