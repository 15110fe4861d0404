// K3 / K4 on the 5th-generation tensor cores: grouped bf16 GEMMs over the plan's row tiles with
// TMA-fed shared-memory pipelines, tcgen05.mma accumulating in tensor memory, and warp-specialised
// persistent CTAs (warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-5 = epilogue).
//
//  gemm2_tc_kernel : y[rows, H]  = h[rows, I] x down_proj[e][H, I]^T
//  gemm1_tc_kernel : gate|up     = xp[rows, H] x gate_up_proj[e][2I, H]^T, then the Radial NormSiLU
//                    epilogue r = sqrt(mean g^2 + 1e-6), a = silu(g/r) r^p, h = a * up.  The row
//                    reduction spans all I gate columns: a CTA owns NC <= 256 of them (gate and up
//                    accumulators = 2*NC tensor-memory columns), so for I = 512 two CTAs of a
//                    cluster split the columns and exchange their partial sums of squares through
//                    distributed shared memory.
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "tc_common.cuh"

namespace bibo {
namespace tc {

// =====================================================================================================
// K4: down projection
// =====================================================================================================
template <int BN, int STAGES>
struct G2Layout {
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_C = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_BAR = OFF_C + 2 * C_SUB;
  static constexpr int BYTES = OFF_BAR + 256 + 1024;  // barriers + alignment slack
};

// RES: the epilogue adds residual[row][col] (same shape and pitch as y) to the rounded product,
// y = bf16(bf16(acc) + residual): the decoder layer's `hidden_states + mlp(...)` (src/modeling/layers.py:61-66)
// for the dense layers, without a pass of its own over the activations.
template <int BN, int STAGES, bool RES = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm2_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, int32_t* __restrict__ plan, int64_t tiles_off,
                int n_chunks, int k_blocks, int n_out, const __nv_bfloat16* __restrict__ residual = nullptr) {
  using L = G2Layout<BN, STAGES>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 4); }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB); prefetch_tmap(&tmC);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 2 * BN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int n_work = plan[PLAN_N_TILES] * n_chunks;
  const int4* tiles = reinterpret_cast<const int4*>(plan + tiles_off);

  if (warp == 0) {
    if (elect_one()) {
      PipeState ps;
      for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
        const int4 t = tiles[w / n_chunks];
        const int n0 = (w % n_chunks) * BN;
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
          ok = mbar_wait(&empty[ps.stage], ps.phase ^ 1, abort_flag);
          if (!ok) break;
          mbar_expect_tx(&full[ps.stage], A_BYTES + L::B_BYTES);
          tma_load_2d(smem + L::OFF_A + ps.stage * A_BYTES, &tmA, &full[ps.stage], kb * BK, t.y);
          tma_load_2d(smem + L::OFF_B + ps.stage * L::B_BYTES, &tmB, &full[ps.stage], kb * BK, t.x * n_out + n0);
          ps.next<STAGES>();
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
      PipeState ps;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) break;
        tc_fence_after();
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(&full[ps.stage], ps.phase, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint64_t da = make_sdesc_k128(smem_u32(smem + L::OFF_A + ps.stage * A_BYTES));
          const uint64_t db = make_sdesc_k128(smem_u32(smem + L::OFF_B + ps.stage * L::B_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UK; ++k)
            umma_bf16(tmem_base + acc * BN, da + k * 2, db + k * 2, idesc, (kb | k) != 0);
          umma_commit(&empty[ps.stage]);
          ps.next<STAGES>();
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int q = warp & 3;                     // TMEM lane quadrant this warp may read
    const int row = q * 32 + lane;
    const bool issuer = (threadIdx.x == 64);
    int acc = 0, buf = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
      const int4 t = tiles[w / n_chunks];
      const int n0 = (w % n_chunks) * BN;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
#pragma unroll 1
      for (int g = 0; g < BN / 64; ++g) {
        if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        named_bar_sync(1, EPI_THREADS);
        unsigned char* cbuf = smem + L::OFF_C + buf * C_SUB;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t r[32];
          uint4 res[4];
          if (RES) {   // issued before the accumulator is read, so the loads fly under the tensor-memory load
            const bool live = row < t.z;
            const uint4* rp = reinterpret_cast<const uint4*>(residual + (int64_t)(t.y + row) * n_out + n0 + g * 64 + hh * 32);
#pragma unroll
            for (int j = 0; j < 4; ++j) res[j] = live ? __ldg(rp + j) : make_uint4(0, 0, 0, 0);
          }
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + g * 64 + hh * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            if (RES) {
              const uint32_t* rv = reinterpret_cast<const uint32_t*>(&res[j]);
              uint32_t o[4];
#pragma unroll
              for (int i = 0; i < 4; ++i)
                o[i] = pack_bf16(round_bf16(__uint_as_float(r[8 * j + 2 * i])) + bf16_lo(rv[i]),
                                 round_bf16(__uint_as_float(r[8 * j + 2 * i + 1])) + bf16_hi(rv[i]));
              v = make_uint4(o[0], o[1], o[2], o[3]);
            } else {
              v.x = pack_bf16(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
              v.y = pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              v.z = pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              v.w = pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            }
            *reinterpret_cast<uint4*>(cbuf + swz(row, hh * 4 + j)) = v;
          }
        }
        if (g == BN / 64 - 1) {  // accumulator fully read: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[acc]);
        }
        fence_proxy_async_smem();
        named_bar_sync(1, EPI_THREADS);
        if (issuer) {
          tma_store_2d(&tmC, cbuf, n0 + g * 64, t.y);
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
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 2 * BN); }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&plan[PLAN_STATUS], 100);
}

// =====================================================================================================
// K3: gate/up projection + Radial NormSiLU
// =====================================================================================================
template <int NC, int STAGES>
struct G1Layout {
  static constexpr int B_BYTES = NC * BK * 2;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_STASH = OFF_B + STAGES * B_BYTES;        // [NC/64][128][128B] bf16 gate, then h
  static constexpr int OFF_PART = OFF_STASH + (NC / 64) * C_SUB;    // float [2][128] partial sums from the peer
  static constexpr int OFF_BAR = OFF_PART + 2 * BM * 4;
  static constexpr int BYTES = OFF_BAR + 256 + 1024;
};

template <int NC, int CL, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm1_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmH, const float* __restrict__ theta,
                int32_t* __restrict__ plan, int64_t tiles_off, int k_blocks, int inter,
                __nv_bfloat16* __restrict__ gate_up_out, float* __restrict__ rnorm_out) {
  using L = G1Layout<NC, STAGES>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  float* part = reinterpret_cast<float*>(smem + L::OFF_PART);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* empty = full + STAGES;
  uint64_t* gfull = empty + STAGES;   // gate accumulator complete
  uint64_t* gempty = gfull + 1;       // gate accumulator drained
  uint64_t* ufull = gempty + 1;
  uint64_t* uempty = ufull + 1;
  uint64_t* xbar = uempty + 1;        // [2] partial-sum exchange, arrivals come from the peer CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xbar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cr = (CL > 1) ? cluster_ctarank() : 0;   // column block of this CTA
  const int cluster_id = blockIdx.x / CL, n_clusters = gridDim.x / CL;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(gfull, 1); mbar_init(ufull, 1);
    mbar_init(gempty, 4); mbar_init(uempty, 4);
    mbar_init(&xbar[0], EPI_THREADS); mbar_init(&xbar[1], EPI_THREADS);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB); prefetch_tmap(&tmH);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 2 * NC); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  if (CL > 1) cluster_sync_all();   // peer barriers are initialised before anyone arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int n_tiles = plan[PLAN_N_TILES];
  const int4* tiles = reinterpret_cast<const int4*>(plan + tiles_off);

  if (warp == 0) {
    if (elect_one()) {
      PipeState ps;
      bool ok = true;
      for (int ti = cluster_id; ti < n_tiles && ok; ti += n_clusters) {
        const int4 t = tiles[ti];
        for (int pass = 0; pass < 2 && ok; ++pass) {
          const int brow = t.x * 2 * inter + pass * inter + cr * NC;   // gate rows, then up rows
          for (int kb = 0; kb < k_blocks; ++kb) {
            ok = mbar_wait(&empty[ps.stage], ps.phase ^ 1, abort_flag);
            if (!ok) break;
            mbar_expect_tx(&full[ps.stage], A_BYTES + L::B_BYTES);
            tma_load_2d(smem + L::OFF_A + ps.stage * A_BYTES, &tmA, &full[ps.stage], kb * BK, t.y);
            tma_load_2d(smem + L::OFF_B + ps.stage * L::B_BYTES, &tmB, &full[ps.stage], kb * BK, brow);
            ps.next<STAGES>();
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, NC);
      PipeState ps;
      uint32_t it = 0;
      bool ok = true;
      for (int ti = cluster_id; ti < n_tiles && ok; ti += n_clusters, ++it) {
        for (int pass = 0; pass < 2 && ok; ++pass) {
          ok = mbar_wait(pass == 0 ? gempty : uempty, (it & 1) ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          for (int kb = 0; kb < k_blocks; ++kb) {
            ok = mbar_wait(&full[ps.stage], ps.phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint64_t da = make_sdesc_k128(smem_u32(smem + L::OFF_A + ps.stage * A_BYTES));
            const uint64_t db = make_sdesc_k128(smem_u32(smem + L::OFF_B + ps.stage * L::B_BYTES));
#pragma unroll
            for (int k = 0; k < BK / UK; ++k)
              umma_bf16(tmem_base + pass * NC, da + k * 2, db + k * 2, idesc, (kb | k) != 0);
            umma_commit(&empty[ps.stage]);
            ps.next<STAGES>();
          }
          if (ok) umma_commit(pass == 0 ? gfull : ufull);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool issuer = (threadIdx.x == 64);
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    unsigned char* stash = smem + L::OFF_STASH;
    uint32_t it = 0;
    for (int ti = cluster_id; ti < n_tiles; ti += n_clusters, ++it) {
      const int4 t = tiles[ti];
      // the previous tile's stores must have finished reading the stash before it is overwritten
      if (issuer) tma_store_wait_read();
      named_bar_sync(1, EPI_THREADS);
      if (!mbar_wait(gfull, it & 1, abort_flag)) break;
      tc_fence_after();
      float ss = 0.f;
#pragma unroll 1
      for (int c = 0; c < NC / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_addr + c * 32, r);
        tmem_ld_wait();
        unsigned char* sub = stash + (c >> 1) * C_SUB;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t pk = pack_bf16(__uint_as_float(r[8 * j + 2 * i]), __uint_as_float(r[8 * j + 2 * i + 1]));
            const float a = bf16_lo(pk), b = bf16_hi(pk);   // the reference squares the bf16-rounded gate
            ss = fmaf(a, a, ss);
            ss = fmaf(b, b, ss);
            pv[i] = pk;
          }
          *reinterpret_cast<uint4*>(sub + swz(row, (c & 1) * 4 + j)) = v;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(gempty);
      if (CL > 1) {
        const uint32_t peer = cr ^ 1u;
        st_remote_f32(&part[(it & 1) * BM + row], peer, ss);
        mbar_arrive_remote(&xbar[it & 1], peer);
        if (!mbar_wait<true>(&xbar[it & 1], (it >> 1) & 1, abort_flag)) break;
        ss += part[(it & 1) * BM + row];
      }
      const float rn = sqrtf(ss / (float)inter + 1e-6f);
      const float p = sigmoid_accurate(__ldg(theta + t.x));
      const float gain = powf(rn, p);
      const float inv_r = __fdiv_rn(1.0f, rn);
      if (rnorm_out != nullptr && cr == 0) rnorm_out[t.y + row] = rn;

      if (!mbar_wait(ufull, it & 1, abort_flag)) break;
      tc_fence_after();
      __nv_bfloat16* gu_row = gate_up_out ? gate_up_out + (int64_t)(t.y + row) * 2 * inter + cr * NC : nullptr;
#pragma unroll 1
      for (int c = 0; c < NC / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_addr + NC + c * 32, r);
        tmem_ld_wait();
        unsigned char* sub = stash + (c >> 1) * C_SUB;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4* slot = reinterpret_cast<uint4*>(sub + swz(row, (c & 1) * 4 + j));
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
              const float z = g * inv_r;
              const float a = round_bf16(__fdividef(z, 1.0f + __expf(-z)) * gain);   // activation is cast to bf16
              hval[s] = a * u;                                                       // then multiplied in bf16
            }
            ph[i] = pack_bf16(hval[0], hval[1]);
          }
          *slot = hv;
          if (gu_row != nullptr) {
            *reinterpret_cast<uint4*>(gu_row + c * 32 + j * 8) = gv;
            *reinterpret_cast<uint4*>(gu_row + inter + c * 32 + j * 8) = uv;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(uempty);
      fence_proxy_async_smem();
      named_bar_sync(1, EPI_THREADS);
      if (issuer) {
#pragma unroll
        for (int s = 0; s < NC / 64; ++s) tma_store_2d(&tmH, stash + s * C_SUB, cr * NC + s * 64, t.y);
        tma_store_commit();
      }
    }
    if (issuer) tma_store_wait_all();
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (CL > 1) cluster_sync_all();   // nobody leaves while a peer may still write into this CTA
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 2 * NC); }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&plan[PLAN_STATUS], 101);
}

// =====================================================================================================
// K3 on CTA pairs.  Cluster of 2*CLN CTAs: rank r -> pr = r & 1 (position in the MMA pair, i.e. which
// of the two row tiles), ch = r >> 1 (which 256-column block of the gate / up projections).  The pair
// (r, r^1) runs 256-row tcgen05.mma.cta_group::2 instructions: each CTA stages its own A tile and 128
// of the 256 B rows, so a k-block costs 32 KB of shared memory per CTA instead of 48 KB (five pipeline
// stages beside the 64 KB gate stash).  For I = 512 the CTAs r and r^2 hold the two column blocks of
// the same rows and exchange their partial sums of squares exactly as the one-CTA kernel does.
// =====================================================================================================
template <int STAGES>
struct G1PairLayout {
  static constexpr int NC = 256;
  static constexpr int BH_BYTES = (NC / 2) * BK * 2;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_STASH = OFF_B + STAGES * BH_BYTES;
  static constexpr int OFF_PART = OFF_STASH + (NC / 64) * C_SUB;
  static constexpr int OFF_BAR = OFF_PART + 2 * BM * 4;
  static constexpr int BYTES = OFF_BAR + 256 + 1024;
};

// XG: the two column blocks of a row pair live in two separate 2-CTA clusters (blockIdx.x ^ 2) and
// exchange their partial sums through global memory (flag + 128 floats per CTA and parity) instead of
// distributed shared memory, so the cluster size stays 2 and every SM can host a CTA; the launcher
// guarantees that all CTAs are resident (grid <= SM count, one CTA per SM).
//
// GATHER: the kernel also builds its own A operand.  Six extra warps per CTA copy token rows
// src[row_src[r]] into the expert-contiguous buffer behind tmA, up to two row pairs ahead of the loads: the
// GROUP CTAs that work on a pair split its rows, every gather warp adds one to the pair's arrival
// counter (release, after a generic->async proxy fence) and each CTA's load thread waits for the
// GROUP * GATHER_WARPS arrivals (acquire) before its first tile load of that pair.  The copied rows are
// read back by the tile loads while they are still in L2.  Measured on 32768 tokens, hidden 2048,
// intermediate 512: the copies cost this kernel about as much as the separate permute pass takes
// (0.76 ms against 0.56 + 0.16 ms), because the kernel already moves ~14 TB/s through L2 and the copies
// add to that; the variant is therefore opt-in.  All waits are bounded like every other wait of this kernel.
constexpr int GATHER_WARPS = 6;
struct GatherArgs {
  const uint8_t* src;       // source rows, pitch row_bytes (token-major)
  uint8_t* dst;             // expert-contiguous rows: the tensor tmA describes
  const int32_t* row_src;   // [rows] source row of every valid expert-contiguous row
  int* ready;               // [pairs] arrival counters, zero at launch
  int row_bytes;
  int zero_padding;         // write zeros into the rows of a tile beyond its valid rows
};

template <int CLN, int STAGES, bool XG, bool GATHER = false>
__global__ void __launch_bounds__(NUM_THREADS + (GATHER ? GATHER_WARPS * 32 : 0), 1)
gemm1_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmH, const float* __restrict__ theta,
                  int32_t* __restrict__ plan, int64_t tiles_off, int64_t pairs_off, int k_blocks, int inter,
                  __nv_bfloat16* __restrict__ gate_up_out, float* __restrict__ rnorm_out, float* xg_part,
                  int* xg_flags, const GatherArgs ga = GatherArgs{}) {
  using L = G1PairLayout<STAGES>;
  constexpr int NC = L::NC;
  constexpr int CL = XG ? 2 : 2 * CLN;          // hardware cluster size
  constexpr int GROUP = 2 * CLN;                // CTAs that share one row pair
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  float* part = reinterpret_cast<float*>(smem + L::OFF_PART);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);   // used in the pair leader only
  uint64_t* empty = full + STAGES;
  uint64_t* gfull = empty + STAGES;
  uint64_t* gempty = gfull + 1;       // pair leader: 8 arrivals (4 epilogue warps of each CTA)
  uint64_t* ufull = gempty + 1;
  uint64_t* uempty = ufull + 1;       // pair leader
  uint64_t* xbar = uempty + 1;        // [2] partial-sum exchange with CTA r^2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xbar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* load_iter = reinterpret_cast<volatile int*>(tmem_slot + 2);   // pair iteration the load thread is on

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cr = cluster_ctarank();
  const uint32_t pr = cr & 1u, leader = cr & ~1u;
  const uint32_t ch = XG ? ((blockIdx.x >> 1) & (CLN - 1)) : (cr >> 1);
  const uint16_t pair_mask = (uint16_t)(3u << leader);
  const int cluster_id = blockIdx.x / GROUP, n_clusters = gridDim.x / GROUP;   // row-pair groups

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(gfull, 1); mbar_init(ufull, 1);
    mbar_init(gempty, 8); mbar_init(uempty, 8);
    mbar_init(&xbar[0], EPI_THREADS); mbar_init(&xbar[1], EPI_THREADS);
    *abort_flag = 0;
    *load_iter = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB); prefetch_tmap(&tmH);
  }
  if (warp == 1) { tmem_alloc_cg2(tmem_slot, 2 * NC); tmem_relinquish_cg2(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int n_pairs = plan[PLAN_N_PAIRS];
  const int4* tiles = reinterpret_cast<const int4*>(plan + tiles_off);
  const int2* pairs = reinterpret_cast<const int2*>(plan + pairs_off);

  if (warp == 0) {
    if (elect_one()) {
      PipeState ps;
      bool ok = true;
      int it = 0;
      for (int p = cluster_id; p < n_pairs && ok; p += n_clusters, ++it) {
        const int2 pp = pairs[p];
        const int4 t = tiles[(pr == 1 && pp.y >= 0) ? pp.y : pp.x];
        if (GATHER) {   // the rows of this pair have been copied by the gather warps of the whole group
          *load_iter = it;
          bool got = false;
          for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ga.ready + p) : "memory");
            if (v >= GROUP * GATHER_WARPS) { got = true; break; }
            if ((spin & 255u) == 255u && *abort_flag) break;
          }
          if (!got) { *abort_flag = 1; ok = false; break; }
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int pass = 0; pass < 2 && ok; ++pass) {
          const int brow = t.x * 2 * inter + pass * inter + (int)ch * NC + (int)pr * (NC / 2);
          for (int kb = 0; kb < k_blocks; ++kb) {
            ok = mbar_wait(&empty[ps.stage], ps.phase ^ 1, abort_flag);
            if (!ok) break;
            if (pr == 0) mbar_expect_tx(&full[ps.stage], 2 * (A_BYTES + L::BH_BYTES));
            const uint32_t bar0 = map_to_cta(&full[ps.stage], leader);
            tma_load_2d_cg2(smem + L::OFF_A + ps.stage * A_BYTES, &tmA, bar0, kb * BK, t.y);
            tma_load_2d_cg2(smem + L::OFF_B + ps.stage * L::BH_BYTES, &tmB, bar0, kb * BK, brow);
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
      for (int p = cluster_id; p < n_pairs && ok; p += n_clusters, ++it) {
        for (int pass = 0; pass < 2 && ok; ++pass) {
          ok = mbar_wait<true>(pass == 0 ? gempty : uempty, (it & 1) ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          for (int kb = 0; kb < k_blocks; ++kb) {
            ok = mbar_wait<true>(&full[ps.stage], ps.phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint64_t da = make_sdesc_k128(smem_u32(smem + L::OFF_A + ps.stage * A_BYTES));
            const uint64_t db = make_sdesc_k128(smem_u32(smem + L::OFF_B + ps.stage * L::BH_BYTES));
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
  } else if (GATHER && warp >= 6) {
    // ---- gather warps: copy this CTA's share of the rows of pair `it`, at most two pairs ahead of the loads
    const int gw = warp - 6;
    const int gi = blockIdx.x % GROUP;               // pr = gi & 1 (which tile), gi >> 1 = which part of its rows
    constexpr int SHARE = BM / CLN;
    const int chunks = ga.row_bytes >> 4;
    int it = 0;
    for (int p = cluster_id; p < n_pairs; p += n_clusters, ++it) {
      bool go = true;
      if (it >= 3) {
        go = false;
        for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
          if (*load_iter >= it - 2) { go = true; break; }
          if (*abort_flag) break;
          __nanosleep(200);
        }
      }
      if (!go) { *abort_flag = 1; break; }
      const int2 pp = pairs[p];
      const int ti = (gi & 1) ? pp.y : pp.x;
      if (ti >= 0) {
        const int4 t = tiles[ti];
        const int r0 = (gi >> 1) * SHARE;
        // this warp's rows are r0 + gw + i * GATHER_WARPS, taken two at a time: the sixteen 16-byte loads of a
        // lane (eight per row) are all issued before the first store; loads bypass L1 (the carve-out leaves
        // next to none), and the loop has no division: the warps next to this one issue the MMAs
        for (int ra = r0 + gw; ra < r0 + SHARE; ra += 2 * GATHER_WARPS) {
          const int rb = ra + GATHER_WARPS;
          const bool la = ra < t.z, lb = rb < r0 + SHARE && rb < t.z;
          const bool wa = la || (ga.zero_padding & 1), wb = rb < r0 + SHARE && (lb || (ga.zero_padding & 1));
          const uint4* sa = reinterpret_cast<const uint4*>(ga.src + (int64_t)(la ? __ldg(ga.row_src + t.y + ra) : 0) * ga.row_bytes);
          const uint4* sb = reinterpret_cast<const uint4*>(ga.src + (int64_t)(lb ? __ldg(ga.row_src + t.y + rb) : 0) * ga.row_bytes);
          uint4* da = reinterpret_cast<uint4*>(ga.dst + (int64_t)(t.y + ra) * ga.row_bytes);
          uint4* db = reinterpret_cast<uint4*>(ga.dst + (int64_t)(t.y + rb) * ga.row_bytes);
          for (int c0 = lane; c0 < chunks; c0 += 256) {
            uint4 va[8], vb[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int c = c0 + u * 32;
              va[u] = (la && c < chunks) ? __ldcg(sa + c) : make_uint4(0, 0, 0, 0);
              vb[u] = (lb && c < chunks) ? __ldcg(sb + c) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int c = c0 + u * 32;
              if (wa && c < chunks) da[c] = va[u];
              if (wb && c < chunks) db[c] = vb[u];
            }
          }
        }
      }
      asm volatile("fence.proxy.async.global;" ::: "memory");
      __threadfence();
      __syncwarp();
      if (lane == 0) asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(ga.ready + p) : "memory");
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool issuer = (threadIdx.x == 64);
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    unsigned char* stash = smem + L::OFF_STASH;
    uint32_t it = 0;
    for (int p = cluster_id; p < n_pairs; p += n_clusters, ++it) {
      const int2 pp = pairs[p];
      const bool twin = (pr == 1 && pp.y < 0);     // duplicate of the leader's tile: compute, write nothing
      const int4 t = tiles[(pr == 1 && pp.y >= 0) ? pp.y : pp.x];
      if (issuer) tma_store_wait_read();           // the previous tile's stores are done with the stash
      named_bar_sync(1, EPI_THREADS);
      if (!mbar_wait(gfull, it & 1, abort_flag)) break;
      tc_fence_after();
      float ss = 0.f;
#pragma unroll 1
      for (int c = 0; c < NC / 64; ++c) {
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
            uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t pk = pack_bf16(__uint_as_float(r[8 * j + 2 * i]), __uint_as_float(r[8 * j + 2 * i + 1]));
              const float a = bf16_lo(pk), b = bf16_hi(pk);
              ss = fmaf(a, a, ss);
              ss = fmaf(b, b, ss);
              pv[i] = pk;
            }
            *reinterpret_cast<uint4*>(sub + swz(row, hh * 4 + j)) = v;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_addr(map_to_cta(gempty, leader));
      if (CLN > 1 && !XG) {
        const uint32_t peer = cr ^ 2u;
        st_remote_f32(&part[(it & 1) * BM + row], peer, ss);
        mbar_arrive_remote(&xbar[it & 1], peer);
        if (!mbar_wait<true>(&xbar[it & 1], (it >> 1) & 1, abort_flag)) break;
        ss += part[(it & 1) * BM + row];
      }
      if (CLN > 1 && XG) {
        const int par = it & 1, epoch = (int)(it >> 1) + 1;
        xg_part[((int64_t)blockIdx.x * 2 + par) * BM + row] = ss;
        __threadfence();
        named_bar_sync(1, EPI_THREADS);
        if (threadIdx.x == 64) asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(xg_flags + blockIdx.x * 2 + par), "r"(epoch) : "memory");
        const int peer_cta = blockIdx.x ^ 2;
        const int* pf = xg_flags + peer_cta * 2 + par;
        bool got = false;
        for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
          int v;
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(pf) : "memory");
          if (v >= epoch) { got = true; break; }
          if ((spin & 255u) == 255u && *abort_flag) break;
        }
        if (!got) { *abort_flag = 1; break; }
        ss += __ldcg(&xg_part[((int64_t)peer_cta * 2 + par) * BM + row]);
      }
      const float rn = sqrtf(ss / (float)inter + 1e-6f);
      const float pw = sigmoid_accurate(__ldg(theta + t.x));
      const float gain = powf(rn, pw);
      const float inv_r_half = 0.5f * __fdiv_rn(1.0f, rn);
      if (rnorm_out != nullptr && ch == 0 && !twin) rnorm_out[t.y + row] = rn;

      if (!mbar_wait(ufull, it & 1, abort_flag)) break;
      tc_fence_after();
      __nv_bfloat16* gu_row =
          (gate_up_out && !twin) ? gate_up_out + (int64_t)(t.y + row) * 2 * inter + ch * NC : nullptr;
#pragma unroll 1
      for (int c2 = 0; c2 < NC / 64; ++c2) {
        uint32_t rr0[32], rr1[32];
        tmem_ld32(lane_addr + NC + c2 * 64, rr0);
        tmem_ld32(lane_addr + NC + c2 * 64 + 32, rr1);
        tmem_ld_wait();
        unsigned char* sub = stash + c2 * C_SUB;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int c = c2 * 2 + (jj >> 2), j = jj & 3;
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
              const float zh = g * inv_r_half;
              float th;
              asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(zh));
              const float a = round_bf16(fmaf(zh, th, zh) * gain);
              hval[s] = a * u;
            }
            ph[i] = pack_bf16(hval[0], hval[1]);
          }
          *slot = hv;
          if (gu_row != nullptr) {
            *reinterpret_cast<uint4*>(gu_row + c * 32 + j * 8) = gv;
            *reinterpret_cast<uint4*>(gu_row + inter + c * 32 + j * 8) = uv;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_addr(map_to_cta(uempty, leader));
      fence_proxy_async_smem();
      named_bar_sync(1, EPI_THREADS);
      if (issuer && !twin) {
#pragma unroll
        for (int s = 0; s < NC / 64; ++s) tma_store_2d(&tmH, stash + s * C_SUB, ch * NC + s * 64, t.y);
        tma_store_commit();
      }
    }
    if (issuer) tma_store_wait_all();
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // nobody leaves while a cluster peer may still signal or write into this CTA
  if (warp == 1) { tc_fence_after(); tmem_dealloc_cg2(tmem_base, 2 * NC); }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&plan[PLAN_STATUS], 104);
}

// =====================================================================================================
// host side
// =====================================================================================================
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
                      uint32_t box_rows) {
  using Key = std::tuple<const void*, uint64_t, uint64_t, uint64_t, uint32_t>;
  static std::mutex mu;
  static std::map<Key, CUtensorMap> cache;
  const Key key{base, rows, cols, pitch_elems, box_rows};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return BIBO_OK; }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(BIBO_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(BIBO_ERR_CUDA, "cuTensorMapEncodeTiled(rows=%llu cols=%llu box_rows=%u) -> %d",
                (unsigned long long)rows, (unsigned long long)cols, box_rows, (int)r);
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 256) cache.clear();
  cache[key] = *out;
  return BIBO_OK;
}

template <typename Kern>
static int set_smem(Kern kern, int bytes) {
  BIBO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return BIBO_OK;
}

}  // namespace tc

using namespace tc;

int gemm2_tc_supported(int hidden, int inter, int dtype) {
  return dtype == BIBO_BF16 && hidden % 256 == 0 && inter % 64 == 0 && inter >= 64;
}

template <int BN, int STAGES, bool RES = false>
static int gemm2_launch_t(const void* h, const void* down_proj, const PlanView& pv, int hidden, int inter,
                          int n_weight_experts, void* y, cudaStream_t st, const void* residual = nullptr) {
  using L = G2Layout<BN, STAGES>;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tmA, h, pv.rows_alloc, inter, inter, BM))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmB, down_proj, (uint64_t)n_weight_experts * hidden, inter, inter, BN))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmC, y, pv.rows_alloc, hidden, hidden, BM))) return rc;
  auto kern = gemm2_tc_kernel<BN, STAGES, RES>;
  static DeviceOnce once;
  if ((rc = once.get([&](int*) { return set_smem(kern, L::BYTES); }))) return rc;
  const int64_t work_cap = pv.tiles_cap * (hidden / BN);
  const int sms = pv.max_ctas > 0 ? std::min(pv.max_ctas, sm_count()) : sm_count();
  const int grid = (int)std::min<int64_t>(sms, work_cap);
  kern<<<grid, NUM_THREADS, L::BYTES, st>>>(tmA, tmB, tmC, const_cast<int32_t*>(pv.plan), pv.tiles_off, hidden / BN,
                                           inter / BK, hidden, static_cast<const __nv_bfloat16*>(residual));
  BIBO_CHECK_LAUNCH("gemm2_tc_kernel");
  return BIBO_OK;
}

int gemm2_tc_launch(const void* h, const void* down_proj, const PlanView& pv, int hidden, int inter,
                    int n_weight_experts, void* y, cudaStream_t st) {
  return gemm2_launch_t<256, 4>(h, down_proj, pv, hidden, inter, n_weight_experts, y, st);
}

// y = bf16(bf16(h x down_proj^T) + residual); residual has y's shape and pitch
int gemm2_tc_residual_launch(const void* h, const void* down_proj, const PlanView& pv, int hidden, int inter,
                             int n_weight_experts, void* y, const void* residual, cudaStream_t st) {
  return gemm2_launch_t<256, 4, true>(h, down_proj, pv, hidden, inter, n_weight_experts, y, st, residual);
}

int gemm1_tc_supported(int hidden, int inter, int dtype) {
  return dtype == BIBO_BF16 && hidden % 64 == 0 && hidden >= 64 && (inter == 128 || inter == 256 || inter == 512);
}

template <int NC, int CL, int STAGES>
static int gemm1_launch_t(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmH, const float* theta,
                          const int32_t* plan, int64_t tiles_off, int64_t tile_cap, int max_ctas, int k_blocks,
                          int inter, void* gate_up_out, float* rnorm_out, cudaStream_t st) {
  using L = G1Layout<NC, STAGES>;
  auto kern = gemm1_tc_kernel<NC, CL, STAGES>;
  static DeviceOnce once;
  int rc;
  if ((rc = once.get([&](int*) { return set_smem(kern, L::BYTES); }))) return rc;
  const int sms = max_ctas > 0 ? std::min(max_ctas, sm_count()) : sm_count();
  int clusters = (int)std::min<int64_t>(sms / CL, tile_cap);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(clusters * CL);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = L::BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  BIBO_CUDA(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmH, theta, const_cast<int32_t*>(plan), tiles_off, k_blocks, inter,
                               reinterpret_cast<__nv_bfloat16*>(gate_up_out), rnorm_out));
  launch_counter().fetch_add(1, std::memory_order_relaxed);
  return BIBO_OK;
}

template <int CLN, int STAGES, bool XG, bool GATHER>
static int gemm1_pair_launch_t(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmH,
                               const float* theta, const PlanView& pv, int k_blocks, int inter, void* gate_up_out,
                               float* rnorm_out, cudaStream_t st, GatherArgs ga = GatherArgs{}) {
  using L = G1PairLayout<STAGES>;
  constexpr int CL = XG ? 2 : 2 * CLN;      // hardware cluster size
  constexpr int GROUP = 2 * CLN;            // CTAs per row pair
  constexpr int THREADS = NUM_THREADS + (GATHER ? GATHER_WARPS * 32 : 0);
  auto kern = gemm1_pair_kernel<CLN, STAGES, XG, GATHER>;
  int rc;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = L::BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  static DeviceOnce once;
  int max_clusters = 0;
  rc = once.get([&](int* v) {
    int r = set_smem(kern, L::BYTES);
    if (r) return r;
    cfg.gridDim = dim3((sm_count() / CL) * CL);
    int n = 0;
    BIBO_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));   // clusters of CL CTAs that fit at once
    *v = n > 0 ? n : 1;
    return (int)BIBO_OK;
  }, &max_clusters);
  if (rc) return rc;
  const int sms = pv.max_ctas > 0 ? std::min(pv.max_ctas, sm_count()) : sm_count();
  // resident CTAs only: the CTAs of a group wait on one another through global memory (XG, GATHER)
  const int ctas = std::min(std::min(max_clusters * CL, sms), XG_MAX_CTAS);
  const int groups = (int)std::max<int64_t>(1, std::min<int64_t>(ctas / GROUP, pv.tiles_cap));
  cfg.gridDim = dim3(groups * GROUP);
  int32_t* scratch = const_cast<int32_t*>(pv.plan) + pv.scratch_off;
  float* xg_part = reinterpret_cast<float*>(scratch);
  int* xg_flags = scratch + XG_PART_WORDS;
  // the exchange flags and, behind them, the gather arrival counters start every launch at zero
  const size_t clear_words = (XG ? XG_MAX_CTAS * 2 : 0) + (GATHER ? (size_t)pv.tiles_cap : 0);
  if (GATHER) ga.ready = scratch + XG_WORDS;
  if (clear_words) {
    int* from = XG ? xg_flags : scratch + XG_WORDS;
    BIBO_CUDA(cudaMemsetAsync(from, 0, sizeof(int) * clear_words, st));
  }
  BIBO_CUDA(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmH, theta, const_cast<int32_t*>(pv.plan), pv.tiles_off,
                               pv.pairs_off, k_blocks, inter, reinterpret_cast<__nv_bfloat16*>(gate_up_out),
                               rnorm_out, xg_part, xg_flags, ga));
  launch_counter().fetch_add(1, std::memory_order_relaxed);
  return BIBO_OK;
}

// rows of `src` (pitch = hidden bf16) are gathered by the kernel itself: intermediate sizes with a CTA-pair kernel
int gemm1_gather_supported(int hidden, int inter, int dtype) {
  return dtype == BIBO_BF16 && hidden % 64 == 0 && hidden >= 64 && (inter == 256 || inter == 512);
}

// gather != nullptr: `xp` is written by the kernel from gather_src rows (see GatherArgs), not read from a permute pass
int gemm1_tc_launch(const void* xp, const void* gate_up_proj, const float* theta, const PlanView& pv, int hidden,
                    int inter, int n_weight_experts, void* h, void* gate_up_out, float* rnorm_out, cudaStream_t st,
                    const void* gather_src, const int32_t* row_src, int zero_padding) {
  const int nc = inter >= 256 ? 256 : 128;
  CUtensorMap tmA, tmB, tmH;
  int rc;
  if (gather_src != nullptr && (!gemm1_gather_supported(hidden, inter, BIBO_BF16) || row_src == nullptr))
    return fail(BIBO_ERR_UNSUPPORTED, "gate/up kernel: no row-gathering variant for hidden=%d inter=%d", hidden, inter);
  if (inter >= 256) {
    if ((rc = make_tmap_bf16_2d(&tmA, xp, pv.rows_alloc, hidden, hidden, BM))) return rc;
    if ((rc = make_tmap_bf16_2d(&tmB, gate_up_proj, (uint64_t)n_weight_experts * 2 * inter, hidden, hidden, 128))) return rc;
    if ((rc = make_tmap_bf16_2d(&tmH, h, pv.rows_alloc, inter, inter, BM))) return rc;
    if (gather_src != nullptr) {
      GatherArgs ga{static_cast<const uint8_t*>(gather_src), static_cast<uint8_t*>(const_cast<void*>(xp)), row_src,
                    nullptr, hidden * 2, zero_padding & 1};
      if (inter == 512)
        return gemm1_pair_launch_t<2, 5, true, true>(tmA, tmB, tmH, theta, pv, hidden / BK, inter, gate_up_out,
                                                     rnorm_out, st, ga);
      return gemm1_pair_launch_t<1, 5, false, true>(tmA, tmB, tmH, theta, pv, hidden / BK, inter, gate_up_out,
                                                    rnorm_out, st, ga);
    }
    // A capped grid shares the GPU with another stream's kernels, and nothing guarantees that every CTA of it
    // is resident at once: the variant whose column-block pairs exchange through distributed shared memory
    // inside ONE 4-CTA cluster (co-scheduled by the hardware) waits on nobody outside its cluster.
    if (inter == 512 && pv.max_ctas > 0)
      return gemm1_pair_launch_t<2, 5, false, false>(tmA, tmB, tmH, theta, pv, hidden / BK, inter, gate_up_out,
                                                     rnorm_out, st);
    if (inter == 512)
      return gemm1_pair_launch_t<2, 5, true, false>(tmA, tmB, tmH, theta, pv, hidden / BK, inter, gate_up_out,
                                                    rnorm_out, st);
    return gemm1_pair_launch_t<1, 5, false, false>(tmA, tmB, tmH, theta, pv, hidden / BK, inter, gate_up_out,
                                                   rnorm_out, st);
  }
  if ((rc = make_tmap_bf16_2d(&tmA, xp, pv.rows_alloc, hidden, hidden, BM))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmB, gate_up_proj, (uint64_t)n_weight_experts * 2 * inter, hidden, hidden, nc))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmH, h, pv.rows_alloc, inter, inter, BM))) return rc;
  return gemm1_launch_t<128, 1, 4>(tmA, tmB, tmH, theta, pv.plan, pv.tiles_off, pv.tiles_cap, pv.max_ctas,
                                   hidden / BK, inter, gate_up_out, rnorm_out, st);
}

// router on tensor cores: see router_tc.cu
}  // namespace bibo
