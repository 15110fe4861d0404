// Expert-parallel forward with a de-duplicated exchange: a token row crosses NVLink ONCE per destination
// rank (not once per selected expert), and ONE partial result row per (token, rank) comes back.
//
// Sharding as in ep.cu: rank d owns experts [d*EL, (d+1)*EL), EL = E/R; tokens stay on their home rank;
// the router is replicated.  Every rank provides, mapped into all processes of the group,
//   xu   [R*n_cap, H]  rows received from every source rank, slot v = s*n_cap + t (no compaction: the
//                      position of a row depends only on its source rank and token, so the sender needs
//                      no counts from anybody before it can store);
//   midx [R*n_cap, k]  the LOCAL expert index of every slot of every token of every rank (-1 where the
//   mw   [R*n_cap, k]  slot belongs to another rank, or the token does not exist) and its routing weight;
//   part [R*n_cap, H]  on the HOME rank: part[d*n_cap + t] = what owner d contributes to token t.
// n_cap = the largest token count of any rank (ranks may hold different numbers of tokens).
//
// Per forward and rank:
//   home   ep_dedup_dispatch_kernel  x[t] -> xu of every DISTINCT owner among the token's k experts (peer
//                                    stores), routing records -> midx / mw of ALL ranks (48 bytes each)
//   -- barrier --
//   owner  the caller-routed single-GPU chain over the R*n_cap "virtual tokens" of its receive buffer with
//          its EL experts (rank_kernel with empty slots -> plan -> permute -> gate/up -> down), then
//          ep_dedup_partial_kernel: sum_j w_j * y[row_j] over the virtual token's local slots in ascending
//          expert order (fp32), rounded to bf16 and stored into the home rank's `part` (peer stores)
//   -- barrier --
//   home   ep_dedup_final_kernel     out[t] = bf16( sum over owners d in ascending order of part[d][t] )
//
// Against the single-GPU chain the sum over a token's slots is taken in the same order (experts are
// sharded contiguously, so "ascending expert" = "ascending owner, then ascending expert"), but every
// owner's partial is rounded to bf16 before the last addition: results are within the bf16 parity bars of
// the fp32 oracle, not bit-identical to one GPU (the per-slot exchange in ep.cu is).
// Bytes per direction and rank: (distinct remote owners per token) * 2H instead of (remote slots) * 2H:
// with 64 experts and top-6 that is 0.99 / 2.50 / 3.96 rows instead of 2.98 / 4.49 / 5.25 at 2 / 4 / 8 ranks.
#include <algorithm>

#include "ep_common.cuh"

namespace bibo {

constexpr int DW = 8;        // warps per block of the exchange kernels when they have the GPU to themselves
constexpr int DW_TAGGED = 16; // warps per block of a capped grid
// A capped exchange grid (comm_ctas > 0: token slices pipelined against another slice's grouped GEMMs) runs
// blocks of 16 warps that ask for this much dynamic shared memory and never touch it.  Two such blocks do
// not fit on one SM and none fits beside a GEMM CTA (which takes all but 1 KB of the shared memory), so the
// hardware places every exchange block on an SM of its own, whichever kernel arrives first: comm_ctas IS the
// number of SMs the exchange uses, and the grouped GEMMs (capped by the caller to the rest) keep theirs.
// Without the tag the block scheduler spreads small blocks over as many SMs as it can, each of which then
// lacks the shared memory for a GEMM CTA: the GEMMs ran 1.5-1.75x slower while an exchange kernel was active.
constexpr int COMM_TAG_BYTES = 120 * 1024;

__device__ __forceinline__ void fma_bf16x8_d(const uint4& v, float w, float* acc) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] = fmaf(__uint_as_float(u[i] << 16), w, acc[2 * i]);
    acc[2 * i + 1] = fmaf(__uint_as_float(u[i] & 0xffff0000u), w, acc[2 * i + 1]);
  }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float* a) {
  uint4 o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
  return o;
}

// Warp per token slot t in [0, n_cap).  t >= n_tokens: only "no such token" records are written.
__global__ void __launch_bounds__(DW_TAGGED * 32, 1)
ep_dedup_dispatch_kernel(const uint8_t* __restrict__ x, const int32_t* __restrict__ topk_idx,
                         const float* __restrict__ topk_w, PeerPtrs xu, PeerPtrs midx, PeerPtrs mw,
                         int64_t n_tokens, int64_t n_cap, int row_bytes, int n_experts, int rank, int world,
                         int top_k, int records) {
  const int lane = threadIdx.x & 31;
  const int el = n_experts / world;
  for (int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < n_cap; t += (int64_t)gridDim.x * (blockDim.x >> 5)) {
    const int64_t v = (int64_t)rank * n_cap + t;
    int e = -1;
    float w = 0.f;
    if (t < n_tokens && lane < top_k) {
      e = topk_idx[t * top_k + lane];
      w = topk_w[t * top_k + lane];
      if (e >= n_experts) e = -1;
    }
    const int owner = e >= 0 ? e / el : -1;
    unsigned hit = 0;                                  // bit d: some slot of this token lives on rank d
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) {
      const int o = __shfl_sync(0xffffffffu, owner, j);
      if (j < top_k && o >= 0) hit |= 1u << o;
    }
    if (records && lane < top_k) {
      for (int d = 0; d < world; ++d) {
        static_cast<int32_t*>(midx.p[d])[v * top_k + lane] = owner == d ? e - d * el : -1;
        static_cast<float*>(mw.p[d])[v * top_k + lane] = w;
      }
    }
    if (hit == 0) continue;
    const uint4* src = reinterpret_cast<const uint4*>(x + t * row_bytes);
    const int chunks = row_bytes >> 4;
    for (int c0 = lane; c0 < chunks; c0 += 256) {      // eight 16-byte loads in flight per lane
      uint4 val[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (c0 + u * 32 < chunks) val[u] = __ldg(src + c0 + u * 32);
      for (int d = 0; d < world; ++d) {
        if (!((hit >> d) & 1u)) continue;
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(xu.p[d]) + v * row_bytes);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (c0 + u * 32 < chunks) dst[c0 + u * 32] = val[u];
      }
    }
  }
}

// Routing records that arrived as plain copies of every rank's top-k table (GLOBAL expert indices, -1 for
// "no such token"): keep the slots of this rank's experts, as local indices; everything else becomes -1.
__global__ void __launch_bounds__(256)
ep_localize_kernel(const int32_t* __restrict__ raw, int64_t n_slots, int lo, int el, int32_t* __restrict__ midx) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n_slots) return;
  const int e = raw[i] - lo;
  midx[i] = (e >= 0 && e < el) ? e : -1;
}

// Warp per virtual token v = s*n_cap + t of this owner.  Its local slots are summed in ascending slot order:
// with the router's ascending expert lists that is ascending expert order (the order of the single-GPU
// combine); a caller-routed list in another order changes only the order of the fp32 additions.
template <int K>
__global__ void __launch_bounds__(DW_TAGGED * 32, 1)
ep_dedup_partial_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ slot_row,
                        const float* __restrict__ mw, PeerPtrs part, const int32_t* __restrict__ plan,
                        int64_t n_virtual, int64_t n_cap, int hidden, int rank) {
  const int lane = threadIdx.x & 31;
  if (plan[PLAN_STATUS] != 0) return;
  const int world = (int)(n_virtual / n_cap);
  for (int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n_virtual; i += (int64_t)gridDim.x * (blockDim.x >> 5)) {
    // consecutive warps take the same token slot of consecutive home ranks, starting at rank+1: at any moment
    // every owner stores to ALL home ranks at once, its own included (walking the blocks of home ranks one after
    // the other in the same order on every owner aimed all owners at one receiver at a time: 0.4 ms of waiting
    // for the slowest rank at 4 GPUs; walking them in a rotated order left the local, HBM-only part for the end
    // instead of under the NVLink stores)
    const int64_t t = i / world, blk = i - t * world;
    const int64_t s = (rank + 1 + blk) % world;
    const int64_t v = s * n_cap + t;
    int row = -1;
    float w = 0.f;
    if (lane < K) { row = slot_row[v * K + lane]; w = mw[v * K + lane]; }
    const unsigned valid = __ballot_sync(0xffffffffu, row >= 0);
    if (valid == 0) continue;
    const int cnt = __popc(valid);
    const uint4* src[K];
    float ws[K];
    unsigned rest = valid;                             // the local slots in ascending slot order, wherever they sit
#pragma unroll
    for (int i = 0; i < K; ++i) {
      const int j = rest ? __ffs(rest) - 1 : 0;
      rest &= rest - 1;
      const int r = __shfl_sync(0xffffffffu, row, j);
      ws[i] = __shfl_sync(0xffffffffu, w, j);
      src[i] = reinterpret_cast<const uint4*>(y + (int64_t)(i < cnt ? r : 0) * hidden);
    }
    uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(part.p[s]) + ((int64_t)rank * n_cap + t) * hidden);
    const int chunks = hidden >> 3;
    if (cnt <= 2) {
      // the common case (a token rarely has more than two experts on one rank): four chunks per lane in flight
      for (int c0 = lane; c0 < chunks; c0 += 128) {
        uint4 va[4], vb[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (c0 + u * 32 < chunks) {
            va[u] = __ldcs(src[0] + c0 + u * 32);
            if (cnt == 2) vb[u] = __ldcs(src[1] + c0 + u * 32);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (c0 + u * 32 >= chunks) continue;
          float a[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) a[q] = 0.f;
          fma_bf16x8_d(va[u], ws[0], a);
          if (cnt == 2) fma_bf16x8_d(vb[u], ws[1], a);
          dst[c0 + u * 32] = pack_bf16x8(a);
        }
      }
      continue;
    }
    for (int c0 = lane; c0 < chunks; c0 += 64) {       // two chunks per lane in flight, times the local slots
      uint4 val[2][K];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int i = 0; i < K; ++i)
          if (i < cnt && c0 + u * 32 < chunks) val[u][i] = __ldcs(src[i] + c0 + u * 32);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (c0 + u * 32 >= chunks) continue;
        float a[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) a[q] = 0.f;
#pragma unroll
        for (int i = 0; i < K; ++i)
          if (i < cnt) fma_bf16x8_d(val[u][i], ws[i], a);
        dst[c0 + u * 32] = pack_bf16x8(a);
      }
    }
  }
}

// Partial rows that were summed into a LOCAL staging buffer (laid out like `part`: row s*n_cap + t for home
// rank s) travel to the home ranks: warp per virtual token with local slots, a plain 16-byte copy loop with
// eight loads in flight per lane.  Nothing but streaming, so a handful of SMs keeps NVLink busy while the
// rest of the GPU runs another token slice's grouped GEMMs.  Home ranks in the rotated order rank+1, ...
__global__ void __launch_bounds__(DW_TAGGED * 32, 1)
ep_dedup_push_kernel(const uint8_t* __restrict__ stage, const int32_t* __restrict__ midx, PeerPtrs part,
                     const int32_t* __restrict__ plan, int64_t n_virtual, int64_t n_cap, int row_bytes, int top_k,
                     int rank) {
  const int lane = threadIdx.x & 31;
  if (plan[PLAN_STATUS] != 0) return;
  const int world = (int)(n_virtual / n_cap);
  const int chunks = row_bytes >> 4;
  for (int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n_virtual - n_cap;
       i += (int64_t)gridDim.x * (blockDim.x >> 5)) {
    const int64_t blk = i / n_cap, t = i - blk * n_cap;
    const int64_t s = (rank + 1 + blk) % world;          // never the own rank: its rows are summed in place
    const int64_t v = s * n_cap + t;
    const bool any = __any_sync(0xffffffffu, lane < top_k && midx[v * top_k + lane] >= 0);
    if (!any) continue;
    const uint4* src = reinterpret_cast<const uint4*>(stage + v * row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(part.p[s]) + ((int64_t)rank * n_cap + t) * row_bytes);
    for (int c0 = lane; c0 < chunks; c0 += 256) {
      uint4 val[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (c0 + u * 32 < chunks) val[u] = __ldcs(src + c0 + u * 32);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (c0 + u * 32 < chunks) dst[c0 + u * 32] = val[u];
    }
  }
}

// Warp per home token: adds the partial rows of the owners the token was sent to, ascending owner.
// W = ranks the kernel is compiled for (2, 4 or 8): 8 / W chunks of every owner's row are in flight per lane.
template <int W>
__global__ void __launch_bounds__(DW_TAGGED * 32, 1)
ep_dedup_final_kernel(const __nv_bfloat16* __restrict__ part, const int32_t* __restrict__ topk_idx,
                      const int32_t* __restrict__ status, int64_t n_tokens, int64_t n_cap, int hidden, int n_experts,
                      int world, int top_k, __nv_bfloat16* __restrict__ out) {
  constexpr int U = 8 / W;
  const int lane = threadIdx.x & 31;
  if (status[0] != 0) return;
  const int el = n_experts / world;
  for (int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < n_tokens; t += (int64_t)gridDim.x * (blockDim.x >> 5)) {
    int owner = -1;
    if (lane < top_k) {
      const int e = topk_idx[t * top_k + lane];
      if (e >= 0 && e < n_experts) owner = e / el;
    }
    unsigned hit = 0;
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j) {
      const int o = __shfl_sync(0xffffffffu, owner, j);
      if (j < top_k && o >= 0) hit |= 1u << o;
    }
    uint4* dst = reinterpret_cast<uint4*>(out + t * hidden);
    const int chunks = hidden >> 3;
    for (int c0 = lane; c0 < chunks; c0 += 32 * U) {
      uint4 val[U][W];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int d = 0; d < W; ++d)
          if (((hit >> d) & 1u) && c0 + u * 32 < chunks)
            val[u][d] = __ldcs(reinterpret_cast<const uint4*>(part + ((int64_t)d * n_cap + t) * hidden) + c0 + u * 32);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (c0 + u * 32 >= chunks) continue;
        float a[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) a[q] = 0.f;
#pragma unroll
        for (int d = 0; d < W; ++d)
          if ((hit >> d) & 1u) fma_bf16x8_d(val[u][d], 1.0f, a);
        dst[c0 + u * 32] = pack_bf16x8(a);
      }
    }
  }
}

// gemm_tc.cu
int gemm1_tc_supported(int hidden, int inter, int dtype);
int gemm1_tc_launch(const void* xp, const void* gate_up_proj, const float* theta, const PlanView& pv, int hidden,
                    int inter, int n_weight_experts, void* h, void* gate_up_out, float* rnorm_out, cudaStream_t st,
                    const void* gather_src = nullptr, const int32_t* row_src = nullptr, int zero_padding = 0);
int gemm2_tc_supported(int hidden, int inter, int dtype);
int gemm2_tc_launch(const void* h, const void* down_proj, const PlanView& pv, int hidden, int inter,
                    int n_weight_experts, void* y, cudaStream_t st);

}  // namespace bibo

using namespace bibo;

template <typename Kern>
static void prefer_max_smem_d(Kern kern) {
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}
// same carve-out as the grouped GEMMs, so these kernels can share SMs with another token slice's GEMMs
template <typename Kern>
static void allow_tag_smem(Kern kern) {
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, COMM_TAG_BYTES);
}
static void dedup_set_carveouts() {
  static DeviceOnce once;
  once.get([](int*) {
    allow_tag_smem(ep_dedup_dispatch_kernel);
    allow_tag_smem(ep_dedup_final_kernel<2>); allow_tag_smem(ep_dedup_final_kernel<4>);
    allow_tag_smem(ep_dedup_final_kernel<8>);
    allow_tag_smem(ep_dedup_push_kernel);
    prefer_max_smem_d(ep_dedup_push_kernel);
    allow_tag_smem(ep_dedup_partial_kernel<1>); allow_tag_smem(ep_dedup_partial_kernel<2>);
    allow_tag_smem(ep_dedup_partial_kernel<3>); allow_tag_smem(ep_dedup_partial_kernel<4>);
    allow_tag_smem(ep_dedup_partial_kernel<5>); allow_tag_smem(ep_dedup_partial_kernel<6>);
    allow_tag_smem(ep_dedup_partial_kernel<7>); allow_tag_smem(ep_dedup_partial_kernel<8>);
    prefer_max_smem_d(ep_dedup_dispatch_kernel);
    prefer_max_smem_d(ep_dedup_final_kernel<2>); prefer_max_smem_d(ep_dedup_final_kernel<4>);
    prefer_max_smem_d(ep_dedup_final_kernel<8>);
    prefer_max_smem_d(ep_dedup_partial_kernel<1>); prefer_max_smem_d(ep_dedup_partial_kernel<2>);
    prefer_max_smem_d(ep_dedup_partial_kernel<3>); prefer_max_smem_d(ep_dedup_partial_kernel<4>);
    prefer_max_smem_d(ep_dedup_partial_kernel<5>); prefer_max_smem_d(ep_dedup_partial_kernel<6>);
    prefer_max_smem_d(ep_dedup_partial_kernel<7>); prefer_max_smem_d(ep_dedup_partial_kernel<8>);
    return (int)BIBO_OK;
  });
}

static int dedup_check(const char* who, int world, int rank, int n_experts, int top_k, int hidden, int64_t n_cap) {
  if (world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world)
    return fail(BIBO_ERR_ARG, "%s: rank %d of %d (max %d ranks)", who, rank, world, EP_MAX_RANKS);
  if (n_experts < world || n_experts > BIBO_MAX_EXPERTS || n_experts % world != 0)
    return fail(BIBO_ERR_UNSUPPORTED, "%s: %d experts do not shard evenly over %d ranks", who, n_experts, world);
  if (top_k < 1 || top_k > BIBO_MAX_TOP_K) return fail(BIBO_ERR_UNSUPPORTED, "%s: top_k=%d", who, top_k);
  if (hidden < 8 || hidden % 8 != 0) return fail(BIBO_ERR_UNSUPPORTED, "%s: hidden=%d", who, hidden);
  if (n_cap <= 0 || n_cap * world * (int64_t)top_k > 0x7fffffffLL)
    return fail(BIBO_ERR_ARG, "%s: n_cap=%lld", who, (long long)n_cap);
  return BIBO_OK;
}

static int fill_peers(const char* who, void* const* in, int world, PeerPtrs* out) {
  if (!in) return fail(BIBO_ERR_ARG, "%s: null peer table", who);
  for (int i = 0; i < world; ++i) {
    if (!in[i] || !aligned16(in[i])) return fail(BIBO_ERR_ALIGN, "%s: peer buffer %d", who, i);
    out->p[i] = in[i];
  }
  return BIBO_OK;
}

static unsigned exchange_grid(int64_t warps, int comm_ctas) {
  if (comm_ctas > 0) return (unsigned)std::max<int64_t>(1, std::min<int64_t>((warps + DW_TAGGED - 1) / DW_TAGGED, comm_ctas));
  return (unsigned)std::max<int64_t>(1, (warps + DW - 1) / DW);
}
static unsigned exchange_block(int comm_ctas) { return (comm_ctas > 0 ? DW_TAGGED : DW) * 32; }
static size_t exchange_smem(int comm_ctas) { return comm_ctas > 0 ? COMM_TAG_BYTES : 0; }

extern "C" int64_t bibo_moe_ep_dedup_virtual_tokens(int world, int64_t n_cap) { return (int64_t)world * n_cap; }

extern "C" int bibo_moe_ep_dedup_dispatch(const void* x, const int32_t* topk_idx, const float* topk_w,
                                          void* const* xu_peers, void* const* midx_peers, void* const* mw_peers,
                                          int64_t n_tokens, int64_t n_cap, int hidden, int n_experts, int rank,
                                          int world, int top_k, int comm_ctas, void* stream) {
  int rc = dedup_check("ep_dedup_dispatch", world, rank, n_experts, top_k, hidden, n_cap);
  if (rc) return rc;
  if (n_tokens < 0 || n_tokens > n_cap) return fail(BIBO_ERR_ARG, "ep_dedup_dispatch: %lld tokens, n_cap %lld",
                                                    (long long)n_tokens, (long long)n_cap);
  if (n_tokens > 0 && (!x || !topk_idx || !topk_w || !aligned16(x)))
    return fail(BIBO_ERR_ARG, "ep_dedup_dispatch: null or unaligned input");
  PeerPtrs xu = {}, mi = {}, mw = {};
  if ((rc = fill_peers("ep_dedup_dispatch", xu_peers, world, &xu))) return rc;
  // without record tables only the rows travel: the caller sends the routing records as two block copies per
  // peer (bibo_moe_ep_copy_to_peers + bibo_moe_ep_localize) instead of 2 * world small remote stores per token
  const int records = midx_peers != nullptr && mw_peers != nullptr;
  if (records) {
    if ((rc = fill_peers("ep_dedup_dispatch", midx_peers, world, &mi))) return rc;
    if ((rc = fill_peers("ep_dedup_dispatch", mw_peers, world, &mw))) return rc;
  }
  dedup_set_carveouts();
  ep_dedup_dispatch_kernel<<<exchange_grid(n_cap, comm_ctas), exchange_block(comm_ctas), exchange_smem(comm_ctas),
                             static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(x), topk_idx, topk_w, xu, mi, mw, n_tokens, n_cap, hidden * 2, n_experts, rank, world,
      top_k, records);
  BIBO_CHECK_LAUNCH("ep_dedup_dispatch_kernel");
  return BIBO_OK;
}

extern "C" int64_t bibo_moe_ep_dedup_rows_cap(int world, int64_t n_cap, int top_k, int n_experts) {
  return rows_cap((int64_t)world * n_cap, top_k, n_experts / std::max(world, 1));
}
extern "C" int64_t bibo_moe_ep_dedup_plan_words(int world, int64_t n_cap, int top_k, int n_experts) {
  const int el = n_experts / std::max(world, 1);
  return plan_words((int64_t)world * n_cap, top_k, el, el);
}

// owner, first half: the caller-routed single-GPU chain over the virtual tokens and this rank's experts
static int dedup_owner_experts(const bibo_moe_ep_dedup_owner_args* a, void* stream) {
  int rc = dedup_check("ep_dedup_owner", a->world, a->rank, a->n_experts, a->top_k, a->hidden, a->n_cap);
  if (rc) return rc;
  if (!a->xu || !a->midx || !a->mw || !a->gate_up_proj || !a->down_proj || !a->theta || !a->slot_rank ||
      !a->block_counts || !a->plan || !a->slot_row || !a->row_token || !a->xp || !a->h || !a->y)
    return fail(BIBO_ERR_ARG, "ep_dedup_owner: null pointer");
  const int el = a->n_experts / a->world;
  const int64_t nv = (int64_t)a->world * a->n_cap;
  if (!gemm1_tc_supported(a->hidden, a->inter, BIBO_BF16) || !gemm2_tc_supported(a->hidden, a->inter, BIBO_BF16))
    return fail(BIBO_ERR_UNSUPPORTED, "ep_dedup_owner: hidden=%d inter=%d is outside the tensor-core kernels",
                a->hidden, a->inter);
  dedup_set_carveouts();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t* status = a->plan + PLAN_STATUS;
  if ((rc = bibo_moe_route_from_indices(a->midx, nv, el, a->top_k, a->slot_rank, a->block_counts, status, stream))) return rc;
  if ((rc = bibo_moe_plan(a->block_counts, nv, a->top_k, el, el, a->plan, stream))) return rc;
  if ((rc = bibo_moe_permute_fwd(a->xu, a->midx, a->slot_rank, a->plan, nv, a->hidden, el, el, a->top_k, BIBO_BF16, 0,
                                 a->xp, a->slot_row, a->row_token, stream)))
    return rc;
  PlanView pv = local_plan_view(a->plan, nv, a->top_k, el, el);
  pv.max_ctas = a->max_ctas;
  if ((rc = gemm1_tc_launch(a->xp, a->gate_up_proj, a->theta, pv, a->hidden, a->inter, el, a->h, nullptr, nullptr, st)))
    return rc;
  return gemm2_tc_launch(a->h, a->down_proj, pv, a->hidden, a->inter, el, a->y, st);
}

// owner, second half: one partial row per virtual token with local slots, stored into its home rank's buffer
static int dedup_owner_partial(const bibo_moe_ep_dedup_owner_args* a, void* stream) {
  PeerPtrs part = {};
  int rc = fill_peers("ep_dedup_owner", a->part_peers, a->world, &part);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t nv = (int64_t)a->world * a->n_cap;
  const unsigned grid = exchange_grid(nv, a->comm_ctas);
#define BIBO_DPART(KK)                                                                                             \
  case KK:                                                                                                         \
    ep_dedup_partial_kernel<KK><<<grid, exchange_block(a->comm_ctas), exchange_smem(a->comm_ctas), st>>>(                              \
        static_cast<const __nv_bfloat16*>(a->y), a->slot_row, a->mw, part, a->plan, nv, a->n_cap, a->hidden, a->rank); \
    break;
  switch (a->top_k) {
    BIBO_DPART(1) BIBO_DPART(2) BIBO_DPART(3) BIBO_DPART(4) BIBO_DPART(5) BIBO_DPART(6) BIBO_DPART(7) BIBO_DPART(8)
    default: return fail(BIBO_ERR_UNSUPPORTED, "ep_dedup_owner: top_k=%d", a->top_k);
  }
#undef BIBO_DPART
  BIBO_CHECK_LAUNCH("ep_dedup_partial_kernel");
  return BIBO_OK;
}

extern "C" int bibo_moe_ep_dedup_owner(const bibo_moe_ep_dedup_owner_args* a, void* stream) {
  if (!a) return fail(BIBO_ERR_ARG, "ep_dedup_owner: null args");
  const int rc = dedup_owner_experts(a, stream);
  return rc ? rc : dedup_owner_partial(a, stream);
}
// the two halves on their own, for a caller that keeps the tensor-core work of one token slice and the
// NVLink work of another on different streams
extern "C" int bibo_moe_ep_dedup_experts(const bibo_moe_ep_dedup_owner_args* a, void* stream) {
  if (!a) return fail(BIBO_ERR_ARG, "ep_dedup_experts: null args");
  return dedup_owner_experts(a, stream);
}
extern "C" int bibo_moe_ep_dedup_partial(const bibo_moe_ep_dedup_owner_args* a, void* stream) {
  if (!a) return fail(BIBO_ERR_ARG, "ep_dedup_partial: null args");
  const int rc = dedup_check("ep_dedup_partial", a->world, a->rank, a->n_experts, a->top_k, a->hidden, a->n_cap);
  if (rc) return rc;
  if (!a->y || !a->slot_row || !a->mw || !a->plan) return fail(BIBO_ERR_ARG, "ep_dedup_partial: null pointer");
  dedup_set_carveouts();
  return dedup_owner_partial(a, stream);
}

// Rows of a local staging buffer [world*n_cap, H] (what bibo_moe_ep_dedup_partial wrote when it was given a
// table that points every other home rank into that buffer) to the home ranks' `part` buffers.
extern "C" int bibo_moe_ep_dedup_push(const void* stage, const int32_t* midx, void* const* part_peers,
                                      const int32_t* plan, int64_t n_cap, int hidden, int top_k, int rank, int world,
                                      int comm_ctas, void* stream) {
  int rc = dedup_check("ep_dedup_push", world, rank, world, top_k, hidden, n_cap);
  if (rc) return rc;
  if (world == 1) return BIBO_OK;
  if (!stage || !midx || !plan || !aligned16(stage)) return fail(BIBO_ERR_ARG, "ep_dedup_push: null or unaligned pointer");
  PeerPtrs part = {};
  if ((rc = fill_peers("ep_dedup_push", part_peers, world, &part))) return rc;
  dedup_set_carveouts();
  const int64_t nv = (int64_t)world * n_cap;
  ep_dedup_push_kernel<<<exchange_grid(nv - n_cap, comm_ctas), exchange_block(comm_ctas), exchange_smem(comm_ctas),
                         static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t*>(stage), midx, part, plan, nv,
                                                              n_cap, hidden * 2, top_k, rank);
  BIBO_CHECK_LAUNCH("ep_dedup_push_kernel");
  return BIBO_OK;
}

extern "C" int bibo_moe_ep_dedup_final(const void* part, const int32_t* topk_idx, const int32_t* status,
                                       int64_t n_tokens, int64_t n_cap, int hidden, int n_experts, int world,
                                       int top_k, int comm_ctas, void* out, void* stream) {
  int rc = dedup_check("ep_dedup_final", world, 0, n_experts, top_k, hidden, n_cap);
  if (rc) return rc;
  if (n_tokens <= 0) return BIBO_OK;
  if (!part || !topk_idx || !status || !out || !aligned16(part) || !aligned16(out))
    return fail(BIBO_ERR_ARG, "ep_dedup_final: null or unaligned pointer");
  dedup_set_carveouts();
  const dim3 grid(exchange_grid(n_tokens, comm_ctas)), block(exchange_block(comm_ctas));
  const size_t smem = exchange_smem(comm_ctas);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* pp = static_cast<const __nv_bfloat16*>(part);
  __nv_bfloat16* oo = static_cast<__nv_bfloat16*>(out);
  if (world <= 2)
    ep_dedup_final_kernel<2><<<grid, block, smem, st>>>(pp, topk_idx, status, n_tokens, n_cap, hidden, n_experts, world, top_k, oo);
  else if (world <= 4)
    ep_dedup_final_kernel<4><<<grid, block, smem, st>>>(pp, topk_idx, status, n_tokens, n_cap, hidden, n_experts, world, top_k, oo);
  else
    ep_dedup_final_kernel<8><<<grid, block, smem, st>>>(pp, topk_idx, status, n_tokens, n_cap, hidden, n_experts, world, top_k, oo);
  BIBO_CHECK_LAUNCH("ep_dedup_final_kernel");
  return BIBO_OK;
}

extern "C" int bibo_moe_ep_localize(const int32_t* raw_idx, int64_t n_virtual, int top_k, int n_experts, int rank,
                                    int world, int32_t* midx, void* stream) {
  if (n_virtual <= 0) return BIBO_OK;
  if (!raw_idx || !midx) return fail(BIBO_ERR_ARG, "ep_localize: null pointer");
  if (world < 1 || rank < 0 || rank >= world || n_experts % world != 0 || top_k < 1 || top_k > BIBO_MAX_TOP_K)
    return fail(BIBO_ERR_ARG, "ep_localize: rank %d of %d, %d experts, top_k %d", rank, world, n_experts, top_k);
  const int el = n_experts / world;
  const int64_t slots = n_virtual * top_k;
  ep_localize_kernel<<<(unsigned)((slots + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      raw_idx, slots, rank * el, el, midx);
  BIBO_CHECK_LAUNCH("ep_localize_kernel");
  return BIBO_OK;
}

// One block of bytes from this rank to the same place in every rank's buffer (an all-gather leg), or from a
// per-destination place of a local buffer to this rank's place in every rank's buffer (an all-to-all leg), as
// asynchronous copies on the copy engines: dst_peers[d] + dst_offset  <-  src + d * src_stride, `bytes` each,
// for d = rank+1, rank+2, ... (every rank starts with another peer), the own rank last and only with
// include_self.  No kernel, no SM: the copies run beside whatever the SMs are doing.
extern "C" int bibo_moe_ep_copy_to_peers(void* const* dst_peers, int64_t dst_offset, const void* src,
                                         int64_t src_stride, int64_t bytes, int rank, int world, int include_self,
                                         void* stream) {
  if (!dst_peers || !src) return fail(BIBO_ERR_ARG, "ep_copy_to_peers: null pointer");
  if (world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world || bytes < 0 || dst_offset < 0)
    return fail(BIBO_ERR_ARG, "ep_copy_to_peers: rank %d of %d, %lld bytes", rank, world, (long long)bytes);
  if (bytes == 0) return BIBO_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int i = 1; i <= world; ++i) {
    const int d = (rank + i) % world;
    if (d == rank && !include_self) continue;
    if (!dst_peers[d]) return fail(BIBO_ERR_ARG, "ep_copy_to_peers: peer %d has no buffer", d);
    BIBO_CUDA(cudaMemcpyAsync(static_cast<char*>(dst_peers[d]) + dst_offset,
                              static_cast<const char*>(src) + (int64_t)d * src_stride, (size_t)bytes,
                              cudaMemcpyDefault, st));
  }
  return BIBO_OK;
}

// The whole forward of one token slice: router -> dispatch -> barrier -> owner chain -> barrier -> final sum.
// Uses barrier epochs epoch_base+1 and epoch_base+2 on flags_peers.
extern "C" int bibo_moe_ep_dedup_forward(const bibo_moe_ep_dedup_args* a, void* stream) {
  if (!a) return fail(BIBO_ERR_ARG, "ep_dedup_forward: null args");
  const bibo_moe_ep_dedup_owner_args* o = &a->owner;
  int rc = dedup_check("ep_dedup_forward", o->world, o->rank, o->n_experts, o->top_k, o->hidden, o->n_cap);
  if (rc) return rc;
  if (!a->flags_peers || !a->xu_peers || !a->midx_peers || !a->mw_peers || !a->part_local || !a->topk_idx || !a->topk_w ||
      !a->slot_rank_home || !a->block_counts_home || !a->out)
    return fail(BIBO_ERR_ARG, "ep_dedup_forward: null pointer");
  if (a->trace && !a->trace->block_sums) return fail(BIBO_ERR_ARG, "ep_dedup_forward: trace without block_sums");
  int32_t* status = o->plan + PLAN_STATUS;
  void* const* ev = a->marks;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define BIBO_MARK(i)                                                                 \
  do {                                                                               \
    if (ev) BIBO_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev[i]), st));         \
  } while (0)
  BIBO_MARK(0);
  if (a->n_tokens > 0) {
    rc = bibo_moe_router_fwd_trace(a->x, a->w_router, a->bias, nullptr, a->n_tokens, o->hidden, o->n_experts, o->top_k,
                                   a->norm_mode, a->scale, BIBO_BF16, nullptr, a->topk_idx, a->topk_w, a->slot_rank_home,
                                   a->block_counts_home, status, a->trace ? a->trace->block_sums : nullptr, stream);
    if (rc) return rc;
  }
  BIBO_MARK(1);
  rc = bibo_moe_ep_dedup_dispatch(a->x, a->topk_idx, a->topk_w, a->xu_peers, a->midx_peers, a->mw_peers, a->n_tokens,
                                  o->n_cap, o->hidden, o->n_experts, o->rank, o->world, o->top_k, o->comm_ctas, stream);
  if (rc) return rc;
  BIBO_MARK(2);
  if ((rc = bibo_moe_ep_barrier(a->flags_peers, o->rank, o->world, a->epoch_base + 1, status, stream))) return rc;
  BIBO_MARK(3);
  if ((rc = dedup_owner_experts(o, stream))) return rc;
  BIBO_MARK(4);
  if ((rc = dedup_owner_partial(o, stream))) return rc;
  BIBO_MARK(5);
  if ((rc = bibo_moe_ep_barrier(a->flags_peers, o->rank, o->world, a->epoch_base + 2, status, stream))) return rc;
  BIBO_MARK(6);
  rc = bibo_moe_ep_dedup_final(a->part_local, a->topk_idx, status, a->n_tokens, o->n_cap, o->hidden, o->n_experts,
                               o->world, o->top_k, o->comm_ctas, a->out, stream);
  if (rc) return rc;
  BIBO_MARK(7);
#undef BIBO_MARK
  return BIBO_OK;
}
