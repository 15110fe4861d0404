// Expert-parallel forward: the 64 experts are sharded contiguously over R GPUs of one NVSwitch box
// (rank d owns experts [d*E/R, (d+1)*E/R)), tokens stay data-parallel, the router is replicated.
//
// There is no separate all-to-all pass.  The two exchange steps are fused into the kernels on either
// side of the grouped GEMMs, over peer (NVLink) memory:
//   dispatch = the permute kernel writes each token row straight into the OWNER rank's
//              expert-contiguous receive buffer (16-byte remote stores);
//   combine  = the combine kernel of the token's home rank reads the k result rows straight out of
//              the owner ranks' y buffers (16-byte remote loads).
// Row positions are agreed without host involvement: every rank holds the all-gathered per-rank
// histograms cnt[R][E] and computes every rank's receive layout itself (ep_plan_kernel).
//
// Receive layout of rank d: for local expert le (ascending), for source rank s (ascending): the
// cnt[s][d*EL+le] rows of (le, s), padded to a multiple of BIBO_TILE_M, so a row tile never mixes
// two (expert, source) groups; tiles carry the LOCAL expert index for the weight lookup.
// Cross-rank ordering (all stores landed before the GEMMs start; all y written before the combine
// reads) is provided by the caller with device-side barriers between the launches.
#include <algorithm>

#include "ep_common.cuh"

namespace bibo {

// One block, E threads.  Thread d < R scans destination d's layout.
__global__ void __launch_bounds__(BIBO_MAX_EXPERTS)
ep_plan_kernel(const int32_t* __restrict__ cnt_all, int rank, int world, int n_experts, int rows_cap_recv,
               int source_major, int32_t* __restrict__ plan) {
  const int el = n_experts / world;
  int32_t* send_base = plan + ep_off_send_base();
  int32_t* recv_off = plan + ep_off_recv_off(n_experts);
  int32_t* recv_cnt = plan + ep_off_recv_cnt(n_experts);
  int4* tiles = reinterpret_cast<int4*>(plan + ep_off_tiles(n_experts));
  int2* pairs = reinterpret_cast<int2*>(plan + ep_off_pairs(n_experts, rows_cap_recv));
  __shared__ int s_pair_off[BIBO_MAX_EXPERTS + 1];
  __shared__ int s_off[BIBO_MAX_EXPERTS + 1];
  __shared__ int s_cnt[BIBO_MAX_EXPERTS];
  __shared__ int s_over;
  const int tid = threadIdx.x;
  if (tid == 0) s_over = 0;
  __syncthreads();
  if (tid < world) {
    const int d = tid;
    int run = 0;
    // expert-major: groups (le, s) in the order le, s; source-major: in the order s, le, so that all rows
    // from one source rank form one contiguous block (what a block copy between ranks needs)
    for (int i = 0; i < n_experts; ++i) {
      const int le = source_major ? i % el : i / world, s = source_major ? i / el : i % world;
      const int c = cnt_all[s * n_experts + d * el + le];
      if (s == rank) send_base[d * el + le] = run;
      if (d == rank) { s_off[le * world + s] = run; s_cnt[le * world + s] = c; }
      run += (c + BIBO_TILE_M - 1) / BIBO_TILE_M * BIBO_TILE_M;
    }
    if (run > rows_cap_recv) s_over = 1;   // some rank's buffer would overflow: everyone learns it
    if (d == rank) s_off[n_experts] = run;
  }
  __syncthreads();
  const bool over = s_over != 0;
  // tiles of one local expert are paired across its source groups (two tiles of a pair only have to
  // share the expert), so at most one pair per expert is left with a single tile
  if (tid == 0) {
    const int rows = over ? 0 : s_off[n_experts];
    int pacc = 0;
    for (int le = 0; le < el; ++le) {
      int nt = 0;
      for (int s = 0; s < world; ++s) nt += (s_cnt[le * world + s] + BIBO_TILE_M - 1) / BIBO_TILE_M;
      s_pair_off[le] = pacc;
      pacc += (nt + 1) / 2;
    }
    plan[PLAN_N_TILES] = rows / BIBO_TILE_M;
    plan[PLAN_ROWS_USED] = rows;
    plan[PLAN_N_PAIRS] = over ? 0 : pacc;
    if (over) atomicMax(&plan[PLAN_STATUS], 4);
  }
  __syncthreads();
  if (tid <= n_experts) recv_off[tid] = s_off[tid];
  if (tid < el) {   // row range of local expert tid: its `world` groups are contiguous (expert-major only)
    const bool em = !source_major && !over;
    plan[ep_off_le_off(n_experts) + tid] = source_major ? 0 : s_off[tid * world];
    plan[ep_off_le_span(n_experts) + tid] =
        em ? (tid + 1 < el ? s_off[(tid + 1) * world] : s_off[n_experts]) - s_off[tid * world] : 0;
    if (tid == el - 1) plan[ep_off_le_off(n_experts) + el] = s_off[n_experts];
  }
  if (tid < n_experts) {
    recv_cnt[tid] = s_cnt[tid];
    if (!over) {
      const int row0 = s_off[tid], cnt = s_cnt[tid], le = tid / world, src = tid % world;
      const int t0 = row0 / BIBO_TILE_M, nt = (cnt + BIBO_TILE_M - 1) / BIBO_TILE_M;
      for (int i = 0; i < nt; ++i)
        tiles[t0 + i] = make_int4(le, row0 + i * BIBO_TILE_M, min(BIBO_TILE_M, cnt - i * BIBO_TILE_M), src);
    }
  }
  if (tid < el && !over) {
    int idx = 0, prev = -1;
    for (int s = 0; s < world; ++s) {
      const int g = tid * world + s;
      const int t0 = s_off[g] / BIBO_TILE_M, nt = (s_cnt[g] + BIBO_TILE_M - 1) / BIBO_TILE_M;
      for (int i = 0; i < nt; ++i, ++idx) {
        if (idx & 1) pairs[s_pair_off[tid] + idx / 2] = make_int2(prev, t0 + i);
        else prev = t0 + i;
      }
    }
    if (idx & 1) pairs[s_pair_off[tid] + idx / 2] = make_int2(prev, -1);
  }
}

constexpr int EPW = 8;

// Dispatch: warp per token; x[t] is read once and written to the k owner ranks' receive buffers.
// slot_row[t][j] = owner * rows_cap_recv + row (the address the combine reads back from).
__global__ void __launch_bounds__(EPW * 32)
ep_dispatch_kernel(const uint8_t* __restrict__ x, const int32_t* __restrict__ topk_idx,
                   const int32_t* __restrict__ slot_rank, const int32_t* __restrict__ local_plan,
                   const int32_t* __restrict__ ep_plan, PeerPtrs xp_peers, int64_t n_tokens, int row_bytes,
                   int n_experts, int world, int top_k, int rows_cap_recv, int32_t* __restrict__ slot_row,
                   int32_t* __restrict__ row_token) {
  const int lane = threadIdx.x & 31;
  if (ep_plan[PLAN_STATUS] != 0) return;   // overflow or earlier error: write nothing
  const int el = n_experts / world;
  const int32_t* block_base = local_plan + plan_off_block_base(n_experts, n_experts);
  const int32_t* send_base = ep_plan + ep_off_send_base();
  // grid-stride over tokens: the grid may be capped to a few CTAs per SM subset (see comm_ctas)
  for (int64_t w = (int64_t)blockIdx.x * EPW + (threadIdx.x >> 5); w < n_tokens; w += (int64_t)gridDim.x * EPW) {
  int my_row = -1, my_owner = 0;
  if (lane < top_k) {
    const int e = topk_idx[w * top_k + lane];
    const int64_t b = w / BIBO_ROUTER_BLOCK_TOKENS;
    my_owner = e / el;
    my_row = send_base[e] + block_base[b * n_experts + e] + slot_rank[w * top_k + lane];
    slot_row[w * top_k + lane] = my_owner * rows_cap_recv + my_row;
    if (row_token != nullptr)   // token of each row of the LOCAL expert-sorted order (router weight gradient)
      row_token[local_plan[plan_off_expert_off(n_experts) + e] + block_base[b * n_experts + e] +
                slot_rank[w * top_k + lane]] = (int32_t)w;
  }
  uint4* dst[BIBO_MAX_TOP_K];
#pragma unroll
  for (int j = 0; j < BIBO_MAX_TOP_K; ++j) {
    const int r = __shfl_sync(0xffffffffu, my_row, j);
    const int o = __shfl_sync(0xffffffffu, my_owner, j);
    dst[j] = reinterpret_cast<uint4*>(static_cast<uint8_t*>(xp_peers.p[o]) + (int64_t)r * row_bytes);
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + w * row_bytes);
  const int chunks = row_bytes / 16;
  for (int c = lane; c < chunks; c += 32) {
    const uint4 v = __ldg(src + c);
#pragma unroll
    for (int j = 0; j < BIBO_MAX_TOP_K; ++j)
      if (j < top_k) dst[j][c] = v;
  }
  }
}

__device__ __forceinline__ void fma_bf16x8(const uint4& v, float w, float* acc) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] = fmaf(__uint_as_float(u[i] << 16), w, acc[2 * i]);
    acc[2 * i + 1] = fmaf(__uint_as_float(u[i] & 0xffff0000u), w, acc[2 * i + 1]);
  }
}

// Combine: warp per token; the k rows are read from the owner ranks' y buffers (peer loads), summed
// in slot order (ascending expert) in fp32, cast once.
template <int K>
__global__ void __launch_bounds__(EPW * 32, 4)
ep_combine_kernel(PeerPtrs y_peers, const int32_t* __restrict__ slot_row, const float* __restrict__ topk_w,
                  const int32_t* __restrict__ ep_plan, int64_t n_tokens, int hidden, int rows_cap_recv,
                  __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  if (ep_plan[PLAN_STATUS] != 0) return;
  for (int64_t t = (int64_t)blockIdx.x * EPW + (threadIdx.x >> 5); t < n_tokens; t += (int64_t)gridDim.x * EPW) {
  int my_g = 0;
  float my_w = 0.f;
  if (lane < K) { my_g = slot_row[t * K + lane]; my_w = topk_w[t * K + lane]; }
  const uint4* src[K];
  float ws[K];
#pragma unroll
  for (int j = 0; j < K; ++j) {
    const int g = __shfl_sync(0xffffffffu, my_g, j);
    ws[j] = __shfl_sync(0xffffffffu, my_w, j);
    const int o = g / rows_cap_recv, r = g % rows_cap_recv;
    src[j] = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(y_peers.p[o]) + (int64_t)r * hidden);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + t * hidden);
  const int chunks = hidden / 8;
  int c = lane;
  for (; c + 32 < chunks; c += 64) {
    uint4 v0[K], v1[K];
#pragma unroll
    for (int j = 0; j < K; ++j) { v0[j] = src[j][c]; v1[j] = src[j][c + 32]; }
    float a0[8], a1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a0[i] = a1[i] = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) { fma_bf16x8(v0[j], ws[j], a0); fma_bf16x8(v1[j], ws[j], a1); }
    uint4 o0, o1;
    __nv_bfloat162* h0 = reinterpret_cast<__nv_bfloat162*>(&o0);
    __nv_bfloat162* h1 = reinterpret_cast<__nv_bfloat162*>(&o1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      h0[i] = __floats2bfloat162_rn(a0[2 * i], a0[2 * i + 1]);
      h1[i] = __floats2bfloat162_rn(a1[2 * i], a1[2 * i + 1]);
    }
    dst[c] = o0;
    dst[c + 32] = o1;
  }
  for (; c < chunks; c += 32) {
    uint4 v0[K];
#pragma unroll
    for (int j = 0; j < K; ++j) v0[j] = src[j][c];
    float a0[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a0[i] = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) fma_bf16x8(v0[j], ws[j], a0);
    uint4 o0;
    __nv_bfloat162* h0 = reinterpret_cast<__nv_bfloat162*>(&o0);
#pragma unroll
    for (int i = 0; i < 4; ++i) h0[i] = __floats2bfloat162_rn(a0[2 * i], a0[2 * i + 1]);
    dst[c] = o0;
  }
  }
}

// Zero the rows of every tile that lie beyond its valid rows (block per tile).
__global__ void __launch_bounds__(128)
ep_zero_tile_padding_kernel(uint8_t* __restrict__ buf, const int32_t* __restrict__ plan, int64_t tiles_off,
                            int row_bytes) {
  if ((int)blockIdx.x >= plan[PLAN_N_TILES]) return;
  const int4 t = reinterpret_cast<const int4*>(plan + tiles_off)[blockIdx.x];
  const int chunks = row_bytes / 16;
  for (int r = t.z + (threadIdx.x >> 5); r < BIBO_TILE_M; r += 4) {
    uint4* dst = reinterpret_cast<uint4*>(buf + (int64_t)(t.y + r) * row_bytes);
    for (int c = threadIdx.x & 31; c < chunks; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
  }
}

// Every rank publishes its histogram row into every peer's cnt_all[rank][:] (peer stores); a
// barrier after this kernel makes all rows visible everywhere, replacing a library all-gather.
__global__ void __launch_bounds__(BIBO_MAX_EXPERTS)
ep_share_counts_kernel(const int32_t* __restrict__ counts, PeerPtrs cnt_peers, int rank, int world, int n_experts) {
  const int e = threadIdx.x;
  if (e >= n_experts) return;
  const int32_t c = counts[e];
  for (int p = 0; p < world; ++p) static_cast<int32_t*>(cnt_peers.p[p])[rank * n_experts + e] = c;
}

__global__ void ep_barrier_kernel(PeerPtrs flags, int rank, int world, int epoch, uint32_t max_polls,
                                  int32_t* status);

int ep_share_counts_launch(const int32_t* counts, void* const* cnt_peers, int rank, int world, int n_experts,
                           cudaStream_t st) {
  PeerPtrs cp = {};
  for (int i = 0; i < world; ++i) {
    if (!cnt_peers[i]) return fail(BIBO_ERR_ARG, "peer %d has no histogram buffer", i);
    cp.p[i] = cnt_peers[i];
  }
  ep_share_counts_kernel<<<1, BIBO_MAX_EXPERTS, 0, st>>>(counts, cp, rank, world, n_experts);
  BIBO_CHECK_LAUNCH("ep_share_counts_kernel");
  return BIBO_OK;
}

// gemm_tc.cu
int gemm1_tc_supported(int hidden, int inter, int dtype);
int gemm1_gather_supported(int hidden, int inter, int dtype);
int gemm1_tc_launch(const void* xp, const void* gate_up_proj, const float* theta, const PlanView& pv, int hidden,
                    int inter, int n_weight_experts, void* h, void* gate_up_out, float* rnorm_out, cudaStream_t st,
                    const void* gather_src = nullptr, const int32_t* row_src = nullptr, int zero_padding = 0);
int gemm2_tc_supported(int hidden, int inter, int dtype);
int gemm2_tc_launch(const void* h, const void* down_proj, const PlanView& pv, int hidden, int inter,
                    int n_weight_experts, void* y, cudaStream_t st);

}  // namespace bibo

using namespace bibo;

// The grouped GEMMs run with the shared-memory carve-out at its maximum.  An SM can only change its
// carve-out while it is idle, so the small kernels of this path ask for the same carve-out: otherwise a
// dispatch / combine kernel of one token slice, resident on every SM, would keep the GEMM kernel of
// another slice from starting and the two would serialise instead of overlapping.
template <typename Kern>
static void prefer_max_smem(Kern kern) {
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}
static void ep_set_carveouts() {
  static DeviceOnce once;
  once.get([](int*) {
  prefer_max_smem(ep_plan_kernel);
  prefer_max_smem(ep_dispatch_kernel);
  prefer_max_smem(ep_barrier_kernel);
  prefer_max_smem(ep_share_counts_kernel);
  prefer_max_smem(ep_combine_kernel<1>); prefer_max_smem(ep_combine_kernel<2>); prefer_max_smem(ep_combine_kernel<3>);
  prefer_max_smem(ep_combine_kernel<4>); prefer_max_smem(ep_combine_kernel<5>); prefer_max_smem(ep_combine_kernel<6>);
  prefer_max_smem(ep_combine_kernel<7>); prefer_max_smem(ep_combine_kernel<8>);
    return (int)BIBO_OK;
  });
}

static int ep_check(const char* who, int world, int rank, int n_experts, int64_t rows_cap_recv) {
  if (world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world)
    return fail(BIBO_ERR_ARG, "%s: rank %d of %d (max %d ranks)", who, rank, world, EP_MAX_RANKS);
  if (n_experts < world || n_experts > BIBO_MAX_EXPERTS || n_experts % world != 0)
    return fail(BIBO_ERR_UNSUPPORTED, "%s: %d experts do not shard evenly over %d ranks", who, n_experts, world);
  if (rows_cap_recv <= 0 || rows_cap_recv % BIBO_TILE_M != 0 || rows_cap_recv * world > 0x7fffffffLL)
    return fail(BIBO_ERR_ARG, "%s: rows_cap_recv=%lld must be a positive multiple of %d", who,
                (long long)rows_cap_recv, BIBO_TILE_M);
  return BIBO_OK;
}

extern "C" int64_t bibo_moe_ep_plan_words(int n_experts, int64_t rows_cap_recv) {
  return ep_plan_words(n_experts, rows_cap_recv);
}
extern "C" int64_t bibo_moe_ep_plan_off(int which, int n_experts) {
  switch (which) {
    case 0: return ep_off_send_base();
    case 1: return ep_off_recv_off(n_experts);
    case 2: return ep_off_recv_cnt(n_experts);
    case 4: return ep_off_le_off(n_experts);
    case 5: return ep_off_le_span(n_experts);
    default: return ep_off_tiles(n_experts);
  }
}

extern "C" int bibo_moe_ep_plan_layout(const int32_t* cnt_all, int rank, int world, int n_experts,
                                       int64_t rows_cap_recv, int source_major, int32_t* ep_plan, void* stream) {
  int rc = ep_check("ep_plan", world, rank, n_experts, rows_cap_recv);
  if (rc) return rc;
  if (!cnt_all || !ep_plan) return fail(BIBO_ERR_ARG, "ep_plan: null pointer");
  ep_set_carveouts();
  ep_plan_kernel<<<1, BIBO_MAX_EXPERTS, 0, static_cast<cudaStream_t>(stream)>>>(
      cnt_all, rank, world, n_experts, (int)rows_cap_recv, source_major != 0, ep_plan);
  BIBO_CHECK_LAUNCH("ep_plan_kernel");
  return BIBO_OK;
}

extern "C" int bibo_moe_ep_plan(const int32_t* cnt_all, int rank, int world, int n_experts, int64_t rows_cap_recv,
                                int32_t* ep_plan, void* stream) {
  return bibo_moe_ep_plan_layout(cnt_all, rank, world, n_experts, rows_cap_recv, 0, ep_plan, stream);
}

extern "C" int bibo_moe_ep_dispatch(const void* x, const int32_t* topk_idx, const int32_t* slot_rank,
                                    const int32_t* local_plan, const int32_t* ep_plan, void* const* xp_peers,
                                    int64_t n_tokens, int hidden, int n_experts, int rank, int world, int top_k,
                                    int64_t rows_cap_recv, int comm_ctas, int32_t* slot_row, int32_t* row_token,
                                    void* stream) {
  int rc = ep_check("ep_dispatch", world, rank, n_experts, rows_cap_recv);
  if (rc) return rc;
  if (n_tokens <= 0) return BIBO_OK;
  if (!x || !topk_idx || !slot_rank || !local_plan || !ep_plan || !xp_peers || !slot_row)
    return fail(BIBO_ERR_ARG, "ep_dispatch: null pointer");
  if (top_k < 1 || top_k > BIBO_MAX_TOP_K) return fail(BIBO_ERR_UNSUPPORTED, "ep_dispatch: top_k=%d", top_k);
  const int row_bytes = hidden * 2;
  if (row_bytes % 16 != 0) return fail(BIBO_ERR_UNSUPPORTED, "ep_dispatch: hidden=%d", hidden);
  PeerPtrs pp = {};
  for (int i = 0; i < world; ++i) {
    if (!xp_peers[i] || !aligned16(xp_peers[i])) return fail(BIBO_ERR_ALIGN, "ep_dispatch: peer buffer %d", i);
    pp.p[i] = xp_peers[i];
  }
  int64_t blocks = (n_tokens + EPW - 1) / EPW;
  if (comm_ctas > 0) blocks = std::min<int64_t>(blocks, comm_ctas);
  dim3 grid((unsigned)blocks);
  ep_dispatch_kernel<<<grid, EPW * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)x, topk_idx, slot_rank, local_plan, ep_plan, pp, n_tokens, row_bytes, n_experts, world, top_k,
      (int)rows_cap_recv, slot_row, row_token);
  BIBO_CHECK_LAUNCH("ep_dispatch_kernel");
  return BIBO_OK;
}

extern "C" int bibo_moe_ep_experts(const void* xp_recv, const void* gate_up_proj, const void* down_proj,
                                   const float* theta, const int32_t* ep_plan, int hidden, int inter, int n_experts,
                                   int world, int64_t rows_cap_recv, int max_ctas, void* h, void* y_recv,
                                   void* gate_up_out, float* rnorm_out, int zero_padding, void* stream) {
  int rc = ep_check("ep_experts", world, 0, n_experts, rows_cap_recv);
  if (rc) return rc;
  if (!xp_recv || !gate_up_proj || !down_proj || !theta || !ep_plan || !h || !y_recv)
    return fail(BIBO_ERR_ARG, "ep_experts: null pointer");
  if (!gemm1_tc_supported(hidden, inter, BIBO_BF16) || !gemm2_tc_supported(hidden, inter, BIBO_BF16))
    return fail(BIBO_ERR_UNSUPPORTED, "ep_experts: hidden=%d inter=%d is outside the tensor-core kernels", hidden, inter);
  const PlanView pv = ep_plan_view(ep_plan, n_experts, rows_cap_recv, max_ctas);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int el = n_experts / world;
  if (zero_padding) {   // training: rows between a group's last token and its tile boundary become zero
    ep_zero_tile_padding_kernel<<<(unsigned)pv.tiles_cap, 128, 0, st>>>(
        static_cast<uint8_t*>(const_cast<void*>(xp_recv)), ep_plan, pv.tiles_off, hidden * 2);
    BIBO_CHECK_LAUNCH("ep_zero_tile_padding_kernel");
  }
  rc = gemm1_tc_launch(xp_recv, gate_up_proj, theta, pv, hidden, inter, el, h, gate_up_out, rnorm_out, st);
  if (rc) return rc;
  return gemm2_tc_launch(h, down_proj, pv, hidden, inter, el, y_recv, st);
}

extern "C" int bibo_moe_ep_combine(void* const* y_peers, const int32_t* slot_row, const float* topk_w,
                                   const int32_t* ep_plan, int64_t n_tokens, int hidden, int world, int top_k,
                                   int64_t rows_cap_recv, int comm_ctas, void* out, void* stream) {
  if (n_tokens <= 0) return BIBO_OK;
  if (!y_peers || !slot_row || !topk_w || !ep_plan || !out) return fail(BIBO_ERR_ARG, "ep_combine: null pointer");
  if (world < 1 || world > EP_MAX_RANKS) return fail(BIBO_ERR_ARG, "ep_combine: world=%d", world);
  if (hidden % 8 != 0) return fail(BIBO_ERR_UNSUPPORTED, "ep_combine: hidden=%d", hidden);
  PeerPtrs pp = {};
  for (int i = 0; i < world; ++i) {
    if (!y_peers[i] || !aligned16(y_peers[i])) return fail(BIBO_ERR_ALIGN, "ep_combine: peer buffer %d", i);
    pp.p[i] = y_peers[i];
  }
  int64_t blocks = (n_tokens + EPW - 1) / EPW;
  if (comm_ctas > 0) blocks = std::min<int64_t>(blocks, comm_ctas);
  dim3 grid((unsigned)blocks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define BIBO_EPC(KK)                                                                                              \
  case KK:                                                                                                        \
    ep_combine_kernel<KK><<<grid, EPW * 32, 0, st>>>(pp, slot_row, topk_w, ep_plan, n_tokens, hidden,             \
                                                     (int)rows_cap_recv, (__nv_bfloat16*)out);                    \
    break;
  switch (top_k) {
    BIBO_EPC(1) BIBO_EPC(2) BIBO_EPC(3) BIBO_EPC(4) BIBO_EPC(5) BIBO_EPC(6) BIBO_EPC(7) BIBO_EPC(8)
    default: return fail(BIBO_ERR_UNSUPPORTED, "ep_combine: top_k=%d", top_k);
  }
#undef BIBO_EPC
  BIBO_CHECK_LAUNCH("ep_combine_kernel");
  return BIBO_OK;
}

// ---- cross-rank barrier on the stream -------------------------------------------------------------
// flags_peers[r] = rank r's int32[EP_MAX_RANKS] flag array as mapped into this process (zeroed once
// at set-up).  Thread p publishes `epoch` into slot [rank] of peer p (release, system scope: every
// earlier write of this GPU, including the previous kernels' peer stores, is visible first) and then
// waits until slot [p] of its own array reaches `epoch`.  The wait is bounded: after about two
// seconds the kernel gives up, raises the status word to 5 and returns.
namespace bibo {
__global__ void ep_barrier_kernel(PeerPtrs flags, int rank, int world, int epoch, uint32_t max_polls,
                                  int32_t* status) {
  const int p = threadIdx.x;
  if (p >= world) return;
  int* remote = static_cast<int*>(flags.p[p]) + rank;
  int* mine = static_cast<int*>(flags.p[rank]) + p;
  __threadfence_system();
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  for (uint32_t i = 0; i < max_polls; ++i) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v >= epoch) return;
    __nanosleep(400);
  }
  if (status) atomicMax(status, 5);
}
}  // namespace bibo

extern "C" int bibo_moe_ep_barrier(void* const* flags_peers, int rank, int world, int epoch, int32_t* status,
                                   void* stream) {
  return bibo_moe_ep_barrier_bounded(flags_peers, rank, world, epoch, 0, status, stream);
}

extern "C" int bibo_moe_ep_barrier_bounded(void* const* flags_peers, int rank, int world, int epoch,
                                           int64_t max_polls, int32_t* status, void* stream) {
  if (!flags_peers) return fail(BIBO_ERR_ARG, "ep_barrier: null pointer");
  if (max_polls <= 0 || max_polls > (1ll << 22)) max_polls = 1ll << 22;   // about two seconds
  if (world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world)
    return fail(BIBO_ERR_ARG, "ep_barrier: rank %d of %d", rank, world);
  PeerPtrs pp = {};
  for (int i = 0; i < world; ++i) {
    if (!flags_peers[i]) return fail(BIBO_ERR_ARG, "ep_barrier: peer %d has no flag array", i);
    pp.p[i] = flags_peers[i];
  }
  ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pp, rank, world, epoch, (uint32_t)max_polls,
                                                                     status);
  BIBO_CHECK_LAUNCH("ep_barrier_kernel");
  return BIBO_OK;
}

// ---- the whole expert-parallel forward of one token slice as ONE call ---------------------------------
// router -> local plan -> publish histogram to peers -> barrier -> EP plan -> dispatch (peer stores) ->
// barrier -> gate/up + radial + down on received rows -> barrier -> combine (peer loads).
// Uses barrier epochs epoch_base+1 .. epoch_base+3 on `flags_peers`.
extern "C" int bibo_moe_ep_forward(const bibo_moe_ep_args* a, void* stream) {
  if (!a) return fail(BIBO_ERR_ARG, "ep_forward: null args");
  int rc = ep_check("ep_forward", a->world, a->rank, a->n_experts, a->rows_cap_recv);
  if (rc) return rc;
  if (!a->cnt_peers || !a->flags_peers || !a->xp_peers || !a->y_peers || !a->local_plan || !a->ep_plan)
    return fail(BIBO_ERR_ARG, "ep_forward: null peer table / plan");
  ep_set_carveouts();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t* status = a->ep_plan + PLAN_STATUS;
  if (a->trace && !a->trace->block_sums) return fail(BIBO_ERR_ARG, "ep_forward: trace without block_sums");
  rc = bibo_moe_router_fwd_trace(a->x, a->w_router, a->bias, nullptr, a->n_tokens, a->hidden, a->n_experts, a->top_k,
                                 a->norm_mode, a->scale, BIBO_BF16, nullptr, a->topk_idx, a->topk_w, a->slot_rank,
                                 a->block_counts, a->local_plan + PLAN_STATUS, a->trace ? a->trace->block_sums : nullptr,
                                 stream);
  if (rc) return rc;
  rc = bibo_moe_plan_trace(a->block_counts, a->n_tokens, a->top_k, a->n_experts, a->n_experts, a->local_plan, a->trace,
                           stream);
  if (rc) return rc;
  rc = ep_share_counts_launch(a->local_plan + plan_off_counts(), a->cnt_peers, a->rank, a->world, a->n_experts, st);
  if (rc) return rc;
  rc = bibo_moe_ep_barrier(a->flags_peers, a->rank, a->world, a->epoch_base + 1, status, stream);
  if (rc) return rc;
  rc = bibo_moe_ep_plan(static_cast<const int32_t*>(a->cnt_peers[a->rank]), a->rank, a->world, a->n_experts,
                        a->rows_cap_recv, a->ep_plan, stream);
  if (rc) return rc;
  rc = bibo_moe_ep_dispatch(a->x, a->topk_idx, a->slot_rank, a->local_plan, a->ep_plan, a->xp_peers, a->n_tokens,
                            a->hidden, a->n_experts, a->rank, a->world, a->top_k, a->rows_cap_recv, a->comm_ctas,
                            a->slot_row, a->row_token, stream);
  if (rc) return rc;
  rc = bibo_moe_ep_barrier(a->flags_peers, a->rank, a->world, a->epoch_base + 2, status, stream);
  if (rc) return rc;
  rc = bibo_moe_ep_experts(a->xp_peers[a->rank], a->gate_up_proj, a->down_proj, a->theta, a->ep_plan, a->hidden,
                           a->inter, a->n_experts, a->world, a->rows_cap_recv, a->max_ctas, a->h, a->y_peers[a->rank],
                           a->gate_up_recv, a->rnorm_recv, a->gate_up_recv != nullptr, stream);
  if (rc) return rc;
  rc = bibo_moe_ep_barrier(a->flags_peers, a->rank, a->world, a->epoch_base + 3, status, stream);
  if (rc) return rc;
  return bibo_moe_ep_combine(a->y_peers, a->slot_row, a->topk_w, a->ep_plan, a->n_tokens, a->hidden, a->world,
                             a->top_k, a->rows_cap_recv, a->comm_ctas, a->out, stream);
}
