// Layout of the expert-parallel plan buffer and the peer-pointer table, shared by ep.cu and ep_bwd.cu.
#pragma once
#include "common.cuh"

namespace bibo {

constexpr int EP_MAX_RANKS = 8;
struct PeerPtrs { void* p[EP_MAX_RANKS]; };

// EP plan words: [0]=n_tiles [1]=rows used [2]=status (sticky) [3]=n_pairs,
// send_base[E] (row in the owner's buffer where this rank's rows of expert e start),
// recv_off[E+1] and recv_cnt[E] (groups g = le*R + s of this rank),
// le_off[E+1] / le_span[E] (row range of each LOCAL expert: its R groups are contiguous; entries
// beyond E/R are unused), then int4 tiles and int2 tile pairs.
__host__ __device__ inline int64_t ep_off_send_base() { return PLAN_HDR; }
__host__ __device__ inline int64_t ep_off_recv_off(int E) { return PLAN_HDR + E; }
__host__ __device__ inline int64_t ep_off_recv_cnt(int E) { return PLAN_HDR + 2 * E + 1; }
__host__ __device__ inline int64_t ep_off_le_off(int E) { return PLAN_HDR + 3 * E + 1; }
__host__ __device__ inline int64_t ep_off_le_span(int E) { return PLAN_HDR + 4 * E + 2; }
__host__ __device__ inline int64_t ep_off_tiles(int E) { return (PLAN_HDR + 5 * E + 2 + 3) / 4 * 4; }
__host__ __device__ inline int64_t ep_off_pairs(int E, int64_t rows_cap_recv) {
  return ep_off_tiles(E) + rows_cap_recv / BIBO_TILE_M * 4;
}
__host__ __device__ inline int64_t ep_off_scratch(int E, int64_t rows_cap_recv) {
  return ep_off_pairs(E, rows_cap_recv) + rows_cap_recv / BIBO_TILE_M * 2;
}
__host__ __device__ inline int64_t ep_plan_words(int E, int64_t rows_cap_recv) {
  return ep_off_scratch(E, rows_cap_recv) + XG_WORDS + rows_cap_recv / BIBO_TILE_M;
}
inline PlanView ep_plan_view(const int32_t* ep_plan, int n_experts, int64_t rows_cap_recv, int max_ctas) {
  return PlanView{ep_plan, ep_off_tiles(n_experts), ep_off_pairs(n_experts, rows_cap_recv),
                  ep_off_scratch(n_experts, rows_cap_recv), rows_cap_recv / BIBO_TILE_M, rows_cap_recv, max_ctas};
}

}  // namespace bibo
