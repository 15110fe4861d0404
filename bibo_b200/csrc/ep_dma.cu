// Expert-parallel forward with the exchange on the copy engines.
//
// Same sharding as ep.cu (rank d owns experts [d*E/R, (d+1)*E/R), tokens stay home, router replicated),
// but the rows do not travel through SM kernels.  The home rank sorts its tokens by expert exactly as
// the single-GPU chain does (permute into xp_send): the experts of owner d then occupy ONE contiguous
// row range, which one asynchronous peer copy moves into owner d's receive buffer.  The receive buffer
// is laid out source-major (all rows of source 0, then source 1, ...), so the results of source s are
// again one contiguous range of the owner's y buffer and one peer copy returns them, in the home
// rank's own expert-sorted layout, where the ordinary combine kernel finishes.  Copies run on the
// copy engines: with token slices on separate streams they overlap another slice's GEMMs without
// taking SMs from them.
//
// The copy sizes depend on the routing, so the host reads the R x E histogram table once per call
// (2 KB, one stream synchronisation after the router).  Everything else is stream-ordered; the three
// cross-rank barriers are the flag kernel of ep.cu.
#include <algorithm>

#include "ep_common.cuh"

using namespace bibo;

namespace bibo {
// ep.cu: publishes this rank's histogram row into every peer's table
int ep_share_counts_launch(const int32_t* counts, void* const* cnt_peers, int rank, int world, int n_experts,
                           cudaStream_t st);
}

namespace {
struct Copy { void* dst; const void* src; size_t bytes; };
// Issue the block copies.  With auxiliary streams every copy gets its own stream (round robin), all of
// them ordered after the work already in `st` and joined back into `st`: the flows to different peers
// then run at the same time and share the links evenly instead of colliding at one receiver.
int issue_copies(const Copy* c, int n, const bibo_moe_ep_dma* d, int event_base, cudaStream_t st) {
  if (n == 0) return BIBO_OK;
  if (d->n_aux <= 0 || !d->aux_streams || !d->aux_events) {
    for (int i = 0; i < n; ++i) BIBO_CUDA(cudaMemcpyAsync(c[i].dst, c[i].src, c[i].bytes, cudaMemcpyDefault, st));
    return BIBO_OK;
  }
  cudaEvent_t fork = static_cast<cudaEvent_t>(d->aux_events[event_base]);
  BIBO_CUDA(cudaEventRecord(fork, st));
  const int used = std::min(n, d->n_aux);
  for (int j = 0; j < used; ++j) BIBO_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(d->aux_streams[j]), fork, 0));
  for (int i = 0; i < n; ++i)
    BIBO_CUDA(cudaMemcpyAsync(c[i].dst, c[i].src, c[i].bytes, cudaMemcpyDefault,
                              static_cast<cudaStream_t>(d->aux_streams[i % used])));
  for (int j = 0; j < used; ++j) {
    cudaEvent_t join = static_cast<cudaEvent_t>(d->aux_events[event_base + 1 + j]);
    BIBO_CUDA(cudaEventRecord(join, static_cast<cudaStream_t>(d->aux_streams[j])));
    BIBO_CUDA(cudaStreamWaitEvent(st, join, 0));
  }
  return BIBO_OK;
}
}  // namespace

static inline int64_t pad_tile(int64_t c) { return (c + BIBO_TILE_M - 1) / BIBO_TILE_M * BIBO_TILE_M; }

// phase 0 = the whole forward; 1 = everything up to (not including) the host's wait for the histogram
// table; 2 = the rest.  A caller with several token slices issues phase 1 of every slice before phase 2
// of the first, so that no slice's router waits behind another slice's host round trip.
extern "C" int bibo_moe_ep_forward_dma(const bibo_moe_ep_args* a, const bibo_moe_ep_dma* d, int phase, void* stream) {
  if (!a || !d) return fail(BIBO_ERR_ARG, "ep_forward_dma: null args");
  const int R = a->world, E = a->n_experts, me = a->rank;
  if (R < 1 || R > EP_MAX_RANKS || me < 0 || me >= R || E < R || E > BIBO_MAX_EXPERTS || E % R != 0)
    return fail(BIBO_ERR_ARG, "ep_forward_dma: rank %d of %d, %d experts", me, R, E);
  if (!a->cnt_peers || !a->flags_peers || !a->xp_peers || !a->local_plan || !a->ep_plan || !d->xp_send ||
      !d->y_owner || !d->y_home_peers || !d->row_token || !d->cnt_host)
    return fail(BIBO_ERR_ARG, "ep_forward_dma: null buffer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int el = E / R;
  const size_t row_bytes = (size_t)a->hidden * 2;
  int32_t* status = a->ep_plan + PLAN_STATUS;

  if (phase < 0 || phase > 2) return fail(BIBO_ERR_ARG, "ep_forward_dma: phase %d", phase);
  if (!d->counts_ready) return fail(BIBO_ERR_ARG, "ep_forward_dma: no event");
  cudaEvent_t counts_ready = static_cast<cudaEvent_t>(d->counts_ready);
  int rc = BIBO_OK;
  // optional timeline: marks[i] is recorded when step i of the list in the header has been issued
#define EP_MARK(i)                                                                          \
  do {                                                                                      \
    if (d->marks) BIBO_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(d->marks[i]), st));    \
  } while (0)
  if (phase != 2) {
  EP_MARK(0);
  if (a->trace && !a->trace->block_sums) return fail(BIBO_ERR_ARG, "ep_forward_dma: trace without block_sums");
  rc = bibo_moe_router_fwd_trace(a->x, a->w_router, a->bias, nullptr, a->n_tokens, a->hidden, E, a->top_k, a->norm_mode,
                                 a->scale, BIBO_BF16, nullptr, a->topk_idx, a->topk_w, a->slot_rank, a->block_counts,
                                 a->local_plan + PLAN_STATUS, a->trace ? a->trace->block_sums : nullptr, stream);
  if (rc) return rc;
  rc = bibo_moe_plan_trace(a->block_counts, a->n_tokens, a->top_k, E, E, a->local_plan, a->trace, stream);
  if (rc) return rc;
  for (int i = 0; i < R; ++i)
    if (!a->cnt_peers[i] || !a->xp_peers[i] || !d->y_home_peers[i])
      return fail(BIBO_ERR_ARG, "ep_forward_dma: peer %d has a null buffer", i);
  rc = ep_share_counts_launch(a->local_plan + plan_off_counts(), a->cnt_peers, me, R, E, st);
  if (rc) return rc;
  rc = bibo_moe_ep_barrier(a->flags_peers, me, R, a->epoch_base + 1, status, stream);
  if (rc) return rc;
  EP_MARK(1);
  BIBO_CUDA(cudaMemcpyAsync(d->cnt_host, a->cnt_peers[me], sizeof(int32_t) * R * E, cudaMemcpyDeviceToHost, st));
  BIBO_CUDA(cudaEventRecord(counts_ready, st));
  // work that needs no host knowledge is queued before the host waits for the table
  rc = bibo_moe_ep_plan_layout(static_cast<const int32_t*>(a->cnt_peers[me]), me, R, E, a->rows_cap_recv, 1,
                               a->ep_plan, stream);
  if (rc) return rc;
  rc = bibo_moe_permute_fwd(a->x, a->topk_idx, a->slot_rank, a->local_plan, a->n_tokens, a->hidden, E, E, a->top_k,
                            BIBO_BF16, 0, d->xp_send, a->slot_row, d->row_token, stream);
  if (rc) return rc;
  EP_MARK(2);
  }
  if (phase == 1) return BIBO_OK;
  BIBO_CUDA(cudaEventSynchronize(counts_ready));

  // host mirror of the layouts: blk[s][o] rows that source s sends to owner o (its experts o*el .. padded
  // per expert), home_off[s][o] = where they start in s's expert-sorted order, recv_off[o][s] = where
  // they start in o's source-major receive buffer
  const int32_t* cnt = d->cnt_host;
  int64_t blk[EP_MAX_RANKS][EP_MAX_RANKS], home_off[EP_MAX_RANKS][EP_MAX_RANKS], recv_off[EP_MAX_RANKS][EP_MAX_RANKS];
  bool over = false;
  for (int s = 0; s < R; ++s) {
    int64_t run = 0;
    for (int o = 0; o < R; ++o) {
      home_off[s][o] = run;
      int64_t b = 0;
      for (int le = 0; le < el; ++le) b += pad_tile(cnt[s * E + o * el + le]);
      blk[s][o] = b;
      run += b;
    }
  }
  for (int o = 0; o < R; ++o) {
    int64_t run = 0;
    for (int s = 0; s < R; ++s) { recv_off[o][s] = run; run += blk[s][o]; }
    if (run > a->rows_cap_recv) over = true;      // every rank computes the same verdict; ep_plan raised status 4
  }
  Copy copies[EP_MAX_RANKS];
  int n_copies = 0;
  if (!over)
    for (int j = 0; j < R; ++j) {                 // staggered start: rank r begins with peer r
      const int o = (me + j) % R;
      if (blk[me][o] == 0) continue;
      copies[n_copies++] = {static_cast<char*>(a->xp_peers[o]) + recv_off[o][me] * row_bytes,
                            static_cast<const char*>(d->xp_send) + home_off[me][o] * row_bytes,
                            (size_t)blk[me][o] * row_bytes};
    }
  rc = issue_copies(copies, n_copies, d, 0, st);
  if (rc) return rc;
  EP_MARK(3);
  rc = bibo_moe_ep_barrier(a->flags_peers, me, R, a->epoch_base + 2, status, stream);
  if (rc) return rc;
  EP_MARK(4);
  rc = bibo_moe_ep_experts(a->xp_peers[me], a->gate_up_proj, a->down_proj, a->theta, a->ep_plan, a->hidden, a->inter,
                           E, R, a->rows_cap_recv, a->max_ctas, a->h, d->y_owner, nullptr, nullptr, 0, stream);
  if (rc) return rc;
  EP_MARK(5);
  n_copies = 0;
  if (!over)
    for (int j = 0; j < R; ++j) {
      const int s = (me + j) % R;
      if (blk[s][me] == 0) continue;
      copies[n_copies++] = {static_cast<char*>(d->y_home_peers[s]) + home_off[s][me] * row_bytes,
                            static_cast<const char*>(d->y_owner) + recv_off[me][s] * row_bytes,
                            (size_t)blk[s][me] * row_bytes};
    }
  rc = issue_copies(copies, n_copies, d, 1 + EP_MAX_RANKS, st);
  if (rc) return rc;
  EP_MARK(6);
  rc = bibo_moe_ep_barrier(a->flags_peers, me, R, a->epoch_base + 3, status, stream);
  if (rc) return rc;
  EP_MARK(7);
  rc = bibo_moe_combine_fwd(d->y_home_peers[me], a->x, a->slot_row, a->topk_idx, a->topk_w, a->n_tokens, a->hidden,
                            a->top_k, E, 0, BIBO_BF16, a->out, stream);
  if (rc) return rc;
  EP_MARK(8);
#undef EP_MARK
  return BIBO_OK;
}
