// extern "C" entry points that dispatch K3/K4 and chain the whole block.
#include <algorithm>
#include <map>
#include <mutex>

#include "common.cuh"

namespace bibo {
// gemm_simt.cu
int gemm_simt_launch(const void* A, const void* B, void* C, const PlanView& pv, int k_dim, int n_out, int dtype,
                     cudaStream_t st, int ldc = 0, int64_t row_limit = INT64_MAX);
int radial_rows_launch(const void* gate_up, const float* theta, const PlanView& pv, int inter, int dtype, void* h,
                       float* rnorm_out, cudaStream_t st);
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

extern "C" int bibo_moe_version(void) { return 100; }
extern "C" const char* bibo_moe_last_error_string(void) { return err_buf(); }
extern "C" int64_t bibo_moe_launch_count(void) { return launch_counter().load(); }

static int check_common(const char* who, int64_t n_tokens, int hidden, int inter, int n_experts,
                        int n_glu, int top_k, int dtype) {
  if (dtype != BIBO_F32 && dtype != BIBO_BF16) return fail(BIBO_ERR_ARG, "%s: dtype=%d", who, dtype);
  if (n_tokens <= 0 || hidden < 1 || inter < 1)
    return fail(BIBO_ERR_ARG, "%s: n_tokens=%lld hidden=%d inter=%d", who, (long long)n_tokens, hidden, inter);
  if (n_experts < 1 || n_experts > BIBO_MAX_EXPERTS || n_glu < 0 || n_glu > n_experts || top_k < 1 ||
      top_k > BIBO_MAX_TOP_K)
    return fail(BIBO_ERR_UNSUPPORTED, "%s: n_experts=%d n_glu=%d top_k=%d", who, n_experts, n_glu, top_k);
  return BIBO_OK;
}

extern "C" int bibo_moe_gemm1_radial_fwd(const void* xp, const void* gate_up_proj, const float* theta,
                                         const int32_t* plan, int64_t n_tokens, int hidden, int inter,
                                         int n_experts, int n_glu, int top_k, int dtype, void* h,
                                         void* gate_up_out, float* rnorm_out, void* stream) {
  int rc = check_common("gemm1_radial_fwd", n_tokens, hidden, inter, n_experts, n_glu, top_k, dtype);
  if (rc) return rc;
  if (n_glu == 0) return BIBO_OK;
  if (!xp || !gate_up_proj || !theta || !plan || !h) return fail(BIBO_ERR_ARG, "gemm1_radial_fwd: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const PlanView pv = local_plan_view(plan, n_tokens, top_k, n_experts, n_glu);
  if (gemm1_tc_supported(hidden, inter, dtype) && aligned16(xp) && aligned16(gate_up_proj) && aligned16(h) &&
      aligned16(gate_up_out))
    return gemm1_tc_launch(xp, gate_up_proj, theta, pv, hidden, inter, n_glu, h, gate_up_out, rnorm_out, st);
  if (!gate_up_out)
    return fail(BIBO_ERR_ARG,
                "gemm1_radial_fwd: this dtype/shape runs the two-kernel path and needs the gate_up buffer");
  rc = gemm_simt_launch(xp, gate_up_proj, gate_up_out, pv, hidden, 2 * inter, dtype, st);
  if (rc) return rc;
  return radial_rows_launch(gate_up_out, theta, pv, inter, dtype, h, rnorm_out, st);
}

extern "C" int bibo_moe_gemm1_gather_supported(int hidden, int inter, int dtype) {
  return gemm1_gather_supported(hidden, inter, dtype);
}

extern "C" int bibo_moe_gemm1_gather_fwd(const void* x, const int32_t* row_token, const void* gate_up_proj,
                                         const float* theta, const int32_t* plan, int64_t n_tokens, int hidden,
                                         int inter, int n_experts, int n_glu, int top_k, int dtype,
                                         int zero_padding, void* xp, void* h, void* gate_up_out, float* rnorm_out,
                                         void* stream) {
  int rc = check_common("gemm1_gather_fwd", n_tokens, hidden, inter, n_experts, n_glu, top_k, dtype);
  if (rc) return rc;
  if (n_glu == 0) return BIBO_OK;
  if (!x || !row_token || !xp || !gate_up_proj || !theta || !plan || !h)
    return fail(BIBO_ERR_ARG, "gemm1_gather_fwd: null pointer");
  if (!gemm1_gather_supported(hidden, inter, dtype))
    return fail(BIBO_ERR_UNSUPPORTED, "gemm1_gather_fwd: bf16 with intermediate 256 or 512 only (hidden=%d inter=%d)",
                hidden, inter);
  if (!aligned16(x) || !aligned16(xp) || !aligned16(gate_up_proj) || !aligned16(h) || !aligned16(gate_up_out))
    return fail(BIBO_ERR_ALIGN, "gemm1_gather_fwd: pointers not 16-byte aligned");
  const PlanView pv = local_plan_view(plan, n_tokens, top_k, n_experts, n_glu);
  return gemm1_tc_launch(xp, gate_up_proj, theta, pv, hidden, inter, n_glu, h, gate_up_out, rnorm_out,
                         static_cast<cudaStream_t>(stream), x, row_token, zero_padding & 1);
}

extern "C" int bibo_moe_gemm1_is_fused(int hidden, int inter, int dtype) {
  return gemm1_tc_supported(hidden, inter, dtype);
}

extern "C" int bibo_moe_gemm2_fwd(const void* h, const void* down_proj, const int32_t* plan,
                                  int64_t n_tokens, int hidden, int inter, int n_experts, int n_glu,
                                  int top_k, int dtype, void* y, void* stream) {
  int rc = check_common("gemm2_fwd", n_tokens, hidden, inter, n_experts, n_glu, top_k, dtype);
  if (rc) return rc;
  if (n_glu == 0) return BIBO_OK;
  if (!h || !down_proj || !plan || !y) return fail(BIBO_ERR_ARG, "gemm2_fwd: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const PlanView pv = local_plan_view(plan, n_tokens, top_k, n_experts, n_glu);
  if (gemm2_tc_supported(hidden, inter, dtype) && aligned16(h) && aligned16(down_proj) && aligned16(y))
    return gemm2_tc_launch(h, down_proj, pv, hidden, inter, n_glu, y, st);
  return gemm_simt_launch(h, down_proj, y, pv, inter, hidden, dtype, st);
}

// The kernel chain.  With norm_w the input is the raw residual stream: the RMSNorm is folded into the
// router's and the permute's loads, and the residual add into the combine (out = h + block(norm(h))).
static int forward_chain(const bibo_moe_shape* s, const void* x, const void* w_router, const float* bias,
                         const void* gate_up_proj, const void* down_proj, const float* theta,
                         const bibo_moe_workspace* ws, void* out, void* stream, const void* norm_w, float eps,
                         float* rstd, void* w_fold, int refold, void* xn) {
  if (!s || !ws) return fail(BIBO_ERR_ARG, "forward: null shape / workspace");
  cudaStream_t st_ = static_cast<cudaStream_t>(stream);
  void* const* ev = ws->stage_events;
#define BIBO_STAGE(i)                                                              \
  do {                                                                             \
    if (ev) BIBO_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev[i]), st_));      \
  } while (0)
  BIBO_STAGE(0);
  const bibo_moe_router_trace* tr = ws->trace;
  if (tr && !tr->block_sums) return fail(BIBO_ERR_ARG, "forward: trace without block_sums");
  int32_t* status = ws->plan ? ws->plan + PLAN_STATUS : nullptr;
  int rc = BIBO_OK;
  if (norm_w && refold) rc = bibo_moe_fold_norm_weight(w_router, norm_w, s->n_experts, s->hidden, w_fold, stream);
  if (rc) return rc;
  rc = norm_w
      ? bibo_moe_router_norm_fwd(x, w_fold, eps, bias, s->n_tokens, s->hidden, s->n_experts, s->top_k,
                                 s->norm_mode, s->scale, ws->logits, ws->topk_idx, ws->topk_w, ws->slot_rank,
                                 ws->block_counts, status, tr ? tr->block_sums : nullptr, rstd, stream)
      : bibo_moe_router_fwd_trace(x, w_router, bias, nullptr, s->n_tokens, s->hidden, s->n_experts, s->top_k,
                                  s->norm_mode, s->scale, s->dtype, ws->logits, ws->topk_idx, ws->topk_w,
                                  ws->slot_rank, ws->block_counts, status, tr ? tr->block_sums : nullptr, stream);
  if (rc) return rc;
  BIBO_STAGE(1);
  rc = bibo_moe_plan_trace(ws->block_counts, s->n_tokens, s->top_k, s->n_experts, s->n_glu, ws->plan, tr, stream);
  if (rc) return rc;
  BIBO_STAGE(2);
  // bit 1 of zero_padding: the gate/up kernel copies its own rows (bf16, intermediate 256 / 512) and the
  // permute pass shrinks to the row maps
  const bool gather = !norm_w && (s->zero_padding & 2) && s->n_glu > 0 &&
                      gemm1_gather_supported(s->hidden, s->inter, s->dtype) && aligned16(x) && aligned16(ws->xp) &&
                      aligned16(gate_up_proj) && aligned16(ws->h) && aligned16(ws->gate_up);
  rc = norm_w
      ? bibo_moe_permute_norm_fwd(x, rstd, norm_w, ws->topk_idx, ws->slot_rank, ws->plan, s->n_tokens, s->hidden,
                                  s->n_experts, s->n_glu, s->top_k, s->zero_padding & 1, ws->xp, ws->slot_row,
                                  ws->row_token, xn, stream)
      : gather
      ? bibo_moe_rowmap_fwd(ws->topk_idx, ws->slot_rank, ws->plan, s->n_tokens, s->n_experts, s->n_glu, s->top_k,
                            ws->slot_row, ws->row_token, stream)
      : bibo_moe_permute_fwd(x, ws->topk_idx, ws->slot_rank, ws->plan, s->n_tokens, s->hidden, s->n_experts,
                             s->n_glu, s->top_k, s->dtype, s->zero_padding & 1, ws->xp, ws->slot_row,
                             ws->row_token, stream);
  if (rc) return rc;
  BIBO_STAGE(3);
  rc = gather
      ? bibo_moe_gemm1_gather_fwd(x, ws->row_token, gate_up_proj, theta, ws->plan, s->n_tokens, s->hidden, s->inter,
                                  s->n_experts, s->n_glu, s->top_k, s->dtype, s->zero_padding, ws->xp, ws->h,
                                  ws->gate_up, ws->rnorm, stream)
      : bibo_moe_gemm1_radial_fwd(ws->xp, gate_up_proj, theta, ws->plan, s->n_tokens, s->hidden, s->inter,
                                  s->n_experts, s->n_glu, s->top_k, s->dtype, ws->h, ws->gate_up, ws->rnorm,
                                  stream);
  if (rc) return rc;
  BIBO_STAGE(4);
  rc = bibo_moe_gemm2_fwd(ws->h, down_proj, ws->plan, s->n_tokens, s->hidden, s->inter, s->n_experts,
                          s->n_glu, s->top_k, s->dtype, ws->y, stream);
  if (rc) return rc;
  BIBO_STAGE(5);
  // with the norm folded in, x is the raw stream: it is the residual, and the identity experts (if any) read xn
  rc = bibo_moe_combine_add_fwd(ws->y, (norm_w && xn) ? xn : x, ws->slot_row, ws->topk_idx, ws->topk_w, norm_w ? x : ws->addend,
                                s->n_tokens, s->hidden, s->top_k, s->n_glu, s->n_pos, s->dtype, out, stream);
  if (rc) return rc;
  BIBO_STAGE(6);
#undef BIBO_STAGE
  return BIBO_OK;
}

extern "C" int bibo_moe_forward(const bibo_moe_shape* s, const void* x, const void* w_router,
                                const float* bias, const void* gate_up_proj, const void* down_proj,
                                const float* theta, const bibo_moe_workspace* ws, void* out, void* stream) {
  return forward_chain(s, x, w_router, bias, gate_up_proj, down_proj, theta, ws, out, stream, nullptr, 0.f, nullptr,
                       nullptr, 0, nullptr);
}

extern "C" int bibo_moe_ffn_supported(const bibo_moe_shape* s) {
  return s && s->dtype == BIBO_BF16 && bibo_moe_router_norm_supported(s->hidden, s->n_experts, s->dtype);
}

extern "C" int bibo_moe_ffn_forward(const bibo_moe_shape* s, const void* h, const void* norm_weight, float eps,
                                    const void* w_router, const float* bias, const void* gate_up_proj,
                                    const void* down_proj, const float* theta, const bibo_moe_workspace* ws,
                                    float* rstd, void* w_fold, int refold, void* xn, void* out, void* stream) {
  if (!s || !ws || !h || !norm_weight || !rstd || !w_fold) return fail(BIBO_ERR_ARG, "ffn_forward: null pointer");
  if (!bibo_moe_ffn_supported(s))
    return fail(BIBO_ERR_UNSUPPORTED, "ffn_forward: bf16, 64 routed experts and hidden %% 64 == 0 only");
  if (s->n_glu < s->n_experts && !xn) return fail(BIBO_ERR_ARG, "ffn_forward: identity experts need the xn buffer");
  if (ws->addend) return fail(BIBO_ERR_ARG, "ffn_forward: the addend slot is taken by the residual");
  return forward_chain(s, h, w_router, bias, gate_up_proj, down_proj, theta, ws, out, stream, norm_weight, eps, rstd,
                       w_fold, refold, xn);
}

// ---- host-buffer call: copies overlapped with the kernels --------------------------------------------
// Tokens are independent, so the batch is cut into slices: the host->device copy of slice i+1 and the
// device->host copy of slice i-1 run on two copy streams while slice i is computed on the caller's
// stream (the link is full duplex).  Streams and events are created once per device and kept.
namespace {
constexpr int HOST_MAX_SLICES = 16;
struct HostPipe {
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t start = nullptr, done = nullptr, copied[HOST_MAX_SLICES] = {}, computed[HOST_MAX_SLICES] = {};
  bool ready = false;
};
int host_pipe(HostPipe** out) {
  static std::mutex mu;
  static std::map<int, HostPipe> pipes;
  int dev = 0;
  BIBO_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> g(mu);
  HostPipe& p = pipes[dev];
  if (!p.ready) {
    BIBO_CUDA(cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking));
    BIBO_CUDA(cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking));
    BIBO_CUDA(cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming));
    BIBO_CUDA(cudaEventCreateWithFlags(&p.done, cudaEventDisableTiming));
    for (int i = 0; i < HOST_MAX_SLICES; ++i) {
      BIBO_CUDA(cudaEventCreateWithFlags(&p.copied[i], cudaEventDisableTiming));
      BIBO_CUDA(cudaEventCreateWithFlags(&p.computed[i], cudaEventDisableTiming));
    }
    p.ready = true;
  }
  *out = &p;
  return BIBO_OK;
}
// Slice lengths: equal slices of about 4096 tokens (a multiple of the router block), at most
// HOST_MAX_SLICES of them.  A tapered tail (shorter last slices) and 2048 / 3072 / 6144 / 8192-token slices
// all measured slower.  BIBO_HOST_SLICE_TOKENS overrides the length (0 = one slice, no overlap).
int host_slices(int64_t n_tokens, int64_t* lens) {
  static const int64_t forced = [] { const char* e = getenv("BIBO_HOST_SLICE_TOKENS"); return e ? atoll(e) : -1; }();
  constexpr int64_t BLK = BIBO_ROUTER_BLOCK_TOKENS;
  int64_t len = forced >= 0 ? forced : 4096;
  if (len <= 0 || n_tokens < 2 * len) { lens[0] = n_tokens; return 1; }
  const int64_t min_len = (n_tokens + HOST_MAX_SLICES - 1) / HOST_MAX_SLICES;
  len = (std::max(len, min_len) + BLK - 1) / BLK * BLK;
  int n = 0;
  for (int64_t left = n_tokens; left > 0; left -= lens[n++]) lens[n] = std::min(len, left);
  return n;
}
}  // namespace

// Waits for the stream and looks at the sticky status word the kernels leave in plan[2] (the read rides on
// the synchronisation the call does anyway): a bounded wait that gave up, or a bad routing index, becomes
// BIBO_ERR_DEVICE_STATUS instead of a silently wrong result.
namespace bibo {
int sync_and_check_status(const int32_t* plan, cudaStream_t st, const char* who) {
  static thread_local int32_t hdr[4];
  hdr[PLAN_STATUS] = 0;
  if (plan) BIBO_CUDA(cudaMemcpyAsync(hdr, plan, sizeof(hdr), cudaMemcpyDeviceToHost, st));
  BIBO_CUDA(cudaStreamSynchronize(st));
  if (hdr[PLAN_STATUS] != 0)
    return fail(BIBO_ERR_DEVICE_STATUS, "%s: the kernels left status %d in the plan (see bibo_moe.h, plan layout)", who,
                hdr[PLAN_STATUS]);
  return BIBO_OK;
}
}  // namespace bibo

extern "C" int bibo_moe_forward_host(const bibo_moe_shape* s, const void* x_host, void* x_dev,
                                     const void* w_router, const float* bias, const void* gate_up_proj,
                                     const void* down_proj, const float* theta,
                                     const bibo_moe_workspace* ws, void* out_dev, void* out_host,
                                     void* stream) {
  if (!s || !ws || !x_host || !x_dev || !out_dev || !out_host) return fail(BIBO_ERR_ARG, "forward_host: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t row_bytes = (size_t)s->hidden * (s->dtype == BIBO_F32 ? 4 : 2);
  int64_t lens[HOST_MAX_SLICES];
  const int n_slices = host_slices(s->n_tokens, lens);
  if (n_slices == 1) {
    const size_t bytes = (size_t)s->n_tokens * row_bytes;
    BIBO_CUDA(cudaMemcpyAsync(x_dev, x_host, bytes, cudaMemcpyHostToDevice, st));
    int rc = bibo_moe_forward(s, x_dev, w_router, bias, gate_up_proj, down_proj, theta, ws, out_dev, stream);
    if (rc) return rc;
    BIBO_CUDA(cudaMemcpyAsync(out_host, out_dev, bytes, cudaMemcpyDeviceToHost, st));
    return sync_and_check_status(ws->plan, st, "forward_host");
  }
  HostPipe* hp = nullptr;
  int rc = host_pipe(&hp);
  if (rc) return rc;
  BIBO_CUDA(cudaEventRecord(hp->start, st));          // earlier work of the caller's stream owns the buffers until here
  BIBO_CUDA(cudaStreamWaitEvent(hp->in, hp->start, 0));
  BIBO_CUDA(cudaStreamWaitEvent(hp->out, hp->start, 0));
  int64_t t0 = 0;
  for (int i = 0; i < n_slices; t0 += lens[i++]) {
    const int64_t nt = lens[i];
    BIBO_CUDA(cudaMemcpyAsync(static_cast<char*>(x_dev) + t0 * row_bytes, static_cast<const char*>(x_host) + t0 * row_bytes,
                              (size_t)nt * row_bytes, cudaMemcpyHostToDevice, hp->in));
    BIBO_CUDA(cudaEventRecord(hp->copied[i], hp->in));
  }
  t0 = 0;
  for (int i = 0; i < n_slices; t0 += lens[i++]) {
    const int64_t nt = lens[i];
    bibo_moe_shape part = *s;
    part.n_tokens = nt;                               // the workspace of the whole batch is large enough for a slice
    bibo_moe_workspace wpart = *ws;
    if (wpart.addend) wpart.addend = static_cast<const char*>(ws->addend) + t0 * row_bytes;   // per-token tensor
    BIBO_CUDA(cudaStreamWaitEvent(st, hp->copied[i], 0));
    rc = bibo_moe_forward(&part, static_cast<const char*>(x_dev) + t0 * row_bytes, w_router, bias, gate_up_proj,
                          down_proj, theta, &wpart, static_cast<char*>(out_dev) + t0 * row_bytes, stream);
    if (rc) return rc;
    BIBO_CUDA(cudaEventRecord(hp->computed[i], st));
    BIBO_CUDA(cudaStreamWaitEvent(hp->out, hp->computed[i], 0));
    BIBO_CUDA(cudaMemcpyAsync(static_cast<char*>(out_host) + t0 * row_bytes, static_cast<const char*>(out_dev) + t0 * row_bytes,
                              (size_t)nt * row_bytes, cudaMemcpyDeviceToHost, hp->out));
  }
  BIBO_CUDA(cudaEventRecord(hp->done, hp->out));
  BIBO_CUDA(cudaStreamWaitEvent(st, hp->done, 0));
  return sync_and_check_status(ws->plan, st, "forward_host");
}

extern "C" int bibo_moe_debug_plan_header(const int32_t* plan, int32_t* header4_host, void* stream) {
  if (!plan || !header4_host) return fail(BIBO_ERR_ARG, "debug_plan_header: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BIBO_CUDA(cudaMemcpyAsync(header4_host, plan, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  BIBO_CUDA(cudaStreamSynchronize(st));
  if (header4_host[PLAN_STATUS] != 0)
    return fail(BIBO_ERR_DEVICE_STATUS, "plan status word = %d", header4_host[PLAN_STATUS]);
  return BIBO_OK;
}
