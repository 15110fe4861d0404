/*
 * bibo_moe.h -- C ABI of libbibo_moe.so: the BiBo sparse-MoE feed-forward block as a chain of
 * sm_100a CUDA kernels.
 *
 * The reference project has no native plug-in interface for this path: it swaps kernels in by
 * assigning Python callables onto its module classes (ablate/common/patches.py:177-180 assigns
 * BiBoFusedExperts.forward, patches.py:290 assigns BiBoDecoderLayer._ffn_forward).  The entry
 * points below sit UNDER that Python seam; each comment names the reference code the call
 * replaces (paths inside the reference project).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the parameter name ends in _host;
 *   - nothing here allocates device memory, synchronises the device or throws (the two _host
 *     entry points and the explicitly named debug calls are the exceptions, documented at the call);
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*);
 *   - return value 0 = success, negative = error; bibo_moe_last_error_string() describes the
 *     last error of the calling thread;
 *   - dtype: 0 = float32, 1 = bfloat16 (activations and weights share one dtype; router scores,
 *     routing weights and all accumulation are float32).
 *
 * Row layout shared by the calls ("the plan")
 *   N tokens, k slots per token, E routed experts of which the first E_glu own weights.  Rows of
 *   expert e occupy [expert_off[e], expert_off[e] + counts[e]) of every expert-contiguous buffer;
 *   expert_off[e] is a multiple of BIBO_TILE_M, so a BIBO_TILE_M-row tile never straddles two
 *   experts.  Inside an expert, rows are in ascending token order.  plan_tiles[] lists the row
 *   tiles: {expert, first row, valid rows, 0}.
 */
#ifndef BIBO_MOE_H_
#define BIBO_MOE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BIBO_TILE_M 128
#define BIBO_ROUTER_BLOCK_TOKENS 128
#define BIBO_MAX_TOP_K 8
#define BIBO_MAX_EXPERTS 256

enum { BIBO_F32 = 0, BIBO_BF16 = 1 };
enum { BIBO_NORM_RAW = 0, BIBO_NORM_SUM = 1, BIBO_NORM_SOFTMAX = 2 };

/* error codes */
enum {
  BIBO_OK = 0,
  BIBO_ERR_ARG = -1,          /* bad size / null pointer / unsupported combination */
  BIBO_ERR_ALIGN = -2,        /* pointer or leading dimension not 16-byte aligned   */
  BIBO_ERR_CUDA = -3,         /* a CUDA runtime/driver call failed                  */
  BIBO_ERR_UNSUPPORTED = -4,  /* shape outside what the kernels cover               */
  BIBO_ERR_DEVICE_STATUS = -5 /* a kernel reported a non-zero status word           */
};

int bibo_moe_version(void);
const char* bibo_moe_last_error_string(void);

/* ---- sizes the caller needs to allocate buffers --------------------------------------------- */
/* Upper bound of rows in an expert-contiguous buffer: N*k + E_glu*(BIBO_TILE_M-1), rounded up.  */
int64_t bibo_moe_rows_cap(int64_t n_tokens, int top_k, int n_glu);
/* Upper bound of row tiles.                                                                      */
int64_t bibo_moe_tiles_cap(int64_t n_tokens, int top_k, int n_glu);
/* Blocks the router kernel splits the tokens into (rows of block_counts / block_base).           */
int64_t bibo_moe_router_blocks(int64_t n_tokens);
/* int32 words in a plan buffer for these sizes (see bibo_moe_plan).                              */
int64_t bibo_moe_plan_words(int64_t n_tokens, int top_k, int n_experts, int n_glu);

/* ---- K1: router ------------------------------------------------------------------------------
 * Replaces BiBoMoERouter.router_logits + forward (src/modeling/ffn/router.py:25-51) and the
 * bincount of BiBoFusedExperts.forward / _balance_step (src/modeling/ffn/moe.py:65,140-143).
 * logits = x @ w_router^T with fp32 accumulation; score = sigmoid(logit); selection on
 * score + bias, ties to the lower expert index; weights from the un-biased scores, normalised per
 * norm_mode and multiplied by scale.  The k experts of a token are written in ASCENDING expert
 * index.  Also writes, per block of BIBO_ROUTER_BLOCK_TOKENS tokens, the per-expert histogram
 * (block_counts [blocks, E]) and each slot's rank among the block's earlier tokens that picked
 * the same expert (slot_rank [N, k]).
 * logits_out may be NULL.  If logits_in is non-NULL the matrix product is skipped and the
 * selection runs on the given fp32 logits (test entry: selection parity on identical logits).
 * status (optional device int32) is set non-zero if a bounded wait inside the kernel gave up.    */
int bibo_moe_router_fwd(const void* x, const void* w_router, const float* bias,
                        const float* logits_in, int64_t n_tokens, int hidden, int n_experts,
                        int top_k, int norm_mode, float scale, int dtype,
                        float* logits_out, int32_t* topk_idx, float* topk_w,
                        int32_t* slot_rank, int32_t* block_counts, int32_t* status, void* stream);

/* ---- router diagnostics without extra launches -------------------------------------------------
 * Replaces the boundary-gap probe of BiBoMoERouter.forward (src/modeling/ffn/router.py:33-36: mean over
 * tokens of the raw score of rank k minus that of rank k+1) and the device-side sums of
 * RouterTrace._hook / _router_hook (ablate/common/router_trace.py:106-130), which the reference
 * computes with a second top-k and about twenty small launches per layer.  The router kernel
 * writes per-block sums (block_sums [router_blocks, BIBO_TRACE_WORDS] fp32, see router_select.cuh
 * for the words); the plan kernel adds them up in a fixed order and folds them into the caller's
 * accumulators:
 *   acc[0] += sum_t max_j p   acc[1] += sum_t entropy(p)   acc[2] += N   acc[3] += sum_t max_j w
 *   acc[4] += sum_t sum_j w   acc[5] += sum_t min_j w      acc[6] += mean gap   acc[7] += 1
 *   counts[e] += tokens routed to expert e (as float)      gap[0] = mean gap of this call
 * with w the weights as written to topk_w and p = w / max(sum_j |w_j|, 1e-9).  acc, counts and gap
 * are optional device pointers; the struct itself lives in HOST memory.                           */
#define BIBO_TRACE_WORDS 8
typedef struct {
  float* block_sums;      /* scratch [router_blocks, BIBO_TRACE_WORDS] */
  float* acc;             /* optional [BIBO_TRACE_WORDS], accumulated  */
  float* counts;          /* optional [E], accumulated                 */
  float* gap;             /* optional [1], overwritten                 */
} bibo_moe_router_trace;
/* bibo_moe_router_fwd that also writes block_sums (NULL = off).                                    */
int bibo_moe_router_fwd_trace(const void* x, const void* w_router, const float* bias,
                              const float* logits_in, int64_t n_tokens, int hidden, int n_experts,
                              int top_k, int norm_mode, float scale, int dtype,
                              float* logits_out, int32_t* topk_idx, float* topk_w,
                              int32_t* slot_rank, int32_t* block_counts, int32_t* status,
                              float* block_sums, void* stream);

/* Histogram and ranks for routing decided by the caller: the BiBoFusedExperts.forward(x, idx, w)
 * seam (src/modeling/ffn/moe.py:47-52).  topk_idx [N,k] int32 in any order.  status (optional
 * device int32, zeroed by the caller) is set to 2 for an index outside [0,E) (treated as expert 0)
 * and to 3 when a token names one expert twice.                                                  */
int bibo_moe_route_from_indices(const int32_t* topk_idx, int64_t n_tokens, int n_experts, int top_k,
                                int32_t* slot_rank, int32_t* block_counts, int32_t* status,
                                void* stream);

/* ---- plan: histogram -> offsets ---------------------------------------------------------------
 * Replaces the sort / bincount / cumsum / .tolist() of BiBoFusedExperts.forward
 * (src/modeling/ffn/moe.py:56-68) without a host synchronisation.
 * plan layout (int32 words): [0]=n_tiles [1]=rows used [2]=status [3]=n_pairs; the status word is
 * STICKY: the caller zeroes it once, kernels only ever raise it (1 = histogram total > N*k,
 * 2 = an expert index >= n_experts (the slot is ignored), 3 = one expert twice in a token,
 * 4 = a receive buffer of the expert-parallel path would overflow, 5 = a cross-rank barrier timed
 * out, 100..111 = a bounded wait inside a tensor-core kernel gave up: 100 down, 101 gate/up,
 * 102 router, 104 the gate/up kernel's exchange between its two column-block clusters),
 * then counts[E], expert_off[E_glu+1], block_base[blocks*E] (exclusive prefix of block_counts over
 * blocks), tiles[tiles_cap*4] (int4 {expert, first row, rows, 0}), pairs[tiles_cap*2] (int2: two
 * consecutive tiles of one expert, or {tile, -1}) and the scratch of the gate/up kernel.
 * bibo_moe_plan_words gives the total; the accessors below return the word offsets.                */
int bibo_moe_plan(const int32_t* block_counts, int64_t n_tokens, int top_k, int n_experts,
                  int n_glu, int32_t* plan, void* stream);
/* bibo_moe_plan that also reduces the router's diagnostic sums (trace NULL = off).                */
int bibo_moe_plan_trace(const int32_t* block_counts, int64_t n_tokens, int top_k, int n_experts,
                        int n_glu, int32_t* plan, const bibo_moe_router_trace* trace, void* stream);
int64_t bibo_moe_plan_off_counts(void);
int64_t bibo_moe_plan_off_expert_off(int n_experts);
int64_t bibo_moe_plan_off_block_base(int n_experts, int n_glu);
int64_t bibo_moe_plan_off_tiles(int64_t n_tokens, int n_experts, int n_glu);

/* ---- K2: permute ------------------------------------------------------------------------------
 * Replaces `current_state = hidden_states[token_idx]` (src/modeling/ffn/moe.py:77,81) for all
 * experts at once: writes x rows into expert-contiguous rows xp [rows_cap, H]; also writes
 * slot_row [N,k] (row of every slot, -1 for an expert without weights) and row_token [rows_cap]
 * (token of every row, -1 for padding).  zero_padding != 0 also zero-fills the padding rows of xp
 * (needed when a later reduction runs over rows, i.e. for weight gradients).                     */
int bibo_moe_permute_fwd(const void* x, const int32_t* topk_idx, const int32_t* slot_rank,
                         const int32_t* plan, int64_t n_tokens, int hidden, int n_experts,
                         int n_glu, int top_k, int dtype, int zero_padding,
                         void* xp, int32_t* slot_row, int32_t* row_token, void* stream);

/* ---- K3: grouped gate/up GEMM + Radial NormSiLU -----------------------------------------------
 * Replaces F.linear(x_e, gate_up_proj[e]), chunk, r = sqrt(mean g^2 + 1e-6), p = sigmoid(theta_e),
 * a = silu(g/r) * r^p, a * up  (src/modeling/ffn/moe.py:84-92 up to the input of the down
 * projection).  xp [rows_cap,H], gate_up_proj [E_glu, 2I, H], theta fp32 [E_glu] -> h [rows_cap,I].
 * gate_up_out (optional, [rows_cap, 2I] in dtype) receives the raw gate|up rows, rnorm_out
 * (optional fp32 [rows_cap]) receives r; both are what the backward pass re-reads.               */
int bibo_moe_gemm1_radial_fwd(const void* xp, const void* gate_up_proj, const float* theta,
                              const int32_t* plan, int64_t n_tokens, int hidden, int inter,
                              int n_experts, int n_glu, int top_k, int dtype,
                              void* h, void* gate_up_out, float* rnorm_out, void* stream);

/* 1 when the fused tensor-core kernel covers this shape (gate_up_out may then be NULL), else 0.   */
int bibo_moe_gemm1_is_fused(int hidden, int inter, int dtype);

/* ---- K2 + K3 in one kernel: the gate/up kernel gathers its own rows ------------------------------
 * Same reference lines as K2 and K3 (src/modeling/ffn/moe.py:77,81,84-92).  bibo_moe_rowmap_fwd writes
 * only the row maps of K2 (slot_row [N,k], row_token [rows_cap]; no row is copied; a negative expert
 * index is an empty slot without a row).  bibo_moe_gemm1_gather_fwd then runs K3 with six extra warps
 * per CTA that copy x[row_token[r]] into xp [rows_cap,H] up to two row-tile pairs ahead of the tile
 * loads, so the copies are read back from L2; xp is left complete (what the backward pass re-reads).
 * bf16, intermediate size 256 or 512 (bibo_moe_gemm1_gather_supported); zero_padding bit 0 as in K2.
 * Results are bit-identical to K2 followed by K3.  Opt-in (bibo_moe_shape.zero_padding bit 1): on the
 * benchmark shape it measured 0.77 ms against 0.73 ms for K2 + K3, the copies' L2 traffic costing the
 * tensor-core kernel what the separate pass costs.                                                  */
int bibo_moe_rowmap_fwd(const int32_t* topk_idx, const int32_t* slot_rank, const int32_t* plan,
                        int64_t n_tokens, int n_experts, int n_glu, int top_k, int32_t* slot_row,
                        int32_t* row_token, void* stream);
int bibo_moe_gemm1_gather_supported(int hidden, int inter, int dtype);
int bibo_moe_gemm1_gather_fwd(const void* x, const int32_t* row_token, const void* gate_up_proj,
                              const float* theta, const int32_t* plan, int64_t n_tokens, int hidden,
                              int inter, int n_experts, int n_glu, int top_k, int dtype, int zero_padding,
                              void* xp, void* h, void* gate_up_out, float* rnorm_out, void* stream);

/* ---- K4: grouped down GEMM ---------------------------------------------------------------------
 * Replaces F.linear(activated * up, down_proj[e]) (src/modeling/ffn/moe.py:92).
 * h [rows_cap, I], down_proj [E_glu, H, I] -> y [rows_cap, H].                                    */
int bibo_moe_gemm2_fwd(const void* h, const void* down_proj, const int32_t* plan,
                       int64_t n_tokens, int hidden, int inter, int n_experts, int n_glu,
                       int top_k, int dtype, void* y, void* stream);

/* ---- K5: weighted combine ----------------------------------------------------------------------
 * Replaces output.index_add_(0, token_idx, expert_output * weights) over all experts and the final
 * cast (src/modeling/ffn/moe.py:70-71,93-101): out[t] = sum_j w[t,j] * y[slot_row[t,j]], fp32
 * accumulation in ascending expert order, one cast at the end.  Slots of +Identity / -Identity
 * experts (index >= n_glu; the first n_pos of them positive) add +w*x[t] / -w*x[t].               */
int bibo_moe_combine_fwd(const void* y, const void* x, const int32_t* slot_row,
                         const int32_t* topk_idx, const float* topk_w, int64_t n_tokens,
                         int hidden, int top_k, int n_glu, int n_pos, int dtype, void* out,
                         void* stream);
/* The same with a second term: out[t] = T(T(sum over slots) + addend[t]) (addend may be NULL).      */
int bibo_moe_combine_add_fwd(const void* y, const void* x, const int32_t* slot_row,
                             const int32_t* topk_idx, const float* topk_w, const void* addend,
                             int64_t n_tokens, int hidden, int top_k, int n_glu, int n_pos, int dtype,
                             void* out, void* stream);

/* ---- whole block -------------------------------------------------------------------------------
 * Replaces BiBoMoELayer.forward in eval mode without shared expert
 * (src/modeling/ffn/moe.py:157-183).  All buffers are caller-allocated; `ws` groups the
 * intermediates so a caller can keep one set per (device, shape).                                 */
typedef struct {
  int32_t* topk_idx;      /* [N,k]                      */
  float* topk_w;          /* [N,k]                      */
  int32_t* slot_rank;     /* [N,k]                      */
  int32_t* block_counts;  /* [router_blocks, E]         */
  int32_t* plan;          /* [plan_words]               */
  int32_t* slot_row;      /* [N,k]                      */
  int32_t* row_token;     /* [rows_cap]                 */
  void* xp;               /* [rows_cap, H]  dtype       */
  void* h;                /* [rows_cap, I]  dtype       */
  void* y;                /* [rows_cap, H]  dtype       */
  void* gate_up;          /* optional [rows_cap, 2I]    */
  float* rnorm;           /* optional [rows_cap]        */
  float* logits;          /* optional [N,E]             */
  void* const* stage_events; /* optional HOST array of 7 cudaEvent_t: [i] is recorded on the stream
                                before stage i (router, plan, permute, gate/up, down, combine) and
                                [6] after the last; lets a caller time each kernel without extra
                                launches or synchronisation                                        */
  const void* addend;     /* optional [N,H] dtype: added to the combined output (the shared expert's
                             result, src/modeling/ffn/moe.py:174-176): out = T(T(sum) + addend)        */
  const bibo_moe_router_trace* trace; /* optional HOST struct: router diagnostics of this call       */
} bibo_moe_workspace;

typedef struct {
  int64_t n_tokens;
  int hidden, inter, n_experts, n_glu, n_pos, top_k, norm_mode, dtype;
  float scale;            /* routed_scaling_factor */
  int zero_padding;       /* bit 0: zero-fill the padding rows of xp (training); bit 1: let the gate/up kernel
                             gather its own rows where it can (bibo_moe_gemm1_gather_fwd) instead of running K2
                             as a pass of its own: same bits, measured slightly slower, see below            */
} bibo_moe_shape;

int bibo_moe_forward(const bibo_moe_shape* shape, const void* x, const void* w_router,
                     const float* bias, const void* gate_up_proj, const void* down_proj,
                     const float* theta, const bibo_moe_workspace* ws, void* out, void* stream);

/* ---- feed-forward half of the decoder layer, norm and residual folded in ---------------------------
 * Replaces BiBoDecoderLayer._ffn_forward (src/modeling/layers.py:57-67) for inference:
 * out = h + block(post_attention_layernorm(h)).  The normalised activations are never written:
 * the router kernel reads h against the router weight with the norm weight folded in
 * (w_fold[e][c] = bf16(w_router[e][c] * norm_weight[c])), adds up h^2 per row beside the tensor core
 * and scales its accumulators by rstd = rsqrt(mean h^2 + eps) (rstd [N] fp32 is an output); the
 * permute kernel writes bf16(w * bf16(h * rstd)), BiBoRMSNorm.forward's rounding
 * (src/modeling/norm.py:19-24), into the expert rows; the combine kernel adds h.
 * bf16, 64 routed experts, hidden % 64 == 0 (bibo_moe_ffn_supported); ws->addend must be NULL.
 * w_fold [E,H] bf16 is caller-owned scratch: refold != 0 recomputes it first (one small extra
 * launch); refold == 0 reuses what an earlier call left there for the same weights.
 * xn [N,H] bf16 is needed only with +/-Identity experts (n_glu < n_experts; NULL otherwise): the
 * permute kernel leaves there the normalised row of every token that picked such an expert (no other
 * row is written or read), which the combine kernel adds as +w*x / -w*x.                            */
int bibo_moe_ffn_supported(const bibo_moe_shape* shape);
int bibo_moe_ffn_forward(const bibo_moe_shape* shape, const void* h, const void* norm_weight, float eps,
                         const void* w_router, const float* bias, const void* gate_up_proj,
                         const void* down_proj, const float* theta, const bibo_moe_workspace* ws,
                         float* rstd, void* w_fold, int refold, void* xn, void* out, void* stream);
/* The pieces on their own.                                                                          */
int bibo_moe_router_norm_supported(int hidden, int n_experts, int dtype);
int bibo_moe_fold_norm_weight(const void* w_router, const void* norm_weight, int n_experts, int hidden,
                              void* w_fold, void* stream);
int bibo_moe_router_norm_fwd(const void* h, const void* w_fold, float eps, const float* bias,
                             int64_t n_tokens, int hidden, int n_experts, int top_k, int norm_mode,
                             float scale, float* logits_out, int32_t* topk_idx, float* topk_w,
                             int32_t* slot_rank, int32_t* block_counts, int32_t* status,
                             float* block_sums, float* rstd_out, void* stream);
int bibo_moe_permute_norm_fwd(const void* h, const float* rstd, const void* norm_weight,
                              const int32_t* topk_idx, const int32_t* slot_rank, const int32_t* plan,
                              int64_t n_tokens, int hidden, int n_experts, int n_glu, int top_k,
                              int zero_padding, void* xp, int32_t* slot_row, int32_t* row_token,
                              void* xn, void* stream);

/* Same block with HOST input and output: copies x_host to x_dev, runs the block, copies the result
 * into out_host and waits for it.  x_dev / out_dev are caller-allocated device staging buffers
 * [N,H]; weights stay resident on the device.  Batches of 8192 tokens or more are cut into slices
 * of about 4096 tokens: the copies of neighbouring slices run on two internal copy streams
 * (created once per device) while a slice is computed on `stream`; tokens are independent, so the
 * result equals bibo_moe_forward bit for bit.  Afterwards the workspace describes the LAST slice
 * only.  x_host / out_host should be pinned.  This is the call the end-to-end timing uses
 * (host->device and device->host copies inside the call).  The environment variable
 * BIBO_HOST_SLICE_TOKENS, read once at the first call, overrides the slice length (0 = one slice,
 * no overlap); it is the library's only environment switch.  The call reads the plan header with its
 * final synchronisation and returns BIBO_ERR_DEVICE_STATUS if a kernel left a status word.          */
int bibo_moe_forward_host(const bibo_moe_shape* shape, const void* x_host, void* x_dev,
                          const void* w_router, const float* bias, const void* gate_up_proj,
                          const void* down_proj, const float* theta, const bibo_moe_workspace* ws,
                          void* out_dev, void* out_host, void* stream);

/* ---- backward ----------------------------------------------------------------------------------------
 * The reference derives its gradients by autograd over src/modeling/ffn/router.py:25-51 and
 * src/modeling/ffn/moe.py:47-101 (there is no hand-written backward to cite); this call computes the
 * same gradients in closed form on the forward's expert-contiguous layout.
 * `ws` is the workspace of the matching bibo_moe_forward call, run with zero_padding = 0 or 1 and
 * with xp, h, y, gate_up, rnorm kept; it is CONSUMED: y is overwritten (dXp) and gate_up becomes
 * dGate|dUp.  dout [N,H] is the gradient of the block output.  Outputs: dx [N,H], d_w_router [E,H],
 * d_gate_up_proj [E_glu,2I,H], d_down_proj [E_glu,H,I] in the model dtype (overwritten, not
 * accumulated), d_theta fp32 [E_glu].  gate.bias receives no gradient (requires_grad=False in the
 * reference).  Every reduction runs in a fixed order: results are bit-reproducible.               */
typedef struct {
  void* dy;           /* [rows_cap, H] dtype */
  void* dh;           /* [rows_cap, I] dtype */
  float* dw;          /* [N,k]               */
  float* dlogit;      /* [N,k]               */
  float* dlogit_row;  /* [rows_cap]          */
  float* dtheta_row;  /* [rows_cap]          */
} bibo_moe_bwd_workspace;

int bibo_moe_backward(const bibo_moe_shape* shape, const void* x, const void* w_router,
                      const void* gate_up_proj, const void* down_proj, const float* theta,
                      const bibo_moe_workspace* ws, const void* dout, const bibo_moe_bwd_workspace* bws,
                      void* dx, void* d_w_router, void* d_gate_up_proj, void* d_down_proj, float* d_theta,
                      void* stream);

/* ---- expert-parallel forward over NVLink peer memory ------------------------------------------------
 * No counterpart in the reference (it has no expert parallelism; its only collective is the
 * all_reduce of accumulated_tpe, src/modeling/ffn/moe.py:150-151).  Experts are sharded contiguously
 * over `world` GPUs of one box, tokens stay on their home rank, the router is replicated.  The two
 * exchange steps are fused into the neighbouring kernels: bibo_moe_ep_dispatch writes token rows
 * straight into the owner ranks' receive buffers (peer stores), bibo_moe_ep_combine reads result rows
 * straight from the owner ranks' y buffers (peer loads).  The caller provides peer-mapped buffers
 * (xp_peers[r], y_peers[r] = rank r's receive / result buffer [rows_cap_recv, H] as mapped into THIS
 * process), the all-gathered histograms cnt_all [world, E] (counts of bibo_moe_plan of every rank),
 * and a cross-rank barrier on the stream between dispatch -> experts and experts -> combine.
 * ep_plan layout: [0]=n_tiles [1]=rows used [2]=sticky status (4 = a receive buffer would overflow:
 * nothing is written, the caller must raise rows_cap_recv) then send_base[E], recv_off[E+1],
 * recv_cnt[E], tiles; bibo_moe_ep_plan_off(which, E) returns the word offsets (0..3).              */
int64_t bibo_moe_ep_plan_words(int n_experts, int64_t rows_cap_recv);
int64_t bibo_moe_ep_plan_off(int which, int n_experts);
int bibo_moe_ep_plan(const int32_t* cnt_all, int rank, int world, int n_experts, int64_t rows_cap_recv,
                     int32_t* ep_plan, void* stream);
/* source_major != 0: the receive buffer holds all rows of source rank 0, then of source 1, ... (groups
 * in the order s, le instead of le, s), so the rows exchanged between two ranks are one contiguous
 * range on both sides (bibo_moe_ep_forward_dma); per-expert row ranges then do not exist.          */
int bibo_moe_ep_plan_layout(const int32_t* cnt_all, int rank, int world, int n_experts,
                            int64_t rows_cap_recv, int source_major, int32_t* ep_plan, void* stream);
int bibo_moe_ep_dispatch(const void* x, const int32_t* topk_idx, const int32_t* slot_rank,
                         const int32_t* local_plan, const int32_t* ep_plan, void* const* xp_peers,
                         int64_t n_tokens, int hidden, int n_experts, int rank, int world, int top_k,
                         int64_t rows_cap_recv, int comm_ctas, int32_t* slot_row, int32_t* row_token,
                         void* stream);
/* gate/up + radial + down on the rows this rank received; gate_up_proj / down_proj / theta hold only
 * this rank's E/world experts.  max_ctas > 0 bounds the persistent grids (leaves SMs to concurrent
 * dispatch / combine kernels of another token chunk).                                              */
int bibo_moe_ep_experts(const void* xp_recv, const void* gate_up_proj, const void* down_proj,
                        const float* theta, const int32_t* ep_plan, int hidden, int inter, int n_experts,
                        int world, int64_t rows_cap_recv, int max_ctas, void* h, void* y_recv,
                        void* gate_up_out, float* rnorm_out, int zero_padding, void* stream);
/* Stream-ordered barrier over the ranks: flags_peers[r] = rank r's zero-initialised int32[8] flag array
 * as mapped into this process; epoch must grow by one per call.  The wait inside is bounded (about
 * two seconds); on timeout *status is raised to 5 and the kernel returns.                          */
int bibo_moe_ep_barrier(void* const* flags_peers, int rank, int world, int epoch, int32_t* status,
                        void* stream);
/* The same with the number of polls (about 0.5 us each) chosen by the caller; max_polls <= 0 or beyond
 * 2^22 means the default.  A caller that wants a short failure-detection timeout, or a test that makes
 * the wait run out on purpose (a flag nobody writes), passes a small number: the kernel then raises
 * *status to 5 and returns, the context stays usable.                                               */
int bibo_moe_ep_barrier_bounded(void* const* flags_peers, int rank, int world, int epoch, int64_t max_polls,
                                int32_t* status, void* stream);
int bibo_moe_ep_combine(void* const* y_peers, const int32_t* slot_row, const float* topk_w,
                        const int32_t* ep_plan, int64_t n_tokens, int hidden, int world, int top_k,
                        int64_t rows_cap_recv, int comm_ctas, void* out, void* stream);

/* The whole expert-parallel forward of one token slice in one call: router, local plan, histogram
 * exchange through peer memory (cnt_peers[r] = rank r's int32 [world, E] table), EP plan, dispatch,
 * experts, combine, with the three stream barriers in between (epochs epoch_base+1..+3; the caller
 * advances epoch_base by 3 per call).  comm_ctas > 0 caps the dispatch / combine grids and max_ctas
 * caps the GEMM grids, so that slices running on different streams overlap their NVLink phases with
 * each other's GEMMs instead of competing for the same SMs.                                        */
typedef struct {
  int64_t n_tokens, rows_cap_recv;
  int hidden, inter, n_experts, top_k, norm_mode, rank, world, max_ctas, comm_ctas, epoch_base;
  float scale;
  const void* x; const void* w_router; const float* bias;
  const void* gate_up_proj; const void* down_proj; const float* theta;      /* this rank's E/world experts */
  int32_t* topk_idx; float* topk_w; int32_t* slot_rank; int32_t* block_counts;
  int32_t* local_plan; int32_t* ep_plan; int32_t* slot_row;
  void* h;                                                                  /* [rows_cap_recv, I] local */
  void* const* xp_peers; void* const* y_peers; void* const* flags_peers; void* const* cnt_peers;
  void* out;
  /* training only (all NULL for inference): raw gate|up rows [rows_cap_recv, 2I] and row norms
   * [rows_cap_recv] of the received rows, and the token of every row of the local expert-sorted
   * order [N*k + E*127]; with these set the padding rows of the receive buffer are zeroed.       */
  void* gate_up_recv; float* rnorm_recv; int32_t* row_token;
  const bibo_moe_router_trace* trace; /* optional HOST struct: diagnostics of this rank's own tokens */
} bibo_moe_ep_args;
int bibo_moe_ep_forward(const bibo_moe_ep_args* args, void* stream);

/* The same forward with the two exchange steps done by asynchronous peer copies (copy engines)
 * instead of SM kernels, so that token slices on different streams overlap their exchange with each
 * other's GEMMs without sharing SMs.  The home rank sorts its rows by expert into xp_send (the
 * single-GPU permute); the rows for owner o are then one range, copied into o's receive buffer
 * (source-major layout); results come back the same way into the home rank's y_home buffer, in its
 * own expert-sorted layout, and the single-GPU combine finishes.  The copy sizes depend on the
 * routing: the call reads the histogram table on the host (cnt_host, pinned int32 [world*E]) and
 * therefore synchronises with `stream` once, after the router.  args->y_peers, comm_ctas and the
 * training fields are not used; inference only.  Epochs as in bibo_moe_ep_forward.                 */
typedef struct {
  void* xp_send;               /* local [N*k + E*127 rounded, H]: this rank's rows sorted by expert      */
  void* y_owner;               /* local [rows_cap_recv, H]: results of this rank's experts                */
  void* const* y_home_peers;   /* y_home_peers[r] = rank r's [N*k + E*127 rounded, H] buffer, peer-mapped  */
  int32_t* row_token;          /* local [N*k + E*127 rounded] scratch                                       */
  int32_t* cnt_host;           /* pinned host int32 [world*E]                                               */
  void* counts_ready;          /* a cudaEvent_t of the caller, one per token slice                          */
  int n_aux;                   /* 0, or the number of auxiliary streams (at most 8)                         */
  void* const* aux_streams;    /* n_aux cudaStream_t of this token slice: the copies to different peers run on
                                  them at the same time (forked from and joined into `stream`)              */
  void* const* aux_events;     /* 18 cudaEvent_t (timing disabled) used for that fork / join                */
  void* const* marks;          /* NULL, or 9 cudaEvent_t recorded on the stream: start, histograms exchanged,
                                  rows sorted, rows sent, all rows received, experts done, results sent, all
                                  results received, combined                                                 */
} bibo_moe_ep_dma;
/* phase 0 = the whole forward; 1 = up to the point where the host must read the table; 2 = the rest
 * (a caller with several token slices issues phase 1 of all slices, then phase 2 of each).          */
int bibo_moe_ep_forward_dma(const bibo_moe_ep_args* args, const bibo_moe_ep_dma* dma, int phase, void* stream);

/* Backward of bibo_moe_ep_forward (bf16, shapes of the tensor-core backward kernels).  `fwd` is the
 * argument block of the matching forward, run with gate_up_recv / rnorm_recv / row_token set; its
 * buffers are consumed (y becomes dXp, gate_up_recv becomes dGate|dUp).  dy_peers[r] = rank r's
 * dY receive buffer [rows_cap_recv, H] as mapped here.  Outputs: dx [N,H]; d_w_router [E,H] = the
 * LOCAL tokens' contribution (all-reduce it across ranks like any replicated parameter);
 * d_gate_up_proj / d_down_proj / d_theta for this rank's E/world experts.  Uses barrier epochs
 * epoch_base+1 .. epoch_base+2.                                                                  */
typedef struct {
  const void* dout;            /* [N,H] */
  void* const* dy_peers;
  void* dh;                    /* [rows_cap_recv, I] */
  float* dw;                   /* [N,k] */
  float* dlogit_row;           /* [N*k + E*127] */
  float* dtheta_row;           /* [rows_cap_recv] */
  void* dx; void* d_w_router; void* d_gate_up_proj; void* d_down_proj; float* d_theta;
  int epoch_base;
} bibo_moe_ep_bwd_args;
int bibo_moe_ep_backward(const bibo_moe_ep_args* fwd, const bibo_moe_ep_bwd_args* bwd, void* stream);

/* ---- expert-parallel forward with a de-duplicated exchange ---------------------------------------------
 * No counterpart in the reference (the reference states the need for expert parallelism with a replicated
 * router, AGENTS.md:174,199,703, and has none).  Same sharding as above, but a token row crosses NVLink once
 * per DESTINATION RANK instead of once per selected expert, and one partial result row per (token, rank)
 * comes back: with 64 experts and top-6, 0.99 / 2.50 / 3.96 rows per token and direction at 2 / 4 / 8 ranks
 * instead of 2.98 / 4.49 / 5.25.  Every rank provides four peer-mapped buffers:
 *   xu   [world*n_cap, H] bf16   received rows, slot v = source*n_cap + token (no compaction, so a sender
 *                                needs nothing from anybody before it stores)
 *   midx [world*n_cap, k] int32  local expert index of every slot (-1: slot of another rank / no such token)
 *   mw   [world*n_cap, k] fp32   routing weights
 *   part [world*n_cap, H] bf16   on the home rank: part[d*n_cap + t] = owner d's contribution to token t
 * n_cap = the largest token count of any rank.  The owner runs the caller-routed single-GPU chain (rank with
 * empty slots, plan, permute, gate/up, down) over the world*n_cap virtual tokens of its receive buffer with
 * its E/world experts and then sums each virtual token's local slots (fp32, in slot order: ascending expert
 * for the router's lists; a caller's list may be in any order and may hold -1 for unused slots) into ONE bf16
 * row stored into the home rank's `part`; the home rank adds the partial rows of the owners a token went to
 * in ascending owner order.  Same summation order as one GPU, one extra bf16 rounding per owner: inside the
 * bf16 parity bars of the fp32 oracle, not bit-identical to the single-GPU chain.
 * Buffers of the owner chain are sized for the worst case (every slot of every token on this rank):
 * bibo_moe_ep_dedup_rows_cap rows for xp / h / y / row_token, bibo_moe_ep_dedup_plan_words for plan,
 * [world*n_cap, k] for slot_rank / slot_row, [router_blocks(world*n_cap), E/world] for block_counts.
 * The stage entry points take explicit pointers, so several ranks can also be played one after another on
 * ONE device (no kernel waits on another kernel): that is how the single-GPU tests cover this path.      */
int64_t bibo_moe_ep_dedup_rows_cap(int world, int64_t n_cap, int top_k, int n_experts);
int64_t bibo_moe_ep_dedup_plan_words(int world, int64_t n_cap, int top_k, int n_experts);
int64_t bibo_moe_ep_dedup_virtual_tokens(int world, int64_t n_cap);
/* home rank: rows to the distinct owners of each token, routing records to every rank.  midx_peers / mw_peers
 * may be NULL: then only rows are stored and the caller ships the records as block copies of its top-k table
 * (bibo_moe_ep_copy_to_peers into a raw table, bibo_moe_ep_localize on the owner).                         */
int bibo_moe_ep_dedup_dispatch(const void* x, const int32_t* topk_idx, const float* topk_w,
                               void* const* xu_peers, void* const* midx_peers, void* const* mw_peers,
                               int64_t n_tokens, int64_t n_cap, int hidden, int n_experts, int rank,
                               int world, int top_k, int comm_ctas, void* stream);
typedef struct {
  int64_t n_cap;
  int hidden, inter, n_experts, top_k, rank, world, max_ctas, comm_ctas;
  const void* xu; const int32_t* midx; const float* mw;                  /* this rank's receive buffers  */
  const void* gate_up_proj; const void* down_proj; const float* theta;   /* this rank's E/world experts  */
  int32_t* slot_rank; int32_t* block_counts; int32_t* plan; int32_t* slot_row; int32_t* row_token;
  void* xp; void* h; void* y;
  void* const* part_peers;        /* part_peers[s] = rank s's `part` buffer as mapped into this process   */
} bibo_moe_ep_dedup_owner_args;
/* owner rank: experts over the received rows, one partial row per (token, this rank) to the home ranks    */
int bibo_moe_ep_dedup_owner(const bibo_moe_ep_dedup_owner_args* args, void* stream);
/* its two halves: the tensor-core part (rank, plan, permute, gate/up, down) and the NVLink part (partial rows
 * to the home ranks), for callers that run them on different streams (pipelined token slices)             */
int bibo_moe_ep_dedup_experts(const bibo_moe_ep_dedup_owner_args* args, void* stream);
int bibo_moe_ep_dedup_partial(const bibo_moe_ep_dedup_owner_args* args, void* stream);
/* A partial call whose part_peers table points every OTHER home rank s into a local staging buffer
 * (entry s = stage + (s - rank) * n_cap * H * 2 bytes, so that the row lands at stage[s*n_cap + t]) sums at
 * full HBM speed without touching NVLink; bibo_moe_ep_dedup_push then streams the staged rows of the virtual
 * tokens with local slots to the home ranks (a pure copy: a few SMs saturate the links).                    */
int bibo_moe_ep_dedup_push(const void* stage, const int32_t* midx, void* const* part_peers, const int32_t* plan,
                           int64_t n_cap, int hidden, int top_k, int rank, int world, int comm_ctas, void* stream);
/* home rank: out[t] = sum of the partial rows of token t's owners; `status` = a device word, the kernel
 * does nothing when it is non-zero (pass the owner plan's status word)                                    */
int bibo_moe_ep_dedup_final(const void* part, const int32_t* topk_idx, const int32_t* status, int64_t n_tokens,
                            int64_t n_cap, int hidden, int n_experts, int world, int top_k, int comm_ctas,
                            void* out, void* stream);
/* The same exchange on the COPY ENGINES, dense: every rank copies ALL its token rows and its whole top-k table
 * to every peer (an all-gather: the slot layout makes each rank's rows one contiguous block of the receiver's
 * xu), the owner keeps the slots of its own experts (bibo_moe_ep_localize turns the gathered GLOBAL indices
 * into local ones, -1 elsewhere) and stores its partial rows into a local staging buffer laid out by home rank,
 * whose blocks go back as one copy per peer.  More bytes than the kernels above send (world-1 rows per token
 * instead of the distinct owners), but no SM and next to no interference with the grouped GEMMs of another token
 * slice: the better trade while (world-1) is close to the distinct-owner count (2 and 4 ranks).
 * bibo_moe_ep_copy_to_peers: dst_peers[d] + dst_offset <- src + d*src_stride, `bytes` each, as asynchronous
 * copies on `stream`, peers in the order rank+1, rank+2, ...; the own rank only with include_self.          */
int bibo_moe_ep_localize(const int32_t* raw_idx, int64_t n_virtual, int top_k, int n_experts, int rank,
                         int world, int32_t* midx, void* stream);
int bibo_moe_ep_copy_to_peers(void* const* dst_peers, int64_t dst_offset, const void* src, int64_t src_stride,
                              int64_t bytes, int rank, int world, int include_self, void* stream);
/* router + the three stages with the two stream barriers in between (epochs epoch_base+1, +2; the caller
 * advances epoch_base by 2 per call).  marks: NULL or 8 cudaEvent_t recorded on the stream: start, routed,
 * dispatched, all rows received, experts done, partials stored, all partials received, summed.          */
typedef struct {
  bibo_moe_ep_dedup_owner_args owner;
  int64_t n_tokens;
  int norm_mode, epoch_base;
  float scale;
  const void* x; const void* w_router; const float* bias;
  int32_t* topk_idx; float* topk_w; int32_t* slot_rank_home; int32_t* block_counts_home;
  void* const* xu_peers; void* const* midx_peers; void* const* mw_peers; void* const* flags_peers;
  const void* part_local; void* out;
  void* const* marks;
  const bibo_moe_router_trace* trace;
} bibo_moe_ep_dedup_args;
int bibo_moe_ep_dedup_forward(const bibo_moe_ep_dedup_args* args, void* stream);

/* ---- RMSNorm in front of the block -------------------------------------------------------------------
 * Replaces BiBoRMSNorm.forward (src/modeling/norm.py:19-24) where BiBoDecoderLayer._ffn_forward
 * applies post_attention_layernorm before the feed-forward block (src/modeling/layers.py:57-67):
 * out = weight * T(float(h) * rsqrt(mean(float(h)^2) + eps)), h / out [N,H], weight [H], all in dtype.
 * The residual add of the same function is the `addend` of the combine kernel.                      */
int bibo_moe_rmsnorm_fwd(const void* h, const void* weight, float eps, int64_t n_rows, int hidden, int dtype,
                         void* out, void* stream);
/* Backward (autograd through BiBoRMSNorm.forward in the reference): dh [N,H] and dweight [H] from dy [N,H];
 * partial is fp32 scratch [bibo_moe_rmsnorm_bwd_parts(N), H].  Deterministic (no float atomics).       */
int64_t bibo_moe_rmsnorm_bwd_parts(int64_t n_rows);
int bibo_moe_rmsnorm_bwd(const void* h, const void* weight, const void* dy, float eps, int64_t n_rows,
                         int hidden, int dtype, void* dh, float* partial, void* dweight, void* stream);

/* ---- dense SwiGLU MLP -----------------------------------------------------------------------------
 * Replaces BiBoMLP.forward, `down_proj(act_fn(gate_proj(x)) * up_proj(x))` with act = SiLU
 * (src/modeling/ffn/mlp.py:33-34): the shared expert of the MoE layer (src/modeling/ffn/moe.py:120-127,
 * 174-176) and the dense feed-forward layers.  x [N,H], gate_proj / up_proj [I,H], down_proj [H,I]
 * (the nn.Linear weights as stored) -> y [N,H]; h [N,I] and plan (bibo_moe_mlp_plan_words(N) int32) are
 * scratch.  bf16 with H % 256 == 0 and I % 256 == 0 (bibo_moe_mlp_supported), forward only.  Rounding
 * points as in the reference run in bf16: gate and up outputs, the activation, their product.      */
int64_t bibo_moe_mlp_plan_words(int64_t n_tokens);
int bibo_moe_mlp_supported(int hidden, int inter, int dtype);
/* gate_up_out: NULL, or [N, 2I] receiving the raw gate | up rows (what the backward re-reads).      */
int bibo_moe_mlp_forward(const void* x, const void* gate_proj, const void* up_proj, const void* down_proj,
                         int64_t n_tokens, int hidden, int inter, int dtype, int32_t* plan, void* h, void* y,
                         void* gate_up_out, void* stream);
/* The same with the decoder layer's residual add (src/modeling/layers.py:61-66) in the down kernel's
 * epilogue: y = T(T(mlp(x)) + residual), residual [N,H] (may alias nothing written here; NULL = plain
 * forward).  Tensor-core shapes only (bibo_moe_mlp_supported).                                      */
int bibo_moe_mlp_forward_residual(const void* x, const void* gate_proj, const void* up_proj,
                                  const void* down_proj, int64_t n_tokens, int hidden, int inter, int dtype,
                                  int32_t* plan, void* h, void* y, void* gate_up_out, const void* residual,
                                  void* stream);
/* Backward of bibo_moe_mlp_forward (autograd through BiBoMLP.forward in the reference).  plan, h and
 * gate_up are the forward's (gate_up is overwritten with [dGate | dUp]); gate_up_weight is
 * [gate_proj ; up_proj] stacked [2I, H] and d_gate_up_weight [2I, H] receives their gradients in the
 * same order; dh [N, I] is scratch.  Every output is written in full.                               */
int bibo_moe_mlp_backward(const void* x, const void* gate_up_weight, const void* down_proj, void* gate_up,
                          const void* h, const void* dout, int64_t n_tokens, int hidden, int inter, int dtype,
                          int32_t* plan, void* dh, void* dx, void* d_gate_up_weight, void* d_down_proj,
                          void* stream);

/* ---- routing without any allocation -------------------------------------------------------------
 * No counterpart in the reference: added for callers that cannot allocate device memory (a runtime
 * that reserves all memory up front, or a loop that must not incur cudaMalloc's implicit device
 * synchronisation).  Same routing as bibo_moe_router_fwd followed by bibo_moe_plan, but the three
 * intermediates (slot ranks, per-block histograms, plan) live in a fixed device array inside the
 * library (about 1.1 MB per GPU), so the caller passes only inputs and outputs:
 * topk_idx [N,k] int32 ascending, topk_w [N,k] fp32, counts [E] int32 (tokens per expert).
 * At most BIBO_NOALLOC_MAX_TOKENS tokens per call, otherwise BIBO_ERR_UNSUPPORTED.  The first call
 * on a device resolves the array's address (do it before any stream capture).  All calls on a
 * device share the array: calls whose kernels overlap on the GPU race; serialise them.           */
#define BIBO_NOALLOC_MAX_TOKENS 16384
int bibo_moe_route_noalloc(const void* x, const void* w_router, const float* bias, int64_t n_tokens,
                           int hidden, int n_experts, int top_k, int norm_mode, float scale, int dtype,
                           int32_t* topk_idx, float* topk_w, int32_t* counts, void* stream);
int64_t bibo_moe_route_noalloc_max_tokens(void);
/* The router / plan kernels' status word of the last call on the current device sits inside the shared array
 * and is otherwise unobservable: this copies it into a caller-owned DEVICE word on `stream` (no allocation,
 * no synchronisation; no counterpart in the reference).  n_tokens <= 0 only zeroes `counts`.              */
int bibo_moe_route_noalloc_status(int32_t* status_out, void* stream);

/* Debug: copies plan[0..3] to the host (synchronises `stream`) and returns plan[2] (status).     */
int bibo_moe_debug_plan_header(const int32_t* plan, int32_t* header4_host, void* stream);

/* Number of kernels this library has launched from the calling process so far.                   */
int64_t bibo_moe_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* BIBO_MOE_H_ */
