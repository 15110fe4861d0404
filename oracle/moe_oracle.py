"""CPU oracle for the BiBo sparse-MoE feed-forward block.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch ops on whatever device its inputs live on (CPU in the
test-suite), the algorithm of the reference's eager MoE block so that the CUDA path can be
checked against it on a machine that does not hold the reference checkout.  It is never
imported by the product package: only the tests, the smoke entry and the benchmark's CPU
baseline leg use it.

Parity of this restatement is PINNED: ``tests/golden/make_golden.py`` imports the reference's own
``BiBoMoELayer`` and stores its outputs and gradients for seeded inputs; ``tests/test_oracle.py``
replays those fixtures through the functions below.

Reference lines each function follows (paths inside the reference project):

* ``router_logits``      src/modeling/ffn/router.py:25-26
* ``router_select``      src/modeling/ffn/router.py:28-51  (sigmoid, +bias for selection only,
                         top-k, gather un-biased scores, "sum" / "softmax" / raw weights)
* ``radial_normsilu``    src/modeling/ffn/moe.py:16,87-90
* ``experts_forward``    src/modeling/ffn/moe.py:47-101    (sort by expert, per-expert loop,
                         fp32 ``index_add_`` in ascending expert order, ±Identity tails)
* ``balance_step`` / ``update_bias``   src/modeling/ffn/moe.py:131-155
* ``moe_forward``        src/modeling/ffn/moe.py:157-183

Two deliberate definitions where the reference leaves behaviour to ``torch.topk``:

* ties in the biased selection score are broken towards the LOWER expert index (the reference's
  ``topk(sorted=False)`` order is implementation-defined);
* the k selected experts are returned in ASCENDING expert index, with their weights in the same
  order (the reference returns them in ``topk``'s unspecified order).  Compare against the
  reference on sorted index sets.

``routed_scaling_factor`` multiplies the normalised weights; the reference's current source has no
such field (only historical documents name it), so values other than 1.0 have no reference to pin
against.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

NORMSILU_EPS = 1e-6          # src/modeling/ffn/moe.py:16
SUM_NORM_EPS = 1e-20         # src/modeling/ffn/router.py:45


# --------------------------------------------------------------------------------------------
# router
# --------------------------------------------------------------------------------------------
def router_logits(x: torch.Tensor, w_router: torch.Tensor) -> torch.Tensor:
    """[N,H] x [E,H]^T in the model dtype, then widened to fp32 (router.py:25-26)."""
    return F.linear(x, w_router).float()


def router_select(
    logits: torch.Tensor,
    bias: torch.Tensor,
    top_k: int,
    norm_topk_prob="sum",
    routed_scaling_factor: float = 1.0,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """fp32 logits [N,E] -> (idx int64 [N,k] ascending, weights fp32 [N,k], counts int64 [E]).

    Selection runs on ``sigmoid(logits) + bias``; the weights are gathered from the UN-biased
    scores (router.py:38-41).  Ties go to the lower expert index.
    """
    scores = torch.sigmoid(logits.float())
    sel = scores + bias.to(scores.dtype)
    # stable descending sort: equal keys keep ascending index order -> lowest index wins a tie
    order = torch.sort(sel, dim=-1, descending=True, stable=True).indices
    idx = torch.sort(order[:, :top_k], dim=-1).values
    w = scores.gather(-1, idx)
    if top_k > 1 and norm_topk_prob == "softmax":
        w = F.softmax(w, dim=-1)
    elif top_k > 1 and norm_topk_prob:
        w = w / (w.sum(dim=-1, keepdim=True) + SUM_NORM_EPS)
    if routed_scaling_factor != 1.0:
        w = w * routed_scaling_factor
    counts = torch.bincount(idx.flatten(), minlength=logits.shape[-1])
    return idx.long(), w.float(), counts


def boundary_gap(logits: torch.Tensor, bias: torch.Tensor, top_k: int) -> torch.Tensor:
    """Per-token gap between the k-th and (k+1)-th BIASED selection score, in fp64.

    Used by the parity tests to adjudicate tokens whose selection legitimately depends on the
    last bit of the sigmoid (a flip is accepted only where this gap is below the stated noise).
    """
    sel = torch.sigmoid(logits.double()) + bias.double()
    top = sel.topk(min(top_k + 1, sel.shape[-1]), dim=-1).values
    if top.shape[-1] <= top_k:
        return torch.full((sel.shape[0],), float("inf"), dtype=torch.float64)
    return top[:, top_k - 1] - top[:, top_k]


def probe_gap(logits: torch.Tensor, top_k: int) -> torch.Tensor:
    """Mean un-biased score gap the reference exposes as ``boundary_gap`` (router.py:33-36)."""
    tk = torch.sigmoid(logits if logits.dtype == torch.float64 else logits.float()).topk(top_k + 1, dim=-1).values
    return (tk[..., top_k - 1] - tk[..., top_k]).mean()


def router_trace_sums(logits: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, top_k: int) -> torch.Tensor:
    """What one training forward adds to the reference's RouterTrace accumulator
    (ablate/common/router_trace.py:106-130): [sum max p, sum entropy(p), tokens, sum max w, sum sum w,
    sum min w, mean boundary gap, 1] with p = w / max(sum |w|, 1e-9), in fp64."""
    wr = w.double()
    p = wr / wr.abs().sum(-1, keepdim=True).clamp_min(1e-9)
    ent = -(p.abs() * p.abs().clamp_min(1e-12).log()).sum(-1)
    gap = probe_gap(logits.double(), top_k) if top_k < logits.shape[-1] else torch.zeros(())
    return torch.stack([p.max(-1).values.sum(), ent.sum(), torch.tensor(float(w.shape[0]), dtype=torch.float64),
                        wr.max(-1).values.sum(), wr.sum(), wr.min(-1).values.sum(), gap.double(),
                        torch.tensor(1.0, dtype=torch.float64)])


# --------------------------------------------------------------------------------------------
# experts
# --------------------------------------------------------------------------------------------
def radial_normsilu(gate: torch.Tensor, theta_e: torch.Tensor) -> torch.Tensor:
    """r^p * SiLU(g / r), r = sqrt(mean g^2 + eps), p = sigmoid(theta_e); fp32 inside, result
    cast back to ``gate.dtype`` (moe.py:87-90)."""
    g = gate.float() if gate.dtype != torch.float64 else gate
    r = torch.sqrt(g.square().mean(-1, keepdim=True) + NORMSILU_EPS)
    p = torch.sigmoid(theta_e.to(g.dtype))
    return (F.silu(g / r) * r.pow(p)).to(gate.dtype)


def experts_forward(
    x: torch.Tensor,
    idx: torch.Tensor,
    w: torch.Tensor,
    gate_up_proj: torch.Tensor,
    down_proj: torch.Tensor,
    radial_theta: torch.Tensor,
    num_routed_experts: Optional[int] = None,
    num_pos_identity: int = 0,
    num_neg_identity: int = 0,
) -> torch.Tensor:
    """x [N,H], idx [N,k], w [N,k] fp32 -> [N,H] in x.dtype (moe.py:47-101).

    gate_up_proj [E_glu, 2I, H] (rows [0,I) gate, [I,2I) up), down_proj [E_glu, H, I].
    Rounding points follow the reference: each F.linear result is in the model dtype, the
    activation is computed in fp32 and cast back, the combine accumulates in fp32 in ascending
    expert order and is cast once at the end.
    """
    n_tok, hidden = x.shape
    e_glu = gate_up_proj.shape[0]
    n_routed = e_glu + num_pos_identity + num_neg_identity if num_routed_experts is None else num_routed_experts
    neg_start = e_glu + num_pos_identity

    flat_e = idx.flatten()
    flat_t = torch.arange(n_tok, device=x.device).unsqueeze(1).expand_as(idx).flatten()
    flat_w = w.flatten()
    # stable: rows of one expert stay in ascending token order (the reference's sort is unstable;
    # the order inside an expert cannot change the result because a token meets an expert once)
    order = torch.sort(flat_e, stable=True).indices
    tok_sorted, w_sorted = flat_t[order], flat_w[order]
    bounds = torch.zeros(n_routed + 1, dtype=torch.long)
    bounds[1:] = torch.cumsum(torch.bincount(flat_e.cpu(), minlength=n_routed), 0)
    bounds = bounds.tolist()

    acc_dtype = torch.promote_types(torch.float32, x.dtype)
    out = torch.zeros(n_tok, hidden, device=x.device, dtype=acc_dtype)
    for e in range(n_routed):
        lo, hi = bounds[e], bounds[e + 1]
        if hi == lo:
            continue
        tok = tok_sorted[lo:hi]
        we = w_sorted[lo:hi].unsqueeze(-1)
        xe = x[tok]
        if e < e_glu:
            gate, up = F.linear(xe, gate_up_proj[e]).chunk(2, dim=-1)
            act = radial_normsilu(gate, radial_theta[e])
            y = F.linear(act * up, down_proj[e])
            out = out.index_add(0, tok, y * we)
        elif e < neg_start:
            out = out.index_add(0, tok, xe * we)
        else:
            out = out.index_add(0, tok, xe * -we)
    return out.to(x.dtype)


# --------------------------------------------------------------------------------------------
# load balancer (host logic of the block)
# --------------------------------------------------------------------------------------------
@dataclass
class BalancerState:
    """The mutable state ``BiBoMoELayer`` keeps for its bias balancer (moe.py:111-114)."""
    accumulated_tpe: torch.Tensor
    fwd_step: int = 0
    update_every: Optional[int] = None


def balance_step(state: BalancerState, counts: torch.Tensor, num_tokens: int,
                 bias_update_threshold: int, all_reduce=None) -> Optional[torch.Tensor]:
    """moe.py:139-155.  ``counts`` is the per-expert histogram of this forward; ``all_reduce`` is an
    optional in-place SUM over ranks (the reference calls ``dist.all_reduce``)."""
    state.accumulated_tpe += counts.float()
    if state.update_every is None:
        state.update_every = max(1, round(bias_update_threshold / max(num_tokens, 1)))
    state.fwd_step += 1
    if state.fwd_step % state.update_every == 0:
        if all_reduce is not None:
            all_reduce(state.accumulated_tpe)
        tpe = state.accumulated_tpe.clone()
        state.accumulated_tpe.zero_()
        return tpe
    return None


def update_bias(bias: torch.Tensor, tokens_per_expert: torch.Tensor, bias_update_factor: float) -> None:
    """bias += u * (mean(share) - share), share = tpe / max(sum tpe, 1)  (moe.py:131-137)."""
    if bias_update_factor <= 0:
        return
    share = tokens_per_expert.detach().float()
    share = share / share.sum().clamp_min(1.0)
    bias.add_(bias_update_factor * (share.mean() - share))


# --------------------------------------------------------------------------------------------
# whole block
# --------------------------------------------------------------------------------------------
def moe_forward(
    x: torch.Tensor,
    w_router: torch.Tensor,
    bias: torch.Tensor,
    gate_up_proj: torch.Tensor,
    down_proj: torch.Tensor,
    radial_theta: torch.Tensor,
    top_k: int,
    norm_topk_prob="sum",
    routed_scaling_factor: float = 1.0,
    num_pos_identity: int = 0,
    num_neg_identity: int = 0,
    return_routing: bool = False,
):
    """[B,S,H] (or [N,H]) -> same shape, same dtype (moe.py:157-183, shared expert off)."""
    shape = x.shape
    flat = x.reshape(-1, shape[-1])
    logits = router_logits(flat, w_router)
    idx, w, counts = router_select(logits, bias, top_k, norm_topk_prob, routed_scaling_factor)
    out = experts_forward(flat, idx, w, gate_up_proj, down_proj, radial_theta,
                          num_routed_experts=w_router.shape[0],
                          num_pos_identity=num_pos_identity, num_neg_identity=num_neg_identity)
    out = out.reshape(shape)
    if return_routing:
        return out, logits, idx, w, counts
    return out


def rmsnorm(h: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """BiBoRMSNorm.forward (src/modeling/norm.py:19-24): fp32 statistics, the normalised value cast back to
    the input dtype, then multiplied by the weight."""
    v = h.to(torch.float32)
    v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    return weight * v.to(h.dtype)


def mlp_forward(x: torch.Tensor, gate_proj: torch.Tensor, up_proj: torch.Tensor, down_proj: torch.Tensor):
    """Dense SwiGLU MLP, BiBoMLP.forward with hidden_act = "silu" (src/modeling/ffn/mlp.py:33-34):
    down_proj(silu(gate_proj(x)) * up_proj(x)); weights as nn.Linear stores them ([I,H], [I,H], [H,I])."""
    return F.linear(F.silu(F.linear(x, gate_proj)) * F.linear(x, up_proj), down_proj)


def make_mlp_weights(hidden: int, inter: int, seed: int = 0):
    """Seeded N(0, 0.02) weights of a dense MLP (own generators, like make_inputs)."""
    def gen(i):
        return torch.Generator().manual_seed(seed * 1000 + 20 + i)
    return dict(gate_proj=torch.randn(inter, hidden, generator=gen(1)) * 0.02,
                up_proj=torch.randn(inter, hidden, generator=gen(2)) * 0.02,
                down_proj=torch.randn(hidden, inter, generator=gen(3)) * 0.02)


# --------------------------------------------------------------------------------------------
# seeded synthetic workloads (shapes and distributions of the benchmark configurations)
# --------------------------------------------------------------------------------------------
def make_inputs(n_tokens: int, hidden: int, inter: int, n_experts: int = 64, seed: int = 0,
                bias_mode: str = "zero", theta_std: float = 0.0, zipf_alpha: float = 1.0,
                dtype=torch.float32):
    """One CPU generator per tensor so every consumer sees identical bits.

    x ~ N(0,1); gate/up/down/router weights ~ N(0, 0.02); bias: "zero", "uniform" (U(-0.01, 0.01))
    or "zipf" (alpha * log of a normalised Zipf(s=1.1) profile over the experts);
    theta ~ N(0, theta_std).
    """
    def gen(i):
        return torch.Generator().manual_seed(seed * 1000 + i)
    x = torch.randn(n_tokens, hidden, generator=gen(1))
    w_gu = torch.randn(n_experts, 2 * inter, hidden, generator=gen(2)) * 0.02
    w_d = torch.randn(n_experts, hidden, inter, generator=gen(3)) * 0.02
    w_r = torch.randn(n_experts, hidden, generator=gen(4)) * 0.02
    if bias_mode == "zero":
        bias = torch.zeros(n_experts)
    elif bias_mode == "uniform":
        bias = (torch.rand(n_experts, generator=gen(5)) * 2 - 1) * 0.01
    elif bias_mode == "zipf":
        prof = 1.0 / torch.arange(1, n_experts + 1, dtype=torch.float64) ** 1.1
        bias = (zipf_alpha * torch.log(prof / prof.sum())).float()
    else:
        raise ValueError(bias_mode)
    theta = torch.randn(n_experts, generator=gen(6)) * theta_std
    cast = lambda t: t.to(dtype)
    return dict(x=cast(x), gate_up_proj=cast(w_gu), down_proj=cast(w_d), w_router=cast(w_r),
                bias=bias.float(), radial_theta=theta.float())
