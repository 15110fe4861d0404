"""Drop-in modules for the BiBo sparse-MoE block, backed by libbibo_moe.so.

The three classes mirror the reference's module API so that checkpoints, hooks and callers keep
working when the classes are swapped (``bibo_b200.install``):

* ``BiBoMoERouter``     <- src/modeling/ffn/router.py:10-51
* ``BiBoFusedExperts``  <- src/modeling/ffn/moe.py:19-101
* ``BiBoMoELayer``      <- src/modeling/ffn/moe.py:104-183

Parameter / buffer names and shapes are the reference's: ``gate.gate_proj.weight [E,H]``,
``gate.bias [E]`` (a Parameter with requires_grad=False), ``experts.gate_up_proj [E_glu,2I,H]``,
``experts.down_proj [E_glu,H,I]``, ``experts.radial_theta [E_glu]``, buffer ``accumulated_tpe [E]``.

Every forward runs CUDA kernels; CPU tensors raise.  ``use_shared_expert=True`` adds the reference's
shared SwiGLU expert (``shared_experts_list.0`` = ``bibo_b200.BiBoMLP``, src/modeling/ffn/moe.py:120-127),
bf16.  Configurations outside the kernels' coverage (convolutional shared expert, float16) raise at
construction or call time instead of silently taking another path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import functional as Fn


@dataclass
class MoEConfig:
    """The fields of the reference's BiBoConfig this block reads (src/configuration_bibo.py:39-59,
    103-137).  Any object with these attributes works, including the reference's own config."""
    hidden_size: int = 2048
    moe_intermediate_size: int = 512
    num_routed_experts: int = 64
    num_experts_per_tok: int = 6
    num_pos_identity_experts: int = 0
    num_neg_identity_experts: int = 0
    norm_topk_prob: object = "sum"
    bias_update_factor: float = 0.4
    bias_update_threshold: int = 8000
    initializer_range: float = 0.02
    use_shared_expert: bool = False
    shared_expert_type: str = "mlp"
    num_shared_experts: int = 1
    hidden_act: str = "silu"
    routed_scaling_factor: float = 1.0

    @property
    def num_glu_experts(self) -> int:
        return self.num_routed_experts - self.num_pos_identity_experts - self.num_neg_identity_experts

    @property
    def special_expert_pairs(self) -> int:
        return max(self.num_pos_identity_experts, self.num_neg_identity_experts)


def _cfg(config, name, default=None):
    v = getattr(config, name, default)
    return default if v is None else v


class BiBoMoERouter(nn.Module):
    """Sigmoid router with bias-adjusted top-k selection (src/modeling/ffn/router.py:10-51)."""

    def __init__(self, config):
        super().__init__()
        self.num_routed_experts = config.num_routed_experts
        self.top_k = config.num_experts_per_tok
        norm = _cfg(config, "norm_topk_prob", "sum")
        self.norm_topk_prob = "sum" if norm is True else norm
        self.routed_scaling_factor = float(_cfg(config, "routed_scaling_factor", 1.0))
        self.bias = nn.Parameter(torch.zeros(self.num_routed_experts), requires_grad=False)
        self._probe_gap = False
        self.boundary_gap = None
        self.gate_proj = nn.Linear(config.hidden_size, self.num_routed_experts, bias=False)
        nn.init.normal_(self.gate_proj.weight, mean=0.0, std=_cfg(config, "initializer_range", 0.02))

    def router_logits(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """fp32 logits [N,E] from the router kernel (router.py:25-26)."""
        flat = hidden_states.reshape(-1, hidden_states.shape[-1]).contiguous()
        return Fn.router_forward(flat, self.gate_proj.weight, self.bias, self.top_k, self.norm_topk_prob,
                                 self.routed_scaling_factor, want_logits=True)[4]

    def _set_gap(self, logits: torch.Tensor) -> None:
        # diagnostic only (router.py:33-36); a handful of torch ops on the fp32 logits
        with torch.no_grad():
            tk = torch.sigmoid(logits).topk(self.top_k + 1, dim=-1).values
            self.boundary_gap = (tk[..., self.top_k - 1] - tk[..., self.top_k]).mean()

    def forward(self, hidden_states: torch.Tensor):
        b, s, h = hidden_states.shape
        flat = hidden_states.reshape(b * s, h).contiguous()
        want_gap = self._probe_gap and self.top_k < self.num_routed_experts
        idx, w, _, _, logits = Fn.router_forward(flat, self.gate_proj.weight, self.bias, self.top_k,
                                                 self.norm_topk_prob, self.routed_scaling_factor,
                                                 want_logits=want_gap)
        if want_gap:
            self._set_gap(logits)
        return idx.view(b, s, -1).long(), w.view(b, s, -1)


class BiBoFusedExperts(nn.Module):
    """Stacked expert weights + the expert kernels on caller-supplied routing
    (src/modeling/ffn/moe.py:19-101)."""

    def __init__(self, config):
        super().__init__()
        n_pos = int(_cfg(config, "num_pos_identity_experts", _cfg(config, "special_expert_pairs", 0)))
        n_neg = int(_cfg(config, "num_neg_identity_experts", _cfg(config, "special_expert_pairs", 0)))
        self.num_routed_experts = config.num_routed_experts
        self.num_glu_experts = int(_cfg(config, "num_glu_experts", self.num_routed_experts - n_pos - n_neg))
        self.special_expert_pairs = int(_cfg(config, "special_expert_pairs", 0))
        self.hidden_size = config.hidden_size
        self.intermediate_size = config.moe_intermediate_size
        std = _cfg(config, "initializer_range", 0.02)
        self.gate_up_proj = nn.Parameter(torch.empty(self.num_glu_experts, 2 * self.intermediate_size, self.hidden_size))
        self.down_proj = nn.Parameter(torch.empty(self.num_glu_experts, self.hidden_size, self.intermediate_size))
        nn.init.normal_(self.gate_up_proj, mean=0.0, std=std)
        nn.init.normal_(self.down_proj, mean=0.0, std=std)
        self.radial_theta = nn.Parameter(torch.zeros(self.num_glu_experts))
        self.pos_start = self.num_glu_experts
        self.pos_end = self.pos_start + n_pos
        self.neg_start = self.pos_end
        self.neg_end = self.neg_start + n_neg

    @property
    def num_pos(self) -> int:
        return self.pos_end - self.pos_start

    @property
    def num_neg(self) -> int:
        return self.neg_end - self.neg_start

    def forward(self, hidden_states: torch.Tensor, top_k_indices: torch.Tensor,
                top_k_weights: torch.Tensor) -> torch.Tensor:
        return experts_forward_seam(self, hidden_states, top_k_indices, top_k_weights)


def _refuse_grad(module: nn.Module, *tensors) -> None:
    """The experts-only seam has no backward kernels for caller-supplied routing weights."""
    if not torch.is_grad_enabled():
        return
    if any(t.requires_grad for t in tensors) or any(p.requires_grad for p in module.parameters()):
        raise NotImplementedError(
            "bibo_b200: BiBoFusedExperts.forward(x, idx, w) is forward-only; train through BiBoMoELayer "
            "(whole-block backward) or call this seam under torch.no_grad()")


class _MoEBlockFunction(torch.autograd.Function):
    """Whole-block forward/backward as one autograd node (the reference relies on autograd over ~900
    eager ops per layer; here both directions are single C-ABI calls)."""

    @staticmethod
    def forward(ctx, x, w_router, gate_up_proj, down_proj, theta, bias, cfg, holder, addend=None):
        top_k, norm, scale, n_pos, n_neg, trace = cfg
        n, hidden = x.shape
        geo = Fn.Geometry(n, hidden, gate_up_proj.shape[1] // 2, w_router.shape[0], gate_up_proj.shape[0], n_pos, top_k,
                          x.dtype)
        # a private workspace: its tensors are what the backward pass re-reads
        # the fp32 logits are kept as well: the backward reads the selected ones instead of recomputing them
        ws = Fn.MoEWorkspace(geo, x.device, keep_logits=True, keep_gate_up=True)
        out, ws = Fn.moe_forward(x, w_router, bias, gate_up_proj, down_proj, theta, top_k, norm, scale, n_pos=n_pos,
                                 n_neg=n_neg, ws=ws, zero_padding=True, addend=addend, trace=trace)
        ctx.save_for_backward(x, w_router, gate_up_proj, down_proj, theta)
        ctx.ws, ctx.norm, ctx.scale = ws, norm, scale
        ctx.has_addend = addend is not None
        holder["ws"] = ws
        return out

    @staticmethod
    def backward(ctx, dout):
        x, w_router, gate_up_proj, down_proj, theta = ctx.saved_tensors
        if ctx.ws is None:
            raise RuntimeError("bibo_b200: the MoE block's backward ran twice (its workspace is consumed)")
        dx, d_wr, d_gu, d_dn, d_th = Fn.moe_backward(dout.contiguous(), x, w_router, gate_up_proj, down_proj, theta,
                                                     ctx.ws, ctx.norm, ctx.scale)
        ctx.ws = None
        # the addend (shared expert output) enters the result by a plain sum: its gradient is dout
        return dx, d_wr, d_gu, d_dn, d_th.to(theta.dtype), None, None, None, (dout if ctx.has_addend else None)


class BiBoMoELayer(nn.Module):
    """Router -> experts -> weighted combine, one C-ABI call (src/modeling/ffn/moe.py:104-183)."""

    def __init__(self, config):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_routed_experts = config.num_routed_experts
        self.num_experts_per_tok = config.num_experts_per_tok
        self.bias_update_factor = _cfg(config, "bias_update_factor", 0.4)
        self.bias_update_threshold = _cfg(config, "bias_update_threshold", 8000)
        self.register_buffer("accumulated_tpe", torch.zeros(config.num_routed_experts, dtype=torch.float))
        self._fwd_step = 0
        self._update_every = None
        self.experts = BiBoFusedExperts(config)
        self.use_shared_expert = bool(_cfg(config, "use_shared_expert", False))
        self.shared_experts_list = nn.ModuleList()
        if self.use_shared_expert:
            # moe.py:120-127: one SwiGLU MLP of width moe_intermediate_size * num_shared_experts
            if _cfg(config, "shared_expert_type", "mlp") == "conv":
                raise NotImplementedError("bibo_b200.BiBoMoELayer: shared_expert_type='conv' is outside the kernels' "
                                          "coverage")
            from .mlp import BiBoMLP
            n_sh = int(_cfg(config, "num_shared_experts", 1))
            self.shared_experts_list.append(BiBoMLP(config, is_expert=True,
                                                    intermediate_size=config.moe_intermediate_size * n_sh))
        self.gate = BiBoMoERouter(config)
        self.last_workspace: Optional[Fn.MoEWorkspace] = None

    # ---- load balancer: host logic unchanged from the reference (moe.py:131-155) --------------------
    @torch.no_grad()
    def update_bias(self, tokens_per_expert: torch.Tensor):
        if self.bias_update_factor <= 0:
            return
        share = tokens_per_expert.detach().float()
        share = share / share.sum().clamp_min(1.0)
        self.gate.bias.add_(self.bias_update_factor * (share.mean() - share))

    @torch.no_grad()
    def _balance_step(self, top_k_indices: torch.Tensor, num_tokens: int):
        """Reference signature (indices [B,S,k]); the forward itself feeds the kernel's histogram."""
        counts = torch.bincount(top_k_indices.reshape(-1), minlength=self.num_routed_experts)
        return _balance_from_counts(self, counts, num_tokens)

    # ---- forward -------------------------------------------------------------------------------------
    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return layer_forward(self, hidden_states)


def _balance_from_counts(layer, counts: torch.Tensor, num_tokens: int):
    """`_balance_step` of the reference (moe.py:139-155) fed with the kernel's histogram.

    As in the reference, the histogram is accumulated in the dtype of the ``accumulated_tpe`` buffer: a module
    cast with ``.to(torch.bfloat16)`` carries a bf16 buffer, which rounds counts above 256.  Callers that want
    exact counts keep that buffer fp32 (``layer.accumulated_tpe = layer.accumulated_tpe.float()``)."""
    with torch.no_grad():
        layer.accumulated_tpe += counts.float()
        if layer._update_every is None:
            layer._update_every = max(1, round(layer.bias_update_threshold / max(num_tokens, 1)))
        layer._fwd_step += 1
        if layer._fwd_step % layer._update_every == 0:
            if dist.is_available() and dist.is_initialized():
                dist.all_reduce(layer.accumulated_tpe, op=dist.ReduceOp.SUM)
            tpe = layer.accumulated_tpe.clone()
            layer.accumulated_tpe.zero_()
            return tpe
    return None


def layer_forward(layer, hidden_states: torch.Tensor, residual: Optional[torch.Tensor] = None,
                  fused_norm=None) -> torch.Tensor:
    """``BiBoMoELayer.forward`` (src/modeling/ffn/moe.py:157-183) on the CUDA kernel chain.

    Written against the REFERENCE's attribute names only, so it serves both this package's layer
    and, through ``bibo_b200.install``, an instance of the reference's own class.
    ``residual`` (same shape; used by ``ffn_forward``) is added to the result, inside the combine
    kernel when the layer has no shared expert.  ``fused_norm`` = (norm weight, eps), inference only and
    only where ``fused_ffn_applies`` says so: ``hidden_states`` is then the raw residual stream, the
    RMSNorm happens inside the router's and the permute's loads and the stream itself is added to the
    result (``bibo_moe_ffn_forward``).
    """
    bsz, seq_len, hidden = hidden_states.shape
    n = bsz * seq_len
    flat = hidden_states.reshape(n, hidden).contiguous()
    shared_out = None
    if getattr(layer, "use_shared_expert", False):
        # moe.py:174-176: final = routed + shared(hidden_states); the sum happens in the combine kernel
        from .mlp import mlp_module_forward
        shared = layer.shared_experts_list[0]
        if not hasattr(shared, "gate_proj"):
            raise NotImplementedError("bibo_b200: only the MLP shared expert is covered by the kernels")
        shared_out = mlp_module_forward(shared, flat)          # its own autograd node when gradients are on
    late_residual = None
    if residual is not None:
        if shared_out is None:
            shared_out = residual.reshape(n, hidden).contiguous()   # the combine kernel's second term
        else:
            late_residual = residual
    gate, ex = layer.gate, layer.experts
    n_pos, n_neg = ex.pos_end - ex.pos_start, ex.neg_end - ex.neg_start
    want_gap = gate._probe_gap and gate.top_k < gate.num_routed_experts
    scale = float(getattr(gate, "routed_scaling_factor", 1.0))
    # routing diagnostics come out of the router / plan kernels themselves (no extra launches): the sums
    # of an attached bibo_b200.RouterTrace, and the boundary gap of router.py:33-36 when it is probed
    tracer = getattr(layer, "_router_trace", None)
    trace = tracer.buffers(layer) if tracer is not None else None
    if want_gap:
        gap = torch.empty(1, dtype=torch.float32, device=flat.device)
        trace = (trace[0], trace[1], gap) if trace is not None else (None, None, gap)
    params = (gate.gate_proj.weight, ex.gate_up_proj, ex.down_proj, ex.radial_theta)
    if torch.is_grad_enabled() and (flat.requires_grad or any(p.requires_grad for p in params)):
        if fused_norm is not None:
            raise RuntimeError("bibo_b200: the fused norm path has no backward; call it under torch.no_grad()")
        holder = {}
        out = _MoEBlockFunction.apply(flat, *params, gate.bias.detach(),
                                      (gate.top_k, gate.norm_topk_prob, scale, n_pos, n_neg, trace), holder,
                                      shared_out)
        ws = holder["ws"]
    elif fused_norm is not None:
        out, ws = Fn.ffn_forward(flat, fused_norm[0], fused_norm[1], gate.gate_proj.weight, gate.bias, ex.gate_up_proj,
                                 ex.down_proj, ex.radial_theta, gate.top_k, gate.norm_topk_prob, scale, trace=trace,
                                 n_pos=n_pos, n_neg=n_neg)
    else:
        out, ws = Fn.moe_forward(flat, gate.gate_proj.weight, gate.bias, ex.gate_up_proj, ex.down_proj,
                                 ex.radial_theta, gate.top_k, gate.norm_topk_prob, scale,
                                 n_pos=n_pos, n_neg=n_neg, addend=shared_out, trace=trace)
    layer.last_workspace = ws
    if want_gap:
        gate.boundary_gap = gap[0]
    # replay the reference's diagnostic hook points only when someone is listening
    if ex._forward_pre_hooks:
        for hook in ex._forward_pre_hooks.values():
            hook(ex, (flat, ws.topk_idx.long(), ws.topk_w))
    if gate._forward_hooks:
        res = (ws.topk_idx.view(bsz, seq_len, -1).long(), ws.topk_w.view(bsz, seq_len, -1))
        for hook in gate._forward_hooks.values():
            hook(gate, (hidden_states,), res)
    if layer.training and layer.bias_update_factor > 0:
        tpe = _balance_from_counts(layer, ws.counts(), n)
        if tpe is not None:
            layer.update_bias(tpe)
    out = out.view(bsz, seq_len, hidden)
    return out if late_residual is None else late_residual + out


class _RMSNormFunction(torch.autograd.Function):
    """BiBoRMSNorm forward / backward as single C-ABI calls (src/modeling/norm.py:19-24)."""

    @staticmethod
    def forward(ctx, h, weight, eps):
        ctx.save_for_backward(h, weight)
        ctx.eps = eps
        return Fn.rmsnorm_forward(h, weight, eps)

    @staticmethod
    def backward(ctx, dy):
        h, weight = ctx.saved_tensors
        dh, dw = Fn.rmsnorm_backward(dy, h, weight, ctx.eps)
        return dh, dw.to(weight.dtype), None


def ffn_forward(decoder_layer, hidden_states: torch.Tensor) -> torch.Tensor:
    """``BiBoDecoderLayer._ffn_forward`` (src/modeling/layers.py:57-67): post-attention RMSNorm, the
    feed-forward block and the residual add.  Inference runs the norm kernel and folds the residual add
    into the combine kernel; with gradients on, norm and block run through their autograd nodes (kernels
    in both directions) and the residual add is torch's.  Written against the reference's attribute
    names (``post_attention_layernorm``, ``mlp``, ``_bf16_moe_out``, ``_bf16_stream``)."""
    from .mlp import mlp_module_forward
    mlp, norm = decoder_layer.mlp, decoder_layer.post_attention_layernorm
    is_moe = hasattr(mlp, "gate") and hasattr(mlp, "experts")
    block = (lambda x, res=None: layer_forward(mlp, x, res)) if is_moe else (lambda x, res=None: mlp_module_forward(mlp, x))
    bf16_out = bool(getattr(decoder_layer, "_bf16_moe_out", False))
    bf16_stream = bool(getattr(decoder_layer, "_bf16_stream", False))
    needs_grad = torch.is_grad_enabled() and (hidden_states.requires_grad or
                                              any(p.requires_grad for p in decoder_layer.parameters()))
    plain = hidden_states.dtype == torch.bfloat16 or not (bf16_out or bf16_stream)   # the casts are no-ops
    if needs_grad or not plain:
        shape = hidden_states.shape
        if hidden_states.is_cuda and norm.weight.dtype == hidden_states.dtype:
            x = _RMSNormFunction.apply(hidden_states.reshape(-1, shape[-1]).contiguous(), norm.weight,
                                       norm.variance_epsilon).view(shape)
        else:
            x = norm(hidden_states)
        out = block(x)
        if bf16_out:
            out = out.to(torch.bfloat16)
        hidden_states = hidden_states + out
        return hidden_states.to(torch.bfloat16) if bf16_stream else hidden_states
    shape = hidden_states.shape
    if is_moe and fused_ffn_applies(mlp, hidden_states, norm):
        return layer_forward(mlp, hidden_states, fused_norm=(norm.weight, float(norm.variance_epsilon)))
    flat = hidden_states.reshape(-1, shape[-1]).contiguous()
    x = Fn.rmsnorm_forward(flat, norm.weight, norm.variance_epsilon).view(shape)
    if is_moe:
        return block(x, hidden_states)
    return mlp_module_forward(mlp, x, residual=hidden_states)     # the add happens in the down kernel's epilogue


def fused_ffn_applies(layer, hidden_states: torch.Tensor, norm) -> bool:
    """Whether ``bibo_moe_ffn_forward`` covers this layer and input: bf16 on a CUDA device, 64 routed experts,
    no shared expert (it reads the normalised activations, which the fused path never writes), and nobody
    listening on the hooks that hand those activations out."""
    gate, ex = layer.gate, layer.experts
    if not hidden_states.is_cuda or hidden_states.dtype != torch.bfloat16 or norm.weight.dtype != torch.bfloat16:
        return False
    if getattr(layer, "use_shared_expert", False):
        return False
    if ex._forward_pre_hooks or gate._forward_hooks:
        return False
    return Fn.ffn_supported(hidden_states.shape[-1], ex.gate_up_proj.shape[1] // 2, gate.num_routed_experts, gate.top_k)


def experts_forward_seam(experts, hidden_states: torch.Tensor, top_k_indices: torch.Tensor,
                         top_k_weights: torch.Tensor) -> torch.Tensor:
    """``BiBoFusedExperts.forward(x, idx, w)`` (src/modeling/ffn/moe.py:47-101) on the kernels."""
    _refuse_grad(experts, hidden_states, top_k_weights)
    out, _ = Fn.experts_forward(hidden_states.contiguous(), top_k_indices, top_k_weights, experts.gate_up_proj,
                                experts.down_proj, experts.radial_theta, experts.num_routed_experts,
                                experts.pos_end - experts.pos_start)
    return out
