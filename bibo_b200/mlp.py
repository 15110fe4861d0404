"""Dense SwiGLU MLP with the reference's module interface (src/modeling/ffn/mlp.py:9-34).

``BiBoMLP(config, is_expert=False, intermediate_size=None)`` owns ``gate_proj``, ``up_proj`` and
``down_proj`` as bias-free ``nn.Linear`` modules (state-dict compatible with the reference) and runs
``down_proj(silu(gate_proj(x)) * up_proj(x))`` on the tensor-core kernels of the MoE block
(``bibo_moe_mlp_forward``).  It serves as the shared expert of ``BiBoMoELayer`` and as a dense
feed-forward layer.  On a CUDA device: bf16 at tile-friendly shapes on tensor cores (forward and backward),
float32 and other shapes on CUDA cores (forward and backward); anything else raises.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import functional as Fn

__all__ = ["BiBoMLP", "mlp_module_forward"]


class _MLPFunction(torch.autograd.Function):
    """Forward and backward of the dense MLP as single C-ABI calls (the reference relies on autograd over
    three nn.Linear modules and the activation)."""

    @staticmethod
    def forward(ctx, x, gate_w, up_w, down_w):
        out, saved = Fn.mlp_forward(x, gate_w, up_w, down_w, keep=True)
        ctx.save_for_backward(x, gate_w, up_w, down_w)
        ctx.saved = saved
        return out

    @staticmethod
    def backward(ctx, dout):
        x, gate_w, up_w, down_w = ctx.saved_tensors
        if ctx.saved is None:
            raise RuntimeError("bibo_b200: the MLP's backward ran twice (its saved tensors are consumed)")
        grads = Fn.mlp_backward(dout.contiguous(), x, gate_w, up_w, down_w, ctx.saved)
        ctx.saved = None
        return grads


def mlp_module_forward(mlp, x: torch.Tensor, residual=None) -> torch.Tensor:
    """``BiBoMLP.forward`` written against the reference's attribute names only (works on an instance of
    the reference's own class).  ``residual`` (inference, x's shape): returns ``residual + mlp(x)`` with the
    add inside the down kernel where the shapes allow it, by torch otherwise."""
    act = getattr(getattr(mlp, "config", None), "hidden_act", "silu")
    if act not in ("silu", "swish"):
        raise NotImplementedError(f"bibo_b200.BiBoMLP: hidden_act={act!r} (the kernels implement SiLU)")
    weights = (mlp.gate_proj.weight, mlp.up_proj.weight, mlp.down_proj.weight)
    flat = x.reshape(-1, x.shape[-1]).contiguous()
    if torch.is_grad_enabled() and (x.requires_grad or any(w.requires_grad for w in weights)):
        out = _MLPFunction.apply(flat, *weights).view(x.shape)
        return out if residual is None else residual + out
    if residual is not None:
        if flat.is_cuda and Fn.mlp_residual_supported(flat.shape[1], weights[0].shape[0], flat.dtype):
            res = residual.reshape(-1, x.shape[-1]).contiguous()
            return Fn.mlp_forward(flat, *weights, residual=res).view(x.shape)
        return residual + Fn.mlp_forward(flat, *weights).view(x.shape)
    return Fn.mlp_forward(flat, *weights).view(x.shape)


class BiBoMLP(nn.Module):
    def __init__(self, config, is_expert: bool = False, intermediate_size=None):
        super().__init__()
        self.config = config
        self.hidden_size = config.hidden_size
        self.intermediate_size = intermediate_size if intermediate_size is not None else (
            config.moe_intermediate_size if is_expert else config.intermediate_size)
        self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.down_proj = nn.Linear(self.intermediate_size, self.hidden_size, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return mlp_module_forward(self, x)
