"""Swap the CUDA kernel chain into the reference's own classes, the way the reference swaps kernels
itself: class-level assignment wrapped in ``torch.compiler.disable``
(ablate/common/patches.py:20-23,177-180,290).

    import bibo_b200
    bibo_b200.install()                      # BiBoMoELayer.forward -> kernel chain
    bibo_b200.install(seam="experts")        # only BiBoFusedExperts.forward(x, idx, w)
    bibo_b200.install(seam="mlp")            # BiBoMLP.forward (dense layers, shared expert) -> SwiGLU kernels
    bibo_b200.install(seam="ffn")            # BiBoDecoderLayer._ffn_forward: norm + block + residual (the
                                             # reference's own "megakernel" seam, patches.py:184-199,290)
    bibo_b200.uninstall()

``ref_moe_module`` is the reference's ``src.modeling.ffn.moe`` module (imported by default; pass it
explicitly when the checkout lives under another package name).  Parameters stay owned by the
reference's modules; nothing is copied.
"""
from __future__ import annotations

import torch

from . import mlp as _mlp
from . import moe as _moe

_saved = {}


def _nc(fn):
    return torch.compiler.disable(fn) if hasattr(torch, "compiler") else fn


def install(ref_moe_module=None, seam: str = "layer") -> None:
    if ref_moe_module is None:
        from src.modeling.ffn import moe as ref_moe_module  # the reference checkout must be importable
    if seam == "layer":
        cls = ref_moe_module.BiBoMoELayer
        _saved.setdefault((cls, "forward"), cls.forward)
        cls.forward = _nc(_moe.layer_forward)
    elif seam == "experts":
        cls = ref_moe_module.BiBoFusedExperts
        _saved.setdefault((cls, "forward"), cls.forward)
        cls.forward = _nc(_moe.experts_forward_seam)
    elif seam == "mlp":
        # the MLP class lives next to the MoE module (src/modeling/ffn/mlp.py); the MoE module imports it
        cls = getattr(ref_moe_module, "BiBoMLP", None)
        if cls is None:
            from src.modeling.ffn.mlp import BiBoMLP as cls
        _saved.setdefault((cls, "forward"), cls.forward)
        cls.forward = _nc(_mlp.mlp_module_forward)
    elif seam == "ffn":
        from src.modeling.layers import BiBoDecoderLayer as cls
        _saved.setdefault((cls, "_ffn_forward"), cls._ffn_forward)
        cls._ffn_forward = _nc(_moe.ffn_forward)
    else:
        raise ValueError(f"seam must be 'layer', 'experts', 'mlp' or 'ffn', got {seam!r}")


def uninstall() -> None:
    for (cls, name), fn in _saved.items():
        setattr(cls, name, fn)
    _saved.clear()
