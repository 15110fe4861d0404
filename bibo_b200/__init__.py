"""bibo_b200: the BiBo sparse-MoE feed-forward block as hand-written sm_100a CUDA kernels behind
the reference's PyTorch module API.  See include/bibo_moe.h for the C ABI underneath."""
from .moe import BiBoFusedExperts, BiBoMoELayer, BiBoMoERouter, MoEConfig  # noqa: F401
from .mlp import BiBoMLP  # noqa: F401
from .trace import RouterTrace  # noqa: F401
from . import functional  # noqa: F401
from .install import install, uninstall  # noqa: F401

__all__ = ["BiBoMoELayer", "BiBoMoERouter", "BiBoFusedExperts", "BiBoMLP", "MoEConfig", "RouterTrace", "functional", "install", "uninstall"]
