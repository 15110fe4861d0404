"""RMSNorm kernel and the decoder layer's feed-forward half (norm + block + residual) on the GPU against
the reference's own outputs (golden fixture, fp32) and the CPU oracle."""
import pathlib
import types

import pytest
import torch

from conftest import mean_rel_err, rel_err
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
GOLDEN = pathlib.Path(__file__).resolve().parent / "golden"
BF16_MAX, BF16_MEAN = 2e-2, 1e-2


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("n,h", [(1, 64), (300, 256), (1000, 2048), (70, 8192 + 64)])
def test_rmsnorm_kernel_matches_the_oracle(dtype, tol, n, h):
    """Rows held in registers and the long-row loop (h > 8192 bf16 elements per warp pass)."""
    from bibo_b200 import functional as Fn
    g = torch.Generator().manual_seed(n + h)
    x = (torch.randn(n, h, generator=g) * 3).to(dtype)
    w = (1.0 + 0.1 * torch.randn(h, generator=g)).to(dtype)
    out = Fn.rmsnorm_forward(x.to(DEV), w.to(DEV), 1e-6)
    ref = orc.rmsnorm(x, w, 1e-6)
    if dtype == torch.float32:
        assert rel_err(out.cpu(), ref) < tol
    else:   # same rounding points as the reference in bf16: at most one bf16 ulp apart
        assert rel_err(out.float().cpu(), ref.float()) < tol


class _Norm(torch.nn.Module):
    def __init__(self, weight, eps):
        super().__init__()
        self.weight = torch.nn.Parameter(weight)
        self.variance_epsilon = eps

    def forward(self, h):
        return orc.rmsnorm(h, self.weight, self.variance_epsilon)


def _decoder_half(rec, dtype):
    """An object with the attributes ffn_forward reads from the reference's decoder layer."""
    from bibo_b200 import BiBoMoELayer, MoEConfig
    inp = orc.make_inputs(rec["n_tokens"], rec["hidden"], rec["inter"], rec["n_experts"], seed=rec["seed"],
                          bias_mode="uniform", theta_std=0.5)
    norm_w = 1.0 + 0.1 * torch.randn(rec["hidden"], generator=torch.Generator().manual_seed(rec["seed"] * 1000 + 31))
    layer = BiBoMoELayer(MoEConfig(hidden_size=rec["hidden"], moe_intermediate_size=rec["inter"],
                                   num_routed_experts=rec["n_experts"], num_experts_per_tok=rec["top_k"],
                                   bias_update_factor=0.0))
    with torch.no_grad():
        layer.gate.gate_proj.weight.copy_(inp["w_router"]); layer.gate.bias.copy_(inp["bias"])
        layer.experts.gate_up_proj.copy_(inp["gate_up_proj"]); layer.experts.down_proj.copy_(inp["down_proj"])
        layer.experts.radial_theta.copy_(inp["radial_theta"])
    dl = torch.nn.Module()
    dl.mlp = layer.to(DEV).to(dtype)
    dl.mlp.gate.bias.data = inp["bias"].to(DEV)
    dl.mlp.experts.radial_theta.data = inp["radial_theta"].to(DEV)
    dl.post_attention_layernorm = _Norm(norm_w.to(dtype), rec["eps"]).to(DEV)
    dl._bf16_moe_out = dl._bf16_stream = False
    return dl, inp


def test_ffn_forward_fp32_matches_the_reference_fixture():
    from bibo_b200.moe import ffn_forward
    rec = torch.load(GOLDEN / "ffn_moe.pt")
    dl, inp = _decoder_half(rec, torch.float32)
    with torch.no_grad():
        out = ffn_forward(dl.eval(), inp["x"].to(DEV).unsqueeze(0))[0]
    assert rel_err(out.cpu(), rec["out"]) < 1e-4


def test_ffn_forward_bf16_and_training_path():
    """bf16 inference (norm kernel + residual inside the combine kernel) against the fp32 fixture, and the
    gradient-enabled path (module norm + autograd node + torch residual) against the inference result."""
    from bibo_b200.moe import ffn_forward
    rec = torch.load(GOLDEN / "ffn_moe.pt")
    dl, inp = _decoder_half(rec, torch.bfloat16)
    h = inp["x"].to(torch.bfloat16).to(DEV).unsqueeze(0)
    with torch.no_grad():
        out = ffn_forward(dl.eval(), h)[0]
    _, _, ref_idx, _, _ = orc.moe_forward(rec["normed"], inp["w_router"], inp["bias"], inp["gate_up_proj"],
                                          inp["down_proj"], inp["radial_theta"], rec["top_k"], return_routing=True)
    same = (dl.mlp.last_workspace.topk_idx.cpu().long() == ref_idx).all(-1)
    assert float(same.float().mean()) > 0.95
    o, r = out.float().cpu()[same], rec["out"][same]
    assert rel_err(o, r) < BF16_MAX and mean_rel_err(o, r) < BF16_MEAN
    hg = h.clone().requires_grad_(True)
    out_t = ffn_forward(dl.train(), hg)[0]
    out_t.float().sum().backward()
    assert hg.grad is not None and bool(torch.isfinite(hg.grad.float()).all())
    assert rel_err(out_t.detach().float().cpu()[same], o) < 8e-3      # same math, one rounding order differs
