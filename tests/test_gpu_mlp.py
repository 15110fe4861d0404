"""Dense SwiGLU MLP and the shared expert of the MoE layer on the GPU against the reference's own
outputs (golden fixtures, fp32) and the CPU oracle, at the bf16 bars."""
import pathlib

import pytest
import torch

from conftest import mean_rel_err, rel_err
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
GOLDEN = pathlib.Path(__file__).resolve().parent / "golden"
BF16_MAX, BF16_MEAN = 2e-2, 1e-2


def _dev(w):
    return {k: v.to(torch.bfloat16).to(DEV).contiguous() for k, v in w.items()}


def test_dense_mlp_matches_the_reference_fixture():
    from bibo_b200 import functional as Fn
    rec = torch.load(GOLDEN / "mlp_dense.pt")
    w = _dev(orc.make_mlp_weights(rec["hidden"], rec["inter"], rec["seed"]))
    x = torch.randn(rec["n_tokens"], rec["hidden"], generator=torch.Generator().manual_seed(rec["seed"] * 1000 + 1))
    out = Fn.mlp_forward(x.to(torch.bfloat16).to(DEV), w["gate_proj"], w["up_proj"], w["down_proj"])
    torch.cuda.synchronize()
    o = out.float().cpu()
    assert rel_err(o, rec["out"]) < BF16_MAX and mean_rel_err(o, rec["out"]) < BF16_MEAN


@pytest.mark.parametrize("n,h,i", [(1, 256, 256), (127, 256, 512), (1000, 1024, 4096), (2050, 2048, 1024)])
def test_dense_mlp_matches_the_oracle(n, h, i):
    """One row, ragged last tile, odd tile counts, the dense-layer width of benchmark configuration 5."""
    from bibo_b200 import functional as Fn
    w = orc.make_mlp_weights(h, i, seed=n)
    x = torch.randn(n, h, generator=torch.Generator().manual_seed(n))
    wd = _dev(w)
    out = Fn.mlp_forward(x.to(torch.bfloat16).to(DEV), wd["gate_proj"], wd["up_proj"], wd["down_proj"])
    again = Fn.mlp_forward(x.to(torch.bfloat16).to(DEV), wd["gate_proj"], wd["up_proj"], wd["down_proj"])
    torch.cuda.synchronize()
    assert torch.equal(out, again)
    r = lambda t: t.to(torch.bfloat16).float()
    ref = orc.mlp_forward(r(x), r(w["gate_proj"]), r(w["up_proj"]), r(w["down_proj"]))
    o = out.float().cpu()
    assert rel_err(o, ref) < BF16_MAX and mean_rel_err(o, ref) < BF16_MEAN


def test_layer_with_shared_expert_matches_the_reference_fixture():
    """BiBoMoELayer(use_shared_expert=True): routed + shared, the sum done in the combine kernel."""
    from bibo_b200 import BiBoMLP, BiBoMoELayer, MoEConfig
    rec = torch.load(GOLDEN / "layer_shared_expert.pt")
    cfg = MoEConfig(hidden_size=rec["hidden"], moe_intermediate_size=rec["moe_inter"], num_routed_experts=rec["n_experts"],
                    num_experts_per_tok=rec["top_k"], use_shared_expert=True, num_shared_experts=rec["n_shared"])
    layer = BiBoMoELayer(cfg)
    assert isinstance(layer.shared_experts_list[0], BiBoMLP)
    assert layer.shared_experts_list[0].gate_proj.weight.shape == (rec["inter"], rec["hidden"])
    inp = orc.make_inputs(rec["n_tokens"], rec["hidden"], rec["moe_inter"], rec["n_experts"], seed=rec["seed"],
                          bias_mode="uniform", theta_std=0.5)
    w = orc.make_mlp_weights(rec["hidden"], rec["inter"], rec["seed"])
    with torch.no_grad():
        layer.gate.gate_proj.weight.copy_(inp["w_router"])
        layer.gate.bias.copy_(inp["bias"])
        layer.experts.gate_up_proj.copy_(inp["gate_up_proj"])
        layer.experts.down_proj.copy_(inp["down_proj"])
        layer.experts.radial_theta.copy_(inp["radial_theta"])
        sh = layer.shared_experts_list[0]
        sh.gate_proj.weight.copy_(w["gate_proj"]); sh.up_proj.weight.copy_(w["up_proj"]); sh.down_proj.weight.copy_(w["down_proj"])
    layer = layer.to(DEV).to(torch.bfloat16).eval()
    layer.gate.bias.data = inp["bias"].to(DEV)                 # selection bias and theta stay fp32
    layer.experts.radial_theta.data = inp["radial_theta"].to(DEV)
    x = inp["x"].to(torch.bfloat16).to(DEV).unsqueeze(0)
    with torch.no_grad():
        out = layer(x)[0]
    torch.cuda.synchronize()
    # bf16 logits may route a near-tie token differently from the fp32 reference: compare the others
    _, _, ref_idx, _, _ = orc.moe_forward(inp["x"], inp["w_router"], inp["bias"], inp["gate_up_proj"], inp["down_proj"],
                                          inp["radial_theta"], rec["top_k"], return_routing=True)
    same = (layer.last_workspace.topk_idx.cpu().long() == ref_idx).all(-1)
    assert float(same.float().mean()) > 0.95
    o, r = out.float().cpu()[same], rec["out"][same]
    assert rel_err(o, r) < BF16_MAX and mean_rel_err(o, r) < BF16_MEAN
    with pytest.raises(NotImplementedError):                   # the shared expert has no backward kernels
        layer.train()(x.clone().requires_grad_(True))


def test_unsupported_mlp_inputs_are_refused():
    from bibo_b200 import functional as Fn
    w = _dev(orc.make_mlp_weights(256, 256, seed=1))
    x = torch.randn(8, 256)
    with pytest.raises(RuntimeError):
        Fn.mlp_forward(x.to(torch.bfloat16), w["gate_proj"], w["up_proj"], w["down_proj"])      # CPU tensor
    with pytest.raises(RuntimeError):
        Fn.mlp_forward(x.to(DEV), w["gate_proj"].float(), w["up_proj"].float(), w["down_proj"].float())   # fp32
    w2 = _dev(orc.make_mlp_weights(256, 192, seed=1))
    with pytest.raises(RuntimeError):
        Fn.mlp_forward(x.to(torch.bfloat16).to(DEV), w2["gate_proj"], w2["up_proj"], w2["down_proj"])     # I % 256
