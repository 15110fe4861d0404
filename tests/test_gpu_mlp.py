"""Dense SwiGLU MLP and the shared expert of the MoE layer on the GPU against the reference's own
outputs (golden fixtures, fp32) and the CPU oracle, at the bf16 bars."""
import pathlib

import pytest
import torch

from conftest import digest_close, grad_digest, mean_rel_err, rel_err, upstream_grad
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


def _bf16_close(got, ref, name=""):
    got = got.float().cpu()
    assert rel_err(got, ref) < BF16_MAX and mean_rel_err(got, ref) < BF16_MEAN, name


def test_dense_mlp_backward_matches_the_reference_fixture():
    """Gradients of BiBoMLP against the reference's autograd (fp32 fixture), bf16 bars."""
    from bibo_b200 import BiBoMLP, MoEConfig
    rec = torch.load(GOLDEN / "mlp_dense.pt")
    w = orc.make_mlp_weights(rec["hidden"], rec["inter"], rec["seed"])
    cfg = MoEConfig(hidden_size=rec["hidden"], moe_intermediate_size=rec["inter"])
    mlp = BiBoMLP(cfg, is_expert=True)
    with torch.no_grad():
        mlp.gate_proj.weight.copy_(w["gate_proj"]); mlp.up_proj.weight.copy_(w["up_proj"]); mlp.down_proj.weight.copy_(w["down_proj"])
    mlp = mlp.to(DEV).to(torch.bfloat16)
    x = torch.randn(rec["n_tokens"], rec["hidden"], generator=torch.Generator().manual_seed(rec["seed"] * 1000 + 1))
    xg = x.to(torch.bfloat16).to(DEV).requires_grad_(True)
    out = mlp(xg)
    (out * upstream_grad(rec).to(torch.bfloat16).to(DEV)).sum().backward()
    _bf16_close(out.detach(), rec["out"], "out")
    _bf16_close(xg.grad, rec["dx"], "dx")
    for key, prm in (("gate_proj", mlp.gate_proj.weight), ("up_proj", mlp.up_proj.weight), ("down_proj", mlp.down_proj.weight)):
        _bf16_close(prm.grad[:8], rec[f"d_{key}_head"], key)
        assert digest_close(grad_digest(prm.grad.float().cpu(), rec["seed"]), rec[f"d_{key}_digest"], BF16_MAX), key


@pytest.mark.parametrize("n,h,i", [(130, 256, 256), (1000, 1024, 2048), (2050, 512, 768)])
def test_dense_mlp_backward_matches_oracle_autograd(n, h, i):
    from bibo_b200 import functional as Fn
    w = orc.make_mlp_weights(h, i, seed=n)
    x = torch.randn(n, h, generator=torch.Generator().manual_seed(n))
    dout = torch.randn(n, h, generator=torch.Generator().manual_seed(n + 1))
    r = lambda t: t.to(torch.bfloat16).float()
    cx = r(x).requires_grad_(True)
    cw = {k: r(v).requires_grad_(True) for k, v in w.items()}
    (orc.mlp_forward(cx, cw["gate_proj"], cw["up_proj"], cw["down_proj"]) * r(dout)).sum().backward()
    wd = _dev(w)
    xd = x.to(torch.bfloat16).to(DEV)
    out, saved = Fn.mlp_forward(xd, wd["gate_proj"], wd["up_proj"], wd["down_proj"], keep=True)
    plain = Fn.mlp_forward(xd, wd["gate_proj"], wd["up_proj"], wd["down_proj"])
    assert torch.equal(out, plain), "keeping the gate/up rows changes the result"
    dx, dg, du, dd = Fn.mlp_backward(dout.to(torch.bfloat16).to(DEV), xd, wd["gate_proj"], wd["up_proj"], wd["down_proj"], saved)
    torch.cuda.synchronize()
    _bf16_close(dx, cx.grad, "dx")
    _bf16_close(dg, cw["gate_proj"].grad, "d_gate_proj")
    _bf16_close(du, cw["up_proj"].grad, "d_up_proj")
    _bf16_close(dd, cw["down_proj"].grad, "d_down_proj")


def test_layer_with_shared_expert_trains():
    """Gradients through BiBoMoELayer(use_shared_expert=True) against autograd through the CPU oracle
    (routed block + shared MLP, inputs rounded to bf16, fp32 math)."""
    from bibo_b200 import BiBoMoELayer, MoEConfig
    n, h, i, n_sh, k = 700, 256, 256, 2, 6
    cfg = MoEConfig(hidden_size=h, moe_intermediate_size=i, num_routed_experts=64, num_experts_per_tok=k,
                    use_shared_expert=True, num_shared_experts=n_sh, bias_update_factor=0.0)
    inp = orc.make_inputs(n, h, i, 64, seed=12, bias_mode="uniform", theta_std=0.5)
    w = orc.make_mlp_weights(h, i * n_sh, seed=12)
    dout = torch.randn(n, h, generator=torch.Generator().manual_seed(13))
    layer = BiBoMoELayer(cfg)
    sh = layer.shared_experts_list[0]
    with torch.no_grad():
        layer.gate.gate_proj.weight.copy_(inp["w_router"]); layer.gate.bias.copy_(inp["bias"])
        layer.experts.gate_up_proj.copy_(inp["gate_up_proj"]); layer.experts.down_proj.copy_(inp["down_proj"])
        layer.experts.radial_theta.copy_(inp["radial_theta"])
        sh.gate_proj.weight.copy_(w["gate_proj"]); sh.up_proj.weight.copy_(w["up_proj"]); sh.down_proj.weight.copy_(w["down_proj"])
    layer = layer.to(DEV).to(torch.bfloat16).train()
    layer.gate.bias.data = inp["bias"].to(DEV)
    layer.experts.radial_theta.data = inp["radial_theta"].to(DEV)
    xg = inp["x"].to(torch.bfloat16).to(DEV).requires_grad_(True)
    out = layer(xg.unsqueeze(0))[0]
    (out * dout.to(torch.bfloat16).to(DEV)).sum().backward()
    r = lambda t: t.to(torch.bfloat16).float()
    c = {kk: (r(v) if kk in ("x", "w_router", "gate_up_proj", "down_proj") else v.clone()) for kk, v in inp.items()}
    cw = {kk: r(v).requires_grad_(True) for kk, v in w.items()}
    for kk in ("x", "w_router", "gate_up_proj", "down_proj", "radial_theta"):
        c[kk].requires_grad_(True)
    routed, _, idx, _, _ = orc.moe_forward(c["x"], c["w_router"], c["bias"], c["gate_up_proj"], c["down_proj"],
                                           c["radial_theta"], k, return_routing=True)
    ref = routed + orc.mlp_forward(c["x"], cw["gate_proj"], cw["up_proj"], cw["down_proj"])
    (ref * r(dout)).sum().backward()
    assert bool((layer.last_workspace.topk_idx.cpu().long() == idx).all()), "routing differs: gradients not comparable"
    _bf16_close(out.detach(), ref.detach(), "out")
    _bf16_close(xg.grad, c["x"].grad, "dx")
    _bf16_close(sh.gate_proj.weight.grad, cw["gate_proj"].grad, "shared d_gate_proj")
    _bf16_close(sh.up_proj.weight.grad, cw["up_proj"].grad, "shared d_up_proj")
    _bf16_close(sh.down_proj.weight.grad, cw["down_proj"].grad, "shared d_down_proj")
    _bf16_close(layer.experts.gate_up_proj.grad, c["gate_up_proj"].grad, "d_gate_up_proj")
    _bf16_close(layer.gate.gate_proj.weight.grad, c["w_router"].grad, "d_w_router")


def test_dense_mlp_fp32_matches_the_reference_fixture():
    """float32 runs the CUDA-core kernels: 1e-4 against the reference's own fp32 output."""
    from bibo_b200 import functional as Fn
    rec = torch.load(GOLDEN / "mlp_dense.pt")
    w = {k: v.to(DEV) for k, v in orc.make_mlp_weights(rec["hidden"], rec["inter"], rec["seed"]).items()}
    x = torch.randn(rec["n_tokens"], rec["hidden"], generator=torch.Generator().manual_seed(rec["seed"] * 1000 + 1))
    out = Fn.mlp_forward(x.to(DEV), w["gate_proj"], w["up_proj"], w["down_proj"])
    torch.cuda.synchronize()
    assert rel_err(out.cpu(), rec["out"]) < 1e-4


def test_dense_mlp_fp32_backward_matches_the_reference_fixture():
    """float32 gradients (CUDA-core kernels) against the reference's autograd at 1e-4."""
    from bibo_b200 import BiBoMLP, MoEConfig
    rec = torch.load(GOLDEN / "mlp_dense.pt")
    w = orc.make_mlp_weights(rec["hidden"], rec["inter"], rec["seed"])
    mlp = BiBoMLP(MoEConfig(hidden_size=rec["hidden"], moe_intermediate_size=rec["inter"]), is_expert=True)
    with torch.no_grad():
        mlp.gate_proj.weight.copy_(w["gate_proj"]); mlp.up_proj.weight.copy_(w["up_proj"]); mlp.down_proj.weight.copy_(w["down_proj"])
    mlp = mlp.to(DEV)
    x = torch.randn(rec["n_tokens"], rec["hidden"], generator=torch.Generator().manual_seed(rec["seed"] * 1000 + 1))
    xg = x.to(DEV).requires_grad_(True)
    out = mlp(xg)
    (out * upstream_grad(rec).to(DEV)).sum().backward()
    assert rel_err(out.detach().cpu(), rec["out"]) < 1e-4
    assert rel_err(xg.grad.cpu(), rec["dx"]) < 1e-4
    for key, prm in (("gate_proj", mlp.gate_proj.weight), ("up_proj", mlp.up_proj.weight), ("down_proj", mlp.down_proj.weight)):
        assert rel_err(prm.grad[:8].cpu(), rec[f"d_{key}_head"]) < 1e-4, key
        assert digest_close(grad_digest(prm.grad.cpu(), rec["seed"]), rec[f"d_{key}_digest"], 1e-4), key


@pytest.mark.parametrize("dtype,n,h,i", [(torch.float32, 77, 96, 80), (torch.bfloat16, 130, 192, 96)])
def test_dense_mlp_on_cuda_cores_for_other_shapes(dtype, n, h, i):
    from bibo_b200 import functional as Fn
    w = orc.make_mlp_weights(h, i, seed=3)
    x = torch.randn(n, h, generator=torch.Generator().manual_seed(3))
    r = lambda t: t.to(dtype).float()
    ref = orc.mlp_forward(r(x), r(w["gate_proj"]), r(w["up_proj"]), r(w["down_proj"]))
    wd = {k: v.to(dtype).to(DEV) for k, v in w.items()}
    out = Fn.mlp_forward(x.to(dtype).to(DEV), wd["gate_proj"], wd["up_proj"], wd["down_proj"]).float().cpu()
    if dtype == torch.float32:
        assert rel_err(out, ref) < 1e-4
    else:
        assert rel_err(out, ref) < BF16_MAX and mean_rel_err(out, ref) < BF16_MEAN


def test_unsupported_mlp_inputs_are_refused():
    from bibo_b200 import functional as Fn
    w = _dev(orc.make_mlp_weights(256, 256, seed=1))
    x = torch.randn(8, 256)
    with pytest.raises(RuntimeError):
        Fn.mlp_forward(x.to(torch.bfloat16), w["gate_proj"], w["up_proj"], w["down_proj"])      # CPU tensor
    with pytest.raises(RuntimeError):
        Fn.mlp_forward(x.to(DEV), w["gate_proj"], w["up_proj"], w["down_proj"])                   # dtype mismatch



def test_layer_with_shared_expert_fp32_forward_and_backward_match_the_reference_fixture():
    """float32: routed block (CUDA-core kernels) + shared MLP against the reference's own forward and
    autograd gradients at 1e-4."""
    from bibo_b200 import BiBoMoELayer, MoEConfig
    rec = torch.load(GOLDEN / "layer_shared_expert.pt")
    cfg = MoEConfig(hidden_size=rec["hidden"], moe_intermediate_size=rec["moe_inter"], num_routed_experts=rec["n_experts"],
                    num_experts_per_tok=rec["top_k"], use_shared_expert=True, num_shared_experts=rec["n_shared"],
                    bias_update_factor=0.0)
    layer = BiBoMoELayer(cfg)
    inp = orc.make_inputs(rec["n_tokens"], rec["hidden"], rec["moe_inter"], rec["n_experts"], seed=rec["seed"],
                          bias_mode="uniform", theta_std=0.5)
    w = orc.make_mlp_weights(rec["hidden"], rec["inter"], rec["seed"])
    sh = layer.shared_experts_list[0]
    with torch.no_grad():
        layer.gate.gate_proj.weight.copy_(inp["w_router"]); layer.gate.bias.copy_(inp["bias"])
        layer.experts.gate_up_proj.copy_(inp["gate_up_proj"]); layer.experts.down_proj.copy_(inp["down_proj"])
        layer.experts.radial_theta.copy_(inp["radial_theta"])
        sh.gate_proj.weight.copy_(w["gate_proj"]); sh.up_proj.weight.copy_(w["up_proj"]); sh.down_proj.weight.copy_(w["down_proj"])
    layer = layer.to(DEV).train()
    xg = inp["x"].to(DEV).requires_grad_(True)
    out = layer(xg.unsqueeze(0))[0]
    (out * upstream_grad(rec).to(DEV)).sum().backward()
    assert rel_err(out.detach().cpu(), rec["out"]) < 1e-4
    assert rel_err(xg.grad.cpu(), rec["dx"]) < 1e-4
    for key, prm in (("gate_proj", sh.gate_proj.weight), ("up_proj", sh.up_proj.weight), ("down_proj", sh.down_proj.weight)):
        assert rel_err(prm.grad[:8].cpu(), rec[f"d_{key}_head"]) < 1e-4, key
        assert digest_close(grad_digest(prm.grad.cpu(), rec["seed"]), rec[f"d_{key}_digest"], 1e-4), key


@pytest.mark.parametrize("n,h,i", [(1, 256, 256), (127, 256, 512), (1000, 1024, 4096), (2050, 2048, 1024)])
def test_dense_mlp_with_the_residual_in_the_down_kernel(n, h, i):
    """y = bf16(bf16(mlp(x)) + residual) from the down kernel's epilogue equals the plain forward followed by
    torch's bf16 add bit for bit (the same two roundings), ragged last tile included; rows past N untouched."""
    from bibo_b200 import functional as Fn
    wd = _dev(orc.make_mlp_weights(h, i, seed=n))
    g = torch.Generator().manual_seed(n + 1)
    x = torch.randn(n, h, generator=g).to(torch.bfloat16).to(DEV)
    res = (3 * torch.randn(n, h, generator=g)).to(torch.bfloat16).to(DEV)
    plain = Fn.mlp_forward(x, wd["gate_proj"], wd["up_proj"], wd["down_proj"])
    buf = torch.full((n + 3, h), 7.0, dtype=torch.bfloat16, device=DEV)
    fused = Fn.mlp_forward(x, wd["gate_proj"], wd["up_proj"], wd["down_proj"], out=buf[:n], residual=res)
    torch.cuda.synchronize()
    assert Fn.mlp_residual_supported(h, i, torch.bfloat16)
    assert torch.equal(fused, plain + res)
    assert bool((buf[n:] == 7.0).all()), "rows past the batch were written"


def test_residual_in_the_down_kernel_is_refused_where_it_does_not_exist():
    from bibo_b200 import functional as Fn
    from bibo_b200 import BiBoMLP, MoEConfig
    assert not Fn.mlp_residual_supported(256, 256, torch.float32) and not Fn.mlp_residual_supported(192, 256, torch.bfloat16)
    w = {k: v.to(DEV) for k, v in orc.make_mlp_weights(256, 256, seed=3).items()}
    x = torch.randn(10, 256, device=DEV)
    with pytest.raises(RuntimeError, match="residual"):
        Fn.mlp_forward(x, w["gate_proj"], w["up_proj"], w["down_proj"], residual=x.clone())
    # the module-level call falls back to torch's add there
    from bibo_b200.mlp import mlp_module_forward
    cfg = MoEConfig(hidden_size=256, moe_intermediate_size=256)
    cfg.intermediate_size = 256
    mlp = BiBoMLP(cfg).to(DEV)
    with torch.no_grad():
        a = mlp_module_forward(mlp, x.view(1, 10, 256), residual=x.view(1, 10, 256))
        b = x.view(1, 10, 256) + mlp_module_forward(mlp, x.view(1, 10, 256))
    assert torch.equal(a, b)
