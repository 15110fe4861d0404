"""Backward of the whole block on the GPU against the reference's autograd gradients (golden
fixtures) and against autograd through the CPU oracle."""
import pytest
import torch

from conftest import digest_close, grad_digest, load_golden, mean_rel_err, rel_err, upstream_grad
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP32_TOL = 1e-4
BF16_MAX, BF16_MEAN = 2e-2, 1e-2


def _layer(inp, top_k, norm, pairs, dtype):
    from bibo_b200 import BiBoMoELayer, MoEConfig
    n_glu, two_i, hidden = inp["gate_up_proj"].shape
    cfg = MoEConfig(hidden_size=hidden, moe_intermediate_size=two_i // 2, num_routed_experts=inp["w_router"].shape[0],
                    num_experts_per_tok=top_k, num_pos_identity_experts=pairs, num_neg_identity_experts=pairs,
                    norm_topk_prob=norm, bias_update_factor=0.0)
    layer = BiBoMoELayer(cfg)
    with torch.no_grad():
        layer.gate.gate_proj.weight.copy_(inp["w_router"])
        layer.gate.bias.copy_(inp["bias"])
        layer.experts.gate_up_proj.copy_(inp["gate_up_proj"])
        layer.experts.down_proj.copy_(inp["down_proj"])
        layer.experts.radial_theta.copy_(inp["radial_theta"])
    layer = layer.to(DEV).to(dtype)
    # the selection bias and theta stay fp32 (a bf16-rounded bias would route differently)
    layer.gate.bias.data = inp["bias"].to(DEV)
    layer.experts.radial_theta.data = inp["radial_theta"].to(DEV)
    return layer.train()


def _grads(layer, x, dout):
    x = x.clone().requires_grad_(True)
    out = layer(x.unsqueeze(0))
    (out[0] * dout).sum().backward()
    e = layer.experts
    return out[0].detach(), dict(dx=x.grad, d_w_router=layer.gate.gate_proj.weight.grad, d_gate_up_proj=e.gate_up_proj.grad,
                                 d_down_proj=e.down_proj.grad, d_radial_theta=e.radial_theta.grad)


@pytest.mark.parametrize("name", ["tiny_glu", "tiny_specials", "tiny_softmax", "tiny_raw", "e64_k6_fp32"])
def test_backward_fp32_matches_reference_autograd(name):
    rec, inp = load_golden(name)
    layer = _layer(inp, rec["top_k"], rec["norm"], rec["pairs"], torch.float32)
    out, g = _grads(layer, inp["x"].to(DEV), upstream_grad(rec).to(DEV))
    assert torch.equal(layer.last_workspace.topk_idx.cpu().to(torch.int16), rec["idx_sorted"])
    assert rel_err(out.cpu(), rec["out"]) < FP32_TOL
    assert rel_err(g["dx"].cpu(), rec["dx"]) < FP32_TOL
    assert rel_err(g["d_w_router"].cpu(), rec["d_w_router"]) < FP32_TOL
    assert rel_err(g["d_radial_theta"].cpu(), rec["d_radial_theta"]) < FP32_TOL
    for key in ("d_gate_up_proj", "d_down_proj"):
        gg = g[key].cpu()
        assert rel_err(gg[rec[key + "_experts"]], rec[key + "_sel"]) < FP32_TOL
        assert digest_close(grad_digest(gg, rec["seed"]), rec[key + "_digest"], FP32_TOL)
    assert layer.gate.bias.grad is None


def _oracle_grads(inp, dout, k, dtype):
    t = {kk: v.clone() for kk, v in inp.items()}
    for kk in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[kk] = t[kk].to(dtype).float()
    for kk in ("x", "w_router", "gate_up_proj", "down_proj", "radial_theta"):
        t[kk].requires_grad_(True)
    out, logits, idx, w, counts = orc.moe_forward(t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"],
                                                  t["radial_theta"], k, return_routing=True)
    (out * dout.to(dtype).float()).sum().backward()
    return idx, dict(dx=t["x"].grad, d_w_router=t["w_router"].grad, d_gate_up_proj=t["gate_up_proj"].grad,
                     d_down_proj=t["down_proj"].grad, d_radial_theta=t["radial_theta"].grad)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,h,i,e,k", [(300, 128, 64, 64, 6), (700, 256, 128, 64, 6), (520, 512, 512, 64, 6),
                                       (900, 256, 256, 64, 6), (2100, 1024, 512, 64, 6)])
def test_backward_matches_oracle_autograd(dtype, n, h, i, e, k):
    inp = orc.make_inputs(n, h, i, e, seed=n + 1, bias_mode="uniform", theta_std=0.5)
    dout = torch.randn(n, h, generator=torch.Generator().manual_seed(5))
    layer = _layer(inp, k, "sum", 0, dtype)
    out, g = _grads(layer, inp["x"].to(dtype).to(DEV), dout.to(dtype).to(DEV))
    idx, ref = _oracle_grads(inp, dout, k, dtype)
    same = (layer.last_workspace.topk_idx.cpu().long() == idx).all(-1)
    assert bool(same.all()), "routing differs from the oracle: gradients are not comparable"
    for key, r in ref.items():
        got = g[key].float().cpu()
        if dtype == torch.float32:
            assert rel_err(got, r) < FP32_TOL, key
        else:
            assert rel_err(got, r) < BF16_MAX and mean_rel_err(got, r) < BF16_MEAN, key


def test_backward_with_unused_experts_writes_zero_gradients():
    """Strongly skewed routing leaves experts without tokens: their weight gradients must come out as
    exact zeros (the gradient buffers are not pre-zeroed) and the rest must match the oracle."""
    n, h, i, k = 1500, 1024, 512, 6
    inp = orc.make_inputs(n, h, i, 64, seed=77, bias_mode="zipf", theta_std=0.5, zipf_alpha=6.0)
    dout = torch.randn(n, h, generator=torch.Generator().manual_seed(8))
    layer = _layer(inp, k, "sum", 0, torch.bfloat16)
    out, g = _grads(layer, inp["x"].to(torch.bfloat16).to(DEV), dout.to(torch.bfloat16).to(DEV))
    idx, ref = _oracle_grads(inp, dout, k, torch.bfloat16)
    counts = torch.bincount(idx.reshape(-1), minlength=64)
    unused = counts == 0
    assert int(unused.sum()) > 0, "the case must leave some experts unused"
    assert bool((layer.last_workspace.topk_idx.cpu().long() == idx).all())
    for key in ("d_gate_up_proj", "d_down_proj"):
        got = g[key].float().cpu()
        assert float(got[unused].abs().max()) == 0.0, key
        assert rel_err(got, ref[key]) < BF16_MAX and mean_rel_err(got, ref[key]) < BF16_MEAN, key
    assert rel_err(g["dx"].float().cpu(), ref["dx"]) < BF16_MAX


def test_backward_is_deterministic_and_eval_forward_unchanged():
    inp = orc.make_inputs(600, 256, 128, 64, seed=3, bias_mode="uniform", theta_std=0.5)
    dout = torch.randn(600, 256, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16).to(DEV)
    x = inp["x"].to(torch.bfloat16).to(DEV)
    runs = []
    for _ in range(2):
        layer = _layer(inp, 6, "sum", 0, torch.bfloat16)
        runs.append(_grads(layer, x, dout))
    for key in runs[0][1]:
        assert torch.equal(runs[0][1][key], runs[1][1][key]), key
    with torch.no_grad():
        out_eval = layer.eval()(x.unsqueeze(0))[0]
    assert torch.equal(out_eval, runs[0][0])


def test_training_mode_drives_the_balancer_from_the_kernel_histogram():
    """5 training forwards: the bias moves once the step threshold is hit, never in eval
    (tests/test_training.py:54-79)."""
    from bibo_b200 import BiBoMoELayer, MoEConfig
    cfg = MoEConfig(hidden_size=128, moe_intermediate_size=64, num_routed_experts=64, num_experts_per_tok=6,
                    bias_update_factor=0.4, bias_update_threshold=200)
    layer = BiBoMoELayer(cfg).to(DEV).train()
    x = torch.randn(1, 100, 128, device=DEV, requires_grad=True)
    layer(x).sum().backward()
    assert float(layer.gate.bias.abs().max()) == 0 and float(layer.accumulated_tpe.sum()) == 600
    layer(x).sum().backward()
    assert float(layer.gate.bias.abs().max()) > 0 and float(layer.accumulated_tpe.sum()) == 0
    assert abs(float(layer.gate.bias.mean())) < 1e-6
    before = layer.gate.bias.clone()
    with torch.no_grad():
        layer.eval()(x)
    assert torch.equal(before, layer.gate.bias)
