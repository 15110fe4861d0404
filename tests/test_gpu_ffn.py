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
    """bf16 inference (norm folded into the router's and the permute's loads, residual inside the combine
    kernel: bibo_moe_ffn_forward) against the fp32 fixture, and the gradient-enabled path (module norm + autograd node + torch residual) against the inference result."""
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
    dout = torch.randn(out_t.shape, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).to(DEV)
    (out_t * dout).sum().backward()
    # same math up to the operand rounding of the router (the fused kernel does not round x before the logits):
    # compared on the tokens both paths route like the reference
    same_t = same & (dl.mlp.last_workspace.topk_idx.cpu().long() == ref_idx).all(-1)
    assert float(same_t.float().mean()) > 0.93
    assert rel_err(out_t.detach().float().cpu()[same_t], out.float().cpu()[same_t]) < 8e-3
    # gradients against autograd through the CPU oracle (norm + block + residual), bf16-rounded inputs
    r = lambda t: t.to(torch.bfloat16).float()
    ch = r(inp["x"]).requires_grad_(True)
    nw = r(dl.post_attention_layernorm.weight.detach().cpu()).requires_grad_(True)
    c = {k: (r(v) if k in ("w_router", "gate_up_proj", "down_proj") else v.clone()) for k, v in inp.items()}
    routed, _, idx2, _, _ = orc.moe_forward(orc.rmsnorm(ch, nw, rec["eps"]), c["w_router"], c["bias"], c["gate_up_proj"],
                                            c["down_proj"], c["radial_theta"], rec["top_k"], return_routing=True)
    ((ch + routed) * dout.float().cpu()).sum().backward()
    # a token at a near-tie may route differently (the oracle normalises in fp32, the kernel rounds x to bf16 first):
    # per-token gradients are compared on the other tokens, the norm weight gradient (a sum over all tokens) loosely
    same2 = (dl.mlp.last_workspace.topk_idx.cpu().long() == idx2).all(-1)
    assert float(same2.float().mean()) > 0.97
    got = hg.grad[0].float().cpu()
    assert rel_err(got[same2], ch.grad[same2]) < BF16_MAX and mean_rel_err(got[same2], ch.grad[same2]) < BF16_MEAN
    gw = dl.post_attention_layernorm.weight.grad.float().cpu()
    cos = float(torch.nn.functional.cosine_similarity(gw, nw.grad, dim=0))
    assert cos > 0.99, cos      # the few differently-routed tokens enter this sum; the kernel itself is checked above


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,h", [(1, 64), (333, 256), (2100, 2048)])
def test_rmsnorm_backward_matches_oracle_autograd(dtype, n, h):
    from bibo_b200 import functional as Fn
    g = torch.Generator().manual_seed(n * 7 + h)
    x = (torch.randn(n, h, generator=g) * 2).to(dtype)
    w = (1.0 + 0.1 * torch.randn(h, generator=g)).to(dtype)
    dy = torch.randn(n, h, generator=g).to(dtype)
    cx, cw = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    (orc.rmsnorm(cx, cw, 1e-6).float() * dy.float()).sum().backward()
    dh, dw = Fn.rmsnorm_backward(dy.to(DEV), x.to(DEV), w.to(DEV), 1e-6)
    dh2, dw2 = Fn.rmsnorm_backward(dy.to(DEV), x.to(DEV), w.to(DEV), 1e-6)
    assert torch.equal(dh, dh2) and torch.equal(dw, dw2)
    if dtype == torch.float32:
        assert rel_err(dh.cpu(), cx.grad) < 1e-4 and rel_err(dw.cpu(), cw.grad) < 1e-4
    else:
        assert rel_err(dh.float().cpu(), cx.grad.float()) < BF16_MAX
        assert rel_err(dw.float().cpu(), cw.grad.float()) < BF16_MAX


@pytest.mark.parametrize("n,h,i,pairs", [(4096 + 37, 1024, 256, 0), (2048, 2048, 512, 0), (130, 4096, 128, 0),
                                         (3000, 1024, 256, 1), (777, 512, 128, 3)])
def test_fused_norm_chain_against_the_separate_norm_kernel(n, h, i, pairs):
    """bibo_moe_ffn_forward (norm inside the router's and the permute's loads) against rmsnorm kernel ->
    block -> residual in the combine: rstd against torch, the normalised expert rows bit for bit where
    rstd has the same bits, the routing equal except at near-ties, the outputs equal on equally routed tokens."""
    from bibo_b200 import functional as Fn
    g = torch.Generator().manual_seed(n + h)
    inp = orc.make_inputs(n, h, i, 64, seed=17, bias_mode="uniform", theta_std=0.5)
    t = {k: v.to(DEV) for k, v in inp.items()}
    for k in ("w_router", "gate_up_proj", "down_proj"):
        t[k] = t[k].to(torch.bfloat16).contiguous()
    g_ = 64 - 2 * pairs        # with pairs > 0 the last experts are +Identity / -Identity (no weights)
    for k in ("gate_up_proj", "down_proj", "radial_theta"):
        t[k] = t[k][:g_].contiguous()
    # a residual stream whose rows have different scales, as after a few layers
    hs = (torch.randn(n, h, generator=g) * (0.5 + 3 * torch.rand(n, 1, generator=g))).to(torch.bfloat16).to(DEV)
    nw = (1.0 + 0.1 * torch.randn(h, generator=g)).to(torch.bfloat16).to(DEV)
    eps = 1e-6
    geo = Fn.Geometry(n, h, i, 64, g_, pairs, 6, torch.bfloat16)
    ws_a, ws_b = Fn.MoEWorkspace(geo, DEV, keep_logits=True), Fn.MoEWorkspace(geo, DEV, keep_logits=True)
    x = Fn.rmsnorm_forward(hs, nw, eps)
    ref, ws_a = Fn.moe_forward(x, t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], 6,
                               ws=ws_a, addend=hs, n_pos=pairs, n_neg=pairs)
    out, ws_b = Fn.ffn_forward(hs, nw, eps, t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"],
                               t["radial_theta"], 6, ws=ws_b, n_pos=pairs, n_neg=pairs)
    torch.cuda.synchronize()
    assert Fn.plan_header(ws_a)[2] == 0 and Fn.plan_header(ws_b)[2] == 0
    rstd = torch.rsqrt(hs.double().pow(2).mean(-1) + eps)
    assert float(((ws_b.rstd.double() - rstd).abs() / rstd).max()) < 2e-6
    # logits: the fused kernel rounds h*w once, the separate chain rounds the normalised row twice
    la, lb = ws_a.logits, ws_b.logits
    assert float((la - lb).abs().max() / la.abs().max()) < 1e-2
    same = (ws_a.topk_idx == ws_b.topk_idx).all(-1)
    assert float(same.float().mean()) > 0.95, float(same.float().mean())
    flipped = ~same
    if bool(flipped.any()):     # only near-ties flip: boundary gap of the reference logits below the logits difference
        gap = orc.boundary_gap(la.cpu(), t["bias"].cpu(), 6)[flipped.cpu()]
        err = (la - lb).abs().max(-1).values.cpu()[flipped.cpu()]
        assert bool((gap <= 2 * err.double() + 1e-7).all())
    o, r = out.float()[same], ref.float()[same]
    assert rel_err(o.cpu(), r.cpu()) < 8e-3, rel_err(o.cpu(), r.cpu())
    if pairs:
        special = (ws_b.topk_idx >= g_).any(-1)
        assert int((special & same).sum()) > 0, "no equally routed token picked an identity expert"
        o2, r2 = out.float()[special & same], ref.float()[special & same]
        assert rel_err(o2.cpu(), r2.cpu()) < 8e-3
    # the expert rows of an equally routed token are the separate kernel's normalised row
    tok = int((same & (ws_b.slot_row[:, 0] >= 0)).nonzero()[0])
    row_a, row_b = int(ws_a.slot_row[tok, 0]), int(ws_b.slot_row[tok, 0])
    assert float((ws_a.xp[row_a].float() - ws_b.xp[row_b].float()).abs().max()) <= 2 ** -7 * float(x[tok].float().abs().max())
    again, _ = Fn.ffn_forward(hs, nw, eps, t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"],
                              t["radial_theta"], 6, ws=ws_b, n_pos=pairs, n_neg=pairs)   # reuses the folded router weight
    assert torch.equal(again, out), "the fused chain is not deterministic"
    fold = (t["w_router"].float() * nw.float()).to(torch.bfloat16)
    assert torch.equal(ws_b.w_fold, fold)
    nw.mul_(2.0)                                                    # an in-place update must be seen
    twice, _ = Fn.ffn_forward(hs, nw, eps, t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"],
                              t["radial_theta"], 6, ws=ws_b, n_pos=pairs, n_neg=pairs)
    assert torch.equal(ws_b.w_fold, (t["w_router"].float() * nw.float()).to(torch.bfloat16))
    assert not torch.equal(twice, out)


def test_fused_norm_is_refused_or_bypassed_where_it_does_not_apply():
    from bibo_b200 import functional as Fn
    from bibo_b200.moe import ffn_forward, fused_ffn_applies
    rec = torch.load(GOLDEN / "ffn_moe.pt")
    dl, inp = _decoder_half(rec, torch.bfloat16)
    h = inp["x"].to(torch.bfloat16).to(DEV).unsqueeze(0)
    assert fused_ffn_applies(dl.mlp, h, dl.post_attention_layernorm)
    assert not fused_ffn_applies(dl.mlp, h.float(), dl.post_attention_layernorm)
    with torch.no_grad():
        fused = ffn_forward(dl.eval(), h)
    seen = []
    handle = dl.mlp.experts.register_forward_pre_hook(lambda m, a: seen.append(a[0]))
    assert not fused_ffn_applies(dl.mlp, h, dl.post_attention_layernorm)
    with torch.no_grad():
        plain = ffn_forward(dl.eval(), h)          # the hook wants the normalised activations: separate norm kernel
    handle.remove()
    assert len(seen) == 1 and seen[0].shape == (rec["n_tokens"], rec["hidden"])
    assert rel_err(fused.float().cpu(), plain.float().cpu()) < 0.5     # a few tokens may route differently
    assert not Fn.ffn_supported(2048 + 32, 512, 64, 6) and not Fn.ffn_supported(2048, 512, 32, 6)
    t = {k: v.to(DEV) for k, v in inp.items()}
    with pytest.raises(RuntimeError, match="bf16 only"):
        Fn.ffn_forward(h[0].float(), dl.post_attention_layernorm.weight.float(), 1e-6, t["w_router"], t["bias"],
                       t["gate_up_proj"], t["down_proj"], t["radial_theta"], 6)


def test_ffn_forward_of_a_dense_layer_adds_the_residual_in_the_down_kernel():
    """A decoder layer whose feed-forward block is the dense BiBoMLP (layers 0 and N-1 of the reference model):
    norm kernel, MLP with the residual added by the down kernel's epilogue; against the separate calls bit for
    bit and against the oracle at the bf16 bars."""
    from bibo_b200 import BiBoMLP, MoEConfig, functional as Fn
    from bibo_b200.moe import ffn_forward
    n, h, i = 700, 512, 1024
    cfg = MoEConfig(hidden_size=h)
    cfg.intermediate_size = i
    w = orc.make_mlp_weights(h, i, seed=5)
    mlp = BiBoMLP(cfg)
    with torch.no_grad():
        mlp.gate_proj.weight.copy_(w["gate_proj"]); mlp.up_proj.weight.copy_(w["up_proj"])
        mlp.down_proj.weight.copy_(w["down_proj"])
    g = torch.Generator().manual_seed(12)
    norm_w = (1.0 + 0.1 * torch.randn(h, generator=g)).to(torch.bfloat16)
    dl = torch.nn.Module()
    dl.mlp = mlp.to(DEV).to(torch.bfloat16)
    dl.post_attention_layernorm = _Norm(norm_w, 1e-6).to(DEV)
    hs = (2 * torch.randn(1, n, h, generator=g)).to(torch.bfloat16).to(DEV)
    with torch.no_grad():
        out = ffn_forward(dl.eval(), hs)
        x = Fn.rmsnorm_forward(hs[0], dl.post_attention_layernorm.weight, 1e-6)
        sep = hs[0] + Fn.mlp_forward(x, dl.mlp.gate_proj.weight, dl.mlp.up_proj.weight, dl.mlp.down_proj.weight)
    assert out.shape == hs.shape and torch.equal(out[0], sep)
    r = lambda t: t.to(torch.bfloat16).float()
    ref = hs[0].float().cpu() + orc.mlp_forward(orc.rmsnorm(hs[0].float().cpu(), norm_w.float(), 1e-6),
                                                r(w["gate_proj"]), r(w["up_proj"]), r(w["down_proj"]))
    assert rel_err(out[0].float().cpu(), ref) < BF16_MAX and mean_rel_err(out[0].float().cpu(), ref) < BF16_MEAN
