"""The whole block (and the experts seam) on the GPU against golden fixtures and the oracle."""
import pytest
import torch

from conftest import load_golden, mean_rel_err, rel_err
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"

FP32_TOL = 1e-4                  # relative, float32 (stated parity bar)
BF16_MAX, BF16_MEAN = 2e-2, 1e-2  # bf16 vs the fp32 reference forward


def _run(inp, rec=None, dtype=torch.float32, top_k=None, norm="sum", pairs=0, scale=1.0):
    from bibo_b200 import functional as Fn
    t = {k: v.to(DEV) for k, v in inp.items()}
    for k in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[k] = t[k].to(dtype).contiguous()
    top_k = rec["top_k"] if rec else top_k
    norm = rec["norm"] if rec else norm
    pairs = rec["pairs"] if rec else pairs
    ws = Fn.MoEWorkspace(Fn.Geometry(t["x"].shape[0], t["x"].shape[1], t["gate_up_proj"].shape[1] // 2,
                                     t["w_router"].shape[0], t["gate_up_proj"].shape[0], pairs, top_k, dtype),
                         DEV, keep_logits=True)
    out, ws = Fn.moe_forward(t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"],
                             top_k, norm, scale, n_pos=pairs, n_neg=pairs, ws=ws)
    torch.cuda.synchronize()
    assert Fn.plan_header(ws)[2] == 0
    return out, ws


def _oracle(inp, top_k, norm="sum", pairs=0, dtype=torch.float32, scale=1.0):
    t = {k: v.clone() for k, v in inp.items()}
    for k in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[k] = t[k].to(dtype).float()   # the same rounded inputs, computed in fp32
    return orc.moe_forward(t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"],
                           top_k, norm, scale, pairs, pairs, return_routing=True)


def _routing_agrees(ws, ref_idx, logits_ref, bias, k):
    same = (ws.topk_idx.cpu().long() == ref_idx).all(-1)
    if bool(same.all()):
        return same
    # a different logits summation order may flip a token whose boundary gap is below the logits error
    err = float((ws.logits.cpu() - logits_ref).abs().max())
    gap = orc.boundary_gap(logits_ref, bias, k)
    assert bool((gap[~same] <= 4 * err + 1e-6).all()), "routing differs away from a near-tie"
    return same


@pytest.mark.parametrize("name", ["tiny_glu", "tiny_specials", "tiny_softmax", "tiny_raw", "e64_k6_fp32", "config1"])
def test_forward_fp32_matches_reference_fixture(name):
    rec, inp = load_golden(name)
    out, ws = _run(inp, rec)
    step = rec["rows_step"]
    ref_out, ref_logits, ref_idx, ref_w, ref_counts = _oracle(inp, rec["top_k"], rec["norm"], rec["pairs"])
    same = _routing_agrees(ws, ref_idx, ref_logits, inp["bias"], rec["top_k"])
    if bool(same.all()):
        assert torch.equal(ws.topk_idx.cpu().to(torch.int16), rec["idx_sorted"]), "bit-exact routing vs the reference"
        assert torch.equal(ws.counts().cpu(), rec["counts"])
    keep = same[::step]
    assert rel_err(out.cpu()[::step][keep], rec["out"][keep]) < FP32_TOL
    assert rel_err(out.cpu()[same], ref_out[same]) < FP32_TOL


def test_forward_bf16_matches_fp32_reference_fixture():
    rec, inp = load_golden("e64_k6_fp32")
    out, ws = _run(inp, rec, dtype=torch.bfloat16)
    # routing is judged on the bf16-rounded inputs the kernel actually saw
    _, ref_logits, ref_idx, _, _ = _oracle(inp, rec["top_k"], rec["norm"], dtype=torch.bfloat16)
    same = _routing_agrees(ws, ref_idx, ref_logits, inp["bias"], rec["top_k"])
    same &= (ref_idx.to(torch.int16) == rec["idx_sorted"]).all(-1)   # tokens the fp32 reference routes alike
    assert same.float().mean() > 0.9
    o, r = out.float().cpu()[same], rec["out"][same]
    assert rel_err(o, r) < BF16_MAX and mean_rel_err(o, r) < BF16_MEAN


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,h,i,e,k,bias_mode", [
    (1, 64, 64, 8, 2, "zero"), (127, 64, 32, 8, 2, "uniform"), (129, 128, 64, 64, 6, "uniform"),
    (1000, 256, 128, 64, 6, "zipf"), (2048, 512, 128, 64, 6, "zero"), (700, 1024, 256, 64, 6, "uniform"),
    (900, 512, 512, 64, 6, "uniform"), (4096, 1024, 512, 64, 6, "zipf")])
def test_forward_matches_oracle(dtype, n, h, i, e, k, bias_mode):
    """Ragged token counts, near-empty experts (zipf bias), both dtypes."""
    inp = orc.make_inputs(n, h, i, e, seed=n, bias_mode=bias_mode, theta_std=0.5, zipf_alpha=1.0)
    out, ws = _run(inp, dtype=dtype, top_k=k)
    ref_out, ref_logits, ref_idx, ref_w, ref_counts = _oracle(inp, k, dtype=dtype)
    same = _routing_agrees(ws, ref_idx, ref_logits, inp["bias"], k)
    if bool(same.all()):
        assert torch.equal(ws.counts().cpu().long(), ref_counts)
    o, r = out.float().cpu()[same], ref_out[same]
    if dtype == torch.float32:
        assert rel_err(o, r) < FP32_TOL
    else:
        assert rel_err(o, r) < BF16_MAX and mean_rel_err(o, r) < BF16_MEAN


@pytest.mark.parametrize("n,h,i", [(700, 256, 128), (1500, 512, 256), (1100, 256, 512)])
def test_saved_gate_up_and_rnorm_bf16(n, h, i):
    """The tensors K3 keeps for the backward pass: raw gate|up rows and the row norm r."""
    from bibo_b200 import functional as Fn
    inp = orc.make_inputs(n, h, i, 64, seed=n, bias_mode="uniform", theta_std=0.5)
    out, ws = _run(inp, dtype=torch.bfloat16, top_k=6)
    rows = Fn.plan_header(ws)[1]
    tok = ws.row_token[:rows].long()
    valid = tok >= 0
    tiles = ws.tiles()[: rows // 128]
    expert_of_row = tiles[:, 0].long().repeat_interleave(128)
    xg = inp["x"].to(torch.bfloat16).to(DEV)[tok[valid]].float()
    wg = inp["gate_up_proj"].to(torch.bfloat16).to(DEV).float()[expert_of_row[valid]]
    gu_ref = torch.einsum("rh,rnh->rn", xg, wg)
    gu = ws.gate_up[:rows][valid].float()
    assert rel_err(gu, gu_ref) < 1e-2 and mean_rel_err(gu, gu_ref) < 5e-3
    r_ref = torch.sqrt(ws.gate_up[:rows][valid][:, :i].float().square().mean(-1) + 1e-6)
    assert torch.allclose(ws.rnorm[:rows][valid], r_ref, rtol=1e-5, atol=0)


@pytest.mark.parametrize("n", [700, 9000, 70000])
def test_host_buffer_call_equals_device_call(n):
    """bibo_moe_forward_host cuts large batches into slices to overlap the copies with the kernels;
    tokens are independent, so the result equals one device call bit for bit (9000: ragged last
    slice; 70000: more slices than the default length allows, so the slice length grows)."""
    from bibo_b200 import functional as Fn
    h, i, k = 512, 256, 6
    inp = orc.make_inputs(n, h, i, 64, seed=11, bias_mode="uniform", theta_std=0.5)
    t = {kk: v.to(DEV) for kk, v in inp.items()}
    for kk in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[kk] = t[kk].to(torch.bfloat16).contiguous()
    ref, _ = Fn.moe_forward(t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], k)
    x_host = t["x"].cpu().pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    x_dev, out_dev = torch.empty_like(t["x"]), torch.empty_like(t["x"])
    for _ in range(2):                                   # twice: the streams and events are reused
        out_host.zero_()
        Fn.moe_forward_host(x_host, out_host, x_dev, out_dev, t["w_router"], t["bias"], t["gate_up_proj"],
                            t["down_proj"], t["radial_theta"], k)
        assert torch.equal(out_host, ref.cpu())


def test_forward_is_cuda_graph_capturable():
    """The single-GPU forward makes no host synchronisation and allocates nothing: after one warm-up
    call it can be captured in a CUDA graph and replayed on new inputs."""
    from bibo_b200 import functional as Fn
    n, h, i, k = 3000, 1024, 512, 6
    inp = orc.make_inputs(n, h, i, 64, seed=4, bias_mode="uniform", theta_std=0.5)
    t = {kk: v.to(DEV) for kk, v in inp.items()}
    for kk in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[kk] = t[kk].to(torch.bfloat16).contiguous()
    args = (t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], k)
    geo = Fn.Geometry(n, h, i, 64, 64, 0, k, torch.bfloat16)
    ws = Fn.get_workspace(geo, t["x"].device, fresh=True)
    x_static, out_static = t["x"].clone(), torch.empty_like(t["x"])
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        Fn.moe_forward(x_static, *args, ws=ws, out=out_static)          # warm-up: attributes, tensor maps
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        Fn.moe_forward(x_static, *args, ws=ws, out=out_static)
    for seed in (1, 2):
        x_new = torch.randn(n, h, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16).to(DEV)
        x_static.copy_(x_new)
        graph.replay()
        torch.cuda.synchronize()
        eager, _ = Fn.moe_forward(x_new, *args, ws=Fn.get_workspace(geo, t["x"].device, fresh=True))
        assert torch.equal(out_static, eager)


def test_forward_is_deterministic():
    inp = orc.make_inputs(1500, 256, 128, 64, seed=4, bias_mode="uniform", theta_std=0.5)
    a, _ = _run(inp, dtype=torch.bfloat16, top_k=6)
    b, _ = _run(inp, dtype=torch.bfloat16, top_k=6)
    assert torch.equal(a, b)


def test_routed_scaling_factor_scales_output():
    inp = orc.make_inputs(256, 128, 64, 64, seed=5, bias_mode="uniform")
    a, _ = _run(inp, top_k=6)
    b, _ = _run(inp, top_k=6, scale=2.0)
    assert rel_err(b, 2.0 * a) < 1e-6


@pytest.mark.parametrize("pairs", [0, 1])
def test_experts_seam_with_caller_routing(pairs):
    """BiBoFusedExperts.forward(x, idx, w) with indices in arbitrary order (tests/test_moe.py:29-33,81-105)."""
    from bibo_b200 import functional as Fn
    n, h, i, e, k = 333, 64, 96, 8, 2
    inp = orc.make_inputs(n, h, i, e, seed=6, theta_std=0.5)
    n_glu = e - 2 * pairs
    g = torch.Generator().manual_seed(1)
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(n)])
    w = torch.rand(n, k, generator=g)
    gu, dn, th = inp["gate_up_proj"][:n_glu].contiguous(), inp["down_proj"][:n_glu].contiguous(), inp["radial_theta"][:n_glu]
    out, _ = Fn.experts_forward(inp["x"].to(DEV), idx.to(DEV), w.to(DEV), gu.to(DEV), dn.to(DEV), th.to(DEV), e, pairs)
    ref = orc.experts_forward(inp["x"], idx, w, gu, dn, th, e, pairs, pairs)
    assert rel_err(out.cpu(), ref) < FP32_TOL


def test_module_api_and_hooks():
    """State-dict names, eval forward, hook replay, balancer untouched in eval (tests/test_training.py:74-79)."""
    from bibo_b200 import BiBoMoELayer, MoEConfig
    cfg = MoEConfig(hidden_size=128, moe_intermediate_size=64, num_routed_experts=64, num_experts_per_tok=6)
    layer = BiBoMoELayer(cfg).to(DEV).eval()
    assert set(layer.state_dict()) == {"accumulated_tpe", "experts.gate_up_proj", "experts.down_proj",
                                       "experts.radial_theta", "gate.bias", "gate.gate_proj.weight"}
    seen = {}
    layer.experts.register_forward_pre_hook(lambda m, a: seen.setdefault("experts", a))
    layer.gate.register_forward_hook(lambda m, a, r: seen.setdefault("gate", r))
    layer.gate._probe_gap = True
    x = torch.randn(2, 50, 128, device=DEV)
    with torch.no_grad():
        y = layer(x)
        idx, w = layer.gate(x)
    assert y.shape == x.shape and y.dtype == x.dtype
    assert seen["experts"][1].dtype == torch.long and seen["experts"][0].shape == (100, 128)
    assert torch.equal(seen["gate"][0], idx) and w.dtype == torch.float32
    assert layer.gate.boundary_gap is not None and float(layer.gate.boundary_gap) > 0
    assert float(layer.gate.bias.abs().max()) == 0 and float(layer.accumulated_tpe.sum()) == 0
    p = {k: v.detach().cpu() for k, v in layer.state_dict().items()}
    ref = orc.moe_forward(x.cpu(), p["gate.gate_proj.weight"], p["gate.bias"], p["experts.gate_up_proj"],
                          p["experts.down_proj"], p["experts.radial_theta"], 6)
    assert rel_err(y.cpu(), ref) < FP32_TOL


def test_cpu_tensor_is_refused():
    from bibo_b200 import BiBoMoELayer, MoEConfig
    layer = BiBoMoELayer(MoEConfig(hidden_size=64, moe_intermediate_size=32, num_routed_experts=8,
                                   num_experts_per_tok=2)).eval()
    with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU implementation"):
        layer(torch.randn(1, 4, 64))
