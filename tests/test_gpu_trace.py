"""Router diagnostics produced inside the router and plan kernels (bibo_moe_router_trace): against the
accumulator of the reference's RouterTrace (fixtures written by tests/golden/make_golden.py
run_trace_case), against the oracle at a tensor-core size, and the claims that come with it: the same
launches as an untraced forward, the same bits every run, nothing accumulated in eval mode."""
import pytest
import torch

from conftest import GOLDEN
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
FLUSH_KEYS = ["balance_entropy", "router_top1_weight", "router_entropy", "max_expert_load", "router_w_top1",
              "router_w_sum", "router_w_min", "special_load", "neg_identity_load", "router_boundary_gap"]


def _layer_from_fixture(rec):
    from bibo_b200 import BiBoMoELayer, MoEConfig
    cfg = MoEConfig(hidden_size=rec["hidden"], moe_intermediate_size=rec["inter"], num_routed_experts=rec["n_experts"],
                    num_experts_per_tok=rec["top_k"], num_pos_identity_experts=rec["pairs"],
                    num_neg_identity_experts=rec["pairs"], norm_topk_prob=rec["norm"], bias_update_factor=0.0)
    layer = BiBoMoELayer(cfg).to(DEV).train()
    inp = orc.make_inputs(rec["n_tokens"], rec["hidden"], rec["inter"], rec["n_experts"], seed=rec["seeds"][0],
                          bias_mode="uniform", theta_std=0.5)
    g = rec["n_glu"]
    with torch.no_grad():
        layer.gate.gate_proj.weight.copy_(inp["w_router"])
        layer.gate.bias.copy_(inp["bias"])
        layer.experts.gate_up_proj.copy_(inp["gate_up_proj"][:g])
        layer.experts.down_proj.copy_(inp["down_proj"][:g])
        layer.experts.radial_theta.copy_(inp["radial_theta"][:g])
    return layer


def _x(rec, seed):
    return orc.make_inputs(rec["n_tokens"], rec["hidden"], rec["inter"], rec["n_experts"], seed=seed,
                           bias_mode="uniform", theta_std=0.5)["x"].reshape(1, rec["n_tokens"], rec["hidden"]).to(DEV)


@pytest.mark.parametrize("name", ["router_trace_sum", "router_trace_raw"])
@pytest.mark.parametrize("grad", [False, True])
def test_trace_matches_the_reference_trace(name, grad):
    from bibo_b200 import RouterTrace
    rec = torch.load(GOLDEN / f"{name}.pt", weights_only=True)
    layer = _layer_from_fixture(rec)
    layer.gate._probe_gap = True
    trace = RouterTrace(torch.nn.ModuleDict({"mlp": layer}), rec["n_experts"], DEV)
    for i, seed in enumerate(rec["seeds"]):
        with torch.set_grad_enabled(grad):
            layer(_x(rec, seed))
        assert torch.allclose(trace.acc.cpu(), rec["acc"][i], rtol=1e-5, atol=1e-6), (i, trace.acc.cpu(), rec["acc"][i])
        assert torch.equal(trace.counts.cpu(), rec["counts"][i])
        assert abs(float(layer.gate.boundary_gap) - float(rec["gap"][i])) < 1e-6
    got = trace.flush()
    assert list(got) == ["train/" + k for k in FLUSH_KEYS]
    for k, v in rec["flush"].items():
        assert abs(got[k] - v) <= 1e-5 * max(1.0, abs(v)), (k, got[k], v)
    assert float(trace.acc.abs().sum()) == 0 and float(trace.counts.sum()) == 0, "flush resets"
    layer.eval()
    with torch.no_grad():
        layer(_x(rec, rec["seeds"][0]))
    assert float(trace.acc.abs().sum()) == 0, "an eval forward is not traced (router_trace.py:108,115)"
    assert trace.flush() == {}
    trace.close()
    layer.train()
    with torch.no_grad():
        layer(_x(rec, rec["seeds"][0]))
    assert float(trace.acc.abs().sum()) == 0, "closed trace still attached"


def _bf16_block(n=8192, h=512, i=128, e=64, seed=21):
    inp = orc.make_inputs(n, h, i, e, seed=seed, bias_mode="uniform", theta_std=0.5)
    t = {k: v.to(DEV) for k, v in inp.items()}
    for k in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[k] = t[k].to(torch.bfloat16).contiguous()
    return t


def _traced_forward(t, k=6, norm="sum", scale=1.0, trace=True):
    from bibo_b200 import functional as Fn
    n, h = t["x"].shape
    geo = Fn.Geometry(n, h, t["gate_up_proj"].shape[1] // 2, 64, 64, 0, k, torch.bfloat16)
    ws = Fn.MoEWorkspace(geo, t["x"].device, keep_logits=True)
    bufs = (torch.zeros(8, device=DEV), torch.zeros(64, device=DEV), torch.zeros(1, device=DEV)) if trace else None
    before = Fn.launch_count()
    out, ws = Fn.moe_forward(t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], k,
                             norm, scale, ws=ws, trace=bufs)
    launches = Fn.launch_count() - before
    torch.cuda.synchronize()
    assert Fn.plan_header(ws)[2] == 0
    return out, ws, bufs, launches


@pytest.mark.parametrize("norm,scale", [("sum", 1.0), (False, 1.0), ("softmax", 2.5)])
def test_tensor_core_router_trace_matches_the_oracle_on_its_own_routing(norm, scale):
    """bf16, 8192 tokens (64 router blocks, tensor-core router): the sums against the oracle's formula on
    the kernel's own logits, indices and weights, accumulated twice."""
    t = _bf16_block()
    out, ws, bufs, launches = _traced_forward(t, norm=norm, scale=scale)
    ref = orc.router_trace_sums(ws.logits.cpu(), ws.topk_idx.cpu().long(), ws.topk_w.cpu(), 6)
    acc, counts, gap = (b.cpu() for b in bufs)
    assert torch.allclose(acc.double(), ref, rtol=2e-5, atol=1e-6), (acc, ref)
    assert torch.equal(counts, ws.counts().float().cpu())
    assert abs(float(gap) - float(ref[6])) < 1e-6
    out_plain, ws_plain, _, launches_plain = _traced_forward(t, norm=norm, scale=scale, trace=False)
    assert launches == launches_plain, "tracing added launches"
    assert torch.equal(out, out_plain) and torch.equal(ws.topk_w, ws_plain.topk_w)
    _, _, bufs2, _ = _traced_forward(t, norm=norm, scale=scale)
    for a, b in zip(bufs, bufs2):
        assert torch.equal(a, b), "the diagnostic sums are not deterministic"


def test_trace_pieces_are_optional_and_checked():
    from bibo_b200 import functional as Fn
    t = _bf16_block(n=1000)            # ragged last router block
    geo = Fn.Geometry(1000, 512, 128, 64, 64, 0, 6, torch.bfloat16)
    ws = Fn.MoEWorkspace(geo, DEV, keep_logits=True)
    gap = torch.zeros(1, device=DEV)
    args = (t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], 6)
    Fn.moe_forward(*args, ws=ws, trace=(None, None, gap))
    assert abs(float(gap) - float(orc.probe_gap(ws.logits.cpu(), 6))) < 1e-6
    acc = torch.zeros(8, device=DEV)
    Fn.moe_forward(*args, ws=ws, trace=(acc, None, None))
    assert float(acc[2]) == 1000 and float(acc[7]) == 1 and abs(float(acc[6]) - float(gap)) < 1e-7
    with pytest.raises(RuntimeError, match="trace tensors"):
        Fn.moe_forward(*args, ws=ws, trace=(torch.zeros(7, device=DEV), None, None))
    with pytest.raises(RuntimeError, match="trace tensors"):
        Fn.moe_forward(*args, ws=ws, trace=(None, torch.zeros(64), None))


def test_traced_and_fused_forwards_replay_from_a_cuda_graph():
    """The traced block and the fused feed-forward half are plain stream work (no host synchronisation): both
    are captured in one CUDA graph; every replay adds one forward to the trace accumulators and reproduces the
    eager results on new inputs."""
    from bibo_b200 import functional as Fn
    n, h, i = 2048, 512, 128
    t = _bf16_block(n=n, h=h, i=i)
    args = (t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], 6)
    geo = Fn.Geometry(n, h, i, 64, 64, 0, 6, torch.bfloat16)
    ws, ws_f = Fn.MoEWorkspace(geo, DEV), Fn.MoEWorkspace(geo, DEV)
    nw = (1.0 + 0.1 * torch.randn(h, generator=torch.Generator().manual_seed(3))).to(torch.bfloat16).to(DEV)
    bufs = (torch.zeros(8, device=DEV), torch.zeros(64, device=DEV), torch.zeros(1, device=DEV))
    x_static, out_a, out_b = t["x"].clone(), torch.empty_like(t["x"]), torch.empty_like(t["x"])

    def both():
        Fn.moe_forward(x_static, *args, ws=ws, out=out_a, trace=bufs)
        Fn.ffn_forward(x_static, nw, 1e-6, *args, ws=ws_f, out=out_b)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        both()                                  # warm-up: attributes, tensor maps, the folded router weight
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        both()
    for b in bufs:
        b.zero_()
    counts = torch.zeros(64, device=DEV)
    for rep, seed in enumerate((1, 2, 3)):
        x_new = torch.randn(n, h, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16).to(DEV)
        x_static.copy_(x_new)
        graph.replay()
        torch.cuda.synchronize()
        eager, w1 = Fn.moe_forward(x_new, *args, ws=Fn.MoEWorkspace(geo, DEV))
        fused, _ = Fn.ffn_forward(x_new, nw, 1e-6, *args, ws=Fn.MoEWorkspace(geo, DEV))
        assert torch.equal(out_a, eager) and torch.equal(out_b, fused)
        counts += w1.counts().float()
        assert float(bufs[0][7]) == rep + 1 and float(bufs[0][2]) == (rep + 1) * n
        assert torch.equal(bufs[1], counts)
