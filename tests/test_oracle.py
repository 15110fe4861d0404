"""The oracle restatement against fixtures produced by the unmodified reference (CPU only)."""
import pytest
import torch

from conftest import GOLDEN, GOLDEN_CASES, digest_close, grad_digest, load_golden, rel_err, upstream_grad
from oracle import moe_oracle as orc


def _run(rec, inp, dtype=torch.float32, grad=False):
    t = {k: (v.to(dtype) if k not in ("bias", "radial_theta") else v.clone()) for k, v in inp.items()}
    if dtype != torch.float32:
        t["radial_theta"] = t["radial_theta"].to(dtype)   # the reference casts the whole module
    if grad:
        for k in ("x", "gate_up_proj", "down_proj", "radial_theta", "w_router"):
            t[k].requires_grad_(True)
    out, logits, idx, w, counts = orc.moe_forward(
        t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"],
        top_k=rec["top_k"], norm_topk_prob=rec["norm"], num_pos_identity=rec["pairs"],
        num_neg_identity=rec["pairs"], return_routing=True)
    return t, out, logits, idx, w, counts


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_forward_matches_reference(name):
    rec, inp = load_golden(name)
    _, out, logits, idx, w, counts = _run(rec, inp)
    assert torch.equal(logits, rec["logits"]), "same F.linear on the same bits"
    assert torch.equal(idx.to(torch.int16), rec["idx_sorted"]), "selected expert sets"
    assert torch.equal(counts.to(torch.int32), rec["counts"])
    assert torch.allclose(w, rec["w_sorted"], rtol=0, atol=1e-6)
    assert rel_err(out, rec["out"]) < 1e-6


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_backward_matches_reference_autograd(name):
    rec, inp = load_golden(name)
    t, out, *_ = _run(rec, inp, grad=True)
    (out * upstream_grad(rec)).sum().backward()
    assert rel_err(t["x"].grad, rec["dx"]) < 1e-5
    assert rel_err(t["w_router"].grad, rec["d_w_router"]) < 1e-5
    assert rel_err(t["radial_theta"].grad, rec["d_radial_theta"]) < 1e-5
    for key, g in (("d_gate_up_proj", t["gate_up_proj"].grad), ("d_down_proj", t["down_proj"].grad)):
        assert rel_err(g[rec[key + "_experts"]], rec[key + "_sel"]) < 1e-5
        dig = grad_digest(g.detach(), rec["seed"])
        assert digest_close(dig, rec[key + "_digest"], 1e-5)


def test_bf16_rounding_points_match_reference():
    rec, inp = load_golden("e64_k6_bf16")
    _, out, logits, idx, w, counts = _run(rec, inp, dtype=torch.bfloat16)
    assert torch.equal(logits, rec["logits"])
    assert torch.equal(idx.to(torch.int16), rec["idx_sorted"])
    assert torch.equal(counts.to(torch.int32), rec["counts"])
    # identical rounding points -> only fp32 summation-order noise ahead of one bf16 rounding
    assert rel_err(out.float(), rec["out"].float()) < 1e-2
    assert float((out.float() - rec["out"].float()).abs().mean() / rec["out"].float().abs().mean()) < 1e-3


def test_config1_matches_reference():
    rec, inp = load_golden("config1")
    _, out, logits, idx, w, counts = _run(rec, inp)
    step = rec["rows_step"]
    assert torch.equal(idx.to(torch.int16), rec["idx_sorted"])
    assert torch.equal(counts.to(torch.int32), rec["counts"])
    assert torch.allclose(w, rec["w_sorted"], rtol=0, atol=1e-6)
    assert torch.allclose(logits[::step], rec["logits"], rtol=0, atol=1e-6)
    assert rel_err(out[::step], rec["out"]) < 1e-5


def test_radial_matches_fp64_definition():
    # the definition the reference's own unit test uses (tests/test_moe.py:35-50)
    g = torch.randn(5, 96, generator=torch.Generator().manual_seed(0))
    for theta in (-2.0, 0.0, 1.5, 3.0):
        th = torch.tensor(theta)
        gd = g.double()
        r = (gd.square().mean(-1, keepdim=True) + 1e-6).sqrt()
        ref = torch.nn.functional.silu(gd / r) * r.pow(torch.sigmoid(th.double()))
        assert rel_err(orc.radial_normsilu(g, th), ref) < 1e-6


def test_tie_break_is_lowest_index():
    logits = torch.zeros(3, 8)
    idx, w, counts = orc.router_select(logits, torch.zeros(8), 2)
    assert idx.tolist() == [[0, 1]] * 3
    assert torch.allclose(w, torch.full((3, 2), 0.5))
    assert counts.tolist() == [3, 3, 0, 0, 0, 0, 0, 0]


def test_bias_moves_selection_not_weights():
    # tests/test_moe.py:177-185
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(6, 8, generator=g)
    bias = torch.zeros(8)
    bias[0] = 5.0
    idx, w, _ = orc.router_select(logits, bias, 2)
    assert (idx == 0).any(dim=-1).all()
    assert w.max() <= 1.0 + 1e-6


def test_balancer_interval_and_direction():
    # tests/test_moe.py:206-249
    st = orc.BalancerState(torch.zeros(8))
    counts = torch.zeros(8, dtype=torch.long)
    counts[0] = 32
    fired = [orc.balance_step(st, counts, 16, 48) is not None for _ in range(7)]
    assert st.update_every == 3 and fired == [False, False, True, False, False, True, False]
    bias = torch.zeros(8)
    tpe = torch.full((8,), 10.0)
    tpe[0] = 100.0
    orc.update_bias(bias, tpe, 0.4)
    assert bias[0] < 0 and (bias[1:] > 0).all() and abs(float(bias.mean())) < 1e-6


def test_dense_mlp_oracle_matches_the_reference_fixture():
    """oracle.mlp_forward against the reference's BiBoMLP (src/modeling/ffn/mlp.py), fp32."""
    rec = torch.load(GOLDEN / "mlp_dense.pt")
    w = orc.make_mlp_weights(rec["hidden"], rec["inter"], rec["seed"])
    x = torch.randn(rec["n_tokens"], rec["hidden"], generator=torch.Generator().manual_seed(rec["seed"] * 1000 + 1))
    x.requires_grad_(True)
    for v in w.values():
        v.requires_grad_(True)
    out = orc.mlp_forward(x, w["gate_proj"], w["up_proj"], w["down_proj"])
    assert rel_err(out.detach(), rec["out"]) < 1e-6
    (out * upstream_grad(rec)).sum().backward()
    assert rel_err(x.grad, rec["dx"]) < 1e-5
    for key in ("gate_proj", "up_proj", "down_proj"):
        assert rel_err(w[key].grad[:8], rec[f"d_{key}_head"]) < 1e-5
        assert digest_close(grad_digest(w[key].grad, rec["seed"]), rec[f"d_{key}_digest"], 1e-5)


def test_layer_with_shared_expert_oracle_matches_the_reference_fixture():
    """Routed experts + shared SwiGLU expert (src/modeling/ffn/moe.py:120-127,174-176), fp32."""
    rec = torch.load(GOLDEN / "layer_shared_expert.pt")
    inp = orc.make_inputs(rec["n_tokens"], rec["hidden"], rec["moe_inter"], rec["n_experts"], seed=rec["seed"],
                          bias_mode="uniform", theta_std=0.5)
    w = orc.make_mlp_weights(rec["hidden"], rec["inter"], rec["seed"])
    routed = orc.moe_forward(inp["x"], inp["w_router"], inp["bias"], inp["gate_up_proj"], inp["down_proj"],
                             inp["radial_theta"], rec["top_k"])
    out = routed + orc.mlp_forward(inp["x"], w["gate_proj"], w["up_proj"], w["down_proj"])
    assert rel_err(out, rec["out"]) < 1e-6


def test_ffn_half_of_the_decoder_layer_oracle_matches_the_reference_fixture():
    """RMSNorm + MoE block + residual (BiBoDecoderLayer._ffn_forward, src/modeling/layers.py:57-67), fp32."""
    rec = torch.load(GOLDEN / "ffn_moe.pt")
    inp = orc.make_inputs(rec["n_tokens"], rec["hidden"], rec["inter"], rec["n_experts"], seed=rec["seed"],
                          bias_mode="uniform", theta_std=0.5)
    norm_w = 1.0 + 0.1 * torch.randn(rec["hidden"], generator=torch.Generator().manual_seed(rec["seed"] * 1000 + 31))
    x = orc.rmsnorm(inp["x"], norm_w, rec["eps"])
    assert rel_err(x, rec["normed"]) < 1e-6
    out = inp["x"] + orc.moe_forward(x, inp["w_router"], inp["bias"], inp["gate_up_proj"], inp["down_proj"],
                                     inp["radial_theta"], rec["top_k"])
    assert rel_err(out, rec["out"]) < 1e-6


def _trace_forwards(rec):
    """The routing of the trace fixture's forwards through the oracle: (logits, idx, w, counts) per seed."""
    n_glu, first = rec["n_glu"], None
    for seed in rec["seeds"]:
        inp = orc.make_inputs(rec["n_tokens"], rec["hidden"], rec["inter"], rec["n_experts"], seed=seed,
                              bias_mode="uniform", theta_std=0.5)
        first = first or inp
        logits = orc.router_logits(inp["x"], first["w_router"])
        idx, w, counts = orc.router_select(logits, first["bias"], rec["top_k"], rec["norm"])
        yield logits, idx, w, counts


@pytest.mark.parametrize("name", ["router_trace_sum", "router_trace_raw"])
def test_router_trace_sums_match_the_reference_trace(name):
    """oracle.router_trace_sums against the accumulator of the reference's RouterTrace, hooked onto the
    reference layer for two training forwards (fixture: tests/golden/make_golden.py run_trace_case)."""
    rec = torch.load(GOLDEN / f"{name}.pt", weights_only=True)
    acc, counts = torch.zeros(8, dtype=torch.float64), torch.zeros(rec["n_experts"], dtype=torch.float64)
    for i, (logits, idx, w, c) in enumerate(_trace_forwards(rec)):
        acc += orc.router_trace_sums(logits, idx, w, rec["top_k"])
        counts += c
        assert torch.allclose(acc, rec["acc"][i].double(), rtol=2e-6, atol=1e-7), (i, acc, rec["acc"][i])
        assert torch.equal(counts.float(), rec["counts"][i])
        assert abs(float(orc.probe_gap(logits, rec["top_k"])) - float(rec["gap"][i])) < 1e-7
