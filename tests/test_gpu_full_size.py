"""The block at the full sizes of the benchmark configurations, through properties that do not need the
oracle on the whole batch: structural invariants of the routing and of the plan, independence of
the tokens (slices, permutations), determinism, and an oracle check on a random sample of tokens
(tokens are independent, so the CPU oracle on 256 of them checks the same rows of the full run).

Configurations: 2 (16384 tokens, H=1024, I=256, uniform bias), 3 (65536 tokens, H=2048, I=512,
Zipf bias: experts from near-empty to very full), 4 per GPU (32768 tokens, H=2048, I=512)."""
import pytest
import torch

from conftest import mean_rel_err, rel_err
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
K, E = 6, 64
BF16_MAX, BF16_MEAN = 2e-2, 1e-2
CONFIGS = {
    "config2": dict(n=16384, h=1024, i=256, bias_mode="uniform", zipf_alpha=0.0),
    "config3": dict(n=65536, h=2048, i=512, bias_mode="zipf", zipf_alpha=1.0),
    "config4": dict(n=32768, h=2048, i=512, bias_mode="zero", zipf_alpha=0.0),
}


def _inputs(cfg, seed=3):
    inp = orc.make_inputs(cfg["n"], cfg["h"], cfg["i"], E, seed=seed, bias_mode=cfg["bias_mode"], theta_std=0.5,
                          zipf_alpha=cfg["zipf_alpha"])
    t = {k: v.to(DEV) for k, v in inp.items()}
    for k in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[k] = t[k].to(torch.bfloat16).contiguous()
    return inp, t


def _forward(t, x=None, keep_logits=False):
    from bibo_b200 import functional as Fn
    x = t["x"] if x is None else x
    geo = Fn.Geometry(x.shape[0], x.shape[1], t["gate_up_proj"].shape[1] // 2, E, E, 0, K, torch.bfloat16)
    ws = Fn.MoEWorkspace(geo, x.device, keep_logits=keep_logits)
    out, ws = Fn.moe_forward(x, t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], K, ws=ws)
    torch.cuda.synchronize()
    assert Fn.plan_header(ws)[2] == 0, "device status word"
    return out, ws


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def run(request):
    cfg = CONFIGS[request.param]
    inp, t = _inputs(cfg)
    out, ws = _forward(t, keep_logits=True)
    return cfg, inp, t, out, ws


def test_routing_and_plan_invariants(run):
    from bibo_b200 import functional as Fn
    cfg, inp, t, out, ws = run
    n = cfg["n"]
    idx, w = ws.topk_idx.long(), ws.topk_w
    assert int(idx.min()) >= 0 and int(idx.max()) < E
    assert bool((idx[:, 1:] > idx[:, :-1]).all()), "the k experts of a token are distinct and ascending"
    assert float((w.sum(-1) - 1).abs().max()) < 1e-5 and float(w.min()) > 0
    counts = ws.counts().long()
    assert int(counts.sum()) == n * K
    assert torch.equal(counts, torch.bincount(idx.reshape(-1), minlength=E))
    n_tiles, rows_used, status = Fn.plan_header(ws)
    off = ws.expert_off().long()
    assert bool((off % 128 == 0).all()) and int(off[0]) == 0 and int(off[-1]) == rows_used == n_tiles * 128
    assert torch.equal(off[1:] - off[:-1], (counts + 127) // 128 * 128)
    tiles = ws.tiles()[:n_tiles].long()
    assert torch.equal(tiles[:, 1], torch.arange(n_tiles, device=tiles.device) * 128), "tiles cover the rows in order"
    assert int(tiles[:, 2].sum()) == n * K and int(tiles[:, 2].min()) >= 1 and int(tiles[:, 2].max()) <= 128
    expert_of_tile = torch.bucketize(tiles[:, 1].contiguous(), off[1:].contiguous(), right=True)
    assert torch.equal(tiles[:, 0], expert_of_tile)
    # slot_row is a bijection between the N*k slots and the non-padding rows; row_token inverts it
    rows = ws.slot_row.long().reshape(-1)
    assert int(rows.min()) >= 0 and int(rows.unique().numel()) == n * K
    tok = ws.row_token[:rows_used].long()
    assert int((tok >= 0).sum()) == n * K
    assert torch.equal(tok[rows], torch.arange(n, device=rows.device).repeat_interleave(K))
    # every slot lies inside its expert's row range
    e_flat = idx.reshape(-1)
    assert bool(((rows >= off[e_flat]) & (rows < off[e_flat] + counts[e_flat])).all())
    assert bool(torch.isfinite(out.float()).all())


def test_tokens_are_independent_and_the_forward_is_deterministic(run):
    cfg, inp, t, out, ws = run
    n = cfg["n"]
    again, _ = _forward(t)
    assert torch.equal(again, out), "two runs differ"
    cut = n // 2 + 128 * 3 + 17                                   # ragged slices
    lo, _ = _forward(t, t["x"][:cut].contiguous())
    hi, _ = _forward(t, t["x"][cut:].contiguous())
    assert torch.equal(torch.cat([lo, hi]), out), "a token's result depends on the other tokens of the batch"
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(1)).to(DEV)
    shuffled, _ = _forward(t, t["x"][perm].contiguous())
    assert torch.equal(shuffled, out[perm]), "permuting the tokens does not permute the results"


def test_sampled_tokens_match_the_cpu_oracle(run):
    cfg, inp, t, out, ws = run
    n = cfg["n"]
    pick = torch.randperm(n, generator=torch.Generator().manual_seed(2))[:256].sort().values
    c = {k: (v.to(torch.bfloat16).float() if k in ("x", "w_router", "gate_up_proj", "down_proj") else v)
         for k, v in inp.items()}
    ref, logits, idx, w, _ = orc.moe_forward(c["x"][pick], c["w_router"], c["bias"], c["gate_up_proj"], c["down_proj"],
                                             c["radial_theta"], K, return_routing=True)
    got_idx = ws.topk_idx.cpu().long()[pick]
    same = (got_idx == idx).all(-1)
    if not bool(same.all()):   # only a near-tie may flip: boundary gap below the logits difference
        err = float((ws.logits.cpu()[pick] - logits).abs().max())
        gap = orc.boundary_gap(logits, c["bias"], K)
        assert bool((gap[~same] <= 4 * err + 1e-6).all()), "routing differs away from a near-tie"
    assert float(same.float().mean()) > 0.97
    assert float((ws.topk_w.cpu()[pick][same] - w[same]).abs().max()) < 1e-3
    o, r = out.float().cpu()[pick][same], ref[same]
    assert rel_err(o, r) < BF16_MAX and mean_rel_err(o, r) < BF16_MEAN


def _fwd_bwd(t, x, dout):
    from bibo_b200 import functional as Fn
    geo = Fn.Geometry(x.shape[0], x.shape[1], t["gate_up_proj"].shape[1] // 2, E, E, 0, K, torch.bfloat16)
    ws = Fn.MoEWorkspace(geo, x.device, keep_logits=True, keep_gate_up=True)
    out, ws = Fn.moe_forward(x, t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], K,
                             ws=ws, zero_padding=True)
    grads = Fn.moe_backward(dout, x, t["w_router"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], ws, "sum")
    torch.cuda.synchronize()
    assert Fn.plan_header(ws)[2] == 0, "device status word"
    return out, grads


def test_backward_at_configuration_4_size():
    """Forward + backward on 32768 tokens (H=2048, I=512): deterministic; the weight gradients of the
    whole batch equal the sum over two token slices (a gradient is a sum over tokens); dx of sampled
    tokens against autograd through the CPU oracle on those tokens alone (dx of a token depends only
    on that token)."""
    cfg = CONFIGS["config4"]
    inp, t = _inputs(cfg, seed=5)
    n = cfg["n"]
    dout = torch.randn(n, cfg["h"], generator=torch.Generator().manual_seed(11)).to(torch.bfloat16).to(DEV)
    out, g = _fwd_bwd(t, t["x"], dout)
    out2, g2 = _fwd_bwd(t, t["x"], dout)
    for a, b in zip(g, g2):
        assert torch.equal(a, b), "backward is not deterministic"
    cut = n // 2 + 333
    _, ga = _fwd_bwd(t, t["x"][:cut].contiguous(), dout[:cut].contiguous())
    _, gb = _fwd_bwd(t, t["x"][cut:].contiguous(), dout[cut:].contiguous())
    assert torch.equal(torch.cat([ga[0], gb[0]]), g[0]), "dx of a token depends on the other tokens"
    for name, whole, pa, pb in zip(("d_w_router", "d_gate_up_proj", "d_down_proj", "d_theta"), g[1:], ga[1:], gb[1:]):
        s = pa.float() + pb.float()                      # each part is rounded to bf16 once more than the whole
        assert rel_err(whole.float(), s) < BF16_MAX and mean_rel_err(whole.float(), s) < BF16_MEAN, name
    pick = torch.randperm(n, generator=torch.Generator().manual_seed(4))[:192].sort().values
    c = {k: (v.to(torch.bfloat16).float() if k in ("x", "w_router", "gate_up_proj", "down_proj") else v.clone())
         for k, v in inp.items()}
    xs = c["x"][pick].clone().requires_grad_(True)
    ref, logits, idx, w, _ = orc.moe_forward(xs, c["w_router"], c["bias"], c["gate_up_proj"], c["down_proj"],
                                             c["radial_theta"], K, return_routing=True)
    (ref * dout.cpu()[pick].float()).sum().backward()
    got = g[0].float().cpu()[pick]
    assert rel_err(got, xs.grad) < BF16_MAX and mean_rel_err(got, xs.grad) < BF16_MEAN
