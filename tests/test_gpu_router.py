"""K1 + plan + K2 on the GPU against the oracle (through the C-ABI)."""
import pytest
import torch

from conftest import GOLDEN_CASES, load_golden, rel_err
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _fn():
    from bibo_b200 import functional as Fn
    return Fn


def _check_selection(logits_cpu, bias_cpu, k, norm, idx, w, gap_tol=1e-6):
    """Exact set equality with the oracle, except tokens whose k/k+1 biased-score gap is below
    gap_tol (there the last bit of the sigmoid decides and both answers are accepted)."""
    ref_idx, ref_w, ref_counts = orc.router_select(logits_cpu, bias_cpu, k, norm)
    same = (idx.cpu().long() == ref_idx).all(-1)
    gap = orc.boundary_gap(logits_cpu, bias_cpu, k)
    bad = (~same) & (gap >= gap_tol)
    assert int(bad.sum()) == 0, f"{int(bad.sum())} tokens differ from the oracle away from a tie"
    assert torch.allclose(w.cpu()[same], ref_w[same], rtol=0, atol=1e-6)
    return int((~same).sum()), ref_counts


@pytest.mark.parametrize("name", GOLDEN_CASES + ["config1"])
def test_selection_from_reference_logits(name):
    """Golden logits (written by the reference) in -> selected sets, weights, counts out."""
    Fn = _fn()
    rec, inp = load_golden(name)
    if rec["rows_step"] != 1:
        logits = orc.router_logits(inp["x"], inp["w_router"])
    else:
        logits = rec["logits"]
    idx, w, rank, bc, _ = Fn.router_forward(None, None, inp["bias"].to(DEV), rec["top_k"], rec["norm"],
                                            logits_in=logits.to(DEV))
    flips, _ = _check_selection(logits, inp["bias"], rec["top_k"], rec["norm"], idx, w)
    if flips == 0:
        assert torch.equal(idx.cpu().to(torch.int16), rec["idx_sorted"])
        assert torch.equal(bc.sum(0).cpu(), rec["counts"])
        assert torch.allclose(w.cpu(), rec["w_sorted"], rtol=0, atol=1e-6)


@pytest.mark.parametrize("n,e,k,bias_mode", [(4096, 64, 6, "uniform"), (1000, 64, 6, "zipf"), (257, 22, 2, "uniform"),
                                             (128, 8, 8, "zero"), (1, 64, 6, "uniform"), (300, 256, 8, "uniform")])
def test_selection_matches_oracle_on_the_same_device(n, e, k, bias_mode):
    """With the oracle's ops running on the same GPU (same sigmoid), selection is bit-exact."""
    Fn = _fn()
    g = torch.Generator().manual_seed(n + e)
    logits = torch.randn(n, e, generator=g) * 0.9
    inp = orc.make_inputs(8, 8, 8, e, seed=3, bias_mode=bias_mode, zipf_alpha=0.1)
    bias = inp["bias"]
    for norm in ("sum", "softmax", False):
        idx, w, rank, bc, _ = Fn.router_forward(None, None, bias.to(DEV), k, norm, logits_in=logits.to(DEV))
        ref_idx, ref_w, ref_counts = orc.router_select(logits.to(DEV), bias.to(DEV), k, norm)
        assert torch.equal(idx.long(), ref_idx)
        assert torch.equal(bc.sum(0).long(), ref_counts)
        assert torch.allclose(w, ref_w, rtol=0, atol=1e-6)
        _check_selection(logits, bias, k, norm, idx, w)


def test_ties_go_to_the_lowest_index():
    Fn = _fn()
    logits = torch.zeros(5, 64, device=DEV)
    idx, w, *_ = Fn.router_forward(None, None, torch.zeros(64, device=DEV), 6, "sum", logits_in=logits)
    assert idx.cpu().tolist() == [[0, 1, 2, 3, 4, 5]] * 5
    assert torch.allclose(w, torch.full_like(w, 1 / 6), atol=1e-7)


def test_routed_scaling_factor_scales_weights():
    Fn = _fn()
    logits = torch.randn(64, 64, device=DEV)
    b = torch.zeros(64, device=DEV)
    _, w1, *_ = Fn.router_forward(None, None, b, 6, "sum", 1.0, logits_in=logits)
    _, w2, *_ = Fn.router_forward(None, None, b, 6, "sum", 2.5, logits_in=logits)
    assert torch.allclose(w2, w1 * 2.5, rtol=1e-6, atol=0)


@pytest.mark.parametrize("dtype,n,h,e", [(torch.float32, 300, 64, 8), (torch.float32, 2048, 512, 64),
                                         (torch.bfloat16, 1000, 1024, 64), (torch.bfloat16, 130, 72, 22)])
def test_logits_match_fp32_product(dtype, n, h, e):
    Fn = _fn()
    inp = orc.make_inputs(n, h, 8, e, seed=11, bias_mode="uniform")
    x, wr = inp["x"].to(dtype), inp["w_router"].to(dtype)
    *_, logits = Fn.router_forward(x.to(DEV), wr.to(DEV), inp["bias"].to(DEV), min(6, e), "sum", want_logits=True)
    ref = x.double() @ wr.double().T
    assert rel_err(logits.cpu(), ref) < (1e-5 if dtype == torch.float32 else 1e-5)


@pytest.mark.parametrize("n,e,n_glu,k", [(1000, 64, 64, 6), (130, 8, 6, 2), (128, 64, 64, 6), (5, 8, 8, 2)])
def test_plan_and_permute_layout(n, e, n_glu, k):
    """counts / offsets / tiles agree with a host recomputation; permuted rows hold the right
    tokens in ascending token order; padding rows are marked and zeroed."""
    Fn = _fn()
    from bibo_b200 import _lib
    lib = _lib.load()
    h = 64
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, h, generator=g).to(DEV)
    logits = torch.randn(n, e, generator=g).to(DEV)
    geo = Fn.Geometry(n, h, 16, e, n_glu, (e - n_glu) // 2, k, torch.float32)
    ws = Fn.MoEWorkspace(geo, DEV)
    ws.xp.fill_(float("nan"))
    idx, w, rank, bc, _ = Fn.router_forward(None, None, torch.zeros(e, device=DEV), k, "sum", ws=ws, logits_in=logits)
    st = torch.cuda.current_stream().cuda_stream
    p = _lib.ptr
    _lib.check(lib.bibo_moe_plan(p(ws.block_counts), n, k, e, n_glu, p(ws.plan), st), "plan")
    _lib.check(lib.bibo_moe_permute_fwd(p(x), p(idx), p(rank), p(ws.plan), n, h, e, n_glu, k, 0, 1, p(ws.xp),
                                        p(ws.slot_row), p(ws.row_token), st), "permute")
    n_tiles, rows_used, status = Fn.plan_header(ws)
    assert status == 0
    counts = torch.bincount(idx.flatten().long().cpu(), minlength=e)
    assert torch.equal(ws.counts().cpu().long(), counts)
    padded = (counts[:n_glu] + 127) // 128 * 128
    off = torch.cat([torch.zeros(1, dtype=torch.long), padded.cumsum(0)])
    assert torch.equal(ws.expert_off().cpu().long(), off)
    assert rows_used == int(off[-1]) and n_tiles == rows_used // 128
    tiles = ws.tiles().cpu()[:n_tiles]
    t = 0
    for ex in range(n_glu):
        for r in range(0, int(counts[ex]), 128):
            assert tiles[t].tolist() == [ex, int(off[ex]) + r, min(128, int(counts[ex]) - r), 0]
            t += 1
    assert t == n_tiles
    slot_row, row_token, xp = ws.slot_row.cpu().long(), ws.row_token.cpu().long(), ws.xp.cpu()
    idx_c = idx.cpu().long()
    for ex in range(e):
        sel = (idx_c == ex)
        toks = sel.any(-1).nonzero().flatten()
        rows = slot_row[sel]
        if ex < n_glu:
            assert torch.equal(rows, int(off[ex]) + torch.arange(len(toks))), "ascending token order inside an expert"
            assert torch.equal(row_token[rows], toks)
            assert torch.equal(xp[rows], x.cpu()[toks])
            pad = torch.arange(int(off[ex]) + int(counts[ex]), int(off[ex + 1]))
            assert (row_token[pad] == -1).all() and (xp[pad] == 0).all()
        else:
            assert (rows == -1).all()
