"""The gate/up kernel that gathers its own rows (bibo_moe_rowmap_fwd + bibo_moe_gemm1_gather_fwd) against the
permute pass followed by the plain gate/up kernel: every buffer must come out bit-identical, on ragged
token counts, near-empty experts (Zipf bias), both intermediate sizes with a CTA-pair kernel, with and
without zero-filled padding rows, and through the stage entry points as well as the whole block."""
import pytest
import torch

from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
K, E = 6, 64

CASES = {
    "ragged_i256": dict(n=5000, h=1024, i=256, bias_mode="uniform", zipf_alpha=0.0),
    "small_i512": dict(n=300, h=512, i=512, bias_mode="uniform", zipf_alpha=0.0),
    "c4_slice_i512": dict(n=8192, h=2048, i=512, bias_mode="zero", zipf_alpha=0.0),
    "zipf_i512": dict(n=6000, h=2048, i=512, bias_mode="zipf", zipf_alpha=1.0),
    "many_pairs_i256": dict(n=40000, h=1024, i=256, bias_mode="uniform", zipf_alpha=0.0),
}


def _inputs(cfg, seed=11):
    inp = orc.make_inputs(cfg["n"], cfg["h"], cfg["i"], E, seed=seed, bias_mode=cfg["bias_mode"], theta_std=0.5,
                          zipf_alpha=cfg["zipf_alpha"] or 1.0)
    t = {k: v.to(DEV) for k, v in inp.items()}
    for k in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[k] = t[k].to(torch.bfloat16).contiguous()
    return t


def _run(t, separate, zero_padding):
    from bibo_b200 import functional as Fn
    x = t["x"]
    geo = Fn.Geometry(x.shape[0], x.shape[1], t["gate_up_proj"].shape[1] // 2, E, E, 0, K, torch.bfloat16)
    ws = Fn.MoEWorkspace(geo, x.device, keep_gate_up=True)
    ws.xp.fill_(float("nan"))          # a row nobody writes must not look right by accident
    ws.row_token.fill_(-7)
    out, ws = Fn.moe_forward(x, t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], K,
                             ws=ws, zero_padding=zero_padding, gather_in_gemm=not separate)
    torch.cuda.synchronize()
    assert Fn.plan_header(ws)[2] == 0, "device status word"
    return out, ws


@pytest.mark.parametrize("zero_padding", [False, True])
@pytest.mark.parametrize("name", sorted(CASES))
def test_gathering_kernel_equals_permute_then_gemm(name, zero_padding):
    from bibo_b200 import _lib
    cfg = CASES[name]
    assert _lib.load().bibo_moe_gemm1_gather_supported(cfg["h"], cfg["i"], _lib.BF16) == 1
    t = _inputs(cfg)
    out_a, ws_a = _run(t, separate=True, zero_padding=zero_padding)
    out_b, ws_b = _run(t, separate=False, zero_padding=zero_padding)
    assert torch.equal(ws_a.plan[:4], ws_b.plan[:4])
    assert torch.equal(ws_a.slot_row, ws_b.slot_row)
    rows = int(ws_a.plan[1])
    tok_a, tok_b = ws_a.row_token[:rows], ws_b.row_token[:rows]
    valid = tok_a >= 0
    assert torch.equal(tok_a[valid], tok_b[valid]) and bool((tok_b[~valid] < 0).all())
    # every valid row holds its token's activations, in both buffers
    assert torch.equal(ws_b.xp[:rows][valid].view(torch.int16), t["x"][tok_a[valid].long()].view(torch.int16))
    assert torch.equal(ws_a.xp[:rows][valid].view(torch.int16), ws_b.xp[:rows][valid].view(torch.int16))
    if zero_padding:
        assert bool((ws_b.xp[:rows][~valid] == 0).all()), "padding rows inside the tiles are zero"
    for name_ in ("h", "y", "gate_up", "rnorm"):
        a, b = getattr(ws_a, name_)[:rows][valid], getattr(ws_b, name_)[:rows][valid]
        assert torch.equal(a.view(torch.int16 if a.dtype == torch.bfloat16 else torch.int32),
                           b.view(torch.int16 if b.dtype == torch.bfloat16 else torch.int32)), name_
    assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))


def test_stage_entry_points_and_repeat_calls():
    """rowmap + gather entry called directly, three times on one workspace (the arrival counters of the
    gather are cleared by every launch), against permute + plain kernel."""
    from bibo_b200 import _lib, functional as Fn
    lib, p = _lib.load(), _lib.ptr
    cfg = CASES["ragged_i256"]
    t = _inputs(cfg, seed=5)
    n, h, i = cfg["n"], cfg["h"], cfg["i"]
    geo = Fn.Geometry(n, h, i, E, E, 0, K, torch.bfloat16)
    ws = Fn.MoEWorkspace(geo, DEV, keep_gate_up=False)
    st = torch.cuda.current_stream().cuda_stream
    Fn.router_forward(t["x"], t["w_router"], t["bias"], K, ws=ws)
    _lib.check(lib.bibo_moe_plan(p(ws.block_counts), n, K, E, E, p(ws.plan), st), "plan")
    _lib.check(lib.bibo_moe_permute_fwd(p(t["x"]), p(ws.topk_idx), p(ws.slot_rank), p(ws.plan), n, h, E, E, K, _lib.BF16,
                                        0, p(ws.xp), p(ws.slot_row), p(ws.row_token), st), "permute")
    _lib.check(lib.bibo_moe_gemm1_radial_fwd(p(ws.xp), p(t["gate_up_proj"]), p(t["radial_theta"]), p(ws.plan), n, h, i,
                                             E, E, K, _lib.BF16, p(ws.h), None, None, st), "gemm1")
    torch.cuda.synchronize()
    rows = int(ws.plan[1])
    valid = ws.row_token[:rows] >= 0
    h_ref, slot_row_ref = ws.h[:rows][valid].clone(), ws.slot_row.clone()
    for _ in range(3):
        ws.xp.fill_(float("nan")); ws.h.zero_(); ws.slot_row.fill_(-5)
        _lib.check(lib.bibo_moe_rowmap_fwd(p(ws.topk_idx), p(ws.slot_rank), p(ws.plan), n, E, E, K, p(ws.slot_row),
                                           p(ws.row_token), st), "rowmap")
        _lib.check(lib.bibo_moe_gemm1_gather_fwd(p(t["x"]), p(ws.row_token), p(t["gate_up_proj"]), p(t["radial_theta"]),
                                                 p(ws.plan), n, h, i, E, E, K, _lib.BF16, 0, p(ws.xp), p(ws.h), None, None,
                                                 st), "gemm1_gather")
        torch.cuda.synchronize()
        assert int(ws.plan[2]) == 0
        assert torch.equal(ws.slot_row, slot_row_ref)
        assert torch.equal(ws.h[:rows][valid].view(torch.int16), h_ref.view(torch.int16))


def test_unsupported_shape_is_refused():
    from bibo_b200 import _lib
    lib = _lib.load()
    assert lib.bibo_moe_gemm1_gather_supported(1024, 128, _lib.BF16) == 0
    assert lib.bibo_moe_gemm1_gather_supported(1024, 256, _lib.F32) == 0
