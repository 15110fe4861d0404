"""Host-side logic that needs no GPU: library symbols, module API, balancer, install seam."""
import ctypes
import os
import pathlib
import re
import sys

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
REF = pathlib.Path(os.environ.get("BIBO_REFERENCE", "/root/reference"))   # a checkout of the reference, where present


def test_library_exports_every_declared_symbol():
    from bibo_b200 import _lib, build
    build.build()
    lib = _lib.load()
    header = (ROOT / "include" / "bibo_moe.h").read_text()
    declared = set(re.findall(r"\b(bibo_moe_\w+)\s*\(", header))
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name)
    assert lib.bibo_moe_version() >= 100


def test_argument_errors_of_the_newer_entry_points_without_a_gpu():
    """Every check below fails before the first CUDA call."""
    from bibo_b200 import _lib
    lib = _lib.load()
    one = ctypes.c_int(0)
    p = ctypes.addressof(one) & ~15 | 16          # a non-null, 16-byte aligned dummy that is never dereferenced
    assert lib.bibo_moe_rowmap_fwd(None, None, None, 10, 64, 64, 6, None, None, None) == -1
    assert lib.bibo_moe_gemm1_gather_supported(1024, 128, _lib.BF16) == 0 and lib.bibo_moe_gemm1_gather_supported(2048, 512, _lib.BF16) == 1
    rc = lib.bibo_moe_gemm1_gather_fwd(p, p, p, p, p, 10, 1024, 128, 64, 64, 6, _lib.BF16, 0, p, p, None, None, None)
    assert rc == -4 and b"intermediate 256 or 512" in lib.bibo_moe_last_error_string()
    assert lib.bibo_moe_ep_copy_to_peers(None, 0, None, 0, 16, 0, 2, 1, None) == -1
    assert lib.bibo_moe_ep_copy_to_peers((ctypes.c_void_p * 2)(p, p), 0, p, 0, 16, 3, 2, 1, None) == -1      # rank >= world
    assert lib.bibo_moe_ep_localize(None, 10, 6, 64, 0, 2, None, None) == -1
    assert lib.bibo_moe_ep_localize(p, 10, 6, 63, 0, 2, p, None) == -1                                        # 63 experts over 2 ranks
    assert lib.bibo_moe_ep_dedup_push(None, None, None, None, 128, 512, 6, 0, 2, 0, None) == -1
    assert lib.bibo_moe_ep_dedup_experts(None, None) == -1 and lib.bibo_moe_ep_dedup_partial(None, None) == -1
    assert lib.bibo_moe_ep_dedup_forward(None, None) == -1
    assert lib.bibo_moe_ep_barrier_bounded(None, 0, 2, 1, 100, None, None) == -1
    assert lib.bibo_moe_route_noalloc_status(None, None) == -1
    assert lib.bibo_moe_ep_dedup_virtual_tokens(8, 1000) == 8000
    assert lib.bibo_moe_ep_dedup_plan_words(4, 1024, 6, 64) == lib.bibo_moe_plan_words(4096, 6, 16, 16)


def test_size_helpers_and_argument_errors_without_a_gpu():
    from bibo_b200 import _lib
    lib = _lib.load()
    assert lib.bibo_moe_rows_cap(1000, 6, 64) == (6000 + 64 * 127 + 127) // 128 * 128
    assert lib.bibo_moe_router_blocks(129) == 2
    assert lib.bibo_moe_tiles_cap(1000, 6, 64) * 128 == lib.bibo_moe_rows_cap(1000, 6, 64)
    # argument validation happens before any CUDA call
    rc = lib.bibo_moe_router_fwd(None, None, None, None, 10, 64, 64, 6, 1, 1.0, 1, None, None, None, None, None, None, None)
    assert rc == -1 and b"null" in lib.bibo_moe_last_error_string()
    rc = lib.bibo_moe_plan(None, 10, 6, 64, 64, None, None)
    assert rc == -1
    one = ctypes.c_int(0)
    p = ctypes.addressof(one)
    rc = lib.bibo_moe_router_fwd(p, p, p, None, 10, 64, 1000, 6, 1, 1.0, 1, None, p, p, p, p, None, None)
    assert rc == -4


def test_module_mirrors_reference_names_and_shapes():
    from bibo_b200 import BiBoMoELayer, MoEConfig
    cfg = MoEConfig(hidden_size=64, moe_intermediate_size=96, num_routed_experts=8, num_experts_per_tok=2,
                    num_pos_identity_experts=1, num_neg_identity_experts=1)
    layer = BiBoMoELayer(cfg)
    sd = layer.state_dict()
    assert sd["experts.gate_up_proj"].shape == (6, 192, 64) and sd["experts.down_proj"].shape == (6, 64, 96)
    assert sd["experts.radial_theta"].shape == (6,) and sd["gate.gate_proj.weight"].shape == (8, 64)
    assert sd["gate.bias"].shape == (8,) and sd["accumulated_tpe"].dtype == torch.float32
    assert layer.gate.bias.requires_grad is False
    e = layer.experts
    assert (e.pos_start, e.pos_end, e.neg_start, e.neg_end) == (6, 7, 7, 8)
    # shared expert: one SwiGLU MLP of width moe_intermediate_size * num_shared_experts (moe.py:120-127)
    shared = BiBoMoELayer(MoEConfig(use_shared_expert=True, num_shared_experts=2, hidden_size=64,
                                    moe_intermediate_size=32, num_routed_experts=8))
    sd = shared.state_dict()
    assert sd["shared_experts_list.0.gate_proj.weight"].shape == (64, 64)
    assert sd["shared_experts_list.0.up_proj.weight"].shape == (64, 64)
    assert sd["shared_experts_list.0.down_proj.weight"].shape == (64, 64)
    with pytest.raises(NotImplementedError):
        BiBoMoELayer(MoEConfig(use_shared_expert=True, shared_expert_type="conv", hidden_size=64,
                               moe_intermediate_size=32, num_routed_experts=8))


def test_balancer_host_logic_matches_reference_tests():
    # tests/test_moe.py:206-249,278-310
    from bibo_b200 import BiBoMoELayer, MoEConfig
    cfg = MoEConfig(hidden_size=64, moe_intermediate_size=32, num_routed_experts=8, num_experts_per_tok=2,
                    bias_update_threshold=48)
    layer = BiBoMoELayer(cfg).train()
    idx = torch.zeros(2, 8, 2, dtype=torch.long)
    fired = [layer._balance_step(idx, 16) is not None for _ in range(7)]
    assert layer._update_every == 3 and fired == [False, False, True, False, False, True, False]
    tpe = torch.full((8,), 10.0)
    tpe[0] = 100.0
    layer.update_bias(tpe)
    assert layer.gate.bias[0] < 0 and (layer.gate.bias[1:] > 0).all()
    assert abs(float(layer.gate.bias.mean())) < 1e-6


@pytest.mark.skipif(not REF.exists(), reason="reference checkout not present on this machine")
def test_install_patches_reference_classes_and_state_dict_is_compatible():
    sys.path.insert(0, str(REF))
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    sys.dont_write_bytecode = True
    from src.configuration_bibo import BiBoConfig
    from src.modeling.ffn import moe as ref
    import bibo_b200
    cfg = BiBoConfig(vocab_size=512, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                     intermediate_size=96, moe_intermediate_size=96, num_routed_experts=8, special_expert_pairs=1,
                     num_experts_per_tok=2)
    ref_layer = ref.BiBoMoELayer(cfg)
    mine = bibo_b200.BiBoMoELayer(cfg)                 # the reference's config object is accepted as is
    mine.load_state_dict(ref_layer.state_dict())       # identical names and shapes
    assert mine.experts.num_glu_experts == 6 and mine.experts.neg_end == 8
    orig = ref.BiBoMoELayer.forward
    bibo_b200.install(ref)
    try:
        assert ref.BiBoMoELayer.forward is not orig
        with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU implementation"):
            ref_layer.eval()(torch.randn(1, 4, 64))    # the patched class refuses CPU tensors loudly
    finally:
        bibo_b200.uninstall()
    assert ref.BiBoMoELayer.forward is orig


@pytest.mark.skipif(not REF.exists(), reason="needs the reference checkout")
def test_install_mlp_seam_and_shared_expert_state_dict():
    sys.path.insert(0, str(REF))
    sys.dont_write_bytecode = True
    from src.configuration_bibo import BiBoConfig
    from src.modeling.ffn import moe as ref
    from src.modeling.ffn.mlp import BiBoMLP as RefMLP
    import bibo_b200
    cfg = BiBoConfig(vocab_size=512, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                     intermediate_size=256, moe_intermediate_size=32, num_routed_experts=8, special_expert_pairs=0,
                     num_experts_per_tok=2, use_shared_expert=True, shared_expert_type="mlp", num_shared_experts=2)
    ref_layer = ref.BiBoMoELayer(cfg)
    mine = bibo_b200.BiBoMoELayer(cfg)
    mine.load_state_dict(ref_layer.state_dict())       # shared_experts_list.0.{gate,up,down}_proj.weight included
    assert mine.shared_experts_list[0].intermediate_size == 64
    dense = bibo_b200.BiBoMLP(cfg)                      # dense layer form: intermediate_size of the config
    dense.load_state_dict(RefMLP(cfg).state_dict())
    assert dense.gate_proj.weight.shape == (256, 64)
    orig = RefMLP.forward
    bibo_b200.install(ref, seam="mlp")
    try:
        assert RefMLP.forward is not orig
        with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU implementation"):
            RefMLP(cfg)(torch.randn(4, 64))
    finally:
        bibo_b200.uninstall()
    assert RefMLP.forward is orig
    from src.modeling.layers import BiBoDecoderLayer
    orig_ffn = BiBoDecoderLayer._ffn_forward
    bibo_b200.install(ref, seam="ffn")
    try:
        assert BiBoDecoderLayer._ffn_forward is not orig_ffn
    finally:
        bibo_b200.uninstall()
    assert BiBoDecoderLayer._ffn_forward is orig_ffn
    with pytest.raises(ValueError):
        bibo_b200.install(ref, seam="attention")


@pytest.mark.parametrize("name", ["router_trace_sum", "router_trace_raw"])
def test_router_trace_flush_matches_the_reference_flush(name):
    """bibo_b200.RouterTrace on CPU buffers: attach / detach, eval forwards skipped, and flush() on the
    accumulator the reference's RouterTrace held after two forwards gives the reference's metrics
    (fixture: tests/golden/make_golden.py run_trace_case)."""
    import torch
    from conftest import GOLDEN
    from bibo_b200 import BiBoMoELayer, MoEConfig, RouterTrace
    rec = torch.load(GOLDEN / f"{name}.pt", weights_only=True)
    cfg = MoEConfig(hidden_size=rec["hidden"], moe_intermediate_size=rec["inter"], num_routed_experts=rec["n_experts"],
                    num_experts_per_tok=rec["top_k"], num_pos_identity_experts=rec["pairs"],
                    num_neg_identity_experts=rec["pairs"], norm_topk_prob=rec["norm"])
    model = torch.nn.ModuleDict({"a": BiBoMoELayer(cfg), "b": BiBoMoELayer(cfg), "other": torch.nn.Linear(4, 4)})
    trace = RouterTrace(model, rec["n_experts"], "cpu")
    assert model["a"]._router_trace is trace and model["b"]._router_trace is trace
    assert trace.n_glu == rec["n_glu"] and trace.pos_end == rec["n_glu"] + rec["pairs"]
    bufs = trace.buffers(model["a"].train())
    assert bufs[0] is trace.acc and bufs[1] is trace.counts and bufs[2] is None
    assert trace.buffers(model["a"].eval()) is None
    assert trace.flush() == {}, "nothing accumulated yet"
    trace.acc.copy_(rec["acc"][-1])
    trace.counts.copy_(rec["counts"][-1])
    got = trace.flush()
    assert list(got) == list(rec["flush"])
    for k, v in rec["flush"].items():
        assert abs(got[k] - v) <= 1e-6 * max(1.0, abs(v)), (k, got[k], v)
    assert float(trace.acc.abs().sum()) == 0 and float(trace.counts.sum()) == 0
    trace.close()
    assert model["a"]._router_trace is None and model["b"]._router_trace is None


def test_ffn_seam_host_logic_without_a_gpu():
    """Which path the feed-forward seam takes is decided on the host: CPU tensors never qualify for the fused
    chain and are refused by the kernels' entry check rather than served by a slower path."""
    import torch
    from bibo_b200 import BiBoMoELayer, MoEConfig
    from bibo_b200.moe import ffn_forward, fused_ffn_applies

    class Norm(torch.nn.Module):
        def __init__(self, h):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.ones(h, dtype=torch.bfloat16))
            self.variance_epsilon = 1e-6

    dl = torch.nn.Module()
    dl.mlp = BiBoMoELayer(MoEConfig(hidden_size=128, moe_intermediate_size=64)).to(torch.bfloat16).eval()
    dl.post_attention_layernorm = Norm(128)
    h = torch.randn(1, 8, 128).to(torch.bfloat16)
    assert not fused_ffn_applies(dl.mlp, h, dl.post_attention_layernorm)
    with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU implementation"):
        ffn_forward(dl, h)
