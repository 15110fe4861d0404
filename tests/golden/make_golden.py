"""Generate the golden fixtures in this folder by running the UNMODIFIED reference.

Usage (only where the reference checkout exists; the fixtures themselves are committed):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <path to BiBo checkout>

The script imports ``src.modeling.ffn.moe.BiBoMoELayer`` from the reference checkout, copies
seeded weights into it, runs forward (and backward) on CPU and stores outputs and gradients (inputs are
regenerated from the seed by ``oracle.moe_oracle.make_inputs``).  ``tests/test_oracle.py`` replays the files through ``oracle/moe_oracle.py``; the GPU
parity tests replay them through the CUDA path.
"""
import argparse
import os
import pathlib
import sys

import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
from oracle import moe_oracle as orc  # noqa: E402  (input generator only)


def KEEP_EXPERTS(n_glu):
    return [0, n_glu // 2, n_glu - 1]


def upstream_grad(n_tokens, hidden, seed):
    """The seeded dOut every backward fixture uses."""
    return torch.randn(1, n_tokens, hidden, generator=torch.Generator().manual_seed(seed * 1000 + 77))


def grad_digest(g, seed):
    """[E, 2]: per-expert L2 norm and inner product with a seeded N(0,1) probe of g's shape."""
    probe = torch.randn(g.shape, generator=torch.Generator().manual_seed(seed * 1000 + 99))
    flat, pf = g.reshape(g.shape[0], -1).double(), probe.reshape(g.shape[0], -1).double()
    return torch.stack([flat.norm(dim=1), (flat * pf).sum(1)], dim=1)


def build_layer(ref_root, hidden, inter, n_experts, top_k, pairs, norm, dtype):
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    from src.configuration_bibo import BiBoConfig
    from src.modeling.ffn.moe import BiBoMoELayer
    cfg = BiBoConfig(vocab_size=512, hidden_size=hidden, num_hidden_layers=4, num_attention_heads=4,
                     num_key_value_heads=2, intermediate_size=inter, moe_intermediate_size=inter,
                     num_routed_experts=n_experts, special_expert_pairs=pairs,
                     num_experts_per_tok=top_k, norm_topk_prob=norm, bias_update_factor=0.4)
    layer = BiBoMoELayer(cfg).eval()
    return layer.to(dtype)


def run_case(ref_root, name, n_tokens, hidden, inter, n_experts, top_k, pairs=0, norm="sum",
             bias_mode="uniform", theta_std=0.5, seed=1, dtype=torch.float32, backward=True,
             keep_rows=None):
    n_glu = n_experts - 2 * pairs
    inp = orc.make_inputs(n_tokens, hidden, inter, n_experts, seed=seed, bias_mode=bias_mode,
                          theta_std=theta_std)
    layer = build_layer(ref_root, hidden, inter, n_experts, top_k, pairs, norm, dtype)
    with torch.no_grad():
        layer.gate.gate_proj.weight.copy_(inp["w_router"])
        layer.gate.bias.copy_(inp["bias"])
        layer.experts.gate_up_proj.copy_(inp["gate_up_proj"][:n_glu])
        layer.experts.down_proj.copy_(inp["down_proj"][:n_glu])
        layer.experts.radial_theta.copy_(inp["radial_theta"][:n_glu])
    x = inp["x"].to(dtype).reshape(1, n_tokens, hidden).clone().requires_grad_(backward)
    logits = layer.gate.router_logits(x.detach())
    idx, w = layer.gate(x)
    out = layer(x)
    rec = dict(name=name, n_tokens=n_tokens, hidden=hidden, inter=inter, n_experts=n_experts,
               n_glu=n_glu, pairs=pairs, top_k=top_k, norm=norm, seed=seed, bias_mode=bias_mode,
               theta_std=theta_std, dtype=str(dtype).split(".")[-1])
    order = idx[0].argsort(-1)
    rec["idx_sorted"] = idx[0].gather(-1, order).to(torch.int16)
    rec["w_sorted"] = w[0].detach().gather(-1, order)
    rec["counts"] = torch.bincount(idx.flatten(), minlength=n_experts).to(torch.int32)
    rows = slice(None) if keep_rows is None else slice(0, n_tokens, n_tokens // keep_rows)
    rec["rows_step"] = 1 if keep_rows is None else n_tokens // keep_rows
    rec["logits"] = logits.detach()[rows].clone()
    rec["out"] = out.detach()[0][rows].clone()
    if backward:
        dout = upstream_grad(n_tokens, hidden, seed).to(dtype)
        (out * dout).sum().backward()
        rec["dx"] = x.grad[0].clone()
        rec["d_radial_theta"] = layer.experts.radial_theta.grad.clone()
        rec["d_w_router"] = layer.gate.gate_proj.weight.grad.clone()
        # expert-weight gradients are large: keep three experts whole plus, for every expert, the
        # L2 norm and the inner product with a seeded probe tensor (see grad_digest)
        for key, g in (("d_gate_up_proj", layer.experts.gate_up_proj.grad),
                       ("d_down_proj", layer.experts.down_proj.grad)):
            rec[key + "_digest"] = grad_digest(g.float(), seed)
            rec[key + "_experts"] = KEEP_EXPERTS(n_glu)
            rec[key + "_sel"] = g[KEEP_EXPERTS(n_glu)].clone()
    torch.save(rec, HERE / f"{name}.pt")
    sz = os.path.getsize(HERE / f"{name}.pt") / 1024
    print(f"{name}: out abs-mean {out.abs().mean():.4e}  counts min/max "
          f"{int(rec['counts'].min())}/{int(rec['counts'].max())}  {sz:.0f} KiB")


def run_mlp_case(ref_root, name, n_tokens, hidden, inter, seed, shared_in_layer=False, n_experts=64, top_k=6,
                 moe_inter=64, n_shared=2):
    """The reference's dense SwiGLU MLP (src/modeling/ffn/mlp.py) alone, or as the shared expert of the
    MoE layer (use_shared_expert=True, width moe_inter * n_shared); fp32 on CPU."""
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    from src.configuration_bibo import BiBoConfig
    from src.modeling.ffn.mlp import BiBoMLP
    from src.modeling.ffn.moe import BiBoMoELayer
    rec = dict(name=name, n_tokens=n_tokens, hidden=hidden, inter=inter, seed=seed, shared_in_layer=shared_in_layer)
    w = orc.make_mlp_weights(hidden, inter, seed)
    if not shared_in_layer:
        cfg = BiBoConfig(vocab_size=512, hidden_size=hidden, num_hidden_layers=4, num_attention_heads=4,
                         num_key_value_heads=2, intermediate_size=inter, moe_intermediate_size=moe_inter,
                         num_routed_experts=n_experts, special_expert_pairs=0, num_experts_per_tok=top_k)
        mlp = BiBoMLP(cfg).eval()
        x = torch.randn(n_tokens, hidden, generator=torch.Generator().manual_seed(seed * 1000 + 1))
    else:
        assert inter == moe_inter * n_shared
        cfg = BiBoConfig(vocab_size=512, hidden_size=hidden, num_hidden_layers=4, num_attention_heads=4,
                         num_key_value_heads=2, intermediate_size=4 * hidden, moe_intermediate_size=moe_inter,
                         num_routed_experts=n_experts, special_expert_pairs=0, num_experts_per_tok=top_k,
                         use_shared_expert=True, shared_expert_type="mlp", num_shared_experts=n_shared,
                         bias_update_factor=0.4)
        layer = BiBoMoELayer(cfg).eval()
        inp = orc.make_inputs(n_tokens, hidden, moe_inter, n_experts, seed=seed, bias_mode="uniform", theta_std=0.5)
        with torch.no_grad():
            layer.gate.gate_proj.weight.copy_(inp["w_router"])
            layer.gate.bias.copy_(inp["bias"])
            layer.experts.gate_up_proj.copy_(inp["gate_up_proj"])
            layer.experts.down_proj.copy_(inp["down_proj"])
            layer.experts.radial_theta.copy_(inp["radial_theta"])
        mlp = layer.shared_experts_list[0]
        x = inp["x"]
        rec.update(n_experts=n_experts, top_k=top_k, moe_inter=moe_inter, n_shared=n_shared)
    with torch.no_grad():
        mlp.gate_proj.weight.copy_(w["gate_proj"])
        mlp.up_proj.weight.copy_(w["up_proj"])
        mlp.down_proj.weight.copy_(w["down_proj"])
    # forward and autograd gradients (upstream gradient = the seeded dOut of the other fixtures)
    xg = x.clone().requires_grad_(True)
    out = layer(xg.reshape(1, n_tokens, hidden))[0] if shared_in_layer else mlp(xg)
    (out * upstream_grad(n_tokens, hidden, seed)[0]).sum().backward()
    rec["out"] = out.detach().clone()
    rec["dx"] = xg.grad.clone()
    for key, prm in (("d_gate_proj", mlp.gate_proj.weight), ("d_up_proj", mlp.up_proj.weight),
                     ("d_down_proj", mlp.down_proj.weight)):
        rec[key + "_digest"] = grad_digest(prm.grad.float(), seed)      # per row: L2 norm, probe inner product
        rec[key + "_head"] = prm.grad[:8].clone()
    torch.save(rec, HERE / f"{name}.pt")
    print(f"{name}: out abs-mean {out.abs().mean():.4e}  {os.path.getsize(HERE / f'{name}.pt') / 1024:.0f} KiB")


def run_ffn_case(ref_root, name, n_tokens, hidden, inter, n_experts, top_k, seed):
    """BiBoDecoderLayer._ffn_forward of a MoE layer (src/modeling/layers.py:57-67): post-attention RMSNorm,
    MoE block, residual add; fp32 on CPU.  The norm weight is 1 + 0.1 N(0,1) from its own generator."""
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    from src.configuration_bibo import BiBoConfig
    from src.modeling.layers import BiBoDecoderLayer
    cfg = BiBoConfig(vocab_size=512, hidden_size=hidden, num_hidden_layers=4, num_attention_heads=4,
                     num_key_value_heads=2, intermediate_size=4 * hidden, moe_intermediate_size=inter,
                     num_routed_experts=n_experts, special_expert_pairs=0, num_experts_per_tok=top_k)
    layer_idx = next(i for i in range(cfg.num_hidden_layers) if i not in cfg.mlp_only_layers)
    dl = BiBoDecoderLayer(cfg, layer_idx=layer_idx).eval()
    inp = orc.make_inputs(n_tokens, hidden, inter, n_experts, seed=seed, bias_mode="uniform", theta_std=0.5)
    norm_w = 1.0 + 0.1 * torch.randn(hidden, generator=torch.Generator().manual_seed(seed * 1000 + 31))
    with torch.no_grad():
        dl.post_attention_layernorm.weight.copy_(norm_w)
        dl.mlp.gate.gate_proj.weight.copy_(inp["w_router"])
        dl.mlp.gate.bias.copy_(inp["bias"])
        dl.mlp.experts.gate_up_proj.copy_(inp["gate_up_proj"])
        dl.mlp.experts.down_proj.copy_(inp["down_proj"])
        dl.mlp.experts.radial_theta.copy_(inp["radial_theta"])
        out = dl._ffn_forward(inp["x"].reshape(1, n_tokens, hidden))[0]
        normed = dl.post_attention_layernorm(inp["x"])
    rec = dict(name=name, n_tokens=n_tokens, hidden=hidden, inter=inter, n_experts=n_experts, top_k=top_k, seed=seed,
               eps=float(dl.post_attention_layernorm.variance_epsilon), out=out.clone(), normed=normed.clone())
    torch.save(rec, HERE / f"{name}.pt")
    print(f"{name}: out abs-mean {out.abs().mean():.4e}  {os.path.getsize(HERE / f'{name}.pt') / 1024:.0f} KiB")


def run_trace_case(ref_root, name, n_tokens, hidden, inter, n_experts, top_k, pairs, norm, seeds):
    """The reference's RouterTrace (ablate/common/router_trace.py) hooked onto its own layer in training
    mode: its accumulator and expert counts after each forward, and what flush() reports."""
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    from ablate.common.router_trace import RouterTrace
    n_glu = n_experts - 2 * pairs
    layer = build_layer(ref_root, hidden, inter, n_experts, top_k, pairs, norm, torch.float32).train()
    layer.bias_update_factor = 0.0           # keep the bias fixed between the forwards
    model = torch.nn.ModuleDict({"mlp": layer})
    trace = RouterTrace(model, n_experts, "cpu")
    rec = dict(name=name, n_tokens=n_tokens, hidden=hidden, inter=inter, n_experts=n_experts, n_glu=n_glu,
               pairs=pairs, top_k=top_k, norm=norm, seeds=list(seeds), acc=[], counts=[], gap=[])
    for seed in seeds:
        inp = orc.make_inputs(n_tokens, hidden, inter, n_experts, seed=seed, bias_mode="uniform", theta_std=0.5)
        if seed == seeds[0]:                 # weights of the first seed; later seeds only change x
            with torch.no_grad():
                layer.gate.gate_proj.weight.copy_(inp["w_router"])
                layer.gate.bias.copy_(inp["bias"])
                layer.experts.gate_up_proj.copy_(inp["gate_up_proj"][:n_glu])
                layer.experts.down_proj.copy_(inp["down_proj"][:n_glu])
                layer.experts.radial_theta.copy_(inp["radial_theta"][:n_glu])
        with torch.no_grad():
            layer(inp["x"].reshape(1, n_tokens, hidden))
        rec["acc"].append(trace.acc.clone())
        rec["counts"].append(trace.counts.clone())
        rec["gap"].append(layer.gate.boundary_gap.clone())
    rec["flush"] = trace.flush()
    trace.close()
    torch.save(rec, HERE / f"{name}.pt")
    print(f"{name}: " + ", ".join(f"{k.split('/')[-1]} {v:.4f}" for k, v in rec["flush"].items()))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    a = ap.parse_args()
    torch.set_num_threads(8)
    r = a.reference
    # the reference's own test geometry: hidden 64, 8 experts, top-2, intermediate 96
    run_case(r, "tiny_glu", 16, 64, 96, 8, 2, pairs=0, seed=1)
    run_case(r, "tiny_specials", 16, 64, 96, 8, 2, pairs=1, seed=2)
    run_case(r, "tiny_softmax", 16, 64, 96, 8, 2, pairs=0, norm="softmax", seed=3)
    run_case(r, "tiny_raw", 16, 64, 96, 8, 2, pairs=0, norm=False, seed=4)
    # 64 experts / top-6 at a size the tensor-core kernels accept (hidden, intermediate % 64 == 0)
    run_case(r, "e64_k6_fp32", 320, 128, 64, 64, 6, seed=5)
    run_case(r, "e64_k6_bf16", 320, 128, 64, 64, 6, seed=5, dtype=torch.bfloat16)
    # benchmark configuration 1 (2048 tokens, hidden 512, intermediate 128, bias 0, theta 0,
    # seed 0); every 32nd output row is kept.  Inputs of every case are regenerated from the seed
    # by oracle.moe_oracle.make_inputs and are not stored.
    run_case(r, "config1", 2048, 512, 128, 64, 6, bias_mode="zero", theta_std=0.0, seed=0,
             backward=False, keep_rows=64)
    # dense SwiGLU MLP alone and as the shared expert of the layer (shapes the tensor-core kernels accept)
    run_mlp_case(r, "mlp_dense", 300, 256, 512, seed=7)
    run_mlp_case(r, "layer_shared_expert", 300, 256, 512, seed=8, shared_in_layer=True, moe_inter=256, n_shared=2)
    # the decoder layer's feed-forward half: RMSNorm + MoE block + residual
    run_ffn_case(r, "ffn_moe", 300, 256, 256, 64, 6, seed=9)
    # RouterTrace of the reference over two training forwards: sum-normalised top-6 of 64, and raw weights
    # with one +/-Identity pair
    run_trace_case(r, "router_trace_sum", 320, 128, 64, 64, 6, pairs=0, norm="sum", seeds=(11, 12))
    run_trace_case(r, "router_trace_raw", 320, 128, 64, 64, 6, pairs=1, norm=False, seeds=(13, 14))


if __name__ == "__main__":
    main()
