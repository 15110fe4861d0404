"""Worker of the expert-parallel MODULE test (launched by tests/test_gpu_ep.py through torch.distributed.run).

Every rank builds the same single-GPU BiBoMoELayer (seeded weights), shards it into an
ExpertParallelMoELayer and trains one step on its own tokens; results are compared with the
single-GPU layer run on the concatenated batch of all ranks: forward bit-identical, gradients at the
bf16 bars (the two paths sum the same bf16 values in a different order), and the balancer's bias
update identical.  A RouterTrace on each layer: the sharded layer's sums over this rank's tokens against
the single-GPU layer's trace of the same tokens."""
import os
import pathlib
import sys

import torch
import torch.distributed as dist

ROOT = pathlib.Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def rel(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


def main():
    n, hidden, inter, n_exp, k = (int(a) for a in sys.argv[1:6])
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from bibo_b200 import BiBoMoELayer, MoEConfig, RouterTrace, ep
    from oracle import moe_oracle as orc

    # the balancer updates every round(threshold / tokens of this rank's forward) forwards: with these thresholds both
    # layers update on their first forward (the sharded layer sees n tokens per rank, the full one n * world)
    cfg = MoEConfig(hidden_size=hidden, moe_intermediate_size=inter, num_routed_experts=n_exp, num_experts_per_tok=k,
                    bias_update_factor=0.4, bias_update_threshold=n * world)
    cfg_shard = MoEConfig(hidden_size=hidden, moe_intermediate_size=inter, num_routed_experts=n_exp, num_experts_per_tok=k,
                          bias_update_factor=0.4, bias_update_threshold=n)
    inp = orc.make_inputs(n * world, hidden, inter, n_exp, seed=41, bias_mode="uniform", theta_std=0.5)
    dout = torch.randn(n * world, hidden, generator=torch.Generator().manual_seed(42)).to(torch.bfloat16).to(dev)
    full = BiBoMoELayer(cfg)
    with torch.no_grad():
        full.gate.gate_proj.weight.copy_(inp["w_router"]); full.gate.bias.copy_(inp["bias"])
        full.experts.gate_up_proj.copy_(inp["gate_up_proj"]); full.experts.down_proj.copy_(inp["down_proj"])
        full.experts.radial_theta.copy_(inp["radial_theta"])
    full = full.to(dev).to(torch.bfloat16).train()
    full.gate.bias.data = inp["bias"].to(dev)
    full.experts.radial_theta.data = inp["radial_theta"].to(dev)
    shard = ep.ExpertParallelMoELayer.from_full_layer(full, cfg_shard, dist.group.WORLD, capacity_factor=float(world)).to(dev)
    shard = shard.to(torch.bfloat16).train()
    shard.gate.bias.data = full.gate.bias.data.clone()
    lo, hi = rank * shard.el, (rank + 1) * shard.el
    shard.radial_theta.data = inp["radial_theta"][lo:hi].to(dev)
    # the cast above also took the balancer's histogram buffer to bf16 (8 bits of mantissa: counts above 256 would be
    # rounded, differently in the two layers, which sum them in a different order); keep it fp32 like bias and theta
    full.accumulated_tpe = full.accumulated_tpe.float()
    shard.accumulated_tpe = shard.accumulated_tpe.float()

    x_all = inp["x"].to(torch.bfloat16).to(dev)
    xs = x_all[rank * n:(rank + 1) * n].clone().requires_grad_(True)
    # routing diagnostics of this rank's tokens: the single-GPU layer on the same tokens (bias not yet updated)
    full.bias_update_factor, keep = 0.0, full.bias_update_factor
    trace_full = RouterTrace(torch.nn.ModuleDict({"m": full}), n_exp, dev)
    full.gate._probe_gap = True
    with torch.no_grad():
        full(xs.detach().unsqueeze(0))
    want_acc, want_counts, want_gap = trace_full.acc.clone(), trace_full.counts.clone(), full.gate.boundary_gap.clone()
    trace_full.close()
    full.gate._probe_gap = False
    full.bias_update_factor = keep
    trace_shard = RouterTrace(torch.nn.ModuleDict({"m": shard}), n_exp, dev)
    shard.gate._probe_gap = True
    out = shard(xs.unsqueeze(0))[0]
    (out * dout[rank * n:(rank + 1) * n]).sum().backward()
    xf = x_all.clone().requires_grad_(True)
    ref = full(xf.unsqueeze(0))[0]
    (ref * dout).sum().backward()
    torch.cuda.synchronize()

    ok = True
    msgs = []
    same_fwd = torch.equal(out.detach(), ref.detach()[rank * n:(rank + 1) * n])
    ok &= same_fwd
    msgs.append(f"forward identical {same_fwd}")
    checks = {
        "dx": (xs.grad, xf.grad[rank * n:(rank + 1) * n]),
        "d_gate_up_proj": (shard.gate_up_proj.grad, full.experts.gate_up_proj.grad[lo:hi]),
        "d_down_proj": (shard.down_proj.grad, full.experts.down_proj.grad[lo:hi]),
        "d_radial_theta": (shard.radial_theta.grad.float(), full.experts.radial_theta.grad[lo:hi].float()),
        "d_w_router": (shard.gate.gate_proj.weight.grad, full.gate.gate_proj.weight.grad),
    }
    for name, (got, want) in checks.items():
        r = rel(got.float(), want.float())
        msgs.append(f"{name} {r:.2e}")
        ok &= r < 2e-2
    trace_same = (torch.equal(trace_shard.acc, want_acc) and torch.equal(trace_shard.counts, want_counts)
                  and torch.equal(shard.gate.boundary_gap, want_gap) and float(want_acc[2]) == n)
    msgs.append(f"router trace identical {trace_same}")
    ok &= trace_same
    bias_same = torch.allclose(shard.gate.bias.data, full.gate.bias.data, rtol=0, atol=1e-7)
    moved = float((full.gate.bias.data - inp["bias"].to(dev)).abs().max()) > 0
    bias_diff = float((shard.gate.bias.data - full.gate.bias.data).abs().max())
    msgs.append(f"bias update identical {bias_same} (moved {moved}, max diff {bias_diff:.2e}, update every "
                f"{shard._update_every} / {full._update_every} forwards, forwards {shard._fwd_step} / {full._fwd_step})")
    ok &= bias_same and moved
    print(f"rank {rank}: " + "; ".join(msgs), flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
