"""Worker of the expert-parallel BACKWARD test; launched by tests/test_gpu_ep.py through torch.distributed.run.

Every rank owns `n` tokens and E/world experts.  Forward + backward run expert-parallel; the gradients
are compared with autograd through the CPU oracle on the concatenated batch with all experts:
dx per rank slice, expert weight / theta gradients per owner rank, router weight gradient after the
all-reduce a data-parallel caller would do.
"""
import os
import pathlib
import sys

import torch
import torch.distributed as dist

ROOT = pathlib.Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def rel(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


def mean_rel(a, b):
    return float((a.double() - b.double()).abs().mean() / b.double().abs().mean().clamp_min(1e-30))


def main():
    n, hidden, inter, n_exp, k = (int(a) for a in sys.argv[1:6])
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from bibo_b200 import ep
    from oracle import moe_oracle as orc

    full = orc.make_inputs(n * world, hidden, inter, n_exp, seed=33, bias_mode="uniform", theta_std=0.5)
    dout_full = torch.randn(n * world, hidden, generator=torch.Generator().manual_seed(9))
    t = {kk: v.to(dev) for kk, v in full.items()}
    for kk in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[kk] = t[kk].to(torch.bfloat16).contiguous()
    x_local = t["x"][rank * n:(rank + 1) * n].contiguous()
    dout_local = dout_full[rank * n:(rank + 1) * n].to(torch.bfloat16).to(dev).contiguous()
    weights = dict(w_router=t["w_router"], bias=t["bias"], gate_up_proj=t["gate_up_proj"], down_proj=t["down_proj"],
                   radial_theta=t["radial_theta"])
    moe = ep.ExpertParallelMoE(weights, k, dist.group.WORLD)
    res = []
    for _ in range(2):                                  # twice: buffers and barrier epochs are reused
        out = moe.forward(x_local, training=True)
        res.append([g.clone() for g in moe.backward(dout_local)])
    torch.cuda.synchronize()
    assert moe.status() == 0, f"rank {rank}: status {moe.status()}"
    for a, b in zip(res[0], res[1]):
        assert torch.equal(a, b), "expert-parallel backward is not deterministic"
    dx, d_wr, d_gu, d_dn, d_th = res[0]
    dist.all_reduce(d_wr_f := d_wr.float())              # what a data-parallel caller does for a replicated weight

    # oracle autograd on the concatenated batch (bf16-rounded inputs, fp32 math)
    c = {kk: (v.to(torch.bfloat16).float() if kk in ("x", "w_router", "gate_up_proj", "down_proj") else v.clone())
         for kk, v in full.items()}
    for kk in ("x", "w_router", "gate_up_proj", "down_proj", "radial_theta"):
        c[kk].requires_grad_(True)
    ref_out, logits, idx, w, counts = orc.moe_forward(c["x"], c["w_router"], c["bias"], c["gate_up_proj"], c["down_proj"],
                                                      c["radial_theta"], k, return_routing=True)
    (ref_out * dout_full.to(torch.bfloat16).float()).sum().backward()
    same = (moe.topk_idx.cpu().long() == idx[rank * n:(rank + 1) * n]).all(-1)
    el = n_exp // world
    lo, hi = rank * el, (rank + 1) * el
    checks = {
        "dx": (dx.float().cpu(), c["x"].grad[rank * n:(rank + 1) * n]),
        "d_gate_up_proj": (d_gu.float().cpu(), c["gate_up_proj"].grad[lo:hi]),
        "d_down_proj": (d_dn.float().cpu(), c["down_proj"].grad[lo:hi]),
        "d_radial_theta": (d_th.cpu(), c["radial_theta"].grad[lo:hi]),
        "d_w_router": (d_wr_f.cpu(), c["w_router"].grad),
    }
    ok = bool(same.all())
    msg = [f"rank {rank}: routing identical {bool(same.all())}"]
    for name, (got, ref) in checks.items():
        r, m = rel(got, ref), mean_rel(got, ref)
        msg.append(f"{name} max-rel {r:.2e} mean-rel {m:.2e}")
        ok &= r < 2e-2 and m < 1e-2
    print("; ".join(msg), flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
