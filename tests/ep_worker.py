"""Worker of the expert-parallel tests; launched by tests/test_gpu_ep.py through torch.distributed.run.

Every rank owns `n` tokens (rank-seeded) and E/world experts of one common, seeded weight set.  The
expert-parallel forward of all ranks is compared on rank 0 with (a) the single-GPU kernel chain on
the concatenated batch and (b) the CPU oracle on the concatenated batch.
"""
import os
import pathlib
import sys

import torch
import torch.distributed as dist

ROOT = pathlib.Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def main():
    n, hidden, inter, n_exp, k = (int(a) for a in sys.argv[1:6])
    bias_mode = sys.argv[6] if len(sys.argv) > 6 else "uniform"
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from bibo_b200 import ep, functional as Fn
    from oracle import moe_oracle as orc

    full = orc.make_inputs(n * world, hidden, inter, n_exp, seed=21, bias_mode=bias_mode, theta_std=0.5, zipf_alpha=0.2)
    t = {kk: v.to(dev) for kk, v in full.items()}
    for kk in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[kk] = t[kk].to(torch.bfloat16).contiguous()
    x_local = t["x"][rank * n:(rank + 1) * n].contiguous()
    weights = dict(w_router=t["w_router"], bias=t["bias"], gate_up_proj=t["gate_up_proj"], down_proj=t["down_proj"],
                   radial_theta=t["radial_theta"])
    moe = ep.ExpertParallelMoE(weights, k, dist.group.WORLD, capacity_factor=float(os.environ.get("EP_CF", "2.0")))
    outs = []
    for _ in range(3):                      # repeated calls reuse the peer buffers and the barrier epochs
        outs.append(moe.forward(x_local).clone())
    torch.cuda.synchronize()
    status = moe.status()
    assert status == 0, f"rank {rank}: status {status}"
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), "expert-parallel forward is not deterministic"
    # host-buffer call on token slices (copies of one slice under the kernels of another): same result
    piped = ep.PipelinedExpertParallelMoE(weights, k, dist.group.WORLD, chunks=3, comm_sms=20,
                                          capacity_factor=float(os.environ.get("EP_CF", "2.0")))
    x_host, out_host = x_local.cpu().pin_memory(), torch.empty_like(x_local, device="cpu").pin_memory()
    piped.forward_host(x_host, out_host, torch.empty_like(x_local), torch.empty_like(x_local))
    assert piped.status() == 0, f"rank {rank}: sliced status {piped.status()}"
    assert torch.equal(out_host, outs[0].cpu()), "sliced host-buffer forward differs from the device forward"
    # exchange on the copy engines (block copies between ranks), single slice and three slices
    cf = float(os.environ.get("EP_CF", "2.0"))
    dma = ep.ExpertParallelMoE(weights, k, dist.group.WORLD, capacity_factor=cf, dma=True)
    for _ in range(2):
        o = dma.forward(x_local)
        torch.cuda.synchronize()
        assert dma.status() == 0, f"rank {rank}: copy-engine status {dma.status()}"
        assert torch.equal(o, outs[0]), "copy-engine exchange differs from the kernel exchange"
    dma3 = ep.PipelinedExpertParallelMoE(weights, k, dist.group.WORLD, chunks=3, capacity_factor=cf, dma=True)
    o = dma3.forward(x_local)
    torch.cuda.synchronize()
    assert dma3.status() == 0 and torch.equal(o, outs[0]), "sliced copy-engine forward differs"
    out_host.zero_()
    dma3.forward_host(x_host, out_host, torch.empty_like(x_local), torch.empty_like(x_local))
    assert torch.equal(out_host, outs[0].cpu()), "sliced copy-engine host-buffer forward differs"
    # a receive buffer that is too small: every rank sees the overflow on the device (status 4), no row is
    # exchanged, the barriers still pass, and the host layer raises instead of handing out an unwritten result
    small = ep.ExpertParallelMoE(weights, k, dist.group.WORLD, capacity_factor=0.01)   # the padding allowance alone
    sentinel = torch.full_like(x_local, 3.0)
    small.forward(x_local, out=sentinel)
    try:
        small.raise_if_failed(wait=True)
        raise AssertionError("an overflowing receive buffer went unnoticed")
    except RuntimeError as err:
        assert "device status 4" in str(err), str(err)
    assert bool((sentinel == 3.0).all()), "the combine must not write anything after an overflow"
    assert small.status() == 0, "the status word is cleared once it has been reported"
    gathered = [torch.empty_like(outs[0]) for _ in range(world)] if rank == 0 else None
    dist.gather(outs[0], gathered, dst=0)
    ok = True
    if rank == 0:
        got = torch.cat(gathered).float().cpu()
        single, ws = Fn.moe_forward(t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"],
                                    t["radial_theta"], k, "sum")
        torch.cuda.synchronize()
        single = single.float().cpu()
        # same kernels, same per-row arithmetic, same summation order: bit-identical
        same = torch.equal(got, single)
        c = {kk: (v.to(torch.bfloat16).float() if kk in ("x", "w_router", "gate_up_proj", "down_proj") else v)
             for kk, v in full.items()}
        ref, logits, idx, w, counts = orc.moe_forward(c["x"], c["w_router"], c["bias"], c["gate_up_proj"],
                                                      c["down_proj"], c["radial_theta"], k, return_routing=True)
        routed_same = (ws.topk_idx.cpu().long() == idx).all(-1)
        rel = float((got[routed_same] - ref[routed_same]).abs().max() / ref[routed_same].abs().max())
        mean_rel = float((got[routed_same] - ref[routed_same]).abs().mean() / ref[routed_same].abs().mean())
        print(f"EP world={world}: identical to single-GPU chain: {same}; vs CPU oracle max-rel {rel:.3e} "
              f"mean-rel {mean_rel:.3e} on {int(routed_same.sum())}/{n * world} tokens", flush=True)
        ok = same and rel < 2e-2 and mean_rel < 1e-2 and float(routed_same.float().mean()) > 0.99
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, src=0)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
