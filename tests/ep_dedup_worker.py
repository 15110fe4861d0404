"""Worker of the de-duplicated expert-parallel test; launched by tests/test_gpu_ep.py through torch.distributed.run.

Every rank owns a DIFFERENT number of tokens (rank-seeded) and E/world experts of one common, seeded weight
set.  The forward of all ranks (one slice, then three pipelined slices on separate streams, then the
host-buffer call) is compared on rank 0 with the single-GPU kernel chain on the concatenated batch (identical
routing, outputs apart only by the bf16 rounding of the per-rank partial sums) and with the fp32 CPU oracle
at the bf16 bars.
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

    counts = [n - 37 * r for r in range(world)]                 # ragged: rank r holds n - 37 r tokens
    offs = [sum(counts[:r]) for r in range(world + 1)]
    full = orc.make_inputs(offs[-1], hidden, inter, n_exp, seed=23, bias_mode=bias_mode, theta_std=0.5, zipf_alpha=0.2)
    t = {kk: v.to(dev) for kk, v in full.items()}
    for kk in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[kk] = t[kk].to(torch.bfloat16).contiguous()
    x_local = t["x"][offs[rank]:offs[rank + 1]].contiguous()
    weights = dict(w_router=t["w_router"], bias=t["bias"], gate_up_proj=t["gate_up_proj"], down_proj=t["down_proj"],
                   radial_theta=t["radial_theta"])
    moe = ep.DedupExpertParallelMoE(weights, k, dist.group.WORLD)
    outs = [moe.forward(x_local).clone() for _ in range(3)]     # repeated calls reuse the peer buffers and the epochs
    torch.cuda.synchronize()
    moe.raise_if_failed(wait=True)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), "forward is not deterministic"
    piped = ep.PipelinedExpertParallelMoE(weights, k, dist.group.WORLD, chunks=3, dedup=True, gemm_ctas=96, comm_ctas=16)
    o3 = piped.forward(x_local)
    torch.cuda.synchronize()
    assert piped.status() == 0, f"rank {rank}: sliced status {piped.status()}"
    assert torch.equal(o3, outs[0]), "three pipelined slices differ from one slice (tokens are independent)"
    x_host, out_host = x_local.cpu().pin_memory(), torch.empty_like(x_local, device="cpu").pin_memory()
    piped.forward_host(x_host, out_host, torch.empty_like(x_local), torch.empty_like(x_local))
    assert torch.equal(out_host, outs[0].cpu()), "sliced host-buffer forward differs from the device forward"
    # slices pipelined by resource (one stream for the NVLink work, one for the tensor-core work)
    staged = ep.PipelinedDedupMoE(weights, k, dist.group.WORLD, chunks=3, comm_sms=16)
    for _ in range(2):
        o4 = staged.forward(x_local)
        torch.cuda.synchronize()
        assert staged.status() == 0, f"rank {rank}: staged status {staged.status()}"
        assert torch.equal(o4, outs[0]), "resource-pipelined slices differ from one slice"
    out_host.zero_()
    staged.forward_host(x_host, out_host, torch.empty_like(x_local), torch.empty_like(x_local))
    assert torch.equal(out_host, outs[0].cpu()), "resource-pipelined host-buffer forward differs"

    # the same exchange on the copy engines (dense all-gather, blocks back), three slices and one
    for chunks in (3, 1):
        ag = ep.PipelinedAllGatherMoE(weights, k, dist.group.WORLD, chunks=chunks)
        for _ in range(2):
            o5 = ag.forward(x_local)
            torch.cuda.synchronize()
            assert ag.status() == 0, f"rank {rank}: copy-engine status {ag.status()}"
            assert torch.equal(o5, outs[0]), f"copy-engine exchange ({chunks} slices) differs from the kernel exchange"
        out_host.zero_()
        ag.forward_host(x_host, out_host, torch.empty_like(x_local), torch.empty_like(x_local))
        assert torch.equal(out_host, outs[0].cpu()), "copy-engine host-buffer forward differs"

    pad = torch.zeros(n, hidden, dtype=torch.bfloat16, device=dev)
    pad[:counts[rank]] = outs[0]
    gathered = [torch.empty_like(pad) for _ in range(world)] if rank == 0 else None
    dist.gather(pad, gathered, dst=0)
    idx_pad = torch.full((n, k), -1, dtype=torch.int32, device=dev)
    idx_pad[:counts[rank]] = moe.buf.topk_idx[:counts[rank]]
    idx_g = [torch.empty_like(idx_pad) for _ in range(world)] if rank == 0 else None
    dist.gather(idx_pad, idx_g, dst=0)
    ok = True
    if rank == 0:
        got = torch.cat([g[:c] for g, c in zip(gathered, counts)]).float().cpu()
        idx_all = torch.cat([g[:c] for g, c in zip(idx_g, counts)])
        single, ws = Fn.moe_forward(t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"],
                                    t["radial_theta"], k, "sum")
        torch.cuda.synchronize()
        single = single.float().cpu()
        same_routing = torch.equal(idx_all, ws.topk_idx)
        d_max = float((got - single).abs().max() / single.abs().max())
        d_mean = float((got - single).abs().mean() / single.abs().mean())
        c = {kk: (v.to(torch.bfloat16).float() if kk in ("x", "w_router", "gate_up_proj", "down_proj") else v)
             for kk, v in full.items()}
        ref, logits, idx, w, _ = orc.moe_forward(c["x"], c["w_router"], c["bias"], c["gate_up_proj"], c["down_proj"],
                                                 c["radial_theta"], k, return_routing=True)
        routed_same = (ws.topk_idx.cpu().long() == idx).all(-1)
        rel = float((got[routed_same] - ref[routed_same]).abs().max() / ref[routed_same].abs().max())
        mean_rel = float((got[routed_same] - ref[routed_same]).abs().mean() / ref[routed_same].abs().mean())
        print(f"dedup EP world={world}: routing identical to single GPU: {same_routing}; vs single-GPU chain max-rel "
              f"{d_max:.3e} mean-rel {d_mean:.3e}; vs CPU oracle max-rel {rel:.3e} mean-rel {mean_rel:.3e} on "
              f"{int(routed_same.sum())}/{offs[-1]} tokens", flush=True)
        ok = (same_routing and d_max < 1.2e-2 and d_mean < 4e-3 and rel < 2e-2 and mean_rel < 1e-2
              and float(routed_same.float().mean()) > 0.99)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, src=0)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
