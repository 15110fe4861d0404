#!/usr/bin/env python
"""Benchmark of the BiBo sparse-MoE feed-forward block (forward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c2|c3|c3a] [--impl reference]

One "step" is one forward pass of the MoE layer over one batch of synthetic tokens.  Prints ONE JSON
line (rank 0).  `value` is tokens/s of the whole job with the batch already resident in HBM, from ONE
timed region of --steps steps; `repeats` gives median / min / max of further regions and `sustained`
seconds of back-to-back steps with the clocks seen; `e2e` is the same metric through the host-buffer
call (pinned host input copied to the device and the result copied back inside the timed region);
`roofline` describes the dominant kernel, timed with CUDA events recorded around each kernel of the
chain inside the timed steps (at N > 1: the NVLink phase against the measured peer-copy rate);
`cpu_baseline` is the reference's own eager layer (from oracle/_ref when it has been built, else the
CPU oracle, a restatement of its per-expert loop) timed on this machine's host cores on a bounded
sample of the same workload; `gpu_eager_reference` is that layer in bf16 on this GPU; at N > 1
`ep_check` compares sampled tokens of every rank with the single-GPU chain and the CPU oracle and the
run exits non-zero outside the bf16 bars.

Workloads (synthetic, seeded; shapes and distributions of the benchmark configurations):
  c4  32768 tokens per GPU, hidden 2048, 64 experts, top-6, intermediate 512, bias 0   (default)
  c2  16384 tokens, hidden 1024, intermediate 256, bias ~ U(-0.01, 0.01)
  c3  65536 tokens, hidden 2048, intermediate 512, bias = log Zipf(1.1) profile (literal)
  c3a same with the bias scaled by 0.07 (per-expert counts span about 20x)
  c5layer  one MoE layer of benchmark configuration 5 (32768 tokens, hidden 1024, intermediate 256)
  c5  the reference's 10-layer model (from oracle/_ref), prefill of 8 x 4096 tokens, with and without its
      feed-forward blocks swapped for the kernels (one GPU; a line of its own)
"""
import argparse
import json
import os
import pathlib
import sys
import threading
import time

import torch

ROOT = pathlib.Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

WORKLOADS = {
    "c4": dict(n_tokens=32768, hidden=2048, inter=512, bias="zero", zipf_alpha=0.0),
    "c2": dict(n_tokens=16384, hidden=1024, inter=256, bias="uniform", zipf_alpha=0.0),
    "c3": dict(n_tokens=65536, hidden=2048, inter=512, bias="zipf", zipf_alpha=1.0),
    "c3a": dict(n_tokens=65536, hidden=2048, inter=512, bias="zipf", zipf_alpha=0.07),
    # one MoE layer of benchmark configuration 5 (batch 8 x 4096 tokens, hidden 1024, intermediate 256)
    "c5layer": dict(n_tokens=32768, hidden=1024, inter=256, bias="uniform", zipf_alpha=0.0),
    # benchmark configuration 5 itself: the reference's 10-layer model with its feed-forward blocks swapped (run_c5)
    "c5": dict(n_tokens=32768, hidden=1024, inter=256, bias="uniform", zipf_alpha=0.0, model=True),
}
N_EXPERTS, TOP_K = 64, 6
METRIC, UNIT = "moe_layer_fwd_tokens_per_s", "tokens/s"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=float(d["hbm_gbs"]), tf=float(d["bf16_tflops"]), tf_sus=float(d.get("bf16_tflops_sustained", 0)),
                    src="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sus=1400.0, src="fallback")


def synth(wl, device, seed, rank=0, dtype=torch.bfloat16):
    """Seeded synthetic tensors generated on `device`: x ~ N(0,1) (rank-seeded); weights ~ N(0,0.02) and
    theta ~ N(0,0.5) from a seed common to all ranks."""
    g = torch.Generator(device=device).manual_seed(seed)
    gx = torch.Generator(device=device).manual_seed(seed + 7919 * (rank + 1))
    n, h, i = wl["n_tokens"], wl["hidden"], wl["inter"]
    rn = lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32)
    t = dict(x=torch.randn(n, h, generator=gx, device=device, dtype=torch.float32).to(dtype),
             gate_up_proj=(rn(N_EXPERTS, 2 * i, h) * 0.02).to(dtype),
             down_proj=(rn(N_EXPERTS, h, i) * 0.02).to(dtype), w_router=(rn(N_EXPERTS, h) * 0.02).to(dtype),
             radial_theta=rn(N_EXPERTS) * 0.5)
    if wl["bias"] == "zero":
        t["bias"] = torch.zeros(N_EXPERTS, device=device)
    elif wl["bias"] == "uniform":
        t["bias"] = (torch.rand(N_EXPERTS, generator=g, device=device) * 2 - 1) * 0.01
    else:
        prof = 1.0 / torch.arange(1, N_EXPERTS + 1, dtype=torch.float64) ** 1.1
        t["bias"] = (wl["zipf_alpha"] * torch.log(prof / prof.sum())).float().to(device)
    return t


def bind_to_gpu_cpus(index):
    """Pin this process to the CPUs NVML reports as local to GPU `index` (read-only query), so that the
    pinned host buffers of the end-to-end path are allocated on the GPU's own NUMA node.  Several ranks
    copying over PCIe at once otherwise all pull from one socket's memory.  Returns the CPU count or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {w * 64 + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""
    BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._stop_evt = index, [], set(), None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        while self.nv and not self._stop_evt.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                r = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.reasons |= {n for b, n in self.BITS.items() if r & b}
            except Exception:
                pass
            time.sleep(0.004)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def reference_layer(wl, tensors, device, dtype):
    """The UNMODIFIED reference BiBoMoELayer (from oracle/_ref, built by oracle/make_ref.py) carrying the
    benchmark's weights, or None where oracle/_ref is absent.  Checker / baseline only."""
    from oracle import make_ref
    if not make_ref.available():
        return None
    make_ref.activate()
    from src.configuration_bibo import BiBoConfig
    from src.modeling.ffn.moe import BiBoMoELayer
    cfg = BiBoConfig(hidden_size=wl["hidden"], num_attention_heads=wl["hidden"] // 256, num_key_value_heads=2,
                     moe_intermediate_size=wl["inter"], num_routed_experts=N_EXPERTS, num_experts_per_tok=TOP_K,
                     special_expert_pairs=0)
    layer = BiBoMoELayer(cfg).to(dtype).to(device).eval()
    with torch.no_grad():
        layer.gate.gate_proj.weight.copy_(tensors["w_router"])
        layer.gate.bias.copy_(tensors["bias"])
        layer.experts.gate_up_proj.copy_(tensors["gate_up_proj"])
        layer.experts.down_proj.copy_(tensors["down_proj"])
        layer.experts.radial_theta.copy_(tensors["radial_theta"])
    return layer


def gpu_eager_reference(wl, t, dev, steps=5):
    """tokens/s of the reference's own eager BiBoMoELayer.forward (per-expert Python loop, one host sync per
    forward) in bf16 on this GPU, same tokens and weights: the only GPU implementation the reference ships."""
    layer = reference_layer(wl, t, dev, torch.bfloat16)
    if layer is None:
        return None
    x = t["x"][None]
    with torch.no_grad():
        for _ in range(2):
            ref_out = layer(x)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            layer(x)
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"value": wl["n_tokens"] / (ms * 1e-3), "unit": UNIT, "ms_per_step": round(ms, 3), "steps": steps,
            "kind": "the reference's BiBoMoELayer.forward, eager PyTorch, bf16, same GPU, same tokens and weights"}, ref_out[0]


def cpu_oracle_rate(wl, seconds_cap=20.0, sample_tokens=2048, threads=None):
    """tokens/s of the CPU oracle (fp32, all host threads) on a bounded sample of the workload."""
    from oracle import moe_oracle as orc
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    bias_mode = {"zero": "zero", "uniform": "uniform", "zipf": "zipf"}[wl["bias"]]
    inp = orc.make_inputs(sample_tokens, wl["hidden"], wl["inter"], N_EXPERTS, seed=0, bias_mode=bias_mode,
                          theta_std=0.5, zipf_alpha=wl["zipf_alpha"] or 1.0)
    run = lambda: orc.moe_forward(inp["x"], inp["w_router"], inp["bias"], inp["gate_up_proj"], inp["down_proj"],
                                  inp["radial_theta"], TOP_K)
    kind, what = "port", "CPU oracle = restatement of the reference's eager per-expert loop"
    layer = reference_layer(wl, inp, "cpu", torch.float32)
    if layer is not None:
        x3 = inp["x"][None]
        run = lambda: layer(x3)
        kind, what = "reference", "the reference's own BiBoMoELayer.forward (unmodified, from oracle/_ref)"
    with torch.no_grad():
        run()
        t0, reps = time.perf_counter(), 0
        while True:
            run()
            reps += 1
            dt = time.perf_counter() - t0
            if dt > seconds_cap or (reps >= 3 and dt > 10.0):
                break
    return dict(value=sample_tokens * reps / dt, unit=UNIT, cores=torch.get_num_threads(), kind=kind,
                sample=f"{reps} passes of {sample_tokens} tokens (same hidden/intermediate/experts/top-k, fp32) "
                       f"in {dt:.1f} s; {what}")


def run_reference(args, wl, rank, world):
    """The reference arm: the reference's CPU algorithm (oracle port) on host cores, rank 0 only."""
    if rank != 0:
        return
    from oracle import moe_oracle as orc
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    sample = 2048
    inp = orc.make_inputs(sample, wl["hidden"], wl["inter"], N_EXPERTS, seed=0, bias_mode=wl["bias"], theta_std=0.5,
                          zipf_alpha=wl["zipf_alpha"] or 1.0)
    run = lambda: orc.moe_forward(inp["x"], inp["w_router"], inp["bias"], inp["gate_up_proj"], inp["down_proj"],
                                  inp["radial_theta"], TOP_K)
    kind = "port"
    desc = (f"each step = one fp32 forward of {sample} tokens of the workload through the CPU oracle "
            f"(restatement of the reference's eager per-expert loop; oracle/_ref is not present on this machine)")
    layer = reference_layer(wl, inp, "cpu", torch.float32)
    if layer is not None:
        kind = "reference"
        x3 = inp["x"][None]
        run = lambda: layer(x3)
        desc = (f"each step = one fp32 forward of {sample} tokens of the workload through the reference's own "
                f"BiBoMoELayer.forward (unmodified, byte-compiled into oracle/_ref) on the host cores")
    with torch.no_grad():
        for _ in range(args.warmup):
            run()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            run()
        dt = time.perf_counter() - t0
    val = sample * args.steps / dt
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, wl, world),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind, "sample": desc},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def workload_config(args, wl, world):
    return {"workload": f"{args.workload}: MoE layer forward, {wl['n_tokens']} tokens per GPU, hidden {wl['hidden']}, "
                        f"{N_EXPERTS} experts, top-{TOP_K}, intermediate {wl['inter']}, router bias {wl['bias']}"
                        + (f" (alpha {wl['zipf_alpha']})" if wl["bias"] == "zipf" else ""),
            "tokens_per_gpu": wl["n_tokens"], "global_tokens": wl["n_tokens"] * world,
            "parallelism": "single GPU" if world == 1 else
            f"expert-parallel ep{world} (tokens data-parallel), exchange by {args.ep_exchange}, {args.ep_chunks} token slice(s)",
            "l2": "per-step working set (activations + expert weights + intermediates) exceeds the 126 MB L2"}


BF16_MAX_REL, BF16_MEAN_REL = 2e-2, 1e-2      # the bf16 parity bars against the fp32 oracle
PEER_COPY_GBS = 770.0                         # peer copy per direction measured on this pool's B200s (nominal 900)


def _lane_topk_idx(lane):
    return lane.buf.topk_idx if hasattr(lane, "buf") else lane.topk_idx


def run_ep_check(args, wl, t, runner, rank, world, dev, fwdbwd_step):
    """After the timed region: one more expert-parallel step, then the first 256 tokens of every rank are
    gathered on rank 0 and compared with (i) the single-GPU kernel chain on those tokens with the full expert
    set and (ii) the fp32 CPU oracle on them (tokens are independent, so a sample checks the same rows).
    Forward + backward mode compares the sampled rows of dx with the single-GPU backward."""
    import torch.distributed as dist
    from bibo_b200 import functional as Fn
    sample = min(256, wl["n_tokens"])
    h, i = wl["hidden"], wl["inter"]
    if fwdbwd_step is None:
        out = runner.forward(t["x"])
        dx = None
    else:
        lane = runner.lanes[0]
        out = lane.forward(t["x"], training=True)
        dout = torch.randn(t["x"].shape, generator=torch.Generator(device=dev).manual_seed(77 + rank), device=dev,
                           dtype=torch.float32).to(torch.bfloat16)
        dx = lane.backward(dout)[0]
    torch.cuda.synchronize()
    status = runner.status()
    pieces = [t["x"][:sample], out[:sample]] + ([dout[:sample], dx[:sample]] if dx is not None else [])
    mine = torch.cat([p_.contiguous().reshape(sample, -1) for p_ in pieces], dim=1).contiguous()
    idx_mine = _lane_topk_idx(runner.lanes[0])[:sample].contiguous()
    gathered = torch.empty(world * sample, mine.shape[1], dtype=torch.bfloat16, device=dev)
    idx_all = torch.empty(world * sample, TOP_K, dtype=torch.int32, device=dev)
    st_all = torch.empty(world, dtype=torch.int32, device=dev)
    dist.all_gather_into_tensor(gathered, mine)
    dist.all_gather_into_tensor(idx_all, idx_mine)
    dist.all_gather_into_tensor(st_all, torch.tensor([status], dtype=torch.int32, device=dev))
    if rank != 0:
        return None
    cols = gathered.split(h, dim=1)
    xs, outs = cols[0].contiguous(), cols[1].contiguous()
    geo = Fn.Geometry(xs.shape[0], h, i, N_EXPERTS, N_EXPERTS, 0, TOP_K, torch.bfloat16)
    ws1 = Fn.MoEWorkspace(geo, dev, keep_logits=True, keep_gate_up=True)
    ref1, _ = Fn.moe_forward(xs, t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], TOP_K,
                             "sum", ws=ws1, zero_padding=dx is not None)
    rel = lambda a, b: float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))
    mrel = lambda a, b: float((a.double() - b.double()).abs().mean() / b.double().abs().mean().clamp_min(1e-30))
    res = {"sample_tokens_per_rank": sample, "status": int(st_all.max()),
           "routing_identical": bool(torch.equal(idx_all, ws1.topk_idx)),
           "vs_single_gpu_max_rel": rel(outs.float(), ref1.float()),
           "vs_single_gpu_bit_identical": bool(torch.equal(outs.view(torch.int16), ref1.view(torch.int16)))}
    from oracle import moe_oracle as orc
    f32 = lambda k_: t[k_].float().cpu()
    ref, _, idx_o, _, _ = orc.moe_forward(xs.float().cpu(), f32("w_router"), f32("bias"), f32("gate_up_proj"),
                                          f32("down_proj"), f32("radial_theta"), TOP_K, return_routing=True)
    same = (idx_all.cpu().long() == idx_o).all(-1)
    res.update(oracle_same_routing_frac=float(same.float().mean()),
               vs_oracle_max_rel=rel(outs.float().cpu()[same], ref[same]),
               vs_oracle_mean_rel=mrel(outs.float().cpu()[same], ref[same]))
    ok = (res["status"] == 0 and res["routing_identical"] and res["vs_oracle_max_rel"] < BF16_MAX_REL
          and res["vs_oracle_mean_rel"] < BF16_MEAN_REL and res["oracle_same_routing_frac"] > 0.97)
    if dx is not None:
        douts, dxs = cols[2].contiguous(), cols[3].contiguous()
        dx1 = Fn.moe_backward(douts, xs, t["w_router"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], ws1, "sum")[0]
        res["dx_vs_single_gpu_max_rel"] = rel(dxs.float(), dx1.float())
        res["dx_vs_single_gpu_mean_rel"] = mrel(dxs.float(), dx1.float())
        ok = ok and res["dx_vs_single_gpu_max_rel"] < BF16_MAX_REL and res["dx_vs_single_gpu_mean_rel"] < BF16_MEAN_REL
    res["ok"] = bool(ok)
    res["bars"] = {"max_rel": BF16_MAX_REL, "mean_rel": BF16_MEAN_REL}
    return res


def nvlink_roofline(args, wl, t, runner, world, rank, ep_phases):
    """N > 1: the NVLink phase of the profiled step against the measured peer-copy rate.  Bytes = rows this
    rank sends to OTHER ranks in the dispatch phase (counted from its routing) x row size; the return phase
    moves the same number of rows the other way."""
    el = N_EXPERTS // world
    rows = 0
    dedup = args.ep_exchange in ("dedup", "allgather")
    for lane in runner.lanes:
        if args.ep_exchange == "allgather":       # every row to every peer
            rows += lane._n_cap * (world - 1)
            continue
        n_lane = lane._n_cap if dedup else lane._n
        idx = _lane_topk_idx(lane)[:n_lane].long()
        owner = idx // el
        remote = owner != rank
        if dedup:     # distinct remote owners per token
            onehot = torch.zeros(idx.shape[0], world, dtype=torch.bool, device=idx.device)
            onehot.scatter_(1, owner, True)
            onehot[:, rank] = False
            rows += int(onehot.sum())
        else:
            rows += int(remote.sum())
    nbytes = rows * wl["hidden"] * 2
    if rank != 0:
        return None
    # time during which any slice was in its dispatch phase / its return phase
    names = ("dispatch", "partial") if dedup else ("dispatch", "combine")
    starts = {"dispatch": "route" if dedup else "gather_plan", "partial": "experts", "combine": "barrier2"}
    if args.ep_exchange == "allgather":          # rows leave at "start"; all of a slice's rows and records are in at "received"
        names, starts = ("received", "returned"), {"received": "start", "returned": "experts"}
    out = {}
    for nm in names:
        t0 = min(ph[starts[nm]] for ph in ep_phases if starts[nm] in ph)
        t1 = max(ph[nm] for ph in ep_phases if nm in ph)
        out[nm] = max(t1 - t0, 1e-6)
    top = max(out, key=out.get)
    ach = nbytes / (out[top] * 1e-3) / 1e9
    return {"kernel": "ep_" + top, "bound": "nvlink", "achieved": round(ach, 1), "peak": PEER_COPY_GBS, "unit": "GB/s",
            "frac": round(ach / PEER_COPY_GBS, 4), "traffic": None, "bytes_per_direction_per_rank": nbytes,
            "phase_ms": {k_: round(v, 4) for k_, v in out.items()},
            "peak_source": "peer copy per direction measured on this pool (nominal 900 GB/s); the phase interval "
                           "spans all token slices, whose phases overlap other slices' GEMMs"}


def run_c5(args, rank=0, world=1, local=0):
    """Benchmark configuration 5: the reference's own 10-layer BiBoModel (from oracle/_ref), bf16, a prefill of
    8 x 4096 token ids on one GPU (on N GPUs: data-parallel replicas, one sequence of 4096 ids per GPU, every
    replica with all 64 experts; times are the maximum over the ranks), first unmodified (eager PyTorch
    everywhere), then with ONLY the feed-forward blocks swapped for the kernels (bibo_b200.install() +
    install(seam="mlp")).  Prints one JSON line: prefill
    tokens/s with the kernels, the unmodified model's figure, the share of the prefill spent inside the
    feed-forward blocks in both runs (CUDA events around every .mlp module), and how far the two last hidden
    states are apart."""
    from oracle import make_ref
    batch = 8 if world == 1 else 1
    line = {"metric": "c5_prefill_tokens_per_s", "unit": UNIT, "n_gpus": world, "higher_is_better": True, "dtype": "bf16",
            "scaling": "weak" if world == 1 else "replicas only (one sequence per GPU, no exchange)",
            "data": "synthetic", "config": {"workload": f"c5: 10-layer BiBo prefill, batch {batch} x sequence 4096 per GPU, "
                                            "hidden 1024, layers 0/9 dense MLP (4096), layers 1-8 MoE (64 experts, top-6, 256)"}}
    if not make_ref.available():
        line["unavailable"] = "oracle/_ref is absent on this machine (python oracle/make_ref.py needs a checkout of the reference)"
        if rank == 0:
            print(json.dumps(line))
        return
    make_ref.activate()
    import bibo_b200
    from src.configuration_bibo import BiBoConfig
    from src.modeling.models import BiBoModel
    dev = torch.device("cuda", local)
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    cfg = BiBoConfig(vocab_size=32000, hidden_size=1024, intermediate_size=4096, num_hidden_layers=10,
                     num_attention_heads=4, num_key_value_heads=2, moe_intermediate_size=256, num_routed_experts=N_EXPERTS,
                     num_experts_per_tok=TOP_K, special_expert_pairs=0, hybrid_layer_pattern=[0, 1, 1, 0, 1, 1, 0, 1, 1, 0],
                     sliding_window=128, tie_word_embeddings=True, mlp_only_layers=[0, 9], use_cache=False)
    torch.manual_seed(0)
    model = BiBoModel(cfg).to(torch.bfloat16).to(dev).eval()
    seq = 4096
    ids = torch.randint(0, 32000, (batch, seq), generator=torch.Generator().manual_seed(1 + rank)).to(dev)

    def over_ranks(ms):
        if world == 1:
            return ms
        v = torch.tensor([ms], device=dev)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v)

    def timed(steps):
        spans = []
        hooks = []
        for layer in model.layers:
            def pre(m, a, spans=spans):
                e = torch.cuda.Event(enable_timing=True); e.record(); spans.append([e, None])
            def post(m, a, o, spans=spans):
                e = torch.cuda.Event(enable_timing=True); e.record(); spans[-1][1] = e
            hooks += [layer.mlp.register_forward_pre_hook(pre), layer.mlp.register_forward_hook(post)]
        with torch.no_grad():
            out = model(input_ids=ids, use_cache=False).last_hidden_state      # warm-up (and the compared output)
            spans.clear()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0.record()
            for _ in range(steps):
                model(input_ids=ids, use_cache=False)
            e1.record()
            torch.cuda.synchronize()
        for h in hooks:
            h.remove()
        total = over_ranks(e0.elapsed_time(e1) / steps)
        ffn = over_ranks(sum(a.elapsed_time(b) for a, b in spans) / steps)
        return total, ffn, out

    steps = max(1, min(args.steps, 5))
    ref_ms, ref_ffn, ref_out = timed(steps)
    launches0 = 0
    from bibo_b200 import functional as Fn
    bibo_b200.install()
    bibo_b200.install(seam="mlp")
    try:
        launches0 = Fn.launch_count()
        ms, ffn, out = timed(steps)
        launches = (Fn.launch_count() - launches0) // (steps + 1)
    finally:
        bibo_b200.uninstall()
    g, r = out.reshape(-1, 1024).float(), ref_out.reshape(-1, 1024).float()
    per_tok = (g - r).norm(dim=-1) / r.norm(dim=-1).clamp_min(1e-30)
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    line.update({
        "value": world * batch * seq / (ms * 1e-3), "steps": steps, "warmup": 1, "ms_per_step": round(ms, 3),
        "feed_forward_ms": round(ffn, 3), "feed_forward_share": round(ffn / ms, 4),
        "unmodified_reference": {"ms_per_step": round(ref_ms, 3), "feed_forward_ms": round(ref_ffn, 3),
                                 "feed_forward_share": round(ref_ffn / ref_ms, 4),
                                 "value": world * batch * seq / (ref_ms * 1e-3)},
        "prefill_speedup": round(ref_ms / ms, 3), "feed_forward_speedup": round(ref_ffn / ffn, 2),
        "gpu_launches": int(launches),
        "last_hidden_state_vs_unmodified": {"median_token_rel": float(per_tok.median()),
                                            "tokens_above_1e-1": int((per_tok > 1e-1).sum()), "tokens": int(per_tok.numel())},
        "note": "attention, norms and embedding stay the reference's eager PyTorch in both runs; eval mode"})
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gpu-reference", action="store_true",
                    help="skip timing the reference's eager layer on this GPU (needs oracle/_ref)")
    ap.add_argument("--ep-chunks", type=int, default=None,
                    help="token slices pipelined on separate streams (N>1; default 1)")
    ap.add_argument("--ep-exchange", default="auto", choices=["auto", "allgather", "dedup", "copy", "kernel"],
                    help="N>1: dedup = one row per (token, destination rank) each way through exchange kernels (auto at "
                         "2 and 4 GPUs; at 8 the per-slot kernels are as fast and auto picks them); "
                         "allgather = every rank's rows to every peer and partial rows back on the copy engines, token "
                         "slices pipelined; kernel = one row per slot through the dispatch/combine kernels (training "
                         "path); copy = per-slot rows by peer copies")
    ap.add_argument("--ep-lockstep", action="store_true",
                    help="N>1, dedup: one stream per token slice (all slices in the same phase at once) instead of "
                         "one stream per resource (NVLink work / tensor-core work)")
    ap.add_argument("--gemm-ctas", type=int, default=None, help="N>1: cap of the grouped-GEMM grids (0 = none)")
    ap.add_argument("--comm-ctas", type=int, default=None, help="N>1: cap of the exchange kernels' grids (0 = none)")
    ap.add_argument("--repeats", type=int, default=9, help="extra timed regions of --steps steps (median / min / max)")
    ap.add_argument("--sustained-s", type=float, default=2.0, help="seconds of back-to-back steps for the sustained figure (0 = skip)")
    ap.add_argument("--no-ep-check", action="store_true", help="N>1: skip the parity check of sampled tokens")
    ap.add_argument("--copy-streams", type=int, default=0, help="copy exchange: 1 = one stream per peer, 0 = one stream")
    ap.add_argument("--no-numa-bind", action="store_true",
                    help="N>1: do not pin each rank to the CPUs local to its GPU (pinned host buffers then land anywhere)")
    ap.add_argument("--e2e-chunks", type=int, default=4, help="token slices of the host-buffer (e2e) forward (N>1)")
    ap.add_argument("--comm-sms", type=int, default=16, help="SMs set aside for the exchange kernels (N>1, several slices)")
    ap.add_argument("--gather-in-gemm", action="store_true",
                    help="1 GPU: the gate/up kernel gathers its own rows instead of a separate permute kernel (A/B)")
    ap.add_argument("--mode", default="fwd", choices=["fwd", "fwdbwd", "ffn", "ffn_separate"],
                    help="fwd = the headline metric; fwdbwd = forward + backward of the block (1 GPU); ffn = the decoder "
                         "layer's feed-forward half (RMSNorm + block + residual) with the norm folded into the router's and "
                         "the permute's loads; ffn_separate = the same with the norm as a kernel of its own (1 GPU)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.ep_exchange == "auto":      # measured: dedup 1.74 / 2.42 / 3.20 ms, kernel 2.24 / 2.84 / 3.15 ms at 2 / 4 / 8 GPUs
        args.ep_exchange = "dedup" if world <= 4 else "kernel"
    if args.mode == "fwdbwd" and args.ep_exchange in ("dedup", "allgather"):
        args.ep_exchange = "kernel"            # the de-duplicated exchanges are forward-only
    if args.ep_chunks is None:
        args.ep_chunks = 1          # every pipelined form measured slower than one slice at 2 GPUs, equal at 4
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return run_reference(args, wl, rank, world)
    if wl.get("model"):
        return run_c5(args, rank, world, local)
    if args.warmup < 3:
        args.warmup = 3

    import torch.distributed as dist
    from bibo_b200 import functional as Fn
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        if not args.no_numa_bind:
            bind_to_gpu_cpus(local)
    t = synth(wl, dev, seed=1234, rank=rank)
    n, h, i = wl["n_tokens"], wl["hidden"], wl["inter"]
    dtype = torch.bfloat16

    if world > 1:
        from bibo_b200 import ep
        dma = args.ep_exchange == "copy" and args.mode == "fwd"
        dedup = args.ep_exchange == "dedup"
        ep_kw = dict(comm_sms=args.comm_sms, dedup=dedup, gemm_ctas=args.gemm_ctas, comm_ctas=args.comm_ctas)
        if not dedup:
            ep_kw.update(dma=dma, copy_streams=bool(args.copy_streams))
        make_runner = lambda chunks: (
            ep.PipelinedAllGatherMoE(t, TOP_K, dist.group.WORLD, n_tokens=wl["n_tokens"], chunks=chunks)
            if args.ep_exchange == "allgather" else
            ep.PipelinedDedupMoE(t, TOP_K, dist.group.WORLD, n_tokens=wl["n_tokens"], chunks=chunks,
                                 comm_sms=args.comm_sms, gemm_ctas=args.gemm_ctas, comm_ctas=args.comm_ctas)
            if dedup and not args.ep_lockstep else
            ep.PipelinedExpertParallelMoE(t, TOP_K, dist.group.WORLD, n_tokens=wl["n_tokens"], chunks=chunks,
                                          **dict(ep_kw, **(dict(gemm_ctas=args.gemm_ctas or 0, comm_ctas=args.comm_ctas or 0)
                                                           if dedup else {}))))
        runner = make_runner(args.ep_chunks)
        step = lambda: runner.forward(t["x"])
        ws = None
        if args.mode == "fwdbwd":
            lane = runner.lanes[0]
            dout = torch.randn_like(t["x"])

            def step():
                lane.forward(t["x"], training=True)
                return lane.backward(dout)
    else:
        geo = Fn.Geometry(n, h, i, N_EXPERTS, N_EXPERTS, 0, TOP_K, dtype)
        ws = Fn.MoEWorkspace(geo, dev, keep_gate_up=False)
        out = torch.empty_like(t["x"])
        step = lambda: Fn.moe_forward(t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"],
                                      t["radial_theta"], TOP_K, "sum", ws=ws, out=out,
                                      gather_in_gemm=args.gather_in_gemm)
        if args.mode in ("ffn", "ffn_separate"):
            norm_w = (1.0 + 0.1 * torch.randn(h, generator=torch.Generator().manual_seed(99))).to(dtype).to(dev)
            if args.mode == "ffn":
                step = lambda: Fn.ffn_forward(t["x"], norm_w, 1e-6, t["w_router"], t["bias"], t["gate_up_proj"],
                                              t["down_proj"], t["radial_theta"], TOP_K, "sum", ws=ws, out=out)
            else:
                def step():
                    xn = Fn.rmsnorm_forward(t["x"], norm_w, 1e-6)
                    return Fn.moe_forward(xn, t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"],
                                          t["radial_theta"], TOP_K, "sum", ws=ws, out=out, addend=t["x"])
        if args.mode == "fwdbwd":
            ws = None                       # no per-kernel events: the backward consumes its workspace
            dout = torch.randn_like(t["x"])
            ws_b = Fn.MoEWorkspace(geo, dev, keep_logits=True, keep_gate_up=True)

            def step():
                o, w = Fn.moe_forward(t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"],
                                      t["radial_theta"], TOP_K, "sum", ws=ws_b, out=out, zero_padding=True)
                return Fn.moe_backward(dout, t["x"], t["w_router"], t["gate_up_proj"], t["down_proj"],
                                       t["radial_theta"], w, "sum")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    # ---- timed region: K steps, events on the launching stream, per-kernel events inside ------------
    stage_sets = []
    if ws is not None:   # events are created (first record) before the timed region
        stage_sets = [[torch.cuda.Event(enable_timing=True) for _ in range(7)] for _ in range(args.steps)]
        for evs in stage_sets:
            for e in evs:
                e.record()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = Fn.launch_count()
    barrier()
    e0.record()
    for k in range(args.steps):
        if ws is not None:
            ws.stage_events = stage_sets[k]
        step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    launches = Fn.launch_count() - launches0
    ms_total = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms_total, op=dist.ReduceOp.MAX)
    ms_step = float(ms_total) / args.steps
    value = n * world / (ms_step * 1e-3)

    # ---- the same region repeated: spread of the per-step time, then seconds of back-to-back steps -------
    if ws is not None:
        ws.stage_events = None

    def timed_region(k_steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for _ in range(k_steps):
            step()
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / k_steps

    rep = sorted(timed_region(args.steps) for _ in range(max(0, args.repeats)))
    repeats = ({"regions": len(rep), "steps_each": args.steps, "ms_median": round(rep[len(rep) // 2], 4),
                "ms_min": round(rep[0], 4), "ms_max": round(rep[-1], 4)} if rep else None)
    sustained = None
    if args.sustained_s > 0:
        k_sus = max(args.steps, int(args.sustained_s * 1e3 / ms_step))
        sus_sampler = ClockSampler(local)
        sus_sampler.start()
        ms_sus = timed_region(k_sus)
        sus_clocks = sus_sampler.stop()
        sustained = {"steps": k_sus, "seconds": round(ms_sus * k_sus * 1e-3, 2), "ms_per_step": round(ms_sus, 4),
                     "clocks": sus_clocks}

    # ---- end-to-end: host buffers through the C-ABI host entry (N=1) / the public forward (N>1) ------
    x_host = t["x"].cpu().pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    x_dev, out_dev = torch.empty_like(t["x"]), torch.empty_like(t["x"])
    if world > 1:
        # token slices on separate streams: the copies of one slice run under the kernels of another
        if dedup:     # host buffers: one stream per slice (copy-in, forward, copy-out), every kernel with the whole GPU
            e2e_runner = ep.PipelinedExpertParallelMoE(t, TOP_K, dist.group.WORLD, n_tokens=wl["n_tokens"],
                                                       chunks=args.e2e_chunks, dedup=True, gemm_ctas=0, comm_ctas=0)
        else:
            e2e_runner = runner if args.e2e_chunks == args.ep_chunks else make_runner(args.e2e_chunks)
        e2e_step = lambda: e2e_runner.forward_host(x_host, out_host, x_dev, out_dev)
    else:
        if ws is not None:
            ws.stage_events = None
        e2e_step = lambda: Fn.moe_forward_host(x_host, out_host, x_dev, out_dev, t["w_router"], t["bias"],
                                               t["gate_up_proj"], t["down_proj"], t["radial_theta"], TOP_K, "sum", ws=ws)
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=dev)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_val = n * world * args.steps / float(e2e_s)

    ep_phases = None
    if world > 1 and args.mode == "fwd":      # one extra profiled step: when each phase of each token slice ended (ms from step start)
        for lane in runner.lanes:
            lane.profile = True
        barrier()
        step()
        step()                                # the marks of the second of two back-to-back steps survive
        barrier()
        t_start = min((lane.marks[0][1] for lane in runner.lanes), key=lambda ev: runner.lanes[0].marks[0][1].elapsed_time(ev))
        ep_phases = [{n: round(t_start.elapsed_time(ev), 3) for n, ev in lane.marks} for lane in runner.lanes]
        for lane in runner.lanes:
            lane.profile = False
    ep_check = None
    if world > 1 and not args.no_ep_check:
        ep_check = run_ep_check(args, wl, t, runner, rank, world, dev, step if args.mode == "fwdbwd" else None)
    nvlink = None
    if world > 1 and ep_phases:
        nvlink = nvlink_roofline(args, wl, t, runner, world, rank, ep_phases)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    pk = peaks()
    S = n * TOP_K
    stages, roof = {}, None
    if stage_sets:
        names = Fn.MoEWorkspace.STAGES
        ms = {nm: sum(ev[k].elapsed_time(ev[k + 1]) for ev in stage_sets) / len(stage_sets) for k, nm in enumerate(names)}
        eb = 2  # bf16 bytes
        alg = {  # algorithmic work per launch: (flops, bytes)
            "router": (2.0 * n * h * N_EXPERTS, n * (eb * h + 8 * TOP_K) + eb * N_EXPERTS * h),
            "plan": (0.0, 0.0),
            "permute": (0.0, n * (eb * h + eb * TOP_K * h + 8 * TOP_K)),
            "gemm1_radial": (4.0 * S * h * i, eb * (S * h + S * i + 2 * N_EXPERTS * h * i)),
            "gemm2": (2.0 * S * h * i, eb * (S * i + S * h + N_EXPERTS * h * i)),
            "combine": (0.0, n * (eb * TOP_K * h + eb * h + 8 * TOP_K)),
        }
        for nm in names:
            fl, by = alg[nm]
            tensor = nm.startswith("gemm")
            ach = (fl / (ms[nm] * 1e-3) / 1e12) if tensor else (by / (ms[nm] * 1e-3) / 1e9)
            peak = pk["tf"] if tensor else pk["hbm"]
            stages[nm] = {"ms": round(ms[nm], 4), "bound": "tensor" if tensor else "hbm", "achieved": round(ach, 2),
                          "unit": "TFLOP/s" if tensor else "GB/s", "frac": round(ach / peak, 4) if nm != "plan" else None}
        top = max(names, key=lambda nm: ms[nm])
        # DRAM bytes per launch of the c4 workload from ncu (dram__bytes_read.sum + dram__bytes_write.sum),
        # profiles/c4_forward_gemm1_global_exchange.md; other workloads were not captured
        ncu_traffic = {"gemm1_radial": 1.307e9, "gemm2": 1.110e9} if args.workload == "c4" else {}
        roof = {"kernel": top, "bound": stages[top]["bound"], "achieved": stages[top]["achieved"],
                "peak": pk["tf"] if stages[top]["bound"] == "tensor" else pk["hbm"], "unit": stages[top]["unit"],
                "frac": stages[top]["frac"], "traffic": ncu_traffic.get(top),
                "peak_source": f"of {pk['src']} (burst figure)", "ms_per_launch": stages[top]["ms"]}
    layer_flops = (36.0 * n * h * i + 2.0 * n * h * N_EXPERTS) * (3.0 if args.mode == "fwdbwd" else 1.0)
    line = {
        "metric": {"fwd": METRIC, "fwdbwd": "moe_layer_fwdbwd_tokens_per_s"}.get(args.mode, "ffn_half_fwd_tokens_per_s"), "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args, wl, world),
        "layer_tflops": round(layer_flops * world / (ms_step * 1e-3) / 1e12, 2),
        "layer_frac_of_bf16_peak": round(layer_flops / (ms_step * 1e-3) / 1e12 / pk["tf"], 4),
        "roofline": roof if roof is not None else nvlink, "stages": stages, "ep_phases_ms": ep_phases,
        "ep_check": ep_check, "repeats": repeats, "sustained": sustained, "clocks": clocks, "gpu_launches": launches,
        "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2 * world,
                "d2h_bytes_per_step": out_host.numel() * 2 * world},
    }
    if sustained is not None:
        sustained["layer_frac_of_sustained_bf16_peak"] = (
            round(layer_flops / (sustained["ms_per_step"] * 1e-3) / 1e12 / pk["tf_sus"], 4) if pk["tf_sus"] else None)
    if ep_check is not None and not ep_check["ok"]:
        print(json.dumps(line))
        sys.exit("expert-parallel parity check failed: " + json.dumps(ep_check))
    if args.mode != "fwd":      # the host-buffer call is the block's forward: it says nothing about the other modes
        line["e2e"]["note"] = "host-buffer forward of the block alone (mode fwd), not of mode " + args.mode
    if world == 1 and args.mode == "fwd" and not args.no_gpu_reference:
        res = gpu_eager_reference(wl, t, dev)
        if res is not None:
            line["gpu_eager_reference"], ref_out = res
            ours, _ = Fn.moe_forward(t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"],
                                     t["radial_theta"], TOP_K, "sum")
            torch.cuda.synchronize()
            per_tok = (ours.float() - ref_out.float()).norm(dim=-1) / ref_out.float().norm(dim=-1).clamp_min(1e-30)
            line["gpu_eager_reference"]["our_output_vs_it"] = {
                "median_token_rel": float(per_tok.median()), "tokens_above_5e-2": int((per_tok > 5e-2).sum()),
                "note": "both bf16; a token above the bar took another expert at a bf16 near-tie of the router"}
            line["gpu_eager_reference"]["speedup_device_timed"] = round(value / line["gpu_eager_reference"]["value"], 1)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_oracle_rate(wl)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
