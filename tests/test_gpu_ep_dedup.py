"""The de-duplicated expert-parallel exchange with ALL ranks played on ONE device: the three stages take
explicit buffer pointers and no kernel waits on another one, so rank after rank can run each stage in turn
(home dispatch of every rank, then owner chain of every rank, then final sum of every rank).

Checked against the single-GPU chain on the concatenated batch with the full expert set (same router
kernel: identical routing; outputs differ only by the bf16 rounding of the per-rank partial sums) and
against the fp32 CPU oracle at the bf16 bars.  World sizes 1, 2, 4, 8; ragged token counts per rank; a rank
without tokens; a run repeated on the same buffers with other tokens (stale rows and records of the previous
run must not leak)."""
import ctypes as C

import pytest
import torch

from conftest import mean_rel_err, rel_err
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
K, E = 6, 64
BF16_MAX, BF16_MEAN = 2e-2, 1e-2


def _weights(hidden, inter, seed):
    inp = orc.make_inputs(8, hidden, inter, E, seed=seed, bias_mode="uniform", theta_std=0.5)
    t = {k: v.to(DEV) for k, v in inp.items() if k != "x"}
    for k in ("w_router", "gate_up_proj", "down_proj"):
        t[k] = t[k].to(torch.bfloat16).contiguous()
    return inp, t


def _play(world, counts, t, hidden, inter, xs, bufs=None, comm_ctas=0, staged=False, shuffle=None):
    """One forward of `world` ranks on this device; returns (outs per rank, buffers).  ``staged``: the owners sum
    their partial rows into a local staging buffer and a separate streaming kernel moves them to the home ranks.
    ``shuffle``: a generator; every token's k slots are put into a random order before the dispatch (a caller
    that routes by itself, as ``torch.topk(sorted=False)`` gives no order) and one slot in eight is emptied."""
    from bibo_b200 import _lib, ep, functional as Fn
    lib, p = _lib.load(), _lib.ptr
    n_cap = max(max(counts), 1)
    el = E // world
    if bufs is None:
        bufs = [ep.DedupBuffers(world, n_cap, K, E, hidden, inter, DEV) for _ in range(world)]
    arr = lambda name: (C.c_void_p * world)(*[getattr(b, name).data_ptr() for b in bufs])
    xu, midx, mw, part = arr("xu"), arr("midx"), arr("mw"), arr("part")
    st = torch.cuda.current_stream().cuda_stream
    for r in range(world):                                    # home: route and dispatch
        b, n = bufs[r], counts[r]
        if n:
            _lib.check(lib.bibo_moe_router_fwd(p(xs[r]), p(t["w_router"]), p(t["bias"]), None, n, hidden, E, K,
                                               _lib.NORM_SUM, 1.0, _lib.BF16, None, p(b.topk_idx), p(b.topk_w),
                                               p(b.slot_rank_home), p(b.block_counts_home), p(b.plan[2:]), st), "router")
            if shuffle is not None:
                perm = torch.argsort(torch.rand(n, K, generator=shuffle), dim=1).to(DEV)
                drop = (torch.rand(n, K, generator=shuffle) < 0.125).to(DEV)
                b.topk_idx[:n] = torch.where(drop, -1, b.topk_idx[:n].gather(1, perm))
                b.topk_w[:n] = b.topk_w[:n].gather(1, perm)
        _lib.check(lib.bibo_moe_ep_dedup_dispatch(p(xs[r]) if n else None, p(b.topk_idx), p(b.topk_w), xu, midx, mw, n,
                                                  n_cap, hidden, E, r, world, K, comm_ctas, st), "dispatch")
    for r in range(world):                                    # owner: experts + partial sums
        b = bufs[r]
        gu, dn = t["gate_up_proj"][r * el:(r + 1) * el].contiguous(), t["down_proj"][r * el:(r + 1) * el].contiguous()
        th = t["radial_theta"][r * el:(r + 1) * el].contiguous()
        b._keep = (gu, dn, th)
        if staged:
            b.pstage = torch.full((world * n_cap, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)
            row = n_cap * hidden * 2
            table = [b.pstage.data_ptr() + (s_ - r) * row for s_ in range(world)]
            table[r] = b.part.data_ptr()
            a = b.owner_args(r, hidden, inter, E, gu, dn, th, (C.c_void_p * world)(*table), 0, 0)
            _lib.check(lib.bibo_moe_ep_dedup_owner(C.byref(a), st), "owner")
            _lib.check(lib.bibo_moe_ep_dedup_push(p(b.pstage), p(b.midx), part, p(b.plan), n_cap, hidden, K, r, world,
                                                  comm_ctas, st), "push")
            continue
        a = b.owner_args(r, hidden, inter, E, gu, dn, th, part, 0, comm_ctas)
        _lib.check(lib.bibo_moe_ep_dedup_owner(C.byref(a), st), "owner")
    outs = []
    for r in range(world):                                    # home: final sum
        b, n = bufs[r], counts[r]
        out = torch.full((n, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)
        _lib.check(lib.bibo_moe_ep_dedup_final(p(b.part), p(b.topk_idx), p(b.plan[2:]), n, n_cap, hidden, E, world, K,
                                               comm_ctas, p(out), st), "final")
        outs.append(out)
    torch.cuda.synchronize()
    for b in bufs:
        assert int(b.plan[2]) == 0, "device status word"
    return outs, bufs


def _check(world, counts, hidden, inter, seed, bufs=None, comm_ctas=0, staged=False):
    from bibo_b200 import functional as Fn
    inp, t = _weights(hidden, inter, seed=3)
    g = torch.Generator().manual_seed(seed)
    xs_cpu = [torch.randn(n, hidden, generator=g).to(torch.bfloat16) for n in counts]
    xs = [x.to(DEV) for x in xs_cpu]
    outs, bufs = _play(world, counts, t, hidden, inter, xs, bufs, comm_ctas, staged)
    x_all = torch.cat(xs)
    ref_gpu, ws = Fn.moe_forward(x_all, t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], K)
    torch.cuda.synchronize()
    got = torch.cat(outs)
    assert not bool(torch.isnan(got.float()).any())
    # same router kernel on the same rows: the routing each rank used is the single-GPU routing
    idx_all = torch.cat([bufs[r].topk_idx[:n] for r, n in enumerate(counts)])
    assert torch.equal(idx_all, ws.topk_idx)
    if world == 1:
        assert torch.equal(got.view(torch.int16), ref_gpu.view(torch.int16)), "one rank: one partial, no extra rounding"
    # every rank's partial is rounded to bf16 once: a handful of bf16 ulps of the largest partial
    assert rel_err(got.float(), ref_gpu.float()) < 1.2e-2
    assert mean_rel_err(got.float(), ref_gpu.float()) < 4e-3
    # fp32 oracle on the same (bf16-valued) inputs, on the tokens it routes identically
    c = {k: (v.to(torch.bfloat16).float() if k in ("w_router", "gate_up_proj", "down_proj") else v) for k, v in inp.items()}
    xf = torch.cat(xs_cpu).float()
    ref, logits, idx, w, _ = orc.moe_forward(xf, c["w_router"], c["bias"], c["gate_up_proj"], c["down_proj"],
                                             c["radial_theta"], K, return_routing=True)
    same = (idx_all.cpu().long() == idx).all(-1)
    assert float(same.float().mean()) > 0.97
    assert rel_err(got.float().cpu()[same], ref[same]) < BF16_MAX
    assert mean_rel_err(got.float().cpu()[same], ref[same]) < BF16_MEAN
    return bufs


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_all_ranks_on_one_device(world):
    counts = [700, 513, 128, 1000, 300, 999, 64, 257][:world]
    _check(world, counts, hidden=512, inter=256, seed=world)


def test_rank_without_tokens_and_reuse_of_buffers():
    bufs = _check(4, [900, 0, 450, 1], hidden=512, inter=256, seed=21)
    # same buffers, fewer tokens on rank 0 and tokens on rank 1: records of the first run must be overwritten
    _check(4, [300, 900, 450, 0], hidden=512, inter=256, seed=22, bufs=bufs)


def test_capped_exchange_grids_and_intermediate_512():
    _check(2, [2048, 1500], hidden=1024, inter=512, seed=5, comm_ctas=16)


@pytest.mark.parametrize("world,comm_ctas", [(4, 0), (8, 12)])
def test_partial_rows_through_a_staging_buffer(world, comm_ctas):
    """Same result when the owners sum into a local staging buffer and a streaming kernel carries the rows home."""
    counts = [600, 333, 128, 900, 1, 512, 64, 257][:world]
    _check(world, counts, hidden=512, inter=256, seed=30 + world, comm_ctas=comm_ctas, staged=True)


def test_caller_routed_lists_in_any_order_with_empty_slots():
    """Slots of a token in random order and some of them empty (-1): against the caller-routed single-GPU chain
    on the same lists (the order changes only the order of the fp32 additions)."""
    from bibo_b200 import functional as Fn
    world, counts, hidden, inter = 4, [800, 257, 1, 600], 512, 256
    _, t = _weights(hidden, inter, seed=3)
    g = torch.Generator().manual_seed(77)
    xs = [torch.randn(n, hidden, generator=g).to(torch.bfloat16).to(DEV) for n in counts]
    outs, bufs = _play(world, counts, t, hidden, inter, xs, shuffle=g)
    idx = torch.cat([bufs[r].topk_idx[:n] for r, n in enumerate(counts)])
    w = torch.cat([bufs[r].topk_w[:n] for r, n in enumerate(counts)])
    assert bool((idx < 0).any()) and not bool((idx[:, 1:] >= idx[:, :-1]).all())
    ref, _ = Fn.experts_forward(torch.cat(xs), idx, w, t["gate_up_proj"], t["down_proj"], t["radial_theta"], E)
    torch.cuda.synchronize()
    got = torch.cat(outs)
    assert not bool(torch.isnan(got.float()).any())
    assert rel_err(got.float(), ref.float()) < 1.2e-2
    assert mean_rel_err(got.float(), ref.float()) < 4e-3
    empty = (idx < 0).all(-1)
    assert not bool(got[empty].float().abs().any())


def test_argument_checks():
    from bibo_b200 import _lib
    lib = _lib.load()
    assert lib.bibo_moe_ep_dedup_dispatch(None, None, None, None, None, None, 10, 5, 512, E, 0, 2, K, 0, None) != 0
    assert lib.bibo_moe_ep_dedup_dispatch(None, None, None, None, None, None, 0, 128, 512, 63, 0, 2, K, 0, None) != 0
    assert lib.bibo_moe_ep_dedup_final(None, None, None, 10, 128, 512, E, 2, K, 0, None, None) != 0
    assert lib.bibo_moe_ep_dedup_rows_cap(8, 1024, K, E) == (8 * 1024 * K + 8 * 127 + 127) // 128 * 128
