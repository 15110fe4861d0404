"""Host-side logic of the expert-parallel path on CPU ranks (gloo, world_size 2 and 4)."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, path, n_exp):
    from bibo_b200.ep import ep_layout, recv_rows_cap
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(100 + rank)
    counts = torch.randint(0, 700, (n_exp,), generator=g, dtype=torch.int32)
    counts[rank] = 0                                   # an empty (expert, source) group
    cnt_all = torch.zeros(world, n_exp, dtype=torch.int32)
    dist.all_gather_into_tensor(cnt_all.view(-1), counts)
    lay = ep_layout(cnt_all, rank, world)
    el = n_exp // world
    # every rank's view of "where do rank s's rows of expert e start in owner d's buffer" must agree
    send = [torch.zeros(n_exp, dtype=torch.int64) for _ in range(world)]
    recv = [torch.zeros(n_exp + 1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(send, lay["send_base"])
    dist.all_gather(recv, lay["recv_off"])
    for s in range(world):
        for e in range(n_exp):
            d, le = divmod(e, el)
            assert int(send[s][e]) == int(recv[d][le * world + s])
    # groups are tile-aligned, disjoint and in (expert, source) order
    off, cnt = lay["recv_off"], lay["recv_cnt"]
    assert (off % 128 == 0).all()
    assert (off[1:] - off[:-1] >= cnt).all() and (off[1:] - off[:-1] < cnt + 128).all()
    assert int(lay["rows"][rank]) == int(off[-1])
    total = int(cnt_all.sum())
    assert int(lay["recv_cnt"].sum()) == int(cnt_all[:, rank * el:(rank + 1) * el].sum())
    cap = recv_rows_cap(1000, 6, n_exp, world, 2.0)
    assert cap % 128 == 0 and cap >= 2 * 6000
    assert total > 0
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ep_layout_is_consistent_across_ranks(world):
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, os.path.join(d, "store"), 64), nprocs=world, join=True)


def test_ep_layout_matches_hand_example():
    from bibo_b200.ep import ep_layout
    cnt = torch.tensor([[130, 0, 5, 128], [1, 300, 0, 0]], dtype=torch.int32)   # 2 ranks, 4 experts
    l0, l1 = ep_layout(cnt, 0, 2), ep_layout(cnt, 1, 2)
    # rank 0 owns experts 0,1: groups (e0,s0) 130->256, (e0,s1) 1->128, (e1,s0) 0, (e1,s1) 300->384
    assert l0["recv_off"].tolist() == [0, 256, 384, 384, 768]
    assert l0["recv_cnt"].tolist() == [130, 1, 0, 300]
    # rank 1 owns experts 2,3: (e2,s0) 5->128, (e2,s1) 0, (e3,s0) 128->128, (e3,s1) 0
    assert l1["recv_off"].tolist() == [0, 128, 128, 256, 256]
    assert l0["send_base"].tolist() == [0, 384, 0, 128] and l1["send_base"].tolist() == [256, 384, 128, 256]
    assert l0["rows"].tolist() == [768, 256]


def test_source_major_layout_makes_each_exchange_one_block():
    """Copy-engine exchange: owner d's buffer holds all rows of source 0, then source 1, ...; the rows
    of one (source, owner) pair are one contiguous, tile-aligned range, in the source's own expert
    order, so one peer copy moves them in either direction."""
    from bibo_b200.ep import ep_layout
    cnt = torch.tensor([[130, 0, 5, 128], [1, 300, 0, 0]], dtype=torch.int32)   # 2 ranks, 4 experts
    l0, l1 = ep_layout(cnt, 0, 2, source_major=True), ep_layout(cnt, 1, 2, source_major=True)
    # rank 0 owns experts 0,1: from s0: e0 130->256, e1 0 | from s1: e0 1->128, e1 300->384
    assert l0["recv_off"].tolist() == [0, 256, 256, 384, 768]          # index g = le*2 + s
    assert l0["recv_cnt"].tolist() == [130, 1, 0, 300]
    assert l0["send_base"].tolist() == [0, 256, 0, 128] and l1["send_base"].tolist() == [256, 384, 256, 256]
    g = torch.Generator().manual_seed(5)
    world, n_exp = 4, 64
    el = n_exp // world
    cnt_all = torch.randint(0, 500, (world, n_exp), generator=g, dtype=torch.int32)
    pad = (cnt_all.long() + 127) // 128 * 128
    lays = [ep_layout(cnt_all, r, world, source_major=True) for r in range(world)]
    for d in range(world):
        run = 0
        for s in range(world):
            for le in range(el):
                assert int(lays[d]["recv_off"][le * world + s]) == run
                assert int(lays[s]["send_base"][d * el + le]) == run
                run += int(pad[s, d * el + le])
        assert int(lays[d]["rows"][d]) == run


def _module_worker(rank, world, path):
    import bibo_b200
    from bibo_b200 import ep
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    cfg = bibo_b200.MoEConfig(hidden_size=64, moe_intermediate_size=32, num_routed_experts=8, num_experts_per_tok=2)
    torch.manual_seed(0)                                  # the same full layer on every rank
    full = bibo_b200.BiBoMoELayer(cfg)
    shard = ep.ExpertParallelMoELayer.from_full_layer(full, cfg)
    el = 8 // world
    lo, hi = rank * el, (rank + 1) * el
    assert shard.gate_up_proj.shape == (el, 64, 64) and shard.down_proj.shape == (el, 64, 32)
    assert torch.equal(shard.gate_up_proj, full.experts.gate_up_proj[lo:hi])
    assert torch.equal(shard.down_proj, full.experts.down_proj[lo:hi])
    assert torch.equal(shard.radial_theta, full.experts.radial_theta[lo:hi])
    assert torch.equal(shard.gate.gate_proj.weight, full.gate.gate_proj.weight)      # router replicated
    sd = shard.state_dict()
    assert set(sd) == {"gate.bias", "gate.gate_proj.weight", "gate_up_proj", "down_proj", "radial_theta", "accumulated_tpe"}
    # the balancer all-reduces the token counts: every rank applies the same bias update
    counts = torch.zeros(8)
    counts[rank] = 100.0
    from bibo_b200.moe import _balance_from_counts
    shard.bias_update_threshold = 50
    tpe = _balance_from_counts(shard, counts, 50)
    assert tpe is not None and float(tpe.sum()) == 100.0 * world
    shard.update_bias(tpe)
    biases = [torch.zeros(8) for _ in range(world)]
    dist.all_gather(biases, shard.gate.bias.data)
    assert all(torch.equal(b, biases[0]) for b in biases) and float(biases[0].abs().max()) > 0
    for bad in (dict(num_pos_identity_experts=1, num_neg_identity_experts=1), dict(use_shared_expert=True)):
        try:
            ep.ExpertParallelMoELayer(bibo_b200.MoEConfig(hidden_size=64, moe_intermediate_size=32,
                                                          num_routed_experts=8 + 2 * ("num_pos_identity_experts" in bad),
                                                          num_experts_per_tok=2, **bad))
            raise AssertionError("identity / shared experts must be refused")
        except NotImplementedError:
            pass
    dist.destroy_process_group()


def test_expert_parallel_module_shards_and_balances_on_cpu_ranks():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_module_worker, args=(2, os.path.join(d, "store")), nprocs=2, join=True)


def _dedup_worker(rank, world, path):
    """The de-duplicated exchange restated on CPU ranks (fp32, gloo collectives in place of peer stores): fixed
    slots v = source*n_cap + token, local expert indices with empty slots, one partial sum per (token, owner) in
    ascending expert order, partial rows added on the home rank in ascending owner order.  Must reproduce the
    single-process oracle on the concatenated batch to fp32 rounding, with ragged token counts per rank."""
    from oracle import moe_oracle as orc
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    n_exp, k, hidden, inter = 16, 4, 32, 24
    counts = [37 - 9 * r for r in range(world)]
    offs = [sum(counts[:r]) for r in range(world + 1)]
    full = orc.make_inputs(offs[-1], hidden, inter, n_exp, seed=3, bias_mode="uniform", theta_std=0.5)
    x = full["x"][offs[rank]:offs[rank + 1]]
    n = x.shape[0]
    cap = torch.tensor([n])
    dist.all_reduce(cap, op=dist.ReduceOp.MAX)
    n_cap = int(cap)
    assert n_cap == max(counts)
    idx, w, _ = orc.router_select(orc.router_logits(x, full["w_router"]), full["bias"], k)
    # "dispatch": every rank's rows and records into the slot layout of every rank (dense here; the kernels
    # send a row only to the ranks that own one of the token's experts)
    pad = lambda t, fill: torch.cat([t, torch.full((n_cap - n,) + t.shape[1:], fill, dtype=t.dtype)])
    xu = torch.empty(world * n_cap, hidden)
    gidx = torch.empty(world * n_cap, k, dtype=torch.int64)
    gw = torch.empty(world * n_cap, k)
    dist.all_gather_into_tensor(xu, pad(x, 0.0))
    dist.all_gather_into_tensor(gidx, pad(idx, -1))
    dist.all_gather_into_tensor(gw, pad(w, 0.0))
    el = n_exp // world
    lo = rank * el
    local = (gidx >= lo) & (gidx < lo + el)
    midx = torch.where(local, gidx - lo, torch.full_like(gidx, -1))
    # owner: its experts over the virtual tokens; an empty slot contributes nothing (index 0 with weight 0)
    part = orc.experts_forward(xu, midx.clamp_min(0), torch.where(local, gw, torch.zeros_like(gw)),
                               full["gate_up_proj"][lo:lo + el], full["down_proj"][lo:lo + el],
                               full["radial_theta"][lo:lo + el])
    # "return": block s of every owner's partial rows to home rank s, summed in ascending owner order
    blocks = [torch.empty(world * n_cap, hidden) for _ in range(world)]
    dist.all_gather(blocks, part)
    out = torch.zeros(n, hidden)
    for d in range(world):
        hit = ((idx >= d * el) & (idx < (d + 1) * el)).any(-1)
        out[hit] += blocks[d][rank * n_cap:rank * n_cap + n][hit]
    ref = orc.moe_forward(full["x"], full["w_router"], full["bias"], full["gate_up_proj"], full["down_proj"],
                          full["radial_theta"], k)[offs[rank]:offs[rank + 1]]
    assert float((out - ref).abs().max() / ref.abs().max()) < 1e-6
    # distinct owners per token = rows the kernels send: never more than the slots, never more than the ranks
    owners = torch.zeros(n, world, dtype=torch.bool).scatter_(1, idx // el, True)
    assert int(owners.sum(-1).max()) <= min(k, world) and int(owners.sum()) <= n * k
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_deduplicated_exchange_semantics_on_cpu_ranks(world):
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_dedup_worker, args=(world, os.path.join(d, "store")), nprocs=world, join=True)
