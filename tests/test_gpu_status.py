"""Failure paths that must not go unnoticed, each provoked WITHOUT faulting or hanging the GPU:
a cross-rank barrier whose peer never arrives (the bounded wait runs out: status 5), an expert-parallel
receive buffer that is too small (status 4: nothing is written), routing indices out of range (status 2),
and the host layer turning a status word that a kernel left behind into a RuntimeError."""
import ctypes as C

import pytest
import torch

from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
K, E = 6, 64


def _ptr_array(tensors):
    return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def test_barrier_wait_runs_out_and_reports_status_5():
    """One GPU plays rank 0 of 2; the flag array of "rank 1" is a second local buffer that nobody writes
    into rank 0's slot, so the wait gives up after max_polls polls, raises the status word and returns."""
    from bibo_b200 import _lib
    lib = _lib.load()
    flags = [torch.zeros(8, dtype=torch.int32, device=DEV) for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.bibo_moe_ep_barrier_bounded(_ptr_array(flags), 0, 2, 1, 2000, status.data_ptr(), st), "barrier")
    torch.cuda.synchronize()
    assert int(status) == 5
    assert int(flags[1][0]) == 1, "rank 0 published its epoch into the peer's array before waiting"
    # the context is still usable, and a barrier whose peer HAS arrived passes without touching the status
    status.zero_()
    flags[0][1] = 2                      # what rank 1 would have stored
    _lib.check(lib.bibo_moe_ep_barrier_bounded(_ptr_array(flags), 0, 2, 2, 2000, status.data_ptr(), st), "barrier")
    torch.cuda.synchronize()
    assert int(status) == 0 and int(flags[1][0]) == 2


def test_receive_buffer_overflow_is_status_4_and_nothing_is_written():
    from bibo_b200 import _lib, functional as Fn
    lib, p = _lib.load(), _lib.ptr
    n, hidden, world = 1024, 256, 2
    inp = orc.make_inputs(n, hidden, 128, E, seed=2, bias_mode="uniform")
    x = inp["x"].to(DEV).to(torch.bfloat16)
    w_r = inp["w_router"].to(DEV).to(torch.bfloat16)
    geo = Fn.Geometry(n, hidden, 128, E, E, 0, K, torch.bfloat16)
    ws = Fn.MoEWorkspace(geo, DEV)
    st = torch.cuda.current_stream().cuda_stream
    Fn.router_forward(x, w_r, inp["bias"].to(DEV), K, ws=ws)
    _lib.check(lib.bibo_moe_plan(p(ws.block_counts), n, K, E, E, p(ws.plan), st), "plan")
    cnt_all = torch.stack([ws.counts(), ws.counts()]).contiguous()       # both "ranks" route alike
    cap = 1024                                                           # far below the ~6000 rows a rank receives
    ep_plan = torch.zeros(int(lib.bibo_moe_ep_plan_words(E, cap)), dtype=torch.int32, device=DEV)
    _lib.check(lib.bibo_moe_ep_plan(p(cnt_all), 0, world, E, cap, p(ep_plan), st), "ep_plan")
    torch.cuda.synchronize()
    assert int(ep_plan[2]) == 4 and int(ep_plan[0]) == 0 and int(ep_plan[1]) == 0 and int(ep_plan[3]) == 0
    recv = [torch.full((cap, hidden), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    slot_row = torch.full((n, K), -9, dtype=torch.int32, device=DEV)
    _lib.check(lib.bibo_moe_ep_dispatch(p(x), p(ws.topk_idx), p(ws.slot_rank), p(ws.plan), p(ep_plan), _ptr_array(recv),
                                        n, hidden, E, 0, world, K, cap, 0, p(slot_row), None, st), "ep_dispatch")
    torch.cuda.synchronize()
    assert all(bool((r == 7.0).all()) for r in recv), "no row may be stored once the overflow is known"
    assert bool((slot_row == -9).all())


def _small(dtype=torch.bfloat16, n=512, hidden=256, inter=256):
    inp = orc.make_inputs(n, hidden, inter, E, seed=4, bias_mode="uniform", theta_std=0.5)
    t = {k: v.to(DEV) for k, v in inp.items()}
    for k in ("x", "w_router", "gate_up_proj", "down_proj"):
        t[k] = t[k].to(dtype).contiguous()
    return inp, t


def test_host_layer_raises_on_a_status_word_left_by_a_kernel():
    from bibo_b200 import functional as Fn
    _, t = _small()
    geo = Fn.Geometry(512, 256, 256, E, E, 0, K, torch.bfloat16)
    ws = Fn.MoEWorkspace(geo, DEV)
    run = lambda: Fn.moe_forward(t["x"], t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"],
                                 t["radial_theta"], K, ws=ws)
    out0, _ = run()
    torch.cuda.synchronize()
    ws.raise_if_failed()                              # clean run: nothing to report
    ws.plan[2] = 104                                  # what a gate/up kernel whose wait gave up leaves behind
    run()                                             # this call cannot know yet; its trailing copy carries the word out
    with pytest.raises(RuntimeError, match="device status 104"):
        ws.raise_if_failed(wait=True)
    out1, _ = run()                                   # reported once, then cleared: the workspace works again
    torch.cuda.synchronize()
    ws.raise_if_failed()
    assert torch.equal(out0, out1)
    # without an explicit check the NEXT call on the workspace raises
    ws.plan[2] = 100
    run()
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="device status 100"):
        run()


def test_host_buffer_call_returns_device_status():
    from bibo_b200 import functional as Fn
    _, t = _small()
    geo = Fn.Geometry(512, 256, 256, E, E, 0, K, torch.bfloat16)
    ws = Fn.MoEWorkspace(geo, DEV)
    xh = t["x"].cpu().pin_memory()
    oh = torch.empty_like(xh).pin_memory()
    xd, od = torch.empty_like(t["x"]), torch.empty_like(t["x"])
    args = (xh, oh, xd, od, t["w_router"], t["bias"], t["gate_up_proj"], t["down_proj"], t["radial_theta"], K)
    Fn.moe_forward_host(*args, ws=ws)
    ws.plan[2] = 101
    with pytest.raises(RuntimeError, match="code -5"):
        Fn.moe_forward_host(*args, ws=ws)
    ws.plan[2] = 0
    Fn.moe_forward_host(*args, ws=ws)


def test_caller_routing_with_empty_and_bad_slots():
    """BiBoFusedExperts.forward(x, idx, w) seam: a slot with index -1 is an empty slot (no row, contributes
    nothing); an index >= n_experts is ignored too but reported (status 2 -> RuntimeError at the next check).
    The reference raises a Python error for both; nothing here may write out of bounds."""
    from bibo_b200 import functional as Fn
    inp, t = _small(torch.float32, n=300, hidden=128, inter=64)
    logits = orc.router_logits(inp["x"], inp["w_router"])
    idx, w, _ = orc.router_select(logits, inp["bias"], K)
    idx_e, w_e = idx.clone(), w.clone()
    idx_e[::3, 2] = -1                               # every third token loses its third slot
    w_ref = w_e.clone()
    w_ref[::3, 2] = 0.0
    ref = orc.experts_forward(inp["x"], idx, w_ref, inp["gate_up_proj"], inp["down_proj"], inp["radial_theta"])
    out, ws = Fn.experts_forward(t["x"], idx_e.to(DEV), w_e.to(DEV), t["gate_up_proj"], t["down_proj"],
                                 t["radial_theta"], E)
    torch.cuda.synchronize()
    ws.raise_if_failed()
    err = float((out.cpu() - ref).abs().max() / ref.abs().max())
    assert err < 1e-4, err
    idx_bad = idx.clone()
    idx_bad[5, 0] = E + 3
    Fn.experts_forward(t["x"], idx_bad.to(DEV), w.to(DEV), t["gate_up_proj"], t["down_proj"], t["radial_theta"], E, ws=ws)
    with pytest.raises(RuntimeError, match="device status 2"):
        ws.raise_if_failed(wait=True)
