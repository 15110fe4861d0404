"""Expert-parallel forward of the MoE block over the GPUs of one NVSwitch box.

One process per GPU (``torch.distributed``, NCCL).  Rank d owns experts ``[d*E/R, (d+1)*E/R)``; tokens
stay on their home rank; the router is replicated.  The exchange steps are not separate collectives:
the dispatch kernel stores token rows straight into the owner ranks' receive buffers and the combine
kernel loads result rows straight from the owners' buffers, both over NVLink peer memory
(``include/bibo_moe.h``, section "expert-parallel forward").  torch supplies the plumbing only:
symmetric (peer-mapped) buffers and one tiny NCCL all-gather of the per-rank histograms.

The reference has no expert parallelism; the oracle for this path is the single-process block on the
concatenation of all ranks' tokens with the full set of expert weights.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib
from . import functional as Fn

TILE_M = _lib.TILE_M


def ep_layout(cnt_all: torch.Tensor, rank: int, world: int, source_major: bool = False):
    """Host mirror of ``ep_plan_kernel`` (used to size buffers and to check the kernel).
    ``source_major``: groups in the order (source, local expert) instead of (local expert, source).

    cnt_all [world, E] = tokens-per-expert histogram of every rank.  Returns a dict with
    ``send_base [E]`` (row in the owner's receive buffer where THIS rank's rows of expert e start),
    ``recv_off [E+1]`` / ``recv_cnt [E]`` of this rank's groups g = le*world + s, ``rows`` per rank.
    """
    cnt = cnt_all.to(torch.int64).cpu()
    n_exp = cnt.shape[1]
    el = n_exp // world
    pad = (cnt + TILE_M - 1) // TILE_M * TILE_M
    send_base = torch.zeros(n_exp, dtype=torch.int64)
    rows = torch.zeros(world, dtype=torch.int64)
    recv_off = torch.zeros(n_exp + 1, dtype=torch.int64)
    recv_cnt = torch.zeros(n_exp, dtype=torch.int64)
    for d in range(world):
        run = 0
        order = [(le, s) for s in range(world) for le in range(el)] if source_major else \
                [(le, s) for le in range(el) for s in range(world)]
        for le, s in order:
            if s == rank:
                send_base[d * el + le] = run
            if d == rank:
                recv_off[le * world + s] = run
                recv_cnt[le * world + s] = cnt[s, d * el + le]
            run += int(pad[s, d * el + le])
        rows[d] = run
        if d == rank:
            recv_off[n_exp] = run
    return dict(send_base=send_base, recv_off=recv_off, recv_cnt=recv_cnt, rows=rows)


def recv_rows_cap(n_tokens: int, top_k: int, n_experts: int, world: int, capacity_factor: Optional[float]) -> int:
    """Rows provisioned per rank for received tokens: capacity_factor x the balanced share, plus the
    worst-case padding of the E groups, rounded to the tile size (never more than every row of every
    rank).  ``None`` = the worst case (every slot of every rank lands here): dropless, like the reference."""
    balanced = n_tokens * top_k                      # world * N * k / world
    worst = world * n_tokens * top_k
    rows = (worst if capacity_factor is None else min(int(balanced * capacity_factor), worst)) + n_experts * (TILE_M - 1)
    return (rows + TILE_M - 1) // TILE_M * TILE_M


class _Symmetric:
    """A tensor every rank allocates identically, mapped into every process of the group."""

    def __init__(self, shape, dtype, device, group):
        import torch.distributed._symmetric_memory as symm_mem
        self.tensor = symm_mem.empty(*shape, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group.group_name)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.ptr_array = (C.c_void_p * len(self.ptrs))(*self.ptrs)


class ExpertParallelMoE:
    """Forward of the MoE block with the experts sharded over ``group``.

    ``weights`` holds the FULL tensors (``w_router [E,H]``, ``bias [E]``, ``gate_up_proj [E,2I,H]``,
    ``down_proj [E,H,I]``, ``radial_theta [E]``) or already-sharded expert tensors (leading dimension
    E/world); only this rank's shard is kept.
    """

    def __init__(self, weights, top_k: int, group=None, n_tokens: Optional[int] = None, norm_mode="sum",
                 scale: float = 1.0, capacity_factor: Optional[float] = None, max_ctas: int = 0, comm_ctas: int = 0,
                 dma: bool = False, copy_streams: bool = False):
        """``capacity_factor``: receive buffers hold this multiple of the balanced load; ``None`` (default)
        provisions the worst case, so no routing can overflow them (the reference is dropless).  With a cap, an
        overflow is detected on the device by every rank (status 4), nothing is written, and the next call on
        this object raises."""
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads/stores only
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.top_k, self.norm_mode, self.scale = top_k, norm_mode, scale
        self.capacity_factor, self.max_ctas, self.comm_ctas = capacity_factor, max_ctas, comm_ctas
        # dma: rows travel by asynchronous peer copies (copy engines) instead of the dispatch / combine
        # kernels (bibo_moe_ep_forward_dma); inference forward only, training calls use the kernels
        self.dma = bool(dma)
        self.copy_streams = bool(copy_streams)     # copies to different peers on separate streams (concurrent)
        w_r = weights["w_router"]
        self.device = w_r.device
        self.n_experts, self.hidden = w_r.shape
        if self.n_experts % self.world:
            raise RuntimeError(f"{self.n_experts} experts do not shard evenly over {self.world} ranks")
        self.el = self.n_experts // self.world
        lo, hi = self.rank * self.el, (self.rank + 1) * self.el
        shard = lambda t: (t[lo:hi] if t.shape[0] == self.n_experts else t).contiguous()
        self.w_router, self.bias = w_r.contiguous(), weights["bias"].float().contiguous()
        self.gate_up, self.down = shard(weights["gate_up_proj"]), shard(weights["down_proj"])
        self.theta = shard(weights["radial_theta"]).float().contiguous()
        self.inter = self.gate_up.shape[1] // 2
        if w_r.dtype != torch.bfloat16:
            raise RuntimeError("the expert-parallel path runs the bf16 tensor-core kernels only")
        self._n = None
        self._epoch = 0
        if n_tokens is not None:
            self._allocate(n_tokens)

    # ---- buffers --------------------------------------------------------------------------------------
    def _allocate(self, n_tokens: int) -> None:
        lib = _lib.load()
        dev, k, e = self.device, self.top_k, self.n_experts
        self._n = n_tokens
        self.cap = recv_rows_cap(n_tokens, k, e, self.world, self.capacity_factor)
        geo = Fn.Geometry(n_tokens, self.hidden, self.inter, e, e, 0, k, torch.bfloat16)
        i32 = dict(dtype=torch.int32, device=dev)
        self.topk_idx = torch.empty(n_tokens, k, **i32)
        self.topk_w = torch.empty(n_tokens, k, dtype=torch.float32, device=dev)
        self.slot_rank = torch.empty(n_tokens, k, **i32)
        self.block_counts = torch.empty(geo.router_blocks, e, **i32)
        self.local_plan = torch.zeros(geo.plan_words, **i32)
        self.slot_row = torch.empty(n_tokens, k, **i32)
        self.ep_plan = torch.zeros(int(lib.bibo_moe_ep_plan_words(e, self.cap)), **i32)
        self.cnt = _Symmetric((self.world, e), torch.int32, dev, self.group)   # histograms, written by peers
        self.cnt_all = self.cnt.tensor
        self.h = torch.empty(self.cap, self.inter, dtype=torch.bfloat16, device=dev)
        self.xp = _Symmetric((self.cap, self.hidden), torch.bfloat16, dev, self.group)
        self.y = _Symmetric((self.cap, self.hidden), torch.bfloat16, dev, self.group)
        if self.dma:
            self.xp_send = torch.empty(geo.rows_cap, self.hidden, dtype=torch.bfloat16, device=dev)
            self.y_owner = torch.empty(self.cap, self.hidden, dtype=torch.bfloat16, device=dev)
            self.y_home = _Symmetric((geo.rows_cap, self.hidden), torch.bfloat16, dev, self.group)
            self.row_token_dma = torch.empty(geo.rows_cap, **i32)
            self.cnt_host = torch.zeros(self.world * e, dtype=torch.int32).pin_memory()
            self.counts_ready = torch.cuda.Event()
            self.counts_ready.record()          # creates the underlying event
            n_aux = min(self.world, 8) if self.copy_streams else 0
            self._aux_streams = [torch.cuda.Stream(device=dev) for _ in range(n_aux)]
            self._aux_events = [torch.cuda.Event() for _ in range(18)]
            for ev in self._aux_events:
                ev.record()
            self._aux_stream_ptrs = (C.c_void_p * max(n_aux, 1))(*[s_.cuda_stream for s_ in self._aux_streams])
            self._aux_event_ptrs = (C.c_void_p * 18)(*[ev.cuda_event for ev in self._aux_events])
        self.flags = _Symmetric((64,), torch.int32, dev, self.group)
        self.flags.tensor.zero_()
        self.header_host = torch.zeros(8, dtype=torch.int32).pin_memory()   # both plans' headers, see raise_if_failed
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)            # every rank's flags are zero before the first device barrier
        o = int(lib.bibo_moe_plan_off_counts())
        self._counts = self.local_plan[o:o + e]
        self._args = None

    def _barrier(self, st) -> None:
        self._epoch += 1
        _lib.check(_lib.load().bibo_moe_ep_barrier(self.flags.ptr_array, self.rank, self.world, self._epoch,
                                                   _lib.ptr(self.ep_plan[2:]), st), "bibo_moe_ep_barrier")

    # ---- forward ----------------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, training: bool = False,
                phase: int = 0) -> torch.Tensor:
        """``phase`` (copy-engine path only): 1 = issue the part before the host reads the histogram table
        and return; ``finish()`` issues the rest."""
        lib, p = _lib.load(), _lib.ptr
        n, hidden = x.shape
        if self._n != n:
            self._allocate(n)
            self._train_ready = False
        if out is None:
            out = torch.empty_like(x)
        k, e, st = self.top_k, self.n_experts, torch.cuda.current_stream(self.device).cuda_stream
        if phase != 2:
            self.raise_if_failed()
        if training or self.dma or not getattr(self, "profile", False):
            out = self._forward_one_call(x, out, st, training, phase if self.dma and not training else 0)
            if phase != 1:
                self._post_status()
            return out
        ev = self._mark
        ev("start")
        _lib.check(lib.bibo_moe_router_fwd(p(x), p(self.w_router), p(self.bias), None, n, hidden, e, k,
                                           Fn.norm_code(self.norm_mode), float(self.scale), _lib.BF16, None,
                                           p(self.topk_idx), p(self.topk_w), p(self.slot_rank), p(self.block_counts),
                                           p(self.local_plan[2:]), st), "bibo_moe_router_fwd")
        _lib.check(lib.bibo_moe_plan(p(self.block_counts), n, k, e, e, p(self.local_plan), st), "bibo_moe_plan")
        ev("route")
        dist.all_gather_into_tensor(self.cnt_all.view(-1), self._counts, group=self.group)
        _lib.check(lib.bibo_moe_ep_plan(p(self.cnt_all), self.rank, self.world, e, self.cap, p(self.ep_plan), st),
                   "bibo_moe_ep_plan")
        ev("gather_plan")
        _lib.check(lib.bibo_moe_ep_dispatch(p(x), p(self.topk_idx), p(self.slot_rank), p(self.local_plan),
                                            p(self.ep_plan), self.xp.ptr_array, n, hidden, e, self.rank, self.world, k,
                                            self.cap, self.comm_ctas, p(self.slot_row), None, st),
                   "bibo_moe_ep_dispatch")
        ev("dispatch")
        self._barrier(st)                   # every rank's rows have landed
        ev("barrier1")
        _lib.check(lib.bibo_moe_ep_experts(p(self.xp.tensor), p(self.gate_up), p(self.down), p(self.theta),
                                           p(self.ep_plan), hidden, self.inter, e, self.world, self.cap, self.max_ctas,
                                           p(self.h), p(self.y.tensor), None, None, 0, st), "bibo_moe_ep_experts")
        ev("experts")
        self._barrier(st)                   # every rank's results are written
        ev("barrier2")
        _lib.check(lib.bibo_moe_ep_combine(self.y.ptr_array, p(self.slot_row), p(self.topk_w), p(self.ep_plan), n,
                                           hidden, self.world, k, self.cap, self.comm_ctas, p(out), st),
                   "bibo_moe_ep_combine")
        ev("combine")
        self._post_status()
        return out

    def _post_status(self) -> None:
        self.header_host[:4].copy_(self.ep_plan[:4], non_blocking=True)
        self.header_host[4:].copy_(self.local_plan[:4], non_blocking=True)

    def raise_if_failed(self, wait: bool = False) -> None:
        """RuntimeError if a kernel of an earlier call on this object left a status word (4 = a receive buffer
        would have overflowed: nothing was exchanged; 5 = a cross-rank barrier timed out; 100.. = a bounded
        wait in a kernel gave up).  Looks at what an asynchronous copy behind that call brought to the host, so
        without ``wait`` nothing is synchronised; the words are cleared once reported."""
        if self._n is None:
            return
        if wait:
            torch.cuda.current_stream(self.device).synchronize()
        code = max(int(self.header_host[2]), int(self.header_host[6]))
        if code != 0:
            self.header_host.zero_()
            self.ep_plan[2:3].zero_()
            self.local_plan[2:3].zero_()
            hint = " (raise capacity_factor, or leave it at None for the dropless worst case)" if code == 4 else ""
            raise RuntimeError(f"bibo_b200: an expert-parallel call reported device status {code} "
                               f"({Fn.STATUS_TEXT.get(code, 'see the plan layout in bibo_moe.h')}){hint}; its results "
                               "and those of the calls issued since are invalid")

    def _allocate_training(self) -> None:
        """Extra buffers the backward pass needs (allocated on the first training forward)."""
        dev, n, k, e = self.device, self._n, self.top_k, self.n_experts
        rows_local = Fn.Geometry(n, self.hidden, self.inter, e, e, 0, k, torch.bfloat16).rows_cap
        f32 = dict(dtype=torch.float32, device=dev)
        self.gate_up_recv = torch.empty(self.cap, 2 * self.inter, dtype=torch.bfloat16, device=dev)
        self.rnorm_recv = torch.empty(self.cap, **f32)
        self.row_token = torch.zeros(rows_local, dtype=torch.int32, device=dev)
        self.dy = _Symmetric((self.cap, self.hidden), torch.bfloat16, dev, self.group)
        self.dh = torch.empty(self.cap, self.inter, dtype=torch.bfloat16, device=dev)
        self.dw = torch.empty(n, k, **f32)
        self.dlogit_row = torch.zeros(rows_local, **f32)
        self.dtheta_row = torch.zeros(self.cap, **f32)
        self._train_ready = True

    def backward(self, dout: torch.Tensor):
        """Gradients of the last TRAINING forward (``forward(x, training=True)``): returns
        (dx [N,H], d_w_router [E,H] = this rank's tokens only, d_gate_up_proj, d_down_proj, d_theta)
        for this rank's experts."""
        if getattr(self, "_last_args", None) is None:
            raise RuntimeError("backward needs a preceding forward(x, training=True)")
        p, dev = _lib.ptr, self.device
        dout = dout.contiguous()
        dx = torch.empty_like(dout)
        d_wr = torch.zeros_like(self.w_router)
        d_gu, d_dn = torch.empty_like(self.gate_up), torch.empty_like(self.down)   # written in full by the kernels
        d_th = torch.zeros(self.el, dtype=torch.float32, device=dev)
        b = _lib.EpBwdArgs(p(dout), C.cast(self.dy.ptr_array, C.c_void_p), p(self.dh), p(self.dw), p(self.dlogit_row),
                           p(self.dtheta_row), p(dx), p(d_wr), p(d_gu), p(d_dn), p(d_th), self._epoch)
        self._epoch += 2
        st = torch.cuda.current_stream(dev).cuda_stream
        _lib.check(_lib.load().bibo_moe_ep_backward(C.byref(self._last_args), C.byref(b), st), "bibo_moe_ep_backward")
        self._last_args = None
        self._post_status()
        return dx, d_wr, d_gu, d_dn, d_th

    DMA_MARKS = ("start", "histograms", "sorted", "sent", "received", "experts", "returned", "all_returned", "combine")

    def _mark_array(self):
        """profile=True: nine timing events the copy-engine forward records (see ``marks``)."""
        if not getattr(self, "profile", False):
            return None
        evs = [torch.cuda.Event(enable_timing=True) for _ in self.DMA_MARKS]
        for e in evs:
            e.record()                           # creates the underlying events
        self.marks = list(zip(self.DMA_MARKS, evs))
        self._mark_ptrs = (C.c_void_p * len(evs))(*[e.cuda_event for e in evs])
        return C.cast(self._mark_ptrs, C.c_void_p)

    def finish(self) -> None:
        """Second half of a ``forward(..., phase=1)`` of the copy-engine path (same stream)."""
        a, d, st = self._dma_call
        _lib.check(_lib.load().bibo_moe_ep_forward_dma(C.byref(a), C.byref(d), 2, st), "bibo_moe_ep_forward_dma")
        self._post_status()

    def _forward_one_call(self, x: torch.Tensor, out: torch.Tensor, st: int, training: bool = False,
                          phase: int = 0) -> torch.Tensor:
        """The product path: bibo_moe_ep_forward (histograms exchanged through peer memory, no library
        collective)."""
        if training and not getattr(self, "_train_ready", False):
            self._allocate_training()
        p = _lib.ptr
        C_vp = C.c_void_p
        cast = lambda arr: C.cast(arr, C_vp)
        a = _lib.EpArgs(
            x.shape[0], self.cap, self.hidden, self.inter, self.n_experts, self.top_k, Fn.norm_code(self.norm_mode),
            self.rank, self.world, self.max_ctas, self.comm_ctas, self._epoch, float(self.scale),
            p(x), p(self.w_router), p(self.bias), p(self.gate_up), p(self.down), p(self.theta),
            p(self.topk_idx), p(self.topk_w), p(self.slot_rank), p(self.block_counts), p(self.local_plan),
            p(self.ep_plan), p(self.slot_row), p(self.h), cast(self.xp.ptr_array), cast(self.y.ptr_array),
            cast(self.flags.ptr_array), cast(self.cnt.ptr_array), p(out),
            p(self.gate_up_recv) if training else None, p(self.rnorm_recv) if training else None,
            p(self.row_token) if training else None, self._trace_struct())
        self._epoch += 3
        if self.dma and not training:
            d = _lib.EpDma(p(self.xp_send), p(self.y_owner), cast(self.y_home.ptr_array), p(self.row_token_dma),
                           p(self.cnt_host), self.counts_ready.cuda_event, len(self._aux_streams),
                           C.cast(self._aux_stream_ptrs, C.c_void_p), C.cast(self._aux_event_ptrs, C.c_void_p),
                           self._mark_array())
            self._dma_call = (a, d, st)
            if phase != 2:
                _lib.check(_lib.load().bibo_moe_ep_forward_dma(C.byref(a), C.byref(d), phase, st),
                           "bibo_moe_ep_forward_dma")
            return out
        _lib.check(_lib.load().bibo_moe_ep_forward(C.byref(a), st), "bibo_moe_ep_forward")
        self._last_args, self._last_x = (a, x) if training else (None, None)
        return out

    def _trace_struct(self):
        """Pointer to a bibo_moe_router_trace for this call when ``self.trace`` = (acc, counts, gap) is set
        (the router and plan kernels then fold this rank's routing diagnostics into those tensors)."""
        trace = getattr(self, "trace", None)
        if trace is None:
            return None
        blocks = _lib.load().bibo_moe_router_blocks(self._n)
        if getattr(self, "_trace_blocks", None) is None or self._trace_blocks.shape[0] != blocks:
            self._trace_blocks = torch.empty(blocks, _lib.TRACE_WORDS, dtype=torch.float32, device=self.device)
        self._trace_c = _lib.RouterTrace(_lib.ptr(self._trace_blocks), *[_lib.ptr(t) for t in trace])
        return C.cast(C.pointer(self._trace_c), C.c_void_p)

    def _mark(self, name: str) -> None:
        """profile=True: record a timing event after each phase of the current forward."""
        if name == "start":
            self.marks = []
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.marks.append((name, e))

    def phase_ms(self):
        """Device time of each phase of the last profiled forward (call after a synchronize)."""
        return {n: self.marks[i - 1][1].elapsed_time(ev) for i, (n, ev) in enumerate(self.marks) if i > 0}

    def status(self) -> int:
        """Sticky status words of both plans (synchronises): 0 = fine, 4 = receive buffer overflow,
        5 = a cross-rank barrier timed out, 100-102 = a bounded wait in a kernel gave up."""
        return max(int(self.ep_plan[2].item()), int(self.local_plan[2].item()))


class DedupBuffers:
    """The buffers one rank needs for the de-duplicated exchange (``include/bibo_moe.h``, "expert-parallel
    forward with a de-duplicated exchange").  ``group`` given: the four exchange buffers and the barrier flags are
    symmetric (peer-mapped) allocations; ``group=None``: plain local tensors, for playing several ranks on
    one device (tests)."""

    def __init__(self, world: int, n_cap: int, top_k: int, n_experts: int, hidden: int, inter: int, device, group=None):
        lib = _lib.load()
        self.world, self.n_cap, self.top_k = world, n_cap, top_k
        nv = world * n_cap
        el = n_experts // world
        rows = int(lib.bibo_moe_ep_dedup_rows_cap(world, n_cap, top_k, n_experts))
        i32 = dict(dtype=torch.int32, device=device)
        bf = dict(dtype=torch.bfloat16, device=device)

        def shared(shape, dtype):
            if group is None:
                return None, torch.empty(*shape, dtype=dtype, device=device)
            sym = _Symmetric(shape, dtype, device, group)
            return sym, sym.tensor

        self.sym_xu, self.xu = shared((nv, hidden), torch.bfloat16)
        self.sym_midx, self.midx = shared((nv, top_k), torch.int32)
        self.sym_mw, self.mw = shared((nv, top_k), torch.float32)
        self.sym_part, self.part = shared((nv, hidden), torch.bfloat16)
        self.sym_flags, self.flags = shared((64,), torch.int32)
        self.flags.zero_()
        self.midx.fill_(-1)              # until a source rank has written its records, its tokens do not exist
        self.slot_rank = torch.empty(nv, top_k, **i32)
        self.block_counts = torch.empty(int(lib.bibo_moe_router_blocks(nv)), el, **i32)
        self.plan = torch.zeros(int(lib.bibo_moe_ep_dedup_plan_words(world, n_cap, top_k, n_experts)), **i32)
        self.slot_row = torch.empty(nv, top_k, **i32)
        self.row_token = torch.empty(rows, **i32)
        self.xp = torch.empty(rows, hidden, **bf)
        self.h = torch.empty(rows, inter, **bf)
        self.y = torch.empty(rows, hidden, **bf)
        # home side: routing of this rank's own tokens
        self.topk_idx = torch.empty(n_cap, top_k, **i32)
        self.topk_w = torch.empty(n_cap, top_k, dtype=torch.float32, device=device)
        self.slot_rank_home = torch.empty(n_cap, top_k, **i32)
        self.block_counts_home = torch.empty(int(lib.bibo_moe_router_blocks(n_cap)), n_experts, **i32)

    def owner_args(self, rank: int, hidden: int, inter: int, n_experts: int, gate_up, down, theta, part_ptr_array,
                   max_ctas: int = 0, comm_ctas: int = 0) -> _lib.EpDedupOwner:
        p = _lib.ptr
        return _lib.EpDedupOwner(self.n_cap, hidden, inter, n_experts, self.top_k, rank, self.world, max_ctas, comm_ctas,
                                 p(self.xu), p(self.midx), p(self.mw), p(gate_up), p(down), p(theta), p(self.slot_rank),
                                 p(self.block_counts), p(self.plan), p(self.slot_row), p(self.row_token), p(self.xp),
                                 p(self.h), p(self.y), C.cast(part_ptr_array, C.c_void_p))


class DedupExpertParallelMoE:
    """Inference forward of the MoE block with the experts sharded over ``group`` and a de-duplicated exchange:
    one row per (token, destination rank) goes out, one partial result row per (token, rank) comes back
    (``bibo_moe_ep_dedup_forward``).  Dropless: the owner's buffers hold the worst case.  Results are within
    the bf16 parity bars of the fp32 oracle; they are not bit-identical to the single-GPU chain (every rank's
    partial sum is rounded to bf16 once).  ``weights`` as for ``ExpertParallelMoE``.

    Every rank calls ``forward`` the same number of times (each call holds two device barriers); token counts may
    differ between ranks and between calls up to the capacity the group agreed on at the first call (the largest
    count of any rank then, or ``n_tokens``).  A call above that capacity re-allocates the peer buffers with a
    collective, so it has to happen on every rank in the same call: pass ``n_tokens`` = the largest count that
    will ever occur when the ranks' counts grow independently."""

    MARKS = ("start", "route", "dispatch", "received", "experts", "partial", "returned", "sum")

    def __init__(self, weights, top_k: int, group=None, n_tokens: Optional[int] = None, norm_mode="sum",
                 scale: float = 1.0, max_ctas: int = 0, comm_ctas: int = 0, **_unused):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads/stores only
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.top_k, self.norm_mode, self.scale = top_k, norm_mode, scale
        self.max_ctas, self.comm_ctas = max_ctas, comm_ctas
        w_r = weights["w_router"]
        self.device = w_r.device
        self.n_experts, self.hidden = w_r.shape
        if self.n_experts % self.world:
            raise RuntimeError(f"{self.n_experts} experts do not shard evenly over {self.world} ranks")
        if w_r.dtype != torch.bfloat16:
            raise RuntimeError("the expert-parallel path runs the bf16 tensor-core kernels only")
        self.el = self.n_experts // self.world
        lo, hi = self.rank * self.el, (self.rank + 1) * self.el
        shard = lambda t: (t[lo:hi] if t.shape[0] == self.n_experts else t).contiguous()
        self.w_router, self.bias = w_r.contiguous(), weights["bias"].float().contiguous()
        self.gate_up, self.down = shard(weights["gate_up_proj"]), shard(weights["down_proj"])
        self.theta = shard(weights["radial_theta"]).float().contiguous()
        self.inter = self.gate_up.shape[1] // 2
        self.dma = False
        self._n_cap, self._epoch, self.buf, self.profile, self.trace = None, 0, None, False, None
        if n_tokens is not None:
            self._allocate(n_tokens)

    def _allocate(self, n_tokens: int) -> None:
        cap = torch.tensor([n_tokens], dtype=torch.int64, device=self.device)
        dist.all_reduce(cap, op=dist.ReduceOp.MAX, group=self.group)      # ranks may hold different token counts
        self._n_cap = int(cap)
        self.buf = DedupBuffers(self.world, self._n_cap, self.top_k, self.n_experts, self.hidden, self.inter,
                                self.device, self.group)
        self.header_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        self._epoch = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)            # every rank's flags and records are initialised before the first step

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, training: bool = False,
                phase: int = 0) -> torch.Tensor:
        if training:
            raise RuntimeError("the de-duplicated exchange is forward-only; train through ExpertParallelMoE")
        n, hidden = x.shape
        if self.buf is None or n > self._n_cap:
            self._allocate(n)
        self.raise_if_failed()
        if out is None:
            out = torch.empty_like(x)
        b, p = self.buf, _lib.ptr
        cast = lambda sym: C.cast(sym.ptr_array, C.c_void_p)
        marks = None
        if self.profile:
            evs = [torch.cuda.Event(enable_timing=True) for _ in self.MARKS]
            for e in evs:
                e.record()
            self.marks = list(zip(self.MARKS, evs))
            self._mark_ptrs = (C.c_void_p * len(evs))(*[e.cuda_event for e in evs])
            marks = C.cast(self._mark_ptrs, C.c_void_p)
        owner = b.owner_args(self.rank, hidden, self.inter, self.n_experts, self.gate_up, self.down, self.theta,
                             b.sym_part.ptr_array, self.max_ctas, self.comm_ctas)
        a = _lib.EpDedup(owner, n, Fn.norm_code(self.norm_mode), self._epoch, float(self.scale), p(x), p(self.w_router),
                         p(self.bias), p(b.topk_idx), p(b.topk_w), p(b.slot_rank_home), p(b.block_counts_home),
                         cast(b.sym_xu), cast(b.sym_midx), cast(b.sym_mw), cast(b.sym_flags), p(b.part), p(out), marks,
                         self._trace_struct(n))
        self._epoch += 2
        st = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.load().bibo_moe_ep_dedup_forward(C.byref(a), st), "bibo_moe_ep_dedup_forward")
        self.header_host.copy_(b.plan[:4], non_blocking=True)
        return out

    # ---- the forward in three stream-ordered stages (used by PipelinedDedupMoE) -------------------------
    def _mark(self, name: str) -> None:
        if self.profile:
            if name == "start":
                self.marks = []
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.marks.append((name, e))

    def _barrier(self, st: int) -> None:
        self._epoch += 1
        b = self.buf
        _lib.check(_lib.load().bibo_moe_ep_barrier(b.sym_flags.ptr_array, self.rank, self.world, self._epoch,
                                                   _lib.ptr(b.plan[2:]), st), "bibo_moe_ep_barrier")

    def stage_home(self, x: torch.Tensor) -> None:
        """Router and dispatch of this rank's tokens, then the barrier after which every rank's rows have
        landed (current stream)."""
        lib, p, b = _lib.load(), _lib.ptr, self.buf
        n, hidden = x.shape
        if b is None or n > self._n_cap:
            raise RuntimeError("allocate the lane before staging it")
        self.raise_if_failed()
        st = torch.cuda.current_stream(self.device).cuda_stream
        self._mark("start")
        if n:
            _lib.check(lib.bibo_moe_router_fwd(p(x), p(self.w_router), p(self.bias), None, n, hidden, self.n_experts,
                                               self.top_k, Fn.norm_code(self.norm_mode), float(self.scale), _lib.BF16, None,
                                               p(b.topk_idx), p(b.topk_w), p(b.slot_rank_home), p(b.block_counts_home),
                                               p(b.plan[2:]), st), "bibo_moe_router_fwd")
        self._mark("route")
        raw = getattr(b, "sym_raw", None)
        if raw is None:
            _lib.check(lib.bibo_moe_ep_dedup_dispatch(p(x) if n else None, p(b.topk_idx), p(b.topk_w), b.sym_xu.ptr_array,
                                                      b.sym_midx.ptr_array, b.sym_mw.ptr_array, n, self._n_cap, hidden,
                                                      self.n_experts, self.rank, self.world, self.top_k, self.comm_ctas,
                                                      st), "bibo_moe_ep_dedup_dispatch")
        else:
            # pipelined form: the records travel as two block copies per peer (copy engines), the kernel stores rows only
            if n < b.n_routed:
                b.topk_idx[n:].fill_(-1)
            b.n_routed = n
            block = self._n_cap * self.top_k * 4
            for sym, src in ((raw, b.topk_idx), (b.sym_mw, b.topk_w)):
                _lib.check(lib.bibo_moe_ep_copy_to_peers(sym.ptr_array, self.rank * block, p(src), 0, block, self.rank,
                                                         self.world, 1, st), "bibo_moe_ep_copy_to_peers")
            _lib.check(lib.bibo_moe_ep_dedup_dispatch(p(x) if n else None, p(b.topk_idx), p(b.topk_w), b.sym_xu.ptr_array,
                                                      None, None, n, self._n_cap, hidden, self.n_experts, self.rank,
                                                      self.world, self.top_k, self.comm_ctas, st),
                       "bibo_moe_ep_dedup_dispatch")
        self._mark("dispatch")
        self._barrier(st)
        self._mark("received")
        self._n_last = n

    def _owner(self) -> _lib.EpDedupOwner:
        b = self.buf
        return b.owner_args(self.rank, self.hidden, self.inter, self.n_experts, self.gate_up, self.down, self.theta,
                            b.sym_part.ptr_array, self.max_ctas, self.comm_ctas)

    def stage_experts(self) -> None:
        """The tensor-core part of the owner's work on the received rows (current stream).  With a staging
        buffer (``add_staging``) the partial rows are summed here too, at full HBM speed, into that buffer."""
        st = torch.cuda.current_stream(self.device).cuda_stream
        lib, b = _lib.load(), self.buf
        if getattr(b, "sym_raw", None) is not None:      # records arrived as raw top-k tables: keep this rank's slots
            _lib.check(lib.bibo_moe_ep_localize(_lib.ptr(b.sym_raw.tensor), self.world * self._n_cap, self.top_k,
                                                self.n_experts, self.rank, self.world, _lib.ptr(b.midx), st),
                       "bibo_moe_ep_localize")
        if getattr(b, "pstage", None) is None:
            _lib.check(lib.bibo_moe_ep_dedup_experts(C.byref(self._owner()), st), "bibo_moe_ep_dedup_experts")
            return
        owner = b.owner_args(self.rank, self.hidden, self.inter, self.n_experts, self.gate_up, self.down, self.theta,
                             b.stage_table, self.max_ctas, 0)
        _lib.check(lib.bibo_moe_ep_dedup_owner(C.byref(owner), st), "bibo_moe_ep_dedup_owner")

    def add_staging(self) -> None:
        """A local buffer for the partial rows of other ranks' tokens (the own rank's go straight into ``part``),
        and a peer-mapped table for the raw top-k records of every rank (sent as block copies)."""
        b = self.buf
        nv = self.world * self._n_cap
        b.sym_raw = _Symmetric((nv, self.top_k), torch.int32, self.device, self.group)
        b.sym_raw.tensor.fill_(-1)
        b.topk_idx.fill_(-1)
        b.n_routed = self._n_cap
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        b.pstage = torch.empty(nv, self.hidden, dtype=torch.bfloat16, device=self.device)
        row = self._n_cap * self.hidden * 2
        table = [b.pstage.data_ptr() + (s_ - self.rank) * row for s_ in range(self.world)]
        table[self.rank] = b.part.data_ptr()
        b.stage_table = (C.c_void_p * self.world)(*table)

    def stage_push(self) -> None:
        """Staged partial rows to the home ranks (a streaming kernel on the exchange SMs), then the barrier."""
        lib, p, b = _lib.load(), _lib.ptr, self.buf
        st = torch.cuda.current_stream(self.device).cuda_stream
        self._mark("experts")
        _lib.check(lib.bibo_moe_ep_dedup_push(p(b.pstage), p(b.midx), b.sym_part.ptr_array, p(b.plan), self._n_cap,
                                              self.hidden, self.top_k, self.rank, self.world, self.comm_ctas, st),
                   "bibo_moe_ep_dedup_push")
        self._mark("partial")
        self._barrier(st)
        self._mark("returned")

    def stage_final(self, out: torch.Tensor) -> None:
        """The final sum of the partial rows into ``out`` (current stream; full GPU, HBM-bound)."""
        lib, p, b = _lib.load(), _lib.ptr, self.buf
        st = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(lib.bibo_moe_ep_dedup_final(p(b.part), p(b.topk_idx), p(b.plan[2:]), self._n_last, self._n_cap,
                                               self.hidden, self.n_experts, self.world, self.top_k, 0, p(out), st),
                   "bibo_moe_ep_dedup_final")
        self._mark("sum")
        self.header_host.copy_(b.plan[:4], non_blocking=True)

    def stage_back(self, out: torch.Tensor) -> None:
        """Partial rows to the home ranks, the barrier, and the final sum into ``out`` (current stream)."""
        lib, p, b = _lib.load(), _lib.ptr, self.buf
        st = torch.cuda.current_stream(self.device).cuda_stream
        self._mark("experts")
        _lib.check(lib.bibo_moe_ep_dedup_partial(C.byref(self._owner()), st), "bibo_moe_ep_dedup_partial")
        self._mark("partial")
        self._barrier(st)
        self._mark("returned")
        _lib.check(lib.bibo_moe_ep_dedup_final(p(b.part), p(b.topk_idx), p(b.plan[2:]), self._n_last, self._n_cap,
                                               self.hidden, self.n_experts, self.world, self.top_k, self.comm_ctas,
                                               p(out), st), "bibo_moe_ep_dedup_final")
        self._mark("sum")
        self.header_host.copy_(b.plan[:4], non_blocking=True)

    def _trace_struct(self, n: int):
        if self.trace is None:
            return None
        blocks = _lib.load().bibo_moe_router_blocks(n)
        if getattr(self, "_trace_blocks", None) is None or self._trace_blocks.shape[0] != blocks:
            self._trace_blocks = torch.empty(blocks, _lib.TRACE_WORDS, dtype=torch.float32, device=self.device)
        self._trace_c = _lib.RouterTrace(_lib.ptr(self._trace_blocks), *[_lib.ptr(t) for t in self.trace])
        return C.cast(C.pointer(self._trace_c), C.c_void_p)

    def raise_if_failed(self, wait: bool = False) -> None:
        """RuntimeError if a kernel of an earlier forward left a status word (5 = a cross-rank barrier timed
        out, 100.. = a bounded wait in a kernel gave up); see ``functional.MoEWorkspace.raise_if_failed``."""
        if self.buf is None:
            return
        if wait:
            torch.cuda.current_stream(self.device).synchronize()
        code = int(self.header_host[2])
        if code != 0:
            self.header_host[2] = 0
            self.buf.plan[2:3].zero_()
            raise RuntimeError(f"bibo_b200: an expert-parallel forward reported device status {code} "
                               f"({Fn.STATUS_TEXT.get(code, 'see the plan layout in bibo_moe.h')}); its results and "
                               "those of the calls issued since are invalid")

    def phase_ms(self):
        return {n: self.marks[i - 1][1].elapsed_time(ev) for i, (n, ev) in enumerate(self.marks) if i > 0}

    def status(self) -> int:
        return int(self.buf.plan[2].item()) if self.buf is not None else 0


class PipelinedDedupMoE:
    """The de-duplicated forward on ``chunks`` token slices, pipelined over TWO streams by resource: one stream
    carries everything that uses NVLink (router + dispatch + barrier of every slice, later the push of the
    staged partial rows + barrier), the other the work that wants the whole GPU (rank, plan, permute, grouped
    GEMMs, the partial sums into a local staging buffer, the final sum) of every slice.  Work on one resource runs in slice order and never competes with itself; slice i's GEMMs run
    while slice i+1's rows travel and slice i-1's partial rows return.  Every rank issues the same sequence
    per stream, so the per-slice barriers pair up across ranks.  Results equal the one-slice forward bit for
    bit (tokens are independent)."""

    def __init__(self, weights, top_k: int, group=None, n_tokens: Optional[int] = None, chunks: int = 4,
                 comm_sms: int = 16, gemm_ctas: Optional[int] = None, comm_ctas: Optional[int] = None, **kw):
        """``comm_sms`` SMs are set aside for the exchange kernels (one block of 16 warps each, tagged with shared
        memory so that it never shares an SM with a GEMM CTA); the grouped GEMMs get the rest minus one SM per
        GPC (their 4-CTA clusters need four free SMs in one GPC), rounded down to whole clusters.
        ``gemm_ctas`` / ``comm_ctas`` override the two caps (0 = no cap, no tag)."""
        self.chunks = max(1, int(chunks))
        dev = weights["w_router"].device
        self.device = dev
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        if self.chunks == 1:
            comm_sms = 0                                        # nothing to overlap with: every kernel gets the whole GPU
        if gemm_ctas is None:
            gemm_ctas = (sms - comm_sms - 8) // 4 * 4 if comm_sms > 0 else 0
        if comm_ctas is None:
            comm_ctas = comm_sms
        self.lanes = [DedupExpertParallelMoE(weights, top_k, group, max_ctas=gemm_ctas, comm_ctas=comm_ctas, **kw)
                      for _ in range(self.chunks)]
        # the grouped GEMMs' CTAs are placed first whenever SMs come free; exchange blocks take what is left
        # (the opposite priorities measured the same: 2.22 vs 2.26 ms at 2 GPUs with 4 slices)
        self.link = torch.cuda.Stream(device=dev)
        self.tensor = torch.cuda.Stream(device=dev, priority=-1)
        self.copy_in, self.copy_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        ev = lambda: [torch.cuda.Event() for _ in range(self.chunks)]
        self._received, self._computed, self._returned, self._copied, self._done = ev(), ev(), ev(), ev(), ev()
        if n_tokens is not None:
            for lane, (lo, hi) in zip(self.lanes, self._bounds(n_tokens)):
                lane._allocate(hi - lo)
                lane.add_staging()

    def _bounds(self, n: int):
        per = (n + self.chunks - 1) // self.chunks
        return [(min(c * per, n), min((c + 1) * per, n)) for c in range(self.chunks)]

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, x_host=None, out_host=None) -> torch.Tensor:
        if out is None:
            out = torch.empty_like(x)
        n = x.shape[0]
        if self.chunks == 1:                 # nothing to pipeline: the one-call forward (partial rows stored directly)
            if x_host is not None:
                x.copy_(x_host, non_blocking=True)
            self.lanes[0].forward(x, out)
            if out_host is not None:
                out_host.copy_(out, non_blocking=True)
            return out
        bounds = self._bounds(n)
        for lane, (lo, hi) in zip(self.lanes, bounds):
            if lane.buf is None or hi - lo > lane._n_cap:
                lane._allocate(hi - lo)
                lane.add_staging()
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for st in (self.link, self.tensor, self.copy_in, self.copy_out):
            st.wait_event(start)
        if x_host is not None:
            with torch.cuda.stream(self.copy_in):
                for i, (lo, hi) in enumerate(bounds):
                    x[lo:hi].copy_(x_host[lo:hi], non_blocking=True)
                    self._copied[i].record()
        work = list(enumerate(zip(self.lanes, bounds)))
        with torch.cuda.stream(self.link):
            for i, (lane, (lo, hi)) in work:
                if x_host is not None:
                    self.link.wait_event(self._copied[i])
                lane.stage_home(x[lo:hi])
                self._received[i].record()

        def finish(i):
            lane, (lo, hi) = self.lanes[i], bounds[i]
            with torch.cuda.stream(self.tensor):
                self.tensor.wait_event(self._returned[i])
                lane.stage_final(out[lo:hi])
                self._done[i].record()
            if out_host is not None:
                with torch.cuda.stream(self.copy_out):
                    self.copy_out.wait_event(self._done[i])
                    out_host[lo:hi].copy_(out[lo:hi], non_blocking=True)

        for i, (lane, _) in work:                                # tensor stream: E0 E1 F0 E2 F1 ... F(last)
            with torch.cuda.stream(self.tensor):
                self.tensor.wait_event(self._received[i])
                lane.stage_experts()
                self._computed[i].record()
            with torch.cuda.stream(self.link):
                self.link.wait_event(self._computed[i])
                lane.stage_push()
                self._returned[i].record()
            if i >= 1:
                finish(i - 1)
        finish(len(work) - 1)
        if out_host is not None:
            cur.wait_stream(self.copy_out)
        cur.wait_stream(self.link)
        cur.wait_stream(self.tensor)
        return out

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor, x_dev: torch.Tensor,
                     out_dev: torch.Tensor) -> torch.Tensor:
        """Host-buffer forward (pinned tensors): the copies of the slices run on two more streams under the
        kernels of other slices; waits for the result."""
        self.forward(x_dev, out_dev, x_host=x_host, out_host=out_host)
        torch.cuda.current_stream(self.device).synchronize()
        return out_host

    def status(self) -> int:
        return max(lane.status() for lane in self.lanes)


class PipelinedAllGatherMoE:
    """The forward on ``chunks`` token slices with the exchange on the COPY ENGINES (dense all-gather out, one
    block per peer back; see ``bibo_moe_ep_copy_to_peers`` in the header).  Two streams by resource: the copy
    stream carries the peer copies and the cross-rank barriers of every slice, the tensor stream every kernel
    (router, the owner chain over the gathered rows, the partial sums, the final sum).  No SM moves a row over
    NVLink, so the grouped GEMMs keep the whole GPU while other slices' rows travel.  More bytes than the
    de-duplicated kernels send: ``world - 1`` rows per token each way."""

    def __init__(self, weights, top_k: int, group=None, n_tokens: Optional[int] = None, chunks: int = 4, **kw):
        self.chunks = max(1, int(chunks))
        dev = weights["w_router"].device
        self.device = dev
        self.lanes = [DedupExpertParallelMoE(weights, top_k, group, **kw) for _ in range(self.chunks)]
        self.copy = torch.cuda.Stream(device=dev, priority=-1)
        self.tensor = torch.cuda.Stream(device=dev)
        self.copy_in, self.copy_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        ev = lambda: [torch.cuda.Event() for _ in range(self.chunks)]
        self._routed, self._received, self._computed, self._returned, self._copied, self._done = (ev() for _ in range(6))
        if n_tokens is not None:
            for lane, (lo, hi) in zip(self.lanes, self._bounds(n_tokens)):
                self._prepare(lane, hi - lo)

    def _bounds(self, n: int):
        per = (n + self.chunks - 1) // self.chunks
        return [(min(c * per, n), min((c + 1) * per, n)) for c in range(self.chunks)]

    @staticmethod
    def _prepare(lane, n: int) -> None:
        """Buffers of the de-duplicated path plus the gathered raw top-k table (peer-mapped) and the local staging
        buffer of the partial rows; the partial kernel's destination table points into the staging buffer for
        every other home rank and into this rank's own ``part`` for its own tokens."""
        lane._allocate(n)
        b, dev = lane.buf, lane.device
        nv = lane.world * lane._n_cap
        b.sym_raw = _Symmetric((nv, lane.top_k), torch.int32, dev, lane.group)
        b.sym_raw.tensor.fill_(-1)
        b.topk_idx.fill_(-1)
        b.pstage = torch.empty(nv, lane.hidden, dtype=torch.bfloat16, device=dev)
        row = lane._n_cap * lane.hidden * 2
        table = [b.pstage.data_ptr() + (s_ - lane.rank) * row for s_ in range(lane.world)]
        table[lane.rank] = b.part.data_ptr()
        b.stage_table = (C.c_void_p * lane.world)(*table)
        b.n_routed = lane._n_cap
        torch.cuda.synchronize(dev)
        dist.barrier(lane.group)

    # ---- per-slice stages ---------------------------------------------------------------------------------
    @staticmethod
    def _send_rows(lane, x) -> None:
        b, st = lane.buf, torch.cuda.current_stream(lane.device).cuda_stream
        row = lane.hidden * 2
        _lib.check(_lib.load().bibo_moe_ep_copy_to_peers(b.sym_xu.ptr_array, lane.rank * lane._n_cap * row, _lib.ptr(x), 0,
                                                         x.shape[0] * row, lane.rank, lane.world, 1, st),
                   "bibo_moe_ep_copy_to_peers")

    @staticmethod
    def _route(lane, x) -> None:
        lib, p, b = _lib.load(), _lib.ptr, lane.buf
        n, st = x.shape[0], torch.cuda.current_stream(lane.device).cuda_stream
        lane.raise_if_failed()
        if n < b.n_routed:
            b.topk_idx[n:].fill_(-1)              # slots past this call's tokens: "no such token"
        b.n_routed = n
        if n:
            _lib.check(lib.bibo_moe_router_fwd(p(x), p(lane.w_router), p(lane.bias), None, n, lane.hidden, lane.n_experts,
                                               lane.top_k, Fn.norm_code(lane.norm_mode), float(lane.scale), _lib.BF16, None,
                                               p(b.topk_idx), p(b.topk_w), p(b.slot_rank_home), p(b.block_counts_home),
                                               p(b.plan[2:]), st), "bibo_moe_router_fwd")
        lane._n_last = n

    @staticmethod
    def _send_records(lane) -> None:
        lib, p, b = _lib.load(), _lib.ptr, lane.buf
        st = torch.cuda.current_stream(lane.device).cuda_stream
        block = lane._n_cap * lane.top_k * 4
        for sym, src in ((b.sym_raw, b.topk_idx), (b.sym_mw, b.topk_w)):
            _lib.check(lib.bibo_moe_ep_copy_to_peers(sym.ptr_array, lane.rank * block, p(src), 0, block, lane.rank,
                                                     lane.world, 1, st), "bibo_moe_ep_copy_to_peers")
        lane._barrier(st)

    @staticmethod
    def _experts(lane) -> None:
        lib, p, b = _lib.load(), _lib.ptr, lane.buf
        st = torch.cuda.current_stream(lane.device).cuda_stream
        nv = lane.world * lane._n_cap
        _lib.check(lib.bibo_moe_ep_localize(p(b.sym_raw.tensor), nv, lane.top_k, lane.n_experts, lane.rank, lane.world,
                                            p(b.midx), st), "bibo_moe_ep_localize")
        owner = b.owner_args(lane.rank, lane.hidden, lane.inter, lane.n_experts, lane.gate_up, lane.down, lane.theta,
                             b.stage_table, lane.max_ctas, 0)
        _lib.check(lib.bibo_moe_ep_dedup_owner(C.byref(owner), st), "bibo_moe_ep_dedup_owner")

    @staticmethod
    def _return(lane) -> None:
        b, st = lane.buf, torch.cuda.current_stream(lane.device).cuda_stream
        block = lane._n_cap * lane.hidden * 2
        _lib.check(_lib.load().bibo_moe_ep_copy_to_peers(b.sym_part.ptr_array, lane.rank * block, _lib.ptr(b.pstage), block,
                                                         block, lane.rank, lane.world, 0, st), "bibo_moe_ep_copy_to_peers")
        lane._barrier(st)

    @staticmethod
    def _final(lane, out) -> None:
        lib, p, b = _lib.load(), _lib.ptr, lane.buf
        st = torch.cuda.current_stream(lane.device).cuda_stream
        _lib.check(lib.bibo_moe_ep_dedup_final(p(b.part), p(b.topk_idx), p(b.plan[2:]), lane._n_last, lane._n_cap,
                                               lane.hidden, lane.n_experts, lane.world, lane.top_k, 0, p(out), st),
                   "bibo_moe_ep_dedup_final")
        lane.header_host.copy_(b.plan[:4], non_blocking=True)

    @staticmethod
    def _mark(lane, name: str, stream) -> None:
        if lane.profile:
            if name == "start":
                lane.marks = []
            e = torch.cuda.Event(enable_timing=True)
            e.record(stream)
            lane.marks.append((name, e))

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, x_host=None, out_host=None) -> torch.Tensor:
        if out is None:
            out = torch.empty_like(x)
        bounds = self._bounds(x.shape[0])
        for lane, (lo, hi) in zip(self.lanes, bounds):
            if lane.buf is None or hi - lo > lane._n_cap or not hasattr(lane.buf, "pstage"):
                self._prepare(lane, hi - lo)
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for st in (self.copy, self.tensor, self.copy_in, self.copy_out):
            st.wait_event(start)
        work = list(enumerate(zip(self.lanes, bounds)))
        if x_host is not None:
            with torch.cuda.stream(self.copy_in):
                for i, (lane, (lo, hi)) in work:
                    x[lo:hi].copy_(x_host[lo:hi], non_blocking=True)
                    self._copied[i].record()
        for i, (lane, (lo, hi)) in work:
            with torch.cuda.stream(self.copy):                   # the rows need no routing: they leave at once
                if x_host is not None:
                    self.copy.wait_event(self._copied[i])
                self._mark(lane, "start", self.copy)
                self._send_rows(lane, x[lo:hi])
            with torch.cuda.stream(self.tensor):
                if x_host is not None:
                    self.tensor.wait_event(self._copied[i])
                self._route(lane, x[lo:hi])
                self._routed[i].record()
                self._mark(lane, "route", self.tensor)
            with torch.cuda.stream(self.copy):
                self.copy.wait_event(self._routed[i])
                self._mark(lane, "dispatch", self.copy)
                self._send_records(lane)
                self._received[i].record()
                self._mark(lane, "received", self.copy)
        for i, (lane, (lo, hi)) in work:                         # E0 R0 | E1 R1 F0 | E2 R2 F1 | ... | F(last)
            with torch.cuda.stream(self.tensor):
                self.tensor.wait_event(self._received[i])
                self._experts(lane)
                self._computed[i].record()
                self._mark(lane, "experts", self.tensor)
            with torch.cuda.stream(self.copy):
                self.copy.wait_event(self._computed[i])
                self._return(lane)
                self._returned[i].record()
                self._mark(lane, "partial", self.copy)
                self._mark(lane, "returned", self.copy)
            if i >= 1:
                self._finish(i - 1, bounds[i - 1], out, out_host)
        self._finish(len(work) - 1, bounds[-1], out, out_host)
        if out_host is not None:
            cur.wait_stream(self.copy_out)
        cur.wait_stream(self.copy)
        cur.wait_stream(self.tensor)
        return out

    def _finish(self, i, bound, out, out_host) -> None:
        lane, (lo, hi) = self.lanes[i], bound
        with torch.cuda.stream(self.tensor):
            self.tensor.wait_event(self._returned[i])
            self._final(lane, out[lo:hi])
            self._done[i].record()
            self._mark(lane, "sum", self.tensor)
        if out_host is not None:
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(self._done[i])
                out_host[lo:hi].copy_(out[lo:hi], non_blocking=True)

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor, x_dev: torch.Tensor,
                     out_dev: torch.Tensor) -> torch.Tensor:
        self.forward(x_dev, out_dev, x_host=x_host, out_host=out_host)
        torch.cuda.current_stream(self.device).synchronize()
        return out_host

    def status(self) -> int:
        return max(lane.status() for lane in self.lanes)


class PipelinedExpertParallelMoE:
    """The expert-parallel forward on ``chunks`` token slices, each on its own CUDA stream.

    A slice is a complete, independent forward (tokens are independent), with its own peer buffers,
    plans and barrier flags.  Running the slices on separate streams lets the GPU overlap the NVLink
    phases of one slice (dispatch stores, combine loads) with the grouped GEMMs of another; the GEMM
    grids are capped at ``148 - comm_sms`` CTAs so the exchange kernels always find free SMs.
    Every rank issues the same sequence of launches per stream, so the per-slice barriers and the NCCL
    all-gathers pair up across ranks in the same order.
    """

    def __init__(self, weights, top_k: int, group=None, n_tokens: Optional[int] = None, chunks: int = 2,
                 comm_sms: int = 20, dedup: bool = False, gemm_ctas: Optional[int] = None,
                 comm_ctas: Optional[int] = None, **kw):
        """``dedup``: lanes use the de-duplicated exchange (``DedupExpertParallelMoE``, forward only).
        ``gemm_ctas`` / ``comm_ctas`` override the grid caps derived from ``comm_sms`` (0 = no cap)."""
        self.chunks = max(1, int(chunks))
        dev = weights["w_router"].device
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        sm_exchange = self.chunks > 1 and not kw.get("dma", False)   # copy-engine exchange needs no SMs
        max_ctas = max(8, sms - comm_sms) if sm_exchange else 0
        c_ctas = comm_sms * 4 if sm_exchange else 0             # 4 resident 8-warp blocks per exchange SM
        if gemm_ctas is not None:
            max_ctas = int(gemm_ctas)
        if comm_ctas is not None:
            c_ctas = int(comm_ctas)
        cls = DedupExpertParallelMoE if dedup else ExpertParallelMoE
        self.lanes = [cls(weights, top_k, group, max_ctas=max_ctas, comm_ctas=c_ctas, **kw)
                      for _ in range(self.chunks)]
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(self.chunks)]
        self.device = dev
        if n_tokens is not None:
            for lane, (lo, hi) in zip(self.lanes, self._bounds(n_tokens)):
                lane._allocate(hi - lo)

    def _bounds(self, n: int):
        per = (n + self.chunks - 1) // self.chunks
        return [(min(c * per, n), min((c + 1) * per, n)) for c in range(self.chunks)]

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty_like(x)
        if self.chunks == 1:
            return self.lanes[0].forward(x, out)
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        self._run_lanes(lambda lo, hi: (x[lo:hi], out[lo:hi]), x.shape[0], start, None)
        for st in self.streams:
            cur.wait_stream(st)
        return out

    def _run_lanes(self, views, n: int, start, after) -> None:
        """Issue every slice on its stream.  Copy-engine lanes are issued in two passes (everything up to
        the host's read of the histogram table for all slices, then the rest), so that no slice's router
        waits behind another slice's host round trip.  ``after(lane_index, lo, hi)`` runs on the slice's
        stream once its forward is issued."""
        work = [(i, lane, st, lo, hi) for i, (lane, st, (lo, hi)) in
                enumerate(zip(self.lanes, self.streams, self._bounds(n))) if hi > lo]
        two_pass = all(lane.dma for lane in self.lanes)
        for i, lane, st, lo, hi in work:
            st.wait_event(start)
            with torch.cuda.stream(st):
                xs, os_ = views(lo, hi)
                lane.forward(xs, os_, phase=1 if two_pass else 0)
                if not two_pass and after is not None:
                    after(i, lo, hi)
        if two_pass:
            for i, lane, st, lo, hi in work:
                with torch.cuda.stream(st):
                    lane.finish()
                    if after is not None:
                        after(i, lo, hi)

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor, x_dev: torch.Tensor,
                     out_dev: torch.Tensor) -> torch.Tensor:
        """Host-buffer forward: every slice copies its tokens in, runs and copies its result out on its
        own stream, so the copies of one slice overlap the kernels of another (pinned host tensors);
        waits for the result."""
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        if self.chunks == 1:
            x_dev.copy_(x_host, non_blocking=True)
            self.lanes[0].forward(x_dev, out_dev)
            out_host.copy_(out_dev, non_blocking=True)
            cur.synchronize()
            return out_host

        def views(lo, hi):
            x_dev[lo:hi].copy_(x_host[lo:hi], non_blocking=True)      # on the slice's stream, before its router
            return x_dev[lo:hi], out_dev[lo:hi]

        self._run_lanes(views, x_host.shape[0], start,
                        lambda i, lo, hi: out_host[lo:hi].copy_(out_dev[lo:hi], non_blocking=True))
        for st in self.streams:
            st.synchronize()
        return out_host

    def status(self) -> int:
        return max(lane.status() for lane in self.lanes)


# ---- module interface --------------------------------------------------------------------------------
class _EPBlockFunction(torch.autograd.Function):
    """Expert-parallel forward / backward as one autograd node (bibo_moe_ep_forward / _backward)."""

    @staticmethod
    def forward(ctx, x, w_router, gate_up, down, theta, layer):
        runner = layer._runner
        out = runner.forward(x, training=True)
        ctx.layer = layer
        return out

    @staticmethod
    def backward(ctx, dout):
        layer = ctx.layer
        dx, d_wr, d_gu, d_dn, d_th = layer._runner.backward(dout.contiguous())
        if layer.reduce_router_grad and layer._runner.world > 1:
            # the router is replicated and the tokens are data-parallel: its gradient is the sum over ranks
            acc = d_wr.float()
            dist.all_reduce(acc, group=layer.group)
            d_wr = acc.to(d_wr.dtype)
        return dx, d_wr, d_gu, d_dn, d_th.to(layer.radial_theta.dtype), None


class ExpertParallelMoELayer(torch.nn.Module):
    """``BiBoMoELayer`` with the experts sharded over a process group (one rank per GPU of one box).

    Same ``forward([B,S,H]) -> [B,S,H]`` and balancer semantics as the single-GPU layer
    (src/modeling/ffn/moe.py:104-183); the reference itself has no expert parallelism.  Every rank keeps the
    full router (``gate``, replicated) and the E/world experts ``[rank*E/world, (rank+1)*E/world)`` as
    ``gate_up_proj [E/world, 2I, H]``, ``down_proj [E/world, H, I]``, ``radial_theta [E/world]``; tokens stay
    on their rank.  Training runs through one autograd node; the router weight gradient is all-reduced over
    the group (``reduce_router_grad``), expert gradients stay with their owner.  bf16, no ±Identity
    experts, no shared expert.
    """

    def __init__(self, config, group=None, capacity_factor: Optional[float] = None, reduce_router_grad: bool = True):
        super().__init__()
        from .moe import BiBoMoERouter, _cfg
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        e = config.num_routed_experts
        n_special = int(_cfg(config, "num_pos_identity_experts", 0)) + int(_cfg(config, "num_neg_identity_experts", 0))
        if n_special == 0 and _cfg(config, "special_expert_pairs", 0):
            n_special = 2 * int(config.special_expert_pairs)
        if n_special or _cfg(config, "use_shared_expert", False):
            raise NotImplementedError("ExpertParallelMoELayer: identity and shared experts are not sharded")
        if e % self.world:
            raise RuntimeError(f"{e} experts do not shard evenly over {self.world} ranks")
        self.num_routed_experts, self.el = e, e // self.world
        h, i = config.hidden_size, config.moe_intermediate_size
        std = float(_cfg(config, "initializer_range", 0.02))
        self.gate = BiBoMoERouter(config)
        self.gate_up_proj = torch.nn.Parameter(torch.randn(self.el, 2 * i, h) * std)
        self.down_proj = torch.nn.Parameter(torch.randn(self.el, h, i) * std)
        self.radial_theta = torch.nn.Parameter(torch.zeros(self.el))
        self.register_buffer("accumulated_tpe", torch.zeros(e, dtype=torch.float))
        self.bias_update_factor = _cfg(config, "bias_update_factor", 0.4)
        self.bias_update_threshold = _cfg(config, "bias_update_threshold", 8000)
        self._fwd_step, self._update_every = 0, None
        self.capacity_factor, self.reduce_router_grad = capacity_factor, reduce_router_grad
        self._runner, self._runner_key = None, None

    @classmethod
    def from_full_layer(cls, layer, config, group=None, **kw):
        """Shard a single-GPU ``BiBoMoELayer`` (or the reference's) into this rank's slice."""
        ep = cls(config, group, **kw)
        lo, hi = ep.rank * ep.el, (ep.rank + 1) * ep.el
        with torch.no_grad():
            ep.gate.gate_proj.weight.copy_(layer.gate.gate_proj.weight)
            ep.gate.bias.copy_(layer.gate.bias)
            ep.gate_up_proj.copy_(layer.experts.gate_up_proj[lo:hi])
            ep.down_proj.copy_(layer.experts.down_proj[lo:hi])
            ep.radial_theta.copy_(layer.experts.radial_theta[lo:hi])
        return ep

    @torch.no_grad()
    def update_bias(self, tokens_per_expert: torch.Tensor):
        """src/modeling/ffn/moe.py:131-137 (proportional bias update)."""
        if self.bias_update_factor <= 0:
            return
        share = tokens_per_expert.detach().float()
        share = share / share.sum().clamp_min(1.0)
        self.gate.bias.add_(self.bias_update_factor * (share.mean() - share))

    def _get_runner(self) -> ExpertParallelMoE:
        w = dict(w_router=self.gate.gate_proj.weight.data, bias=self.gate.bias.data, gate_up_proj=self.gate_up_proj.data,
                 down_proj=self.down_proj.data, radial_theta=self.radial_theta.data)
        key = tuple(t.data_ptr() for t in w.values())
        if self._runner is None or key != self._runner_key:     # first call, or the parameters were moved / cast
            self._runner = ExpertParallelMoE(w, self.gate.top_k, self.group, norm_mode=self.gate.norm_topk_prob,
                                             scale=float(getattr(self.gate, "routed_scaling_factor", 1.0)),
                                             capacity_factor=self.capacity_factor)
            self._runner_key = key
        # the runner keeps fp32 copies of bias / theta when the parameters are not fp32: refresh them
        r = self._runner
        if r.bias.data_ptr() != self.gate.bias.data_ptr():
            r.bias.copy_(self.gate.bias.data)
        if r.theta.data_ptr() != self.radial_theta.data_ptr():
            r.theta.copy_(self.radial_theta.data)
        return r

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        from .moe import _balance_from_counts
        bsz, seq_len, hidden = hidden_states.shape
        flat = hidden_states.reshape(-1, hidden).contiguous()
        runner = self._get_runner()
        params = (self.gate.gate_proj.weight, self.gate_up_proj, self.down_proj, self.radial_theta)
        # routing diagnostics of this rank's tokens, produced by the router / plan kernels (bibo_b200.RouterTrace,
        # gate._probe_gap), as in the single-GPU layer
        tracer = getattr(self, "_router_trace", None)
        trace = tracer.buffers(self) if tracer is not None else None
        want_gap = self.gate._probe_gap and self.gate.top_k < self.gate.num_routed_experts
        if want_gap:
            gap = torch.empty(1, dtype=torch.float32, device=flat.device)
            trace = (trace[0], trace[1], gap) if trace is not None else (None, None, gap)
        runner.trace = trace
        if torch.is_grad_enabled() and (flat.requires_grad or any(p.requires_grad for p in params)):
            out = _EPBlockFunction.apply(flat, *params, self)
        else:
            out = runner.forward(flat)
        runner.trace = None
        if want_gap:
            self.gate.boundary_gap = gap[0]
        if self.training and self.bias_update_factor > 0:
            tpe = _balance_from_counts(self, runner._counts, flat.shape[0])   # all-reduces accumulated_tpe
            if tpe is not None:
                self.update_bias(tpe)
        return out.view(bsz, seq_len, hidden)
