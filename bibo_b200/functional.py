"""Host-side driver of the kernel chain: buffers, launches, and the stage-by-stage entry points.

All arithmetic happens in libbibo_moe.so.  This module only allocates torch tensors (outputs and
one workspace per shape) and passes their raw pointers through ctypes.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}
_NORMS = {"sum": _lib.NORM_SUM, True: _lib.NORM_SUM, "softmax": _lib.NORM_SOFTMAX,
          False: _lib.NORM_RAW, None: _lib.NORM_RAW}


def dtype_code(dt: torch.dtype) -> int:
    if dt not in _DTYPES:
        raise RuntimeError(f"bibo_b200 kernels take float32 or bfloat16 tensors, got {dt}")
    return _DTYPES[dt]


def norm_code(mode) -> int:
    if mode not in _NORMS:
        raise RuntimeError(f"unknown norm_topk_prob {mode!r}")
    return _NORMS[mode]


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _need_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"{name} is on {t.device}: the bibo_b200 MoE block runs only as CUDA kernels "
            "(there is no CPU implementation)")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


@dataclass(frozen=True)
class Geometry:
    n_tokens: int
    hidden: int
    inter: int
    n_experts: int
    n_glu: int
    n_pos: int
    top_k: int
    dtype: torch.dtype

    @property
    def rows_cap(self) -> int:
        return int(_lib.load().bibo_moe_rows_cap(self.n_tokens, self.top_k, self.n_glu))

    @property
    def router_blocks(self) -> int:
        return int(_lib.load().bibo_moe_router_blocks(self.n_tokens))

    @property
    def plan_words(self) -> int:
        return int(_lib.load().bibo_moe_plan_words(self.n_tokens, self.top_k, self.n_experts, self.n_glu))


class MoEWorkspace:
    """Every intermediate buffer of one forward, allocated once per (device, geometry)."""

    def __init__(self, geo: Geometry, device, keep_logits: bool = False, keep_gate_up: bool = True):
        n, k, e = geo.n_tokens, geo.top_k, geo.n_experts
        rows = geo.rows_cap
        i32 = dict(dtype=torch.int32, device=device)
        self.geo = geo
        self.topk_idx = torch.empty(n, k, **i32)
        self.topk_w = torch.empty(n, k, dtype=torch.float32, device=device)
        self.slot_rank = torch.empty(n, k, **i32)
        self.block_counts = torch.empty(geo.router_blocks, e, **i32)
        self.plan = torch.zeros(geo.plan_words, **i32)
        self.slot_row = torch.empty(n, k, **i32)
        self.row_token = torch.empty(rows, **i32)
        self.xp = torch.empty(rows, geo.hidden, dtype=geo.dtype, device=device)
        self.h = torch.empty(rows, geo.inter, dtype=geo.dtype, device=device)
        self.y = torch.empty(rows, geo.hidden, dtype=geo.dtype, device=device)
        fused = bool(_lib.load().bibo_moe_gemm1_is_fused(geo.hidden, geo.inter, dtype_code(geo.dtype)))
        keep_gate_up = keep_gate_up or not fused   # the two-kernel path always needs the buffer
        self.gate_up = (torch.empty(rows, 2 * geo.inter, dtype=geo.dtype, device=device)
                        if keep_gate_up else None)
        self.rnorm = torch.empty(rows, dtype=torch.float32, device=device) if keep_gate_up else None
        self.logits = torch.empty(n, e, dtype=torch.float32, device=device) if keep_logits else None
        self.status = torch.zeros(1, **i32)
        # host copy of the plan header {n_tiles, rows, status, n_pairs}: refreshed by an asynchronous 16-byte
        # copy behind every call, looked at (without waiting) before the next one -- see raise_if_failed
        self.header_host = torch.zeros(4, dtype=torch.int32).pin_memory() if torch.device(device).type == "cuda" else None
        self.stage_events = None      # optional list of 7 torch.cuda.Event(enable_timing=True)
        self._stage_event_array = None
        self.trace_blocks = None      # [router_blocks, 8] fp32 scratch of the router diagnostics, on first use
        self._trace_struct = None

    def c_struct(self) -> _lib.Workspace:
        p = _lib.ptr
        ev = None
        if self.stage_events is not None:
            # torch creates the CUDA event lazily on first record
            for e in self.stage_events:
                if e.cuda_event == 0:
                    e.record()
            self._stage_event_array = (C.c_void_p * 7)(*[e.cuda_event for e in self.stage_events])
            ev = C.cast(self._stage_event_array, C.c_void_p)
        tr = None
        trace = getattr(self, "trace", None)       # (acc, counts, gap) tensors or None each, for this call only
        if trace is not None:
            if self.trace_blocks is None:
                self.trace_blocks = torch.empty(self.geo.router_blocks, _lib.TRACE_WORDS, dtype=torch.float32,
                                                device=self.plan.device)
            self._trace_struct = _lib.RouterTrace(p(self.trace_blocks), *[p(t) for t in trace])
            tr = C.cast(C.pointer(self._trace_struct), C.c_void_p)
        return _lib.Workspace(p(self.topk_idx), p(self.topk_w), p(self.slot_rank), p(self.block_counts),
                              p(self.plan), p(self.slot_row), p(self.row_token), p(self.xp), p(self.h),
                              p(self.y), p(self.gate_up), p(self.rnorm), p(self.logits), ev,
                              p(getattr(self, "addend", None)), tr)

    def post_status(self) -> None:
        """Enqueue the copy of the plan header into pinned host memory behind the kernels just launched."""
        if self.header_host is not None:
            self.header_host.copy_(self.plan[:4], non_blocking=True)

    def raise_if_failed(self, wait: bool = False) -> None:
        """Raise RuntimeError if a kernel of an EARLIER call on this workspace left a non-zero status word
        (a bounded wait that gave up, a routing index out of range, ...).  Without ``wait`` nothing is
        synchronised: the check sees what has reached the host so far, so a failure is reported at the
        latest by the call after the one in which it became visible (kernels skip their work while the word
        is non-zero).  The word is cleared once it has been reported."""
        if self.header_host is None:
            return
        if wait:
            torch.cuda.current_stream(self.plan.device).synchronize()
        code = int(self.header_host[2])
        if code != 0:
            self.header_host[2] = 0
            self.plan[2:3].zero_()
            raise RuntimeError(f"bibo_b200: a kernel of an earlier call reported device status {code} "
                               f"({STATUS_TEXT.get(code, 'see the plan layout in bibo_moe.h')}); its results and those "
                               "of the calls issued since are invalid")

    def enable_stage_timing(self) -> None:
        """Ask bibo_moe_forward to record an event around every stage (see stage_ms)."""
        self.stage_events = [torch.cuda.Event(enable_timing=True) for _ in range(7)]

    STAGES = ("router", "plan", "permute", "gemm1_radial", "gemm2", "combine")

    def stage_ms(self):
        """Per-stage device time of the last forward (call after a synchronize)."""
        ev = self.stage_events
        return {n: ev[i].elapsed_time(ev[i + 1]) for i, n in enumerate(self.STAGES)}

    # views into the plan buffer
    def counts(self) -> torch.Tensor:
        o = int(_lib.load().bibo_moe_plan_off_counts())
        return self.plan[o:o + self.geo.n_experts]

    def expert_off(self) -> torch.Tensor:
        o = int(_lib.load().bibo_moe_plan_off_expert_off(self.geo.n_experts))
        return self.plan[o:o + self.geo.n_glu + 1]

    def tiles(self) -> torch.Tensor:
        g = self.geo
        o = int(_lib.load().bibo_moe_plan_off_tiles(g.n_tokens, g.n_experts, g.n_glu))
        n_rec = self.geo.rows_cap // _lib.TILE_M
        return self.plan[o:o + 4 * n_rec].view(-1, 4)


STATUS_TEXT = {
    1: "per-expert histogram total exceeds tokens x top_k", 2: "an expert index is out of range",
    3: "one expert appears twice in a token", 4: "an expert-parallel receive buffer would overflow",
    5: "a cross-rank barrier timed out", 100: "down kernel: a bounded wait gave up",
    101: "gate/up kernel: a bounded wait gave up", 102: "router kernel: a bounded wait gave up",
    104: "gate/up CTA-pair kernel: a bounded wait gave up (exchange or row gather)",
    110: "backward dX kernel: a bounded wait gave up", 111: "backward dW kernel: a bounded wait gave up",
}

_WS_CACHE: Dict[Tuple, MoEWorkspace] = {}


def get_workspace(geo: Geometry, device, keep_logits=False, keep_gate_up=True, fresh=False) -> MoEWorkspace:
    key = (torch.device(device), geo, keep_logits, keep_gate_up)
    if fresh:
        return MoEWorkspace(geo, device, keep_logits, keep_gate_up)
    ws = _WS_CACHE.get(key)
    if ws is None:
        if len(_WS_CACHE) > 8:
            _WS_CACHE.clear()
        ws = _WS_CACHE[key] = MoEWorkspace(geo, device, keep_logits, keep_gate_up)
    return ws


def _shape(geo: Geometry, norm_mode, scale: float, zero_padding: bool, gather: bool = False) -> _lib.Shape:
    """zero_padding field: bit 0 = zero-fill padding rows, bit 1 = the gate/up kernel gathers its own rows."""
    return _lib.Shape(geo.n_tokens, geo.hidden, geo.inter, geo.n_experts, geo.n_glu, geo.n_pos, geo.top_k,
                      norm_code(norm_mode), dtype_code(geo.dtype), float(scale),
                      int(bool(zero_padding)) | (2 if gather else 0))


# ---------------------------------------------------------------------------------------------------
# stage entry points (each is one C-ABI call)
# ---------------------------------------------------------------------------------------------------
def router_forward(x: Optional[torch.Tensor], w_router: Optional[torch.Tensor], bias: torch.Tensor,
                   top_k: int, norm_mode="sum", scale: float = 1.0, ws: Optional[MoEWorkspace] = None,
                   logits_in: Optional[torch.Tensor] = None, want_logits: bool = False):
    """K1.  Returns (topk_idx int32 [N,k] ascending, topk_w fp32 [N,k], slot_rank, block_counts, logits|None)."""
    lib = _lib.load()
    src = x if logits_in is None else logits_in
    _need_cuda(src, "router input")
    n = src.shape[0]
    e = bias.shape[0]
    dev = src.device
    hidden = x.shape[1] if x is not None else 0
    dt = dtype_code(x.dtype) if x is not None else _lib.F32
    if x is not None and w_router is not None and w_router.dtype != x.dtype:
        raise RuntimeError(f"router weight dtype {w_router.dtype} != activation dtype {x.dtype}")
    if ws is None:
        i32 = dict(dtype=torch.int32, device=dev)
        idx = torch.empty(n, top_k, **i32)
        w = torch.empty(n, top_k, dtype=torch.float32, device=dev)
        rank = torch.empty(n, top_k, **i32)
        bc = torch.empty(int(lib.bibo_moe_router_blocks(n)), e, **i32)
    else:
        idx, w, rank, bc = ws.topk_idx, ws.topk_w, ws.slot_rank, ws.block_counts
    logits = torch.empty(n, e, dtype=torch.float32, device=dev) if want_logits else None
    bias32 = bias if bias.dtype == torch.float32 else bias.float()
    rc = lib.bibo_moe_router_fwd(_lib.ptr(x), _lib.ptr(w_router), _lib.ptr(bias32), _lib.ptr(logits_in), n, hidden,
                                 e, top_k, norm_code(norm_mode), float(scale), dt, _lib.ptr(logits),
                                 _lib.ptr(idx), _lib.ptr(w), _lib.ptr(rank), _lib.ptr(bc),
                                 _lib.ptr(ws.plan[2:]) if ws is not None else None, _stream(dev))
    _lib.check(rc, "bibo_moe_router_fwd")
    return idx, w, rank, bc, logits


def launch_count() -> int:
    return int(_lib.load().bibo_moe_launch_count())


def moe_forward(x: torch.Tensor, w_router: torch.Tensor, bias: torch.Tensor, gate_up_proj: torch.Tensor,
                down_proj: torch.Tensor, theta: torch.Tensor, top_k: int, norm_mode="sum", scale: float = 1.0,
                n_pos: int = 0, n_neg: int = 0, ws: Optional[MoEWorkspace] = None, out: Optional[torch.Tensor] = None,
                zero_padding: bool = False, keep_logits: bool = False,
                addend: Optional[torch.Tensor] = None,
                trace: Optional[Tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]] = None,
                gather_in_gemm: bool = False) -> Tuple[torch.Tensor, MoEWorkspace]:
    """The whole block on flat tokens x [N,H]: one call of bibo_moe_forward.  Returns (out, workspace).
    ``gather_in_gemm`` lets the gate/up kernel gather its own rows where it can (bf16, intermediate 256 / 512)
    instead of running the permute as a kernel of its own: same bits, measured slightly slower.
    ``addend`` [N,H] (the shared expert's output) is added in the combine kernel.
    ``trace`` = (acc [8], counts [E], gap [1]) fp32 device tensors, each optional: the router and plan
    kernels fold this call's routing diagnostics into them (see bibo_moe_router_trace in the header)."""
    lib = _lib.load()
    for name, t in (("x", x), ("w_router", w_router), ("bias", bias), ("gate_up_proj", gate_up_proj),
                    ("down_proj", down_proj), ("radial_theta", theta)):
        _need_cuda(t, name)
    n, hidden = x.shape
    n_glu, two_i, _ = gate_up_proj.shape
    geo = Geometry(n, hidden, two_i // 2, w_router.shape[0], n_glu, n_pos, top_k, x.dtype)
    if geo.n_experts != n_glu + n_pos + n_neg:
        raise RuntimeError(f"{geo.n_experts} routed experts != {n_glu} GLU + {n_pos} + {n_neg} identity experts")
    for name, t in (("w_router", w_router), ("gate_up_proj", gate_up_proj), ("down_proj", down_proj)):
        if t.dtype != x.dtype:
            raise RuntimeError(f"{name} dtype {t.dtype} != activation dtype {x.dtype}")
    if ws is None:
        ws = get_workspace(geo, x.device, keep_logits=keep_logits)
    if out is None:
        out = torch.empty_like(x)
    if n == 0:
        return out, ws
    bias32 = bias if bias.dtype == torch.float32 else bias.float()
    theta32 = theta if theta.dtype == torch.float32 else theta.float()
    shape = _shape(geo, norm_mode, scale, zero_padding, gather_in_gemm)
    if addend is not None and (addend.shape != x.shape or addend.dtype != x.dtype or not addend.is_contiguous()):
        raise RuntimeError("addend must be a contiguous tensor of the activations' shape and dtype")
    if trace is not None:
        for t, words in zip(trace, (_lib.TRACE_WORDS, geo.n_experts, 1)):
            if t is not None and (t.dtype != torch.float32 or t.numel() != words or t.device != x.device
                                  or not t.is_contiguous()):
                raise RuntimeError("trace tensors must be contiguous fp32 device tensors of 8 / n_experts / 1 elements")
    ws.raise_if_failed()
    ws.addend, ws.trace = addend, trace
    cws = ws.c_struct()
    ws.addend = ws.trace = None
    rc = lib.bibo_moe_forward(C.byref(shape), _lib.ptr(x), _lib.ptr(w_router), _lib.ptr(bias32),
                              _lib.ptr(gate_up_proj), _lib.ptr(down_proj), _lib.ptr(theta32), C.byref(cws),
                              _lib.ptr(out), _stream(x.device))
    _lib.check(rc, "bibo_moe_forward")
    ws.post_status()
    return out, ws


def ffn_supported(hidden: int, inter: int, n_experts: int, top_k: int) -> bool:
    geo = Geometry(1, hidden, inter, n_experts, n_experts, 0, top_k, torch.bfloat16)
    shape = _shape(geo, "sum", 1.0, False)
    return bool(_lib.load().bibo_moe_ffn_supported(C.byref(shape)))


def ffn_forward(h: torch.Tensor, norm_weight: torch.Tensor, eps: float, w_router: torch.Tensor, bias: torch.Tensor,
                gate_up_proj: torch.Tensor, down_proj: torch.Tensor, theta: torch.Tensor, top_k: int, norm_mode="sum",
                scale: float = 1.0, ws: Optional[MoEWorkspace] = None, out: Optional[torch.Tensor] = None,
                keep_logits: bool = False, trace=None, n_pos: int = 0, n_neg: int = 0,
                ) -> Tuple[torch.Tensor, MoEWorkspace]:
    """out = h + block(rmsnorm(h)) on flat bf16 rows h [N,H] with the norm folded into the router's and the
    permute's loads (bibo_moe_ffn_forward).  The per-row rstd is left in ``ws.rstd``.  The router weight with
    the norm weight folded in lives in ``ws.w_fold`` and is recomputed only when one of the two tensors
    changed (another tensor, or an in-place update: torch's version counter)."""
    lib = _lib.load()
    for name, t in (("hidden_states", h), ("norm weight", norm_weight), ("w_router", w_router), ("bias", bias),
                    ("gate_up_proj", gate_up_proj), ("down_proj", down_proj), ("radial_theta", theta)):
        _need_cuda(t, name)
    n, hidden = h.shape
    n_glu, two_i, _ = gate_up_proj.shape
    geo = Geometry(n, hidden, two_i // 2, w_router.shape[0], n_glu, n_pos, top_k, h.dtype)
    if geo.n_experts != n_glu + n_pos + n_neg:
        raise RuntimeError(f"{geo.n_experts} routed experts != {n_glu} GLU + {n_pos} + {n_neg} identity experts")
    for name, t in (("norm weight", norm_weight), ("w_router", w_router), ("gate_up_proj", gate_up_proj),
                    ("down_proj", down_proj)):
        if t.dtype != torch.bfloat16 or h.dtype != torch.bfloat16:
            raise RuntimeError(f"ffn_forward is bf16 only ({name} is {t.dtype}, activations {h.dtype})")
    if not h.is_contiguous() or not norm_weight.is_contiguous():
        raise RuntimeError("ffn_forward: hidden_states and the norm weight must be contiguous")
    if ws is None:
        ws = get_workspace(geo, h.device, keep_logits=keep_logits)
    if out is None:
        out = torch.empty_like(h)
    if n == 0:
        return out, ws
    if getattr(ws, "rstd", None) is None:
        ws.rstd = torch.empty(n, dtype=torch.float32, device=h.device)
        ws.w_fold, ws.w_fold_key = torch.empty_like(w_router), None
        # normalised rows of the tokens that pick a +/-Identity expert (only those rows are ever touched)
        ws.xn = torch.empty_like(h) if n_glu < geo.n_experts else None
    key = (w_router.data_ptr(), w_router._version, norm_weight.data_ptr(), norm_weight._version)
    refold = int(ws.w_fold_key != key)
    ws.w_fold_key = key
    bias32 = bias if bias.dtype == torch.float32 else bias.float()
    theta32 = theta if theta.dtype == torch.float32 else theta.float()
    shape = _shape(geo, norm_mode, scale, False)
    ws.raise_if_failed()
    ws.addend, ws.trace = None, trace
    cws = ws.c_struct()
    ws.trace = None
    rc = lib.bibo_moe_ffn_forward(C.byref(shape), _lib.ptr(h), _lib.ptr(norm_weight), float(eps), _lib.ptr(w_router),
                                  _lib.ptr(bias32), _lib.ptr(gate_up_proj), _lib.ptr(down_proj), _lib.ptr(theta32),
                                  C.byref(cws), _lib.ptr(ws.rstd), _lib.ptr(ws.w_fold), refold, _lib.ptr(ws.xn),
                                  _lib.ptr(out), _stream(h.device))
    _lib.check(rc, "bibo_moe_ffn_forward")
    ws.post_status()
    return out, ws


def moe_forward_host(x_host: torch.Tensor, out_host: torch.Tensor, x_dev: torch.Tensor, out_dev: torch.Tensor,
                     w_router, bias, gate_up_proj, down_proj, theta, top_k: int, norm_mode="sum",
                     scale: float = 1.0, ws: Optional[MoEWorkspace] = None) -> torch.Tensor:
    """Host-buffer variant (bibo_moe_forward_host): x_host -> device, block, -> out_host, then waits."""
    lib = _lib.load()
    n, hidden = x_host.shape
    n_glu, two_i, _ = gate_up_proj.shape
    geo = Geometry(n, hidden, two_i // 2, w_router.shape[0], n_glu, 0, top_k, x_host.dtype)
    if ws is None:
        ws = get_workspace(geo, x_dev.device)
    shape = _shape(geo, norm_mode, scale, False)
    cws = ws.c_struct()
    rc = lib.bibo_moe_forward_host(C.byref(shape), _lib.ptr(x_host), _lib.ptr(x_dev), _lib.ptr(w_router),
                                   _lib.ptr(bias), _lib.ptr(gate_up_proj), _lib.ptr(down_proj), _lib.ptr(theta),
                                   C.byref(cws), _lib.ptr(out_dev), _lib.ptr(out_host), _stream(x_dev.device))
    _lib.check(rc, "bibo_moe_forward_host")
    return out_host


def experts_forward(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, gate_up_proj: torch.Tensor,
                    down_proj: torch.Tensor, theta: torch.Tensor, n_experts: int, n_pos: int = 0,
                    ws: Optional[MoEWorkspace] = None, zero_padding: bool = False) -> Tuple[torch.Tensor, MoEWorkspace]:
    """Experts on routing decided by the caller (the BiBoFusedExperts.forward seam): rank, plan,
    permute, the two grouped GEMMs and the combine as separate C-ABI calls."""
    lib = _lib.load()
    for name, t in (("x", x), ("top_k_indices", topk_idx), ("top_k_weights", topk_w)):
        _need_cuda(t, name)
    n, hidden = x.shape
    k = topk_idx.shape[1]
    n_glu, two_i, _ = gate_up_proj.shape
    inter = two_i // 2
    geo = Geometry(n, hidden, inter, n_experts, n_glu, n_pos, k, x.dtype)
    if ws is None:
        ws = get_workspace(geo, x.device)
    out = torch.empty_like(x)
    if n == 0:
        return out, ws
    dt, st = dtype_code(x.dtype), _stream(x.device)
    idx32 = topk_idx.to(torch.int32).contiguous()
    w32 = topk_w.to(torch.float32).contiguous()
    theta32 = theta if theta.dtype == torch.float32 else theta.float()
    p = _lib.ptr
    ws.raise_if_failed()
    # bad indices (status 2 / 3) land in the plan's status word, which raise_if_failed reports
    _lib.check(lib.bibo_moe_route_from_indices(p(idx32), n, n_experts, k, p(ws.slot_rank), p(ws.block_counts),
                                               p(ws.plan[2:]), st), "bibo_moe_route_from_indices")
    _lib.check(lib.bibo_moe_plan(p(ws.block_counts), n, k, n_experts, n_glu, p(ws.plan), st), "bibo_moe_plan")
    _lib.check(lib.bibo_moe_permute_fwd(p(x), p(idx32), p(ws.slot_rank), p(ws.plan), n, hidden, n_experts, n_glu, k,
                                        dt, int(zero_padding), p(ws.xp), p(ws.slot_row), p(ws.row_token), st),
               "bibo_moe_permute_fwd")
    _lib.check(lib.bibo_moe_gemm1_radial_fwd(p(ws.xp), p(gate_up_proj), p(theta32), p(ws.plan), n, hidden, inter,
                                             n_experts, n_glu, k, dt, p(ws.h), p(ws.gate_up), p(ws.rnorm), st),
               "bibo_moe_gemm1_radial_fwd")
    _lib.check(lib.bibo_moe_gemm2_fwd(p(ws.h), p(down_proj), p(ws.plan), n, hidden, inter, n_experts, n_glu, k, dt,
                                      p(ws.y), st), "bibo_moe_gemm2_fwd")
    _lib.check(lib.bibo_moe_combine_fwd(p(ws.y), p(x), p(ws.slot_row), p(idx32), p(w32), n, hidden, k, n_glu, n_pos,
                                        dt, p(out), st), "bibo_moe_combine_fwd")
    ws.topk_idx_external = idx32  # keep alive until the stream has consumed it
    ws.topk_w_external = w32
    ws.post_status()
    return out, ws


def rmsnorm_forward(h: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """BiBoRMSNorm.forward on flat rows h [N,H] (bibo_moe_rmsnorm_fwd)."""
    lib = _lib.load()
    _need_cuda(h, "hidden_states")
    _need_cuda(weight, "norm weight")
    if weight.dtype != h.dtype:
        weight = weight.to(h.dtype)
    out = torch.empty_like(h)
    n, hidden = h.shape
    _lib.check(lib.bibo_moe_rmsnorm_fwd(_lib.ptr(h), _lib.ptr(weight.contiguous()), float(eps), n, hidden,
                                        dtype_code(h.dtype), _lib.ptr(out), _stream(h.device)), "bibo_moe_rmsnorm_fwd")
    return out


def rmsnorm_backward(dy: torch.Tensor, h: torch.Tensor, weight: torch.Tensor, eps: float):
    """Gradients of ``rmsnorm_forward``: (dh [N,H], dweight [H]) (bibo_moe_rmsnorm_bwd)."""
    lib = _lib.load()
    _need_cuda(dy, "dy")
    if weight.dtype != h.dtype:
        weight = weight.to(h.dtype)
    n, hidden = h.shape
    dh = torch.empty_like(h)
    dweight = torch.empty(hidden, dtype=h.dtype, device=h.device)
    partial = torch.empty(int(lib.bibo_moe_rmsnorm_bwd_parts(n)), hidden, dtype=torch.float32, device=h.device)
    p = _lib.ptr
    _lib.check(lib.bibo_moe_rmsnorm_bwd(p(h), p(weight.contiguous()), p(dy.contiguous()), float(eps), n, hidden,
                                        dtype_code(h.dtype), p(dh), p(partial), p(dweight), _stream(h.device)),
               "bibo_moe_rmsnorm_bwd")
    return dh, dweight


def mlp_forward(x: torch.Tensor, gate_proj: torch.Tensor, up_proj: torch.Tensor, down_proj: torch.Tensor,
                out: Optional[torch.Tensor] = None, keep: bool = False, residual: Optional[torch.Tensor] = None):
    """Dense SwiGLU MLP ``down(silu(gate(x)) * up(x))`` on flat tokens x [N,H] (bibo_moe_mlp_forward);
    weights are the ``nn.Linear`` weights as stored: gate/up [I,H], down [H,I].  bf16.
    ``keep=True`` returns ``(out, saved)`` with the tensors ``mlp_backward`` needs.
    ``residual`` [N,H] is added in the down kernel's epilogue (tensor-core shapes only: ``mlp_residual_supported``)."""
    lib = _lib.load()
    for name, t in (("x", x), ("gate_proj", gate_proj), ("up_proj", up_proj), ("down_proj", down_proj)):
        _need_cuda(t, name)
        if t.dtype != x.dtype:
            raise RuntimeError(f"{name} dtype {t.dtype} != activation dtype {x.dtype}")
    n, hidden = x.shape
    inter = gate_proj.shape[0]
    dt = dtype_code(x.dtype)
    # bf16 with hidden % 256 == 0 and intermediate % 256 == 0 runs on tensor cores; float32 and other shapes run
    # the CUDA-core kernels, which stage gate | up in a buffer
    tensor_cores = bool(lib.bibo_moe_mlp_supported(hidden, inter, dt))
    if out is None:
        out = torch.empty_like(x)
    if n == 0:
        return (out, None) if keep else out
    plan = torch.empty(int(lib.bibo_moe_mlp_plan_words(n)), dtype=torch.int32, device=x.device)
    h = torch.empty(n, inter, dtype=x.dtype, device=x.device)
    gate_up = torch.empty(n, 2 * inter, dtype=x.dtype, device=x.device) if (keep or not tensor_cores) else None
    p = _lib.ptr
    if residual is not None:
        if residual.shape != x.shape or residual.dtype != x.dtype or not residual.is_contiguous() or not residual.is_cuda:
            raise RuntimeError("residual must be a contiguous CUDA tensor of the activations' shape and dtype")
        _lib.check(lib.bibo_moe_mlp_forward_residual(p(x), p(gate_proj), p(up_proj), p(down_proj), n, hidden, inter, dt,
                                                     p(plan), p(h), p(out), p(gate_up), p(residual), _stream(x.device)),
                   "bibo_moe_mlp_forward_residual")
        return (out, (plan, h, gate_up)) if keep else out
    _lib.check(lib.bibo_moe_mlp_forward(p(x), p(gate_proj), p(up_proj), p(down_proj), n, hidden, inter, dt, p(plan),
                                        p(h), p(out), p(gate_up), _stream(x.device)), "bibo_moe_mlp_forward")
    return (out, (plan, h, gate_up)) if keep else out


def mlp_residual_supported(hidden: int, inter: int, dtype) -> bool:
    """Whether ``mlp_forward(residual=...)`` can add the residual inside the down kernel for these sizes."""
    return bool(_lib.load().bibo_moe_mlp_supported(hidden, inter, dtype_code(dtype)))


def mlp_backward(dout: torch.Tensor, x: torch.Tensor, gate_proj: torch.Tensor, up_proj: torch.Tensor,
                 down_proj: torch.Tensor, saved):
    """Gradients of ``mlp_forward(..., keep=True)`` (bibo_moe_mlp_backward); ``saved`` is consumed.
    Returns (dx, d_gate_proj, d_up_proj, d_down_proj)."""
    lib = _lib.load()
    plan, h, gate_up = saved
    n, hidden = x.shape
    inter = gate_proj.shape[0]
    w_gu = torch.cat([gate_proj, up_proj])                      # [2I, H]: one K-stacked operand for dX
    dh = torch.empty(n, inter, dtype=x.dtype, device=x.device)
    dx = torch.empty_like(x)
    d_gu = torch.empty_like(w_gu)
    d_dn = torch.empty_like(down_proj)
    p = _lib.ptr
    _lib.check(lib.bibo_moe_mlp_backward(p(x), p(w_gu), p(down_proj), p(gate_up), p(h), p(dout), n, hidden, inter,
                                         dtype_code(x.dtype), p(plan), p(dh), p(dx), p(d_gu), p(d_dn),
                                         _stream(x.device)), "bibo_moe_mlp_backward")
    return dx, d_gu[:inter], d_gu[inter:], d_dn


def moe_backward(dout: torch.Tensor, x: torch.Tensor, w_router: torch.Tensor, gate_up_proj: torch.Tensor,
                 down_proj: torch.Tensor, theta: torch.Tensor, ws: MoEWorkspace, norm_mode="sum", scale: float = 1.0,
                 zero_padded: bool = True):
    """Gradients of the block (one call of bibo_moe_backward).  ``ws`` is the workspace of the matching
    forward (kept gate_up / rnorm); it is consumed.  Returns (dx, d_w_router, d_gate_up_proj,
    d_down_proj, d_theta fp32)."""
    lib = _lib.load()
    geo = ws.geo
    for name, t in (("dout", dout), ("x", x)):
        _need_cuda(t, name)
    if ws.gate_up is None or ws.rnorm is None:
        raise RuntimeError("the forward workspace was created without the tensors the backward needs")
    dev, rows = x.device, geo.rows_cap
    f32 = dict(dtype=torch.float32, device=dev)
    dy = torch.empty(rows, geo.hidden, dtype=geo.dtype, device=dev)
    dh = torch.empty(rows, geo.inter, dtype=geo.dtype, device=dev)
    dw = torch.empty(geo.n_tokens, geo.top_k, **f32)
    dlogit = torch.empty(geo.n_tokens, geo.top_k, **f32)
    dlogit_row = torch.empty(rows, **f32)
    dtheta_row = torch.empty(rows, **f32)
    dx = torch.empty_like(x)
    d_wr = torch.zeros_like(w_router)
    d_gu = torch.empty_like(gate_up_proj)    # written in full by the weight-gradient kernels (zeros for unused experts)
    d_dn = torch.empty_like(down_proj)
    d_theta = torch.zeros(geo.n_glu, **f32)
    p = _lib.ptr
    bws = _lib.BwdWorkspace(p(dy), p(dh), p(dw), p(dlogit), p(dlogit_row), p(dtheta_row))
    # zero_padded: the forward ran with zero_padding=True (lets the weight-gradient GEMMs use tensor cores)
    shape = _shape(geo, norm_mode, scale, zero_padded)
    ws.raise_if_failed()
    cws = ws.c_struct()
    theta32 = theta if theta.dtype == torch.float32 else theta.float()
    rc = lib.bibo_moe_backward(C.byref(shape), p(x), p(w_router), p(gate_up_proj), p(down_proj), p(theta32),
                               C.byref(cws), p(dout), C.byref(bws), p(dx), p(d_wr), p(d_gu), p(d_dn), p(d_theta),
                               _stream(dev))
    _lib.check(rc, "bibo_moe_backward")
    ws.post_status()
    return dx, d_wr, d_gu, d_dn, d_theta


def plan_header(ws: MoEWorkspace):
    """Debug: (n_tiles, rows_used, status) read back from the device (synchronises the stream)."""
    lib = _lib.load()
    hdr = (C.c_int32 * 4)()
    rc = lib.bibo_moe_debug_plan_header(_lib.ptr(ws.plan), C.cast(hdr, C.c_void_p), _stream(ws.plan.device))
    _lib.check(rc, "bibo_moe_debug_plan_header")
    return int(hdr[0]), int(hdr[1]), int(hdr[2])
