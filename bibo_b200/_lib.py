"""ctypes binding of libbibo_moe.so (declarations mirror include/bibo_moe.h).

There is no CPU or PyTorch fallback behind these calls: if the library is missing or a call
returns an error, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes as C
import pathlib

_HERE = pathlib.Path(__file__).resolve().parent
LIB_PATH = _HERE / "csrc" / "libbibo_moe.so"

F32, BF16 = 0, 1
NORM_RAW, NORM_SUM, NORM_SOFTMAX = 0, 1, 2
TILE_M = 128
ROUTER_BLOCK_TOKENS = 128
MAX_TOP_K = 8
MAX_EXPERTS = 256

_vp, _i32, _i64, _f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float


class Workspace(C.Structure):
    _fields_ = [(n, _vp) for n in (
        "topk_idx", "topk_w", "slot_rank", "block_counts", "plan", "slot_row", "row_token",
        "xp", "h", "y", "gate_up", "rnorm", "logits", "stage_events", "addend", "trace")]


class RouterTrace(C.Structure):
    _fields_ = [(n, _vp) for n in ("block_sums", "acc", "counts", "gap")]


TRACE_WORDS = 8


class BwdWorkspace(C.Structure):
    _fields_ = [(n, _vp) for n in ("dy", "dh", "dw", "dlogit", "dlogit_row", "dtheta_row")]


class EpArgs(C.Structure):
    _fields_ = ([("n_tokens", _i64), ("rows_cap_recv", _i64)] +
                [(n, _i32) for n in ("hidden", "inter", "n_experts", "top_k", "norm_mode", "rank", "world", "max_ctas",
                                     "comm_ctas", "epoch_base")] +
                [("scale", _f32)] +
                [(n, _vp) for n in ("x", "w_router", "bias", "gate_up_proj", "down_proj", "theta", "topk_idx", "topk_w",
                                    "slot_rank", "block_counts", "local_plan", "ep_plan", "slot_row", "h", "xp_peers",
                                    "y_peers", "flags_peers", "cnt_peers", "out", "gate_up_recv", "rnorm_recv",
                                    "row_token", "trace")])


class EpDma(C.Structure):
    _fields_ = ([(n, _vp) for n in ("xp_send", "y_owner", "y_home_peers", "row_token", "cnt_host", "counts_ready")] +
                [("n_aux", _i32)] + [(n, _vp) for n in ("aux_streams", "aux_events", "marks")])


class EpBwdArgs(C.Structure):
    _fields_ = ([(n, _vp) for n in ("dout", "dy_peers", "dh", "dw", "dlogit_row", "dtheta_row", "dx", "d_w_router",
                                    "d_gate_up_proj", "d_down_proj", "d_theta")] + [("epoch_base", _i32)])


class EpDedupOwner(C.Structure):
    _fields_ = ([("n_cap", _i64)] +
                [(n, _i32) for n in ("hidden", "inter", "n_experts", "top_k", "rank", "world", "max_ctas", "comm_ctas")] +
                [(n, _vp) for n in ("xu", "midx", "mw", "gate_up_proj", "down_proj", "theta", "slot_rank", "block_counts",
                                    "plan", "slot_row", "row_token", "xp", "h", "y", "part_peers")])


class EpDedup(C.Structure):
    _fields_ = ([("owner", EpDedupOwner), ("n_tokens", _i64), ("norm_mode", _i32), ("epoch_base", _i32), ("scale", _f32)] +
                [(n, _vp) for n in ("x", "w_router", "bias", "topk_idx", "topk_w", "slot_rank_home", "block_counts_home",
                                    "xu_peers", "midx_peers", "mw_peers", "flags_peers", "part_local", "out", "marks",
                                    "trace")])


class Shape(C.Structure):
    _fields_ = [("n_tokens", _i64), ("hidden", _i32), ("inter", _i32), ("n_experts", _i32),
                ("n_glu", _i32), ("n_pos", _i32), ("top_k", _i32), ("norm_mode", _i32),
                ("dtype", _i32), ("scale", _f32), ("zero_padding", _i32)]


# name -> (restype, argtypes); every symbol include/bibo_moe.h declares
SIGNATURES = {
    "bibo_moe_version": (_i32, []),
    "bibo_moe_last_error_string": (C.c_char_p, []),
    "bibo_moe_rows_cap": (_i64, [_i64, _i32, _i32]),
    "bibo_moe_tiles_cap": (_i64, [_i64, _i32, _i32]),
    "bibo_moe_router_blocks": (_i64, [_i64]),
    "bibo_moe_plan_words": (_i64, [_i64, _i32, _i32, _i32]),
    "bibo_moe_router_fwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _f32, _i32,
                                   _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bibo_moe_router_fwd_trace": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _f32, _i32,
                                         _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bibo_moe_router_norm_supported": (_i32, [_i32, _i32, _i32]),
    "bibo_moe_fold_norm_weight": (_i32, [_vp, _vp, _i32, _i32, _vp, _vp]),
    "bibo_moe_router_norm_fwd": (_i32, [_vp, _vp, _f32, _vp, _i64, _i32, _i32, _i32, _i32, _f32,
                                        _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bibo_moe_permute_norm_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32,
                                         _vp, _vp, _vp, _vp, _vp]),
    "bibo_moe_ffn_supported": (_i32, [_vp]),
    "bibo_moe_ffn_forward": (_i32, [_vp, _vp, _vp, _f32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp]),
    "bibo_moe_route_from_indices": (_i32, [_vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp]),
    "bibo_moe_plan": (_i32, [_vp, _i64, _i32, _i32, _i32, _vp, _vp]),
    "bibo_moe_plan_trace": (_i32, [_vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp]),
    "bibo_moe_plan_off_counts": (_i64, []),
    "bibo_moe_plan_off_expert_off": (_i64, [_i32]),
    "bibo_moe_plan_off_block_base": (_i64, [_i32, _i32]),
    "bibo_moe_plan_off_tiles": (_i64, [_i64, _i32, _i32]),
    "bibo_moe_permute_fwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _i32,
                                    _vp, _vp, _vp, _vp]),
    "bibo_moe_gemm1_radial_fwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32,
                                         _i32, _vp, _vp, _vp, _vp]),
    "bibo_moe_gemm1_is_fused": (_i32, [_i32, _i32, _i32]),
    "bibo_moe_rowmap_fwd": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp]),
    "bibo_moe_gemm1_gather_supported": (_i32, [_i32, _i32, _i32]),
    "bibo_moe_gemm1_gather_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
                                         _vp, _vp, _vp, _vp, _vp]),
    "bibo_moe_gemm2_fwd": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "bibo_moe_combine_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32,
                                    _vp, _vp]),
    "bibo_moe_combine_add_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32,
                                        _vp, _vp]),
    "bibo_moe_forward": (_i32, [C.POINTER(Shape), _vp, _vp, _vp, _vp, _vp, _vp,
                                C.POINTER(Workspace), _vp, _vp]),
    "bibo_moe_forward_host": (_i32, [C.POINTER(Shape), _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                     C.POINTER(Workspace), _vp, _vp, _vp]),
    "bibo_moe_backward": (_i32, [C.POINTER(Shape), _vp, _vp, _vp, _vp, _vp, C.POINTER(Workspace), _vp,
                                 C.POINTER(BwdWorkspace), _vp, _vp, _vp, _vp, _vp, _vp]),
    "bibo_moe_ep_plan_words": (_i64, [_i32, _i64]),
    "bibo_moe_ep_plan_off": (_i64, [_i32, _i32]),
    "bibo_moe_ep_plan": (_i32, [_vp, _i32, _i32, _i32, _i64, _vp, _vp]),
    "bibo_moe_ep_dispatch": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _i64, _i32, _vp, _vp,
                                    _vp]),
    "bibo_moe_rmsnorm_fwd": (_i32, [_vp, _vp, _f32, _i64, _i32, _i32, _vp, _vp]),
    "bibo_moe_rmsnorm_bwd_parts": (_i64, [_i64]),
    "bibo_moe_rmsnorm_bwd": (_i32, [_vp, _vp, _vp, _f32, _i64, _i32, _i32, _vp, _vp, _vp, _vp]),
    "bibo_moe_mlp_plan_words": (_i64, [_i64]),
    "bibo_moe_mlp_supported": (_i32, [_i32, _i32, _i32]),
    "bibo_moe_mlp_forward": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp]),
    "bibo_moe_mlp_forward_residual": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp,
                                             _vp]),
    "bibo_moe_mlp_backward": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp,
                                     _vp]),
    "bibo_moe_ep_forward": (_i32, [C.POINTER(EpArgs), _vp]),
    "bibo_moe_ep_forward_dma": (_i32, [C.POINTER(EpArgs), C.POINTER(EpDma), _i32, _vp]),
    "bibo_moe_ep_plan_layout": (_i32, [_vp, _i32, _i32, _i32, _i64, _i32, _vp, _vp]),
    "bibo_moe_ep_backward": (_i32, [C.POINTER(EpArgs), C.POINTER(EpBwdArgs), _vp]),
    "bibo_moe_ep_experts": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i64, _i32, _vp, _vp, _vp, _vp, _i32,
                                   _vp]),
    "bibo_moe_ep_barrier": (_i32, [_vp, _i32, _i32, _i32, _vp, _vp]),
    "bibo_moe_ep_barrier_bounded": (_i32, [_vp, _i32, _i32, _i32, _i64, _vp, _vp]),
    "bibo_moe_ep_combine": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i64, _i32, _vp, _vp]),
    "bibo_moe_ep_dedup_rows_cap": (_i64, [_i32, _i64, _i32, _i32]),
    "bibo_moe_ep_dedup_plan_words": (_i64, [_i32, _i64, _i32, _i32]),
    "bibo_moe_ep_dedup_virtual_tokens": (_i64, [_i32, _i64]),
    "bibo_moe_ep_dedup_dispatch": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32,
                                          _vp]),
    "bibo_moe_ep_dedup_owner": (_i32, [C.POINTER(EpDedupOwner), _vp]),
    "bibo_moe_ep_dedup_experts": (_i32, [C.POINTER(EpDedupOwner), _vp]),
    "bibo_moe_ep_dedup_partial": (_i32, [C.POINTER(EpDedupOwner), _vp]),
    "bibo_moe_ep_dedup_push": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp]),
    "bibo_moe_ep_dedup_final": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "bibo_moe_ep_localize": (_i32, [_vp, _i64, _i32, _i32, _i32, _i32, _vp, _vp]),
    "bibo_moe_ep_copy_to_peers": (_i32, [_vp, _i64, _vp, _i64, _i64, _i32, _i32, _i32, _vp]),
    "bibo_moe_ep_dedup_forward": (_i32, [C.POINTER(EpDedup), _vp]),
    "bibo_moe_route_noalloc": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _f32, _i32, _vp, _vp, _vp, _vp]),
    "bibo_moe_route_noalloc_max_tokens": (_i64, []),
    "bibo_moe_route_noalloc_status": (_i32, [_vp, _vp]),
    "bibo_moe_debug_plan_header": (_i32, [_vp, _vp, _vp]),
    "bibo_moe_launch_count": (_i64, []),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m bibo_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().bibo_moe_last_error_string().decode(errors="replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def ptr(t) -> int | None:
    """Raw data pointer of a torch tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()
