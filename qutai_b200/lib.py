"""ctypes binding of ``libqutai_moe.so`` (declared in ``include/qutai_moe.h``).

Dependency-free: only the standard library.  Importing this module never touches CUDA; the
library is loaded on first use (the upstream package behaves the same way,
tests/test_cuda.py:12-16).  There is no CPU fallback: when the library cannot be loaded every
operation raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import (POINTER, Structure, byref, c_char_p, c_double, c_float, c_int, c_int32, c_int64,
                    c_uint64, c_void_p)

QMOE_F32, QMOE_BF16 = 0, 1
ENGINE_AUTO, ENGINE_SIMT, ENGINE_TCGEN05 = 0, 1, 2
VARIANT_SINGLE_CTA_GEMM, VARIANT_WGRAD_PER_PRODUCT, VARIANT_NARROW_SCATTER, VARIANT_PLAIN_GEMM_ON_CUDA_CORES = 0, 1, 2, 3
ROW_PAD, MAX_EXPERTS, MAX_TOP_K = 128, 256, 8
DTYPE_CODES = {"float32": QMOE_F32, "bfloat16": QMOE_BF16}
ITEM_BYTES = {"float32": 4, "bfloat16": 2, "int32": 4, "int64": 8, "float64": 8}


class Route(Structure):
    """``qmoe_route_t``."""
    _fields_ = [("tokens", c_int64), ("experts", c_int32), ("top_k", c_int32), ("rows_bound", c_int64)] + [
        (name, c_uint64) for name in (
            "probs", "gate_weights", "expert_index", "dest_row", "row_source", "counts", "offsets",
            "tile_expert", "meta", "utilization", "aux", "block_counts", "block_base", "block_colsum")]


class Experts(Structure):
    """``qmoe_experts_t``."""
    _fields_ = [("experts", c_int32), ("dtype", c_int32), ("engine", c_int32), ("reserved", c_int32),
                ("width", c_int64), ("hidden", c_int64),
                ("w_gate", c_uint64), ("w_up", c_uint64), ("w_down", c_uint64)]


class Segment(Structure):
    """``qmoe_ep_segment_t``."""
    _fields_ = [("peer", c_int32), ("reserved", c_int32), ("offset_rows", c_int64), ("rows", c_int64)]


EP_MAX_RANKS = 16


class Peers(Structure):
    """``qmoe_ep_peers_t``."""
    _fields_ = [("world", c_int32), ("rank", c_int32), ("buffer", c_uint64 * EP_MAX_RANKS),
                ("ret", c_uint64 * EP_MAX_RANKS)]


class OptimItem(Structure):
    """``qmoe_optim_item_t``."""
    _fields_ = [("values", c_uint64), ("grad", c_uint64), ("exp_avg", c_uint64), ("exp_avg_sq", c_uint64),
                ("shadow", c_uint64), ("size", c_int64), ("first_chunk", c_int64), ("c1", c_float), ("c2", c_float)]


class Layer(Structure):
    """``qmoe_layer_t``."""
    _fields_ = [("route", Route), ("experts", Experts)] + [
        (name, c_uint64) for name in (
            "x", "w_router", "scores", "x_dispatched", "g", "u", "h", "y_dispatched", "out",
            "grad_out", "grad_aux", "dy_dispatched", "d_h", "d_g", "d_u", "dx_dispatched",
            "d_gate_weights", "d_scores", "dx_router", "router_partials", "dx", "d_w_router",
            "d_w_gate", "d_w_up", "d_w_down", "master_gate", "master_up", "master_down")]


class Block(Structure):
    """``qmoe_block_t``."""
    _fields_ = [("layer", Layer)] + [(name, c_uint64) for name in (
        "norm_weight", "inverse", "w_router_folded", "d_norm_weight", "norm_partials")] + [("norm_eps", c_double)]


class Head(Structure):
    """``qmoe_head_t``."""
    _fields_ = [("batch", c_int32), ("time", c_int32), ("dtype", c_int32), ("reserved", c_int32),
                ("width", c_int64), ("vocab", c_int64), ("rows_bound", c_int64)] + [(name, c_uint64) for name in (
        "hidden", "weight", "labels", "inputs", "logits", "row_loss", "loss", "meta", "d_inputs", "d_hidden", "d_weight")]


class Attention(Structure):
    """``qmoe_attention_t``."""
    _fields_ = [(name, c_int32) for name in ("batch", "time", "heads", "kv_heads", "dim", "dtype")] + [(name, c_uint64) for name in (
        "q", "k", "v", "out", "lse", "grad_out", "delta", "dq", "dk", "dv")]


_U, _I32, _I64 = c_uint64, c_int32, c_int64
_RP, _EP, _LP, _SP = POINTER(Route), POINTER(Experts), POINTER(Layer), POINTER(Segment)

# name -> (restype, argtypes); every symbol declared in include/qutai_moe.h
SIGNATURES = {
    "qmoe_version": (c_int, []),
    "qmoe_last_error": (c_char_p, []),
    "qmoe_device_info": (c_int, [POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_uint64)]),
    "qmoe_malloc": (c_int, [POINTER(c_uint64), _U]),
    "qmoe_free": (c_int, [_U]),
    "qmoe_host_alloc": (c_int, [POINTER(c_void_p), _U]),
    "qmoe_host_free": (c_int, [c_void_p]),
    "qmoe_memcpy_h2d": (c_int, [_U, c_void_p, _U, _U]),
    "qmoe_memcpy_d2h": (c_int, [c_void_p, _U, _U, _U]),
    "qmoe_memcpy_d2d": (c_int, [_U, _U, _U, _U]),
    "qmoe_memset": (c_int, [_U, c_int, _U, _U]),
    "qmoe_stream_sync": (c_int, [_U]),
    "qmoe_stream_create": (c_int, [POINTER(c_uint64)]),
    "qmoe_stream_destroy": (c_int, [_U]),
    "qmoe_event_create": (c_int, [POINTER(c_uint64)]),
    "qmoe_event_destroy": (c_int, [_U]),
    "qmoe_event_record": (c_int, [_U, _U]),
    "qmoe_stream_wait_event": (c_int, [_U, _U]),
    "qmoe_event_sync": (c_int, [_U]),
    "qmoe_launch_count": (c_int64, []),
    "qmoe_tensor_core_launch_count": (c_int64, []),
    "qmoe_timing_enable": (c_int, [c_int]),
    "qmoe_timing_classes": (c_int, []),
    "qmoe_timing_class_name": (c_char_p, [c_int]),
    "qmoe_timing_read": (c_int, [POINTER(c_double), POINTER(c_int64), c_int]),
    "qmoe_device_status": (c_int, [_U, POINTER(c_int)]),
    "qmoe_device_status_clear": (c_int, [_U]),
    "qmoe_device_status_async": (c_int, [_U, c_void_p]),
    "qmoe_gather_rows": (c_int, [_U, _U, _U, _I32, _I32, _I64, _U]),
    "qmoe_ep_set_barrier_timeout_ms": (c_int, [_I64]),
    "qmoe_test_select_variant": (c_int, [_I32, _I32]),
    "qmoe_rows_bound": (c_int64, [_I64, _I32, _I32]),
    "qmoe_route_blocks": (c_int64, [_I64]),
    "qmoe_router_logits": (c_int, [_U, _I32, _U, _U, _I64, _I64, _I32, _U]),
    "qmoe_router_scratch_bytes": (c_int64, [_I64, _I32, _I64]),
    "qmoe_router_forward": (c_int, [_U, _I32, _U, _U, _U, _I64, _I64, _I32, _U]),
    "qmoe_router_grad_partials": (c_int64, [_I64, _I32, _I64]),
    "qmoe_router_backward": (c_int, [_U, _U, _I32, _U, _U, _U, _U, _I64, _I64, _I32, _U]),
    "qmoe_route": (c_int, [_RP, _U, _U]),
    "qmoe_route_static": (c_int, [_RP, _U, _U]),
    "qmoe_route_export_i64": (c_int, [_RP, _U, _U, _U, _U, _U, _I64, _U]),
    "qmoe_route_backward": (c_int, [_RP, _U, _U, _U, _U]),
    "qmoe_permute": (c_int, [_RP, _U, _U, _I32, _I64, _U]),
    "qmoe_unpermute_reduce": (c_int, [_RP, _U, _U, _U, _I32, _I64, _U]),
    "qmoe_combine": (c_int, [_RP, _U, _U, _I32, _I64, _U]),
    "qmoe_combine_backward": (c_int, [_RP, _U, _U, _U, _U, _I32, _I64, _U]),
    "qmoe_cast_bf16": (c_int, [_U, _U, _I64, _U]),
    "qmoe_expert_forward": (c_int, [_RP, _EP, _U, _U, _U, _U, _U, _U]),
    "qmoe_expert_backward": (c_int, [_RP, _EP] + [_U] * 13),
    "qmoe_expert_forward_parts": (c_int, [_RP, _EP, _U, _U, _U, _U, _U, _I32, _U]),
    "qmoe_expert_backward_parts": (c_int, [_RP, _EP] + [_U] * 12 + [_I32, _U]),
    "qmoe_gemm": (c_int, [_U, _I32, _U, _I32, _U, _I32, _I64, _I64, _I64, _I32, _I32, _I32, _U]),
    "qmoe_gemm_wgrad_partials": (c_int64, [_I64, _I64, _I64]),
    "qmoe_gemm_wgrad_split": (c_int, [_U, _U, _U, _U, _I64, _I64, _I64, _U]),
    "qmoe_silu": (c_int, [_U, _U, _U, _I32, _I64, _I32, _U]),
    "qmoe_add": (c_int, [_U, _U, _U, _I32, _I64, _U]),
    "qmoe_normal_fill": (c_int, [_U, _I32, _I64, c_double, c_double, _U, _U]),
    "qmoe_rms_inverse": (c_int, [_U, _I32, _U, _I64, _I64, c_double, _U]),
    "qmoe_scale_f32": (c_int, [_U, _U, _U, _U, _I64, _I64, _U]),
    "qmoe_permute_norm": (c_int, [_RP, _U, _U, _U, _U, _I32, _I64, _U]),
    "qmoe_combine_residual": (c_int, [_RP, _U, _U, _U, _I32, _I64, _U]),
    "qmoe_norm_backward_partials": (c_int64, [_I64, _I64]),
    "qmoe_unpermute_norm_backward": (c_int, [_RP, _U, _U, _I32] + [_U] * 7 + [_I32, _I64, _U]),
    "qmoe_block_forward": (c_int, [POINTER(Block), _U]),
    "qmoe_block_backward": (c_int, [POINTER(Block), _U]),
    "qmoe_head_forward": (c_int, [POINTER(Head), _U]),
    "qmoe_head_backward": (c_int, [POINTER(Head), _U, _U]),
    "qmoe_head_rows": (c_int, [_U, _U, _I32, _I64, _I64, _I64, _I64, _I32, _U]),
    "qmoe_head_loss": (c_int, [_U, _I32, _U, _U, _U, _I64, _I64, _I64, _U]),
    "qmoe_head_gradient": (c_int, [_U, _I32, _U, _U, _U, _I64, _I64, _I64, _I64, _U]),
    "qmoe_rms_norm": (c_int, [_U, _I32, _U, _U, _I32, _U, _I64, _I64, c_double, _U]),
    "qmoe_rms_norm_partials": (c_int64, [_I64, _I64]),
    "qmoe_rms_norm_backward": (c_int, [_U, _I32, _U, _I32, _U, _U, _U, _U, _U, _I64, _I64, _U]),
    "qmoe_rope": (c_int, [_U, _U, _I32, _I64, _I64, _I32, _I32, c_double, _I32, _I32, _U]),
    "qmoe_embedding": (c_int, [_U, _U, _U, _I32, _I64, _I64, _I64, _U]),
    "qmoe_embedding_backward": (c_int, [_U, _I32, _U, _U, _U, _U, _I64, _I64, _I64, _I64, _U]),
    "qmoe_attention_forward": (c_int, [POINTER(Attention), _U]),
    "qmoe_attention_backward": (c_int, [POINTER(Attention), _U]),
    "qmoe_layer_forward": (c_int, [_LP, _U]),
    "qmoe_layer_backward": (c_int, [_LP, _U]),
    "qmoe_ep_unique_id": (c_int, [c_void_p]),
    "qmoe_ep_init": (c_int, [_I32, _I32, c_void_p]),
    "qmoe_ep_finalize": (c_int, [_I32]),
    "qmoe_ep_info": (c_int, [POINTER(c_int32), POINTER(c_int32)]),
    "qmoe_ep_gather_stats": (c_int, [_RP, _U, _U, c_void_p, _U]),
    "qmoe_ep_plan": (c_int, [_U, _RP, _RP, _I64, _U]),
    "qmoe_ep_zero_pad_rows": (c_int, [_RP, _U, _I32, _I64, _U]),
    "qmoe_ep_exchange": (c_int, [_U, _SP, _I32, _U, _SP, _I32, _I64, _I32, _U]),
    "qmoe_ep_all_reduce_f32": (c_int, [_U, _I64, _U]),
    "qmoe_set_device": (c_int, [_I32]),
    "qmoe_ep_ipc_export": (c_int, [_U, c_void_p]),
    "qmoe_ep_ipc_open": (c_int, [c_void_p, POINTER(c_uint64)]),
    "qmoe_ep_ipc_close": (c_int, [_U]),
    "qmoe_ep_barrier": (c_int, [_U, _U]),
    "qmoe_ep_dest_base": (c_int, [_U, _I32, _I32, _U, _U]),
    "qmoe_ep_push_dispatch": (c_int, [_RP, _U, _U, POINTER(Peers), _I32, _I32, _I32, _I64, _U]),
    "qmoe_ep_flag_barrier": (c_int, [POINTER(Peers), _I32, _U, _I32, POINTER(Peers), _U]),
    "qmoe_ep_pack_stats": (c_int, [_RP, _U, _U]),
    "qmoe_ep_permute_push": (c_int, [_RP, _U, _U, POINTER(Peers), _I32, _I64, _U]),
    "qmoe_ep_combine_backward_push": (c_int, [_RP, _U, _U, _U, POINTER(Peers), _U, _I32, _I64, _U]),
    "qmoe_ep_permute_push_range": (c_int, [_RP, _U, _U, POINTER(Peers), _I32, _I32, _I32, _I64, _U]),
    "qmoe_ep_combine_backward_push_range": (c_int, [_RP, _U, _U, _U, POINTER(Peers), _U, _I32, _I32, _I32, _I64, _U]),
    "qmoe_ep_expert_down_push": (c_int, [_RP, _EP, _U, _U, POINTER(Peers), _U]),
    "qmoe_ep_expert_dx_push": (c_int, [_RP, _EP, _U, _U, _U, POINTER(Peers), _U]),
    "qmoe_ep_push_return": (c_int, [_RP, _U, _U, POINTER(Peers), _I32, _I32, _I32, _I32, _I64, _U]),
    "qmoe_graph_begin": (c_int, [_U]),
    "qmoe_graph_end": (c_int, [_U, POINTER(c_uint64)]),
    "qmoe_graph_abandon": (c_int, [_U]),
    "qmoe_graph_launch": (c_int, [_U, _U]),
    "qmoe_graph_destroy": (c_int, [_U]),
    "qmoe_optim_table_bytes": (c_int64, [_I32]),
    "qmoe_clip_scratch_bytes": (c_int64, []),
    "qmoe_adamw_multi": (c_int, [POINTER(OptimItem), _I32, _U, c_float, c_float, c_float, c_float, c_float, _U]),
    "qmoe_clip_grad_norm": (c_int, [POINTER(OptimItem), _I32, _U, c_double, _U, _U]),
}

_lock = threading.Lock()
_library = None


def library_path():
    override = os.environ.get("QUTAI_MOE_LIBRARY")
    if override:
        return override
    from . import build

    return build.ensure_built()


def load(path=None):
    """Load the shared library (once) and attach the signatures."""
    global _library
    with _lock:
        if _library is not None and path is None:
            return _library
        handle = ctypes.CDLL(path or library_path())
        for name, (restype, argtypes) in SIGNATURES.items():
            function = getattr(handle, name)  # AttributeError if an export is missing
            function.restype, function.argtypes = restype, argtypes
        if path is None:
            _library = handle
        return handle


def last_error():
    text = load().qmoe_last_error()
    return text.decode("utf-8", "replace") if text else ""


def check(code):
    """Turn a return code into the upstream error convention: ValueError for argument errors
    (raised upstream before any launch, src/qutai/backends/cuda.py:307-334), RuntimeError for
    CUDA failures (src/qutai/backends/cuda_runtime.py:165-177)."""
    if code == 0:
        return
    message = last_error() or f"libqutai_moe error {code}"
    if code in (-1, -2):
        raise ValueError(message)
    raise RuntimeError(f"{message} [code {code}]")


def call(name, *args):
    check(getattr(load(), name)(*args))


def rows_bound(tokens, experts, top_k):
    return int(load().qmoe_rows_bound(tokens, experts, top_k))


def route_blocks(tokens):
    return int(load().qmoe_route_blocks(tokens))


def device_info():
    sms, major, minor, total = c_int(), c_int(), c_int(), c_uint64()
    call("qmoe_device_info", byref(sms), byref(major), byref(minor), byref(total))
    return dict(sm_count=sms.value, compute_capability=(major.value, minor.value), total_bytes=total.value)


def timing(enable):
    call("qmoe_timing_enable", 1 if enable else 0)


def timing_read():
    """{class name: (milliseconds, scopes)} since ``timing(True)``; synchronises the device."""
    handle = load()
    n = handle.qmoe_timing_classes()
    ms, scopes = (c_double * n)(), (c_int64 * n)()
    call("qmoe_timing_read", ms, scopes, n)
    return {handle.qmoe_timing_class_name(i).decode(): (ms[i], scopes[i]) for i in range(n)}


def device_status(stream=0):
    status = c_int()
    call("qmoe_device_status", stream, byref(status))
    return status.value
