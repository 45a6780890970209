"""Causal self-attention with grouped key/value heads over ``qmoe_attention_forward`` / ``qmoe_attention_backward``.

Upstream's ``attention(q, k, v, heads, kv_heads)`` (src/qutai/lm/layers.py:119-130) takes ``q`` [batch, time,
heads * dim] and ``k``, ``v`` [batch, time, kv_heads * dim], calls the backend's ``attention`` (output and the
log-sum-exp of every row) and records a backward that calls ``attention_backward`` with the saved storages.
``attention`` here has that signature and returns a tensor whose ``parents`` / ``backward_rule`` are what upstream's
``record`` would have filled in.  bfloat16 and head width 64 only — the case of upstream's tensor-core kernels
(src/qutai/backends/cuda/lm.cu:91-285).  Dependency-free: ctypes and the standard library only.
"""
from __future__ import annotations

import ctypes

from . import lib
from .layers import Tensor
from .storage import DeviceStorage


def _describe(q, k, v, heads, kv_heads):
    if len(q.shape) != 3 or tuple(k.shape) != tuple(v.shape) or len(k.shape) != 3 or k.shape[:2] != q.shape[:2]:
        raise ValueError("q must be [batch, time, heads * dim] and k, v [batch, time, kv_heads * dim]")
    batch, time, features = q.shape
    if heads <= 0 or kv_heads <= 0 or heads % kv_heads or features % heads:
        raise ValueError("heads must be a positive multiple of kv_heads and divide the width of q")
    dim = features // heads
    if k.shape[2] != kv_heads * dim:
        raise ValueError("the width of k and v must be kv_heads * dim")
    for tensor in (q, k, v):
        if tensor.storage.dtype != "bfloat16":
            raise ValueError("attention takes bfloat16 tensors")
    a = lib.Attention()
    a.batch, a.time, a.heads, a.kv_heads, a.dim, a.dtype = batch, time, heads, kv_heads, dim, lib.QMOE_BF16
    a.q, a.k, a.v = q.storage.ptr, k.storage.ptr, v.storage.ptr
    return a


def attention_forward(q, k, v, heads, kv_heads, stream=0):
    """Returns ``(out, lse)`` as device storages (bfloat16 [batch * time * heads * dim], float32 [batch * time * heads])."""
    a = _describe(q, k, v, heads, kv_heads)
    out = DeviceStorage(q.storage.size, "bfloat16")
    lse = DeviceStorage(a.batch * a.time * a.heads, "float32")
    a.out, a.lse = out.ptr, lse.ptr
    lib.call("qmoe_attention_forward", ctypes.byref(a), stream)
    return out, lse


def attention_backward(gradient, q, k, v, out, lse, heads, kv_heads, stream=0):
    """``gradient``: storage (or tensor) like ``out``.  Returns ``(dq, dk, dv)`` as device storages."""
    a = _describe(q, k, v, heads, kv_heads)
    gradient = getattr(gradient, "storage", gradient)
    if gradient.dtype != "bfloat16" or gradient.size != q.storage.size:
        raise ValueError("the gradient must be bfloat16 and shaped like the output")
    dq = DeviceStorage(q.storage.size, "bfloat16")
    dk = DeviceStorage(k.storage.size, "bfloat16")
    dv = DeviceStorage(v.storage.size, "bfloat16")
    delta = DeviceStorage(lse.size, "float32")
    a.out, a.lse, a.grad_out, a.delta = out.ptr, lse.ptr, gradient.ptr, delta.ptr
    a.dq, a.dk, a.dv = dq.ptr, dk.ptr, dv.ptr
    lib.call("qmoe_attention_backward", ctypes.byref(a), stream)
    return dq, dk, dv


def attention(q, k, v, heads, kv_heads, stream=0):
    """Upstream's ``attention`` (src/qutai/lm/layers.py:119-130)."""
    out, lse = attention_forward(q, k, v, heads, kv_heads, stream)
    result = Tensor(out, q.shape)
    result.parents = (q, k, v)
    result.backward_rule = lambda gradient: attention_backward(gradient, q, k, v, out, lse, heads, kv_heads, stream)
    return result
