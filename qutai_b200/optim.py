"""``AdamW`` and ``clip_grad_norm`` for parameters that live on the device, mirroring the upstream
optimizer interface (src/qutai/nn/optimizers.py:19-31, :121-153): per-parameter step counters and moments,
parameters whose ``grad`` is ``None`` are skipped, ``clip_grad_norm`` returns the norm before clipping.

Upstream launches one kernel per parameter tensor; here every tensor that has a gradient goes into one
table and one launch (``qmoe_adamw_multi`` / ``qmoe_clip_grad_norm``).  When ``shadows`` maps a parameter
to a bf16 storage, the step also writes the rounded parameter there, so a layer whose tensor-core operands
are those storages need not convert its weights again (``SparseMoE.operand_shadows``).
"""
from __future__ import annotations

import ctypes
from math import isfinite

from . import lib
from .storage import DeviceStorage


def _parameters(source):
    """A model, a layer or an iterable of tensors; a shared parameter is kept once (upstream ``_parameters``)."""
    if hasattr(source, "parameters"):
        source = source.parameters()
    return tuple(dict.fromkeys(source))


class _Table:
    """Host item array plus the device buffer it is copied into, grown on demand."""

    def __init__(self):
        self.capacity, self.items, self.device = 0, None, None

    def fill(self, rows):
        if len(rows) > self.capacity:
            self.capacity = max(64, 2 * len(rows))
            self.items = (lib.OptimItem * self.capacity)()
            self.device = DeviceStorage(int(lib.load().qmoe_optim_table_bytes(self.capacity)) // 4, "int32")
        for item, (values, grad, average, square, shadow, size, c1, c2) in zip(self.items, rows):
            item.values, item.grad, item.exp_avg, item.exp_avg_sq, item.shadow = values, grad, average, square, shadow
            item.size, item.first_chunk, item.c1, item.c2 = size, 0, c1, c2
        return self.items, len(rows), self.device.ptr


def clip_grad_norm(parameters, max_norm=1.0, *, stream=0, scratch=None):
    """Scale all gradients so that their joint L2 norm is at most ``max_norm``; returns the norm before
    clipping (reading it waits for the device, as upstream's download does)."""
    if not isfinite(max_norm) or max_norm < 0:
        raise ValueError("max_norm must be a non-negative finite number")
    gradients = [p.grad for p in _parameters(parameters) if p.grad is not None]
    if not gradients:
        return 0.0
    if any(g.dtype != "float32" for g in gradients):
        raise ValueError("gradients must be float32")
    table = _Table()
    items, count, device = table.fill([(0, g.storage.ptr, 0, 0, 0, g.storage.size, 1.0, 1.0) for g in gradients])
    scratch = scratch or DeviceStorage(int(lib.load().qmoe_clip_scratch_bytes()) // 4, "int32")
    lib.call("qmoe_clip_grad_norm", items, count, device, float(max_norm), scratch.ptr, stream)
    host = (ctypes.c_double * 2)()
    lib.call("qmoe_memcpy_d2h", ctypes.cast(host, ctypes.c_void_p), scratch.ptr, 16, stream)
    lib.call("qmoe_stream_sync", stream)
    norm = float(host[0])
    if not isfinite(norm):
        raise ValueError("the gradients contain non-finite values")
    return norm


def clip_grad_norm_sharded(replicated, sharded, max_norm=1.0, *, stream=0):
    """``clip_grad_norm`` for one rank of an expert-parallel job (no counterpart upstream, which is single-device):
    the gradients of ``replicated`` parameters are the same on every rank and count once, those of ``sharded``
    parameters (this rank's experts) exist only here and count together with the other ranks'.  Every rank calls it
    at the same point; all return the same norm and scale by the same factor.  Built from the single-rank kernels:
    two passes that only measure (replicated, sharded), one all-reduce of the sharded square, and one pass over all
    local gradients whose limit is chosen so that the kernel's own ``max_norm / norm`` comes out as
    ``max_norm / joint norm``."""
    if not isfinite(max_norm) or max_norm < 0:
        raise ValueError("max_norm must be a non-negative finite number")
    replicated, sharded = _parameters(replicated), _parameters(sharded)
    measure_only = 1.7e308      # the largest limit the kernel takes: nothing is scaled, the norm is reported
    norm_replicated = clip_grad_norm(replicated, measure_only, stream=stream)
    norm_sharded = clip_grad_norm(sharded, measure_only, stream=stream)
    square = DeviceStorage.from_values([norm_sharded * norm_sharded], "float32", stream)
    lib.call("qmoe_ep_all_reduce_f32", square.ptr, 1, stream)
    joint = (norm_replicated * norm_replicated + float(square.tolist(stream)[0])) ** 0.5
    if not isfinite(joint):
        raise ValueError("the gradients contain non-finite values")
    local = (norm_replicated * norm_replicated + norm_sharded * norm_sharded) ** 0.5
    if joint > max_norm and local > 0:
        # the kernel scales by limit / local when local > limit: limit = max_norm * local / joint gives max_norm / joint
        clip_grad_norm(tuple(replicated) + tuple(sharded), max_norm * local / joint, stream=stream)
    return joint


class AdamW:
    """Adam with decoupled weight decay; state per parameter object (``steps``, ``averages``,
    ``square_averages``), created when the parameter first has a gradient."""

    def __init__(self, parameters, *, learning_rate=0.001, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 shadows=None, stream=0):
        if learning_rate < 0 or weight_decay < 0 or eps < 0:
            raise ValueError("learning rate, weight decay and eps must not be negative")
        if len(betas) != 2 or any(beta < 0 or beta >= 1 for beta in betas):
            raise ValueError("betas must be two numbers in [0, 1)")
        self.parameters = _parameters(parameters)
        if any(p.dtype != "float32" for p in self.parameters):
            raise ValueError("parameters must be float32")
        self.learning_rate, self.betas, self.eps, self.weight_decay = learning_rate, tuple(betas), eps, weight_decay
        self.shadows = dict(shadows or {})
        self.stream = stream
        self.steps, self.averages, self.square_averages = {}, {}, {}
        self._table = _Table()

    def zero_grad(self):
        for parameter in self.parameters:
            parameter.zero_grad()

    def step(self):
        beta1, beta2 = self.betas
        rows, updated = [], []
        for parameter in self.parameters:
            gradient = parameter.grad
            if gradient is None:
                continue
            if gradient.storage.size != parameter.storage.size or gradient.dtype != "float32":
                raise ValueError("a gradient must be float32 and have its parameter's size")
            step = self.steps.get(parameter, 0) + 1
            if parameter not in self.averages:
                self.averages[parameter] = DeviceStorage.zeros(parameter.storage.size, "float32", self.stream)
                self.square_averages[parameter] = DeviceStorage.zeros(parameter.storage.size, "float32", self.stream)
            shadow = self.shadows.get(parameter)
            if shadow is not None and (shadow.dtype != "bfloat16" or shadow.size != parameter.storage.size):
                raise ValueError("a shadow must be a bfloat16 storage of its parameter's size")
            rows.append((parameter.storage.ptr, gradient.storage.ptr, self.averages[parameter].ptr,
                         self.square_averages[parameter].ptr, shadow.ptr if shadow is not None else 0,
                         parameter.storage.size, 1 - beta1 ** step, 1 - beta2 ** step))
            self.steps[parameter] = step
            updated.append((parameter.storage, shadow))
        if not rows:
            return
        items, count, device = self._table.fill(rows)
        # Change tracking (storage.py): the parameters' generation grows.  A bf16 copy that was current before the
        # step and whose every updated part was rewritten by this launch is current afterwards as well; a copy of
        # an allocation in which some updated parameter had no shadow is left stale for its owner to rebuild.
        groups = {}
        for master, shadow in updated:
            group = groups.setdefault(id(master._root), dict(master=master, shadows={}, complete=True))
            if shadow is None:
                group["complete"] = False
            else:
                group["shadows"][id(shadow._root)] = shadow
        for group in groups.values():
            group["current"] = [s for s in group["shadows"].values() if group["complete"] and len(group["shadows"]) == 1
                                and s.is_derived_from(group["master"])]
        lib.call("qmoe_adamw_multi", items, count, device, self.learning_rate, beta1, beta2, self.eps, self.weight_decay,
                 self.stream)
        for group in groups.values():
            group["master"].touch()
            for shadow in group["current"]:
                shadow.mark_derived_from(group["master"])
