"""The language-model head with its cross-entropy loss, over ``qmoe_head_forward`` / ``qmoe_head_backward``.

Upstream's ``projection_loss(hidden, weight, labels, chunk_size, *, prepared_labels=None)``
(src/qutai/lm/layers.py:187-257, called from ``Decoder.loss`` src/qutai/lm/decoder.py:143-175) drops the last
position of every sequence, multiplies by the (tied embedding) weight chunk by chunk, takes each row's
``log sum exp - picked logit`` for labels other than -100 and divides by the number of counted rows; its backward
forms every chunk's logits again.  ``projection_loss`` here keeps that signature and meaning — ``chunk_size`` is
accepted and ignored: the logits of all rows are formed once and kept (see ``csrc/head.cu``) — and returns a tensor
whose ``parents`` / ``backward_rule`` are what upstream's ``record`` would have filled in, so either autograd can
walk it.  Dependency-free: ctypes and the standard library only.
"""
from __future__ import annotations

import ctypes
from array import array

from . import lib
from .layers import Tensor
from .storage import DeviceStorage

ROW_PAD = 128


def prepare_labels(labels, stream=0):
    """Token ids ``[batch][time]`` (nested sequences, -100 = no target) as an int64 device storage, the form
    ``projection_loss`` takes as ``prepared_labels``.  Upstream's ``prepare_labels`` uploads the targets
    ``row[1:]`` of every sequence (src/qutai/lm/layers.py:193-196, src/qutai/backends/cuda_lm.py); here the whole
    ``[batch, time]`` table goes up and the kernels read position ``t + 1`` for row ``t``."""
    flat = array("q", (int(label) for row in labels for label in row))
    return DeviceStorage.from_bytes(flat.tobytes(), "int64", stream)


class LMHead:
    """Buffers and the two calls of one head.  ``forward`` leaves the loss (fp32 scalar on the device) and keeps
    the gradient of the logits; ``backward`` returns ``(d_hidden, d_weight)``."""

    def __init__(self, stream=0):
        self.stream = stream
        self._buffers, self._key = {}, None
        self._operand = None      # bf16 copy of an fp32 weight
        self._call = None

    def _buffer(self, name, size, dtype):
        current = self._buffers.get(name)
        if current is None or current.size < size or current.dtype != dtype:
            current = self._buffers[name] = DeviceStorage(size, dtype)
        return current

    def _weight_operand(self, weight, dtype):
        if weight.storage.dtype == dtype:
            return weight.storage
        if weight.storage.dtype != "float32" or dtype != "bfloat16":
            raise ValueError("the head's weight must have the activations' dtype, or be float32 with bfloat16 activations")
        shadow = self._operand
        if shadow is None or shadow.size != weight.storage.size:
            shadow = self._operand = DeviceStorage(weight.storage.size, "bfloat16")
        if not shadow.is_derived_from(weight.storage):
            lib.call("qmoe_cast_bf16", weight.storage.ptr, shadow.ptr, weight.storage.size, self.stream)
            shadow.mark_derived_from(weight.storage)
        return shadow

    def forward(self, hidden, weight, labels):
        """``hidden`` [batch, time, width] (bfloat16 or float32), ``weight`` [vocab, width], ``labels`` an int64
        device storage of batch * time token ids (``prepare_labels``) or nested sequences."""
        if len(hidden.shape) != 3 or len(weight.shape) != 2 or weight.shape[1] != hidden.shape[2]:
            raise ValueError("hidden must be [batch, time, width] and weight [vocab, width]")
        batch, time, width = hidden.shape
        vocab = weight.shape[0]
        if time < 2:
            raise ValueError("a sequence needs at least two positions to have a target")
        dtype = hidden.storage.dtype
        if dtype not in lib.DTYPE_CODES:
            raise ValueError("hidden must be float32 or bfloat16")
        if not isinstance(labels, DeviceStorage):
            labels = prepare_labels(labels, self.stream)
        if labels.dtype != "int64" or labels.size != batch * time:
            raise ValueError("labels must hold batch * time int64 token ids")
        rows = batch * (time - 1)
        bound = (rows + ROW_PAD - 1) // ROW_PAD * ROW_PAD
        operand = self._weight_operand(weight, dtype)
        h = lib.Head()
        h.batch, h.time, h.dtype, h.width, h.vocab, h.rows_bound = batch, time, lib.DTYPE_CODES[dtype], width, vocab, bound
        h.hidden, h.weight, h.labels = hidden.storage.ptr, operand.ptr, labels.ptr
        h.inputs = self._buffer("inputs", bound * width, dtype).ptr
        h.logits = self._buffer("logits", bound * vocab, dtype).ptr
        h.row_loss = self._buffer("row_loss", rows, "float32").ptr
        h.meta = self._buffer("meta", 8, "float32").ptr
        loss = DeviceStorage(1, "float32")
        h.loss = loss.ptr
        lib.call("qmoe_head_forward", ctypes.byref(h), self.stream)
        self._call = (h, hidden, weight, labels, loss)
        return Tensor(loss, ())

    def backward(self, gradient=None, *, need_hidden=True, need_weight=True):
        """``gradient``: fp32 device storage (or tensor) of one element, ``None`` = 1.  Returns ``(d_hidden,
        d_weight)`` — the first in the dtype of ``hidden`` with zero rows at the last positions, the second fp32 —
        ``None`` for the one not asked for."""
        if self._call is None:
            raise RuntimeError("backward needs a forward first")
        h, hidden, weight, labels, loss = self._call
        dtype = hidden.storage.dtype
        d_hidden = d_weight = None
        h.d_inputs = h.d_hidden = h.d_weight = 0
        if need_hidden:
            d_hidden = DeviceStorage(hidden.storage.size, dtype)
            h.d_inputs = self._buffer("d_inputs", h.rows_bound * h.width, dtype).ptr
            h.d_hidden = d_hidden.ptr
        if need_weight:
            d_weight = DeviceStorage(weight.storage.size, "float32")
            h.d_weight = d_weight.ptr
        if not (need_hidden or need_weight):
            return None, None
        storage = getattr(gradient, "storage", gradient)
        if storage is not None and (storage.dtype != "float32" or storage.size != 1):
            raise ValueError("the incoming gradient must be one float32 value on the device")
        lib.call("qmoe_head_backward", ctypes.byref(h), 0 if storage is None else storage.ptr, self.stream)
        return (None if d_hidden is None else Tensor(d_hidden, hidden.shape),
                None if d_weight is None else Tensor(d_weight, weight.shape))


def projection_loss(hidden, weight, labels, chunk_size=None, *, prepared_labels=None, head=None):
    """Upstream's ``projection_loss`` (src/qutai/lm/layers.py:187-257): the mean cross-entropy of predicting token
    ``t + 1`` from position ``t``.  Returns the loss as a tensor recorded with parents ``(hidden, weight)``."""
    head = head or LMHead()
    loss = head.forward(hidden, weight, labels if prepared_labels is None else prepared_labels)

    def backward(gradient):
        d_hidden, d_weight = head.backward(gradient, need_hidden=getattr(hidden, "requires_grad", True),
                                           need_weight=getattr(weight, "requires_grad", True))
        return (None if d_hidden is None else d_hidden.storage, None if d_weight is None else d_weight.storage)

    loss.parents, loss.backward_rule = (hidden, weight), backward
    return loss
