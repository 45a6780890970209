"""Backend function table for ``device="cuda"`` on B200: the MoE subset of the upstream
``qutai.backends.cuda_lm`` (same function names, argument meaning and error behaviour), implemented
over ``libqutai_moe.so``.

Upstream selects a backend *module* per device and calls ``b.<name>(storage, ...)``
(src/qutai/lm/layers.py:9-17).  A host that keeps that per-op structure can point the MoE ops at
this module; storages only need ``ptr`` / ``size`` / ``dtype`` (the upstream ``CUDAStorage`` has
them).  The fused layer of ``qutai_b200.layers`` is the fast path; this table exists so that code
written against the upstream per-expert functions keeps working, and it does strictly more device
work (one dispatched buffer per call where upstream had one buffer per expert).

``route`` is the upstream dict (``weights, aux, counts, utilization, rows, experts, top_k, probs,
indices, ids, slots, locations, capacity``; src/qutai/backends/cuda_lm.py:435-449) plus a private
``_tables`` entry holding this library's routing tables.  As upstream, ``routing`` waits for the
device once to return ``counts`` as Python ints (src/qutai/backends/cuda_lm.py:432-434).
"""
from __future__ import annotations

import ctypes

from . import lib
from .storage import DeviceStorage

_REAL = ("float32", "bfloat16")


def _code(dtype):
    if dtype not in lib.DTYPE_CODES:
        raise ValueError(f"dtype {dtype!r} is not supported on this path (float32 or bfloat16)")
    return lib.DTYPE_CODES[dtype]


def normal(size, mean=0.0, std=1.0, *, seed=None, dtype="float32"):
    """N(mean, std) draws (src/qutai/backends/cuda_lm.py:27-28).  Like upstream, the generator's
    stream differs from the CPU backend's for the same seed."""
    out = DeviceStorage(size, dtype)
    lib.call("qmoe_normal_fill", out.ptr, _code(dtype), size, float(mean), float(std),
             (0x5EED if seed is None else seed) & (2 ** 64 - 1), 0)
    return out


def gemm(a, b, rows, inner, cols, *, transpose_left=False, transpose_right=False, out_dtype=None, out=None,
         accumulate=False):
    """``C[rows, cols] = op(A) op(B)`` with the upstream dispatcher's checks
    (src/qutai/backends/cuda.py:305-334): float32 / bfloat16 operands, fp32 accumulation, optional
    ``out`` (must not overlap an input) and ``accumulate``."""
    for value in (a, b):
        if not hasattr(value, "ptr") or value.dtype not in _REAL:
            raise ValueError("GEMM inputs must be device storages of float32 or bfloat16")
    dtype = "float32" if out_dtype is None else out_dtype
    if dtype not in _REAL:
        raise ValueError("GEMM output dtype must be float32 or bfloat16")
    if any(type(x) is not int or x < 0 for x in (rows, inner, cols)):
        raise ValueError("GEMM sizes must be non-negative integers")
    if a.size < rows * inner or b.size < inner * cols:
        raise ValueError("GEMM input storage is too small")
    if accumulate and out is None:
        raise ValueError("an accumulating GEMM needs out")
    size = rows * cols
    if out is not None:
        if not hasattr(out, "ptr") or out.dtype != dtype or out.size != size:
            raise ValueError("GEMM out has the wrong dtype or size")
        for value in (a, b):
            if out.nbytes and value.nbytes and out.ptr < value.ptr + value.nbytes and value.ptr < out.ptr + out.nbytes:
                raise ValueError("GEMM out must not share storage with an input")
    result = out if out is not None else DeviceStorage(size, dtype)
    if not size:
        return result
    if not inner:
        if not accumulate:
            result.fill_zero()
        return result
    lib.call("qmoe_gemm", a.ptr, _code(a.dtype), b.ptr, _code(b.dtype), result.ptr, _code(dtype), rows, inner, cols,
             1 if transpose_left else 0, 1 if transpose_right else 0, 1 if accumulate else 0, 0)
    return result


def take(values, start, size):
    """Copy of ``values[start:start + size]`` (src/qutai/backends/cuda_lm.py:58-63)."""
    out = DeviceStorage(size, values.dtype)
    lib.call("qmoe_memcpy_d2d", out.ptr, values.ptr + start * lib.ITEM_BYTES[values.dtype], out.nbytes, 0)
    return out


def add_into(target, source):
    """``target += source`` (src/qutai/backends/cuda_lm.py:66-75)."""
    lib.call("qmoe_add", target.ptr, source.ptr, target.ptr, _code(target.dtype), target.size, 0)


def silu(values):
    """src/qutai/backends/cuda_lm.py:180-192."""
    out = DeviceStorage(values.size, values.dtype)
    lib.call("qmoe_silu", values.ptr, 0, out.ptr, _code(values.dtype), values.size, 0, 0)
    return out


def silu_backward(gradient, values):
    """src/qutai/backends/cuda_lm.py:195-207."""
    out = DeviceStorage(values.size, values.dtype)
    lib.call("qmoe_silu", values.ptr, gradient.ptr, out.ptr, _code(values.dtype), values.size, 1, 0)
    return out


# ------------------------------------------------------------------------------------------------
# routing
# ------------------------------------------------------------------------------------------------
class _Tables:
    """Caller-allocated routing tables and the ``qmoe_route_t`` pointing at them."""

    def __init__(self, rows, experts, top_k):
        A, R, blocks = rows * top_k, lib.rows_bound(rows, experts, top_k), lib.route_blocks(rows)
        S = DeviceStorage
        self.rows_bound = R
        self.buf = dict(
            probs=S(rows * experts, "float32"), gate_weights=S(A, "float32"), expert_index=S(A, "int32"),
            dest_row=S(A, "int32"), row_source=S(R, "int32"), counts=S(experts, "int32"), offsets=S(experts + 1, "int32"),
            tile_expert=S(R // lib.ROW_PAD, "int32"), meta=S(4, "int32"), utilization=S(experts, "float32"),
            aux=S(1, "float32"), block_counts=S(blocks * experts, "int32"), block_base=S(blocks * experts, "int32"),
            block_colsum=S(blocks * experts, "float32"))
        self.struct = lib.Route()
        self.struct.tokens, self.struct.experts, self.struct.top_k, self.struct.rows_bound = rows, experts, top_k, R
        for name, storage in self.buf.items():
            setattr(self.struct, name, storage.ptr)

    def ref(self, weights=None):
        """The struct, optionally with another gate-weight storage in place of the routed one."""
        if weights is None or weights.ptr == self.buf["gate_weights"].ptr:
            return ctypes.byref(self.struct)
        other = lib.Route.from_buffer_copy(self.struct)
        other.gate_weights = weights.ptr
        self._keep = other
        return ctypes.byref(other)


def routing(scores, rows, experts, top_k):
    """Softmax / top-k gating and the dispatch tables (src/qutai/backends/cuda_lm.py:368-449,
    CPU statement src/qutai/backends/cpu_lm.py:204-242).  bfloat16 scores are widened first, as
    upstream does."""
    if scores.size != rows * experts:
        raise ValueError("scores do not match rows * experts")
    if scores.dtype == "bfloat16":
        wide = DeviceStorage(scores.size, "float32")
        lib.call("qmoe_gemm", scores.ptr, lib.QMOE_BF16, _one().ptr, lib.QMOE_F32, wide.ptr, lib.QMOE_F32,
                 scores.size, 1, 1, 0, 0, 0, 0)  # [n, 1] x [1, 1] product with 1.0: an exact widening copy
        scores = wide
    elif scores.dtype != "float32":
        raise ValueError("scores must be float32 or bfloat16")
    tables = _Tables(rows, experts, top_k)
    lib.call("qmoe_route", tables.ref(), scores.ptr, 0)
    capacity = rows * top_k
    indices, locations = DeviceStorage(capacity, "int64"), DeviceStorage(capacity, "int64")
    ids, slots = DeviceStorage(experts * capacity, "int64"), DeviceStorage(experts * capacity, "int64")
    counts64 = DeviceStorage(experts, "int64")
    lib.call("qmoe_route_export_i64", tables.ref(), indices.ptr, ids.ptr, slots.ptr, locations.ptr, counts64.ptr, capacity, 0)
    counts = tuple(counts64.tolist())  # the one host wait: integer counts decide the GEMM shapes
    offsets = tuple(tables.buf["offsets"].tolist())
    return dict(probs=tables.buf["probs"], weights=tables.buf["gate_weights"], indices=indices, counts=counts, ids=ids,
                slots=slots, locations=locations, utilization=tables.buf["utilization"], aux=tables.buf["aux"], rows=rows,
                experts=experts, top_k=top_k, capacity=capacity, _tables=tables, _offsets=offsets, _dispatched={})


_ONE = []


def _one():
    if not _ONE:
        _ONE.append(DeviceStorage.from_values([1.0], "float32"))
    return _ONE[0]


def routing_backward(gradient, route, auxiliary=False):
    """d(scores) of the gate weights, or of the auxiliary loss when ``auxiliary``
    (src/qutai/backends/cuda_lm.py:452-468)."""
    out = DeviceStorage(route["rows"] * route["experts"], "float32")
    tables = route["_tables"]
    if auxiliary:
        lib.call("qmoe_route_backward", tables.ref(), 0, gradient.ptr, out.ptr, 0)
    else:
        lib.call("qmoe_route_backward", tables.ref(), gradient.ptr, 0, out.ptr, 0)
    return out


def _expert_rows(route, expert):
    return route["_offsets"][expert], route["counts"][expert]


def route_gather(values, route, expert, width):
    """Rows of ``values`` routed to ``expert`` (src/qutai/backends/cuda_lm.py:471-485).  All experts
    are gathered by one launch the first time; later calls for the same ``values`` return views."""
    key = (values.ptr, width, values.dtype)
    cache = route["_dispatched"]
    if key not in cache:
        tables = route["_tables"]
        dispatched = DeviceStorage(tables.rows_bound * width, values.dtype)
        lib.call("qmoe_permute", tables.ref(), values.ptr, dispatched.ptr, _code(values.dtype), width, 0)
        cache.clear()  # one input at a time keeps memory bounded
        cache[key] = dispatched
    start, count = _expert_rows(route, expert)
    return cache[key].view(start * width, count * width)


def _assemble(route, pairs, width, dtype):
    """Dispatched buffer holding every given expert's rows (zero elsewhere)."""
    tables = route["_tables"]
    buffer = DeviceStorage.zeros(tables.rows_bound * width, dtype)
    item = lib.ITEM_BYTES[dtype]
    for expert, values in pairs:
        start, count = _expert_rows(route, expert)
        if values.size != count * width or values.dtype != dtype:
            raise ValueError(f"expert {expert}: expected {count} x {width} values of {dtype}")
        lib.call("qmoe_memcpy_d2d", buffer.ptr + start * width * item, values.ptr, values.nbytes, 0)
    return buffer


def route_gather_backward(gradient, route, expert, width):
    """(rows, width) zeros with the expert's gradient rows scattered back
    (src/qutai/backends/cuda_lm.py:488-502)."""
    tables = route["_tables"]
    buffer = _assemble(route, ((expert, gradient),), width, gradient.dtype)
    out = DeviceStorage(route["rows"] * width, gradient.dtype)
    lib.call("qmoe_unpermute_reduce", tables.ref(), buffer.ptr, 0, out.ptr, _code(gradient.dtype), width, 0)
    return out


def combine(outputs, weights, route, width):
    """``out[row] = sum_slot weights[row, slot] * y_expert[location]`` in fp32, rounded once to the
    experts' dtype (src/qutai/backends/cuda_lm.py:521-541); ``outputs = ((expert, storage), ...)``."""
    dtype = outputs[0][1].dtype if outputs else weights.dtype
    tables = route["_tables"]
    buffer = _assemble(route, outputs, width, dtype)
    out = DeviceStorage(route["rows"] * width, dtype)
    lib.call("qmoe_combine", tables.ref(weights), buffer.ptr, out.ptr, _code(dtype), width, 0)
    return out


def combine_backward(gradient, outputs, weights, route, width):
    """``(*dy_per_expert, dw)``: ``dy = g[row] * weight`` in the experts' dtype, ``dw = <g[row], y>``
    in float32 (src/qutai/backends/cuda_lm.py:544-581)."""
    dtype = outputs[0][1].dtype if outputs else gradient.dtype
    tables = route["_tables"]
    buffer = _assemble(route, outputs, width, dtype)
    dy = DeviceStorage(tables.rows_bound * width, dtype)
    dw = DeviceStorage.zeros(weights.size, "float32")
    lib.call("qmoe_combine_backward", tables.ref(weights), gradient.ptr, buffer.ptr, dy.ptr, dw.ptr, _code(dtype), width, 0)
    grads = []
    for expert, _ in outputs:
        start, count = _expert_rows(route, expert)
        grads.append(dy.view(start * width, count * width))
    return (*grads, dw)


# ------------------------------------------------------------------------------------------------
# the operations around attention and the feed-forward half of a block
# ------------------------------------------------------------------------------------------------
def _acc_dtype(dtype):
    """Upstream's accumulation dtype (src/qutai/backends/cuda_lm.py:9-10): bfloat16 activations are paired with
    float32 weights, statistics and norm outputs."""
    return "float32" if dtype == "bfloat16" else dtype


def embedding(weight, ids, width, *, out_dtype=None):
    """Rows ``ids`` of the float32 table ``weight`` (src/qutai/backends/cuda_lm.py:77-93)."""
    dtype = out_dtype or weight.dtype
    if _acc_dtype(dtype) != weight.dtype or weight.dtype != "float32":
        raise ValueError("the embedding table must be float32 and the output float32 or bfloat16")
    ids = list(ids)
    identifiers = DeviceStorage.from_values(ids, "int64")
    result = DeviceStorage(len(ids) * width, dtype)
    if ids:
        lib.call("qmoe_embedding", weight.ptr, identifiers.ptr, result.ptr, _code(dtype), len(ids), width, weight.size // width, 0)
    return result


def embedding_backward(gradient, ids, count, width):
    """Gradient of the table, ``[count, width]`` float32: row ``token`` is the sum of the gradient rows of the
    positions that held it, added in ascending position order (src/qutai/backends/cuda_lm.py:96-123 builds the same
    three tables on the host)."""
    groups = {}
    for row, token in enumerate(ids):
        groups.setdefault(token, []).append(row)
    tokens = sorted(groups)
    starts, positions = [0], []
    for token in tokens:
        positions.extend(groups[token])
        starts.append(len(positions))
    result = DeviceStorage.zeros(count * width, _acc_dtype(gradient.dtype))
    if tokens:
        tables = [DeviceStorage.from_values(values, "int64") for values in (tokens, starts, positions)]
        lib.call("qmoe_embedding_backward", gradient.ptr, _code(gradient.dtype), tables[0].ptr, tables[1].ptr, tables[2].ptr,
                 result.ptr, len(tokens), len(positions), width, count, 0)
    return result


def rms_norm(values, weight, width, eps):
    """``(out, inverse)``, both in the accumulation dtype (src/qutai/backends/cuda_lm.py:126-145)."""
    rows = values.size // width
    out = DeviceStorage(values.size, _acc_dtype(values.dtype))
    inverse = DeviceStorage(rows, "float32")
    lib.call("qmoe_rms_norm", values.ptr, _code(values.dtype), weight.ptr, out.ptr, _code(out.dtype), inverse.ptr, rows, width,
             float(eps), 0)
    return out, inverse


def rms_norm_backward(gradient, values, weight, inverse, width):
    """``(dx, dw)``: ``dx`` in the dtype of ``values``, ``dw`` float32 (src/qutai/backends/cuda_lm.py:148-177)."""
    rows = inverse.size
    dx = DeviceStorage(values.size, values.dtype)
    dw = DeviceStorage(width, "float32")
    partials = DeviceStorage(lib.load().qmoe_rms_norm_partials(rows, width), "float32")
    lib.call("qmoe_rms_norm_backward", gradient.ptr, _code(gradient.dtype), values.ptr, _code(values.dtype), weight.ptr,
             inverse.ptr, dx.ptr, dw.ptr, partials.ptr, rows, width, 0)
    return dx, dw


def rope(values, batch, time, heads, dim, theta, offset=0, inverse=False):
    """Rotary position embedding (src/qutai/backends/cuda_lm.py:210-226); ``inverse`` is its backward."""
    result = DeviceStorage(values.size, values.dtype)
    lib.call("qmoe_rope", values.ptr, result.ptr, _code(values.dtype), batch, time, heads, dim, float(theta), int(offset),
             1 if inverse else 0, 0)
    return result


class _View:
    """A storage seen as a tensor of some shape (what ``qutai_b200.attention`` reads: ``storage`` and ``shape``)."""

    def __init__(self, storage, shape):
        self.storage, self.shape = storage, shape


def attention(q, k, v, batch, time, heads, kv_heads, dim):
    """``(out, lse)`` of causal attention with grouped key/value heads (src/qutai/backends/cuda_lm.py:229-275):
    bfloat16 and head width 64 on the tensor cores; anything else raises ``ValueError`` (upstream serves it with
    its CUDA-core kernel)."""
    from .attention import attention_forward

    return attention_forward(_View(q, (batch, time, heads * dim)), _View(k, (batch, time, kv_heads * dim)),
                             _View(v, (batch, time, kv_heads * dim)), heads, kv_heads)


def attention_backward(gradient, q, k, v, out, lse, batch, time, heads, kv_heads, dim):
    """``(dq, dk, dv)`` (src/qutai/backends/cuda_lm.py:278-365)."""
    from .attention import attention_backward as backward

    return backward(gradient, _View(q, (batch, time, heads * dim)), _View(k, (batch, time, kv_heads * dim)),
                    _View(v, (batch, time, kv_heads * dim)), out, lse, heads, kv_heads)


# ------------------------------------------------------------------------------------------------
# the language-model head, chunk by chunk (the fused form is qutai_b200.head)
# ------------------------------------------------------------------------------------------------
def head_rows(values, start, count, width, time):
    """Rows ``start .. start + count`` of the head's inputs: every position but the last of each sequence
    (src/qutai/backends/cuda_lm.py:584-598)."""
    out = DeviceStorage(count * width, values.dtype)
    if count:
        lib.call("qmoe_head_rows", values.ptr, out.ptr, _code(values.dtype), start, count, width, time, 0, 0)
    return out


def head_rows_backward(target, gradient, start, count, width, time):
    """``target[position(start + i)] += gradient[i]`` (src/qutai/backends/cuda_lm.py:601-613)."""
    if count:
        lib.call("qmoe_head_rows", gradient.ptr, target.ptr, _code(target.dtype), start, count, width, time, 1, 0)


def prepare_labels(labels):
    """The targets as an int64 device storage (src/qutai/backends/cuda_lm.py:616-617)."""
    return DeviceStorage.from_values(list(labels), "int64")


def head_loss(logits, labels, rows, vocab, *, start=0):
    """One-element float32 storage: the sum over the chunk's counted rows of ``log sum exp - picked logit``
    (src/qutai/backends/cuda_lm.py:629-643); ``labels`` from ``prepare_labels``."""
    out = DeviceStorage(1, "float32")
    scratch = DeviceStorage(rows, "float32")
    lib.call("qmoe_head_loss", logits.ptr, _code(logits.dtype), labels.ptr, scratch.ptr, out.ptr, rows, vocab, start, 0)
    return out


def head_gradient(logits, labels, rows, vocab, gradient, count, *, start=0):
    """``logits`` overwritten by ``gradient[0] / count * (softmax - one_hot)``, zero rows where the label is -100
    (src/qutai/backends/cuda_lm.py:646-660).  Returns ``logits``."""
    factor = DeviceStorage(1, "float32")
    lib.call("qmoe_head_gradient", logits.ptr, _code(logits.dtype), labels.ptr, gradient.ptr, factor.ptr, int(count), rows, vocab, start, 0)
    return logits
