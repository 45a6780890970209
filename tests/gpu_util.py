"""Helpers for the GPU parity tests: move numpy arrays to device storages and back, and run the
layer through the C ABI.  The oracle is imported here only as the checker."""
import ctypes

import numpy as np

from qutai_b200 import lib
from qutai_b200.storage import DeviceStorage


def bf16_bytes(a):
    """numpy float array -> bytes of bfloat16 (round to nearest even)."""
    a32 = np.ascontiguousarray(np.asarray(a, dtype=np.float32))
    bits = a32.view(np.uint32).astype(np.uint64)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16).tobytes()


def to_device(a, dtype):
    a = np.asarray(a)
    if dtype == "bfloat16":
        return DeviceStorage.from_bytes(bf16_bytes(a), "bfloat16")
    np_dtype = {"float32": np.float32, "int32": np.int32, "int64": np.int64}[dtype]
    return DeviceStorage.from_bytes(np.ascontiguousarray(a, dtype=np_dtype).tobytes(), dtype)


def to_host(storage, shape=None):
    data = storage.tobytes()
    if storage.dtype == "bfloat16":
        out = (np.frombuffer(data, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    else:
        np_dtype = {"float32": np.float32, "int32": np.int32, "int64": np.int64}[storage.dtype]
        out = np.frombuffer(data, dtype=np_dtype).copy()
        if storage.dtype == "float32":
            out = out.astype(np.float64)
    return out if shape is None else out.reshape(shape)


class RouteTables:
    """Caller-allocated routing tables + the ``qmoe_route_t`` that points at them."""

    def __init__(self, tokens, experts, top_k):
        self.tokens, self.experts, self.top_k = tokens, experts, top_k
        A, R, blocks = tokens * top_k, lib.rows_bound(tokens, experts, top_k), lib.route_blocks(tokens)
        S = DeviceStorage
        self.rows_bound = R
        self.buf = dict(
            probs=S(tokens * experts, "float32"), gate_weights=S(A, "float32"), expert_index=S(A, "int32"),
            dest_row=S(A, "int32"), row_source=S(R, "int32"), counts=S(experts, "int32"),
            offsets=S(experts + 1, "int32"), tile_expert=S(R // lib.ROW_PAD, "int32"), meta=S(4, "int32"),
            utilization=S(experts, "float32"), aux=S(1, "float32"), block_counts=S(blocks * experts, "int32"),
            block_base=S(blocks * experts, "int32"), block_colsum=S(blocks * experts, "float32"))
        self.struct = lib.Route()
        self.struct.tokens, self.struct.experts, self.struct.top_k, self.struct.rows_bound = tokens, experts, top_k, R
        for name, storage in self.buf.items():
            setattr(self.struct, name, storage.ptr)

    @property
    def ref(self):
        return ctypes.byref(self.struct)

    def run(self, scores):
        lib.call("qmoe_route", self.ref, scores.ptr, 0)

    def host(self, name, shape=None):
        return to_host(self.buf[name], shape)

    def export_i64(self):
        A, E = self.tokens * self.top_k, self.experts
        out = dict(indices=DeviceStorage(A, "int64"), ids=DeviceStorage(E * A, "int64"),
                   slots=DeviceStorage(E * A, "int64"), locations=DeviceStorage(A, "int64"),
                   counts=DeviceStorage(E, "int64"))
        lib.call("qmoe_route_export_i64", self.ref, out["indices"].ptr, out["ids"].ptr, out["slots"].ptr,
                 out["locations"].ptr, out["counts"].ptr, A, 0)
        return {k: to_host(v) for k, v in out.items()}


def check_route_against_oracle(tables, expected, float_tol=2e-6):
    """Integer tables exactly, floats within ``float_tol``; ``expected`` is the oracle's dict."""
    T, E, k = tables.tokens, tables.experts, tables.top_k
    A = T * k
    assert np.array_equal(tables.host("expert_index", (T, k)), expected["indices"])
    counts = tables.host("counts")
    assert tuple(counts.tolist()) == expected["counts"]
    offsets = tables.host("offsets")
    pad = lib.ROW_PAD
    assert offsets[0] == 0
    for e in range(E):
        assert offsets[e] % pad == 0 and offsets[e + 1] - offsets[e] == -(-counts[e] // pad) * pad
    meta = tables.host("meta")
    assert meta[0] == offsets[E] and meta[1] == offsets[E] // pad and meta[2] == A
    dest = tables.host("dest_row")
    source = tables.host("row_source")[: offsets[E]]
    # dispatched rows of expert e hold its assignments in increasing (token, slot) order, pads are -1
    for e in range(E):
        want = expected["ids"][e] * k + expected["slots"][e]
        got = source[offsets[e]: offsets[e] + counts[e]]
        assert np.array_equal(got, want)
        assert np.all(source[offsets[e] + counts[e]: offsets[e + 1]] == -1)
        assert np.array_equal(dest[want], offsets[e] + np.arange(counts[e]))
    tiles = tables.host("tile_expert")[: meta[1]]
    for e in range(E):
        assert np.all(tiles[offsets[e] // pad: offsets[e + 1] // pad] == e)
    exported = tables.export_i64()
    assert np.array_equal(exported["indices"].reshape(T, k), expected["indices"])
    assert np.array_equal(exported["locations"].reshape(T, k), expected["locations"])
    assert tuple(exported["counts"].tolist()) == expected["counts"]
    for e in range(E):
        assert np.array_equal(exported["ids"][e * A: e * A + counts[e]], expected["ids"][e])
        assert np.array_equal(exported["slots"][e * A: e * A + counts[e]], expected["slots"][e])
    assert np.abs(tables.host("probs", (T, E)) - expected["probs"]).max() <= float_tol
    assert np.abs(tables.host("gate_weights", (T, k)) - expected["weights"]).max() <= float_tol
    assert np.abs(tables.host("utilization") - expected["utilization"]).max() <= float_tol
    assert abs(tables.host("aux")[0] - expected["aux"]) <= 4 * float_tol * max(1.0, abs(expected["aux"]))


class Config:
    """The fields of the upstream ``Config`` (src/qutai/lm/config.py:5-21) this layer reads."""

    def __init__(self, d_model, n_experts, top_k, d_expert, n_layers=1):
        self.d_model, self.n_experts, self.top_k, self.d_expert, self.n_layers = d_model, n_experts, top_k, d_expert, n_layers


def make_layer(x_shape, router, gate, up, down, top_k, engine="auto"):
    """A ``qutai_b200.layers.SparseMoE`` whose parameters are overwritten with the given arrays
    (the upstream parity tests copy weights the same way, tests/test_lm_moe.py:105-108)."""
    from qutai_b200.layers import SparseMoE

    experts, hidden, width = gate.shape[0], gate.shape[1], gate.shape[2]
    layer = SparseMoE(Config(width, experts, top_k, hidden), device="cuda", dtype="float32", seed=1, engine=engine)
    layer.router.weight.storage.upload_bytes(np.ascontiguousarray(router, dtype=np.float32).tobytes())
    layer._gate.upload_bytes(np.ascontiguousarray(gate, dtype=np.float32).tobytes())
    layer._up.upload_bytes(np.ascontiguousarray(up, dtype=np.float32).tobytes())
    layer._down.upload_bytes(np.ascontiguousarray(down, dtype=np.float32).tobytes())
    return layer


def run_layer(layer, x, grad_y, grad_aux, dtype):
    """Forward + backward through the public layer; returns numpy results and the fp32 logits."""
    from qutai_b200.layers import Tensor

    T, d = x.shape
    E, h = layer.n_experts, layer.d_expert
    for p in layer.parameters():
        p.zero_grad()
    xs = to_device(x, dtype)
    y, aux = layer(Tensor(xs, (T, d)))
    ga = to_device(np.array([grad_aux]), "float32") if grad_aux is not None else None
    dx = layer.backward(Tensor(to_device(grad_y, dtype), (T, d)), ga)
    work = layer._saved[0]
    out = dict(
        y=to_host(y.storage, (T, d)), aux=float(to_host(aux.storage)[0]), dx=to_host(dx.storage, (T, d)),
        counts=layer.last_counts, scores=to_host(work["buf"]["scores"], (T, E)),
        utilization=to_host(layer.utilization.storage),
        d_router=to_host(layer.router.weight.grad.storage, (E, d)),
        d_gate=[None if ex.gate.weight.grad is None else to_host(ex.gate.weight.grad.storage, (h, d)) for ex in layer.experts],
        d_up=[None if ex.up.weight.grad is None else to_host(ex.up.weight.grad.storage, (h, d)) for ex in layer.experts],
        d_down=[None if ex.down.weight.grad is None else to_host(ex.down.weight.grad.storage, (d, h)) for ex in layer.experts],
    )
    assert lib.device_status() == 0, "a kernel recorded a failed self-check"
    return out
