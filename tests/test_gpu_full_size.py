"""Parity at the full benchmark sizes (C2: 16384 tokens, d 1024, 8 experts top-2, hidden 2816; C3: 32768
tokens, d 2048, 64 experts top-6, hidden 1408; one layer of C4: 65536 tokens, d 1024, 16 experts top-2, hidden
2048; bf16 activations, tcgen05 engine), where the float64 oracle cannot run the whole layer in seconds, and
the whole layer at the decode shape C5 (64 tokens on C3's layer), which it can.  What is checked at the full sizes:

* routing tables bit-exact against the oracle on the device's own fp32 logits (the oracle's routing is
  vectorised and fast at any size), counts summing to T * k;
* permute followed by un-permute-reduce returns k * x (round trip through the dispatched layout);
* y and dx of a sample of tokens against the oracle run on just those tokens (a token's output and input
  gradient depend on no other token);
* the three weight gradients of three whole experts — the one with the fewest rows, the one with the most
  (the longest contraction and the most row tiles) and one with an odd number of 128-row tiles (a pair-tile
  whose second half holds no rows) — against the oracle's expert body run on exactly the rows routed to them;
* linearity: doubling the upstream gradient doubles every gradient bit for bit;
* determinism: a second forward gives the same bits.
"""
import ctypes

import numpy as np
import pytest

from oracle import moe_oracle as oracle

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2   # max |a - b| / max |b| for bf16 activations
SIZES = {
    "c2": dict(T=16384, d=1024, E=8, k=2, h=2816, router_std=0.01, bias_std=0.0),
    "c3": dict(T=32768, d=2048, E=64, k=6, h=1408, router_std=0.02, bias_std=0.5),
    "c4layer": dict(T=65536, d=1024, E=16, k=2, h=2048, router_std=0.02, bias_std=0.0),
}
# Element-wise bar in the upstream form |x - y| <= tol max(unit, |y|) (tests/test_lm_bfloat16.py:129-167).  Upstream
# uses unit 1 and tol 0.012 on data of order one and short contractions; these sums run over thousands of
# bf16-rounded terms of arbitrary magnitude, whose error does not shrink with the sum: unit = the tensor's root mean
# square, tol 0.08 (measured worst case 0.054, a weight gradient of the decode shape: sums of a handful of
# heavy-tailed products).
BF16_ELEMENT_TOL = 0.08


def element_err(actual, expected):
    return oracle.elementwise_err(actual, expected, bf16=True, unit=oracle.rms(expected))


def bf16_exact(values):
    """float32 array rounded in place to values a bfloat16 holds exactly (nearest even)."""
    bits = values.view(np.uint32)
    step = 1 << 22
    for start in range(0, bits.size, step):
        chunk = bits.reshape(-1)[start:start + step]
        wide = chunk.astype(np.uint64)
        chunk[:] = ((wide + 0x7FFF + ((wide >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return values


def normal32(rng, shape, std):
    out = rng.standard_normal(shape, dtype=np.float32)
    out *= np.float32(std)
    return bf16_exact(out)


def rel(actual, expected):
    return oracle.max_rel_err(actual, expected)


@pytest.mark.parametrize("name", sorted(SIZES))
def test_full_size_layer_properties(name):
    from gpu_util import RouteTables, check_route_against_oracle, make_layer, to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.layers import Tensor
    from qutai_b200.storage import DeviceStorage

    cfg = SIZES[name]
    T, d, E, k, h = cfg["T"], cfg["d"], cfg["E"], cfg["k"], cfg["h"]
    rng = np.random.default_rng(20240 + T)
    x = normal32(rng, (T, d), 1.0)
    grad_y = normal32(rng, (T, d), 1.0)
    router = rng.standard_normal((E, d)).astype(np.float32) * np.float32(cfg["router_std"])
    if cfg["bias_std"]:
        # the router has no bias: a constant input column times a per-expert weight acts as one (skewed loads)
        x[:, d - 1] = 1.0
        router[:, d - 1] = rng.standard_normal(E).astype(np.float32) * np.float32(cfg["bias_std"])
    gate = normal32(rng, (E, h, d), 1.0 / np.sqrt(d))
    up = normal32(rng, (E, h, d), 1.0 / np.sqrt(d))
    down = normal32(rng, (E, d, h), 1.0 / np.sqrt(h))

    layer = make_layer((T, d), router, gate, up, down, k, engine="tcgen05")
    xs, gs = to_device(x, "bfloat16"), to_device(grad_y, "bfloat16")
    for p in layer.parameters():
        p.zero_grad()
    y, aux = layer(Tensor(xs, (T, d)))
    dx = layer.backward(Tensor(gs, (T, d)), None)
    assert lib.device_status() == 0
    work = layer._saved[0]
    scores = to_host(work["buf"]["scores"], (T, E))
    y_host, dx_host = to_host(y.storage, (T, d)), to_host(dx.storage, (T, d))

    # --- routing: bit-exact tables on the device's own logits --------------------------------------------
    expected = oracle.routing(scores, k)
    tables = RouteTables(T, E, k)
    tables.run(work["buf"]["scores"])
    check_route_against_oracle(tables, expected)
    assert layer.last_counts == expected["counts"] and sum(layer.last_counts) == T * k
    assert abs(float(to_host(aux.storage)[0]) - expected["aux"]) <= 1e-5 * max(1.0, abs(expected["aux"]))

    # --- round trip through the dispatched layout: un-permute(permute(x)) + 0 = k * x -------------------
    dispatched = DeviceStorage(tables.rows_bound * d, "bfloat16")
    zeros = DeviceStorage.zeros(T * d, "float32")
    back = DeviceStorage(T * d, "bfloat16")
    lib.call("qmoe_permute", tables.ref, xs.ptr, dispatched.ptr, lib.QMOE_BF16, d, 0)
    lib.call("qmoe_unpermute_reduce", tables.ref, dispatched.ptr, zeros.ptr, back.ptr, lib.QMOE_BF16, d, 0)
    assert np.array_equal(to_host(back, (T, d)), oracle.round_bf16(k * x.astype(np.float64)))
    del dispatched, zeros, back

    # --- a sample of tokens: y and dx depend on the token alone ------------------------------------------
    sample = np.sort(rng.choice(T, size=48, replace=False))
    ys, _, ctx = oracle.moe_forward(x[sample], router, gate, up, down, k, scores=scores[sample])
    grads = oracle.moe_backward(ctx, grad_y[sample], 0.0)
    assert rel(y_host[sample], ys) <= BF16_TOL
    assert rel(dx_host[sample], grads["x"]) <= BF16_TOL
    assert element_err(y_host[sample], ys) <= BF16_ELEMENT_TOL
    assert element_err(dx_host[sample], grads["x"]) <= BF16_ELEMENT_TOL

    # --- whole experts: their weight gradients need exactly the rows routed to them ----------------------
    counts = np.array(expected["counts"])
    smallest = int(np.argmin(np.where(counts > 0, counts, counts.max() + 1)))
    largest = int(np.argmax(counts))
    tiles = -(-counts // 128)
    odd = [e for e in np.argsort(-counts) if tiles[e] % 2 == 1 and e not in (smallest, largest)]
    checked = [smallest, largest] + [int(e) for e in odd[:1]]
    kept = {}
    for chosen in checked:
        members, slots = expected["ids"][chosen], expected["slots"][chosen]
        assert np.unique(members).size == counts[chosen]          # a token uses an expert at most once
        dy = grad_y[members].astype(np.float64) * expected["weights"][members, slots][:, None]
        _, saved = oracle.expert_forward(x[members], gate[chosen], up[chosen], down[chosen])
        want = oracle.expert_backward(saved, dy, gate[chosen], up[chosen], down[chosen])
        expert = layer.experts[chosen]
        got = dict(gate=to_host(expert.gate.weight.grad.storage, (h, d)), up=to_host(expert.up.weight.grad.storage, (h, d)),
                   down=to_host(expert.down.weight.grad.storage, (d, h)))
        for key, reference in zip(("gate", "up", "down"), want):
            assert rel(got[key], reference) <= BF16_TOL, (key, chosen, int(counts[chosen]))
            assert element_err(got[key], reference) <= BF16_ELEMENT_TOL, (key, chosen)
        if chosen == smallest:
            kept = got
    got, chosen = kept, smallest

    # --- linearity in the upstream gradient: 2 g gives exactly 2 x every gradient ------------------------
    d_router = to_host(layer.router.weight.grad.storage, (E, d))
    for p in layer.parameters():
        p.zero_grad()
    y2, _ = layer(Tensor(xs, (T, d)))
    assert y2.storage.tobytes() == y.storage.tobytes()      # determinism of the forward
    doubled = to_device(2.0 * grad_y, "bfloat16")
    dx2 = layer.backward(Tensor(doubled, (T, d)), None)
    assert lib.device_status() == 0
    assert np.array_equal(to_host(dx2.storage, (T, d)), 2.0 * dx_host)
    assert np.array_equal(to_host(layer.router.weight.grad.storage, (E, d)), 2.0 * d_router)
    expert = layer.experts[chosen]
    assert np.array_equal(to_host(expert.gate.weight.grad.storage, (h, d)), 2.0 * got["gate"])
    assert np.array_equal(to_host(expert.up.weight.grad.storage, (h, d)), 2.0 * got["up"])
    assert np.array_equal(to_host(expert.down.weight.grad.storage, (d, h)), 2.0 * got["down"])


def test_decode_shape_whole_layer_matches_the_oracle():
    """The decode configuration in full (64 tokens on the 64-expert layer: most groups hold a handful of rows,
    some none, every 128-row tile is mostly padding): every output and every expert's gradients against the
    oracle, experts without tokens get no gradient; the recorded CUDA graph replays the same bits."""
    from gpu_util import make_layer, to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.layers import Tensor

    T, d, E, k, h = 64, 2048, 64, 6, 1408
    rng = np.random.default_rng(64)
    x, grad_y = normal32(rng, (T, d), 1.0), normal32(rng, (T, d), 1.0)
    router = rng.standard_normal((E, d)).astype(np.float32) * np.float32(0.02)
    x[:, d - 1] = 1.0
    router[:, d - 1] = rng.standard_normal(E).astype(np.float32) * np.float32(0.5)
    gate = normal32(rng, (E, h, d), 1.0 / np.sqrt(d))
    up = normal32(rng, (E, h, d), 1.0 / np.sqrt(d))
    down = normal32(rng, (E, d, h), 1.0 / np.sqrt(h))
    layer = make_layer((T, d), router, gate, up, down, k, engine="tcgen05")
    stream = ctypes.c_uint64()
    lib.call("qmoe_stream_create", ctypes.byref(stream))
    layer.stream = stream.value
    xs, gs = Tensor(to_device(x, "bfloat16"), (T, d)), Tensor(to_device(grad_y, "bfloat16"), (T, d))
    aux_grad = to_device(np.array([0.3]), "float32")
    y, aux = layer(xs)
    dx = layer.backward(gs, aux_grad)
    lib.call("qmoe_stream_sync", layer.stream)
    assert lib.device_status() == 0
    work = layer._saved[0]
    scores = to_host(work["buf"]["scores"], (T, E))
    want_y, want_aux, ctx = oracle.moe_forward(x, router, gate, up, down, k, scores=scores)
    grads = oracle.moe_backward(ctx, grad_y, 0.3)
    counts = ctx["route"]["counts"]
    assert layer.last_counts == counts and sum(counts) == T * k
    assert min(counts) == 0 or max(counts) < 128          # the shape this test is about: tiny groups
    y_eager = y.storage.tobytes()
    for name, got, want in (("y", to_host(y.storage, (T, d)), want_y), ("dx", to_host(dx.storage, (T, d)), grads["x"]),
                            ("d_router", to_host(layer.router.weight.grad.storage, (E, d)), grads["router"])):
        assert rel(got, want) <= BF16_TOL, name
        assert element_err(got, want) <= BF16_ELEMENT_TOL, name
    assert abs(float(to_host(aux.storage)[0]) - want_aux) <= 1e-5
    for e, expert in enumerate(layer.experts):
        for key, parameter, shape in (("gate", expert.gate.weight, (h, d)), ("up", expert.up.weight, (h, d)),
                                      ("down", expert.down.weight, (d, h))):
            if counts[e] == 0:
                assert parameter.grad is None and grads[key][e] is None
            else:
                got = to_host(parameter.grad.storage, shape)
                assert rel(got, grads[key][e]) <= BF16_TOL, (key, e, counts[e])
                assert element_err(got, grads[key][e]) <= BF16_ELEMENT_TOL, (key, e)
    graph = layer.capture_forward(xs)
    for _ in range(2):
        y_replayed, _ = graph.replay()
        lib.call("qmoe_stream_sync", layer.stream)
        assert y_replayed.storage.tobytes() == y_eager
    assert lib.device_status(layer.stream) == 0
    del graph
    lib.call("qmoe_stream_destroy", stream.value)
