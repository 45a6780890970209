"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the golden fixtures.
Needs a B200: run with ``-m gpu``."""
import os

import numpy as np
import pytest

from conftest import golden_files
from oracle import moe_oracle as oracle

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4   # max relative error of outputs and gradients, fp32 activations
BF16_TOL = 2e-2   # the same bar for bf16 activations
# Element-wise bars in the form of the upstream GPU-against-CPU tests (a tensor-wide relative error lets small
# entries hide behind large ones): fp32 |x - y| <= 2e-5 (1 + |y|), upstream's own value (tests/test_lm_moe.py:105-138);
# bf16 |x - y| <= tol max(unit, |y|) (tests/test_lm_bfloat16.py:129-167).  Upstream applies the bf16 bar with unit 1
# and tol 0.012 to data of order one and contractions a few terms long; test_layer_bf16_at_upstream_scale does the
# same.  The other shapes here sum bf16-rounded products of arbitrary magnitude (heavy-tailed: a product of two
# normal factors reaches ten times its root mean square among millions of entries): the error of such a sum is
# about 2^-8 x the size of its terms whether or not the sum itself comes out small, so there the unit is the
# tensor's root mean square and the tolerance 0.08 (measured worst case 0.054).
FP32_ELEMENT_TOL = 2e-5
BF16_ELEMENT_TOL = 0.012
BF16_ELEMENT_TOL_LONG = 0.08


def rel(a, b):
    return oracle.max_rel_err(a, b)


def close(actual, expected, tol, bf16, upstream_scale=False):
    """Both bars: tensor-wide relative error within ``tol`` and every element within the element-wise bar."""
    if not bf16:
        return rel(actual, expected) <= tol and oracle.elementwise_err(actual, expected) <= FP32_ELEMENT_TOL
    if upstream_scale:
        return rel(actual, expected) <= tol and oracle.elementwise_err(actual, expected, bf16=True) <= BF16_ELEMENT_TOL
    element = oracle.elementwise_err(actual, expected, bf16=True, unit=oracle.rms(expected))
    return rel(actual, expected) <= tol and element <= BF16_ELEMENT_TOL_LONG


# ------------------------------------------------------------------------------------------------
# routing: bit-exact integer tables
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("path", golden_files("routing"), ids=os.path.basename)
def test_routing_golden(path):
    from gpu_util import RouteTables, check_route_against_oracle, to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.storage import DeviceStorage

    g = np.load(path)
    scores, k = g["scores"], int(g["top_k"])
    T, E = scores.shape
    tables = RouteTables(T, E, k)
    dev_scores = to_device(scores, "float32")
    expected = oracle.routing(scores.astype(np.float32).astype(np.float64), k)
    assert np.array_equal(expected["indices"], g["indices"])  # the fixture itself
    for _ in range(3):  # run-to-run identical, like the upstream test repeats it (tests/test_lm_moe.py:151)
        tables.run(dev_scores)
        check_route_against_oracle(tables, expected)
    # backward of both paths, separately and fused
    gw, ga = to_device(g["grad_weights"], "float32"), to_device(np.array([float(g["grad_aux"])]), "float32")
    out = DeviceStorage(T * E, "float32")
    lib.call("qmoe_route_backward", tables.ref, gw.ptr, 0, out.ptr, 0)
    assert np.abs(to_host(out, (T, E)) - g["d_scores_gate"]).max() <= 2e-6
    lib.call("qmoe_route_backward", tables.ref, 0, ga.ptr, out.ptr, 0)
    assert np.abs(to_host(out, (T, E)) - g["d_scores_aux"]).max() <= 2e-6
    lib.call("qmoe_route_backward", tables.ref, gw.ptr, ga.ptr, out.ptr, 0)
    assert np.abs(to_host(out, (T, E)) - (g["d_scores_gate"] + g["d_scores_aux"])).max() <= 4e-6


@pytest.mark.parametrize("T,E,k,skew", [(1, 1, 1, 0.0), (1, 8, 2, 0.0), (127, 8, 2, 0.0), (129, 9, 3, 0.0),
                                        (5000, 64, 6, 0.5), (16384, 8, 2, 0.0), (4099, 256, 8, 1.0),
                                        (3000, 33, 8, 0.0)])
def test_routing_random_and_quantised(T, E, k, skew):
    from gpu_util import RouteTables, check_route_against_oracle, to_device

    rng = np.random.default_rng(T * 131 + E)
    for quantise in (False, True):
        scores = rng.standard_normal((T, E)) + skew * rng.standard_normal(E)[None, :]
        if quantise:  # many exact ties in every row
            scores = np.round(scores * 2) / 2
        scores = scores.astype(np.float32)
        tables = RouteTables(T, E, k)
        tables.run(to_device(scores, "float32"))
        check_route_against_oracle(tables, oracle.routing(scores.astype(np.float64), k), float_tol=4e-6)


def test_routing_orders_logits_one_ulp_apart_like_the_float64_oracle():
    """Ranking runs on the raw fp32 logits (softmax is monotone).  Two logits one ulp apart have distinct float64
    probabilities, so the float64 CPU path — the oracle — prefers the larger one, as this kernel does.  (A path
    that ranks on fp32 probabilities, like the upstream CUDA kernel src/qutai/backends/cuda/lm.cu:345-352, may see
    them round to the same probability and then prefer the LOWER index: that deviation from the float64 path is
    not reproduced here.)"""
    from gpu_util import RouteTables, check_route_against_oracle, to_device

    rng = np.random.default_rng(77)
    T, E, k = 512, 16, 4
    scores = rng.standard_normal((T, E)).astype(np.float32)
    # in every row make the higher-index expert of a pair the larger one by exactly one ulp, near the top of the row
    top = scores.max(axis=1) + np.float32(0.5)
    low = rng.integers(0, E - 1, size=T)
    high = low + 1 + rng.integers(0, E - 1 - low)
    rows = np.arange(T)
    scores[rows, low] = top
    scores[rows, high] = np.nextafter(top, np.float32(np.inf))
    assert np.all(scores[rows, high] > scores[rows, low])
    expected = oracle.routing(scores.astype(np.float64), k)
    assert np.array_equal(expected["indices"][:, 0], high) and np.array_equal(expected["indices"][:, 1], low)
    tables = RouteTables(T, E, k)
    tables.run(to_device(scores, "float32"))
    check_route_against_oracle(tables, expected, float_tol=4e-6)


@pytest.mark.parametrize("E,k", [(8, 2), (64, 6), (33, 8)])
def test_routing_of_rows_with_nan_or_infinite_logits_stays_inside_the_tables(E, k):
    """Logits that are not numbers (a diverged step) must not send an index outside the tables: a NaN ranks as
    -inf, every row still gets k distinct experts in [0, E), the counts add up to T * k, and rows of ordinary
    numbers are routed exactly as without their neighbours."""
    from gpu_util import RouteTables, to_device

    rng = np.random.default_rng(E * 7 + k)
    T = 700
    scores = rng.standard_normal((T, E)).astype(np.float32)
    clean = scores.copy()
    scores[5] = np.nan                                   # a whole row of NaN
    scores[6, ::2] = np.nan                              # half a row
    scores[7] = np.inf
    scores[8] = -np.inf
    scores[9, 1] = np.inf
    scores[10, : E - 1] = np.nan                         # a single number left
    bad = (5, 6, 7, 8, 9, 10)
    tables = RouteTables(T, E, k)
    tables.run(to_device(scores, "float32"))
    indices = tables.host("expert_index", (T, k))
    assert indices.min() >= 0 and indices.max() < E
    assert all(len(set(row)) == k for row in indices.tolist())
    counts = tables.host("counts")
    assert counts.sum() == T * k and np.array_equal(counts, np.bincount(indices.reshape(-1), minlength=E))
    dest = tables.host("dest_row")
    assert dest.min() >= 0 and dest.max() < tables.rows_bound and len(set(dest.tolist())) == T * k
    expected = oracle.routing(clean.astype(np.float64), k)
    good = np.setdiff1d(np.arange(T), bad)
    assert np.array_equal(indices[good], np.asarray(expected["indices"]).reshape(T, k)[good])
    assert np.isfinite(tables.host("gate_weights", (T, k))[good]).all()
    numbers = np.flatnonzero(~np.isnan(scores[6]))       # in the half-NaN row the numbers win, largest first
    assert set(indices[6, : min(k, len(numbers))]) <= set(numbers.tolist())
    assert indices[10, 0] == E - 1


def test_routing_rejects_bad_arguments():
    from gpu_util import RouteTables, to_device
    from qutai_b200 import lib

    tables = RouteTables(8, 4, 2)
    scores = to_device(np.zeros((8, 4)), "float32")
    tables.struct.top_k = 5
    with pytest.raises(ValueError):
        lib.call("qmoe_route", tables.ref, scores.ptr, 0)
    tables.struct.top_k = 2
    tables.struct.counts = 0
    with pytest.raises(ValueError):
        lib.call("qmoe_route", tables.ref, scores.ptr, 0)


# ------------------------------------------------------------------------------------------------
# permute / combine and their backwards
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,k,d", [(5, 3, 2, 4), (37, 4, 2, 16), (300, 8, 3, 72), (1000, 64, 6, 256), (64, 5, 1, 1030)])
def test_permute_combine_and_backwards(T, E, k, d, dtype):
    from gpu_util import RouteTables, to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.storage import DeviceStorage

    rng = np.random.default_rng(T + d)
    code = lib.DTYPE_CODES[dtype]
    rnd = oracle.round_bf16 if dtype == "bfloat16" else (lambda a: np.asarray(a, dtype=np.float32).astype(np.float64))
    tol = 1e-2 if dtype == "bfloat16" else 2e-6
    scores = rng.standard_normal((T, E)).astype(np.float32)
    x, gout = rnd(rng.standard_normal((T, d))), rnd(rng.standard_normal((T, d)))
    route = oracle.routing(scores.astype(np.float64), k)
    tables = RouteTables(T, E, k)
    tables.run(to_device(scores, "float32"))
    R = tables.rows_bound
    offsets, counts = tables.host("offsets"), tables.host("counts")
    weights = tables.host("gate_weights", (T, k))

    xd = DeviceStorage(R * d, dtype)
    lib.call("qmoe_memset", xd.ptr, 0x7f, xd.nbytes, 0)  # stale data must not survive in pad rows
    x_dev = to_device(x, dtype)  # kept alive by name: a temporary would be released before the call is made
    lib.call("qmoe_permute", tables.ref, x_dev.ptr, xd.ptr, code, d, 0)
    xh = to_host(xd, (R, d))
    for e in range(E):
        assert np.array_equal(xh[offsets[e]: offsets[e] + counts[e]], oracle.route_gather(x, route, e))
        assert np.all(xh[offsets[e] + counts[e]: offsets[e + 1]] == 0)

    # expert outputs: any values in the dispatched layout
    yd_host = np.zeros((R, d))
    outputs = []
    for e in range(E):
        if counts[e]:
            ye = rnd(rng.standard_normal((counts[e], d)))
            yd_host[offsets[e]: offsets[e] + counts[e]] = ye
            outputs.append((e, ye))
    yd = to_device(yd_host, dtype)
    out = DeviceStorage(T * d, dtype)
    lib.call("qmoe_combine", tables.ref, yd.ptr, out.ptr, code, d, 0)
    route_w = dict(route, weights=weights)
    assert rel(to_host(out, (T, d)), oracle.combine(outputs, weights, route_w)) <= tol

    dy, dw = DeviceStorage(R * d, dtype), DeviceStorage(T * k, "float32")
    lib.call("qmoe_memset", dy.ptr, 0x7f, dy.nbytes, 0)
    gout_dev = to_device(gout, dtype)
    lib.call("qmoe_combine_backward", tables.ref, gout_dev.ptr, yd.ptr, dy.ptr, dw.ptr, code, d, 0)
    want_dy, want_dw = oracle.combine_backward(gout, outputs, weights, route_w)
    dyh = to_host(dy, (R, d))
    for (e, _), want in zip(outputs, want_dy):
        assert rel(dyh[offsets[e]: offsets[e] + counts[e]], want) <= tol
        assert np.all(dyh[offsets[e] + counts[e]: offsets[e + 1]] == 0)
    assert rel(to_host(dw, (T, k)), want_dw) <= 1e-5

    # unpermute-reduce == sum over experts of route_gather_backward, plus the optional fp32 addend
    extra = rng.standard_normal((T, d)).astype(np.float32)
    dx = DeviceStorage(T * d, dtype)
    extra_dev = to_device(extra, "float32")
    lib.call("qmoe_unpermute_reduce", tables.ref, yd.ptr, extra_dev.ptr, dx.ptr, code, d, 0)
    want = extra.astype(np.float64)
    for e, ye in outputs:
        want = want + oracle.route_gather_backward(ye, route, e)
    assert rel(to_host(dx, (T, d)), want) <= tol
    lib.call("qmoe_unpermute_reduce", tables.ref, yd.ptr, 0, dx.ptr, code, d, 0)
    assert rel(to_host(dx, (T, d)), want - extra) <= tol


# ------------------------------------------------------------------------------------------------
# the layer against the golden fixtures (fp32 activations, 1e-4) and against the oracle (bf16, 2e-2)
# ------------------------------------------------------------------------------------------------
def check_layer(out, g, y, aux, grads, counts, tol, sample=1, bf16=True, upstream_scale=False):
    close_ = lambda a, b: close(a, b, tol, bf16, upstream_scale)
    assert out["counts"] == tuple(counts)
    assert close_(out["y"], y)
    assert abs(out["aux"] - aux) <= 1e-4 * max(1.0, abs(aux))
    assert close_(out["dx"], grads["x"])
    assert close_(out["d_router"], grads["router"])
    # every expert's row of the router gradient on its own scale (a rarely used expert's row is small)
    assert oracle.rowwise_rel_err(out["d_router"], grads["router"]) <= 2 * tol
    for e in range(len(counts)):
        for key in ("gate", "up", "down"):
            mine, want = out["d_" + key][e], grads[key][e]
            if counts[e] == 0:
                assert mine is None and want is None  # upstream: such an expert gets no gradient object
            else:
                assert close_(mine.reshape(-1)[::sample], np.asarray(want).reshape(-1)[::sample]), (key, e)


@pytest.mark.parametrize("path", golden_files("layer"), ids=os.path.basename)
def test_layer_fp32_matches_golden(path):
    from gpu_util import make_layer, run_layer

    g = np.load(path)
    layer = make_layer(g["x"].shape, g["router"], g["gate"], g["up"], g["down"], int(g["top_k"]))
    out = run_layer(layer, g["x"], g["grad_y"], float(g["grad_aux"]), "float32")
    E, step = g["gate"].shape[0], int(g["sample"])
    grads = dict(x=g["dx"], router=g["d_router"])
    for key in ("gate", "up", "down"):
        grads[key] = [g[f"d_{key}_{e}"] if g["has_grad"][e] else None for e in range(E)]
    assert out["counts"] == tuple(g["counts"].tolist())
    assert close(out["y"], g["y"], FP32_TOL, False)
    assert abs(out["aux"] - float(g["aux"])) <= 1e-5
    assert close(out["dx"], g["dx"], FP32_TOL, False)
    assert close(out["d_router"], g["d_router"], FP32_TOL, False)
    assert rel(out["utilization"], g["utilization"]) <= 1e-6
    for e in range(E):
        for key in ("gate", "up", "down"):
            mine = out["d_" + key][e]
            if not g["has_grad"][e]:
                assert mine is None
            else:
                assert close(mine.reshape(-1)[::step], grads[key][e], FP32_TOL, False), (key, e)
    # a second pass gives bit-identical results (no floating-point atomics anywhere)
    again = run_layer(layer, g["x"], g["grad_y"], float(g["grad_aux"]), "float32")
    assert np.array_equal(again["y"], out["y"]) and np.array_equal(again["dx"], out["dx"])
    assert np.array_equal(again["d_router"], out["d_router"])


def oracle_for(x, router, gate, up, down, k, grad_y, grad_aux, scores):
    y, aux, ctx = oracle.moe_forward(x, router, gate, up, down, k, scores=scores)
    grads = oracle.moe_backward(ctx, grad_y, grad_aux)
    return y, aux, grads, ctx["route"]["counts"]


LAYER_SHAPES = [
    # T, d, E, k, h
    (64, 64, 4, 2, 128),      # single tile per expert
    (300, 72, 5, 2, 136),     # widths that are multiples of 8 but not of the tile sizes
    (1000, 256, 8, 2, 512),   # several tiles, several k blocks
    (777, 128, 16, 4, 264),   # ragged counts, partial N tile
    (2048, 512, 8, 2, 1408),  # half-filled last N tile (1408 = 5.5 x 256)
    (900, 384, 3, 1, 640),    # odd numbers of 128-row tiles per expert, d and h = 1.5 and 2.5 x 256
]


@pytest.mark.parametrize("engine", ["simt", "tcgen05", "tcgen05-1cta"])
@pytest.mark.parametrize("T,d,E,k,h", LAYER_SHAPES)
def test_layer_bf16_matches_oracle(T, d, E, k, h, engine, kernel_variant):
    from gpu_util import make_layer, run_layer
    from qutai_b200 import lib

    # "tcgen05" runs the expert GEMMs as CTA pairs (256-row tiles), "tcgen05-1cta" one CTA per 128-row tile
    if engine == "tcgen05-1cta":
        kernel_variant(lib.VARIANT_SINGLE_CTA_GEMM)
        engine = "tcgen05"
    rng = np.random.default_rng(T + d + E)
    r16 = oracle.round_bf16
    x, grad_y = r16(rng.standard_normal((T, d))), r16(rng.standard_normal((T, d)))
    router = rng.standard_normal((E, d)).astype(np.float32) * 0.05
    gate = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    up = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    down = rng.standard_normal((E, d, h)).astype(np.float32) / np.sqrt(h)
    layer = make_layer(x.shape, router, gate, up, down, k, engine=engine)
    out = run_layer(layer, x, grad_y, 0.37, "bfloat16")
    # router logits: fp32 arithmetic on exactly these inputs
    assert rel(out["scores"], x @ router.astype(np.float64).T) <= FP32_TOL
    # everything downstream is checked given the device's own fp32 logits (identical routing)
    y, aux, grads, counts = oracle_for(x, router, r16(gate), r16(up), r16(down), k, grad_y, 0.37, out["scores"])
    check_layer(out, None, y, aux, grads, counts, BF16_TOL)


@pytest.mark.parametrize("engine", ["simt", "tcgen05"])
def test_layer_bf16_at_upstream_scale(engine):
    """Data of order one and contractions a few terms long, as in the upstream bf16 test
    (tests/test_lm_bfloat16.py:129-167): upstream's own element-wise bar, |x - y| <= 0.012 max(1, |y|)."""
    from gpu_util import make_layer, run_layer

    T, d, E, k, h = 40, 16, 3, 2, 24
    rng = np.random.default_rng(41)
    r16 = oracle.round_bf16
    x, grad_y = r16(rng.standard_normal((T, d)) * 0.5), r16(rng.standard_normal((T, d)) * 0.5)
    router = rng.standard_normal((E, d)).astype(np.float32) * 0.3
    gate = rng.standard_normal((E, h, d)).astype(np.float32) * 0.3
    up = rng.standard_normal((E, h, d)).astype(np.float32) * 0.3
    down = rng.standard_normal((E, d, h)).astype(np.float32) * 0.3
    layer = make_layer(x.shape, router, gate, up, down, k, engine=engine)
    out = run_layer(layer, x, grad_y, 0.37, "bfloat16")
    y, aux, grads, counts = oracle_for(x, router, r16(gate), r16(up), r16(down), k, grad_y, 0.37, out["scores"])
    check_layer(out, None, y, aux, grads, counts, BF16_TOL, upstream_scale=True)


def test_tcgen05_agrees_with_cuda_core_engine():
    from gpu_util import make_layer, run_layer

    T, d, E, k, h = 1500, 256, 6, 2, 768
    rng = np.random.default_rng(5)
    x, grad_y = oracle.round_bf16(rng.standard_normal((T, d))), oracle.round_bf16(rng.standard_normal((T, d)))
    router = rng.standard_normal((E, d)).astype(np.float32) * 0.05
    gate = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    up = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    down = rng.standard_normal((E, d, h)).astype(np.float32) / np.sqrt(h)
    results = {}
    for engine in ("simt", "tcgen05"):
        layer = make_layer(x.shape, router, gate, up, down, k, engine=engine)
        results[engine] = run_layer(layer, x, grad_y, None, "bfloat16")
    a, b = results["simt"], results["tcgen05"]
    assert a["counts"] == b["counts"]
    # same operands, same fp32 accumulation up to summation order: differences are bf16 roundings
    assert rel(b["y"], a["y"]) <= 1e-2 and rel(b["dx"], a["dx"]) <= 1e-2
    for e in range(E):
        for key in ("d_gate", "d_up", "d_down"):
            assert rel(b[key][e], a[key][e]) <= 1e-2


def test_empty_expert_gets_no_gradient_and_its_buffer_is_untouched():
    from gpu_util import make_layer, run_layer

    T, d, E, k, h = 200, 64, 4, 1, 128
    rng = np.random.default_rng(9)
    x = np.abs(oracle.round_bf16(rng.standard_normal((T, d))))
    router = rng.standard_normal((E, d)).astype(np.float32) * 0.01
    router[2] = -1.0  # expert 2 is never the arg-max
    gate = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    up = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    down = rng.standard_normal((E, d, h)).astype(np.float32) / np.sqrt(h)
    for engine in ("simt", "tcgen05"):
        layer = make_layer(x.shape, router, gate, up, down, k, engine=engine)
        out = run_layer(layer, x, oracle.round_bf16(rng.standard_normal((T, d))), 0.1, "bfloat16")
        assert out["counts"][2] == 0 and sum(out["counts"]) == T
        assert out["d_gate"][2] is None and out["d_up"][2] is None and out["d_down"][2] is None
        assert all(g is not None for i, g in enumerate(out["d_gate"]) if out["counts"][i])


def test_gradient_accumulates_over_two_backwards():
    from gpu_util import make_layer, run_layer, to_device, to_host
    from qutai_b200.layers import Tensor

    g = np.load(os.path.join(os.path.dirname(golden_files("layer")[0]), "layer_mid.npz"))
    layer = make_layer(g["x"].shape, g["router"], g["gate"], g["up"], g["down"], int(g["top_k"]))
    once = run_layer(layer, g["x"], g["grad_y"], float(g["grad_aux"]), "float32")
    T, d = g["x"].shape
    layer(Tensor(to_device(g["x"], "float32"), (T, d)))
    layer.backward(Tensor(to_device(g["grad_y"], "float32"), (T, d)), to_device(np.array([float(g["grad_aux"])]), "float32"))
    twice = to_host(layer.router.weight.grad.storage, once["d_router"].shape)
    assert rel(twice, 2 * once["d_router"]) <= 1e-6
    e = int(np.argmax(g["counts"]))
    got = to_host(layer.experts[e].down.weight.grad.storage, once["d_down"][e].shape)
    assert rel(got, 2 * once["d_down"][e]) <= 1e-6


# ------------------------------------------------------------------------------------------------
# router projection: fp32 semantics on the tensor cores (split bf16 terms) and on the CUDA cores
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("T,d,E", [(1000, 256, 8), (4133, 2048, 64), (300, 512, 33), (128, 64, 1), (77, 72, 5)])
def test_router_forward_backward_fp32_semantics(T, d, E, dtype):
    from gpu_util import to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.storage import DeviceStorage

    rng = np.random.default_rng(T + E)
    x = rng.standard_normal((T, d))
    x = oracle.round_bf16(x) if dtype == "bfloat16" else x.astype(np.float32).astype(np.float64)
    w = (rng.standard_normal((E, d)) * 0.05).astype(np.float32)
    ds = (rng.standard_normal((T, E)) * 0.01).astype(np.float32)
    code = lib.DTYPE_CODES[dtype]
    scratch = DeviceStorage(int(lib.load().qmoe_router_scratch_bytes(T, E, d)) // 4 + 64, "float32")
    xd, wd, dsd = to_device(x, dtype), to_device(w, "float32"), to_device(ds, "float32")
    scores, dxr, dwr = DeviceStorage(T * E, "float32"), DeviceStorage(T * d, "float32"), DeviceStorage(E * d, "float32")
    lib.call("qmoe_router_forward", xd.ptr, code, wd.ptr, scores.ptr, scratch.ptr, T, d, E, 0)
    lib.call("qmoe_router_backward", dsd.ptr, xd.ptr, code, wd.ptr, dxr.ptr, dwr.ptr, scratch.ptr, T, d, E, 0)
    w64, ds64 = w.astype(np.float64), ds.astype(np.float64)
    # fp32 accumulation over up to thousands of terms: a few 1e-6 relative; the bar for logits is 1e-4
    assert rel(to_host(scores, (T, E)), x @ w64.T) <= 1e-5
    assert rel(to_host(dwr, (E, d)), ds64.T @ x) <= 1e-5
    assert rel(to_host(dxr, (T, d)), ds64 @ w64) <= 2e-5
    first = to_host(dwr, (E, d))
    lib.call("qmoe_router_backward", dsd.ptr, xd.ptr, code, wd.ptr, dxr.ptr, dwr.ptr, scratch.ptr, T, d, E, 0)
    assert np.array_equal(first, to_host(dwr, (E, d)))  # fixed reduction order: bit-identical
    assert lib.device_status() == 0


def test_launch_variants_of_the_weight_gradients_agree_bit_for_bit(kernel_variant):
    """One launch for the three weight gradients (default) against one launch each (the comparison form of
    ``qmoe_test_select_variant``): the same tiles in a different order give the same bits."""
    from gpu_util import make_layer, run_layer
    from qutai_b200 import lib

    T, d, E, k, h = 1100, 384, 5, 2, 1408
    rng = np.random.default_rng(11)
    x, grad_y = oracle.round_bf16(rng.standard_normal((T, d))), oracle.round_bf16(rng.standard_normal((T, d)))
    router = rng.standard_normal((E, d)).astype(np.float32) * 0.05
    gate = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    up = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    down = rng.standard_normal((E, d, h)).astype(np.float32) / np.sqrt(h)
    results = []
    for per_product in (False, True):
        if per_product:
            kernel_variant(lib.VARIANT_WGRAD_PER_PRODUCT)
        layer = make_layer(x.shape, router, gate, up, down, k, engine="tcgen05")
        results.append(run_layer(layer, x, grad_y, None, "bfloat16"))
    a, b = results
    for e in range(E):
        for key in ("d_gate", "d_up", "d_down"):
            assert np.array_equal(a[key][e], b[key][e]), (key, e)
