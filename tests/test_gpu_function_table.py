"""The per-op backend function table (``qutai_b200.cuda_lm``) against the oracle, written after the
upstream GPU tests of the same functions (tests/test_lm_moe.py:140-162,
tests/test_lm_bfloat16.py:129-167, tests/test_gemm_precision.py)."""
import os

import numpy as np
import pytest

from conftest import golden_files
from oracle import moe_oracle as oracle

pytestmark = pytest.mark.gpu


def close(actual, expected, tolerance):
    actual, expected = np.asarray(actual, dtype=np.float64), np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape
    assert np.all(np.abs(actual - expected) <= tolerance * np.maximum(1.0, np.abs(expected)))


def test_route_pack_has_stable_token_slot_order_across_blocks():
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm

    rows, experts, top_k = 517, 5, 3
    scores = np.array([[((row * 37 + expert * 11) % 101) / 13 for expert in range(experts)] for row in range(rows)],
                      dtype=np.float32)
    reference = oracle.routing(scores.astype(np.float64), top_k)
    values = to_device(scores, "float32")
    for _ in range(3):
        route = cuda_lm.routing(values, rows, experts, top_k)
        assert route["counts"] == reference["counts"]
        for expert, count in enumerate(route["counts"]):
            ids = to_host(cuda_lm.take(route["ids"], expert * route["capacity"], count))
            slots = to_host(cuda_lm.take(route["slots"], expert * route["capacity"], count))
            assert np.array_equal(ids, reference["ids"][expert])
            assert np.array_equal(slots, reference["slots"][expert])
        assert np.array_equal(to_host(route["indices"]).reshape(rows, top_k), reference["indices"])
        assert np.array_equal(to_host(route["locations"]).reshape(rows, top_k), reference["locations"])


def test_router_fp32_and_bfloat16_expert_gather_combine():
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm

    scores = np.array([[3, 1, -2], [0, 2, 1], [1, -2, 4], [-1, 3, 2], [4, 0, 1]], dtype=np.float32)
    raw_values = np.array([0.03 * i - 0.2 for i in range(20)]).reshape(5, 4)
    raw_gradient = np.array([0.05 * i - 0.4 for i in range(20)]).reshape(5, 4)
    values, gradient = to_device(raw_values, "bfloat16"), to_device(raw_gradient, "bfloat16")
    reference, reference_g = oracle.round_bf16(raw_values), oracle.round_bf16(raw_gradient)
    route = cuda_lm.routing(to_device(scores, "float32"), 5, 3, 2)
    outputs = tuple((e, cuda_lm.route_gather(values, route, e, 4)) for e in range(3) if route["counts"][e])
    combined = cuda_lm.combine(outputs, route["weights"], route, 4)
    gradients = cuda_lm.combine_backward(gradient, outputs, route["weights"], route, 4)
    cpu_route = oracle.routing(scores.astype(np.float64), 2)
    assert route["counts"] == cpu_route["counts"] == (3, 3, 4)
    cpu_outputs = [(e, oracle.route_gather(reference, cpu_route, e)) for e in range(3) if cpu_route["counts"][e]]
    expected = oracle.combine(cpu_outputs, cpu_route["weights"], cpu_route)
    expected_dy, expected_dw = oracle.combine_backward(reference_g, cpu_outputs, cpu_route["weights"], cpu_route)
    assert (route["weights"].dtype, route["aux"].dtype, combined.dtype) == ("float32", "float32", "bfloat16")
    assert combined.nbytes == 40
    close(to_host(combined, (5, 4)), expected, 0.012)
    for (e, storage), want_rows in zip(outputs, cpu_outputs):
        assert np.array_equal(to_host(storage).reshape(-1, 4), want_rows[1])
    for actual, want in zip(gradients[:-1], expected_dy):
        close(to_host(actual).reshape(-1, 4), want, 0.012)
    assert gradients[-1].dtype == "float32"
    close(to_host(gradients[-1], (5, 2)), expected_dw, 0.012)
    # bfloat16 scores are widened exactly before routing
    again = cuda_lm.routing(to_device(scores, "bfloat16"), 5, 3, 2)
    assert again["counts"] == route["counts"] and np.array_equal(to_host(again["indices"]), to_host(route["indices"]))
    # routing backward: both paths
    g = np.random.default_rng(0).standard_normal((5, 2)).astype(np.float32)
    close(to_host(cuda_lm.routing_backward(to_device(g, "float32"), route), (5, 3)), oracle.routing_backward(g, cpu_route), 1e-5)
    close(to_host(cuda_lm.routing_backward(to_device(np.array([0.5]), "float32"), route, True), (5, 3)),
          oracle.routing_backward([0.5], cpu_route, True), 1e-5)


@pytest.mark.parametrize("transpose_left", [False, True])
@pytest.mark.parametrize("transpose_right", [False, True])
def test_gemm_transposes_mixed_precision_and_accumulate(transpose_left, transpose_right):
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm

    rows, inner, cols = 65, 129, 33     # partial tiles in every dimension
    rng = np.random.default_rng(3)
    a, b = rng.standard_normal((rows, inner)), rng.standard_normal((inner, cols))
    a16, b32 = oracle.round_bf16(a), b.astype(np.float32).astype(np.float64)
    left = to_device(a16.T if transpose_left else a16, "bfloat16")
    right = to_device(b32.T if transpose_right else b32, "float32")
    kw = dict(transpose_left=transpose_left, transpose_right=transpose_right)
    product = a16 @ b32
    out = cuda_lm.gemm(left, right, rows, inner, cols, **kw)
    assert out.dtype == "float32"
    close(to_host(out, (rows, cols)), product, 5e-5)   # fp32 accumulation of 129 products
    rounded = cuda_lm.gemm(left, right, rows, inner, cols, out_dtype="bfloat16", **kw)
    assert rounded.dtype == "bfloat16" and rounded.nbytes == rows * cols * 2
    assert np.array_equal(to_host(rounded, (rows, cols)), oracle.round_bf16(to_host(out, (rows, cols))))  # RNE of the fp32 result
    cuda_lm.gemm(left, right, rows, inner, cols, out=out, accumulate=True, **kw)
    close(to_host(out, (rows, cols)), 2 * product, 5e-5)
    with pytest.raises(ValueError):
        cuda_lm.gemm(left, right, rows, inner, cols, accumulate=True, **kw)          # accumulate needs out
    square = to_device(np.eye(16), "float32")
    with pytest.raises(ValueError):
        cuda_lm.gemm(square, square, 16, 16, 16, out=square)                           # out must not overlap an input
    with pytest.raises(ValueError):
        cuda_lm.gemm(square, square, 16, 16, 16, out_dtype="float64")


def test_gemm_long_inner_dimension_keeps_fp32_sums():
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm

    rows, inner, cols = 129, 8193, 65
    a, b = np.ones((rows, inner)), np.full((inner, cols), 0.5)
    out = cuda_lm.gemm(to_device(a, "bfloat16"), to_device(b, "bfloat16"), rows, inner, cols)
    assert np.array_equal(to_host(out, (rows, cols)), np.full((rows, cols), inner * 0.5))  # exact in fp32


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_forward_and_backward(dtype):
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm

    rng = np.random.default_rng(4)
    rnd = oracle.round_bf16 if dtype == "bfloat16" else (lambda v: v.astype(np.float32).astype(np.float64))
    x, g = rnd(rng.standard_normal(1000) * 4), rnd(rng.standard_normal(1000))
    x[:4] = [0.0, -80.0, 80.0, -1e-3]
    x = rnd(x)
    tol = 0.012 if dtype == "bfloat16" else 2e-6
    close(to_host(cuda_lm.silu(to_device(x, dtype))), oracle.silu(x), tol)
    close(to_host(cuda_lm.silu_backward(to_device(g, dtype), to_device(x, dtype))), oracle.silu_backward(g, x), tol)


def test_upstream_style_expert_loop_matches_golden_layer():
    """The upstream ``SparseMoE.__call__`` written against this function table
    (src/qutai/lm/layers.py:376-402) reproduces the golden fixture of the upstream CPU layer."""
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm as b

    g = np.load(os.path.join(os.path.dirname(golden_files("layer")[0]), "layer_mid.npz"))
    T, d = g["x"].shape
    E, h = g["gate"].shape[0], g["gate"].shape[1]
    k = int(g["top_k"])
    x = to_device(g["x"], "float32")
    scores = b.gemm(x, to_device(g["router"], "float32"), T, d, E, transpose_right=True)
    route = b.routing(scores, T, E, k)
    assert route["counts"] == tuple(g["counts"].tolist())
    outputs = []
    for e in range(E):
        if route["counts"][e]:
            xe, c = b.route_gather(x, route, e, d), route["counts"][e]
            gate = b.gemm(xe, to_device(g["gate"][e], "float32"), c, d, h, transpose_right=True)
            up = b.gemm(xe, to_device(g["up"][e], "float32"), c, d, h, transpose_right=True)
            act = b.silu(gate)
            outputs.append((e, (act, up, c)))
    # element-wise product silu(gate) * up through the table's gemm is not available; use numpy for that one op
    ys = []
    for e, (act, up, c) in outputs:
        hidden = to_device(to_host(act) * to_host(up), "float32")
        ys.append((e, b.gemm(hidden, to_device(g["down"][e], "float32"), c, h, d, transpose_right=True)))
    y = b.combine(tuple(ys), route["weights"], route, d)
    assert oracle.max_rel_err(to_host(y, (T, d)), g["y"]) <= 1e-4
    assert abs(to_host(route["aux"])[0] - float(g["aux"])) <= 1e-5
    # gather backward of one expert: rows scattered into zeros
    e0 = ys[0][0]
    grad_rows = np.random.default_rng(1).standard_normal((route["counts"][e0], d)).astype(np.float32)
    scattered = to_host(b.route_gather_backward(to_device(grad_rows, "float32"), route, e0, d), (T, d))
    cpu_route = oracle.routing(to_host(scores, (T, E)), k)
    assert np.array_equal(scattered, oracle.route_gather_backward(grad_rows, cpu_route, e0))


@pytest.mark.parametrize("rows,inner,cols", [(128, 64, 72), (384, 1024, 264), (1024, 264, 1024)])
def test_gemm_takes_the_tensor_cores_for_the_three_products_of_a_linear_layer(rows, inner, cols, kernel_variant):
    """bf16 x bf16 in the forms of a linear layer's forward (x W^T), input gradient (g W) and weight gradient
    (g^T x, float32) run on the tcgen05 kernels when the sizes allow, and give what the CUDA-core kernel gives."""
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm, lib

    rng = np.random.default_rng(rows + cols)
    x, w = oracle.round_bf16(rng.standard_normal((rows, inner))), oracle.round_bf16(rng.standard_normal((cols, inner)) * 0.1)
    g = oracle.round_bf16(rng.standard_normal((rows, cols)))
    xs, ws, gs = to_device(x, "bfloat16"), to_device(w, "bfloat16"), to_device(g, "bfloat16")
    count = lib.load().qmoe_tensor_core_launch_count

    def products():
        y = cuda_lm.gemm(xs, ws, rows, inner, cols, transpose_right=True, out_dtype="bfloat16")
        dx = cuda_lm.gemm(gs, ws, rows, cols, inner, out_dtype="bfloat16")
        dw = cuda_lm.gemm(gs, xs, cols, rows, inner, transpose_left=True, out_dtype="float32")
        return to_host(y, (rows, cols)), to_host(dx, (rows, inner)), to_host(dw, (cols, inner))

    before = count()
    fast = products()
    assert count() - before == 3
    kernel_variant(lib.VARIANT_PLAIN_GEMM_ON_CUDA_CORES)
    before = count()
    slow = products()
    assert count() == before
    for got, reference, exact in zip(fast, slow, (x @ w.T, g @ w, g.T @ x)):
        assert oracle.max_rel_err(got, exact) <= 1e-2
        assert oracle.max_rel_err(got, reference) <= 8e-3          # both round fp32 sums of the same products to bf16 (or keep fp32)
    # a row count that is not a multiple of 128 stays on the CUDA cores (a tile of the tensor-core kernel writes 128 rows)
    kernel_variant(lib.VARIANT_PLAIN_GEMM_ON_CUDA_CORES, 0)
    before = count()
    cuda_lm.gemm(to_device(x[:100], "bfloat16"), ws, 100, inner, cols, transpose_right=True, out_dtype="bfloat16")
    assert count() == before


@pytest.mark.parametrize("rows,cols_out,cols_in", [(8192, 1024, 1024), (4104, 256, 1024), (1096, 512, 264)])
def test_split_weight_gradient_of_a_linear_layer(rows, cols_out, cols_in):
    """``qmoe_gemm_wgrad_split``: g^T x with the rows cut into ranges that run side by side, the ranges' products
    added in a fixed order — the value of the one-launch product, the same bits on every run; row counts that leave a
    ragged last range included."""
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm, lib
    from qutai_b200.storage import DeviceStorage

    rng = np.random.default_rng(rows)
    x, g = oracle.round_bf16(rng.standard_normal((rows, cols_in))), oracle.round_bf16(rng.standard_normal((rows, cols_out)))
    xs, gs = to_device(x, "bfloat16"), to_device(g, "bfloat16")
    partials = lib.load().qmoe_gemm_wgrad_partials(cols_out, rows, cols_in)
    assert partials > 64 + cols_out * cols_in                 # these shapes are split
    scratch, out = DeviceStorage(partials, "float32"), DeviceStorage(cols_out * cols_in, "float32")
    results = []
    for _ in range(2):
        lib.call("qmoe_gemm_wgrad_split", gs.ptr, xs.ptr, out.ptr, scratch.ptr, cols_out, rows, cols_in, 0)
        results.append(to_host(out, (cols_out, cols_in)))
    assert np.array_equal(results[0], results[1])
    assert lib.device_status() == 0
    assert oracle.max_rel_err(results[0], g.T @ x) <= 1e-5
    whole = to_host(cuda_lm.gemm(gs, xs, cols_out, rows, cols_in, transpose_left=True, out_dtype="float32"), (cols_out, cols_in))
    assert oracle.max_rel_err(results[0], whole) <= 1e-5
    # a shape with enough tiles of its own is not split, and the call says so
    assert lib.load().qmoe_gemm_wgrad_partials(32000, 8192, 1024) == 0
    with pytest.raises(ValueError):
        lib.call("qmoe_gemm_wgrad_split", gs.ptr, xs.ptr, out.ptr, scratch.ptr, 32000, 8192, 1024, 0)
