"""The functions of the backend table around attention and the feed-forward half of a block
(``qutai_b200.cuda_lm``: ``rms_norm``, ``rms_norm_backward``, ``rope``, ``embedding``, ``embedding_backward``,
``attention``, ``attention_backward``) with upstream's call signatures: float32 against the fixtures the upstream CPU
backend produced, bfloat16 and larger shapes against the oracle.  Needs a B200: ``-m gpu``."""
import os
import sys

import numpy as np
import pytest

from oracle import moe_oracle as oracle

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from attention_inputs import attention_inputs  # noqa: E402

pytestmark = pytest.mark.gpu

FP32_ELEMENT_TOL = 2e-5      # |x - y| <= 2e-5 (1 + |y|)
BF16_TOL = 2e-2


def fixture():
    return np.load(os.path.join(os.path.dirname(__file__), "golden", "lm_ops.npz"))


def near(got, want, tol=FP32_ELEMENT_TOL):
    assert oracle.elementwise_err(got, want) <= tol


def test_rms_norm_and_its_backward_fp32_match_the_upstream_fixture():
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm

    g = fixture()
    rows, width = g["norm_x"].shape
    x, w, grad = to_device(g["norm_x"], "float32"), to_device(g["norm_w"], "float32"), to_device(g["norm_g"], "float32")
    out, inverse = cuda_lm.rms_norm(x, w, width, float(g["norm_eps"]))
    assert out.dtype == "float32" and inverse.size == rows
    near(to_host(out, (rows, width)), g["norm_out"])
    near(to_host(inverse), g["norm_inverse"])
    dx, dw = cuda_lm.rms_norm_backward(grad, x, w, inverse, width)
    near(to_host(dx, (rows, width)), g["norm_dx"])
    near(to_host(dw), g["norm_dw"])


@pytest.mark.parametrize("rows,width", [(1, 8), (300, 1024), (4099, 2048), (77, 72), (64, 1030)])
def test_rms_norm_bf16_rows_against_the_oracle(rows, width):
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm

    rng = np.random.default_rng(rows + width)
    x = oracle.round_bf16(rng.standard_normal((rows, width)) * 1.5 + 0.3)
    grad = oracle.round_bf16(rng.standard_normal((rows, width)))
    w = (1 + 0.1 * rng.standard_normal(width)).astype(np.float32)
    xs, gs, ws = to_device(x, "bfloat16"), to_device(grad, "bfloat16"), to_device(w, "float32")
    out, inverse = cuda_lm.rms_norm(xs, ws, width, 1e-6)
    assert out.dtype == "float32"                       # upstream's norm hands float32 on (cuda_lm.py:128-131)
    want_out, want_inverse = oracle.rms_norm(x, w, 1e-6)
    near(to_host(out, (rows, width)), want_out)
    near(to_host(inverse), want_inverse)
    dx, dw = cuda_lm.rms_norm_backward(gs, xs, ws, inverse, width)
    want_dx, want_dw = oracle.rms_norm_backward(grad, x, w, want_inverse)
    assert dx.dtype == "bfloat16" and oracle.max_rel_err(to_host(dx, (rows, width)), want_dx) <= BF16_TOL
    assert oracle.max_rel_err(to_host(dw), want_dw) <= 1e-4
    again = cuda_lm.rms_norm_backward(gs, xs, ws, inverse, width)[1]
    assert np.array_equal(to_host(again), to_host(dw))   # fixed summation order


def test_rope_matches_the_upstream_fixture_and_undoes_itself():
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm

    g = fixture()
    v = g["rope_v"]
    batch, time, features = v.shape
    heads, theta, offset = int(g["rope_heads"]), float(g["rope_theta"]), int(g["rope_offset"])
    dims = (batch, time, heads, features // heads, theta, offset)
    turned = cuda_lm.rope(to_device(v, "float32"), *dims)
    near(to_host(turned, v.shape), g["rope_out"])
    near(to_host(cuda_lm.rope(to_device(v, "float32"), *dims, inverse=True), v.shape), g["rope_inverse"])
    near(to_host(cuda_lm.rope(turned, *dims, inverse=True), v.shape), v)
    # bfloat16, the shape of the decoder step's keys: positions up to 2047
    rng = np.random.default_rng(3)
    big = oracle.round_bf16(rng.standard_normal((2, 2048, 4 * 64)))
    got = to_host(cuda_lm.rope(to_device(big, "bfloat16"), 2, 2048, 4, 64, 10000.0), big.shape)
    assert oracle.elementwise_err(got, oracle.rope(big, 4, 10000.0), bf16=True) <= 0.012


def test_embedding_and_its_backward_match_the_upstream_fixture():
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm

    g = fixture()
    table, ids, grad = g["emb_table"], g["emb_ids"].tolist(), g["emb_grad"]
    vocab, width = table.shape
    ts = to_device(table, "float32")
    np.testing.assert_array_equal(to_host(cuda_lm.embedding(ts, ids, width), (len(ids), width)), g["emb_out"])
    half = to_host(cuda_lm.embedding(ts, ids, width, out_dtype="bfloat16"), (len(ids), width))
    np.testing.assert_array_equal(half, oracle.round_bf16(g["emb_out"]))
    d_table = cuda_lm.embedding_backward(to_device(grad, "float32"), ids, vocab, width)
    near(to_host(d_table, (vocab, width)), g["emb_d_table"])
    with pytest.raises(ValueError):
        cuda_lm.embedding(to_device(table, "bfloat16"), ids, width)          # the table must be float32
    # many repeats of few tokens (Zipf-like), bfloat16 gradients: sums in position order, the same bits every time
    rng = np.random.default_rng(8)
    ids = np.minimum(rng.zipf(1.3, size=5000) - 1, 999).tolist()
    grad = oracle.round_bf16(rng.standard_normal((5000, 64)))
    first = to_host(cuda_lm.embedding_backward(to_device(grad, "bfloat16"), ids, 1000, 64), (1000, 64))
    assert oracle.max_rel_err(first, oracle.embedding_backward(grad, ids, 1000)) <= 1e-5
    assert np.array_equal(first, to_host(cuda_lm.embedding_backward(to_device(grad, "bfloat16"), ids, 1000, 64), (1000, 64)))


def test_attention_of_the_function_table_has_upstreams_signature():
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm

    batch, time, heads, kv_heads, dim = 2, 70, 4, 2, 64
    q, k, v, grad = attention_inputs(batch, time, heads, kv_heads, seed=12, scale=0.8)
    qs, ks, vs, gs = (to_device(a, "bfloat16") for a in (q, k, v, grad))
    out, lse = cuda_lm.attention(qs, ks, vs, batch, time, heads, kv_heads, dim)
    want_out, want_lse = oracle.attention_forward(q, k, v, heads, kv_heads)
    assert oracle.max_rel_err(to_host(out, q.shape), want_out) <= BF16_TOL
    assert np.abs(to_host(lse, (batch, time, heads)) - want_lse).max() <= 1e-3
    dq, dk, dv = cuda_lm.attention_backward(gs, qs, ks, vs, out, lse, batch, time, heads, kv_heads, dim)
    want = oracle.attention_backward(grad, q, k, v, want_out, want_lse, heads, kv_heads)
    for got, expected, shape in ((dq, want[0], q.shape), (dk, want[1], k.shape), (dv, want[2], v.shape)):
        assert oracle.max_rel_err(to_host(got, shape), expected) <= BF16_TOL
    with pytest.raises(ValueError):
        cuda_lm.attention(qs, ks, vs, batch, time, heads * 2, kv_heads * 2, dim // 2)      # head width 32


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_chunked_head_loop_over_the_function_table_reproduces_the_upstream_loss(dtype):
    """A host that keeps upstream's chunk loop (src/qutai/lm/layers.py:199-255: head_rows, gemm, head_loss and, in
    the backward, head_gradient, two more gemms, head_rows_backward) and points every call at this table gets the
    fixture's loss and gradients (float32), or the oracle's on bf16 values."""
    from gpu_util import to_device, to_host
    from qutai_b200 import cuda_lm

    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "head_mid.npz"))
    hidden, weight, labels = g["hidden"], g["weight"], g["labels"]
    if dtype == "bfloat16":
        hidden, weight = oracle.round_bf16(hidden), oracle.round_bf16(weight)
    batch, time, width = hidden.shape
    vocab, chunk = weight.shape[0], 7
    targets = labels[:, 1:].reshape(-1).tolist()
    count = max(1, sum(t != -100 for t in targets))
    hs, ws = to_device(hidden, dtype), to_device(weight, dtype)
    prepared = cuda_lm.prepare_labels(targets)
    total = to_device(np.zeros(1), "float32")
    for start in range(0, len(targets), chunk):
        rows = min(chunk, len(targets) - start)
        inputs = cuda_lm.head_rows(hs, start, rows, width, time)
        logits = cuda_lm.gemm(inputs, ws, rows, width, vocab, transpose_right=True, out_dtype=dtype)
        cuda_lm.add_into(total, cuda_lm.head_loss(logits, prepared, rows, vocab, start=start))
    loss = to_host(total)[0] / count
    incoming = to_device(np.array([float(g["gradient"])]), "float32")
    dx = to_device(np.zeros(hidden.size), dtype)
    dw = to_device(np.zeros(weight.size), "float32")
    for start in range(0, len(targets), chunk):
        rows = min(chunk, len(targets) - start)
        inputs = cuda_lm.head_rows(hs, start, rows, width, time)
        logits = cuda_lm.gemm(inputs, ws, rows, width, vocab, transpose_right=True, out_dtype=dtype)
        cuda_lm.head_gradient(logits, prepared, rows, vocab, incoming, count, start=start)
        cuda_lm.head_rows_backward(dx, cuda_lm.gemm(logits, ws, rows, vocab, width, out_dtype=dtype), start, rows, width, time)
        cuda_lm.gemm(logits, inputs, vocab, rows, width, transpose_left=True, out_dtype="float32", out=dw, accumulate=True)
    got_dx, got_dw = to_host(dx, hidden.shape), to_host(dw, weight.shape)
    if dtype == "float32":
        assert abs(loss - float(g["loss"])) <= FP32_ELEMENT_TOL * (1 + abs(float(g["loss"])))
        near(got_dx, g["d_hidden"])
        near(got_dw, g["d_weight"])
    else:
        want_loss, ctx = oracle.head_loss_forward(hidden, weight, labels)
        want_dx, want_dw, _ = oracle.head_loss_backward(ctx, float(g["gradient"]))
        assert abs(loss - want_loss) <= BF16_TOL * max(1.0, abs(want_loss))
        assert oracle.max_rel_err(got_dx, want_dx) <= BF16_TOL and oracle.max_rel_err(got_dw, want_dw) <= BF16_TOL
