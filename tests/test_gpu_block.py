"""The feed-forward half of a block with the norm and the residual fused into the layer,
``out = x + MoE(rms_norm(x))`` (``qutai_b200.layers.MoEFeedForward`` over ``qmoe_block_forward`` / ``_backward``),
against the fixtures the upstream package produced (fp32, 1e-4) and against the oracle (bf16, 2e-2), through the
C ABI.  Needs a B200: run with ``-m gpu``."""
import os

import numpy as np
import pytest

from conftest import golden_files
from oracle import moe_oracle as oracle

pytestmark = pytest.mark.gpu

FP32_TOL, BF16_TOL = 1e-4, 2e-2
FP32_ELEMENT_TOL = 2e-5      # |x - y| <= 2e-5 (1 + |y|), upstream's fp32 bar (tests/test_lm_moe.py:105-138)


def rel(a, b):
    return oracle.max_rel_err(a, b)


def make_block(norm_weight, eps, router, gate, up, down, top_k, engine="auto"):
    from gpu_util import make_layer
    from qutai_b200.layers import MoEFeedForward, RMSNorm

    layer = make_layer(None, router, gate, up, down, top_k, engine=engine)
    norm = RMSNorm(gate.shape[2], eps)
    norm.weight.storage.upload_bytes(np.ascontiguousarray(norm_weight, dtype=np.float32).tobytes())
    return MoEFeedForward(norm, layer)


def run_block(block, x, grad_out, grad_aux, dtype):
    from gpu_util import to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.layers import Tensor

    T, d = x.shape
    layer = block.ffn
    E, h = layer.n_experts, layer.d_expert
    for p in block.parameters():
        p.zero_grad()
    xs = to_device(x, dtype)
    out, aux = block(Tensor(xs, (T, d)))
    ga = to_device(np.array([grad_aux]), "float32") if grad_aux is not None else None
    dx = block.backward(Tensor(to_device(grad_out, dtype), (T, d)), ga)
    work = layer._saved[0]
    result = dict(
        out=to_host(out.storage, (T, d)), aux=float(to_host(aux.storage)[0]), dx=to_host(dx.storage, (T, d)),
        counts=layer.last_counts, scores=to_host(work["buf"]["scores"], (T, E)),
        d_norm_weight=to_host(block.ffn_norm.weight.grad.storage),
        d_router=to_host(layer.router.weight.grad.storage, (E, d)),
        d_gate=[None if ex.gate.weight.grad is None else to_host(ex.gate.weight.grad.storage, (h, d)) for ex in layer.experts],
        d_up=[None if ex.up.weight.grad is None else to_host(ex.up.weight.grad.storage, (h, d)) for ex in layer.experts],
        d_down=[None if ex.down.weight.grad is None else to_host(ex.down.weight.grad.storage, (d, h)) for ex in layer.experts])
    assert lib.device_status() == 0
    return result


@pytest.mark.parametrize("path", golden_files("block"), ids=os.path.basename)
def test_block_fp32_matches_the_upstream_fixture(path):
    g = np.load(path)
    block = make_block(g["norm_weight"], float(g["eps"]), g["router"], g["gate"], g["up"], g["down"], int(g["top_k"]))
    got = run_block(block, g["x"], g["grad_out"], float(g["grad_aux"]), "float32")
    E, step = g["gate"].shape[0], int(g["sample"])
    assert got["counts"] == tuple(g["counts"].tolist())
    assert abs(got["aux"] - float(g["aux"])) <= 1e-5
    for name, want in (("out", g["out"]), ("dx", g["dx"]), ("d_norm_weight", g["d_norm_weight"]), ("d_router", g["d_router"])):
        assert rel(got[name], want) <= FP32_TOL, name
        assert oracle.elementwise_err(got[name], want) <= FP32_ELEMENT_TOL, name
    for e in range(E):
        for key in ("gate", "up", "down"):
            mine = got["d_" + key][e]
            if not g["has_grad"][e]:
                assert mine is None
            else:
                assert rel(mine.reshape(-1)[::step], g[f"d_{key}_{e}"]) <= FP32_TOL, (key, e)
    again = run_block(block, g["x"], g["grad_out"], float(g["grad_aux"]), "float32")
    for name in ("out", "dx", "d_norm_weight", "d_router"):     # no floating-point atomics: a second pass gives the same bits
        assert np.array_equal(again[name], got[name]), name


BLOCK_SHAPES = [(64, 64, 4, 2, 128), (300, 72, 5, 2, 136), (1000, 256, 8, 2, 512), (777, 128, 16, 4, 264), (900, 384, 3, 1, 640)]


@pytest.mark.parametrize("engine", ["simt", "tcgen05"])
@pytest.mark.parametrize("T,d,E,k,h", BLOCK_SHAPES)
def test_block_bf16_matches_the_oracle(T, d, E, k, h, engine):
    rng = np.random.default_rng(T + d + E + 1)
    r16 = oracle.round_bf16
    x, grad_out = r16(rng.standard_normal((T, d)) * 1.5 + 0.1), r16(rng.standard_normal((T, d)))
    norm_weight = (1.0 + 0.2 * rng.standard_normal(d)).astype(np.float32)
    router = rng.standard_normal((E, d)).astype(np.float32) * 0.05
    gate = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    up = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    down = rng.standard_normal((E, d, h)).astype(np.float32) / np.sqrt(h)
    block = make_block(norm_weight, 1e-6, router, gate, up, down, k, engine=engine)
    got = run_block(block, x, grad_out, 0.37, "bfloat16")
    # router logits of the normalised activations: fp32 arithmetic on exactly these inputs
    normed, _ = oracle.rms_norm(x, norm_weight, 1e-6)
    assert rel(got["scores"], normed @ router.astype(np.float64).T) <= 1e-4
    out, aux, ctx = oracle.block_ffn_forward(x, norm_weight, 1e-6, router, r16(gate), r16(up), r16(down), k, scores=got["scores"])
    grads = oracle.block_ffn_backward(ctx, grad_out, 0.37)
    counts = ctx["moe"]["route"]["counts"]
    assert got["counts"] == counts
    assert abs(got["aux"] - aux) <= 1e-4 * max(1.0, abs(aux))
    for name, want in (("out", out), ("dx", grads["x"]), ("d_norm_weight", grads["norm_weight"]), ("d_router", grads["router"])):
        assert rel(got[name], want) <= BF16_TOL, name
    for e in range(E):
        for key in ("gate", "up", "down"):
            mine, want = got["d_" + key][e], grads[key][e]
            if counts[e] == 0:
                assert mine is None and want is None
            else:
                assert rel(mine, want) <= BF16_TOL, (key, e)


def test_fused_block_agrees_with_the_unfused_chain_at_full_size():
    """C2's shape (16384 tokens, d 1024, 8 experts top-2, hidden 2816, bf16): routing bit-exact on the device's own
    logits; out and dx of sampled tokens against the oracle on those tokens; and the norm weight's gradient — a sum
    over ALL tokens — against the oracle's norm backward applied to the input gradient that the UNFUSED layer
    returns for the same normalised activations (run in fp32, so that it routes the tokens the same way: the sum
    over tokens is a sum of terms of either sign, and re-routing even one token in a hundred moves it by more than
    a tenth of its size)."""
    from gpu_util import make_layer, to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.layers import Tensor

    T, d, E, k, h = 16384, 1024, 8, 2, 2816
    rng = np.random.default_rng(7)

    def normal32(shape, std):
        out = rng.standard_normal(shape, dtype=np.float32)
        out *= np.float32(std)
        return oracle.round_bf16(out).astype(np.float32)

    x, grad_out = normal32((T, d), 1.3), normal32((T, d), 1.0)
    norm_weight = (1.0 + 0.2 * rng.standard_normal(d)).astype(np.float32)
    router = rng.standard_normal((E, d)).astype(np.float32) * np.float32(0.01)
    gate, up, down = normal32((E, h, d), d ** -0.5), normal32((E, h, d), d ** -0.5), normal32((E, d, h), h ** -0.5)
    block = make_block(norm_weight, 1e-6, router, gate, up, down, k, engine="tcgen05")
    got = run_block(block, x, grad_out, None, "bfloat16")
    expected = oracle.routing(got["scores"], k)
    assert got["counts"] == expected["counts"] and sum(got["counts"]) == T * k
    sample = np.sort(rng.choice(T, size=48, replace=False))
    out, _, ctx = oracle.block_ffn_forward(x[sample], norm_weight, 1e-6, router, gate, up, down, k, scores=got["scores"][sample])
    grads = oracle.block_ffn_backward(ctx, grad_out[sample], 0.0)
    assert rel(got["out"][sample], out) <= BF16_TOL
    assert rel(got["dx"][sample], grads["x"]) <= BF16_TOL
    # the unfused chain on the same normalised activations: its input gradient is the gradient of rms_norm(x)
    normed, inverse = oracle.rms_norm(x, norm_weight, 1e-6)
    plain = make_layer(None, router, gate, up, down, k)
    xn = Tensor(to_device(normed, "float32"), (T, d))
    plain(xn)
    d_normed = to_host(plain.backward(Tensor(to_device(grad_out, "float32"), (T, d)), None).storage, (T, d))
    # logits that nearly tie may still order differently by a rounding: those few tokens are left out of the row-wise check
    routed_alike = np.all(to_host(plain._saved[0]["buf"]["expert_index"], (T, k)) ==
                          to_host(block.ffn._saved[0]["buf"]["expert_index"], (T, k)), axis=1)
    assert routed_alike.mean() >= 0.999
    dx_norm, d_weight = oracle.rms_norm_backward(d_normed, x, norm_weight, inverse)
    assert rel(got["d_norm_weight"], d_weight) <= BF16_TOL
    assert rel(got["dx"][routed_alike], (grad_out.astype(np.float64) + dx_norm)[routed_alike]) <= BF16_TOL
    assert lib.device_status() == 0
