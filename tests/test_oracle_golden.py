"""Pin the CPU oracle: every function of ``oracle/moe_oracle.py`` (and the pure-Python restatement)
against the fixtures produced by the upstream package itself (``tests/golden/make_golden.py``)."""
import os
import sys

import numpy as np
import pytest

from conftest import golden_files
from oracle import moe_oracle as oracle
from oracle import moe_pure as pure

RTOL = 1e-12


def close(a, b, tol=RTOL):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape
    scale = max(1.0, float(np.abs(b).max()) if b.size else 1.0)
    assert float(np.abs(a - b).max() if a.size else 0.0) <= tol * scale


def split(flat, counts):
    return np.split(flat, np.cumsum(counts)[:-1])


@pytest.mark.parametrize("path", golden_files("routing"), ids=os.path.basename)
def test_routing_matches_upstream(path):
    g = np.load(path)
    route = oracle.routing(g["scores"], int(g["top_k"]))
    assert np.array_equal(route["indices"], g["indices"])
    assert route["counts"] == tuple(g["counts"].tolist())
    for mine, theirs in zip(route["ids"], split(g["ids"], g["counts"])):
        assert np.array_equal(mine, theirs)
    for mine, theirs in zip(route["slots"], split(g["slots"], g["counts"])):
        assert np.array_equal(mine, theirs)
    close(route["probs"], g["probs"])
    close(route["weights"], g["weights"])
    close(route["utilization"], g["utilization"])
    close(route["aux"], g["aux"])
    close(route["weights"].sum(axis=1), np.ones(route["rows"]))
    close(oracle.routing_backward(g["grad_weights"], route), g["d_scores_gate"])
    close(oracle.routing_backward([float(g["grad_aux"])], route, True), g["d_scores_aux"])
    # locations are implied by ids/slots: assignment (row, slot) sits at row `location` of its expert
    for e in range(route["experts"]):
        at = route["ids"][e] * route["top_k"] + route["slots"][e]
        assert np.array_equal(route["locations"].reshape(-1)[at], np.arange(at.size))


def test_known_answers_of_upstream_tests():
    route = oracle.routing(np.array([[3.0, 2.0, -1.0], [-1.0, 2.0, 3.0]]), 2)
    assert route["indices"].reshape(-1).tolist() == [0, 1, 2, 1]
    assert route["counts"] == (1, 2, 1)
    route = oracle.routing(np.zeros((4, 5)), 2)   # all equal: lowest expert indices win
    assert route["indices"].tolist() == [[0, 1]] * 4
    assert abs(sum(route["utilization"]) - 1) < 1e-12


@pytest.mark.parametrize("path", golden_files("layer"), ids=os.path.basename)
def test_layer_matches_upstream(path):
    g = np.load(path)
    experts, step = g["gate"].shape[0], int(g["sample"])
    y, aux, ctx = oracle.moe_forward(g["x"], g["router"], g["gate"], g["up"], g["down"], int(g["top_k"]))
    grads = oracle.moe_backward(ctx, g["grad_y"], float(g["grad_aux"]))
    assert ctx["route"]["counts"] == tuple(g["counts"].tolist())
    close(y, g["y"])
    close(aux, g["aux"])
    close(ctx["route"]["utilization"], g["utilization"])
    close(grads["x"], g["dx"])
    close(grads["router"], g["d_router"])
    for e in range(experts):
        for key in ("gate", "up", "down"):
            mine, theirs = grads[key][e], g[f"d_{key}_{e}"]
            if not g["has_grad"][e]:
                assert mine is None and theirs.size == 0
            else:
                close(mine.reshape(-1)[::step], theirs)


@pytest.mark.parametrize("name", ["layer_small", "layer_k_eq_e", "layer_empty_expert", "layer_tied_router_rows"])
def test_pure_python_restatement_matches(name):
    from array import array

    g = np.load(os.path.join(os.path.dirname(golden_files("layer")[0]), name + ".npz"))
    rows, width = g["x"].shape
    experts, hidden = g["gate"].shape[0], g["gate"].shape[1]
    flat = lambda a: array("d", np.asarray(a, dtype=np.float64).reshape(-1).tolist())
    y, aux, grads, route = pure.moe_forward_backward(
        flat(g["x"]), flat(g["router"]), [flat(w) for w in g["gate"]], [flat(w) for w in g["up"]],
        [flat(w) for w in g["down"]], rows, width, hidden, int(g["top_k"]), flat(g["grad_y"]),
        float(g["grad_aux"]))
    assert route["counts"] == tuple(g["counts"].tolist())
    close(np.array(y).reshape(rows, width), g["y"])
    close(aux, g["aux"])
    close(np.array(grads["x"]).reshape(rows, width), g["dx"])
    close(np.array(grads["router"]).reshape(experts, width), g["d_router"])
    for e in range(experts):
        if not g["has_grad"][e]:
            assert grads["gate"][e] is None
        else:
            close(np.array(grads["down"][e]), g[f"d_down_{e}"])
            close(np.array(grads["gate"][e]), g[f"d_gate_{e}"])


def test_bf16_rounding_helper():
    a = np.array([1.0, 1.00390625, 1.0 + 2 ** -8, 1.0 + 3 * 2 ** -8, -2.5, 3.1415926])
    r = oracle.round_bf16(a)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == 1.0            # 1+2^-8 ties to even (1.0)
    assert r[3] == 1.0 + 2 ** -6                                  # 1+3*2^-8 ties to even upward
    assert r[4] == -2.5 and abs(r[5] - 3.140625) < 1e-12


@pytest.mark.parametrize("path", golden_files("block"), ids=os.path.basename)
def test_block_oracle_matches_the_upstream_norm_layer_and_residual(path):
    """``x + ffn(ffn_norm(x))`` (RMS norm, the layer, the residual add) against what the upstream package produced
    for it on its CPU float64 path (tests/golden/make_golden_block.py)."""
    g = np.load(path)
    experts, step = g["gate"].shape[0], int(g["sample"])
    out, aux, ctx = oracle.block_ffn_forward(g["x"], g["norm_weight"], float(g["eps"]), g["router"], g["gate"], g["up"],
                                             g["down"], int(g["top_k"]))
    grads = oracle.block_ffn_backward(ctx, g["grad_out"], float(g["grad_aux"]))
    assert ctx["moe"]["route"]["counts"] == tuple(g["counts"].tolist())
    close(out, g["out"])
    close(aux, g["aux"])
    close(grads["x"], g["dx"])
    close(grads["norm_weight"], g["d_norm_weight"])
    close(grads["router"], g["d_router"])
    for e in range(experts):
        for key in ("gate", "up", "down"):
            mine, theirs = grads[key][e], g[f"d_{key}_{e}"]
            if not g["has_grad"][e]:
                assert mine is None and theirs.size == 0
            else:
                close(mine.reshape(-1)[::step], theirs)


@pytest.mark.parametrize("path", golden_files("head"), ids=os.path.basename)
def test_head_oracle_matches_the_upstream_projection_loss(path):
    """The language-model head and its cross-entropy loss against what the upstream package's chunked
    ``projection_loss`` produced on its CPU float64 path (tests/golden/make_golden_head.py): the loss, and the
    gradients of the hidden states and of the weight for the stored incoming gradient."""
    g = np.load(path)
    loss, ctx = oracle.head_loss_forward(g["hidden"], g["weight"], g["labels"])
    d_hidden, d_weight, _ = oracle.head_loss_backward(ctx, float(g["gradient"]))
    close(loss, g["loss"])
    close(d_hidden, g["d_hidden"])
    close(d_weight, g["d_weight"])
    assert not d_hidden[:, -1, :].any()          # the last position of a sequence has no target


@pytest.mark.parametrize("path", golden_files("attention"), ids=os.path.basename)
def test_attention_oracle_matches_the_upstream_cpu_backend(path):
    """Causal attention with grouped key/value heads, forward and backward, against what the upstream pure-Python
    CPU backend produced (tests/golden/make_golden_attention.py)."""
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    from attention_inputs import attention_inputs

    g = np.load(path)
    heads, kv_heads = int(g["heads"]), int(g["kv_heads"])
    q, k, v, grad = attention_inputs(int(g["batch"]), int(g["time"]), heads, kv_heads, int(g["seed"]), float(g["scale"]))
    out, lse = oracle.attention_forward(q, k, v, heads, kv_heads)
    dq, dk, dv = oracle.attention_backward(grad, q, k, v, out, lse, heads, kv_heads)
    for mine, theirs in ((out, g["out"]), (lse, g["lse"]), (dq, g["dq"]), (dk, g["dk"]), (dv, g["dv"])):
        assert np.abs(mine - theirs).max() <= 2e-6 * (1 + np.abs(theirs).max())      # the fixtures are stored in float32


def test_small_lm_operations_of_the_oracle_match_the_upstream_cpu_backend():
    """RMS norm and its backward, the rotary embedding and its inverse, the token embedding and its backward against
    what the upstream pure-Python CPU backend produced (tests/golden/make_golden_lm_ops.py)."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "lm_ops.npz"))
    out, inverse = oracle.rms_norm(g["norm_x"], g["norm_w"], float(g["norm_eps"]))
    dx, dw = oracle.rms_norm_backward(g["norm_g"], g["norm_x"], g["norm_w"], inverse)
    for mine, theirs in ((out, g["norm_out"]), (inverse, g["norm_inverse"]), (dx, g["norm_dx"]), (dw, g["norm_dw"])):
        close(mine, theirs)
    heads, theta, offset = int(g["rope_heads"]), float(g["rope_theta"]), int(g["rope_offset"])
    close(oracle.rope(g["rope_v"], heads, theta, offset), g["rope_out"])
    close(oracle.rope(g["rope_v"], heads, theta, offset, inverse=True), g["rope_inverse"])
    close(oracle.rope(oracle.rope(g["rope_v"], heads, theta, offset), heads, theta, offset, inverse=True), g["rope_v"])
    close(oracle.embedding(g["emb_table"], g["emb_ids"]), g["emb_out"])
    close(oracle.embedding_backward(g["emb_grad"], g["emb_ids"], g["emb_table"].shape[0]), g["emb_d_table"])
