"""Pure-Python (no numpy) restatement of the upstream CPU path of the Mixture-of-Experts layer.

TEST INFRASTRUCTURE ONLY — the checker and the timed "what the upstream CPU path costs"
baseline, never the product.  It mirrors the upstream loop structure (scalar triple-loop matrix
products over flat ``array('d')`` buffers) so that timing it on a token subsample measures the
same kind of work as the upstream package on ``device="cpu"``; the numpy oracle in
``moe_oracle.py`` is the one used for parity at real sizes.  Parity status: pinned through
``tests/test_oracle_golden.py`` (it must agree with the numpy oracle, which is itself pinned to
the upstream package's own outputs).

Only small cases are practical: the matrix product below runs at a few million
multiply-accumulates per second.
"""
from __future__ import annotations

from array import array
from math import exp, fsum


def zeros(n):
    return array("d", bytes(8 * n))


def gemm(a, b, rows, inner, cols, *, transpose_left=False, transpose_right=False):
    """``C[rows, cols] = op(A) op(B)`` by scalar loops; src/qutai/backends/cpu_lm.py:11-42."""
    out = zeros(rows * cols)
    for i in range(rows):
        for j in range(cols):
            value = 0.0
            for k in range(inner):
                value += (a[k * rows + i if transpose_left else i * inner + k]
                          * b[j * inner + k if transpose_right else k * cols + j])
            out[i * cols + j] = value
    return out


def _sigmoid(x):
    return 1 / (1 + exp(-x)) if x >= 0 else exp(x) / (1 + exp(x))


def silu(values):
    """src/qutai/backends/cpu_lm.py:107-111."""
    return array("d", (x * _sigmoid(x) for x in values))


def silu_backward(gradient, values):
    """src/qutai/backends/cpu_lm.py:114-122."""
    out = zeros(len(values))
    for i, (g, x) in enumerate(zip(gradient, values)):
        s = _sigmoid(x)
        out[i] = g * s * (1 + x * (1 - s))
    return out


def routing(scores, rows, experts, top_k):
    """src/qutai/backends/cpu_lm.py:204-242 with the softmax of src/qutai/backends/cpu.py:250-260."""
    probs = zeros(rows * experts)
    for row in range(rows):
        items = scores[row * experts:(row + 1) * experts]
        peak = max(items)
        weights = [exp(v - peak) for v in items]
        total = fsum(weights)
        for e, w in enumerate(weights):
            probs[row * experts + e] = w / total
    weights = zeros(rows * top_k)
    indices = array("q", bytes(8 * rows * top_k))
    ids = [[] for _ in range(experts)]
    slots = [[] for _ in range(experts)]
    for row in range(rows):
        selected = sorted(range(experts), key=lambda e: probs[row * experts + e], reverse=True)[:top_k]
        total = sum(probs[row * experts + e] for e in selected)
        for slot, e in enumerate(selected):
            indices[row * top_k + slot] = e
            weights[row * top_k + slot] = probs[row * experts + e] / total
            ids[e].append(row)
            slots[e].append(slot)
    counts = tuple(map(len, ids))
    utilization = array("d", (c / (rows * top_k) for c in counts))
    aux = experts * sum(
        utilization[e] * sum(probs[row * experts + e] for row in range(rows)) / rows
        for e in range(experts))
    return dict(probs=probs, weights=weights, indices=indices, counts=counts, ids=ids,
                slots=slots, utilization=utilization, aux=aux, rows=rows, experts=experts,
                top_k=top_k)


def routing_backward(gradient, route, auxiliary=False):
    """src/qutai/backends/cpu_lm.py:245-276."""
    rows, experts, top_k = route["rows"], route["experts"], route["top_k"]
    probs, util, w = route["probs"], route["utilization"], route["weights"]
    out = zeros(rows * experts)
    for row in range(rows):
        if auxiliary:
            center = sum(probs[row * experts + e] * util[e] for e in range(experts))
            for e in range(experts):
                out[row * experts + e] = (gradient[0] * experts / rows * probs[row * experts + e]
                                          * (util[e] - center))
        else:
            center = sum(gradient[row * top_k + s] * w[row * top_k + s] for s in range(top_k))
            for s in range(top_k):
                e = route["indices"][row * top_k + s]
                out[row * experts + e] = w[row * top_k + s] * (gradient[row * top_k + s] - center)
    return out


def moe_forward_backward(x, router, gate, up, down, rows, width, hidden, top_k, grad_y, grad_aux):
    """One forward plus backward of the layer on flat buffers (src/qutai/lm/layers.py:376-402 and
    the closures it registers).  ``gate[e]``/``up[e]`` are (hidden, width), ``down[e]`` is
    (width, hidden), all flat row-major.  Returns ``(y, aux, grads)`` with the same keys as the
    numpy oracle's ``moe_backward``.
    """
    experts = len(gate)
    scores = gemm(x, router, rows, width, experts, transpose_right=True)
    route = routing(scores, rows, experts, top_k)
    w = route["weights"]
    y = zeros(rows * width)
    saved = {}
    for e in range(experts):
        count = route["counts"][e]
        if not count:
            continue
        xe = array("d", (x[row * width + j] for row in route["ids"][e] for j in range(width)))
        g = gemm(xe, gate[e], count, width, hidden, transpose_right=True)
        u = gemm(xe, up[e], count, width, hidden, transpose_right=True)
        act = silu(g)
        hid = array("d", (a * b for a, b in zip(act, u)))
        ye = gemm(hid, down[e], count, hidden, width, transpose_right=True)
        saved[e] = (xe, g, u, act, hid, ye)
        for i, (row, slot) in enumerate(zip(route["ids"][e], route["slots"][e])):
            factor = w[row * top_k + slot]
            for j in range(width):
                y[row * width + j] += factor * ye[i * width + j]
    # backward
    dw = zeros(rows * top_k)
    dx = zeros(rows * width)
    grads = dict(gate=[None] * experts, up=[None] * experts, down=[None] * experts)
    for e, (xe, g, u, act, hid, ye) in saved.items():
        count = route["counts"][e]
        dy = zeros(count * width)
        for i, (row, slot) in enumerate(zip(route["ids"][e], route["slots"][e])):
            at = row * top_k + slot
            for j in range(width):
                dy[i * width + j] = grad_y[row * width + j] * w[at]
                dw[at] += grad_y[row * width + j] * ye[i * width + j]
        d_hid = gemm(dy, down[e], count, width, hidden)
        grads["down"][e] = gemm(dy, hid, width, count, hidden, transpose_left=True)
        d_up = array("d", (a * b for a, b in zip(d_hid, act)))
        d_gate = silu_backward(array("d", (a * b for a, b in zip(d_hid, u))), g)
        grads["gate"][e] = gemm(d_gate, xe, hidden, count, width, transpose_left=True)
        grads["up"][e] = gemm(d_up, xe, hidden, count, width, transpose_left=True)
        dxe_a = gemm(d_gate, gate[e], count, hidden, width)
        dxe_b = gemm(d_up, up[e], count, hidden, width)
        for i, row in enumerate(route["ids"][e]):
            for j in range(width):
                dx[row * width + j] += dxe_a[i * width + j] + dxe_b[i * width + j]
    d_scores = routing_backward(dw, route)
    if grad_aux:
        extra = routing_backward([grad_aux], route, True)
        for i in range(len(d_scores)):
            d_scores[i] += extra[i]
    grads["scores"] = d_scores
    grads["router"] = gemm(d_scores, x, experts, rows, width, transpose_left=True)
    dxr = gemm(d_scores, router, rows, experts, width)
    for i in range(rows * width):
        dx[i] += dxr[i]
    grads["x"] = dx
    grads["weights"] = dw
    return y, route["aux"], grads, route
