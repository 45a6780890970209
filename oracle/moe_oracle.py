"""CPU float64 oracle for the Mixture-of-Experts layer: a numpy restatement of the upstream
pure-Python CPU path.

TEST INFRASTRUCTURE ONLY.  This file is the checker, never the product: only the test-suite,
the smoke check and the CPU-baseline / reference legs of the benchmark may import it.  The
shipped package never does, and has no CPU fallback.

Parity status: PINNED.  ``tests/golden/*.npz`` hold outputs of the upstream package itself
(``SparseMoE`` on ``device="cpu"``, ``dtype="float64"``), produced by
``tests/golden/make_golden.py``; ``tests/test_oracle_golden.py`` checks every function below
against them (integer tables exactly, floats to 1e-12 relative), and also against the
known-answer cases of the upstream tests (tests/test_lm_moe.py:65-71, :140-162;
tests/test_lm_bfloat16.py:129-167).

Each function cites the upstream file:line it follows.  Arrays are row-major numpy float64
unless stated; integer tables are int64 like the upstream ``array('q')`` storages.
"""
from __future__ import annotations

import numpy as np


# --------------------------------------------------------------------------------------
# element-wise pieces
# --------------------------------------------------------------------------------------
def sigmoid(v):
    """Two-branch stable logistic, as in src/qutai/backends/cpu_lm.py:107-111."""
    v = np.asarray(v, dtype=np.float64)
    out = np.empty_like(v)
    pos = v >= 0
    out[pos] = 1.0 / (1.0 + np.exp(-v[pos]))
    ev = np.exp(v[~pos])
    out[~pos] = ev / (1.0 + ev)
    return out


def silu(v):
    """``x * sigmoid(x)``; src/qutai/backends/cpu_lm.py:107-111."""
    return np.asarray(v, dtype=np.float64) * sigmoid(v)


def silu_backward(g, v):
    """``g * s * (1 + x * (1 - s))``; src/qutai/backends/cpu_lm.py:114-122."""
    s = sigmoid(v)
    return np.asarray(g, dtype=np.float64) * s * (1.0 + np.asarray(v, dtype=np.float64) * (1.0 - s))


def softmax_rows(scores):
    """Row softmax with the row maximum subtracted; src/qutai/backends/cpu.py:250-260.

    The upstream code totals the exponentials with ``math.fsum``; ``np.sum`` differs from that
    by at most a few ulp, far inside every tolerance used with this oracle.
    """
    scores = np.asarray(scores, dtype=np.float64)
    weights = np.exp(scores - scores.max(axis=1, keepdims=True))
    return weights / weights.sum(axis=1, keepdims=True)


# --------------------------------------------------------------------------------------
# routing
# --------------------------------------------------------------------------------------
def routing(scores, top_k):
    """Softmax / top-k gating and the per-expert dispatch tables.

    Follows ``routing`` in src/qutai/backends/cpu_lm.py:204-242:

    * ``probs`` = row softmax of the scores;
    * per row the ``top_k`` experts with the largest probability, ordered by descending
      probability; Python's stable sort with ``reverse=True`` keeps EQUAL probabilities in
      ascending expert index, which a stable argsort of ``-probs`` reproduces;
    * ``weights[r, s] = probs[r, e_s] / sum_s' probs[r, e_s']``;
    * per expert the list of token rows (``ids``) and slot numbers (``slots``) in increasing
      (row, slot) scan order; ``counts``; ``utilization = counts / (rows * top_k)``;
    * ``aux = experts * sum_e utilization[e] * mean_r probs[r, e]``.

    ``locations[r, s]`` (row of assignment (r, s) inside its expert's group) is the extra table
    the upstream CUDA path keeps (src/qutai/backends/cuda/lm.cu:353-383); it is implied by
    ``ids``/``slots`` and is included so the device tables can be compared one to one.
    """
    scores = np.asarray(scores, dtype=np.float64)
    rows, experts = scores.shape
    probs = softmax_rows(scores)
    order = np.argsort(-probs, axis=1, kind="stable")[:, :top_k]
    indices = order.astype(np.int64)
    picked = np.take_along_axis(probs, order, axis=1)
    # Python's sum() over the selected probabilities is a left-to-right float64 sum.
    total = np.zeros(rows, dtype=np.float64)
    for slot in range(top_k):
        total = total + picked[:, slot]
    weights = picked / total[:, None]
    flat = indices.reshape(-1)
    ids, slots = [], []
    locations = np.zeros(rows * top_k, dtype=np.int64)
    for e in range(experts):
        at = np.nonzero(flat == e)[0]
        ids.append((at // top_k).astype(np.int64))
        slots.append((at % top_k).astype(np.int64))
        locations[at] = np.arange(at.size, dtype=np.int64)
    counts = tuple(int(a.size) for a in ids)
    utilization = np.array([c / (rows * top_k) for c in counts], dtype=np.float64)
    aux = experts * float(sum(utilization[e] * probs[:, e].sum() / rows for e in range(experts)))
    return dict(probs=probs, weights=weights, indices=indices, counts=counts, ids=ids,
                slots=slots, locations=locations.reshape(rows, top_k), utilization=utilization,
                aux=aux, rows=rows, experts=experts, top_k=top_k)


def routing_backward(gradient, route, auxiliary=False):
    """Gradient of the gate weights (or of the auxiliary loss) with respect to the scores.

    Follows ``routing_backward`` in src/qutai/backends/cpu_lm.py:245-276.  Gate path:
    ``d[r, e_s] = w[r, s] * (g[r, s] - sum_s' g[r, s'] * w[r, s'])`` and zero for experts that
    were not selected.  Auxiliary path (``utilization`` held constant):
    ``d[r, e] = g * E / T * p[r, e] * (util[e] - sum_j p[r, j] * util[j])``.
    """
    rows, experts, top_k = route["rows"], route["experts"], route["top_k"]
    out = np.zeros((rows, experts), dtype=np.float64)
    if auxiliary:
        g = float(np.asarray(gradient, dtype=np.float64).reshape(-1)[0])
        probs, util = route["probs"], route["utilization"]
        center = probs @ util
        out[:] = g * experts / rows * probs * (util[None, :] - center[:, None])
        return out
    g = np.asarray(gradient, dtype=np.float64).reshape(rows, top_k)
    w = route["weights"]
    center = (g * w).sum(axis=1, keepdims=True)
    np.put_along_axis(out, route["indices"], w * (g - center), axis=1)
    return out


def route_gather(values, route, expert):
    """Rows of ``values`` routed to ``expert``; src/qutai/backends/cpu_lm.py:279-283."""
    return np.asarray(values)[route["ids"][expert]]


def route_gather_backward(gradient, route, expert):
    """Scatter-add into a zero (rows, width) array; src/qutai/backends/cpu_lm.py:286-291."""
    gradient = np.asarray(gradient, dtype=np.float64)
    out = np.zeros((route["rows"], gradient.shape[1]), dtype=np.float64)
    np.add.at(out, route["ids"][expert], gradient)
    return out


def combine(outputs, weights, route):
    """Weighted un-permute: ``out[row] += w[row, slot] * y_e[i]``, expert by expert.

    Follows ``combine`` in src/qutai/backends/cpu_lm.py:294-303; ``outputs`` is a sequence of
    ``(expert, array(c_e, width))`` pairs for the experts that received tokens.
    """
    weights = np.asarray(weights, dtype=np.float64).reshape(route["rows"], route["top_k"])
    width = outputs[0][1].shape[1] if outputs else 0
    result = np.zeros((route["rows"], width), dtype=np.float64)
    for expert, values in outputs:
        rows_e, slots_e = route["ids"][expert], route["slots"][expert]
        # each token appears at most once per expert, so a plain indexed add is exact
        result[rows_e] += weights[rows_e, slots_e][:, None] * np.asarray(values, dtype=np.float64)
    return result


def combine_backward(gradient, outputs, weights, route):
    """``dy_e[i] = g[row] * w[row, slot]`` and ``dw[row, slot] = <g[row], y_e[i]>``.

    Follows ``combine_backward`` in src/qutai/backends/cpu_lm.py:306-320.  Returns
    ``([dy_e for each entry of outputs], dw)``.
    """
    gradient = np.asarray(gradient, dtype=np.float64)
    weights = np.asarray(weights, dtype=np.float64).reshape(route["rows"], route["top_k"])
    dw = np.zeros_like(weights)
    grads = []
    for expert, values in outputs:
        rows_e, slots_e = route["ids"][expert], route["slots"][expert]
        grads.append(gradient[rows_e] * weights[rows_e, slots_e][:, None])
        dw[rows_e, slots_e] = (gradient[rows_e] * np.asarray(values, dtype=np.float64)).sum(axis=1)
    return grads, dw


# --------------------------------------------------------------------------------------
# one expert
# --------------------------------------------------------------------------------------
def expert_forward(xe, w_gate, w_up, w_down):
    """``down(silu(gate(x)) * up(x))`` of one expert on its rows ``xe`` (c_e, d); the expert body of
    src/qutai/lm/layers.py:310-311 with the bias-free linear maps of src/qutai/lm/layers.py:35-48.
    Returns ``(ye, saved)`` with ``saved = (xe, g, u, hidden)`` for the backward."""
    xe = np.asarray(xe, dtype=np.float64)
    g = xe @ np.asarray(w_gate, dtype=np.float64).T
    u = xe @ np.asarray(w_up, dtype=np.float64).T
    hidden = silu(g) * u
    return hidden @ np.asarray(w_down, dtype=np.float64).T, (xe, g, u, hidden)


def expert_backward(saved, dy, w_gate, w_up, w_down):
    """Backward of ``expert_forward`` for the upstream gradient ``dy`` (c_e, d): the closures of
    src/qutai/lm/layers.py:50-70 (linear), :99-105 (silu) and
    src/qutai/core/operations/elementwise.py:40-51 (multiply).  Returns
    ``(d_w_gate, d_w_up, d_w_down, dxe)``."""
    xe, g, u, hidden = saved
    dy = np.asarray(dy, dtype=np.float64)
    wg, wu, wd = (np.asarray(w, dtype=np.float64) for w in (w_gate, w_up, w_down))
    d_hidden = dy @ wd
    d_up = d_hidden * silu(g)
    d_gate = silu_backward(d_hidden * u, g)
    return d_gate.T @ xe, d_up.T @ xe, dy.T @ hidden, d_gate @ wg + d_up @ wu


# --------------------------------------------------------------------------------------
# the layer
# --------------------------------------------------------------------------------------
def moe_forward(x, router, gate, up, down, top_k, scores=None):
    """Forward of the sparse layer; src/qutai/lm/layers.py:376-402 with the expert body of
    src/qutai/lm/layers.py:310-311 (``down(silu(gate(x)) * up(x))``, no biases) and the linear
    maps of src/qutai/lm/layers.py:35-48 (``x @ W.T`` with ``W`` stored (out, in)).

    ``x`` (T, d); ``router`` (E, d); ``gate``/``up`` sequences of (h, d); ``down`` sequence of
    (d, h).  ``scores`` overrides the router product (used to feed identical fp32 logits).
    Returns ``(y, aux, ctx)`` where ``ctx`` keeps what the backward needs.
    """
    x = np.asarray(x, dtype=np.float64)
    router = np.asarray(router, dtype=np.float64)
    if scores is None:
        scores = x @ router.T
    route = routing(scores, top_k)
    saved, outputs = {}, []
    for e in range(route["experts"]):
        if not route["counts"][e]:
            continue
        ye, saved[e] = expert_forward(route_gather(x, route, e), gate[e], up[e], down[e])
        outputs.append((e, ye))
    y = combine(outputs, route["weights"], route)
    ctx = dict(x=x, router=router, gate=gate, up=up, down=down, route=route, saved=saved,
               outputs=outputs, scores=np.asarray(scores, dtype=np.float64))
    return y, route["aux"], ctx


def moe_backward(ctx, grad_y, grad_aux=0.0):
    """Backward of the sparse layer, following the closures registered by the forward:
    combine (src/qutai/lm/layers.py:144-152), the expert body (src/qutai/lm/layers.py:50-70,
    :99-105, src/qutai/core/operations/elementwise.py:40-51), route_gather
    (src/qutai/lm/layers.py:133-141), the two routing closures (src/qutai/lm/layers.py:382-391)
    and the router projection.

    Returns a dict with ``x``, ``router``, ``scores`` and per-expert lists ``gate``, ``up``,
    ``down`` whose entries are ``None`` for experts that received no token (the upstream layer
    never calls such an expert, so its parameters get no gradient object at all).
    """
    route = ctx["route"]
    experts = route["experts"]
    x = ctx["x"]
    grad_y = np.asarray(grad_y, dtype=np.float64).reshape(x.shape)
    dys, dw = combine_backward(grad_y, ctx["outputs"], route["weights"], route)
    dx = np.zeros_like(x)
    grads = dict(gate=[None] * experts, up=[None] * experts, down=[None] * experts)
    for (e, _), dy in zip(ctx["outputs"], dys):
        grads["gate"][e], grads["up"][e], grads["down"][e], dxe = expert_backward(
            ctx["saved"][e], dy, ctx["gate"][e], ctx["up"][e], ctx["down"][e])
        dx += route_gather_backward(dxe, route, e)
    d_scores = routing_backward(dw, route)
    if grad_aux:
        d_scores = d_scores + routing_backward([grad_aux], route, True)
    grads["scores"] = d_scores
    grads["router"] = d_scores.T @ x
    grads["x"] = dx + d_scores @ ctx["router"]
    grads["weights"] = dw
    return grads


# --------------------------------------------------------------------------------------
# the step either side of the layer inside a block: RMS norm before, residual after
# --------------------------------------------------------------------------------------
def rms_norm(x, weight, eps):
    """``out[t, j] = x[t, j] * inverse[t] * weight[j]`` with ``inverse[t] = 1 / sqrt(mean_j x[t, j]^2 + eps)``;
    src/qutai/backends/cpu_lm.py:84-97.  Returns ``(out, inverse)``."""
    x = np.asarray(x, dtype=np.float64)
    weight = np.asarray(weight, dtype=np.float64)
    inverse = 1.0 / np.sqrt((x * x).sum(axis=1) / x.shape[1] + eps)
    return x * inverse[:, None] * weight[None, :], inverse


def rms_norm_backward(gradient, x, weight, inverse):
    """``dx[t, j] = inverse * (g[t, j] w[j] - x[t, j] inverse^2 projected[t])`` with
    ``projected[t] = mean_j g[t, j] w[j] x[t, j]``, and ``dw[j] = sum_t g[t, j] x[t, j] inverse[t]``;
    src/qutai/backends/cpu_lm.py:100-117.  Returns ``(dx, dw)``."""
    g = np.asarray(gradient, dtype=np.float64)
    x = np.asarray(x, dtype=np.float64)
    weight = np.asarray(weight, dtype=np.float64)
    projected = (g * weight[None, :] * x).sum(axis=1) / x.shape[1]
    dx = inverse[:, None] * (g * weight[None, :] - x * (inverse * inverse * projected)[:, None])
    dw = (g * x * inverse[:, None]).sum(axis=0)
    return dx, dw


def block_ffn_forward(x, norm_weight, eps, router, gate, up, down, top_k, scores=None):
    """The feed-forward half of ``Block.__call__`` for a mixture-of-experts block,
    src/qutai/lm/layers.py:430-437: ``(x + ffn(ffn_norm(x)), aux)``.  ``scores`` overrides the router product
    (identical fp32 logits).  Returns ``(out, aux, ctx)``."""
    x = np.asarray(x, dtype=np.float64)
    normed, inverse = rms_norm(x, norm_weight, eps)
    y, aux, ctx = moe_forward(normed, router, gate, up, down, top_k, scores=scores)
    return x + y, aux, dict(moe=ctx, x=x, norm_weight=np.asarray(norm_weight, dtype=np.float64), inverse=inverse)


def block_ffn_backward(ctx, grad_out, grad_aux=0.0):
    """Backward of ``block_ffn_forward``: the layer's gradients (as ``moe_backward`` returns them, ``x`` being
    the gradient of the block's input, residual included) plus ``norm_weight``."""
    grad_out = np.asarray(grad_out, dtype=np.float64).reshape(ctx["x"].shape)
    grads = moe_backward(ctx["moe"], grad_out, grad_aux)
    dx, dw = rms_norm_backward(grads["x"], ctx["x"], ctx["norm_weight"], ctx["inverse"])
    grads["normed"] = grads["x"]
    grads["x"] = grad_out + dx
    grads["norm_weight"] = dw
    return grads


# --------------------------------------------------------------------------------------
# the language-model head and its loss (the caller after the last block)
# --------------------------------------------------------------------------------------
def head_loss_forward(hidden, weight, labels):
    """``projection_loss`` (src/qutai/lm/layers.py:187-257) without its chunking: every position but the last of
    each sequence (``head_rows``, src/qutai/backends/cpu_lm.py:323-331) times ``weight^T``, then per row
    ``log sum exp(z - max) - (z[label] - max)`` for labels other than -100 (``head_loss``, :345-355; the label
    of position t is the token at t + 1, layers.py:193), summed and divided by ``max(1, counted rows)``
    (:198, :213).  ``hidden`` [batch, time, width], ``weight`` [vocab, width], ``labels`` [batch, time] integers.
    Returns ``(loss, ctx)``."""
    hidden = np.asarray(hidden, dtype=np.float64)
    weight = np.asarray(weight, dtype=np.float64)
    labels = np.asarray(labels, dtype=np.int64)
    batch, time, width = hidden.shape
    inputs = hidden[:, :-1, :].reshape(batch * (time - 1), width)
    targets = labels[:, 1:].reshape(-1)
    counted = targets != -100
    count = max(1, int(counted.sum()))
    logits = inputs @ weight.T
    peak = logits.max(axis=1, keepdims=True)
    exps = np.exp(logits - peak)
    total = exps.sum(axis=1, keepdims=True)
    safe = np.where(counted, targets, 0)
    picked = logits[np.arange(len(targets)), safe] - peak[:, 0]
    row_loss = np.where(counted, np.log(total[:, 0]) - picked, 0.0)
    loss = row_loss.sum() / count
    ctx = dict(inputs=inputs, weight=weight, shape=hidden.shape, probabilities=exps / total, targets=safe, counted=counted,
               count=count, logits=logits)
    return loss, ctx


def head_loss_backward(ctx, gradient=1.0):
    """Backward closure of ``projection_loss`` (src/qutai/lm/layers.py:215-255): per row
    ``gradient / count * (softmax - one_hot)``, zero for rows that are not counted (``head_gradient``,
    src/qutai/backends/cpu_lm.py:358-371); ``dx`` rows = that times ``weight`` put back at their positions, the last
    position of each sequence getting nothing (``head_rows_backward``, :334-338); ``dw`` = its transpose times the
    gathered rows.  Returns ``(d_hidden [batch, time, width], d_weight [vocab, width], d_logits)``."""
    batch, time, width = ctx["shape"]
    g = ctx["probabilities"].copy()
    g[np.arange(g.shape[0]), ctx["targets"]] -= 1.0
    g *= float(gradient) / ctx["count"]
    g[~ctx["counted"]] = 0.0
    d_hidden = np.zeros((batch, time, width))
    d_hidden[:, :-1, :] = (g @ ctx["weight"]).reshape(batch, time - 1, width)
    return d_hidden, g.T @ ctx["inputs"], g


# --------------------------------------------------------------------------------------
# rotary position embedding, token embedding
# --------------------------------------------------------------------------------------
def rope(values, heads, theta, offset=0, inverse=False):
    """``rope`` of the CPU backend, src/qutai/backends/cpu_lm.py:125-138: in every head of ``values``
    [batch, time, heads * dim] the pair ``(2 i, 2 i + 1)`` is turned by ``(offset + t) theta ** (-2 i / dim)``
    (the other way round with ``inverse``, which is the backward)."""
    values = np.asarray(values, dtype=np.float64)
    batch, time, features = values.shape
    dim = features // heads
    x = values.reshape(batch, time, heads, dim // 2, 2)
    angle = (offset + np.arange(time))[:, None] * theta ** (-np.arange(0, dim, 2) / dim)[None, :]
    if inverse:
        angle = -angle
    c, s = np.cos(angle)[None, :, None, :], np.sin(angle)[None, :, None, :]
    out = np.stack([x[..., 0] * c - x[..., 1] * s, x[..., 0] * s + x[..., 1] * c], axis=-1)
    return out.reshape(batch, time, features)


def embedding(weight, ids):
    """Rows ``ids`` of ``weight`` (src/qutai/backends/cpu_lm.py:54-58)."""
    return np.asarray(weight, dtype=np.float64)[np.asarray(ids, dtype=np.int64)]


def embedding_backward(gradient, ids, count):
    """Row ``token`` = the sum of the gradient rows of the positions that held it
    (src/qutai/backends/cpu_lm.py:61-66)."""
    gradient = np.asarray(gradient, dtype=np.float64)
    result = np.zeros((count, gradient.shape[-1]))
    np.add.at(result, np.asarray(ids, dtype=np.int64), gradient.reshape(-1, gradient.shape[-1]))
    return result


# --------------------------------------------------------------------------------------
# causal self-attention with grouped key/value heads
# --------------------------------------------------------------------------------------
def attention_forward(q, k, v, heads, kv_heads):
    """``attention`` of the CPU backend, src/qutai/backends/cpu_lm.py:141-173: per sequence, query position t and
    head h, scores ``q . k[s] / sqrt(dim)`` over the key positions ``s <= t`` of key/value head
    ``h // (heads // kv_heads)``, a softmax over them, and the weighted sum of the values; ``lse`` is
    ``max + log(sum exp(score - max))`` of each row.  ``q`` [batch, time, heads * dim], ``k``, ``v``
    [batch, time, kv_heads * dim].  Returns ``(out [batch, time, heads * dim], lse [batch, time, heads])``."""
    q, k, v = (np.asarray(a, dtype=np.float64) for a in (q, k, v))
    batch, time, features = q.shape
    dim = features // heads
    group = heads // kv_heads
    qh = q.reshape(batch, time, heads, dim)
    kh = k.reshape(batch, time, kv_heads, dim)[:, :, np.arange(heads) // group, :]
    vh = v.reshape(batch, time, kv_heads, dim)[:, :, np.arange(heads) // group, :]
    scores = np.einsum("bthd,bshd->bhts", qh, kh) / np.sqrt(dim)
    mask = np.tril(np.ones((time, time), dtype=bool))
    scores = np.where(mask, scores, -np.inf)
    peak = scores.max(axis=-1, keepdims=True)
    weights = np.exp(scores - peak)
    total = weights.sum(axis=-1, keepdims=True)
    out = np.einsum("bhts,bshd->bthd", weights / total, vh).reshape(batch, time, features)
    lse = (peak + np.log(total))[..., 0].transpose(0, 2, 1)
    return out, lse


def attention_backward(gradient, q, k, v, out, lse, heads, kv_heads):
    """``attention_backward``, src/qutai/backends/cpu_lm.py:176-201: with ``p = exp(score - lse)``,
    ``delta = <gradient, out>`` per row and ``ds = p (gradient . v[s] - delta) / sqrt(dim)``:
    ``dq += ds k[s]``, ``dk[s] += ds q``, ``dv[s] += p gradient`` (the key/value gradients summed over the query heads
    of a group).  Returns ``(dq, dk, dv)`` in the shapes of ``q, k, v``."""
    gradient, q, k, v, out, lse = (np.asarray(a, dtype=np.float64) for a in (gradient, q, k, v, out, lse))
    batch, time, features = q.shape
    dim = features // heads
    group = heads // kv_heads
    head_of = np.arange(heads) // group
    qh, gh, oh = (a.reshape(batch, time, heads, dim) for a in (q, gradient, out))
    kh = k.reshape(batch, time, kv_heads, dim)[:, :, head_of, :]
    vh = v.reshape(batch, time, kv_heads, dim)[:, :, head_of, :]
    scale = 1.0 / np.sqrt(dim)
    scores = np.einsum("bthd,bshd->bhts", qh, kh) * scale
    mask = np.tril(np.ones((time, time), dtype=bool))
    p = np.where(mask, np.exp(scores - lse.transpose(0, 2, 1)[..., None]), 0.0)
    delta = np.einsum("bthd,bthd->bht", gh, oh)
    dp = np.einsum("bthd,bshd->bhts", gh, vh)
    ds = p * (dp - delta[..., None]) * scale
    dq = np.einsum("bhts,bshd->bthd", ds, kh).reshape(batch, time, features)
    dk_heads = np.einsum("bhts,bthd->bshd", ds, qh)
    dv_heads = np.einsum("bhts,bthd->bshd", p, gh)
    dk = dk_heads.reshape(batch, time, kv_heads, group, dim).sum(axis=3).reshape(batch, time, kv_heads * dim)
    dv = dv_heads.reshape(batch, time, kv_heads, group, dim).sum(axis=3).reshape(batch, time, kv_heads * dim)
    return dq, dk, dv


# --------------------------------------------------------------------------------------
# helpers used by tests and by the benchmark's CPU leg
# --------------------------------------------------------------------------------------
def round_bf16(a):
    """Round float values to the nearest bfloat16 (ties to even), returned as float64."""
    a32 = np.ascontiguousarray(np.asarray(a, dtype=np.float32))
    bits = a32.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return rounded.view(np.float32).astype(np.float64).reshape(a32.shape)


def elementwise_err(actual, expected, bf16=False, unit=1.0):
    """Element-wise error in the form of the upstream GPU-against-CPU checks: ``max |a - b| / (unit + |b|)``
    (``|x - y| <= tol * (1 + |y|)``, tests/test_lm_moe.py:105-138) or, with ``bf16``,
    ``max |a - b| / max(unit, |b|)`` (``tol * max(1, |y|)``, tests/test_lm_bfloat16.py:129-167).  Upstream's
    test data are of order one, hence its ``1``; ``unit`` is that scale (pass the tensor's root mean square for
    data of another magnitude).  Unlike ``max_rel_err`` an entry cannot hide behind the largest one of its tensor."""
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    if not expected.size:
        return 0.0
    scale = np.maximum(unit, np.abs(expected)) if bf16 else unit + np.abs(expected)
    return float((np.abs(actual - expected) / scale).max())


def rms(values):
    values = np.asarray(values, dtype=np.float64)
    return float(np.sqrt(np.mean(values * values))) if values.size else 0.0


def rowwise_rel_err(actual, expected):
    """``max over rows of (max |a - b| over the row / max |b| over the row)`` for 2-D arrays: every row (an
    expert's router gradient, a token's output) is held to the relative bar on its own scale."""
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    if not expected.size:
        return 0.0
    scale = np.abs(expected).max(axis=1)
    error = np.abs(actual - expected).max(axis=1)
    return float((error[scale > 0] / scale[scale > 0]).max()) if np.any(scale > 0) else float(error.max())


def max_rel_err(actual, expected):
    """``max |a - b| / max |b|`` — the layer-level relative error used for the parity bars."""
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    scale = float(np.abs(expected).max()) if expected.size else 0.0
    if scale == 0.0:
        return float(np.abs(actual).max()) if actual.size else 0.0
    return float(np.abs(actual - expected).max() / scale)
