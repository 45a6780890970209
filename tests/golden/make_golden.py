"""Generate the golden fixtures ``tests/golden/*.npz`` from the upstream package itself.

Run where a checkout of the upstream sources is mounted (``QUTAI_REFERENCE_SRC`` or the default
location used by ``oracle/ref_loader.py``):

    python tests/golden/make_golden.py

Every fixture holds the INPUTS (numpy ``default_rng`` draws, stored so the fixture does not depend
on a generator's stream) and the OUTPUTS of the upstream CPU float64 path: ``cpu_lm.routing`` for
the routing cases, and ``SparseMoE`` forward + backward on ``device="cpu"``,
``dtype="float64"`` for the layer cases (src/qutai/lm/layers.py:354-408,
src/qutai/backends/cpu_lm.py:204-320).  The fixtures travel with the repository; the upstream
sources do not, so nothing but this script reads them.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import ref_loader  # noqa: E402

ref_loader.load()
from qutai.backends import cpu, cpu_lm  # noqa: E402
from qutai.core.tensor import Tensor  # noqa: E402
from qutai.lm.config import Config  # noqa: E402
from qutai.lm.layers import SparseMoE  # noqa: E402


def _store(a):
    return cpu.storage([float(v) for v in np.asarray(a, dtype=np.float64).reshape(-1)], dtype="float64")


def _arr(storage, shape=None):
    a = np.array(storage.tolist() if hasattr(storage, "tolist") else list(storage), dtype=np.float64)
    return a if shape is None else a.reshape(shape)


def _ragged(lists):
    """Concatenate per-expert lists; the split points are the cumulative counts."""
    return np.array([v for part in lists for v in part], dtype=np.int64)


def routing_case(name, scores, top_k):
    scores = np.asarray(scores, dtype=np.float64)
    rows, experts = scores.shape
    route = cpu_lm.routing(_store(scores), rows, experts, top_k)
    g = np.random.default_rng(1234).standard_normal((rows, top_k))
    d_gate = cpu_lm.routing_backward(_store(g), route)
    d_aux = cpu_lm.routing_backward(_store([0.37]), route, True)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        kind="routing", scores=scores, top_k=top_k,
        probs=_arr(route["probs"], (rows, experts)),
        weights=_arr(route["weights"], (rows, top_k)),
        indices=np.array(route["indices"].tolist(), dtype=np.int64).reshape(rows, top_k),
        counts=np.array(route["counts"], dtype=np.int64),
        ids=_ragged(route["ids"]), slots=_ragged(route["slots"]),
        utilization=_arr(route["utilization"]), aux=_arr(route["aux"])[0],
        grad_weights=g, d_scores_gate=_arr(d_gate, (rows, experts)),
        grad_aux=0.37, d_scores_aux=_arr(d_aux, (rows, experts)))
    print(name, "counts", route["counts"])


def layer_case(name, x, router, gate, up, down, top_k, grad_y, grad_aux, sample=1):
    rows, width = x.shape
    experts, hidden = len(gate), gate[0].shape[0]
    cfg = Config(d_model=width, n_heads=2, n_kv_heads=1, ffn_type="moe", n_experts=experts,
                 top_k=top_k, d_expert=hidden, n_layers=1)
    layer = SparseMoE(cfg, device="cpu", dtype="float64", seed=0)

    def leaf(a):
        return Tensor(_store(a), shape=tuple(a.shape), requires_grad=True)

    layer.router.weight = leaf(router)
    for e, expert in enumerate(layer.experts):
        expert.gate.weight, expert.up.weight, expert.down.weight = leaf(gate[e]), leaf(up[e]), leaf(down[e])
    xt = leaf(x)
    y, aux = layer(xt)
    y.backward(Tensor(_store(grad_y), shape=tuple(grad_y.shape)))
    aux.backward(Tensor(_store([grad_aux]), shape=()))

    def grad(t):
        return None if t.grad is None else _arr(t.grad.storage, t.shape)

    empty = np.zeros((0,))
    out = dict(
        kind="layer", x=x.astype(np.float32), router=router.astype(np.float32),
        gate=np.stack(gate).astype(np.float32), up=np.stack(up).astype(np.float32),
        down=np.stack(down).astype(np.float32), top_k=top_k, grad_y=grad_y.astype(np.float32), grad_aux=grad_aux, sample=sample,
        y=_arr(y.storage, (rows, width)), aux=_arr(aux.storage)[0],
        counts=np.array(layer.last_counts, dtype=np.int64),
        utilization=_arr(layer.utilization.storage),
        dx=grad(xt), d_router=grad(layer.router.weight))
    has = []
    for e, expert in enumerate(layer.experts):
        for key, p in (("gate", expert.gate.weight), ("up", expert.up.weight), ("down", expert.down.weight)):
            g = grad(p)
            if key == "gate":
                has.append(g is not None)
            out[f"d_{key}_{e}"] = empty if g is None else g.reshape(-1)[::sample]
    out["has_grad"] = np.array(has)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, "counts", layer.last_counts, "aux", out["aux"])


def random_layer(name, rows, width, experts, top_k, hidden, seed, *, std=0.3, tweak=None, sample=1):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, width))
    router = rng.standard_normal((experts, width)) * std
    gate = [rng.standard_normal((hidden, width)) * std for _ in range(experts)]
    up = [rng.standard_normal((hidden, width)) * std for _ in range(experts)]
    down = [rng.standard_normal((width, hidden)) * std for _ in range(experts)]
    if tweak:
        x, router = tweak(x, router)
    grad_y = rng.standard_normal((rows, width))
    # inputs are made exactly representable in float32 so a float32 device run sees the same values
    f32 = lambda a: np.asarray(a, dtype=np.float32).astype(np.float64)
    x, router, grad_y = f32(x), f32(router), f32(grad_y)
    gate, up, down = [f32(a) for a in gate], [f32(a) for a in up], [f32(a) for a in down]
    layer_case(name, x, router, gate, up, down, top_k, grad_y, 0.37, sample=sample)


def main():
    # known answers of the upstream tests (tests/test_lm_moe.py:65-71, tests/test_lm_bfloat16.py:130)
    routing_case("routing_known_2x3", [[3.0, 2.0, -1.0], [-1.0, 2.0, 3.0]], 2)
    routing_case("routing_bf16_test_5x3",
                 [[3, 1, -2], [0, 2, 1], [1, -2, 4], [-1, 3, 2], [4, 0, 1]], 2)
    # stable (token, slot) order across blocks (tests/test_lm_moe.py:140-162); the values are
    # rounded to float32 first, as the device path receives them
    rows, experts = 517, 5
    scores = np.array([[((r * 37 + e * 11) % 101) / 13 for e in range(experts)] for r in range(rows)])
    routing_case("routing_pack_517x5", scores.astype(np.float32).astype(np.float64), 3)
    # exact ties: quantised logits, many equal values per row -> lowest expert index first
    rng = np.random.default_rng(7)
    routing_case("routing_ties_64x16", rng.integers(-2, 3, size=(64, 16)).astype(np.float64), 4)
    routing_case("routing_all_equal_9x6", np.zeros((9, 6)), 3)
    routing_case("routing_wide_33x64", np.random.default_rng(8).standard_normal((33, 64)).astype(np.float32).astype(np.float64), 6)
    routing_case("routing_k1_40x7", np.random.default_rng(9).standard_normal((40, 7)).astype(np.float32).astype(np.float64), 1)

    random_layer("layer_small", 5, 8, 3, 2, 6, 11)
    random_layer("layer_mid", 37, 16, 4, 2, 24, 12)
    random_layer("layer_k_eq_e", 9, 8, 3, 3, 8, 13)

    def empty_expert(x, router):
        x = np.abs(x)
        router = router * 0.05
        router[2] = -1.0
        return x, router

    random_layer("layer_empty_expert", 11, 8, 4, 1, 8, 14, tweak=empty_expert)

    def tied_rows(x, router):
        router[3] = router[1]
        return x, router

    random_layer("layer_tied_router_rows", 8, 8, 4, 2, 8, 15, tweak=tied_rows)
    # the layer shape of the CPU-runnable configuration (4 experts, top-2, d 64, hidden 128,
    # 128 tokens, weights N(0, 0.02)); expert gradients stored as every 7th element
    random_layer("layer_c1_shape", 128, 64, 4, 2, 128, 16, std=0.02, sample=7)


if __name__ == "__main__":
    main()
