"""Golden vectors for the feed-forward half of a mixture-of-experts block — RMS norm, the MoE layer and the
residual add, ``x + ffn(ffn_norm(x))`` (src/qutai/lm/layers.py:430-437) — produced by the UPSTREAM package itself
on ``device="cpu"``, ``dtype="float64"``: its ``RMSNorm``, ``SparseMoE`` and ``residual_add`` under its own autograd.

Run in a container that has a checkout of the upstream sources (``python tests/golden/make_golden_block.py``);
the fixtures ``block_*.npz`` are committed, this script documents how they were made.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import ref_loader  # noqa: E402

ref_loader.load()
from qutai.backends import cpu  # noqa: E402
from qutai.core.tensor import Tensor  # noqa: E402
from qutai.lm.config import Config  # noqa: E402
from qutai.lm.layers import RMSNorm, SparseMoE, residual_add  # noqa: E402


def _store(a):
    return cpu.storage(np.asarray(a, dtype=np.float64).reshape(-1).tolist(), dtype="float64")


def _arr(storage, shape=None):
    out = np.array(storage.tolist(), dtype=np.float64)
    return out if shape is None else out.reshape(shape)


def block_case(name, rows, width, experts, top_k, hidden, seed, eps=1e-6, std=0.3, sample=1):
    rng = np.random.default_rng(seed)
    f32 = lambda a: np.asarray(a, dtype=np.float32).astype(np.float64)   # exactly representable on a float32 device
    x = f32(rng.standard_normal((rows, width)) * 1.7 + 0.2)
    norm_weight = f32(1.0 + 0.3 * rng.standard_normal(width))
    router = f32(rng.standard_normal((experts, width)) * std)
    gate = [f32(rng.standard_normal((hidden, width)) * std) for _ in range(experts)]
    up = [f32(rng.standard_normal((hidden, width)) * std) for _ in range(experts)]
    down = [f32(rng.standard_normal((width, hidden)) * std) for _ in range(experts)]
    grad_out, grad_aux = f32(rng.standard_normal((rows, width))), 0.37
    cfg = Config(d_model=width, n_heads=2, n_kv_heads=1, ffn_type="moe", n_experts=experts, top_k=top_k,
                 d_expert=hidden, n_layers=1, norm_eps=eps)
    norm = RMSNorm(width, eps, device="cpu", dtype="float64")
    layer = SparseMoE(cfg, device="cpu", dtype="float64", seed=0)
    leaf = lambda a: Tensor(_store(a), shape=tuple(a.shape), requires_grad=True)
    norm.weight = leaf(norm_weight)
    layer.router.weight = leaf(router)
    for e, expert in enumerate(layer.experts):
        expert.gate.weight, expert.up.weight, expert.down.weight = leaf(gate[e]), leaf(up[e]), leaf(down[e])
    xt = leaf(x)
    y, aux = layer(norm(xt))
    out = residual_add(xt, y)                                    # Block.__call__, src/qutai/lm/layers.py:436-437
    out.backward(Tensor(_store(grad_out), shape=tuple(grad_out.shape)))
    aux.backward(Tensor(_store([grad_aux]), shape=()))
    grad = lambda t: None if t.grad is None else _arr(t.grad.storage, t.shape)
    data = dict(kind="block", x=x.astype(np.float32), norm_weight=norm_weight.astype(np.float32), eps=eps,
                router=router.astype(np.float32), gate=np.stack(gate).astype(np.float32), up=np.stack(up).astype(np.float32),
                down=np.stack(down).astype(np.float32), top_k=top_k, grad_out=grad_out.astype(np.float32), grad_aux=grad_aux,
                sample=sample, out=_arr(out.storage, (rows, width)), aux=_arr(aux.storage)[0],
                counts=np.array(layer.last_counts, dtype=np.int64), dx=grad(xt), d_norm_weight=grad(norm.weight),
                d_router=grad(layer.router.weight))
    has = []
    for e, expert in enumerate(layer.experts):
        for key, p in (("gate", expert.gate.weight), ("up", expert.up.weight), ("down", expert.down.weight)):
            g = grad(p)
            if key == "gate":
                has.append(g is not None)
            data[f"d_{key}_{e}"] = np.zeros((0,)) if g is None else g.reshape(-1)[::sample]
    data["has_grad"] = np.array(has)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **data)
    print(name, "counts", layer.last_counts, "aux", data["aux"])


if __name__ == "__main__":
    block_case("block_small", 6, 8, 3, 2, 8, 21)
    block_case("block_mid", 41, 24, 4, 2, 32, 22)
    block_case("block_k1_wide", 19, 72, 5, 1, 40, 23, eps=1e-5, sample=3)
