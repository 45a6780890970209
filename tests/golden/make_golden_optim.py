"""Generate ``tests/golden/optim_*.npz`` from the upstream package itself (run where its sources are
mounted, like ``make_golden.py``):

    python tests/golden/make_golden_optim.py

``optim_adamw``: four parameter tensors, three ``AdamW.step()`` calls on ``device="cpu"``,
``dtype="float64"`` (src/qutai/nn/optimizers.py:121-153); the third tensor has no gradient in step 2 and the
fourth never has one, so the per-parameter step counters differ.  ``optim_clip``: ``clip_grad_norm``
(src/qutai/nn/optimizers.py:19-31) once above and once below the limit.  Inputs are stored with the outputs.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import ref_loader  # noqa: E402

ref_loader.load()
from qutai.backends import cpu  # noqa: E402
from qutai.core.tensor import Tensor  # noqa: E402
from qutai.nn.optimizers import AdamW, clip_grad_norm  # noqa: E402


def _store(a):
    return cpu.storage([float(v) for v in np.asarray(a, dtype=np.float64).reshape(-1)], dtype="float64")


def _arr(storage):
    return np.array(storage.tolist(), dtype=np.float64)


def _leaf(a):
    return Tensor(_store(a), shape=tuple(np.shape(a)), requires_grad=True)


def adamw_case():
    rng = np.random.default_rng(2024)
    shapes = [(7, 5), (33,), (4, 9), (6,)]
    initial = [rng.standard_normal(s) * 0.3 for s in shapes]
    settings = dict(learning_rate=0.01, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    parameters = [_leaf(a) for a in initial]
    optimizer = AdamW(parameters, **settings)
    out = dict(kind="adamw", learning_rate=settings["learning_rate"], beta1=settings["betas"][0], beta2=settings["betas"][1],
               eps=settings["eps"], weight_decay=settings["weight_decay"], tensors=len(shapes), steps=3)
    for i, a in enumerate(initial):
        out[f"initial_{i}"] = a
    for step in range(3):
        for i, parameter in enumerate(parameters):
            has = not (i == 3 or (i == 2 and step == 1))
            gradient = rng.standard_normal(shapes[i]) * (10.0 ** (step - 1))
            out[f"has_grad_{step}_{i}"] = has
            out[f"grad_{step}_{i}"] = gradient
            parameter.grad = Tensor(_store(gradient), shape=shapes[i]) if has else None
        optimizer.step()
        for i, parameter in enumerate(parameters):
            out[f"values_{step}_{i}"] = _arr(parameter.storage).reshape(shapes[i])
            out[f"count_{step}_{i}"] = optimizer.steps.get(parameter, 0)
            if parameter in optimizer.averages:
                out[f"average_{step}_{i}"] = _arr(optimizer.averages[parameter]).reshape(shapes[i])
                out[f"square_{step}_{i}"] = _arr(optimizer.square_averages[parameter]).reshape(shapes[i])
    np.savez_compressed(os.path.join(HERE, "optim_adamw.npz"), **out)
    print("optim_adamw", [out[f"count_2_{i}"] for i in range(4)])


def clip_case():
    rng = np.random.default_rng(77)
    shapes = [(5, 3), (17,), (2, 2)]
    gradients = [rng.standard_normal(s) for s in shapes]
    out = dict(kind="clip", tensors=len(shapes))
    for name, limit in (("above", 1.5), ("below", 100.0)):
        parameters = [_leaf(np.zeros(s)) for s in shapes]
        for i, parameter in enumerate(parameters):
            parameter.grad = None if i == 2 and name == "below" else Tensor(_store(gradients[i]), shape=shapes[i])
        norm = clip_grad_norm(parameters, limit)
        out[f"{name}_limit"], out[f"{name}_norm"] = limit, norm
        for i, parameter in enumerate(parameters):
            out[f"{name}_has_{i}"] = parameter.grad is not None
            if parameter.grad is not None:
                out[f"{name}_after_{i}"] = _arr(parameter.grad.storage).reshape(shapes[i])
    for i, g in enumerate(gradients):
        out[f"grad_{i}"] = g
    np.savez_compressed(os.path.join(HERE, "optim_clip.npz"), **out)
    print("optim_clip", out["above_norm"], out["below_norm"])


if __name__ == "__main__":
    adamw_case()
    clip_case()
