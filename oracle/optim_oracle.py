"""CPU restatement (numpy float64) of the upstream optimizer step either side of the MoE layer.

Test infrastructure only: imported by ``tests/`` as the checker, never by the product.

* ``adamw_step``      src/qutai/backends/cpu.py:557-566 (the arithmetic),
* ``AdamW``           src/qutai/nn/optimizers.py:121-153 (per-parameter step counters, zero-initialised moments,
                      parameters whose ``grad`` is ``None`` are skipped and keep their counter),
* ``global_norm``     src/qutai/backends/cpu.py:534-536,
* ``clip_grad_norm``  src/qutai/nn/optimizers.py:19-31 (scale by ``max_norm / norm`` only when ``norm > max_norm``;
                      returns the norm before clipping).

Pinned by ``tests/golden/optim_*.npz``, which the upstream package itself produced
(``tests/golden/make_golden_optim.py``).
"""
from __future__ import annotations

import numpy as np


def adamw_step(values, gradient, average, square_average, *, step, learning_rate, betas, eps, weight_decay):
    beta1, beta2 = betas
    values, gradient = np.asarray(values, dtype=np.float64), np.asarray(gradient, dtype=np.float64)
    average = beta1 * np.asarray(average, dtype=np.float64) + (1 - beta1) * gradient
    square_average = beta2 * np.asarray(square_average, dtype=np.float64) + (1 - beta2) * gradient * gradient
    correction1, correction2 = 1 - beta1 ** step, 1 - beta2 ** step
    decay = 1 - learning_rate * weight_decay
    result = values * decay - learning_rate * (average / correction1) / (np.sqrt(square_average / correction2) + eps)
    return result, average, square_average


class AdamW:
    """State per parameter index: ``steps[i]``, ``averages[i]``, ``square_averages[i]`` (absent until the
    parameter first has a gradient)."""

    def __init__(self, *, learning_rate=0.001, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01):
        self.learning_rate, self.betas, self.eps, self.weight_decay = learning_rate, tuple(betas), eps, weight_decay
        self.steps, self.averages, self.square_averages = {}, {}, {}

    def step(self, values, gradients):
        """``values``: list of arrays (replaced in the returned list); ``gradients``: list of arrays or ``None``."""
        out = []
        for index, (value, gradient) in enumerate(zip(values, gradients)):
            if gradient is None:
                out.append(np.asarray(value, dtype=np.float64))
                continue
            step = self.steps.get(index, 0) + 1
            zeros = np.zeros(np.shape(value))
            new, average, square = adamw_step(value, gradient, self.averages.get(index, zeros),
                                              self.square_averages.get(index, zeros), step=step,
                                              learning_rate=self.learning_rate, betas=self.betas, eps=self.eps,
                                              weight_decay=self.weight_decay)
            self.steps[index], self.averages[index], self.square_averages[index] = step, average, square
            out.append(new)
        return out


def global_norm(gradients):
    total = 0.0
    for gradient in gradients:
        g = np.asarray(gradient, dtype=np.float64)
        total += float(np.sum(g * g))
    return float(np.sqrt(total))


def clip_grad_norm(gradients, max_norm=1.0):
    """Returns ``(norm before clipping, gradients after clipping)``; ``None`` entries are passed through."""
    present = [g for g in gradients if g is not None]
    norm = global_norm(present)
    if norm > max_norm:
        scale = max_norm / norm
        gradients = [None if g is None else np.asarray(g, dtype=np.float64) * scale for g in gradients]
    return norm, gradients
