"""The optimizer oracle against the fixtures the upstream package produced (CPU only)."""
import os

import numpy as np

from conftest import ROOT
from oracle import optim_oracle

GOLDEN = os.path.join(ROOT, "tests", "golden")


def test_adamw_oracle_reproduces_the_upstream_steps():
    f = np.load(os.path.join(GOLDEN, "optim_adamw.npz"))
    n, steps = int(f["tensors"]), int(f["steps"])
    optimizer = optim_oracle.AdamW(learning_rate=float(f["learning_rate"]), betas=(float(f["beta1"]), float(f["beta2"])),
                                   eps=float(f["eps"]), weight_decay=float(f["weight_decay"]))
    values = [f[f"initial_{i}"] for i in range(n)]
    for step in range(steps):
        gradients = [f[f"grad_{step}_{i}"] if bool(f[f"has_grad_{step}_{i}"]) else None for i in range(n)]
        values = optimizer.step(values, gradients)
        for i in range(n):
            assert np.allclose(values[i], f[f"values_{step}_{i}"], rtol=1e-13, atol=0)
            assert optimizer.steps.get(i, 0) == int(f[f"count_{step}_{i}"])
            if f"average_{step}_{i}" in f:
                assert np.allclose(optimizer.averages[i], f[f"average_{step}_{i}"], rtol=1e-13, atol=0)
                assert np.allclose(optimizer.square_averages[i], f[f"square_{step}_{i}"], rtol=1e-13, atol=0)
            else:
                assert i not in optimizer.averages
    assert [optimizer.steps.get(i, 0) for i in range(n)] == [3, 3, 2, 0]   # skipped steps do not count


def test_clip_oracle_reproduces_the_upstream_norm_and_scaling():
    f = np.load(os.path.join(GOLDEN, "optim_clip.npz"))
    n = int(f["tensors"])
    for name in ("above", "below"):
        gradients = [f[f"grad_{i}"] if bool(f[f"{name}_has_{i}"]) else None for i in range(n)]
        norm, after = optim_oracle.clip_grad_norm(gradients, float(f[f"{name}_limit"]))
        assert abs(norm - float(f[f"{name}_norm"])) <= 1e-13 * norm
        for i in range(n):
            if after[i] is None:
                assert not bool(f[f"{name}_has_{i}"])
            else:
                assert np.allclose(after[i], f[f"{name}_after_{i}"], rtol=1e-13, atol=0)
    assert float(f["above_norm"]) > float(f["above_limit"]) and float(f["below_norm"]) < float(f["below_limit"])
