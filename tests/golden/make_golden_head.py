"""Golden vectors for the language-model head and its cross-entropy loss, produced by the UPSTREAM package itself on
``device="cpu"``, ``dtype="float64"``: its ``projection_loss`` (src/qutai/lm/layers.py:187-257) with a chunk size that
does not divide the rows, under its own autograd, with an incoming gradient other than 1.

Run in a container that has a checkout of the upstream sources (``python tests/golden/make_golden_head.py``); the
fixtures ``head_*.npz`` are committed, this script documents how they were made.
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
from qutai.lm.layers import projection_loss  # noqa: E402


def _store(a):
    return cpu.storage(np.asarray(a, dtype=np.float64).reshape(-1).tolist(), dtype="float64")


def _arr(storage, shape):
    return np.array(storage.tolist(), dtype=np.float64).reshape(shape)


def head_case(name, batch, time, width, vocab, seed, chunk, ignored=0.2, gradient=1.0, scale=1.0):
    rng = np.random.default_rng(seed)
    f32 = lambda a: np.asarray(a, dtype=np.float32).astype(np.float64)   # exactly representable on a float32 device
    hidden = f32(rng.standard_normal((batch, time, width)) * scale)
    weight = f32(rng.standard_normal((vocab, width)) * 0.5)
    labels = rng.integers(0, vocab, size=(batch, time))
    labels[rng.random((batch, time)) < ignored] = -100
    leaf = lambda a: Tensor(_store(a), shape=tuple(a.shape), requires_grad=True)
    h, w = leaf(hidden), leaf(weight)
    loss = projection_loss(h, w, [list(map(int, row)) for row in labels], chunk)
    loss.backward(Tensor(_store([gradient]), shape=()))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), kind="head", hidden=hidden.astype(np.float32),
                        weight=weight.astype(np.float32), labels=labels.astype(np.int64), gradient=gradient,
                        loss=_arr(loss.storage, ())[()], d_hidden=_arr(h.grad.storage, hidden.shape),
                        d_weight=_arr(w.grad.storage, weight.shape))
    print(name, "loss", _arr(loss.storage, ())[()], "counted", int((labels[:, 1:] != -100).sum()))


if __name__ == "__main__":
    head_case("head_small", 2, 5, 8, 11, 31, chunk=3)
    head_case("head_mid", 3, 17, 24, 40, 32, chunk=7, gradient=0.37)
    head_case("head_all_ignored", 2, 4, 8, 16, 33, chunk=4, ignored=1.1)
    head_case("head_wide", 2, 17, 64, 136, 34, chunk=20, ignored=0.0, gradient=-1.5, scale=2.0)
