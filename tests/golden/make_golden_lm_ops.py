"""Golden vectors for the small operations around attention and the feed-forward half of a decoder block, produced by
the UPSTREAM package itself: ``rms_norm`` / ``rms_norm_backward``, ``rope`` and ``embedding`` /
``embedding_backward`` of its pure-Python CPU backend (src/qutai/backends/cpu_lm.py:54-138) in float64.

Run in a container that has a checkout of the upstream sources (``python tests/golden/make_golden_lm_ops.py``); the
fixture ``lm_ops.npz`` is committed, this script documents how it was made.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import ref_loader  # noqa: E402

ref_loader.load()
from qutai.backends import cpu, cpu_lm  # noqa: E402


def _store(a, dtype="float64"):
    return cpu.storage(np.asarray(a).reshape(-1).tolist(), dtype=dtype)


def _arr(storage, shape):
    return np.array(storage.tolist(), dtype=np.float64).reshape(shape)


if __name__ == "__main__":
    rng = np.random.default_rng(51)
    f32 = lambda a: np.asarray(a, dtype=np.float32).astype(np.float64)
    data = {}
    # RMS norm: 13 rows of width 40 (not a power of two), eps 1e-5
    rows, width, eps = 13, 40, 1e-5
    x, w, g = f32(rng.standard_normal((rows, width)) * 1.3 + 0.1), f32(1 + 0.2 * rng.standard_normal(width)), f32(rng.standard_normal((rows, width)))
    out, inverse = cpu_lm.rms_norm(_store(x), _store(w), width, eps)
    dx, dw = cpu_lm.rms_norm_backward(_store(g), _store(x), _store(w), inverse, width)
    data.update(norm_x=x, norm_w=w, norm_g=g, norm_eps=eps, norm_out=_arr(out, x.shape), norm_inverse=_arr(inverse, (rows,)),
                norm_dx=_arr(dx, x.shape), norm_dw=_arr(dw, (width,)))
    # rotary embedding: batch 2, time 7, 3 heads of width 8, theta 10000, offset 5; and its inverse
    batch, time, heads, dim, theta, offset = 2, 7, 3, 8, 10000.0, 5
    v = f32(rng.standard_normal((batch, time, heads * dim)))
    turned = cpu_lm.rope(_store(v), batch, time, heads, dim, theta, offset)
    back = cpu_lm.rope(_store(v), batch, time, heads, dim, theta, offset, inverse=True)
    data.update(rope_v=v, rope_heads=heads, rope_theta=theta, rope_offset=offset, rope_out=_arr(turned, v.shape), rope_inverse=_arr(back, v.shape))
    # embedding: vocabulary 11, width 6, 9 positions with repeats
    vocab, width = 11, 6
    table = f32(rng.standard_normal((vocab, width)))
    ids = [3, 7, 3, 0, 10, 7, 3, 5, 0]
    grad = f32(rng.standard_normal((len(ids), width)))
    rows_out = cpu_lm.embedding(_store(table), ids, width)
    d_table = cpu_lm.embedding_backward(_store(grad), ids, vocab, width)
    data.update(emb_table=table, emb_ids=np.array(ids), emb_grad=grad, emb_out=_arr(rows_out, (len(ids), width)), emb_d_table=_arr(d_table, (vocab, width)))
    np.savez_compressed(os.path.join(HERE, "lm_ops.npz"), kind="lm_ops", **data)
    print("written", len(data), "arrays")
