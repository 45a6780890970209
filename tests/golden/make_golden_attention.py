"""Golden vectors for causal self-attention with grouped key/value heads, produced by the UPSTREAM package itself:
``attention`` and ``attention_backward`` of its pure-Python CPU backend (src/qutai/backends/cpu_lm.py:141-201) in
float64, head width 64 (the width of its tensor-core kernels).

Run in a container that has a checkout of the upstream sources (``python tests/golden/make_golden_attention.py``); the
fixtures ``attention_*.npz`` are committed, this script documents how they were made.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)
from attention_inputs import attention_inputs  # noqa: E402
from oracle import ref_loader  # noqa: E402

ref_loader.load()
from qutai.backends import cpu, cpu_lm  # noqa: E402


def _store(a):
    return cpu.storage(np.asarray(a, dtype=np.float64).reshape(-1).tolist(), dtype="float64")


def _arr(storage, shape):
    return np.array(storage.tolist(), dtype=np.float64).reshape(shape)


def attention_case(name, batch, time, heads, kv_heads, seed, scale=1.0, dim=64):
    q, k, v, grad = attention_inputs(batch, time, heads, kv_heads, seed, scale, dim)
    dims = (batch, time, heads, kv_heads, dim)
    out, lse = cpu_lm.attention(_store(q), _store(k), _store(v), *dims)
    dq, dk, dv = cpu_lm.attention_backward(_store(grad), _store(q), _store(k), _store(v), out, lse, *dims)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), kind="attention", batch=batch, time=time, heads=heads,
                        kv_heads=kv_heads, seed=seed, scale=scale, out=_arr(out, q.shape).astype(np.float32), lse=_arr(lse, (batch, time, heads)).astype(np.float32),
                        dq=_arr(dq, q.shape).astype(np.float32), dk=_arr(dk, k.shape).astype(np.float32),
                        dv=_arr(dv, v.shape).astype(np.float32))
    print(name, "out rms", float(np.sqrt(np.mean(_arr(out, q.shape) ** 2))))


if __name__ == "__main__":
    attention_case("attention_small", 2, 5, 4, 2, 41)
    attention_case("attention_one_position", 1, 1, 2, 1, 42)
    attention_case("attention_two_blocks", 1, 150, 1, 1, 43, scale=0.7)
    attention_case("attention_heads_equal", 1, 33, 2, 2, 44, scale=1.5)
