"""Seeded inputs of the attention fixtures (values a bfloat16 holds exactly), shared by the script that made the
fixtures and by the tests, so that the fixtures store the upstream results only."""
import numpy as np


def attention_inputs(batch, time, heads, kv_heads, seed, scale=1.0, dim=64):
    rng = np.random.default_rng(seed)
    bf = lambda a: (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) & 0xFFFF0000).view(np.float32)
    q = bf(rng.standard_normal((batch, time, heads * dim)) * scale)
    k = bf(rng.standard_normal((batch, time, kv_heads * dim)) * scale)
    v = bf(rng.standard_normal((batch, time, kv_heads * dim)))
    grad = bf(rng.standard_normal((batch, time, heads * dim)))
    return q, k, v, grad
