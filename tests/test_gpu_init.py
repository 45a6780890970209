"""Parameter initialisation of the layer (src/qutai/lm/layers.py:355-374, :261-266, :292-308 upstream): every
tensor is N(0, 0.02) except the down projections, which get 0.02 / sqrt(2 n_layers); the router is drawn with
the layer's seed ``s`` and expert ``i`` with ``s + 1 + 3 i`` (gate), ``+ 1`` (up), ``+ 2`` (down).  The draws come
from the library's counter-based generator (``qmoe_normal_fill``): deterministic per key, independent between
keys.  Like upstream's device generator it is not the CPU generator's stream (tests/test_lm_moe.py:105-108
copies weights for that reason), so what is pinned here are moments, determinism and the key schedule."""
from math import sqrt

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def draws(n, std, seed, mean=0.0, dtype="float32"):
    from gpu_util import to_host
    from qutai_b200.storage import DeviceStorage

    storage = DeviceStorage(n, dtype)
    storage.fill_normal(mean, std, seed)
    return to_host(storage)


def test_normal_fill_moments_determinism_and_key_independence():
    n = 1 << 20
    a = draws(n, 0.02, 7)
    assert np.array_equal(a, draws(n, 0.02, 7))                      # same key, same draws
    b = draws(n, 0.02, 8)
    assert not np.array_equal(a, b)
    # N(0, 0.02) over 2^20 draws: the mean is within 5 standard errors, the standard deviation within 1 %
    assert abs(a.mean()) <= 5 * 0.02 / sqrt(n)
    assert abs(a.std() / 0.02 - 1) <= 0.01
    assert abs(np.corrcoef(a, b)[0, 1]) <= 5 / sqrt(n)               # neighbouring keys are uncorrelated
    assert abs(np.corrcoef(a[:-1], a[1:])[0, 1]) <= 5 / sqrt(n)      # and so are neighbouring draws of one key
    # shape of the distribution: the standardised fourth moment of a normal is 3, 4.55 % lie beyond two sigma
    z = a / a.std()
    assert abs((z ** 4).mean() - 3.0) <= 0.05
    assert abs((np.abs(z) > 2).mean() - 0.0455) <= 0.002
    shifted = draws(n, 0.5, 7, mean=3.0)
    assert abs(shifted.mean() - 3.0) <= 5 * 0.5 / sqrt(n) and abs(shifted.std() / 0.5 - 1) <= 0.01
    assert np.allclose(shifted, 3.0 + a * 25.0, atol=1e-5)           # the same underlying standard normal draws
    # a prefix of a longer fill is the shorter fill (the generator is indexed by position, not by launch shape)
    assert np.array_equal(draws(1000, 0.02, 7), a[:1000])
    rounded = draws(4096, 0.02, 7, dtype="bfloat16")
    assert np.abs(rounded - a[:4096]).max() <= 0.02 * 6 * 2.0 ** -8   # bf16 storage rounds the same draws


@pytest.mark.parametrize("n_layers", [1, 12])
def test_layer_parameters_follow_the_upstream_initialisation(n_layers):
    from gpu_util import Config, to_host
    from qutai_b200.layers import SparseMoE

    d, E, k, h, seed = 128, 6, 2, 256, 40
    layer = SparseMoE(Config(d, E, k, h, n_layers=n_layers), device="cuda", dtype="float32", seed=seed)
    parameters = layer.parameters()
    assert len(parameters) == 1 + 3 * E and parameters[0] is layer.router.weight
    assert layer.router.weight.shape == (E, d) and all(p.requires_grad and p.dtype == "float32" for p in parameters)
    assert np.array_equal(to_host(layer.router.weight.storage), draws(E * d, 0.02, seed))
    down_std = 0.02 / sqrt(2 * n_layers)
    for i, expert in enumerate(layer.experts):
        assert parameters[1 + 3 * i: 4 + 3 * i] == (expert.gate.weight, expert.up.weight, expert.down.weight)
        assert expert.gate.weight.shape == (h, d) and expert.up.weight.shape == (h, d) and expert.down.weight.shape == (d, h)
        base = seed + 1 + 3 * i
        assert np.array_equal(to_host(expert.gate.weight.storage), draws(h * d, 0.02, base))
        assert np.array_equal(to_host(expert.up.weight.storage), draws(h * d, 0.02, base + 1))
        down = to_host(expert.down.weight.storage)
        assert np.array_equal(down, draws(d * h, down_std, base + 2))
        assert abs(down.std() / down_std - 1) <= 0.02 and abs(to_host(expert.gate.weight.storage).std() / 0.02 - 1) <= 0.02
    assert layer.last_counts == (0,) * E and layer.utilization is None and layer.top_k == k and layer.n_experts == E
    # another seed gives other weights; the same seed the same ones
    again = SparseMoE(Config(d, E, k, h, n_layers=n_layers), device="cuda", dtype="float32", seed=seed)
    other = SparseMoE(Config(d, E, k, h, n_layers=n_layers), device="cuda", dtype="float32", seed=seed + 1)
    assert np.array_equal(to_host(again._down), to_host(layer._down))
    assert not np.array_equal(to_host(other._gate), to_host(layer._gate))
