"""Rank-sharded checkpoint files with real device storages: a layer's weights written in two pieces (as two ranks
would), read back into a fresh layer, which then computes the same bits — its bf16 operand copies included.
Needs a B200: ``-m gpu``."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_a_layer_saved_in_two_pieces_loads_into_a_fresh_layer(tmp_path):
    from gpu_util import make_layer, run_layer
    from qutai_b200 import checkpoint

    rng = np.random.default_rng(5)
    T, d, E, k, h = 200, 64, 4, 2, 128
    weights = dict(router=rng.standard_normal((E, d)) * 0.3, gate=rng.standard_normal((E, h, d)) * 0.1,
                   up=rng.standard_normal((E, h, d)) * 0.1, down=rng.standard_normal((E, d, h)) * 0.1)
    x, grad = rng.standard_normal((T, d)), rng.standard_normal((T, d))
    layer = make_layer(x.shape, weights["router"], weights["gate"], weights["up"], weights["down"], k)
    want = run_layer(layer, x, grad, 0.3, "bfloat16")
    named = checkpoint.layer_tensors(layer, "blocks.0.ffn")
    half = 1 + 3 * 2                                         # the router and experts 0, 1 / experts 2, 3
    checkpoint.save_sharded(tmp_path, named[half:], rank=1, world=2, generation=3, chunk_bytes=4096)
    checkpoint.save_sharded(tmp_path, named[:half], rank=0, world=2, generation=3, chunk_bytes=4096, metadata={"step": 3})
    fresh = make_layer(x.shape, *(np.zeros_like(weights[key]) for key in ("router", "gate", "up", "down")), k)
    stale = run_layer(fresh, x, grad, 0.3, "bfloat16")      # a forward with the zero weights: operand copies exist and are stale
    assert not stale["y"].any()
    assert checkpoint.load_sharded(tmp_path, checkpoint.layer_tensors(fresh, "blocks.0.ffn"), verify=True) == {"step": 3}
    got = run_layer(fresh, x, grad, 0.3, "bfloat16")
    for name in ("y", "dx", "d_router"):
        assert np.array_equal(got[name], want[name]), name
    assert got["counts"] == want["counts"]


def test_a_decoder_saved_and_loaded_into_another_gives_the_same_loss_bits(tmp_path):
    """``checkpoint.model_tensors`` over a whole decoder (the upstream parameter names): a second decoder built from
    another seed computes the first one's loss, bit for bit, after loading — the bf16 operand copies of its first
    forward are renewed."""
    from gpu_util import to_host
    from qutai_b200 import checkpoint
    from qutai_b200.decoder import Config, Decoder

    config = Config(vocab_size=40, d_model=128, n_heads=2, n_kv_heads=1, n_layers=2, n_experts=4, top_k=2, d_expert=16)
    tokens = np.random.default_rng(2).integers(0, 40, size=(2, 9)).tolist()
    first, second = Decoder(config, seed=11), Decoder(config, seed=12)
    want = to_host(first.loss(tokens).storage)[0]
    assert to_host(second.loss(tokens).storage)[0] != want
    named = checkpoint.model_tensors(first)
    assert [name for name, _ in named] == [name for name, _ in first.named_parameters()]
    checkpoint.save_sharded(tmp_path, named, metadata={"step": 1})
    assert checkpoint.load_sharded(tmp_path, checkpoint.model_tensors(second), verify=True) == {"step": 1}
    assert to_host(second.loss(tokens).storage)[0] == want
