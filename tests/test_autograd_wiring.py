"""The autograd wiring of the fused layer (``qutai_b200.autograd.recorded_call``) driven by the UPSTREAM engine:
upstream's own ``record`` / ``backward`` (src/qutai/core/grad.py), ``checkpoint`` (src/qutai/lm/recompute.py),
``Block.packed`` with ``pack`` / ``unpack`` (src/qutai/lm/layers.py:155-184, :443-444) and ``Decoder.loss``
(src/qutai/lm/decoder.py:143-175) run a tiny MoE decoder whose ``SparseMoE`` layers were swapped for the glue
over a stand-in with the fused layer's interface (``forward`` / ``backward_contributions`` / ``backward_aux`` /
``parameters``; its arithmetic is the numpy oracle, on upstream CPU storages).  Every parameter gradient must
equal the unmodified upstream model's, with and without activation checkpointing, and an expert without tokens
must keep ``grad is None``.

Runs only where a checkout of the upstream sources is present (this is a CPU test; the GPU counterpart,
tests/test_gpu_autograd.py, drives the same glue over the CUDA layer with a minimal engine of the same rules).
"""
import numpy as np
import pytest

from oracle import moe_oracle as oracle
from oracle import ref_loader
from qutai_b200.autograd import recorded_call

pytestmark = pytest.mark.skipif(ref_loader.reference_root() is None, reason="upstream sources are not on this machine")


class _Value:
    def __init__(self, storage, shape):
        self.storage, self.shape = storage, shape


class OracleLayer:
    """The fused layer's interface over the numpy oracle, holding the upstream layer's own parameter tensors."""

    def __init__(self, upstream_layer, cpu):
        self.upstream, self.cpu = upstream_layer, cpu
        self.top_k, self.n_experts = upstream_layer.top_k, upstream_layer.n_experts
        self.calls = dict(forward=0, backward=0, backward_aux=0)

    def parameters(self):
        return self.upstream.parameters()

    def _array(self, tensor):
        return np.array(tensor.storage.tolist(), dtype=np.float64).reshape(tensor.shape)

    def _storage(self, array):
        return self.cpu.storage(np.asarray(array, dtype=np.float64).reshape(-1).tolist(), dtype="float64")

    def forward(self, x):
        self.calls["forward"] += 1
        experts = self.upstream.experts
        self.x_shape = tuple(x.shape)
        rows = self._array(x).reshape(-1, x.shape[-1])
        y, aux, self.ctx = oracle.moe_forward(
            rows, self._array(self.upstream.router.weight), [self._array(e.gate.weight) for e in experts],
            [self._array(e.up.weight) for e in experts], [self._array(e.down.weight) for e in experts], self.top_k)
        self.upstream.last_counts = self.ctx["route"]["counts"]
        return _Value(self._storage(y), self.x_shape), _Value(self._storage([aux]), ())

    def backward_contributions(self, gradient, grad_aux=None):
        self.calls["backward"] += 1
        assert grad_aux is None
        g = np.array(gradient.tolist(), dtype=np.float64).reshape(self.ctx["x"].shape)
        grads = oracle.moe_backward(self.ctx, g, 0.0)
        experts = [None if grads["gate"][e] is None else tuple(_Value(self._storage(grads[key][e]), None) for key in ("gate", "up", "down"))
                   for e in range(self.n_experts)]
        return _Value(self._storage(grads["x"]), self.x_shape), _Value(self._storage(grads["router"]), None), experts

    def backward_aux(self, gradient):
        self.calls["backward_aux"] += 1
        d_scores = oracle.routing_backward(gradient.tolist(), self.ctx["route"], True)
        return (_Value(self._storage(d_scores @ self.ctx["router"]), self.x_shape),
                _Value(self._storage(d_scores.T @ self.ctx["x"]), None))


def models(checkpointing, top_k=2, seed=2):
    qutai = ref_loader.load()
    from qutai.backends import cpu
    from qutai.core.grad import record
    from qutai.core.tensor import Tensor
    from qutai.lm.config import Config
    from qutai.lm.decoder import Decoder

    config = Config(vocab_size=17, n_layers=2, d_model=8, n_heads=2, n_kv_heads=1, d_ff=12, max_seq_len=8, ffn_type="moe",
                    n_experts=3, top_k=top_k, d_expert=6, activation_checkpointing=checkpointing)
    plain, wired = Decoder(config, dtype="float64", seed=seed), Decoder(config, dtype="float64", seed=seed)
    stand_ins = []
    for block in wired.blocks:
        stand_in = OracleLayer(block.ffn, cpu)
        stand_ins.append(stand_in)

        class Wired:   # what replaces SparseMoE.__call__: the glue, with upstream's record and Tensor
            def __init__(self, inner):
                self.inner = inner

            def __call__(self, x):
                return recorded_call(self.inner, x, record=record, tensor=Tensor)

            def parameters(self):
                return self.inner.parameters()

            def __getattr__(self, name):   # router, experts, utilization, ...: the upstream layer's own attributes
                return getattr(self.inner.upstream, name)

        block.ffn = Wired(stand_in)
    return plain, wired, stand_ins


@pytest.mark.parametrize("checkpointing", [False, True])
def test_gradients_through_the_upstream_engine_match_the_upstream_layer(checkpointing):
    plain, wired, stand_ins = models(checkpointing)
    tokens = [[1, 2, 3, 4], [2, 3, 4, 5]]
    loss_plain, loss_wired = plain.loss(tokens), wired.loss(tokens)
    assert abs(loss_plain.item() - loss_wired.item()) <= 1e-12
    loss_plain.backward()
    loss_wired.backward()
    compared = 0
    for a, b in zip(plain.parameters(), wired.parameters()):
        assert (a.grad is None) == (b.grad is None)
        if a.grad is not None:
            assert np.abs(np.array(a.grad.storage.tolist()) - np.array(b.grad.storage.tolist())).max() <= 1e-11
            compared += 1
    assert compared >= 10
    for stand_in in stand_ins:   # checkpointing runs the forward twice (once unrecorded, once in the backward)
        assert stand_in.calls == dict(forward=2 if checkpointing else 1, backward=1, backward_aux=1)


def test_an_expert_without_tokens_keeps_no_gradient_through_the_glue():
    plain, wired, _ = models(False, top_k=1, seed=8)
    for model in (plain, wired):
        block = model.blocks[0]
        router = block.ffn.parameters()[0]
        d = model.config.d_model
        for i in range(block.attn.out.weight.size):
            block.attn.out.weight.storage[i] = 0           # attention contributes nothing: every row is the embedding
        for j in range(d):
            model.embedding.weight.storage[d + j] = 0.1
        for row in range(model.config.n_experts):          # every token prefers expert 1 (tests/test_lm_moe.py:74-100)
            for j in range(d):
                router.storage[row * d + j] = 0.3 if row == 1 else -0.1
        model.loss([[1, 1, 1, 1]]).backward(retain_graph=False)
    first_plain, first_wired = plain.blocks[0].ffn, wired.blocks[0].ffn
    assert all(p.grad is None for p in first_plain.experts[0].parameters())
    wired_parameters = first_wired.parameters()
    assert all(p.grad is None for p in wired_parameters[1:4])                  # expert 0: gate, up, down
    assert all(p.grad is not None for p in wired_parameters[4:7])              # expert 1 received every token
    for a, b in zip(first_plain.parameters(), wired_parameters):
        if a.grad is not None:
            assert np.abs(np.array(a.grad.storage.tolist()) - np.array(b.grad.storage.tolist())).max() <= 1e-11
