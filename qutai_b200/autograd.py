"""Wiring of the fused layer into a reverse-mode autograd of the upstream kind.

Upstream every operation returns ``record(result, parents, rule)`` (src/qutai/core/grad.py:7-13): ``rule``
maps the gradient of ``result`` to one contribution per parent (``None`` = nothing), ``backward`` walks the
nodes in reverse topological order, sums the contributions a tensor receives and hands leaves to a sink
that accumulates ``.grad`` (src/qutai/core/grad.py:34-65, src/qutai/core/tensor.py:191-216).  Its
``SparseMoE.__call__`` registers one node for the gate weights, one for the auxiliary loss, one per linear
map of every expert and an identity node for the output (src/qutai/lm/layers.py:382-402).

``recorded_call`` registers TWO nodes for the whole fused layer instead:

* the output ``y`` with parents ``(x, router.weight, expert 0's gate, up, down weights, expert 1's ...)`` —
  the order of ``parameters()`` — whose rule is one ``qmoe_layer_backward`` and returns the input gradient,
  the router gradient and the three weight gradients of every expert that received tokens, ``None`` for the
  others (such an expert's parameters keep ``grad is None``, pinned by tests/test_lm_moe.py:74-100);
* the auxiliary loss with parents ``(x, router.weight)`` whose rule is the routing backward of the auxiliary
  path followed by the router's backward.

Nothing else is needed for activation checkpointing (src/qutai/lm/recompute.py:13-79): under
``checkpoint(block.packed, hidden, parameters=block.parameters())`` the first call runs with recording
off (both nodes come back without parents), the backward re-runs the call under recording and walks these
two nodes; the parameters are leaves of that inner walk exactly as upstream's are.

``record`` and the tensor class are passed in, so the same function serves upstream's own engine (with its
``Tensor`` over storages that carry ``ptr``) and this package's minimal ``Tensor``.
"""
from __future__ import annotations


def recorded_call(layer, x, *, record, tensor):
    """``layer(x)`` registered with autograd.  ``record(result, parents, rule)`` and ``tensor(storage,
    shape=...)`` are the host framework's; ``layer`` is a ``qutai_b200.layers.SparseMoE`` (or anything with
    its ``forward`` / ``backward_contributions`` / ``backward_aux`` / ``parameters``).  Returns
    ``(y, aux)`` as the host framework's tensors."""
    y, aux = layer.forward(x)
    parameters = tuple(layer.parameters())
    n_experts = (len(parameters) - 1) // 3

    def output_rule(gradient):
        dx, d_router, experts = layer.backward_contributions(gradient, None)
        contributions = [dx.storage, d_router.storage]
        for expert in experts:
            contributions.extend((None, None, None) if expert is None else (t.storage for t in expert))
        return tuple(contributions)

    def auxiliary_rule(gradient):
        dx, d_router = layer.backward_aux(gradient)
        return dx.storage, d_router.storage

    assert len(parameters) == 1 + 3 * n_experts
    result = record(tensor(y.storage, shape=tuple(x.shape)), (x, *parameters), output_rule)
    auxiliary = record(tensor(aux.storage, shape=()), (x, parameters[0]), auxiliary_rule)
    return result, auxiliary
