"""The autograd wiring of the fused layer on the GPU.  The upstream engine itself cannot run here (it is not on
the GPU machine; tests/test_autograd_wiring.py drives it on CPU), so a minimal engine with the same rules —
``record`` keeps parents and a rule when recording is on, ``backward`` walks nodes in reverse topological order,
sums contributions and accumulates leaves into ``.grad`` (src/qutai/core/grad.py:7-65,
src/qutai/core/tensor.py:203-210), a checkpoint runs the function unrecorded and re-runs it inside the backward
(src/qutai/lm/recompute.py:13-79) — drives ``qutai_b200.autograd.recorded_call`` over the CUDA layer.  Checked:
gradients equal the golden fixture the upstream package produced, the expert weight gradients are bit-identical
to the direct ``layer.backward``, and checkpointing changes no bit."""
import os

import numpy as np
import pytest

from conftest import GOLDEN
from oracle import moe_oracle as oracle

pytestmark = pytest.mark.gpu


class Engine:
    """The upstream autograd rules in miniature, over ``qutai_b200.layers.Tensor``."""

    def __init__(self):
        self.recording = True

    def record(self, result, parents, rule=None):
        result.requires_grad = self.recording and any(p.requires_grad for p in parents)
        if result.requires_grad:
            result.parents, result.backward_rule = parents, rule
        return result

    @staticmethod
    def add(a, b):
        from qutai_b200 import lib
        from qutai_b200.storage import DeviceStorage

        out = DeviceStorage(a.size, a.dtype)
        lib.call("qmoe_add", a.ptr, b.ptr, out.ptr, lib.DTYPE_CODES[a.dtype], a.size, 0)
        return out

    def backward(self, outputs):
        """``outputs``: [(tensor, gradient storage)].  Leaves accumulate into ``.grad`` (a copy for the first
        contribution, a sum afterwards), as upstream's leaf sink does."""
        from qutai_b200.layers import Tensor

        order, seen = [], set()

        def visit(t):
            if id(t) in seen:
                return
            seen.add(id(t))
            for p in t.parents:
                if p.requires_grad:
                    visit(p)
            order.append(t)

        gradients = {}
        for tensor, gradient in outputs:
            visit(tensor)
            gradients[id(tensor)] = gradient
        while order:
            t = order.pop()
            incoming = gradients.pop(id(t), None)
            if incoming is None:
                continue
            if t.backward_rule is None:
                t.grad = Tensor(incoming.copy() if t.grad is None else self.add(t.grad.storage, incoming), t.shape)
                continue
            for parent, contribution in zip(t.parents, t.backward_rule(incoming), strict=True):
                if parent.requires_grad and contribution is not None:
                    gradients[id(parent)] = self.add(gradients[id(parent)], contribution) if id(parent) in gradients else contribution

    def checkpoint(self, function, argument, parameters):
        """Run ``function`` unrecorded now and again, recorded, when the gradient arrives."""
        from qutai_b200.layers import Tensor

        was, self.recording = self.recording, False
        try:
            outputs = function(argument)
        finally:
            self.recording = was
        results = []
        state = {}

        def rerun():   # both outputs share one recomputation
            if "graph" not in state:
                replacement = Tensor(argument.storage, argument.shape, requires_grad=argument.requires_grad)
                state["graph"] = (replacement, function(replacement))
            return state["graph"]

        pending = {}

        def rule_for(index):
            def rule(gradient):
                pending[index] = gradient
                if len(pending) < len(outputs):
                    return (None,) * (1 + len(parameters))
                replacement, recomputed = rerun()
                before = [p.grad for p in parameters]
                for p in parameters:
                    p.grad = None
                self.backward([(recomputed[i], pending[i]) for i in sorted(pending)])
                inner = [replacement.grad] + [p.grad for p in parameters]
                for p, g in zip(parameters, before):
                    p.grad = g
                return tuple(None if g is None else g.storage for g in inner)
            return rule

        for index, output in enumerate(outputs):
            results.append(self.record(Tensor(output.storage, output.shape), (argument, *parameters), rule_for(index)))
        return tuple(results)


def run(layer, g, engine, checkpointing):
    from gpu_util import to_device, to_host
    from qutai_b200.autograd import recorded_call
    from qutai_b200.layers import Tensor

    T, d = g["x"].shape
    for p in layer.parameters():
        p.zero_grad()
    x = Tensor(to_device(g["x"], "float32"), (T, d), requires_grad=True)
    call = lambda value: recorded_call(layer, value, record=engine.record, tensor=Tensor)
    y, aux = engine.checkpoint(call, x, layer.parameters()) if checkpointing else call(x)
    assert y.requires_grad and aux.requires_grad
    engine.backward([(y, to_device(g["grad_y"], "float32")), (aux, to_device(np.array([float(g["grad_aux"])]), "float32"))])
    E, h = layer.n_experts, layer.d_expert
    grads = dict(x=to_host(x.grad.storage, (T, d)), router=to_host(layer.router.weight.grad.storage, (E, d)))
    for key in ("gate", "up", "down"):
        grads[key] = [None if getattr(e, key).weight.grad is None else to_host(getattr(e, key).weight.grad.storage) for e in layer.experts]
    return to_host(y.storage, (T, d)), float(to_host(aux.storage)[0]), grads


@pytest.mark.parametrize("fixture", ["layer_mid.npz", "layer_empty_expert.npz"])
def test_recorded_layer_under_a_minimal_engine(fixture):
    from gpu_util import make_layer, run_layer

    g = np.load(os.path.join(GOLDEN, fixture))
    layer = make_layer(g["x"].shape, g["router"], g["gate"], g["up"], g["down"], int(g["top_k"]))
    direct = run_layer(layer, g["x"], g["grad_y"], float(g["grad_aux"]), "float32")
    engine = Engine()
    results = {flag: run(layer, g, engine, flag) for flag in (False, True)}
    y, aux, grads = results[False]
    E, step = g["gate"].shape[0], int(g["sample"])
    assert oracle.max_rel_err(y, g["y"]) <= 1e-4 and abs(aux - float(g["aux"])) <= 1e-5
    assert oracle.max_rel_err(grads["x"], g["dx"]) <= 1e-4
    assert oracle.max_rel_err(grads["router"], g["d_router"]) <= 1e-4
    for e in range(E):
        for key in ("gate", "up", "down"):
            if not g["has_grad"][e]:
                assert grads[key][e] is None               # no contribution, so no gradient object
            else:
                assert oracle.max_rel_err(grads[key][e][::step], g[f"d_{key}_{e}"]) <= 1e-4
                # the expert weights do not depend on the auxiliary path: the same bits as the fused backward
                assert np.array_equal(grads[key][e], direct["d_" + key][e].reshape(-1))
    # the output node's and the auxiliary node's contributions are rounded separately and then added, the fused
    # backward adds them before its one product: equal to fp32 rounding
    assert oracle.max_rel_err(grads["router"], direct["d_router"]) <= 1e-5
    assert oracle.max_rel_err(grads["x"], direct["dx"]) <= 1e-5
    # checkpointing recomputes the same bits
    y2, aux2, grads2 = results[True]
    assert np.array_equal(y, y2) and aux == aux2
    assert np.array_equal(grads["x"], grads2["x"]) and np.array_equal(grads["router"], grads2["router"])
    for e in range(E):
        for key in ("gate", "up", "down"):
            assert (grads[key][e] is None) == (grads2[key][e] is None)
            if grads[key][e] is not None:
                assert np.array_equal(grads[key][e], grads2[key][e])
