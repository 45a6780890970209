"""Host logic of ``qutai_b200.optim`` that needs no device: argument checks happen before any launch
(upstream raises in the constructor and in ``clip_grad_norm`` the same way, src/qutai/nn/optimizers.py:19-21,
:125-128), a shared parameter is kept once, and a step without gradients does nothing."""
import pytest

from qutai_b200.optim import AdamW, _parameters, clip_grad_norm


class FakeParameter:
    dtype = "float32"

    def __init__(self):
        self.grad = None

    def zero_grad(self):
        self.grad = None


class FakeModel:
    def __init__(self, parameters):
        self._parameters = parameters

    def parameters(self):
        return self._parameters


def test_parameter_collection_accepts_models_and_drops_duplicates():
    a, b = FakeParameter(), FakeParameter()
    assert _parameters(FakeModel((a, b, a))) == (a, b)
    assert _parameters([b, b, a]) == (b, a)


@pytest.mark.parametrize("bad", [dict(learning_rate=-1e-3), dict(eps=-1.0), dict(weight_decay=-0.5),
                                 dict(betas=(0.9, 1.0)), dict(betas=(-0.1, 0.9)), dict(betas=(0.9,))])
def test_adamw_rejects_settings_before_touching_the_device(bad):
    with pytest.raises(ValueError):
        AdamW([FakeParameter()], **bad)


def test_adamw_rejects_parameters_that_are_not_float32():
    p = FakeParameter()
    p.dtype = "bfloat16"
    with pytest.raises(ValueError):
        AdamW([p])


def test_step_and_clip_without_gradients_do_nothing():
    parameters = [FakeParameter(), FakeParameter()]
    optimizer = AdamW(FakeModel(parameters))
    optimizer.step()                       # no gradient anywhere: no table, no launch, no counters
    assert optimizer.steps == {} and optimizer.averages == {}
    assert clip_grad_norm(parameters, 1.0) == 0.0
    for bad in (-1.0, float("inf"), float("nan")):
        with pytest.raises(ValueError):
            clip_grad_norm(parameters, bad)
