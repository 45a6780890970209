"""A whole mixture-of-experts decoder step (``qutai_b200.decoder.Decoder``: embedding, two blocks of grouped-query
attention with rotary embedding and a MoE feed-forward half, final norm, tied head with its loss and the auxiliary
term) against what the upstream ``Decoder`` produced on its CPU float64 path for the same parameters and tokens
(tests/golden/make_golden_decoder.py).  Everything runs in bfloat16 here, so the bars are those of bf16 products
carried through two blocks.  Needs a B200: ``-m gpu``."""
import os
import sys

import numpy as np
import pytest

from oracle import moe_oracle as oracle

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden_decoder as fixture  # noqa: E402  (only its seeded inputs are used; upstream is not imported)

pytestmark = pytest.mark.gpu


def build():
    from qutai_b200.decoder import Config, Decoder

    model = Decoder(Config(aux_loss_coef=0.05, **fixture.SHAPE), seed=3)
    named = model.named_parameters()
    values = fixture.decoder_parameters([(name, tuple(p.shape)) for name, p in named])
    for name, parameter in named:
        parameter.storage.upload_bytes(np.ascontiguousarray(values[name], dtype=np.float32).tobytes())
    return model, named


def test_decoder_loss_and_every_gradient_match_the_upstream_decoder():
    from gpu_util import to_host
    from qutai_b200 import lib

    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "decoder_small.npz"))
    model, named = build()
    assert [name for name, _ in named] == [key[5:] for key in g.files if key.startswith("grad:")]      # upstream's names and order
    tokens, labels = fixture.decoder_tokens()
    loss = model.loss(tokens, labels)
    model.backward()
    assert lib.device_status() == 0
    assert abs(to_host(loss.storage)[0] - float(g["loss"])) <= 2e-2 * abs(float(g["loss"]))
    assert abs(to_host(model.last_lm_loss.storage)[0] - float(g["lm_loss"])) <= 2e-2 * abs(float(g["lm_loss"]))
    assert abs(to_host(model.last_auxiliary_loss.storage)[0] - float(g["aux_loss"])) <= 1e-2 * abs(float(g["aux_loss"]))
    worst = {}
    for name, parameter in named:
        want = g["grad:" + name]
        if want.size == 0:
            assert parameter.grad is None, name             # an expert that received no token
            continue
        assert parameter.grad is not None, name
        got = to_host(parameter.grad.storage, want.shape)
        worst[name] = oracle.max_rel_err(got, want)
    loose = {name: error for name, error in worst.items() if error > 6e-2}
    assert not loose, loose
    assert np.median(list(worst.values())) <= 2e-2


def test_decoder_steps_with_adamw_and_the_loss_falls():
    from gpu_util import to_host
    from qutai_b200.optim import AdamW

    tokens, labels = fixture.decoder_tokens()
    curves = []
    for with_shadows in (False, True):
        model, named = build()
        if with_shadows:
            model.loss(tokens, labels)                     # makes the operand copies the optimizer is to keep current
        optimizer = AdamW(model.parameters(), learning_rate=3e-3, shadows=model.operand_shadows() if with_shadows else None)
        losses = []
        for _ in range(6):
            model.zero_grad()
            loss = model.loss(tokens, labels)
            model.backward()
            optimizer.step()
            losses.append(float(to_host(loss.storage)[0]))
        assert losses[-1] < losses[0] - 0.3, losses
        curves.append(losses)
    assert curves[0] == curves[1]          # the copies the optimizer writes are the ones a forward would have made


def test_decoder_rejects_what_it_does_not_cover():
    from qutai_b200.decoder import Config, Decoder

    with pytest.raises(ValueError):
        Decoder(Config(vocab_size=10, d_model=64, n_heads=2, n_kv_heads=1, n_layers=1, n_experts=2, top_k=1, d_expert=8))   # head width 32
    model, _ = build()
    with pytest.raises(ValueError):
        model.loss([[1]])
    with pytest.raises(ValueError):
        model.loss([[1, 2, 999]])
    with pytest.raises(RuntimeError):
        model.backward()
