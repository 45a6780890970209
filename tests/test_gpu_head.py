"""The language-model head with its cross-entropy loss (``qutai_b200.head`` over ``qmoe_head_forward`` /
``qmoe_head_backward``) against the fixtures the upstream package's ``projection_loss`` produced (fp32), against the
oracle on bf16-rounded inputs (bf16: tcgen05 products when width and vocab are multiples of 8, CUDA cores
otherwise), and at the size of a full training step through row and column samples.  Needs a B200: ``-m gpu``."""
import os

import numpy as np
import pytest

from conftest import golden_files
from oracle import moe_oracle as oracle

pytestmark = pytest.mark.gpu

FP32_TOL, BF16_TOL = 1e-4, 2e-2
FP32_ELEMENT_TOL = 2e-5      # |x - y| <= 2e-5 (1 + |y|), upstream's fp32 bar (tests/test_lm_moe.py:105-138)
BF16_ELEMENT_TOL = 0.08      # |x - y| <= 0.08 max(rms(y), |y|): sums of many bf16 products


def run_head(hidden, weight, labels, dtype, gradient=None, weight_dtype=None):
    from gpu_util import to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.head import LMHead, prepare_labels
    from qutai_b200.layers import Tensor

    head = LMHead()
    h = Tensor(to_device(hidden, dtype), hidden.shape)
    w = Tensor(to_device(weight, weight_dtype or dtype), weight.shape)
    loss = head.forward(h, w, prepare_labels(labels.tolist()))
    g = None if gradient is None else to_device(np.array([gradient]), "float32")
    d_hidden, d_weight = head.backward(g)
    assert lib.device_status() == 0
    rows = hidden.shape[0] * (hidden.shape[1] - 1)
    return dict(loss=float(to_host(loss.storage)[0]), d_hidden=to_host(d_hidden.storage, hidden.shape),
                d_weight=to_host(d_weight.storage, weight.shape), head=head,
                row_loss=to_host(head._buffers["row_loss"])[:rows])


@pytest.mark.parametrize("path", golden_files("head"), ids=os.path.basename)
def test_head_fp32_matches_the_upstream_fixture(path):
    g = np.load(path)
    gradient = float(g["gradient"])
    got = run_head(g["hidden"], g["weight"], g["labels"], "float32", None if gradient == 1.0 else gradient)
    assert abs(got["loss"] - float(g["loss"])) <= FP32_ELEMENT_TOL * (1 + abs(float(g["loss"])))
    for name in ("d_hidden", "d_weight"):
        assert oracle.max_rel_err(got[name], g[name]) <= FP32_TOL, name
        assert oracle.elementwise_err(got[name], g[name]) <= FP32_ELEMENT_TOL, name
    assert not got["d_hidden"][:, -1, :].any()
    again = run_head(g["hidden"], g["weight"], g["labels"], "float32", None if gradient == 1.0 else gradient)
    for name in ("loss", "d_hidden", "d_weight"):          # fixed summation orders: the same bits on every run
        assert np.array_equal(again[name], got[name]), name


@pytest.mark.parametrize("path", golden_files("head"), ids=os.path.basename)
@pytest.mark.parametrize("master", [False, True], ids=["bf16-weight", "fp32-weight"])
def test_head_bf16_matches_the_oracle(path, master):
    g = np.load(path)
    hidden, weight = oracle.round_bf16(g["hidden"]), oracle.round_bf16(g["weight"])
    gradient = float(g["gradient"])
    want_loss, ctx = oracle.head_loss_forward(hidden, weight, g["labels"])
    want_dx, want_dw, _ = oracle.head_loss_backward(ctx, gradient)
    got = run_head(hidden, weight, g["labels"], "bfloat16", None if gradient == 1.0 else gradient,
                   weight_dtype="float32" if master else None)
    assert abs(got["loss"] - want_loss) <= BF16_TOL * max(1.0, abs(want_loss))
    if not ctx["counted"].any():
        assert not got["d_hidden"].any() and not got["d_weight"].any()
        return
    for name, want in (("d_hidden", want_dx), ("d_weight", want_dw)):
        assert oracle.max_rel_err(got[name], want) <= BF16_TOL, name
        assert oracle.elementwise_err(got[name], want, bf16=True, unit=oracle.rms(want)) <= BF16_ELEMENT_TOL, name


def test_head_labels_outside_the_vocabulary_count_as_ignored():
    """A label that is not a class (negative other than -100, or >= vocab) must not be used as an index: such rows
    are left out exactly like -100."""
    g = np.load([p for p in golden_files("head") if p.endswith("head_mid.npz")][0])
    vocab = g["weight"].shape[0]
    labels = g["labels"].copy()
    wild = labels.copy()
    wild[0, 1], wild[1, 2], wild[2, 3] = vocab, -7, 2 ** 40
    labels[0, 1] = labels[1, 2] = labels[2, 3] = -100
    got = run_head(g["hidden"], g["weight"], wild, "float32")
    want = run_head(g["hidden"], g["weight"], labels, "float32")
    for name in ("loss", "d_hidden", "d_weight"):
        assert np.array_equal(got[name], want[name]), name


def test_head_rejects_bad_arguments():
    from gpu_util import to_device
    from qutai_b200.head import LMHead
    from qutai_b200.layers import Tensor

    head = LMHead()
    hidden = Tensor(to_device(np.zeros((2, 1, 8)), "float32"), (2, 1, 8))
    weight = Tensor(to_device(np.zeros((16, 8)), "float32"), (16, 8))
    with pytest.raises(ValueError):
        head.forward(hidden, weight, [[0], [1]])                      # a sequence of one position has no target
    hidden = Tensor(to_device(np.zeros((2, 3, 8)), "float32"), (2, 3, 8))
    with pytest.raises(ValueError):
        head.forward(hidden, weight, [[0, 1, 2]])                     # labels do not cover the batch
    with pytest.raises(RuntimeError):
        LMHead().backward()


def test_head_at_the_size_of_a_training_step():
    """Vocabulary 32000, width 1024, 4 sequences of 2048 positions (one rank's share of the full decoder step):
    the loss of sampled rows, their rows of the input gradient and sampled rows of the weight gradient against
    float64 arithmetic on the same bf16 values."""
    batch, time, width, vocab = 4, 2048, 1024, 32000
    rng = np.random.default_rng(7)
    hidden = oracle.round_bf16(rng.standard_normal((batch, time, width), dtype=np.float32))
    weight = oracle.round_bf16(rng.standard_normal((vocab, width), dtype=np.float32) * 0.02)
    labels = np.minimum(rng.zipf(1.1, size=(batch, time)) - 1, vocab - 1).astype(np.int64)
    labels[rng.random((batch, time)) < 0.05] = -100
    got = run_head(hidden, weight, labels, "bfloat16")
    rows = batch * (time - 1)
    targets = labels[:, 1:].reshape(-1)
    counted = targets != -100
    count = max(1, int(counted.sum()))
    inputs = hidden[:, :-1, :].reshape(rows, width)
    # the loss of every row from the device's own row losses, and sampled rows in float64
    assert abs(got["loss"] - got["row_loss"].sum() / count) <= 1e-4 * abs(got["loss"])
    assert not got["row_loss"][~counted].any()
    sample = np.concatenate([rng.choice(rows, 24, replace=False), np.flatnonzero(~counted)[:4], [0, rows - 1]])
    z = oracle.round_bf16(inputs[sample] @ weight.T)          # the logits are kept in bf16
    peak = z.max(axis=1, keepdims=True)
    total = np.exp(z - peak).sum(axis=1)
    for i, r in enumerate(sample):
        want = 0.0 if not counted[r] else np.log(total[i]) - (z[i, targets[r]] - peak[i, 0])
        assert abs(got["row_loss"][r] - want) <= 2e-2 * max(1.0, abs(want)), r
    # the kept gradient of the logits: every row sums to zero; sampled rows against float64
    head = got["head"]
    raw = np.frombuffer(head._buffers["logits"].tobytes(), dtype=np.uint16)[:rows * vocab]
    kept = (raw.astype(np.uint32) << 16).view(np.float32).reshape(rows, vocab)
    del raw
    assert np.abs(kept.sum(axis=1, dtype=np.float64)).max() <= 2e-2 / count * 8
    assert not kept[~counted].any()
    want_rows = np.exp(z - peak) / total[:, None]
    for i, r in enumerate(sample):
        if counted[r]:
            want_rows[i, targets[r]] -= 1.0
        else:
            want_rows[i] = 0.0
    want_rows /= count
    assert oracle.elementwise_err(kept[sample], want_rows, bf16=True, unit=oracle.rms(want_rows)) <= BF16_ELEMENT_TOL
    # the two products of the backward on the kept gradient (what the device multiplied), sampled
    d_hidden = got["d_hidden"].reshape(batch, time, width)
    assert not d_hidden[:, -1, :].any()
    got_rows = d_hidden[:, :-1, :].reshape(rows, width)[sample]
    want_dx = kept[sample].astype(np.float64) @ weight
    assert oracle.elementwise_err(got_rows, want_dx, bf16=True, unit=oracle.rms(want_dx)) <= BF16_ELEMENT_TOL
    classes = np.concatenate([rng.choice(vocab, 12, replace=False), [0, vocab - 1, int(np.bincount(targets[counted]).argmax())]])
    want_dw = kept[:, classes].T.astype(np.float64) @ inputs
    got_dw = got["d_weight"][classes]
    assert oracle.max_rel_err(got_dw, want_dw) <= 1e-3       # fp32 accumulation of exact bf16 products


def test_projection_loss_keeps_the_upstream_signature_and_record_shape():
    """``projection_loss(hidden, weight, labels, chunk_size, prepared_labels=...)`` returns the loss with
    ``parents = (hidden, weight)`` and a rule that maps the incoming gradient to one contribution per parent
    (``None`` for a parent that needs no gradient), the shape upstream's ``record`` takes
    (src/qutai/core/grad.py:7-13, src/qutai/lm/layers.py:215-257)."""
    from gpu_util import to_device, to_host
    from qutai_b200.head import prepare_labels, projection_loss
    from qutai_b200.layers import Tensor

    g = np.load([p for p in golden_files("head") if p.endswith("head_mid.npz")][0])
    hidden = Tensor(to_device(g["hidden"], "float32"), g["hidden"].shape, requires_grad=True)
    weight = Tensor(to_device(g["weight"], "float32"), g["weight"].shape, requires_grad=False)
    labels = [list(map(int, row)) for row in g["labels"]]
    loss = projection_loss(hidden, weight, labels, 7)
    assert loss.shape == () and loss.parents == (hidden, weight)
    assert abs(to_host(loss.storage)[0] - float(g["loss"])) <= FP32_ELEMENT_TOL * (1 + abs(float(g["loss"])))
    d_hidden, d_weight = loss.backward_rule(to_device(np.array([float(g["gradient"])]), "float32"))
    assert d_weight is None                                         # the weight did not ask for a gradient
    assert oracle.elementwise_err(to_host(d_hidden, g["hidden"].shape), g["d_hidden"]) <= FP32_ELEMENT_TOL
    again = projection_loss(hidden, weight, None, 7, prepared_labels=prepare_labels(labels))
    assert to_host(again.storage)[0] == to_host(loss.storage)[0]
