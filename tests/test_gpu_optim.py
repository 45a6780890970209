"""AdamW and the gradient-norm clip on the device (one launch over many tensors, through the C ABI) against
the fixtures the upstream package produced and against the float64 oracle."""
import os

import numpy as np
import pytest

from conftest import ROOT
from oracle import moe_oracle, optim_oracle

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(ROOT, "tests", "golden")
FP32_TOL = 2e-6   # relative to the largest magnitude of the compared tensor


def rel(actual, expected):
    return moe_oracle.max_rel_err(actual, expected)


def parameter(values):
    from gpu_util import to_device
    from qutai_b200.layers import Tensor

    values = np.asarray(values)
    return Tensor(to_device(values.reshape(-1), "float32"), values.shape, requires_grad=True)


def set_grad(p, gradient):
    from gpu_util import to_device
    from qutai_b200.layers import Tensor

    p.grad = None if gradient is None else Tensor(to_device(np.asarray(gradient).reshape(-1), "float32"), p.shape)


def test_adamw_matches_the_upstream_fixture_with_skipped_parameters():
    from gpu_util import to_host
    from qutai_b200.optim import AdamW

    f = np.load(os.path.join(GOLDEN, "optim_adamw.npz"))
    n, steps = int(f["tensors"]), int(f["steps"])
    parameters = [parameter(f[f"initial_{i}"]) for i in range(n)]
    optimizer = AdamW(parameters, learning_rate=float(f["learning_rate"]), betas=(float(f["beta1"]), float(f["beta2"])),
                      eps=float(f["eps"]), weight_decay=float(f["weight_decay"]))
    for step in range(steps):
        for i, p in enumerate(parameters):
            set_grad(p, f[f"grad_{step}_{i}"] if bool(f[f"has_grad_{step}_{i}"]) else None)
        optimizer.step()
        for i, p in enumerate(parameters):
            assert rel(to_host(p.storage, p.shape), f[f"values_{step}_{i}"]) <= 5 * FP32_TOL
            assert optimizer.steps.get(p, 0) == int(f[f"count_{step}_{i}"])
            if f"average_{step}_{i}" in f:
                assert rel(to_host(optimizer.averages[p], p.shape), f[f"average_{step}_{i}"]) <= FP32_TOL
                assert rel(to_host(optimizer.square_averages[p], p.shape), f[f"square_{step}_{i}"]) <= FP32_TOL
            else:
                assert p not in optimizer.averages


def test_adamw_many_ragged_tensors_views_and_bf16_shadows():
    from gpu_util import to_device, to_host
    from qutai_b200.layers import Tensor
    from qutai_b200.optim import AdamW
    from qutai_b200.storage import DeviceStorage

    rng = np.random.default_rng(5)
    sizes = [1, 3, 4097, 8192, 12289, 70001, 5, 4096 * 3 + 2]
    slab = to_device(rng.standard_normal(sum(sizes) + 1), "float32")
    parameters, offset = [], 1                      # views at odd offsets: not 16-byte aligned
    for size in sizes:
        parameters.append(Tensor(slab.view(offset, size), (size,), requires_grad=True))
        offset += size
    initial = [to_host(p.storage) for p in parameters]
    shadows = {p: DeviceStorage(p.storage.size, "bfloat16") for p in parameters[::2]}
    settings = dict(learning_rate=3e-3, betas=(0.8, 0.99), eps=1e-6, weight_decay=0.05)
    optimizer = AdamW(parameters, shadows=shadows, **settings)
    oracle = optim_oracle.AdamW(**settings)
    values = initial
    for step in range(4):
        gradients = [None if (step + i) % 5 == 0 else rng.standard_normal(size).astype(np.float32).astype(np.float64)
                     for i, size in enumerate(sizes)]
        for p, g in zip(parameters, gradients):
            set_grad(p, g)
        optimizer.step()
        values = oracle.step(values, gradients)
        for i, p in enumerate(parameters):
            got = to_host(p.storage)
            assert rel(got, values[i]) <= 5 * FP32_TOL, (step, i)
            assert optimizer.steps.get(p, 0) == oracle.steps.get(i, 0)
            if p in shadows and gradients[i] is not None:
                assert np.array_equal(to_host(shadows[p]), moe_oracle.round_bf16(got))   # exactly the rounded parameter


def test_adamw_rejects_bad_settings():
    from qutai_b200.optim import AdamW

    p = parameter(np.ones(8))
    for bad in (dict(learning_rate=-1.0), dict(eps=-1e-3), dict(weight_decay=-0.1), dict(betas=(1.0, 0.9)), dict(betas=(0.9,))):
        with pytest.raises(ValueError):
            AdamW([p], **bad)


def test_clip_grad_norm_matches_the_upstream_fixture():
    from gpu_util import to_host
    from qutai_b200.optim import clip_grad_norm

    f = np.load(os.path.join(GOLDEN, "optim_clip.npz"))
    n = int(f["tensors"])
    for name in ("above", "below"):
        parameters = [parameter(np.zeros(f[f"grad_{i}"].shape)) for i in range(n)]
        for i, p in enumerate(parameters):
            set_grad(p, f[f"grad_{i}"] if bool(f[f"{name}_has_{i}"]) else None)
        norm = clip_grad_norm(parameters, float(f[f"{name}_limit"]))
        assert abs(norm - float(f[f"{name}_norm"])) <= 1e-6 * norm
        for i, p in enumerate(parameters):
            if p.grad is not None:
                assert rel(to_host(p.grad.storage, p.shape), f[f"{name}_after_{i}"]) <= FP32_TOL


def test_clip_grad_norm_large_is_deterministic_and_matches_the_oracle():
    from gpu_util import to_host
    from qutai_b200.optim import clip_grad_norm

    rng = np.random.default_rng(9)
    gradients = [rng.standard_normal(size).astype(np.float32) for size in (3_000_001, 17, 1 << 20, 4095)]
    norms = []
    for _ in range(2):
        parameters = [parameter(np.zeros(g.shape)) for g in gradients]
        for p, g in zip(parameters, gradients):
            set_grad(p, g)
        norms.append(clip_grad_norm(parameters, 10.0))
        want_norm, want = optim_oracle.clip_grad_norm([g.astype(np.float64) for g in gradients], 10.0)
        assert abs(norms[-1] - want_norm) <= 1e-12 * want_norm     # double accumulation of exact fp32 squares
        for p, w in zip(parameters, want):
            assert rel(to_host(p.grad.storage), w) <= FP32_TOL
    assert norms[0] == norms[1]
    assert clip_grad_norm([parameter(np.zeros(4))], 1.0) == 0.0    # nothing has a gradient


def test_optimizer_keeps_the_layer_operands_current():
    """AdamW writing the bf16 operand copies: a layer that no longer converts its weights per forward gives the
    same bits as one that does."""
    from gpu_util import make_layer, to_device
    from qutai_b200.layers import Tensor
    from qutai_b200.optim import AdamW

    T, d, E, k, h = 600, 128, 6, 2, 256
    rng = np.random.default_rng(3)
    x, grad_y = moe_oracle.round_bf16(rng.standard_normal((T, d))), moe_oracle.round_bf16(rng.standard_normal((T, d)))
    router = rng.standard_normal((E, d)).astype(np.float32) * 0.05
    gate = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    up = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    down = rng.standard_normal((E, d, h)).astype(np.float32) / np.sqrt(h)
    outputs = []
    for fused in (False, True):
        layer = make_layer((T, d), router, gate, up, down, k, engine="tcgen05")
        xs, gs = Tensor(to_device(x, "bfloat16"), (T, d)), Tensor(to_device(grad_y, "bfloat16"), (T, d))
        layer(xs)                                   # builds the workspace and the operand copies
        optimizer = AdamW(layer.parameters(), learning_rate=1e-2, shadows=layer.operand_shadows() if fused else None)
        layer.refresh_operands = not fused
        for _ in range(3):
            optimizer.zero_grad()
            layer(xs)
            layer.backward(gs, None)
            optimizer.step()
        y, _ = layer(xs)
        outputs.append(y.storage.tobytes())
    assert outputs[0] == outputs[1]


def test_operand_copies_are_rebuilt_only_after_a_weight_was_written():
    """``refresh_operands = "auto"`` (the default): a forward converts the fp32 weights to their bf16 operand
    copies only when a weight storage was written since the copies were made (optimizer step, upload).  The bits
    are those of a layer that converts at every forward, and a forward on unchanged weights launches three
    kernels fewer (the three conversions)."""
    from gpu_util import make_layer, to_device
    from qutai_b200 import lib
    from qutai_b200.layers import Tensor
    from qutai_b200.optim import AdamW

    T, d, E, k, h = 300, 64, 4, 2, 128
    rng = np.random.default_rng(17)
    x, grad_y = moe_oracle.round_bf16(rng.standard_normal((T, d))), moe_oracle.round_bf16(rng.standard_normal((T, d)))
    router = rng.standard_normal((E, d)).astype(np.float32) * 0.05
    gate = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    up = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    down = rng.standard_normal((E, d, h)).astype(np.float32) / np.sqrt(h)
    new_up = (rng.standard_normal((h, d)) / np.sqrt(d)).astype(np.float32)
    count = lib.load().qmoe_launch_count
    outputs, launches = [], []
    for mode in (True, "auto"):
        layer = make_layer((T, d), router, gate, up, down, k, engine="tcgen05")
        assert layer.refresh_operands == "auto"
        layer.refresh_operands = mode
        xs, gs = Tensor(to_device(x, "bfloat16"), (T, d)), Tensor(to_device(grad_y, "bfloat16"), (T, d))
        seen, per_forward = [], []

        def forward():
            before = count()
            y, _ = layer(xs)
            per_forward.append(count() - before)
            seen.append(y.storage.tobytes())

        forward()                                             # builds the copies
        forward()                                             # nothing was written in between
        optimizer = AdamW(layer.parameters(), learning_rate=1e-2)   # no shadows: the step only writes the fp32 weights
        optimizer.zero_grad()
        layer.backward(gs, None)
        optimizer.step()
        forward()                                             # after an optimizer step
        forward()
        layer.experts[1].up.weight.storage.upload_bytes(new_up.tobytes())   # through a view of the stacked buffer
        forward()                                             # after an upload
        shadowed = AdamW(layer.parameters(), learning_rate=1e-2, shadows=layer.operand_shadows())
        shadowed.zero_grad()
        layer.backward(gs, None)
        shadowed.step()                                       # writes weights and copies together
        forward()
        outputs.append(seen)
        launches.append(per_forward)
    assert outputs[0] == outputs[1]
    always, auto = launches
    assert len(set(always)) == 1                              # the forced layer converts every time
    full = always[0]
    assert auto == [full, full - 3, full, full - 3, full, full - 3], (always, auto)
