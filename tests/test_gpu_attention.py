"""Causal self-attention with grouped key/value heads (``qutai_b200.attention`` over ``qmoe_attention_forward`` /
``_backward``, tcgen05, head width 64, bf16) against the fixtures the upstream CPU backend produced, against the oracle
on other shapes (sequence lengths that are not multiples of the 128-position block, one and many blocks, key/value
groups of 1, 2 and 4 heads), and at the size of the full decoder step through sampled heads.  Needs a B200: ``-m gpu``."""
import os
import sys

import numpy as np
import pytest

from conftest import golden_files
from oracle import moe_oracle as oracle

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from attention_inputs import attention_inputs  # noqa: E402

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2              # max |a - b| / max |b| per tensor (the bar of the layer's bf16 outputs and gradients)
BF16_ELEMENT_TOL = 0.08      # |x - y| <= 0.08 max(rms(y), |y|)


def run_attention(q, k, v, grad, heads, kv_heads):
    from gpu_util import to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.attention import attention
    from qutai_b200.layers import Tensor

    tensors = [Tensor(to_device(a, "bfloat16"), a.shape) for a in (q, k, v)]
    out = attention(*tensors, heads, kv_heads)
    assert out.parents == tuple(tensors)
    dq, dk, dv = out.backward_rule(to_device(grad, "bfloat16"))
    assert lib.device_status() == 0
    return dict(out=to_host(out.storage, q.shape), dq=to_host(dq, q.shape), dk=to_host(dk, k.shape), dv=to_host(dv, v.shape))


def check(got, want, element_tol=BF16_ELEMENT_TOL):
    for name in ("out", "dq", "dk", "dv"):
        if not np.any(want[name]):        # a single position: the gradients of q and k are exactly zero upstream
            assert np.abs(got[name]).max() <= 1e-6, name
            continue
        assert oracle.max_rel_err(got[name], want[name]) <= BF16_TOL, name
        assert oracle.elementwise_err(got[name], want[name], bf16=True, unit=oracle.rms(want[name])) <= element_tol, name


@pytest.mark.parametrize("path", golden_files("attention"), ids=os.path.basename)
def test_attention_matches_the_upstream_fixture(path):
    g = np.load(path)
    heads, kv_heads = int(g["heads"]), int(g["kv_heads"])
    q, k, v, grad = attention_inputs(int(g["batch"]), int(g["time"]), heads, kv_heads, int(g["seed"]), float(g["scale"]))
    got = run_attention(q, k, v, grad, heads, kv_heads)
    check(got, g)
    again = run_attention(q, k, v, grad, heads, kv_heads)
    for name in ("out", "dq", "dk", "dv"):                 # no atomics anywhere: the same bits on every run
        assert np.array_equal(again[name], got[name]), name


@pytest.mark.parametrize("batch,time,heads,kv_heads", [(1, 128, 1, 1), (2, 129, 2, 1), (1, 256, 4, 1), (3, 300, 4, 2),
                                                       (1, 1000, 2, 2), (2, 64, 8, 2)])
def test_attention_matches_the_oracle(batch, time, heads, kv_heads):
    q, k, v, grad = attention_inputs(batch, time, heads, kv_heads, seed=time * 7 + heads, scale=0.8)
    out, lse = oracle.attention_forward(q, k, v, heads, kv_heads)
    dq, dk, dv = oracle.attention_backward(grad, q, k, v, out, lse, heads, kv_heads)
    check(run_attention(q, k, v, grad, heads, kv_heads), dict(out=out, dq=dq, dk=dk, dv=dv))


def test_attention_at_the_size_of_the_decoder_step():
    """4 sequences of 2048 positions, 16 heads in 4 key/value groups (one rank's share of the full decoder step):
    two sampled sequences x key/value groups against the oracle (a group's heads depend on nothing else).  The
    tensor-wide bar is the usual 2e-2; the element-wise one is 0.2 of the tensor's root mean square here: over 2048
    keys dS = P (dP - delta) loses digits where dP and delta (formed from the bf16 output) nearly cancel, and the
    worst of two million elements was 0.11."""
    batch, time, heads, kv_heads, dim = 4, 2048, 16, 4, 64
    q, k, v, grad = attention_inputs(batch, time, heads, kv_heads, seed=99, scale=0.6)
    got = run_attention(q, k, v, grad, heads, kv_heads)
    group = heads // kv_heads
    for b, g in ((0, 0), (3, 2)):
        wide = slice(g * group * dim, (g + 1) * group * dim)
        narrow = slice(g * dim, (g + 1) * dim)
        qs, ks, vs, gs = q[b:b + 1, :, wide], k[b:b + 1, :, narrow], v[b:b + 1, :, narrow], grad[b:b + 1, :, wide]
        out, lse = oracle.attention_forward(qs, ks, vs, group, 1)
        dq, dk, dv = oracle.attention_backward(gs, qs, ks, vs, out, lse, group, 1)
        check(dict(out=got["out"][b:b + 1, :, wide], dq=got["dq"][b:b + 1, :, wide], dk=got["dk"][b:b + 1, :, narrow],
                   dv=got["dv"][b:b + 1, :, narrow]), dict(out=out, dq=dq, dk=dk, dv=dv), element_tol=0.2)


def test_attention_rejects_what_it_does_not_cover():
    from gpu_util import to_device
    from qutai_b200.attention import attention
    from qutai_b200.layers import Tensor

    q = Tensor(to_device(np.zeros((1, 4, 64)), "bfloat16"), (1, 4, 64))
    kv = Tensor(to_device(np.zeros((1, 4, 64)), "bfloat16"), (1, 4, 64))
    with pytest.raises(ValueError):
        attention(q, kv, kv, 2, 1)                      # head width 32
    q32 = Tensor(to_device(np.zeros((1, 4, 64)), "float32"), (1, 4, 64))
    with pytest.raises(ValueError):
        attention(q32, kv, kv, 1, 1)                    # float32
    q3 = Tensor(to_device(np.zeros((1, 4, 192)), "bfloat16"), (1, 4, 192))
    kv2 = Tensor(to_device(np.zeros((1, 4, 128)), "bfloat16"), (1, 4, 128))
    with pytest.raises(ValueError):
        attention(q3, kv2, kv2, 3, 2)                   # heads not a multiple of kv_heads
