"""The forward recorded as a CUDA graph (``SparseMoE.capture_forward``) gives the bits of the call-by-call
forward, follows new contents of its input buffer, and leaves the layer ready for a backward."""
import ctypes

import numpy as np
import pytest

from oracle import moe_oracle as oracle

pytestmark = pytest.mark.gpu


def _layer_on_its_own_stream(T, d, E, k, h, seed):
    from gpu_util import make_layer
    from qutai_b200 import lib

    rng = np.random.default_rng(seed)
    router = rng.standard_normal((E, d)).astype(np.float32) * 0.05
    gate = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    up = rng.standard_normal((E, h, d)).astype(np.float32) / np.sqrt(d)
    down = rng.standard_normal((E, d, h)).astype(np.float32) / np.sqrt(h)
    layer = make_layer((T, d), router, gate, up, down, k, engine="tcgen05")
    stream = ctypes.c_uint64()
    lib.call("qmoe_stream_create", ctypes.byref(stream))
    lib.call("qmoe_stream_sync", 0)          # the uploads above ran on the default stream
    layer.stream = stream.value
    return layer, rng


def test_capture_needs_a_stream_of_its_own():
    from gpu_util import make_layer, to_device
    from qutai_b200.layers import Tensor

    rng = np.random.default_rng(0)
    layer = make_layer((8, 64), rng.standard_normal((4, 64)).astype(np.float32), rng.standard_normal((4, 64, 64)).astype(np.float32),
                       rng.standard_normal((4, 64, 64)).astype(np.float32), rng.standard_normal((4, 64, 64)).astype(np.float32), 2)
    with pytest.raises(ValueError):
        layer.capture_forward(Tensor(to_device(np.zeros((8, 64)), "bfloat16"), (8, 64)))


@pytest.mark.parametrize("T,d,E,k,h", [(64, 256, 8, 2, 512), (200, 128, 16, 4, 264)])
def test_replayed_forward_matches_the_eager_forward_bit_for_bit(T, d, E, k, h):
    from gpu_util import bf16_bytes, to_device
    from qutai_b200 import lib
    from qutai_b200.layers import Tensor

    layer, rng = _layer_on_its_own_stream(T, d, E, k, h, seed=T + d)
    sync = lambda: (lib.call("qmoe_stream_sync", layer.stream), lib.call("qmoe_stream_sync", 0))
    first, second = oracle.round_bf16(rng.standard_normal((T, d))), oracle.round_bf16(rng.standard_normal((T, d)))
    grad = Tensor(to_device(oracle.round_bf16(rng.standard_normal((T, d))), "bfloat16"), (T, d))
    x = Tensor(to_device(first, "bfloat16"), (T, d))
    sync()
    for refresh in (True, False):
        layer.refresh_operands = refresh
        graph = layer.capture_forward(x)
        for values in (first, second):
            x.storage.upload_bytes(bf16_bytes(values))
            sync()
            y_eager, aux_eager = layer(x)
            sync()
            want = (y_eager.storage.tobytes(), aux_eager.storage.tobytes(), layer.last_counts)
            dx_eager = layer.backward(grad, None)
            sync()
            want_dx = dx_eager.storage.tobytes()
            y, aux = graph.replay()
            assert layer.last_counts == want[2] and sum(want[2]) == T * k     # read through the stream
            sync()
            assert (y.storage.tobytes(), aux.storage.tobytes()) == want[:2]
            dx = layer.backward(grad, None)                                   # the replay left what backward needs
            sync()
            assert dx.storage.tobytes() == want_dx
        assert lib.device_status(layer.stream) == 0
