"""The routing entry point that needs no caller-allocated scratch (``qmoe_route_static``).

It exists for hosts that cannot allocate device memory themselves — a serving loop that must not
call cudaMalloc while handling a request, or a plug-in that only has the buffers it was given at
start-up — and keeps its three scratch tables in an array built into the library.  The checks
here: called through the C ABI it fills every output table exactly as ``qmoe_route`` does, on two
calls in a row (the second on different scores, so nothing left over from the first may leak
through the shared array), and it refuses problems larger than the built-in array.

This file is named so that pytest collects it last.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TABLES = ("probs", "gate_weights", "expert_index", "dest_row", "row_source", "counts", "offsets",
          "tile_expert", "meta", "utilization", "aux")


def _run(entry, scores, top_k, with_scratch):
    from gpu_util import RouteTables, to_device
    from qutai_b200 import lib

    T, E = scores.shape
    tables = RouteTables(T, E, top_k)
    if not with_scratch:  # the static variant must not need (or touch) caller scratch
        tables.struct.block_counts = tables.struct.block_base = tables.struct.block_colsum = 0
    for name in ("tile_expert", "row_source"):  # entries past the used range are never written: make them comparable
        lib.call("qmoe_memset", tables.buf[name].ptr, 0, tables.buf[name].nbytes, 0)
    scores_dev = to_device(scores, "float32")  # kept alive by name until the call has been made
    lib.call(entry, tables.ref, scores_dev.ptr, 0)
    return {name: tables.host(name) for name in TABLES}


def test_static_scratch_routing_matches_the_allocating_entry_point_twice_in_a_row():
    rng = np.random.default_rng(42)
    first = rng.standard_normal((3000, 64)).astype(np.float32)
    second = (rng.standard_normal((777, 8)) * 3).astype(np.float32)  # other shape, other values
    for scores, top_k in ((first, 6), (second, 2)):
        got = _run("qmoe_route_static", scores, top_k, with_scratch=False)
        want = _run("qmoe_route", scores, top_k, with_scratch=True)
        for name in TABLES:
            used = slice(None)
            if name == "row_source":
                used = slice(0, int(want["meta"][0]))
            elif name == "tile_expert":
                used = slice(0, int(want["meta"][1]))
            assert np.array_equal(got[name][used], want[name][used]), name  # same kernels: bit-identical


def test_static_scratch_routing_rejects_sizes_beyond_the_built_in_array():
    from gpu_util import RouteTables, to_device
    from qutai_b200 import lib

    T, E = 32 * 513, 256  # 513 blocks x 256 experts > 131072 entries
    tables = RouteTables(T, E, 2)
    scores = to_device(np.zeros((1, 1)), "float32")  # never read: the call must fail before any launch
    with pytest.raises(ValueError, match="exceed the built-in"):
        lib.call("qmoe_route_static", tables.ref, scores.ptr, 0)


def test_a_route_filled_without_caller_scratch_feeds_the_other_entry_points():
    """A host that could not allocate the scratch tables still has to permute, combine and run the routing
    backward with the struct the static variant filled: those calls must accept the three scratch fields left
    at 0 and give the bits they give for a route filled by ``qmoe_route``."""
    from gpu_util import RouteTables, to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.storage import DeviceStorage

    rng = np.random.default_rng(7)
    T, E, k, d = 500, 8, 2, 64
    scores = to_device(rng.standard_normal((T, E)).astype(np.float32), "float32")
    x = to_device(rng.standard_normal((T, d)).astype(np.float32), "float32")
    grad_w = to_device(rng.standard_normal((T, k)).astype(np.float32), "float32")
    results = []
    for entry, with_scratch in (("qmoe_route_static", False), ("qmoe_route", True)):
        tables = RouteTables(T, E, k)
        if not with_scratch:
            tables.struct.block_counts = tables.struct.block_base = tables.struct.block_colsum = 0
        lib.call(entry, tables.ref, scores.ptr, 0)
        R = tables.rows_bound
        # rows past the last expert group are never written: start them equal on both sides
        dispatched, out = DeviceStorage.zeros(R * d, "float32"), DeviceStorage(T * d, "float32")
        dy, dw = DeviceStorage.zeros(R * d, "float32"), DeviceStorage(T * k, "float32")
        back, d_scores = DeviceStorage(T * d, "float32"), DeviceStorage(T * E, "float32")
        lib.call("qmoe_permute", tables.ref, x.ptr, dispatched.ptr, lib.QMOE_F32, d, 0)
        lib.call("qmoe_combine", tables.ref, dispatched.ptr, out.ptr, lib.QMOE_F32, d, 0)
        lib.call("qmoe_combine_backward", tables.ref, x.ptr, dispatched.ptr, dy.ptr, dw.ptr, lib.QMOE_F32, d, 0)
        lib.call("qmoe_unpermute_reduce", tables.ref, dy.ptr, 0, back.ptr, lib.QMOE_F32, d, 0)
        lib.call("qmoe_route_backward", tables.ref, grad_w.ptr, 0, d_scores.ptr, 0)
        results.append([to_host(s) for s in (dispatched, out, dy, dw, back, d_scores)])
        if not with_scratch:  # the statistics packer reads the column sums out of the scratch: it has to say so
            stats = DeviceStorage(2 * E, "int32")
            with pytest.raises(ValueError, match="block_colsum"):
                lib.call("qmoe_ep_pack_stats", tables.ref, stats.ptr, 0)
    for got, want in zip(*results):
        assert np.array_equal(got, want)
    assert lib.device_status() == 0
