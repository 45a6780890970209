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
