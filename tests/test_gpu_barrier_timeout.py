"""Failure detection of the peer-memory barrier, without faulting or hanging the GPU: a barrier
whose partner never arrives (its flag is simply never set) must give up after its bounded wait,
report a status the host can read, and leave the context usable."""
import ctypes
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_flag_barrier_gives_up_when_a_rank_never_arrives():
    from gpu_util import to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.storage import DeviceStorage

    assert lib.device_status() == 0
    lib.call("qmoe_ep_set_barrier_timeout_ms", 1000)             # the default (10 s) is sized for training jobs
    mine, absent = DeviceStorage.zeros(16, "int32"), DeviceStorage.zeros(16, "int32")
    flags = lib.Peers()
    flags.world, flags.rank = 2, 0
    flags.buffer[0], flags.buffer[1] = mine.ptr, absent.ptr     # "rank 1" is memory nobody writes to
    start = time.monotonic()
    lib.call("qmoe_ep_flag_barrier", ctypes.byref(flags), 1, 0, 0, None, 0)
    status = lib.device_status()                                 # waits for the kernel
    elapsed = time.monotonic() - start
    assert status == 201, "the barrier must report that a rank never arrived"
    assert 0.5 < elapsed < 10, f"the wait is bounded to about a second (took {elapsed:.2f} s)"
    assert to_host(absent)[0] == 1 and to_host(mine)[0] == 1     # our own arrival was published to both arrays
    lib.call("qmoe_device_status_clear", 0)
    assert lib.device_status() == 0
    # the context is still usable: a barrier whose partner HAS arrived passes immediately
    absent_arrived = to_device(np.array([0, 2] + [0] * 14), "int32")
    lib.call("qmoe_memcpy_d2d", mine.ptr + 4, absent_arrived.ptr + 4, 4, 0)
    start = time.monotonic()
    lib.call("qmoe_ep_flag_barrier", ctypes.byref(flags), 2, 0, 0, None, 0)
    assert lib.device_status() == 0 and time.monotonic() - start < 0.5
    lib.call("qmoe_ep_set_barrier_timeout_ms", 10000)


def test_layer_raises_when_a_barrier_of_its_step_timed_out(tmp_path):
    """The expert-parallel layer surfaces the barrier's status: a step during which a rank never arrived raises
    instead of handing back rows that were read before their owners wrote them (child process: the layer needs
    a communicator of its own)."""
    import os
    import subprocess
    import sys

    here = os.path.dirname(os.path.abspath(__file__))
    proc = subprocess.run([sys.executable, os.path.join(here, "ep_timeout_worker.py"), str(tmp_path)],
                          capture_output=True, text=True, timeout=240)
    out = proc.stdout + proc.stderr
    assert proc.returncode == 0, out[-3000:]
    assert "raised in backward" in out and "raised in check_status" in out and "timeout worker done" in out, out[-3000:]
