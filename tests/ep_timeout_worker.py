"""Child process of the failure-detection test of the expert-parallel layer: one GPU, one rank, whose flag
barrier is told about a second rank that does not exist (a flag array nobody writes to).  The barrier's
bounded wait runs out, the kernel reports a status, and the layer must turn that into an exception where the
host next looks at the step — no GPU is faulted or hung.  Usage: python ep_timeout_worker.py OUT_DIR"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def main():
    out_dir = sys.argv[1]
    from gpu_util import Config, to_device
    from qutai_b200 import lib
    from qutai_b200.expert_parallel import ExpertParallelMoE, finalize_communicator, init_communicator
    from qutai_b200.layers import Tensor
    from qutai_b200.storage import DeviceStorage

    init_communicator(0, 1, rendezvous_path=os.path.join(out_dir, "nccl_id"), timeout=60)
    T, d, E, k, h = 256, 64, 4, 2, 128
    layer = ExpertParallelMoE(Config(d, E, k, h), rank=0, world=1, seed=5, gather=lambda data: [data])
    rng = np.random.default_rng(0)
    x = Tensor(to_device(rng.standard_normal((T, d)), "bfloat16"), (T, d))
    g = Tensor(to_device(rng.standard_normal((T, d)), "bfloat16"), (T, d))
    layer(x)
    layer.backward(g, 0.1)
    layer.check_status()                       # a healthy step: nothing to report
    # from here on the barrier believes in a rank 1 whose flags nobody ever raises
    lib.call("qmoe_ep_set_barrier_timeout_ms", 300)
    absent, absent_stats = DeviceStorage.zeros(16, "int32"), DeviceStorage.zeros(4 * E, "int32")
    flags, stats = layer._work["peers"]["flags"], layer._work["peers"]["stats_all"]
    flags.world = stats.world = 2
    flags.buffer[1], stats.buffer[1] = absent.ptr, absent_stats.ptr
    layer(x)
    try:
        layer.backward(g, 0.1)                 # reads the counts, and with them the status the barrier left
    except RuntimeError as error:
        assert "barrier" in str(error) and "201" in str(error), error
        print("raised in backward")
    else:
        raise AssertionError("a step whose barrier timed out returned without an error")
    try:
        layer.check_status()
    except RuntimeError:
        print("raised in check_status")
    else:
        raise AssertionError("check_status did not report the failed barrier")
    # the context is still usable once the cause is gone and the status is cleared
    flags.world = stats.world = 1
    lib.call("qmoe_device_status_clear", 0)
    layer._work["host_status"][0] = layer._work["host_status"][1] = 0
    layer(x)
    layer.backward(g, 0.1)
    layer.check_status()
    finalize_communicator()
    print("timeout worker done")


if __name__ == "__main__":
    main()
