"""Child process of the expert-parallel GPU test: one rank = one GPU (picked through
CUDA_VISIBLE_DEVICES by the parent).  Runs forward + backward of ExpertParallelMoE on this rank's
token shard and writes its results to OUT/rank{r}.npz for the parent to check against the oracle.
Usage: python ep_gpu_worker.py RANK WORLD OUT_DIR TRANSPORT [PLACEMENT]

PLACEMENT: "contiguous" (default), "interleaved" (expert e on rank e % world) or "rebalanced" (built
contiguous, then moved to the interleaved placement with ``rebalance``, weights travelling over NCCL)."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def problem():
    T, d, E, k, h = 768, 128, 8, 2, 256
    rng = np.random.default_rng(21)
    bf = lambda a: (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) & 0xFFFF0000).view(np.float32).astype(np.float64)
    x, grad = bf(rng.standard_normal((T, d))), bf(rng.standard_normal((T, d)))
    router = (rng.standard_normal((E, d)) * 0.05).astype(np.float32)
    router[:, -1] += np.linspace(-0.6, 0.6, E).astype(np.float32)  # skewed load
    x[:, -1] = 1.0
    gate = (rng.standard_normal((E, h, d)) / np.sqrt(d)).astype(np.float32)
    up = (rng.standard_normal((E, h, d)) / np.sqrt(d)).astype(np.float32)
    down = (rng.standard_normal((E, d, h)) / np.sqrt(h)).astype(np.float32)
    return dict(T=T, d=d, E=E, k=k, h=h, x=x, grad=grad, router=router, gate=gate, up=up, down=down, grad_aux=0.25)


def main():
    rank, world, out_dir, transport = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    placement_kind = sys.argv[5] if len(sys.argv) > 5 else "contiguous"
    engine, overlap = "tcgen05", False
    if transport.endswith("-simt"):  # the direct transport without the fused tensor-core producers
        transport, engine = transport[:-5], "simt"
    if transport.endswith("-overlap"):  # the fused direct transport with the two-phase overlap of push and first product
        transport, overlap = transport[:-8], True
    from gpu_util import Config, to_device, to_host
    from qutai_b200 import lib
    from qutai_b200.expert_parallel import ExpertParallelMoE, file_all_gather, finalize_communicator, init_communicator
    from qutai_b200.layers import Tensor

    if transport == "p2p":  # every GPU of the job is visible to every rank; pick ours
        lib.call("qmoe_set_device", rank)

    p = problem()
    T, d, E, k, h = p["T"], p["d"], p["E"], p["k"], p["h"]
    init_communicator(rank, world, rendezvous_path=os.path.join(out_dir, "nccl_id"), timeout=120)
    interleaved = [e % world for e in range(E)]
    exchanges = iter(range(100))   # a tag of its own for every exchange of IPC handles (a rebuilt workspace makes a second one)
    layer = ExpertParallelMoE(Config(d, E, k, h), rank=rank, world=world, seed=3, engine=engine, transport=transport,
                              placement=interleaved if placement_kind == "interleaved" else None, overlap=overlap,
                              gather=lambda data: file_all_gather(out_dir, f"ipc{next(exchanges)}", rank, world, data))
    mine = list(layer.expert_ids)   # the model's numbers of this rank's experts, in slot order
    layer.router.weight.storage.upload_bytes(p["router"].tobytes())
    layer._gate.upload_bytes(np.ascontiguousarray(p["gate"][mine]).tobytes())
    layer._up.upload_bytes(np.ascontiguousarray(p["up"][mine]).tobytes())
    layer._down.upload_bytes(np.ascontiguousarray(p["down"][mine]).tobytes())
    if placement_kind == "rebalanced":
        assert layer.rebalance(placement=interleaved) == tuple(interleaved)
        moved = list(layer.expert_ids)
        assert moved == [e for e in range(E) if e % world == rank]
        assert np.array_equal(to_host(layer._gate, (len(moved), h, d)), p["gate"][moved].astype(np.float64))
        assert np.array_equal(to_host(layer._down, (len(moved), d, h)), p["down"][moved].astype(np.float64))
        names = [name for name, _ in layer.named_expert_parameters()]
        assert names[:3] == [f"experts.{moved[0]}.{kind}.weight" for kind in ("gate", "up", "down")]
    shard = slice(rank * T // world, (rank + 1) * T // world)
    Tl = T // world
    results = {}
    for attempt in range(2):  # twice: the second pass must reproduce the first bit for bit
        for parameter in layer.parameters():
            parameter.grad = None
        y, aux = layer(Tensor(to_device(p["x"][shard], "bfloat16"), (Tl, d)))
        dx = layer.backward(Tensor(to_device(p["grad"][shard], "bfloat16"), (Tl, d)), p["grad_aux"])
        work = layer._saved[0]
        out = dict(y=to_host(y.storage, (Tl, d)), aux=to_host(aux.storage), dx=to_host(dx.storage, (Tl, d)),
                   # the workspace keeps the logits in the layer's internal (physical) expert order
                   scores=to_host(work["buf"]["scores"], (Tl, E))[:, list(layer._physical_of_logical)],
                   counts=np.array(layer.last_counts),
                   utilization=to_host(layer.utilization.storage),
                   d_router=to_host(layer.router.weight.grad.storage, (E, d)))
        has = []
        for e, expert in zip(layer.expert_ids, layer.experts):   # keyed by the model's expert number
            has.append(expert.gate.weight.grad is not None)
            if has[-1]:
                out[f"d_gate_{e}"] = to_host(expert.gate.weight.grad.storage, (h, d))
                out[f"d_up_{e}"] = to_host(expert.up.weight.grad.storage, (h, d))
                out[f"d_down_{e}"] = to_host(expert.down.weight.grad.storage, (d, h))
        out["has_grad"] = np.array(has)
        out["expert_ids"] = np.array(layer.expert_ids)
        results[attempt] = out
    for key, value in results[0].items():
        assert np.array_equal(value, results[1][key]), f"rank {rank}: {key} differs between two identical steps"
    assert lib.device_status() == 0
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **results[0])
    finalize_communicator()
    print(f"rank {rank} done")


if __name__ == "__main__":
    main()
