"""Child process of the 2-rank CPU test: runs the dispatch and combine exchanges of the
expert-parallel plan over torch.distributed (gloo) on CPU tensors and checks them against the
oracle's global routing.  Usage: python ep_gloo_worker.py RANK WORLD PORT"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import moe_oracle as oracle  # noqa: E402
from qutai_b200.expert_parallel import plan_exchange  # noqa: E402


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    T, d, E, k = 96, 8, 4, 2
    rng = np.random.default_rng(3)
    x = rng.standard_normal((T, d))
    scores = rng.standard_normal((T, E)) + np.array([1.0, 0.0, -0.5, 0.3])
    shard = slice(rank * T // world, (rank + 1) * T // world)
    local = oracle.routing(scores[shard], k)
    mine = torch.tensor(local["counts"], dtype=torch.int64)
    gathered = [torch.zeros(E, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(gathered, mine)                       # the count exchange
    counts = [g.tolist() for g in gathered]
    plan = plan_exchange(counts, rank, world, pad=4)
    send = np.zeros((plan["send_offsets"][-1], d))
    for e in range(E):
        send[plan["send_offsets"][e]: plan["send_offsets"][e] + local["counts"][e]] = oracle.route_gather(x[shard], local, e)
    send_t, recv_t = torch.from_numpy(send), torch.zeros((max(1, plan["expert_offsets"][-1]), d), dtype=torch.float64)

    def exchange(src, sends, dst, recvs):
        # gloo has no channel from a rank to itself: pair those segments locally, in list order
        # (NCCL, which the product uses, handles them inside the group)
        own_out = [seg for seg in sends if seg[0] == rank]
        own_in = [seg for seg in recvs if seg[0] == rank]
        for (_, so, rows), (_, ro, _) in zip(own_out, own_in):
            dst[ro: ro + rows] = src[so: so + rows]
        ops = []
        for peer, off, rows in sends:
            if peer != rank:
                ops.append(dist.P2POp(dist.isend, src[off: off + rows].contiguous(), peer))
        bufs = []
        for peer, off, rows in recvs:
            if peer == rank:
                continue
            buf = torch.empty((rows, d), dtype=torch.float64)
            bufs.append((off, rows, buf))
            ops.append(dist.P2POp(dist.irecv, buf, peer))
        for work in dist.batch_isend_irecv(ops):
            work.wait()
        for off, rows, buf in bufs:
            dst[off: off + rows] = buf

    exchange(send_t, plan["sends"], recv_t, plan["recvs"])
    full = oracle.routing(scores, k)                      # what one GPU would have built
    local_experts = E // world
    for j in range(local_experts):
        e = rank * local_experts + j
        rows = recv_t[plan["expert_offsets"][j]: plan["expert_offsets"][j] + plan["expert_counts"][j]].numpy()
        assert plan["expert_counts"][j] == full["counts"][e]
        assert np.array_equal(rows, oracle.route_gather(x, full, e)), f"rank {rank}: expert {e} rows are not in global order"
    # combine direction: send every row back (times 2) and check it lands where it came from
    back = torch.zeros_like(send_t)
    exchange(recv_t * 2, plan["recvs"], back, plan["sends"])
    for e in range(E):
        o, c = plan["send_offsets"][e], local["counts"][e]
        assert np.array_equal(back[o: o + c].numpy(), 2 * send[o: o + c])
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok")


if __name__ == "__main__":
    main()
