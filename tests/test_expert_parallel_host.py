"""Host-side logic of the expert-parallel layer, on CPU: the exchange plan (in-process with 1, 2,
4 and 8 simulated ranks, and over torch.distributed/gloo with 2 real ranks), and the rendezvous
time-out that reports a rank that never arrives."""
import os
import socket
import subprocess
import sys
import time

import numpy as np
import pytest

from oracle import moe_oracle as oracle
from qutai_b200.expert_parallel import file_rendezvous, padded_offsets, plan_exchange

HERE = os.path.dirname(os.path.abspath(__file__))


def test_padded_offsets():
    assert padded_offsets([0, 1, 128, 129]) == [0, 0, 128, 256, 512]
    assert padded_offsets([3, 4], pad=4) == [0, 4, 8]


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_plan_reproduces_the_global_token_slot_order(world):
    T, d, E, k = 64 * world, 4, 8, 3
    rng = np.random.default_rng(world)
    x = rng.standard_normal((T, d))
    scores = np.round(rng.standard_normal((T, E)) * 2) / 2 + rng.standard_normal(E)  # ties and skew
    full = oracle.routing(scores, k)
    shards = [slice(p * T // world, (p + 1) * T // world) for p in range(world)]
    local = [oracle.routing(scores[s], k) for s in shards]
    counts = [list(r["counts"]) for r in local]
    plans = [plan_exchange(counts, p, world, pad=8) for p in range(world)]
    send = []
    for p in range(world):
        buf = np.zeros((plans[p]["send_offsets"][-1], d))
        for e in range(E):
            o = plans[p]["send_offsets"][e]
            buf[o: o + counts[p][e]] = oracle.route_gather(x[shards[p]], local[p], e)
        send.append(buf)
    # deliver: between a pair of ranks the i-th send matches the i-th receive
    recv = [np.full((max(1, plans[p]["expert_offsets"][-1]), d), np.nan) for p in range(world)]
    for src in range(world):
        for dst in range(world):
            outgoing = [seg for seg in plans[src]["sends"] if seg[0] == dst]
            incoming = [seg for seg in plans[dst]["recvs"] if seg[0] == src]
            assert [s[2] for s in outgoing] == [r[2] for r in incoming]
            for (_, so, rows), (_, ro, _) in zip(outgoing, incoming):
                recv[dst][ro: ro + rows] = send[src][so: so + rows]
    L = E // world
    for p in range(world):
        assert all(o % 8 == 0 for o in plans[p]["expert_offsets"])
        for j in range(L):
            e = p * L + j
            o, c = plans[p]["expert_offsets"][j], plans[p]["expert_counts"][j]
            assert c == full["counts"][e]
            assert np.array_equal(recv[p][o: o + c], oracle.route_gather(x, full, e))
    assert sum(sum(pl["expert_counts"]) for pl in plans) == T * k


def test_plan_rejects_uneven_expert_split():
    with pytest.raises(ValueError):
        plan_exchange([[1, 2, 3]], 0, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gloo_ranks_exchange_in_global_order():
    port = str(_free_port())
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "ep_gloo_worker.py"), str(r), "2", port],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outputs = []
    for proc in procs:
        try:
            out, _ = proc.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            proc.kill()
            out, _ = proc.communicate()
        outputs.append(out)
    for r, (proc, out) in enumerate(zip(procs, outputs)):
        assert proc.returncode == 0 and f"rank {r} ok" in out, out[-2000:]


def test_rendezvous_times_out_when_rank_zero_never_arrives(tmp_path):
    start = time.monotonic()
    with pytest.raises(TimeoutError, match="rank 1"):
        file_rendezvous(str(tmp_path / "missing"), 1, timeout=0.3)
    assert time.monotonic() - start < 5
    path = str(tmp_path / "id")
    assert file_rendezvous(path, 0, b"x" * 128) == b"x" * 128
    assert file_rendezvous(path, 1, timeout=1.0) == b"x" * 128


def test_repeated_file_exchanges_never_hand_back_an_older_payload(tmp_path):
    """Two all-gathers in a row through the same directory, one rank lagging a whole exchange behind: the fast
    rank's second gather must wait for the slow rank's SECOND payload, not pick up its first one again."""
    import threading

    from qutai_b200.expert_parallel import FileExchange

    world, results = 3, {}

    def rank_main(rank):
        exchange = FileExchange(str(tmp_path), "ipc_job", rank, world, timeout=20.0)
        got = []
        for round_number in (1, 2):
            if rank == 2:
                time.sleep(0.4)            # always late: the others finish a round long before it publishes
            got.append(exchange.all_gather(f"rank{rank}-round{round_number}".encode()))
        results[rank] = (got, exchange)

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
    for rank in range(world):
        got, _ = results[rank]
        for round_number, payloads in zip((1, 2), got):
            assert payloads == [f"rank{p}-round{round_number}".encode() for p in range(world)]
    for rank in range(world):
        results[rank][1].close()
    assert not [name for name in os.listdir(tmp_path) if name.startswith("ipc_job")]   # every rank removed its own files


def test_placement_maps_and_parameter_names():
    from qutai_b200.expert_parallel import balanced_placement, contiguous_placement, physical_numbering

    assert contiguous_placement(8, 4) == [0, 0, 1, 1, 2, 2, 3, 3]
    counts = [900, 100, 800, 200, 700, 300, 600, 400]
    placement = balanced_placement(counts, 4)
    loads = [sum(c for c, p in zip(counts, placement) if p == r) for r in range(4)]
    assert sorted(placement) == [0, 0, 1, 1, 2, 2, 3, 3] and loads == [1000] * 4     # LPT pairs large with small
    physical_of_logical, logical_of_physical = physical_numbering(placement, 4)
    assert sorted(logical_of_physical) == list(range(8))
    for physical, e in enumerate(logical_of_physical):
        assert physical_of_logical[e] == physical and placement[e] == physical // 2    # rank p owns slots 2p, 2p + 1
    for rank in range(4):                                                              # ascending inside a rank
        mine = logical_of_physical[2 * rank: 2 * rank + 2]
        assert mine == sorted(mine)
    assert physical_numbering(contiguous_placement(8, 2), 2)[1] == list(range(8))      # contiguous blocks = identity
    with pytest.raises(ValueError):
        physical_numbering([0, 0, 0, 1], 2)          # a rank with three experts
    with pytest.raises(ValueError):
        balanced_placement([1, 2, 3], 2)
