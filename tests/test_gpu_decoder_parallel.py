"""The decoder as ranks of a data- and expert-parallel job (``Decoder(..., rank=, world=)``): every rank takes its share
of the sequences of the upstream-made fixture, the experts of every block are spread over the ranks.  The job's loss and
every gradient must be what upstream's single-device ``Decoder`` produced on the whole batch
(tests/golden/make_golden_decoder.py), the replicated gradients and parameters must be the same bits on every rank.
Each rank is a child process on its own GPU; skipped on a box with fewer GPUs than ranks.  Needs B200s: ``-m gpu``."""
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import moe_oracle as oracle

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for line in out.splitlines() if line.startswith("GPU "))
    except Exception:
        return 0


def run_ranks(world, out_dir):
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "decoder_parallel_worker.py"), str(rank), str(world), out_dir],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=dict(os.environ, NCCL_DEBUG="WARN"))
             for rank in range(world)]
    for rank, proc in enumerate(procs):
        try:
            out, _ = proc.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            proc.kill()
            out, _ = proc.communicate()
        assert proc.returncode == 0 and f"rank {rank} done" in out, out[-3000:]
    return [np.load(os.path.join(out_dir, f"rank{rank}.npz")) for rank in range(world)]


def test_two_ranks_reproduce_the_upstream_decoder_on_the_whole_batch(tmp_path):
    world = 2
    if gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    g = np.load(os.path.join(HERE, "golden", "decoder_small.npz"))
    ranks = run_ranks(world, str(tmp_path))
    wanted = [key[5:] for key in g.files if key.startswith("grad:")]
    experts = 4
    for rank, r in enumerate(ranks):
        for key, bar in (("loss", 2e-2), ("lm_loss", 2e-2), ("aux_loss", 1e-2)):
            assert abs(float(r[key][0]) - float(g[key])) <= bar * abs(float(g[key])), (rank, key)
        # upstream's names and order, minus the experts that live on the other rank (contiguous blocks of experts)
        held = [name for name in wanted if ".ffn.experts." not in name
                or int(name.split(".ffn.experts.")[1].split(".")[0]) // (experts // world) == rank]
        assert r["names"].tolist() == held
        worst = {}
        for name in held:
            want = g["grad:" + name]
            if want.size == 0:
                assert not bool(r["has:" + name]), name          # an expert that received no token from any rank
                continue
            assert bool(r["has:" + name]), name
            worst[name] = oracle.max_rel_err(r["grad:" + name], want)
        loose = {name: error for name, error in worst.items() if error > 6e-2}
        assert not loose, (rank, loose)
        # the norm before the expert-parallel layer hands over a bf16 tensor and the residual is added in a step of its
        # own: two roundings the fused block of the one-GPU decoder (median bar 2e-2 there) does not have
        assert np.median(list(worst.values())) <= 3e-2
        assert r["losses"][-1] < r["losses"][0] - 0.3, r["losses"]
    first, second = ranks
    # gradient clipping over the whole model: upstream's joint norm of ALL gradients, the same on both ranks, and
    # every gradient (replicated or one rank's expert) scaled by max_norm / norm
    joint = np.sqrt(sum(float((g[key].astype(np.float64) ** 2).sum()) for key in g.files if key.startswith("grad:")))
    assert float(first["clip_norm"]) == float(second["clip_norm"])
    assert abs(float(first["clip_norm"]) - joint) <= 3e-2 * joint
    factor = 1e-3 / float(first["clip_norm"])
    for r in ranks:
        assert oracle.max_rel_err(r["clipped:embedding.weight"], r["grad:embedding.weight"] * factor) <= 1e-5
        assert oracle.max_rel_err(r["clipped_expert"], r["grad:" + str(r["clipped_expert_name"])] * factor) <= 1e-5
    assert float(first["loss"][0]) == float(second["loss"][0])
    for name in first["replicated"].tolist() + [n for n in first["names"].tolist() if n.endswith("router.weight")]:
        assert np.array_equal(first["grad:" + name], second["grad:" + name]), name
    assert first["losses"].tolist() == second["losses"].tolist()
    assert np.array_equal(first["embedding_after"], second["embedding_after"])     # the replicas stay in step
    assert np.array_equal(first["router_after"], second["router_after"])
