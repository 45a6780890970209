"""Rank-sharded checkpoint files (``qutai_b200.checkpoint``) on host-memory stand-ins for the device storages: every
rank writes what it owns, rank 0 publishes the manifest, and a differently sharded run reads it back."""
import hashlib
import json
import os
import threading

import pytest

from qutai_b200 import checkpoint


class HostStorage:
    """What ``checkpoint`` needs of a storage, over a bytearray."""
    WIDTH = {"float32": 4, "bfloat16": 2}

    def __init__(self, size, dtype="float32", data=None, parent=None, start=0):
        self.size, self.dtype, self.nbytes = size, dtype, size * self.WIDTH[dtype]
        self._data = data if data is not None else bytearray(self.nbytes)
        self._start, self.uploads = start, 0

    def view(self, start, size):
        assert 0 <= start and start + size <= self.size
        return HostStorage(size, self.dtype, self._data, self, self._start + start * self.WIDTH[self.dtype])

    def tobytes(self):
        return bytes(self._data[self._start:self._start + self.nbytes])

    def upload_bytes(self, data):
        assert len(data) == self.nbytes
        self._data[self._start:self._start + self.nbytes] = data


def tensors_of(experts, prefix="blocks.3.ffn", width=24, fill=None, with_router=False, n_experts=6):
    named = []
    if with_router:
        named.append((f"{prefix}.router.weight", HostStorage(n_experts * width)))
    for e in experts:
        for kind in ("gate", "up", "down"):
            named.append((f"{prefix}.experts.{e}.{kind}.weight", HostStorage(width * 10, "bfloat16" if kind == "up" else "float32")))
    if fill is not None:
        for name, storage in named:
            storage.upload_bytes(hashlib.shake_128((fill + name).encode()).digest(storage.nbytes))
    return named


def test_two_ranks_write_and_one_reads_everything(tmp_path):
    placement = {0: [0, 2, 5], 1: [1, 3, 4]}
    written = {r: tensors_of(placement[r], fill="a", with_router=r == 0) for r in (0, 1)}
    results = {}

    def save(rank):
        results[rank] = checkpoint.save_sharded(tmp_path, written[rank], rank=rank, world=2, generation=17, metadata={"step": 17},
                                                chunk_bytes=64)

    late = threading.Thread(target=save, args=(1,))
    first = threading.Thread(target=save, args=(0,))
    first.start(); late.start(); first.join(); late.join()              # rank 0 waits for rank 1's part
    manifest = checkpoint.read_manifest(tmp_path)
    assert results[0] == tmp_path / "manifest.json" and manifest["world"] == 2 and len(manifest["shards"]) == 2
    assert sorted(os.listdir(tmp_path)) == ["data-17-rank00000.bin", "data-17-rank00001.bin", "manifest.json"]
    # one process with all six experts (another world size) reads everything back, shards verified
    whole = tensors_of(range(6), with_router=True)
    assert checkpoint.load_sharded(tmp_path, whole, verify=True, chunk_bytes=100) == {"step": 17}
    expected = dict(written[0] + written[1])
    for name, storage in whole:
        assert storage.tobytes() == expected[name].tobytes(), name
    # another placement: a rank that now owns experts 4 and 0 reads them from two different shards
    mine = tensors_of([4, 0])
    checkpoint.load_sharded(tmp_path, mine)
    for name, storage in mine:
        assert storage.tobytes() == expected[name].tobytes(), name


def test_a_new_checkpoint_replaces_the_old_one_only_after_it_is_published(tmp_path):
    checkpoint.save_sharded(tmp_path, tensors_of([0, 1], fill="old", with_router=True), generation="s1")
    old_files = set(os.listdir(tmp_path))
    with pytest.raises(TimeoutError):                                # rank 1 never writes: nothing is published, nothing removed
        checkpoint.save_sharded(tmp_path, tensors_of([0], fill="new", with_router=True), rank=0, world=2, generation="s2", timeout=0.2)
    assert checkpoint.read_manifest(tmp_path)["generation"] == "s1" and old_files <= set(os.listdir(tmp_path))
    got = tensors_of([0, 1], with_router=True)
    checkpoint.load_sharded(tmp_path, got, verify=True)
    assert dict(got)["blocks.3.ffn.experts.1.up.weight"].tobytes() == dict(tensors_of([0, 1], fill="old"))["blocks.3.ffn.experts.1.up.weight"].tobytes()
    checkpoint.save_sharded(tmp_path, tensors_of([0, 1], fill="new", with_router=True), generation="s3")
    assert checkpoint.read_manifest(tmp_path)["generation"] == "s3"
    assert not any(name.startswith("data-s1-") for name in os.listdir(tmp_path))


def test_what_does_not_fit_is_refused_before_anything_is_written(tmp_path):
    checkpoint.save_sharded(tmp_path, tensors_of([0, 1], fill="x", with_router=True), generation=1)
    with pytest.raises(KeyError):
        checkpoint.load_sharded(tmp_path, tensors_of([0, 7]))                       # expert 7 was never saved
    wrong = tensors_of([0], width=25)
    marker = wrong[0][1].tobytes()
    with pytest.raises(ValueError):
        checkpoint.load_sharded(tmp_path, tensors_of([1]) + wrong)                  # another size
    assert wrong[0][1].tobytes() == marker
    # a damaged shard is found when asked to verify
    shard = tmp_path / checkpoint.read_manifest(tmp_path)["shards"][0]["file"]
    data = bytearray(shard.read_bytes())
    data[10] ^= 0xFF
    shard.write_bytes(bytes(data))
    with pytest.raises(ValueError):
        checkpoint.load_sharded(tmp_path, tensors_of([0]), verify=True)
    shard.unlink()
    with pytest.raises(FileNotFoundError):
        checkpoint.load_sharded(tmp_path, tensors_of([0]))
    with pytest.raises(ValueError):
        checkpoint.save_sharded(tmp_path, tensors_of([0]), rank=0, world=2)         # ranks must agree on a generation
    with pytest.raises(ValueError):
        checkpoint.save_sharded(tmp_path / "d", tensors_of([0]) + tensors_of([0]))  # a name twice
    (tmp_path / "other").mkdir()
    (tmp_path / "other" / "manifest.json").write_text(json.dumps({"format": "qutai-training", "version": 1}))
    with pytest.raises(ValueError):
        checkpoint.read_manifest(tmp_path / "other")


def test_layer_tensors_uses_the_models_expert_numbers():
    class P:
        def __init__(self, tag):
            self.storage = tag

    class Expert:
        def __init__(self, e):
            self.gate, self.up, self.down = (type("Projection", (), {"weight": P(f"{e}{k}")})() for k in "gud")

    class Sharded:
        router = type("Router", (), {"weight": P("router")})()
        expert_ids = [5, 2]
        experts = [Expert(5), Expert(2)]

        def named_expert_parameters(self, prefix="experts"):
            for j, e in enumerate(self.expert_ids):
                for kind in ("gate", "up", "down"):
                    yield f"{prefix}.{e}.{kind}.weight", getattr(self.experts[j], kind).weight

    names = [name for name, _ in checkpoint.layer_tensors(Sharded(), "blocks.0.ffn", rank=1)]
    assert names == [f"blocks.0.ffn.experts.{e}.{k}.weight" for e in (5, 2) for k in ("gate", "up", "down")]
    first = checkpoint.layer_tensors(Sharded(), "blocks.0.ffn", rank=0)
    assert first[0] == ("blocks.0.ffn.router.weight", "router")

    class Single:
        router = Sharded.router
        experts = [Expert(0), Expert(1)]

    assert [name for name, _ in checkpoint.layer_tensors(Single(), "ffn")][1:4] == [f"ffn.experts.0.{k}.weight" for k in ("gate", "up", "down")]


def test_model_tensors_writes_every_name_exactly_once_across_ranks(tmp_path):
    """``model_tensors`` over stand-ins with a decoder's interface: rank 0 writes the replicated tensors and its experts,
    the other ranks only their experts; together the ranks' lists are the whole model's names, and a one-GPU model reads
    all of it back."""
    class Parameter:
        def __init__(self, size, value):
            self.storage = HostStorage(size)
            self.storage.upload_bytes(bytes([value]) * self.storage.nbytes)

    class Model:
        def __init__(self, rank, world, experts):
            self.rank, self.world = rank, world
            self.replicated = [("embedding.weight", Parameter(8, 1)), ("blocks.0.ffn.router.weight", Parameter(4, 2)), ("norm.weight", Parameter(2, 3))]
            self.experts = [(f"blocks.0.ffn.experts.{e}.gate.weight", Parameter(6, 10 + e)) for e in experts]

        def named_parameters(self):
            return self.replicated[:2] + self.experts + self.replicated[2:]

        def replicated_parameters(self):
            return tuple(p for _, p in self.replicated)

    ranks = [Model(0, 2, [0, 3]), Model(1, 2, [1, 2])]
    lists = [checkpoint.model_tensors(model) for model in ranks]
    assert [name for name, _ in lists[1]] == ["blocks.0.ffn.experts.1.gate.weight", "blocks.0.ffn.experts.2.gate.weight"]
    names = [name for named in lists for name, _ in named]
    assert len(names) == len(set(names)) == 3 + 4
    threads = [threading.Thread(target=checkpoint.save_sharded, args=(tmp_path, lists[r]), kwargs=dict(rank=r, world=2, generation=7)) for r in (1, 0)]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    whole = Model(0, 1, [0, 1, 2, 3])
    for _, parameter in whole.named_parameters():
        parameter.storage.upload_bytes(bytes(parameter.storage.nbytes))
    checkpoint.load_sharded(tmp_path, checkpoint.model_tensors(whole), verify=True)
    assert [p.storage.tobytes()[0] for _, p in whole.named_parameters()] == [1, 2, 10, 11, 12, 13, 3]


def test_a_rank_waits_for_the_manifest_of_its_own_generation(tmp_path):
    """Rank 1 saves, then waits for rank 0 to publish generation 2 (an older manifest of generation 1 lies there), and only
    then loads; a generation nobody publishes runs into the time limit."""
    import time

    first = tensors_of([0], with_router=True)
    checkpoint.save_sharded(tmp_path, first, generation=1)
    mine, theirs = tensors_of([1]), tensors_of([0], with_router=True)
    for _, storage in mine + theirs:
        storage.upload_bytes(bytes([7]) * storage.nbytes)
    checkpoint.save_sharded(tmp_path, mine, rank=1, world=2, generation=2)
    late = threading.Timer(0.3, checkpoint.save_sharded, args=(tmp_path, theirs), kwargs=dict(rank=0, world=2, generation=2))
    late.start()
    begin = time.monotonic()
    document = checkpoint.wait_for_manifest(tmp_path, 2, timeout=30)
    assert time.monotonic() - begin >= 0.2 and document["generation"] == "2" and document["world"] == 2
    late.join()
    fresh = tensors_of([1])
    checkpoint.load_sharded(tmp_path, fresh)
    assert all(storage.tobytes() == bytes([7]) * storage.nbytes for _, storage in fresh)
    with pytest.raises(TimeoutError):
        checkpoint.wait_for_manifest(tmp_path, 3, timeout=0.2)
