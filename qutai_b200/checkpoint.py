"""Checkpoint files for expert-parallel layers: every rank writes the tensors it owns, nobody gathers.

Upstream's ``save_checkpoint`` / ``load_checkpoint`` (src/qutai/lm/checkpoint.py:211-595) stream every parameter of a
single-GPU model through one writer into ``data-*.bin`` shards and publish a ``manifest.json`` whose ``tensors`` table
maps a name to ``{dtype, size, nbytes, segments: [{file, offset, nbytes}]}`` and whose ``shards`` table carries each
file's size and sha256; files are written as ``.part`` and renamed, the manifest last.  With experts sharded over
ranks the weights of one layer live on several GPUs.  This module keeps that manifest layout and those names
(``{prefix}.router.weight``, ``{prefix}.experts.{e}.gate.weight`` ... with the model's expert numbers,
src/qutai/lm/decoder.py:57-68) and changes only who writes:

* ``save_sharded(directory, named, rank=, world=)`` — every rank streams ITS tensors (device memory in 4 MiB pieces)
  into ``data-<generation>-rank<r>.bin`` and leaves ``manifest-<generation>-rank<r>.json`` beside it; rank 0 waits
  for all the pieces (files are the only channel, so it works under any launcher), merges them into
  ``manifest.json`` (atomic rename) and removes the pieces and the shards of the checkpoint it replaces.
* ``wait_for_manifest(directory, generation)`` — what a rank other than 0 calls before it loads the checkpoint it has
  just helped to write.
* ``load_sharded(directory, named)`` — a rank reads the tensors it owns NOW, from whichever shard holds them: the
  world size and the expert placement may differ from those at saving time.  Sizes and dtypes are checked, and with
  ``verify=True`` every shard a rank touches is hashed first.

``named`` is an iterable of ``(name, storage)``; a storage needs ``dtype``, ``size``, ``nbytes``, ``view(start, size)``,
``tobytes()`` and ``upload_bytes(data)`` — ``qutai_b200.storage.DeviceStorage`` has them.  ``layer_tensors`` builds
that list for a ``SparseMoE`` or an ``ExpertParallelMoE``.  Standard library only.
"""
from __future__ import annotations

import hashlib
import json
import os
import time
import uuid
from pathlib import Path

FORMAT, VERSION = "qutai-training-sharded", 1
CHUNK_BYTES = 4 << 20
_WIDTHS = {"float32": 4, "bfloat16": 2, "float64": 8, "int32": 4, "int64": 8}


def layer_tensors(layer, prefix, *, rank=0):
    """``(name, storage)`` of what this rank writes for one MoE layer: its experts' weights under the model's
    expert numbers, and on rank 0 the replicated router weight."""
    named = []
    if rank == 0:
        named.append((f"{prefix}.router.weight", layer.router.weight.storage))
    if hasattr(layer, "named_expert_parameters"):
        pairs = layer.named_expert_parameters(prefix=f"{prefix}.experts")
    else:
        pairs = ((f"{prefix}.experts.{e}.{kind}.weight", getattr(expert, kind).weight)
                 for e, expert in enumerate(layer.experts) for kind in ("gate", "up", "down"))
    named.extend((name, parameter.storage) for name, parameter in pairs)
    return named


def model_tensors(model):
    """``(name, storage)`` of what this rank writes for a ``qutai_b200.decoder.Decoder``: every tensor of
    ``named_parameters()`` on one GPU; as a rank of a data- and expert-parallel job the experts it holds (under their
    numbers in the model) and, on rank 0 only, the replicated tensors — so every name is written exactly once."""
    named = model.named_parameters()
    if getattr(model, "world", 1) == 1 or model.rank == 0:
        return [(name, parameter.storage) for name, parameter in named]
    replicated = {id(parameter) for parameter in model.replicated_parameters()}
    return [(name, parameter.storage) for name, parameter in named if id(parameter) not in replicated]


def _pieces(storage, chunk_bytes):
    width = _WIDTHS[storage.dtype]
    step = max(1, chunk_bytes // width)
    for start in range(0, storage.size, step):
        yield storage.view(start, min(step, storage.size - start)).tobytes()


def _fsync_write(path, text):
    with open(path, "x", encoding="utf8") as file:
        file.write(text)
        file.flush()
        os.fsync(file.fileno())


def save_sharded(directory, named, *, rank=0, world=1, generation=None, metadata=None, timeout=600.0, chunk_bytes=CHUNK_BYTES):
    """Write this rank's tensors and (rank 0) publish the manifest.  ``generation`` names this checkpoint's files;
    every rank must pass the same one when ``world > 1`` (a step number will do), a single writer may leave it out.
    Returns the manifest path on rank 0, the path of this rank's piece elsewhere."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    if generation is None:
        if world > 1:
            raise ValueError("ranks of one checkpoint must agree on its generation")
        generation = uuid.uuid4().hex
    generation = str(generation)
    shard_name = f"data-{generation}-rank{rank:05d}.bin"
    piece_path = directory / f"manifest-{generation}-rank{rank:05d}.json"
    temporary = directory / (shard_name + ".part")
    tensors, digest, offset = {}, hashlib.sha256(), 0
    try:
        with open(temporary, "xb") as file:
            for name, storage in named:
                if name in tensors:
                    raise ValueError(f"tensor name {name!r} appears twice")
                begin = offset
                for piece in _pieces(storage, chunk_bytes):
                    file.write(piece)
                    digest.update(piece)
                    offset += len(piece)
                if offset - begin != storage.nbytes:
                    raise RuntimeError(f"{name}: wrote {offset - begin} of {storage.nbytes} bytes")
                tensors[name] = {"dtype": storage.dtype, "size": storage.size, "nbytes": storage.nbytes, "rank": rank,
                                 "segments": [{"file": shard_name, "offset": begin, "nbytes": storage.nbytes}]}
            file.flush()
            os.fsync(file.fileno())
        os.replace(temporary, directory / shard_name)
    finally:
        if temporary.exists():
            temporary.unlink()
    piece = {"rank": rank, "tensors": tensors, "shard": {"file": shard_name, "nbytes": offset, "sha256": digest.hexdigest()}}
    piece_temporary = directory / (piece_path.name + ".part")
    piece_temporary.unlink(missing_ok=True)
    _fsync_write(piece_temporary, json.dumps(piece))
    os.replace(piece_temporary, piece_path)
    if rank != 0:
        return piece_path
    # rank 0: wait for every rank's piece, merge, publish, clean up
    deadline = time.monotonic() + timeout
    pieces = {}
    while len(pieces) < world:
        for r in range(world):
            path = directory / f"manifest-{generation}-rank{r:05d}.json"
            if r not in pieces and path.exists():
                pieces[r] = json.loads(path.read_text(encoding="utf8"))
        if len(pieces) < world:
            if time.monotonic() > deadline:
                missing = sorted(set(range(world)) - set(pieces))
                raise TimeoutError(f"ranks {missing} did not write their part of checkpoint {generation} within {timeout} s")
            time.sleep(0.05)
    merged, shards = {}, []
    for r in range(world):
        for name, record in pieces[r]["tensors"].items():
            if name in merged:
                raise ValueError(f"tensor {name!r} was written by ranks {merged[name]['rank']} and {r}")
            merged[name] = record
        shards.append(pieces[r]["shard"])
    manifest = directory / "manifest.json"
    previous = json.loads(manifest.read_text(encoding="utf8")) if manifest.exists() else None
    document = {"format": FORMAT, "version": VERSION, "generation": generation, "world": world, "tensors": merged,
                "shards": shards, "metadata": metadata or {}}
    manifest_temporary = directory / f"manifest-{generation}.json.part"
    manifest_temporary.unlink(missing_ok=True)
    _fsync_write(manifest_temporary, json.dumps(document, indent=2, allow_nan=False))
    os.replace(manifest_temporary, manifest)
    for r in range(world):
        (directory / f"manifest-{generation}-rank{r:05d}.json").unlink(missing_ok=True)
    if previous and previous.get("generation") != generation:   # only after the new one is published
        for shard in previous.get("shards", []):
            old = Path(shard["file"])
            if old.name == str(old) and old.name.startswith("data-"):
                (directory / old).unlink(missing_ok=True)
    return manifest


def read_manifest(directory):
    document = json.loads((Path(directory) / "manifest.json").read_text(encoding="utf8"))
    if document.get("format") != FORMAT or document.get("version") != VERSION:
        raise ValueError("not a sharded checkpoint of this format")
    return document


def wait_for_manifest(directory, generation, *, timeout=600.0, poll=0.05):
    """Wait until the published manifest is that of checkpoint ``generation`` and return it: what a rank other than 0
    does between its ``save_sharded`` and a ``load_sharded`` of the same checkpoint (rank 0 publishes last; files are the
    only channel between the ranks here)."""
    deadline, path = time.monotonic() + timeout, Path(directory) / "manifest.json"
    while True:
        if path.exists():
            try:
                document = json.loads(path.read_text(encoding="utf8"))
            except ValueError:
                document = None         # replaced under our eyes: look again
            if document is not None and str(document.get("generation")) == str(generation):
                return document
        if time.monotonic() > deadline:
            raise TimeoutError(f"checkpoint {generation} was not published within {timeout} s")
        time.sleep(poll)


def _verify(directory, shard):
    digest, size = hashlib.sha256(), 0
    with open(Path(directory) / shard["file"], "rb") as file:
        while True:
            piece = file.read(CHUNK_BYTES)
            if not piece:
                break
            digest.update(piece)
            size += len(piece)
    if size != shard["nbytes"] or digest.hexdigest() != shard["sha256"]:
        raise ValueError(f"shard {shard['file']} does not match the manifest (size or sha256)")


def load_sharded(directory, named, *, verify=False, chunk_bytes=CHUNK_BYTES):
    """Fill the storages of ``named`` from the checkpoint.  Returns the manifest's ``metadata``.  A name the
    checkpoint does not hold, or a tensor of another size or dtype, raises before anything is written."""
    directory = Path(directory)
    document = read_manifest(directory)
    named = list(named)
    shards = {shard["file"]: shard for shard in document["shards"]}
    needed = set()
    for name, storage in named:
        record = document["tensors"].get(name)
        if record is None:
            raise KeyError(f"the checkpoint holds no tensor named {name!r}")
        if record["dtype"] != storage.dtype or record["size"] != storage.size:
            raise ValueError(f"{name}: the checkpoint has {record['dtype']}[{record['size']}], the model {storage.dtype}[{storage.size}]")
        for segment in record["segments"]:
            if segment["file"] not in shards:
                raise ValueError(f"{name}: shard {segment['file']} is not listed in the manifest")
            if segment["offset"] + segment["nbytes"] > shards[segment["file"]]["nbytes"]:
                raise ValueError(f"{name}: segment reaches past the end of {segment['file']}")
            needed.add(segment["file"])
    for file in sorted(needed):
        if not (directory / file).exists():
            raise FileNotFoundError(f"shard {file} is missing")
        if verify:
            _verify(directory, shards[file])
    for name, storage in named:
        record = document["tensors"][name]
        width = _WIDTHS[storage.dtype]
        step = max(1, chunk_bytes // width)
        done = 0                                     # elements of the tensor filled so far
        for segment in record["segments"]:
            with open(directory / segment["file"], "rb") as file:
                file.seek(segment["offset"])
                remaining = segment["nbytes"]
                while remaining:
                    take = min(remaining, step * width)
                    data = file.read(take)
                    if len(data) != take or take % width:
                        raise ValueError(f"{name}: {segment['file']} ended early")
                    storage.view(done, take // width).upload_bytes(data)
                    done += take // width
                    remaining -= take
        if done != storage.size:
            raise ValueError(f"{name}: the segments hold {done} of {storage.size} elements")
    return document.get("metadata", {})
