"""Expert-parallel ``SparseMoE``: one process per GPU, tokens sharded by rank (contiguous shards of
equal size), experts sharded by rank (E / world each; contiguous blocks unless a placement map says
otherwise), rows exchanged by direct stores into peer memory over NVLink or by NCCL send/receive.

The upstream project is single-GPU; this module keeps its layer semantics across ranks: routing is
decided per token exactly as on one GPU, an expert's rows arrive ordered by source rank — with
contiguous token shards that is the upstream global (token, slot) order
(src/qutai/backends/cuda/lm.cu:353-383) — and utilisation / auxiliary loss are taken over all ranks'
tokens (src/qutai/backends/cpu_lm.py:221-229).  Host code is standard-library Python; the NCCL id
travels through a small file rendezvous (or any callable the caller supplies).

With the NCCL transport the host waits once per step for the device, to read the [world, E] matrix of
counts that sizes the exchanges (the upstream layer also reads its counts in every forward,
src/qutai/backends/cuda_lm.py:432-434); with the direct transport it waits for nothing inside a step.

Expert placement.  ``placement[e]`` names the rank that owns expert ``e``.  Inside the layer experts are
numbered physically — rank ``p`` owns physical experts ``p * L .. p * L + L - 1``, its logical experts in
ascending order — and every kernel works on physical numbers; only the small expert-indexed tables
(router weight rows, their gradient, utilisation, counts) are permuted at the layer's boundary, so
``router.weight``, ``utilization``, ``last_counts`` and the parameter names (``expert_ids``) keep the
model's own expert numbering (src/qutai/lm/decoder.py:57-68).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import time
from math import sqrt

from . import lib
from .layers import Projection, SwiGLU, Tensor, _accumulate
from .storage import DeviceStorage


# ------------------------------------------------------------------------------------------------
# host logic (no GPU needed)
# ------------------------------------------------------------------------------------------------
def padded_offsets(counts, pad=lib.ROW_PAD):
    """First row of each group when every group is padded to a multiple of ``pad`` rows."""
    offsets, at = [], 0
    for c in counts:
        offsets.append(at)
        at += -(-c // pad) * pad
    offsets.append(at)
    return offsets


def plan_exchange(counts, rank, world, pad=lib.ROW_PAD):
    """Segments of the dispatch all-to-all for ``rank``.

    ``counts[p][e]`` = rows that rank ``p`` routes to global expert ``e``.  Token side: this rank's
    dispatched buffer holds expert ``e``'s rows at ``send_offsets[e]`` (padded groups, all E
    experts).  Expert side: local expert ``j`` (global ``rank * E_loc + j``) receives the rows of
    rank 0, rank 1, ... one after the other, groups padded to ``pad``.

    Returns a dict: ``sends`` / ``recvs`` lists of ``(peer, offset_rows, rows)`` in the order they
    must be posted (for a fixed pair of ranks both lists walk the experts in ascending order, so
    the i-th send matches the i-th receive), ``expert_counts``, ``expert_offsets``.  The combine
    all-to-all is the same plan with the two lists swapped.
    """
    experts = len(counts[0])
    if experts % world:
        raise ValueError("the number of experts must be a multiple of the number of ranks")
    local = experts // world
    send_offsets = padded_offsets(counts[rank], pad)
    sends = [(e // local, send_offsets[e], counts[rank][e]) for e in range(experts) if counts[rank][e]]
    mine = range(rank * local, (rank + 1) * local)
    expert_counts = [sum(counts[p][e] for p in range(world)) for e in mine]
    expert_offsets = padded_offsets(expert_counts, pad)
    recvs = []
    for p in range(world):
        for j, e in enumerate(mine):
            if counts[p][e]:
                before = sum(counts[q][e] for q in range(p))
                recvs.append((p, expert_offsets[j] + before, counts[p][e]))
    return dict(sends=sends, recvs=recvs, expert_counts=expert_counts, expert_offsets=expert_offsets,
                send_offsets=send_offsets)


def file_rendezvous(path, rank, payload=None, timeout=60.0, poll=0.02):
    """Share ``payload`` (bytes, given by rank 0) with every rank through a file.  Rank 0 publishes
    atomically; the others poll until the file appears or ``timeout`` seconds pass (TimeoutError:
    rank 0 never arrived)."""
    if rank == 0:
        tmp = f"{path}.tmp.{os.getpid()}"
        with open(tmp, "wb") as handle:
            handle.write(payload)
        os.replace(tmp, path)
        return payload
    deadline = time.monotonic() + timeout
    while True:
        try:
            with open(path, "rb") as handle:
                data = handle.read()
            if data:
                return data
        except FileNotFoundError:
            pass
        if time.monotonic() > deadline:
            raise TimeoutError(f"rank {rank}: no NCCL id at {path} after {timeout:.0f} s (is rank 0 alive?)")
        time.sleep(poll)


_JOB = {"token": "job"}


def default_rendezvous_dir():
    return os.path.join("/tmp", "qutai_moe_%s_%s" % (os.environ.get("MASTER_ADDR", "local"), os.environ.get("MASTER_PORT", "0")))


def file_all_gather(directory, tag, rank, world, payload, timeout=120.0, poll=0.02):
    """All-gather of one bytes object per rank through files in ``directory`` (every rank publishes
    ``tag.rank`` atomically and polls for the others; TimeoutError names the ranks that never came)."""
    os.makedirs(directory, exist_ok=True)
    tmp = os.path.join(directory, f"{tag}.{rank}.tmp.{os.getpid()}")
    with open(tmp, "wb") as handle:
        handle.write(payload)
    os.replace(tmp, os.path.join(directory, f"{tag}.{rank}"))
    deadline, result = time.monotonic() + timeout, [None] * world
    while True:
        for p in range(world):
            if result[p] is None:
                try:
                    with open(os.path.join(directory, f"{tag}.{p}"), "rb") as handle:
                        data = handle.read()
                    if data:
                        result[p] = data
                except FileNotFoundError:
                    pass
        if all(item is not None for item in result):
            return result
        if time.monotonic() > deadline:
            missing = [p for p in range(world) if result[p] is None]
            raise TimeoutError(f"rank {rank}: ranks {missing} never published '{tag}' in {directory}")
        time.sleep(poll)


class FileExchange:
    """Repeated all-gathers between the ranks of one job through files in one directory.  Every exchange
    uses a tag of its own (``<name>_<n>``, n counted the same way on every rank), so a rank that is one
    exchange ahead can never be handed a file a slower rank wrote for the previous one; the rank's own
    files are removed by ``close()``, after which the directory can be reused."""

    def __init__(self, directory, name, rank, world, timeout=120.0):
        self.directory, self.name, self.rank, self.world, self.timeout = directory, name, rank, world, timeout
        self.exchanges = 0

    def all_gather(self, payload):
        self.exchanges += 1
        return file_all_gather(self.directory, f"{self.name}_{self.exchanges}", self.rank, self.world, payload, self.timeout)

    def close(self):
        for n in range(1, self.exchanges + 1):
            try:
                os.remove(os.path.join(self.directory, f"{self.name}_{n}.{self.rank}"))
            except OSError:
                pass
        self.exchanges = 0


def contiguous_placement(experts, world):
    """Expert ``e`` on rank ``e // (experts / world)``."""
    if experts % world:
        raise ValueError("the number of experts must be a multiple of the number of ranks")
    return [e // (experts // world) for e in range(experts)]


def balanced_placement(counts, world):
    """Load-aware placement from per-expert row counts: longest-processing-time greedy (experts by falling
    count, each to the least loaded rank that still has a free slot).  Returns ``placement[e] = rank``."""
    experts = len(counts)
    if experts % world:
        raise ValueError("the number of experts must be a multiple of the number of ranks")
    slots = experts // world
    loads, filled, placement = [0] * world, [0] * world, [0] * experts
    for e in sorted(range(experts), key=lambda i: (-counts[i], i)):
        p = min((r for r in range(world) if filled[r] < slots), key=lambda r: (loads[r], r))
        placement[e] = p
        loads[p] += counts[e]
        filled[p] += 1
    return placement


def physical_numbering(placement, world):
    """``(physical_of_logical, logical_of_physical)`` for a placement: rank ``p`` owns physical experts
    ``p * L + j`` where ``j`` counts its logical experts in ascending order.  Raises when a rank does not
    own exactly E / world experts."""
    experts = len(placement)
    if experts % world:
        raise ValueError("the number of experts must be a multiple of the number of ranks")
    slots = experts // world
    owned = [[e for e in range(experts) if placement[e] == p] for p in range(world)]
    if any(not 0 <= p < world for p in placement) or any(len(o) != slots for o in owned):
        raise ValueError(f"every rank must own exactly {slots} experts")
    logical_of_physical = [e for p in range(world) for e in owned[p]]
    physical_of_logical = [0] * experts
    for physical, e in enumerate(logical_of_physical):
        physical_of_logical[e] = physical
    return physical_of_logical, logical_of_physical


def init_communicator(rank, world, share=None, rendezvous_path=None, timeout=60.0):
    """Create the process' NCCL communicator.  ``share(payload_or_None) -> bytes`` broadcasts rank
    0's 128-byte id (rank 0 passes it, the others pass None); without it a file rendezvous at
    ``rendezvous_path`` is used."""
    payload = None
    if rank == 0:
        buffer = ctypes.create_string_buffer(128)
        lib.call("qmoe_ep_unique_id", ctypes.cast(buffer, ctypes.c_void_p))
        payload = buffer.raw
    if share is not None:
        payload = share(payload)
    else:
        if rendezvous_path is None:
            rendezvous_path = os.path.join(
                "/tmp", "qutai_moe_id_%s_%s" % (os.environ.get("MASTER_ADDR", "local"), os.environ.get("MASTER_PORT", "0")))
        payload = file_rendezvous(rendezvous_path, rank, payload, timeout)
    if len(payload) != 128:
        raise ValueError("the NCCL id must be 128 bytes")
    _JOB["token"] = hashlib.sha1(payload).hexdigest()[:12]  # names this job's rendezvous files
    buffer = ctypes.create_string_buffer(payload, 128)
    lib.call("qmoe_ep_init", rank, world, ctypes.cast(buffer, ctypes.c_void_p))


def finalize_communicator(abort=False):
    lib.call("qmoe_ep_finalize", 1 if abort else 0)
    for exchange in _IPC_EXCHANGES.values():   # this process' rendezvous files of the job
        exchange.close()
    _IPC_EXCHANGES.clear()


def _segments(triples):
    array = (lib.Segment * max(1, len(triples)))()
    for i, (peer, offset, rows) in enumerate(triples):
        array[i].peer, array[i].offset_rows, array[i].rows = peer, offset, rows
    return array, len(triples)


# ------------------------------------------------------------------------------------------------
# the layer
# ------------------------------------------------------------------------------------------------
_IPC_EXCHANGES = {}   # job token -> FileExchange of this process (the default channel for swapping IPC handles)


class ExpertParallelMoE:
    """``SparseMoE`` over ``world`` GPUs.  Same constructor fields as the single-GPU layer plus
    ``rank`` / ``world``; ``experts`` holds only this rank's E / world experts (``expert_ids[j]`` is the
    model's number of ``experts[j]``), ``router`` is replicated and its gradient is summed over ranks."""

    def __init__(self, config, *, rank, world, device="cuda", dtype="float32", seed=None, engine="auto", stream=0,
                 transport="p2p", barrier="flags", placement=None, gather=None, overlap=False):
        """``transport``: "p2p" (default) = rows pushed straight into the peers' buffers over NVLink (CUDA IPC
        mappings, destinations computed on the device, no host read in the forward); "nccl" = grouped NCCL
        send/receive sized by counts the host reads once per step.  ``barrier`` (p2p only): "flags" = the
        bounded flag barrier over peer memory, which also carries the count all-gather; "nccl" = NCCL
        collectives instead.  ``placement[e]`` = rank owning expert ``e`` (default: contiguous blocks); every
        rank passes the same list.  ``gather(payload) -> [payload of rank 0, ...]`` all-gathers a bytes object
        between the ranks (needed for "p2p" to swap the IPC handles); without it files in a per-job directory
        are used.  ``overlap`` (p2p with the flag barrier and the tensor-core engine, at least two local experts):
        the rows of the second half of every rank's experts travel on a side stream while the first product
        already runs on the first half (forward: dispatch behind SwiGLU; backward: the gradient rows behind
        dSwiGLU); the results are bit-identical to the serial order.  Off by default: at two GPUs it measured
        no faster than the serial order (two more barriers, two smaller product launches, and the push slows the
        product it runs beside)."""
        if device != "cuda" or dtype != "float32":
            raise ValueError("parameters are float32 on device='cuda'")
        if transport not in ("nccl", "p2p"):
            raise ValueError("transport must be 'nccl' or 'p2p'")
        if barrier not in ("flags", "nccl"):
            raise ValueError("barrier must be 'flags' or 'nccl'")
        if world > lib.EP_MAX_RANKS:
            raise ValueError(f"at most {lib.EP_MAX_RANKS} ranks")
        self.transport, self.barrier, self._gather, self.overlap = transport, barrier, gather, bool(overlap)
        d, E, h = config.d_model, config.n_experts, config.d_expert
        if E % world:
            raise ValueError("n_experts must be a multiple of the number of ranks")
        self.rank, self.world, self.stream = rank, world, stream
        self.top_k, self.n_experts, self.d_model, self.d_expert = config.top_k, E, d, h
        self.local_experts = L = E // world
        self.engine = {"auto": lib.ENGINE_AUTO, "simt": lib.ENGINE_SIMT, "tcgen05": lib.ENGINE_TCGEN05}[engine]
        self._down_std = 0.02 / sqrt(2 * config.n_layers)
        router = DeviceStorage(E * d, "float32")
        router.fill_normal(0.0, 0.02, 0x5EED if seed is None else seed, stream)
        self.router = Projection(Tensor(router, (E, d), requires_grad=True))
        self._set_placement(contiguous_placement(E, world) if placement is None else list(placement))
        self._gate = DeviceStorage(L * h * d, "float32")
        self._up = DeviceStorage(L * h * d, "float32")
        self._down = DeviceStorage(L * d * h, "float32")
        self._make_experts()
        for j, i in enumerate(self.expert_ids):   # the model's expert number decides the generator key, as on one GPU
            base = None if seed is None else seed + 1 + 3 * i
            expert = self.experts[j]
            expert.gate.weight.storage.fill_normal(0.0, 0.02, 0x5EED if base is None else base, stream)
            expert.up.weight.storage.fill_normal(0.0, 0.02, 0x5EED if base is None else base + 1, stream)
            expert.down.weight.storage.fill_normal(0.0, self._down_std, 0x5EED if base is None else base + 2, stream)
        self.utilization = None
        self._side = None   # second stream and its events: work that nothing on the main stream waits for soon
        # "auto": rebuild the bf16 weight copies only after a weight storage was written (DeviceStorage.generation);
        # True: at every forward; False: never after the first forward
        self.refresh_operands = "auto"
        # False: backward leaves THIS rank's part of the router gradient in ``router.weight.grad`` and the caller sums
        # it over the ranks (a model that reduces all its replicated gradients in one collective)
        self.reduce_router_gradient = True
        self._sequence = 0  # barriers issued so far (the flag barrier's growing sequence number)
        self._work = None
        self._saved = None

    # ------------------------------------------------------------------------------------------
    def _set_placement(self, placement):
        E = self.n_experts
        if len(placement) != E:
            raise ValueError("placement needs one rank per expert")
        self._physical_of_logical, self._logical_of_physical = physical_numbering(placement, self.world)
        self.placement = tuple(placement)
        L = self.local_experts
        self.expert_ids = tuple(self._logical_of_physical[self.rank * L:(self.rank + 1) * L])
        self._identity = self._logical_of_physical == list(range(E))
        if not self._identity:
            ints = lambda values: DeviceStorage.from_bytes(b"".join(int(v).to_bytes(4, "little") for v in values), "int32")
            self._to_physical = ints(self._logical_of_physical)   # gather index: physical row p <- logical row
            self._to_logical = ints(self._physical_of_logical)    # gather index: logical row e <- physical row
            self._router_physical = DeviceStorage(E * self.d_model, "float32")

    def _make_experts(self):
        L, h, d = self.local_experts, self.d_expert, self.d_model
        experts = []
        for j in range(L):
            views = (self._gate.view(j * h * d, h * d), self._up.view(j * h * d, h * d), self._down.view(j * d * h, d * h))
            experts.append(SwiGLU(Tensor(views[0], (h, d), requires_grad=True), Tensor(views[1], (h, d), requires_grad=True),
                                  Tensor(views[2], (d, h), requires_grad=True)))
        self.experts = tuple(experts)

    def parameters(self):
        return (*self.router.parameters(), *(p for expert in self.experts for p in expert.parameters()))

    def named_expert_parameters(self, prefix="experts"):
        """``(name, parameter)`` pairs of this rank's expert weights under the model's expert numbers
        (``experts.{e}.gate.weight`` ..., the names src/qutai/lm/decoder.py:57-68 gives them on one GPU)."""
        for j, e in enumerate(self.expert_ids):
            expert = self.experts[j]
            yield f"{prefix}.{e}.gate.weight", expert.gate.weight
            yield f"{prefix}.{e}.up.weight", expert.up.weight
            yield f"{prefix}.{e}.down.weight", expert.down.weight

    def operand_shadows(self):
        """``{parameter: bf16 storage}`` of the tensor-core operand copies of this rank's expert weights, for
        ``qutai_b200.optim.AdamW(shadows=...)`` (see ``SparseMoE.operand_shadows``)."""
        work = self._work
        if work is None or "w_gate" not in work["buf"]:
            raise RuntimeError("no bfloat16 forward has run yet")
        buf, h, d = work["buf"], self.d_expert, self.d_model
        shadows = {}
        for j, expert in enumerate(self.experts):
            shadows[expert.gate.weight] = buf["w_gate"].view(j * h * d, h * d)
            shadows[expert.up.weight] = buf["w_up"].view(j * h * d, h * d)
            shadows[expert.down.weight] = buf["w_down"].view(j * d * h, d * h)
        return shadows

    def rebalance(self, counts=None, placement=None):
        """Move the expert weights to a new placement: ``placement`` if given, else the load-balanced one for
        the per-expert ``counts`` (default: the counts of the last forward).  Every rank calls it with the same
        arguments; the weights travel through one grouped NCCL exchange per kind.  ``experts`` and
        ``expert_ids`` are rebuilt (new parameter objects over the moved weights), gradients are dropped:
        call it before an optimizer is created, or move the optimizer's moments the same way with
        ``move_expert_tensors``.  Returns the new placement."""
        if placement is None:
            placement = balanced_placement(list(self.last_counts if counts is None else counts), self.world)
        old_ids = self.expert_ids
        old_owner = dict(zip(range(self.n_experts), self.placement))
        self._set_placement(list(placement))
        h, d = self.d_expert, self.d_model
        moved = [self.move_expert_tensors(storage, rows, width, old_ids, old_owner)
                 for storage, rows, width in ((self._gate, h, d), (self._up, h, d), (self._down, d, h))]
        self._gate, self._up, self._down = moved
        self._make_experts()
        self.router.weight.grad = None
        self._work, self._saved = self._close_workspace(), None
        return self.placement

    def move_expert_tensors(self, stacked, rows, width, old_ids, old_owner):
        """One stacked fp32 buffer of per-expert blocks (``rows`` x ``width`` each, in the slot order of
        ``old_ids``) re-sharded to the layer's current placement; returns the new stacked storage."""
        s = self.stream
        out = DeviceStorage(stacked.size, "float32")
        sends = [(self.placement[e], j * rows, rows) for j, e in enumerate(old_ids)]
        recvs = [(old_owner[e], j * rows, rows) for j, e in enumerate(self.expert_ids)]
        (sa, sn), (ra, rn) = _segments(sends), _segments(recvs)
        lib.call("qmoe_ep_exchange", stacked.ptr, sa, sn, out.ptr, ra, rn, width, lib.QMOE_F32, s)
        lib.call("qmoe_stream_sync", s)   # the old buffer may be released once the exchange has run
        out.touch()
        return out

    # ------------------------------------------------------------------------------------------
    def _close_workspace(self):
        """Unmap the peers' buffers of the workspace that is being replaced."""
        work = self._work
        if work is not None and work.get("opened"):
            lib.call("qmoe_stream_sync", self.stream)
            for address in work["opened"]:
                lib.load().qmoe_ep_ipc_close(address)
            work["opened"] = []
        return None

    def _workspace(self, tokens, dtype):
        if self._work is not None and self._work["key"] == (tokens, dtype):
            return self._work
        self._work = self._close_workspace()
        E, L, k, d, h, N = self.n_experts, self.local_experts, self.top_k, self.d_model, self.d_expert, self.world
        A = tokens * k
        Rt = lib.rows_bound(tokens, E, k)
        Rx = lib.rows_bound(tokens * N, L, k)
        blocks = lib.route_blocks(tokens)
        S = DeviceStorage
        buf = dict(
            probs=S(tokens * E, "float32"), gate_weights=S(A, "float32"), expert_index=S(A, "int32"),
            dest_row=S(A, "int32"), row_source=S(Rt, "int32"), counts=S(E, "int32"), offsets=S(E + 1, "int32"),
            tile_expert=S(Rt // lib.ROW_PAD, "int32"), meta=S(4, "int32"), utilization=S(E, "float32"),
            aux=S(1, "float32"), block_counts=S(blocks * E, "int32"), block_base=S(blocks * E, "int32"),
            block_colsum=S(blocks * E, "float32"),
            scores=S(tokens * E, "float32"), stats_local=S(2 * E, "int32"), stats_all=S(N * 2 * E, "int32"),
            x_send=S(Rt * d, dtype), y_send=S(Rt * d, dtype), dy_send=S(Rt * d, dtype),
            x_counts=S(L, "int32"), x_offsets=S(L + 1, "int32"), x_tile_expert=S(Rx // lib.ROW_PAD, "int32"), x_meta=S(4, "int32"),
            x_recv=S(Rx * d, dtype), g=S(Rx * h, dtype), u=S(Rx * h, dtype), h=S(Rx * h, dtype), y_recv=S(Rx * d, dtype),
            dy_recv=S(Rx * d, dtype), d_h=S(Rx * h, dtype), d_g=S(Rx * h, dtype), d_u=S(Rx * h, dtype),
            d_gate_weights=S(A, "float32"), d_scores=S(tokens * E, "float32"), dx_router=S(tokens * d, "float32"),
            router_partials=S(int(lib.load().qmoe_router_grad_partials(tokens, E, d)), "float32"),
            d_w_router=S(E * d, "float32"), d_w_gate=S(L * h * d, "float32"), d_w_up=S(L * h * d, "float32"),
            d_w_down=S(L * d * h, "float32"), aux_grad=S(1, "float32"),
            ret_table=S(Rx, "int32"), dest_base=S(E, "int32"), barrier=S.zeros(1, "int32"),
            flags=S.zeros(lib.EP_MAX_RANKS, "int32"),
        )
        if not self._identity:   # the expert-indexed outputs in the model's numbering
            buf.update(utilization_logical=S(E, "float32"), d_w_router_logical=S(E * d, "float32"))
        if self.transport == "p2p":
            buf["dx_recv"] = S(Rx * d, dtype)  # dX gets its own buffer so it can travel while the weight gradients run
        if dtype == "bfloat16":
            buf.update(w_gate=S(L * h * d, "bfloat16"), w_up=S(L * h * d, "bfloat16"), w_down=S(L * d * h, "bfloat16"))
        token_route = lib.Route()
        token_route.tokens, token_route.experts, token_route.top_k, token_route.rows_bound = tokens, E, k, Rt
        for name in ("probs", "gate_weights", "expert_index", "dest_row", "row_source", "counts", "offsets", "tile_expert",
                     "meta", "utilization", "aux", "block_counts", "block_base", "block_colsum"):
            setattr(token_route, name, buf[name].ptr)
        # expert side: only counts / offsets / tile_expert / meta are meaningful; the other tables
        # are never touched through this struct and just need valid addresses
        expert_route = lib.Route()
        expert_route.tokens, expert_route.experts, expert_route.top_k, expert_route.rows_bound = tokens * N, L, k, Rx
        for name in ("probs", "gate_weights", "expert_index", "dest_row", "row_source", "utilization", "aux",
                     "block_counts", "block_base", "block_colsum"):
            setattr(expert_route, name, buf["x_meta"].ptr)
        expert_route.counts, expert_route.offsets = buf["x_counts"].ptr, buf["x_offsets"].ptr
        expert_route.tile_expert, expert_route.meta = buf["x_tile_expert"].ptr, buf["x_meta"].ptr
        ex = lib.Experts()
        ex.experts, ex.dtype, ex.engine, ex.width, ex.hidden = L, lib.DTYPE_CODES[dtype], self.engine, d, h
        if dtype == "bfloat16":
            ex.w_gate, ex.w_up, ex.w_down = buf["w_gate"].ptr, buf["w_up"].ptr, buf["w_down"].ptr
        else:
            ex.w_gate, ex.w_up, ex.w_down = self._gate.ptr, self._up.ptr, self._down.ptr
        host, status, stats_event = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_uint64()
        lib.call("qmoe_host_alloc", ctypes.byref(host), 4 * N * 2 * E)
        lib.call("qmoe_host_alloc", ctypes.byref(status), 8)
        lib.call("qmoe_event_create", ctypes.byref(stats_event))
        host_status = ctypes.cast(status, ctypes.POINTER(ctypes.c_int32))
        host_status[0] = host_status[1] = 0
        router_grad = buf["d_w_router"] if self._identity else buf["d_w_router_logical"]
        grad_views = [Tensor(router_grad, (E, d))]
        for j in range(L):
            grad_views.append((Tensor(buf["d_w_gate"].view(j * h * d, h * d), (h, d)),
                               Tensor(buf["d_w_up"].view(j * h * d, h * d), (h, d)),
                               Tensor(buf["d_w_down"].view(j * d * h, d * h), (d, h))))
        self._work = dict(key=(tokens, dtype), buf=buf, token_route=token_route, expert_route=expert_route, experts=ex,
                          host_stats=ctypes.cast(host, ctypes.POINTER(ctypes.c_int32)), host_status=host_status,
                          grad_views=grad_views, stats_event=stats_event.value, opened=[])
        tensor_cores = dtype == "bfloat16" and self.engine != lib.ENGINE_SIMT and d % 8 == 0 and h % 8 == 0
        # fused: the producing kernels (permute, combine-backward, and the tensor-core epilogues of the down
        # projection and of dX) store their rows straight into the owning GPU's buffer
        self._work["fused"] = self.transport == "p2p" and tensor_cores
        if self._side is None:
            side = ctypes.c_uint64()
            lib.call("qmoe_stream_create", ctypes.byref(side))
            self._side = {"stream": side.value}
            for name in ("ready", "done", "stats", "grads", "reduced", "ended", "first_sent", "rest_landed"):
                event = ctypes.c_uint64()
                lib.call("qmoe_event_create", ctypes.byref(event))
                self._side[name] = event.value
        if self.transport == "p2p":
            self._work["peers"] = self._open_peers(buf, self._work["opened"])
            # barriers and the count all-gather go through flags in peer memory unless NCCL is asked for
            self._work["flag_barrier"] = self.barrier == "flags"
        self._work["groups"] = None
        if self.overlap and self._work["fused"] and self._work.get("flag_barrier") and L >= 2:
            # two groups of local experts, [0, split) and [split, L): routes and weight tables that cover one group each
            split, item = L // 2, lib.ITEM_BYTES[dtype]
            groups = []
            for begin, end in ((0, split), (split, L)):
                route, experts = lib.Route(), lib.Experts()
                ctypes.memmove(ctypes.byref(route), ctypes.byref(expert_route), ctypes.sizeof(route))
                ctypes.memmove(ctypes.byref(experts), ctypes.byref(ex), ctypes.sizeof(experts))
                route.experts = experts.experts = end - begin
                route.counts, route.offsets = buf["x_counts"].ptr + 4 * begin, buf["x_offsets"].ptr + 4 * begin
                experts.w_gate, experts.w_up = ex.w_gate + begin * h * d * item, ex.w_up + begin * h * d * item
                experts.w_down = ex.w_down + begin * d * h * item
                groups.append((begin, end, route, experts))
            self._work["groups"] = groups
        return self._work

    def _open_peers(self, buf, opened):
        """Swap CUDA IPC handles of the buffers other ranks write into and map every peer's."""
        names = ("x_recv", "dy_recv", "y_send", "dy_send", "ret_table", "flags", "stats_all")
        lib.call("qmoe_stream_sync", 0)  # the zero-fill of the flag array must have run before any peer can write it
        payload = b""
        for name in names:
            handle = ctypes.create_string_buffer(64)
            lib.call("qmoe_ep_ipc_export", buf[name].ptr, ctypes.cast(handle, ctypes.c_void_p))
            payload += handle.raw
        gather = self._gather
        if gather is None:
            # one exchange object per job and process: every exchange (a second layer of the model, a workspace
            # rebuilt for another token count) gets a tag of its own, counted alike on all ranks
            token = _JOB["token"]
            if token not in _IPC_EXCHANGES:
                _IPC_EXCHANGES[token] = FileExchange(default_rendezvous_dir(), "ipc_" + token, self.rank, self.world)
            gather = _IPC_EXCHANGES[token].all_gather
        everyone = gather(payload)
        if len(everyone) != self.world or any(len(item) != 64 * len(names) for item in everyone):
            raise ValueError("the IPC handle all-gather returned a wrong shape")
        address = {name: [0] * self.world for name in names}
        for p in range(self.world):
            for i, name in enumerate(names):
                if p == self.rank:
                    address[name][p] = buf[name].ptr
                else:
                    mapped = ctypes.c_uint64()
                    handle = ctypes.create_string_buffer(everyone[p][64 * i: 64 * (i + 1)], 64)
                    lib.call("qmoe_ep_ipc_open", ctypes.cast(handle, ctypes.c_void_p), ctypes.byref(mapped))
                    address[name][p] = mapped.value
                    opened.append(mapped.value)
        peers = {}
        for name in ("x_recv", "dy_recv", "y_send", "dy_send", "flags", "stats_all"):
            table = lib.Peers()
            table.world, table.rank = self.world, self.rank
            for p in range(self.world):
                table.buffer[p] = address[name][p]
                table.ret[p] = address["ret_table"][p]
            peers[name] = table
        return peers

    def __call__(self, x):
        return self.forward(x)

    def _barrier(self, w, stream=None):
        """Order everything the ranks enqueued so far (on ``stream``) against what they enqueue next."""
        stream = self.stream if stream is None else stream
        if w.get("flag_barrier"):
            self._sequence += 1
            lib.call("qmoe_ep_flag_barrier", ctypes.byref(w["peers"]["flags"]), self._sequence, 0, 0, None, stream)
        else:
            lib.call("qmoe_ep_barrier", w["buf"]["barrier"].ptr, stream)

    def _two_phase(self, w, push, product):
        """The overlapped order of one exchange: ``push(begin, end, stream)`` sends the rows of the local experts
        [begin, end) of every rank, ``product(route, experts)`` runs the first tensor-core product on one group.
        Group 0 travels and is waited for on the main stream; group 1 travels (and is waited for) on the side
        stream while the product of group 0 runs."""
        s, side = self.stream, self._side
        (b0, e0, route0, experts0), (b1, e1, route1, experts1) = w["groups"]
        push(b0, e0, s)
        self._barrier(w)
        lib.call("qmoe_event_record", side["first_sent"], s)
        lib.call("qmoe_stream_wait_event", side["stream"], side["first_sent"])
        push(b1, e1, side["stream"])
        self._barrier(w, side["stream"])
        lib.call("qmoe_event_record", side["rest_landed"], side["stream"])
        product(route0, experts0)
        lib.call("qmoe_stream_wait_event", s, side["rest_landed"])
        product(route1, experts1)

    def _raise_on_status(self, code):
        if code:
            what = ("a rank did not arrive at an expert-parallel barrier within the time limit" if code == 201
                    else "a kernel gave up a bounded wait")
            raise RuntimeError(f"{what} (device status {code}): the results of the steps in flight are invalid; "
                               "qmoe_device_status_clear after the cause has been dealt with")

    def _host_counts(self, w):
        """[world][E] counts (physical expert numbers) of the last forward as Python ints.  Waits for that
        forward's count exchange only, not for work enqueued after it, and raises if a kernel up to that point
        (or in the step before) reported a failed bounded wait."""
        lib.call("qmoe_event_sync", w["stats_event"])
        self._raise_on_status(w["host_status"][0] or w["host_status"][1])
        stats, E = w["host_stats"], self.n_experts
        return [[stats[p * 2 * E + e] for e in range(E)] for p in range(self.world)]

    def check_status(self):
        """Wait for everything enqueued on the layer's stream and raise if any kernel reported a failed bounded
        wait (a rank missing at a barrier): the way to be certain about a step's results before using them."""
        self._raise_on_status(lib.device_status(self.stream))

    @property
    def last_counts(self):
        """Global per-expert counts (all ranks' tokens, the model's expert numbers) of the last forward."""
        if self._saved is None:
            return (0,) * self.n_experts
        counts = self._host_counts(self._saved[0])
        physical = [sum(counts[p][e] for p in range(self.world)) for e in range(self.n_experts)]
        return tuple(physical[self._physical_of_logical[e]] for e in range(self.n_experts))

    def _router_operand(self, s):
        """Address of the router weight with rows in physical expert order."""
        weight = self.router.weight.storage
        if self._identity:
            return weight.ptr
        if not self._router_physical.is_derived_from(weight):
            E, d = self.n_experts, self.d_model
            lib.call("qmoe_gather_rows", weight.ptr, self._router_physical.ptr, self._to_physical.ptr, E, E, 4 * d, s)
            self._router_physical.mark_derived_from(weight)
        return self._router_physical.ptr

    def forward(self, x):
        """``x``: this rank's (T / world, d) shard.  Returns ``(y, aux)``; ``aux`` is the global
        auxiliary loss (identical on every rank)."""
        storage = x.storage if hasattr(x, "storage") else x
        d, E, L, k, h, N = self.d_model, self.n_experts, self.local_experts, self.top_k, self.d_expert, self.world
        tokens, dtype = storage.size // d, storage.dtype
        shape = tuple(x.shape) if hasattr(x, "storage") else (tokens, d)
        code, s = lib.DTYPE_CODES[dtype], self.stream
        w = self._workspace(tokens, dtype)
        buf, tr, xr, ex = w["buf"], ctypes.byref(w["token_route"]), ctypes.byref(w["expert_route"]), ctypes.byref(w["experts"])
        side = self._side

        def cast_weights(stream):
            if dtype != "bfloat16":
                return
            pairs = ((self._gate, buf["w_gate"]), (self._up, buf["w_up"]), (self._down, buf["w_down"]))
            if w.get("operands_built") and self.refresh_operands is not True:
                if self.refresh_operands is False or all(copy.is_derived_from(master) for master, copy in pairs):
                    return
            w["operands_built"] = True
            for master, copy in pairs:
                lib.call("qmoe_cast_bf16", master.ptr, copy.ptr, master.size, stream)
                copy.mark_derived_from(master)

        def route_and_plan():
            lib.call("qmoe_router_forward", storage.ptr, code, self._router_operand(s), buf["scores"].ptr,
                     buf["router_partials"].ptr, tokens, d, E, s)
            lib.call("qmoe_route", tr, buf["scores"].ptr, s)
            # the all-gather is also the point no rank passes before every rank has finished its previous step
            if w.get("flag_barrier"):
                self._sequence += 1
                lib.call("qmoe_ep_pack_stats", tr, buf["stats_local"].ptr, s)
                lib.call("qmoe_ep_flag_barrier", ctypes.byref(w["peers"]["flags"]), self._sequence, buf["stats_local"].ptr,
                         2 * E, ctypes.byref(w["peers"]["stats_all"]), s)
                # the host's copy of the counts is only read when gradients are handed out: it leaves on the side
                # stream, together with the status word the barrier kernels report a missing rank in
                lib.call("qmoe_event_record", side["stats"], s)
                lib.call("qmoe_stream_wait_event", side["stream"], side["stats"])
                lib.call("qmoe_memcpy_d2h", ctypes.cast(w["host_stats"], ctypes.c_void_p), buf["stats_all"].ptr, 4 * N * 2 * E,
                         side["stream"])
                lib.call("qmoe_device_status_async", side["stream"], ctypes.cast(w["host_status"], ctypes.c_void_p))
                lib.call("qmoe_event_record", w["stats_event"], side["stream"])
            else:
                lib.call("qmoe_ep_gather_stats", tr, buf["stats_local"].ptr, buf["stats_all"].ptr,
                         ctypes.cast(w["host_stats"], ctypes.c_void_p), s)
                lib.call("qmoe_device_status_async", s, ctypes.cast(w["host_status"], ctypes.c_void_p))
                lib.call("qmoe_event_record", w["stats_event"], s)
            lib.call("qmoe_ep_plan", buf["stats_all"].ptr, tr, xr, tokens * N, s)
            lib.call("qmoe_ep_zero_pad_rows", xr, buf["x_recv"].ptr, code, d, s)

        out = DeviceStorage(storage.size, dtype)
        acts = (buf["x_recv"].ptr, buf["g"].ptr, buf["u"].ptr, buf["h"].ptr, buf["y_recv"].ptr)
        if self.transport == "p2p":
            peers = w["peers"]
            ready, done = side["ready"], side["done"]
            # the bf16 weight copies are refreshed on the side stream while this stream routes and dispatches
            lib.call("qmoe_event_record", ready, s)
            lib.call("qmoe_stream_wait_event", side["stream"], ready)
            cast_weights(side["stream"])
            lib.call("qmoe_event_record", done, side["stream"])
            route_and_plan()
            lib.call("qmoe_ep_dest_base", buf["stats_all"].ptr, E, L, buf["dest_base"].ptr, s)
            if w["groups"]:
                lib.call("qmoe_stream_wait_event", s, done)   # the first product starts right behind its rows
                self._two_phase(
                    w,
                    lambda begin, end, stream: lib.call("qmoe_ep_permute_push_range", tr, buf["dest_base"].ptr, storage.ptr,
                                                        ctypes.byref(peers["x_recv"]), begin, end, code, d, stream),
                    lambda route, experts: lib.call("qmoe_expert_forward_parts", ctypes.byref(route), ctypes.byref(experts),
                                                    *acts, 1, s))
                lib.call("qmoe_ep_expert_down_push", xr, ex, buf["h"].ptr, buf["ret_table"].ptr, ctypes.byref(peers["y_send"]), s)
                self._barrier(w)
                lib.call("qmoe_combine", tr, buf["y_send"].ptr, out.ptr, code, d, s)
                return self._finish_forward(w, buf, out, storage, shape)
            if w["fused"]:
                lib.call("qmoe_ep_permute_push", tr, buf["dest_base"].ptr, storage.ptr, ctypes.byref(peers["x_recv"]), code, d, s)
            else:
                lib.call("qmoe_permute", tr, storage.ptr, buf["x_send"].ptr, code, d, s)
                lib.call("qmoe_ep_push_dispatch", tr, buf["dest_base"].ptr, buf["x_send"].ptr, ctypes.byref(peers["x_recv"]), 1, 0, code, d, s)
            self._barrier(w)
            lib.call("qmoe_stream_wait_event", s, done)
            if w["fused"]:
                lib.call("qmoe_expert_forward_parts", xr, ex, *acts, 1, s)
                lib.call("qmoe_ep_expert_down_push", xr, ex, buf["h"].ptr, buf["ret_table"].ptr, ctypes.byref(peers["y_send"]), s)
            else:
                lib.call("qmoe_expert_forward", xr, ex, *acts, s)
                lib.call("qmoe_ep_push_return", xr, buf["ret_table"].ptr, buf["y_recv"].ptr, ctypes.byref(peers["y_send"]), 0, L, 0, code, d, s)
            self._barrier(w)
        else:
            cast_weights(s)
            route_and_plan()
            lib.call("qmoe_permute", tr, storage.ptr, buf["x_send"].ptr, code, d, s)
            counts = self._host_counts(w)                                              # the one host wait of the step
            plan = plan_exchange(counts, self.rank, N)
            w["sends"], w["recvs"] = _segments(plan["sends"]), _segments(plan["recvs"])
            (sa, sn), (ra, rn) = w["sends"], w["recvs"]
            lib.call("qmoe_ep_exchange", buf["x_send"].ptr, sa, sn, buf["x_recv"].ptr, ra, rn, d, code, s)
            lib.call("qmoe_expert_forward", xr, ex, *acts, s)
            lib.call("qmoe_ep_exchange", buf["y_recv"].ptr, ra, rn, buf["y_send"].ptr, sa, sn, d, code, s)
        lib.call("qmoe_combine", tr, buf["y_send"].ptr, out.ptr, code, d, s)
        return self._finish_forward(w, buf, out, storage, shape)

    def _finish_forward(self, w, buf, out, storage, shape):
        E, s = self.n_experts, self.stream
        if self._identity:
            self.utilization = Tensor(buf["utilization"], (E,))
        else:
            lib.call("qmoe_gather_rows", buf["utilization"].ptr, buf["utilization_logical"].ptr, self._to_logical.ptr, E, E, 4, s)
            self.utilization = Tensor(buf["utilization_logical"], (E,))
        self._saved = (w, storage, shape)
        return Tensor(out, shape), Tensor(buf["aux"], ())

    def backward(self, grad_y, grad_aux=None):
        """Backward of the last forward.  ``grad_aux`` (host float or None) is the gradient of the
        GLOBAL auxiliary loss; every rank passes the same value.  Leaves local expert gradients and
        the all-reduced router gradient in ``parameter.grad``; returns this rank's ``dx``."""
        if self._saved is None:
            raise RuntimeError("backward called before forward")
        w, x_storage, shape = self._saved
        g = grad_y.storage if hasattr(grad_y, "storage") else grad_y
        d, E, L, k, h, N = self.d_model, self.n_experts, self.local_experts, self.top_k, self.d_expert, self.world
        tokens, dtype = x_storage.size // d, x_storage.dtype
        code, s = lib.DTYPE_CODES[dtype], self.stream
        buf, tr, xr, ex = w["buf"], ctypes.byref(w["token_route"]), ctypes.byref(w["expert_route"]), ctypes.byref(w["experts"])
        side = self._side
        ga = 0
        if grad_aux is not None:
            # the routing-backward kernel scales by E / (local tokens); the loss is over all ranks' tokens
            value = float(grad_aux) / N
            if w.get("aux_value") != value:  # uploaded only when it changes (the copy waits for the stream)
                buf["aux_grad"].upload_bytes(ctypes.string_at(ctypes.byref(ctypes.c_float(value)), 4), s)
                w["aux_value"] = value
            ga = buf["aux_grad"].ptr
        views = w["grad_views"]
        owned = {id(views[0])} | {id(t) for group in views[1:] for t in group}
        for parameter in self.parameters():
            if parameter.grad is not None and id(parameter.grad) in owned:
                parameter.grad = Tensor(parameter.grad.storage.copy(s), parameter.shape)
        lib.call("qmoe_ep_zero_pad_rows", xr, buf["dy_recv"].ptr, code, d, s)
        grads = (buf["d_w_gate"].ptr, buf["d_w_up"].ptr, buf["d_w_down"].ptr)
        saved = (buf["x_recv"].ptr, buf["g"].ptr, buf["u"].ptr, buf["h"].ptr, buf["d_h"].ptr, buf["d_g"].ptr, buf["d_u"].ptr)
        flags = bool(w.get("flag_barrier"))
        overlapped = flags and self.reduce_router_gradient   # no other NCCL call in the step: the all-reduce can leave the main stream

        def router_backward():
            lib.call("qmoe_route_backward", tr, buf["d_gate_weights"].ptr, ga, buf["d_scores"].ptr, s)
            lib.call("qmoe_router_backward", buf["d_scores"].ptr, x_storage.ptr, code, self._router_operand(s),
                     buf["dx_router"].ptr, buf["d_w_router"].ptr, buf["router_partials"].ptr, tokens, d, E, s)
            # overlapped: the all-reduce runs on the side stream, beside the last barrier and the un-permute, and
            # is waited for where the router gradient is handed out
            stream = side["stream"] if overlapped else s
            if overlapped:
                lib.call("qmoe_event_record", side["grads"], s)
                lib.call("qmoe_stream_wait_event", stream, side["grads"])
            if self.reduce_router_gradient:
                lib.call("qmoe_ep_all_reduce_f32", buf["d_w_router"].ptr, E * d, stream)
            if not self._identity:   # rows back into the model's expert order
                lib.call("qmoe_gather_rows", buf["d_w_router"].ptr, buf["d_w_router_logical"].ptr, self._to_logical.ptr,
                         E, E, 4 * d, stream)
            if overlapped:
                lib.call("qmoe_event_record", side["reduced"], stream)

        if self.transport == "p2p" and w["fused"]:
            peers = w["peers"]
            if w["groups"]:
                self._two_phase(
                    w,
                    lambda begin, end, stream: lib.call("qmoe_ep_combine_backward_push_range", tr, buf["dest_base"].ptr, g.ptr,
                                                        buf["y_send"].ptr, ctypes.byref(peers["dy_recv"]), buf["d_gate_weights"].ptr,
                                                        begin, end, code, d, stream),
                    lambda route, experts: lib.call("qmoe_expert_backward_parts", ctypes.byref(route), ctypes.byref(experts),
                                                    buf["dy_recv"].ptr, *saved, buf["dx_recv"].ptr, *grads, 1 | 4, s))
            else:
                lib.call("qmoe_ep_combine_backward_push", tr, buf["dest_base"].ptr, g.ptr, buf["y_send"].ptr,
                         ctypes.byref(peers["dy_recv"]), buf["d_gate_weights"].ptr, code, d, s)
                self._barrier(w)
                lib.call("qmoe_expert_backward_parts", xr, ex, buf["dy_recv"].ptr, *saved, buf["dx_recv"].ptr, *grads, 1 | 4, s)
            # dX leaves from the tensor-core epilogue; it has landed long before the barrier below
            lib.call("qmoe_ep_expert_dx_push", xr, ex, buf["d_g"].ptr, buf["d_u"].ptr, buf["ret_table"].ptr, ctypes.byref(peers["dy_send"]), s)
            lib.call("qmoe_expert_backward_parts", xr, ex, buf["dy_recv"].ptr, *saved, buf["dx_recv"].ptr, *grads, 2, s)
            router_backward()
            if flags:  # peers overwrite the gathered counts after this barrier: the host's copy has left by then
                lib.call("qmoe_stream_wait_event", s, w["stats_event"])
            self._barrier(w)
        elif self.transport == "p2p":
            peers = w["peers"]
            lib.call("qmoe_combine_backward", tr, g.ptr, buf["y_send"].ptr, buf["dy_send"].ptr, buf["d_gate_weights"].ptr, code, d, s)
            lib.call("qmoe_ep_push_dispatch", tr, buf["dest_base"].ptr, buf["dy_send"].ptr, ctypes.byref(peers["dy_recv"]), 0, 0, code, d, s)
            self._barrier(w)
            lib.call("qmoe_expert_backward_parts", xr, ex, buf["dy_recv"].ptr, *saved, buf["dx_recv"].ptr, *grads, 3, s)
            lib.call("qmoe_ep_push_return", xr, buf["ret_table"].ptr, buf["dx_recv"].ptr, ctypes.byref(peers["dy_send"]), 0, L, 0, code, d, s)
            router_backward()
            if flags:
                lib.call("qmoe_stream_wait_event", s, w["stats_event"])
            self._barrier(w)
        else:
            lib.call("qmoe_combine_backward", tr, g.ptr, buf["y_send"].ptr, buf["dy_send"].ptr, buf["d_gate_weights"].ptr, code, d, s)
            (sa, sn), (ra, rn) = w["sends"], w["recvs"]
            lib.call("qmoe_ep_exchange", buf["dy_send"].ptr, sa, sn, buf["dy_recv"].ptr, ra, rn, d, code, s)
            lib.call("qmoe_expert_backward", xr, ex, buf["dy_recv"].ptr, *saved, buf["dy_recv"].ptr, *grads, s)  # dX reuses dY's buffer
            lib.call("qmoe_ep_exchange", buf["dy_recv"].ptr, ra, rn, buf["dy_send"].ptr, sa, sn, d, code, s)
            router_backward()
        dx = DeviceStorage(x_storage.size, dtype)
        lib.call("qmoe_unpermute_reduce", tr, buf["dy_send"].ptr, buf["dx_router"].ptr, dx.ptr, code, d, s)
        # the status word at the end of the step leaves on the side stream; it is looked at together with the next
        # step's counts (or by check_status), so the host still waits for nothing here
        lib.call("qmoe_event_record", side["ended"], s)
        lib.call("qmoe_stream_wait_event", side["stream"], side["ended"])
        lib.call("qmoe_device_status_async", side["stream"], ctypes.cast(ctypes.addressof(w["host_status"].contents) + 4, ctypes.c_void_p))
        # which local experts received rows decides who gets a gradient object: host logic on the forward's
        # counts, read only now so that the device never waits for the host inside the step
        counts = self._host_counts(w)
        received = [sum(counts[p][self.rank * L + j] for p in range(N)) for j in range(L)]
        if overlapped:
            lib.call("qmoe_stream_wait_event", s, side["reduced"])
        _accumulate(self.router.weight, views[0], s)
        for j, expert in enumerate(self.experts):
            if not received[j]:
                continue
            gate, up, down = views[1 + j]
            _accumulate(expert.gate.weight, gate, s)
            _accumulate(expert.up.weight, up, s)
            _accumulate(expert.down.weight, down, s)
        return Tensor(dx, shape)
