"""``SparseMoE`` for ``device="cuda"`` on B200: the host-side mirror of the upstream layer
(src/qutai/lm/layers.py:354-408) over ``libqutai_moe.so``.

Same constructor (``SparseMoE(config, *, device, dtype, seed)``), same attributes (``router``,
``experts[i].gate/up/down`` with ``.weight`` of shape (outputs, inputs), ``top_k``, ``n_experts``,
``utilization``, ``last_counts``) and the same ``parameters()`` order, so the parameter naming used
by checkpoints (src/qutai/lm/decoder.py:57-68) is unchanged.  What differs is how the work runs:
one fused call per direction (router logits, routing, permute, grouped expert FFN, combine) instead
of a Python loop over experts, with no host synchronisation inside the layer.  The expert weights
of one kind live in ONE stacked buffer ([E, h, d] / [E, d, h]); every ``weight`` is a view into it.

``__call__``/``forward`` returns ``(y, aux)``; ``backward(grad_y, grad_aux)`` plays the role of the
closures the upstream layer registers with autograd and leaves gradients in ``parameter.grad``
(``None`` for an expert that received no token, as upstream, src/qutai/lm/layers.py:396).  A
gradient produced by ``backward`` is a view of the layer's stacked gradient buffer and stays valid
until the next ``backward`` of the same layer (which first copies out any gradient still in use).
"""
from __future__ import annotations

import ctypes
from math import prod, sqrt

from . import lib
from .storage import DeviceStorage


class Tensor:
    """Shape + storage + grad, with the attribute names of the upstream ``Tensor``
    (src/qutai/core/tensor.py:14-33); just enough for parameters and activations of this layer."""

    def __init__(self, storage, shape=None, requires_grad=False):
        self.parents, self.backward_rule = (), None     # the fields upstream's ``record`` fills in
        self.storage = storage
        self.shape = tuple(shape) if shape is not None else (storage.size,)
        if prod(self.shape) != storage.size:
            raise ValueError("element count does not match the shape")
        self.requires_grad = requires_grad
        self.grad = None

    device = "cuda"

    @property
    def dtype(self):
        return self.storage.dtype

    @property
    def size(self):
        return self.storage.size

    def tolist(self):
        return self.storage.tolist()

    def zero_grad(self):
        self.grad = None


class ForwardGraph:
    """A recorded forward of one ``SparseMoE`` on one input buffer (``SparseMoE.capture_forward``).  Keeps the
    workspace, the input and the output alive; a forward with another token count in between does not disturb it."""

    def __init__(self, layer, graph, work, x_storage, shape, y, aux):
        self.layer, self.graph, self.work, self.x_storage, self.shape, self.y, self.aux = layer, graph, work, x_storage, shape, y, aux

    def replay(self):
        layer = self.layer
        lib.call("qmoe_graph_launch", self.graph, layer.stream)
        layer._counts_valid = "stream"
        layer.utilization = Tensor(self.work["buf"]["utilization"], (layer.n_experts,))
        layer._saved = (self.work, self.x_storage, self.shape)
        return self.y, self.aux

    def __del__(self):
        graph, self.graph = getattr(self, "graph", 0), 0
        if graph:
            try:
                lib.load().qmoe_graph_destroy(graph)
            except Exception:
                pass


class Projection:
    """Bias-free linear map with ``weight`` of shape (outputs, inputs) (src/qutai/lm/layers.py:260-272)."""

    def __init__(self, weight):
        self.weight = weight

    def parameters(self):
        return (self.weight,)


class SwiGLU:
    """Holder of one expert's three projections (src/qutai/lm/layers.py:291-314)."""

    def __init__(self, gate, up, down):
        self.gate, self.up, self.down = Projection(gate), Projection(up), Projection(down)

    def parameters(self):
        return (*self.gate.parameters(), *self.up.parameters(), *self.down.parameters())


def _accumulate(parameter, view, stream):
    """Leaf accumulation (src/qutai/core/tensor.py:203-210).  The first contribution is handed out
    as a view of the layer's stacked gradient buffer (no copy); a later one is summed into a fresh
    storage."""
    if parameter.grad is None:
        parameter.grad = view
        return
    out = DeviceStorage(view.size, view.storage.dtype)
    lib.call("qmoe_add", parameter.grad.storage.ptr, view.storage.ptr, out.ptr,
             lib.DTYPE_CODES[view.storage.dtype], view.size, stream)
    parameter.grad = Tensor(out, parameter.shape)


class SparseMoE:
    def __init__(self, config, *, device="cuda", dtype="float32", seed=None, engine="auto", stream=0):
        if device != "cuda":
            raise ValueError("this layer only runs on device='cuda' (there is no CPU fallback)")
        if dtype != "float32":
            raise ValueError("parameters are float32 (bf16 is an activation dtype, as upstream)")
        d, E, h = config.d_model, config.n_experts, config.d_expert
        if not 1 <= config.top_k <= min(E, lib.MAX_TOP_K) or E > lib.MAX_EXPERTS:
            raise ValueError(f"need 1 <= top_k <= min(n_experts, {lib.MAX_TOP_K}) and n_experts <= {lib.MAX_EXPERTS}")
        self.top_k, self.n_experts, self.d_model, self.d_expert = config.top_k, E, d, h
        self.stream = stream
        self.engine = {"auto": lib.ENGINE_AUTO, "simt": lib.ENGINE_SIMT, "tcgen05": lib.ENGINE_TCGEN05}[engine]
        self._gate = DeviceStorage(E * h * d, "float32")
        self._up = DeviceStorage(E * h * d, "float32")
        self._down = DeviceStorage(E * d * h, "float32")
        router = DeviceStorage(E * d, "float32")
        down_std = 0.02 / sqrt(2 * config.n_layers)

        def fill(storage, std, tensor_seed):
            # one generator stream per parameter tensor, keyed like upstream: router seed, expert i
            # gate seed+1+3i, up +1, down +2 (src/qutai/lm/layers.py:355-371, :292-308)
            storage.fill_normal(0.0, std, 0x5EED if tensor_seed is None else tensor_seed, stream)

        fill(router, 0.02, seed)
        self.router = Projection(Tensor(router, (E, d), requires_grad=True))
        experts = []
        for i in range(E):
            views = (self._gate.view(i * h * d, h * d), self._up.view(i * h * d, h * d), self._down.view(i * d * h, d * h))
            base = None if seed is None else seed + 1 + 3 * i
            fill(views[0], 0.02, base)
            fill(views[1], 0.02, None if base is None else base + 1)
            fill(views[2], down_std, None if base is None else base + 2)
            experts.append(SwiGLU(Tensor(views[0], (h, d), requires_grad=True),
                                  Tensor(views[1], (h, d), requires_grad=True),
                                  Tensor(views[2], (d, h), requires_grad=True)))
        self.experts = tuple(experts)
        self.utilization = None
        # "auto": the bf16 operand copies of the fp32 weights are rebuilt by a forward only when a weight storage
        # was written since they were made (``DeviceStorage.generation``; upstream pays nothing either, it rounds
        # while staging tiles, src/qutai/backends/cuda/gemm.cu:122-127).  True rebuilds at every forward (for
        # weights that are written through raw addresses), False never after the first forward.
        self.refresh_operands = "auto"
        self._counts_host = None
        self._counts_valid = False
        self._zero_counts = (0,) * E
        self._work = {}
        self._saved = None

    # ------------------------------------------------------------------------------------------
    def parameters(self):
        return (*self.router.parameters(), *(p for expert in self.experts for p in expert.parameters()))

    def operand_shadows(self, tokens=None):
        """``{parameter: bf16 storage}`` of the tensor-core operand copies of the expert weights (those of the
        last bf16 forward, or of the workspace for ``tokens``).  An optimizer that writes the rounded weights
        there (``qutai_b200.optim.AdamW(shadows=...)``) keeps them current across its steps, so the forward
        after a step converts nothing (with ``refresh_operands`` left at "auto")."""
        works = [w for (t, dtype), w in self._work.items() if dtype == "bfloat16" and (tokens is None or t == tokens)]
        if self._saved is not None and any(w is self._saved[0] for w in works):
            works = [self._saved[0]]
        if not works:
            raise RuntimeError("no bfloat16 forward has run yet")
        buf, h, d = works[-1]["buf"], self.d_expert, self.d_model
        shadows = {}
        for i, expert in enumerate(self.experts):
            shadows[expert.gate.weight] = buf["w_gate"].view(i * h * d, h * d)
            shadows[expert.up.weight] = buf["w_up"].view(i * h * d, h * d)
            shadows[expert.down.weight] = buf["w_down"].view(i * d * h, d * h)
        return shadows

    @property
    def last_counts(self):
        """Tokens routed to each expert in the last forward, as Python ints.  Reading it is the
        only thing that waits for the device (upstream downloads the counts inside every forward,
        src/qutai/backends/cuda_lm.py:432-434)."""
        if not self._counts_valid:
            return self._zero_counts
        if self._counts_valid == "stream":  # the last forward was a graph replay: its copy is a node of the graph
            lib.call("qmoe_stream_sync", self.stream)
        else:
            lib.call("qmoe_event_sync", self._counts_event)  # waits for the forward's routing only, not for later work
        return tuple(self._counts_host[i] for i in range(self.n_experts))

    # ------------------------------------------------------------------------------------------
    def _workspace(self, tokens, dtype):
        key = (tokens, dtype)
        work = self._work.get(key)
        if work is not None:
            return work
        E, k, d, h = self.n_experts, self.top_k, self.d_model, self.d_expert
        A = tokens * k
        R = lib.rows_bound(tokens, E, k)
        blocks = lib.route_blocks(tokens)
        S = DeviceStorage
        buf = dict(
            probs=S(tokens * E, "float32"), gate_weights=S(A, "float32"), expert_index=S(A, "int32"),
            dest_row=S(A, "int32"), row_source=S(R, "int32"), counts=S(E, "int32"), offsets=S(E + 1, "int32"),
            tile_expert=S(R // lib.ROW_PAD, "int32"), meta=S(4, "int32"), utilization=S(E, "float32"),
            aux=S(1, "float32"), block_counts=S(blocks * E, "int32"), block_base=S(blocks * E, "int32"),
            block_colsum=S(blocks * E, "float32"),
            scores=S(tokens * E, "float32"),
            x_dispatched=S(R * d, dtype), g=S(R * h, dtype), u=S(R * h, dtype), h=S(R * h, dtype),
            y_dispatched=S(R * d, dtype),
            dy_dispatched=S(R * d, dtype), d_h=S(R * h, dtype), d_g=S(R * h, dtype), d_u=S(R * h, dtype),
            d_gate_weights=S(A, "float32"), d_scores=S(tokens * E, "float32"), dx_router=S(tokens * d, "float32"),
            router_partials=S(int(lib.load().qmoe_router_grad_partials(tokens, E, d)), "float32"),
            d_w_router=S(E * d, "float32"), d_w_gate=S(E * h * d, "float32"), d_w_up=S(E * h * d, "float32"),
            d_w_down=S(E * d * h, "float32"),
        )
        if dtype == "bfloat16":
            buf.update(w_gate=S(E * h * d, "bfloat16"), w_up=S(E * h * d, "bfloat16"), w_down=S(E * d * h, "bfloat16"))
        layer = lib.Layer()
        route = layer.route
        route.tokens, route.experts, route.top_k, route.rows_bound = tokens, E, k, R
        for name in ("probs", "gate_weights", "expert_index", "dest_row", "row_source", "counts", "offsets",
                     "tile_expert", "meta", "utilization", "aux", "block_counts", "block_base", "block_colsum"):
            setattr(route, name, buf[name].ptr)
        ex = layer.experts
        ex.experts, ex.dtype, ex.engine, ex.width, ex.hidden = E, lib.DTYPE_CODES[dtype], self.engine, d, h
        if dtype == "bfloat16":
            ex.w_gate, ex.w_up, ex.w_down = buf["w_gate"].ptr, buf["w_up"].ptr, buf["w_down"].ptr
            layer.master_gate, layer.master_up, layer.master_down = self._gate.ptr, self._up.ptr, self._down.ptr
        else:
            ex.w_gate, ex.w_up, ex.w_down = self._gate.ptr, self._up.ptr, self._down.ptr
        layer.w_router = self.router.weight.storage.ptr
        for name in ("scores", "x_dispatched", "g", "u", "h", "y_dispatched", "dy_dispatched", "d_h", "d_g", "d_u",
                     "d_gate_weights", "d_scores", "dx_router", "router_partials", "d_w_router", "d_w_gate",
                     "d_w_up", "d_w_down"):
            setattr(layer, name, buf[name].ptr)
        layer.dx_dispatched = buf["dy_dispatched"].ptr  # dX reuses dY's buffer (written after its last reader)
        if self._counts_host is None:
            host, event, routed, side = ctypes.c_void_p(), ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
            lib.call("qmoe_host_alloc", ctypes.byref(host), 4 * E)
            lib.call("qmoe_event_create", ctypes.byref(event))
            lib.call("qmoe_event_create", ctypes.byref(routed))
            lib.call("qmoe_stream_create", ctypes.byref(side))
            self._counts_host = ctypes.cast(host, ctypes.POINTER(ctypes.c_int32))
            self._counts_event, self._routed_event, self._copy_stream = event.value, routed.value, side.value
        grad_views = [Tensor(buf["d_w_router"], (E, d))]
        for i in range(E):
            grad_views.append((Tensor(buf["d_w_gate"].view(i * h * d, h * d), (h, d)),
                               Tensor(buf["d_w_up"].view(i * h * d, h * d), (h, d)),
                               Tensor(buf["d_w_down"].view(i * d * h, d * h), (d, h))))
        work = dict(buf=buf, layer=layer, rows_bound=R, grad_views=grad_views)
        self._work = {key: work}  # one token count at a time keeps memory bounded
        return work

    def _operands_current(self, work):
        """True when this forward can keep the bf16 operand copies it finds in the workspace."""
        buf = work["buf"]
        if "w_gate" not in buf or not work.get("operands_built") or self.refresh_operands is True:
            return False
        if self.refresh_operands is False:
            return True
        return (buf["w_gate"].is_derived_from(self._gate) and buf["w_up"].is_derived_from(self._up)
                and buf["w_down"].is_derived_from(self._down))

    def _operands_made(self, work):
        """A forward that converted the weights has been enqueued: the copies follow the weights as they are now."""
        buf = work["buf"]
        work["operands_built"] = True
        if "w_gate" in buf:
            buf["w_gate"].mark_derived_from(self._gate)
            buf["w_up"].mark_derived_from(self._up)
            buf["w_down"].mark_derived_from(self._down)

    def __call__(self, x):
        return self.forward(x)

    def forward(self, x):
        """``x``: Tensor (or storage + implicit (T, d)) of float32 or bfloat16 activations on the
        device.  Returns ``(y, aux)``: ``y`` shaped like ``x`` in the same dtype, ``aux`` a float32
        scalar tensor (src/qutai/lm/layers.py:376-402)."""
        storage = x.storage if hasattr(x, "storage") else x
        shape = tuple(x.shape) if hasattr(x, "shape") and not hasattr(x, "ptr") else (storage.size // self.d_model, self.d_model)
        if shape[-1] != self.d_model or storage.dtype not in lib.DTYPE_CODES:
            raise ValueError("input must be (..., d_model) float32 or bfloat16")
        tokens = storage.size // self.d_model
        work = self._workspace(tokens, storage.dtype)
        layer, buf = work["layer"], work["buf"]
        out = DeviceStorage(storage.size, storage.dtype)
        layer.x, layer.out = storage.ptr, out.ptr
        masters = (layer.master_gate, layer.master_up, layer.master_down)
        keep = self._operands_current(work)
        if keep:
            layer.master_gate = layer.master_up = layer.master_down = 0   # keep the bf16 copies of the last forward
        if self._counts_valid is True:  # the previous forward's counts have left before routing overwrites them
            lib.call("qmoe_stream_wait_event", self.stream, self._counts_event)
        lib.call("qmoe_layer_forward", ctypes.byref(layer), self.stream)
        layer.master_gate, layer.master_up, layer.master_down = masters
        if not keep:
            self._operands_made(work)
        self._publish_counts(buf)
        self.utilization = Tensor(buf["utilization"], (self.n_experts,))
        self._saved = (work, storage, shape)
        return Tensor(out, shape), Tensor(buf["aux"], ())

    def _publish_counts(self, buf):
        """Start the host's copy of the counts of the forward just enqueued.  It travels on a stream of its own: a
        device-to-host copy queued on the caller's stream would wait behind whatever large copy-out the caller
        has in flight on the same copy engine, and every kernel after it would wait too."""
        lib.call("qmoe_event_record", self._routed_event, self.stream)
        lib.call("qmoe_stream_wait_event", self._copy_stream, self._routed_event)
        lib.call("qmoe_memcpy_d2h", ctypes.cast(self._counts_host, ctypes.c_void_p), buf["counts"].ptr,
                 4 * self.n_experts, self._copy_stream)
        lib.call("qmoe_event_record", self._counts_event, self._copy_stream)
        self._counts_valid = True

    def _release_aliased_gradients(self, work):
        """A ``parameter.grad`` that still aliases the stacked gradient buffers about to be overwritten is copied out."""
        views = work["grad_views"]
        owned = {id(views[0].storage)} | {id(t.storage) for group in views[1:] for t in group}
        for parameter in self.parameters():
            if parameter.grad is not None and id(parameter.grad.storage) in owned:
                parameter.grad = type(parameter.grad)(parameter.grad.storage.copy(self.stream), shape=parameter.shape)

    def capture_forward(self, x):
        """Record the forward on ``x``'s buffer as a CUDA graph (the decode-shaped call is a dozen short kernels:
        one graph launch replaces their launches).  Returns a ``ForwardGraph``; ``replay()`` reruns the forward on
        whatever ``x`` holds then and returns the same ``(y, aux)`` tensors every time.  The layer must run on a
        stream of its own (``stream != 0``).  Unless ``refresh_operands`` is True the recording keeps the bf16
        operand copies as they are at capture time: after a weight update run one plain ``forward`` (which
        rebuilds them) before the next replay."""
        if not self.stream:
            raise ValueError("capture needs a layer whose stream is not the default stream")
        self.forward(x)                                    # once without capture: workspace, kernel attributes
        storage = x.storage if hasattr(x, "storage") else x
        work, _, shape = self._saved
        layer, buf = work["layer"], work["buf"]
        out = DeviceStorage(storage.size, storage.dtype)   # allocated before the capture starts
        lib.call("qmoe_event_sync", self._counts_event)
        layer.x, layer.out = storage.ptr, out.ptr
        masters = (layer.master_gate, layer.master_up, layer.master_down)
        if self.refresh_operands is not True:   # the forward above has just built them
            layer.master_gate = layer.master_up = layer.master_down = 0
        graph = ctypes.c_uint64()
        lib.call("qmoe_graph_begin", self.stream)
        try:
            lib.call("qmoe_layer_forward", ctypes.byref(layer), self.stream)
            lib.call("qmoe_memcpy_d2h", ctypes.cast(self._counts_host, ctypes.c_void_p), buf["counts"].ptr,
                     4 * self.n_experts, self.stream)
        except Exception:
            lib.load().qmoe_graph_abandon(self.stream)
            raise
        finally:
            layer.master_gate, layer.master_up, layer.master_down = masters
        lib.call("qmoe_graph_end", self.stream, ctypes.byref(graph))
        return ForwardGraph(self, graph.value, work, storage, shape, Tensor(out, shape), Tensor(buf["aux"], ()))

    def backward_contributions(self, grad_y, grad_aux=None):
        """The backward of the last forward as autograd sees it: returns ``(dx, d_router, experts)`` where
        ``experts[i]`` is ``None`` for an expert that received no token (upstream never calls such an expert, so
        its parameters get no contribution, src/qutai/lm/layers.py:396) and else the ``(d_gate, d_up, d_down)``
        tensors.  ``parameter.grad`` is not touched.  The weight contributions are views of the layer's stacked
        gradient buffers and stay valid until the next backward of this layer; a ``parameter.grad`` that still
        aliases them is copied out first."""
        if self._saved is None:
            raise RuntimeError("backward called before forward")
        work, x_storage, shape = self._saved
        layer, buf = work["layer"], work["buf"]
        g = grad_y.storage if hasattr(grad_y, "storage") else grad_y
        if g.size != x_storage.size or g.dtype != x_storage.dtype:
            raise ValueError("grad_y must match the output's size and dtype")
        ga = None if grad_aux is None else (grad_aux.storage if hasattr(grad_aux, "storage") else grad_aux)
        views = work["grad_views"]
        self._release_aliased_gradients(work)
        dx = DeviceStorage(x_storage.size, x_storage.dtype)
        layer.grad_out, layer.grad_aux, layer.dx = g.ptr, 0 if ga is None else ga.ptr, dx.ptr
        lib.call("qmoe_layer_backward", ctypes.byref(layer), self.stream)
        # which experts get a gradient object is host logic on the forward's counts; they are read only
        # now, after the whole backward is enqueued, so the device never idles waiting for the host
        counts = self.last_counts
        return Tensor(dx, shape), views[0], [views[1 + i] if counts[i] else None for i in range(self.n_experts)]

    def backward_aux(self, grad_aux):
        """The auxiliary loss' own path through the last forward (upstream records it as a node of its own,
        src/qutai/lm/layers.py:387-391): returns ``(dx, d_router)`` for the float32 scalar ``grad_aux`` in fresh
        storages; touches neither ``parameter.grad`` nor the buffers of ``backward_contributions``."""
        if self._saved is None:
            raise RuntimeError("backward_aux called before forward")
        work, x_storage, shape = self._saved
        layer, buf = work["layer"], work["buf"]
        ga = grad_aux.storage if hasattr(grad_aux, "storage") else grad_aux
        tokens, d, E = x_storage.size // self.d_model, self.d_model, self.n_experts
        code = lib.DTYPE_CODES[x_storage.dtype]
        d_router = DeviceStorage(E * d, "float32")
        dx32 = DeviceStorage(tokens * d, "float32")
        lib.call("qmoe_route_backward", ctypes.byref(layer.route), 0, ga.ptr, buf["d_scores"].ptr, self.stream)
        lib.call("qmoe_router_backward", buf["d_scores"].ptr, x_storage.ptr, code, self.router.weight.storage.ptr,
                 dx32.ptr, d_router.ptr, buf["router_partials"].ptr, tokens, d, E, self.stream)
        if x_storage.dtype == "bfloat16":
            dx = DeviceStorage(tokens * d, "bfloat16")
            lib.call("qmoe_cast_bf16", dx32.ptr, dx.ptr, tokens * d, self.stream)
        else:
            dx = dx32
        return Tensor(dx, shape), Tensor(d_router, (E, d))

    def backward(self, grad_y, grad_aux=None):
        """Propagate ``grad_y`` (shaped like the output) and optionally ``grad_aux`` (float32
        scalar storage/tensor) through the last forward.  Accumulates into ``parameter.grad`` and
        returns the gradient of the input as a Tensor."""
        dx, d_router, experts = self.backward_contributions(grad_y, grad_aux)
        _accumulate(self.router.weight, d_router, self.stream)
        for expert, contribution in zip(self.experts, experts):
            if contribution is None:
                continue
            gate, up, down = contribution
            _accumulate(expert.gate.weight, gate, self.stream)
            _accumulate(expert.up.weight, up, self.stream)
            _accumulate(expert.down.weight, down, self.stream)
        return dx


class RMSNorm:
    """Holder of the norm's weight and epsilon, with upstream's constructor (src/qutai/lm/layers.py:275-288):
    ``weight`` of shape (width,), ones, float32.  The arithmetic runs inside ``MoEFeedForward``."""

    def __init__(self, width, eps, *, device="cuda", dtype="float32", stream=0):
        if device != "cuda" or dtype != "float32":
            raise ValueError("the norm weight is float32 on device='cuda'")
        storage = DeviceStorage.from_values([1.0] * width, "float32", stream)
        self.weight = Tensor(storage, (width,), requires_grad=True)
        self.eps = float(eps)

    def parameters(self):
        return (self.weight,)


class MoEFeedForward:
    """The feed-forward half of upstream's ``Block.__call__`` for a mixture-of-experts block
    (src/qutai/lm/layers.py:430-437): ``(x + ffn(ffn_norm(x)), aux)``, with the norm and the residual fused into
    the layer's first read and last write (``qmoe_block_forward`` / ``qmoe_block_backward``): no normalised copy of
    the activations is written, the expert input is normalised while it is gathered, the residual is added
    before the combine's single rounding, and in the backward the gather-sum of the input gradient applies the
    norm's backward and adds the residual's gradient.  ``ffn_norm`` and ``ffn`` carry upstream's attribute names."""

    def __init__(self, ffn_norm, ffn):
        if ffn_norm.weight.size != ffn.d_model:
            raise ValueError("the norm's width must be the layer's d_model")
        self.ffn_norm, self.ffn = ffn_norm, ffn
        self._blocks = {}

    def parameters(self):
        return (*self.ffn_norm.parameters(), *self.ffn.parameters())

    def _block(self, work, tokens):
        block = self._blocks.get(id(work))
        if block is None:
            moe = self.ffn
            E, d = moe.n_experts, moe.d_model
            S = DeviceStorage
            extra = dict(inverse=S(tokens, "float32"), w_router_folded=S(E * d, "float32"), d_norm_weight=S(d, "float32"),
                         norm_partials=S(int(lib.load().qmoe_norm_backward_partials(tokens, d)), "float32"))
            block = dict(struct=lib.Block(), extra=extra, work=work)
            for name, storage in extra.items():
                setattr(block["struct"], name, storage.ptr)
            self._blocks = {id(work): block}   # follows the layer's one-workspace-at-a-time rule
        return block

    def __call__(self, x):
        return self.forward(x)

    def forward(self, x):
        """``x``: (..., d_model) float32 or bfloat16.  Returns ``(x + ffn(ffn_norm(x)), aux)``."""
        moe = self.ffn
        storage = x.storage if hasattr(x, "storage") else x
        shape = tuple(x.shape) if hasattr(x, "shape") and not hasattr(x, "ptr") else (storage.size // moe.d_model, moe.d_model)
        if shape[-1] != moe.d_model or storage.dtype not in lib.DTYPE_CODES:
            raise ValueError("input must be (..., d_model) float32 or bfloat16")
        tokens = storage.size // moe.d_model
        work = moe._workspace(tokens, storage.dtype)
        block = self._block(work, tokens)
        layer, buf, struct = work["layer"], work["buf"], block["struct"]
        out = DeviceStorage(storage.size, storage.dtype)
        layer.x, layer.out = storage.ptr, out.ptr
        masters = (layer.master_gate, layer.master_up, layer.master_down)
        keep = moe._operands_current(work)
        if keep:
            layer.master_gate = layer.master_up = layer.master_down = 0
        struct.layer = layer
        struct.norm_weight, struct.norm_eps = self.ffn_norm.weight.storage.ptr, self.ffn_norm.eps
        if moe._counts_valid is True:
            lib.call("qmoe_stream_wait_event", moe.stream, moe._counts_event)
        lib.call("qmoe_block_forward", ctypes.byref(struct), moe.stream)
        layer.master_gate, layer.master_up, layer.master_down = masters
        if not keep:
            moe._operands_made(work)
        moe._publish_counts(buf)
        moe.utilization = Tensor(buf["utilization"], (moe.n_experts,))
        moe._saved = (work, storage, shape)
        return Tensor(out, shape), Tensor(buf["aux"], ())

    def backward(self, grad_out, grad_aux=None):
        """Gradient of the block's input for ``grad_out`` (shaped like the output; it also flows through the
        residual) and the optional float32 scalar ``grad_aux``; accumulates into every ``parameter.grad``."""
        moe = self.ffn
        if moe._saved is None:
            raise RuntimeError("backward called before forward")
        work, x_storage, shape = moe._saved
        block = self._blocks.get(id(work))
        if block is None:
            raise RuntimeError("the last forward of the layer did not go through this block")
        layer, struct = work["layer"], block["struct"]
        g = grad_out.storage if hasattr(grad_out, "storage") else grad_out
        if g.size != x_storage.size or g.dtype != x_storage.dtype:
            raise ValueError("grad_out must match the output's size and dtype")
        ga = None if grad_aux is None else (grad_aux.storage if hasattr(grad_aux, "storage") else grad_aux)
        moe._release_aliased_gradients(work)
        dx = DeviceStorage(x_storage.size, x_storage.dtype)
        layer.x, layer.grad_out, layer.grad_aux, layer.dx = x_storage.ptr, g.ptr, 0 if ga is None else ga.ptr, dx.ptr
        struct.layer = layer
        struct.norm_weight, struct.norm_eps = self.ffn_norm.weight.storage.ptr, self.ffn_norm.eps
        lib.call("qmoe_block_backward", ctypes.byref(struct), moe.stream)
        views = work["grad_views"]
        counts = moe.last_counts
        d_norm = Tensor(block["extra"]["d_norm_weight"].copy(moe.stream), (moe.d_model,))   # the buffer is reused by the next backward
        _accumulate(self.ffn_norm.weight, d_norm, moe.stream)
        _accumulate(moe.router.weight, views[0], moe.stream)
        for i, expert in enumerate(moe.experts):
            if not counts[i]:
                continue
            gate, up, down = views[1 + i]
            _accumulate(expert.gate.weight, gate, moe.stream)
            _accumulate(expert.up.weight, up, moe.stream)
            _accumulate(expert.down.weight, down, moe.stream)
        return Tensor(dx, shape)
