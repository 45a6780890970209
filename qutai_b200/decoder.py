"""A mixture-of-experts decoder over this package's layers and function table: the upstream ``Decoder`` with
``ffn_type="moe"`` (src/qutai/lm/decoder.py:20-175, blocks src/qutai/lm/layers.py:316-449) — token embedding, per block
``x += attn(attn_norm(x))`` (grouped-query attention with rotary embedding) and ``x += ffn(ffn_norm(x))`` (the MoE
layer), a final norm, and the tied-embedding head with its cross-entropy loss plus ``aux_loss_coef`` times the mean
auxiliary loss of the blocks.

Same constructor fields, parameter names (``named_parameters``) and loss as upstream; forward and backward are
written out by hand over the fused pieces instead of a general autograd: ``loss(tokens)`` runs the forward and keeps
what the backward needs, ``backward()`` fills ``parameter.grad`` of every parameter (float32), ready for
``qutai_b200.optim.AdamW``.  With ``world > 1`` the decoder is one rank of a data- and expert-parallel job (upstream has
no such mode): every rank holds its own sequences, the dense parameters are replicated and their gradients summed over
the ranks, every block's experts are spread over the ranks (``ExpertParallelMoE``), and the loss is the mean over all
ranks' targets.  Activations are bfloat16 throughout (the residual stream too: upstream keeps float32
there and hands float32 from its norms to bf16 products), parameters float32 with bf16 operand copies that are
renewed only when a parameter's storage changed.  Head width 64 only (``qutai_b200.attention``).  Dependency-free.
"""
from __future__ import annotations

from array import array
from dataclasses import dataclass
from math import sqrt

from . import lib
from .attention import attention_backward, attention_forward
from .expert_parallel import ExpertParallelMoE
from .head import LMHead
from .layers import MoEFeedForward, RMSNorm, SparseMoE, Tensor
from .storage import DeviceStorage


@dataclass
class Config:
    """The fields of upstream's ``Config`` (src/qutai/lm/config.py:5-21) that a MoE decoder reads."""
    vocab_size: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    n_layers: int
    n_experts: int
    top_k: int
    d_expert: int
    norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    aux_loss_coef: float = 0.01
    ffn_type: str = "moe"


def _accumulate(parameter, storage, stream):
    """Leaf accumulation (src/qutai/core/tensor.py:203-210): the first contribution becomes ``grad``, later ones are added."""
    if parameter.grad is None:
        parameter.grad = Tensor(storage, parameter.shape)
    else:
        lib.call("qmoe_add", parameter.grad.storage.ptr, storage.ptr, parameter.grad.storage.ptr, lib.QMOE_F32, storage.size, stream)


class Linear:
    """``y = x W^T`` without bias (upstream ``Projection`` + ``linear``, src/qutai/lm/layers.py:35-74, :260-272):
    ``weight`` [out, in] float32, bf16 operand copy, bf16 activations; the three products go through ``qmoe_gemm``
    (tensor cores when the row count is a multiple of 128)."""

    def __init__(self, width_in, width_out, *, std, seed, stream=0):
        storage = DeviceStorage(width_out * width_in, "float32")
        storage.fill_normal(0.0, std, 0x5EED if seed is None else seed, stream)
        self.weight = Tensor(storage, (width_out, width_in), requires_grad=True)
        self.width_in, self.width_out, self.stream = width_in, width_out, stream
        self._operand = DeviceStorage(storage.size, "bfloat16")

    def parameters(self):
        return (self.weight,)

    def operand(self):
        if not self._operand.is_derived_from(self.weight.storage):
            lib.call("qmoe_cast_bf16", self.weight.storage.ptr, self._operand.ptr, self.weight.storage.size, self.stream)
            self._operand.mark_derived_from(self.weight.storage)
        return self._operand

    def _gemm(self, a, b, c, m, k, n, ta, tb, c_dtype):
        lib.call("qmoe_gemm", a.ptr, lib.QMOE_BF16, b.ptr, lib.QMOE_BF16, c.ptr, c_dtype, m, k, n, ta, tb, 0, self.stream)

    def forward(self, x, rows):
        y = DeviceStorage(rows * self.width_out, "bfloat16")
        self._gemm(x, self.operand(), y, rows, self.width_in, self.width_out, 0, 1, lib.QMOE_BF16)
        return y

    def backward(self, dy, x, rows):
        """Input gradient [rows, in] (bf16); the weight gradient [out, in] (float32) is accumulated into ``weight.grad``."""
        dx = DeviceStorage(rows * self.width_in, "bfloat16")
        self._gemm(dy, self.operand(), dx, rows, self.width_out, self.width_in, 0, 0, lib.QMOE_BF16)
        dw = DeviceStorage(self.weight.storage.size, "float32")
        partials = lib.load().qmoe_gemm_wgrad_partials(self.width_out, rows, self.width_in)
        if partials:    # few output tiles, many rows: the rows are cut into ranges that run side by side
            scratch = DeviceStorage(partials, "float32")
            lib.call("qmoe_gemm_wgrad_split", dy.ptr, x.ptr, dw.ptr, scratch.ptr, self.width_out, rows, self.width_in, self.stream)
        else:
            self._gemm(dy, x, dw, self.width_out, rows, self.width_in, 1, 0, lib.QMOE_F32)
        _accumulate(self.weight, dw, self.stream)
        return dx


def _rms_norm(x, norm, rows, width, stream):
    out, inverse = DeviceStorage(rows * width, "bfloat16"), DeviceStorage(rows, "float32")
    lib.call("qmoe_rms_norm", x.ptr, lib.QMOE_BF16, norm.weight.storage.ptr, out.ptr, lib.QMOE_BF16, inverse.ptr, rows, width,
             norm.eps, stream)
    return out, inverse


def _rms_norm_backward(gradient, x, norm, inverse, rows, width, stream):
    dx, dw = DeviceStorage(rows * width, "bfloat16"), DeviceStorage(width, "float32")
    partials = DeviceStorage(lib.load().qmoe_rms_norm_partials(rows, width), "float32")
    lib.call("qmoe_rms_norm_backward", gradient.ptr, lib.QMOE_BF16, x.ptr, lib.QMOE_BF16, norm.weight.storage.ptr, inverse.ptr,
             dx.ptr, dw.ptr, partials.ptr, rows, width, stream)
    _accumulate(norm.weight, dw, stream)
    return dx


def _add(a, b, stream):
    out = DeviceStorage(a.size, a.dtype)
    lib.call("qmoe_add", a.ptr, b.ptr, out.ptr, lib.DTYPE_CODES[a.dtype], a.size, stream)
    return out


class GQA:
    """Grouped-query attention with rotary embedding (src/qutai/lm/layers.py:316-349)."""

    def __init__(self, config, *, seed, stream=0):
        width = config.d_model
        self.heads, self.kv_heads, self.theta = config.n_heads, config.n_kv_heads, config.rope_theta
        self.dim = width // config.n_heads
        kv_width = config.n_kv_heads * self.dim
        s = (lambda k: None if seed is None else seed + k)
        self.q = Linear(width, width, std=0.02, seed=s(0), stream=stream)
        self.k = Linear(width, kv_width, std=0.02, seed=s(1), stream=stream)
        self.v = Linear(width, kv_width, std=0.02, seed=s(2), stream=stream)
        self.out = Linear(width, width, std=0.02 / sqrt(2 * config.n_layers), seed=s(3), stream=stream)
        self.width, self.kv_width, self.stream = width, kv_width, stream

    def parameters(self):
        return tuple(p for layer in (self.q, self.k, self.v, self.out) for p in layer.parameters())

    def _rope(self, values, batch, time, heads, inverse):
        out = DeviceStorage(values.size, "bfloat16")
        lib.call("qmoe_rope", values.ptr, out.ptr, lib.QMOE_BF16, batch, time, heads, self.dim, float(self.theta), 0, 1 if inverse else 0,
                 self.stream)
        return out

    def forward(self, x, batch, time):
        rows = batch * time
        view = lambda storage, width: Tensor(storage, (batch, time, width))
        q = self._rope(self.q.forward(x, rows), batch, time, self.heads, False)
        k = self._rope(self.k.forward(x, rows), batch, time, self.kv_heads, False)
        v = self.v.forward(x, rows)
        qt, kt, vt = view(q, self.width), view(k, self.kv_width), view(v, self.kv_width)
        attended, lse = attention_forward(qt, kt, vt, self.heads, self.kv_heads, self.stream)
        saved = (x, qt, kt, vt, attended, lse)
        return self.out.forward(attended, rows), saved

    def backward(self, dy, saved, batch, time):
        rows = batch * time
        x, qt, kt, vt, attended, lse = saved
        d_attended = self.out.backward(dy, attended, rows)
        dq, dk, dv = attention_backward(d_attended, qt, kt, vt, attended, lse, self.heads, self.kv_heads, self.stream)
        dq = self._rope(dq, batch, time, self.heads, True)
        dk = self._rope(dk, batch, time, self.kv_heads, True)
        dx = self.q.backward(dq, x, rows)
        dx = _add(dx, self.k.backward(dk, x, rows), self.stream)
        return _add(dx, self.v.backward(dv, x, rows), self.stream)


class Block:
    """``x += attn(attn_norm(x)); x += ffn(ffn_norm(x))`` (src/qutai/lm/layers.py:412-449).  On one GPU the second half
    is the fused ``MoEFeedForward``; as a rank of an expert-parallel job it is norm, ``ExpertParallelMoE`` (experts
    spread over the ranks, rows exchanged over NVLink) and the residual add as three steps."""

    def __init__(self, config, *, seed, stream=0, rank=0, world=1, parallel=None):
        self.attn_norm = RMSNorm(config.d_model, config.norm_eps, stream=stream)
        self.ffn_norm = RMSNorm(config.d_model, config.norm_eps, stream=stream)
        self.attn = GQA(config, seed=seed, stream=stream)
        ffn_seed = None if seed is None else seed + 4
        if world == 1:
            self.ffn = SparseMoE(config, seed=ffn_seed, stream=stream)
            self.feed_forward = MoEFeedForward(self.ffn_norm, self.ffn)
        else:
            self.ffn = ExpertParallelMoE(config, rank=rank, world=world, seed=ffn_seed, stream=stream, **(parallel or {}))
            self.ffn.reduce_router_gradient = False      # summed over the ranks with the other replicated gradients, in one collective
            self.feed_forward = None
        self._aux_gradient_value = config.aux_loss_coef / config.n_layers
        self.width, self.stream = config.d_model, stream
        self._saved = None

    def parameters(self):
        return (*self.attn_norm.parameters(), *self.ffn_norm.parameters(), *self.attn.parameters(), *self.ffn.parameters())

    def forward(self, x, batch, time):
        rows = batch * time
        normed, inverse = _rms_norm(x, self.attn_norm, rows, self.width, self.stream)
        y, attention_saved = self.attn.forward(normed, batch, time)
        middle = _add(x, y, self.stream)
        if self.feed_forward is not None:
            out, aux = self.feed_forward(Tensor(middle, (rows, self.width)))
            self._saved = (x, inverse, attention_saved, None, None)
            return out.storage, aux
        normed, ffn_inverse = _rms_norm(middle, self.ffn_norm, rows, self.width, self.stream)
        y, aux = self.ffn.forward(Tensor(normed, (rows, self.width)))
        self._saved = (x, inverse, attention_saved, middle, ffn_inverse)
        return _add(middle, y.storage, self.stream), aux

    def backward(self, d_out, d_aux, batch, time):
        rows = batch * time
        x, inverse, attention_saved, middle, ffn_inverse = self._saved
        if self.feed_forward is not None:
            d_middle = self.feed_forward.backward(Tensor(d_out, (rows, self.width)), d_aux).storage
        else:   # every rank hands the layer the same gradient of the auxiliary loss over all ranks' tokens
            d_normed = self.ffn.backward(Tensor(d_out, (rows, self.width)), self._aux_gradient_value).storage
            d_middle = _add(_rms_norm_backward(d_normed, middle, self.ffn_norm, ffn_inverse, rows, self.width, self.stream), d_out,
                            self.stream)
        d_normed = self.attn.backward(d_middle, attention_saved, batch, time)
        dx = _rms_norm_backward(d_normed, x, self.attn_norm, inverse, rows, self.width, self.stream)
        self._saved = None
        return _add(dx, d_middle, self.stream)


class Decoder:
    def __init__(self, config, *, device="cuda", dtype="float32", seed=None, stream=0, rank=0, world=1, parallel=None):
        """``rank`` / ``world``: this process's place in a data- and expert-parallel job (the communicator of
        ``qutai_b200.expert_parallel.init_communicator`` must be up when ``world > 1``); every rank passes the same
        ``seed``, so the replicated parameters start equal and an expert's weights depend on its number in the model,
        not on where it lives.  ``parallel``: keyword arguments for every block's ``ExpertParallelMoE``
        (``transport``, ``placement``, ``gather`` ...)."""
        if device != "cuda" or dtype != "float32":
            raise ValueError("parameters are float32 on device='cuda' (there is no CPU fallback)")
        if not 0 <= rank < world:
            raise ValueError("rank must be in [0, world)")
        self.rank, self.world = rank, world
        if config.ffn_type != "moe":
            raise ValueError("this decoder has mixture-of-experts blocks only")
        if config.d_model % config.n_heads or config.d_model // config.n_heads != 64:
            raise ValueError("the head width d_model / n_heads must be 64")
        self.config, self.stream = config, stream
        table = DeviceStorage(config.vocab_size * config.d_model, "float32")
        table.fill_normal(0.0, 0.02, 0x5EED if seed is None else seed, stream)
        self.embedding = type("Projection", (), {})()
        self.embedding.weight = Tensor(table, (config.vocab_size, config.d_model), requires_grad=True)
        self.blocks = tuple(Block(config, seed=None if seed is None else seed + 1 + 100 * i, stream=stream, rank=rank, world=world,
                                  parallel=parallel) for i in range(config.n_layers))
        self.norm = RMSNorm(config.d_model, config.norm_eps, stream=stream)
        self.head = LMHead(stream=stream)
        self.last_lm_loss = self.last_auxiliary_loss = None
        self._saved = None
        one = lambda value: DeviceStorage.from_values([value], "float32", stream)
        self._one_over_layers, self._aux_coef = one(1.0 / config.n_layers), one(config.aux_loss_coef)
        self._aux_gradient = one(config.aux_loss_coef / config.n_layers)     # d total / d (one block's auxiliary loss)
        self._share = (None, None)     # this rank's share of all ranks' targets: (value, device storage)

    # -- parameters -------------------------------------------------------------------------------------------
    def named_parameters(self):
        """Names and order of upstream's ``Decoder.named_parameters`` (src/qutai/lm/decoder.py:38-80); as a rank of an
        expert-parallel job, only the experts this rank holds, under their numbers in the model."""
        result = [("embedding.weight", self.embedding.weight)]
        for i, block in enumerate(self.blocks):
            prefix = f"blocks.{i}."
            result.extend((prefix + name + ".weight", getattr(block, name).weight) for name in ("attn_norm", "ffn_norm"))
            result.extend((prefix + "attn." + name + ".weight", getattr(block.attn, name).weight) for name in ("q", "k", "v", "out"))
            result.append((prefix + "ffn.router.weight", block.ffn.router.weight))
            if self.world > 1:
                result.extend(block.ffn.named_expert_parameters(prefix=prefix + "ffn.experts"))
                continue
            for e, expert in enumerate(block.ffn.experts):
                result.extend((f"{prefix}ffn.experts.{e}.{name}.weight", getattr(expert, name).weight) for name in ("gate", "up", "down"))
        result.append(("norm.weight", self.norm.weight))
        return result

    def replicated_parameters(self):
        """The parameters every rank holds a copy of and whose gradients ``backward`` sums over the ranks: everything
        but the experts."""
        skip = {id(p) for block in self.blocks for expert in block.ffn.experts for p in expert.parameters()}
        return tuple(p for p in self.parameters() if id(p) not in skip)

    def parameters(self):
        return tuple(parameter for _, parameter in self.named_parameters())

    def zero_grad(self):
        for parameter in self.parameters():
            parameter.grad = None

    def operand_shadows(self):
        """``{parameter: bf16 storage}`` of the tensor-core operand copies (expert weights, projections, the tied table)
        once a forward has made them: an ``AdamW(shadows=...)`` that writes the rounded weights there keeps them
        current, and no forward after a step converts anything."""
        shadows = {}
        for block in self.blocks:
            shadows.update(block.ffn.operand_shadows())
            for layer in (block.attn.q, block.attn.k, block.attn.v, block.attn.out):
                shadows[layer.weight] = layer.operand()
        if self.head._operand is not None:
            shadows[self.embedding.weight] = self.head._operand
        return shadows

    def clip_grad_norm(self, max_norm=1.0):
        """Upstream's ``clip_grad_norm(model.parameters(), max_norm)`` (src/qutai/nn/optimizers.py:19-31) over the WHOLE
        model: with ``world > 1`` the experts of the other ranks count too (``clip_grad_norm_sharded``), and every
        rank scales by the same factor.  Returns the norm before clipping."""
        from .optim import clip_grad_norm, clip_grad_norm_sharded

        if self.world == 1:
            return clip_grad_norm(self.parameters(), max_norm, stream=self.stream)
        replicated = self.replicated_parameters()
        held = {id(p) for p in replicated}
        return clip_grad_norm_sharded(replicated, [p for p in self.parameters() if id(p) not in held], max_norm, stream=self.stream)

    # -- forward ------------------------------------------------------------------------------------------------
    def loss(self, tokens, labels=None, *, targets_of_all_ranks=None):
        """``tokens`` (and ``labels``, default the tokens): nested sequences [batch][time] of token ids (-100 in the
        labels = no target).  Returns the loss as a float32 device tensor of one element; ``last_lm_loss`` and
        ``last_auxiliary_loss`` (mean over the blocks) are set like upstream's (src/qutai/lm/decoder.py:143-175).
        With ``world > 1`` the sequences are this rank's, and the loss (the same value on every rank) is the mean over
        the targets of all ranks: ``targets_of_all_ranks`` is their number, by default ``world`` times this rank's."""
        c, stream = self.config, self.stream
        batch, time = len(tokens), len(tokens[0])
        if time < 2 or any(len(row) != time for row in tokens):
            raise ValueError("tokens must be a non-empty rectangular batch of at least two positions")
        flat = [int(t) for row in tokens for t in row]
        if any(t < 0 or t >= c.vocab_size for t in flat):
            raise ValueError("token id outside the vocabulary")
        targets = flat if labels is None else [int(t) for row in labels for t in row]
        if len(targets) != len(flat) or any(t != -100 and not 0 <= t < c.vocab_size for t in targets):
            raise ValueError("labels must have the shape of the tokens and be token ids or -100")
        rows, width = batch * time, c.d_model
        # The embedding's backward wants, per distinct token, the list of its positions (upstream builds the same tables,
        # src/qutai/backends/cuda_lm.py:97-106).  They depend on the ids alone, so they are built and uploaded here,
        # next to the ids: an upload waits for the stream, and at this point of a training loop the device is just
        # finishing the previous step, while at the end of the backward the wait would leave it idle through the
        # host's preparation of the optimizer step.
        groups = {}
        for position, token in enumerate(flat):
            groups.setdefault(token, []).append(position)
        distinct = sorted(groups)
        starts, positions = [0], []
        for token in distinct:
            positions.extend(groups[token])
            starts.append(len(positions))
        ids = DeviceStorage.from_bytes(array("q", flat).tobytes(), "int64", stream)
        tables = tuple(DeviceStorage.from_bytes(array("q", values).tobytes(), "int64", stream) for values in (distinct, starts, positions))
        label_ids = ids if labels is None else DeviceStorage.from_bytes(array("q", targets).tobytes(), "int64", stream)
        x = DeviceStorage(rows * width, "bfloat16")
        lib.call("qmoe_embedding", self.embedding.weight.storage.ptr, ids.ptr, x.ptr, lib.QMOE_BF16, rows, width, c.vocab_size, stream)
        auxiliary = []
        for block in self.blocks:
            x, aux = block.forward(x, batch, time)
            auxiliary.append(aux)
        hidden, inverse = _rms_norm(x, self.norm, rows, width, stream)
        lm = self.head.forward(Tensor(hidden, (batch, time, width)), self.embedding.weight, label_ids)
        share = None
        if self.world > 1:
            # mean over all ranks' targets = sum over ranks of (this rank's mean) x (its share of the targets)
            mine = sum(1 for b in range(batch) for t in range(1, time) if targets[b * time + t] != -100)
            value = 1.0 / self.world if targets_of_all_ranks is None else max(mine, 1) / float(targets_of_all_ranks)
            if self._share[0] != value:
                self._share = (value, DeviceStorage.from_values([value], "float32", stream))
            share = self._share[1]
            weighted = DeviceStorage(1, "float32")
            lib.call("qmoe_scale_f32", lm.storage.ptr, weighted.ptr, 0, share.ptr, 1, 1, stream)
            lib.call("qmoe_ep_all_reduce_f32", weighted.ptr, 1, stream)
            lm = Tensor(weighted, ())
        # total = lm + coef * mean(aux): three tiny device operations keep the host out of the step
        total = DeviceStorage.zeros(1, "float32", stream)
        mean_aux = DeviceStorage.zeros(1, "float32", stream)
        for aux in auxiliary:
            lib.call("qmoe_add", mean_aux.ptr, aux.storage.ptr, mean_aux.ptr, lib.QMOE_F32, 1, stream)
        lib.call("qmoe_scale_f32", mean_aux.ptr, mean_aux.ptr, 0, self._one_over_layers.ptr, 1, 1, stream)
        scaled = DeviceStorage(1, "float32")
        lib.call("qmoe_scale_f32", mean_aux.ptr, scaled.ptr, 0, self._aux_coef.ptr, 1, 1, stream)
        lib.call("qmoe_add", lm.storage.ptr, scaled.ptr, total.ptr, lib.QMOE_F32, 1, stream)
        self.last_lm_loss, self.last_auxiliary_loss = lm, Tensor(mean_aux, ())
        self._saved = (tables, len(distinct), len(positions), batch, time, x, inverse, share)
        return Tensor(total, ())

    # -- backward -----------------------------------------------------------------------------------------------
    def backward(self):
        """Gradient of the last ``loss`` with respect to every parameter, accumulated into ``parameter.grad``."""
        if self._saved is None:
            raise RuntimeError("backward needs a loss first")
        c, stream = self.config, self.stream
        tables, distinct, positions, batch, time, x_last, inverse, share = self._saved
        rows, width = batch * time, c.d_model
        d_hidden, d_table = self.head.backward(share)
        _accumulate(self.embedding.weight, d_table.storage, stream)
        dx = _rms_norm_backward(d_hidden.storage, x_last, self.norm, inverse, rows, width, stream)
        for block in reversed(self.blocks):
            dx = block.backward(dx, self._aux_gradient, batch, time)
        # the embedding's share of the tied table's gradient, through the token -> positions tables of the forward
        lib.call("qmoe_embedding_backward", dx.ptr, lib.QMOE_BF16, tables[0].ptr, tables[1].ptr, tables[2].ptr,
                 self.embedding.weight.grad.storage.ptr, distinct, positions, width, c.vocab_size, stream)
        self._saved = None
        if self.world > 1:
            self._sum_replicated_gradients(stream)

    def _sum_replicated_gradients(self, stream):
        """ONE all-reduce for the gradients of all replicated tensors of this backward: they are copied side by side
        into one buffer (a quarter of a gigabyte at 12 blocks of width 1024: the copies cost less than the latency of
        the seventy small collectives they replace), summed over the ranks there, and ``parameter.grad`` becomes a
        view of that buffer.  A gradient that was already there before this backward (accumulation over several
        backwards) would be summed twice: reduce once per optimizer step then, by calling ``zero_grad`` between
        steps as upstream's training loop does."""
        held = [p for p in self.replicated_parameters() if p.grad is not None]
        if not held:
            return
        flat = DeviceStorage(sum(p.grad.storage.size for p in held), "float32")
        offset = 0
        for parameter in held:
            size = parameter.grad.storage.size
            lib.call("qmoe_memcpy_d2d", flat.ptr + 4 * offset, parameter.grad.storage.ptr, 4 * size, stream)
            offset += size
        lib.call("qmoe_ep_all_reduce_f32", flat.ptr, flat.size, stream)
        offset = 0
        for parameter in held:
            size = parameter.grad.storage.size
            parameter.grad = Tensor(flat.view(offset, size), parameter.shape)
            offset += size
