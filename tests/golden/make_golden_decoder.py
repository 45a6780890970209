"""Golden vectors for a whole mixture-of-experts decoder step — loss and the gradient of every parameter — produced by
the UPSTREAM package itself: its ``Decoder`` (src/qutai/lm/decoder.py:20-175) on ``device="cpu"``, ``dtype="float64"``,
activation checkpointing off, under its own autograd.  Head width 64 (the width of this package's attention kernels),
two heads sharing one key/value head, two blocks, four experts.

The parameters come from a seeded numpy generator (``decoder_parameters`` below, values a float32 holds exactly), so the
fixture stores the upstream results only.  Run in a container that has a checkout of the upstream sources
(``python tests/golden/make_golden_decoder.py``); ``decoder_small.npz`` is committed, this script documents how it
was made.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SHAPE = dict(vocab_size=40, n_layers=2, d_model=128, n_heads=2, n_kv_heads=1, n_experts=4, top_k=2, d_expert=16)
BATCH, TIME, SEED = 2, 9, 61


def decoder_tokens():
    rng = np.random.default_rng(SEED)
    tokens = rng.integers(0, SHAPE["vocab_size"], size=(BATCH, TIME))
    labels = tokens.copy()
    labels[0, 3] = labels[1, 7] = -100
    return tokens.tolist(), labels.tolist()


def decoder_parameters(names_and_shapes):
    """name -> float32 array, drawn in the order given (norm weights near one, everything else N(0, 0.15))."""
    rng = np.random.default_rng(SEED + 1)
    out = {}
    for name, shape in names_and_shapes:
        if name.endswith("norm.weight"):
            out[name] = (1 + 0.2 * rng.standard_normal(shape)).astype(np.float32)
        else:
            out[name] = (0.15 * rng.standard_normal(shape)).astype(np.float32)
    return out


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle import ref_loader

    ref_loader.load()
    from qutai.backends import cpu
    from qutai.core.tensor import Tensor
    from qutai.lm.config import Config
    from qutai.lm.decoder import Decoder

    config = Config(ffn_type="moe", d_ff=64, max_seq_len=16, activation_checkpointing=False, aux_loss_coef=0.05, **SHAPE)
    model = Decoder(config, device="cpu", dtype="float64", seed=0)
    named = model.named_parameters()
    values = decoder_parameters([(name, tuple(p.shape)) for name, p in named])
    for name, parameter in named:
        data = values[name].astype(np.float64).reshape(-1).tolist()
        parameter.storage = cpu.storage(data, dtype="float64")
    tokens, labels = decoder_tokens()
    loss = model.loss(tokens, labels, chunk_size=5)
    loss.backward()
    result = dict(kind="decoder", loss=np.array(loss.storage.tolist())[0], lm_loss=np.array(model.last_lm_loss.storage.tolist())[0],
                  aux_loss=np.array(model.last_auxiliary_loss.storage.tolist())[0])
    for name, parameter in named:
        result["grad:" + name] = (np.zeros(0, dtype=np.float32) if parameter.grad is None
                                  else np.array(parameter.grad.storage.tolist(), dtype=np.float32).reshape(parameter.shape))
    np.savez_compressed(os.path.join(HERE, "decoder_small.npz"), **result)
    print("loss", result["loss"], "lm", result["lm_loss"], "aux", result["aux_loss"], "tensors", len(named))
