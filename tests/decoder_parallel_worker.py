"""Child process of the data- and expert-parallel decoder test: one rank = one GPU.  Builds
``Decoder(..., rank=, world=)`` with the parameters of the upstream-made fixture, takes its share of the fixture's
sequences, runs loss + backward and writes loss, gradients and (after a few AdamW steps) the replicated parameters to
OUT/rank{r}.npz for the parent to compare with what upstream's single-device ``Decoder`` produced on the whole batch.
Usage: python decoder_parallel_worker.py RANK WORLD OUT_DIR"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(HERE, "golden"))


def main():
    rank, world, out_dir = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    import make_golden_decoder as fixture   # only its seeded inputs are used; upstream is not imported
    from gpu_util import to_host
    from qutai_b200 import lib
    from qutai_b200.decoder import Config, Decoder
    from qutai_b200.expert_parallel import file_all_gather, finalize_communicator, init_communicator
    from qutai_b200.optim import AdamW

    lib.call("qmoe_set_device", rank)
    init_communicator(rank, world, rendezvous_path=os.path.join(out_dir, "nccl_id"), timeout=120)
    exchanges = iter(range(1000))
    model = Decoder(Config(aux_loss_coef=0.05, **fixture.SHAPE), seed=3, rank=rank, world=world,
                    parallel=dict(gather=lambda data: file_all_gather(out_dir, f"ipc{next(exchanges)}", rank, world, data)))
    # the fixture draws its parameters in the order of the whole model's names: rebuild that list, keep what this rank holds
    E = fixture.SHAPE["n_experts"]
    d, h = fixture.SHAPE["d_model"], fixture.SHAPE["d_expert"]
    named = model.named_parameters()
    mine = {name for name, _ in named}
    full = []
    for name, parameter in named:
        if ".ffn.experts." not in name:
            full.append((name, tuple(parameter.shape)))
            if name.endswith("ffn.router.weight"):
                prefix = name[:-len("router.weight")]
                for e in range(E):
                    full.extend([(f"{prefix}experts.{e}.gate.weight", (h, d)), (f"{prefix}experts.{e}.up.weight", (h, d)),
                                 (f"{prefix}experts.{e}.down.weight", (d, h))])
    values = fixture.decoder_parameters(full)
    assert mine <= set(values)
    for name, parameter in named:
        parameter.storage.upload_bytes(np.ascontiguousarray(values[name], dtype=np.float32).tobytes())

    tokens, labels = fixture.decoder_tokens()
    share = len(tokens) // world
    rows = slice(rank * share, (rank + 1) * share)
    all_targets = sum(1 for row in labels for label in row[1:] if label != -100)
    loss = model.loss(tokens[rows], labels[rows], targets_of_all_ranks=all_targets)
    model.backward()
    assert lib.device_status() == 0
    out = dict(loss=to_host(loss.storage), lm_loss=to_host(model.last_lm_loss.storage), aux_loss=to_host(model.last_auxiliary_loss.storage),
               names=np.array([name for name, _ in named]),
               replicated=np.array([name for name, p in named if any(p is q for q in model.replicated_parameters())]))
    for name, parameter in named:
        out["has:" + name] = np.array(parameter.grad is not None)
        if parameter.grad is not None:
            out["grad:" + name] = to_host(parameter.grad.storage, tuple(parameter.shape))

    # clipping over the whole model: the norm counts the other rank's experts too, both ranks scale alike
    out["clip_norm"] = np.array(model.clip_grad_norm(1e-3))
    out["clipped:embedding.weight"] = to_host(model.embedding.weight.grad.storage, tuple(model.embedding.weight.shape))
    first_expert = next(name for name, p in named if ".ffn.experts." in name and p.grad is not None)
    out["clipped_expert_name"] = np.array(first_expert)
    out["clipped_expert"] = to_host(dict(named)[first_expert].grad.storage, tuple(dict(named)[first_expert].shape))

    optimizer = AdamW(model.parameters(), learning_rate=3e-3, shadows=model.operand_shadows())
    losses = []
    for _ in range(5):
        model.zero_grad()
        loss = model.loss(tokens[rows], labels[rows], targets_of_all_ranks=all_targets)
        model.backward()
        optimizer.step()
        losses.append(float(to_host(loss.storage)[0]))
    out["losses"] = np.array(losses)
    out["embedding_after"] = to_host(model.embedding.weight.storage, tuple(model.embedding.weight.shape))
    out["router_after"] = to_host(model.blocks[0].ffn.router.weight.storage, (E, d))
    assert lib.device_status() == 0
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **out)
    finalize_communicator()
    print(f"rank {rank} done")


if __name__ == "__main__":
    main()
