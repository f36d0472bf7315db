"""Checkpoint / resume in HuggingFace-style torch ``state_dict`` form.

``save_checkpoint(dir, trainer)`` writes, from DP rank 0 of every TP coordinate,
  ``trainer_state_tp{t}.pt`` {"model": native state dict of this TP shard, "optimizer": ..., "step": ...,
                             "rng": torch / cuda RNG states, "data": data-stream cursor, "config": ...}
and, from global rank 0,
  ``pytorch_model.bin``      HF-named FULL model state dict (the TP shards are joined first; loads into the
                             ``transformers`` class of the family with ``load_state_dict``)
``load_checkpoint(dir, trainer)`` restores all of it, so that a resumed run continues with the same
parameters, moments, RNG and token stream.  When the checkpoint was written with another tensor-parallel size,
the shards of the model AND of the optimizer state (moments, master weights) are joined and cut again for the
current layout, so a run can be resumed on a different number of GPUs.  The reference has no checkpoint code
(its runs stop after at most 100 steps, train.py:94,213-214).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def _unwrap(trainer):
    return trainer.model.unwrap()


def save_checkpoint(path: str, trainer) -> None:
    mesh = trainer.plugin.pg_mesh
    if mesh.dp_rank == 0:
        os.makedirs(path, exist_ok=True)
        model = _unwrap(trainer)
        state = {
            "model": {k: v.detach().cpu() for k, v in model.state_dict().items()},
            "optimizer": trainer.optimizer.state_dict(),
            "step": trainer.step_count,
            "rng": {"cpu": torch.get_rng_state(),
                    "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None},
            "data": trainer.data.state_dict(),
            "config": trainer.cfg.to_dict(),
            "sparse_sync": {"sparse_embedding": trainer.cfg.sparse_embedding, "method": trainer.cfg.method,
                            "top_k": trainer.cfg.top_k},
        }
        state["tp_size"] = mesh.tp_size
        torch.save(state, os.path.join(path, f"trainer_state_tp{mesh.tp_rank}.pt"))
        if mesh.tp_rank == 0:             # shards of an earlier save with a larger TP size would be stale
            t = mesh.tp_size
            while os.path.exists(os.path.join(path, f"trainer_state_tp{t}.pt")):
                os.remove(os.path.join(path, f"trainer_state_tp{t}.pt"))
                t += 1
        if mesh.tp_size == 1:
            hf = {k: v.cpu() for k, v in model.hf_state_dict().items()}
            torch.save(hf, os.path.join(path, "pytorch_model.bin"))
    if dist.is_initialized():
        dist.barrier()
    if mesh.tp_size > 1 and mesh.dp_rank == 0 and mesh.tp_rank == 0:
        # every shard file is on disk now: join them into the HF-format full model
        from ..models import build_model
        from ..models.sharding import unshard_state_dicts

        shards = [torch.load(os.path.join(path, f"trainer_state_tp{t}.pt"), map_location="cpu", weights_only=False)["model"]
                  for t in range(mesh.tp_size)]
        full = build_model(trainer.model_cfg, dtype=shards[0]["wte"].dtype, device="cpu")
        full.load_state_dict(unshard_state_dicts(shards, trainer.model_cfg))
        torch.save({k: v.cpu() for k, v in full.hf_state_dict().items()}, os.path.join(path, "pytorch_model.bin"))
    if dist.is_initialized():
        dist.barrier()


def _saved_tp_size(path: str) -> int:
    """Tensor-parallel size recorded in shard 0 (older checkpoints without the field: the number of shard files)."""
    f0 = os.path.join(path, "trainer_state_tp0.pt")
    if not os.path.exists(f0):
        return 0
    tp = torch.load(f0, map_location="cpu", weights_only=False).get("tp_size")
    if tp is None:
        tp = 0
        while os.path.exists(os.path.join(path, f"trainer_state_tp{tp}.pt")):
            tp += 1
    return int(tp)


def _resharded_state(path: str, trainer, saved_tp: int) -> dict:
    """The trainer state of this rank's TP coordinate, rebuilt from a checkpoint written with ``saved_tp`` shards."""
    from ..models.sharding import shard_state_dict, unshard_state_dicts

    mesh, mc = trainer.plugin.pg_mesh, trainer.model_cfg
    states = [torch.load(os.path.join(path, f"trainer_state_tp{t}.pt"), map_location="cpu", weights_only=False)
              for t in range(saved_tp)]
    for t, st in enumerate(states):      # shards of one save only: a stale file of an earlier save must not be joined in
        if st.get("tp_size", saved_tp) != saved_tp or st["step"] != states[0]["step"]:
            raise RuntimeError(f"checkpoint shard {t} in {path} (tp_size {st.get('tp_size')}, step {st['step']}) does not "
                               f"belong to the save of shard 0 (tp_size {saved_tp}, step {states[0]['step']})")
    names = list(states[0]["model"].keys())                # parameter order = optimizer index order
    out = dict(states[0])
    out["model"] = shard_state_dict(unshard_state_dicts([s["model"] for s in states], mc), mc, mesh.tp_rank, mesh.tp_size)
    opt = {"state": {}, "param_groups": states[0]["optimizer"]["param_groups"]}
    for k, v in states[0]["optimizer"].items():
        if k not in ("state", "param_groups"):
            opt[k] = v
    kinds = set()
    for st in states[0]["optimizer"]["state"].values():
        kinds |= {k for k, v in st.items() if torch.is_tensor(v) and v.dim() > 0}
    for kind in sorted(kinds):
        per_rank = [{names[i]: st[kind] for i, st in s["optimizer"]["state"].items() if kind in st} for s in states]
        if not per_rank[0]:
            continue
        cut = shard_state_dict(unshard_state_dicts(per_rank, mc), mc, mesh.tp_rank, mesh.tp_size)
        for i, st in states[0]["optimizer"]["state"].items():
            if kind in st:
                opt["state"].setdefault(i, {k: v for k, v in st.items() if not (torch.is_tensor(v) and v.dim() > 0)})
                opt["state"][i][kind] = cut[names[i]]
    out["optimizer"] = opt
    return out


def load_checkpoint(path: str, trainer, strict: bool = True) -> int:
    mesh = trainer.plugin.pg_mesh
    saved_tp = _saved_tp_size(path)
    if saved_tp and saved_tp != mesh.tp_size:
        state = _resharded_state(path, trainer, saved_tp)
    else:
        f = os.path.join(path, f"trainer_state_tp{mesh.tp_rank}.pt")
        state = torch.load(f, map_location="cpu", weights_only=False)
    model = _unwrap(trainer)
    model.load_state_dict(state["model"], strict=strict)
    trainer.optimizer.load_state_dict(state["optimizer"])
    # moments / master weights follow the parameters' device
    for st in trainer.optimizer.state.values():
        for k, v in list(st.items()):
            if torch.is_tensor(v):
                st[k] = v.to(trainer.device)
    trainer.step_count = int(state["step"])
    torch.set_rng_state(state["rng"]["cpu"])
    if state["rng"]["cuda"] is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(state["rng"]["cuda"])
    trainer.data.load_state_dict(state["data"])
    if dist.is_initialized():
        dist.barrier()
    return trainer.step_count


def load_hf_weights(path: str, trainer) -> None:
    """Load ``pytorch_model.bin`` (HF names) into the trainer's model."""
    sd = torch.load(os.path.join(path, "pytorch_model.bin"), map_location="cpu", weights_only=True)
    _unwrap(trainer).load_hf_state_dict(sd)
