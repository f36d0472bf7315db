"""Checkpoint / resume in HuggingFace-style torch ``state_dict`` form.

``save_checkpoint(dir, trainer)`` writes, from DP rank 0 of every TP coordinate,
  ``pytorch_model.bin``      HF-named full model state dict (TP = 1 only; loads into the ``transformers``
                             class of the family with ``load_state_dict``)
  ``trainer_state_tp{t}.pt`` {"model": native state dict of this TP shard, "optimizer": ..., "step": ...,
                             "rng": torch / cuda RNG states, "data": data-stream cursor, "config": ...}
``load_checkpoint(dir, trainer)`` restores all of it, so that a resumed run continues with the same
parameters, moments, RNG and token stream.  The reference has no checkpoint code (its runs stop after
at most 100 steps, train.py:94,213-214).
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
        torch.save(state, os.path.join(path, f"trainer_state_tp{mesh.tp_rank}.pt"))
        if mesh.tp_size == 1:
            hf = {k: v.cpu() for k, v in model.hf_state_dict().items()}
            torch.save(hf, os.path.join(path, "pytorch_model.bin"))
    if dist.is_initialized():
        dist.barrier()


def load_checkpoint(path: str, trainer, strict: bool = True) -> int:
    mesh = trainer.plugin.pg_mesh
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
