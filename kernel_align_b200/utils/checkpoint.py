"""Checkpoint / resume: model shards, optimizer state, sampler random stream and step counter
in one ``torch.save`` file per rank (``CheckpointFormat.PT``). Because every kernel of the
training step is deterministic, a run resumed from a checkpoint reproduces the loss of the
uninterrupted run bit for bit; the tests rely on exactly that.

The reference declares ``CheckpointFormat`` (rl_engine/platforms/constants.py:69-73) and has no
checkpoint code.
"""
from __future__ import annotations

import os
from typing import Any, Optional

import torch


def _rank_path(path: str, rank: int, world: int) -> str:
    return path if world == 1 else f"{path}.rank{rank}of{world}"


def save_checkpoint(path: str, model, optimizer=None, sampler=None, step: int = 0, extra: Optional[dict] = None,
                    rank: int = 0, world: int = 1) -> str:
    payload: dict[str, Any] = {
        "format": "pt",
        "step": int(step),
        "model": {k: v.detach().cpu() for k, v in model.state_dict().items()},
        "optimizer": optimizer.state_dict() if optimizer is not None else None,
        "sampler": sampler.rng_state() if sampler is not None else None,
        "extra": extra or {},
    }
    if payload["optimizer"] is not None:
        payload["optimizer"] = {k: ([{n: t.cpu() for n, t in st.items()} for st in v] if k == "state" else v)
                                for k, v in payload["optimizer"].items()}
    out = _rank_path(path, rank, world)
    os.makedirs(os.path.dirname(os.path.abspath(out)), exist_ok=True)
    tmp = out + ".tmp"
    torch.save(payload, tmp)
    os.replace(tmp, out)  # never leave a half-written checkpoint under the final name
    return out


def load_checkpoint(path: str, model, optimizer=None, sampler=None, rank: int = 0, world: int = 1) -> dict:
    payload = torch.load(_rank_path(path, rank, world), map_location="cpu", weights_only=False)
    model.load_state_dict(payload["model"])
    if optimizer is not None and payload["optimizer"] is not None:
        optimizer.load_state_dict(payload["optimizer"])
    if sampler is not None and payload["sampler"] is not None:
        sampler.set_rng_state(payload["sampler"])
    return {"step": payload["step"], "extra": payload["extra"]}
