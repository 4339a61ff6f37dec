"""Checkpoint / pretrained-directory IO.

On-disk contract shared with the reference (``astrai/serialization.py:19-182``):

* pretrained dir: ``config.json`` + ``model.safetensors`` (full, unsharded state dict; a tied
  ``lm_head.weight`` is omitted)
* checkpoint dir: ``meta.json {epoch, iteration, timestamp}``, ``config.json``,
  ``model.safetensors`` and one ``<key>.pt`` (``torch.save``) per entry of ``extra``
  (``optimizer.pt``, ``scheduler.pt``); only rank 0 writes.

``broadcast=True`` makes rank 0 read and ship the content to the other ranks over the
process group (objects with ``broadcast_object_list``, tensors one by one).
"""

from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, Union

import torch
import torch.distributed as dist
from safetensors.torch import load_file, save_file

CONFIG_FILE = "config.json"
WEIGHTS_FILE = "model.safetensors"
META_FILE = "meta.json"
PathLike = Union[str, Path]


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _share(read, broadcast: bool):
    """Run ``read()`` everywhere, or on rank 0 only and broadcast the python object."""
    if not (broadcast and dist.is_available() and dist.is_initialized()):
        return read()
    box = [read() if _rank() == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return box[0]


# -- primitives ---------------------------------------------------------------------------
def _atomically(path: PathLike, write) -> None:
    """``write(tmp_path)`` then rename over ``path``: a reader (or a job restarted after a crash)
    sees either the old file or the complete new one, never a torn write."""
    target = Path(path)
    tmp = target.with_name(target.name + ".tmp")
    try:
        write(tmp)
        os.replace(tmp, target)
    finally:
        if tmp.exists():
            tmp.unlink()


def save_safetensors(state_dict: Dict[str, torch.Tensor], path: PathLike) -> None:
    tensors = {k: v.detach().contiguous().cpu() for k, v in state_dict.items()}
    _atomically(path, lambda tmp: save_file(tensors, str(tmp)))


def load_safetensors(path: PathLike, broadcast: bool = False) -> Dict[str, torch.Tensor]:
    return load_state_dict(path, broadcast=broadcast)


def save_json(data: dict, path: PathLike) -> None:
    text = json.dumps(data, indent=2, ensure_ascii=False)
    _atomically(path, lambda tmp: tmp.write_text(text, encoding="utf-8"))


def load_json(path: PathLike, broadcast: bool = False) -> dict:
    return _share(lambda: json.loads(Path(path).read_text(encoding="utf-8")), broadcast)


def save_torch(obj: Any, path: PathLike) -> None:
    _atomically(path, lambda tmp: torch.save(obj, str(tmp)))


def load_torch(path: PathLike, broadcast: bool = False) -> Any:
    return _share(lambda: torch.load(str(path), map_location="cpu", weights_only=False), broadcast)


def load_state_dict(path: PathLike, broadcast: bool = False) -> Dict[str, torch.Tensor]:
    if not (broadcast and dist.is_available() and dist.is_initialized()):
        return load_file(str(path))
    rank = _rank()
    local = load_file(str(path)) if rank == 0 else {}
    layout = [[(k, tuple(local[k].shape), local[k].dtype) for k in sorted(local)] if rank == 0 else None]
    dist.broadcast_object_list(layout, src=0)
    out: Dict[str, torch.Tensor] = {}
    for key, shape, dtype in layout[0]:
        buf = local[key].contiguous().cpu() if rank == 0 else torch.empty(shape, dtype=dtype)
        dist.broadcast(buf, src=0)
        out[key] = buf
    return out


# -- pretrained directories ---------------------------------------------------------------
def save_model(config: dict, state_dict: Dict[str, torch.Tensor], save_directory: str) -> None:
    root = Path(save_directory)
    root.mkdir(parents=True, exist_ok=True)
    save_json(config, root / CONFIG_FILE)
    save_safetensors(state_dict, root / WEIGHTS_FILE)


def load_model_config(save_directory: str) -> dict:
    return load_json(Path(save_directory) / CONFIG_FILE)


def load_model_weights(save_directory: str) -> Dict[str, torch.Tensor]:
    return load_state_dict(Path(save_directory) / WEIGHTS_FILE)


# -- training checkpoints -----------------------------------------------------------------
@dataclass
class Checkpoint:
    state_dict: Dict[str, Any] = field(default_factory=dict)
    epoch: int = 0
    iteration: int = 0
    extra: Dict[str, Any] = field(default_factory=dict)
    meta: Dict[str, Any] = field(default_factory=dict)
    config: Dict[str, Any] = field(default_factory=dict)

    def save(self, save_dir: str) -> None:
        root = Path(save_dir)
        root.mkdir(parents=True, exist_ok=True)
        if _rank() != 0:
            return
        stamp = {"epoch": self.epoch, "iteration": self.iteration, "timestamp": time.strftime("%Y-%m-%dT%H:%M:%S")}
        save_json(self.config, root / CONFIG_FILE)
        save_safetensors(self.state_dict, root / WEIGHTS_FILE)
        for name, payload in self.extra.items():
            save_torch(payload, root / f"{name}.pt")
        # last: its presence says that everything else is complete (what an automatic resume looks for)
        save_json({**stamp, **self.meta}, root / META_FILE)

    @classmethod
    def load(cls, save_dir: str, broadcast: bool = False) -> "Checkpoint":
        root = Path(save_dir)
        meta = load_json(root / META_FILE, broadcast)
        extra = {p.stem: load_torch(p, broadcast) for p in sorted(root.glob("*.pt"))}
        return cls(state_dict=load_state_dict(root / WEIGHTS_FILE, broadcast=broadcast), epoch=meta.get("epoch", 0),
                   iteration=meta.get("iteration", 0), extra=extra, config=load_json(root / CONFIG_FILE, broadcast))


def find_latest_checkpoint(ckpt_dir: str):
    """``(directory, meta)`` of the newest complete checkpoint under ``ckpt_dir`` (ordered by epoch, then
    iteration), or ``None``.  The reference resumes only from a directory and a position given by hand
    (``scripts/tools/train.py:144-149``); an emergency checkpoint written by the error path counts too."""
    best = None
    if not os.path.isdir(ckpt_dir):
        return None
    for name in os.listdir(ckpt_dir):
        root = os.path.join(ckpt_dir, name)
        if not (os.path.isfile(os.path.join(root, META_FILE)) and os.path.isfile(os.path.join(root, WEIGHTS_FILE))):
            continue
        try:
            with open(os.path.join(root, META_FILE)) as fh:
                meta = json.load(fh)
        except (OSError, ValueError):       # a checkpoint that was being written when the job died
            continue
        key = (int(meta.get("epoch", 0)), int(meta.get("iteration", 0)))
        if best is None or key > best[0]:
            best = (key, root, meta)
    return None if best is None else (best[1], best[2])
